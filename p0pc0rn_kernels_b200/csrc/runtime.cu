// Device context, buffers with the reference's accounting and same-size reuse pool, copies.
// Replaces, for the gemm path, class Gpu / Runner of the reference (src/core/gpu.js:29-257): a CUDA stream
// is the in-order queue, so there is no batching layer and no per-dispatch bind group.
#include <cstring>

#include "ctx.h"

using namespace p0p;

extern "C" {

uint32_t p0p_abi_version(void) { return P0P_ABI_VERSION; }

int p0p_open(int device, const p0p_opts* opts, p0p_ctx** out) {
  if (!out) return -1;
  *out = nullptr;
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n == 0) return e != cudaSuccess ? (int)e : (int)cudaErrorNoDevice;   // createGpu throws GpuError('no ... adapter')
  if (device < 0 || device >= n) return -2;
  p0p_ctx* c = new p0p_ctx();
  c->device = device;
  DeviceGuard g(device);
  if ((e = cudaGetDeviceProperties(&c->prop, device)) != cudaSuccess) { delete c; return (int)e; }
  if (c->prop.major < 10) { delete c; return -3; }   // sm_100a code only: the analogue of the missing 'shader-f16' feature (src/core/gpu.js:49)
  if (opts && opts->struct_size >= sizeof(p0p_opts) && (opts->flags & P0P_OPT_USE_STREAM)) { c->stream = (cudaStream_t)opts->stream; c->own_stream = false; }
  else if ((e = cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking)) != cudaSuccess) { delete c; return (int)e; }
  if ((e = cudaEventCreateWithFlags(&c->ev, cudaEventDisableTiming)) != cudaSuccess) { if (c->own_stream) cudaStreamDestroy(c->stream); delete c; return (int)e; }
  if ((e = cudaHostAlloc((void**)&c->host_status, sizeof(int), cudaHostAllocMapped)) != cudaSuccess ||
      (e = cudaHostGetDevicePointer((void**)&c->dev_status, c->host_status, 0)) != cudaSuccess) {
    if (c->host_status) cudaFreeHost(c->host_status);
    cudaEventDestroy(c->ev); if (c->own_stream) cudaStreamDestroy(c->stream); delete c; return (int)e;
  }
  *c->host_status = 0;
  *out = c;
  return 0;
}

// after a stream sync: did a kernel give up on a bounded wait?
static int check_kernel_status(p0p_ctx* c) {
  if (c->host_status && *c->host_status) {
    int code = *c->host_status; *c->host_status = 0;
    return fail(c, -10, "a kernel gave up on a bounded wait (code %d); results of the queued work are invalid", code);
  }
  return 0;
}

static void destroy_buf(p0p_ctx* c, p0p_buf* b) {
  if (b->owned && b->ptr) { if (b->plain) { cudaStreamSynchronize(c->stream); cudaFree(b->ptr); } else cudaFreeAsync(b->ptr, c->stream); }
  delete b;
}

// destroy pooled buffers, oldest first, until at most `room` bytes stay pooled (src/core/gpu.js:123-133)
static void evict(p0p_ctx* c, uint64_t room) {
  while (c->pooled > room) {
    p0p_buf* oldest = nullptr; uint64_t key = 0;
    for (auto& kv : c->pool) for (p0p_buf* b : kv.second) if (!oldest || b->seq < oldest->seq) { oldest = b; key = kv.first; }
    if (!oldest) break;
    auto& L = c->pool[key];
    for (size_t i = 0; i < L.size(); i++) if (L[i] == oldest) { L.erase(L.begin() + i); break; }
    if (L.empty()) c->pool.erase(key);
    c->pooled -= oldest->size; c->pooledN--; c->evictions++;
    destroy_buf(c, oldest);
  }
}
static inline uint64_t pool_cap(const p0p_ctx* c) { return c->hw + c->maxBuf; }   // src/core/gpu.js:136

int p0p_close(p0p_ctx* c) {
  if (!c) return -1;
  DeviceGuard g(c->device);
  cudaStreamSynchronize(c->stream);
  for (p0p_buf* b : c->bufs) destroy_buf(c, b);
  c->bufs.clear();
  evict(c, 0);
  if (c->scratch) cudaFree(c->scratch);
  if (c->host_status) cudaFreeHost(c->host_status);
  for (void* p : c->pinned) cudaFreeHost(p);
  cudaStreamSynchronize(c->stream);
  if (c->ev) cudaEventDestroy(c->ev);
  if (c->own_stream) cudaStreamDestroy(c->stream);
  delete c;
  return 0;
}

const char* p0p_last_error(const p0p_ctx* c) { return c ? c->err.c_str() : "null context"; }
int p0p_status(const p0p_ctx* c) { return c ? c->status : -1; }
void* p0p_stream(const p0p_ctx* c) { return c ? (void*)c->stream : nullptr; }

size_t p0p_describe(const p0p_ctx* c, char* dst, size_t cap) {
  if (!c) return 0;
  char b[512];
  int n = snprintf(b, sizeof b,
                   "{\"vendor\":\"nvidia\",\"architecture\":\"sm_%d%d\",\"device\":\"%s\",\"f16\":true,\"subgroups\":true,\"sgMin\":32,\"sgMax\":32,"
                   "\"sms\":%d,\"memMB\":%llu,\"l2MB\":%d,\"wgMem\":%zu,\"wgInv\":%d}",
                   c->prop.major, c->prop.minor, c->prop.name, c->prop.multiProcessorCount, (unsigned long long)(c->prop.totalGlobalMem >> 20),
                   c->prop.l2CacheSize >> 20, (size_t)c->prop.sharedMemPerBlockOptin, c->prop.maxThreadsPerBlock);
  if (dst && cap) { size_t m = (size_t)n < cap - 1 ? (size_t)n : cap - 1; memcpy(dst, b, m); dst[m] = 0; }
  return (size_t)n + 1;
}

int p0p_alloc(p0p_ctx* c, uint64_t bytes, p0p_buf** out) {
  P0P_ALIVE(c);
  if (!out) return fail(c, -1, "buffer: null result pointer");
  *out = nullptr;
  uint64_t size = bytes < 16 ? 16 : (bytes + 15) / 16 * 16;                       // src/core/gpu.js:88
  if (size > c->prop.totalGlobalMem) return fail(c, -2, "buffer %llu B exceeds maxBufferSize", (unsigned long long)size);
  DeviceGuard g(c->device);
  auto it = c->pool.find(size);
  p0p_buf* b = nullptr;
  if (it != c->pool.end() && !it->second.empty()) {                               // pooled: cleared like a new one (:92-101)
    b = it->second.back(); it->second.pop_back();
    if (it->second.empty()) c->pool.erase(it);
    c->pooled -= size; c->pooledN--; c->reuses++;
  } else {
    uint64_t cap = pool_cap(c), want = c->alive + size;
    evict(c, (cap > want ? cap : want) - want);                                   // :104
    b = new p0p_buf();
    cudaError_t e = cudaMallocAsync(&b->ptr, size, c->stream);
    if (e != cudaSuccess) { delete b; return cuda_fail(c, e, "buffer"); }
    b->size = size; c->creates++;
    if (size > c->maxBuf) c->maxBuf = size;
  }
  cudaError_t e = cudaMemsetAsync(b->ptr, 0, size, c->stream);
  if (e != cudaSuccess) { destroy_buf(c, b); return cuda_fail(c, e, "buffer clear"); }
  c->bufs.insert(b); c->alive += size;
  if (c->alive > c->peak) c->peak = c->alive;
  if (c->alive > c->hw) c->hw = c->alive;
  *out = b;
  return 0;
}

int p0p_wrap(p0p_ctx* c, void* device_ptr, uint64_t bytes, p0p_buf** out) {
  P0P_ALIVE(c);
  if (!out || !device_ptr || !bytes) return fail(c, -1, "wrap: null pointer or empty range");
  p0p_buf* b = new p0p_buf();
  b->ptr = device_ptr; b->size = bytes; b->owned = false;
  c->bufs.insert(b);
  *out = b;
  return 0;
}

int p0p_alloc_shareable(p0p_ctx* c, uint64_t bytes, p0p_buf** out) {
  P0P_ALIVE(c);
  if (!out) return fail(c, -1, "buffer: null result pointer");
  *out = nullptr;
  const uint64_t size = bytes < 16 ? 16 : (bytes + 15) / 16 * 16;
  if (size > c->prop.totalGlobalMem) return fail(c, -2, "buffer %llu B exceeds maxBufferSize", (unsigned long long)size);
  DeviceGuard g(c->device);
  p0p_buf* b = new p0p_buf();
  cudaError_t e = cudaMalloc(&b->ptr, size);             // not the stream-ordered pool: its memory has no IPC handle
  if (e != cudaSuccess) { delete b; return cuda_fail(c, e, "shareable buffer"); }
  b->size = size; b->plain = true; c->creates++;
  e = cudaMemsetAsync(b->ptr, 0, size, c->stream);
  if (e != cudaSuccess) { cudaFree(b->ptr); delete b; return cuda_fail(c, e, "buffer clear"); }
  c->bufs.insert(b); c->alive += size;
  if (c->alive > c->peak) c->peak = c->alive;
  if (c->alive > c->hw) c->hw = c->alive;
  *out = b;
  return 0;
}
int p0p_ipc_export(p0p_ctx* c, const p0p_buf* b, void* handle64) {
  P0P_ALIVE(c);
  if (!b || !handle64 || !c->bufs.count(const_cast<p0p_buf*>(b)) || !b->owned || !b->plain) return fail(c, -1, "ipc_export: needs a buffer made by p0p_alloc_shareable");
  DeviceGuard g(c->device);
  cudaIpcMemHandle_t h;
  static_assert(sizeof(h) == 64, "CUDA IPC handles are 64 bytes");
  P0P_CUDA(c, cudaIpcGetMemHandle(&h, b->ptr), "ipc_export");
  memcpy(handle64, &h, sizeof h);
  return 0;
}
int p0p_ipc_open(p0p_ctx* c, const void* handle64, uint64_t bytes, p0p_buf** out) {
  P0P_ALIVE(c);
  if (!handle64 || !out || !bytes) return fail(c, -1, "ipc_open: null pointer or empty range");
  DeviceGuard g(c->device);
  cudaIpcMemHandle_t h; memcpy(&h, handle64, sizeof h);
  void* ptr = nullptr;
  P0P_CUDA(c, cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess), "ipc_open");
  p0p_buf* b = new p0p_buf();
  b->ptr = ptr; b->size = bytes; b->owned = false; b->ipc = true;
  c->bufs.insert(b);
  *out = b;
  return 0;
}
int p0p_free(p0p_ctx* c, p0p_buf* b) {
  if (!c) return -1;
  if (!b || !c->bufs.count(b)) return 0;                                          // double free is a no-op (:113)
  DeviceGuard g(c->device);
  c->bufs.erase(b);
  if (!b->owned) { if (b->ipc) (void)cudaIpcCloseMemHandle(b->ptr); delete b; return 0; }
  c->alive -= b->size;
  if (!b->plain && !c->status && c->alive + c->pooled + b->size <= pool_cap(c)) {  // :115-118
    b->seq = ++c->poolSeq;
    c->pool[b->size].push_back(b); c->pooled += b->size; c->pooledN++;
    return 0;
  }
  destroy_buf(c, b);
  return 0;
}

int p0p_drain_pool(p0p_ctx* c) { if (!c) return -1; DeviceGuard g(c->device); evict(c, 0); return 0; }
int p0p_reset_peak(p0p_ctx* c) { if (!c) return -1; c->peak = c->alive; return 0; }
int p0p_pool_stats(const p0p_ctx* c, uint64_t o[9]) {
  if (!c || !o) return -1;
  uint64_t live = 0; for (p0p_buf* b : c->bufs) if (b->owned) live++;
  o[0] = c->alive; o[1] = c->pooled; o[2] = c->peak; o[3] = c->hw; o[4] = live; o[5] = c->pooledN; o[6] = c->creates; o[7] = c->reuses; o[8] = c->evictions;
  return 0;
}
uint64_t p0p_buf_size(const p0p_buf* b) { return b ? b->size : 0; }
void* p0p_buf_ptr(const p0p_buf* b) { return b ? b->ptr : nullptr; }

static int check_range(p0p_ctx* c, const p0p_buf* b, uint64_t off, uint64_t bytes, const char* what) {
  if (!b || !c->bufs.count(const_cast<p0p_buf*>(b))) return fail(c, -1, "%s: not a live buffer of this context", what);
  if (off > b->size || bytes > b->size - off) return fail(c, -2, "%s: range [%llu, +%llu) outside the buffer of %llu bytes", what, (unsigned long long)off, (unsigned long long)bytes, (unsigned long long)b->size);
  return 0;
}

int p0p_write(p0p_ctx* c, p0p_buf* b, uint64_t dst_off, const void* host, uint64_t bytes) {
  P0P_ALIVE(c);
  if (int r = check_range(c, b, dst_off, bytes, "upload")) return r;
  if (!bytes) return 0;
  if (!host) return fail(c, -1, "upload: null host pointer");
  DeviceGuard g(c->device);
  P0P_CUDA(c, cudaMemcpyAsync((char*)b->ptr + dst_off, host, bytes, cudaMemcpyHostToDevice, c->stream), "upload");
  // Pageable memory is staged before the call returns.  A page-locked source is read by the copy engine
  // later, so wait for this copy: the caller may reuse the range on return either way.
  cudaPointerAttributes at{};
  if (cudaPointerGetAttributes(&at, host) == cudaSuccess && at.type == cudaMemoryTypeHost) {
    P0P_CUDA(c, cudaEventRecord(c->ev, c->stream), "upload");
    P0P_CUDA(c, cudaEventSynchronize(c->ev), "upload");
  } else (void)cudaGetLastError();
  return 0;
}

int p0p_read(p0p_ctx* c, const p0p_buf* b, uint64_t off, void* host, uint64_t bytes) {
  P0P_ALIVE(c);
  if (int r = check_range(c, b, off, bytes, "read")) return r;
  if (!bytes) return 0;
  if (!host) return fail(c, -1, "read: null host pointer");
  DeviceGuard g(c->device);
  P0P_CUDA(c, cudaMemcpyAsync(host, (const char*)b->ptr + off, bytes, cudaMemcpyDeviceToHost, c->stream), "read");
  P0P_CUDA(c, cudaStreamSynchronize(c->stream), "read");
  return check_kernel_status(c);
}

int p0p_clear(p0p_ctx* c, p0p_buf* b, uint64_t off, uint64_t bytes) {
  P0P_ALIVE(c);
  if (int r = check_range(c, b, off, bytes, "clear")) return r;
  DeviceGuard g(c->device);
  if (bytes) P0P_CUDA(c, cudaMemsetAsync((char*)b->ptr + off, 0, bytes, c->stream), "clear");
  return 0;
}

int p0p_copy(p0p_ctx* c, const p0p_buf* src, uint64_t so, p0p_buf* dst, uint64_t d_o, uint64_t bytes) {
  P0P_ALIVE(c);
  if (int r = check_range(c, src, so, bytes, "copy source")) return r;
  if (int r = check_range(c, dst, d_o, bytes, "copy destination")) return r;
  DeviceGuard g(c->device);
  if (bytes) P0P_CUDA(c, cudaMemcpyAsync((char*)dst->ptr + d_o, (const char*)src->ptr + so, bytes, cudaMemcpyDeviceToDevice, c->stream), "copy");
  return 0;
}

int p0p_sync(p0p_ctx* c) {
  P0P_ALIVE(c);
  DeviceGuard g(c->device);
  P0P_CUDA(c, cudaStreamSynchronize(c->stream), "done");
  return check_kernel_status(c);
}

int p0p_host_alloc(p0p_ctx* c, uint64_t bytes, void** out) {
  P0P_ALIVE(c);
  if (!out) return fail(c, -1, "host_alloc: null result pointer");
  DeviceGuard g(c->device);
  P0P_CUDA(c, cudaMallocHost(out, bytes ? bytes : 1), "host_alloc");
  c->pinned.insert(*out);
  return 0;
}
int p0p_host_free(p0p_ctx* c, void* p) {
  if (!c) return -1;
  if (!p || !c->pinned.count(p)) return 0;
  DeviceGuard g(c->device);
  c->pinned.erase(p);
  cudaFreeHost(p);
  return 0;
}

struct p0p_graph { cudaGraph_t graph = nullptr; cudaGraphExec_t exec = nullptr; };

int p0p_capture_begin(p0p_ctx* c) {
  P0P_ALIVE(c);
  if (c->capturing) return fail(c, -1, "capture: already recording");
  DeviceGuard g(c->device);
  P0P_CUDA(c, cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal), "capture begin");
  c->capturing = true;
  return 0;
}
int p0p_capture_end(p0p_ctx* c, p0p_graph** out) {
  if (!c || !out) return -1;
  if (!c->capturing) return fail(c, -1, "capture: not recording");
  DeviceGuard g(c->device);
  c->capturing = false;
  p0p_graph* gr = new p0p_graph();
  cudaError_t e = cudaStreamEndCapture(c->stream, &gr->graph);
  if (e == cudaSuccess) e = cudaGraphInstantiate(&gr->exec, gr->graph, 0);
  if (e != cudaSuccess) { if (gr->graph) cudaGraphDestroy(gr->graph); delete gr; return cuda_fail(c, e, "capture end"); }
  *out = gr;
  return 0;
}
int p0p_graph_launch(p0p_ctx* c, p0p_graph* gr) {
  P0P_ALIVE(c);
  if (!gr || !gr->exec) return fail(c, -1, "graph: null graph");
  DeviceGuard g(c->device);
  P0P_CUDA(c, cudaGraphLaunch(gr->exec, c->stream), "graph launch");
  return 0;
}
int p0p_graph_free(p0p_ctx* c, p0p_graph* gr) {
  if (!c) return -1;
  if (!gr) return 0;
  DeviceGuard g(c->device);
  if (gr->exec) cudaGraphExecDestroy(gr->exec);
  if (gr->graph) cudaGraphDestroy(gr->graph);
  delete gr;
  return 0;
}

}  // extern "C"

namespace p0p {
// is the context's stream recording a graph, whoever began the capture (p0p_capture_begin, or the owner of a shared stream)?
static bool stream_is_capturing(p0p_ctx* c) {
  if (c->capturing) return true;
  cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(c->stream, &st) != cudaSuccess) { (void)cudaGetLastError(); return false; }
  return st != cudaStreamCaptureStatusNone;
}

int ensure_scratch(p0p_ctx* c, uint64_t bytes) {
  if (c->scratch_bytes >= bytes) return 0;
  if (stream_is_capturing(c)) return fail(c, -11, "this call needs %llu bytes of scratch memory, which cannot be sized while recording: run it once before p0p_capture_begin", (unsigned long long)bytes);
  if (c->scratch) { cudaStreamSynchronize(c->stream); cudaFree(c->scratch); c->scratch = nullptr; c->scratch_bytes = 0; }
  uint64_t want = bytes < (8ull << 20) ? (8ull << 20) : (bytes + (1ull << 20) - 1) & ~((1ull << 20) - 1);
  cudaError_t e = cudaMalloc(&c->scratch, want);
  if (e != cudaSuccess) return cuda_fail(c, e, "split-K scratch");
  c->scratch_bytes = want;
  return 0;
}
}  // namespace p0p
