// Internal state behind the opaque handles of include/p0p.h.
#pragma once
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <map>
#include <string>
#include <unordered_set>
#include <vector>

#include "../../include/p0p.h"

struct p0p_buf {
  void* ptr = nullptr;
  uint64_t size = 0;      // the reference's _pf
  bool owned = true;      // false: wrapped foreign memory
  bool ipc = false;       // a peer allocation mapped by p0p_ipc_open (unmapped on free)
  bool plain = false;     // cudaMalloc'd outside the stream-ordered pool (p0p_alloc_shareable): has an IPC handle, never pooled
  uint64_t seq = 0;       // pool age
};

struct p0p_ctx {
  int device = 0;
  cudaStream_t stream = nullptr;
  bool own_stream = true;
  cudaEvent_t ev = nullptr;
  int status = 0;         // sticky CUDA error, 0 while usable
  std::string err;
  cudaDeviceProp prop{};
  // buffer accounting and the same-size reuse pool (src/core/gpu.js:32-34, 87-139)
  std::unordered_set<p0p_buf*> bufs;
  std::map<uint64_t, std::vector<p0p_buf*>> pool;
  uint64_t alive = 0, peak = 0, pooled = 0, pooledN = 0, hw = 0, maxBuf = 0, creates = 0, reuses = 0, evictions = 0, poolSeq = 0;
  // op bookkeeping
  int last_kernel = 0;
  uint32_t last_plan[8] = {};   // the tensor-core kernel's plan of the last call (p0p_last_plan)
  uint64_t launches = 0;
  // split-K partial sums of the decode kernel (grown on demand, owned by the context)
  void* scratch = nullptr;
  uint64_t scratch_bytes = 0;
  bool capturing = false;
  std::unordered_set<void*> pinned;
  // a host-visible word kernels write when a bounded wait runs out (0 = fine)
  int* host_status = nullptr;
  int* dev_status = nullptr;
};

namespace p0p {

inline int fail(p0p_ctx* c, int code, const char* fmt, ...) {
  char b[512];
  va_list ap; va_start(ap, fmt); vsnprintf(b, sizeof b, fmt, ap); va_end(ap);
  if (c) c->err = b;
  return code;
}
// CUDA failure -> positive status; errors that poison the context mark it lost
inline int cuda_fail(p0p_ctx* c, cudaError_t e, const char* what) {
  if (c) {
    c->err = std::string(what) + ": " + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ")";
    switch (e) {
      case cudaErrorInvalidValue: case cudaErrorMemoryAllocation: case cudaErrorInvalidDevice: case cudaErrorNotReady:
      case cudaErrorInvalidConfiguration: case cudaErrorLaunchOutOfResources: break;
      default: c->status = (int)e;
    }
  }
  (void)cudaGetLastError();
  return (int)e;
}
struct DeviceGuard {
  int prev = -1; bool ok;
  explicit DeviceGuard(int dev) { ok = cudaGetDevice(&prev) == cudaSuccess; if (ok && prev != dev) ok = cudaSetDevice(dev) == cudaSuccess; else if (!ok) ok = cudaSetDevice(dev) == cudaSuccess; }
  ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
};
#define P0P_CUDA(ctx, call, what) do { cudaError_t e__ = (call); if (e__ != cudaSuccess) return ::p0p::cuda_fail((ctx), e__, (what)); } while (0)
#define P0P_ALIVE(ctx) do { if (!(ctx)) return -1; if ((ctx)->status) return ::p0p::fail((ctx), (ctx)->status, "GPU device lost: %s", (ctx)->err.c_str()); } while (0)

int ensure_scratch(p0p_ctx* c, uint64_t bytes);

}  // namespace p0p
