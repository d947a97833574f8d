// p0p_decode_q4_static: the decode-sized q4 multiply for callers that must not allocate device memory.
//
// Some hosts own every byte of device memory themselves and give a library none of it at run time: an inference
// server that reserved the whole GPU for its own arena at start-up, a plug-in running inside another runtime's
// memory manager, a real-time loop in which cudaMalloc's implicit device-wide synchronisation is unacceptable.
// The regular path (p0p_open / p0p_gemm) allocates: a context, a stream, and the split-K scratch of the decode
// kernel.  This entry point needs none of that.  Inputs and outputs are plain device pointers of the caller,
// work is enqueued on the caller's stream, and the kernel's split-K partial sums live in a fixed array inside
// this library's device image (P0P_STATIC_SCRATCH_BYTES, held by every GPU that loads the library until the
// process exits).
//
// Sharing rules.  Every call on a device uses the same array and leaves its partial sums there.  Nothing in it
// has to start at zero (each call overwrites exactly the words it later reads), but two calls whose kernels
// overlap on the GPU - different streams, or graph branches - race on it: keep calls on one device in one
// stream order.  The first call on each device looks up the array's device address (and raises one kernel
// attribute); make that first call before any stream capture begins.  The kernels bound every wait they make; whether
// one ran out is read back with p0p_decode_q4_static_status, which allocates nothing either.
#include <cstdio>
#include <cstring>
#include <mutex>

#include "k_decode.cuh"

namespace {

__device__ __align__(256) unsigned char g_static_scratch[P0P_STATIC_SCRATCH_BYTES];
__device__ __align__(16) int g_static_status[4];

constexpr int MAX_DEVICES = 64;
struct PerDevice { bool ready = false; float* scratch = nullptr; int* status = nullptr; int sms = 0; int smem_per_sm = 0; };
PerDevice g_dev[MAX_DEVICES];
std::mutex g_mu;

int say(char* err, size_t cap, int code, const char* msg) {
  if (err && cap) { size_t n = strlen(msg); if (n >= cap) n = cap - 1; memcpy(err, msg, n); err[n] = 0; }
  return code;
}

}  // namespace

extern "C" int p0p_decode_q4_static(int device, void* stream, const void* w, const void* x, void* y, uint32_t M, uint32_t N, uint32_t K,
                                    char* err, size_t err_cap) {
  using namespace p0p;
  if (err && err_cap) err[0] = 0;
  if (device < 0 || device >= MAX_DEVICES) return say(err, err_cap, -1, "decode_q4_static: device ordinal out of range");
  if (!w || !x || !y) return say(err, err_cap, -1, "decode_q4_static: null pointer");
  if (M < 1u || M > 16u) return say(err, err_cap, -2, "decode_q4_static: M must be 1..16");
  if (!N || N % 64u) return say(err, err_cap, -2, "decode_q4_static: N must be a positive multiple of 64 (whole q4 row tiles)");
  if (!K || K % D_STAGE_K) return say(err, err_cap, -2, "decode_q4_static: K must be a positive multiple of 256");
  if (((uintptr_t)w | (uintptr_t)x | (uintptr_t)y) & 15u) return say(err, err_cap, -2, "decode_q4_static: w, x and y must be 16-byte aligned");

  DeviceGuard guard(device);
  if (!guard.ok) return say(err, err_cap, -3, "decode_q4_static: cannot make the device current");
  PerDevice& pd = g_dev[device];
  {
    // set-up, once per device, with that device current: the array's NAME is a host-side stand-in for the symbol,
    // not an address a kernel could use, so the device address is looked up here and handed to the kernels.
    std::lock_guard<std::mutex> lock(g_mu);
    if (!pd.ready) {
      void* sp = nullptr; void* st = nullptr;
      cudaError_t e = cudaGetSymbolAddress(&sp, g_static_scratch);
      if (e == cudaSuccess) e = cudaGetSymbolAddress(&st, g_static_status);
      if (e == cudaSuccess) e = cudaDeviceGetAttribute(&pd.sms, cudaDevAttrMultiProcessorCount, device);
      if (e == cudaSuccess) e = cudaDeviceGetAttribute(&pd.smem_per_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, device);
      if (e != cudaSuccess) { (void)cudaGetLastError(); return say(err, err_cap, (int)e, cudaGetErrorString(e)); }
      pd.scratch = reinterpret_cast<float*>(sp); pd.status = reinterpret_cast<int*>(st); pd.ready = true;
    }
  }

  // ---- the plan of the decode kernel for a plain q4 multiply (fp16 tokens [M][K], fp16 result [M][N])
  DecodeP d{};
  KP& p = d.p;
  p.M = M; p.N = N; p.K = K; p.ldx = K; p.wG = K / 32u; p.ldy = N; p.Nw = N; p.eps = 1e-6f; p.stride = 1; p.ks = 1;
  p.enc = P0P_ENC_Q4; p.xmode = P0P_X_F16; p.epi = P0P_EPI_F16; p.vecx = 1;
  p.X = x; p.W = reinterpret_cast<const uint8_t*>(w); p.Y = y;
  DecodeLaunch L{};
  const uint64_t need = plan_decode(d, L, pd.sms, (size_t)pd.smem_per_sm);
  if (need > (uint64_t)P0P_STATIC_SCRATCH_BYTES) {
    char msg[200];
    snprintf(msg, sizeof msg, "decode_q4_static: this shape needs %llu bytes of split-K scratch, the built-in array holds %llu; use p0p_gemm",
             (unsigned long long)need, (unsigned long long)P0P_STATIC_SCRATCH_BYTES);
    return say(err, err_cap, -4, msg);
  }
  d.scratch = pd.scratch; d.status = pd.status;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemsetAsync(pd.status, 0, sizeof(int), st);          // the one word that must start at zero
  if (e == cudaSuccess) e = launch_decode_pair(d, L, device, st);
  if (e != cudaSuccess) { (void)cudaGetLastError(); return say(err, err_cap, (int)e, cudaGetErrorString(e)); }
  return 0;
}

// The kernels of p0p_decode_q4_static bound every wait; one that ran out leaves a code in a status word next to the scratch
// array and the results of that call are invalid.  This reads the word back (a 4-byte copy into a local variable and a wait
// for `stream`: no allocation either) after the calls queued on `stream`: 0 = fine, -10 = a wait ran out (the code is in `err`).
extern "C" int p0p_decode_q4_static_status(int device, void* stream, char* err, size_t err_cap) {
  using namespace p0p;
  if (err && err_cap) err[0] = 0;
  if (device < 0 || device >= MAX_DEVICES) return say(err, err_cap, -1, "decode_q4_static_status: device ordinal out of range");
  DeviceGuard guard(device);
  if (!guard.ok) return say(err, err_cap, -3, "decode_q4_static_status: cannot make the device current");
  int* word = nullptr;
  { std::lock_guard<std::mutex> lock(g_mu); if (g_dev[device].ready) word = g_dev[device].status; }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int code = 0;
  cudaError_t e = word ? cudaMemcpyAsync(&code, word, sizeof code, cudaMemcpyDeviceToHost, st) : cudaSuccess;
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) { (void)cudaGetLastError(); return say(err, err_cap, (int)e, cudaGetErrorString(e)); }
  if (code) {
    char msg[120];
    snprintf(msg, sizeof msg, "decode_q4_static: a kernel gave up on a bounded wait (code %d); the results of the queued calls are invalid", code);
    return say(err, err_cap, -10, msg);
  }
  return 0;
}
