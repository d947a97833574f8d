// p0p_peer_barrier: a stream-ordered barrier between the GPUs of one node, made of plain stores into the other GPUs'
// memory and polling of the GPU's own memory.  It orders the ranks after the gemm epilogues have stored their columns into
// every rank's copy of y (p0p_gemm_args.y_peers) and before those rows are read; being a kernel of this library it can be
// recorded into a CUDA graph like the multiplies around it.  Nothing here loads from another GPU's memory.
//
// Each rank owns a flag block of 64 words: word r (r < world) is the latest barrier number rank r has reached, written by
// rank r; word 32 is this rank's own barrier count.  A barrier adds one to the count, stores it into word `rank` of every
// rank's block and polls its own block until every other rank's word has reached the count.  All ranks must issue the same
// sequence of barriers.  The wait is bounded: when it runs out the kernel records a code in the context's status word (the
// next p0p_sync / p0p_read returns -10) and returns; the context stays usable.
#include "ctx.h"
#include "sync.cuh"

using namespace p0p;

namespace {

struct PeerFlags { uint32_t* p[8]; };

__device__ __forceinline__ void st_release_sys(uint32_t* a, uint32_t v) { asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(a), "r"(v) : "memory"); }
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* a) { uint32_t v; asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(a) : "memory"); return v; }

__global__ void __launch_bounds__(32) k_peer_barrier(uint32_t* mine, PeerFlags peers, uint32_t rank, uint32_t world, long long limit, int* status) {
  const uint32_t t = threadIdx.x;
  uint32_t seq = 0;
  if (t == 0) { seq = mine[32] + 1u; mine[32] = seq; }
  seq = __shfl_sync(0xffffffffu, seq, 0);
  if (t < world) {
    __threadfence_system();                                   // everything this GPU wrote before (its columns in the peers' buffers) comes first
    st_release_sys((t == rank ? mine : peers.p[t]) + rank, seq);
  }
  if (t < world && t != rank) {
    const long long t0 = clock64();
    uint32_t n = 0;
    while ((int)(ld_acquire_sys(mine + t) - seq) < 0) {
      __nanosleep(64);
      if ((++n & 15u) == 0u && clock64() - t0 > limit) { atomicCAS(status, 0, 301); break; }
    }
  }
}

inline bool live(const p0p_ctx* c, const p0p_buf* b) { return b && c->bufs.count(const_cast<p0p_buf*>(b)); }

}  // namespace

extern "C" int p0p_peer_barrier(p0p_ctx* c, p0p_buf* flags, p0p_buf* const* peer_flags, uint32_t rank, uint32_t world, uint64_t wait_cycles) {
  P0P_ALIVE(c);
  if (!world || world > 8u || rank >= world) return fail(c, -1, "peer_barrier: world must be 1..8 and rank below it");
  if (!live(c, flags) || flags->size < P0P_PEER_FLAG_BYTES) return fail(c, -4, "peer_barrier: the flag block must be a live buffer of at least %u bytes", (unsigned)P0P_PEER_FLAG_BYTES);
  PeerFlags pf{};
  for (uint32_t r = 0; r < world; r++) {
    if (r == rank) { pf.p[r] = (uint32_t*)flags->ptr; continue; }
    if (!peer_flags || !live(c, peer_flags[r]) || peer_flags[r]->size < P0P_PEER_FLAG_BYTES) return fail(c, -4, "peer_barrier: missing flag block of rank %u", r);
    pf.p[r] = (uint32_t*)peer_flags[r]->ptr;
  }
  DeviceGuard g(c->device);
  const long long limit = wait_cycles ? (long long)wait_cycles : WAIT_LIMIT_CYCLES;
  k_peer_barrier<<<1, 32, 0, c->stream>>>((uint32_t*)flags->ptr, pf, rank, world, limit, c->dev_status);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(c, e, "peer barrier launch");
  c->launches += 1;
  return 0;
}
