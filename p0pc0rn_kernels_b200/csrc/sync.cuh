// Thin wrappers over the PTX this library uses for asynchronous data movement on sm_100a: mbarriers,
// bulk (TMA) copies and tensor-map copies.  Every wait is bounded: after the limit it records a code in a
// host-visible status word and reports failure, so a protocol error ends the kernel instead of hanging the GPU.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace p0p {

constexpr long long WAIT_LIMIT_CYCLES = 4000000000LL;   // about two seconds at boost clock

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory"); }
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) { asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory"); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
// One try: the hardware parks the thread for a short, system-chosen time unless the phase completes first.  (An explicit, longer
// suspend-time hint was measured: the waiters then wake late and every kernel here got 10-20 % slower.)
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// bounded wait; false after the limit (the code lands in *status).  sleep_ns > 0: the thread also backs off between tries, for
// waits that are long and off the critical path (a polling warp otherwise takes issue slots from the warps that work).  The
// clock is read only every 256 tries.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* status, int code, uint32_t sleep_ns = 0) {
  if (mbar_try(bar, parity)) return true;
  const long long t0 = clock64();
  uint32_t n = 0;
  while (!mbar_try(bar, parity)) {
    if (sleep_ns) __nanosleep(sleep_ns);
    if ((++n & 255u) == 0u && clock64() - t0 > WAIT_LIMIT_CYCLES) { if (status) atomicCAS(status, 0, code); return false; }
  }
  return true;
}

// Programmatic dependent launch.  A kernel launched with the programmatic-serialization attribute may start while the
// kernel before it in the stream still runs; it must call grid_dependency_wait() before it touches anything that kernel
// writes (the wait returns once that kernel has finished and its writes are visible; without the attribute it returns
// at once).  grid_launch_dependents() tells the scheduler that the kernel after this one may begin to launch.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// global -> shared bulk copy; both addresses 16-byte aligned, bytes a multiple of 16; completes on `bar`
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// 2-D tiled tensor-map copy global -> shared, to this block only; x is the innermost coordinate
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
// 3-D tiled tensor-map copy (c0 innermost)
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
               ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar) : "memory");
}
// 4-D tiled tensor-map copy (c0 innermost); coordinates outside the tensor read as zero, which is the convolution's padding
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
               ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar) : "memory");
}

}  // namespace p0p
