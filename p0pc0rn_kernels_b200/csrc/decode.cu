// Host side of the decode-sized multiply (k_decode.cuh): which calls it takes, the plan of a call (k-blocks, grid, shared
// memory, split-K scratch) and the launches; and the instantiations of the stream kernel.  The second-stage kernels are
// instantiated in decode_finish.cu.
#include <algorithm>

#include "device_once.h"
#include "k_decode.cuh"

namespace p0p {

typedef void (*decode_stream_fn)(const DecodeP);
typedef void (*decode_finish_fn)(const DecodeP);
decode_finish_fn decode_finish_kernel(uint32_t mp, uint32_t epi);      // decode_finish.cu

static decode_stream_fn stream_kernel(uint32_t enc, uint32_t xmode, uint32_t mp) {
  // [encoding][prologue: f16, lnmod, rms][8 | 16 token columns]
  static const decode_stream_fn table[2][3][2] = {
      {{k_decode_stream<P0P_ENC_Q4, P0P_X_F16, 8>, k_decode_stream<P0P_ENC_Q4, P0P_X_F16, 16>},
       {k_decode_stream<P0P_ENC_Q4, P0P_X_LNMOD, 8>, k_decode_stream<P0P_ENC_Q4, P0P_X_LNMOD, 16>},
       {k_decode_stream<P0P_ENC_Q4, P0P_X_RMS, 8>, k_decode_stream<P0P_ENC_Q4, P0P_X_RMS, 16>}},
      {{k_decode_stream<P0P_ENC_Q8, P0P_X_F16, 8>, k_decode_stream<P0P_ENC_Q8, P0P_X_F16, 16>},
       {k_decode_stream<P0P_ENC_Q8, P0P_X_LNMOD, 8>, k_decode_stream<P0P_ENC_Q8, P0P_X_LNMOD, 16>},
       {k_decode_stream<P0P_ENC_Q8, P0P_X_RMS, 8>, k_decode_stream<P0P_ENC_Q8, P0P_X_RMS, 16>}}};
  return table[enc][xmode][mp == 8u ? 0 : 1];
}

bool decode_supported(const KP& p) {
  if (p.M > 16u) return false;
  if (p.enc != P0P_ENC_Q4 && p.enc != P0P_ENC_Q8) return false;
  if (p.xmode != P0P_X_F16 && p.xmode != P0P_X_LNMOD && p.xmode != P0P_X_RMS) return false;
  if (p.wR0 % 64u) return false;
  if (p.epi == P0P_EPI_SWIGLU && (p.wR1 % 64u)) return false;
  if (p.K % D_STAGE_K) return false;                  // k-blocks are whole stages
  if ((uintptr_t)p.W & 15u) return false;             // bulk copies need 16-byte aligned sources
  if (p.enc == P0P_ENC_Q8 && (p.wk0 % 64u)) return false;
  if (p.epi == P0P_EPI_HEADS && ((uintptr_t)p.RP & 7u)) return false;      // the epilogue reads (cos, sin) as one 8-byte load
  return true;
}

uint64_t plan_decode(DecodeP& d, DecodeLaunch& L, int sms, size_t smem_per_sm) {
  const KP& p = d.p;
  d.Mp = p.M <= 8u ? 8u : 16u;
  d.vec32 = (p.xmode != P0P_X_F16 && (((uintptr_t)p.X | (uintptr_t)(p.PV + p.pvOff)) & 15u) == 0u && p.ldx % 4u == 0u && p.kx0 % 4u == 0u && (p.xmode != P0P_X_LNMOD || p.pvStride % 4u == 0u)) ? 1u : 0u;
  const uint32_t cols = p.epi == P0P_EPI_SWIGLU ? p.N / 2u : ((p.epi == P0P_EPI_HEADS || p.epi == P0P_EPI_ONORMGATE) ? (p.N + 127u) / 128u * 128u : p.N);
  d.th = (cols + 63u) / 64u;
  // tiles past the weight's last row do not exist: columns there read the last tile (their outputs are never stored)
  const uint32_t avail = (p.Nw - p.wR0) / 64u;
  if (p.epi != P0P_EPI_SWIGLU && d.th > avail) d.th = avail;
  d.tiles = p.epi == P0P_EPI_SWIGLU ? 2u * d.th : d.th;
  d.nslots = d.tiles * 64u;
  // k-block: as long as the token tile allows (about 32 KB); the blocks share the stages evenly whatever its length, but a
  // block's range must be at least one unit long (a unit is shared by at most two blocks), and every block wants work
  uint32_t kc = p.M <= 8u ? 2048u : 1024u;                                // token tile of (M + 1) * kc fp16 stays near 32 KB
  while (kc > p.K) kc >>= 1;                                              // (K is a multiple of 256)
  d.T = d.tiles * (p.K / (uint32_t)D_STAGE_K);
  const uint32_t tok_stride0 = kc * 2u + 64u;
  const size_t smem0 = (size_t)D_STAGES * D_STAGE_BYTES_Q8 + (size_t)(p.M + 1u) * tok_stride0 + 16384u;      // upper estimate: how many blocks an SM holds
  const uint32_t slots = (uint32_t)std::max<size_t>(1, std::min<size_t>(4, smem_per_sm / (smem0 + 1024))) * (uint32_t)sms;
  while (kc > (uint32_t)D_STAGE_K && d.T / std::min(d.T, slots) < kc / (uint32_t)D_STAGE_K) kc >>= 1;
  d.KC = kc; d.S = (p.K + kc - 1u) / kc; d.units = d.tiles * d.S;
  const uint32_t tok_stride = d.KC * 2u + (p.enc == P0P_ENC_Q4 ? 64u : 16u);
  const size_t ct_bytes = p.enc == P0P_ENC_Q4 ? (size_t)(d.KC / 32u) * (d.Mp / 2u) * 24u : (size_t)(d.KC / 64u) * (d.Mp / 2u) * 16u;
  L.smem = (size_t)D_STAGES * (p.enc == P0P_ENC_Q4 ? D_STAGE_BYTES_Q4 : D_STAGE_BYTES_Q8) + (((p.M + 1u) * tok_stride + 127u) & ~127u) + ct_bytes + 4u * 32u * (d.Mp / 2u) * 4u + 2u * D_STAGES * 8u + 128u;
  const uint32_t per_sm = (uint32_t)std::max<size_t>(1, std::min<size_t>(4, smem_per_sm / (L.smem + 1024)));
  // every block is resident: the ranges run side by side.  At least KC / 256 stages per block (see above).
  L.grid = (int)std::min<uint64_t>(d.T / (d.KC / (uint32_t)D_STAGE_K), (uint64_t)per_sm * (uint64_t)sms);
  while ((uint64_t)d.T * (uint64_t)L.grid >= (1ull << 32)) L.grid = (L.grid + 1) / 2;      // the kernels' range arithmetic is 32-bit
  d.G = (uint32_t)L.grid;
  d.whole = (p.K % d.KC == 0u && d.units >= 4u * d.G) ? 1u : 0u;
  L.fin_blocks = (p.epi == P0P_EPI_HEADS || p.epi == P0P_EPI_ONORMGATE) ? (p.N + 127u) / 128u : (((p.N + 3u) & ~3u) + 127u) / 128u;
  return 2ull * d.S * p.M * d.nslots * 4ull;
}

cudaError_t launch_decode_pair(const DecodeP& d, const DecodeLaunch& L, int device, cudaStream_t st) {
  const KP& p = d.p;
  if (L.smem > (size_t)D_SMEM_MAX) return cudaErrorInvalidValue;
  const decode_stream_fn stream = stream_kernel(p.enc, p.xmode, d.Mp);
  // the dynamic shared memory ceiling is an attribute of (kernel, device): raised once for each pair
  static DeviceOnce once[2][3][2];
  cudaError_t e = cudaSuccess;
  if (once[p.enc][p.xmode][d.Mp == 8u ? 0 : 1].run(device, [&] { e = cudaFuncSetAttribute(reinterpret_cast<const void*>(stream), cudaFuncAttributeMaxDynamicSharedMemorySize, D_SMEM_MAX); return (int)e; }))
    return e != cudaSuccess ? e : cudaErrorInvalidDevice;
  // both kernels are programmatic dependents of whatever precedes them in the stream (see k_decode.cuh)
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization; at[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)L.grid); cfg.blockDim = dim3(D_THREADS); cfg.dynamicSmemBytes = L.smem; cfg.stream = st; cfg.attrs = at; cfg.numAttrs = 1;
  if ((e = cudaLaunchKernelEx(&cfg, stream, d)) != cudaSuccess) return e;
  cfg.gridDim = dim3(L.fin_blocks); cfg.blockDim = dim3(128); cfg.dynamicSmemBytes = 0;
  return cudaLaunchKernelEx(&cfg, decode_finish_kernel(d.Mp, p.epi), d);
}

int launch_decode(p0p_ctx* c, const KP& p) {
  DecodeP d{};
  d.p = p;
  DecodeLaunch L{};
  const uint64_t sbytes = plan_decode(d, L, c->prop.multiProcessorCount, (size_t)c->prop.sharedMemPerMultiprocessor);
  if (int r = ensure_scratch(c, sbytes + 256)) return r;
  d.scratch = reinterpret_cast<float*>(c->scratch);
  d.status = c->dev_status;
  const uint32_t plan[8] = {d.G, d.T, d.KC, d.S, d.whole, d.units, d.tiles, 0u};
  std::copy(plan, plan + 8, c->last_plan);
  const cudaError_t e = launch_decode_pair(d, L, c->device, c->stream);
  if (e != cudaSuccess) return cuda_fail(c, e, "decode launch");
  c->launches += 2;
  return 0;
}

}  // namespace p0p
