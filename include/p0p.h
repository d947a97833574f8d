/*
 * p0p.h — C ABI of the B200-native `gemm` path of p0pc0rn-kernels.
 *
 * This is the boundary a foreign-function binding (Node N-API, Python ctypes, cgo ...) attaches to.  It
 * replaces, for the gemm path only, the reference's WebGPU runtime (src/core/gpu.js) and its generated
 * shader op (src/ops/gemm.js).  Plain pointers and sizes only; no exceptions cross it; every call returns
 * an int status:   0 = ok,   < 0 = invalid argument (p0p_last_error() holds the message, worded like the
 * reference's thrown Error where one exists),   > 0 = a CUDA error code (sticky ones mark the context lost).
 *
 * One context = one device + one in-order stream.  Calls on one context must come from one thread at a
 * time (the reference's caller is a single JavaScript thread).
 *
 * Citations are paths inside the reference project (file:line).
 */
#ifndef P0P_H
#define P0P_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define P0P_ABI_VERSION 1

typedef struct p0p_ctx p0p_ctx;   /* replaces class Gpu + Runner           (src/core/gpu.js:29-199, 203-257) */
typedef struct p0p_buf p0p_buf;   /* replaces a GPUBuffer with its _pf size (src/core/gpu.js:105-106)        */

/* ---- enumerations: the strings of the reference's argument object, as integers ------------------------ */
enum { P0P_ENC_Q4 = 0, P0P_ENC_Q8 = 1, P0P_ENC_F16 = 2 };                    /* 'q4g32a.t64' | 'q8g64s.t64' | 'f16'  (src/ops/gemm.js:269-271) */
enum { P0P_X_F16 = 0, P0P_X_LNMOD = 1, P0P_X_RMS = 2, P0P_X_CONV = 3, P0P_X_CONV3 = 4 };   /* x.mode / conv.kind        (src/ops/gemm.js:275)     */
enum { P0P_EPI_F16 = 0, P0P_EPI_F32 = 1, P0P_EPI_RESADD = 2, P0P_EPI_SWIGLU = 3, P0P_EPI_HEADS = 4, P0P_EPI_BIAS = 5, P0P_EPI_ONORMGATE = 6 };
enum {                                                                       /* booleans of the config object       (src/ops/gemm.js:276-277)  */
  P0P_F_GATE = 1,        /* resadd: ev given -> per-column gate       */
  P0P_F_RES = 2,         /* bias: add the fp16 Y already there        */
  P0P_F_STORE = 4,       /* resadd: write instead of accumulate       */
  P0P_F_GN = 8,          /* conv: fused GroupNorm-apply + SiLU        */
  P0P_F_UP2 = 16,        /* conv: fused nearest 2x upsample           */
  P0P_F_PN = 32,         /* conv3: fused PixelNorm + SiLU             */
  P0P_F_BIAS = 64,       /* resadd / swiglu: bv given                 */
  P0P_F_GELU = 128,      /* swiglu: act 'gelu' (GeGLU)                */
  P0P_F_ROPE_HALF = 256  /* heads: ropeMode 'half' (pairs d, d+64)    */
};
/* which kernel family served the last p0p_gemm call (p0p_last_kernel) or is forced (p0p_gemm_args.force_kernel) */
enum { P0P_K_AUTO = 0, P0P_K_GENERIC = 1, P0P_K_DECODE = 2, P0P_K_UMMA = 3,
       /* p0p_attention: the warp-level kernel / the tensor-memory kernel (p0p_attn_args.kernel forces one of them) */
       P0P_K_ATTN_WARP = 16, P0P_K_ATTN_TMEM = 17 };

enum { P0P_OPT_USE_STREAM = 1 };

/* ---- context ------------------------------------------------------------------------------------------- */
typedef struct p0p_opts {
  uint32_t struct_size;        /* sizeof(p0p_opts) */
  uint32_t flags;              /* P0P_OPT_* */
  void*    stream;             /* with P0P_OPT_USE_STREAM: the cudaStream_t to enqueue on (NULL = the legacy default stream);
                                  otherwise ignored and the context creates and owns a stream */
} p0p_opts;

/* createGpu(opts) (src/core/gpu.js:15-20, 41-77): open device `device` (ordinal). */
int p0p_open(int device, const p0p_opts* opts, p0p_ctx** out);
/* freeAll + destroy (src/core/gpu.js:138). */
int p0p_close(p0p_ctx* ctx);
/* message of the last failed call on this context (never NULL). Replaces thrown Error / GpuError text. */
const char* p0p_last_error(const p0p_ctx* ctx);
/* 0 while usable; the sticky CUDA error once the device is lost (gpu.lost, src/core/gpu.js:79, 171-176). */
int p0p_status(const p0p_ctx* ctx);
/* gpu.describe() (src/core/gpu.js:80-84): writes a short JSON text about the device; returns bytes needed. */
size_t p0p_describe(const p0p_ctx* ctx, char* dst, size_t cap);
/* the cudaStream_t work is enqueued on (for callers that interleave their own device work) */
void* p0p_stream(const p0p_ctx* ctx);

/* ---- buffers (src/core/gpu.js:87-139) ------------------------------------------------------------------ */
/* gpu.buffer(size): size -> max(16, ceil16(size)); contents zero (new or pooled); counted in alive/peak. */
int p0p_alloc(p0p_ctx* ctx, uint64_t bytes, p0p_buf** out);
/* adopt device memory owned by someone else (e.g. a tensor of the host framework); p0p_free only drops the handle */
int p0p_wrap(p0p_ctx* ctx, void* device_ptr, uint64_t bytes, p0p_buf** out);
/* gpu.free(b): back to the same-size pool or released; unknown / already freed handles are ignored. */
int p0p_free(p0p_ctx* ctx, p0p_buf* buf);
/* gpu.drainPool() (src/core/gpu.js:134) */
int p0p_drain_pool(p0p_ctx* ctx);
/* gpu.poolStats() fields (src/core/gpu.js:137): alive, pooled, peak, high-water bytes; live / pooled counts; creates, reuses, evictions */
int p0p_pool_stats(const p0p_ctx* ctx, uint64_t out[9]);
int p0p_reset_peak(p0p_ctx* ctx);
uint64_t p0p_buf_size(const p0p_buf* buf);          /* GPUBuffer._pf */
void*    p0p_buf_ptr(const p0p_buf* buf);           /* the device address */

/* gpu.upload(data, label, dst, dstOff) / device.queue.writeBuffer (src/core/gpu.js:141-148): copies `bytes`
 * from host memory into buf at dst_off, in stream order; the host range may be reused when the call returns. */
int p0p_write(p0p_ctx* ctx, p0p_buf* buf, uint64_t dst_off, const void* host, uint64_t bytes);
/* gpu.read(buf, off, size) (src/core/gpu.js:150-170): waits for queued work, copies to host. */
int p0p_read(p0p_ctx* ctx, const p0p_buf* buf, uint64_t off, void* host, uint64_t bytes);
/* enc.clearBuffer (src/core/gpu.js:97) on a byte range */
int p0p_clear(p0p_ctx* ctx, p0p_buf* buf, uint64_t off, uint64_t bytes);
/* Runner.copy (src/core/gpu.js:240-245) */
int p0p_copy(p0p_ctx* ctx, const p0p_buf* src, uint64_t src_off, p0p_buf* dst, uint64_t dst_off, uint64_t bytes);
/* gpu.done() (src/core/gpu.js:171-176) */
int p0p_sync(p0p_ctx* ctx);
/* page-locked host memory for callers that want asynchronous uploads / fast reads */
int p0p_host_alloc(p0p_ctx* ctx, uint64_t bytes, void** out);
int p0p_host_free(p0p_ctx* ctx, void* p);

/* ---- recorded launch sequences ---------------------------------------------------------------------------- */
/* The reference's Runner batches dispatches into one command buffer per submit (src/core/gpu.js:203-257) to keep
 * the GPU fed; the CUDA analogue is a graph.  Between begin and end, p0p_gemm / p0p_rowstats / p0p_copy /
 * p0p_clear calls are recorded instead of run; p0p_graph_launch replays them in stream order.  Run the same
 * calls once before recording (first calls size the library's scratch memory). */
typedef struct p0p_graph p0p_graph;
int p0p_capture_begin(p0p_ctx* ctx);
int p0p_capture_end(p0p_ctx* ctx, p0p_graph** out);
int p0p_graph_launch(p0p_ctx* ctx, p0p_graph* g);
int p0p_graph_free(p0p_ctx* ctx, p0p_graph* g);

/* ---- the op -------------------------------------------------------------------------------------------- */
/* The uniform block of the reference shader (struct P, src/ops/gemm.js:39-41, filled at :317-322) plus the
 * bindings (:304-313) and the configuration key (:275-277).  Offsets are in the unit the reference uses:
 * bytes for x/w/y, floats for ev/pv/bv, rows for stats. */
typedef struct p0p_gemm_args {
  uint32_t struct_size;            /* sizeof(p0p_gemm_args) */
  uint32_t enc, xmode, epi, flags; /* enums above */
  uint32_t M, N, K;
  uint32_t ldx, kx0;               /* x.ld || K, x.k0 */
  uint32_t wr0, wr1, wk0;          /* first weight row, first 'up' row (swiglu), first weight column */
  uint32_t w_rows, w_cols, w_ld;   /* w.rows (Nw), w.cols (Ktot), w.ld (f16 row stride in halves; 0 = cols) */
  uint32_t ldy, ny0;               /* y.ld || N, y.n0 */
  uint32_t rowOff, Ltot, Hq, Hkv;  /* heads */
  float    eps;                    /* heads.eps (default 1e-6) */
  uint32_t pv_off, pv_stride, ev_off, st_off, bv_off, bv_up;
  uint32_t Hi, Wi, Ci, Ho, Wo, stride, padT, padL, ks;   /* conv (stride defaults 1, ks defaults 1) */
  uint32_t tile_bm, tile_bn;       /* a.tile: accepted for compatibility; 0 = default. Results do not depend on it. */
  uint32_t acc_f16;                /* a.acc == 'f16': accepted; accumulation is always fp32 */
  uint32_t force_kernel;           /* P0P_K_AUTO, or a family to force (tests); unsupported combinations fail */
  p0p_buf *x, *w, *y;              /* required */
  p0p_buf *st, *pv, *ev, *bv, *rp, *gt;   /* optional, NULL when the configuration does not bind them */
  uint64_t x_off, w_off, y_off;    /* bytes */
  uint64_t w_bytes;                /* w.bytes (size of the encoded tensor) */
  uint64_t x_size, y_size;         /* x.size / y.size when given, else 0 = to the end of the buffer */
  /* No counterpart in the reference (multi-GPU extension): peer copies of y.  Every result is stored to y AND, at the same
   * byte offset, to each y_peers[i] - device memory of another GPU opened with p0p_ipc_open.  This is the all-gather of an
   * N-sharded output fused into the store: each rank writes its columns into every rank's full-row buffer (y.ld = full N,
   * y.n0 = the rank's first column); the caller still orders the ranks (any stream-ordered barrier) before the rows are read.
   * Plain peer stores over NVLink; nothing waits inside the kernel. */
  uint32_t n_ypeers, reserved0;
  p0p_buf* y_peers[7];
} p0p_gemm_args;

/* gemm(gpu, a) (src/ops/gemm.js:268-327): validates, picks the kernel, enqueues.  *flops = 2*M*N*K. */
int p0p_gemm(p0p_ctx* ctx, const p0p_gemm_args* a, double* flops);
/* the kernel family the last successful p0p_gemm used (P0P_K_*), and how many kernels it launched */
int p0p_last_kernel(const p0p_ctx* ctx);
uint64_t p0p_launch_count(const p0p_ctx* ctx);
/* Test convenience (no counterpart in the reference): the plan of the last call the tensor-core kernel served, so that tests can
 * tell which variant they covered.  out8 = {tokens per tile, k-steps of 64 k per pipeline step, lock-step rings (0 / 1), token
 * stages, operand stages, accumulator buffers, split-K units per tile, tiles left unsplit}.  After a call the decode kernel
 * served: {blocks, stages of 256 k in the call, k-block length, k-blocks, 1 if the blocks' ranges are whole units, units, 64-row
 * tiles, 0}. */
int p0p_last_plan(const p0p_ctx* ctx, uint32_t* out8);

/* No counterpart in the reference (a browser page never manages device memory).  The decode-sized q4 multiply
 * (M <= 16 tokens: y[M][N] fp16 = x[M][K] fp16 * W^T, W in q4g32a.t64) for callers that cannot allocate on the
 * device: hosts that hand a library no device memory at run time (a serving process that reserved the GPU for its
 * own arena, a plug-in under another runtime's allocator, a loop that cannot afford cudaMalloc's device-wide
 * synchronisation).  It takes no context: w, x, y are the caller's own device pointers (16-byte aligned), work is
 * enqueued on the caller's cudaStream_t, and it calls no allocating routine.  The kernel's split-K partial sums
 * live in an array of P0P_STATIC_SCRATCH_BYTES built into the library's device image (every GPU that loads the
 * library holds it until the process exits); a shape that needs more (8 * M * N * ceil(K / 2048) bytes; above 8 tokens
 * 8 * M * N * ceil(K / 1024))
 * is refused with a message in `err`.  All calls on a device share that array: calls whose kernels overlap on
 * the GPU race, so keep them in one stream order.  The first call on each device resolves the array's device
 * address; make it before any stream capture.  Conditions: 1 <= M <= 16, N % 64 == 0, K % 256 == 0.
 * Returns 0, < 0 for refused arguments, > 0 for a CUDA error; `err` (optional) receives the reason. */
#define P0P_STATIC_SCRATCH_BYTES (8u << 20)
int p0p_decode_q4_static(int device, void* stream, const void* w, const void* x, void* y, uint32_t M, uint32_t N, uint32_t K,
                         char* err, size_t err_cap);
/* No counterpart in the reference.  The kernels of p0p_decode_q4_static bound every wait they make; one that ran out leaves a
 * code in a word next to the built-in array and the results of that call are invalid.  This reads the word after the work
 * queued on `stream` (a 4-byte copy into a local variable plus a wait for the stream: it allocates nothing either).
 * Returns 0, -10 when a wait ran out (`err` names the code), > 0 for a CUDA error. */
int p0p_decode_q4_static_status(int device, void* stream, char* err, size_t err_cap);

/* Peer memory (no counterpart in the reference).  p0p_alloc_shareable is p0p_alloc (zeroed, 16-byte rounded, counted) on
 * memory that other processes can map: plain cudaMalloc instead of the stream-ordered pool, never recycled.
 * p0p_ipc_export writes the 64-byte CUDA IPC handle of such a buffer (whole allocation) to `handle64`; p0p_ipc_open maps the allocation another process exported (on another GPU of
 * the node) and returns it as a non-owning buffer of `bytes` bytes, unmapped by p0p_free.  Such a buffer is valid as a
 * y_peers entry of p0p_gemm; pass the handle bytes between processes by any means. */
int p0p_alloc_shareable(p0p_ctx* ctx, uint64_t bytes, p0p_buf** out);
int p0p_ipc_export(p0p_ctx* ctx, const p0p_buf* buf, void* handle64);
int p0p_ipc_open(p0p_ctx* ctx, const void* handle64, uint64_t bytes, p0p_buf** out);
/* Barrier between the ranks of one node, in stream order (no counterpart in the reference).  It is the "order the ranks"
 * step of the y_peers scheme: queued after a p0p_gemm that stored into the peers' buffers and before the call that reads
 * the gathered rows.  `flags` is this rank's flag block: P0P_PEER_FLAG_BYTES of zeroed memory from p0p_alloc_shareable, kept
 * for the life of the group; peer_flags[r] (r < world, the entry at `rank` is ignored) are the other ranks' blocks opened
 * with p0p_ipc_open.  The kernel stores this rank's barrier count into every rank's block (plain stores over NVLink) and polls
 * its OWN block until every rank has arrived; it never loads from a peer.  Every rank must issue the same sequence of
 * barriers.  The wait is bounded by `wait_cycles` SM clock cycles (0 = about two seconds): when it runs out, the next
 * p0p_sync / p0p_read returns -10 and the context stays usable.  May be recorded into a graph. */
#define P0P_PEER_FLAG_BYTES 256u
int p0p_peer_barrier(p0p_ctx* ctx, p0p_buf* flags, p0p_buf* const* peer_flags, uint32_t rank, uint32_t world, uint64_t wait_cycles);

/* attention, head_dim 128 (src/ops/attention.js:168-193; argument object types/index.d.ts `AttentionArgs`): the step after the
 * 'heads' projection.  Q [Hq][Lq][128] f16, K / V [Hkv][Lk][128] f16 head-major, O [Lq][ldo] f16 token-major at column h*128.
 * mode 0 none, 1 causal + valid length (key j visible to query i iff j <= min(i, nvalid-1)), 2 valid length (j < nvalid);
 * Hkv 0 = Hq, Lk 0 = Lq, ldo 0 = Hq*128, scale 0 = 1/sqrt(128), nvalid 0 = Lk.  *flops = 4*Lq*Lk*128*Hq (:192).
 * Calls with at least 128 queries per head run on the tensor-memory kernel (tcgen05), which first writes a transposed copy
 * of V into the context's scratch memory (sized on the first such call: not while recording a graph). */
typedef struct p0p_attn_args {
  uint32_t struct_size;
  uint32_t Hq, Hkv, Lq, Lk, ldo, mode, nvalid;
  float scale;
  p0p_buf *q, *k, *v, *o;
  uint64_t q_off, k_off, v_off, o_off;   /* bytes */
  uint32_t kernel;                       /* 0 = the library chooses; P0P_K_ATTN_WARP / P0P_K_ATTN_TMEM force one (tests).  A caller
                                            built before this field existed passes a smaller struct_size and gets 0. */
} p0p_attn_args;
int p0p_attention(p0p_ctx* ctx, const p0p_attn_args* args, double* flops);

/* Debug op: writes the fp16 tile values the kernels feed to the multiply, rows [r0, r0+nr) x all w_cols
 * columns, row-major into `out` (fp16).  path 0 = the fp32-FMA conversion, 1 = the packed half2 conversion
 * the tensor-core kernels use.  Both must equal f16(q*s+min) / f16(q*s) of docs/FORMAT.md bit for bit. */
int p0p_dequant(p0p_ctx* ctx, uint32_t enc, const p0p_buf* w, uint64_t w_off, uint32_t w_cols, uint32_t w_ld,
                uint32_t r0, uint32_t nr, uint32_t path, p0p_buf* out, uint64_t out_off);

/* rowstats (src/ops/misc.js:16-44): ST[(st_off+r)*2] = (mean, rstd) of fp32 rows; mode 0 LayerNorm, 1 RMS.
 * The producer of the `stats` input of the fused norm prologues. */
int p0p_rowstats(p0p_ctx* ctx, const p0p_buf* x, uint64_t x_off, uint32_t ld, uint32_t c0, uint32_t rows, uint32_t cols,
                 uint32_t mode, float eps, p0p_buf* st, uint32_t st_off);

/* pixstats (src/ops/video.js:301-318): r[ro + v] = rsqrt(sum_c x[v][c]^2 / C + eps) for the V voxels of an fp16 tensor [V][C]
 * (eps 0 = 1e-8).  The producer of `stats` for conv3's fused PixelNorm (`pn`). */
int p0p_pixstats(p0p_ctx* ctx, const p0p_buf* x, uint64_t x_off, uint32_t V, uint32_t C, float eps, p0p_buf* r, uint32_t ro);
/* gnPartial (src/ops/misc.js:50-73, 110-115): partial GroupNorm(32) statistics of an HWC fp16 tensor [pix][C], C a power of two
 * 32..512: one row of 32 x (count, mean, M2, 0) per 64 pixels into rows [wgOff, wgOff + ceil(pix / 64)) of `part` (512 bytes
 * per row, gnPartBytes).  Rows of separate calls merge, as in the reference.  *nwg (optional) = the number of rows written. */
int p0p_gn_partial(p0p_ctx* ctx, const p0p_buf* x, uint64_t x_off, uint32_t pix, uint32_t C, p0p_buf* part, uint32_t wgOff, uint32_t* nwg);
/* gnFinalize (src/ops/misc.js:75-104, 117-120): merges nwg partial rows (Chan's formula) and writes, at float offset ab_off of
 * `ab`, a[C] = gamma * rstd and b[C] = beta - mean * a, so that GroupNorm(x) = a * x + b per channel: the `pv` input of conv's
 * fused `gn`.  gamma / beta at float offsets g_off / b_off of `gb`; eps 0 = 1e-6. */
int p0p_gn_finalize(p0p_ctx* ctx, const p0p_buf* part, uint32_t nwg, uint32_t C, float eps, const p0p_buf* gb, uint32_t g_off, uint32_t b_off,
                    p0p_buf* ab, uint32_t ab_off);

/* ---- host-side helpers (no device work) ------------------------------------------------------------------ */
uint16_t p0p_f2h(float v);                                   /* f2h  (src/core/gpu.js:276-291) */
float    p0p_h2f(uint16_t h);                                /* h2f  (src/core/gpu.js:292-297) */
void p0p_to_f16(const float* src, uint16_t* dst, size_t n);  /* toF16   (src/core/gpu.js:298) */
void p0p_from_f16(const uint16_t* src, float* dst, size_t n);/* fromF16 (src/core/gpu.js:299) */
/* packQ4 / packQ8 (src/convert/encode.js:56-90): out holds rows*K*5/8 resp. rows*K*33/32 bytes; deq may be NULL. */
int p0p_pack_q4(const float* W, uint32_t rows, uint32_t K, uint8_t* out, float* deq);
int p0p_pack_q8(const float* W, uint32_t rows, uint32_t K, uint8_t* out, float* deq);
/* reorderConvRows (src/convert/encode.js:118-122) */
void p0p_reorder_conv_rows(const float* W, float* out, uint32_t rows, uint32_t I, uint32_t taps);
/* encodedBytes (src/convert/convert.js:11); enc 3 = f32 */
uint64_t p0p_encoded_bytes(uint32_t enc, uint64_t rows, uint64_t cols);
/* The byte range and row range of shard `rank` of `world` when a weight is split along N on 64-row tile
 * boundaries (docs/FORMAT.md:20, 41: a tile-aligned row range is one contiguous byte range).  rows must be a
 * multiple of 64*world for q4/q8.  No counterpart in the reference (it is single-device). */
int p0p_shard_rows(uint32_t enc, uint64_t rows, uint64_t cols, uint32_t rank, uint32_t world,
                   uint64_t* row0, uint64_t* nrows, uint64_t* byte_off, uint64_t* bytes);

uint32_t p0p_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* P0P_H */
