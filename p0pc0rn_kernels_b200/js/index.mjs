// Drop-in for the reference's src/core/gpu.js + src/ops/gemm.js on a B200: the same names and argument objects
// (`createGpu`, `gpu.buffer / upload / read / free / done`, `gemm(gpu, args)`, `toF16 / fromF16 / f2h / h2f`,
// `packQ4 / packQ8`), marshalled into the native addon (addon.cc) over the C ABI of include/p0p.h.
// UNVERIFIED where this project is built (no Node.js there); the verified boundary is the C ABI, exercised by
// the Python mirror of this same API.
import { createRequire } from 'node:module';
const addon = createRequire(import.meta.url)('./build/Release/p0p_addon.node');

export class GpuError extends Error {}
const ENC = { 'q4g32a.t64': 0, 'q8g64s.t64': 1, f16: 2 };
const XMODE = { f16: 0, lnmod: 1, rms: 2, conv: 3, conv3: 4 };
const EPI = { f16: 0, f32: 1, resadd: 2, swiglu: 3, heads: 4, bias: 5, onormgate: 6 };

class Buf { constructor(handle, size, label) { this.handle = handle; this._pf = size; this.size = size; this.label = label; } }

export class Gpu {
  constructor(opts = {}) {
    this.opts = Object.assign({ powerPreference: 'high-performance', wantSubgroups: true, wantF16: true, maxDispatchSeconds: 0.2, device: 0 }, opts);
    try { this._h = addon.open(this.opts.device); } catch (e) { throw new GpuError(e.message); }
    this.bufs = new Set(); this.lostInfo = null; this.tune = null;
    this.rate = { mm: 1e15, mm32: 1e15, mm16: 1e15, attn: 0.5e15, mem: 6.5e12 };   // dispatch sizing does not exist on CUDA; callers read the fields
    this.f16 = true; this.subgroups = true; this.sgMin = 32; this.sgMax = 32; this.sgOK16 = true;
    this.info = { vendor: 'nvidia', architecture: 'sm_100', device: 'B200', description: 'B200' };
    this.limits = { maxStorageBufferBindingSize: Number.MAX_SAFE_INTEGER, maxComputeWorkgroupStorageSize: 232448 };
    const self = this;
    this.device = { queue: { writeBuffer(buf, dstOff, data, srcOff = 0, size = undefined) {
      // a typed-array source counts srcOff / size in ELEMENTS (the WebGPU rule the reference's ring test relies on)
      const view = ArrayBuffer.isView(data) ? data.subarray(srcOff, size === undefined ? undefined : srcOff + size) : new Uint8Array(data, srcOff, size);
      self._call(() => addon.write(self._h, buf.handle, dstOff, view));
    } } };
  }
  _call(fn) { try { return fn(); } catch (e) { if (e.code === 'GpuError') { this.lostInfo = { reason: 'cuda', message: e.message }; if (this.opts.onLost) this.opts.onLost(this.lostInfo); throw new GpuError(e.message); } throw e; } }
  get lost() { return !!this.lostInfo; }
  describe() { return Object.assign({}, this.info, { f16: true, subgroups: true, sgMin: 32, sgMax: 32 }); }
  buffer(size, label = '') { const r = this._call(() => addon.alloc(this._h, size)); const b = new Buf(r.handle, r.size, label); this.bufs.add(b); return b; }
  free(b) { if (!b || !this.bufs.has(b)) return; this.bufs.delete(b); addon.free(this._h, b.handle); }
  freeAll() { for (const b of Array.from(this.bufs)) this.free(b); }
  upload(data, label = '', dst = null, dstOff = 0) {
    const u8 = data instanceof ArrayBuffer ? new Uint8Array(data) : new Uint8Array(data.buffer, data.byteOffset, data.byteLength);
    const b = dst || this.buffer(u8.byteLength, label);
    if (u8.byteLength) this._call(() => addon.write(this._h, b.handle, dstOff, u8));
    return b;
  }
  async read(buf, off = 0, size = null) { return this._call(() => addon.read(this._h, buf.handle, off, size == null ? buf._pf - off : size)); }
  async done() { if (this.lost) throw new GpuError('GPU device lost: ' + JSON.stringify(this.lostInfo)); this._call(() => addon.sync(this._h)); }
  cap(kind = 'mm') { return this.rate[kind] * this.opts.maxDispatchSeconds; }
}
export async function createGpu(opts = {}) { return new Gpu(opts); }

export const f2h = (v) => addon.f2h(v);
export const h2f = (h) => addon.h2f(h);
export function toF16(a) { const o = new Uint16Array(a.length); for (let i = 0; i < a.length; i++) o[i] = addon.f2h(a[i]); return o; }
export function fromF16(u) { const o = new Float32Array(u.length); for (let i = 0; i < u.length; i++) o[i] = addon.h2f(u[i]); return o; }
export const packQ4 = (W, rows, K, deq = null) => new Uint8Array(addon.packQ(4, W, rows, K, deq));
export const packQ8 = (W, rows, K, deq = null) => new Uint8Array(addon.packQ(8, W, rows, K, deq));
export const DEFAULT_TILE = { BM: 64, BN: 128 };

/** gemm(gpu, a): the reference's argument object (src/ops/gemm.js:259-267), flattened to p0p_gemm_args; returns 2*M*N*K */
export function gemm(gpu, a) {
  const enc = ENC[a.w.enc];
  if (enc === undefined) throw new Error('gemm: unsupported weight encoding ' + a.w.enc);
  const cv = a.conv || null, h = a.heads || {}, epi = a.epi || 'f16';
  let flags = 0;
  if (a.ev && epi === 'resadd') flags |= 1; if (a.res) flags |= 2; if (a.store) flags |= 4; if (cv && cv.gn) flags |= 8; if (cv && cv.up2) flags |= 16;
  if (cv && cv.pn) flags |= 32; if (a.bv) flags |= 64; if (a.act === 'gelu') flags |= 128; if (h.ropeMode === 'half') flags |= 256;
  const t = a.tile || {};
  if (a.tile && (t.BM % 32 || t.BN % 64 || (t.BM / 8) * (t.BN / 8) > 256)) throw new Error('bad tile ' + t.BM + 'x' + t.BN);
  const flat = {
    enc, xmode: cv ? (cv.kind === 'conv3' ? 4 : 3) : XMODE[a.x.mode || 'f16'], epi: EPI[epi], flags, M: a.M, N: a.N, K: a.K,
    ldx: a.x.ld || a.K, kx0: a.x.k0 || 0, wr0: a.wr0 || 0, wr1: a.wr1 || 0, wk0: a.wk0 || 0, w_rows: a.w.rows, w_cols: a.w.cols, w_ld: a.w.ld || 0,
    ldy: a.y.ld || a.N, ny0: a.y.n0 || 0, rowOff: h.rowOff || 0, Ltot: h.Ltot || 0, Hq: h.Hq || 0, Hkv: h.Hkv || 0, eps: h.eps || 1e-6,
    pv_off: a.pv ? a.pv.off || 0 : 0, pv_stride: a.pv ? a.pv.stride || 0 : 0, ev_off: a.ev ? a.ev.off || 0 : 0, st_off: a.stats ? a.stats.off || 0 : 0,
    bv_off: a.bv ? a.bv.off || 0 : 0, bv_up: a.bv ? a.bv.up || 0 : 0,
    Hi: cv ? cv.Hi : 0, Wi: cv ? cv.Wi : 0, Ci: cv ? cv.Ci : 0, Ho: cv ? cv.Ho : 0, Wo: cv ? cv.Wo : 0, stride: cv ? cv.stride || 1 : 1,
    padT: cv ? cv.padT || 0 : 0, padL: cv ? cv.padL || 0 : 0, ks: cv ? cv.ks || 1 : 1, tile_bm: t.BM || 0, tile_bn: t.BN || 0,
    acc_f16: (a.acc || (gpu.tune && gpu.tune.acc)) === 'f16' ? 1 : 0,
    x: a.x.buf.handle, w: a.w.buf.handle, y: a.y.buf.handle, st: a.stats && a.stats.buf.handle, pv: a.pv && a.pv.buf.handle, ev: a.ev && a.ev.buf.handle,
    bv: a.bv && a.bv.buf.handle, rp: h.rope && h.rope.buf.handle, gt: a.gt && a.gt.buf.handle,
    x_off: a.x.off || 0, w_off: a.w.off || 0, y_off: a.y.off || 0, w_bytes: a.w.bytes || 0, x_size: a.x.size || 0, y_size: a.y.size || 0,
    y_peers: a.y.peers ? a.y.peers.map((b) => b.handle) : undefined,   // multi-GPU extension: other ranks' copies of y (not in the reference)
  };
  return gpu._call(() => addon.gemm(gpu._h, flat));
}
