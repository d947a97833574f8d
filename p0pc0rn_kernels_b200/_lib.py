"""ctypes binding of ``libp0p.so`` (the C ABI declared in ``include/p0p.h``).

There is no fallback: when the library is missing or does not load, importing this module raises."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libp0p.so")

# every symbol include/p0p.h declares
SYMBOLS = [
    "p0p_open", "p0p_close", "p0p_last_error", "p0p_status", "p0p_describe", "p0p_stream",
    "p0p_alloc", "p0p_wrap", "p0p_free", "p0p_drain_pool", "p0p_pool_stats", "p0p_reset_peak", "p0p_buf_size", "p0p_buf_ptr",
    "p0p_write", "p0p_read", "p0p_clear", "p0p_copy", "p0p_sync", "p0p_host_alloc", "p0p_host_free",
    "p0p_capture_begin", "p0p_capture_end", "p0p_graph_launch", "p0p_graph_free",
    "p0p_decode_q4_static", "p0p_decode_q4_static_status", "p0p_alloc_shareable", "p0p_ipc_export", "p0p_ipc_open", "p0p_peer_barrier",
    "p0p_gemm", "p0p_attention", "p0p_last_kernel", "p0p_launch_count", "p0p_last_plan", "p0p_dequant", "p0p_rowstats",
    "p0p_pixstats", "p0p_gn_partial", "p0p_gn_finalize",
    "p0p_f2h", "p0p_h2f", "p0p_to_f16", "p0p_from_f16", "p0p_pack_q4", "p0p_pack_q8", "p0p_reorder_conv_rows",
    "p0p_encoded_bytes", "p0p_shard_rows", "p0p_abi_version",
]

ENC = {"q4g32a.t64": 0, "q8g64s.t64": 1, "f16": 2}
XMODE = {"f16": 0, "lnmod": 1, "rms": 2, "conv": 3, "conv3": 4}
EPI = {"f16": 0, "f32": 1, "resadd": 2, "swiglu": 3, "heads": 4, "bias": 5, "onormgate": 6}
F_GATE, F_RES, F_STORE, F_GN, F_UP2, F_PN, F_BIAS, F_GELU, F_ROPE_HALF = 1, 2, 4, 8, 16, 32, 64, 128, 256
K_AUTO, K_GENERIC, K_DECODE, K_UMMA = 0, 1, 2, 3
KERNEL_NAMES = {0: "auto", 1: "generic", 2: "decode", 3: "umma", 16: "attention (warp-level)", 17: "attention (tcgen05)"}


class Opts(C.Structure):
    _fields_ = [("struct_size", C.c_uint32), ("flags", C.c_uint32), ("stream", C.c_void_p)]


class GemmArgs(C.Structure):
    _fields_ = ([(n, C.c_uint32) for n in ("struct_size", "enc", "xmode", "epi", "flags", "M", "N", "K", "ldx", "kx0", "wr0", "wr1", "wk0",
                                            "w_rows", "w_cols", "w_ld", "ldy", "ny0", "rowOff", "Ltot", "Hq", "Hkv")]
                + [("eps", C.c_float)]
                + [(n, C.c_uint32) for n in ("pv_off", "pv_stride", "ev_off", "st_off", "bv_off", "bv_up", "Hi", "Wi", "Ci", "Ho", "Wo",
                                              "stride", "padT", "padL", "ks", "tile_bm", "tile_bn", "acc_f16", "force_kernel")]
                + [(n, C.c_void_p) for n in ("x", "w", "y", "st", "pv", "ev", "bv", "rp", "gt")]
                + [(n, C.c_uint64) for n in ("x_off", "w_off", "y_off", "w_bytes", "x_size", "y_size")]
                + [("n_ypeers", C.c_uint32), ("reserved0", C.c_uint32), ("y_peers", C.c_void_p * 7)])


class AttnArgs(C.Structure):
    _fields_ = ([(n, C.c_uint32) for n in ("struct_size", "Hq", "Hkv", "Lq", "Lk", "ldo", "mode", "nvalid")] + [("scale", C.c_float)]
                + [(n, C.c_void_p) for n in ("q", "k", "v", "o")] + [(n, C.c_uint64) for n in ("q_off", "k_off", "v_off", "o_off")] + [("kernel", C.c_uint32)])


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is missing: build it with `python p0pc0rn_kernels_b200/build.py` (needs nvcc); there is no CPU fallback")
    L = C.CDLL(LIB_PATH)
    vp, u32, u64, i = C.c_void_p, C.c_uint32, C.c_uint64, C.c_int
    sig = {
        "p0p_open": (i, [i, C.POINTER(Opts), C.POINTER(vp)]), "p0p_close": (i, [vp]), "p0p_last_error": (C.c_char_p, [vp]),
        "p0p_status": (i, [vp]), "p0p_describe": (C.c_size_t, [vp, C.c_char_p, C.c_size_t]), "p0p_stream": (vp, [vp]),
        "p0p_alloc": (i, [vp, u64, C.POINTER(vp)]), "p0p_wrap": (i, [vp, vp, u64, C.POINTER(vp)]), "p0p_free": (i, [vp, vp]),
        "p0p_drain_pool": (i, [vp]), "p0p_pool_stats": (i, [vp, C.POINTER(u64)]), "p0p_reset_peak": (i, [vp]),
        "p0p_buf_size": (u64, [vp]), "p0p_buf_ptr": (vp, [vp]),
        "p0p_write": (i, [vp, vp, u64, vp, u64]), "p0p_read": (i, [vp, vp, u64, vp, u64]), "p0p_clear": (i, [vp, vp, u64, u64]),
        "p0p_copy": (i, [vp, vp, u64, vp, u64, u64]), "p0p_sync": (i, [vp]), "p0p_host_alloc": (i, [vp, u64, C.POINTER(vp)]), "p0p_host_free": (i, [vp, vp]),
        "p0p_capture_begin": (i, [vp]), "p0p_capture_end": (i, [vp, C.POINTER(vp)]), "p0p_graph_launch": (i, [vp, vp]), "p0p_graph_free": (i, [vp, vp]),
        "p0p_decode_q4_static": (i, [i, vp, vp, vp, vp, u32, u32, u32, C.c_char_p, C.c_size_t]),
        "p0p_decode_q4_static_status": (i, [i, vp, C.c_char_p, C.c_size_t]),
        "p0p_peer_barrier": (i, [vp, vp, C.POINTER(vp), u32, u32, u64]),
        "p0p_pixstats": (i, [vp, vp, u64, u32, u32, C.c_float, vp, u32]),
        "p0p_gn_partial": (i, [vp, vp, u64, u32, u32, vp, u32, C.POINTER(u32)]),
        "p0p_gn_finalize": (i, [vp, vp, u32, u32, C.c_float, vp, u32, u32, vp, u32]),
        "p0p_alloc_shareable": (i, [vp, u64, C.POINTER(vp)]), "p0p_ipc_export": (i, [vp, vp, vp]), "p0p_ipc_open": (i, [vp, vp, u64, C.POINTER(vp)]),
        "p0p_gemm": (i, [vp, C.POINTER(GemmArgs), C.POINTER(C.c_double)]), "p0p_attention": (i, [vp, C.POINTER(AttnArgs), C.POINTER(C.c_double)]), "p0p_last_kernel": (i, [vp]), "p0p_launch_count": (u64, [vp]), "p0p_last_plan": (i, [vp, C.POINTER(C.c_uint32)]),
        "p0p_dequant": (i, [vp, u32, vp, u64, u32, u32, u32, u32, u32, vp, u64]),
        "p0p_rowstats": (i, [vp, vp, u64, u32, u32, u32, u32, u32, C.c_float, vp, u32]),
        "p0p_f2h": (C.c_uint16, [C.c_float]), "p0p_h2f": (C.c_float, [C.c_uint16]),
        "p0p_to_f16": (None, [vp, vp, C.c_size_t]), "p0p_from_f16": (None, [vp, vp, C.c_size_t]),
        "p0p_pack_q4": (i, [vp, u32, u32, vp, vp]), "p0p_pack_q8": (i, [vp, u32, u32, vp, vp]),
        "p0p_reorder_conv_rows": (None, [vp, vp, u32, u32, u32]), "p0p_encoded_bytes": (u64, [u32, u64, u64]),
        "p0p_shard_rows": (i, [u32, u64, u64, u32, u32, C.POINTER(u64), C.POINTER(u64), C.POINTER(u64), C.POINTER(u64)]),
        "p0p_abi_version": (u32, []),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype = res; fn.argtypes = args
    return L


lib = _load()
