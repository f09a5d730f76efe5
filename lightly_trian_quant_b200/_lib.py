"""ctypes binding of libkf_b200.so (the C-ABI declared in include/kf_b200.h).

The library is the only compute path: if it is missing or fails to load, importing the operators raises
(there is no CPU or PyTorch fallback).
"""
from __future__ import annotations

import ctypes as C
import re
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "libkf_b200.so"
HEADER = PKG.parent / "include" / "kf_b200.h"
HEADERS = sorted((PKG.parent / "include").glob("*.h"))

KF_FMT = {"mx8": 0, "nv4": 1, "mx4": 2, "bf16": 3}
KF_DT = {"f32": 0, "bf16": 1, "f16": 2}
KF_Q_GELU, KF_Q_ROUND_BF16, KF_Q_RECIP_DIV, KF_Q_FAST_NV4 = 1, 2, 4, 64

KF_EPI = {"plain": 0, "res": 1, "rope": 2, "quant": 3}
KF_G_GELU, KF_G_ROUND_BF16, KF_G_PRE_ROUND_BF16, KF_G_ROPE_HALF = 8, 16, 32, 128


class GemmParams(C.Structure):
    """mirror of kf_gemm_params (include/kf_b200.h)."""
    _fields_ = [("fmt", C.c_int), ("epi", C.c_int), ("M", C.c_int), ("N", C.c_int), ("K", C.c_int), ("out_dtype", C.c_int),
                ("flags", C.c_int), ("Ntok", C.c_int), ("prefix", C.c_int), ("H", C.c_int), ("out_fmt", C.c_int),
                ("A", C.c_void_p), ("SFA", C.c_void_p), ("W", C.c_void_p), ("SFW", C.c_void_p), ("ts_a", C.c_void_p),
                ("ts_w", C.c_void_p), ("bias", C.c_void_p), ("gamma", C.c_void_p), ("R", C.c_void_p), ("sin", C.c_void_p),
                ("cos", C.c_void_p), ("C", C.c_void_p), ("Qo", C.c_void_p), ("SFo", C.c_void_p), ("tso", C.c_void_p),
                ("out_row_group", C.c_int), ("out_row_stride", C.c_int), ("out_row_offset", C.c_int), ("y_dbg", C.c_void_p), ("batch", C.c_int), ("a_rows_per_batch", C.c_int), ("w_rows_per_batch", C.c_int)]


_lib = None


class KfError(RuntimeError):
    pass


def declared_symbols() -> list[str]:
    """every function name the headers under include/ declare."""
    text = re.sub(r"/\*.*?\*/", "", "\n".join(h.read_text() for h in HEADERS), flags=re.S)
    return sorted(set(re.findall(r"\b(kf_[a-z0-9_]+)\s*\(", text)))


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise KfError(f"{LIB_PATH} not built: run `python -m lightly_trian_quant_b200.build` (no fallback path exists)")
        L = C.CDLL(str(LIB_PATH))
        L.kf_version.restype = C.c_char_p
        L.kf_last_error_string.restype = C.c_char_p
        L.kf_sf_bytes.restype = C.c_int64
        L.kf_sf_bytes.argtypes = [C.c_int64, C.c_int64, C.c_int]
        vp, i32, i64, f32 = C.c_void_p, C.c_int, C.c_int64, C.c_float
        sigs = {
            "kf_quant_rows": [i32, i32, vp, i64, i32, i32, vp, vp, i32, vp, vp, vp],
            "kf_ln_quant": [i32, vp, vp, vp, f32, i32, i32, vp, i32, vp, vp, vp, vp],
            "kf_ln_rows": [vp, vp, vp, f32, i32, i32, i32, vp, vp],
            "kf_gemm_bs": [C.POINTER(GemmParams), vp],
            "kf_check_device_error": [],
            "kf_attn_fwd": [i32, vp, vp, i32, i32, i32, f32, vp],
            "kf_tensor_peak_probe": [i32, i32, i32, i32, C.POINTER(C.c_double), vp],
            "kf_fill_rate_probe": [vp, C.c_int64, i32, i32, C.POINTER(C.c_double), vp],
            "kf_selftest_rcp": [i32, vp, vp],
            "kf_attn_fwd_quant": [i32, vp, i32, i32, i32, f32, i32, vp, vp, vp, i32, vp],
            "kf_ln_tail": [vp, vp, vp, f32, i32, i32, i32, i32, i32, vp, vp, vp, vp, i32, vp, vp],
            "kf_broadcast_rows": [vp, vp, i32, i32, i32, i64, i64, vp],
            "kf_im2col_patch16": [vp, vp, i32, i32, vp],
            "kf_patch_embed_static": [vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, vp],
            "kf_dw_ln": [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, f32, i32, vp],
            "kf_semantic": [vp, vp, i32, i32, i32, i32, vp, vp, vp],
            "kf_resize_norm": [vp, vp, i32, i32, i32, i32, C.POINTER(C.c_float), C.POINTER(C.c_float), vp],
        }
        for name, args in sigs.items():
            fn = getattr(L, name)
            fn.restype = C.c_int
            fn.argtypes = args
        _lib = L
    return _lib


def check(status: int, what: str) -> None:
    if status != 0:
        msg = lib().kf_last_error_string().decode()
        raise KfError(f"{what} failed with status {status}: {msg}")
