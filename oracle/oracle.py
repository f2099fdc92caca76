"""ctypes front end of the CPU oracle (TEST INFRASTRUCTURE ONLY).

Loads ``libvelox_oracle.so`` (built by ``make -C oracle``) and exposes numpy-facing helpers.
Only tests, the smoke check and the benchmark's CPU-baseline leg import this module; the
product package never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libvelox_oracle.so")

FMT_F32, FMT_BF16, FMT_FP8, FMT_NVFP4, FMT_Q4K = 0, 1, 2, 3, 17
ACT_EXACT, ACT_BF16, ACT_FP8_ROW, ACT_NVFP4 = 0, 1, 2, 3


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "velox_oracle.c")
    stale = (not os.path.exists(_LIB_PATH)) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src)
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B", "libvelox_oracle.so"], check=True,
                       capture_output=True)
    return _LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB_PATH)
        sz, f32, u8p, f32p = C.c_size_t, C.c_float, C.c_void_p, C.c_void_p
        L.vo_bf16_to_f32.restype = f32
        L.vo_bf16_to_f32.argtypes = [C.c_uint16]
        L.vo_f32_to_bf16.restype = C.c_uint16
        L.vo_f32_to_bf16.argtypes = [f32]
        L.vo_f16_to_f32.restype = f32
        L.vo_f16_to_f32.argtypes = [C.c_uint16]
        L.vo_f32_to_f16.restype = C.c_uint16
        L.vo_f32_to_f16.argtypes = [f32]
        L.vo_e4m3fn_to_f32.restype = f32
        L.vo_e4m3fn_to_f32.argtypes = [C.c_uint8]
        L.vo_e2m1_to_f32.restype = f32
        L.vo_e2m1_to_f32.argtypes = [C.c_uint8]
        for name in ("vo_f32_to_e4m3fn_lower", "vo_f32_to_e4m3fn", "vo_f32_to_e2m1"):
            getattr(L, name).restype = C.c_uint8
            getattr(L, name).argtypes = [f32]
        L.vo_align256.restype = sz
        L.vo_align256.argtypes = [sz]
        L.vo_nvfp4_scale_offset.restype = sz
        L.vo_nvfp4_scale_offset.argtypes = [sz, sz, sz]
        L.vo_check_shape.restype = C.c_int
        L.vo_check_shape.argtypes = [C.c_int, sz, sz]
        L.vo_payload_bytes.restype = sz
        L.vo_payload_bytes.argtypes = [C.c_int, sz, sz]
        L.vo_q4k_decode_block.argtypes = [u8p, f32p]
        L.vo_decode_rows.restype = C.c_int
        L.vo_decode_rows.argtypes = [C.c_int, u8p, sz, sz, sz, sz, sz, f32p]
        for name in ("vo_encode_nvfp4_ref", "vo_encode_nvfp4_rne", "vo_encode_fp8_row",
                     "vo_encode_q4k"):
            getattr(L, name).argtypes = [f32p, sz, sz, u8p]
        L.vo_quantize_activations.argtypes = [f32p, sz, sz, C.c_int, f32]
        L.vo_act_codes_fp8.argtypes = [f32p, sz, sz, u8p, f32p]
        L.vo_act_codes_nvfp4.argtypes = [f32p, sz, sz, f32, u8p, u8p]
        L.vo_matmul.argtypes = [f32p, f32p, f32p, sz, sz, sz, C.c_int]
        L.vo_linear.restype = C.c_int
        L.vo_linear.argtypes = [f32p, sz, u8p, sz, C.c_int, sz, sz, sz, sz, sz, f32p, sz, C.c_int]
        L.vo_silu_mul.argtypes = [f32p, f32p, sz]
        L.vo_swiglu.argtypes = [f32p, sz, sz, sz, sz, sz, f32p]
        L.vo_add.argtypes = [f32p, f32p, sz]
        L.vo_rms_norm.argtypes = [f32p, f32p, f32p, sz, sz, f32, C.c_int]
        L.vo_rng_new.argtypes = [C.c_void_p, C.c_uint64]
        L.vo_rng_next.restype = C.c_uint64
        L.vo_rng_next.argtypes = [C.c_void_p]
        L.vo_rng_uniform.restype = f32
        L.vo_rng_uniform.argtypes = [C.c_void_p]
        L.vo_rng_vec.argtypes = [C.c_void_p, sz, f32, f32p]
        L.vo_random_weight.restype = C.c_int
        L.vo_random_weight.argtypes = [C.c_void_p, C.c_int, sz, sz, u8p]
        L.vo_kat_q4k_blocks.argtypes = [C.c_uint64, u8p]
        for name in ("vo_max_err", "vo_max_abs_diff"):
            getattr(L, name).restype = C.c_double
            getattr(L, name).argtypes = [f32p, f32p, sz]
        L.vo_rms.restype = C.c_double
        L.vo_rms.argtypes = [f32p, sz]
        _lib = L
    return _lib


def _p(a: np.ndarray) -> int:
    return a.ctypes.data


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _u8(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.uint8)


class Rng:
    """The reference's xorshift generator (crates/velox-core/src/rng.rs)."""

    def __init__(self, seed: int):
        self._s = C.c_uint64(0)
        lib().vo_rng_new(C.byref(self._s), seed)

    def next_u64(self) -> int:
        return lib().vo_rng_next(C.byref(self._s))

    def uniform(self) -> float:
        return lib().vo_rng_uniform(C.byref(self._s))

    def vec(self, n: int, scale: float) -> np.ndarray:
        out = np.empty(n, dtype=np.float32)
        lib().vo_rng_vec(C.byref(self._s), n, scale, _p(out))
        return out

    def random_weight(self, fmt: int, n: int, k: int) -> np.ndarray:
        out = np.zeros(payload_bytes(fmt, n, k), dtype=np.uint8)
        rc = lib().vo_random_weight(C.byref(self._s), fmt, n, k, _p(out))
        if rc != 0:
            raise ValueError(f"random_weight: format {fmt} not covered")
        return out


def payload_bytes(fmt: int, n: int, k: int) -> int:
    return lib().vo_payload_bytes(fmt, n, k)


def check_shape(fmt: int, n: int, k: int) -> int:
    return lib().vo_check_shape(fmt, n, k)


def nvfp4_scale_offset(n: int, g: int, k: int) -> int:
    return lib().vo_nvfp4_scale_offset(n, g, k)


def decode_rows(fmt: int, payload: np.ndarray, n: int, k: int, row_begin: int, rows: int):
    payload = _u8(payload)
    out = np.empty((rows, k), dtype=np.float32)
    rc = lib().vo_decode_rows(fmt, _p(payload), payload.size, n, k, row_begin, rows, _p(out))
    if rc != 0:
        raise ValueError(f"decode_rows: shape error ({rc})")
    return out


def _encode(fn: str, fmt: int, w: np.ndarray) -> np.ndarray:
    w = _f32(w)
    n, k = w.shape
    if check_shape(fmt, n, k) != 0:
        raise ValueError("illegal shape for format")
    out = np.zeros(payload_bytes(fmt, n, k), dtype=np.uint8)
    getattr(lib(), fn)(_p(w), n, k, _p(out))
    return out


def encode_nvfp4_ref(w):
    return _encode("vo_encode_nvfp4_ref", FMT_NVFP4, w)


def encode_nvfp4_rne(w):
    return _encode("vo_encode_nvfp4_rne", FMT_NVFP4, w)


def encode_fp8_row(w):
    return _encode("vo_encode_fp8_row", FMT_FP8, w)


def encode_q4k(w):
    return _encode("vo_encode_q4k", FMT_Q4K, w)


def quantize_activations(x: np.ndarray, k: int, act: int, divisor: float = 0.0) -> np.ndarray:
    out = _f32(x).copy()
    rows = out.size // k
    lib().vo_quantize_activations(_p(out), rows, k, act, divisor)
    return out


def act_codes_fp8(x: np.ndarray):
    x = _f32(x)
    rows, k = x.shape
    codes = np.empty((rows, k), dtype=np.uint8)
    scales = np.empty(rows, dtype=np.float32)
    lib().vo_act_codes_fp8(_p(x), rows, k, _p(codes), _p(scales))
    return codes, scales


def act_codes_nvfp4(x: np.ndarray, divisor: float):
    x = _f32(x)
    rows, k = x.shape
    codes = np.empty((rows, k // 2), dtype=np.uint8)
    scales = np.empty((rows, k // 16), dtype=np.uint8)
    lib().vo_act_codes_nvfp4(_p(x), rows, k, divisor, _p(codes), _p(scales))
    return codes, scales


def matmul(x, w, threads: int = 0):
    x, w = _f32(x), _f32(w)
    m, k = x.shape
    n = w.shape[0]
    y = np.empty((m, n), dtype=np.float32)
    lib().vo_matmul(_p(x), _p(w), _p(y), m, n, k, threads)
    return y


def linear(x, payload, fmt, n, k, row_begin, rows, m, threads: int = 0,
           act: int = ACT_EXACT, divisor: float = 0.0):
    """The oracle's ``linear`` on the view, after rounding x as ``act`` declares."""
    x = _f32(x).reshape(-1)
    if act != ACT_EXACT:
        x = quantize_activations(x[: m * k], k, act, divisor)
    payload = _u8(payload)
    y = np.empty(m * rows if m * rows else 1, dtype=np.float32)
    rc = lib().vo_linear(_p(x), x.size, _p(payload), payload.size, fmt, n, k, row_begin, rows, m,
                         _p(y), m * rows, threads)
    if rc != 0:
        raise ValueError(f"linear: shape error ({rc})")
    return y.reshape(m, rows)


def linear_rc(x_len, payload_len, fmt, n, k, row_begin, rows, m, y_len) -> int:
    """Return code of the oracle's shape check alone (buffers are dummies of the given sizes)."""
    x = np.zeros(max(x_len, 1), dtype=np.float32)
    p = np.zeros(max(payload_len, 1), dtype=np.uint8)
    y = np.zeros(max(y_len, 1), dtype=np.float32)
    return lib().vo_linear(_p(x), x_len, _p(p), payload_len, fmt, n, k, row_begin, rows, m,
                           _p(y), y_len, 1)


def silu_mul(gate, up):
    g = _f32(gate).copy()
    u = _f32(up)
    lib().vo_silu_mul(_p(g), _p(u), g.size)
    return g


def swiglu(src, rows, src_cols, gate, up, width):
    src = _f32(src)
    out = np.empty((rows, width), dtype=np.float32)
    lib().vo_swiglu(_p(src), rows, src_cols, gate, up, width, _p(out))
    return out


def rms_norm(x, weight, eps: float, offset: bool = False):
    x, weight = _f32(x), _f32(weight)
    rows, dim = x.shape
    y = np.empty_like(x)
    lib().vo_rms_norm(_p(x), _p(weight), _p(y), rows, dim, eps, int(offset))
    return y


def max_err(got, want) -> float:
    got, want = _f32(got).reshape(-1), _f32(want).reshape(-1)
    if got.size != want.size:
        return float("inf")
    return lib().vo_max_err(_p(got), _p(want), got.size)


def max_abs_diff(got, want) -> float:
    got, want = _f32(got).reshape(-1), _f32(want).reshape(-1)
    return lib().vo_max_abs_diff(_p(got), _p(want), got.size)


def rms(v) -> float:
    v = _f32(v).reshape(-1)
    return lib().vo_rms(_p(v), v.size)


def kat_q4k_blocks(seed: int) -> np.ndarray:
    out = np.zeros(288, dtype=np.uint8)
    lib().vo_kat_q4k_blocks(seed, _p(out))
    return out
