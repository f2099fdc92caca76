"""Loader of the CUDA library (``libvelox_sm100.so``) and its ctypes signatures.

There is no CPU fallback: if the library is missing or fails to load, importing an operator
raises. ``build()`` compiles it in-tree with nvcc for sm_100a.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libvelox_sm100.so")
CSRC = os.path.join(_HERE, "csrc")

ERR_UNSUPPORTED = -1
ERR_SHAPE = -2


class View(C.Structure):
    """``velox_sm100_view`` (include/velox_sm100.h)."""

    _fields_ = [
        ("w", C.c_void_p),
        ("format", C.c_int32),
        ("policy", C.c_int32),
        ("n", C.c_int64),
        ("k", C.c_int64),
        ("row_begin", C.c_int64),
        ("rows", C.c_int32),
        ("divisor", C.c_float),
    ]


class PartQ4(C.Structure):
    """velox_sm100_part_q4."""
    _fields_ = [("view", View), ("yb", C.c_void_p), ("out_codes", C.c_void_p), ("out_atoms", C.c_void_p),
                ("out_divisor", C.c_float)]


class TpSync(C.Structure):
    """``velox_sm100_tp_sync``: the flags one launch of a tensor-parallel step waits for and raises."""
    _fields_ = [("flag_tables", C.c_uint64 * 8), ("epoch", C.c_uint64), ("n", C.c_int32), ("rank", C.c_int32),
                ("wait_phase", C.c_int32), ("signal_phase", C.c_int32)]


class Part(C.Structure):
    """``velox_sm100_part`` (include/velox_sm100.h)."""

    _fields_ = [("view", View), ("y", C.c_void_p), ("ld", C.c_int64), ("col", C.c_int64)]


# name -> (restype, argtypes); every symbol include/velox_sm100.h declares
_VP, _I, _LL, _F = C.c_void_p, C.c_int, C.c_longlong, C.c_float
_PV = C.POINTER(View)
SIGNATURES = {
    "velox_sm100_abi_version": (_I, []),
    "velox_sm100_set_stream": (_I, [_VP]),
    "velox_sm100_debug_status": (_I, []),
    "velox_sm100_debug_status_reset": (_I, []),
    "velox_sm100_tp_step_begin": (_I, [_VP]),
    "velox_sm100_tp_wait": (_I, [_VP]),
    "velox_sm100_tp_signal": (_I, [_VP]),
    "velox_sm100_tp_barrier": (_I, [_VP]),
    "velox_sm100_tp_set_wait_limit_ms": (_I, [_I]),
    "velox_sm100_tp_linears_q4": (_I, [_VP, _VP, _F, _VP, _I, _I, _VP]),
    "velox_sm100_tp_linear_swiglu_q4_to_q4": (_I, [_VP, _VP, _F, _PV, _PV, _I, _VP, _VP, _VP, _F, _VP]),
    "velox_sm100_launch_count": (C.c_longlong, []),
    "velox_sm100_timing_enable": (_I, [_I]),
    "velox_sm100_timing_collect": (_I, [_VP, _VP, _I]),
    "velox_sm100_add_bf16_rms_norm_twin": (_I, [_VP, _VP, _VP, _VP, _VP, _I, _I, _F, _I]),
    "velox_sm100_add_bf16": (_I, [_VP, _VP, _LL]),
    "velox_sm100_add_rms_norm_q4": (_I, [_VP, _VP, _VP, _VP, _VP, _VP, _VP, _I, _I, _F, _I, _F]),
    "velox_sm100_linear_q4": (_I, [_VP, _VP, _F, _PV, _I, _VP, _VP]),
    "velox_sm100_linear_swiglu_q4": (_I, [_VP, _VP, _F, _PV, _PV, _I, _VP, _VP]),
    "velox_sm100_linears_q4": (_I, [_VP, _VP, _F, _VP, _I, _I]),
    "velox_sm100_tp_make_maps": (_I, [_VP, _VP, _I, _I, _LL]),
    "velox_sm100_tp_linear_q4_scatter": (_I, [_VP, _VP, _F, _PV, _I, _VP, _I, _VP]),
    "velox_sm100_tp_norm_q4": (_I, [_VP, _VP, _I, _LL, _VP, _VP, _VP, _I, _LL, _I, _I, _F, _I, _F, _VP]),
    "velox_sm100_tp_finish": (_I, [_VP, _VP, _I, _LL, _VP, _I, _LL, _I, _I, _VP]),
    "velox_sm100_linear_q4_to_q4": (_I, [_VP, _VP, _F, _PV, _I, _VP, _VP, _VP, _F]),
    "velox_sm100_linear_swiglu_q4_to_q4": (_I, [_VP, _VP, _F, _PV, _PV, _I, _VP, _VP, _VP, _F]),
    "velox_sm100_linear_act": (_I, [_PV, _I, C.POINTER(C.c_float)]),
    "velox_sm100_linear": (_I, [_VP, _VP, _I, _LL, _LL, _LL, _I, _I, _VP]),
    "velox_sm100_linear_view": (_I, [_VP, _PV, _I, _VP, _VP]),
    "velox_sm100_linear_bf16": (_I, [_VP, _PV, _I, _VP, _VP]),
    "velox_sm100_linear_nvfp4_a4_static": (_I, [_VP, _PV, _I, _VP, _VP]),
    "velox_sm100_linear_swiglu": (_I, [_VP, _PV, _PV, _I, _VP, _VP]),
    "velox_sm100_linear_swiglu_bf16": (_I, [_VP, _PV, _PV, _I, _VP, _VP]),
    "velox_sm100_linear_swiglu_act": (_I, [_PV, _PV, _I, C.POINTER(C.c_float)]),
    "velox_sm100_linears": (_I, [_VP, _VP, C.POINTER(Part), _I, _I]),
    "velox_sm100_dequant_rows": (_I, [_PV, _VP]),
    "velox_sm100_embed": (_I, [_VP, _I, _VP, _I, _LL, _LL, _LL, _VP]),
    "velox_sm100_matmul": (_I, [_VP, _VP, _VP, _I, _I, _I]),
    "velox_sm100_quantize_act_fp8row": (_I, [_VP, _I, _LL, _VP, _VP]),
    "velox_sm100_quantize_act_nvfp4": (_I, [_VP, _I, _LL, _F, _VP, _VP]),
    "velox_sm100_encode_nvfp4": (_I, [_VP, _LL, _LL, _F, _VP]),
    "velox_sm100_swiglu": (_I, [_VP, _LL, _I, _I, _I, _I, _VP]),
    "velox_sm100_silu_mul": (_I, [_VP, _VP, _LL]),
    "velox_sm100_add": (_I, [_VP, _VP, _LL]),
    "velox_sm100_add_rms_norm_twin": (_I, [_VP, _VP, _VP, _VP, _VP, _I, _I, _F, _I]),
    "velox_sm100_bf16_twin": (_I, [_VP, _VP, _LL]),
}


def build(verbose: bool = False) -> str:
    """Compile every CUDA source for sm_100a into ``libvelox_sm100.so`` (nvcc, in-tree)."""
    r = subprocess.run(["make", "-C", CSRC, "-j8"], capture_output=True, text=True)
    if verbose or r.returncode != 0:
        print(r.stdout[-4000:])
        print(r.stderr[-4000:])
    if r.returncode != 0:
        raise RuntimeError("building libvelox_sm100.so failed")
    return LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: run `python -c 'import __graft_entry__ as g; g.build()'` "
                "(there is no CPU fallback for the sm_100a kernels)")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)  # AttributeError if the library does not export it
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib
