"""Shared helpers of the GPU parity tests: build views from oracle-made payloads and compare the
CUDA path (through the C ABI) with the CPU oracle."""
import numpy as np
import torch

from oracle import oracle as O
from velox_inferer_b200 import ActPolicy, ActQuant, WeightFormat, WeightView

FMT_O = {WeightFormat.NVFP4: O.FMT_NVFP4, WeightFormat.FP8_ROW_BF16: O.FMT_FP8,
         WeightFormat.GGML_Q4_K: O.FMT_Q4K}
ACT_O = {ActQuant.EXACT: O.ACT_EXACT, ActQuant.BF16: O.ACT_BF16, ActQuant.FP8_ROW: O.ACT_FP8_ROW,
         ActQuant.NVFP4: O.ACT_NVFP4}


def backend():
    from velox_inferer_b200 import Sm100Backend
    return Sm100Backend(0)


def make_view(b, payload: np.ndarray, fmt, n, k, begin, rows, policy=ActPolicy()):
    buf = b.upload_bytes(payload)
    return WeightView.full(buf, fmt, n, k).rows_view(begin, rows).with_act(policy)


def oracle_linear(x, payload, fmt, n, k, begin, rows, m, act: ActQuant, threads=0):
    return O.linear(x, payload, FMT_O[fmt], n, k, begin, rows, m, threads=threads,
                    act=ACT_O[act.kind], divisor=act.divisor)


def both_metrics(got, want):
    """(conformance metric max|d|/(1+|want|), max|d| / rms(want))."""
    got = np.asarray(got, dtype=np.float32)
    want = np.asarray(want, dtype=np.float32)
    return O.max_err(got, want), O.max_abs_diff(got, want) / max(O.rms(want), 1e-30)


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().view(torch.int16).numpy().view(np.uint16)


def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
