"""The prefill entry point that never allocates (velox_sm100_linear_nvfp4_a4_static).

Some hosts cannot call cudaMalloc once the model is running: the device's memory is fully planned
out, or the serving loop must not touch the allocator. For them the library offers one NVFP4
prefill linear whose working memory (the quantised activations) lives in a fixed 8 MiB array built
into the library instead of grow-only cudaMalloc'd scratch. This test drives it through the C ABI
twice in a row - a large call, then a smaller one that finds the first call's leftovers in the
shared array - and requires the same bits as the regular entry point, plus the documented refusal
of a call that would not fit. It is collected last so that a failure here cannot hide any other
test."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import oracle as O
from velox_inferer_b200 import ActPolicy, WeightFormat, _lib

from .gpu_util import backend, bf16_bits, make_view

pytestmark = pytest.mark.gpu


def _view_struct(v):
    return _lib.View(v.buf.data_ptr(), int(v.format), v.act.kind, v.parent_rows, v.k, v.row_begin, v.rows,
                     v.act.divisor)


def test_static_scratch_entry_matches_regular_entry_twice_in_a_row():
    b = backend()
    r = O.Rng(0x51a7)
    n, k = 512, 1024
    payload = r.random_weight(O.FMT_NVFP4, n, k)
    policy = ActPolicy.allow_a4(600.0)
    full = make_view(b, payload, WeightFormat.NVFP4, n, k, 0, n, policy)
    cases = [(full, 300), (full.rows_view(128, 256), 70)]   # second call: fewer rows of x and of W
    for view, m in cases:
        xb = b.bf16_twin(b.upload(r.vec(m * k, 1.0)))
        want_f32 = b.alloc(m * view.rows)
        want_bf = torch.zeros(m * view.rows, dtype=torch.bfloat16, device=b.device)
        b.linear_bf16(xb, view, want_f32, m)
        b.linear_bf16(xb, view, None, m, yb=want_bf)
        got_f32 = b.alloc(m * view.rows)
        got_bf = torch.zeros(m * view.rows, dtype=torch.bfloat16, device=b.device)
        b._bind()
        s = _view_struct(view)
        assert b.lib.velox_sm100_linear_nvfp4_a4_static(xb.data_ptr(), C.byref(s), m, got_f32.data_ptr(), None) == 0
        assert b.lib.velox_sm100_linear_nvfp4_a4_static(xb.data_ptr(), C.byref(s), m, None, got_bf.data_ptr()) == 0
        assert b.lib.velox_sm100_debug_status() == 0
        # same kernels on the same operands: identical bits (the suite's linear tolerance is 2e-4)
        assert O.max_err(got_f32.cpu().numpy(), want_f32.cpu().numpy()) <= 2e-4
        assert np.array_equal(got_f32.cpu().numpy().view(np.uint32), want_f32.cpu().numpy().view(np.uint32))
        assert np.array_equal(bf16_bits(got_bf), bf16_bits(want_bf))


def test_static_scratch_entry_refuses_what_does_not_fit_or_apply():
    b = backend()
    n, k = 128, 8192
    payload = O.Rng(3).random_weight(O.FMT_NVFP4, n, k)
    view = make_view(b, payload, WeightFormat.NVFP4, n, k, 0, n, ActPolicy.allow_a4(600.0))
    m = 4096                                   # 16 MiB of codes alone: over the 8 MiB array
    xb = torch.zeros(m * k, dtype=torch.bfloat16, device=b.device)
    y = b.alloc(m * n)
    b._bind()
    s = _view_struct(view)
    assert b.lib.velox_sm100_linear_nvfp4_a4_static(xb.data_ptr(), C.byref(s), m, y.data_ptr(), None) == -3
    assert float(y.abs().max()) == 0.0          # nothing was launched
    a16 = _view_struct(view.with_act(ActPolicy.a16_only()))
    assert b.lib.velox_sm100_linear_nvfp4_a4_static(xb.data_ptr(), C.byref(a16), 64, y.data_ptr(), None) == -1
    assert b.lib.velox_sm100_linear_nvfp4_a4_static(xb.data_ptr(), C.byref(s), 8, y.data_ptr(), None) == -1
