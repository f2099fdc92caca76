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


def test_static_scratch_entry_allocates_nothing_and_serves_its_documented_sizes():
    """What the entry point is for: after its first call on a device (which only looks up the
    array's address) no call changes the free device memory, whatever its size; the documented fit
    (m = 2048 at k = 5120) and a view that starts inside a 128-row scale tile give the regular entry
    point's bits; a call that needs exactly the 8 MiB array is served and one row more is refused."""
    b = backend()
    r = O.Rng(0x57a7)
    policy = ActPolicy.allow_a4(256.0)
    b._bind()

    def run(view, m, xb, y):
        s = _view_struct(view)
        return b.lib.velox_sm100_linear_nvfp4_a4_static(xb.data_ptr(), C.byref(s), m, y.data_ptr(), None)

    # every buffer the calls below use exists before the memory reading is taken
    n, k, m = 384, 5120, 2048
    payload = r.random_weight(O.FMT_NVFP4, n, k)
    full = make_view(b, payload, WeightFormat.NVFP4, n, k, 0, n, policy)
    inner = full.rows_view(72, 200)                       # starts and ends inside scale tiles
    xb = b.bf16_twin(b.upload(r.vec(m * k, 1.0)))
    got, want = b.alloc(m * n), b.alloc(m * n)
    n2, k2, m2 = 128, 1024, 14560                         # 7,454,720 B of codes + 933,888 B of scale atoms = 8 MiB
    view2 = make_view(b, r.random_weight(O.FMT_NVFP4, n2, k2), WeightFormat.NVFP4, n2, k2, 0, n2, policy)
    xb2 = b.bf16_twin(b.upload(r.vec((m2 + 1) * k2, 1.0)))
    got2, want2 = b.alloc((m2 + 1) * n2), b.alloc((m2 + 1) * n2)
    b.linear_bf16(xb, full, want, m)                      # (the regular entry grows its scratch here, once)
    b.linear_bf16(xb2, view2, want2, m2)
    assert run(full, 64, xb, got) == 0                    # first call on this device: address look-up
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info(b.device)[0]
    launches0 = b.launch_count()
    assert run(full, m, xb, got) == 0
    torch.cuda.synchronize()
    assert b.launch_count() - launches0 == 2              # the quantiser and the GEMM, both counted
    assert np.array_equal(got.cpu().numpy().view(np.uint32), want.cpu().numpy().view(np.uint32))
    got.zero_()
    want.zero_()
    b.linear_bf16(xb, inner, want, m)
    assert run(inner, m, xb, got) == 0
    assert np.array_equal(got.cpu().numpy().view(np.uint32), want.cpu().numpy().view(np.uint32))
    assert run(view2, m2, xb2, got2) == 0                 # needs the whole array
    assert np.array_equal(got2.cpu().numpy()[: m2 * n2].view(np.uint32), want2.cpu().numpy()[: m2 * n2].view(np.uint32))
    assert run(view2, m2 + 1, xb2, got2) == -3            # 512 bytes more than the array holds
    torch.cuda.synchronize()
    assert b.debug_status() == 0
    assert torch.cuda.mem_get_info(b.device)[0] == free0  # nothing was allocated (or freed) by any of these calls
