"""CPU-side checks: the C-ABI library loads and exports every symbol the header declares, and the
host-side mirror of the reference's contract types behaves as the reference's does. No GPU work."""
import os
import re

import pytest

from oracle import oracle as O
from velox_inferer_b200 import (ActPolicy, ActQuant, ShapeError, Unsupported, WeightFormat,
                                WeightView, _lib, check_linear, nvfp4_scale_offset, swiglu_pair)
from velox_inferer_b200.errors import BackendError, status

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "velox_sm100.h")).read()
    declared = set(re.findall(r"\b(velox_sm100_[a-z0-9_]+)\s*\(", header))
    assert len(declared) >= 19
    lib = _lib.lib()
    for name in declared:
        assert hasattr(lib, name), name
    assert declared == set(_lib.SIGNATURES)
    assert lib.velox_sm100_abi_version() == 1


def test_view_struct_layout_matches_header():
    import ctypes as C
    # 8 + 4 + 4 + 8 + 8 + 8 + 4 + 4
    assert C.sizeof(_lib.View) == 48 and C.sizeof(_lib.Part) == 72 and C.sizeof(_lib.PartQ4) == 80
    assert _lib.View.rows.offset == 40 and _lib.View.divisor.offset == 44


def test_payload_bytes_and_swizzle_agree_with_oracle():
    fm = {WeightFormat.NVFP4: O.FMT_NVFP4, WeightFormat.FP8_ROW_BF16: O.FMT_FP8,
          WeightFormat.GGML_Q4_K: O.FMT_Q4K}
    for fmt, code in fm.items():
        for n, k in ((128, 256), (25600, 5120), (14336, 4096), (5120, 25600)):
            assert fmt.payload_bytes(n, k) == O.payload_bytes(code, n, k)
    # sizes the survey derives for the benchmark configurations
    assert WeightFormat.NVFP4.payload_bytes(25600, 5120) == 73_728_004
    assert WeightFormat.FP8_ROW_BF16.payload_bytes(14336, 4096) == 58_748_928
    assert WeightFormat.GGML_Q4_K.payload_bytes(14336, 4096) == 33_030_144
    for r, g in ((0, 0), (37, 5), (129, 3), (255, 7)):
        assert nvfp4_scale_offset(r, g, 128) == O.nvfp4_scale_offset(r, g, 128)


def test_format_names_and_shape_rules():
    assert WeightFormat.from_names("nvfp4", "block_scale_k16_m128x4_v1") is WeightFormat.NVFP4
    assert WeightFormat.from_names("ggml_q4_k", "ggml_block_v1") is WeightFormat.GGML_Q4_K
    with pytest.raises(Unsupported):
        WeightFormat.from_names("q8_g32_fp16", "row_split_k128_v1")
    with pytest.raises(ShapeError):
        WeightFormat.NVFP4.check_shape(100, 64)
    with pytest.raises(ShapeError):
        WeightFormat.GGML_Q4_K.check_shape(4, 200)
    WeightFormat.FP8_ROW_BF16.check_shape(96, 300)


def test_act_policy_meet_and_permitted():
    a16, a8, a4 = ActPolicy.a16_only(), ActPolicy.allow_a8(), ActPolicy.allow_a4(600.0)
    assert a4.meet(a16) == a16 and a8.meet(a4) == a8 and a4.meet(a4) == a4
    assert a4.meet(ActPolicy.allow_a4(500.0)) == a8
    assert ActQuant(ActQuant.BF16).permitted(a16)
    assert not ActQuant(ActQuant.FP8_ROW).permitted(a16)
    assert ActQuant(ActQuant.FP8_ROW).permitted(a4)
    assert ActQuant(ActQuant.NVFP4, 600.0).permitted(a4)
    assert not ActQuant(ActQuant.NVFP4, 500.0).permitted(a4)
    assert not ActQuant(ActQuant.NVFP4, 600.0).permitted(a8)


def test_swiglu_pair_detects_both_row_orders():
    buf = object()
    parent = WeightView.full(buf, WeightFormat.NVFP4, 512, 256)
    g, u = parent.rows_view(0, 256), parent.rows_view(256, 256)
    both, go, uo = swiglu_pair(g, u)
    assert (both.row_begin, both.rows, go, uo) == (0, 512, 0, 256)
    both, go, uo = swiglu_pair(u, g)
    assert (both.row_begin, both.rows, go, uo) == (0, 512, 256, 0)
    assert swiglu_pair(g, WeightView.full(object(), WeightFormat.NVFP4, 512, 256).rows_view(256, 256)) is None
    assert swiglu_pair(g, parent.rows_view(128, 256)) is None


def test_check_linear_rejects_what_the_oracle_rejects():
    class Buf:
        pass
    n, k = 128, 64
    pb = WeightFormat.NVFP4.payload_bytes(n, k)
    v = WeightView.full(Buf(), WeightFormat.NVFP4, n, k)
    cases = [
        (k, v, pb, n, 1), (k, v, pb, n, 0), (k, v.rows_view(100, 29), pb, 29, 1),
        (k, v, pb - 8, n, 1), (k - 1, v, pb, n, 1), (k, v, pb, n - 1, 1),
    ]
    for x_len, view, w_bytes, y_len, m in cases:
        rc = O.linear_rc(x_len, w_bytes, O.FMT_NVFP4, n, k, view.row_begin, view.rows, m, y_len)
        try:
            check_linear(x_len, view, w_bytes, y_len, m)
            ok = True
        except ShapeError:
            ok = False
        assert ok == (rc == 0)


def test_status_maps_return_codes_like_the_reference():
    status(0, "x")
    with pytest.raises(Unsupported):
        status(-1, "x")
    with pytest.raises(ShapeError):
        status(-2, "x")
    with pytest.raises(BackendError):
        status(1, "x")
