"""GPU parity: the sm_100a kernels through the C ABI against the CPU oracle on identical inputs.
Integer/byte work (dequantisation, activation codes, weight encoding, bf16 twins) is bit-exact;
products are held to the reference's conformance tolerance, max|got-want|/(1+|want|) <= 2e-4
(crates/velox-conformance/src/lib.rs:43-58, 356), and to the benchmark's
max|err| <= 1e-2 * rms(oracle output)."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from velox_inferer_b200 import (ActPolicy, ActQuant, LinearDst, LinearPart, ShapeError,
                                WeightFormat, WeightView, nvfp4_scale_offset)

from .gpu_util import (FMT_O, backend, bf16_bits, both_metrics, f32_to_bf16_bits, make_view,
                       oracle_linear)

pytestmark = pytest.mark.gpu

LINEAR_TOL = 2e-4   # conformance lib.rs:356
SWIGLU_TOL = 5e-4   # conformance lib.rs:91
RMS_TOL = 1e-2      # benchmark: max|err| <= 1e-2 * rms(reference output)

NV, F8, Q4 = WeightFormat.NVFP4, WeightFormat.FP8_ROW_BF16, WeightFormat.GGML_Q4_K


@pytest.fixture(scope="module")
def b():
    return backend()


# ---- bit-exact unpack ---------------------------------------------------------------------------

@pytest.mark.parametrize("fmt,n,k,begin,rows", [
    (NV, 256, 320, 0, 256), (NV, 384, 192, 128, 200), (NV, 256, 1024, 64, 192),
    (F8, 160, 1024, 16, 128), (F8, 64, 512, 0, 64),
    (Q4, 64, 512, 3, 50), (Q4, 8, 2560, 0, 8),
])
def test_dequant_rows_bit_exact_random_encodings(b, fmt, n, k, begin, rows):
    payload = O.Rng(7).random_weight(FMT_O[fmt], n, k)
    got = b.dequant_rows(make_view(b, payload, fmt, n, k, begin, rows)).cpu().numpy()
    want = O.decode_rows(FMT_O[fmt], payload, n, k, begin, rows)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("fmt,enc", [(NV, O.encode_nvfp4_rne), (NV, O.encode_nvfp4_ref),
                                     (F8, O.encode_fp8_row), (Q4, O.encode_q4k)])
def test_dequant_rows_bit_exact_constructed_weights(b, fmt, enc):
    n, k = 256, 1024
    w = (np.random.default_rng(0).standard_normal((n, k)) * 0.02).astype(np.float32)
    payload = enc(w)
    got = b.dequant_rows(make_view(b, payload, fmt, n, k, 0, n)).cpu().numpy()
    want = O.decode_rows(FMT_O[fmt], payload, n, k, 0, n)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_q4k_known_answer_on_device(b):
    # the gguf-py known answer of crates/velox-core/src/ggml.rs:4524-4553 decoded by the kernel
    data = O.kat_q4k_blocks(2)
    got = b.dequant_rows(make_view(b, data, Q4, 1, 512, 0, 1)).cpu().numpy().reshape(-1)
    want = O.decode_rows(O.FMT_Q4K, data, 1, 512, 0, 1).reshape(-1)
    assert np.array_equal(got, want)
    assert got[16] == np.float32(10.790267944335938) and got[383] == np.float32(13.024139404296875)


# ---- activation quantisers and the weight constructor, bit-exact --------------------------------

@pytest.mark.parametrize("m,k", [(1, 64), (37, 640), (130, 1024)])
def test_quantize_act_fp8row_bit_exact(b, m, k):
    x = O.Rng(11).vec(m * k, 1.0).reshape(m, k)
    x[0, :5] = [0.0, -0.0, 3.0, -1e-9, 1e-3]
    codes, scales = b.quantize_act_fp8row(b.upload(x).reshape(m, k))
    wc, ws = O.act_codes_fp8(x)
    assert np.array_equal(scales.cpu().numpy().view(np.uint32), ws.view(np.uint32))
    assert np.array_equal(codes.cpu().numpy(), wc)


@pytest.mark.parametrize("m,k,div", [(1, 64, 600.0), (37, 640, 600.0), (300, 256, 256.0)])
def test_quantize_act_nvfp4_bit_exact(b, m, k, div):
    x = O.Rng(13).vec(m * k, 1.0).reshape(m, k)
    x[0, :16] = 0.0                      # an all-zero group: scale code 0, codes 0
    x[m - 1, :4] = [0.25, 0.75, 1.25, -2.5]
    codes, atoms = b.quantize_act_nvfp4(b.upload(x).reshape(m, k), div)
    wc, ws = O.act_codes_nvfp4(x, div)
    assert np.array_equal(codes.cpu().numpy(), wc)
    atoms = atoms.cpu().numpy()
    mp = (m + 127) // 128 * 128
    want_atoms = np.zeros(mp * k // 16, dtype=np.uint8)
    for r in range(m):
        for g in range(k // 16):
            want_atoms[nvfp4_scale_offset(r, g, k)] = ws[r, g]
    assert np.array_equal(atoms, want_atoms)


def test_encode_nvfp4_matches_oracle_encoder(b):
    n, k = 256, 512
    w = (np.random.default_rng(3).standard_normal((n, k)) * 0.02).astype(np.float32)
    got = b.encode_nvfp4(b.upload(w).reshape(n, k)).cpu().numpy()
    want = O.encode_nvfp4_rne(w)
    assert np.array_equal(got[: want.size], want)


# ---- decode GEMV (m <= 16) --------------------------------------------------------------------------

GEMV_CASES = [
    # (fmt, n, k, begin, rows, m): shapes of crates/velox-conformance/src/lib.rs:3219-3365, 3962-3970
    (NV, 256, 128, 0, 256, 1), (NV, 384, 192, 128, 200, 5), (NV, 512, 2048, 128, 384, 8),
    (NV, 384, 640, 128, 256, 8), (NV, 256, 1024, 64, 192, 3), (NV, 256, 5120, 0, 256, 16),
    (NV, 384, 1024, 128, 192, 2), (NV, 128, 64, 0, 128, 1), (NV, 256, 320, 7, 100, 13),
    (F8, 64, 512, 0, 64, 9), (F8, 64, 128, 0, 64, 2), (F8, 512, 2048, 64, 384, 8),
    (F8, 300, 192, 0, 300, 5), (F8, 160, 1024, 16, 128, 16),
    (Q4, 48, 512, 0, 48, 1), (Q4, 40, 1024, 3, 33, 8), (Q4, 64, 2560, 0, 64, 16),
    # Q4_K on the MMA kernel: one K block for four K parts, ragged rows and tokens, both token-tile
    # counts, and row counts large enough for two row tiles per block
    (Q4, 100, 256, 5, 77, 11), (Q4, 72, 5120, 0, 72, 4), (Q4, 2100, 1024, 16, 2050, 2),
    (Q4, 28700, 256, 0, 28700, 3), (Q4, 28700, 512, 9, 28650, 12),
    (Q4, 48, 25600, 0, 48, 2),    # a down projection's K: eight K parts per block, the longest sums
    # FP8 rows with bf16 activations on the MMA kernel: two row tiles per block (many rows), eight K
    # parts (few rows, long K), one and two token tiles, ragged rows and a view off the row-tile grid
    (F8, 38000, 128, 5, 37990, 3), (F8, 38000, 64, 0, 38000, 12), (F8, 48, 8192, 0, 48, 10),
    (F8, 100, 4096, 7, 77, 6), (F8, 64, 64, 0, 64, 2),
]


@pytest.mark.parametrize("fmt,n,k,begin,rows,m", GEMV_CASES)
def test_linear_decode_widths_match_oracle(b, fmt, n, k, begin, rows, m):
    r = O.Rng(7)
    payload = r.random_weight(FMT_O[fmt], n, k)
    x = r.vec(m * k, 1.0)
    view = make_view(b, payload, fmt, n, k, begin, rows)
    act = b.linear_act(view, m)
    assert act.permitted(view.act)
    want = oracle_linear(x, payload, fmt, n, k, begin, rows, m, act)
    y = b.alloc(m * rows + 2)
    yb = torch.zeros(m * rows, dtype=torch.bfloat16, device=y.device)
    b.linear(b.upload(x), view, y, m, yb=yb)
    got = y.cpu().numpy()
    assert got[-2:].tolist() == [0.0, 0.0]          # nothing written past [m, rows]
    got = got[:-2].reshape(m, rows)
    e_conf, e_rms = both_metrics(got, want)
    assert e_conf <= LINEAR_TOL and e_rms <= RMS_TOL, (e_conf, e_rms)
    # bf16 twin of the output is the RNE of the f32 output, bit for bit (lib.rs:95-112)
    assert np.array_equal(bf16_bits(yb).reshape(-1), f32_to_bf16_bits(got.reshape(-1)))
    # the twin entry point gives the same bits as the f32 entry point where linear rounds to bf16
    if act.kind == ActQuant.BF16:
        assert b.takes_bf16(view, m)
        y2 = b.alloc(m * rows)
        b.linear_bf16(b.bf16_twin(b.upload(x)), view, y2, m)
        assert np.array_equal(y2.cpu().numpy().view(np.uint32), got.reshape(-1).view(np.uint32))


def test_fp8_decode_takes_every_code_and_a_wide_range_of_activations(b):
    """The FP8-row decode kernel for bf16 activations re-labels E4M3 bytes as bf16 numbers: every
    finite code (subnormals, zeros and the largest values of both signs) and activations over sixteen
    decades must come out as the oracle's exact decode gives them."""
    n, k, m = 64, 512, 8
    codes = (np.arange(n * k, dtype=np.int64) * 37 % 256).astype(np.uint8)
    codes[(codes & 0x7F) == 0x7F] = 0x06           # the two NaN codes: a subnormal instead
    scales = (2.0 ** np.linspace(-10, 6, n)).astype(np.float32)
    plane = (n * k + 255) // 256 * 256
    payload = np.zeros(plane + 2 * n, dtype=np.uint8)
    payload[: n * k] = codes
    payload[plane:] = f32_to_bf16_bits(scales).astype("<u2").view(np.uint8)
    rng = np.random.default_rng(11)
    x = (rng.standard_normal(m * k) * 10.0 ** rng.uniform(-8, 8, m * k)).astype(np.float32)
    view = make_view(b, payload, F8, n, k, 0, n)
    act = b.linear_act(view, m)
    assert act == ActQuant(ActQuant.BF16)
    want = oracle_linear(x, payload, F8, n, k, 0, n, m, act)
    y = b.alloc(m * n)
    b.linear(b.upload(x), view, y, m)
    got = y.cpu().numpy().reshape(m, n)
    assert np.all(np.isfinite(got))
    # sums of terms sixteen decades apart: held relative to the size of the terms, not of the sum
    scale = np.abs(x.reshape(m, k)).max(axis=1)[:, None] * scales[None, :] * 448.0
    assert np.max(np.abs(got - want) / scale) <= 1e-5
    # and one-hot activations pick single weights: each output is one decoded weight times x, exactly
    for col in (0, 1, 2, 3, 17, 255, 511):
        xh = np.zeros((m, k), dtype=np.float32)
        xh[:, col] = 2.0 ** np.arange(-3, m - 3)
        b.linear(b.upload(xh.reshape(-1)), view, y, m)
        w = O.decode_rows(O.FMT_FP8, payload, n, k, 0, n)[:, col]
        assert np.array_equal(y.cpu().numpy().reshape(m, n), (xh[:, col][:, None] * w[None, :]).astype(np.float32))


# ---- decode on the block-scaled tensor cores (views that admit NVFP4 activations) --------------

@pytest.mark.parametrize("fmt,n,k,begin,rows,m", [c for c in GEMV_CASES if c[0] == NV] + [
    (NV, 256, 8192, 0, 256, 4),       # few tiles, long K: K splits with the ordered fix-up
    (NV, 1280, 256, 128, 1024, 16),   # one k-block per item
])
def test_linear_decode_nvfp4_activations_match_oracle(b, fmt, n, k, begin, rows, m):
    r = O.Rng(11)
    payload = r.random_weight(FMT_O[fmt], n, k)
    x = r.vec(m * k, 1.0)
    policy = ActPolicy.allow_a4(600.0)
    view = make_view(b, payload, fmt, n, k, begin, rows, policy)
    act = b.linear_act(view, m)
    assert act == ActQuant(ActQuant.NVFP4, 600.0)     # the tensor-core decode path declares itself
    want = oracle_linear(x, payload, fmt, n, k, begin, rows, m, act)
    y = b.alloc(m * rows + 2)
    yb = torch.zeros(m * rows, dtype=torch.bfloat16, device=y.device)
    for _ in range(2):                                 # twice: the split counters return to zero
        y.zero_()
        b.linear(b.upload(x), view, y, m, yb=yb)
        assert b.lib.velox_sm100_debug_status() == 0
        got = y.cpu().numpy()
        assert got[-2:].tolist() == [0.0, 0.0]
        got = got[:-2].reshape(m, rows)
        e_conf, e_rms = both_metrics(got, want)
        assert e_conf <= LINEAR_TOL and e_rms <= RMS_TOL, (e_conf, e_rms)
        assert np.array_equal(bf16_bits(yb).reshape(-1), f32_to_bf16_bits(got.reshape(-1)))


@pytest.mark.parametrize("k,w,m,order", [(512, 256, 1, "gate_up"), (1024, 128, 16, "up_gate"), (5120, 128, 3, "gate_up")])
def test_linear_swiglu_decode_nvfp4_activations(b, k, w, m, order):
    r = O.Rng(0x5e2)
    x = r.vec(m * k, 1.0)
    p = r.random_weight(FMT_O[NV], 2 * w, k)
    parent = WeightView.full(b.upload_bytes(p), NV, 2 * w, k).with_act(ActPolicy.allow_a4(600.0))
    bg, bu = (0, w) if order == "gate_up" else (w, 0)
    gate, up = parent.rows_view(bg, w), parent.rows_view(bu, w)
    act = b.linear_swiglu_act(gate, up, m)
    assert act == ActQuant(ActQuant.NVFP4, 600.0)
    want = _swiglu_want(x, p, p, NV, 2 * w, 2 * w, k, bg, bu, w, m, act)
    out = b.alloc(m * w)
    b.linear_swiglu(b.upload(x), gate, up, out, m)
    assert b.lib.velox_sm100_debug_status() == 0
    assert O.max_err(out.cpu().numpy(), want) <= 5e-4


@pytest.mark.parametrize("n,k,begin,rows,m", [
    (64, 512, 0, 64, 9), (64, 128, 0, 64, 2), (512, 2048, 64, 384, 8), (300, 256, 0, 300, 5),
    (160, 1024, 16, 128, 16), (1280, 4096, 0, 1280, 3),
])
def test_linear_decode_fp8_rows_under_allow_a8(b, n, k, begin, rows, m):
    """FP8-row views that admit FP8 activations still decode with bf16 activations (the warp-MMA
    kernel is faster than quantiser + block-scaled kernel at these widths, and rounds less): ragged
    row counts, views starting inside a 128-row tile, long K with few tiles."""
    r = O.Rng(17)
    payload = r.random_weight(FMT_O[F8], n, k)
    x = r.vec(m * k, 1.0)
    view = make_view(b, payload, F8, n, k, begin, rows, ActPolicy.allow_a8())
    act = b.linear_act(view, m)
    assert act == ActQuant(ActQuant.BF16) and act.permitted(view.act)
    want = oracle_linear(x, payload, F8, n, k, begin, rows, m, act)
    y = b.alloc(m * rows + 2)
    yb = torch.zeros(m * rows, dtype=torch.bfloat16, device=y.device)
    for _ in range(2):
        y.zero_()
        b.linear(b.upload(x), view, y, m, yb=yb)
        assert b.lib.velox_sm100_debug_status() == 0
        got = y.cpu().numpy()
        assert got[-2:].tolist() == [0.0, 0.0]
        got = got[:-2].reshape(m, rows)
        e_conf, e_rms = both_metrics(got, want)
        assert e_conf <= LINEAR_TOL and e_rms <= RMS_TOL, (e_conf, e_rms)
        assert np.array_equal(bf16_bits(yb).reshape(-1), f32_to_bf16_bits(got.reshape(-1)))


def test_linear_swiglu_decode_fp8_rows(b):
    r = O.Rng(0x5e3)
    k, w, m = 512, 128, 4
    x = r.vec(m * k, 1.0)
    p = r.random_weight(FMT_O[F8], 2 * w, k)
    parent = WeightView.full(b.upload_bytes(p), F8, 2 * w, k).with_act(ActPolicy.allow_a8())
    gate, up = parent.rows_view(0, w), parent.rows_view(w, w)
    act = b.linear_swiglu_act(gate, up, m)
    assert act == ActQuant(ActQuant.BF16)
    want = _swiglu_want(x, p, p, F8, 2 * w, 2 * w, k, 0, w, w, m, act)
    out = b.alloc(m * w)
    b.linear_swiglu(b.upload(x), gate, up, out, m)
    assert b.lib.velox_sm100_debug_status() == 0
    assert O.max_err(out.cpu().numpy(), want) <= 5e-4


# ---- small batches (17 to 64 tokens): streaming kernel where the GEMM would have few tiles --------

@pytest.mark.parametrize("fmt,n,k,begin,rows,m,streams", [
    (NV, 256, 25600, 0, 256, 37, True),      # two 128-row tiles, each cut over many CTAs
    (NV, 384, 20480, 128, 200, 64, True),    # view inside its parent, full token capacity
    (NV, 256, 25600, 0, 256, 17, True),      # second token chunk holds a single token
    (F8, 256, 16384, 0, 256, 40, True),
    (F8, 300, 16384, 20, 270, 33, True),
    (NV, 512, 1024, 0, 512, 37, False),      # short K: the GEMM keeps it
])
def test_small_batches_take_the_streaming_kernel_where_it_wins(b, fmt, n, k, begin, rows, m, streams):
    r = O.Rng(19)
    payload = r.random_weight(FMT_O[fmt], n, k)
    x = r.vec(m * k, 1.0)
    policy = ActPolicy.allow_a4(600.0) if fmt == NV else ActPolicy.allow_a8()
    view = make_view(b, payload, fmt, n, k, begin, rows, policy)
    act = b.linear_act(view, m)
    assert act == (ActQuant(ActQuant.NVFP4, 600.0) if fmt == NV else ActQuant(ActQuant.FP8_ROW))
    want = oracle_linear(x, payload, fmt, n, k, begin, rows, m, act)
    y = b.alloc(m * rows + 2)
    yb = torch.zeros(m * rows, dtype=torch.bfloat16, device=y.device)
    b.timing_enable(True)
    b.timing_collect()
    try:
        for _ in range(2):                             # twice: the split counters return to zero
            y.zero_()
            b.linear(b.upload(x), view, y, m, yb=yb)
            assert b.lib.velox_sm100_debug_status() == 0
            got = y.cpu().numpy()
            assert got[-2:].tolist() == [0.0, 0.0]
            got = got[:-2].reshape(m, rows)
            e_conf, e_rms = both_metrics(got, want)
            assert e_conf <= LINEAR_TOL and e_rms <= RMS_TOL, (e_conf, e_rms)
            assert np.array_equal(bf16_bits(yb).reshape(-1), f32_to_bf16_bits(got.reshape(-1)))
        launches = {name: cnt for name, (_, cnt) in b.timing_collect().items()}
    finally:
        b.timing_enable(False)
    gemm_class = "gemm_nvfp4" if fmt == NV else "gemm_fp8"
    assert (launches["gemv"], launches[gemm_class]) == ((2, 0) if streams else (0, 2)), launches


def test_portable_signature_entry_point(b):
    # velox_sm100_linear has velox_portable_linear's signature (portable.rs:81-91)
    n, k, m = 256, 512, 4
    r = O.Rng(3)
    payload = r.random_weight(O.FMT_NVFP4, n, k)
    x = r.vec(m * k, 1.0)
    wbuf, xd, y = b.upload_bytes(payload), b.upload(x), b.alloc(m * 128)
    b._bind()
    rc = b.lib.velox_sm100_linear(xd.data_ptr(), wbuf.data_ptr(), 3, n, k, 128, 128, m, y.data_ptr())
    assert rc == 0
    want = O.linear(x, payload, O.FMT_NVFP4, n, k, 128, 128, m, act=O.ACT_BF16)
    assert both_metrics(y.cpu().numpy().reshape(m, 128), want)[0] <= LINEAR_TOL


# ---- shapes only the generic kernel takes ---------------------------------------------------------

@pytest.mark.parametrize("fmt,n,k,begin,rows,m", [
    (F8, 96, 300, 10, 40, 1), (F8, 200, 300, 17, 150, 70), (F8, 96, 300, 0, 96, 40),
])
def test_linear_awkward_k_matches_oracle(b, fmt, n, k, begin, rows, m):
    r = O.Rng(7)
    payload = r.random_weight(FMT_O[fmt], n, k)
    x = r.vec(m * k, 1.0)
    view = make_view(b, payload, fmt, n, k, begin, rows)
    act = b.linear_act(view, m)
    want = oracle_linear(x, payload, fmt, n, k, begin, rows, m, act)
    y = b.alloc(m * rows)
    b.linear(b.upload(x), view, y, m)
    e_conf, e_rms = both_metrics(y.cpu().numpy().reshape(m, rows), want)
    assert e_conf <= LINEAR_TOL and e_rms <= RMS_TOL, (e_conf, e_rms)


# ---- fused SwiGLU -------------------------------------------------------------------------------------

def _swiglu_want(x, payload_g, payload_u, fmt, ng, nu, k, bg, bu, w, m, act):
    g = oracle_linear(x, payload_g, fmt, ng, k, bg, w, m, act)
    u = oracle_linear(x, payload_u, fmt, nu, k, bu, w, m, act)
    both = np.concatenate([g, u], axis=1)
    return O.swiglu(both, m, 2 * w, 0, w, w)


@pytest.mark.parametrize("fmt,k,w,m,order", [
    (NV, 512, 256, 1, "gate_up"), (NV, 512, 256, 7, "up_gate"), (NV, 1024, 128, 16, "split"),
    (F8, 512, 96, 4, "gate_up"), (Q4, 512, 40, 3, "split"),
    (F8, 1024, 72, 2, "up_gate"), (F8, 4096, 100, 13, "gate_up"), (F8, 64, 38000, 9, "gate_up"), (F8, 256, 50, 16, "split"),
    # Q4_K pairs on the MMA kernel: both row orders in one parent, ragged rows, one and two token tiles
    (Q4, 1024, 72, 1, "gate_up"), (Q4, 2560, 100, 8, "up_gate"), (Q4, 512, 200, 13, "gate_up"),
])
def test_linear_swiglu_fused_matches_composed_oracle(b, fmt, k, w, m, order):
    # both row orders in one parent and separate parents: conformance lib.rs:3856-3861
    r = O.Rng(0x5e1)
    x = r.vec(m * k, 1.0)
    if order == "split":
        pg, pu = r.random_weight(FMT_O[fmt], w, k), r.random_weight(FMT_O[fmt], w, k)
        gate, up = make_view(b, pg, fmt, w, k, 0, w), make_view(b, pu, fmt, w, k, 0, w)
        want_args = (pg, pu, fmt, w, w, k, 0, 0)
    else:
        p = r.random_weight(FMT_O[fmt], 2 * w, k)
        buf = b.upload_bytes(p)
        parent = WeightView.full(buf, fmt, 2 * w, k)
        bg, bu = (0, w) if order == "gate_up" else (w, 0)
        gate, up = parent.rows_view(bg, w), parent.rows_view(bu, w)
        want_args = (p, p, fmt, 2 * w, 2 * w, k, bg, bu)
    act = b.linear_swiglu_act(gate, up, m)
    want = _swiglu_want(x, *want_args, w, m, act)
    out = b.alloc(m * w)
    outb = torch.zeros(m * w, dtype=torch.bfloat16, device=out.device)
    b.linear_swiglu(b.upload(x), gate, up, out, m, outb=outb)
    got = out.cpu().numpy().reshape(m, w)
    assert O.max_err(got, want) <= SWIGLU_TOL
    assert np.array_equal(bf16_bits(outb), f32_to_bf16_bits(got.reshape(-1)))
    out2 = b.alloc(m * w)
    b.linear_swiglu_twin(b.bf16_twin(b.upload(x)), gate, up, out2, None, m)
    assert np.array_equal(out2.cpu().numpy(), got.reshape(-1))


# ---- linears: column ranges ---------------------------------------------------------------------------

def test_linears_writes_column_ranges_and_nothing_else(b):
    # conformance lib.rs:365-470: ld = parts' rows + 2, the last two columns must stay zero
    r = O.Rng(0x11)
    k, m = 512, 5
    p = r.random_weight(O.FMT_NVFP4, 384, k)
    x = r.vec(m * k, 1.0)
    buf = b.upload_bytes(p)
    parent = WeightView.full(buf, NV, 384, k)
    parts = [LinearPart(parent.rows_view(0, 256), 0), LinearPart(parent.rows_view(256, 128), 256)]
    ld = 384 + 2
    y = b.alloc(m * ld)
    b.linears(b.upload(x), None, [LinearDst(y, ld, parts)], m)
    got = y.cpu().numpy().reshape(m, ld)
    want = O.linear(x, p, O.FMT_NVFP4, 384, k, 0, 384, m, act=O.ACT_BF16)
    assert np.all(got[:, 384:] == 0.0)
    assert both_metrics(got[:, :384], want)[0] <= LINEAR_TOL
    with pytest.raises(ShapeError):
        b.linears(b.upload(x), None, [LinearDst(y, 300, parts)], m)


# ---- shape rejection follows check::linear ---------------------------------------------------------------

def test_shape_errors_match_the_oracle(b):
    n, k = 128, 64
    payload = O.Rng(1).random_weight(O.FMT_NVFP4, n, k)
    view = make_view(b, payload, NV, n, k, 0, n)
    x, y = b.alloc(k), b.alloc(n)
    for bad in (dict(m=0), dict(view=view.rows_view(100, 29)), dict(x=b.alloc(k - 1)),
                dict(y=b.alloc(n - 1))):
        args = dict(x=x, view=view, y=y, m=1)
        args.update(bad)
        with pytest.raises(ShapeError):
            b.linear(args["x"], args["view"], args["y"], args["m"])
    # the C ABI itself refuses what check::linear refuses
    v = make_view(b, payload, NV, n, k, 0, n)
    from velox_inferer_b200 import _lib
    import ctypes as C
    s = _lib.View(v.buf.data_ptr(), 3, 0, 100, k, 0, 100, 0.0)      # N % 128 != 0
    assert b.lib.velox_sm100_linear_view(x.data_ptr(), C.byref(s), 1, y.data_ptr(), None) == -2
    s = _lib.View(v.buf.data_ptr(), 9, 0, n, k, 0, n, 0.0)          # a format not served
    assert b.lib.velox_sm100_linear_view(x.data_ptr(), C.byref(s), 1, y.data_ptr(), None) == -1


# ---- elementwise neighbours ----------------------------------------------------------------------------

def test_elementwise_ops_match_oracle(b):
    r = O.Rng(5)
    rows, w = 7, 96
    src = r.vec(rows * 2 * w, 3.0)
    out = b.alloc(rows * w)
    b.swiglu(b.upload(src), rows, 2 * w, w, 0, w, out)
    assert O.max_err(out.cpu().numpy(), O.swiglu(src, rows, 2 * w, w, 0, w).reshape(-1)) <= 1e-6
    g, u = r.vec(500, 4.0), r.vec(500, 2.0)
    gd = b.upload(g)
    b.silu_mul(gd, b.upload(u), 500)
    assert O.max_err(gd.cpu().numpy(), O.silu_mul(g, u)) <= 1e-6
    acc, xx, wt = r.vec(5 * 320, 1.0), r.vec(5 * 320, 1.0), r.vec(320, 1.0)
    accd, y = b.upload(acc), b.alloc(5 * 320)
    yb = torch.zeros(5 * 320, dtype=torch.bfloat16, device=y.device)
    b.add_rms_norm_twin(accd, b.upload(xx), b.upload(wt), y, yb, 5, 320, 1e-6, offset=True)
    s = (acc + xx).astype(np.float32)
    assert np.array_equal(accd.cpu().numpy(), s)
    want = O.rms_norm(s.reshape(5, 320), wt, 1e-6, offset=True)
    assert O.max_err(y.cpu().numpy(), want.reshape(-1)) <= 1e-5
    assert np.array_equal(bf16_bits(yb), f32_to_bf16_bits(y.cpu().numpy()))


@pytest.mark.parametrize("fmt,n,k,m", [(NV, 128, 256, 3), (NV, 256, 256, 40), (F8, 96, 256, 5), (Q4, 64, 512, 20)])
def test_payload_off_the_16_byte_grid_takes_the_exact_kernel(b, fmt, n, k, m):
    """A payload that starts 8 bytes into a buffer is a legal view: linear_act reports the rounding
    of the per-element kernel (none) and linear serves it, instead of a fast path failing late."""
    r = O.Rng(0xa11)
    payload = r.random_weight(FMT_O[fmt], n, k)
    raw = np.concatenate([np.zeros(8, np.uint8), payload])
    buf = b.upload_bytes(raw)
    view = WeightView.full(buf[8:], fmt, n, k).with_act(ActPolicy.allow_a4(600.0))
    assert view.buf.data_ptr() % 16 == 8
    act = b.linear_act(view, m)
    assert act.kind == ActQuant.EXACT
    x = r.vec(m * k, 1.0)
    y = b.alloc(m * n)
    b.linear(b.upload(x), view, y, m)
    want = oracle_linear(x, payload, fmt, n, k, 0, n, m, act)
    e_conf, e_rms = both_metrics(y.cpu().numpy().reshape(m, n), want)
    assert e_conf <= LINEAR_TOL and e_rms <= RMS_TOL, (e_conf, e_rms)
