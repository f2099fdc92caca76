"""GPU parity of the tensor-core prefill path (m > 16) against the CPU oracle applying the rounding
the kernel declares through linear_act, exactly as the reference's conformance suite does
(crates/velox-conformance/src/lib.rs:311-366). Shapes follow its prefill cases (lib.rs:3261-3364,
3843-3875, 3962-3970): MMA tile edges in tokens, rows and K, row views starting inside a 128-row
scale tile, both SwiGLU row orders."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from velox_inferer_b200 import ActPolicy, ActQuant, WeightFormat, WeightView

from .gpu_util import FMT_O, backend, bf16_bits, both_metrics, f32_to_bf16_bits, make_view, oracle_linear

pytestmark = pytest.mark.gpu

LINEAR_TOL = 2e-4
SWIGLU_TOL = 5e-4
RMS_TOL = 1e-2
NV, F8, Q4 = WeightFormat.NVFP4, WeightFormat.FP8_ROW_BF16, WeightFormat.GGML_Q4_K
A16, A8, A4 = ActPolicy.a16_only(), ActPolicy.allow_a8(), ActPolicy.allow_a4(600.0)


@pytest.fixture(scope="module")
def b():
    return backend()


def _run_linear(b, fmt, n, k, begin, rows, m, policy, seed=7):
    r = O.Rng(seed)
    payload = r.random_weight(FMT_O[fmt], n, k)
    x = r.vec(m * k, 1.0)
    view = make_view(b, payload, fmt, n, k, begin, rows, policy)
    act = b.linear_act(view, m)
    assert act.permitted(policy), (act, policy)
    want = oracle_linear(x, payload, fmt, n, k, begin, rows, m, act)
    y = b.alloc(m * rows + 2)
    yb = torch.zeros(m * rows, dtype=torch.bfloat16, device=y.device)
    b.linear(b.upload(x), view, y, m, yb=yb)
    assert b.lib.velox_sm100_debug_status() == 0
    got = y.cpu().numpy()
    assert got[-2:].tolist() == [0.0, 0.0]
    got = got[:-2].reshape(m, rows)
    assert np.array_equal(bf16_bits(yb).reshape(-1), f32_to_bf16_bits(got.reshape(-1)))
    return act, got, want


@pytest.mark.parametrize("n,k,begin,rows,m", [
    (384, 640, 128, 256, 37), (512, 1024, 0, 512, 130), (256, 256, 128, 128, 300),
    (256, 1024, 64, 192, 33), (256, 64, 0, 256, 17), (768, 320, 100, 600, 129),
])
def test_nvfp4_prefill_with_nvfp4_activations(b, n, k, begin, rows, m):
    act, got, want = _run_linear(b, NV, n, k, begin, rows, m, A4)
    assert act == ActQuant(ActQuant.NVFP4, 600.0)      # the FP4 tensor-core path ran
    e_conf, e_rms = both_metrics(got, want)
    assert e_conf <= LINEAR_TOL and e_rms <= RMS_TOL, (e_conf, e_rms)


@pytest.mark.parametrize("n,k,begin,rows,m", [
    (512, 1024, 64, 384, 130), (256, 512, 0, 256, 64), (96, 384, 0, 96, 40), (300, 256, 7, 290, 100),
    (300, 8192, 40, 200, 257),    # a long K: sums in chunks, added by the epilogue
])
def test_fp8_prefill_with_fp8_row_activations(b, n, k, begin, rows, m):
    act, got, want = _run_linear(b, F8, n, k, begin, rows, m, A8)
    assert act.kind == ActQuant.FP8_ROW
    e_conf, e_rms = both_metrics(got, want)
    assert e_conf <= LINEAR_TOL and e_rms <= RMS_TOL, (e_conf, e_rms)


@pytest.mark.parametrize("fmt,n,k,begin,rows,m", [
    (NV, 384, 1024, 64, 256, 21), (NV, 384, 1024, 64, 256, 96), (NV, 256, 512, 0, 256, 64),
    (F8, 256, 512, 0, 256, 64), (F8, 200, 320, 17, 150, 70), (NV, 8192, 256, 0, 8192, 100),
    # FP8 rows above one token tile: stored bytes converted inside the GEMM (no bf16 scratch): ragged
    # tokens and rows, a view starting off the tile grid and ending at the parent's last row, a long
    # K (several passes over both rings), many tiles per CTA pair
    (F8, 256, 512, 0, 256, 130), (F8, 700, 1024, 17, 683, 300), (F8, 300, 8192, 40, 200, 257),
    (F8, 40000, 64, 128, 39000, 513),
])
def test_a16_only_views_round_to_bf16_at_most(b, fmt, n, k, begin, rows, m):
    act, got, want = _run_linear(b, fmt, n, k, begin, rows, m, A16)
    assert act.kind in (ActQuant.EXACT, ActQuant.BF16)
    e_conf, e_rms = both_metrics(got, want)
    assert e_conf <= LINEAR_TOL and e_rms <= RMS_TOL, (e_conf, e_rms)


@pytest.mark.parametrize("n,k,rows,m", [(64, 512, 64, 33), (300, 1024, 300, 130), (96, 2560, 96, 70), (520, 2560, 520, 300)])
def test_q4k_prefill_meets_both_bounds(b, n, k, rows, m):
    # Q4_K values (d*sc*q - dmin*m) go to the tensor cores as three bf16 terms, summed in chunks of
    # four k-blocks that the epilogue adds: the 2e-4 conformance metric holds on the reference's
    # random blocks too (values up to 30, sums that cancel).
    act, got, want = _run_linear(b, Q4, n, k, 0, rows, m, A16)
    assert act.kind == ActQuant.BF16
    e_conf, e_rms = both_metrics(got, want)
    assert e_conf <= LINEAR_TOL and e_rms <= RMS_TOL, (e_conf, e_rms)


@pytest.mark.parametrize("fmt,policy,k,w,m,order", [
    (NV, A4, 512, 256, 37, "gate_up"), (NV, A4, 512, 256, 130, "up_gate"), (NV, A4, 1024, 128, 64, "split"),
    (NV, A16, 512, 256, 40, "gate_up"), (F8, A8, 512, 192, 70, "gate_up"), (F8, A16, 512, 96, 33, "split"),
    # FP8 rows with bf16 activations above one token tile: converted inside the GEMM
    (F8, A16, 1024, 200, 300, "up_gate"), (F8, A16, 512, 96, 130, "split"), (F8, A16, 2048, 300, 257, "gate_up"),
])
def test_linear_swiglu_prefill(b, fmt, policy, k, w, m, order):
    r = O.Rng(0x5e2)
    x = r.vec(m * k, 1.0)
    if order == "split":
        pg, pu = r.random_weight(FMT_O[fmt], w, k), r.random_weight(FMT_O[fmt], w, k)
        gate = make_view(b, pg, fmt, w, k, 0, w, policy)
        up = make_view(b, pu, fmt, w, k, 0, w, policy)
        wa = (pg, pu, w, w, 0, 0)
    else:
        p = r.random_weight(FMT_O[fmt], 2 * w, k)
        parent = WeightView.full(b.upload_bytes(p), fmt, 2 * w, k).with_act(policy)
        bg, bu = (0, w) if order == "gate_up" else (w, 0)
        gate, up = parent.rows_view(bg, w), parent.rows_view(bu, w)
        wa = (p, p, 2 * w, 2 * w, bg, bu)
    act = b.linear_swiglu_act(gate, up, m)
    assert act.permitted(policy)
    g = oracle_linear(x, wa[0], fmt, wa[2], k, wa[4], w, m, act)
    u = oracle_linear(x, wa[1], fmt, wa[3], k, wa[5], w, m, act)
    want = O.swiglu(np.concatenate([g, u], axis=1), m, 2 * w, 0, w, w)
    out = b.alloc(m * w)
    outb = torch.zeros(m * w, dtype=torch.bfloat16, device=out.device)
    b.linear_swiglu(b.upload(x), gate, up, out, m, outb=outb)
    assert b.lib.velox_sm100_debug_status() == 0
    got = out.cpu().numpy().reshape(m, w)
    assert O.max_err(got, want) <= SWIGLU_TOL, O.max_err(got, want)
    assert np.array_equal(bf16_bits(outb), f32_to_bf16_bits(got.reshape(-1)))


def test_one_hot_operands_pin_nibble_order_and_scale_placement(b):
    # W has a single non-zero code per row at a known k; x is one-hot per token. Any mix-up of
    # nibble order, swizzle or scale-atom placement moves the single non-zero product.
    n, k, m = 256, 256, 128
    payload = np.zeros(WeightFormat.NVFP4.payload_bytes(n, k), dtype=np.uint8)
    plane = (n * k // 2 + 255) // 256 * 256
    cols = [(37 * r + 11) % k for r in range(n)]
    from velox_inferer_b200 import nvfp4_scale_offset
    for r, c in enumerate(cols):
        payload[(r * k + c) // 2] = 0x2 << (4 * (c % 2))                  # code 2 = 1.0
        payload[plane + nvfp4_scale_offset(r, c // 16, k)] = 0x38 + (r % 8)  # 1.0 .. 1.875
    payload[plane + n * k // 16:plane + n * k // 16 + 4] = np.frombuffer(np.float32(2.0).tobytes(), np.uint8)
    x = np.zeros((m, k), dtype=np.float32)
    for t in range(m):
        x[t, (53 * t + 5) % k] = 3.0
    view = make_view(b, payload, NV, n, k, 0, n, ActPolicy.allow_a4(64.0))
    act = b.linear_act(view, m)
    want = oracle_linear(x.reshape(-1), payload, NV, n, k, 0, n, m, act)
    y = b.alloc(m * n)
    b.linear(b.upload(x.reshape(-1)), view, y, m)
    assert b.lib.velox_sm100_debug_status() == 0
    got = y.cpu().numpy().reshape(m, n)
    assert np.count_nonzero(want) > 50
    assert np.array_equal(got != 0, want != 0)
    assert both_metrics(got, want)[0] <= 1e-6


@pytest.mark.parametrize("fmt,policy,n,k,begin,rows,m", [
    (NV, A4, 512, 1024, 0, 512, 130), (NV, A4, 768, 320, 104, 600, 257), (NV, A4, 1024, 512, 128, 896, 300),
    (F8, A8, 512, 1024, 64, 384, 130), (NV, A16, 384, 1024, 64, 256, 96), (NV, A4, 2048, 256, 0, 2048, 700),
])
def test_bf16_only_output_takes_the_staged_store_and_matches(b, fmt, policy, n, k, begin, rows, m):
    # bf16-only output goes through shared memory and a tensor-map store; it must equal the RNE of
    # the f32 output the direct path writes, bit for bit, and leave neighbouring memory alone.
    r = O.Rng(21)
    payload = r.random_weight(FMT_O[fmt], n, k)
    x = r.vec(m * k, 1.0)
    view = make_view(b, payload, fmt, n, k, begin, rows, policy)
    xb = b.bf16_twin(b.upload(x))
    y = b.alloc(m * rows)
    b.linear_bf16(xb, view, y, m)                      # f32 output: direct stores
    guard = 64
    yb = torch.full((m * rows + guard,), 7.0, dtype=torch.bfloat16, device=y.device)
    b.linear_bf16(xb, view, None, m, yb=yb[: m * rows])   # bf16 only: staged tensor-map stores
    assert b.lib.velox_sm100_debug_status() == 0
    assert np.array_equal(bf16_bits(yb[: m * rows]), f32_to_bf16_bits(y.cpu().numpy()))
    act = b.linear_act(view, m)
    want = oracle_linear(xb.float().cpu().numpy().reshape(-1), payload, fmt, n, k, begin, rows, m, act)
    assert both_metrics(y.cpu().numpy().reshape(m, rows), want)[0] <= LINEAR_TOL
    assert torch.all(yb[m * rows:] == 7.0)


def test_swiglu_bf16_only_output_staged(b):
    fmt, policy, k, w, m = NV, A4, 512, 256, 200
    r = O.Rng(0x5e3)
    x = r.vec(m * k, 1.0)
    p = r.random_weight(FMT_O[fmt], 2 * w, k)
    parent = WeightView.full(b.upload_bytes(p), fmt, 2 * w, k).with_act(policy)
    gate, up = parent.rows_view(0, w), parent.rows_view(w, w)
    xd = b.upload(x)
    out = b.alloc(m * w)
    b.linear_swiglu(xd, gate, up, out, m)
    outb = torch.zeros(m * w, dtype=torch.bfloat16, device=out.device)
    # f32 x and its twin quantise to the same NVFP4 codes only if x is bf16-exact: use the twin for both
    xb = b.bf16_twin(xd)
    out2 = b.alloc(m * w)
    b.linear_swiglu_twin(xb, gate, up, out2, None, m)
    b.linear_swiglu_twin(xb, gate, up, None, outb, m)
    assert b.lib.velox_sm100_debug_status() == 0
    assert np.array_equal(bf16_bits(outb), f32_to_bf16_bits(out2.cpu().numpy()))


def _atoms_of(scales: np.ndarray, m: int, k: int) -> np.ndarray:
    from velox_inferer_b200.weights import nvfp4_scale_offset
    mp = (m + 127) // 128 * 128
    want = np.zeros(mp * k // 16, dtype=np.uint8)
    r, g = np.meshgrid(np.arange(m), np.arange(k // 16), indexing="ij")
    want[nvfp4_scale_offset(r, g, k)] = scales
    return want


@pytest.mark.parametrize("m,dim,addend", [(37, 640, "bf16"), (130, 256, "f32"), (300, 1024, None)])
def test_norm_emits_the_nvfp4_blob_the_quantiser_would(b, m, dim, addend):
    """add_rms_norm_q4: the bf16 twin matches the plain norm's, and codes and scale atoms are,
    bit for bit, the oracle's Nvfp4 quantiser applied to that twin (padding rows zeroed)."""
    r = O.Rng(31)
    acc0, add, w = r.vec(m * dim, 1.0), r.vec(m * dim, 0.5), 1.0 + r.vec(dim, 0.1)
    div = 256.0
    acc = b.upload(acc0)
    acc_ref = b.upload(acc0)
    yb = torch.zeros(m * dim, dtype=torch.bfloat16, device=acc.device)
    yb_ref = torch.zeros_like(yb)
    q4 = b.q4_blob(m, dim)
    q4[1].fill_(0xAB)                                     # stale bytes must not survive in padding rows
    x = xb = None
    if addend == "f32":
        x = b.upload(add)
    elif addend == "bf16":
        xb = b.upload(add).to(torch.bfloat16)
    b.add_rms_norm_q4(acc, x, b.upload(w), yb, q4, m, dim, 1e-6, div, xb=xb)
    b.add_rms_norm_twin(acc_ref, x, b.upload(w), None, yb_ref, m, dim, 1e-6, xb=xb)
    assert torch.equal(acc, acc_ref)
    # the two kernels add the squares in different orders: the norm may differ in the last f32 bit,
    # the bf16 twin by at most one unit in the last place
    d = np.abs(bf16_bits(yb).astype(np.int32) - bf16_bits(yb_ref).astype(np.int32))
    assert d.max() <= 1 and np.mean(d != 0) < 0.01
    want = O.rms_norm(acc.cpu().numpy().reshape(m, dim), w, 1e-6)
    assert O.max_err(yb.float().cpu().numpy(), want) <= 2.0 ** -8
    twin = yb.float().cpu().numpy().reshape(m, dim)
    wc, ws = O.act_codes_nvfp4(twin, div)
    assert np.array_equal(q4[0].cpu().numpy().reshape(m, dim // 2), wc)
    assert np.array_equal(q4[1].cpu().numpy(), _atoms_of(ws, m, dim))


@pytest.mark.parametrize("n,k,m", [(256, 640, 37), (512, 1024, 300)])
def test_linear_q4_equals_linear_bf16_on_the_same_twin(b, n, k, m):
    """A linear fed the pre-quantised blob is the same launch minus the quantiser: bit-equal."""
    r = O.Rng(41)
    payload = r.random_weight(FMT_O[NV], n, k)
    view = make_view(b, payload, NV, n, k, 0, n, ActPolicy.allow_a4(256.0))
    acc = b.upload(r.vec(m * k, 1.0))
    yb = torch.zeros(m * k, dtype=torch.bfloat16, device=acc.device)
    q4 = b.q4_blob(m, k)
    b.add_rms_norm_q4(acc, None, b.upload(np.ones(k, np.float32)), yb, q4, m, k, 1e-6, 256.0)
    y1, y2 = b.alloc(m * n), b.alloc(m * n)
    b.linear_bf16(yb, view, y1, m)
    b.linear_q4(q4, 256.0, view, y2, m)
    assert b.lib.velox_sm100_debug_status() == 0
    assert torch.equal(y1, y2)
    want = oracle_linear(yb.float().cpu().numpy(), payload, NV, n, k, 0, n, m, ActQuant(ActQuant.NVFP4, 256.0))
    e_conf, e_rms = both_metrics(y2.cpu().numpy().reshape(m, n), want)
    assert e_conf <= LINEAR_TOL and e_rms <= RMS_TOL
    # SwiGLU twin
    half = n // 2
    g = make_view(b, payload, NV, n, k, 0, half, ActPolicy.allow_a4(256.0))
    u = make_view(b, payload, NV, n, k, half, half, ActPolicy.allow_a4(256.0))
    o1 = torch.zeros(m * half, dtype=torch.bfloat16, device=acc.device)
    o2 = torch.zeros_like(o1)
    b.linear_swiglu_twin(yb, g, u, None, o1, m)
    b.linear_swiglu_q4(q4, 256.0, g, u, None, o2, m)
    assert torch.equal(o1, o2)


def test_linear_q4_refuses_what_the_fp4_gemm_does_not_serve(b):
    from velox_inferer_b200.errors import Unsupported
    r = O.Rng(43)
    n, k = 256, 256
    payload = r.random_weight(FMT_O[NV], n, k)
    q4 = b.q4_blob(128, k)
    y = b.alloc(128 * n)
    with pytest.raises(Unsupported):                     # divisor differs from the view's
        b.linear_q4(q4, 128.0, make_view(b, payload, NV, n, k, 0, n, ActPolicy.allow_a4(256.0)), y, 128)
    with pytest.raises(Unsupported):                     # policy does not allow FP4 activations
        b.linear_q4(q4, 256.0, make_view(b, payload, NV, n, k, 0, n, A16), y, 128)
    # decode sizes are served too (tensor-core decode path reads the same blob)
    b.linear_q4(q4, 256.0, make_view(b, payload, NV, n, k, 0, n, ActPolicy.allow_a4(256.0)), y, 4)
    assert b.lib.velox_sm100_debug_status() == 0


def _assert_atoms_equal(got, want, m, cols):
    """Scale atoms agree: everywhere after a prefill call, over rows < m after a call served by the
    streaming kernel (decode and small batches, which leave the other rows' bytes alone)."""
    got, want = got.cpu().numpy().reshape(-1), want.cpu().numpy().reshape(-1)
    if m > 64:
        assert np.array_equal(got, want)
        return
    from velox_inferer_b200.weights import nvfp4_scale_offset
    r, g = np.meshgrid(np.arange(m), np.arange(cols // 16), indexing="ij")
    idx = nvfp4_scale_offset(r, g, cols)
    assert np.array_equal(got[idx], want[idx])


@pytest.mark.parametrize("n,k,m", [(256, 640, 37), (512, 1024, 300), (1024, 512, 513), (512, 1024, 1), (256, 5120, 13),
                                   (256, 20480, 37)])   # (the last: a small batch on the streaming kernel)
def test_linears_emit_the_next_linears_nvfp4_input(b, n, k, m):
    """linear_q4_to_q4 / linear_swiglu_q4_to_q4: the bf16 result is unchanged, and the codes and
    scale atoms written by the GEMM epilogue are bit for bit the stand-alone quantiser's output on
    that bf16 result (which the oracle's quantiser pins in test_gpu_parity). m covers a lone CTA,
    a CTA pair whose second half runs past the last token tile, and several pair tiles."""
    r = O.Rng(47)
    payload = r.random_weight(FMT_O[NV], n, k)
    view = make_view(b, payload, NV, n, k, 0, n, ActPolicy.allow_a4(256.0))
    acc = b.upload(r.vec(m * k, 1.0))
    q4 = b.q4_blob(m, k)
    b.add_rms_norm_q4(acc, None, b.upload(np.ones(k, np.float32)), None, q4, m, k, 1e-6, 256.0)
    dev = acc.device
    for out_div in (128.0, 16.0):
        yb_ref = torch.zeros(m * n, dtype=torch.bfloat16, device=dev)
        b.linear_q4(q4, 256.0, view, None, m, yb=yb_ref)
        want_codes, want_atoms = b.quantize_act_nvfp4(yb_ref.float().reshape(m, n), out_div)
        for with_bf16 in (True, False):
            yb = torch.zeros(m * n, dtype=torch.bfloat16, device=dev) if with_bf16 else None
            oq = b.q4_blob(m, n)
            oq[0].fill_(0x5A)
            oq[1].fill_(0x5A)
            b.linear_q4_to_q4(q4, 256.0, view, m, oq, out_div, yb=yb)
            assert b.lib.velox_sm100_debug_status() == 0
            if with_bf16:
                assert torch.equal(yb, yb_ref)
            assert torch.equal(oq[0].reshape(m, n // 2), want_codes.reshape(m, n // 2))
            _assert_atoms_equal(oq[1], want_atoms, m, n)
    # SwiGLU producer
    half = n // 2
    g = make_view(b, payload, NV, n, k, 0, half, ActPolicy.allow_a4(256.0))
    u = make_view(b, payload, NV, n, k, half, half, ActPolicy.allow_a4(256.0))
    ob_ref = torch.zeros(m * half, dtype=torch.bfloat16, device=dev)
    b.linear_swiglu_q4(q4, 256.0, g, u, None, ob_ref, m)
    want_codes, want_atoms = b.quantize_act_nvfp4(ob_ref.float().reshape(m, half), 16.0)
    oq = b.q4_blob(m, half)
    oq[1].fill_(0x5A)
    ob = torch.zeros_like(ob_ref)
    b.linear_swiglu_q4_to_q4(q4, 256.0, g, u, m, oq, 16.0, outb=ob)
    assert b.lib.velox_sm100_debug_status() == 0
    assert torch.equal(ob, ob_ref)
    assert torch.equal(oq[0].reshape(m, half // 2), want_codes.reshape(m, half // 2))
    _assert_atoms_equal(oq[1], want_atoms, m, half)


@pytest.mark.parametrize("m", [1, 8, 40, 130, 300, 513])
def test_linears_q4_equals_separate_calls(b, m):
    """q, k and v of one input through linears_q4 (one launch: the streaming kernel at decode
    sizes, one persistent GEMM grid over all three views' tiles at prefill sizes) give the bits the
    per-view entry points give, including the FP4 hand-over of the first view."""
    r = O.Rng(53)
    k = 1024
    shapes = (512, 128, 256)
    payloads = [r.random_weight(FMT_O[NV], n, k) for n in shapes]
    views = [make_view(b, p, NV, n, k, 0, n, ActPolicy.allow_a4(256.0)) for p, n in zip(payloads, shapes)]
    acc = b.upload(r.vec(m * k, 1.0))
    q4 = b.q4_blob(m, k)
    b.add_rms_norm_q4(acc, None, b.upload(np.ones(k, np.float32)), None, q4, m, k, 1e-6, 256.0)
    dev = acc.device
    want = []
    for v, n in zip(views, shapes):
        yb = torch.zeros(m * n, dtype=torch.bfloat16, device=dev)
        b.linear_q4(q4, 256.0, v, None, m, yb=yb)
        want.append(yb)
    oq_ref = b.q4_blob(m, shapes[0])
    b.linear_q4_to_q4(q4, 256.0, views[0], m, oq_ref, 128.0)
    oq = b.q4_blob(m, shapes[0])
    got = [torch.zeros_like(w) for w in want]
    b.linears_q4(q4, 256.0, [(views[0], got[0], oq, 128.0), (views[1], got[1], None, 0.0), (views[2], got[2], None, 0.0)], m)
    assert b.lib.velox_sm100_debug_status() == 0
    for g, w in zip(got, want):
        assert torch.equal(g, w)
    assert torch.equal(oq[0], oq_ref[0])
    _assert_atoms_equal(oq[1], oq_ref[1], m, shapes[0])


@pytest.mark.parametrize("m", [33, 257])
def test_grouped_prefill_linears_on_ragged_views(b, m):
    """The grouped GEMM launch with views that start inside a 128-row scale tile, have ragged row
    counts and different parents: each part equals its own single launch bit for bit and matches
    the oracle. Reference: Backend::linears, crates/velox-core/src/backend.rs:938-958."""
    r = O.Rng(59)
    k = 640
    specs = ((640, 128, 384), (256, 7, 100), (384, 130, 250))      # (parent rows, row_begin, rows)
    payloads = [r.random_weight(FMT_O[NV], n, k) for n, _, _ in specs]
    views = [make_view(b, p, NV, n, k, r0, rows, ActPolicy.allow_a4(256.0)) for p, (n, r0, rows) in zip(payloads, specs)]
    acc = b.upload(r.vec(m * k, 1.0))
    hb = torch.zeros(m * k, dtype=torch.bfloat16, device=acc.device)
    q4 = b.q4_blob(m, k)
    b.add_rms_norm_q4(acc, None, b.upload(np.ones(k, np.float32)), hb, q4, m, k, 1e-6, 256.0)
    want = []
    for v in views:
        yb = torch.zeros(m * v.rows, dtype=torch.bfloat16, device=acc.device)
        b.linear_q4(q4, 256.0, v, None, m, yb=yb)
        want.append(yb)
    got = [torch.zeros_like(w) for w in want]
    b.linears_q4(q4, 256.0, [(v, g, None, 0.0) for v, g in zip(views, got)], m)
    assert b.lib.velox_sm100_debug_status() == 0
    for g, w, v, p, (n, r0, rows) in zip(got, want, views, payloads, specs):
        assert torch.equal(g, w)
        ref = oracle_linear(hb.float().cpu().numpy(), p, NV, n, k, r0, rows, m, ActQuant(ActQuant.NVFP4, 256.0))
        e_conf, e_rms = both_metrics(g.float().cpu().numpy().reshape(m, rows), ref)
        # bf16 output: half a unit in the last place of every value, so the conformance metric (relative for
        # large values) is held to 2^-8; max|d|/rms grows with the largest output and is not the measure here
        assert e_conf <= 2.0 ** -8 and e_rms <= 4e-2, (e_conf, e_rms)
