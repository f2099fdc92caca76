"""GPU parity at the benchmark's own shapes: BASELINE.json configs 0-3 as worded (seed 0, weights
N(0, 0.02^2) quantised by the oracle's constructors, activations N(0, 1)).

The GPU computes the full shape through the C ABI; the oracle checks a subset of it that touches the
first, a middle and the last row tile and token tile (the oracle rounds activations per token, so a
token subset is an exact sub-problem). Both error metrics are asserted: the reference's conformance
metric max|d| / (1 + |want|) <= 2e-4 (5e-4 after SwiGLU; crates/velox-conformance/src/lib.rs:43-58,
91, 356) and max|d| <= 1e-2 * rms(want). Every case also checks that a row subset of the very same
payload decodes bit for bit. Reference cases of the same kind (several hundred tiles, ragged rows,
m = 1030): crates/velox-conformance/src/lib.rs:3843-3875.

Where the kernel rounds activations further than bf16 (NVFP4 or FP8 rows, as the view's policy
allows), the distance of its result from the oracle with bf16 activations is reported in the
terminal summary: that is what the declared rounding costs on this data."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from velox_inferer_b200 import ActPolicy, ActQuant, WeightFormat, WeightView

from .conftest import report_line
from .gpu_util import ACT_O, FMT_O, backend, bf16_bits, both_metrics, f32_to_bf16_bits

pytestmark = pytest.mark.gpu

LINEAR_TOL, SWIGLU_TOL, RMS_TOL = 2e-4, 5e-4, 1e-2
NV, F8, Q4 = WeightFormat.NVFP4, WeightFormat.FP8_ROW_BF16, WeightFormat.GGML_Q4_K
DIV_X, DIV_H = 256.0, 16.0          # the benchmark's activation divisors (norm output; silu(g)*u)


@pytest.fixture(scope="module")
def b():
    return backend()


def _weights(seed, n, k):
    # seeded N(0, 0.02^2); drawn on the device (a host generator needs ten seconds per matrix here)
    gen = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(n, k, generator=gen, device="cuda", dtype=torch.float32) * 0.02).cpu().numpy()


def _x(m, k, seed=0):
    # bf16-representable N(0, 1), as the configs word it ("x is bf16 [M, K]")
    x = np.random.default_rng(1000 + seed).standard_normal((m, k)).astype(np.float32)
    return O.quantize_activations(x.reshape(-1), k, O.ACT_BF16).reshape(m, k)


def _row_slices(n):
    mid = (n // 2) // 128 * 128
    return [(0, 128), (mid - 64, 128), (n - 128, 128)]       # first tile, across a tile edge, last tile


def _token_subset(m):
    if m <= 64:
        return np.arange(m)
    mid = m // 2 // 128 * 128
    return np.unique(np.concatenate([np.arange(0, 24), np.arange(mid - 8, mid + 8), np.arange(m - 24, m)]))


@pytest.fixture(scope="module")
def c0_payload():
    return O.encode_nvfp4_rne(_weights(0, 25600, 5120))


@pytest.fixture(scope="module")
def c0_dev(b, c0_payload):
    return b.upload_bytes(c0_payload)


def _check_linear(b, name, fmt, payload, buf, n, k, m, policy, tol=LINEAR_TOL):
    view = WeightView.full(buf, fmt, n, k).with_act(policy)
    act = b.linear_act(view, m)
    assert act.permitted(policy), (act, policy)
    x = _x(m, k)
    y = b.alloc(m * n)
    yb = torch.zeros(m * n, dtype=torch.bfloat16, device=b.device)
    b.linear(b.upload(x), view, y, m, yb=yb)
    assert b.lib.velox_sm100_debug_status() == 0
    got = y.cpu().numpy().reshape(m, n)
    assert np.array_equal(bf16_bits(yb).reshape(-1), f32_to_bf16_bits(got.reshape(-1)))   # the twin is RNE of y
    toks = _token_subset(m)
    xs = np.ascontiguousarray(x[toks])
    worst = (0.0, 0.0)
    dist_bf16 = 0.0
    for r0, rows in _row_slices(n):
        want = O.linear(xs, payload, FMT_O[fmt], n, k, r0, rows, len(toks), act=ACT_O[act.kind], divisor=act.divisor)
        sub = got[toks][:, r0:r0 + rows]
        e = both_metrics(sub, want)
        worst = (max(worst[0], e[0]), max(worst[1], e[1]))
        if act.kind in (ActQuant.NVFP4, ActQuant.FP8_ROW):
            wb = O.linear(xs, payload, FMT_O[fmt], n, k, r0, rows, len(toks), act=O.ACT_BF16)
            dist_bf16 = max(dist_bf16, O.max_abs_diff(sub, wb) / O.rms(wb))
        # the same payload decodes bit for bit
        dq = b.dequant_rows(view.rows_view(r0, 16)).cpu().numpy()
        assert np.array_equal(dq.view(np.uint32), O.decode_rows(FMT_O[fmt], payload, n, k, r0, 16).view(np.uint32))
    assert worst[0] <= tol and worst[1] <= RMS_TOL, (name, act, worst)
    line = f"{name}: act {act}, conformance metric {worst[0]:.2e}, max|d|/rms {worst[1]:.2e}"
    if dist_bf16:
        line += f"; distance from the bf16-activation oracle {dist_bf16:.2e} of rms"
    report_line(line)
    return got


# ---- config 0: decode GEMV, M = 1, whole output against the oracle --------------------------------

@pytest.mark.parametrize("policy", [ActPolicy.a16_only(), ActPolicy.allow_a4(DIV_X)], ids=["a16", "a4"])
def test_config0_decode_gemv(b, c0_payload, c0_dev, policy):
    n, k, m = 25600, 5120, 1
    view = WeightView.full(c0_dev, NV, n, k).with_act(policy)
    act = b.linear_act(view, m)
    x = _x(m, k)
    yb = torch.zeros(m * n, dtype=torch.bfloat16, device=b.device)
    y = b.alloc(m * n)
    b.linear(b.upload(x), view, y, m, yb=yb)
    assert b.lib.velox_sm100_debug_status() == 0
    want = O.linear(x, c0_payload, O.FMT_NVFP4, n, k, 0, n, m, act=ACT_O[act.kind], divisor=act.divisor)
    e = both_metrics(y.cpu().numpy(), want.reshape(-1))
    assert e[0] <= LINEAR_TOL and e[1] <= RMS_TOL, (act, e)
    line = f"C0 [25600,5120] M=1 {act}: conformance {e[0]:.2e}, max|d|/rms {e[1]:.2e}"
    if act.kind == ActQuant.NVFP4:
        wb = O.linear(x, c0_payload, O.FMT_NVFP4, n, k, 0, n, m, act=O.ACT_BF16)
        line += f"; distance from the bf16-activation oracle {O.max_abs_diff(y.cpu().numpy(), wb) / O.rms(wb):.2e} of rms"
    report_line(line)
    # bf16 output, as the config words it: the RNE of the f32 result
    assert np.array_equal(bf16_bits(yb), f32_to_bf16_bits(y.cpu().numpy()))


# ---- config 1: the same matrix across the M sweep, both activation policies -----------------------

@pytest.mark.parametrize("m", [4, 16, 64, 256, 2048])
def test_config1_sweep_nvfp4_activations(b, c0_payload, c0_dev, m):
    _check_linear(b, f"C1 [25600,5120] M={m} AllowA4", NV, c0_payload, c0_dev, 25600, 5120, m,
                  ActPolicy.allow_a4(DIV_X))


@pytest.mark.parametrize("m", [4, 16, 64, 256])
def test_config1_sweep_bf16_activations(b, c0_payload, c0_dev, m):
    _check_linear(b, f"C1 [25600,5120] M={m} A16Only", NV, c0_payload, c0_dev, 25600, 5120, m,
                  ActPolicy.a16_only())


# ---- config 2: gate|up (one parent, one divisor) -> SwiGLU -> down ---------------------------------

@pytest.fixture(scope="module")
def mlp(b):
    w, k = 25600, 5120
    gu = O.encode_nvfp4_rne(_weights(2, 2 * w, k))
    down = O.encode_nvfp4_rne(_weights(3, k, w))
    return gu, b.upload_bytes(gu), down, b.upload_bytes(down)


@pytest.mark.parametrize("m", [1, 16, 2048])
def test_config2_mlp(b, mlp, m):
    gu, gu_dev, down, down_dev = mlp
    w, k = 25600, 5120
    parent = WeightView.full(gu_dev, NV, 2 * w, k).with_act(ActPolicy.allow_a4(DIV_X))
    gate, up = parent.rows_view(0, w), parent.rows_view(w, w)
    dview = WeightView.full(down_dev, NV, k, w).with_act(ActPolicy.allow_a4(DIV_H))
    act = b.linear_swiglu_act(gate, up, m)
    act_d = b.linear_act(dview, m)
    x = _x(m, k, seed=2)
    h = b.alloc(m * w)
    y = b.alloc(m * k)
    b.linear_swiglu(b.upload(x), gate, up, h, m)
    b.linear(h, dview, y, m)
    assert b.lib.velox_sm100_debug_status() == 0
    hg = h.cpu().numpy().reshape(m, w)
    yg = y.cpu().numpy().reshape(m, k)
    toks = _token_subset(m)[:: max(1, len(_token_subset(m)) // 8)][:8] if m > 16 else np.arange(m)
    xs = np.ascontiguousarray(x[toks])
    # stage 1 on column slices: silu(x . gate_i) * (x . up_i)
    worst_h = 0.0
    for r0, rows in _row_slices(w):
        g = O.linear(xs, gu, O.FMT_NVFP4, 2 * w, k, r0, rows, len(toks), act=ACT_O[act.kind], divisor=act.divisor)
        u = O.linear(xs, gu, O.FMT_NVFP4, 2 * w, k, w + r0, rows, len(toks), act=ACT_O[act.kind], divisor=act.divisor)
        want = O.swiglu(np.concatenate([g, u], axis=1), len(toks), 2 * rows, 0, rows, rows)
        worst_h = max(worst_h, O.max_err(hg[toks][:, r0:r0 + rows], want))
    assert worst_h <= SWIGLU_TOL, worst_h
    # stage 2 from the GPU's own intermediate: down on the whole K of these tokens
    hs = np.ascontiguousarray(hg[toks])
    want_y = O.linear(hs, down, O.FMT_NVFP4, k, w, 0, k, len(toks), act=ACT_O[act_d.kind], divisor=act_d.divisor)
    e = both_metrics(yg[toks], want_y)
    assert e[0] <= LINEAR_TOL and e[1] <= RMS_TOL, e
    # the whole MLP against the oracle's own chain for a few tokens
    t2 = toks[:4]
    g = O.linear(x[t2], gu, O.FMT_NVFP4, 2 * w, k, 0, 2 * w, len(t2), act=ACT_O[act.kind], divisor=act.divisor)
    hw = O.swiglu(g, len(t2), 2 * w, 0, w, w)
    yw = O.linear(hw, down, O.FMT_NVFP4, k, w, 0, k, len(t2), act=ACT_O[act_d.kind], divisor=act_d.divisor)
    # Across the two stages the comparison is statistical: the GPU's intermediate and the oracle's
    # differ in last bits, and where a value sits on a rounding boundary of the NVFP4 quantiser one
    # code of down's input changes by a whole step. Each stage is exact above; the chain is held to
    # a relative RMS error and its largest deviation is reported.
    chain_rms = float(np.sqrt(np.mean((yg[t2] - yw) ** 2))) / O.rms(yw)
    chain_max = O.max_abs_diff(yg[t2], yw) / O.rms(yw)
    assert chain_rms <= 2e-2, chain_rms
    report_line(f"C2 MLP M={m}: swiglu act {act} metric {worst_h:.2e}; down act {act_d} conformance {e[0]:.2e}, "
                f"max|d|/rms {e[1]:.2e}; whole MLP vs oracle chain: rms error {chain_rms:.2e}, max {chain_max:.2e} of rms")


# ---- config 3: FP8 rows and Q4_K on [14336, 4096] --------------------------------------------------

@pytest.fixture(scope="module")
def c3(b):
    w = _weights(4, 14336, 4096)
    f8 = O.encode_fp8_row(w)
    q4 = O.encode_q4k(w)
    return f8, b.upload_bytes(f8), q4, b.upload_bytes(q4)


@pytest.mark.parametrize("m", [1, 512])
@pytest.mark.parametrize("policy", [ActPolicy.a16_only(), ActPolicy.allow_a8()], ids=["a16", "a8"])
def test_config3a_fp8_rows(b, c3, m, policy):
    f8, f8_dev, _, _ = c3
    _check_linear(b, f"C3a FP8 [14336,4096] M={m} policy {policy.kind}", F8, f8, f8_dev, 14336, 4096, m, policy)


@pytest.mark.parametrize("m", [1, 512])
def test_config3b_q4k(b, c3, m):
    _, _, q4, q4_dev = c3
    # held to the conformance metric at prefill width too, as the reference holds Q4_K
    # (crates/velox-conformance/src/lib.rs:3966)
    _check_linear(b, f"C3b Q4_K [14336,4096] M={m}", Q4, q4, q4_dev, 14336, 4096, m, ActPolicy.a16_only())
