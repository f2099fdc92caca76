"""The reference's conformance cases of the linear family, for the three formats this kernel set
executes, replayed through the C ABI: same shapes, row views, token counts, policies and the 2e-4
bound of `velox selftest` (crates/velox-conformance/src/lib.rs:3219-3365 linear / linear_act,
3843-3875 prefill grids and fused SwiGLU, 3909-3939 linears, 3962-3970 GGML blocks, 4153-4176 Q4_K
at K = 2560). Data follows the suite's recipe (`random_weight`, `vec` of the xorshift generator) on a
seed per case; as there, the oracle rounds x the way the backend says it does (`linear_act`), and a
rounding the policy forbids fails whatever the numbers say."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from velox_inferer_b200 import ActPolicy, LinearDst, LinearPart, WeightFormat, WeightView

from .gpu_util import FMT_O, backend, make_view, oracle_linear

pytestmark = pytest.mark.gpu
TOL = 2e-4
NV, F8, Q4 = WeightFormat.NVFP4, WeightFormat.FP8_ROW_BF16, WeightFormat.GGML_Q4_K
A16, A8, A4 = ActPolicy.a16_only(), ActPolicy.allow_a8(), ActPolicy.allow_a4(600.0)


@pytest.fixture(scope="module")
def b():
    return backend()


LINEAR_CASES = (
    # lib.rs:3223-3231, 3253-3255: plain `linear` (A16Only views)
    [(F8, *c, A16) for c in [(96, 300, 10, 40, 1), (64, 512, 0, 64, 9), (160, 1024, 16, 128, 24), (96, 512, 0, 96, 40),
                             (64, 768, 0, 64, 64), (64, 512, 0, 64, 90), (200, 300, 17, 150, 70)]]
    + [(NV, *c, A16) for c in [(256, 320, 0, 256, 33), (256, 128, 0, 256, 1), (384, 192, 128, 200, 5)]]
    # :3258-3273 NVFP4 under AllowA4{600}; :3274-3293 FP8 rows under AllowA8; :3294-3328 A16-only windows
    + [(NV, *c, A4) for c in [(256, 512, 0, 256, 16), (384, 640, 128, 256, 37), (512, 1024, 0, 512, 130),
                              (256, 256, 128, 128, 300), (128, 64, 0, 128, 1), (512, 2048, 128, 384, 8),
                              (384, 640, 128, 256, 8), (256, 1024, 64, 192, 3)]]
    + [(F8, *c, A8) for c in [(256, 512, 0, 256, 16), (200, 320, 17, 150, 70), (512, 1024, 64, 384, 130),
                              (96, 300, 0, 96, 40), (64, 128, 0, 64, 2), (512, 2048, 64, 384, 8), (300, 192, 0, 300, 5)]]
    + [(NV, *c, A16) for c in [(512, 2048, 64, 384, 8), (256, 5120, 0, 256, 16), (384, 1024, 128, 192, 2),
                               (256, 512, 0, 256, 64)]]
    + [(F8, 256, 512, 0, 256, 64, A16)]
    # :3366-3375 batched drafting with A16-only NVFP4
    + [(NV, 384, 1024, 64, 256, m, A16) for m in (21, 42, 48, 96)]
    # :3847-3854 prefill widths: a view starting mid-tile with ragged rows, a full chunk, several hundred tiles
    + [(NV, 384, 512, 40, 300, 100, A16), (NV, 256, 448, 0, 256, 1030, A16),
       (NV, 8448, 256, 128, 8200, 1030, A4), (F8, 8448, 256, 64, 8200, 1030, A8)]
    # :3962-3966 GGML blocks: decode, a verify window over an odd row view, the tiled path
    + [(Q4, *c, A16) for c in [(96, 512, 0, 96, 1), (130, 768, 3, 100, 8), (72, 512, 0, 72, 16), (200, 256, 17, 150, 33)]]
    # :4153-4176 Q4_K with K = 2560 under AllowA8
    + [(Q4, 96, 2560, 0, 96, m, A8) for m in (1, 3, 8, 70, 300, 600)]
)


def _id(c):
    fmt, n, k, begin, rows, m, pol = c
    return f"{fmt.format_name}-{n}x{k}-{begin}+{rows}-m{m}-p{pol.kind}"


@pytest.mark.parametrize("case", LINEAR_CASES, ids=_id)
def test_linear_cases(b, case):
    fmt, n, k, begin, rows, m, policy = case
    r = O.Rng(hash((int(fmt), n, k, begin, rows, m, policy.kind)) & 0x7FFFFFFF)
    payload = r.random_weight(FMT_O[fmt], n, k)
    x = r.vec(m * k, 1.0)
    view = make_view(b, payload, fmt, n, k, begin, rows, policy)
    act = b.linear_act(view, m)
    assert act.permitted(policy), f"rounding {act} not permitted under {policy}"
    want = oracle_linear(x, payload, fmt, n, k, begin, rows, m, act)
    y = b.alloc(m * rows)
    b.linear(b.upload(x), view, y, m)
    assert b.debug_status() == 0
    assert O.max_err(y.cpu().numpy(), want.reshape(-1)) <= TOL, (act, O.max_err(y.cpu().numpy(), want.reshape(-1)))


# lib.rs:3329-3364: a drafter's NVFP4 MLP (hidden 2048, width 6144) at every block width of a draft window
@pytest.mark.parametrize("m", range(1, 10))
def test_drafter_mlp_widths(b, m):
    for n, k in ((6144, 2048), (2048, 6144)):
        test_linear_cases(b, (NV, n, k, 0, n, m, A16))
    _swiglu_case(b, NV, 2048, 6144, 0, m, False, False, A16)


def _swiglu_case(b, fmt, k, width, begin, m, swap, split, policy):
    """`linear_swiglu_with` (lib.rs:786-880): gate and up of `width` rows from `begin`, in one parent
    (either order) or two."""
    n = (begin + 2 * width + 16 + 127) // 128 * 128
    r = O.Rng(hash((int(fmt), k, width, begin, m, swap, split, policy.kind)) & 0x7FFFFFFF)
    p1, p2 = r.random_weight(FMT_O[fmt], n, k), r.random_weight(FMT_O[fmt], n, k)
    x = r.vec(m * k, 1.0)
    gb, ub = (begin + width, begin) if swap else (begin, begin + width)
    gate = make_view(b, p1, fmt, n, k, gb, width, policy)
    up = make_view(b, p2, fmt, n, k, ub, width, policy) if split else gate.rows_view(ub - gb, width)
    act = b.linear_swiglu_act(gate, up, m)
    assert act.permitted(policy)
    g = oracle_linear(x, p1, fmt, n, k, gb, width, m, act)
    u = oracle_linear(x, p2 if split else p1, fmt, n, k, ub, width, m, act)
    want = O.silu_mul(g, u)
    out = b.alloc(m * width)
    b.linear_swiglu(b.upload(x), gate, up, out, m)
    assert b.debug_status() == 0
    assert O.max_err(out.cpu().numpy(), want.reshape(-1)) <= TOL, (act, O.max_err(out.cpu().numpy(), want.reshape(-1)))


@pytest.mark.parametrize("fmt,k,width,begin,m,swap,split,policy", [
    # lib.rs:3858-3875: fused SwiGLU under A4 / A8 at prefill widths
    (NV, 512, 256, 0, 100, False, False, A4), (NV, 256, 128, 128, 300, True, False, A4),
    (NV, 256, 256, 0, 70, False, True, A4), (NV, 256, 4096, 0, 1030, False, False, A4),
    (F8, 256, 192, 0, 130, False, True, A8), (F8, 320, 200, 17, 300, True, False, A8),
    (F8, 128, 4096, 0, 1030, False, True, A8),
    # lib.rs:3968: GGML blocks, separate parents, two tokens
    (Q4, 512, 24, 0, 2, False, True, A16),
])
def test_fused_swiglu_cases(b, fmt, k, width, begin, m, swap, split, policy):
    _swiglu_case(b, fmt, k, width, begin, m, swap, split, policy)


def test_embed_case(b):
    """lib.rs:3967, 1059-1077: rows 11, 0, 5 of a [12, 512] Q4_K table, decoded exactly (1e-6)."""
    for fmt, n, k in ((Q4, 12, 512), (F8, 12, 512), (NV, 128, 512)):
        r = O.Rng(0xe3bed + int(fmt))
        payload = r.random_weight(FMT_O[fmt], n, k)
        table = make_view(b, payload, fmt, n, k, 0, n)
        ids = [11, 0, 5]
        out = b.alloc(len(ids) * k)
        b.embed(ids, table, out)
        want = np.concatenate([O.decode_rows(FMT_O[fmt], payload, n, k, i, 1) for i in ids])
        assert np.array_equal(out.cpu().numpy().view(np.uint32), want.reshape(-1).view(np.uint32))
    # device ids are not checked by the host: a row that does not exist decodes to zeros
    dev_ids = torch.tensor([3, 4000, 1], dtype=torch.int32, device=b.device)
    out = b.alloc(3 * k)
    b.embed_from(dev_ids, 0, 3, table, out)
    got = out.cpu().numpy().reshape(3, k)
    assert np.array_equal(got[0], O.decode_rows(FMT_O[fmt], payload, n, k, 3, 1)[0]) and not got[1].any()


def test_matmul_cases(b):
    """lib.rs:3215-3220 `matmul` shapes (here a spread of tile edges) and velox-cpu's own known answer
    (crates/velox-cpu/src/lib.rs:1264-1271)."""
    y = b.alloc(4)
    b.matmul(b.upload([1, 2, 3, 4, 5, 6]), b.upload([1, 0, 0, 0, 1, 1]), y, 2, 2, 3)
    assert y.cpu().tolist() == [1.0, 5.0, 4.0, 11.0]
    r = O.Rng(0x3a7)
    for m, n, k in ((1, 1, 1), (3, 5, 7), (2, 33, 130), (70, 65, 300), (130, 257, 64)):
        x, w = r.vec(m * k, 1.0), r.vec(n * k, 1.0)
        y = b.alloc(m * n + 1)
        b.matmul(b.upload(x), b.upload(w), y, m, n, k)
        got = y.cpu().numpy()
        assert got[-1] == 0.0
        assert O.max_err(got[:-1], O.matmul(x.reshape(m, k), w.reshape(n, k)).reshape(-1)) <= 1e-5


@pytest.mark.parametrize("m", [1, 8, 70, 130])
def test_linears_cases(b, m):
    """lib.rs:3909-3939 `linears`: runs into column ranges of destinations with two spare columns that
    must stay zero, several destinations, parts that are views of shared parents; the formats here
    are this kernel set's."""
    k = 512
    layout = [[(NV, 256, 0, 128), (F8, 192, 64, 96)], [(Q4, 160, 32, 128)], [(NV, 256, 128, 128), (NV, 128, 8, 24)]]
    r = O.Rng(0x11ea5 + m)
    x = r.vec(m * k, 1.0)
    dsts, wants = [], []
    for parts in layout:
        ld = sum(rows for _, _, _, rows in parts) + 2
        y = b.alloc(m * ld)
        lps, col, want = [], 0, np.zeros((m, ld), np.float32)
        for fmt, n, begin, rows in parts:
            payload = r.random_weight(FMT_O[fmt], n, k)
            view = make_view(b, payload, fmt, n, k, begin, rows, A8)
            act = b.linear_act(view, m)
            assert act.permitted(A8)
            want[:, col:col + rows] = oracle_linear(x, payload, fmt, n, k, begin, rows, m, act)
            lps.append(LinearPart(view, col))
            col += rows
        dsts.append(LinearDst(y, ld, lps))
        wants.append(want)
    b.linears(b.upload(x), None, dsts, m)
    assert b.debug_status() == 0
    for d, want in zip(dsts, wants):
        got = d.y.cpu().numpy().reshape(m, d.ld)
        assert not got[:, -2:].any()
        assert O.max_err(got, want) <= TOL
