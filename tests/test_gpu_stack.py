"""The layer stack on one GPU against the oracle running the identical op sequence with the
roundings the kernels declare (bf16 twins between ops, NVFP4 activations with the per-use
divisors at prefill width, bf16 partial sums)."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from velox_inferer_b200 import ActQuant
from velox_inferer_b200.stack import DIV_DOWN_IN, DIV_NORM_OUT, DIV_O_IN, LinearStack, StackSpec

from .gpu_util import backend

pytestmark = pytest.mark.gpu


def _bf16(a):
    return O.quantize_activations(np.asarray(a, dtype=np.float32).reshape(-1), 1, O.ACT_BF16).reshape(np.shape(a))


def _oracle_stack(b, stack, spec, x, m):
    def lin(inp, view, div):
        n, k = view.parent_rows, view.k
        payload = view.buf.cpu().numpy()
        act = b.linear_act(view, m)                       # the rounding the backend declares
        assert act.kind in (ActQuant.NVFP4, ActQuant.BF16)
        if act.kind == ActQuant.NVFP4:
            assert act.divisor == div
            return O.linear(inp, payload, O.FMT_NVFP4, n, k, 0, n, m, act=O.ACT_NVFP4, divisor=div)
        return O.linear(inp, payload, O.FMT_NVFP4, n, k, 0, n, m, act=O.ACT_BF16, divisor=0.0)

    ones = np.ones(spec.hidden, dtype=np.float32)
    x = _bf16(x).astype(np.float32)
    pb = None
    for l in stack.layers:
        if pb is not None:
            x = (x + pb).astype(np.float32)
        hb = _bf16(O.rms_norm(x, ones, spec.norm_eps))
        qb = _bf16(lin(hb, l.q, DIV_NORM_OUT))
        kv = (_bf16(lin(hb, l.k, DIV_NORM_OUT)), _bf16(lin(hb, l.v, DIV_NORM_OUT)))
        pb = _bf16(lin(qb, l.o, DIV_O_IN))
        x = (x + pb).astype(np.float32)
        hb = _bf16(O.rms_norm(x, ones, spec.norm_eps))
        g, u = lin(hb, l.gate, DIV_NORM_OUT), lin(hb, l.up, DIV_NORM_OUT)
        gb = _bf16(O.swiglu(np.concatenate([g, u], axis=1), m, 2 * g.shape[1], 0, g.shape[1], g.shape[1]))
        pb = _bf16(lin(gb, l.down, DIV_DOWN_IN))
    return _bf16((x + pb).astype(np.float32)), kv


@pytest.mark.parametrize("m", [3, 40, 200])
def test_stack_matches_oracle_sequence(m):
    b = backend()
    spec = StackSpec(layers=2, hidden=256, intermediate=512, heads=2, kv_heads=1, head_dim=128)
    stack = LinearStack(b, spec, max_tokens=m, a4=True, seed=3)
    x = np.random.default_rng(m).standard_normal((m, spec.hidden)).astype(np.float32)
    xb = torch.from_numpy(x).to(torch.bfloat16).to(b.device)
    out = stack.forward(xb, m)
    torch.cuda.synchronize()
    assert b.lib.velox_sm100_debug_status() == 0
    got = out[: m * spec.hidden].float().cpu().numpy().reshape(m, spec.hidden)
    want, (want_k, want_v) = _oracle_stack(b, stack, spec, xb.float().cpu().numpy(), m)
    # every stage rounds to bf16 (2^-9 relative); two layers of it stay within a few bf16 ulps
    err = O.max_abs_diff(got, want) / O.rms(want)
    assert err <= 2e-2, err
    assert np.mean(np.abs(got - want) <= 2.0 ** -7 * (np.abs(want) + 0.05)) > 0.999
    # the k and v projections of the last layer (they feed nothing further in this stack): same launch
    # as q, checked on their own
    for buf, want_p in ((stack.kb, want_k), (stack.vb, want_v)):
        got_p = buf[: m * spec.kv_dim].float().cpu().numpy().reshape(m, spec.kv_dim)
        assert O.max_abs_diff(got_p, want_p) / O.rms(want_p) <= 2e-2
        assert np.mean(np.abs(got_p - want_p) <= 2.0 ** -7 * (np.abs(want_p) + 0.05)) > 0.999
