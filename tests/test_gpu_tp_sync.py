"""The flag protocol of the tensor-parallel step on one GPU: flags are raised with the step's
epoch and accepted by the waits of the same step (rank count 1, everything stream-ordered), and a
wait on a flag nobody raises gives up after its limit, reports through the status word, and leaves
the device usable. No kernel here waits for another kernel: every signal precedes its wait in the
stream, and the wait that runs out has no signaller at all."""
import time

import numpy as np
import pytest
import torch

from oracle import oracle as O
from velox_inferer_b200 import ActPolicy, ActQuant, WeightFormat, _lib

from .gpu_util import FMT_O, backend, both_metrics, make_view, oracle_linear

pytestmark = pytest.mark.gpu
NV = WeightFormat.NVFP4


def _sync(flags, epoch, wait, signal):
    t = _lib.TpSync()
    t.flag_tables[0] = flags.data_ptr()
    t.epoch = epoch.data_ptr()
    t.n, t.rank, t.wait_phase, t.signal_phase = 1, 0, wait, signal
    return t


def test_single_rank_step_raises_and_accepts_flags():
    b = backend()
    r = O.Rng(71)
    m, dim, n = 256, 512, 512
    flags = torch.zeros(4 * 8, dtype=torch.int32, device=b.device)
    epoch = torch.zeros(1, dtype=torch.int32, device=b.device)
    payload = r.random_weight(FMT_O[NV], n, dim)
    view = make_view(b, payload, NV, n, dim, 0, n, ActPolicy.allow_a4(256.0))
    acc = b.upload(r.vec(m * dim, 1.0))
    ones = b.upload(np.ones(dim, np.float32))
    q4 = b.q4_blob(m, dim)
    slots = torch.zeros(m * n, dtype=torch.bfloat16, device=b.device)
    maps = torch.zeros(128, dtype=torch.uint8, device=b.device)
    b.tp_make_maps(maps, [slots.data_ptr()], m, n)
    want = torch.zeros(m * n, dtype=torch.bfloat16, device=b.device)
    for step in (1, 2):                                    # twice: the flags are never reset, the epoch moves on
        b.tp_step_begin(epoch)
        b.tp_norm_q4(acc, None, 0, 0, ones, [q4[0].data_ptr()], [q4[1].data_ptr()], 0, m, dim, 1e-6, 256.0,
                     sync=_sync(flags, epoch, -1, 0))
        slots.zero_()
        b.tp_linear_q4_scatter(q4, 256.0, view, m, maps, m, sync=_sync(flags, epoch, 0, 1))
        b.tp_wait(_sync(flags, epoch, 1, -1))
        torch.cuda.synchronize()
        assert b.debug_status() == 0
        assert int(epoch.item()) == step
        f = flags.cpu().numpy().reshape(4, 8)
        assert f[0, 0] == step and f[1, 0] == step and f[2:].sum() == 0 and f[:, 1:].sum() == 0
        b.linear_q4(q4, 256.0, view, None, m, yb=want)
        assert torch.equal(slots, want)                    # the scattering launch is the plain linear, stored elsewhere
    hb = O.quantize_activations(O.rms_norm(acc.cpu().numpy().reshape(m, dim), np.ones(dim, np.float32), 1e-6).reshape(-1),
                                dim, O.ACT_BF16).reshape(m, dim)
    ref = oracle_linear(hb, payload, NV, n, dim, 0, n, m, ActQuant(ActQuant.NVFP4, 256.0))
    assert both_metrics(slots.float().cpu().numpy().reshape(m, n), ref)[0] <= 2.0 ** -8     # bf16 output


def test_a_wait_nobody_answers_gives_up_and_the_status_can_be_cleared():
    b = backend()
    flags = torch.zeros(2 * 8, dtype=torch.int32, device=b.device)
    epoch = torch.ones(1, dtype=torch.int32, device=b.device)      # step 1; no flag has reached it
    assert b.lib.velox_sm100_tp_set_wait_limit_ms(50) == 0
    try:
        t0 = time.time()
        b.tp_wait(_sync(flags, epoch, 1, -1))
        torch.cuda.synchronize()
        assert time.time() - t0 < 5.0
        assert b.debug_status() == 6                       # a peer's flag did not arrive
        assert b.debug_status() == 6                       # sticky until cleared
        b.debug_status_reset()
        assert b.debug_status() == 0
        # a prefill linear that waits on the same dead flag: gives up, says so, and exits normally
        r = O.Rng(73)
        m, k, n = 130, 256, 256
        payload = r.random_weight(FMT_O[NV], n, k)
        view = make_view(b, payload, NV, n, k, 0, n, ActPolicy.allow_a4(256.0))
        q4 = b.q4_blob(m, k)
        acc = b.upload(r.vec(m * k, 1.0))
        hb = torch.zeros(m * k, dtype=torch.bfloat16, device=b.device)
        b.add_rms_norm_q4(acc, None, b.upload(np.ones(k, np.float32)), hb, q4, m, k, 1e-6, 256.0)
        yb = torch.zeros(m * n, dtype=torch.bfloat16, device=b.device)
        b.tp_linears_q4(q4, 256.0, [(view, yb, None, 0.0)], m, _sync(flags, epoch, 1, -1))
        torch.cuda.synchronize()
        assert b.debug_status() != 0
        b.debug_status_reset()
    finally:
        assert b.lib.velox_sm100_tp_set_wait_limit_ms(2000) == 0
    # the device and the library are fine afterwards: the same linear without the dead wait is right
    b.linear_q4(q4, 256.0, view, None, m, yb=yb)
    torch.cuda.synchronize()
    assert b.debug_status() == 0
    ref = oracle_linear(hb.float().cpu().numpy(), payload, NV, n, k, 0, n, m, ActQuant(ActQuant.NVFP4, 256.0))
    assert both_metrics(yb.float().cpu().numpy().reshape(m, n), ref)[0] <= 2.0 ** -8        # bf16 output
