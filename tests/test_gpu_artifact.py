"""From a container on disk to the kernels: open a .vi holding NVFP4, FP8-row and Q4_K matrices,
load bindings as views with the policies its `uses` state, run `linear` through the C ABI and
compare with the oracle on the very bytes the file holds."""
import numpy as np
import pytest

from oracle import oracle as O
from velox_inferer_b200.artifact import Artifact, Loader, PAGE

from .artifact_fixture import write_vi
from .gpu_util import ACT_O, backend, both_metrics

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m", [3, 70])
def test_linear_on_views_loaded_from_a_multi_part_vi(tmp_path, m):
    b = backend()
    path, mats = write_vi(str(tmp_path), part_limit=12 * PAGE)
    ld = Loader(b, Artifact.open(path))
    rng = np.random.default_rng(m)
    for name, oid in (("text/q", "w.qkv"), ("text/k", "w.qkv"), ("text/v", "w.qkv"), ("text/o", "w.o"),
                      ("text/down", "w.down")):
        view = ld.matrix(name)
        _, _, ofmt, n, k, payload = mats[oid]
        act = b.linear_act(view, m)
        assert act.permitted(view.act)
        x = rng.standard_normal((m, k)).astype(np.float32)
        y = b.alloc(m * view.rows)
        b.linear(b.upload(x), view, y, m)
        assert b.debug_status() == 0
        want = O.linear(x, payload, ofmt, n, k, view.row_begin, view.rows, m, act=ACT_O[act.kind], divisor=act.divisor)
        e_conf, e_rms = both_metrics(y.cpu().numpy().reshape(m, view.rows), want)
        assert e_conf <= 2e-4 and e_rms <= 1e-2, (name, act, e_conf, e_rms)
    assert len(ld.parents) == 3                            # q, k and v share one uploaded parent
