"""Multi-GPU checks of the fused tensor-parallel step (two GPUs, and four and eight where the box
has them; skipped on fewer). Ranks run as child processes with NVLS off."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


def _gpus() -> int:
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_tp_step_is_exact_and_matches_the_all_reduce_step(world):
    if _gpus() < world:
        pytest.skip(f"needs {world} GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
           "--master-addr", "127.0.0.1", "--master-port", str(29533 + world), os.path.join(here, "tp_fused_worker.py")]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=420, env=env)
    fail = out.stdout[out.stdout.find("TP_FUSED_FAIL"):][:3000] if "TP_FUSED_FAIL" in out.stdout else ""
    assert out.returncode == 0, fail + out.stdout[-1500:] + out.stderr[-1500:]
    assert "TP_FUSED_OK" in out.stdout
