"""Every tile of large prefill products, checked on the device: the NVFP4 GEMM against a plain f32
matrix product of the exactly decoded operands (decoded activations x decoded weights; the decoders
are bit-exact against the oracle in test_gpu_parity), over all token tiles and row tiles, repeated.

Why on top of the oracle subsets of test_gpu_configs: a persistent CTA walks many tiles of such a
product, and a hand-over inside its pipeline that is only wrong some of the time shows up as a few
tiles in a few runs. An earlier form of the scale ring did exactly that (a bulk copy could land
in a stage while a lane's read of it was still in flight): no test of a few tiles per CTA saw it."""
import numpy as np
import pytest
import torch

from velox_inferer_b200 import ActPolicy, WeightFormat, WeightView

from .gpu_util import backend

pytestmark = pytest.mark.gpu
NV = WeightFormat.NVFP4


def _blob_values(b, q4, m, k, div):
    """The values an NVFP4 activation blob stands for, through the weight decoder (same layout)."""
    plane = (m * k // 2 + 255) // 256 * 256
    buf = torch.zeros(plane + m * k // 16 + 256, dtype=torch.uint8, device=b.device)
    buf[: m * k // 2] = q4[0][: m * k // 2]
    buf[plane:plane + m * k // 16] = q4[1][: m * k // 16]
    buf[plane + m * k // 16:plane + m * k // 16 + 4] = torch.tensor(
        np.frombuffer(np.float32(div).tobytes(), dtype=np.uint8).copy(), device=b.device)
    return b.dequant_rows(WeightView.full(buf, NV, m, k))


@pytest.mark.parametrize("n,k,m,div,reps", [
    (25600, 5120, 2048, 256.0, 3),      # 800 pair tiles, eleven per CTA pair
    (5120, 25600, 2048, 16.0, 3),       # 100 k-blocks per tile
    (25600, 5120, 256, 256.0, 3),       # one pair tile per row tile: second tiles of some pairs
    (8192, 5120, 128, 256.0, 2),        # a CTA alone per tile
])
def test_every_tile_of_a_large_nvfp4_product(n, k, m, div, reps):
    b = backend()
    torch.backends.cuda.matmul.allow_tf32 = False
    gen = torch.Generator(device=b.device).manual_seed(n + k + m)
    w = torch.randn(n, k, generator=gen, device=b.device) * 0.02
    view = WeightView.full(b.encode_nvfp4(w), NV, n, k).with_act(ActPolicy.allow_a4(div))
    del w
    x = torch.randn(m, k, generator=gen, device=b.device).to(torch.bfloat16).float()
    codes, atoms = b.quantize_act_nvfp4(x, div)
    q4 = (codes.reshape(-1), atoms)
    ref = _blob_values(b, q4, m, k, div) @ b.dequant_rows(view).t()
    rms = float(ref.pow(2).mean().sqrt())
    for rep in range(reps):
        y = b.alloc(m * n)
        b.linear_q4(q4, div, view, y, m)
        torch.cuda.synchronize()
        assert b.debug_status() == 0
        err = (y.view(m, n) - ref).abs() / rms
        tiles = err.view(m // 128, 128, n // 256, 256).amax(dim=(1, 3))
        bad = (tiles > 1e-4).nonzero().tolist()
        assert not bad, (rep, len(bad), bad[:8], float(tiles.max()))
        del y
    # the bf16 output through the tile stores of the same launch
    yb = torch.zeros(m * n, dtype=torch.bfloat16, device=b.device)
    b.linear_q4(q4, div, view, None, m, yb=yb)
    torch.cuda.synchronize()
    rel = ((yb.view(m, n).float() - ref).abs() / (1.0 + ref.abs())).max()
    assert float(rel) <= 2.0 ** -8, float(rel)
