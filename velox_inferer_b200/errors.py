"""Error convention of the reference (crates/velox-core/src/error.rs:4-45,
crates/velox-cuda/src/lib.rs:85-112): launcher return codes become exceptions; sticky CUDA
errors mark the device lost for the whole process."""
from __future__ import annotations


class VeloxError(Exception):
    pass


class ShapeError(VeloxError):
    """``Error::Shape``: arguments every backend must reject (check.rs)."""


class Unsupported(VeloxError):
    """``Error::Unsupported``: this kernel set does not serve the shape; callers fall back."""


class BackendError(VeloxError):
    """``Error::Backend``: a CUDA error code from a launcher."""


_STICKY = {700, 702, 709, 710, 714, 715, 716, 717, 718, 719, 999}
_device_lost: str | None = None


def device_lost() -> str | None:
    return _device_lost


def status(code: int, what: str) -> None:
    """``status()`` of crates/velox-cuda/src/lib.rs:96-112."""
    global _device_lost
    if code == 0:
        return
    if code == -1:
        raise Unsupported(f"{what}: shape not supported by this kernel")
    if code == -2:
        raise ShapeError(f"{what}: arguments rejected")
    msg = f"{what}: CUDA error {code}"
    if code in _STICKY:
        _device_lost = msg
    raise BackendError(msg)
