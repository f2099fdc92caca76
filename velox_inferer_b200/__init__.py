"""velox_inferer_b200: B200-native (sm_100a) kernels for velox-inferer's quantized linear path,
behind the reference's operator boundary. The CUDA library is mandatory: operators raise if it is
missing; nothing here computes on the CPU."""
from .errors import BackendError, ShapeError, Unsupported, VeloxError, device_lost
from .weights import (ActPolicy, ActQuant, LinearDst, LinearPart, WeightFormat, WeightView,
                      align256, check_linear, check_weight, nvfp4_scale_offset, swiglu_pair)


def build(verbose: bool = False) -> str:
    from . import _lib
    return _lib.build(verbose)


def __getattr__(name):
    if name == "Sm100Backend":
        from .backend import Sm100Backend
        return Sm100Backend
    if name in ("Artifact", "ArtifactError", "Loader", "write_container"):
        from . import artifact
        return getattr(artifact, name)
    if name in ("LinearStack", "StackSpec"):
        from . import stack
        return getattr(stack, name)
    raise AttributeError(name)
