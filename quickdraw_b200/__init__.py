"""B200-native batch-one decode path behind quickdraw's engine / kernel / kvcache surface.

Exports mirror the reference package (quickdraw/__init__.py:3-23); ``load_checkpoint`` is
not part of this package (weights are handed over as ``Checkpoint`` containers).
"""

from .weights import (Checkpoint, FP8Linear, FullAttnWeights, GDNWeights, LayerWeights,
                      ModelConfig, MoEWeights, NVFP4Linear)
from .state import DecodeState


def __getattr__(name):
    # Engine and the operator table need the CUDA library; load them on first use so the
    # containers stay importable for host-only tooling.
    if name == "Engine":
        from .engine import Engine
        return Engine
    if name == "bind_kernels":
        import importlib
        return importlib.import_module(".kernels", __name__).bind_kernels
    raise AttributeError(name)


__all__ = ["ModelConfig", "Checkpoint", "FP8Linear", "NVFP4Linear", "Engine", "DecodeState",
           "bind_kernels", "GDNWeights", "FullAttnWeights", "MoEWeights", "LayerWeights"]
