"""A small Qwen3 inference library for NVIDIA B200 (sm_100a): configuration, weights, a decoder
put together from parts, a paged sequence cache, one step function, a generation loop, sampling,
and hand-written CUDA kernels.

    from builderforce_inference_b200 import Model, SampleParams
    model = Model.load("/path/to/folder", dtype="bfloat16", max_tokens=65536)
    ids = model.generate_batch([[1, 2, 3], [4, 5]], SampleParams(max_tokens=32))
"""
from .config import ConfigError, Qwen3Config
from .registry import (Architecture, architecture_for, describe_model, register_architecture,
                       registered_architectures, unregister_architecture)
from .sampling import SampleParams
from .weights import WeightsError, write_model_folder

__all__ = ["ConfigError", "Qwen3Config", "Architecture", "architecture_for", "describe_model",
           "register_architecture", "registered_architectures", "unregister_architecture", "SampleParams",
           "WeightsError", "write_model_folder", "Engine", "SequenceStep", "Model", "registry"]


def registry():
    """Names of the registered architectures."""
    return registered_architectures()


def __getattr__(name):
    # the engine imports torch's CUDA side and the kernel libraries; load it on first use
    if name in ("Engine", "SequenceStep", "StepError"):
        from .engine import engine as _e
        return getattr(_e, name)
    if name in ("Model", "GreedyTrace"):
        from .engine import api as _a
        return getattr(_a, name)
    raise AttributeError(name)
