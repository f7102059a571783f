"""vllm_cpp_b200: a small, whole inference engine for one NVIDIA B200.

From a model folder (config.json + safetensors) to next tokens: typed configuration
and architecture registry, weights by name, layers assembled from parts, a paged
cache with per-request block tables and state slots, one step function for mixed
batches, a continuous-batching scheduler, device-side sampling, and hand-written
sm_100a kernels underneath.
"""
from .config import ConfigError, EngineConfig, Qwen3Config
from .registry import (LayerRun, LayerSpec, ModelSpec, PartSpec, register_architecture, register_part,
                       unregister_architecture, unregister_part)

__version__ = "0.1.0"


def __getattr__(name):
    # heavier pieces load on first use so that reading a configuration needs no GPU and no compiler
    if name in ("LLM", "EngineOutput"):
        from .engine import llm
        return getattr(llm, name)
    if name in ("ModelRunner", "StepEntry", "StepContext"):
        from .engine import step
        return getattr(step, name)
    if name in ("load_config", "build_model", "expected_tensors"):
        from . import models
        return getattr(models, name)
    if name in ("write_random_model", "open_model_weights", "WeightError"):
        from . import weights
        return getattr(weights, name)
    raise AttributeError(name)


__all__ = ["ConfigError", "EngineConfig", "Qwen3Config", "LLM", "EngineOutput", "ModelRunner", "StepEntry",
           "load_config", "build_model", "expected_tensors", "write_random_model", "open_model_weights",
           "PartSpec", "LayerSpec", "LayerRun", "ModelSpec", "register_architecture", "register_part",
           "unregister_architecture", "unregister_part"]
