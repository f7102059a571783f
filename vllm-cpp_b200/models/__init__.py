"""Model descriptions (one file per architecture) and the generic decoder that runs them."""
from __future__ import annotations

import torch

from ..config.base import load_config_dict
from ..parts import BuildContext  # registers the parts
from ..registry import architecture_of, get_architecture
from . import qwen3  # registers Qwen3ForCausalLM
from .decoder import DecoderModel


def load_config(model_dir):
    """The typed configuration of a model folder, its class chosen by ``architectures[0]``."""
    data = load_config_dict(model_dir)
    return architecture_of(data).config_cls.from_dict(data)


def build_model(config, compute_dtype: torch.dtype, device) -> DecoderModel:
    arch = get_architecture(config.architecture)
    return DecoderModel(arch.describe(config), BuildContext(compute_dtype, torch.device(device)))


def expected_tensors(config):
    """Names, shapes and roles of every tensor a checkpoint of this configuration holds."""
    arch = get_architecture(config.architecture)
    model = DecoderModel(arch.describe(config), BuildContext(torch.float32, torch.device("cpu")))
    return model.tensor_specs()


__all__ = ["load_config", "build_model", "expected_tensors", "DecoderModel"]
