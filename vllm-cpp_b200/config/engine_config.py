"""Options of the engine (not of the model).

Counterpart of the reference's PagedEngine constructor arguments
(src/paged_engine.h:26-30: max_num_seqs, max_total_tokens, num_gpu_blocks)
and of its global BLOCK_SIZE (src/config.h:48), as explicit options.
"""
from __future__ import annotations

from dataclasses import dataclass

from .base import ConfigError

DTYPES = {"bfloat16": "bfloat16", "bf16": "bfloat16", "float32": "float32", "fp32": "float32"}


@dataclass(frozen=True)
class EngineConfig:
    dtype: str = "bfloat16"            # "bfloat16": serving kernels; "float32": everything in true 32-bit
    page_size: int = 16                # tokens per cache page (the reference's BLOCK_SIZE)
    max_tokens: int = 8192             # tokens the cache pool holds (the reference's --max-tokens)
    max_num_seqs: int = 4              # live requests (the reference's --max-batch)
    max_step_tokens: int = 2048        # token budget of one step
    max_model_len: int | None = None   # longest request; default: the model's max positions
    device: str = "cuda:0"
    cuda_graphs: bool = True           # replay decode-only steps from captured graphs
    profile: bool = False              # time the groups of kernels of every step (embedding, each layer's mixer and
                                       # feed-forward, head, sampling) with CUDA events; steps then run kernel by kernel

    def __post_init__(self):
        if self.dtype not in DTYPES:
            raise ConfigError(f"dtype '{self.dtype}' is not one of {sorted(DTYPES)}")
        object.__setattr__(self, "dtype", DTYPES[self.dtype])
        for name in ("page_size", "max_tokens", "max_num_seqs", "max_step_tokens"):
            if getattr(self, name) < 1:
                raise ConfigError(f"{name} must be >= 1")
        if self.max_tokens % self.page_size:
            raise ConfigError(f"max_tokens={self.max_tokens} must be a multiple of page_size={self.page_size}")

    @property
    def num_pages(self) -> int:
        return self.max_tokens // self.page_size
