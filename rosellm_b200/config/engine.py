"""Options of the engine itself (not of a model): cache size, batch limits, precision.

The reference passes these as keyword arguments of ``InferenceEngine.__init__``
(rosellm/roseinfer/engine.py:88-113: ``kv_cache_max_tokens``,
``kv_cache_max_concurrency``, ``max_position_embeddings`` ...) and of its
schedulers (``max_batch_size``, ``prefill_chunk_size``,
rosellm/roseinfer/engine.py:3531-3560).
"""
from __future__ import annotations

from dataclasses import dataclass

from .base import ConfigError

DTYPE_NAMES = {
    "bfloat16": "bfloat16",
    "bf16": "bfloat16",
    "float32": "float32",
    "fp32": "float32",
}


@dataclass(frozen=True)
class EngineConfig:
    dtype: str = "bfloat16"
    """``bfloat16``: the serving path.  ``float32``: every product and sum in IEEE 32-bit."""
    page_size: int = 16
    """Tokens per cache page (the reference fixes 64, rosellm/roseinfer/engine.py:230)."""
    num_pages: int | None = None
    """Pages in the pool of each layer group.  The pool's size is given once: by this, by
    ``kv_cache_tokens``, by ``kv_cache_mem_fraction`` or by ``gpu_memory_utilization``; with
    none of them it is ``max_num_seqs * max_model_len`` tokens like the reference's default
    (rosellm/roseinfer/engine.py:316-317).  The arithmetic is in ``rosellm_b200/cache/sizing.py``."""
    kv_cache_tokens: int | None = None
    """Tokens the pool holds (the reference's ``kv_cache_max_tokens``), rounded up to whole pages."""
    gpu_memory_utilization: float | None = None
    """Share of the whole device that the engine may fill: the cache gets what is left of it
    once the weights are loaded, ``(total * utilization - used) / bytes per token``
    (rosellm/roseinfer/engine.py:25-51, 296-314)."""
    kv_cache_mem_fraction: float | None = None
    """Share of the memory that is free after the weights are loaded
    (rosellm/roseinfer/engine.py:278-295)."""
    max_num_seqs: int = 64
    """Requests live at once (rows of the block table, state slots)."""
    max_num_batched_tokens: int = 2048
    """Token budget of one step: decoded tokens plus prompt portions."""
    prefill_chunk_size: int = 512
    """Longest prompt portion one request contributes to a step."""
    max_model_len: int | None = None
    """Longest sequence; ``None`` takes the model's own limit."""
    cuda_graphs: bool = True
    """Replay decode-only steps from captured CUDA graphs."""
    capture_graphs_at_start: bool = True
    """Capture the graph of every batch-size bucket when the engine is built; otherwise the
    first step that needs a bucket captures it (and takes a few milliseconds longer)."""
    reuse_launch_lists: bool = True
    """A step that is not replayed from a CUDA graph notes its library calls; a later step of
    the same sizes issues them again without walking through the parts (the calls depend on the
    sizes, the contents lie in device buffers)."""
    seed: int = 0
    """Base of the random streams of requests that bring no seed of their own: such a
    request's seed is derived from this, its id and its prompt's length, the same in every run."""
    device: str = "cuda:0"

    def __post_init__(self) -> None:
        if self.dtype not in DTYPE_NAMES:
            raise ConfigError(f"dtype must be one of {sorted(DTYPE_NAMES)}, got {self.dtype!r}")
        object.__setattr__(self, "dtype", DTYPE_NAMES[self.dtype])
        if self.page_size <= 0:
            raise ConfigError("page_size must be positive")
        for name in ("max_num_seqs", "max_num_batched_tokens", "prefill_chunk_size"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"{name} must be positive")
        sized = [n for n in ("num_pages", "kv_cache_tokens", "gpu_memory_utilization", "kv_cache_mem_fraction")
                 if getattr(self, n) is not None]
        if len(sized) > 1:
            raise ConfigError(f"the cache's size is given {len(sized)} times ({', '.join(sized)}); give one")
        for name in ("num_pages", "kv_cache_tokens"):
            if getattr(self, name) is not None and getattr(self, name) <= 0:
                raise ConfigError(f"{name} must be positive")
        for name in ("gpu_memory_utilization", "kv_cache_mem_fraction"):
            v = getattr(self, name)
            if v is not None and not 0.0 < v <= 1.0:
                raise ConfigError(f"{name} must be in (0, 1]")
