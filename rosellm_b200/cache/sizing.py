"""How large the page pools are made.

The reference sizes its cache in tokens (rosellm/roseinfer/engine.py:276-333):
an explicit ``kv_cache_max_tokens``; or a fraction of the memory that is free
when the engine is built, ``free * kv_cache_mem_fraction / bytes_per_token``;
or what is left of a share of the whole device, ``(total *
gpu_memory_utilization - used) / bytes_per_token`` (helper at engine.py:25-51);
or ``max_context * max_concurrency``.  ``bytes_per_token`` is ``layers * 2 *
heads * head_dim * element size``.  When a sequence's share of the pool
(``tokens // max_concurrency``) is shorter than the context, the reference
shortens the context to it with a warning (engine.py:319-329).

Here the same arithmetic runs over the layer groups of the model (a token
costs the sum over all layers that keep keys and values, whatever group they
are in), and an explicit number of pages is one more way to say the size.
The context is shortened only when the size was derived from memory: a pool
whose size the caller gave may be smaller than ``max_num_seqs`` whole
contexts on purpose (the scheduler preempts when pages run out, and refuses
a request that could never fit).

Everything here is plain arithmetic on numbers the caller passes in, so it is
tested without a GPU.
"""
from __future__ import annotations

from dataclasses import dataclass

ELEMENT_BYTES = {"bfloat16": 2, "float32": 4}


def kv_bytes_per_token(kv_specs, dtype: str) -> int:
    """Bytes of keys and values that one cached token takes over all layers
    (``kv_specs``: the ``KVCacheSpec`` of every layer that writes a cache)."""
    specs = kv_specs.values() if hasattr(kv_specs, "values") else kv_specs
    return sum(2 * s.num_kv_heads * s.head_dim * ELEMENT_BYTES[dtype] for s in specs)


def tokens_from_total_utilization(free_bytes: int, total_bytes: int, gpu_memory_utilization: float,
                                  bytes_per_token: int) -> int:
    """``(total * utilization - used) // bytes_per_token``: the cache gets what is left of the
    share of the device that the engine may use (rosellm/roseinfer/engine.py:25-51)."""
    if total_bytes <= 0 or not 0 <= free_bytes <= total_bytes:
        raise ValueError(f"free {free_bytes} and total {total_bytes} bytes do not describe a device")
    if not 0.0 < gpu_memory_utilization <= 1.0:
        raise ValueError("gpu_memory_utilization must be in (0, 1]")
    if bytes_per_token <= 0:
        raise ValueError("bytes_per_token must be positive")
    used = total_bytes - free_bytes
    budget = int(total_bytes * gpu_memory_utilization) - used
    if budget <= 0:
        raise ValueError(
            f"gpu_memory_utilization {gpu_memory_utilization} of {total_bytes} bytes leaves nothing for the cache: "
            f"{used} bytes are in use already"
        )
    return max(1, budget // bytes_per_token)


def tokens_from_free_fraction(free_bytes: int, kv_cache_mem_fraction: float, bytes_per_token: int) -> int:
    """``free * fraction // bytes_per_token`` (rosellm/roseinfer/engine.py:278-295)."""
    if not 0.0 < kv_cache_mem_fraction <= 1.0:
        raise ValueError("kv_cache_mem_fraction must be in (0, 1]")
    if bytes_per_token <= 0:
        raise ValueError("bytes_per_token must be positive")
    return max(1, int(free_bytes * kv_cache_mem_fraction) // bytes_per_token)


@dataclass(frozen=True)
class CachePlan:
    num_pages: int
    max_model_len: int
    how: str  # which rule gave the size
    clamped_from: int | None = None  # the context before it was shortened, if it was


def plan_cache(*, page_size: int, max_num_seqs: int, max_model_len: int, bytes_per_token: int,
               num_pages: int | None = None, kv_cache_tokens: int | None = None,
               gpu_memory_utilization: float | None = None, kv_cache_mem_fraction: float | None = None,
               mem_get_info=None, reserve_bytes: int = 0) -> CachePlan:
    """Pages of the pool and the longest sequence, from the engine's options.

    Precedence: ``num_pages``, ``kv_cache_tokens``, ``kv_cache_mem_fraction``,
    ``gpu_memory_utilization``, else ``max_num_seqs * max_model_len`` tokens.
    ``mem_get_info``: a callable returning (free, total) bytes of the device, asked only by the
    two rules that read memory, after the weights are on the device.  ``reserve_bytes`` is taken
    off the free memory first (state slots, workspace).
    """
    given = [n for n, v in (("num_pages", num_pages), ("kv_cache_tokens", kv_cache_tokens),
                            ("kv_cache_mem_fraction", kv_cache_mem_fraction),
                            ("gpu_memory_utilization", gpu_memory_utilization)) if v is not None]
    if len(given) > 1:
        raise ValueError(f"the cache's size is given {len(given)} times ({', '.join(given)}); give one")
    if num_pages is not None:
        if num_pages <= 0:
            raise ValueError("num_pages must be positive")
        return CachePlan(int(num_pages), max_model_len, "num_pages")
    if kv_cache_tokens is not None:
        if kv_cache_tokens <= 0:
            raise ValueError("kv_cache_tokens must be positive")
        return CachePlan(-(-int(kv_cache_tokens) // page_size), max_model_len, "kv_cache_tokens")
    if kv_cache_mem_fraction is None and gpu_memory_utilization is None:
        return CachePlan(-(-max_num_seqs * max_model_len // page_size), max_model_len, "max_num_seqs * max_model_len")
    if mem_get_info is None:
        raise ValueError("sizing the cache from memory needs a device to ask")
    free, total = mem_get_info()
    free = max(0, int(free) - int(reserve_bytes))
    if kv_cache_mem_fraction is not None:
        tokens, how = tokens_from_free_fraction(free, kv_cache_mem_fraction, bytes_per_token), "kv_cache_mem_fraction"
    else:
        tokens = tokens_from_total_utilization(free, int(total), gpu_memory_utilization, bytes_per_token)
        how = "gpu_memory_utilization"
    pages = max(1, tokens // page_size)  # whole pages that fit the budget
    per_seq = max(1, pages * page_size // max_num_seqs)
    if per_seq < max_model_len:
        return CachePlan(pages, per_seq, how, clamped_from=max_model_len)
    return CachePlan(pages, max_model_len, how)
