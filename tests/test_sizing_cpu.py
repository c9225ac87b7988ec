"""The cache's size from the engine's options: plain arithmetic, with a made-up device."""
import pytest

from rosellm_b200.cache.sizing import (kv_bytes_per_token, plan_cache, tokens_from_free_fraction,
                                       tokens_from_total_utilization)
from rosellm_b200.config import ConfigError, EngineConfig
from rosellm_b200.parts.base import KVCacheSpec

GB = 1 << 30


def test_bytes_per_token_sums_over_layers_of_all_groups():
    specs = {0: KVCacheSpec(12, 64), 1: KVCacheSpec(12, 64), 2: KVCacheSpec(2, 32, window=128)}
    assert kv_bytes_per_token(specs, "bfloat16") == 2 * (2 * 12 * 64 * 2) + 2 * 2 * 32 * 2
    assert kv_bytes_per_token(specs, "float32") == 2 * kv_bytes_per_token(specs, "bfloat16")
    # GPT-2 124M: 12 layers x 2 x 768 x 2 bytes
    assert kv_bytes_per_token({i: KVCacheSpec(12, 64) for i in range(12)}, "bfloat16") == 36864


def test_the_reference_arithmetic():
    # (total * utilization - used) // bytes per token
    assert tokens_from_total_utilization(150 * GB, 180 * GB, 0.9, 36864) == (int(180 * GB * 0.9) - 30 * GB) // 36864
    assert tokens_from_free_fraction(100 * GB, 0.5, 36864) == 50 * GB // 36864
    with pytest.raises(ValueError, match="leaves nothing"):
        tokens_from_total_utilization(10 * GB, 180 * GB, 0.5, 36864)
    for bad in (0.0, 1.5):
        with pytest.raises(ValueError):
            tokens_from_total_utilization(1, 2, bad, 1)
        with pytest.raises(ValueError):
            tokens_from_free_fraction(1, bad, 1)


def common(**kw):
    base = dict(page_size=16, max_num_seqs=64, max_model_len=1024, bytes_per_token=36864)
    base.update(kw)
    return base


def test_precedence_and_defaults():
    never = lambda: (_ for _ in ()).throw(AssertionError("memory must not be asked"))
    p = plan_cache(**common(), mem_get_info=never)
    assert (p.num_pages, p.max_model_len, p.clamped_from) == (64 * 1024 // 16, 1024, None)
    assert plan_cache(**common(num_pages=77), mem_get_info=never).num_pages == 77
    assert plan_cache(**common(kv_cache_tokens=100), mem_get_info=never).num_pages == 7  # whole pages
    # a pool whose size the caller gave keeps the context, however small it is
    assert plan_cache(**common(kv_cache_tokens=64), mem_get_info=never).max_model_len == 1024
    with pytest.raises(ValueError, match="given 2 times"):
        plan_cache(**common(num_pages=1, kv_cache_tokens=16))


def test_sizes_from_memory_and_the_shortened_context():
    asked = []

    def device():
        asked.append(1)
        return 20 * GB, 180 * GB

    p = plan_cache(**common(kv_cache_mem_fraction=0.5), mem_get_info=device)
    assert p.num_pages == (10 * GB // 36864) // 16 and p.max_model_len == 1024 and asked == [1]
    p = plan_cache(**common(gpu_memory_utilization=0.9), mem_get_info=device, reserve_bytes=GB)
    assert p.num_pages == ((int(180 * GB * 0.9) - 161 * GB) // 36864) // 16
    # too little memory for 64 whole contexts: every sequence gets its share, as in the reference
    small = plan_cache(**common(kv_cache_mem_fraction=0.5), mem_get_info=lambda: (2 * GB, 180 * GB))
    tokens = small.num_pages * 16
    assert tokens < 64 * 1024 and small.max_model_len == tokens // 64 and small.clamped_from == 1024
    with pytest.raises(ValueError, match="needs a device"):
        plan_cache(**common(gpu_memory_utilization=0.5))


def test_engine_config_checks_the_options():
    ec = EngineConfig(num_pages=12, seed=5)
    assert (ec.num_pages, ec.seed, ec.kv_cache_tokens) == (12, 5, None)
    for kw in (dict(num_pages=0), dict(gpu_memory_utilization=1.2), dict(kv_cache_mem_fraction=0.0),
               dict(num_pages=4, gpu_memory_utilization=0.5)):
        with pytest.raises(ConfigError):
            EngineConfig(**kw)
