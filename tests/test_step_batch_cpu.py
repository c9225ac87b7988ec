"""The host side of a step: index arrays, the decode attention plan, the workspace and noted launches."""
import numpy as np
import pytest

from rosellm_b200.engine.context import ATTENTION_TILE_Q, ATTENTION_TILE_Q_WIDE, build_host_batch


def test_mixed_batch_arrays():
    hb = build_host_batch([(3, 10, [5, 6, 7], [0, 2]), (0, 99, [8], [0]), (7, 0, np.arange(40), [])])
    assert hb.token_ids.tolist() == [5, 6, 7, 8] + list(range(40))
    assert hb.positions.tolist() == [10, 11, 12, 99] + list(range(40))
    assert hb.req_of_token.tolist() == [0, 0, 0, 1] + [2] * 40
    assert hb.q_start.tolist() == [0, 3, 4, 44] and hb.kv_len.tolist() == [13, 100, 40]
    assert hb.slots.tolist() == [3, 0, 7] and hb.logit_rows.tolist() == [0, 2, 3]
    assert hb.decode_reqs.tolist() == [1]
    want = [(0, 0)] + [(2, t) for t in range(0, 40, ATTENTION_TILE_Q)]
    assert [tuple(t) for t in hb.tiles.tolist()] == want
    want = [(0, 0)] + [(2, t) for t in range(0, 40, ATTENTION_TILE_Q_WIDE)]
    assert [tuple(t) for t in hb.tiles_wide.tolist()] == want
    for a in (hb.token_ids, hb.positions, hb.tiles, hb.tiles_wide, hb.logit_rows):
        assert a.dtype == np.int32


def test_decode_only_batch_equals_the_general_form():
    """More than four single-token requests take a vectorised path; it gives the arrays that
    the general path gives for the same requests (here: in groups of three)."""
    entries = [(3 * i + 1, 500 + 7 * i, [-(i + 1) if i % 2 else 11 * i], [0]) for i in range(9)]
    fast = build_host_batch(entries)
    parts = [build_host_batch(entries[i:i + 3]) for i in range(0, 9, 3)]
    for name in ("token_ids", "positions", "kv_len", "slots"):
        assert getattr(fast, name).tolist() == sum((getattr(p, name).tolist() for p in parts), []), name
        assert getattr(fast, name).dtype == np.int32 and getattr(fast, name).flags.c_contiguous
    assert fast.q_start.tolist() == list(range(10))
    assert fast.req_of_token.tolist() == fast.logit_rows.tolist() == fast.decode_reqs.tolist() == list(range(9))
    assert fast.tiles.shape == (0, 2) and fast.tiles_wide.shape == (0, 2)
    # a request that wants nothing, or brings two tokens, leaves the vectorised path
    odd = build_host_batch(entries[:5] + [(40, 3, [1], [])] + entries[5:])
    assert odd.logit_rows.tolist() == [0, 1, 2, 3, 4, 6, 7, 8, 9] and len(odd.decode_reqs) == 10


def test_bad_entries_are_refused():
    with pytest.raises(ValueError, match="no token"):
        build_host_batch([(0, 0, [], [])])
    with pytest.raises(ValueError, match="outside"):
        build_host_batch([(0, 0, [1, 2], [2])])


def test_decode_attention_plan(monkeypatch):
    """How decoded requests are spread over blocks: wide blocks while there are few (request,
    head) pairs, narrow ones beyond; no split while all narrow blocks run at once; never more
    parts than 64-key pieces, nor than 32.  The device's SM count and shared memory are asked
    from the device; here they are given (those of a B200)."""
    import torch

    from rosellm_b200.ops import kernels as K
    from rosellm_b200.parts.standard import CausalSelfAttention, narrow_decode_blocks_at_once

    monkeypatch.setattr(K, "device_facts_given", (148, 233472))
    NARROW_BLOCKS_AT_ONCE = narrow_decode_blocks_at_once(64, 2)
    assert NARROW_BLOCKS_AT_ONCE == 3 * 148  # rings of 32 KB in half of an SM's 228 KB
    assert narrow_decode_blocks_at_once(64, 4) == 3 * 148 and narrow_decode_blocks_at_once(256, 4) == 148
    assert narrow_decode_blocks_at_once(64, 2, 80) == 5 * 148 and narrow_decode_blocks_at_once(64, 2, 100) == 6 * 148
    att = CausalSelfAttention(hidden_size=768, num_heads=12, head_dim=64)
    assert att.decode_plan_for(0, 512) == (1, False)
    for n in (1, 2, 8, 24, 25, 32, 37, 40, 64, 256):
        for span in (1, 63, 64, 512, 1024, 5000, 100_000):
            parts, wide = att.decode_plan_for(n, span)
            assert wide == (n * 12 <= 296)
            assert 1 <= parts <= 32 and (parts == 1 or parts <= span // 64 or wide)
            if not wide and n * 12 <= NARROW_BLOCKS_AT_ONCE and span <= 2048:
                assert parts == 1
    assert att.decode_plan_for(32, 512) == (1, False)   # measured: 10.3 us whole, 15.7 us in two parts
    assert att.decode_plan_for(48, 1024)[0] == 1        # one round of dense blocks (two rounds measured 35.0 us whole, 33.6 in two parts)
    assert att.decode_plan_for(64, 512) == (1, False) and att.decode_plan_for(40, 512) == (1, False)
    windowed = CausalSelfAttention(hidden_size=768, num_heads=12, head_dim=64, window=128)
    assert windowed.decode_plan_for(48, 100_000) == windowed.decode_plan_for(48, 128)
    # half as many SMs: the wide form ends at half as many (request, head) pairs
    monkeypatch.setattr(K, "device_facts_given", (74, 233472))
    assert att.decode_plan_for(13, 512)[1] is False and att.decode_plan_for(12, 512)[1] is True
    # a 32-bit cache costs twice the bytes a key: a split pays earlier
    monkeypatch.setattr(K, "device_facts_given", (148, 233472))
    assert att.decode_plan_for(48, 1024, torch.float32)[0] >= att.decode_plan_for(48, 1024, torch.bfloat16)[0]


def test_workspace_keeps_views_until_a_buffer_moves():
    import torch

    from rosellm_b200.engine.context import Workspace

    ws = Workspace(torch.device("cpu"))
    a = ws.get("x", (4, 8), torch.float32)
    assert ws.get("x", (4, 8), torch.float32) is a and ws.version == 1
    b = ws.get("x", (2, 8), torch.float32)  # a smaller request: the same memory, another view
    assert b.data_ptr() == a.data_ptr() and b.shape == (2, 8) and ws.version == 1
    c = ws.get("x", (16, 8), torch.float32)  # the buffer grows: earlier views are dropped
    assert ws.version == 2 and ws.get("x", (4, 8), torch.float32) is not a
    assert ws.get("x", (4, 8), torch.float32).data_ptr() == c.data_ptr()
    ws.get("y", (3,), torch.int32)
    assert ws.version == 3
    z = ws.get_zeroed("z", (5,), torch.float32)
    assert float(z.abs().sum()) == 0.0
    z += 1
    assert ws.get_zeroed("z", (5,), torch.float32) is z and float(z.sum()) == 5.0  # its users leave it zero
    ws.frozen = True
    with pytest.raises(RuntimeError, match="frozen"):
        ws.get("x", (64, 8), torch.float32)


def test_noted_library_calls_are_issued_again_in_order(monkeypatch):
    """``recording`` notes every launch with its arguments but the stream; ``replay`` makes the
    same calls on the current stream; queries of the library are not noted; a failing call
    raises."""
    from rosellm_b200.ops import kernels as K

    calls = []

    class FakeLibrary:
        def rl_one(self, *args):
            calls.append(("one",) + args)
            return 0

        def rl_two(self, *args):
            calls.append(("two",) + args)
            return 0 if args[0] != 13 else 7

        def rl_gemm_tc_rows_fits(self, *args):
            calls.append(("fits",) + args)
            return 1

    monkeypatch.setattr(K, "_loaded", FakeLibrary())
    monkeypatch.setattr(K, "_stream", lambda: "stream B")
    with K.recording() as launches:
        lib = K._lib()
        assert lib.rl_one(1, 2.5, "stream A") == 0
        assert lib.rl_gemm_tc_rows_fits(64, 768, 3072) == 1
        assert lib.rl_two(None, "stream A") == 0
        with pytest.raises(K.KernelError, match="already"):
            K.recording().__enter__()
    assert K._lib() is K._loaded  # recording is over
    assert [c[0] for c in calls] == ["one", "fits", "two"] and len(launches.calls) == 2
    del calls[:]
    launches.replay()
    assert calls == [("one", 1, 2.5, "stream B"), ("two", None, "stream B")]
    with K.recording() as bad:
        K._lib().rl_two(13, "stream A")
    with pytest.raises(K.KernelError, match="code 7"):
        bad.replay()
