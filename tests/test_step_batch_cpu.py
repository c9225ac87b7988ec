"""The host side of a step's description: index arrays for mixed and for decode-only batches."""
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
