"""What one step is, for the parts that run it.

A step is a flat list of tokens: each request in it contributes one or more
consecutive tokens that continue what the cache already holds of it (a single
token is a decoded one, more are a portion of a prompt).  ``StepContext``
carries the index arrays every part needs, on the device and (for parts that
loop on the host) on the host, plus access to the cache and to scratch
buffers.  The reference builds a ``PagedKVCache`` record per forward pass for
the same purpose (rosellm/rosetrainer/paged_attention.py:22-37) with separate
fields for its decode and its chunked-prefill route; here one record serves
any mix of the two.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import numpy as np
import torch

# queries per block of the prompt-portion attention kernels: the CUDA-core kernel
# (csrc/attention_kernels.cuh TILE_Q) and the tensor-core kernel (csrc/attention_mma.cuh)
ATTENTION_TILE_Q = 16
ATTENTION_TILE_Q_WIDE = 64


class Workspace:
    """Named scratch buffers that keep their address from step to step.

    A buffer grows when a step needs more; growing inside a CUDA-graph capture
    is an error, so graphs are captured after a warm-up at the largest size.
    """

    def __init__(self, device: torch.device) -> None:
        self.device = device
        self._bufs: dict[str, torch.Tensor] = {}
        self._views: dict[tuple, torch.Tensor] = {}
        self.frozen = False
        self.version = 0  # counts (re)allocations: addresses noted before a change are stale

    def get(self, name: str, shape: tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        """The buffer ``name`` as ``shape``: the same tensor object for the same request as long
        as the buffer has not grown (making a view costs microseconds, and a step asks often)."""
        key = (name, shape, dtype)
        view = self._views.get(key)
        if view is not None:
            return view
        n = 1
        for s in shape:
            n *= int(s)
        buf = self._bufs.get(name)
        if buf is None or buf.dtype != dtype or buf.numel() < n:
            if self.frozen:
                raise RuntimeError(f"workspace buffer {name!r} would have to grow while frozen")
            grow = max(n, 1)
            if buf is not None and buf.dtype == dtype:
                grow = max(grow, int(buf.numel() * 1.5))
            buf = torch.empty(grow, dtype=dtype, device=self.device)
            self._bufs[name] = buf
            self.version += 1
            for k in [k for k in self._views if k[0] == name]:
                del self._views[k]
        if len(self._views) > 512:  # steps of ever new sizes: start over rather than grow
            self._views.clear()
        view = self._views[key] = buf[:n].view(*shape)
        return view

    def get_zeroed(self, name: str, shape: tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        """Like ``get``, for buffers whose users leave them zero: zero-filled when (re)allocated."""
        before = self._bufs.get(name)
        out = self.get(name, shape, dtype)
        if self._bufs[name] is not before:
            self._bufs[name].zero_()
        return out


@dataclass
class HostBatch:
    """The step's index arrays on the host (numpy, int32)."""

    token_ids: np.ndarray
    positions: np.ndarray
    req_of_token: np.ndarray
    q_start: np.ndarray      # [requests + 1]
    kv_len: np.ndarray       # [requests] tokens of the request after this step
    slots: np.ndarray        # [requests]
    logit_rows: np.ndarray   # token indices whose logits are wanted
    decode_reqs: np.ndarray  # requests with exactly one token
    tiles: np.ndarray        # [n_tiles, 2] (request, first query) for requests with more
    tiles_wide: np.ndarray   # the same portions cut into 64-query tiles


@dataclass
class StepContext:
    device: torch.device
    act_dtype: torch.dtype
    host: HostBatch
    token_ids: torch.Tensor
    positions: torch.Tensor
    req_of_token: torch.Tensor
    q_start: torch.Tensor
    kv_len: torch.Tensor
    slots: torch.Tensor
    logit_rows: torch.Tensor
    decode_reqs: torch.Tensor
    tiles: torch.Tensor
    tiles_wide: torch.Tensor
    n_tokens: int
    n_reqs: int
    n_logit_rows: int
    n_decode: int
    n_tiles: int
    n_tiles_wide: int
    max_kv_len: int
    cache: Any
    workspace: Workspace
    position: Any = None            # the model's position-encoding part
    extras: dict = field(default_factory=dict)

    @property
    def max_tile_kv_len(self) -> int:
        """The longest context among the requests that bring a portion of a prompt (0: none does)."""
        got = self.extras.get("_max_tile_kv_len")
        if got is None:
            hb = self.host
            got = int(hb.kv_len[hb.tiles[:, 0]].max()) if len(hb.tiles) else 0
            self.extras["_max_tile_kv_len"] = got
        return got

    # ``layer``: a cache key, i.e. a layer's index or (layer, name) for a layer's further mixers
    # (``RunEntry.cache_key`` / ``state_key``)
    def kv_pool(self, layer) -> torch.Tensor:
        return self.cache.kv_pool(layer)

    def block_table(self, layer) -> torch.Tensor:
        return self.cache.block_table(layer)

    def state(self, layer) -> torch.Tensor:
        """Per-request state rows ``[slots, ...]`` of a layer that declared a ``StateSpec``."""
        return self.cache.state(layer)


def build_host_batch(entries: list[tuple[int, int, list[int], list[int]]]) -> HostBatch:
    """``entries``: per request (slot, tokens already cached, new token ids, wanted places).

    Wanted places index the request's new tokens.
    """
    n_reqs = len(entries)
    if n_reqs > 4 and all(len(e[2]) == 1 and e[3] == [0] for e in entries):
        # a decode step: every request brings one token and wants its logits
        cols = np.array([(e[0], e[1], e[2][0]) for e in entries], dtype=np.int64).astype(np.int32)
        ident = np.arange(n_reqs + 1, dtype=np.int32)
        none = np.empty((0, 2), dtype=np.int32)
        return HostBatch(
            token_ids=np.ascontiguousarray(cols[:, 2]), positions=np.ascontiguousarray(cols[:, 1]),
            req_of_token=ident[:-1], q_start=ident, kv_len=cols[:, 1] + 1, slots=np.ascontiguousarray(cols[:, 0]),
            logit_rows=ident[:-1], decode_reqs=ident[:-1], tiles=none, tiles_wide=none,
        )
    total = sum(len(e[2]) for e in entries)
    token_ids = np.empty(total, dtype=np.int32)
    positions = np.empty(total, dtype=np.int32)
    req_of_token = np.empty(total, dtype=np.int32)
    q_start = np.zeros(n_reqs + 1, dtype=np.int32)
    kv_len = np.empty(n_reqs, dtype=np.int32)
    slots = np.empty(n_reqs, dtype=np.int32)
    logit_rows: list[int] = []
    decode_reqs: list[int] = []
    tiles: list[np.ndarray] = []  # per request [(request, first new token of the tile)]
    tiles_wide: list[np.ndarray] = []
    at = 0
    for r, (slot, cached, new_ids, want) in enumerate(entries):
        n = len(new_ids)
        if n < 1:
            raise ValueError(f"request {r} of the step brings no token")
        token_ids[at:at + n] = new_ids
        positions[at:at + n] = np.arange(cached, cached + n, dtype=np.int32)
        req_of_token[at:at + n] = r
        q_start[r + 1] = at + n
        kv_len[r] = cached + n
        slots[r] = slot
        for w in want:
            if not 0 <= w < n:
                raise ValueError(f"request {r}: wanted place {w} outside its {n} new tokens")
            logit_rows.append(at + w)
        if n == 1:
            decode_reqs.append(r)
        else:
            for out, step in ((tiles, ATTENTION_TILE_Q), (tiles_wide, ATTENTION_TILE_Q_WIDE)):
                t = np.empty((-(-n // step), 2), dtype=np.int32)
                t[:, 0] = r
                t[:, 1] = np.arange(0, n, step, dtype=np.int32)
                out.append(t)
        at += n
    return HostBatch(
        token_ids=token_ids,
        positions=positions,
        req_of_token=req_of_token,
        q_start=q_start,
        kv_len=kv_len,
        slots=slots,
        logit_rows=np.asarray(logit_rows, dtype=np.int32),
        decode_reqs=np.asarray(decode_reqs, dtype=np.int32),
        tiles=np.concatenate(tiles) if tiles else np.empty((0, 2), dtype=np.int32),
        tiles_wide=np.concatenate(tiles_wide) if tiles_wide else np.empty((0, 2), dtype=np.int32),
    )


def standalone_context(cache, entries: list[tuple[int, int, list[int], list[int]]], act_dtype: torch.dtype,
                       workspace: Workspace | None = None) -> StepContext:
    """A ``StepContext`` outside ``ModelRunner``, for running a part by itself.

    ``entries`` as in ``build_host_batch``; ``cache`` is a ``CacheManager`` (its pages must
    already be reserved) or anything with ``kv_pool`` / ``block_table`` / ``state``.
    Each array is uploaded by itself; ``ModelRunner`` packs them into one copy.
    """
    hb = build_host_batch(entries)
    device = cache.device

    def dev(a: np.ndarray) -> torch.Tensor:
        return torch.from_numpy(np.ascontiguousarray(a)).to(device)

    return StepContext(
        device=device, act_dtype=act_dtype, host=hb,
        token_ids=dev(hb.token_ids), positions=dev(hb.positions), req_of_token=dev(hb.req_of_token),
        q_start=dev(hb.q_start), kv_len=dev(hb.kv_len), slots=dev(hb.slots), logit_rows=dev(hb.logit_rows),
        decode_reqs=dev(hb.decode_reqs), tiles=dev(hb.tiles.reshape(-1)), tiles_wide=dev(hb.tiles_wide.reshape(-1)),
        n_tokens=len(hb.token_ids), n_reqs=len(hb.slots), n_logit_rows=len(hb.logit_rows),
        n_decode=len(hb.decode_reqs), n_tiles=len(hb.tiles), n_tiles_wide=len(hb.tiles_wide),
        max_kv_len=int(hb.kv_len.max()),
        cache=cache, workspace=workspace or Workspace(device),
    )
