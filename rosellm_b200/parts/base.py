"""Interfaces of the parts a model is assembled from, and their registry.

A part is constructed from its ``PartSpec.params`` alone: sizes, constants and
options.  It declares the tensors it needs (``param_specs``), what cache or
per-request state it wants (``cache_spec`` / ``state_spec``), receives its
tensors with ``bind`` and does its work on one step's tokens in ``forward``.
No part knows which model it is in.

Categories and the signature of ``forward``:

``embedding``      ``forward(ctx, position) -> x``: the residual stream
                   ``[tokens, hidden]`` in float32 for ``ctx.token_ids``.
``position``       ``table()``: a learned table the embedding adds, or ``None``;
                   ``rotate(ctx, q, k)``: in-place encoding of queries and keys.
``norm``           ``forward(ctx, x, rows=None) -> h``: normalised rows of the
                   residual stream in the activation dtype.
``mixer``          ``forward(ctx, run, h, x)``: mixes tokens of a request and
                   adds the result to ``x`` in place.  ``run`` tells which
                   layer's cache or state to use and whether to append to it.
``feed_forward``   ``forward(ctx, h, x)``: adds its result to ``x`` in place.
``block``          ``forward(ctx, run, layer, x)``: arranges norms, mixer and
                   feed-forward of one layer around the residual stream.
``head``           ``forward(ctx, h) -> logits`` ``[rows, vocab]`` float32.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable

import torch

CATEGORIES = ("embedding", "position", "norm", "mixer", "feed_forward", "block", "head")

_PARTS: dict[tuple[str, str], type] = {}


def register_part(category: str, kind: str) -> Callable[[type], type]:
    """Class decorator: make ``kind`` constructible for ``category``."""
    if category not in CATEGORIES:
        raise ValueError(f"unknown part category {category!r}; one of {CATEGORIES}")

    def deco(cls: type) -> type:
        _PARTS[(category, kind)] = cls
        cls.category = category
        cls.kind = kind
        return cls

    return deco


def unregister_part(category: str, kind: str) -> None:
    _PARTS.pop((category, kind), None)


def part_class(category: str, kind: str) -> type:
    try:
        return _PARTS[(category, kind)]
    except KeyError:
        known = sorted(k for c, k in _PARTS if c == category)
        raise KeyError(f"no {category} part named {kind!r}; registered: {known}") from None


@dataclass(frozen=True)
class ParamSpec:
    """One tensor a part reads.

    ``role`` is the part's own name for it; the ``PartSpec.tensors`` map gives
    its name in the weight file.  ``shape`` is the shape in the file.
    ``kind`` decides how it is kept on the device:
    ``matrix``: the engine's compute dtype (bfloat16 or float32);
    ``vector``: float32 in both modes (norm scales, biases: small, and read
    by 32-bit arithmetic); ``int_table``: int32.
    ``transpose``: the file holds ``[in, out]`` and the part wants ``[out, in]``.
    """

    role: str
    shape: tuple[int, ...]
    kind: str = "matrix"
    transpose: bool = False
    # how the random-weights mode fills it: "normal" or "ones" (a norm's scale)
    init: str = "normal"


@dataclass(frozen=True)
class KVCacheSpec:
    """Keys and values in pages.  ``window``: how many latest keys a query sees
    (``None``: all of them); older pages are given back while the request lives."""

    num_kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class StateSpec:
    """Per-request state of fixed size, one slot per live request."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


class Part:
    category = ""
    kind = ""

    def param_specs(self) -> list[ParamSpec]:
        return []

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        """Receive the device tensors named by ``param_specs`` (by role)."""
        for role, t in tensors.items():
            setattr(self, role, t)

    def cache_spec(self) -> KVCacheSpec | None:
        return None

    def state_spec(self) -> StateSpec | None:
        return None

    # whether ``forward`` may be captured in a CUDA graph (no host reads,
    # no allocation whose address changes between replays)
    graph_safe = False

    # whether ``forward`` does all its device work through ``rosellm_b200.ops.kernels`` (no torch
    # operation on device tensors) and chooses it from the step's sizes and ``launch_key`` alone
    launches_replayable = False

    def launch_key(self, ctx) -> tuple:
        """What this part's launches depend on besides the step's sizes (``ctx.n_tokens``,
        ``n_reqs``, ``n_logit_rows``, ``n_decode``, ``n_tiles``, ``n_tiles_wide``): two steps of a
        model whose parts are all ``launches_replayable``, with equal sizes and equal keys, make
        the same library calls with the same arguments, so the engine may issue a recorded list
        of them again."""
        return ()


def build_part(category: str, spec: Any, **extra: Any) -> Part:
    cls = part_class(category, spec.kind)
    return cls(**spec.params, **extra)
