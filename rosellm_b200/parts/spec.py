"""What a model is made of, as data.

An architecture's builder (registered with ``register_architecture``) turns
its typed configuration into a ``ModelSpec``: which embedding, which position
encoding, and, layer by layer, which mixer, feed-forward, norms and block
arrangement, each a ``PartSpec`` naming a registered part and giving it its
sizes and constants.  ``run_order`` is the order in which layers run; it may
name a layer twice, and an entry may read another layer's cache instead of
writing its own.  The reference has one fixed stack
(rosellm/rosetrainer/model.py:494-497: a ``ModuleList`` of identical blocks);
here the stack is a list so that models mixing kinds of layers need no new
code outside their builder.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any


@dataclass(frozen=True)
class PartSpec:
    """A registered part's name with the parameters it is constructed from."""

    kind: str
    params: dict[str, Any] = field(default_factory=dict)
    # tensor names in the weight file, by the part's own role names
    # (for example {"qkv_weight": "h.0.attn.c_attn.weight"})
    tensors: dict[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    block: PartSpec
    mixer: PartSpec
    feed_forward: PartSpec
    norm_mixer: PartSpec
    norm_feed_forward: PartSpec


@dataclass(frozen=True)
class RunEntry:
    """One position of the run order.

    ``layer`` indexes ``ModelSpec.layers``.  With ``cache_of`` unset the run uses the
    layer's own cache and appends the step's keys and values to it before reading.  With
    ``cache_of`` set (to another layer, or to the layer itself when it runs a second
    time) the run only reads that layer's cache, which an earlier run has filled.
    """

    layer: int
    cache_of: int | None = None

    @property
    def cache_layer(self) -> int:
        return self.layer if self.cache_of is None else self.cache_of

    @property
    def writes_cache(self) -> bool:
        return self.cache_of is None


@dataclass(frozen=True)
class ModelSpec:
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    position: PartSpec
    layers: tuple[LayerSpec, ...]
    run_order: tuple[RunEntry, ...]
    final_norm: PartSpec
    head: PartSpec
    eos_token_id: int | None = None
    # prefixes a file may put before every tensor name
    optional_prefixes: tuple[str, ...] = ()
    # glob patterns of tensors a file may hold that no part reads
    ignored_tensors: tuple[str, ...] = ()

    def __post_init__(self) -> None:
        n = len(self.layers)
        seen_writer: set[int] = set()
        for pos, entry in enumerate(self.run_order):
            if not 0 <= entry.layer < n:
                raise ValueError(f"run_order[{pos}] names layer {entry.layer}; there are {n}")
            if entry.writes_cache:
                if entry.layer in seen_writer:
                    raise ValueError(
                        f"run_order[{pos}] runs layer {entry.layer} a second time with its own "
                        "cache; a repeated layer must read another run's cache (cache_of)"
                    )
                seen_writer.add(entry.layer)
            elif entry.cache_layer not in seen_writer:
                raise ValueError(
                    f"run_order[{pos}] reads the cache of layer {entry.cache_layer}, "
                    "which has not run before it"
                )
