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

import dataclasses
from dataclasses import dataclass, field
from typing import Any


@dataclass(frozen=True)
class Concat:
    """One tensor of a part made of several tensors of the weight file, joined along ``dim``
    of the file's layout: a checkpoint that stores queries, keys and values apart feeds a
    mixer that wants them packed.  ``sizes``: the pieces' extents along ``dim`` (``None``:
    equal parts)."""

    names: tuple[str, ...]
    dim: int = 0
    sizes: tuple[int, ...] | None = None

    def piece_shapes(self, shape: tuple[int, ...]) -> list[tuple[int, ...]]:
        """The shape each piece must have for the whole to be ``shape``."""
        total = shape[self.dim]
        sizes = self.sizes
        if sizes is None:
            if total % len(self.names) != 0:
                raise ValueError(f"{total} does not split evenly over {self.names}")
            sizes = (total // len(self.names),) * len(self.names)
        if len(sizes) != len(self.names) or sum(sizes) != total:
            raise ValueError(f"pieces {self.names} of sizes {sizes} do not make up {total} along dimension {self.dim}")
        return [tuple(n if d == self.dim else s for d, s in enumerate(shape)) for n in sizes]


@dataclass(frozen=True)
class PartSpec:
    """A registered part's name with the parameters it is constructed from."""

    kind: str
    params: dict[str, Any] = field(default_factory=dict)
    # tensor names in the weight file, by the part's own role names
    # (for example {"qkv_weight": "h.0.attn.c_attn.weight"}); a ``Concat`` where the file
    # holds the tensor in pieces
    tensors: dict[str, "str | Concat"] = field(default_factory=dict)


# The sub-parts of the layers GPT-2 and its like are made of, by name and category.
STANDARD_SUBPARTS = (("mixer", "mixer"), ("feed_forward", "feed_forward"), ("norm_mixer", "norm"),
                     ("norm_feed_forward", "norm"))


@dataclass(frozen=True)
class LayerSpec:
    """A layer: a block arrangement and the named sub-parts it arranges.

    ``parts`` holds (name within the layer, category, spec) for every sub-part.  Which names
    there are is up to the block part, which declares the ones it uses (``Part.uses``): the
    shipped ``pre_norm`` block wants ``norm_mixer``, ``mixer``, ``norm_feed_forward`` and
    ``feed_forward``; a block with norms after its mixer, one norm shared by two branches, or
    two mixers, names them as it likes and nothing outside the block has to know.
    ``LayerSpec.standard`` builds the usual five.
    """

    block: PartSpec
    parts: tuple[tuple[str, str, PartSpec], ...]

    @staticmethod
    def standard(block: PartSpec, mixer: PartSpec, feed_forward: PartSpec, norm_mixer: PartSpec,
                 norm_feed_forward: PartSpec) -> "LayerSpec":
        given = dict(mixer=mixer, feed_forward=feed_forward, norm_mixer=norm_mixer, norm_feed_forward=norm_feed_forward)
        return LayerSpec(block, tuple((name, cat, given[name]) for name, cat in STANDARD_SUBPARTS))

    @staticmethod
    def of(block: PartSpec, **named: "tuple[str, PartSpec]") -> "LayerSpec":
        """``LayerSpec.of(block, name=(category, spec), ...)``."""
        return LayerSpec(block, tuple((name, cat, spec) for name, (cat, spec) in named.items()))

    def __post_init__(self) -> None:
        names = [n for n, _, _ in self.parts]
        if len(set(names)) != len(names):
            raise ValueError(f"a layer's sub-parts need distinct names, got {names}")

    def part(self, name: str) -> PartSpec:
        for n, _, spec in self.parts:
            if n == name:
                return spec
        raise KeyError(f"the layer has no sub-part {name!r}; it has {[n for n, _, _ in self.parts]}")


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
    # which of the layer's sub-parts this entry is handed to ("mixer" unless a block with
    # several mixers says otherwise through ``for_part``)
    part: str = "mixer"

    @property
    def cache_layer(self) -> int:
        return self.layer if self.cache_of is None else self.cache_of

    # Keys under which the cache manager keeps a mixer's pages and state rows: the layer's
    # index for the sub-part called "mixer", (layer, name) for any other.
    @property
    def cache_key(self):
        return self.cache_layer if self.part == "mixer" else (self.cache_layer, self.part)

    @property
    def state_key(self):
        return self.layer if self.part == "mixer" else (self.layer, self.part)

    def for_part(self, name: str) -> "RunEntry":
        """This entry as seen by the layer's sub-part ``name`` (a block with more than one
        mixer hands each its own, so that each finds its own cache and state)."""
        return self if name == self.part else dataclasses.replace(self, part=name)

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
