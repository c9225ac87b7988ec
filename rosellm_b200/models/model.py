"""A model: the parts of a ``ModelSpec`` built, given their weights, and run in order.

This class knows no architecture.  It constructs every part from the
registry, collects the tensors the parts declare, hands each part its own
tensors and, for one step, runs embedding, the layers in ``run_order``, the
final norm on the rows whose logits are wanted, and the head.  The reference's
counterpart is ``GPTModel.forward_varlen`` (rosellm/rosetrainer/model.py:654-701),
which computes logits for every token and lets the caller select
(rosellm/roseinfer/engine.py:975-976); here rows are selected before the
final norm.
"""
from __future__ import annotations

import torch

from ..parts.base import Part, build_part
from ..parts.spec import Concat, ModelSpec, PartSpec
from ..weights.loader import NamedParam, match_tensors, to_device_tensor


class Layer:
    """The built parts of one layer: the block arrangement and the sub-parts it arranges, by the
    names the layer's spec gives them (``layer.mixer``, ``layer.norm_mixer``, or whatever a
    block of another shape calls its own)."""

    def __init__(self, block: Part, parts: dict[str, Part], categories: dict[str, str]) -> None:
        self.block = block
        self.parts = parts
        self.categories = categories

    def __getattr__(self, name: str) -> Part:
        try:
            return self.__dict__["parts"][name]
        except KeyError:
            raise AttributeError(f"the layer has no sub-part {name!r}; it has {sorted(self.__dict__.get('parts', {}))}") from None


def _cache_key(layer: int, name: str):
    """Key of a sub-part's pages and state rows: see ``RunEntry.cache_key``."""
    return layer if name == "mixer" else (layer, name)


def _file_names(source) -> tuple[str, ...]:
    return source.names if isinstance(source, Concat) else (source,)


def _named(part: Part, spec: PartSpec) -> list[NamedParam]:
    out = []
    for p in part.param_specs():
        if p.role not in spec.tensors:
            raise KeyError(f"part {spec.kind!r} reads tensor {p.role!r}; the model spec names no file tensor for it")
        source = spec.tensors[p.role]
        if isinstance(source, Concat):
            out.append(NamedParam(source.names[0], p, source))
        else:
            out.append(NamedParam(source, p))
    return out


def _build_layer(ls) -> Layer:
    block = build_part("block", ls.block)
    parts = {name: build_part(cat, spec) for name, cat, spec in ls.parts}
    cats = {name: cat for name, cat, _ in ls.parts}
    for name, cat in getattr(block, "uses", {}).items():
        if cats.get(name) != cat:
            raise ValueError(
                f"block {ls.block.kind!r} arranges a {cat} called {name!r}; the layer's spec gives "
                f"{ {n: c for n, c in cats.items()} }"
            )
    return Layer(block, parts, cats)


def _parts_with_specs(spec: ModelSpec, model: "Model | None" = None):
    """(part, PartSpec) pairs in a fixed order; builds throw-away parts when no model is given."""
    pairs = []

    def one(category: str, ps: PartSpec, built: Part | None):
        pairs.append((built if built is not None else build_part(category, ps), ps))

    one("embedding", spec.embedding, model.embedding if model else None)
    one("position", spec.position, model.position if model else None)
    for i, ls in enumerate(spec.layers):
        layer = model.layers[i] if model else None
        for name, cat, ps in ls.parts:
            one(cat, ps, layer.parts[name] if layer else None)
    one("norm", spec.final_norm, model.final_norm if model else None)
    one("head", spec.head, model.head if model else None)
    return pairs


def named_params_of_spec(spec: ModelSpec) -> list[NamedParam]:
    """Every tensor a model of this spec reads from its weight file."""
    out: list[NamedParam] = []
    for part, ps in _parts_with_specs(spec):
        out.extend(_named(part, ps))
    return out


class Model:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device: torch.device | str) -> None:
        self.spec = spec
        self.dtype = dtype
        self.device = torch.device(device)
        self.embedding = build_part("embedding", spec.embedding)
        self.position = build_part("position", spec.position)
        self.layers = [_build_layer(ls) for ls in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm)
        self.head = build_part("head", spec.head)
        self.loaded = False
        self._keyed_parts: list | None = None

    # ---- what the cache manager has to provide --------------------------------
    def kv_specs(self) -> dict:
        """``KVCacheSpec`` of every sub-part that keeps keys and values, by cache key (the layer's
        index for the sub-part called ``mixer``, ``(layer, name)`` for any other)."""
        out = {}
        writers = {e.layer for e in self.spec.run_order if e.writes_cache}
        for i, layer in enumerate(self.layers):
            for name, part in layer.parts.items():
                cs = part.cache_spec()
                if cs is not None and i in writers:
                    out[_cache_key(i, name)] = cs
        for pos, e in enumerate(self.spec.run_order):
            if e.writes_cache:
                continue
            for name, part in self.layers[e.layer].parts.items():
                own = part.cache_spec()
                if own is not None and own != out.get(_cache_key(e.cache_layer, name)):
                    raise ValueError(
                        f"run_order[{pos}]: {name!r} of layer {e.layer} reads the cache of layer {e.cache_layer}, "
                        "whose geometry differs from what it expects"
                    )
        return out

    def state_specs(self) -> dict:
        out = {}
        for i, layer in enumerate(self.layers):
            for name, part in layer.parts.items():
                ss = part.state_spec()
                if ss is not None:
                    out[_cache_key(i, name)] = ss
        return out

    @property
    def graph_safe(self) -> bool:
        parts = [p for p, _ in _parts_with_specs(self.spec, self)] + [l.block for l in self.layers]
        return all(getattr(p, "graph_safe", False) for p in parts)

    def _all_parts(self) -> list:
        return [p for p, _ in _parts_with_specs(self.spec, self)] + [l.block for l in self.layers]

    @property
    def launches_replayable(self) -> bool:
        """Whether a step's library calls follow from its sizes and ``launch_key`` alone."""
        return all(getattr(p, "launches_replayable", False) for p in self._all_parts())

    def launch_key(self, ctx) -> tuple:
        """The parts' ``launch_key``s for this step (only of parts that define one)."""
        if self._keyed_parts is None:
            base = Part.launch_key
            self._keyed_parts = [p for p in self._all_parts() if getattr(type(p), "launch_key", base) is not base]
        return tuple(p.launch_key(ctx) for p in self._keyed_parts)

    # ---- weights ---------------------------------------------------------------
    def named_params(self) -> list[NamedParam]:
        out: list[NamedParam] = []
        for part, ps in _parts_with_specs(self.spec, self):
            out.extend(_named(part, ps))
        return out

    def load_tensors(self, file_tensors: dict[str, torch.Tensor], source: str = "<tensors>") -> None:
        """Check ``file_tensors`` (by file name) against the parts and bind them on the device."""
        by_name = match_tensors(
            self.named_params(), file_tensors, source=source,
            optional_prefixes=self.spec.optional_prefixes, ignored=self.spec.ignored_tensors,
        )
        for part, ps in _parts_with_specs(self.spec, self):
            bound = {
                np_.spec.role: to_device_tensor(by_name[np_.key], np_.spec, self.dtype, self.device)
                for np_ in _named(part, ps)
            }
            part.bind(bound)
        if getattr(self.head, "tied", False):
            self.head.weight = self.embedding.weight
        self.loaded = True

    def weight_bytes(self) -> int:
        """Bytes of every distinct weight tensor on the device (a tied head counts once; copies a
        part keeps in another layout for one of its kernels, under names with a leading
        underscore, are not counted)."""
        seen: dict[int, int] = {}
        parts = [p for p, _ in _parts_with_specs(self.spec, self)]
        for part in parts:
            for name, v in vars(part).items():
                if isinstance(v, torch.Tensor) and not name.startswith("_"):
                    seen[v.data_ptr()] = v.numel() * v.element_size()
        return sum(seen.values())

    # ---- one step ----------------------------------------------------------------
    def samples_in_head(self, n_rows: int, with_temperature: bool = False) -> bool:
        """Whether a step with this many wanted rows (some with a temperature, or all taking the
        arg-max) should have its next tokens chosen by the head (``ctx.extras["sample_into"]``)
        instead of getting logits."""
        can = getattr(self.head, "can_sample", None)
        return can is not None and n_rows > 0 and bool(can(n_rows, self.dtype, with_temperature))

    def forward(self, ctx) -> torch.Tensor | None:
        """Run the step's tokens; logits float32 ``[wanted rows, vocab]`` (``None`` if none wanted).
        With ``ctx.extras["sample_into"]`` (a ``K.SampleInto``; the caller has asked
        ``samples_in_head``) the head chooses the wanted rows' next tokens into it and no
        logits are made: ``None`` then too."""
        ctx.position = self.position
        x = self.embedding.forward(ctx, self.position)
        for run in self.spec.run_order:
            layer = self.layers[run.layer]
            layer.block.forward(ctx, run, layer, x)
        if ctx.n_logit_rows == 0:
            return None
        rows = ctx.host.logit_rows
        every_row = len(rows) == ctx.n_tokens and int(rows[0]) == 0 and int(rows[-1]) == ctx.n_tokens - 1
        if (every_row and ctx.n_tokens <= 2 and getattr(self.final_norm, "can_defer", False)
                and getattr(self.head, "takes_norm_input", False)):
            # one or two rows, all wanted: nothing to gather, and the norm may be handed to the head
            # unevaluated, to be computed inside its product (every block of a product normalises
            # the rows for itself: with more rows, and the thousands of blocks of a head, that
            # costs more than the norm's own kernel; measured at 8 rows, vocabulary 50,257: +80 us)
            h = self.final_norm.forward(ctx, x, defer=True, name="final_normed")
        else:
            h = self.final_norm.forward(ctx, x, rows=ctx.logit_rows, n_rows=ctx.n_logit_rows, name="final_normed")
        into = ctx.extras.get("sample_into")
        if into is not None:
            if not self.samples_in_head(ctx.n_logit_rows):
                raise ValueError(f"the head does not choose the tokens of {ctx.n_logit_rows} rows itself")
            self.head.forward_sample(ctx, h, into)
            return None
        return self.head.forward(ctx, h)
