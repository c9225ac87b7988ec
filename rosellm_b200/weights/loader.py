"""Weights from safetensors, by tensor name.

The reference goes through ``transformers`` and a renaming table
(rosellm/rosetrainer/hf_gpt2.py:37-78, 96-108) and lets
``load_state_dict(strict=True)`` complain.  Here the file is read directly
and matched against the tensors the model's parts declare; everything that is
wrong with a file (missing tensors, tensors no part reads, wrong shapes) is
reported in one ``WeightError``.

Device dtypes: a ``matrix`` is kept in the engine's compute dtype (bfloat16
for serving, float32 for the 32-bit path), a ``vector`` (norm scale, bias) in
float32 (a value stored in bfloat16 widens exactly; one stored in 32-bit stays
as it is), an ``int_table`` in int32.
"""
from __future__ import annotations

import fnmatch
import json
import os
from dataclasses import dataclass
from typing import Iterable

import torch

from ..parts.base import ParamSpec
from ..parts.spec import Concat


class WeightError(ValueError):
    """Lists every missing, unexpected and wrongly shaped tensor of a weight file."""

    def __init__(
        self,
        source: str,
        missing: list[str],
        unexpected: list[str],
        wrong_shape: list[tuple[str, tuple[int, ...], tuple[int, ...]]],
        wrong_dtype: list[tuple[str, str]] = (),
    ) -> None:
        self.source = source
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)
        lines = [f"weights in {source} do not fit the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + ", ".join(
                f"{n}: expected {list(e)}, file has {list(g)}" for n, e, g in self.wrong_shape))
        if self.wrong_dtype:
            lines.append(f"  wrong dtype ({len(self.wrong_dtype)}): " + ", ".join(
                f"{n}: {why}" for n, why in self.wrong_dtype))
        super().__init__("\n".join(lines))


@dataclass(frozen=True)
class NamedParam:
    """A part's tensor with its name in the weight file; ``pieces`` when the file holds it as
    several tensors to be joined (``file_name`` is then the first of them)."""

    file_name: str
    spec: ParamSpec
    pieces: Concat | None = None

    @property
    def key(self) -> str:
        """What the matched tensor is filed under: the file name, or the pieces' names joined."""
        return self.file_name if self.pieces is None else "+".join(self.pieces.names)

    def sources(self) -> list[tuple[str, tuple[int, ...]]]:
        """(file name, shape in the file) of every file tensor this one is made of."""
        if self.pieces is None:
            return [(self.file_name, tuple(self.spec.shape))]
        return list(zip(self.pieces.names, self.pieces.piece_shapes(tuple(self.spec.shape))))


def read_safetensors(model_dir: str) -> dict[str, torch.Tensor]:
    """All tensors of ``model.safetensors`` (or of the shards its index names), on the CPU."""
    from safetensors.torch import load_file

    single = os.path.join(model_dir, "model.safetensors")
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.isfile(single):
        return load_file(single, device="cpu")
    if os.path.isfile(index):
        with open(index, "r", encoding="utf-8") as f:
            shards = sorted(set(json.load(f)["weight_map"].values()))
        out: dict[str, torch.Tensor] = {}
        for shard in shards:
            out.update(load_file(os.path.join(model_dir, shard), device="cpu"))
        return out
    raise FileNotFoundError(f"no model.safetensors (or its index) in {model_dir!r}")


def _strip_prefix(names: Iterable[str], wanted: set[str], prefixes: tuple[str, ...]) -> str:
    """The one optional prefix that every wanted tensor of the file carries, or ''."""
    names = set(names)
    for prefix in prefixes:
        if any(w in names for w in wanted):
            break
        if any(prefix + w in names for w in wanted):
            return prefix
    return ""


def match_tensors(
    params: list[NamedParam],
    file_tensors: dict[str, torch.Tensor],
    *,
    source: str,
    optional_prefixes: tuple[str, ...] = (),
    ignored: tuple[str, ...] = (),
) -> dict[str, torch.Tensor]:
    """Check ``file_tensors`` against ``params``; return them by ``NamedParam.key`` (the file
    name, prefix removed), pieces joined.

    Raises one ``WeightError`` naming everything that does not fit.
    """
    wanted = {name for p in params for name, _ in p.sources()}
    prefix = _strip_prefix(file_tensors.keys(), wanted, optional_prefixes)
    have: dict[str, torch.Tensor] = {}
    for name, t in file_tensors.items():
        have[name[len(prefix):] if prefix and name.startswith(prefix) else name] = t

    missing = sorted(w for w in wanted if w not in have)
    unexpected = sorted(
        n for n in have
        if n not in wanted and not any(fnmatch.fnmatchcase(n, pat) for pat in ignored)
    )
    wrong_shape = []
    wrong_dtype = []
    for p in params:
        for name, shape in p.sources():
            t = have.get(name)
            if t is None:
                continue
            if tuple(t.shape) != shape:
                wrong_shape.append((name, shape, tuple(t.shape)))
            if p.spec.kind == "int_table":
                if t.dtype.is_floating_point:
                    wrong_dtype.append((name, f"integer table stored as {t.dtype}"))
            elif not t.dtype.is_floating_point:
                wrong_dtype.append((name, f"expected a floating-point tensor, file has {t.dtype}"))
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightError(source, missing, unexpected, wrong_shape, wrong_dtype)
    out = {}
    for p in params:
        if p.pieces is None:
            out[p.key] = have[p.file_name]
        else:
            out[p.key] = torch.cat([have[n] for n in p.pieces.names], dim=p.pieces.dim)
    return out


def to_device_tensor(
    t: torch.Tensor, spec: ParamSpec, compute_dtype: torch.dtype, device: torch.device | str
) -> torch.Tensor:
    """One file tensor as the part wants it on the device (see the module docstring)."""
    if spec.kind == "matrix":
        t = t.to(compute_dtype)
    elif spec.kind == "vector":
        t = t.to(torch.float32)
    elif spec.kind == "int_table":
        t = t.to(torch.int32)
    else:
        raise ValueError(f"unknown ParamSpec.kind {spec.kind!r}")
    if spec.transpose:
        t = t.t()
    return t.contiguous().to(device)
