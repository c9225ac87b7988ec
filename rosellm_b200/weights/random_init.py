"""Random-weights mode: a model folder from a configuration and a seed.

The reference's tests build ``GPTModel(cfg)`` under ``torch.manual_seed``
(rosellm/rosetrainer/model.py:506-527: N(0, 0.02) matrices, zero biases, unit
norm scales).  Here every tensor is drawn from its own generator, seeded by
the seed and the tensor's name, so that a tensor's values do not depend on
which other tensors exist or on their order.  Matrices are written in
bfloat16, so that the bfloat16 and the 32-bit path start from the same
values; norm scales and biases are written in float32.
"""
from __future__ import annotations

import hashlib
import json
import os

import torch

from ..config.base import ModelConfig, resolve_architecture
from .loader import NamedParam


def _generator_for(seed: int, name: str) -> torch.Generator:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    g = torch.Generator(device="cpu")
    g.manual_seed(int.from_bytes(digest[:8], "little") & 0x7FFF_FFFF_FFFF_FFFF)
    return g


def random_tensors(
    params: list[NamedParam],
    seed: int,
    *,
    std: float = 0.02,
    norm_affine: str = "random",
    matrix_dtype: torch.dtype = torch.bfloat16,
) -> dict[str, torch.Tensor]:
    """Tensors by file name, in the shapes and layout of the file.

    ``norm_affine``: ``"identity"`` leaves norm scales at one and their biases
    at zero; ``"random"`` perturbs both by N(0, std) so that tests exercise them.
    """
    if norm_affine not in ("identity", "random"):
        raise ValueError("norm_affine must be 'identity' or 'random'")
    out: dict[str, torch.Tensor] = {}
    for p in params:
        if p.spec.kind == "int_table":
            raise ValueError(f"{p.file_name}: no random rule for integer tables")
        for name, shape in p.sources():  # a tensor the file holds in pieces: each piece by its own name
            g = _generator_for(seed, name)
            noise = torch.randn(shape, generator=g, dtype=torch.float32) * std
            if p.spec.init == "ones":
                t = torch.ones(shape) + (noise if norm_affine == "random" else 0.0)
            elif p.spec.init == "zeros":
                t = noise if norm_affine == "random" else torch.zeros(shape)
            else:
                t = noise
            out[name] = t.to(matrix_dtype if p.spec.kind == "matrix" else torch.float32)
    return out


def write_model_folder(
    config: ModelConfig,
    seed: int,
    out_dir: str,
    *,
    std: float = 0.02,
    norm_affine: str = "random",
    matrix_dtype: torch.dtype = torch.bfloat16,
) -> str:
    """Write ``config.json`` and ``model.safetensors`` for ``config``; returns ``out_dir``."""
    from safetensors.torch import save_file

    from ..models.model import named_params_of_spec

    raw = config.to_dict()
    spec = resolve_architecture(raw).build_spec(config)
    tensors = random_tensors(
        named_params_of_spec(spec), seed, std=std, norm_affine=norm_affine, matrix_dtype=matrix_dtype
    )
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(raw, f, indent=1, sort_keys=True)
    save_file({k: v.contiguous() for k, v in tensors.items()}, os.path.join(out_dir, "model.safetensors"))
    return out_dir
