"""GPT-2's typed configuration, read from the keys of its own ``config.json``.

Keys and their meaning follow rosellm/rosetrainer/hf_gpt2.py:16-34
(``gpt_config_from_hf_gpt2``): ``n_embd``, ``n_layer``, ``n_head``,
``n_inner`` (absent or null means four times ``n_embd``), ``vocab_size``,
``n_positions`` (fallback ``max_position_embeddings``) and
``activation_function``.  Unlike the reference, which leaves every LayerNorm
at torch's default epsilon (rosellm/rosetrainer/model.py:355-356, 498),
``layer_norm_epsilon`` is read and used.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, ClassVar

from .base import ConfigError, ModelConfig, optional, require

# activation_function values and the formula each one means
# (rosellm/rosetrainer/model.py:274-277 for the tanh form, :343-346 for erf).
TANH_GELU_NAMES = ("gelu_new", "gelu_pytorch_tanh", "gelu_fast")
ERF_GELU_NAMES = ("gelu",)


@dataclass(frozen=True)
class GPT2Config(ModelConfig):
    architecture: ClassVar[str] = "GPT2LMHeadModel"

    n_layer: int
    n_embd: int
    n_head: int
    n_inner: int
    vocab_size: int
    n_positions: int
    layer_norm_epsilon: float
    activation_function: str
    tie_word_embeddings: bool = True
    eos_token_id: int | None = None
    bos_token_id: int | None = None

    @property
    def head_dim(self) -> int:
        return self.n_embd // self.n_head

    def __post_init__(self) -> None:
        for name in ("n_layer", "n_embd", "n_head", "n_inner", "vocab_size", "n_positions"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"config.json: {name} must be positive, got {getattr(self, name)}")
        if self.n_embd % self.n_head != 0:
            raise ConfigError(
                f"config.json: n_embd={self.n_embd} is not divisible by n_head={self.n_head}"
            )
        if self.layer_norm_epsilon <= 0.0:
            raise ConfigError("config.json: layer_norm_epsilon must be positive")
        if self.activation_function not in TANH_GELU_NAMES + ERF_GELU_NAMES:
            raise ConfigError(
                f"config.json: activation_function={self.activation_function!r} is not supported "
                f"(tanh form: {TANH_GELU_NAMES}; erf form: {ERF_GELU_NAMES})"
            )
        if not self.tie_word_embeddings:
            raise ConfigError(
                "config.json: tie_word_embeddings=false: GPT-2's head is its token table "
                "(rosellm/rosetrainer/model.py:503-504); an untied head is not supported"
            )

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "GPT2Config":
        n_embd = require(raw, "n_embd", int)
        # Options of HF GPT-2 that the reference's model has no code for
        # (rosellm/rosetrainer/model.py:169: scale is always head_dim**-0.5).
        if optional(raw, "scale_attn_weights", bool, True) is not True:
            raise ConfigError("config.json: scale_attn_weights=false is not supported")
        if optional(raw, "scale_attn_by_inverse_layer_idx", bool, False):
            raise ConfigError("config.json: scale_attn_by_inverse_layer_idx=true is not supported")
        if optional(raw, "add_cross_attention", bool, False):
            raise ConfigError("config.json: add_cross_attention=true is not supported")
        n_inner = optional(raw, "n_inner", int, None)
        return cls(
            n_layer=require(raw, "n_layer", int),
            n_embd=n_embd,
            n_head=require(raw, "n_head", int),
            n_inner=n_inner if n_inner is not None else 4 * n_embd,
            vocab_size=require(raw, "vocab_size", int),
            n_positions=require(raw, "n_positions", int, "max_position_embeddings"),
            layer_norm_epsilon=optional(raw, "layer_norm_epsilon", float, 1e-5),
            activation_function=optional(raw, "activation_function", str, "gelu_new"),
            tie_word_embeddings=optional(raw, "tie_word_embeddings", bool, True),
            eos_token_id=optional(raw, "eos_token_id", int, None),
            bos_token_id=optional(raw, "bos_token_id", int, None),
        )

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": "gpt2",
            "n_layer": self.n_layer,
            "n_embd": self.n_embd,
            "n_head": self.n_head,
            "n_inner": self.n_inner,
            "vocab_size": self.vocab_size,
            "n_positions": self.n_positions,
            "layer_norm_epsilon": self.layer_norm_epsilon,
            "activation_function": self.activation_function,
            "tie_word_embeddings": self.tie_word_embeddings,
        }
        if self.eos_token_id is not None:
            out["eos_token_id"] = self.eos_token_id
        if self.bos_token_id is not None:
            out["bos_token_id"] = self.bos_token_id
        return out
