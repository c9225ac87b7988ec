"""GPT-2 as a list of parts.

The reference's ``GPTModel`` (rosellm/rosetrainer/model.py:484-701): learned
token and position tables, ``n_layer`` pre-LayerNorm blocks of multi-head
causal attention and a GELU MLP, a final LayerNorm and a head tied to the
token table.  Tensor names and layouts are those of a Hugging Face GPT-2
checkpoint, which the reference renames and transposes in
rosellm/rosetrainer/hf_gpt2.py:45-76: ``Conv1D`` weights are stored
``[in, out]``.
"""
from __future__ import annotations

from ..config.base import register_architecture
from ..config.gpt2 import ERF_GELU_NAMES, GPT2Config
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry


def build_gpt2_spec(cfg: GPT2Config) -> ModelSpec:
    activation = "gelu_erf" if cfg.activation_function in ERF_GELU_NAMES else "gelu_tanh"
    layers = []
    for i in range(cfg.n_layer):
        h = f"h.{i}."
        layers.append(LayerSpec.standard(
            block=PartSpec("pre_norm"),
            mixer=PartSpec(
                "causal_self_attention",
                dict(hidden_size=cfg.n_embd, num_heads=cfg.n_head, head_dim=cfg.head_dim,
                     num_kv_heads=cfg.n_head, window=None, bias=True, weights_in_out=True),
                {"qkv_weight": h + "attn.c_attn.weight", "qkv_bias": h + "attn.c_attn.bias",
                 "out_weight": h + "attn.c_proj.weight", "out_bias": h + "attn.c_proj.bias"},
            ),
            feed_forward=PartSpec(
                "dense_mlp",
                dict(hidden_size=cfg.n_embd, inner_size=cfg.n_inner, activation=activation,
                     bias=True, weights_in_out=True),
                {"in_weight": h + "mlp.c_fc.weight", "in_bias": h + "mlp.c_fc.bias",
                 "out_weight": h + "mlp.c_proj.weight", "out_bias": h + "mlp.c_proj.bias"},
            ),
            norm_mixer=PartSpec(
                "layer_norm", dict(hidden_size=cfg.n_embd, eps=cfg.layer_norm_epsilon),
                {"weight": h + "ln_1.weight", "bias": h + "ln_1.bias"},
            ),
            norm_feed_forward=PartSpec(
                "layer_norm", dict(hidden_size=cfg.n_embd, eps=cfg.layer_norm_epsilon),
                {"weight": h + "ln_2.weight", "bias": h + "ln_2.bias"},
            ),
        ))
    return ModelSpec(
        hidden_size=cfg.n_embd,
        vocab_size=cfg.vocab_size,
        max_positions=cfg.n_positions,
        embedding=PartSpec("token_table", dict(vocab_size=cfg.vocab_size, hidden_size=cfg.n_embd),
                           {"weight": "wte.weight"}),
        position=PartSpec("learned_absolute", dict(max_positions=cfg.n_positions, hidden_size=cfg.n_embd),
                          {"weight": "wpe.weight"}),
        layers=tuple(layers),
        run_order=tuple(RunEntry(i) for i in range(cfg.n_layer)),
        final_norm=PartSpec("layer_norm", dict(hidden_size=cfg.n_embd, eps=cfg.layer_norm_epsilon),
                            {"weight": "ln_f.weight", "bias": "ln_f.bias"}),
        head=PartSpec("tied_to_embedding", dict(vocab_size=cfg.vocab_size, hidden_size=cfg.n_embd)),
        eos_token_id=cfg.eos_token_id,
        optional_prefixes=("transformer.",),
        # buffers and the tied copy that Hugging Face checkpoints carry
        # (rosellm/rosetrainer/hf_gpt2.py:53 ties lm_head to wte and skips the rest)
        ignored_tensors=("h.*.attn.bias", "h.*.attn.masked_bias", "lm_head.weight"),
    )


register_architecture("GPT2LMHeadModel", GPT2Config, build_gpt2_spec, model_types=("gpt2",), replace=True)
