"""A plain, slow GPT-2: whole sequences, no cache, one function per part.

Written from the formulas of the reference's model code (each function cites
file:line of chtho-like/rosellm); it reads the model folder itself and shares
no code with ``rosellm_b200``.  ``tests/golden/make_golden.py`` compares it
once with the reference's own ``GPTModel`` run on the CPU and commits the
outputs; the tests compare the engine with it.

Tensors are in the checkpoint's own names and layout (Hugging Face GPT-2:
``Conv1D`` weights are ``[in, out]``), so ``y = x @ W + b`` needs no transpose
(rosellm/rosetrainer/hf_gpt2.py:12-13, 66-76 transposes them into
``nn.Linear`` layout instead).
"""
from __future__ import annotations

import json
import math
import os

import numpy as np
import torch


def load_folder(model_dir: str, dtype: torch.dtype = torch.float64, device: str = "cpu"):
    """(config dict, tensors by name in ``dtype``) of a model folder.  ``device``: where the
    tensors live; every function below computes where its inputs are (the large models of the
    tests run this plain code in float64 on the GPU, where it takes seconds instead of minutes)."""
    from safetensors.torch import load_file

    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    tensors = {k: v.to(device=device, dtype=dtype)
               for k, v in load_file(os.path.join(model_dir, "model.safetensors")).items()}
    return cfg, tensors


def embed(ids: torch.Tensor, wte: torch.Tensor, wpe: torch.Tensor) -> torch.Tensor:
    """x[t] = wte[id_t] + wpe[t]  (rosellm/rosetrainer/model.py:543-562)."""
    return wte[ids] + wpe[torch.arange(ids.numel(), device=wte.device)]


def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float) -> torch.Tensor:
    """(x - mean) / sqrt(var + eps) * weight + bias, biased variance over the last dim
    (rosellm/rosetrainer/fused_layernorm.py:99-120; nn.LayerNorm in model.py:355-356)."""
    mean = x.mean(dim=-1, keepdim=True)
    var = ((x - mean) ** 2).mean(dim=-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * weight + bias


def gelu_tanh(u: torch.Tensor) -> torch.Tensor:
    """0.5 u (1 + tanh(sqrt(2/pi) (u + 0.044715 u^3)))  (rosellm/rosetrainer/model.py:274-277)."""
    return 0.5 * u * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (u + 0.044715 * u ** 3)))


def gelu_erf(u: torch.Tensor) -> torch.Tensor:
    """0.5 u (1 + erf(u / sqrt 2)): F.gelu, taken for every activation name but "gelu_new"
    (rosellm/rosetrainer/model.py:343-346)."""
    return 0.5 * u * (1.0 + torch.erf(u / math.sqrt(2.0)))


def activation_of(name: str):
    return gelu_erf if name == "gelu" else gelu_tanh


def _same(x: torch.Tensor) -> torch.Tensor:
    return x


def to_bfloat16_and_back(x: torch.Tensor) -> torch.Tensor:
    """Rounds to bfloat16: passed as ``rounding`` below it shows how much noise storing the
    activations between products, and the cache, in 16 bits puts on the logits."""
    return x.to(torch.bfloat16).to(x.dtype)


def attention(h: torch.Tensor, w_attn, b_attn, w_proj, b_proj, n_head: int,
              window: int | None = None, rounding=_same) -> torch.Tensor:
    """Causal multi-head self-attention over a whole sequence [T, D]
    (rosellm/rosetrainer/model.py:95-98 packed qkv and head split, :169-185 scores, mask,
    softmax, :218-220 merge and output projection)."""
    T, D = h.shape
    dh = D // n_head
    qkv = rounding(h @ w_attn + b_attn)
    q, k, v = qkv.split(D, dim=-1)
    q = q.view(T, n_head, dh).transpose(0, 1)
    k = k.view(T, n_head, dh).transpose(0, 1)
    v = v.view(T, n_head, dh).transpose(0, 1)
    scores = q @ k.transpose(-2, -1) * dh ** -0.5
    i = torch.arange(T, device=h.device)
    visible = i[None, :] <= i[:, None]
    if window is not None:
        visible &= i[None, :] > i[:, None] - window
    scores = scores.masked_fill(~visible, float("-inf"))
    probs = torch.softmax(scores, dim=-1)
    o = rounding((probs @ v).transpose(0, 1).reshape(T, D))
    return o @ w_proj + b_proj


def mlp(h: torch.Tensor, w_fc, b_fc, w_proj, b_proj, act, rounding=_same) -> torch.Tensor:
    """act(h W_fc + b) W_proj + b  (rosellm/rosetrainer/model.py:339-347)."""
    return rounding(act(h @ w_fc + b_fc)) @ w_proj + b_proj


def block(x: torch.Tensor, t: dict, i: int, cfg: dict, rounding=_same) -> torch.Tensor:
    """x += attn(ln_1(x)); x += mlp(ln_2(x))  (rosellm/rosetrainer/model.py:372-428)."""
    p = f"h.{i}."
    eps = cfg.get("layer_norm_epsilon", 1e-5)
    a = rounding(layer_norm(x, t[p + "ln_1.weight"], t[p + "ln_1.bias"], eps))
    x = x + attention(a, t[p + "attn.c_attn.weight"], t[p + "attn.c_attn.bias"],
                      t[p + "attn.c_proj.weight"], t[p + "attn.c_proj.bias"], cfg["n_head"], rounding=rounding)
    a = rounding(layer_norm(x, t[p + "ln_2.weight"], t[p + "ln_2.bias"], eps))
    act = activation_of(cfg.get("activation_function", "gelu_new"))
    return x + mlp(a, t[p + "mlp.c_fc.weight"], t[p + "mlp.c_fc.bias"],
                   t[p + "mlp.c_proj.weight"], t[p + "mlp.c_proj.bias"], act, rounding=rounding)


def hidden_states(cfg: dict, t: dict, ids, rounding=_same) -> torch.Tensor:
    ids = torch.as_tensor(ids, dtype=torch.long).to(t["wte.weight"].device)
    x = embed(ids, t["wte.weight"], t["wpe.weight"])
    for i in range(cfg["n_layer"]):
        x = block(x, t, i, cfg, rounding)
    return x


def forward(cfg: dict, t: dict, ids, rounding=_same, rows=None) -> torch.Tensor:
    """Logits [T, V] of a whole sequence: final LayerNorm, then the token table as head
    (rosellm/rosetrainer/model.py:613-641; tied at :503-504).  ``rounding`` is applied where
    a 16-bit engine stores activations (after each norm, the packed qkv, the merged heads,
    the MLP's inner activation); the default leaves everything in full precision.
    ``rows``: positions whose logits are wanted (all when ``None``); the layers run on the
    whole sequence either way."""
    x = hidden_states(cfg, t, ids, rounding)
    if rows is not None:
        x = x[torch.as_tensor(rows, dtype=torch.long).to(x.device)]
    x = rounding(layer_norm(x, t["ln_f.weight"], t["ln_f.bias"], cfg.get("layer_norm_epsilon", 1e-5)))
    return x @ t["wte.weight"].t()


def greedy(cfg: dict, t: dict, prompt: list[int], n_new: int) -> list[int]:
    """Greedy continuation by re-running the whole sequence for each token
    (as rosellm/rosetrainer/generate.py does without a cache)."""
    ids = list(prompt)
    for _ in range(n_new):
        ids.append(int(forward(cfg, t, ids)[-1].argmax()))
    return ids[len(prompt):]


# ---- sampling ---------------------------------------------------------------------------

def top_k_filter(logits: torch.Tensor, top_k: int) -> torch.Tensor:
    """Keep the k largest logits, the rest -inf (rosellm/roseinfer/engine.py:1039-1054)."""
    vocab = logits.numel()
    if top_k <= 0 or top_k >= vocab:
        return logits
    kth = torch.topk(logits, top_k).values[-1]
    return torch.where(logits < kth, torch.full_like(logits, float("-inf")), logits)


def top_p_filter(logits: torch.Tensor, top_p: float) -> torch.Tensor:
    """Sort descending, softmax, cumulative sum; drop entries whose cumulative probability
    (itself included) exceeds p, but never the first (rosellm/roseinfer/engine.py:1056-1084,
    1163-1169)."""
    if top_p <= 0.0 or top_p >= 1.0:
        return logits
    sorted_logits, idx = torch.sort(logits, descending=True)
    cum = torch.cumsum(torch.softmax(sorted_logits, dim=-1), dim=-1)
    drop = cum > top_p
    drop[0] = False
    out = logits.clone()
    out[idx[drop]] = float("-inf")
    return out


def filtered_logits(logits: torch.Tensor, temperature: float, top_k: int, top_p: float) -> torch.Tensor:
    """logits / T, then top-k, then top-p on the softmax of what top-k kept
    (rosellm/roseinfer/engine.py:1149-1171)."""
    return top_p_filter(top_k_filter(logits / temperature, top_k), top_p)


_M0, _M1, _W0, _W1 = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85


def philox_first(c0: np.ndarray, c1: int, seed: int) -> np.ndarray:
    """First word of Philox-4x32-10 with counter (c0, c1, 0, 0) and key = the seed's halves."""
    mask = np.uint64(0xFFFFFFFF)
    c0 = c0.astype(np.uint64)
    c1 = np.full_like(c0, c1, dtype=np.uint64)
    c2 = np.zeros_like(c0)
    c3 = np.zeros_like(c0)
    k0 = np.uint64(seed & 0xFFFFFFFF)
    k1 = np.uint64((seed >> 32) & 0xFFFFFFFF)
    for _ in range(10):
        p0 = np.uint64(_M0) * c0
        p1 = np.uint64(_M1) * c2
        hi0, lo0 = p0 >> np.uint64(32), p0 & mask
        hi1, lo1 = p1 >> np.uint64(32), p1 & mask
        c0, c1, c2, c3 = (hi1 ^ c1 ^ k0) & mask, lo1, (hi0 ^ c3 ^ k1) & mask, lo0
        k0 = (k0 + np.uint64(_W0)) & mask
        k1 = (k1 + np.uint64(_W1)) & mask
    return c0.astype(np.uint32)


def gumbel_noise(seed: int, counter: int, vocab: int) -> np.ndarray:
    x = philox_first(np.arange(vocab, dtype=np.uint64), counter, seed)
    u = ((x >> np.uint32(8)).astype(np.float64) + 0.5) * 2.0 ** -24
    return -np.log(-np.log(u))


def gumbel_sample(logits: torch.Tensor, temperature: float, top_k: int, top_p: float,
                  seed: int, counter: int) -> tuple[int, np.ndarray]:
    """(token, scores): arg-max of filtered logits + Gumbel noise, which draws from their softmax."""
    kept = filtered_logits(logits.double(), temperature, top_k, top_p).numpy()
    scores = kept + gumbel_noise(seed, counter, logits.numel())
    return int(np.argmax(scores)), scores
