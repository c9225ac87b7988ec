"""The parts this package ships: what GPT-2 is assembled from.

Each part takes its sizes and constants as constructor parameters and calls
the sm_100a kernels through ``rosellm_b200.ops.kernels``.  The residual
stream ``x`` is float32 ``[tokens, hidden]`` in both precisions; activations
between a norm and a matrix product are in the compute dtype.
"""
from __future__ import annotations

import torch

from ..ops import kernels as K
from .base import KVCacheSpec, ParamSpec, Part, register_part


@register_part("position", "none")
class NoPositions(Part):
    """No position information is added anywhere."""

    graph_safe = True
    launches_replayable = True
    rotates = False  # rotate() changes nothing: keys may go to the cache straight from the qkv product

    def table(self):
        return None

    def rotate(self, ctx, q, k) -> None:
        return None


@register_part("position", "learned_absolute")
class LearnedAbsolutePositions(Part):
    """A learned table added to the token embedding: ``x = wte[id] + wpe[pos]``
    (rosellm/rosetrainer/model.py:543-562)."""

    graph_safe = True
    launches_replayable = True
    rotates = False

    def __init__(self, max_positions: int, hidden_size: int) -> None:
        self.max_positions = max_positions
        self.hidden_size = hidden_size
        self.weight = None

    def param_specs(self):
        return [ParamSpec("weight", (self.max_positions, self.hidden_size))]

    def table(self):
        return self.weight

    def rotate(self, ctx, q, k) -> None:
        return None


@register_part("embedding", "token_table")
class TokenEmbedding(Part):
    graph_safe = True
    launches_replayable = True

    def __init__(self, vocab_size: int, hidden_size: int) -> None:
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size
        self.weight = None

    def param_specs(self):
        return [ParamSpec("weight", (self.vocab_size, self.hidden_size))]

    def forward(self, ctx, position) -> torch.Tensor:
        x = ctx.workspace.get("residual", (ctx.n_tokens, self.hidden_size), torch.float32)
        K.embed(ctx.token_ids, ctx.positions, self.weight, position.table(), x, ctx.extras.get("token_feedback"))
        return x


@register_part("norm", "layer_norm")
class LayerNorm(Part):
    """``(x - mean) * rsqrt(var + eps) * weight + bias`` over the last dimension
    (rosellm/rosetrainer/fused_layernorm.py:99-120)."""

    graph_safe = True
    launches_replayable = True
    can_defer = True  # forward(..., defer=True) may hand the consumer a K.NormInput to fuse

    def __init__(self, hidden_size: int, eps: float, bias: bool = True) -> None:
        self.hidden_size = hidden_size
        self.eps = eps
        self.has_bias = bias
        self.weight = None
        self.bias = None

    def param_specs(self):
        specs = [ParamSpec("weight", (self.hidden_size,), kind="vector", init="ones")]
        if self.has_bias:
            specs.append(ParamSpec("bias", (self.hidden_size,), kind="vector", init="zeros"))
        return specs

    def forward(self, ctx, x, rows=None, n_rows=None, name="normed", defer: bool = False):
        """Normalised rows in the activation dtype.  With ``defer`` (the consumer has declared
        ``takes_norm_input``) and few, short rows in bfloat16, a ``K.NormInput`` instead: the
        consumer's first product normalises inside its own kernel and no kernel runs here."""
        if defer and rows is None and K.NormInput.possible(x.shape[0], self.hidden_size, ctx.act_dtype):
            return K.NormInput(x, self.weight, self.bias, self.eps)
        n = x.shape[0] if rows is None else int(n_rows)
        out = ctx.workspace.get(name, (n, self.hidden_size), ctx.act_dtype)
        K.layernorm(x, self.weight, self.bias, self.eps, out, rows)
        return out


_NARROW_PARTS: dict[tuple, int] = {}  # (request-head pairs, keys, bytes a key, blocks at once) -> parts, as computed before


def narrow_decode_blocks_at_once(head_dim: int, element_bytes: int, percent: int = 50) -> int:
    """How many four-warp blocks of the decode attention run at once on the device: each holds
    a ring of two tiles of keys and values per warp in shared memory (csrc/attention_kernels.cuh,
    ``DecodeTile``: 4 warps x 2 stages x 2 x the tile's words), and every small kernel of the
    library asks for half of an SM's memory as shared memory.  ``percent``: the denser forms of
    the kernel ask for 80 % or all of it (taken when the blocks would not run at once otherwise)."""
    words = head_dim // 8 * element_bytes // 4
    sub = 4 if words <= 4 else (2 if words <= 8 else 1)
    block = 4 * 2 * 2 * sub * 32 * words * 4 + 1024  # the ring, and what the driver keeps per block
    sms, shared = K.device_facts()
    return sms * max(1, min(16, (shared * percent // 100) // block))


# The forms of the narrow kernel: (share of an SM's memory as shared memory, what a key costs a
# block against the common form; less L1 is left beside the shared memory).  Measured at 40, 48
# and 64 requests of 512 keys: 13.6, 14.0 us (80 %: five blocks an SM) and 18.2 us (all of it:
# six) in one round against 18.4, 19.7 and 20.6 us in two rounds of the common form; 48 requests
# of 1024 keys: 29.7 us whole, 35.5 in two parts, 32.1 in three.
NARROW_FORMS = ((50, 1.0), (80, 1.15), (100, 1.3))


# Longest context of a step from which prompt portions go to the tcgen05 attention kernel
# (measured on B200, 12 heads of 64: 48 against 56 TFLOP/s at 256 tokens, 101 against 86 at
# 1024, 131 against 96 at 2048).
TC_ATTENTION_MIN_CONTEXT = 512


@register_part("mixer", "causal_self_attention")
class CausalSelfAttention(Part):
    """Multi-head causal attention over the paged cache.

    ``qkv = h W_qkv + b``, columns split into queries, keys and values in that
    order, head ``j // head_dim`` owning column ``j`` of each
    (rosellm/rosetrainer/model.py:95-98, 248-255); the step's keys and values
    are written to the cache, then every query attends over the cached keys
    up to its own position (csrc/attention.cu); heads are merged and
    ``x += o W_out + b`` (model.py:218-221, 412-413).
    """

    graph_safe = True
    launches_replayable = True
    takes_norm_input = True  # h may be a K.NormInput: the qkv product then normalises its own input

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, num_kv_heads: int | None = None,
                 window: int | None = None, scale: float | None = None, bias: bool = True,
                 weights_in_out: bool = False) -> None:
        self.hidden_size = hidden_size
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads if num_kv_heads is not None else num_heads
        self.head_dim = head_dim
        self.window = window
        self.scale = scale if scale is not None else head_dim ** -0.5
        self._split = (None, None, None, None)  # the packed qkv buffer last seen and its three views
        self.has_bias = bias
        self.weights_in_out = weights_in_out
        if head_dim % 16 != 0 or head_dim > 256:
            raise ValueError(f"head size {head_dim}: the attention kernels take multiples of 16 up to 256")
        if self.num_heads % self.num_kv_heads != 0:
            raise ValueError(f"{num_heads} heads are not a multiple of {self.num_kv_heads} key/value heads")
        self.q_width = self.num_heads * head_dim
        self.kv_width = self.num_kv_heads * head_dim
        self.qkv_weight = self.qkv_bias = self.out_weight = self.out_bias = None
        self._out_weight_packed = None

    def _matrix(self, role, n_out, n_in):
        shape = (n_in, n_out) if self.weights_in_out else (n_out, n_in)
        return ParamSpec(role, shape, transpose=self.weights_in_out)

    def param_specs(self):
        qkv = self.q_width + 2 * self.kv_width
        specs = [self._matrix("qkv_weight", qkv, self.hidden_size),
                 self._matrix("out_weight", self.hidden_size, self.q_width)]
        if self.has_bias:
            specs += [ParamSpec("qkv_bias", (qkv,), kind="vector"),
                      ParamSpec("out_bias", (self.hidden_size,), kind="vector")]
        return specs

    def cache_spec(self):
        return KVCacheSpec(self.num_kv_heads, self.head_dim, self.window)

    def decode_plan_for(self, n_decode: int, span: int, act_dtype: torch.dtype = torch.bfloat16) -> tuple[int, bool]:
        """(splits, wide): over how many blocks the keys of one decoded request are split when
        ``n_decode`` requests attend over about ``span`` keys each, and whether the blocks have
        sixteen warps instead of four.  With few requests wide blocks take 256 keys a round, so
        that a request's keys need no split and no merge; with many, narrow blocks fill the SMs."""
        if n_decode == 0:
            return 1, False
        if self.window is not None:
            span = min(span, self.window)
        units = n_decode * self.num_heads
        sms = K.sm_count()
        if units <= 2 * sms:
            return max(1, min(span // 1024, 2 * sms // units, 32)), True   # up to four rounds a block
        # Narrow blocks: a few fit on an SM (shared memory); where they do not all run at once the
        # kernel takes its dense form (twice as many an SM, each slower), and what is still left
        # waits for a second round.
        # Measured on B200 with 12 heads of 64 in bfloat16 (three blocks an SM, 256 bytes a key):
        # a round costs about 0.8 us + 0.0152 us a key, and a split adds the merge kernel,
        # 6 us + 1 us a part (32 x 512: 10.3 us whole against 15.7 us in two parts).  Other head
        # sizes and the 32-bit cache scale the cost of a key by the bytes it takes, and change
        # how many blocks fit.
        element_bytes = 2 if act_dtype == torch.bfloat16 else 4
        key_bytes = 2 * self.head_dim * element_bytes
        at_once = narrow_decode_blocks_at_once(self.head_dim, element_bytes)
        span = -(-span // 64) * 64  # in steps of 64 keys: every layer of a step, and most steps, ask the same
        best = _NARROW_PARTS.get((units, span, key_bytes, at_once))
        if best is None:
            best_cost, best = None, 1
            per_key = 0.0152 * key_bytes / 256.0
            forms = [(narrow_decode_blocks_at_once(self.head_dim, element_bytes, pc), f) for pc, f in NARROW_FORMS]
            for parts in range(1, min(span // 64, 32) + 1):
                # the form the kernel takes (csrc/attention_kernels.cuh: launch_decode): the
                # first that holds all blocks at once, else the densest
                room, factor = next(((r, f) for r, f in forms if units * parts <= r), forms[-1])
                rounds, key_cost = -(-units * parts // room), per_key * factor
                cost = rounds * (0.8 + key_cost * span / parts) + (6.0 + 1.0 * parts if parts > 1 else 0.0)
                if best_cost is None or cost < best_cost - 1e-9:
                    best_cost, best = cost, parts
            if len(_NARROW_PARTS) > 4096:
                _NARROW_PARTS.clear()
            _NARROW_PARTS[(units, span, key_bytes, at_once)] = best
        return best, False

    def decode_plan(self, ctx) -> tuple[int, bool]:
        return self.decode_plan_for(ctx.n_decode, ctx.max_kv_len, ctx.act_dtype)

    @staticmethod
    def _tc_prompt_attention(ctx) -> bool:
        """Whether the step's prompt portions go to the tcgen05 kernel: decided by the longest
        context among the requests that bring portions (decoded requests beside them have
        nothing to do with it)."""
        return ctx.max_tile_kv_len >= TC_ATTENTION_MIN_CONTEXT

    def launch_key(self, ctx) -> tuple:
        """The longest context decides how decoded requests are split over blocks and which
        kernel takes the prompt portions."""
        return (ctx.extras.get("decode_plan") or self.decode_plan(ctx) if ctx.n_decode else None,
                self._tc_prompt_attention(ctx) if ctx.n_tiles else None)

    def bind(self, tensors) -> None:
        super().bind(tensors)
        # the fused kernel of a decode step reads W_out slice by slice: laid out for it once, here
        self._out_weight_packed = None
        w = self.out_weight
        if (w is not None and w.is_cuda and self.window is None and self.num_kv_heads == self.num_heads
                and self.q_width == self.hidden_size):
            cluster = K.attn_block_fused_cluster(self.hidden_size, self.num_heads, self.head_dim, w.dtype)
            if cluster:
                self._out_weight_packed = K.attn_pack_out_weight(w, self.num_heads, self.head_dim, cluster)

    def _fused_decode(self, ctx, run, h, x) -> bool:
        """A step of few decoded requests and nothing else: the whole of this part (its norm
        included) in one kernel, where the sizes fit."""
        n = ctx.n_tokens
        return (self._out_weight_packed is not None and K.FUSED_ROWS and n <= 16
                and isinstance(h, K.NormInput) and h.x is x and n == ctx.n_decode == ctx.n_reqs and run.writes_cache
                and not getattr(ctx.position, "rotates", True))

    def forward(self, ctx, run, h, x) -> None:
        if self._fused_decode(ctx, run, h, x):
            K.attn_block_fused(x, h, self.qkv_weight, self.qkv_bias, self._out_weight_packed, self.out_bias,
                               ctx.kv_pool(run.cache_key), ctx.block_table(run.cache_key), ctx.positions, ctx.slots,
                               n_heads=self.num_heads, scale=self.scale, max_pos=ctx.cache.max_seq_len)
            return
        n = ctx.n_tokens
        qkv_w = self.q_width + 2 * self.kv_width
        qkv = ctx.workspace.get("qkv", (n, qkv_w), ctx.act_dtype)
        pool = ctx.kv_pool(run.cache_key)
        table = ctx.block_table(run.cache_key)
        # keys and values can go to their pages straight from the product when nothing has to
        # touch them in between (no rotation) and the product runs the row kernel
        fuse_write = (run.writes_cache and not getattr(ctx.position, "rotates", True)
                      and K.product_writes_cache(n, ctx.act_dtype, qkv_w, self.hidden_size))
        target = None
        if fuse_write:
            target = K.KvTarget(pool, table, ctx.positions, ctx.req_of_token, ctx.slots, self.q_width,
                                ctx.cache.max_seq_len)
        K.linear(h, self.qkv_weight, self.qkv_bias, qkv, kv=target)
        if self._split[0] is not qkv:  # the workspace hands out one tensor object per size
            self._split = (qkv, qkv[:, : self.q_width], qkv[:, self.q_width: self.q_width + self.kv_width],
                           qkv[:, self.q_width + self.kv_width:])
        _, q, k, v = self._split
        if not fuse_write:
            ctx.position.rotate(ctx, q, k)
            if run.writes_cache:
                K.kv_write(k, v, pool, table, ctx.positions, ctx.req_of_token, ctx.slots, ctx.cache.max_seq_len)
        o = ctx.workspace.get("attn_out", (n, self.q_width), ctx.act_dtype)
        splits, wide = ctx.extras.get("decode_plan") or self.decode_plan(ctx)
        part_o = part_ml = None
        if splits > 1:
            rows = ctx.n_decode * self.num_heads * splits
            part_o = ctx.workspace.get("attn_part_o", (rows, self.head_dim), torch.float32)
            part_ml = ctx.workspace.get("attn_part_ml", (rows, 2), torch.float32)
        K.attention(q, pool, table, ctx.q_start, ctx.kv_len, ctx.slots, o, n_heads=self.num_heads,
                    scale=self.scale, window=self.window, tiles=ctx.tiles, n_tiles=ctx.n_tiles,
                    decode_reqs=ctx.decode_reqs, n_decode=ctx.n_decode, n_splits=splits,
                    part_o=part_o, part_ml=part_ml, tiles_wide=ctx.tiles_wide, n_tiles_wide=ctx.n_tiles_wide,
                    decode_wide=wide,
                    # what decoded requests read of the cache beside their newest key is of earlier
                    # steps, and a step begins with a copy to the device that separates it from them
                    old_keys_settled=True,
                    # prompt portions: the tcgen05 kernel (where its sizes fit) wins once a block
                    # walks several tiles of keys; short contexts are faster on mma.sync
                    prefill_path=None if self._tc_prompt_attention(ctx) else "mma")
        K.linear(o, self.out_weight, self.out_bias, x, residual=True)


@register_part("feed_forward", "dense_mlp")
class DenseMLP(Part):
    """``x += act(h W_in + b_in) W_out + b_out`` (rosellm/rosetrainer/model.py:331-349);
    ``activation`` is ``gelu_tanh`` (model.py:274-277) or ``gelu_erf`` (``F.gelu``)."""

    graph_safe = True
    launches_replayable = True
    takes_norm_input = True

    def __init__(self, hidden_size: int, inner_size: int, activation: str, bias: bool = True,
                 weights_in_out: bool = False) -> None:
        if activation not in K.ACTIVATIONS or activation == "none":
            raise ValueError(f"activation {activation!r}; one of gelu_tanh, gelu_erf")
        self.hidden_size = hidden_size
        self.inner_size = inner_size
        self.activation = K.ACTIVATIONS[activation]
        self.has_bias = bias
        self.weights_in_out = weights_in_out
        self.in_weight = self.in_bias = self.out_weight = self.out_bias = None
        self._fused_slice, self._out_weight_packed = 0, None

    def _matrix(self, role, n_out, n_in):
        shape = (n_in, n_out) if self.weights_in_out else (n_out, n_in)
        return ParamSpec(role, shape, transpose=self.weights_in_out)

    def param_specs(self):
        specs = [self._matrix("in_weight", self.inner_size, self.hidden_size),
                 self._matrix("out_weight", self.hidden_size, self.inner_size)]
        if self.has_bias:
            specs += [ParamSpec("in_bias", (self.inner_size,), kind="vector"),
                      ParamSpec("out_bias", (self.hidden_size,), kind="vector")]
        return specs

    def bind(self, tensors) -> None:
        """The products read rows in 16-byte pieces, so an inner size that is no multiple of 8
        is filled up with units whose weights and bias are zero: their activation is 0 (both
        GELU forms map 0 to 0) and they add nothing to the output."""
        super().bind(tensors)
        pad = -self.inner_size % 8
        self.inner_padded = self.inner_size + pad
        if pad:
            self.in_weight = torch.nn.functional.pad(self.in_weight, (0, 0, 0, pad)).contiguous()
            self.out_weight = torch.nn.functional.pad(self.out_weight, (0, pad)).contiguous()
            if self.in_bias is not None:
                self.in_bias = torch.nn.functional.pad(self.in_bias, (0, pad)).contiguous()
        # the fused kernel of few rows reads W_out slice by slice: laid out for it once, here
        self._fused_slice, self._out_weight_packed = 0, None
        if self.out_weight.is_cuda:
            self._fused_slice = K.mlp_fused_slice(1, self.hidden_size, self.inner_padded, True, self.out_weight.dtype)
            if self._fused_slice:
                self._out_weight_packed = K.mlp_pack_out_weight(self.out_weight, self._fused_slice)

    def forward(self, ctx, h, x) -> None:
        # few rows: both products in one kernel, the inner activations never leave the SM
        width = self._fused_slice if ctx.n_tokens <= 16 and K.FUSED_ROWS else 0
        if width:
            K.mlp_fused(x, h, self.in_weight, self.in_bias, self._out_weight_packed, self.out_bias, act=self.activation,
                        slice_width=width)
            return
        u = ctx.workspace.get("mlp_inner", (ctx.n_tokens, self.inner_padded), ctx.act_dtype)
        K.linear(h, self.in_weight, self.in_bias, u, act=self.activation)
        K.linear(u, self.out_weight, self.out_bias, x, residual=True)


@register_part("block", "pre_norm")
class PreNormBlock(Part):
    """``x += mixer(norm(x)); x += feed_forward(norm(x))`` (rosellm/rosetrainer/model.py:372-428)."""

    graph_safe = True
    launches_replayable = True
    # the sub-parts of a layer this block arranges, by name and category
    uses = {"norm_mixer": "norm", "mixer": "mixer", "norm_feed_forward": "norm", "feed_forward": "feed_forward"}

    def forward(self, ctx, run, layer, x) -> None:
        h = self._normed(ctx, layer.norm_mixer, x, layer.mixer)
        layer.mixer.forward(ctx, run, h, x)
        h = self._normed(ctx, layer.norm_feed_forward, x, layer.feed_forward)
        layer.feed_forward.forward(ctx, h, x)

    @staticmethod
    def _normed(ctx, norm, x, consumer):
        """The norm's output; between a norm that can defer and a consumer that takes it, the
        norm is handed over unevaluated for the consumer to fuse into its first product."""
        if getattr(norm, "can_defer", False) and getattr(consumer, "takes_norm_input", False):
            return norm.forward(ctx, x, defer=True)
        return norm.forward(ctx, x)


@register_part("head", "tied_to_embedding")
class TiedHead(Part):
    """``logits = h wte^T`` with the embedding's own table, no bias
    (rosellm/rosetrainer/model.py:503-504, 639-641)."""

    graph_safe = True
    launches_replayable = True

    def __init__(self, vocab_size: int, hidden_size: int) -> None:
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size
        self.weight = None  # set by the model to the embedding's table

    tied = True
    takes_norm_input = True  # h may be a K.NormInput: the product then normalises its own input

    def forward(self, ctx, h) -> torch.Tensor:
        n_rows = h.x.shape[0] if isinstance(h, K.NormInput) else h.shape[0]
        logits = ctx.workspace.get("logits", (n_rows, self.vocab_size), torch.float32)
        K.linear(h, self.weight, None, logits)
        return logits

    def can_sample(self, n_rows: int, dtype: torch.dtype, with_temperature: bool = False) -> bool:
        """Whether ``forward_sample`` should be given this many rows (some of them with a
        temperature, or all taking the arg-max): a head that can choose the next tokens inside
        its product writes no logits for them."""
        return K.sampling_product_possible(n_rows, self.vocab_size, self.hidden_size, dtype, with_temperature)

    def forward_sample(self, ctx, h, into: "K.SampleInto") -> None:
        """The next token of every row of ``h`` into ``into.out_ids`` (arg-max, or by the rows'
        temperatures), chosen in the product's epilogue: what the sampling kernel would choose
        from ``forward``'s logits."""
        K.linear_sample(h, self.weight, None, into)


@register_part("head", "linear")
class LinearHead(TiedHead):
    """``logits = h W^T`` with a table of its own."""

    tied = False

    def param_specs(self):
        return [ParamSpec("weight", (self.vocab_size, self.hidden_size))]
