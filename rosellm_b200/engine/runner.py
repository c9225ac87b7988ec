"""The step function.

``ModelRunner.step`` takes a batch of (request slot, its next tokens, the
places whose logits are wanted), runs exactly those tokens through the model
as one batch against the cache that earlier steps left, and returns the
logits at the wanted places.  Portions of prompts and single decoded tokens
may share a batch and a prompt may be cut anywhere.  The reference runs the
two kinds in two forward passes of one scheduler step
(rosellm/roseinfer/engine.py:3875-3878 decode, then :3931-3938 chunked
prefill through ``prefill_chunk_sessions``, :738-1037, which needs FlashInfer
and a 16-bit dtype); here both are one pass in either precision.

The host packs the step's index arrays into one pinned buffer and copies it
to the device once; steps that only decode can be replayed from a CUDA graph
captured per batch-size bucket (the reference captures one graph per batch
size as well, rosellm/roseinfer/engine.py:1697-1832).
"""
from __future__ import annotations

import array
import warnings
from dataclasses import dataclass

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..cache.sizing import kv_bytes_per_token, plan_cache
from ..config.base import ModelConfig, load_config, resolve_architecture
from ..config.engine import EngineConfig
from ..models.model import Model
from ..ops import kernels as K
from ..weights.loader import read_safetensors
from .context import HostBatch, StepContext, Workspace, build_host_batch


class OutOfPages(RuntimeError):
    """The cache has no pages left for a step's tokens."""


@dataclass
class StepEntry:
    slot: int
    token_ids: list[int]  # or an integer array
    want: list[int]


TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


class _Staging:
    """Pinned host buffers, used in turn, each guarded by an event of its last copy."""

    def __init__(self, n_ints: int, depth: int = 4) -> None:
        self.bufs = [torch.empty(n_ints, dtype=torch.int32, pin_memory=True) for _ in range(depth)]
        self.arrays = [b.numpy() for b in self.bufs]   # the same memory, as numpy sees it
        self.addresses = [b.data_ptr() for b in self.bufs]
        self.events: list[torch.cuda.Event | None] = [None] * depth
        self.at = 0

    def next(self) -> tuple[int, torch.Tensor]:
        i = self.at
        self.at = (self.at + 1) % len(self.bufs)
        if self.events[i] is not None:
            self.events[i].synchronize()
        return i, self.bufs[i]

    def mark(self, i: int) -> None:
        ev = self.events[i]
        if ev is None:
            ev = self.events[i] = torch.cuda.Event()
        K.record_event(ev)


def _layout(n_tokens: int, n_reqs: int, n_rows: int, n_decode: int, n_tiles: int, n_wide: int = 0
            ) -> dict[str, tuple[int, int]]:
    """Offsets (in int32) of the step's arrays inside the packed buffer."""
    out = {}
    at = 0
    for name, n in (("token_ids", n_tokens), ("positions", n_tokens), ("req_of_token", n_tokens),
                    ("q_start", n_reqs + 1), ("kv_len", n_reqs), ("slots", n_reqs),
                    ("logit_rows", n_rows), ("decode_reqs", n_decode), ("tiles", 2 * n_tiles),
                    ("tiles_wide", 2 * n_wide)):
        out[name] = (at, n)
        at += (n + 3) // 4 * 4  # every array starts on a 16-byte boundary
    out["_total"] = (at, 0)
    return out


class ModelRunner:
    def __init__(self, config: ModelConfig, file_tensors: dict[str, torch.Tensor],
                 engine_config: EngineConfig | None = None, source: str = "<tensors>") -> None:
        self.config = config
        self.engine_config = ec = engine_config or EngineConfig()
        self.device = torch.device(ec.device)
        if self.device.type != "cuda" or not torch.cuda.is_available():
            raise RuntimeError(
                "rosellm_b200 runs on a CUDA device only (there is no CPU path); "
                f"device={ec.device!r}, torch.cuda.is_available()={torch.cuda.is_available()}"
            )
        torch.cuda.set_device(self.device)
        K._lib()  # build or load the CUDA library now: fail here, loudly, if it cannot be had
        self.dtype = TORCH_DTYPES[ec.dtype]
        self.spec = resolve_architecture(config.to_dict()).build_spec(config)
        self.model = Model(self.spec, self.dtype, self.device)
        self.model.load_tensors(file_tensors, source)
        kv_specs, state_specs = self.model.kv_specs(), self.model.state_specs()
        self.cache_plan = plan = plan_cache(
            page_size=ec.page_size, max_num_seqs=ec.max_num_seqs,
            max_model_len=min(ec.max_model_len or self.spec.max_positions, self.spec.max_positions),
            bytes_per_token=kv_bytes_per_token(kv_specs, ec.dtype),
            num_pages=ec.num_pages, kv_cache_tokens=ec.kv_cache_tokens,
            gpu_memory_utilization=ec.gpu_memory_utilization, kv_cache_mem_fraction=ec.kv_cache_mem_fraction,
            mem_get_info=lambda: torch.cuda.mem_get_info(self.device),
            reserve_bytes=self._bytes_beside_the_cache(state_specs),
        )
        if plan.clamped_from is not None:
            warnings.warn(
                f"the cache sized by {plan.how} gives each of {ec.max_num_seqs} sequences "
                f"{plan.max_model_len} tokens; the longest sequence is shortened from {plan.clamped_from} to that"
            )
        self.max_model_len = plan.max_model_len
        self.cache = CacheManager(
            kv_specs, state_specs,
            page_size=ec.page_size, num_pages=plan.num_pages, max_slots=ec.max_num_seqs,
            max_seq_len=self.max_model_len, dtype=self.dtype, device=self.device,
        )
        self.workspace = Workspace(self.device)
        t_cap, r_cap = ec.max_num_batched_tokens, ec.max_num_seqs
        cap = _layout(t_cap, r_cap, t_cap, r_cap, t_cap // 16 + r_cap + 1, t_cap // 64 + r_cap + 1)["_total"][0]
        self._staging = _Staging(cap)
        self._dev_ints = torch.zeros(cap, dtype=torch.int32, device=self.device)
        self._graphs: dict[int, tuple] = {}
        self._views: dict[tuple, dict[str, torch.Tensor]] = {}
        self._launch_lists: dict[tuple, tuple] = {}  # step sizes -> (workspace version, K.LaunchList)
        self._replayable = ec.reuse_launch_lists and self.model.launches_replayable
        self.launch_list_replays = 0
        self._decode_layouts: dict[int, dict] = {}
        self._arange = np.arange(ec.max_num_seqs + 2, dtype=np.int32)
        self._graph_safe = self.model.graph_safe
        # int32 device tensor from which a step may take token ids that the host has not read yet
        # (an id -(r+1) in a step's tokens means row r of it); set by the engine that owns the sampler
        self._token_feedback: torch.Tensor | None = None
        self.steps_run = 0
        self.graph_launches = 0  # kernels run through graph replays so far
        self.graph_replays = 0   # steps that were graph replays
        self.h2d_bytes = 0  # bytes of step descriptors copied to the device so far

    def _bytes_beside_the_cache(self, state_specs) -> int:
        """Device memory the engine will take beside weights and pages, as far as it is known
        before the first step: per-request state rows, block tables, and the scratch buffers of
        a step of the largest size (a few activations of ``max_num_batched_tokens`` rows and the
        logits of ``max_num_seqs`` rows)."""
        ec = self.engine_config
        state = 0
        for spec in state_specs.values():
            n = ec.max_num_seqs
            for s in spec.shape:
                n *= int(s)
            state += n * torch.empty((), dtype=spec.dtype).element_size()
        width = self.spec.hidden_size
        scratch = ec.max_num_batched_tokens * width * 4 * 12 + ec.max_num_seqs * self.spec.vocab_size * 4 * 2
        return state + scratch

    @classmethod
    def from_folder(cls, model_dir: str, engine_config: EngineConfig | None = None) -> "ModelRunner":
        return cls(load_config(model_dir), read_safetensors(model_dir), engine_config, source=model_dir)

    # ---- building a step -----------------------------------------------------------
    def _validate(self, entries: list[StepEntry]) -> None:
        ec = self.engine_config
        if not entries:
            raise ValueError("a step needs at least one request")
        if len(entries) > ec.max_num_seqs:
            raise ValueError(f"{len(entries)} requests in a step; at most {ec.max_num_seqs}")
        total = sum(len(e.token_ids) for e in entries)
        if total > ec.max_num_batched_tokens:
            raise ValueError(f"{total} tokens in a step; at most {ec.max_num_batched_tokens}")
        seen = set()
        for e in entries:
            if e.slot in seen:
                raise ValueError(f"slot {e.slot} appears twice in one step")
            seen.add(e.slot)
            if not self.cache.slots.is_held(e.slot):
                raise ValueError(f"slot {e.slot} is not live")
            cached = int(self.cache.num_tokens[e.slot])
            if cached + len(e.token_ids) > self.max_model_len:
                raise ValueError(
                    f"slot {e.slot}: {cached} cached + {len(e.token_ids)} new tokens exceed the "
                    f"longest sequence {self.max_model_len}"
                )
            vocab = self.spec.vocab_size
            n_back = 0 if self.token_feedback is None else self.token_feedback.numel()
            if len(e.token_ids) > 16:  # a long portion: one conversion serves the check and the copy
                if not isinstance(e.token_ids, np.ndarray):
                    try:  # the quickest way from a list of ints to an array
                        e.token_ids = np.frombuffer(array.array("i", e.token_ids), dtype=np.int32)
                    except (OverflowError, TypeError):
                        e.token_ids = np.asarray(e.token_ids, dtype=np.int64)
                lo, hi = int(e.token_ids.min()), int(e.token_ids.max())
            else:
                lo, hi = min(e.token_ids), max(e.token_ids)
            if lo < -n_back or hi >= vocab:
                raise ValueError(f"token id {lo if lo < -n_back else hi} outside the vocabulary of {vocab}")

    def _upload(self, hb: HostBatch, caps: tuple[int, int, int, int, int, int] | None = None) -> StepContext:
        sizes = (len(hb.token_ids), len(hb.slots), len(hb.logit_rows), len(hb.decode_reqs), len(hb.tiles),
                 len(hb.tiles_wide))
        lay = _layout(*(caps or sizes))
        idx, host = self._staging.next()
        h = self._staging.arrays[idx]
        for name in ("token_ids", "positions", "req_of_token", "q_start", "kv_len", "slots",
                     "logit_rows", "decode_reqs"):
            off, _ = lay[name]
            arr = getattr(hb, name)
            h[off:off + len(arr)] = arr
        off, _ = lay["tiles"]
        h[off:off + hb.tiles.size] = hb.tiles.reshape(-1)
        off, _ = lay["tiles_wide"]
        h[off:off + hb.tiles_wide.size] = hb.tiles_wide.reshape(-1)
        total = lay["_total"][0]
        K.copy_to_device_raw(self._dev_ints.data_ptr(), self._staging.addresses[idx], total * 4)
        self.h2d_bytes += total * 4
        self._staging.mark(idx)

        n_tokens, n_reqs, n_rows, n_decode, n_tiles, n_wide = caps or sizes
        views = self._views.get(caps or sizes)
        if views is None:  # the device arrays of a step of these sizes: the same views every time
            if len(self._views) > 256:
                self._views.clear()
            views = self._views[caps or sizes] = {
                name: self._dev_ints[lay[name][0]:lay[name][0] + n]
                for name, n in (("token_ids", n_tokens), ("positions", n_tokens), ("req_of_token", n_tokens),
                                ("q_start", n_reqs + 1), ("kv_len", n_reqs), ("slots", n_reqs),
                                ("logit_rows", n_rows), ("decode_reqs", n_decode), ("tiles", 2 * n_tiles),
                                ("tiles_wide", 2 * n_wide))}
        view = lambda name, n: views[name]
        return StepContext(
            device=self.device, act_dtype=self.dtype, host=hb,
            token_ids=view("token_ids", n_tokens), positions=view("positions", n_tokens),
            req_of_token=view("req_of_token", n_tokens), q_start=view("q_start", n_reqs + 1),
            kv_len=view("kv_len", n_reqs), slots=view("slots", n_reqs),
            logit_rows=view("logit_rows", n_rows), decode_reqs=view("decode_reqs", n_decode),
            tiles=view("tiles", 2 * n_tiles), tiles_wide=view("tiles_wide", 2 * n_wide),
            n_tokens=n_tokens, n_reqs=n_reqs, n_logit_rows=n_rows, n_decode=n_decode, n_tiles=n_tiles,
            n_tiles_wide=n_wide,
            max_kv_len=int(hb.kv_len.max()), cache=self.cache, workspace=self.workspace,
            extras={"token_feedback": self.token_feedback} if self.token_feedback is not None else {},
        )

    @property
    def token_feedback(self) -> torch.Tensor | None:
        """Device int32 buffer from which a token id -(r+1) of a step is replaced by entry r
        (tokens sampled by the step before, which the host has not read yet)."""
        return self._token_feedback

    @token_feedback.setter
    def token_feedback(self, buf: torch.Tensor | None) -> None:
        if buf is not self._token_feedback:
            self._graphs.clear()  # captured kernels hold the old buffer's address
            self._launch_lists.clear()  # and so do noted launches
        self._token_feedback = buf

    # ---- the step ----------------------------------------------------------------------
    def samples_in_head(self, n_wanted: int, with_temperature: bool = False) -> bool:
        """Whether a step with this many wanted places (some sampled with a temperature, or all
        taking the arg-max) should be run with ``sample_into``: the head must take that many
        rows, and the rows of the graph bucket such a step may be replayed in."""
        if not self.model.samples_in_head(n_wanted, with_temperature):
            return False
        b = self._bucket(n_wanted) if self.engine_config.cuda_graphs and self._graph_safe else None
        return b is None or b == n_wanted or self.model.samples_in_head(b, with_temperature)

    def step(self, entries: list[StepEntry], *, reserve: bool = True,
             sample_into: "K.SampleInto | None" = None) -> torch.Tensor | None:
        """Run one batch; returns float32 logits ``[wanted places, vocab]`` in the order of
        ``entries`` and of each entry's ``want`` (``None`` when nothing is wanted).

        The returned tensor is scratch that the next step overwrites.  ``reserve``: take the
        pages the step needs here (raises ``OutOfPages``, and takes none, when they are not
        to be had); a caller that has reserved them itself passes ``False``.
        ``sample_into``: instead of logits, the next token of every wanted place, chosen by the
        head's own product with the options that lie in ``sample_into``'s device tensors when
        the step runs, into ``sample_into.out_ids`` (in the order of the wanted places); returns
        ``None``.  Only where ``samples_in_head`` says so.  Captured graphs hold the tensors'
        addresses: a caller passes the same object every time.
        """
        self._validate(entries)
        if sample_into is not None and not self.samples_in_head(sum(len(e.want) for e in entries)):
            raise ValueError("the head does not choose the tokens of this step's wanted places itself")
        if reserve:
            done = []
            for e in entries:
                if not self.cache.reserve(e.slot, len(e.token_ids)):
                    # nothing of this step has run: pages already taken for it stay with
                    # their requests (they will be needed by the same tokens later)
                    raise OutOfPages(
                        f"no pages for {len(e.token_ids)} more tokens of slot {e.slot} "
                        f"({self.cache.num_free_pages} pages free)"
                    )
                done.append(e)
        hb = build_host_batch(
            [(e.slot, int(self.cache.num_tokens[e.slot]), e.token_ids, e.want) for e in entries]
        )
        self.cache.sync_to_device()
        logits = None
        if self._graph_ok(hb):
            logits = self._replay(hb, sample_into)
        else:
            ctx = self._upload(hb)
            if sample_into is not None:
                ctx.extras["sample_into"] = sample_into
            logits = self._run(ctx)
        for e in entries:
            self.cache.commit(e.slot, len(e.token_ids))
        self.steps_run += 1
        return logits

    # ---- launch lists for the other steps ----------------------------------------------------
    LAUNCH_LISTS_KEPT = 64

    def _run(self, ctx: StepContext) -> torch.Tensor | None:
        """The model on an uploaded step.  Where every part launches through the kernel library
        and from sizes alone, the first step of some sizes notes its calls and later ones issue
        them again: most of a short step's host time is otherwise spent between the launches."""
        if not self._replayable:
            return self.model.forward(ctx)
        key = (ctx.n_tokens, ctx.n_reqs, ctx.n_logit_rows, ctx.n_decode, ctx.n_tiles, ctx.n_tiles_wide,
               self.model.launch_key(ctx), id(ctx.extras.get("sample_into")))
        have = self._launch_lists.get(key)
        if have is not None and have[0] == self.workspace.version:
            have[1].replay()
            self.launch_list_replays += 1
            return have[1].result
        version = self.workspace.version
        with K.recording() as launches:
            launches.result = self.model.forward(ctx)
        if self.workspace.version == version:  # no buffer moved while the addresses were noted
            if len(self._launch_lists) >= self.LAUNCH_LISTS_KEPT:
                self._launch_lists.pop(next(iter(self._launch_lists)))
            self._launch_lists[key] = (version, launches)
        return launches.result

    # ---- CUDA graphs for decode-only steps ------------------------------------------------
    GRAPH_BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128, 256)

    def _bucket(self, n: int) -> int | None:
        for b in self.GRAPH_BUCKETS:
            if n <= b <= self.engine_config.max_num_seqs:
                return b
        return None

    def _graph_ok(self, hb: HostBatch) -> bool:
        """Steps in which every request brings one token and wants its logits, on a model whose
        parts can all be captured, replay a graph captured for their batch-size bucket."""
        if not self.engine_config.cuda_graphs or not self._graph_safe:
            return False
        n = len(hb.slots)
        if len(hb.token_ids) != n or len(hb.logit_rows) != n or len(hb.decode_reqs) != n:
            return False
        return self._bucket(n) is not None

    def _graph_ok_for(self, n: int) -> bool:
        return self.engine_config.cuda_graphs and self._graph_safe and self._bucket(n) is not None

    def _padded(self, hb: HostBatch, b: int) -> HostBatch:
        """``hb`` filled up to ``b`` requests with rows that no kernel acts on (slot -1)."""
        n = len(hb.slots)
        if n == b:
            return hb
        pad = b - n
        z = np.zeros(pad, dtype=np.int32)
        return HostBatch(
            token_ids=np.concatenate([hb.token_ids, z]), positions=np.concatenate([hb.positions, z]),
            req_of_token=np.arange(b, dtype=np.int32), q_start=np.arange(b + 1, dtype=np.int32),
            kv_len=np.concatenate([hb.kv_len, z + 1]), slots=np.concatenate([hb.slots, z - 1]),
            logit_rows=np.arange(b, dtype=np.int32), decode_reqs=np.arange(b, dtype=np.int32),
            tiles=hb.tiles, tiles_wide=hb.tiles_wide,
        )

    def _graph_decode_plan(self, b: int):
        """How the decode attention splits keys over blocks in a graph: fixed for the bucket,
        whatever the context lengths of a replay are (splits beyond a request's keys are empty)."""
        span = self.max_model_len // 2  # a request's context is anywhere below the limit
        plans = [part.decode_plan_for(b, span, self.dtype) for l in self.model.layers for part in l.parts.values()
                 if hasattr(part, "decode_plan_for")]
        return max(plans) if plans else None

    def _stage_decode(self, hb: HostBatch, b: int) -> None:
        """The arrays of a decode-only step of ``b`` rows (``len(hb.slots)`` real, the rest
        padding with slot -1) written to a pinned buffer in the bucket's layout and copied to
        the device: what ``_upload`` does, without building views that a replay never reads."""
        n = len(hb.slots)
        lay = self._decode_layouts.get(b)
        if lay is None:
            lay = self._decode_layouts[b] = _layout(b, b, b, b, 0, 0)
        idx, host = self._staging.next()
        h = self._staging.arrays[idx]
        total = lay["_total"][0]
        for name, arr in (("token_ids", hb.token_ids), ("positions", hb.positions), ("kv_len", hb.kv_len),
                          ("slots", hb.slots)):
            off = lay[name][0]
            h[off:off + n] = arr
            if n < b:
                h[off + n:off + b] = -1 if name == "slots" else (1 if name == "kv_len" else 0)
        ident = self._arange[:b + 1]
        h[lay["req_of_token"][0]:lay["req_of_token"][0] + b] = ident[:b]
        h[lay["q_start"][0]:lay["q_start"][0] + b + 1] = ident
        h[lay["logit_rows"][0]:lay["logit_rows"][0] + b] = ident[:b]
        h[lay["decode_reqs"][0]:lay["decode_reqs"][0] + b] = ident[:b]
        K.copy_to_device_raw(self._dev_ints.data_ptr(), self._staging.addresses[idx], total * 4)
        self.h2d_bytes += total * 4
        self._staging.mark(idx)

    @staticmethod
    def _graph_key(b: int, sample_into):
        """Graphs are kept by bucket and by what their head does: logits (a bare bucket number),
        or tokens into one ``SampleInto`` (the padding rows' tokens land in its ``out_ids`` too,
        beyond the step's own rows, where nobody reads them)."""
        return b if sample_into is None else (b, id(sample_into))

    def _capture(self, b: int, padded: HostBatch, sample_into=None):
        """Capture the decode step of bucket ``b`` on the given (padded) batch."""
        caps = (b, b, b, b, 0, 0)
        ws = Workspace(self.device)  # buffers of its own: their addresses must never change
        plan = self._graph_decode_plan(b)

        def context():
            ctx = self._upload(padded, caps)
            ctx.workspace = ws
            ctx.extras["decode_plan"] = plan
            if sample_into is not None:
                ctx.extras["sample_into"] = sample_into
            return ctx

        # warm-up: sizes the workspace outside the capture.  A head that chooses tokens writes the
        # padding rows' into the caller's buffer, which in a running engine still holds the tokens
        # of the step before (the step to come may read them from there): put back afterwards
        # (and it counts as a launch in the buffer's ring of host slots, which the caller does not know of)
        kept = sample_into.out_ids.clone() if sample_into is not None else None
        kept_step = sample_into.ring_step.clone() if kept is not None and sample_into.ring_step is not None else None
        self.model.forward(context())
        if kept is not None:
            sample_into.out_ids.copy_(kept)
        if kept_step is not None:
            sample_into.ring_step.copy_(kept_step)
        torch.cuda.synchronize()
        ws.frozen = True
        graph = torch.cuda.CUDAGraph()
        before = K.launches()
        ctx = context()
        with torch.cuda.graph(graph):
            logits = self.model.forward(ctx)
        # the workspace stays with the graph: the captured kernels hold its buffers' addresses,
        # which the allocator must not hand to anyone else while the graph can be replayed
        # (and so does the SampleInto, whose identity is part of the graph's key)
        entry = self._graphs[self._graph_key(b, sample_into)] = (graph, logits, K.launches() - before, ws, sample_into)
        return entry

    def capture_graphs(self, largest: int | None = None, sample_into=None) -> int:
        """Capture the decode graphs of every bucket up to ``largest`` requests now, on batches
        of padding rows only (which no kernel acts on), so that no step of a running engine
        pays for a capture (a few milliseconds each).  With ``sample_into``: the graphs whose
        head chooses the tokens into it, where the head can (logits elsewhere).  Returns how
        many were captured."""
        if not self.engine_config.cuda_graphs or not self._graph_safe:
            return 0
        limit = self.engine_config.max_num_seqs if largest is None else min(largest, self.engine_config.max_num_seqs)
        empty = build_host_batch([])
        made = 0
        for b in self.GRAPH_BUCKETS:
            into = sample_into if sample_into is not None and self.model.samples_in_head(b) else None
            if b <= limit and self._graph_key(b, into) not in self._graphs:
                self._capture(b, self._padded(empty, b), into)
                made += 1
        return made

    def _replay(self, hb: HostBatch, sample_into=None):
        n = len(hb.slots)
        b = self._bucket(n)
        if sample_into is not None and not self.model.samples_in_head(b):
            raise ValueError(f"the head does not choose the tokens of the {b} rows of this step's graph itself")
        entry = self._graphs.get(self._graph_key(b, sample_into))
        if entry is None:
            # captured on padding rows only (no kernel acts on them), never on the step's own
            # rows: the warm-up run of a capture would otherwise run them a second time, which
            # a part with state of its own would not forgive
            entry = self._capture(b, self._padded(build_host_batch([]), b), sample_into)
        self._stage_decode(hb, b)
        graph, logits, n_kernels = entry[:3]
        graph.replay()
        self.graph_launches += n_kernels
        self.graph_replays += 1
        return logits[:n] if logits is not None else None

    def check_status(self) -> None:
        """Wait for the device and raise if a kernel flagged bad indices during earlier steps."""
        K.check_status(self.device)
