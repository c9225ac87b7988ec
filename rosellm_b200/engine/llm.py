"""The Python entry point: ``InferenceEngine`` and the batch-oriented ``LLM``.

``InferenceEngine`` keeps the reference's names: ``generate``,
``generate_batch`` and ``stream_generate`` with the keyword arguments
``max_new_tokens, temperature, top_k, top_p, stop_on_eos, do_sample``
(rosellm/roseinfer/engine.py:1187-1196, 1268-1277, 1374-1383), and the
scheduler face ``add_request`` / ``step`` / ``has_unfinished`` /
``pop_finished_ids`` / ``get_generated_ids`` / ``pop_response``
(rosellm/roseinfer/engine.py:2865-3528).  Unlike the reference, whose
``generate`` runs a dense cache outside its schedulers, every call here goes
through the one scheduler, step function and paged cache.  Prompts may be
text (a tokenizer must then be found in the model folder) or token ids.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Iterator

from ..config.base import ModelConfig
from ..config.engine import EngineConfig
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from .runner import ModelRunner, StepEntry
from .scheduler import FINISHED, PENDING, Request, Scheduler


@dataclass
class RequestOutput:
    request_id: int | str
    prompt_token_ids: list[int]
    token_ids: list[int]
    finish_reason: str | None
    text: str | None = None
    num_preemptions: int = 0


def load_tokenizer(path_or_name: str | None):
    """A Hugging Face tokenizer from local files, as the reference's ``build_tokenizer``
    takes one by name (rosellm/rosetrainer/dataset.py:14-26); ``None`` when there is none."""
    if not path_or_name or not os.path.isdir(path_or_name):
        return None
    names = ("tokenizer.json", "vocab.json", "tokenizer.model", "tokenizer_config.json")
    if not any(os.path.isfile(os.path.join(path_or_name, n)) for n in names):
        return None
    from transformers import AutoTokenizer

    return AutoTokenizer.from_pretrained(path_or_name, local_files_only=True)


class InferenceEngine:
    def __init__(
        self,
        model_path: str | None = None,
        *,
        config: ModelConfig | None = None,
        seed: int = 0,
        tokenizer=None,
        tokenizer_name: str | None = None,
        device: str = "cuda",
        use_amp: bool = True,
        bf16: bool = True,
        dtype: str | None = None,
        kv_cache_max_tokens: int | None = None,
        kv_cache_mem_fraction: float | None = None,
        gpu_memory_utilization: float | None = None,
        num_pages: int | None = None,
        sampling_seed: int = 0,
        max_batch_size: int = 64,
        max_num_batched_tokens: int = 2048,
        prefill_chunk_size: int = 512,
        max_position_embeddings: int | None = None,
        page_size: int = 16,
        cuda_graphs: bool = True,
        capture_graphs_at_start: bool = True,
        truncate_prompt: bool = False,
        random_weights_std: float = 0.02,
        overlap_schedule: bool = True,
        sample_in_head: bool = True,
    ) -> None:
        """``model_path``: a folder with config.json and model.safetensors.  Without it,
        ``config`` and ``seed`` give a model with random weights.  ``use_amp=False`` selects
        the 32-bit path (the reference's ``--no-amp``); otherwise bfloat16 (``bf16`` is kept
        for the reference's signature; there is no float16 path).  ``dtype`` overrides both.
        ``overlap_schedule`` (the reference's ``OnlineScheduler(overlap_schedule=...)``,
        rosellm/roseinfer/engine.py:2865-2910): a step is launched before the host has read the
        tokens of the step before it, which it takes from device memory; ``step`` then returns
        tokens one call late.  The generated tokens are the same either way.
        The cache's size is given by one of ``kv_cache_max_tokens``, ``kv_cache_mem_fraction``,
        ``gpu_memory_utilization`` (the reference's three, rosellm/roseinfer/engine.py:96-98, 111)
        or ``num_pages``; by none, it holds ``max_batch_size`` whole contexts.  ``sample_in_head``:
        steps whose rows are greedy or sampled by temperature alone get their tokens chosen in
        the epilogue of the head's own product, where that product has such an epilogue (up to 16
        rows; more rows of a wide vocabulary when all of them take the arg-max), instead of
        logits written and read back by a sampling kernel (the same tokens).  ``sampling_seed``:
        base of the random streams of requests without a seed of their own (the reference seeds
        one engine-wide generator from ``ROSEINFER_SAMPLING_SEED``, engine.py:363-374).
        """
        if dtype is None:
            dtype = "bfloat16" if use_amp else "float32"
        if device == "cuda":
            device = "cuda:0"
        ec = EngineConfig(
            dtype=dtype, page_size=page_size, kv_cache_tokens=kv_cache_max_tokens,
            kv_cache_mem_fraction=kv_cache_mem_fraction, gpu_memory_utilization=gpu_memory_utilization,
            num_pages=num_pages, seed=sampling_seed,
            max_num_seqs=max_batch_size, max_num_batched_tokens=max_num_batched_tokens,
            prefill_chunk_size=prefill_chunk_size, max_model_len=max_position_embeddings,
            cuda_graphs=cuda_graphs, capture_graphs_at_start=capture_graphs_at_start, device=device,
        )
        if model_path is not None:
            self.runner = ModelRunner.from_folder(model_path, ec)
        elif config is not None:
            from ..config.base import resolve_architecture
            from ..models.model import named_params_of_spec
            from ..weights.random_init import random_tensors

            spec = resolve_architecture(config.to_dict()).build_spec(config)
            tensors = random_tensors(named_params_of_spec(spec), seed, std=random_weights_std)
            self.runner = ModelRunner(config, tensors, ec, source=f"<random weights, seed {seed}>")
        else:
            raise ValueError("give model_path, or config (and seed) for random weights")
        self.config = self.runner.config
        self.engine_config = ec
        self.device = self.runner.device
        self.use_amp = dtype == "bfloat16"
        self.tokenizer = tokenizer if tokenizer is not None else load_tokenizer(tokenizer_name or model_path)
        eos = self.runner.spec.eos_token_id
        if eos is None and self.tokenizer is not None:
            eos = getattr(self.tokenizer, "eos_token_id", None)
        self.eos_token_id = eos
        self.scheduler = Scheduler(
            self.runner.cache, max_num_seqs=ec.max_num_seqs, max_num_batched_tokens=ec.max_num_batched_tokens,
            prefill_chunk_size=ec.prefill_chunk_size, max_model_len=self.runner.max_model_len,
            eos_token_id=eos, truncate_prompt=truncate_prompt, seed=ec.seed,
        )
        self.sampler = Sampler(self.device, ec.max_num_seqs)
        self.overlap_schedule = overlap_schedule
        if overlap_schedule:
            self.runner.token_feedback = self.sampler.device_tokens
        self.sample_in_head = sample_in_head
        if ec.cuda_graphs and ec.capture_graphs_at_start:
            # after the feedback buffer is known: the graphs hold its address
            self.runner.capture_graphs(sample_into=self.sampler.target if sample_in_head else None)
        self._inflight = None  # (plan, requests that sample, PendingTokens) of the step not yet read
        self._requests: dict[int | str, Request] = {}
        self._finished_ids: list[int | str] = []
        self.num_steps = 0
        self.num_preemptions = 0
        self._since_status_check = 0

    # ---- text <-> ids ---------------------------------------------------------------------
    def encode(self, prompt: str) -> list[int]:
        if self.tokenizer is None:
            raise ValueError("a text prompt needs a tokenizer, and the model folder has none; pass token ids")
        return list(self.tokenizer.encode(prompt))

    def decode(self, ids: list[int]) -> str:
        if self.tokenizer is None:
            raise ValueError("decoding to text needs a tokenizer; the model folder has none")
        return self.tokenizer.decode(ids)

    # ---- the scheduler's face ------------------------------------------------------------
    def add_request(self, prompt: str | None = None, *, prompt_token_ids: list[int] | None = None,
                    max_new_tokens: int = 64, temperature: float = 1.0, top_k: int = 0, top_p: float = 1.0,
                    stop_on_eos: bool = True, do_sample: bool = False, seed: int | None = None,
                    request_id: int | str | None = None,
                    sampling_params: SamplingParams | None = None) -> int | str:
        ids = prompt_token_ids if prompt_token_ids is not None else self.encode(prompt or "")
        params = sampling_params or SamplingParams(
            max_new_tokens=max_new_tokens, temperature=temperature, top_k=top_k, top_p=top_p,
            do_sample=do_sample, stop_on_eos=stop_on_eos, seed=seed,
        )
        req = self.scheduler.add_request(ids, params, request_id)
        self._requests[req.request_id] = req
        if req.status == FINISHED:
            self._finished_ids.append(req.request_id)
        return req.request_id

    def has_unfinished(self) -> bool:
        return self.scheduler.has_unfinished() or self._inflight is not None

    def _launch(self, plan):
        """Enqueue the plan's step and its sampling; returns (requests that sample, token handle)."""
        entries = []
        for item in plan.items:
            r = item.request
            ids = r.tokens(item.start, item.count)
            if ids[-1] == PENDING:  # sampled by the step still in flight: row of its sampling batch
                ids[-1] = -(r.pending_row + 1)  # (a copy of the output's tail: prompts hold no such mark)
            entries.append(StepEntry(r.slot, ids, [item.count - 1] if item.samples else []))
        sampling = [i.request for i in plan.items if i.samples]
        params = [r.params for r in sampling]
        handle = None
        if (sampling and self.sample_in_head and not self.sampler.needs_logits(params)
                and self.runner.samples_in_head(len(sampling), any(not p.greedy for p in params))):
            # the head's product chooses the tokens itself: no logits, no sampling kernel
            self.sampler.before_step(params, [r.seed for r in sampling], [len(r.output_ids) for r in sampling])
            self.runner.step(entries, reserve=False, sample_into=self.sampler.target)
            handle = self.sampler.after_step(len(sampling))
        else:
            logits = self.runner.step(entries, reserve=False)
            if sampling:
                handle = self.sampler.launch(logits, params, [r.seed for r in sampling],
                                             [len(r.output_ids) for r in sampling])
        self.num_steps += 1
        return sampling, handle

    def _resolve(self, inflight) -> dict[int | str, int]:
        plan, sampling, handle = inflight
        tokens = handle.tokens() if handle is not None else []
        before = {id(r): r.status for r in sampling}
        done = self.scheduler.resolve(plan, tokens)
        self._finished_ids.extend(r.request_id for r in done)
        # a request that had finished before this token arrived does not report it
        return {r.request_id: t for r, t in zip(sampling, tokens) if before[id(r)] != FINISHED}

    STATUS_CHECK_EVERY = 256  # steps between two looks at the kernels' status word while requests keep coming

    def step(self) -> dict[int | str, int]:
        """One step of continuous batching; returns the token sampled for each request that got
        one.  With ``overlap_schedule`` the tokens are those of the step launched by the call
        before: this call launches the next step first and reads them while it runs.

        The kernels' status word (a bad token, position or page; a wait that gave up) is read
        when the last request has finished, and every ``STATUS_CHECK_EVERY`` steps of an engine
        that never runs dry: a raised ``KernelError`` means that tokens since the last check
        may be wrong."""
        out = self._step()
        self._since_status_check += 1
        if not self.has_unfinished() or self._since_status_check >= self.STATUS_CHECK_EVERY:
            self._since_status_check = 0
            self.runner.check_status()
        return out

    def _step(self) -> dict[int | str, int]:
        if not self.overlap_schedule:
            plan = self.scheduler.schedule()
            self.num_preemptions += len(plan.preempted)
            sampling, handle = self._launch(plan)
            self.scheduler.advance(plan)
            return self._resolve((plan, sampling, handle))
        launched = None
        if self.scheduler.has_unfinished():
            plan = self.scheduler.schedule()
            self.num_preemptions += len(plan.preempted)
            if plan.items:
                sampling, handle = self._launch(plan)
                self.scheduler.advance(plan)
                launched = (plan, sampling, handle)
        out = self._resolve(self._inflight) if self._inflight is not None else {}
        self._inflight = launched
        return out

    def pop_finished_ids(self) -> list[int | str]:
        out, self._finished_ids = self._finished_ids, []
        return out

    def get_generated_ids(self, request_id) -> list[int]:
        """The tokens generated so far that the host has read."""
        return [t for t in self._requests[request_id].output_ids if t != PENDING]

    def pop_response(self, request_id) -> RequestOutput:
        req = self._requests.pop(request_id)
        text = self.decode(req.output_ids) if self.tokenizer is not None else None
        return RequestOutput(req.request_id, list(req.prompt_ids), list(req.output_ids), req.finish_reason,
                             text, req.num_preemptions)

    def discard_request(self, request_id) -> None:
        req = self._requests.pop(request_id, None)
        if req is not None and req.status != FINISHED:
            self.scheduler.abort(req)

    # ---- the reference's generate family ----------------------------------------------------
    def generate_batch(self, prompts, max_new_tokens: int = 64, temperature: float = 1.0, top_k: int = 0,
                       top_p: float = 1.0, stop_on_eos: bool = True, do_sample: bool = False,
                       seed: int | None = None) -> list:
        """Text prompts give texts, token-id prompts give lists of generated ids."""
        rids = []
        for i, p in enumerate(prompts):
            kw = dict(max_new_tokens=max_new_tokens, temperature=temperature, top_k=top_k, top_p=top_p,
                      stop_on_eos=stop_on_eos, do_sample=do_sample,
                      seed=None if seed is None else seed + i)
            rids.append(self.add_request(p, **kw) if isinstance(p, str) else self.add_request(prompt_token_ids=p, **kw))
        while self.has_unfinished():
            self.step()  # the last step reads the kernels' status word
        self.pop_finished_ids()
        outs = [self.pop_response(r) for r in rids]
        return [o.text if isinstance(p, str) else o.token_ids for p, o in zip(prompts, outs)]

    def generate(self, prompt, max_new_tokens: int = 64, temperature: float = 1.0, top_k: int = 0,
                 top_p: float = 1.0, stop_on_eos: bool = True, do_sample: bool = False,
                 seed: int | None = None):
        return self.generate_batch([prompt], max_new_tokens, temperature, top_k, top_p, stop_on_eos,
                                   do_sample, seed)[0]

    def stream_generate(self, prompt, max_new_tokens: int = 64, temperature: float = 1.0, top_k: int = 0,
                        top_p: float = 1.0, stop_on_eos: bool = True, do_sample: bool = False,
                        seed: int | None = None) -> Iterator:
        """Yields pieces of text (token ids for a token-id prompt) as they are generated."""
        kw = dict(max_new_tokens=max_new_tokens, temperature=temperature, top_k=top_k, top_p=top_p,
                  stop_on_eos=stop_on_eos, do_sample=do_sample, seed=seed)
        as_text = isinstance(prompt, str)
        rid = self.add_request(prompt, **kw) if as_text else self.add_request(prompt_token_ids=prompt, **kw)
        shown = ""
        while self.has_unfinished():
            got = self.step()
            if rid not in got:
                continue
            if not as_text:
                yield got[rid]
                continue
            eos = self.eos_token_id
            ids = [t for t in self.get_generated_ids(rid) if not (stop_on_eos and t == eos)]
            text = self.decode(ids)
            if text.endswith("�"):  # half of a multi-byte character: wait for the rest
                continue
            if len(text) > len(shown):
                yield text[len(shown):]
                shown = text
        self.pop_finished_ids()
        self._requests.pop(rid, None)


class LLM:
    """Batch generation over token ids or text: ``LLM(model).generate(prompts, SamplingParams(...))``."""

    def __init__(self, model: str | None = None, *, dtype: str = "bfloat16", **engine_options) -> None:
        self.engine = InferenceEngine(model, dtype=dtype, **engine_options)

    def generate(self, prompts, sampling_params: SamplingParams | list[SamplingParams] | None = None
                 ) -> list[RequestOutput]:
        if isinstance(prompts, str) or (prompts and isinstance(prompts[0], int)):
            prompts = [prompts]
        sp = sampling_params or SamplingParams()
        sps = sp if isinstance(sp, list) else [sp] * len(prompts)
        rids = []
        for p, s in zip(prompts, sps):
            if isinstance(p, str):
                rids.append(self.engine.add_request(p, sampling_params=s))
            else:
                rids.append(self.engine.add_request(prompt_token_ids=list(p), sampling_params=s))
        while self.engine.has_unfinished():
            self.engine.step()  # the last step reads the kernels' status word
        self.engine.pop_finished_ids()
        return [self.engine.pop_response(r) for r in rids]
