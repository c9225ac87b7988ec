"""Continuous batching: which requests run which tokens in the next step.

Every request in flight has some tokens not yet in the cache: a new request
its whole prompt, a decoding request the one token sampled last, a preempted
request its prompt plus what it had generated.  A step gives each scheduled
request the next ``n`` of them; when ``n`` reaches the end, the logits of the
last one are wanted and a token is sampled.  So decoding and prompt portions
are the same thing to the scheduler, and one token budget covers both:
requests that need a single token come first, then portions of at most
``prefill_chunk_size`` in order of admission, then new admissions.

The reference keeps decode and prefill apart: up to ``max_batch_size`` decode
rows, then up to ``prefill_max_batch_size`` portions of ``prefill_chunk_size``
(rosellm/roseinfer/engine.py:3822-3865, 3867-4030), no joint budget.  Prompt
rules are the reference's: an empty prompt becomes the end-of-sequence token,
``max_new_tokens`` is cut to the room left in the context, and a request
without room finishes at once (engine.py:3741-3758); a prompt longer than the
context is refused unless ``truncate_prompt`` keeps its last tokens
(engine.py:3744-3747 always truncates).

When pages run out.  The reference's allocator raises from inside the step
(rosellm/roseinfer/engine.py:4410-4417).  Here reservation is all-or-nothing
before the step: a new request is not admitted while its first portion does
not fit; when a request in flight cannot get its next page, the request
admitted last gives everything back and returns to the head of the waiting
line (it is recomputed later from prompt plus generated tokens, and its
random stream continues where it stopped); a request that could never fit in
an empty cache is refused when it is added.
"""
from __future__ import annotations

import zlib
from collections import deque
from dataclasses import dataclass, field

import numpy as np

from ..cache.manager import CacheManager, pages_for
from ..sampling.params import SamplingParams

WAITING, RUNNING, DRAINING, FINISHED = "waiting", "running", "draining", "finished"
# In an output list: a token that a launched step will sample and the host has not read yet.
PENDING = -1


@dataclass
class Request:
    request_id: int | str
    prompt_ids: list[int]
    params: SamplingParams
    seed: int
    max_new_tokens: int
    output_ids: list[int] = field(default_factory=list)
    status: str = WAITING
    finish_reason: str | None = None
    slot: int | None = None
    num_computed: int = 0
    num_preemptions: int = 0
    admitted_at: int = -1
    pending_row: int = -1   # row of the launched step's sampling batch that holds the PENDING token
    _prompt_array: "np.ndarray | None" = field(default=None, repr=False, compare=False)

    @property
    def all_ids(self) -> list[int]:
        return self.prompt_ids + self.output_ids

    def tokens(self, start: int, count: int):
        """``all_ids[start:start + count]`` without putting the two lists together: a decoded
        token is a one-element list; a long portion of the prompt is a view of the prompt as an
        int32 array (made once a request), which the step function takes as it is."""
        n_prompt = len(self.prompt_ids)
        end = start + count
        if start >= n_prompt:
            return self.output_ids[start - n_prompt:end - n_prompt]
        if end <= n_prompt:
            if count <= 16:
                return self.prompt_ids[start:end]
            if self._prompt_array is None:
                self._prompt_array = np.asarray(self.prompt_ids, dtype=np.int32)
            return self._prompt_array[start:end]
        return self.prompt_ids[start:] + self.output_ids[:end - n_prompt]

    @property
    def num_tokens(self) -> int:
        return len(self.prompt_ids) + len(self.output_ids)

    @property
    def remaining(self) -> int:
        return self.num_tokens - self.num_computed


@dataclass
class Scheduled:
    request: Request
    start: int       # first token (index into all_ids) this step computes
    count: int
    samples: bool    # the step reaches the request's last token: a new one is sampled
    out_index: int = -1  # where in output_ids the sampled token goes (set when the step is launched)


@dataclass
class StepPlan:
    items: list[Scheduled]
    preempted: list[Request]

    @property
    def num_tokens(self) -> int:
        return sum(i.count for i in self.items)


class Scheduler:
    def __init__(self, cache: CacheManager, *, max_num_seqs: int, max_num_batched_tokens: int,
                 prefill_chunk_size: int, max_model_len: int, eos_token_id: int | None = None,
                 truncate_prompt: bool = False, seed: int = 0) -> None:
        self.cache = cache
        self.seed = seed
        self.max_num_seqs = max_num_seqs
        self.max_num_batched_tokens = max_num_batched_tokens
        self.prefill_chunk_size = prefill_chunk_size
        self.max_model_len = max_model_len
        self.eos_token_id = eos_token_id
        self.truncate_prompt = truncate_prompt
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []       # in order of admission
        self.finished: list[Request] = []
        self._admissions = 0
        self._next_id = 0

    # ---- requests in ----------------------------------------------------------------
    def add_request(self, prompt_ids: list[int], params: SamplingParams,
                    request_id: int | str | None = None) -> Request:
        prompt = [int(t) for t in prompt_ids]
        eos = params.eos_token_id if params.eos_token_id is not None else self.eos_token_id
        if not prompt:
            if eos is None:
                raise ValueError("empty prompt and no end-of-sequence token to stand for it")
            prompt = [eos]
        if len(prompt) > self.max_model_len:
            if not self.truncate_prompt:
                raise ValueError(f"prompt of {len(prompt)} tokens exceeds the context of {self.max_model_len}")
            prompt = prompt[-self.max_model_len:]
        if request_id is None:
            request_id = self._next_id
        self._next_id += 1
        room = self.max_model_len - len(prompt)
        max_new = min(params.max_new_tokens, room)
        seed = params.seed if params.seed is not None else self.default_seed(request_id, len(prompt))
        req = Request(request_id, prompt, params, seed, max_new)
        if max_new <= 0:
            req.status, req.finish_reason = FINISHED, "length"
            self.finished.append(req)
            return req
        # the last generated token is never run through the model
        most = len(prompt) + max_new - 1
        if any(n > self.cache.num_pages for n in self._pages_to_hold(most)):
            raise ValueError(
                f"request of up to {most} cached tokens can never fit the cache of "
                f"{self.cache.num_pages} pages of {self.cache.page_size} tokens"
            )
        self.waiting.append(req)
        return req

    def default_seed(self, request_id: int | str, prompt_len: int) -> int:
        """The seed of a request that brings none: a checksum of the engine's seed, the
        request's id and its prompt's length, the same in every process (Python's own ``hash``
        of a string differs from run to run)."""
        text = f"{self.seed}:{type(request_id).__name__}:{request_id!r}:{prompt_len}".encode()
        return (zlib.crc32(text) | (zlib.adler32(text) << 32)) & 0x7FFF_FFFF_FFFF_FFFF

    def _pages_to_hold(self, n_tokens: int) -> list[int]:
        out = []
        for g in self.cache.groups:
            if g.spec.window is None:
                out.append(pages_for(n_tokens, self.cache.page_size))
            else:
                span = min(n_tokens, g.spec.window + self.prefill_chunk_size)
                out.append(pages_for(span, self.cache.page_size) + 1)
        return out

    def has_unfinished(self) -> bool:
        """Requests that a further step could run (those only waiting for their last token to be
        read are not among them)."""
        return bool(self.waiting or self.running)

    def abort(self, req: Request) -> None:
        if req.status == RUNNING:
            self.running.remove(req)
            self.cache.release(req.slot)
            req.slot = None
        elif req.status == WAITING:
            self.waiting.remove(req)
        req.output_ids = [t for t in req.output_ids if t != PENDING]
        req.status, req.finish_reason = FINISHED, "abort"
        self.finished.append(req)

    # ---- one step's plan ---------------------------------------------------------------
    def _preempt(self, req: Request) -> None:
        self.running.remove(req)
        self.cache.release(req.slot)
        req.slot = None
        req.num_computed = 0
        req.status = WAITING
        req.num_preemptions += 1
        self.waiting.appendleft(req)

    def schedule(self) -> StepPlan:
        budget = self.max_num_batched_tokens
        items: list[Scheduled] = []
        preempted: list[Request] = []
        # single tokens first, then portions; both in order of admission
        order = [r for r in self.running if r.remaining == 1] + [r for r in self.running if r.remaining > 1]
        scheduled: set[int] = set()
        for req in order:
            if req.status != RUNNING or budget <= 0:
                continue
            n = min(req.remaining, self.prefill_chunk_size, budget)
            while not self.cache.reserve(req.slot, n):
                victim = next((v for v in reversed(self.running) if id(v) not in scheduled), None)
                if victim is None:
                    raise RuntimeError("out of pages with nothing left to preempt")
                self._preempt(victim)
                preempted.append(victim)
                if victim is req:
                    break
            if req.status != RUNNING:
                continue
            items.append(Scheduled(req, req.num_computed, n, n == req.remaining))
            scheduled.add(id(req))
            budget -= n
        while self.waiting and budget > 0 and not preempted and len(self.running) < self.max_num_seqs:
            req = self.waiting[0]
            n = min(req.remaining, self.prefill_chunk_size, budget)
            slot = self.cache.new_request()
            if slot is None:
                break
            if not self.cache.reserve(slot, n):
                self.cache.release(slot)
                break
            self.waiting.popleft()
            req.slot, req.status = slot, RUNNING
            req.admitted_at = self._admissions
            self._admissions += 1
            self.running.append(req)
            items.append(Scheduled(req, req.num_computed, n, n == req.remaining))
            budget -= n
        if not items and self.has_unfinished():
            raise RuntimeError("nothing can be scheduled: the cache is too small for the waiting request")
        return StepPlan(items, preempted)

    # ---- after the step -------------------------------------------------------------------
    def advance(self, plan: StepPlan) -> None:
        """The step has been launched.  Its tokens count as computed, and where it samples a
        token the request's output gets a ``PENDING`` mark in its place, so that the next step
        can be planned (and launched, feeding the token from device memory) before the host has
        read this one's tokens.  A request whose pending token is the last it may generate takes
        part in no further step and gives its slot and pages back now: everything on the device
        is ordered in one stream, so whoever gets those pages next runs after this step."""
        row = 0
        for item in plan.items:
            req = item.request
            req.num_computed += item.count
            if not item.samples:
                continue
            item.out_index = len(req.output_ids)
            req.output_ids.append(PENDING)
            req.pending_row = row
            row += 1
            if len(req.output_ids) >= req.max_new_tokens:
                req.status = DRAINING
                self.running.remove(req)
                self.cache.release(req.slot)
                req.slot = None

    def resolve(self, plan: StepPlan, sampled: list[int]) -> list[Request]:
        """The host has the step's tokens (one per item with ``samples``, in order): they replace
        the marks, and requests that end (end-of-sequence token, or their last token) finish.
        A request that already finished on an earlier token ignores this one: the step that
        sampled it was launched before that token was known.  Returns the requests that finished."""
        done: list[Request] = []
        it = iter(sampled)
        for item in plan.items:
            if not item.samples:
                continue
            token = int(next(it))
            req = item.request
            if req.status == FINISHED:
                continue
            req.output_ids[item.out_index] = token
            eos = req.params.eos_token_id if req.params.eos_token_id is not None else self.eos_token_id
            if req.params.stop_on_eos and eos is not None and token == eos:
                req.finish_reason = "stop"
                del req.output_ids[item.out_index + 1:]  # a mark of a step launched meanwhile
            elif item.out_index + 1 >= req.max_new_tokens:
                req.finish_reason = "length"
            if req.finish_reason is not None:
                if req.status == RUNNING:
                    self.running.remove(req)
                    self.cache.release(req.slot)
                    req.slot = None
                elif req.status == WAITING:  # preempted while its last step was in flight
                    self.waiting.remove(req)
                req.status = FINISHED
                self.finished.append(req)
                done.append(req)
        return done

    def update(self, plan: StepPlan, sampled: list[int]) -> list[Request]:
        """``advance`` and ``resolve`` in one: for steps whose tokens are read before the next
        step is planned."""
        self.advance(plan)
        return self.resolve(plan, sampled)
