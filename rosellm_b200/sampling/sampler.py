"""Chooses the next token of each request from the step's logits, on the device."""
from __future__ import annotations

import numpy as np
import torch

from ..ops import kernels as K
from .params import SamplingParams


class Sampler:
    """Packs the rows' sampling options into one pinned buffer, copies it once and runs
    the sampling kernel (csrc/sampling.cu).  Rows of greedy requests take the arg-max.
    Where the model's head chooses the tokens in its own product (no logits are written:
    ``before_step`` / ``after_step``), only the options' copy and the tokens' copy are left."""

    def __init__(self, device: torch.device, max_rows: int) -> None:
        self.device = device
        self.max_rows = max_rows
        # per row: temperature f32, top_p f32, top_k i32, counter i32, seed i64 (two words)
        # two of each host buffer, used in turn: a step may be launched while the one before it
        # has not been read yet
        self._hosts = [torch.zeros(6 * max_rows, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self._backs = [torch.zeros(max_rows, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self._events: list[torch.cuda.Event | None] = [None, None]
        self._turn = 0
        self._dev = torch.zeros(6 * max_rows, dtype=torch.int32, device=device)
        self._out = torch.zeros(max_rows, dtype=torch.int32, device=device)
        self._dev_all_greedy = True  # the temperatures on the device are all zero
        self._target: K.SampleInto | None = None
        # where a head that chooses the tokens itself also writes them for the host (no copy):
        # SAMPLE_RING slots, the slot of a step being its number among such steps
        self._ring = torch.zeros(K.SAMPLE_RING, max_rows, dtype=torch.int32, pin_memory=True)
        self._ring_step = torch.zeros(1, dtype=torch.int32, device=device)
        self._ring_steps = 0  # what the device's counter reads once everything launched has run
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    def _stage(self, params: list[SamplingParams], seeds: list[int], counters: list[int]) -> None:
        """The rows' options into the pinned buffer whose turn it is, and from there to the device."""
        n, m = len(params), self.max_rows
        host = self._hosts[self._turn]
        if self._events[self._turn] is not None:
            self._events[self._turn].synchronize()  # its last copy to the device is done
        h = host.numpy()
        hf = h.view(np.float32)
        hf[0:n] = [0.0 if p.greedy else p.temperature for p in params]
        hf[m:m + n] = [p.top_p for p in params]
        h[2 * m:2 * m + n] = [p.top_k for p in params]
        h[3 * m:3 * m + n] = counters
        h[4 * m:4 * m + 2 * n].view(np.int64)[:] = [s & 0x7FFF_FFFF_FFFF_FFFF for s in seeds]
        self._dev.copy_(host, non_blocking=True)
        self.h2d_bytes += host.numel() * 4
        self._dev_all_greedy = False

    def _collect(self, n: int) -> "PendingTokens":
        """Starts the copy of the first ``n`` tokens to the host."""
        back = self._backs[self._turn]
        back[:n].copy_(self._out[:n], non_blocking=True)
        event = self._events[self._turn]
        if event is None:
            event = self._events[self._turn] = torch.cuda.Event()
        event.record()
        self._turn ^= 1
        self.d2h_bytes += n * 4
        return PendingTokens(back, n, event)

    @staticmethod
    def needs_logits(params: list[SamplingParams]) -> bool:
        """Whether some row has top-k or top-p switched on: such a row is chosen from its whole
        row of logits, which a head that chooses tokens itself never writes."""
        return any(not p.greedy and (p.top_k > 0 or 0.0 < p.top_p < 1.0) for p in params)

    def launch(self, logits: torch.Tensor, params: list[SamplingParams], seeds: list[int],
               counters: list[int]) -> "PendingTokens":
        """Starts sampling one token per row and the copy of the tokens to the host; returns a
        handle whose ``tokens()`` waits for them.  ``counters[i]`` is how many tokens request i
        has generated.  The tokens also stay in ``self.device_tokens`` (row i: request i) until
        the next launch, for a step that is launched before the host has read them."""
        n = len(params)
        if n > self.max_rows or logits.shape[0] < n:
            raise ValueError("more rows to sample than logits or than the sampler was made for")
        m = self.max_rows
        out = self._out[:n]
        if all(p.greedy for p in params):
            K.sample(logits[:n], None, None, None, None, None, out)
        else:
            self._stage(params, seeds, counters)
            d = self._dev
            K.sample(logits[:n], d[0:m].view(torch.float32), d[2 * m:3 * m], d[m:2 * m].view(torch.float32),
                     d[4 * m:6 * m].view(torch.int64), d[3 * m:4 * m], out, filtered=self.needs_logits(params))
        return self._collect(n)

    # ---- a step whose head chooses the tokens itself ---------------------------------------
    @property
    def target(self) -> K.SampleInto:
        """Where such a step reads its rows' options and writes its tokens: this sampler's own
        device buffers, the same object every time (captured graphs hold the addresses)."""
        if self._target is None:
            m, d = self.max_rows, self._dev
            ring = self._ring if K.host_memory_on_device(self._ring) else None
            self._target = K.SampleInto(self._out, d[0:m].view(torch.float32), d[4 * m:6 * m].view(torch.int64),
                                        d[3 * m:4 * m], host_ring=ring, ring_step=self._ring_step if ring is not None else None)
        return self._target

    def before_step(self, params: list[SamplingParams], seeds: list[int], counters: list[int]) -> None:
        """Puts the rows' options where the step's head will read them (before the step is
        launched).  Greedy batches copy nothing while the temperatures on the device are zero."""
        if len(params) > self.max_rows:
            raise ValueError("more rows to sample than the sampler was made for")
        if self.needs_logits(params):
            raise ValueError("rows with top-k or top-p are sampled from their logits")
        if all(p.greedy for p in params):
            if not self._dev_all_greedy:
                self._dev[0:self.max_rows].zero_()
                self._dev_all_greedy = True
            return
        self._stage(params, seeds, counters)

    def after_step(self, n: int) -> "PendingTokens":
        """The step has been launched.  Its ``n`` tokens reach the host in the ring slot of its
        number, written by the kernel that chose them (an event after the step says when; a slot
        is written again four such steps later, and a step is launched at most one ahead of the
        one being read); without a ring, by a copy as after the sampling kernel."""
        if self.target.host_ring is None:
            return self._collect(n)
        slot = self._ring_steps % K.SAMPLE_RING
        self._ring_steps += 1
        event = self._events[self._turn]
        if event is None:
            event = self._events[self._turn] = torch.cuda.Event()
        event.record()
        self._turn ^= 1
        self.d2h_bytes += n * 4
        return PendingTokens(self._ring[slot], n, event)

    def sample(self, logits: torch.Tensor, params: list[SamplingParams], seeds: list[int],
               counters: list[int]) -> list[int]:
        """One token id per row, read back at once."""
        return self.launch(logits, params, seeds, counters).tokens()

    @property
    def device_tokens(self) -> torch.Tensor:
        return self._out


class PendingTokens:
    """Tokens on their way to the host."""

    def __init__(self, buffer: torch.Tensor, n: int, event: torch.cuda.Event) -> None:
        self._buffer, self._n, self._event = buffer, n, event

    def tokens(self) -> list[int]:
        self._event.synchronize()
        return self._buffer[: self._n].tolist()
