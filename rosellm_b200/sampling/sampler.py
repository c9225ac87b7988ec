"""Chooses the next token of each request from the step's logits, on the device."""
from __future__ import annotations

import numpy as np
import torch

from ..ops import kernels as K
from .params import SamplingParams


class Sampler:
    """Packs the rows' sampling options into one pinned buffer, copies it once and runs
    the sampling kernel (csrc/sampling.cu).  Rows of greedy requests take the arg-max."""

    def __init__(self, device: torch.device, max_rows: int) -> None:
        self.device = device
        self.max_rows = max_rows
        # per row: temperature f32, top_p f32, top_k i32, counter i32, seed i64 (two words)
        self._host = torch.zeros(6 * max_rows, dtype=torch.int32, pin_memory=True)
        self._dev = torch.zeros(6 * max_rows, dtype=torch.int32, device=device)
        self._out = torch.zeros(max_rows, dtype=torch.int32, device=device)
        self._out_host = torch.zeros(max_rows, dtype=torch.int32, pin_memory=True)
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    def sample(self, logits: torch.Tensor, params: list[SamplingParams], seeds: list[int],
               counters: list[int]) -> list[int]:
        """One token id per row.  ``counters[i]`` is how many tokens request i has generated."""
        n = len(params)
        if n > self.max_rows or logits.shape[0] < n:
            raise ValueError("more rows to sample than logits or than the sampler was made for")
        m = self.max_rows
        out = self._out[:n]
        if all(p.greedy for p in params):
            K.sample(logits[:n], None, None, None, None, None, out)
        else:
            h = self._host.numpy()
            hf = h.view(np.float32)
            hf[0:n] = [0.0 if p.greedy else p.temperature for p in params]
            hf[m:m + n] = [p.top_p for p in params]
            h[2 * m:2 * m + n] = [p.top_k for p in params]
            h[3 * m:3 * m + n] = counters
            h[4 * m:4 * m + 2 * n].view(np.int64)[:] = [s & 0x7FFF_FFFF_FFFF_FFFF for s in seeds]
            self._dev.copy_(self._host, non_blocking=True)
            self.h2d_bytes += self._host.numel() * 4
            d = self._dev
            K.sample(logits[:n], d[0:m].view(torch.float32), d[2 * m:3 * m], d[m:2 * m].view(torch.float32),
                     d[4 * m:6 * m].view(torch.int64), d[3 * m:4 * m], out)
        self._out_host[:n].copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        self.d2h_bytes += n * 4
        return self._out_host[:n].tolist()
