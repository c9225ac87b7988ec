"""Per-request sampling options.

Names and meanings follow the reference's ``generate`` keyword arguments and
command-line options (rosellm/roseinfer/engine.py:1187-1196,
rosellm/roseinfer/cli_generate.py:63-104): ``max_new_tokens``,
``temperature``, ``top_k`` (0: off), ``top_p`` (1.0: off), ``do_sample``
(off: greedy, whatever the temperature), ``stop_on_eos``.  ``seed`` is added:
the reference draws from one process-wide generator
(rosellm/roseinfer/engine.py:363-374, 1154), here each request has its own
stream of random numbers.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class SamplingParams:
    max_new_tokens: int = 64
    temperature: float = 1.0
    top_k: int = 0
    top_p: float = 1.0
    do_sample: bool = False
    stop_on_eos: bool = True
    eos_token_id: int | None = None
    seed: int | None = None

    def __post_init__(self) -> None:
        if self.max_new_tokens < 1:
            raise ValueError("max_new_tokens must be at least 1")
        if self.top_k < 0:
            raise ValueError("top_k must be non-negative (0 turns it off)")
        if self.temperature < 0 or self.top_p < 0:
            raise ValueError("temperature and top_p must be non-negative")

    @property
    def greedy(self) -> bool:
        """The reference takes the arg-max unless asked to sample at a positive temperature
        (rosellm/roseinfer/engine.py:1117-1118)."""
        return (not self.do_sample) or self.temperature <= 0.0
