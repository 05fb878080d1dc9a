"""Choosing the next token: greedy and temperature sampling, on the device.

The reference samples greedily, ``int(logits.argmax().item())`` (mini_hisparse/engine.py:72).
Temperature sampling is added here: softmax(logits / T) in float32 and an inverse-CDF draw at a
uniform number that depends only on the request's seed and on how many tokens it has drawn, so
a request's tokens do not depend on which other requests share its batch.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..kernels import api as K


@dataclass(frozen=True)
class SamplingParams:
    max_new_tokens: int = 16
    temperature: float = 0.0
    seed: int = 0
    eos_token_id: int | None = None

    def __post_init__(self):
        if self.max_new_tokens < 1:
            raise ValueError("max_new_tokens must be positive")
        if self.temperature < 0:
            raise ValueError("temperature must not be negative")


class Sampler:
    """Per-step buffers for the sampling kernel; one row of logits per request."""

    def __init__(self, device, max_rows: int = 64):
        self.device = torch.device(device)
        self._cap = 0
        self._grow(max_rows)

    def _grow(self, n: int):
        self._cap = n
        self.temp_host = torch.empty(n, dtype=torch.float32).pin_memory()
        self.draw_host = torch.empty((2, n), dtype=torch.int64).pin_memory()   # seed, counter
        self.temp = torch.empty(n, dtype=torch.float32, device=self.device)
        self.draw = torch.empty((2, n), dtype=torch.int64, device=self.device)
        self.out = torch.empty(n, dtype=torch.int32, device=self.device)
        self.out_host = torch.empty(n, dtype=torch.int32).pin_memory()

    def sample(self, logits: torch.Tensor, temperatures, seeds, counters) -> list[int]:
        """One token per row of ``logits`` [R, V]; host lists in, host list out (one sync)."""
        self.launch(logits, temperatures, seeds, counters)
        return self.collect()

    def launch(self, logits: torch.Tensor, temperatures, seeds, counters) -> None:
        """Start the sampling kernel and the copy of its result to the host; collect() waits for them."""
        R = logits.shape[0]
        if R > self._cap:
            self._grow(max(R, 2 * self._cap))
        if all(t <= 0 for t in temperatures):
            K.sample(logits, None, None, None, self.out[:R])
        else:
            self.temp_host[:R] = torch.tensor(temperatures, dtype=torch.float32)
            self.draw_host[0, :R] = torch.tensor([s & ((1 << 63) - 1) for s in seeds], dtype=torch.int64)
            self.draw_host[1, :R] = torch.tensor(counters, dtype=torch.int64)
            self.temp.copy_(self.temp_host, non_blocking=True)
            self.draw.copy_(self.draw_host, non_blocking=True)
            K.sample(logits, self.temp, self.draw[0], self.draw[1], self.out[:R])
        self.out_host[:R].copy_(self.out[:R], non_blocking=True)
        self._rows = R

    def collect(self) -> list[int]:
        torch.cuda.current_stream().synchronize()
        return self.out_host[: self._rows].tolist()
