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


class _Slot:
    """The buffers of one launch: two slots take turns, so that a step's tokens can still be on their
    way to the host while the next step's sampling is queued behind it."""

    def __init__(self, n: int, device):
        self.temp_host = torch.empty(n, dtype=torch.float32).pin_memory()
        self.draw_host = torch.empty((2, n), dtype=torch.int64).pin_memory()   # seed, counter
        self.temp = torch.empty(n, dtype=torch.float32, device=device)
        self.draw = torch.empty((2, n), dtype=torch.int64, device=device)
        self.out = torch.empty(n, dtype=torch.int32, device=device)
        self.out_host = torch.empty(n, dtype=torch.int32).pin_memory()
        self.done = torch.cuda.Event()
        self.rows = 0
        self.busy = False


class Sampler:
    """Per-step buffers for the sampling kernel; one row of logits per request."""

    def __init__(self, device, max_rows: int = 64):
        self.device = torch.device(device)
        self._cap = max_rows
        self._slots = [_Slot(max_rows, self.device), _Slot(max_rows, self.device)]
        self._turn = 0
        self._last = None

    def sample(self, logits: torch.Tensor, temperatures, seeds, counters) -> list[int]:
        """One token per row of ``logits`` [R, V]; host lists in, host list out (one sync)."""
        return self.collect(self.launch(logits, temperatures, seeds, counters))

    def launch(self, logits: torch.Tensor, temperatures, seeds, counters) -> int:
        """Start the sampling kernel and the copy of its result to the host; returns the ticket that
        collect() and device_tokens() take.  At most two launches may be uncollected."""
        R = logits.shape[0]
        ticket = self._turn
        slot = self._slots[ticket]
        if slot.busy:
            raise RuntimeError("the sampler has two launches in flight already: collect one first")
        if R > self._cap:
            if any(sl.busy for sl in self._slots):
                raise RuntimeError("the sampler cannot grow while a launch is in flight")
            self._cap = max(R, 2 * self._cap)
            self._slots = [_Slot(self._cap, self.device), _Slot(self._cap, self.device)]
            slot = self._slots[ticket]
        self._turn ^= 1
        if all(t <= 0 for t in temperatures):
            K.sample(logits, None, None, None, slot.out[:R])
        else:
            slot.temp_host[:R] = torch.tensor(temperatures, dtype=torch.float32)
            slot.draw_host[0, :R] = torch.tensor([s & ((1 << 63) - 1) for s in seeds], dtype=torch.int64)
            slot.draw_host[1, :R] = torch.tensor(counters, dtype=torch.int64)
            slot.temp.copy_(slot.temp_host, non_blocking=True)
            slot.draw.copy_(slot.draw_host, non_blocking=True)
            K.sample(logits, slot.temp, slot.draw[0], slot.draw[1], slot.out[:R])
        slot.out_host[:R].copy_(slot.out[:R], non_blocking=True)
        slot.done.record()
        slot.rows, slot.busy = R, True
        self._last = ticket
        return ticket

    def reset(self) -> None:
        """Forget launches that will not be collected (their step raised)."""
        torch.cuda.current_stream().synchronize()
        for slot in self._slots:
            slot.busy = False

    def device_tokens(self, ticket: int) -> torch.Tensor:
        """The launch's tokens on the device (int32 [rows]): what a next step that is queued behind it
        can take as its input without waiting for the host."""
        slot = self._slots[ticket]
        return slot.out[: slot.rows]

    def collect(self, ticket: int | None = None) -> list[int]:
        """Wait for a launch's tokens (the last one's if no ticket is given)."""
        slot = self._slots[self._last if ticket is None else ticket]
        slot.done.synchronize()
        slot.busy = False
        return slot.out_host[: slot.rows].tolist()
