"""Runs steps and samples their logits on the device: the backend of the generation loop.

Two ways to take a step.  ``step_and_sample`` runs it and returns the sampled ids.  ``launch`` only queues the
step and its sampling and returns a handle; ``result`` waits for the handle's ids.  A step that is launched
with ``feed=(handle, rows)`` takes its tokens from the ids the handle's step has sampled, on the device, so it
can be queued before anyone has read them: the loop reads the ids of step k while the GPU already runs step
k + 1, and the time the host needs to prepare and launch a step is hidden behind the step before it.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch

from .. import kernels
from .params import SamplerParams
from .rng import request_seed


@dataclass
class Launched:
    """A step that has been queued: where its sampled ids will be, on the device and on the host."""
    ids: torch.Tensor          # int32 [rows] on the device
    host: torch.Tensor         # pinned int32 [rows]
    event: "torch.cuda.Event"  # recorded after the copy to ``host``
    rows: int


class DeviceSampler:
    """``alloc_slot``/``free_slot``/``step_and_sample``/``check`` for
    :func:`ziglm_b200.engine.generate.run_generation`.

    The error words of the kernels' bounded waits are read every ``CHECK_EVERY`` steps and when the loop asks
    (at the end of every batch); a non-zero word ends the generation with a ``KernelError``."""
    CHECK_EVERY = 16

    def __init__(self, engine):
        self.engine = engine
        self._steps = 0
        self.device = engine.device
        self._out = torch.empty(1024, dtype=torch.int32, device=self.device)
        self._out_host = torch.empty(1024, dtype=torch.int32).pin_memory()
        self._ring: List[Optional[Launched]] = [None, None, None]     # buffers of launched steps, used in turn
        self._turn = 0
        self._feed: Optional[torch.Tensor] = None
        kernels.require(("sampling",))

    def alloc_slot(self) -> int:
        return self.engine.alloc_slot()

    def free_slot(self, slot: int) -> None:
        self.engine.free_slot(slot)

    def sample_logits(self, logits: torch.Tensor, requests: Sequence[int], histories: Sequence[Sequence[int]],
                      counters: Sequence[int], params: SamplerParams) -> List[int]:
        rows = logits.shape[0]
        if self._out.numel() < rows:
            self._out = torch.empty(rows, dtype=torch.int32, device=self.device)
            self._out_host = torch.empty(rows, dtype=torch.int32).pin_memory()
        out = self._out[:rows]
        self._sample_into(out, logits, requests, histories, counters, params)
        host = self._out_host[:rows]
        host.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return host.tolist()

    def _sample_into(self, out: torch.Tensor, logits: torch.Tensor, requests: Sequence[int],
                     histories: Sequence[Sequence[int]], counters: Sequence[int], params: SamplerParams) -> None:
        if params.is_greedy():
            kernels.argmax(logits, out)
        else:
            rng = torch.tensor([[request_seed(params.seed, r), c] for r, c in zip(requests, counters)],
                               dtype=torch.int64).pin_memory().to(self.device, non_blocking=True)
            history = None
            if params.has_penalties() and params.repetition_penalty_window > 0:
                w = params.repetition_penalty_window
                rows_h = [([-1] * w + list(h))[-w:] for h in histories]
                history = torch.tensor(rows_h, dtype=torch.int32).pin_memory().to(self.device, non_blocking=True)
            kernels.sample(logits, out, rng, params.temperature, params.top_k, params.top_p, params.min_p,
                           params.repetition_penalty, params.presence_penalty, history)

    # ------------------------------------------------------------ steps that are queued and read later
    @staticmethod
    def can_run_ahead(params: SamplerParams) -> bool:
        """Whether a step may be launched before the ids of the step before are on the host: the penalties
        need every sequence's last ids on the host."""
        return params.is_greedy() or not params.has_penalties()

    def launch(self, entries: Sequence[Tuple[int, Sequence[int]]], requests: Sequence[int],
               histories: Sequence[Sequence[int]], counters: Sequence[int], params: SamplerParams,
               feed: Optional[Tuple[Launched, Sequence[int]]] = None) -> Launched:
        """Queue a step and its sampling.  ``feed`` = (a launched step, rows): entry j takes the id that row
        ``rows[j]`` of that step sampled (the ids in ``entries`` are then place holders)."""
        rows = len(entries)
        device_tokens = None
        if feed is not None:
            src, take = feed
            take = list(take)
            if take == list(range(len(take))):
                device_tokens = src.ids[:rows]
            else:
                if self._feed is None or self._feed.numel() < rows:
                    self._feed = torch.empty(max(rows, 64), dtype=torch.int32, device=self.device)
                j = 0
                while j < rows:                         # runs of neighbouring rows: one small copy each
                    k = j
                    while k + 1 < rows and take[k + 1] == take[k] + 1:
                        k += 1
                    self._feed[j:k + 1].copy_(src.ids[take[j]:take[k] + 1], non_blocking=True)
                    j = k + 1
                device_tokens = self._feed[:rows]
        logits = self.engine.step(entries, device_tokens=device_tokens)
        slot = self._ring[self._turn]
        if slot is None or slot.ids.numel() < rows:
            n = max(rows, 64)
            slot = Launched(torch.empty(n, dtype=torch.int32, device=self.device),
                            torch.empty(n, dtype=torch.int32).pin_memory(), torch.cuda.Event(), 0)
            self._ring[self._turn] = slot
        self._turn = (self._turn + 1) % len(self._ring)
        slot.rows = rows
        self._sample_into(slot.ids[:rows], logits, requests, histories, counters, params)
        slot.host[:rows].copy_(slot.ids[:rows], non_blocking=True)
        slot.event.record()
        self._steps += 1
        return slot

    def result(self, launched: Launched) -> List[int]:
        """The ids a launched step sampled (waits for them)."""
        launched.event.synchronize()
        ids = launched.host[:launched.rows].tolist()
        if self._steps % self.CHECK_EVERY == 0:
            self.check()
        return ids

    def step_and_sample(self, entries: Sequence[Tuple[int, Sequence[int]]], requests: Sequence[int],
                        histories: Sequence[Sequence[int]], counters: Sequence[int],
                        params: SamplerParams) -> List[int]:
        logits = self.engine.step(entries)
        sampled = self.sample_logits(logits, requests, histories, counters, params)
        self._steps += 1
        if self._steps % self.CHECK_EVERY == 0:
            self.check()
        return sampled

    def check(self) -> None:
        self.engine.check_kernels()
