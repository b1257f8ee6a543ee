"""Runs steps and samples their logits on the device: the backend of the generation loop."""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch

from .. import kernels
from .params import SamplerParams
from .rng import request_seed


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
        host = self._out_host[:rows]
        host.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return host.tolist()

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
