"""The generation loop above the step function.

The reference's ``Engine.generate`` (src/engine.zig:382-500) runs one sequence:
prefill, sample, then decode-and-sample until a stop token, ``max_tokens`` or the
end of the context, with the stop token neither stored nor emitted (473-485) and
timings in ``GenerationStats`` (src/types.zig:357-373).  Here the same loop runs
batches: requests that fit the cache together start together with unequal
prompts, a request that ends gives its slot back at once while the others go on,
and batch follows batch until every request is done.  Token ids go in and come
out; tokenising is not part of this library.

The loop only decides; everything that touches the device goes through the calls
of a *backend* (``alloc_slot``, ``free_slot``, ``step_and_sample`` and, if it has
one, ``check``, which is called when a batch ends and raises if the device
reported a fault), so the decisions are tested without a GPU.  If a step raises,
the slots of the live sequences are given back before the error goes on.

A backend that also has ``launch`` and ``result`` (and says ``can_run_ahead`` for
the sampling options) lets the loop run one step ahead: it queues the next step,
whose tokens the device takes from the ids it has just sampled, before it reads
those ids itself, so the host's work on a step hides behind the step before.  The
decisions are the same; a sequence that turns out to have ended is then part of
one more step whose result for it is dropped, and gives its slot back only when
that step is over.  Sequences that are sure to end with the running step (their
token limit or the context's end) are left out of the step ahead.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence, Tuple

from ..sampling.params import SamplerParams


@dataclass
class GenerationOptions:
    """Options of ``generate``; fields and defaults of the reference (src/types.zig:350-355)
    plus ``ignore_eos`` for measurements."""
    max_tokens: int = 512
    sampler: SamplerParams = field(default_factory=SamplerParams)
    stop_tokens: Sequence[int] = ()
    echo_prompt: bool = False
    ignore_eos: bool = False


@dataclass
class GenerationStats:
    """Counters and wall-clock times of one ``generate`` call (src/types.zig:357-373)."""
    prompt_tokens: int = 0
    completion_tokens: int = 0
    prefill_time_ms: float = 0.0
    generation_time_ms: float = 0.0
    total_time_ms: float = 0.0

    def prefill_tokens_per_sec(self) -> float:
        return self.prompt_tokens / self.prefill_time_ms * 1000.0 if self.prefill_time_ms > 0 else 0.0

    def generation_tokens_per_sec(self) -> float:
        return self.completion_tokens / self.generation_time_ms * 1000.0 if self.generation_time_ms > 0 else 0.0


@dataclass
class GenerationResult:
    tokens: List[int]                 # generated ids (after the prompt unless echo_prompt)
    finish_reason: str                # "stop", "length" or "context"
    prompt_tokens: int = 0


@dataclass
class _Live:
    request: int
    slot: int
    length: int                       # tokens the slot holds
    out: List[int]
    history: List[int]
    next_token: int = -1


def plan_batch(pending: Sequence[int], prompt_lens: Sequence[int], max_new: int, max_batch: int, max_tokens: int,
               max_seq_len: int, page: int) -> List[int]:
    """The requests (indices into ``pending`` order) of the next batch: as many, in order, as fit ``max_batch``
    slots and ``max_tokens`` cache positions when each may grow to prompt + max_new (at most max_seq_len),
    rounded up to whole pages."""
    chosen: List[int] = []
    used = 0
    for r in pending:
        need_len = min(prompt_lens[r] + max_new, max_seq_len)
        need = -(-need_len // page) * page
        if chosen and (len(chosen) >= max_batch or used + need > max_tokens):
            break
        if not chosen and need > max_tokens:
            raise ValueError(f"request {r} needs {need} cache positions, the cache holds {max_tokens}")
        chosen.append(r)
        used += need
    return chosen


def run_generation(backend, prompts: Sequence[Sequence[int]], options: GenerationOptions, stop_ids: Sequence[int],
                   max_batch: int, max_tokens: int, max_seq_len: int, page: int,
                   callback: Optional[Callable[[int, int], bool]] = None
                   ) -> Tuple[List[GenerationResult], GenerationStats]:
    """Generate for every prompt.  ``callback(request, token)`` may return False to end that request."""
    stats = GenerationStats()
    t_start = time.perf_counter()
    results: List[Optional[GenerationResult]] = [None] * len(prompts)
    prompt_lens = [len(p) for p in prompts]
    for r, p in enumerate(prompts):
        if len(p) == 0:
            raise ValueError(f"prompt {r} is empty")                      # error.EmptyPrompt, src/engine.zig:322
        if len(p) > max_seq_len:
            raise ValueError(f"prompt {r} has {len(p)} tokens, a sequence holds {max_seq_len}")  # PromptExceedsContext
    stop = set(int(s) for s in options.stop_tokens)
    if not options.ignore_eos:
        stop |= set(int(s) for s in stop_ids)
    pending = list(range(len(prompts)))

    def finish(seq: _Live, reason: str) -> None:
        backend.free_slot(seq.slot)
        head = list(prompts[seq.request]) if options.echo_prompt else []
        results[seq.request] = GenerationResult(head + seq.out, reason, prompt_lens[seq.request])

    while pending:
        batch = plan_batch(pending, prompt_lens, options.max_tokens, max_batch, max_tokens, max_seq_len, page)
        pending = pending[len(batch):]
        live = [_Live(r, backend.alloc_slot(), 0, [], list(prompts[r])) for r in batch]
        ahead = (hasattr(backend, "launch") and hasattr(backend, "result")
                 and getattr(backend, "can_run_ahead", lambda p: False)(options.sampler))
        try:
            if ahead:
                _run_batch_ahead(backend, live, prompts, options, stop, stats, finish, max_seq_len, callback)
            else:
                _run_batch(backend, live, True, prompts, options, stop, stats, finish, max_seq_len, callback)
        except BaseException:
            for s in live:
                if results[s.request] is None:
                    try:
                        backend.free_slot(s.slot)
                    except Exception:
                        pass
            raise
    stats.total_time_ms = (time.perf_counter() - t_start) * 1000.0
    return [r for r in results if r is not None], stats


def _run_batch(backend, live: List[_Live], first: bool, prompts, options: GenerationOptions, stop, stats: GenerationStats,
               finish, max_seq_len: int, callback) -> None:
    """One batch from its prompts to its last sequence's end.  ``live`` is emptied as sequences end."""
    while live:
        t0 = time.perf_counter()
        if first:
            entries = [(s.slot, list(prompts[s.request])) for s in live]
        else:
            entries = [(s.slot, [s.next_token]) for s in live]
        sampled = backend.step_and_sample(entries, [s.request for s in live], [s.history for s in live],
                                          [len(s.out) for s in live], options.sampler)
        dt = (time.perf_counter() - t0) * 1000.0
        if first:
            stats.prefill_time_ms += dt
            stats.prompt_tokens += sum(len(e[1]) for e in entries)
        else:
            stats.generation_time_ms += dt
        still: List[_Live] = []
        for s, e, tok in zip(live, entries, sampled):
            s.length += len(e[1])
            tok = int(tok)
            if tok in stop:
                finish(s, "stop")                                    # the stop token is not emitted
                continue
            s.out.append(tok)
            s.history.append(tok)
            stats.completion_tokens += 1
            keep_going = True
            if callback is not None and callback(s.request, tok) is False:
                keep_going = False
            if not keep_going:
                finish(s, "stop")
            elif len(s.out) >= options.max_tokens:
                finish(s, "length")
            elif s.length >= max_seq_len:
                finish(s, "context")                                 # cur_pos < max_seq_len, src/engine.zig:464
            else:
                s.next_token = tok
                still.append(s)
        live[:] = still
        first = False
    check = getattr(backend, "check", None)
    if check is not None:
        check()


def _run_batch_ahead(backend, live: List[_Live], prompts, options: GenerationOptions, stop, stats: GenerationStats,
                     finish, max_seq_len: int, callback) -> None:
    """One batch, one step ahead of the ids it reads (see the module's text).  ``live`` is kept as the set of
    sequences that have not given their slot back."""
    params = options.sampler
    rows = list(live)                                    # the sequences of the step in flight, in row order
    for s in rows:
        s.length = len(prompts[s.request])
    flying = backend.launch([(s.slot, list(prompts[s.request])) for s in rows], [s.request for s in rows],
                            [s.history for s in rows], [0] * len(rows), params)
    lens = [s.length for s in rows]                      # what each slot holds once the step in flight is over
    ended_early = set()                                  # ended while a step that includes them was already queued
    waiting = []                                         # (sequence, reason): to be finished when that step is over
    t_last = time.perf_counter()
    first = True
    while flying is not None:
        # 1. the step after: every sequence that is not known, or sure, to end with the step in flight
        nxt_rows, take = [], []
        for j, s in enumerate(rows):
            if id(s) in ended_early:
                continue
            if len(s.out) + 1 >= options.max_tokens or lens[j] >= max_seq_len:
                continue                                 # its token limit, or the context's end: sure to end
            nxt_rows.append(s)
            take.append(j)
        nxt = None
        if nxt_rows:
            nxt = backend.launch([(s.slot, [0]) for s in nxt_rows], [s.request for s in nxt_rows],
                                 [s.history for s in nxt_rows], [len(s.out) + 1 for s in nxt_rows], params,
                                 feed=(flying, take))
            for s in nxt_rows:
                s.length += 1
        in_next = set(id(s) for s in nxt_rows)
        # 2. the ids of the step in flight; what waited for its end can go now
        sampled = backend.result(flying)
        now = time.perf_counter()
        if first:
            stats.prefill_time_ms += (now - t_last) * 1000.0
            stats.prompt_tokens += sum(len(prompts[s.request]) for s in rows)
        else:
            stats.generation_time_ms += (now - t_last) * 1000.0
        t_last = now
        for s, reason in waiting:
            finish(s, reason)
            live.remove(s)
        waiting = []
        # 3. the same decisions as without running ahead, in row order
        for j, (s, tok) in enumerate(zip(rows, sampled)):
            if id(s) in ended_early:
                continue                                 # this row was queued before its end was known
            tok = int(tok)
            reason = None
            if tok in stop:
                reason = "stop"                          # the stop token is not emitted
            else:
                s.out.append(tok)
                s.history.append(tok)
                stats.completion_tokens += 1
                if callback is not None and callback(s.request, tok) is False:
                    reason = "stop"
                elif len(s.out) >= options.max_tokens:
                    reason = "length"
                elif lens[j] >= max_seq_len:
                    reason = "context"
            if reason is None:
                continue
            if id(s) in in_next:
                ended_early.add(id(s))                   # its slot is in use by the queued step
                waiting.append((s, reason))
            else:
                finish(s, reason)
                live.remove(s)
        rows, flying = nxt_rows, nxt
        lens = [s.length for s in rows]
        first = False
    check = getattr(backend, "check", None)
    if check is not None:
        check()


def generate(engine, prompts, options: Optional[GenerationOptions] = None, callback=None):
    """``Engine.generate``: one prompt (a list of ids) or several; returns (results, stats)."""
    from ..sampling.device import DeviceSampler
    options = options or GenerationOptions()
    single = len(prompts) > 0 and isinstance(prompts[0], int)
    batch = [list(prompts)] if single else [list(p) for p in prompts]
    backend = DeviceSampler(engine)
    results, stats = run_generation(backend, batch, options, engine.spec.stop_token_ids,
                                    engine.cache.slots.slots.capacity, engine.cache.n_pages * engine.cache.page_size,
                                    engine.max_seq_len, engine.cache.page_size, callback)
    return (results[0] if single else results), stats
