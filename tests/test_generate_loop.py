"""The generation loop's decisions, on a backend that needs no GPU."""
from typing import List

import pytest

from ziglm_b200.engine.generate import GenerationOptions, plan_batch, run_generation
from ziglm_b200.sampling import SamplerParams


class FakeBackend:
    """Next token = (sum of the sequence so far) mod vocab; records every step and slot."""

    def __init__(self, n_slots: int, vocab: int = 50):
        self.free = list(range(n_slots))
        self.held = {}
        self.vocab = vocab
        self.steps: List[list] = []
        self.freed: List[int] = []

    def alloc_slot(self):
        assert self.free, "the loop asked for more slots than exist"
        s = self.free.pop(0)
        self.held[s] = []
        return s

    def free_slot(self, s):
        assert s in self.held, "slot freed twice or never held"
        del self.held[s]
        self.free.append(s)
        self.free.sort()
        self.freed.append(s)

    def step_and_sample(self, entries, requests, histories, counters, params):
        self.steps.append([(s, list(t)) for s, t in entries])
        out = []
        for (s, toks), h in zip(entries, histories):
            assert s in self.held
            self.held[s].extend(toks)
            assert self.held[s] == list(h), "the history handed to the sampler is the sequence so far"
            out.append(sum(self.held[s]) % self.vocab)
        return out


def expected(prompt, n, vocab=50, stop=()):
    seq, out = list(prompt), []
    while len(out) < n:
        t = sum(seq) % vocab
        if t in stop:
            return out, "stop"
        out.append(t); seq.append(t)
    return out, "length"


def run(prompts, opts, n_slots=4, max_tokens=4096, max_seq_len=512, stop_ids=(), callback=None):
    b = FakeBackend(n_slots)
    res, stats = run_generation(b, prompts, opts, stop_ids, n_slots, max_tokens, max_seq_len, 64, callback)
    assert not b.held and sorted(b.free) == list(range(n_slots)), "every slot came back"
    return b, res, stats


def test_unequal_prompts_start_together_then_one_token_each():
    prompts = [[1, 2, 3], [4], [5, 6, 7, 8, 9]]
    b, res, stats = run(prompts, GenerationOptions(max_tokens=4, sampler=SamplerParams(greedy=True)))
    assert b.steps[0] == [(0, [1, 2, 3]), (1, [4]), (2, [5, 6, 7, 8, 9])]
    assert all(len(t) == 1 for step in b.steps[1:] for _, t in step)
    for p, r in zip(prompts, res):
        assert (r.tokens, r.finish_reason) == expected(p, 4)
    assert stats.prompt_tokens == 9 and stats.completion_tokens == 12
    assert len(b.steps) == 4                                   # prompt step + 3 decode steps


def test_stop_token_ends_a_sequence_early_and_is_not_emitted():
    prompts = [[1, 2, 3], [10, 1], [2, 2]]
    want = [expected(p, 8, stop={22}) for p in prompts]
    assert any(r == "stop" for _, r in want) and any(r == "length" for _, r in want)
    b, res, _ = run(prompts, GenerationOptions(max_tokens=8, stop_tokens=[22]))
    for w, r in zip(want, res):
        assert (r.tokens, r.finish_reason) == w and 22 not in r.tokens
    sizes = [len(s) for s in b.steps]
    assert sizes == sorted(sizes, reverse=True) and sizes[0] == 3 and sizes[-1] < 3    # the batch shrinks


def test_eos_from_the_model_and_ignore_eos():
    p = [[1, 2, 3]]
    first = expected(p[0], 1)[0][0]
    _, res, _ = run(p, GenerationOptions(max_tokens=5), stop_ids=[first])
    assert res[0].tokens == [] and res[0].finish_reason == "stop"
    _, res, _ = run(p, GenerationOptions(max_tokens=5, ignore_eos=True), stop_ids=[first])
    assert len(res[0].tokens) == 5


def test_more_requests_than_slots_run_batch_after_batch_and_slots_are_used_again():
    prompts = [[i + 1, i + 2] for i in range(7)]
    b, res, _ = run(prompts, GenerationOptions(max_tokens=3), n_slots=3)
    assert [len(s) for s in b.steps if len(s[0][1]) == 2] == [3, 3, 1]      # three prompt steps
    assert len(b.freed) == 7 and set(b.freed) == {0, 1, 2}
    for p, r in zip(prompts, res):
        assert r.tokens == expected(p, 3)[0]


def test_cache_room_limits_a_batch():
    lens = [100, 100, 100, 100]
    assert plan_batch([0, 1, 2, 3], lens, 28, 8, 256, 512, 64) == [0, 1]        # 128 + 128 positions
    assert plan_batch([2, 3], lens, 28, 8, 256, 512, 64) == [2, 3]
    assert plan_batch([0, 1, 2, 3], lens, 28, 1, 4096, 512, 64) == [0]
    with pytest.raises(ValueError):
        plan_batch([0], [300], 100, 8, 256, 512, 64)


def test_context_limit_and_errors():
    _, res, _ = run([[1] * 10], GenerationOptions(max_tokens=50), max_seq_len=16)
    assert res[0].finish_reason == "context" and len(res[0].tokens) == 7       # positions 10..16
    with pytest.raises(ValueError, match="empty"):
        run([[]], GenerationOptions())
    with pytest.raises(ValueError, match="holds"):
        run([[1] * 20], GenerationOptions(), max_seq_len=16)


def test_callback_may_end_a_request_and_echo_prompt():
    seen = []

    def cb(request, token):
        seen.append((request, token))
        return not (request == 0 and len([1 for r, _ in seen if r == 0]) == 2)

    _, res, _ = run([[1, 2], [3, 4]], GenerationOptions(max_tokens=5, echo_prompt=True), callback=cb)
    assert len(res[0].tokens) == 2 + 2 and res[0].tokens[:2] == [1, 2]
    assert len(res[1].tokens) == 2 + 5


class FaultyBackend(FakeBackend):
    """Reports a device fault: at a given step, or when the loop asks at the end of a batch."""

    def __init__(self, n_slots, fail_at_step=None, fail_at_check=False):
        super().__init__(n_slots)
        self.fail_at_step, self.fail_at_check, self.checks = fail_at_step, fail_at_check, 0

    def step_and_sample(self, entries, requests, histories, counters, params):
        if self.fail_at_step is not None and len(self.steps) == self.fail_at_step:
            raise RuntimeError("a bounded wait ran out")
        return super().step_and_sample(entries, requests, histories, counters, params)

    def check(self):
        self.checks += 1
        if self.fail_at_check:
            raise RuntimeError("a bounded wait ran out")


def test_a_fault_reported_by_the_backend_ends_generation_and_gives_every_slot_back():
    opts = GenerationOptions(max_tokens=6, ignore_eos=True, sampler=SamplerParams(greedy=True))
    prompts = [[1, 2, 3], [4], [5, 6], [7, 8, 9, 10], [11]]
    # in the middle of the first batch, after one request has already ended by itself
    b = FaultyBackend(3, fail_at_step=3)
    short = GenerationOptions(max_tokens=6, ignore_eos=True, stop_tokens=[sum([4]) % 50], sampler=SamplerParams(greedy=True))
    with pytest.raises(RuntimeError, match="bounded wait"):
        run_generation(b, prompts, short, (), 3, 4096, 512, 64)
    assert not b.held and sorted(b.free) == [0, 1, 2], "the slots of the live sequences came back, none twice"
    assert len(b.steps) == 3
    # the loop asks after every batch; a fault found then stops before the next batch starts
    b = FaultyBackend(3, fail_at_check=True)
    with pytest.raises(RuntimeError, match="bounded wait"):
        run_generation(b, prompts, opts, (), 3, 4096, 512, 64)
    assert b.checks == 1 and not b.held and all(len(e) <= 3 for e in b.steps)
    # and a healthy backend is asked once per batch
    b = FaultyBackend(3)
    res, _ = run_generation(b, prompts, opts, (), 3, 4096, 512, 64)
    assert b.checks == 2 and len(res) == 5


def test_engine_check_names_the_code_and_repairs_the_counters():
    """Engine.check_kernels with a stand-in for the device's error words (no GPU)."""
    from ziglm_b200.engine.engine import Engine
    from ziglm_b200.kernels import KernelError

    class Buf:
        def __init__(self): self.zeroed = []
        def zero(self, name): self.zeroed.append(name)

    e = Engine.__new__(Engine)
    e.ws, e.graph_ws, e._repeat = Buf(), Buf(), object()
    e.check_kernels(read=lambda: {"gemm_tc": 0, "attention_tc": 0})
    assert e._repeat is not None and e.ws.zeroed == []
    with pytest.raises(KernelError) as err:
        e.check_kernels(read=lambda: {"gemm_tc": 0, "attention_tc": 11})
    assert "attention_tc" in str(err.value) and "11" in str(err.value) and "page" in str(err.value)
    assert e._repeat is None and e.ws.zeroed == ["attn_flat_counters"] and e.graph_ws.zeroed == ["attn_flat_counters"]


class AheadBackend(FakeBackend):
    """The same model of a device, with steps that are queued (``launch``) and read later (``result``): the ids of
    a queued step stay hidden until then, a step may take its tokens from the ids of a queued one, and a slot
    must not be given back while a queued step that uses it has not been read."""

    def __init__(self, n_slots, vocab=50, ahead=True):
        super().__init__(n_slots, vocab)
        self.ahead = ahead
        self.unread = []            # handles that were launched and not read: each a dict
        self.launched = 0

    def can_run_ahead(self, params):
        return self.ahead

    def launch(self, entries, requests, histories, counters, params, feed=None):
        if feed is not None:
            src, take = feed
            assert len(take) == len(entries) and all(list(t) == [0] for _, t in entries), "fed steps bring place holders"
            entries = [(s, [src["ids"][j]]) for (s, _), j in zip(entries, take)]
        else:
            assert all(h["read"] for h in self.unread), "tokens from the host while a step's ids are still unread"
        ids = []
        for s, toks in entries:
            assert s in self.held, "a step uses a slot nobody holds"
            self.held[s].extend(toks)
            ids.append(sum(self.held[s]) % self.vocab)
        self.steps.append([(s, list(t)) for s, t in entries])
        self.launched += 1
        h = {"ids": ids, "slots": [s for s, _ in entries], "read": False, "counters": list(counters)}
        self.unread.append(h)
        assert sum(1 for x in self.unread if not x["read"]) <= 2, "more than one step ahead"
        return h

    def result(self, h):
        assert not h["read"]
        # steps complete in the order they were queued
        for x in self.unread:
            if x is h:
                break
            assert x["read"], "a step is read before the one queued before it"
        h["read"] = True
        return list(h["ids"])

    def free_slot(self, s):
        assert all(h["read"] or s not in h["slots"] for h in self.unread), "a slot is given back under a queued step"
        super().free_slot(s)


@pytest.mark.parametrize("max_tokens,stop_tokens,n_slots", [(6, (), 3), (9, (7, 13, 21, 33), 2), (1, (), 4), (12, (0, 1, 2, 3, 4, 5), 3),
                                                            (5, (), 1)])
def test_running_one_step_ahead_decides_what_the_plain_loop_decides(max_tokens, stop_tokens, n_slots):
    prompts = [[1, 2, 3], [4], [5, 6], [7, 8, 9, 10], [11], [3, 3, 3, 3, 3, 3, 3]]
    opts = GenerationOptions(max_tokens=max_tokens, ignore_eos=True, stop_tokens=stop_tokens, sampler=SamplerParams(greedy=True))
    plain = FakeBackend(n_slots)
    want, want_stats = run_generation(plain, prompts, opts, (), n_slots, 4096, 512, 64)
    ahead = AheadBackend(n_slots)
    got, stats = run_generation(ahead, prompts, opts, (), n_slots, 4096, 512, 64)
    assert [(r.tokens, r.finish_reason) for r in got] == [(r.tokens, r.finish_reason) for r in want]
    assert (stats.prompt_tokens, stats.completion_tokens) == (want_stats.prompt_tokens, want_stats.completion_tokens)
    assert not ahead.held and sorted(ahead.free) == list(range(n_slots)) and all(h["read"] for h in ahead.unread)
    # a sequence that ends by its token limit is never part of a step ahead: without stop tokens no step is wasted
    if not stop_tokens:
        assert ahead.launched == len(plain.steps)
    else:
        assert len(plain.steps) <= ahead.launched <= len(plain.steps) + len(prompts)
    # a backend that says it cannot run ahead (penalties need the ids on the host) takes the plain loop
    sync = AheadBackend(n_slots, ahead=False)
    again, _ = run_generation(sync, prompts, opts, (), n_slots, 4096, 512, 64)
    assert sync.launched == 0 and [(r.tokens, r.finish_reason) for r in again] == [(r.tokens, r.finish_reason) for r in want]


def test_running_ahead_with_a_callback_that_ends_requests_and_at_the_context_limit():
    prompts = [[1, 2, 3, 4, 5], [9, 9], [2]]
    seen = []

    def cb(request, token):
        seen.append((request, token))
        return not (request == 1 and len([1 for r, _ in seen if r == 1]) == 3)

    opts = GenerationOptions(max_tokens=50, ignore_eos=True, sampler=SamplerParams(greedy=True))
    want, _ = run_generation(FakeBackend(3), prompts, opts, (), 3, 4096, 9, 64, cb)
    plain_seen, seen[:] = list(seen), []
    ahead = AheadBackend(3)
    got, _ = run_generation(ahead, prompts, opts, (), 3, 4096, 9, 64, cb)
    assert [(r.tokens, r.finish_reason) for r in got] == [(r.tokens, r.finish_reason) for r in want]
    assert seen == plain_seen
    assert {r.finish_reason for r in got} == {"context", "stop"}
    assert max(len(h) for h in ahead.held.values()) if ahead.held else True


def test_running_ahead_gives_slots_back_when_a_step_fails():
    class Failing(AheadBackend):
        def result(self, h):
            if self.launched >= 4:
                raise RuntimeError("a bounded wait ran out")
            return super().result(h)

        def free_slot(self, s):              # the device is in an unknown state: no ordering to insist on
            FakeBackend.free_slot(self, s)

    b = Failing(2)
    opts = GenerationOptions(max_tokens=20, ignore_eos=True, sampler=SamplerParams(greedy=True))
    with pytest.raises(RuntimeError, match="bounded wait"):
        run_generation(b, [[1, 2], [3]], opts, (), 2, 4096, 512, 64)
    assert not b.held and sorted(b.free) == [0, 1]
