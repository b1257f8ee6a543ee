"""The engine against the plain implementation, in float32 and in bfloat16, under every way of cutting
requests into steps and batches: whole; the last 32 tokens one by one; batches of unequal lengths whose
shorter requests end earlier, batch after batch so that slots and pages are used again; long decoding;
the first tokens of a sequence."""
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
# request lengths per configuration: a one-token request, lengths around the page size of 64, a long one
LENGTHS = {"A": [5, 11, 17, 70, 45, 128], "B": [1, 9, 23, 40, 97, 64], "C": [3, 65, 33, 128, 12, 50],
           "D": [5, 130, 64, 200, 17, 96], "E": [1, 129, 70, 33, 250, 16], "F": [2, 66, 150, 31, 128, 90],
           "G": [1, 40, 77, 130, 64, 19], "H": [3, 130, 64, 200, 49, 96]}


class Zoo:
    """Model folders, engines and the plain model's logits, made once per (configuration, precision)."""

    def __init__(self, tmp):
        self.tmp = tmp
        self.cache = {}

    def get(self, name, dn, **opts):
        key = (name, dn, tuple(sorted(opts.items())))
        if key not in self.cache:
            from ziglm_b200 import Engine, EngineOptions
            dtype = DTYPES[dn]
            folder = helpers.make_folder(self.tmp, helpers.CONFIGS[name], 17, dtype, helpers.NORM_JITTER[name])
            o = dict(dtype=dn, max_tokens=1024, max_batch=8)
            o.update(opts)
            self.cache[key] = (folder, Engine.load(folder, EngineOptions(**o)))
        return self.cache[key]

    def requests(self, name):
        V = helpers.CONFIGS[name]["vocab_size"]
        return [helpers.random_tokens(n, V, 100 + i) for i, n in enumerate(LENGTHS[name])]

    def plain(self, name, dn):
        key = ("plain", name, dn)
        if key not in self.cache:
            folder, _ = self.get(name, dn)
            act = None if dn == "float32" else torch.bfloat16
            self.cache[key] = [helpers.plain_logits(folder, r, act=act) for r in self.requests(name)]
        return self.cache[key]


@pytest.fixture(scope="module")
def zoo(tmp_path_factory):
    return Zoo(tmp_path_factory.mktemp("models"))


# D and E have the head sizes of the tensor-core attention kernels: in bfloat16 their prompts run the tcgen05
# kernel (or the mma.sync one below 16 tokens) and their decode steps the flat kernel with rotation and cache write
# F (feed-forward biases, linear position stretching) and G (yarn) are what config.json allows beyond the usual
# H has a sliding window in every layer (from config.json): pages behind it are given back as a sequence grows
CASES = [(n, d) for n in ("A", "B", "C", "F", "G", "H") for d in ("float32", "bfloat16")] + [
    ("D", "bfloat16"), ("E", "bfloat16"), ("D", "float32")]


@pytest.mark.parametrize("name,dn", CASES)
def test_each_request_alone_and_whole(zoo, name, dn):
    _, eng = zoo.get(name, dn)
    for req, want in zip(zoo.requests(name), zoo.plain(name, dn)):
        slot = eng.alloc_slot()
        got = eng.step([(slot, req)], [list(range(len(req)))]).clone()
        eng.free_slot(slot)
        helpers.assert_close(got, want, DTYPES[dn], f"{name} {dn} whole, {len(req)} tokens")
    eng.cache.slots.check()


@pytest.mark.parametrize("name,dn", CASES)
def test_last_32_tokens_one_by_one(zoo, name, dn):
    _, eng = zoo.get(name, dn)
    for req, want in zip(zoo.requests(name), zoo.plain(name, dn)):
        head = max(1, len(req) - 32)
        slot = eng.alloc_slot()
        rows = [eng.step([(slot, req[:head])], [list(range(head))]).clone()]
        for t in req[head:]:
            rows.append(eng.step([(slot, [t])]).clone())
        eng.free_slot(slot)
        got = torch.cat(rows)
        helpers.assert_close(got, want, DTYPES[dn], f"{name} {dn} tail one by one, {len(req)} tokens")
        # the first wrong place, if any, is named by assert_close; the prompt's end is row head-1, the first
        # decoded token row head


def run_batches(eng, requests, batches, prompt_lens):
    """Replay ``requests`` in ``batches`` (lists of request indices): the first step of a batch brings each
    request's first ``prompt_lens[r]`` tokens, then every live request brings one token a step; a request ends
    when its tokens are used up and gives its slot back at once.  Returns logits per request, all places."""
    out = {}
    for batch in batches:
        slots = {r: eng.alloc_slot() for r in batch}
        used = {r: 0 for r in batch}
        rows = {r: [] for r in batch}
        live = list(batch)
        first = True
        while live:
            entries, want = [], []
            for r in live:
                n = prompt_lens[r] if first else 1
                entries.append((slots[r], requests[r][used[r]:used[r] + n]))
                want.append(list(range(n)))
            logits = eng.step(entries, want).clone()
            at = 0
            for r, (_, toks) in zip(live, entries):
                rows[r].append(logits[at:at + len(toks)])
                at += len(toks)
                used[r] += len(toks)
            first = False
            for r in list(live):
                if used[r] == len(requests[r]):
                    eng.free_slot(slots[r])
                    live.remove(r)
        for r in batch:
            out[r] = torch.cat(rows[r])
    return out


@pytest.mark.parametrize("name,dn", CASES)
def test_batches_of_unequal_lengths_with_slots_used_again(zoo, name, dn):
    # three slots and few pages: the second and third batch run in slots and pages the first one left
    _, eng = zoo.get(name, dn, max_batch=3, max_tokens=448)
    reqs = zoo.requests(name)
    prompt_lens = [max(1, len(r) - k) for r, k in zip(reqs, (3, 9, 0, 20, 33, 40))]
    prompt_lens = [min(p, len(r)) for p, r in zip(prompt_lens, reqs)]
    order = sorted(range(len(reqs)), key=lambda r: len(reqs[r]))
    batches = [[order[0], order[5], order[2]], [order[4], order[1]], [order[3]]]
    got = run_batches(eng, reqs, batches, prompt_lens)
    for r, want in enumerate(zoo.plain(name, dn)):
        helpers.assert_close(got[r], want, DTYPES[dn], f"{name} {dn} batched, request {r} of {len(reqs[r])} tokens")
    eng.cache.slots.check()
    assert eng.cache.slots.slots.n_held == 0 and all(g.pages.pool.n_held == 0 for g in eng.cache.groups)


@pytest.mark.parametrize("name,dn", [("A", "float32"), ("B", "float32"), ("C", "float32")])
def test_float32_does_not_depend_on_the_schedule(zoo, name, dn):
    """In 32-bit the three schedules agree to the last few bits: every output element is summed in one fixed order."""
    _, eng = zoo.get(name, dn)
    reqs = zoo.requests(name)
    whole = []
    for req in reqs:
        slot = eng.alloc_slot()
        whole.append(eng.step([(slot, req)], [list(range(len(req)))]).clone())
        eng.free_slot(slot)
    got = run_batches(eng, reqs, [[0, 1, 2, 3], [4, 5]], [max(1, len(r) // 2) for r in reqs])
    for r in range(len(reqs)):
        assert (got[r] - whole[r]).abs().max().item() <= 1e-6


@pytest.mark.parametrize("name,dn", [("A", "float32"), ("B", "bfloat16"), ("C", "bfloat16"), ("B", "float32"),
                                     ("D", "bfloat16"), ("E", "bfloat16")])
def test_long_decoding(zoo, name, dn):
    _, eng = zoo.get(name, dn)
    V = helpers.CONFIGS[name]["vocab_size"]
    n = min(200, helpers.CONFIGS[name]["max_position_embeddings"])
    toks = helpers.random_tokens(n, V, 999)
    folder, _ = zoo.get(name, dn)
    want = helpers.plain_logits(folder, toks, act=None if dn == "float32" else torch.bfloat16)
    slot = eng.alloc_slot()
    rows = [eng.step([(slot, toks[:3])], [[0, 1, 2]]).clone()]
    for t in toks[3:]:
        rows.append(eng.step([(slot, [t])]).clone())
    eng.free_slot(slot)
    helpers.assert_close(torch.cat(rows), want, DTYPES[dn], f"{name} {dn} long decoding")


@pytest.mark.parametrize("name,dn", CASES)
def test_first_tokens_of_a_sequence(zoo, name, dn):
    folder, eng = zoo.get(name, dn)
    V = helpers.CONFIGS[name]["vocab_size"]
    act = None if dn == "float32" else torch.bfloat16
    for toks in ([V - 1], [0, 0], [5, V - 1, 5]):
        want = helpers.plain_logits(folder, toks, act=act)
        slot = eng.alloc_slot()
        rows = [eng.step([(slot, [t])]).clone() for t in toks]       # from the very first token, one by one
        eng.free_slot(slot)
        helpers.assert_close(torch.cat(rows), want, DTYPES[dn], f"{name} {dn} first tokens {toks}")
        slot = eng.alloc_slot()
        got = eng.step([(slot, toks)], [list(range(len(toks)))]).clone()
        eng.free_slot(slot)
        helpers.assert_close(got, want, DTYPES[dn], f"{name} {dn} first tokens whole {toks}")


@pytest.mark.parametrize("name,dn", [("D", "bfloat16"), ("E", "bfloat16"), ("F", "bfloat16"), ("D", "float32")])
def test_a_prompt_in_pieces_on_a_slot_that_already_holds_tokens(zoo, name, dn):
    """A prompt of 150 tokens cut into 70 + 50 + 30: the second and third piece are prompt steps of many tokens
    on a slot that is not empty (in bfloat16 with head size 64 or 128 that is the tcgen05 prompt kernel reading
    cached pages before the new tokens).  Every place is wanted and compared with the plain model."""
    folder, eng = zoo.get(name, dn)
    V = helpers.CONFIGS[name]["vocab_size"]
    toks = helpers.random_tokens(150, V, 4242)
    want = helpers.plain_logits(folder, toks, act=None if dn == "float32" else torch.bfloat16)
    slot = eng.alloc_slot()
    rows, at = [], 0
    for n in (70, 50, 30):
        rows.append(eng.step([(slot, toks[at:at + n])], [list(range(n))]).clone())
        at += n
    eng.free_slot(slot)
    helpers.assert_close(torch.cat(rows), want, DTYPES[dn], f"{name} {dn} prompt in pieces 70 + 50 + 30")
    # and two sequences at different depths in one step: 20 new tokens after 70, 45 new tokens after 16
    other = helpers.random_tokens(61, V, 4243)
    want_other = helpers.plain_logits(folder, other, act=None if dn == "float32" else torch.bfloat16)
    a, b = eng.alloc_slot(), eng.alloc_slot()
    eng.step([(a, toks[:70]), (b, other[:16])], [[], []])
    got = eng.step([(a, toks[70:90]), (b, other[16:61])], [list(range(20)), list(range(45))]).clone()
    eng.free_slot(a); eng.free_slot(b)
    helpers.assert_close(got[:20], want[70:90], DTYPES[dn], f"{name} {dn} 20 tokens after 70")
    helpers.assert_close(got[20:], want_other[16:61], DTYPES[dn], f"{name} {dn} 45 tokens after 16")


@pytest.mark.parametrize("name,dn", [("D", "float32"), ("D", "bfloat16"), ("E", "bfloat16")])
def test_a_batch_that_shrinks_through_many_sizes_generates_what_each_request_generates_alone(tmp_path, name, dn):
    """Twelve requests on eight slots, each ended after its own number of tokens, so the batch steps down through
    most sizes from 8 to 1 (twice).  In float32, where logits do not depend on the batch, greedy output equals
    one request at a time token for token.  In bfloat16 a batch and a single request take different kernels for
    their prompts, so two nearly equal logits may be ordered differently; there every token that was chosen must
    be the plain model's best for its place up to the comparison's tolerance."""
    from ziglm_b200 import Engine, EngineOptions, GenerationOptions, SamplerParams
    # a larger spread of the weights separates the logits
    dtype = DTYPES[dn]
    folder = helpers.make_folder(tmp_path, helpers.CONFIGS[name], 29, dtype, helpers.NORM_JITTER[name], std=0.08)
    eng = Engine.load(folder, EngineOptions(dtype=dn, max_batch=8, max_tokens=2048))
    V = helpers.CONFIGS[name]["vocab_size"]
    prompts = [helpers.random_tokens(5 + 7 * i, V, 300 + i) for i in range(12)]
    limits = [3, 9, 14, 6, 21, 11, 17, 25, 4, 8, 13, 2]
    counts = {}

    def stop_at_limit(request, token):
        counts[request] = counts.get(request, 0) + 1
        return counts[request] < limits[request]

    opts = GenerationOptions(max_tokens=64, ignore_eos=True, sampler=SamplerParams(greedy=True))
    together, _ = eng.generate(prompts, opts, callback=stop_at_limit)
    assert [len(r.tokens) for r in together] == limits
    assert len(eng._graphs) >= 5                            # the batch went through at least five sizes
    eng.cache.slots.check()
    assert eng.cache.slots.slots.n_held == 0
    if dn == "float32":
        for i, p in enumerate(prompts):
            counts.clear()
            alone, _ = eng.generate([p], opts, callback=lambda r, t, i=i: stop_at_limit(i, t))
            assert alone[0].tokens == together[i].tokens, f"request {i}"
    else:
        tol = helpers.TOL[dtype]
        for i, p in enumerate(prompts):
            logits = helpers.plain_logits(folder, list(p) + together[i].tokens, act=dtype)
            for k, tok in enumerate(together[i].tokens):
                row = logits[len(p) - 1 + k]
                slack = 2 * (tol["atol"] + tol["rtol"] * row.max().abs().item())
                assert row[tok].item() >= row.max().item() - slack, f"request {i}, token {k}"
    # the captured steps of all batch sizes share one workspace: its size is that of the largest batch
    assert all(g.ws is eng.graph_ws for g in eng._graphs.values())
    assert eng.graph_ws.bytes() < 8 * 1024 * 1024, f"decode graphs hold {eng.graph_ws.bytes()} bytes of scratch"


@pytest.mark.parametrize("dn", ["float32", "bfloat16"])
def test_a_larger_batch_after_a_smaller_one_moves_the_shared_scratch_and_every_size_stays_right(zoo, dn):
    """Decode steps of one sequence are captured first; then four sequences decode together, which makes the
    shared scratch of the captured steps grow and move; then one sequence decodes again.  Its captured launches
    point to memory that is gone, so they are captured anew, and every step's logits match the plain model."""
    folder, eng = zoo.get("D", dn, max_batch=4, max_tokens=1024, seed=5)
    V = helpers.CONFIGS["D"]["vocab_size"]
    act = None if dn == "float32" else torch.bfloat16
    reqs = [helpers.random_tokens(40, V, 900 + i) for i in range(4)]
    want = [helpers.plain_logits(folder, r, act=act) for r in reqs]
    slots = [eng.alloc_slot() for _ in reqs]
    eng.step([(slots[0], reqs[0][:10])], [[]])
    rows0 = [eng.step([(slots[0], [reqs[0][k]])]).clone() for k in range(10, 14)]          # size 1 is captured
    first_graph = eng._graphs[1].graph
    moves = eng.graph_ws.moves
    eng.step([(s, r[:20]) for s, r in zip(slots[1:], reqs[1:])], [[], [], []])
    eng.step([(slots[0], reqs[0][14:20])], [[]])
    rows_all = [eng.step([(s, [r[k]]) for s, r in zip(slots, reqs)]).clone() for k in range(20, 26)]   # size 4
    assert eng.graph_ws.moves > moves
    rows0b = [eng.step([(slots[0], [reqs[0][k]])]).clone() for k in range(26, 32)]         # size 1 again
    assert eng._graphs[1].graph is not first_graph
    helpers.assert_close(torch.cat(rows0), want[0][10:14], DTYPES[dn], "one sequence, first capture")
    for i in range(4):
        helpers.assert_close(torch.stack([r[i] for r in rows_all]), want[i][20:26], DTYPES[dn], f"four sequences, {i}")
    helpers.assert_close(torch.cat(rows0b), want[0][26:32], DTYPES[dn], "one sequence, captured anew")
    for s in slots:
        eng.free_slot(s)


def test_wanted_places_and_nothing_wanted(zoo):
    folder, eng = zoo.get("A", "float32")
    toks = helpers.random_tokens(20, 256, 3)
    want = helpers.plain_logits(folder, toks)
    a, b = eng.alloc_slot(), eng.alloc_slot()
    got = eng.step([(a, toks[:12]), (b, toks[:7])], [[11, 0, 5], []]).clone()
    helpers.assert_close(got, want[[11, 0, 5]], torch.float32, "wanted places in the order asked")
    assert eng.step([(a, toks[12:15]), (b, toks[7:9])], [[], []]) is None
    got = eng.step([(b, toks[9:10]), (a, toks[15:16])]).clone()
    helpers.assert_close(got, want[[9, 15]], torch.float32, "default: the last token of each")
    eng.free_slot(a); eng.free_slot(b)


def test_step_refuses_bad_input(zoo):
    from ziglm_b200 import StepError
    from ziglm_b200.cache import CacheError, CacheFull, SequenceTooLong
    _, eng = zoo.get("A", "float32", max_batch=2, max_tokens=128)
    s = eng.alloc_slot()
    with pytest.raises(StepError, match="vocabulary"):
        eng.step([(s, [256])])
    with pytest.raises(StepError, match="at least one token"):
        eng.step([(s, [])])
    with pytest.raises(StepError, match="twice"):
        eng.step([(s, [1]), (s, [2])])
    with pytest.raises(StepError, match="outside"):
        eng.step([(s, [1, 2])], [[2]])
    with pytest.raises(CacheError):
        eng.step([(1, [1])])                                   # a slot nobody holds
    with pytest.raises(SequenceTooLong):
        eng.step([(s, [1] * 129)])
    t = eng.alloc_slot()
    eng.step([(s, [1] * 65)])
    with pytest.raises(CacheFull):
        eng.step([(t, [1] * 65)])                              # 2 pages each, the cache has 2
    assert eng.length(s) == 65 and eng.length(t) == 0
    eng.free_slot(s); eng.free_slot(t)
    eng.cache.slots.check()


def test_single_sequence_calls_of_the_reference(zoo):
    folder, eng = zoo.get("B", "float32")
    toks = helpers.random_tokens(10, 384, 8)
    want = helpers.plain_logits(folder, toks)
    eng.reset()
    l = eng.prefill(toks[:6]).clone()
    helpers.assert_close(l, want[5], torch.float32, "prefill")
    for pos in range(6, 10):
        l = eng.decode(toks[pos], pos).clone()
        helpers.assert_close(l, want[pos], torch.float32, f"decode at {pos}")
    from ziglm_b200 import StepError
    with pytest.raises(StepError, match="position"):
        eng.decode(1, 3)
    eng.reset()
    helpers.assert_close(eng.prefill(toks[:2]).clone(), want[1], torch.float32, "after reset")
    eng.reset()


@pytest.mark.parametrize("name", ["D", "E"])
def test_tensor_core_head_sizes_take_the_tensor_core_attention(zoo, name, monkeypatch):
    """With head size 64 or 128 in bfloat16 no step goes through the plain attention kernel, and a decode step
    needs no separate rotation kernel (the flat kernel rotates and writes the cache itself)."""
    from ziglm_b200 import kernels
    _, eng = zoo.get(name, "bfloat16")
    V = helpers.CONFIGS[name]["vocab_size"]

    def never(*a, **k):
        raise AssertionError("the plain attention kernel ran")
    monkeypatch.setattr(kernels, "attention_general", never)
    slot = eng.alloc_slot()
    eng.step([(slot, helpers.random_tokens(40, V, 5))])           # tcgen05 prompt kernel
    eng.step([(slot, helpers.random_tokens(3, V, 6))])            # mma.sync prompt kernel (fewer than 16 tokens)

    def no_rotation(*a, **k):
        raise AssertionError("a decode step launched the rotation kernel")
    monkeypatch.setattr(kernels, "rope_store", no_rotation)
    before = kernels.launches()
    eng.options.use_graphs = False
    try:
        eng.step([(slot, [7])])
    finally:
        eng.options.use_graphs = True
    eng.free_slot(slot)
    layers = helpers.CONFIGS[name]["num_hidden_layers"]
    # Once a step: embedding, the first norm, the last norm, the head.  Per layer: q|k|v, attention (with rotation and
    # cache write), o, gate|up with activation, down, and one norm kernel: at these narrow widths the o product is
    # too short to be split over a cluster, so the norm after it is a launch of its own, while the norm after
    # `down` rides on the products around it.  (At real widths both ride: tests/test_gpu_wide.py counts 5 a layer.)
    assert kernels.launches() - before == 6 * layers + 4
    assert kernels.attention_tc_status() == 0 and kernels.attention_fmha_status() == 0


def test_a_decode_step_taken_again_is_the_same_step(zoo):
    """When the same sequences bring one token each again, the engine reuses the packed integers of the step
    before (tokens and lengths change, and one table entry when a sequence starts a page): the logits are those
    of an engine that packs every step anew, over 150 steps that cross page boundaries at different times."""
    from ziglm_b200 import Engine, EngineOptions
    folder, eng = zoo.get("D", "bfloat16")
    plain = Engine.load(folder, EngineOptions(dtype="bfloat16", max_tokens=1024, max_batch=8, use_graphs=False))
    V = helpers.CONFIGS["D"]["vocab_size"]
    prompts = [helpers.random_tokens(n, V, 70 + n) for n in (3, 60, 41)]
    a = [eng.alloc_slot() for _ in prompts]
    b = [plain.alloc_slot() for _ in prompts]
    eng.step(list(zip(a, prompts)))
    plain.step(list(zip(b, prompts)))
    taken_again = 0
    for k in range(150):
        toks = helpers.random_tokens(3, V, 1000 + k)
        if eng._repeat is not None and eng._repeat.left > 0:
            taken_again += 1
        got = eng.step([(s, [t]) for s, t in zip(a, toks)]).clone()
        want = plain.step([(s, [t]) for s, t in zip(b, toks)]).clone()
        assert torch.equal(got, want), f"step {k}"
        assert [eng.length(s) for s in a] == [plain.length(s) for s in b]
    assert taken_again >= 148                        # every step after the first decode step
    for s in a:
        eng.free_slot(s)
    for s in b:
        plain.free_slot(s)
    eng.cache.slots.check()


@pytest.mark.parametrize("which", ["all", "norms"])
def test_tensors_stored_in_32_bit_stay_so_under_the_bfloat16_engine(tmp_path, which):
    """A folder whose tensors (all of them, or only the norms' gains) are stored in float32, run in bfloat16:
    those tensors are kept as they are stored, activations and the cache are bfloat16, and the logits are the
    plain model's with the same weights and activations rounded at the same places."""
    import json
    import os
    from safetensors.torch import save_file
    from ziglm_b200 import Engine, EngineOptions
    cfg = helpers.CONFIGS["D"]
    folder = helpers.make_folder(tmp_path, cfg, 41, torch.float32, 0.1)
    if which == "norms":
        _, tensors = helpers.read_folder(folder)
        mixed = {n: (t if "norm" in n else t.to(torch.bfloat16)) for n, t in tensors.items()}
        folder = os.path.join(str(tmp_path), "mixed")
        os.makedirs(folder)
        save_file(mixed, os.path.join(folder, "model.safetensors"))
        json.dump(cfg, open(os.path.join(folder, "config.json"), "w"))
    eng = Engine.load(folder, EngineOptions(dtype="bfloat16", max_tokens=512, max_batch=4))
    assert eng.model.final_norm.weight.dtype == torch.float32
    assert eng.model.embedding.dtype == (torch.float32 if which == "all" else torch.bfloat16)
    reqs = [helpers.random_tokens(n, cfg["vocab_size"], 60 + n) for n in (150, 7, 66)]
    want = [helpers.plain_logits(folder, r, act=torch.bfloat16) for r in reqs]
    slots = [eng.alloc_slot() for _ in reqs]
    cut = [len(r) - 4 for r in reqs]
    got = eng.step([(s, r[:k]) for s, r, k in zip(slots, reqs, cut)], [list(range(k)) for k in cut]).clone()
    helpers.assert_close(got, torch.cat([w[:k] for w, k in zip(want, cut)]), torch.bfloat16, f"{which}: prompts")
    for j in range(4):
        got = eng.step([(s, [r[k + j]]) for s, r, k in zip(slots, reqs, cut)]).clone()
        helpers.assert_close(got, torch.stack([w[k + j] for w, k in zip(want, cut)]), torch.bfloat16, f"{which}: token {j}")
