"""A mixer that lives in this test only, with fixed-size state of its own per sequence, is registered, built
into a model beside an attention layer, loaded from a random folder and stepped (whole, token by token, in
unequal batches with slots used again) without any change to the library's files.  Another toy replaces the
position encoding, a third one the feed-forward (with a router), and a schedule runs a layer twice."""
import json
import math
import os
from dataclasses import dataclass
from typing import Dict

import pytest
import torch

import helpers
import plain_llama as P

pytestmark = pytest.mark.gpu


# ------------------------------------------------------------- the toy parts
def make_toy_parts():
    from ziglm_b200.parts import KVNeed, ParamDecl, Part, StateNeed

    class DecayMixer(Part):
        """state <- decay * state + W x_t ; output = state.  One vector of state per sequence, no keys."""

        def __init__(self, spec, dtype, device):
            super().__init__(spec, dtype, device)
            self.decay = float(spec.options["decay"])
            self.w = None

        @classmethod
        def declare(cls, spec):
            return {"w.weight": ParamDecl((spec.width, spec.width))}

        def bind(self, tensors):
            self.w = tensors["w.weight"]

        def cache_needs(self):
            return None

        def state_needs(self):
            return StateNeed((self.spec.width,), torch.float32)

        def forward(self, step, io, h, residual):
            start = 0
            proj = h.float() @ self.w.float().t()
            for b, n in enumerate(step.host_new_lens):
                idx = step.slots[b:b + 1].long()
                s = io.state.index_select(0, idx)
                for t in range(start, start + n):
                    s = self.decay * s + proj[t:t + 1]
                    residual[t:t + 1] += s
                io.state.index_copy_(0, idx, s)
                start += n

    class ShiftPosition(Part):
        """A position encoding that is no rotation: adds position * slope to the first element of every q and k head."""

        def rotary_table(self):
            return None

        def apply(self, step, qkv, n_heads, n_kv_heads, head_dim):
            slope = float(self.spec.options["slope"])
            heads = qkv.view(qkv.shape[0], -1, head_dim)[:, :n_heads + n_kv_heads]
            heads[:, :, 0] += (step.positions.float() * slope).to(qkv.dtype)[:, None]

    class RoutedFFN(Part):
        """Two small experts and a router: each token goes through the expert with the larger router logit
        (router logits in float32), scaled by the softmax weight of that expert."""

        def __init__(self, spec, dtype, device):
            super().__init__(spec, dtype, device)
            self.t = None

        @classmethod
        def declare(cls, spec):
            d, i = spec.width, spec.intermediate
            return {"router.weight": ParamDecl((2, d)), "e0.up.weight": ParamDecl((i, d)), "e0.down.weight": ParamDecl((d, i)),
                    "e1.up.weight": ParamDecl((i, d)), "e1.down.weight": ParamDecl((d, i))}

        def bind(self, tensors):
            self.t = tensors

        def forward(self, step, h, residual):
            x = h.float()
            logits = x @ self.t["router.weight"].float().t()
            prob = torch.softmax(logits, -1)
            pick = logits.argmax(-1)
            for e in (0, 1):
                y = torch.relu(x @ self.t[f"e{e}.up.weight"].float().t()) @ self.t[f"e{e}.down.weight"].float().t()
                residual += torch.where((pick == e)[:, None], y * prob[:, e:e + 1], torch.zeros_like(y))

    return DecayMixer, ShiftPosition, RoutedFFN


@dataclass(frozen=True)
class ToyConfig:
    raw: tuple

    @classmethod
    def from_dict(cls, d):
        return cls(tuple(sorted((k, json.dumps(v)) for k, v in d.items())))

    def to_dict(self):
        return {k: json.loads(v) for k, v in self.raw}

    def model_spec(self):
        from ziglm_b200.config.spec import (FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec)
        c = self.to_dict()
        d = c["hidden_size"]
        norm = NormSpec("rmsnorm", d, 1e-5)
        att = MixerSpec(kind="attention", width=d, n_heads=4, n_kv_heads=2, head_dim=16,
                        position=PositionSpec(kind="toy_shift", options={"slope": 0.01}))
        layers = (
            LayerSpec("prenorm", "toy.l0.", norm, att, norm, FeedForwardSpec("gated_mlp", d, 48)),
            LayerSpec("prenorm", "toy.l1.", norm, MixerSpec(kind="toy_decay", width=d, options={"decay": 0.5}), norm,
                      FeedForwardSpec("toy_routed", d, 24)),
        )
        return ModelSpec(architecture="ToyForCausalLM", width=d, vocab_size=c["vocab_size"], layers=layers,
                         schedule=tuple(c["schedule"]), final_norm=norm, embedding_name="toy.embed.weight",
                         final_norm_name="toy.norm.weight", head_name=None, max_positions=256)


@pytest.fixture(scope="module")
def toy(tmp_path_factory):
    from ziglm_b200 import register_architecture
    from ziglm_b200.config import unregister_architecture
    from ziglm_b200.parts import register_feed_forward, register_mixer, register_position, unregister
    Decay, Shift, Routed = make_toy_parts()
    register_mixer("toy_decay", Decay)
    register_position("toy_shift", Shift)
    register_feed_forward("toy_routed", Routed)
    register_architecture("ToyForCausalLM", ToyConfig)
    yield tmp_path_factory.mktemp("toy")
    unregister("mixer", "toy_decay"); unregister("position", "toy_shift"); unregister("feed_forward", "toy_routed")
    unregister_architecture("ToyForCausalLM")


def plain_toy(cfg: dict, w: Dict[str, torch.Tensor], tokens):
    """The toy model over one whole sequence, written out with the plain functions."""
    d, T = cfg["hidden_size"], len(tokens)
    x = P.embedding(tokens, w["toy.embed.weight"])
    for li in cfg["schedule"]:
        p = f"toy.l{li}."
        h = P.rms_norm(x, w[p + "mixer_norm.weight"], 1e-5)
        if li == 0:
            q = P.linear(h, w[p + "mixer.q.weight"]).view(T, 4, 16).clone()
            k = P.linear(h, w[p + "mixer.k.weight"]).view(T, 2, 16).clone()
            v = P.linear(h, w[p + "mixer.v.weight"]).view(T, 2, 16)
            pos = torch.arange(T, dtype=torch.float32) * 0.01
            q[:, :, 0] += pos[:, None]; k[:, :, 0] += pos[:, None]
            x = x + P.linear(P.attention(q, k, v, 0.25).reshape(T, 64), w[p + "mixer.o.weight"])
        else:
            s = torch.zeros(d)
            proj = P.linear(h, w[p + "mixer.w.weight"])
            out = []
            for t in range(T):
                s = 0.5 * s + proj[t]
                out.append(s)
            x = x + torch.stack(out)
        h = P.rms_norm(x, w[p + "ffn_norm.weight"], 1e-5)
        if li == 0:
            x = x + P.swiglu(h, w[p + "ffn.gate.weight"], w[p + "ffn.up.weight"], w[p + "ffn.down.weight"], None)
        else:
            logits = P.linear(h, w[p + "ffn.router.weight"])
            prob = torch.softmax(logits, -1)
            y = torch.zeros_like(x)
            for t in range(T):
                e = int(logits[t].argmax())
                y[t] = P.linear(torch.relu(P.linear(h[t:t + 1], w[p + f"ffn.e{e}.up.weight"])), w[p + f"ffn.e{e}.down.weight"])[0] * prob[t, e]
            x = x + y
    return P.linear(P.rms_norm(x, w["toy.norm.weight"], 1e-5), w["toy.embed.weight"])


@pytest.mark.parametrize("schedule", [[0, 1], [1, 0, 1]])
def test_toy_model_is_built_loaded_and_stepped(toy, schedule):
    from ziglm_b200 import Engine, EngineOptions, config_from_dict, write_random_model
    cfg = {"architectures": ["ToyForCausalLM"], "hidden_size": 64, "vocab_size": 97, "schedule": schedule}
    folder = os.path.join(str(toy), "m" + "".join(map(str, schedule)))
    write_random_model(folder, config_from_dict(cfg), 3, dtype=torch.float32, std=0.1)
    raw, w = helpers.read_folder(folder)
    eng = Engine.load(folder, EngineOptions(dtype="float32", max_tokens=512, max_batch=3, max_seq_len=256))
    # the toy mixer keeps state per sequence and no keys; a layer run twice keeps state (and keys) per place
    assert len(eng.cache.states) == schedule.count(1)
    assert sum(len(g.places) for g in eng.cache.groups) == schedule.count(0)
    reqs = [helpers.random_tokens(n, 97, 300 + n) for n in (9, 70, 3, 30)]
    want = [plain_toy(raw, w, r) for r in reqs]
    for r, wl in zip(reqs, want):                                    # whole
        s = eng.alloc_slot()
        helpers.assert_close(eng.step([(s, r)], [list(range(len(r)))]).clone(), wl, torch.float32, "toy whole")
        eng.free_slot(s)
    for r, wl in zip(reqs, want):                                    # token by token: the state carries over steps
        s = eng.alloc_slot()
        rows = [eng.step([(s, [t])]).clone() for t in r]
        eng.free_slot(s)
        helpers.assert_close(torch.cat(rows), wl, torch.float32, "toy one by one")
    # unequal batches, batch after batch: a slot used again starts from zero state
    from test_gpu_model import run_batches
    got = run_batches(eng, reqs, [[0, 1, 2], [3]], [4, 33, 1, 10])
    for i, wl in enumerate(want):
        helpers.assert_close(got[i], wl, torch.float32, f"toy batched, request {i}")
    eng.cache.slots.check()


def test_unknown_parts_and_layers_read_before_written_are_refused(toy):
    from ziglm_b200.config.spec import (FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec)
    from ziglm_b200.engine.model import Model, declare_parameters
    norm = NormSpec("rmsnorm", 8, 1e-5)
    bad = ModelSpec("X", 8, 5, (LayerSpec("prenorm", "l.", norm, MixerSpec(kind="no_such_mixer", width=8), norm,
                                          FeedForwardSpec("gated_mlp", 8, 8)),), (0,), norm, "e", "n", None)
    with pytest.raises(KeyError, match="no_such_mixer"):
        declare_parameters(bad)
    with pytest.raises(ValueError, match="schedule"):
        ModelSpec("X", 8, 5, (), (0,), norm, "e", "n", None)
    shares = MixerSpec(kind="attention", width=8, n_heads=1, n_kv_heads=1, head_dim=8, cache_from=1)
    spec = ModelSpec("X", 8, 5, (LayerSpec("prenorm", "a.", norm, shares, norm, FeedForwardSpec("gated_mlp", 8, 8)),
                                 LayerSpec("prenorm", "b.", norm, MixerSpec(kind="attention", width=8, n_heads=1, n_kv_heads=1, head_dim=8),
                                           norm, FeedForwardSpec("gated_mlp", 8, 8))), (0, 1), norm, "e", "n", None)
    with pytest.raises(ValueError, match="has not run before"):
        Model(spec, torch.float32, torch.device("cuda:0")).cache_plan()


def test_a_layer_may_read_another_layers_cache(toy, tmp_path):
    """Two attention layers, the second without keys and values of its own (``cache_from``)."""
    from ziglm_b200.config.spec import (FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec)
    from ziglm_b200.engine.engine import Engine, EngineOptions
    from ziglm_b200.engine.model import Model, declare_parameters
    from ziglm_b200.weights import random_tensors
    d = 32
    norm = NormSpec("rmsnorm", d, 1e-5)
    pos = PositionSpec("rope", 16, 10000.0)
    own = MixerSpec(kind="attention", width=d, n_heads=2, n_kv_heads=1, head_dim=16, position=pos)
    shared = MixerSpec(kind="attention", width=d, n_heads=2, n_kv_heads=1, head_dim=16, position=pos, cache_from=0)
    spec = ModelSpec("Shared", d, 50, (LayerSpec("prenorm", "l0.", norm, own, norm, FeedForwardSpec("gated_mlp", d, 40)),
                                       LayerSpec("prenorm", "l1.", norm, shared, norm, FeedForwardSpec("gated_mlp", d, 40))),
                     (0, 1), norm, "embed", "norm", None, max_positions=128)
    decl = declare_parameters(spec)
    assert "l1.mixer.k.weight" not in decl and "l1.mixer.q.weight" in decl
    dev = torch.device("cuda:0")
    w = dict(random_tensors(decl, 1, torch.float32, dev, std=0.1))
    model = Model(spec, torch.float32, dev)
    model.bind(w)
    eng = Engine(None, model, EngineOptions(dtype="float32", max_tokens=256, max_batch=2, max_seq_len=128))
    assert sum(len(g.places) for g in eng.cache.groups) == 1
    toks = helpers.random_tokens(40, 50, 2)
    w = {k: v.cpu() for k, v in w.items()}
    inv = P.rope_inverse_frequencies(16, 10000.0, None)
    x = P.embedding(toks, w["embed"])
    T = len(toks)
    k0 = v0 = None
    for li in (0, 1):
        p = f"l{li}."
        h = P.rms_norm(x, w[p + "mixer_norm.weight"], 1e-5)
        q = P.apply_rope(P.linear(h, w[p + "mixer.q.weight"]).view(T, 2, 16), range(T), inv)
        if li == 0:
            k0 = P.apply_rope(P.linear(h, w[p + "mixer.k.weight"]).view(T, 1, 16), range(T), inv)
            v0 = P.linear(h, w[p + "mixer.v.weight"]).view(T, 1, 16)
        x = x + P.linear(P.attention(q, k0, v0, 0.25).reshape(T, 32), w[p + "mixer.o.weight"])
        h = P.rms_norm(x, w[p + "ffn_norm.weight"], 1e-5)
        x = x + P.swiglu(h, w[p + "ffn.gate.weight"], w[p + "ffn.up.weight"], w[p + "ffn.down.weight"], None)
    want = P.linear(P.rms_norm(x, w["norm"], 1e-5), w["embed"])
    s = eng.alloc_slot()
    rows = [eng.step([(s, toks[:25])], [list(range(25))]).clone()] + [eng.step([(s, [t])]).clone() for t in toks[25:]]
    helpers.assert_close(torch.cat(rows), want, torch.float32, "shared cache")


def test_an_arrangement_with_options_and_hooks_behind_the_embedding_and_the_head(toy):
    """A block kind that lives in this test reads a further norm from ``LayerSpec.options`` and applies it after
    the mixer (a post-norm); a hook adds learned absolute positions to the embedded tokens and another one a
    bias and a soft cap to the logits.  All three are registered from here; no file of the library changes."""
    from ziglm_b200.config.spec import (FeedForwardSpec, HookSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec)
    from ziglm_b200.engine.engine import Engine, EngineOptions
    from ziglm_b200.engine.model import Model, declare_parameters
    from ziglm_b200.parts import (ParamDecl, Part, block_class, norm_class, register_block, register_hook, unregister)
    from ziglm_b200.weights import random_tensors
    PreNorm = block_class("prenorm")

    class PostNormBlock(PreNorm):
        """x += post(mixer(norm(x))); x += ffn(norm(x)): the mixer's output goes through a norm of its own."""

        def __init__(self, spec, dtype, device):
            super().__init__(spec, dtype, device)
            post = spec.options["post_mixer_norm"]
            self.post = norm_class(post.kind)(post, dtype, device)
            self.gain = float(spec.options["mixer_gain"])

        @classmethod
        def declare(cls, spec):
            out = dict(super().declare(spec))
            post = spec.options["post_mixer_norm"]
            for name, decl in norm_class(post.kind).declare(post).items():
                out["post_mixer_norm." + name] = decl
            return out

        def bind(self, tensors):
            super().bind(tensors)
            self.post.bind({k[len("post_mixer_norm."):]: v for k, v in tensors.items() if k.startswith("post_mixer_norm.")})

        def accepts_normed_input(self):
            return False

        def forward(self, step, io, x, h_in=None, next_norm=None):
            h = self.mixer_norm.forward(step, x)
            branch = torch.zeros_like(x)
            self.mixer.forward(step, io, h, branch)
            x += self.post.forward(step, branch, name="post_out").float() * self.gain
            self.ffn.forward(step, self.ffn_norm.forward(step, x), x)
            return None

    class LearnedPositions(Part):
        @classmethod
        def declare(cls, spec):
            return {"table": ParamDecl((spec.options["max_positions"], spec.options["width"]))}

        def bind(self, tensors):
            self.table = tensors["table"]

        def forward(self, step, x):
            x += self.table.float().index_select(0, step.positions.long())

    class BiasAndCap(Part):
        @classmethod
        def declare(cls, spec):
            return {"bias": ParamDecl((spec.options["vocab_size"],))}

        def bind(self, tensors):
            self.bias = tensors["bias"]

        def forward(self, step, logits):
            cap = float(self.spec.options["cap"])
            logits.copy_(torch.tanh((logits + self.bias.float()) / cap) * cap)

    register_block("toy_postnorm", PostNormBlock)
    register_hook("toy_learned_positions", LearnedPositions)
    register_hook("toy_bias_and_cap", BiasAndCap)
    try:
        d, V = 32, 61
        norm = NormSpec("rmsnorm", d, 1e-5)
        att = MixerSpec(kind="attention", width=d, n_heads=2, n_kv_heads=1, head_dim=16)
        layer = LayerSpec("toy_postnorm", "l0.", norm, att, norm, FeedForwardSpec("gated_mlp", d, 40),
                          options={"post_mixer_norm": NormSpec("rmsnorm", d, 1e-6), "mixer_gain": 0.5})
        spec = ModelSpec("Hooked", d, V, (layer,), (0,), norm, "embed", "norm", "head", max_positions=128,
                         embed_hook=HookSpec("toy_learned_positions", {"max_positions": 128, "width": d}, {"table": "positions.table"}),
                         logits_hook=HookSpec("toy_bias_and_cap", {"vocab_size": V, "cap": 2.0}, {"bias": "head.bias"}))
        decl = declare_parameters(spec)
        assert {"positions.table", "head.bias", "l0.post_mixer_norm.weight"} <= set(decl)
        dev = torch.device("cuda:0")
        w = dict(random_tensors(decl, 4, torch.float32, dev, std=0.2, norm_jitter=0.1))
        model = Model(spec, torch.float32, dev)
        model.bind(w)
        eng = Engine(None, model, EngineOptions(dtype="float32", max_tokens=256, max_batch=2, max_seq_len=128))
        toks = helpers.random_tokens(30, V, 6)
        T = len(toks)
        w = {k: v.cpu() for k, v in w.items()}
        x = P.embedding(toks, w["embed"]) + w["positions.table"][:T]
        h = P.rms_norm(x, w["l0.mixer_norm.weight"], 1e-5)
        q = P.linear(h, w["l0.mixer.q.weight"]).view(T, 2, 16)
        k = P.linear(h, w["l0.mixer.k.weight"]).view(T, 1, 16)
        v = P.linear(h, w["l0.mixer.v.weight"]).view(T, 1, 16)
        branch = P.linear(P.attention(q, k, v, 0.25).reshape(T, 32), w["l0.mixer.o.weight"])
        x = x + 0.5 * P.rms_norm(branch, w["l0.post_mixer_norm.weight"], 1e-6)
        h = P.rms_norm(x, w["l0.ffn_norm.weight"], 1e-5)
        x = x + P.swiglu(h, w["l0.ffn.gate.weight"], w["l0.ffn.up.weight"], w["l0.ffn.down.weight"], None)
        want = torch.tanh((P.linear(P.rms_norm(x, w["norm"], 1e-5), w["head"]) + w["head.bias"]) / 2.0) * 2.0
        s = eng.alloc_slot()
        rows = [eng.step([(s, toks[:11])], [list(range(11))]).clone()] + [eng.step([(s, [t])]).clone() for t in toks[11:]]
        helpers.assert_close(torch.cat(rows), want, torch.float32, "post-norm block with hooks")
    finally:
        unregister("block", "toy_postnorm"); unregister("hook", "toy_learned_positions"); unregister("hook", "toy_bias_and_cap")
