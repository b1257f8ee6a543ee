"""Each part of a layer alone (norm, rotary table, attention mixer, gated feed-forward, block), built from its
spec and run on a hand-made step, against the plain functions."""
import math

import pytest
import torch

import plain_llama as P
from test_gpu_kernels import rnd

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


class MiniStep:
    """The fields of a step that parts read, for one or more sequences, with a cache of its own."""

    def __init__(self, dtype, lens_past, lens_new, n_kv, hd, page=64):
        from ziglm_b200.engine.workspace import Workspace
        from ziglm_b200.parts import LayerIO
        self.dtype, self.device = dtype, DEV
        self.ws = Workspace(DEV)
        pos, seq, cu = [], [], [0]
        for b, (p, n) in enumerate(zip(lens_past, lens_new)):
            pos += list(range(p, p + n)); seq += [b] * n; cu.append(cu[-1] + n)
        self.n_tokens, self.n_seqs = len(pos), len(lens_new)
        self.positions = torch.tensor(pos, dtype=torch.int32, device=DEV)
        self.seq_of_token = torch.tensor(seq, dtype=torch.int32, device=DEV)
        self.cu_seqlens = torch.tensor(cu, dtype=torch.int32, device=DEV)
        self.past_lens = torch.tensor(lens_past, dtype=torch.int32, device=DEV)
        self.single_token = all(n == 1 for n in lens_new)
        self.max_new = max(lens_new)
        self.max_total = max(p + n for p, n in zip(lens_past, lens_new))
        pages_per = -(-self.max_total // page)
        table = torch.arange(self.n_seqs * pages_per, dtype=torch.int32).view(self.n_seqs, pages_per).flip(0)
        self.io = LayerIO(k_pages=torch.zeros(self.n_seqs * pages_per, n_kv, page, hd, dtype=dtype, device=DEV),
                          v_pages=torch.zeros(self.n_seqs * pages_per, n_kv, page, hd, dtype=dtype, device=DEV),
                          block_table=table.contiguous().to(DEV), page_size=page)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part(dtype):
    from ziglm_b200.config.spec import NormSpec
    from ziglm_b200.parts import norm_class
    spec = NormSpec("rmsnorm", 200, 1e-6)
    part = norm_class("rmsnorm")(spec, dtype, DEV)
    assert list(norm_class("rmsnorm").declare(spec)) == ["weight"]
    w = (1 + rnd((200,), torch.float32, 0.1, seed=1)).to(dtype)
    part.bind({"weight": w.to(DEV)})
    step = MiniStep(dtype, [0], [7], 1, 16)
    x = rnd((7, 200), torch.float32, 2.0, seed=2)
    out = part.forward(step, x.to(DEV))
    assert out.dtype == dtype
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert torch.allclose(out.float().cpu(), P.rms_norm(x, w, 1e-6), atol=tol, rtol=tol)
    unit = norm_class("rmsnorm")(NormSpec("rmsnorm", 200, 1e-6, {"unit_offset": True}), dtype, DEV)
    unit.bind({"weight": w.to(DEV)})
    assert torch.allclose(unit.forward(step, x.to(DEV)).float().cpu(), P.rms_norm(x, w.float() + 1, 1e-6), atol=tol, rtol=tol)


def test_rope_part_tables():
    from ziglm_b200.config.spec import PositionSpec
    from ziglm_b200.parts import position_class
    scaling = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
               "original_max_position_embeddings": 64}
    part = position_class("rope")(PositionSpec("rope", 32, 500000.0, scaling), torch.float32, DEV)
    table, rot = part.rotary_table()
    assert rot == 32 and torch.allclose(table.cpu(), P.rope_inverse_frequencies(32, 500000.0, scaling), rtol=2e-7, atol=0)
    assert position_class("none")(PositionSpec("none"), torch.float32, DEV).rotary_table() is None


def attention_case(dtype, nh, nkv, hd, d, bias, window, theta, scaling, lens_past, lens_new):
    from ziglm_b200.config.spec import MixerSpec, PositionSpec
    from ziglm_b200.parts import mixer_class
    spec = MixerSpec(kind="attention", width=d, n_heads=nh, n_kv_heads=nkv, head_dim=hd, bias=bias, out_bias=bias,
                     window=window, position=PositionSpec("rope", hd, theta, scaling))
    part = mixer_class("attention")(spec, dtype, DEV)
    decl = mixer_class("attention").declare(spec)
    w = {n: rnd(dcl.shape, dtype, 0.08, seed=10 + i) for i, (n, dcl) in enumerate(decl.items())}
    part.bind({n: t.to(DEV) for n, t in w.items()})
    return part, w


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,d,bias,window", [(4, 2, 16, 64, False, None), (4, 1, 32, 96, True, None),
                                                      (6, 3, 48, 120, False, 40), (8, 2, 64, 256, True, None),
                                                      (4, 4, 128, 64, False, 70)])
def test_attention_part_prompt_then_decode(dtype, nh, nkv, hd, d, bias, window):
    """The mixer on a prompt of two sequences, then on one more token each, against the plain functions over the
    whole sequences: projections, rotation, cache, attention, output projection, residual sum."""
    theta, scaling = 500000.0, {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                "original_max_position_embeddings": 64}
    lens = [70, 23]
    part, w = attention_case(dtype, nh, nkv, hd, d, bias, window, theta, scaling, [0, 0], lens)
    assert part.cache_needs().window == window and part.cache_needs().head_dim == hd and part.state_needs() is None
    act = None if dtype == torch.float32 else torch.bfloat16
    hs = [rnd((n + 1, d), dtype, 1.0, seed=50 + b) for b, n in enumerate(lens)]     # one extra row: the decoded token
    inv = P.rope_inverse_frequencies(hd, theta, scaling)

    def plain(h):
        T = h.shape[0]
        rd = (lambda t: t) if act is None else (lambda t: t.to(act).float())
        q = rd(P.linear(h.float(), w["q.weight"], w.get("q.bias")))
        k = rd(P.linear(h.float(), w["k.weight"], w.get("k.bias")))
        v = rd(P.linear(h.float(), w["v.weight"], w.get("v.bias")))
        q = rd(P.apply_rope(q.view(T, nh, hd), range(T), inv))
        k = rd(P.apply_rope(k.view(T, nkv, hd), range(T), inv))
        o = rd(P.attention(q, k, v.view(T, nkv, hd), 1 / math.sqrt(hd), window).reshape(T, nh * hd))
        return P.linear(o, w["o.weight"], w.get("o.bias"))

    want = [plain(h) for h in hs]
    tol = dict(atol=2e-5, rtol=1e-4) if dtype == torch.float32 else dict(atol=3e-2, rtol=3e-2)
    step = MiniStep(dtype, [0, 0], lens, nkv, hd)
    res = torch.ones(sum(lens), d, device=DEV)
    part.forward(step, step.io, torch.cat([h[:-1] for h in hs]).to(DEV), res)
    got = res.cpu() - 1.0
    assert torch.allclose(got[:lens[0]], want[0][:-1], **tol) and torch.allclose(got[lens[0]:], want[1][:-1], **tol)
    step2 = MiniStep(dtype, lens, [1, 1], nkv, hd)
    step2.io = step.io                                                      # the same cache, one token further
    res2 = torch.zeros(2, d, device=DEV)
    part.forward(step2, step2.io, torch.stack([hs[0][-1], hs[1][-1]]).to(DEV), res2)
    assert torch.allclose(res2.cpu()[0], want[0][-1], **tol) and torch.allclose(res2.cpu()[1], want[1][-1], **tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("d,inter,act_name,bias", [(64, 176, "silu", False), (120, 200, "gelu_tanh", False),
                                                   (256, 1000, "silu", False), (192, 328, "silu", True),
                                                   (120, 200, "gelu_tanh", True)])
def test_gated_mlp_part(dtype, d, inter, act_name, bias):
    from ziglm_b200.config.spec import FeedForwardSpec
    from ziglm_b200.parts import feed_forward_class
    spec = FeedForwardSpec("gated_mlp", d, inter, activation=act_name, bias=bias)
    part = feed_forward_class("gated_mlp")(spec, dtype, DEV)
    w = {n: rnd(dcl.shape, dtype, 0.08, seed=20 + i) for i, (n, dcl) in enumerate(feed_forward_class("gated_mlp").declare(spec).items())}
    part.bind({n: t.to(DEV) for n, t in w.items()})
    for T in (1, 9, 150):
        h = rnd((T, d), dtype, 1.0, seed=30 + T)
        res = torch.ones(T, d, device=DEV)
        part.forward(MiniStep(dtype, [0], [T], 1, 16), h.to(DEV), res)
        g = P.linear(h.float(), w["gate.weight"], w.get("gate.bias"))
        u = P.linear(h.float(), w["up.weight"], w.get("up.bias"))
        a = (P.silu(g) if act_name == "silu" else torch.nn.functional.gelu(g, approximate="tanh")) * u
        if dtype == torch.bfloat16:
            a = a.to(dtype).float()
        want = 1.0 + P.linear(a, w["down.weight"], w.get("down.bias"))
        tol = dict(atol=2e-5, rtol=1e-4) if dtype == torch.float32 else dict(atol=3e-2, rtol=3e-2)
        assert torch.allclose(res.cpu(), want, **tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_prenorm_block_equals_the_plain_layer(dtype, tmp_path):
    """One block built from the layer spec of tiny B and bound to the tensors of a model folder."""
    import helpers
    from ziglm_b200.config import config_from_dict
    from ziglm_b200.parts import block_class
    cfg = helpers.TINY_B
    spec = config_from_dict(cfg).model_spec()
    layer = spec.layers[1]
    folder = helpers.make_folder(tmp_path, cfg, 3, dtype, 0.1)
    raw_cfg, w = helpers.read_folder(folder)
    block = block_class(layer.block)(layer, dtype, DEV)
    block.bind({local: w[layer.prefix + layer.names.get(local, local)].to(DEV)
                for local in block_class(layer.block).declare(layer)})
    T = 37
    x = rnd((T, cfg["hidden_size"]), torch.float32, 0.5, seed=5)
    step = MiniStep(dtype, [0], [T], cfg["num_key_value_heads"], cfg["head_dim"])
    xd = x.to(DEV).clone()
    block.forward(step, step.io, xd)
    inv = P.rope_inverse_frequencies(cfg["head_dim"], cfg["rope_theta"], cfg["rope_scaling"])
    want = P.decoder_layer(raw_cfg, w, 1, x, list(range(T)), inv, None if dtype == torch.float32 else dtype)
    tol = dict(atol=2e-5, rtol=1e-4) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    assert torch.allclose(xd.cpu(), want, **tol)
