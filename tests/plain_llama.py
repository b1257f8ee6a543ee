"""A plain, slow implementation of the Llama-style decoder for the tests to compare against.

Whole sequences, no cache, one function per part, PyTorch on the CPU.  It shares
no code with ``ziglm_b200``: it reads the raw config.json dictionary and the
tensors under their names in the weight file.  Every function is written from the
formulas of the reference's CPU forward pass (src/model.zig, src/math.zig,
src/sampler.zig); the reference's host code is Zig and cannot be compiled or
imported here (no Zig toolchain, no network), so this file rests on the formulas,
each cited below.  Where the reference deviates from the architecture (it
ignores rope_theta, applies a 512-token window and binds post_attention_layernorm
twice; src/model.zig:405-413, src/safetensors.zig:415-425) the architecture's
own definition is followed and the deviation is named.

``act`` is the type activations are rounded to where the engine stores them in
that type (None: nothing is rounded).  With ``act=torch.bfloat16`` the plain
model rounds at the same places as the engine's bfloat16 path, so the comparison
tolerance can stay tight.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch


def _round(t: torch.Tensor, act: Optional[torch.dtype]) -> torch.Tensor:
    return t if act is None else t.to(act).to(torch.float32)


# ----------------------------------------------------------------------- parts
def embedding(tokens: Sequence[int], table: torch.Tensor) -> torch.Tensor:
    """x = W_e[token] widened to float32, no scaling for this architecture (src/model.zig:495-503)."""
    rows = []
    for t in tokens:
        if not 0 <= t < table.shape[0]:
            raise IndexError(f"token {t} out of bounds")          # error.TokenOutOfBounds, src/model.zig:495
        rows.append(table[t].to(torch.float32))
    return torch.stack(rows)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """ss = sum x_i^2; inv = 1/sqrt(ss/n + eps); y_i = (x_i*inv)*w_i (src/math.zig:850-945)."""
    out = torch.empty_like(x)
    w = weight.to(torch.float32)
    for r in range(x.shape[0]):
        row = x[r]
        ss = (row * row).sum()
        inv = 1.0 / torch.sqrt(ss / row.numel() + eps)
        out[r] = (row * inv) * w
    return out


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y[r] = sum_c W[r,c] x[c] with float32 accumulation over widened weights (src/math.zig:121-176,730-758)."""
    y = x @ weight.to(torch.float32).t()
    if bias is not None:
        y = y + bias.to(torch.float32)
    return y


def rope_inverse_frequencies(rot: int, theta: float, scaling: Optional[dict], max_positions: int = 0) -> torch.Tensor:
    """f_i = theta^(-2i/rot) (the reference: exp(-(2i/rot) ln base), src/model.zig:569-597), then the rule of the
    architecture's rope_scaling (the reference has none), one frequency at a time:
    linear: f / factor.
    llama3: wavelength l = 2 pi / f; l < L0/high: keep; l > L0/low: f/factor; else s = (L0/l - low)/(high - low),
            f <- (1-s) f/factor + s f.
    yarn:   the pair that makes r rotations over L0 positions is d(r) = rot ln(L0/(2 pi r)) / (2 ln theta); between
            lo = floor d(beta_fast) and hi = ceil d(beta_slow) (inside [0, rot-1]) the weight g rises from 0 to 1;
            f <- (1-g) f + g f/factor."""
    kind = None if scaling is None else scaling.get("rope_type", scaling.get("type"))
    out = []
    for i in range(rot // 2):
        f = theta ** (-(2.0 * i) / rot)
        if kind == "linear":
            f = f / float(scaling["factor"])
        elif kind == "llama3":
            factor = float(scaling["factor"])
            low = float(scaling["low_freq_factor"])
            high = float(scaling["high_freq_factor"])
            orig = float(scaling["original_max_position_embeddings"])
            wavelen = 2.0 * math.pi / f
            if wavelen < orig / high:
                pass
            elif wavelen > orig / low:
                f = f / factor
            else:
                s = (orig / wavelen - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        elif kind == "yarn":
            factor = float(scaling["factor"])
            orig = float(scaling.get("original_max_position_embeddings") or max_positions)
            lo = rot * math.log(orig / (float(scaling.get("beta_fast", 32.0)) * 2.0 * math.pi)) / (2.0 * math.log(theta))
            hi = rot * math.log(orig / (float(scaling.get("beta_slow", 1.0)) * 2.0 * math.pi)) / (2.0 * math.log(theta))
            if scaling.get("truncate", True):
                lo, hi = math.floor(lo), math.ceil(hi)
            lo, hi = max(lo, 0), min(hi, rot - 1)
            if lo == hi:
                hi += 0.001
            g = min(1.0, max(0.0, (i - lo) / (hi - lo)))
            f = (1.0 - g) * f + g * f / factor
        elif kind not in (None, "default"):
            raise ValueError(f"rope scaling {kind!r}")
        out.append(f)
    return torch.tensor(out, dtype=torch.float64).to(torch.float32)


def rope_score_factor(scaling: Optional[dict]) -> float:
    """yarn multiplies rotated queries and keys by m = attention_factor (default 0.1 ln(factor) + 1), so a score
    grows by m * m; every other rule leaves them alone."""
    if scaling is None or scaling.get("rope_type", scaling.get("type")) != "yarn":
        return 1.0
    m = scaling.get("attention_factor")
    if m is None:
        factor = float(scaling["factor"])
        m = 0.1 * math.log(factor) + 1.0 if factor > 1.0 else 1.0
    return float(m) * float(m)


def apply_rope(x: torch.Tensor, positions: Sequence[int], inv_freq: torch.Tensor) -> torch.Tensor:
    """x: [T, heads, hd].  Pairs (i, i+rot/2): a' = a cos - b sin, b' = a sin + b cos, theta = pos * f_i in
    float32 (src/model.zig:569-597,642-653; src/cuda_bridge.cu:2070-2108)."""
    T, H, hd = x.shape
    half = inv_freq.numel()
    out = x.clone()
    for t in range(T):
        theta = torch.tensor(float(positions[t]), dtype=torch.float32) * inv_freq        # float32 product
        c, s = torch.cos(theta), torch.sin(theta)
        a, b = x[t, :, :half], x[t, :, half:2 * half]
        out[t, :, :half] = a * c - b * s
        out[t, :, half:2 * half] = a * s + b * c
    return out


def attention_row(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                  window: Optional[int] = None) -> torch.Tensor:
    """One token: q [nh, hd] at position p = len(k)-1 over keys k, v [p+1, nkv, hd].  kvh = h // (nh/nkv);
    s_t = (q . k_t) * scale over t in [start, p]; softmax with max subtraction; o = sum p_t v_t
    (src/model.zig:554,659-700; softmax src/math.zig:1088-1106)."""
    nh, hd = q.shape
    nkv = k.shape[1]
    group = nh // nkv
    p = k.shape[0] - 1
    start = 0 if window is None else max(0, p - window + 1)
    out = torch.zeros(nh, hd, dtype=torch.float32)
    for h in range(nh):
        kvh = h // group
        s = (k[start:p + 1, kvh] @ q[h]) * scale
        e = torch.exp(s - s.max())
        prob = e / e.sum()
        out[h] = prob @ v[start:p + 1, kvh]
    return out


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
              window: Optional[int] = None) -> torch.Tensor:
    """q: [T, nh, hd]; k, v: [T, nkv, hd], all of one sequence in order: every token over the keys up to itself."""
    return torch.stack([attention_row(q[p], k[:p + 1], v[:p + 1], scale, window) for p in range(q.shape[0])])


def silu(z: torch.Tensor) -> torch.Tensor:
    """silu(z) = z / (1 + exp(-z)) (src/math.zig:1108-1111)."""
    return z / (1.0 + torch.exp(-z))


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    """0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))) (src/math.zig:1119-1123)."""
    return 0.5 * z * (1.0 + torch.tanh(0.7978845608028654 * (z + 0.044715 * z * z * z)))


def swiglu(x: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor,
           act: Optional[torch.dtype], gate_bias: Optional[torch.Tensor] = None,
           up_bias: Optional[torch.Tensor] = None, down_bias: Optional[torch.Tensor] = None,
           hidden_act: str = "silu") -> torch.Tensor:
    """f = W_d (silu(W_g x) * (W_u x)) (src/model.zig:725-745, src/math.zig:1112-1117), or with the tanh form of
    gelu in silu's place where config.json's hidden_act says so (src/math.zig:1125-1130); the architecture's
    mlp_bias adds a bias to each of the three products (the reference has none)."""
    g = _round(linear(x, gate, gate_bias), act)
    u = _round(linear(x, up, up_bias), act)
    gated = silu(g) if hidden_act in ("silu", "swish") else gelu_tanh(g)
    a = _round(gated * u, act)
    return linear(a, down, down_bias)


# ----------------------------------------------------------------------- model
def head_dim_of(cfg: dict) -> int:
    return cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]


def decoder_layer(cfg: dict, w: Dict[str, torch.Tensor], i: int, x: torch.Tensor, positions: Sequence[int],
                  inv_freq: torch.Tensor, act: Optional[torch.dtype]) -> torch.Tensor:
    """norm, q/k/v, rope, attention, output projection, residual; norm, SwiGLU, residual
    (src/model.zig:545-755).  post_attention_layernorm is the norm before the feed-forward."""
    p = f"model.layers.{i}."
    nh, nkv, hd = cfg["num_attention_heads"], cfg.get("num_key_value_heads") or cfg["num_attention_heads"], head_dim_of(cfg)
    eps = cfg.get("rms_norm_eps", 1e-5)
    bias = cfg.get("attention_bias", False)
    T = x.shape[0]
    h = _round(rms_norm(x, w[p + "input_layernorm.weight"], eps), act)
    q = _round(linear(h, w[p + "self_attn.q_proj.weight"], w.get(p + "self_attn.q_proj.bias") if bias else None), act)
    k = _round(linear(h, w[p + "self_attn.k_proj.weight"], w.get(p + "self_attn.k_proj.bias") if bias else None), act)
    v = _round(linear(h, w[p + "self_attn.v_proj.weight"], w.get(p + "self_attn.v_proj.bias") if bias else None), act)
    q = _round(apply_rope(q.view(T, nh, hd), positions, inv_freq), act)
    k = _round(apply_rope(k.view(T, nkv, hd), positions, inv_freq), act)
    scale = (1.0 / math.sqrt(hd)) * rope_score_factor(cfg.get("rope_scaling"))
    o = attention(q, k, v.view(T, nkv, hd), scale, cfg.get("sliding_window"))
    o = _round(o.reshape(T, nh * hd), act)
    x = x + linear(o, w[p + "self_attn.o_proj.weight"], w.get(p + "self_attn.o_proj.bias") if bias else None)
    h = _round(rms_norm(x, w[p + "post_attention_layernorm.weight"], eps), act)
    mb = cfg.get("mlp_bias", False)
    x = x + swiglu(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"], act,
                   w[p + "mlp.gate_proj.bias"] if mb else None, w[p + "mlp.up_proj.bias"] if mb else None,
                   w[p + "mlp.down_proj.bias"] if mb else None, cfg.get("hidden_act", "silu"))
    return x


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int],
            act: Optional[torch.dtype] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence: embedding, layers, final norm, head (tied to the embedding when
    there is no lm_head) (src/model.zig:495-503,543-802)."""
    hd = head_dim_of(cfg)
    rot = int(hd * float(cfg.get("partial_rotary_factor", 1.0)))    # the rotated part of a head (src/model.zig:571-572)
    inv_freq = rope_inverse_frequencies(rot, float(cfg.get("rope_theta", 10000.0)), cfg.get("rope_scaling"),
                                        cfg.get("max_position_embeddings", 2048))
    positions = list(range(len(tokens)))
    x = embedding(tokens, w["model.embed_tokens.weight"])
    for i in range(cfg["num_hidden_layers"]):
        x = decoder_layer(cfg, w, i, x, positions, inv_freq, act)
    h = _round(rms_norm(x, w["model.norm.weight"], cfg.get("rms_norm_eps", 1e-5)), act)
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return linear(h, head)


# -------------------------------------------------------------------- sampling
def greedy(logits: torch.Tensor) -> int:
    """The largest logit, lowest id on ties.  (The reference's CPU argmax skips id 0 and its GPU argmax does
    not, src/sampler.zig:159-170 vs src/cuda_bridge.cu:2955-2964; all ids are scanned here.)"""
    best, idx = None, 0
    for i, v in enumerate(logits.tolist()):
        if best is None or v > best:
            best, idx = v, i
    return idx


def apply_penalties(logits: torch.Tensor, history: Sequence[int], repetition: float, presence: float,
                    window: int) -> torch.Tensor:
    """For every occurrence of a token in the last ``window`` ids: positive logit / penalty, negative * penalty,
    then minus presence (src/sampler.zig:54-76)."""
    out = logits.clone()
    if repetition == 1.0 and presence == 0.0:
        return out
    for tok in list(history)[-window:] if window > 0 else []:
        if tok < out.numel():
            out[tok] = out[tok] / repetition if out[tok] > 0 else out[tok] * repetition
            out[tok] = out[tok] - presence
    return out


def sample(logits: torch.Tensor, u: float, temperature: float, top_k: int, top_p: float, min_p: float) -> int:
    """The reference's order (src/sampler.zig:78-157): logits/T, softmax, sort by probability (descending; ties by
    lower id), keep k, cut below min_p * p_max (keeping at least one), cut after the cumulative probability reaches
    top_p, then draw r = u * sum(kept) and take the first kept candidate whose running sum is >= r.  With no top_k
    the candidates stay in id order (the draw's distribution is the same); top_p then keeps the same set as the
    sorted chain would (the shortest prefix by descending probability, ties by lower id, whose probability
    reaches top_p; the running probability is summed exactly, in units of 2^-44)."""
    z = logits.to(torch.float32) * torch.tensor(1.0 / temperature, dtype=torch.float32)
    e = torch.exp(z - z.max())
    prob = e / e.sum()
    ids = list(range(prob.numel()))
    if top_k > 0:
        ids.sort(key=lambda i: (-prob[i].item(), i))
        if top_k < len(ids):
            ids = ids[:top_k]
        if min_p > 0.0:
            thresh = prob[ids[0]] * torch.tensor(min_p, dtype=torch.float32)
            for n, i in enumerate(ids):
                if prob[i] < thresh:
                    ids = ids[:max(1, n)]
                    break
        if top_p < 1.0:
            cum = torch.tensor(0.0, dtype=torch.float32)
            for n, i in enumerate(ids):
                cum = cum + prob[i]
                if cum >= top_p:
                    ids = ids[:n + 1]
                    break
    else:
        if min_p > 0.0:
            thresh = prob.max() * torch.tensor(min_p, dtype=torch.float32)
            ids = [i for i in ids if prob[i] >= thresh]
        if top_p < 1.0:
            unit = float(2 ** 44)
            want = int(float(torch.tensor(top_p, dtype=torch.float32)) * unit)
            cum, kept = 0, set()
            for i in sorted(ids, key=lambda i: (-prob[i].item(), i)):
                kept.add(i)
                cum += int(float(prob[i]) * unit)
                if cum >= want:
                    break
            ids = [i for i in ids if i in kept]
    total = torch.tensor(0.0, dtype=torch.float32)
    for i in ids:
        total = total + prob[i]
    r = torch.tensor(u, dtype=torch.float32) * total
    run = torch.tensor(0.0, dtype=torch.float32)
    for i in ids:
        run = run + prob[i]
        if r <= run:
            return i
    return ids[0]
