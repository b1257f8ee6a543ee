"""Typed configuration of the Llama-style dense decoder, read from config.json.

Keys and defaults follow what the reference reads in ``parseHFConfig``
(src/safetensors.zig:482-596) and ``ModelParams.initComputed``
(src/types.zig:246-285): hidden_size, intermediate_size, num_attention_heads,
num_key_value_heads (default: num_attention_heads), num_hidden_layers,
vocab_size, rms_norm_eps (default 1e-5), rope_theta (default 10000),
max_position_embeddings (default 2048), head_dim (default hidden/heads).
The reference parses rope_theta but never uses it and knows no rope_scaling,
attention_bias, tie_word_embeddings or eos ids; those are read here because the
architecture's own config.json carries them.

Nothing is inferred from tensor shapes (the reference overwrites its parameters
from shapes, src/safetensors.zig:181-252); shapes are checked against this
configuration by the weight loader instead.
"""
from __future__ import annotations

from dataclasses import dataclass, asdict
from typing import Any, Dict, Mapping, Optional, Tuple

from .common import (ConfigError, architecture_name, need_bool, need_float, need_floats, need_int, read_config_json,
                     token_ids)
from .spec import (FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec,
                   PositionSpec)


_REFUSED_SCALINGS = {
    "dynamic": "its frequencies depend on the length of the running sequence, so keys already in the cache "
               "would have been rotated with another table than the queries that read them",
    "longrope": "it switches between two tables of factors by the length of the running sequence, so keys already "
                "in the cache would have been rotated with another table than the queries that read them",
}


@dataclass(frozen=True)
class RopeScaling:
    """``rope_scaling`` of config.json: how the table of rotary frequencies is stretched for long contexts.

    ``rope_type`` (older files: ``type``) selects the rule; every rule is a transform of the table, applied
    once when the model is built (the formulas are in ``ziglm_b200/parts/rope.py``):
      "linear"  every frequency is divided by ``factor``;
      "llama3"  low frequencies are divided by ``factor``, high ones stay, those between are blended;
                needs ``low_freq_factor``, ``high_freq_factor``, ``original_max_position_embeddings``;
      "yarn"    frequencies below a band are divided by ``factor``, those above stay, with a linear ramp over
                the band given by ``beta_fast`` (32) and ``beta_slow`` (1) rotations over
                ``original_max_position_embeddings`` (default: max_position_embeddings); queries and keys are
                scaled by ``attention_factor`` (default 0.1 ln(factor) + 1).
    Rules whose table changes with the length of the running sequence ("dynamic", "longrope") are refused.
    The reference knows no rope_scaling at all (src/safetensors.zig:548-591 never reads the key).
    """
    rope_type: str
    factor: float
    low_freq_factor: Optional[float] = None
    high_freq_factor: Optional[float] = None
    original_max_position_embeddings: Optional[int] = None
    beta_fast: Optional[float] = None
    beta_slow: Optional[float] = None
    attention_factor: Optional[float] = None
    truncate: Optional[bool] = None

    @classmethod
    def from_dict(cls, d: Optional[Mapping[str, Any]], max_positions: Optional[int] = None) -> Optional["RopeScaling"]:
        if d is None:
            return None
        if not isinstance(d, Mapping):
            raise ConfigError(f"config.json: 'rope_scaling' must be an object or null, found {d!r}")
        kind = d.get("rope_type", d.get("type"))
        if kind in (None, "default"):
            return None
        if kind in _REFUSED_SCALINGS:
            raise ConfigError(f"config.json: rope_scaling of type {kind!r} is not supported: {_REFUSED_SCALINGS[kind]}")
        if kind == "linear":
            s = cls(rope_type="linear", factor=need_float(d, "factor"))
        elif kind == "llama3":
            s = cls(
                rope_type="llama3",
                factor=need_float(d, "factor"),
                low_freq_factor=need_float(d, "low_freq_factor"),
                high_freq_factor=need_float(d, "high_freq_factor"),
                original_max_position_embeddings=need_int(d, "original_max_position_embeddings"),
            )
            if s.high_freq_factor <= s.low_freq_factor:
                raise ConfigError("config.json: rope_scaling.high_freq_factor must exceed low_freq_factor")
        elif kind == "yarn":
            for key in ("mscale", "mscale_all_dim"):
                if d.get(key) is not None:
                    raise ConfigError(f"config.json: rope_scaling.{key} (a variant of yarn for another architecture) "
                                      "is not supported")
            s = cls(
                rope_type="yarn",
                factor=need_float(d, "factor"),
                original_max_position_embeddings=need_int(d, "original_max_position_embeddings", default=max_positions),
                beta_fast=need_float(d, "beta_fast", default=32.0),
                beta_slow=need_float(d, "beta_slow", default=1.0),
                attention_factor=need_float(d, "attention_factor") if d.get("attention_factor") is not None else None,
                truncate=need_bool(d, "truncate", True),
            )
            if s.beta_fast <= s.beta_slow:
                raise ConfigError("config.json: rope_scaling.beta_fast must exceed beta_slow")
        else:
            raise ConfigError(f"config.json: rope_scaling of type {kind!r} is not known "
                              "(default, linear, llama3, yarn)")
        if s.factor < 1.0:
            raise ConfigError(f"config.json: rope_scaling.factor must be at least 1, found {s.factor}")
        return s

    def to_dict(self) -> Dict[str, Any]:
        return {k: v for k, v in asdict(self).items() if v is not None}


@dataclass(frozen=True)
class LlamaConfig:
    architecture: str
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    rope_scaling: Optional[RopeScaling] = None
    partial_rotary_factor: float = 1.0       # the first head_dim * factor elements of a head are rotated (src/model.zig:571-572)
    max_position_embeddings: int = 2048
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    mlp_bias: bool = False
    hidden_act: str = "silu"
    sliding_window: Optional[int] = None     # position p sees [p - window + 1, p] in every layer (src/model.zig:660-661)
    bos_token_id: Optional[int] = None
    eos_token_ids: Tuple[int, ...] = ()

    ARCHITECTURE = "LlamaForCausalLM"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "LlamaConfig":
        if not isinstance(d, Mapping):
            raise ConfigError("config.json must hold a JSON object")
        arch = architecture_name(d)
        hidden = need_int(d, "hidden_size")
        heads = need_int(d, "num_attention_heads")
        kv_heads = need_int(d, "num_key_value_heads", default=heads)
        if d.get("head_dim") is None:
            if hidden % heads:
                raise ConfigError(
                    f"config.json: hidden_size {hidden} is not a multiple of num_attention_heads {heads} "
                    "and no head_dim is given")
            head_dim = hidden // heads
        else:
            head_dim = need_int(d, "head_dim")
        if heads % kv_heads:
            raise ConfigError(
                f"config.json: num_attention_heads {heads} is not a multiple of num_key_value_heads {kv_heads}")
        if head_dim % 2:
            raise ConfigError(f"config.json: head_dim {head_dim} must be even for rotary positions")
        # Newer files keep theta and the stretching rule together under "rope_parameters"; it wins over the two
        # separate keys.
        rope = d.get("rope_parameters")
        scaling_src = d.get("rope_scaling")
        theta_src: Mapping[str, Any] = d
        partial_src: Mapping[str, Any] = d
        if rope is not None:
            if not isinstance(rope, Mapping):
                raise ConfigError(f"config.json: 'rope_parameters' must be an object, found {rope!r}")
            if rope.get("rope_theta") is not None:
                theta_src = rope
            if rope.get("partial_rotary_factor") is not None:
                partial_src = rope
            scaling_src = {k: v for k, v in rope.items() if k not in ("rope_theta", "partial_rotary_factor")} or None
        partial = need_float(partial_src, "partial_rotary_factor", default=1.0)
        rotary = int(head_dim * partial)
        if partial > 1.0 or rotary < 2 or rotary % 2:
            raise ConfigError(f"config.json: partial_rotary_factor {partial} of head_dim {head_dim} gives {rotary} "
                              "rotated elements; an even number from 2 to head_dim is needed")
        act = d.get("hidden_act", "silu")
        if act in ("silu", "swish"):
            act = "silu"
        elif act in ("gelu_pytorch_tanh", "gelu_tanh"):
            act = "gelu_pytorch_tanh"                    # the tanh form (src/math.zig:1119-1123)
        else:
            raise ConfigError(f"config.json: hidden_act {act!r} is not supported by this architecture "
                              "(silu, gelu_pytorch_tanh)")
        window = d.get("sliding_window")
        if window is not None:
            window = need_int(d, "sliding_window")
        bos = d.get("bos_token_id")
        if bos is not None and (isinstance(bos, bool) or not isinstance(bos, int)):
            raise ConfigError(f"config.json: 'bos_token_id' must be an integer, found {bos!r}")
        cfg = cls(
            architecture=arch,
            hidden_size=hidden,
            intermediate_size=need_int(d, "intermediate_size"),
            num_hidden_layers=need_int(d, "num_hidden_layers"),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            vocab_size=need_int(d, "vocab_size"),
            rms_norm_eps=need_float(d, "rms_norm_eps", default=1e-5),
            rope_theta=need_float(theta_src, "rope_theta", default=10000.0),
            rope_scaling=RopeScaling.from_dict(scaling_src, need_int(d, "max_position_embeddings", default=2048)),
            partial_rotary_factor=partial,
            max_position_embeddings=need_int(d, "max_position_embeddings", default=2048),
            tie_word_embeddings=need_bool(d, "tie_word_embeddings", False),
            attention_bias=need_bool(d, "attention_bias", False),
            mlp_bias=need_bool(d, "mlp_bias", False),
            hidden_act=act,
            sliding_window=window,
            bos_token_id=bos,
            eos_token_ids=token_ids(d, "eos_token_id"),
        )
        return cfg

    @classmethod
    def from_folder(cls, folder: str) -> "LlamaConfig":
        return cls.from_dict(read_config_json(folder))

    def to_dict(self) -> Dict[str, Any]:
        """The config.json that reads back as this configuration."""
        d: Dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": "llama",
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "vocab_size": self.vocab_size,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": self.rope_scaling.to_dict() if self.rope_scaling else None,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "attention_bias": self.attention_bias,
            "mlp_bias": self.mlp_bias,
            "hidden_act": self.hidden_act,
        }
        if self.partial_rotary_factor != 1.0:
            d["partial_rotary_factor"] = self.partial_rotary_factor
        if self.sliding_window is not None:
            d["sliding_window"] = self.sliding_window
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        return d

    @property
    def rotary_dim(self) -> int:
        return int(self.head_dim * self.partial_rotary_factor)

    # ----------------------------------------------------------- model structure
    def model_spec(self) -> ModelSpec:
        """Lay the architecture out as parts: L identical pre-norm blocks of
        (RMSNorm, rotary grouped-query attention, RMSNorm, SwiGLU), run in order
        (src/model.zig:543-789 is the reference's layer loop)."""
        d = self.hidden_size
        scaling = self.rope_scaling.to_dict() if self.rope_scaling else None
        position = PositionSpec(kind="rope", rotary_dim=self.rotary_dim, theta=self.rope_theta,
                                scaling=scaling, max_positions=self.max_position_embeddings)
        layers = []
        for i in range(self.num_hidden_layers):
            layers.append(LayerSpec(
                block="prenorm",
                prefix=f"model.layers.{i}.",
                mixer_norm=NormSpec("rmsnorm", d, self.rms_norm_eps),
                mixer=MixerSpec(kind="attention", width=d, n_heads=self.num_attention_heads,
                                n_kv_heads=self.num_key_value_heads, head_dim=self.head_dim,
                                bias=self.attention_bias, out_bias=self.attention_bias,
                                position=position, window=self.sliding_window),
                ffn_norm=NormSpec("rmsnorm", d, self.rms_norm_eps),
                ffn=FeedForwardSpec(kind="gated_mlp", width=d, intermediate=self.intermediate_size,
                                    activation="silu" if self.hidden_act == "silu" else "gelu_tanh",
                                    bias=self.mlp_bias),
                names={
                    "mixer_norm.weight": "input_layernorm.weight",
                    "mixer.q.weight": "self_attn.q_proj.weight",
                    "mixer.k.weight": "self_attn.k_proj.weight",
                    "mixer.v.weight": "self_attn.v_proj.weight",
                    "mixer.o.weight": "self_attn.o_proj.weight",
                    "mixer.q.bias": "self_attn.q_proj.bias",
                    "mixer.k.bias": "self_attn.k_proj.bias",
                    "mixer.v.bias": "self_attn.v_proj.bias",
                    "mixer.o.bias": "self_attn.o_proj.bias",
                    "ffn_norm.weight": "post_attention_layernorm.weight",
                    "ffn.gate.weight": "mlp.gate_proj.weight",
                    "ffn.up.weight": "mlp.up_proj.weight",
                    "ffn.down.weight": "mlp.down_proj.weight",
                    "ffn.gate.bias": "mlp.gate_proj.bias",
                    "ffn.up.bias": "mlp.up_proj.bias",
                    "ffn.down.bias": "mlp.down_proj.bias",
                },
            ))
        return ModelSpec(
            architecture=self.architecture,
            width=d,
            vocab_size=self.vocab_size,
            layers=tuple(layers),
            schedule=tuple(range(self.num_hidden_layers)),
            final_norm=NormSpec("rmsnorm", d, self.rms_norm_eps),
            embedding_name="model.embed_tokens.weight",
            final_norm_name="model.norm.weight",
            head_name=None if self.tie_word_embeddings else "lm_head.weight",
            embedding_scale=1.0,
            max_positions=self.max_position_embeddings,
            stop_token_ids=self.eos_token_ids,
        )

    # ------------------------------------------------------------------ counting
    def parameter_count(self) -> int:
        d, i, v = self.hidden_size, self.intermediate_size, self.vocab_size
        q = self.num_attention_heads * self.head_dim
        kv = self.num_key_value_heads * self.head_dim
        per_layer = d * q + 2 * d * kv + q * d + 3 * d * i + 2 * d
        if self.attention_bias:
            per_layer += q + 2 * kv + d
        if self.mlp_bias:
            per_layer += 2 * i + d
        total = self.num_hidden_layers * per_layer + v * d + d
        if not self.tie_word_embeddings:
            total += v * d
        return total

