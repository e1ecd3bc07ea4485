"""Typed configurations of the Llama and Qwen2 dense decoders, read from config.json.

Keys and their meanings follow the reference's two parsers: the strict one
(v3/crates/rvllm-core/src/config/model.rs:51-161, helpers config/hf.rs:9-86) and the
lenient one the Llama path runs on (v3/crates/rvllm-loader/src/load.rs:80-238).  Every
problem of a file is collected and reported in one `ConfigError`.  No size or constant
that config.json carries is repeated in code: the parts receive them as parameters
through the `ModelSpec` that `to_spec()` builds.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, asdict
from typing import Any, Dict, List, Optional, Tuple

from ..errors import ConfigError
from .spec import LayerSpec, ModelSpec, PartSpec, default_run_order


class _Reader:
    """Typed access to a JSON object that remembers every problem instead of raising."""

    def __init__(self, obj: Dict[str, Any]):
        self.obj = obj
        self.problems: List[str] = []

    def _get(self, key, types, default, required, what):
        if key not in self.obj or self.obj[key] is None:
            if required:
                self.problems.append(f"missing key `{key}` ({what})")
            return default
        v = self.obj[key]
        if isinstance(v, bool) and bool not in (types if isinstance(types, tuple) else (types,)):
            self.problems.append(f"`{key}` must be {what}, got {v!r}")
            return default
        if not isinstance(v, types):
            self.problems.append(f"`{key}` must be {what}, got {type(v).__name__} {v!r}")
            return default
        return v

    def integer(self, key, default=None, required=False, minimum=None):
        v = self._get(key, int, default, required, "an integer")
        if v is not None and minimum is not None and v < minimum:
            self.problems.append(f"`{key}` must be >= {minimum}, got {v}")
        return v

    def number(self, key, default=None, required=False, positive=False):
        v = self._get(key, (int, float), default, required, "a number")
        if v is not None:
            v = float(v)
            if positive and not v > 0:
                self.problems.append(f"`{key}` must be > 0, got {v}")
        return v

    def boolean(self, key, default=None):
        return self._get(key, bool, default, False, "true or false")

    def string(self, key, default=None, required=False):
        return self._get(key, str, default, required, "a string")


@dataclass(frozen=True)
class RopeScaling:
    """`rope_scaling` of the llama3 kind; the reference never reads this key."""
    rope_type: str
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int

    @staticmethod
    def parse(obj: Any, problems: List[str]) -> Optional["RopeScaling"]:
        if obj is None:
            return None
        if not isinstance(obj, dict):
            problems.append(f"`rope_scaling` must be an object or null, got {obj!r}")
            return None
        kind = obj.get("rope_type", obj.get("type", "default"))
        if kind == "default":
            return None
        if kind != "llama3":
            problems.append(f"`rope_scaling.rope_type` = {kind!r} is not supported (known: default, llama3)")
            return None
        r = _Reader(obj)
        out = RopeScaling(
            rope_type="llama3",
            factor=r.number("factor", required=True, positive=True) or 1.0,
            low_freq_factor=r.number("low_freq_factor", required=True, positive=True) or 1.0,
            high_freq_factor=r.number("high_freq_factor", required=True, positive=True) or 2.0,
            original_max_position_embeddings=r.integer("original_max_position_embeddings", required=True, minimum=1) or 1,
        )
        problems.extend(f"rope_scaling: {p}" for p in r.problems)
        if not r.problems and out.high_freq_factor <= out.low_freq_factor:
            problems.append("rope_scaling: `high_freq_factor` must be larger than `low_freq_factor`")
        return out

    def to_dict(self):
        return asdict(self)


@dataclass(frozen=True)
class DenseDecoderConfig:
    """What the Llama and Qwen2 configurations have in common."""
    architecture: str
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    rope_scaling: Optional[RopeScaling]
    attention_bias: bool                       # bias on q, k and v (Llama: on o as well; never on the MLP)
    tie_word_embeddings: bool
    hidden_act: str
    layer_windows: Tuple[Optional[int], ...]   # per layer: None = all keys, W = the last W keys
    torch_dtype: str = "bfloat16"
    eos_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    raw: Dict[str, Any] = field(default_factory=dict, compare=False, repr=False)

    ARCHITECTURE = ""              # set by subclasses
    BIAS_DEFAULT = False           # default of `attention_bias`
    OUT_BIAS_FOLLOWS = False       # whether `attention_bias` also puts a bias on the output projection

    # ---- reading -----------------------------------------------------------------------
    @classmethod
    def from_dict(cls, obj: Dict[str, Any], where: str = "config.json") -> "DenseDecoderConfig":
        r = _Reader(obj)
        p = r.problems
        H = r.integer("hidden_size", required=True, minimum=1)
        L = r.integer("num_hidden_layers", required=True, minimum=1)
        nh = r.integer("num_attention_heads", required=True, minimum=1)
        nkv = r.integer("num_key_value_heads", default=nh, minimum=1)
        hd = r.integer("head_dim", minimum=2)
        inter = r.integer("intermediate_size", required=True, minimum=1)
        V = r.integer("vocab_size", required=True, minimum=1)
        max_pos = r.integer("max_position_embeddings", required=True, minimum=1)
        eps = r.number("rms_norm_eps", required=True, positive=True)
        theta = r.number("rope_theta", default=10000.0, positive=True)
        scaling = RopeScaling.parse(obj.get("rope_scaling"), p)
        tie = r.boolean("tie_word_embeddings", default=False)
        act = r.string("hidden_act", default=None) or r.string("hidden_activation", default="silu")
        dtype = r.string("torch_dtype", default=None) or r.string("dtype", default="bfloat16")

        if hd is None and H and nh:
            if H % nh:
                p.append(f"`hidden_size` {H} is not a multiple of `num_attention_heads` {nh} and `head_dim` is absent")
            hd = H // nh
        if hd is not None and hd % 2:
            p.append(f"`head_dim` must be even for rotary pairs, got {hd}")
        if nh and nkv and nh % nkv:
            p.append(f"`num_attention_heads` {nh} is not a multiple of `num_key_value_heads` {nkv}")
        if act != "silu":
            p.append(f"`hidden_act` = {act!r} is not supported by this architecture's gated MLP (known: silu)")
        if dtype not in ("bfloat16", "float16", "float32"):
            p.append(f"`torch_dtype` = {dtype!r} is not supported (known: bfloat16, float16, float32)")

        bias = cls._read_bias(r)
        if r.boolean("mlp_bias", default=False):
            p.append("`mlp_bias` = true is not supported: the gated MLP of this engine has no bias")
        windows = cls._read_windows(r, obj, L or 0)
        eos = obj.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids = (eos,)
        elif isinstance(eos, list) and all(isinstance(e, int) for e in eos):
            eos_ids = tuple(eos)
        else:
            p.append(f"`eos_token_id` must be an integer or a list of integers, got {eos!r}")
            eos_ids = ()
        bos = r.integer("bos_token_id", default=None)

        if p:
            raise ConfigError(p, where)
        return cls(architecture=cls.ARCHITECTURE, hidden_size=H, num_hidden_layers=L,
                   num_attention_heads=nh, num_key_value_heads=nkv, head_dim=hd,
                   intermediate_size=inter, vocab_size=V, max_position_embeddings=max_pos,
                   rms_norm_eps=eps, rope_theta=theta, rope_scaling=scaling, attention_bias=bias,
                   tie_word_embeddings=tie, hidden_act=act, layer_windows=windows,
                   torch_dtype=dtype, eos_token_ids=eos_ids, bos_token_id=bos, raw=dict(obj))

    @classmethod
    def _read_bias(cls, r: _Reader) -> bool:
        return bool(r.boolean("attention_bias", default=cls.BIAS_DEFAULT))

    @classmethod
    def _read_windows(cls, r: _Reader, obj, L: int) -> Tuple[Optional[int], ...]:
        """Llama: no window; a `sliding_window` or non-full `layer_types` is refused."""
        if obj.get("sliding_window") is not None:
            r.problems.append("`sliding_window` is not part of this architecture")
        types = obj.get("layer_types")
        if types is not None and any(t != "full_attention" for t in types):
            r.problems.append("`layer_types` other than full_attention are not part of this architecture")
        return tuple([None] * L)

    # ---- writing -----------------------------------------------------------------------
    def to_dict(self) -> Dict[str, Any]:
        """The config.json that reads back as this configuration."""
        d: Dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": self.architecture.replace("ForCausalLM", "").lower(),
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": self.rope_scaling.to_dict() if self.rope_scaling else None,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": self.hidden_act,
            "torch_dtype": self.torch_dtype,
        }
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        self._write_extra(d)
        return d

    def _write_extra(self, d: Dict[str, Any]) -> None:
        d["attention_bias"] = self.attention_bias

    # ---- the model this configuration describes --------------------------------------------
    def to_spec(self) -> ModelSpec:
        """Layer by layer: pre-norm block, paged attention with rotary positions, SiLU-gated MLP.

        Order of operations: v3/crates/rvllm-runtime/src/layer_exec.rs:162-529.
        The softmax scale 1/sqrt(head_dim) is fixed for this architecture
        (v3/crates/rvllm-runtime/src/bring_up.rs:502).
        """
        norm = PartSpec("rmsnorm", {"size": self.hidden_size, "eps": self.rms_norm_eps})
        layers = []
        for i in range(self.num_hidden_layers):
            mixer = PartSpec("paged_attention", {
                "hidden_size": self.hidden_size,
                "num_heads": self.num_attention_heads,
                "num_kv_heads": self.num_key_value_heads,
                "head_dim": self.head_dim,
                "qkv_bias": self.attention_bias,
                "out_bias": self.attention_bias and self.OUT_BIAS_FOLLOWS,
                "scale": self.head_dim ** -0.5,
                "window": self.layer_windows[i],
                "position": "rope",
            })
            ffn = PartSpec("gated_mlp", {
                "hidden_size": self.hidden_size,
                "intermediate_size": self.intermediate_size,
                "activation": self.hidden_act,
            })
            layers.append(LayerSpec.standard(
                prefix=f"model.layers.{i}.", block=PartSpec("prenorm_residual"),
                mixer=mixer, feed_forward=ffn, mixer_norm=norm, feed_forward_norm=norm,
                names={"mixer": "self_attn.", "feed_forward": "mlp.",
                       "mixer_norm": "input_layernorm.", "feed_forward_norm": "post_attention_layernorm."}))
        rope = PartSpec("rotary", {
            "head_dim": self.head_dim, "theta": self.rope_theta,
            "scaling": self.rope_scaling.to_dict() if self.rope_scaling else None,
        })
        return ModelSpec(
            architecture=self.architecture, hidden_size=self.hidden_size, vocab_size=self.vocab_size,
            max_position_embeddings=self.max_position_embeddings,
            embedding_name="model.embed_tokens.weight", layers=tuple(layers),
            run_order=default_run_order(self.num_hidden_layers),
            final_norm=norm, final_norm_prefix="model.norm.",
            lm_head_name=None if self.tie_word_embeddings else "lm_head.weight",
            position_encodings={"rope": rope},
            ignored_tensors=("*.rotary_emb.inv_freq",),
            eos_token_ids=self.eos_token_ids)


@dataclass(frozen=True)
class LlamaConfig(DenseDecoderConfig):
    """`LlamaForCausalLM`: no bias unless `attention_bias`, which then puts one on q, k, v and o
    (the checkpoints of this architecture that have biases carry `o_proj.bias` too); no window."""
    ARCHITECTURE = "LlamaForCausalLM"
    BIAS_DEFAULT = False
    OUT_BIAS_FOLLOWS = True


@dataclass(frozen=True)
class Qwen2Config(DenseDecoderConfig):
    """`Qwen2ForCausalLM`: q, k and v always carry a bias; layers may use a sliding window.

    Window keys: `use_sliding_window` switches it on, `sliding_window` is the number of keys a
    query sees (itself included), and either `layer_types` names the kind of each layer or the
    layers from `max_window_layers` upward get the window.  The reference parses
    `layer_types` and `sliding_window` (v3/crates/rvllm-loader/src/load.rs:122-135,179-182)
    and its attention kernels take the window as `window_size_left` = W - 1
    (v3/kernels/paged_attention_sm89.cu:300-308).
    """
    ARCHITECTURE = "Qwen2ForCausalLM"
    BIAS_DEFAULT = True

    @classmethod
    def _read_bias(cls, r: _Reader) -> bool:
        b = r.boolean("attention_bias", default=True)
        if b is False:
            r.problems.append("`attention_bias` = false contradicts Qwen2ForCausalLM, whose q, k and v always have a bias")
        return True

    @classmethod
    def _read_windows(cls, r: _Reader, obj, L: int) -> Tuple[Optional[int], ...]:
        use = bool(r.boolean("use_sliding_window", default=False))
        w = r.integer("sliding_window", default=None, minimum=1)
        start = r.integer("max_window_layers", default=L, minimum=0)
        types = obj.get("layer_types")
        if not use:
            if types is not None and any(t != "full_attention" for t in types):
                r.problems.append("`layer_types` names sliding_attention layers but `use_sliding_window` is false")
            return tuple([None] * L)
        if w is None:
            r.problems.append("`use_sliding_window` is true but `sliding_window` is absent")
            return tuple([None] * L)
        if types is None:
            types = ["sliding_attention" if i >= start else "full_attention" for i in range(L)]
        if not isinstance(types, list) or len(types) != L:
            r.problems.append(f"`layer_types` must list {L} layers, got {types!r}")
            return tuple([None] * L)
        out = []
        for i, t in enumerate(types):
            if t == "full_attention":
                out.append(None)
            elif t == "sliding_attention":
                out.append(w)
            else:
                r.problems.append(f"`layer_types[{i}]` = {t!r} is not supported (known: full_attention, sliding_attention)")
                out.append(None)
        return tuple(out)

    def _write_extra(self, d: Dict[str, Any]) -> None:
        windows = [w for w in self.layer_windows if w is not None]
        d["use_sliding_window"] = bool(windows)
        if windows:
            d["sliding_window"] = windows[0]
            d["layer_types"] = ["sliding_attention" if w is not None else "full_attention"
                                for w in self.layer_windows]


def read_config_json(model_dir: str) -> Dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path) as f:
            obj = json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"no config.json in {model_dir}") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"config.json is not valid JSON: {e}", path) from None
    if not isinstance(obj, dict):
        raise ConfigError("config.json must hold a JSON object", path)
    return obj
