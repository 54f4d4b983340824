"""Typed configuration of the Qwen3 dense decoder, read from its config.json keys.

Keys and meanings follow crates/synaptix-models/llm/qwen3/src/config.rs:5-49
(field list) and :63-87 (validation).  Differences, all on the side of failing
loudly instead of guessing:

* sizes have no built-in defaults (the reference falls back to Qwen3-1.7B
  numbers, config.rs:28-49); a missing size is an error;
* ``head_dim`` absent means ``hidden_size // num_attention_heads`` (the
  reference's silent 128, config.rs:37, is wrong for small models);
* ``attention_bias: true`` and a non-default ``rope_scaling`` are errors (the
  reference parses and ignores the former, config.rs:20,42);
* ``tie_word_embeddings`` absent is resolved when weights are bound: tied if
  the weights hold no ``lm_head.weight``;
* ``use_sliding_window: true`` (or ``layer_types`` naming sliding layers) gives
  those layers a window; the reference forces full attention
  (config.rs:117-118), which is the same thing for every released Qwen3 model
  because they all ship ``use_sliding_window: false``.
"""
from __future__ import annotations

import dataclasses
from typing import Any, ClassVar, Dict, Optional, Tuple

from .base import ConfigError, ModelConfig, take


@dataclasses.dataclass(frozen=True)
class Qwen3Config(ModelConfig):
    architectures: ClassVar[Tuple[str, ...]] = ("Qwen3ForCausalLM",)
    model_types: ClassVar[Tuple[str, ...]] = ("qwen3",)

    vocab_size: int = 0
    hidden_size: int = 0
    intermediate_size: int = 0
    num_hidden_layers: int = 0
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    rms_norm_eps: float = 0.0
    rope_theta: float = 0.0
    hidden_act: str = "silu"
    max_position_embeddings: Optional[int] = None
    tie_word_embeddings: Optional[bool] = None
    attention_bias: bool = False
    bos_token_id: Optional[int] = None
    eos_token_ids: Tuple[int, ...] = ()
    # one entry per layer: None = all earlier keys, n = the last n keys
    layer_windows: Tuple[Optional[int], ...] = ()
    # carried through so that a written config.json round-trips
    sliding_window: Optional[int] = None
    use_sliding_window: bool = False
    max_window_layers: Optional[int] = None

    # ---- derived sizes -------------------------------------------------
    @property
    def group_size(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    # ---- reading -------------------------------------------------------
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "Qwen3Config":
        hidden = take(d, "hidden_size", int)
        heads = take(d, "num_attention_heads", int)
        layers = take(d, "num_hidden_layers", int)
        if heads <= 0:
            raise ConfigError("config.json: num_attention_heads must be > 0")
        head_dim = take(d, "head_dim", int, default=None)
        if head_dim is None:
            if hidden % heads != 0:
                raise ConfigError(
                    f"config.json: head_dim is absent and hidden_size={hidden} is not "
                    f"divisible by num_attention_heads={heads}")
            head_dim = hidden // heads

        # rope_theta lives at top level, or inside rope_parameters in newer files
        rope_theta = take(d, "rope_theta", float, default=None)
        rope_params = d.get("rope_parameters")
        if rope_theta is None and isinstance(rope_params, dict):
            rope_theta = take(rope_params, "rope_theta", float, default=None,
                              where="config.json rope_parameters")
        if rope_theta is None:
            raise ConfigError("config.json: required key 'rope_theta' is missing")
        for key in ("rope_scaling", "rope_parameters"):
            sc = d.get(key)
            if isinstance(sc, dict):
                kind = sc.get("rope_type", sc.get("type", "default"))
                if kind not in (None, "default"):
                    raise ConfigError(
                        f"config.json: {key} of type {kind!r} is not supported "
                        "(only unscaled rotary frequencies)")

        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids = (eos,)
        elif isinstance(eos, list) and all(isinstance(e, int) and not isinstance(e, bool) for e in eos):
            eos_ids = tuple(eos)
        else:
            raise ConfigError(f"config.json: 'eos_token_id' must be an integer or a list of integers, got {eos!r}")

        use_sw = take(d, "use_sliding_window", bool, default=False)
        sw = take(d, "sliding_window", int, default=None)
        mwl = take(d, "max_window_layers", int, default=None)
        layer_types = d.get("layer_types")
        windows = cls._layer_windows(layers, use_sw, sw, mwl, layer_types)

        cfg = cls(
            vocab_size=take(d, "vocab_size", int),
            hidden_size=hidden,
            intermediate_size=take(d, "intermediate_size", int),
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=take(d, "num_key_value_heads", int, default=heads),
            head_dim=head_dim,
            rms_norm_eps=take(d, "rms_norm_eps", float),
            rope_theta=rope_theta,
            hidden_act=take(d, "hidden_act", str, default="silu"),
            max_position_embeddings=take(d, "max_position_embeddings", int, default=None),
            tie_word_embeddings=take(d, "tie_word_embeddings", bool, default=None),
            attention_bias=take(d, "attention_bias", bool, default=False),
            bos_token_id=take(d, "bos_token_id", int, default=None),
            eos_token_ids=eos_ids,
            layer_windows=windows,
            sliding_window=sw,
            use_sliding_window=use_sw,
            max_window_layers=mwl,
        )
        cfg.validate()
        return cfg

    @staticmethod
    def _layer_windows(layers, use_sw, sw, mwl, layer_types) -> Tuple[Optional[int], ...]:
        if layers is None or layers < 0:
            return ()
        if not use_sw:
            if isinstance(layer_types, list) and any(t == "sliding_attention" for t in layer_types):
                raise ConfigError(
                    "config.json: layer_types names sliding_attention layers but "
                    "use_sliding_window is false")
            return tuple(None for _ in range(layers))
        if sw is None or sw <= 0:
            raise ConfigError("config.json: use_sliding_window is true but sliding_window is not a positive integer")
        if layer_types is not None:
            if not isinstance(layer_types, list) or len(layer_types) != layers:
                raise ConfigError(
                    f"config.json: layer_types must list {layers} entries, one per layer")
            out = []
            for i, t in enumerate(layer_types):
                if t == "full_attention":
                    out.append(None)
                elif t == "sliding_attention":
                    out.append(sw)
                else:
                    raise ConfigError(f"config.json: layer_types[{i}]={t!r} is not supported")
            return tuple(out)
        first_sliding = layers if mwl is None else mwl
        return tuple(sw if i >= first_sliding else None for i in range(layers))

    # ---- checking ------------------------------------------------------
    def validate(self) -> None:
        def positive(name):
            if getattr(self, name) <= 0:
                raise ConfigError(f"config.json: {name} must be > 0, got {getattr(self, name)}")
        for n in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                  "num_attention_heads", "num_key_value_heads", "head_dim"):
            positive(n)
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(
                f"config.json: num_attention_heads={self.num_attention_heads} must be divisible "
                f"by num_key_value_heads={self.num_key_value_heads}")
        if self.head_dim % 2 != 0:
            raise ConfigError(f"config.json: head_dim={self.head_dim} must be even (rotate-half rotary encoding)")
        if not (self.rms_norm_eps > 0.0):
            raise ConfigError(f"config.json: rms_norm_eps must be > 0, got {self.rms_norm_eps}")
        if not (self.rope_theta > 0.0):
            raise ConfigError(f"config.json: rope_theta must be > 0, got {self.rope_theta}")
        if self.hidden_act not in ("silu", "swish"):
            raise ConfigError(f"config.json: hidden_act={self.hidden_act!r} is not supported (only silu/swish)")
        if self.attention_bias:
            raise ConfigError("config.json: attention_bias=true is not supported (Qwen3 dense has no projection bias)")
        if self.max_position_embeddings is not None and self.max_position_embeddings <= 0:
            raise ConfigError("config.json: max_position_embeddings must be > 0")
        if len(self.layer_windows) != self.num_hidden_layers:
            raise ConfigError("layer_windows must hold one entry per layer")

    # ---- writing -------------------------------------------------------
    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {
            "architectures": [self.architectures[0]],
            "model_type": self.model_types[0],
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "hidden_act": self.hidden_act,
            "attention_bias": self.attention_bias,
            "use_sliding_window": self.use_sliding_window,
            "sliding_window": self.sliding_window,
            "torch_dtype": "bfloat16",
        }
        if self.max_position_embeddings is not None:
            d["max_position_embeddings"] = self.max_position_embeddings
        if self.tie_word_embeddings is not None:
            d["tie_word_embeddings"] = self.tie_word_embeddings
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        if len(self.eos_token_ids) == 1:
            d["eos_token_id"] = self.eos_token_ids[0]
        elif self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        if self.max_window_layers is not None:
            d["max_window_layers"] = self.max_window_layers
        if self.use_sliding_window:
            d["layer_types"] = ["full_attention" if w is None else "sliding_attention"
                                for w in self.layer_windows]
        return d
