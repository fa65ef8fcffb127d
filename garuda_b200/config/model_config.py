"""Typed model configuration, read from the architecture's own config.json keys.

The reference reads the same facts from GGUF metadata
(garuda/src/llama/mod.rs:395-465): required sizes have no default, a missing one
is an error that names the key, and inconsistent head counts are refused.
No size or constant of a model lives anywhere but in an instance of this class.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, asdict
from typing import Any, Optional


class ConfigError(ValueError):
    """A config.json (or config.toml) that cannot be honoured."""


_REQUIRED = ("hidden_size", "num_hidden_layers", "num_attention_heads",
             "intermediate_size", "vocab_size")

LAYER_TYPES = ("full_attention", "sliding_attention")


@dataclass(frozen=True)
class LlamaConfig:
    """The dense Llama decoder's parameters.

    Keys and defaults: ``num_key_value_heads`` defaults to
    ``num_attention_heads`` (garuda/src/llama/mod.rs:428-430), ``head_dim`` to
    ``hidden_size / num_attention_heads`` (:450), ``max_position_embeddings`` to
    2048 (:457), ``rms_norm_eps`` to 1e-5 (:458-460), ``rope_theta`` to 10000
    (:461). ``sliding_window`` (0 or null: attend to everything,
    garuda/src/config/mod.rs:34-35) and ``layer_types`` (which layers the window
    applies to; all of them when absent) choose the mixer layer by layer.
    ``rope_layout`` is ``"half"`` for the row order of safetensors folders and
    ``"interleaved"`` for the reference's pairing (garuda/src/simd/mod.rs:196-206).
    """
    architecture: str
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    intermediate_size: int
    vocab_size: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int = 2048
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    rope_layout: str = "half"
    tie_word_embeddings: bool = False
    hidden_act: str = "silu"
    sliding_window: Optional[int] = None
    layer_types: Optional[tuple] = None
    eos_token_ids: tuple = ()        # config.json gives one id or a list; generation ends on any
    bos_token_id: Optional[int] = None
    torch_dtype: Optional[str] = None
    extra: dict = field(default_factory=dict, compare=False)

    # ---- derived ---------------------------------------------------------
    @property
    def eos_token_id(self) -> Optional[int]:
        """The first end-of-sequence id, for callers that want one."""
        return self.eos_token_ids[0] if self.eos_token_ids else None

    @property
    def kv_dim(self) -> int:
        """Width of one stored key or value (garuda/src/llama/mod.rs:468-470)."""
        return self.num_key_value_heads * self.head_dim

    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    def layer_window(self, layer: int) -> Optional[int]:
        if not self.sliding_window:
            return None
        if self.layer_types is None:
            return self.sliding_window
        return self.sliding_window if self.layer_types[layer] == "sliding_attention" else None

    # ---- construction ----------------------------------------------------
    @classmethod
    def from_dict(cls, d: dict) -> "LlamaConfig":
        d = dict(d)
        for key in _REQUIRED:
            if key not in d or d[key] is None:
                raise ConfigError(f"config.json is missing '{key}'")
        archs = d.pop("architectures", None) or [d.pop("architecture", "LlamaForCausalLM")]
        d.pop("architecture", None)
        arch = archs[0]

        def integer(key, value, minimum=1):
            if isinstance(value, bool) or not isinstance(value, int) or value < minimum:
                raise ConfigError(f"config.json: '{key}' must be an integer >= {minimum}, got {value!r}")
            return value

        hidden = integer("hidden_size", d.pop("hidden_size"))
        layers = integer("num_hidden_layers", d.pop("num_hidden_layers"))
        heads = integer("num_attention_heads", d.pop("num_attention_heads"))
        inter = integer("intermediate_size", d.pop("intermediate_size"))
        vocab = integer("vocab_size", d.pop("vocab_size"))
        kv_heads = d.pop("num_key_value_heads", None)
        kv_heads = heads if kv_heads is None else integer("num_key_value_heads", kv_heads)
        head_dim = d.pop("head_dim", None)
        if head_dim is None:
            if hidden % heads:
                raise ConfigError(
                    f"inconsistent head configuration: hidden_size={hidden} is not a multiple "
                    f"of num_attention_heads={heads} and no head_dim is given")
            head_dim = hidden // heads
        head_dim = integer("head_dim", head_dim)
        if heads % kv_heads:
            raise ConfigError(
                f"num_attention_heads {heads} is not a multiple of num_key_value_heads {kv_heads}")
        if head_dim % 2:
            raise ConfigError(f"head_dim {head_dim} must be even for rotary positions")

        act = d.pop("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"hidden_act '{act}' is not supported (the feed-forward is SwiGLU: 'silu')")
        for key in ("attention_bias", "mlp_bias"):
            if d.pop(key, False):
                raise ConfigError(f"'{key}' = true is not supported: the projections have no bias")
        scaling = d.pop("rope_scaling", None)
        if scaling is not None:
            raise ConfigError("'rope_scaling' is not supported: rotation is full-width and unscaled")
        layout = d.pop("rope_layout", "half")
        if layout not in ("half", "interleaved"):
            raise ConfigError(f"rope_layout must be 'half' or 'interleaved', got {layout!r}")

        window = d.pop("sliding_window", None)
        if window is not None:
            window = integer("sliding_window", window, minimum=0) or None
        types = d.pop("layer_types", None)
        if types is not None:
            types = tuple(types)
            if len(types) != layers:
                raise ConfigError(f"layer_types has {len(types)} entries for {layers} layers")
            for t in types:
                if t not in LAYER_TYPES:
                    raise ConfigError(f"layer_types entry {t!r} is not one of {LAYER_TYPES}")
            if "sliding_attention" in types and not window:
                raise ConfigError("layer_types names sliding_attention but sliding_window is not set")

        eps = d.pop("rms_norm_eps", 1e-5)
        theta = d.pop("rope_theta", 10000.0)
        for key, value in (("rms_norm_eps", eps), ("rope_theta", theta)):
            if isinstance(value, bool) or not isinstance(value, (int, float)) or not value > 0:
                raise ConfigError(f"config.json: '{key}' must be a positive number, got {value!r}")

        return cls(
            architecture=arch, hidden_size=hidden, num_hidden_layers=layers,
            num_attention_heads=heads, intermediate_size=inter, vocab_size=vocab,
            num_key_value_heads=kv_heads, head_dim=head_dim,
            max_position_embeddings=integer("max_position_embeddings",
                                            d.pop("max_position_embeddings", 2048)),
            rms_norm_eps=float(eps), rope_theta=float(theta), rope_layout=layout,
            tie_word_embeddings=bool(d.pop("tie_word_embeddings", False)),
            hidden_act=act, sliding_window=window, layer_types=types,
            eos_token_ids=_int_tuple("eos_token_id", d.pop("eos_token_id", None)),
            bos_token_id=_first_int(d.pop("bos_token_id", None)),
            torch_dtype=d.pop("torch_dtype", d.pop("dtype", None)),
            extra=d,
        )

    def to_dict(self) -> dict:
        """The config.json this configuration is read back from."""
        d = asdict(self)
        extra = d.pop("extra")
        eos = d.pop("eos_token_ids")
        if eos:
            d["eos_token_id"] = eos[0] if len(eos) == 1 else list(eos)
        d["architectures"] = [d.pop("architecture")]
        if d["layer_types"] is not None:
            d["layer_types"] = list(d["layer_types"])
        d = {k: v for k, v in d.items() if v is not None}
        d["model_type"] = extra.get("model_type", "llama")
        return d


def _int_tuple(key: str, v: Any) -> tuple:
    """A single id or a list of ids, as a tuple without repeats (order kept)."""
    if v is None:
        return ()
    items = list(v) if isinstance(v, (list, tuple)) else [v]
    out = []
    for x in items:
        if isinstance(x, bool) or not isinstance(x, int) or x < 0:
            raise ConfigError(f"config.json: '{key}' must be a token id or a list of them, got {v!r}")
        if x not in out:
            out.append(x)
    return tuple(out)


def _first_int(v: Any) -> Optional[int]:
    if isinstance(v, (list, tuple)):
        return int(v[0]) if v else None
    return None if v is None else int(v)


def read_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            return json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"{path} does not exist") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path} is not valid JSON: {e}") from None
