"""The engine's config.toml, in the reference's manner.

garuda/src/config/mod.rs: sections ``[model] [memory] [runtime] [server]
[sampling]`` (:221-227); every section rejects unknown keys and fills what is
absent from defaults (``deny_unknown_fields, default``, :16-17); ``validate``
refuses what cannot be honoured instead of ignoring it (:283-347); sizes are
written ``"512MB"``, ``"8 GiB"`` (:232-269). Keys that the reference has keep
their names and meanings (``model.path``, ``model.context``,
``model.sliding_window``, ``model.gpu``, ``server.max_concurrent``,
``server.queue_capacity``, ``server.request_timeout_secs``, ``sampling.*``); the others are this
engine's own.
"""
from __future__ import annotations

import math
import os
import tomllib
from dataclasses import dataclass, field, fields

from .model_config import ConfigError


def parse_size(s) -> int:
    """``"512MB"``, ``"8 GiB"``, ``"1024"`` into bytes; K/M/G/T are powers of 1024
    (garuda/src/config/mod.rs:232-269)."""
    if isinstance(s, int) and not isinstance(s, bool):
        if s < 0:
            raise ConfigError(f"'{s}' is not a valid size")
        return s
    t = str(s).strip().upper().replace(" ", "")
    if not t:
        raise ConfigError("size is empty")
    i = 0
    while i < len(t) and (t[i].isdigit() or t[i] == "."):
        i += 1
    digits, unit = t[:i], t[i:]
    try:
        value = float(digits)
    except ValueError:
        raise ConfigError(f"'{s}' is not a valid size") from None
    if not math.isfinite(value) or value < 0:
        raise ConfigError(f"'{s}' is not a valid size")
    mult = {"": 1, "B": 1, "K": 1 << 10, "KB": 1 << 10, "KIB": 1 << 10, "M": 1 << 20, "MB": 1 << 20,
            "MIB": 1 << 20, "G": 1 << 30, "GB": 1 << 30, "GIB": 1 << 30, "T": 1 << 40, "TB": 1 << 40,
            "TIB": 1 << 40}.get(unit)
    if mult is None:
        raise ConfigError(f"unknown size unit '{unit}' in '{s}'")
    return int(value * mult)


@dataclass
class ModelSection:
    path: str = "./models"        # folder with config.json and model.safetensors
    dtype: str = "bfloat16"       # bfloat16 | float32
    context: int = 4096           # context window; a model caps it at its own (server/mod.rs:419)
    sliding_window: int = 0       # attention window; 0 attends to the whole context
    seed: int = 0                 # random-weights mode: seed of `garuda init`
    gpu: bool = True              # there is no CPU path: false is refused, not ignored
    # modules to import before the model is built: they register architectures or parts of their own
    plugins: list = field(default_factory=list)


@dataclass
class MemorySection:
    kv_cache: str = "0"           # bytes for the paged cache, e.g. "8GB"; "0": size it from kv_tokens
    kv_tokens: int = 0            # positions the cache holds; 0: max_concurrent * context
    page_size: int = 32           # positions per page (garuda/src/llama/mod.rs:483)


@dataclass
class RuntimeSection:
    max_batch_tokens: int = 2048  # tokens of one step: decode tokens and prompt portions together
    # most tokens of one prompt per step (scheduler/mod.rs:319-321, where the default is 512: here a
    # step of 512 tokens runs at 145 tokens/ms, one of 2,048 at 335, so a prompt may fill the step)
    prefill_chunk: int = 2048
    cuda_graphs: bool = True      # replay decode steps from captured graphs
    lookahead: bool = True        # launch the next greedy decode step while this one's tokens travel to the host
    paced_prefill: bool = False   # while something decodes, prompt portions sized to cost about one decode step
    device: int = 0


@dataclass
class ServerSection:
    max_concurrent: int = 4       # requests running at once
    queue_capacity: int = 256     # requests waiting before submissions are refused
    request_timeout_secs: int = 120   # a request ends with "timeout" this long after it was submitted


@dataclass
class SamplingSection:            # garuda/src/config/mod.rs:201-217
    temperature: float = 0.8
    top_p: float = 0.95
    top_k: int = 40
    max_tokens: int = 256


@dataclass
class EngineConfig:
    model: ModelSection = field(default_factory=ModelSection)
    memory: MemorySection = field(default_factory=MemorySection)
    runtime: RuntimeSection = field(default_factory=RuntimeSection)
    server: ServerSection = field(default_factory=ServerSection)
    sampling: SamplingSection = field(default_factory=SamplingSection)

    @classmethod
    def from_dict(cls, d: dict) -> "EngineConfig":
        cfg = cls()
        known = {f.name for f in fields(cls)}
        for section, body in d.items():
            if section not in known:
                raise ConfigError(f"unknown section [{section}] (sections: {', '.join(sorted(known))})")
            if not isinstance(body, dict):
                raise ConfigError(f"[{section}] must be a table")
            target = getattr(cfg, section)
            names = {f.name: f for f in fields(target)}
            for key, value in body.items():
                if key not in names:
                    raise ConfigError(f"unknown key '{key}' in [{section}] (keys: {', '.join(sorted(names))})")
                default = getattr(target, key)
                if isinstance(default, list):
                    ok = isinstance(value, list) and all(isinstance(v, str) for v in value)
                    value = list(value) if ok else value
                elif isinstance(default, bool):
                    ok = isinstance(value, bool)
                elif isinstance(default, int):
                    ok = isinstance(value, int) and not isinstance(value, bool)
                elif isinstance(default, float):
                    ok = isinstance(value, (int, float)) and not isinstance(value, bool)
                    value = float(value) if ok else value
                else:
                    ok = isinstance(value, str) or (key == "kv_cache" and isinstance(value, int))
                if not ok:
                    raise ConfigError(f"[{section}] {key} = {value!r} has the wrong type "
                                      f"(expected {type(default).__name__})")
                setattr(target, key, value)
        cfg.validate()
        return cfg

    @classmethod
    def load(cls, path: str) -> "EngineConfig":
        try:
            with open(path, "rb") as f:
                data = tomllib.load(f)
        except OSError as e:
            raise ConfigError(f"reading {path}: {e}") from None
        except tomllib.TOMLDecodeError as e:
            raise ConfigError(f"parsing {path}: {e}") from None
        return cls.from_dict(data)

    @classmethod
    def load_or_default(cls, path: str) -> "EngineConfig":
        """A missing file means defaults (garuda/src/main.rs:30-36)."""
        return cls.load(path) if os.path.exists(path) else cls()

    def validate(self) -> None:
        """Reject what cannot be honoured (garuda/src/config/mod.rs:283-347)."""
        if not self.model.gpu:
            raise ConfigError("gpu = false, but this engine has no CPU path. Set gpu = true.")
        if self.model.dtype not in ("bfloat16", "float32"):
            raise ConfigError(f"model.dtype must be 'bfloat16' or 'float32', got '{self.model.dtype}'")
        if self.model.context < 2:
            raise ConfigError("model.context must be at least 2")
        if self.model.sliding_window < 0:
            raise ConfigError("model.sliding_window must not be negative")
        if self.model.sliding_window > self.model.context:
            raise ConfigError(f"model.sliding_window ({self.model.sliding_window}) exceeds "
                              f"model.context ({self.model.context})")
        parse_size(self.memory.kv_cache)
        if self.memory.kv_tokens < 0:
            raise ConfigError("memory.kv_tokens must not be negative")
        if self.memory.page_size < 1:
            raise ConfigError("memory.page_size must be at least 1")
        if self.runtime.max_batch_tokens < 1:
            raise ConfigError("runtime.max_batch_tokens must be at least 1")
        if self.runtime.prefill_chunk < 0:
            raise ConfigError("runtime.prefill_chunk must not be negative")
        if self.runtime.device < 0:
            raise ConfigError("runtime.device must not be negative")
        if self.server.max_concurrent < 1:
            raise ConfigError("server.max_concurrent must be at least 1")
        if self.server.queue_capacity < 1:
            raise ConfigError("server.queue_capacity must be at least 1")
        if self.server.request_timeout_secs < 1:           # garuda/src/config/mod.rs:327-330
            raise ConfigError("server.request_timeout_secs must be at least 1")
        from ..sampling.params import SamplingParams
        SamplingParams(temperature=self.sampling.temperature, top_p=self.sampling.top_p,
                       top_k=self.sampling.top_k, max_tokens=self.sampling.max_tokens).validate()
