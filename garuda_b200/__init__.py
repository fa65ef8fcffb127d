"""garuda_b200: a single-GPU inference engine for the dense Llama decoder,
written for NVIDIA B200 (sm_100a).

    from garuda_b200 import Engine, SamplingParams
    engine = Engine("path/to/model_dir", dtype="bfloat16")
    results = engine.generate([[1, 2, 3]], SamplingParams.greedy(max_tokens=16))
"""
from .config import LlamaConfig, ConfigError, register_architecture, registered_architectures
from .config.engine_config import EngineConfig, parse_size
from .sampling import SamplingParams
from . import parts, models
from .engine import Engine, GenerationResult, StreamEvent, StepEntry, StepRunner, StepError
from .weights import write_random_model, WeightError

__all__ = ["Engine", "EngineConfig", "SamplingParams", "GenerationResult", "StreamEvent", "StepEntry", "StepRunner",
           "StepError", "LlamaConfig", "ConfigError", "WeightError", "write_random_model",
           "register_architecture", "registered_architectures", "parse_size", "parts", "models"]
