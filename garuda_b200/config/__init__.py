from .model_config import LlamaConfig, ConfigError, read_config_json
from .registry import (register_architecture, registered_architectures, read_model_config,
                       build_model, architecture_of, load_plugins)
