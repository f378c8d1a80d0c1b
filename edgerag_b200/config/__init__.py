from .model_config import ConfigError, DecoderConfig
from .registry import (Architecture, architecture_names, architecture_of, read_model_folder,
                       register_architecture)

__all__ = ["ConfigError", "DecoderConfig", "Architecture", "architecture_names", "architecture_of",
           "read_model_folder", "register_architecture"]
