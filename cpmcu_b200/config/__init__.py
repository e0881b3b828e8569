from .base import ConfigError, FieldReader, architecture_name, read_config_json
from .minicpm import MiniCPMConfig, RopeScaling, SparseConfig

__all__ = ["ConfigError", "FieldReader", "architecture_name", "read_config_json", "MiniCPMConfig", "RopeScaling",
           "SparseConfig"]
