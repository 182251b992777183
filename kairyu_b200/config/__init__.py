from kairyu_b200.config.engine_config import EngineConfig, normalize_dtype
from kairyu_b200.config.model_config import ConfigError, ModelConfig, RopeScaling, parse_dense_config

__all__ = ["ConfigError", "EngineConfig", "ModelConfig", "RopeScaling", "normalize_dtype", "parse_dense_config"]
