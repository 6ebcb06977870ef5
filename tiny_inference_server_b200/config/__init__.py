from .model_config import ConfigError, GqaMtpConfig, KefisunConfig, MizidraConfig, BiruvikConfig, KubolornConfig, read_config_json, write_config_json, UPSTREAM_ALIASES
from .engine_config import EngineConfig

__all__ = ["ConfigError", "GqaMtpConfig", "KefisunConfig", "MizidraConfig", "BiruvikConfig", "KubolornConfig", "EngineConfig", "read_config_json", "write_config_json",
           "UPSTREAM_ALIASES"]
