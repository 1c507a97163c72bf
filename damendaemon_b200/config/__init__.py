from .reader import ConfigError, parse_config_text, read_config_file
from .bonatar import BonatarConfig
from .derusun import DerusunConfig
from .gpt2 import Gpt2Config
from .zokanex import ZokanexConfig

__all__ = ["ConfigError", "parse_config_text", "read_config_file", "Gpt2Config", "BonatarConfig", "ZokanexConfig", "DerusunConfig"]
