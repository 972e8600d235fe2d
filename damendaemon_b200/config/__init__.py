from .reader import ConfigError, parse_config_text, read_config_file
from .gpt2 import Gpt2Config

__all__ = ["ConfigError", "parse_config_text", "read_config_file", "Gpt2Config"]
