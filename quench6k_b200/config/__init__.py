from .flint import FlintConfig, ConfigError, ARCHITECTURE
from .registry import (register_architecture, get_architecture, known_architectures, load_config,
                       architecture_of, read_config_dict, UnknownArchitecture, Architecture)
