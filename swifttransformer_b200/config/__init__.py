from .base import (ConfigError, ModelConfig, config_class, config_from_dict, known_architectures,
                   load_config, register_config, save_config)
from .fanidra import FanidraConfig
from .nafelix import NafelixConfig
from .norelix import NorelixConfig
from .opt import OptConfig, opt_preset
from .pikadra import PikadraConfig

__all__ = ["ConfigError", "FanidraConfig", "ModelConfig", "NafelixConfig", "NorelixConfig", "OptConfig", "PikadraConfig", "config_class", "config_from_dict",
           "known_architectures", "load_config", "opt_preset", "register_config", "save_config"]
