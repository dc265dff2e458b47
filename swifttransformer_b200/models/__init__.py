from .base import CausalLM, LayerStep, ModelDef
from .registry import (build_model_def, known_models, load_model, random_model, register_model,
                       write_random_model)
from . import opt as _opt  # registers OPTForCausalLM
from . import fanidra as _fanidra  # registers Fanidra
from . import pikadra as _pikadra  # registers Pikadra
from . import norelix as _norelix  # registers Norelix
from . import nafelix as _nafelix  # registers Nafelix

__all__ = ["CausalLM", "LayerStep", "ModelDef", "build_model_def", "known_models", "load_model",
           "random_model", "register_model", "write_random_model"]
