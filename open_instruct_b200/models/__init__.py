from .llama import LlamaModel
from .spec import PRESETS, ModelSpec, ParamLayout, get_spec

__all__ = ["LlamaModel", "ModelSpec", "ParamLayout", "PRESETS", "get_spec"]
