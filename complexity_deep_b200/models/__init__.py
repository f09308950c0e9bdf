"""Model classes with the reference's names (complexity_deep/models/__init__.py:5-16)."""
from .config import ComplexityConfig
from .modeling import ComplexityModel, CausalLMOutput, ModelOutput
from .utils import DecodeGraph, PrefillGraph, create_complexity_model, count_parameters

__all__ = ["ComplexityConfig", "ComplexityModel", "CausalLMOutput", "ModelOutput",
           "create_complexity_model", "count_parameters", "PrefillGraph", "DecodeGraph"]
