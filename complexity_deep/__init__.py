"""Import-name shim: ``complexity_deep`` resolves to the B200 implementation.

A script written against the reference package keeps its import lines
(complexity_deep/__init__.py:21-54, complexity_deep/models/__init__.py:5-16,
complexity_deep/core/__init__.py:13-29 of the reference project) and gets the classes of
``complexity_deep_b200``.  Nothing is implemented here: every public name and every
sub-module path (``complexity_deep.core.token_routed_mlp``, ``complexity_deep.models.modeling``,
...) is an alias of the corresponding ``complexity_deep_b200`` module.  The reference's
``complexity_deep.cuda`` (Triton kernels) has no counterpart: its role is taken by libcdeep.so.
"""
import importlib as _importlib
import sys as _sys

import complexity_deep_b200 as _impl
from complexity_deep_b200 import (RMSNorm, RotaryEmbedding, ComplexityAttention, SwiGLU,  # noqa: F401
                                  TokenRoutedMLP, TransformerBlock, MuGuidance, ComplexityConfig,
                                  ComplexityModel, create_complexity_model, count_parameters)

__version__ = _impl.__version__
__all__ = list(_impl.__all__)

for _name in ("core", "core.normalization", "core.rotary", "core.attention", "core.mlp",
              "core.token_routed_mlp", "core.layer", "models", "models.config",
              "models.modeling", "models.utils"):
    _module = _importlib.import_module("complexity_deep_b200." + _name)
    _sys.modules[__name__ + "." + _name] = _module
    if "." not in _name:
        globals()[_name] = _module
del _name, _module
