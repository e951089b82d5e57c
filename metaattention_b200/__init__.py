"""B200-native attention backend behind the AttentionEngine front-end API.

The reference project is used with its ``attention_engine/`` directory on
``PYTHONPATH`` so that ``attn_engine``, ``core``, ``autotuner`` and
``benchmark`` are top-level packages (docker/Dockerfile.cu128:49 of the
reference).  Importing this package puts its own directory on ``sys.path``
the same way, so ``import metaattention_b200`` followed by
``from attn_engine import AttentionEngine`` works unchanged.
"""

import os as _os
import sys as _sys

_here = _os.path.dirname(_os.path.abspath(__file__))
if _here not in _sys.path:
    _sys.path.insert(0, _here)

__version__ = "0.1.0"

from attn_engine import AttentionEngine, LinearAttentionEngine, OnlineFunc  # noqa: E402
from core import CustomIO, SymbolicArray, SymbolicTensor, SymbolScalar, Var, meta_tensor  # noqa: E402

__all__ = ["AttentionEngine", "LinearAttentionEngine", "OnlineFunc", "CustomIO", "SymbolicArray",
           "SymbolicTensor", "SymbolScalar", "Var", "meta_tensor"]
