"""Front-end objects re-exported at package level (reference: attention_engine/core/__init__.py:1-2)."""
from .transform.core import CustomIO, SymbolicArray, SymbolScalar, SymbolicTensor, Var
from .utils import meta_tensor

__all__ = ["CustomIO", "SymbolicArray", "SymbolScalar", "SymbolicTensor", "Var", "meta_tensor"]
