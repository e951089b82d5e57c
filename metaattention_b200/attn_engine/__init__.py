"""Top-level package ``attn_engine`` (reference: attention_engine/attn_engine/__init__.py:1-2)."""
from .attn_engine import AttentionEngine, OnlineFunc
from .linear_attn_engine import LinearAttentionEngine

__all__ = ["AttentionEngine", "OnlineFunc", "LinearAttentionEngine"]
