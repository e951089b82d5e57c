"""The backward functor derived from a traced score_mod (core/lower/derivative.py): which programs qualify, what is
emitted, and that the generated library compiles for sm_100a without a GPU."""

import pytest
import torch

from core.lower import derivative
from core.native import jit
from examples_b200 import programs


def test_which_programs_are_elementwise():
    B, H, S, D = 1, 2, 128, 128
    assert programs.sigmoid_engine(B, H, S, D, D, is_causal=True)._bwd_source is not None
    assert programs.relu_engine(B, H, S, 64, 64)._bwd_source is not None
    soft = programs.softmax_engine(B, H, S, D, D, is_causal=True)       # built-in softmax: its own backward kernel
    assert soft._bwd_source is None and soft.functor_kind == "builtin_softmax"
    assert programs.relu_engine(B, H, S, 128, 256)._bwd_source is not None  # one backward per 128-column slice of v
    assert programs.relu_engine(B, H, S, 192, 128)._bwd_source is None  # head dims the backward does not cover


def test_emitted_functor_of_sigmoid_attention():
    eng = programs.sigmoid_engine(1, 2, 128, 128, 128, is_causal=False, scale=0.25)
    src = eng._bwd_source
    assert "struct UserBwdFunctor" in src and "attn_b200_elementwise_bwd_jit" in src
    assert "kUsesStats = false" in src
    assert "c.cu[0] = *static_cast<const float*>(p.custom[0]);" in src        # the bias, an fp32 scalar
    assert "b200::fast_tanh" in src and "(1.0f - " in src                       # tanh and its derivative 1 - tanh^2
    assert "0.25f" in src                                                       # the scale inside score_mod
    assert "g_out = d" in src and "return dp * g;" in src


def test_programs_with_row_scales_are_refused():
    from core.lower.trace import trace_parallel
    from core.transform.core import CustomIO
    tr = trace_parallel(lambda s, c, b, h, q, kv: s * 0.5, programs.AbsSumNormaliser(), CustomIO({}))
    assert not derivative.elementwise_program(tr)
    with pytest.raises(NotImplementedError):
        derivative.emit_backward_functor(tr)


def test_generated_library_compiles():
    eng = programs.relu_engine(1, 1, 128, 64, 64, dtype=torch.float16)
    path = jit.build(eng._bwd_source)
    import ctypes
    assert hasattr(ctypes.CDLL(path), "attn_b200_elementwise_bwd_jit")
