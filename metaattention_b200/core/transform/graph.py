"""Expression-node vocabulary of the traced score_mod / online_func DAG.

Mirrors the node names of the reference front-end
(attention_engine/core/transform/graph.py:26-243) so user code that does
``from core import Var`` keeps working.  Only the forward vocabulary is kept:
the native backend lowers these nodes into C++ device functors, it does not
differentiate them.

Every node class is produced from one table (``OP_TABLE``) which also records
the arity and whether the op reduces a tile along its last axis; the C++
emitter in ``core.lower.functor`` keys off the same table, so the set of
supported ops is defined in exactly one place.
"""

from __future__ import annotations


class Node:
    """One operation (or leaf) of the symbolic DAG."""

    type: str = "Node"
    arity: int = 0
    reduces: str | None = None  # None | "row" | "col"

    def __init__(self, *inputs: "Node"):
        if len(inputs) != self.arity:
            raise TypeError(
                f"{self.type} takes {self.arity} operand(s), got {len(inputs)}")
        self.inputs = list(inputs)

    def __str__(self) -> str:
        return f"{self.type}({', '.join(str(i) for i in self.inputs)})"

    __repr__ = __str__


class Var(Node):
    """Named leaf: a kernel input (``scores``, a custom tensor) or an initial
    row-scale value given as a string such as ``"-inf"``, ``"0.0"``, ``"1"``."""

    type = "Var"

    def __init__(self, name: str):
        super().__init__()
        self.name = str(name)

    def __str__(self) -> str:
        return f'Var("{self.name}")'


class Const(Node):
    """Python number captured by value at trace time."""

    type = "Const"

    def __init__(self, value: float):
        super().__init__()
        self.value = value

    def __str__(self) -> str:
        return f"Const({self.value})"


# name -> (arity, reduction kind)
OP_TABLE: dict[str, tuple[int, str | None]] = {
    "Add": (2, None),
    "Sub": (2, None),
    "Mul": (2, None),
    "Div": (2, None),
    "Max": (2, None),
    "Min": (2, None),
    "MaxBwd": (3, None),
    "Neg": (1, None),
    "Abs": (1, None),
    "Exp": (1, None),
    "Exp2": (1, None),
    "Log": (1, None),
    "Log2": (1, None),
    "Tanh": (1, None),
    "ReduceSum": (1, "row"),
    "ReduceMax": (1, "row"),
    "ReduceAbsSum": (1, "row"),
    "ColReduceSum": (1, "col"),
    "ColReduceMax": (1, "col"),
    "ColReduceAbsSum": (1, "col"),
}


def _make_op(name: str, arity: int, reduces: str | None) -> type:
    return type(name, (Node,), {"type": name, "arity": arity, "reduces": reduces,
                                "__doc__": f"{name} node ({arity} operand(s))."})


for _name, (_arity, _red) in OP_TABLE.items():
    globals()[_name] = _make_op(_name, _arity, _red)

__all__ = ["Node", "Var", "Const", "OP_TABLE", *OP_TABLE.keys()]
