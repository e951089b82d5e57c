"""Small helpers shared by the front-end."""


class meta_tensor:
    """Shape/dtype descriptor of q, k or v: ``meta_tensor(B, H, S, D, dtype=...)``.
    Holds no storage (reference: attention_engine/core/utils.py:40-47)."""

    def __init__(self, *shape, **kwargs):
        self.shape = tuple(shape)
        self.kargs = kwargs

    @property
    def dtype(self):
        return self.kargs["dtype"]

    def __repr__(self):
        return f"meta_tensor{self.shape}[{self.kargs.get('dtype')}]"
