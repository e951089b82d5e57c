"""placeholder, filled in with the MLA decode kernel"""


def build_mla_decode(*a, **k):
    raise NotImplementedError("MLA decode not built yet")
