"""Device descriptors.  The import surface ``get_attn_device``, ``H100``,
``AttnDevice``, ``AttnDeviceAMD`` is what the reference's examples use
(attention_engine/autotuner/arch/__init__.py:9-34); only ``.name`` is read by
callers (it selects a tuned-config path, which this backend ignores).  There is
no tuning step here: every kernel family has fixed per-shape configurations,
so a descriptor is informational."""

import warnings

import torch

from .arch_base import Arch
from .devices import A100, B200, H100, RTX4090

AttnDevice = {
    (8, 0): A100,
    (8, 9): RTX4090,
    (9, 0): H100,
    (10, 0): B200,
}

# The reference keeps a second table for ROCm parts; this backend is CUDA sm_100a only.
AttnDeviceAMD: dict = {}


def get_attn_device() -> Arch:
    """Descriptor of the current CUDA device; B200 when no GPU is visible
    (engines can be constructed, and their functors compiled, without one)."""
    if not torch.cuda.is_available():
        return B200()
    cap = torch.cuda.get_device_capability(torch.cuda.current_device())
    if cap in AttnDevice:
        return AttnDevice[cap]()
    warnings.warn(f"no descriptor for compute capability {cap}; using B200 settings")
    return B200()


__all__ = ["Arch", "A100", "RTX4090", "H100", "B200", "AttnDevice", "AttnDeviceAMD", "get_attn_device"]
