"""The allocation-free MLA decode entry point (attn_b200_mla_decode_static) against the regular one.

The static entry point exists for hosts that must not allocate device memory around the decode
(their own arena owns the whole GPU, or a driver allocation's stall is not acceptable).  It keeps
its split-KV scratch in a fixed array inside the library, shared by all calls.  This test calls
it through the C ABI twice in a row with different inputs -- the second call finds the first
call's leftovers in the array -- and compares each result with the regular entry point, which
gets a fresh workspace.  It also checks that the call refuses a problem larger than the array,
and that no device memory is allocated across a call: this process's own allocator view
(torch's reserved bytes) must not change, and the device-wide free memory -- which another
process on the same GPU can move -- must not shrink by as much as the scratch would take.  The file name sorts last so that
a run stopping at the first failure has already run every other test."""

import ctypes as C

import pytest
import torch

from core.native import lib
from oracle import inputs

pytestmark = pytest.mark.gpu


def _args(q, kv, o, lse, splits, workspace=None):
    B, H, D = q.shape
    S = kv.shape[1]
    a = lib.MlaArgs()
    a.q, a.kv, a.o, a.lse = q.data_ptr(), kv.data_ptr(), o.data_ptr(), lse.data_ptr()
    a.q_stride[:] = (q.stride(0), q.stride(1))
    a.kv_stride[:] = (kv.stride(0), kv.stride(1))
    a.shape = lib.MlaShape(B, H, S, D, 512)
    a.num_splits, a.dtype, a.scale = splits, lib.DTYPE_CODES[q.dtype], D ** -0.5
    if workspace is not None:
        a.workspace, a.workspace_bytes = workspace.data_ptr(), workspace.numel()
    return a


def _regular(native, q, kv, splits):
    B, H, _ = q.shape
    o = torch.empty(B, H, 512, dtype=q.dtype, device="cuda")
    lse = torch.empty(B, H, dtype=torch.float32, device="cuda")
    shape = lib.MlaShape(B, H, kv.shape[1], 576, 512)
    need = native.attn_b200_mla_workspace_bytes(C.byref(shape), splits)
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
    assert native.attn_b200_mla_decode(C.byref(_args(q, kv, o, lse, splits, ws)), lib.current_stream_ptr()) == 0
    torch.cuda.synchronize()
    return o, lse


def test_static_entry_matches_regular_entry_on_two_calls_in_a_row():
    native = lib.load_library()
    status = torch.full((1,), 123, dtype=torch.int32, device="cuda")   # a stale value: the call must clear it
    cases = [(2, 128, 1536, 4, 61), (3, 64, 900, 3, 62)]               # different shapes: leftovers differ in layout
    outs = []
    for B, H, S, splits, seed in cases:
        q4, kv4 = inputs.mla_inputs(B, H, S, 576, 512, seed)
        q, kv = q4[:, 0].contiguous().cuda(), kv4[:, :, 0].contiguous().cuda()
        o = torch.full((B, H, 512), float("nan"), dtype=q.dtype, device="cuda")
        lse = torch.full((B, H), float("nan"), dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        reserved_before = torch.cuda.memory_reserved()
        rc = native.attn_b200_mla_decode_static(C.byref(_args(q, kv, o, lse, splits)), status.data_ptr(),
                                                lib.current_stream_ptr())
        assert rc == 0
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert torch.cuda.memory_reserved() == reserved_before   # nothing went through torch's allocator
        if outs:   # the very first call of a process may load the kernels' code; later calls must not take memory
            shape = lib.MlaShape(B, H, S, 576, 512)
            assert free_before - free_after < native.attn_b200_mla_workspace_bytes(C.byref(shape), splits)
        assert int(status.item()) == 0
        outs.append((q, kv, splits, o, lse))
    for q, kv, splits, o, lse in outs:
        want_o, want_lse = _regular(native, q, kv, splits)
        # same kernels, same split: the tolerance of the parity tests (max-abs 2e-2) is met with room to spare
        assert (o.float() - want_o.float()).abs().max().item() <= 2e-2
        assert torch.equal(o, want_o)
        assert (lse - want_lse).abs().max().item() <= 1e-5


def test_static_entry_refuses_what_does_not_fit():
    native = lib.load_library()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    # 128 sequences x 4 splits x 128 heads of fp32 partials = 134 MB of scratch: beyond the 32 MiB array
    q = torch.zeros(128, 128, 576, dtype=torch.bfloat16, device="cuda")
    kv = torch.zeros(128, 1024, 576, dtype=torch.bfloat16, device="cuda")
    o = torch.zeros(128, 128, 512, dtype=torch.bfloat16, device="cuda")
    lse = torch.zeros(128, 128, dtype=torch.float32, device="cuda")
    rc = native.attn_b200_mla_decode_static(C.byref(_args(q, kv, o, lse, 4)), status.data_ptr(), lib.current_stream_ptr())
    assert rc == -6 and "scratch" in lib.ERRORS[rc]
    # without splits no scratch is needed, so the same problem is accepted
    rc = native.attn_b200_mla_decode_static(C.byref(_args(q, kv, o, lse, 1)), status.data_ptr(), lib.current_stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert native.attn_b200_mla_decode_static(C.byref(_args(q, kv, o, lse, 1)), None, lib.current_stream_ptr()) == -1
