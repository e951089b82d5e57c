"""MLA decode on the native split-KV kernels (``kv_shared=True`` engines).

Two calling conventions of the reference are kept:

* ``backend="tl"`` -- ``mod(q, q_pe, kv, k_pe) -> o`` with q ``[B,1,H,Dv]``,
  q_pe ``[B,1,H,D-Dv]``, kv ``[B,S,1,Dv]``, k_pe ``[B,S,1,D-Dv]``
  (core/template/tl_template/attn/mla_decode_tl.py:450-465, testing/test.py:842-848);
* ``backend="cute"`` -- ``mod(q, KV) -> (out, lse)`` with q ``[B,1,H,D]`` and the
  latent cache as 64-token pages ``[B*S/64, 64, 1, D]`` under an identity block
  table (attn_engine.py:199-224, cute_template_kvshared/flash_mla_interface.py:98-115).

As in the reference's MLA lowering (core/lower/lower_decode_mla.py:25-38) the
softmax is fixed: ``score_mod`` / ``online_func`` passed to the engine are not
consulted; the scale is 1/sqrt(D).  The rope part may live in separate tensors:
the kernel reads both through their own tensor maps, nothing is concatenated.
"""

from __future__ import annotations

import ctypes as C

import torch

from core.native import lib as native

_sm_count_cache: dict[int, int] = {}


def _sm_count(device: torch.device) -> int:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _sm_count_cache:
        _sm_count_cache[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _sm_count_cache[idx]


def plan_splits(batch: int, heads: int, seq_kv: int, dim_qk: int, dim_v: int, sm_count: int) -> int:
    shape = native.MlaShape(batch, heads, seq_kv, dim_qk, dim_v)
    out = C.c_int32(0)
    native.check(native.load_library().attn_b200_mla_plan(C.byref(shape), sm_count, C.byref(out)), "attn_b200_mla_plan")
    return out.value


def workspace_bytes(batch: int, heads: int, seq_kv: int, dim_qk: int, dim_v: int, num_splits: int) -> int:
    shape = native.MlaShape(batch, heads, seq_kv, dim_qk, dim_v)
    return int(native.load_library().attn_b200_mla_workspace_bytes(C.byref(shape), num_splits))


def _rows(t: torch.Tensor, what: str):
    """[B, R, C] view of a [B,R,C], [B,1,R,C] or [B,R,1,C] tensor, last dim contiguous."""
    if t.dim() == 4:
        if t.shape[1] == 1:
            t = t[:, 0]
        elif t.shape[2] == 1:
            t = t[:, :, 0]
        else:
            raise ValueError(f"{what}: expected a singleton axis, got shape {tuple(t.shape)}")
    if t.dim() != 3 or t.stride(-1) != 1:
        raise ValueError(f"{what}: expected [batch, rows, cols] with contiguous columns, got {tuple(t.shape)}")
    return t


last_plan = None   # how the most recent mla_decode_forward call was distributed (read by the benchmark)


def num_parts(heads_q: int, device) -> int:
    """Clusters that walk the tile schedule for ``heads_q`` query heads on ``device`` (SM pairs / head blocks)."""
    return int(native.load_library().attn_b200_mla_num_parts(heads_q, _sm_count(device)))


def mla_schedule(cache_seqlens, batch: int, seq_kv: int, heads_q: int, device):
    """(tile_scheduler_metadata int32 [parts, 8], num_splits int32 [batch + 1]) from attn_b200_mla_metadata: the
    equal-payload partition of all sequences' KV tiles over the clusters, computed on the device from the actual
    cache lengths (``cache_seqlens`` None = ``seq_kv`` tokens each).  Enqueued on the current stream."""
    parts = num_parts(heads_q, device)
    meta = torch.empty((parts, 8), dtype=torch.int32, device=device)
    cum = torch.empty((batch + 1,), dtype=torch.int32, device=device)
    native.check(native.load_library().attn_b200_mla_metadata(
        cache_seqlens.data_ptr() if cache_seqlens is not None else None, batch, seq_kv, parts, meta.data_ptr(), cum.data_ptr(),
        native.current_stream_ptr()), "attn_b200_mla_metadata")
    return meta, cum


def mla_decode_forward(q, kv, dim_v: int, scale: float, q_rope=None, kv_rope=None, num_splits: int | None = None,
                       workspace: torch.Tensor | None = None, cache_seqlens: torch.Tensor | None = None,
                       block_table: torch.Tensor | None = None, max_seqlen: int | None = None,
                       tile_scheduler_metadata: torch.Tensor | None = None, num_splits_cum: torch.Tensor | None = None):
    """q: [B,H,D] (or [B,1,H,D]); kv: [B,S,D] (or [B,S,1,D]).  With ``q_rope`` /
    ``kv_rope`` given, q and kv hold only the first ``dim_v`` columns.
    ``cache_seqlens`` (int32 [B], CUDA): tokens of each sequence (1..S); default all S.
    ``block_table`` (int32 [B, max_blocks], CUDA): kv is then a page pool [num_pages, page_size, D] (or
    [num_pages, page_size, 1, D]), page_size a multiple of 64, and entry i of a sequence's row names the
    page with its tokens [i*page_size, (i+1)*page_size); ``max_seqlen`` (default max_blocks*page_size)
    bounds the sequence lengths.
    ``num_splits``: 0 = scheduled -- one cluster per SM pair walks the pieces of sequences that the tile
    scheduler gives it (equal payloads from the actual cache lengths; ``tile_scheduler_metadata`` / ``num_splits_cum``
    from ``mla_schedule`` may be passed to reuse one schedule over many calls); an int >= 1 = that many equal splits
    per sequence; None = scheduled when ``cache_seqlens`` or a schedule is given, else what ``plan_splits`` estimates
    to be faster for equal lengths.
    Returns (o [B,H,dim_v] in the input dtype, lse [B,H] fp32)."""
    global last_plan
    q3, kv3 = _rows(q, "q"), _rows(kv, "kv")
    if not q3.is_cuda:
        raise native.NativeError("MLA decode needs CUDA tensors")
    B, H, dq = q3.shape
    S = kv3.shape[1]
    page_size = num_pages = 0
    if block_table is not None:
        if block_table.dtype != torch.int32 or not block_table.is_cuda or block_table.dim() != 2 or block_table.shape[0] != B:
            raise ValueError("block_table must be a CUDA int32 tensor [batch, max_blocks]")
        if block_table.stride(1) != 1:
            block_table = block_table.contiguous()
        num_pages, page_size = kv3.shape[0], kv3.shape[1]
        S = block_table.shape[1] * page_size if max_seqlen is None else int(max_seqlen)
        if S > block_table.shape[1] * page_size:
            raise ValueError("max_seqlen exceeds the block table")
    if cache_seqlens is not None:
        if cache_seqlens.dtype != torch.int32 or not cache_seqlens.is_cuda or cache_seqlens.numel() != B:
            raise ValueError("cache_seqlens must be a CUDA int32 tensor [batch]")
        cache_seqlens = cache_seqlens.contiguous()
    rope_dim = 0
    qr3 = kr3 = None
    if (q_rope is None) != (kv_rope is None):
        raise ValueError("q_rope and kv_rope must be given together")
    if q_rope is not None:
        qr3, kr3 = _rows(q_rope, "q_rope"), _rows(kv_rope, "kv_rope")
        rope_dim = qr3.shape[2]
    dim_qk = dq + rope_dim
    if q3.dtype not in native.DTYPE_CODES or kv3.dtype != q3.dtype:
        raise native.NativeError("q and kv must share dtype float16 or bfloat16")
    with torch.cuda.device(q3.device):
        if num_splits is None:
            # ragged lengths: scheduled; equal lengths: whichever the plan estimates faster (0 = scheduled)
            num_splits = 0 if (cache_seqlens is not None or tile_scheduler_metadata is not None) else \
                plan_splits(B, H, S, dim_qk, dim_v, _sm_count(q3.device))
        need = workspace_bytes(B, H, S, dim_qk, dim_v, num_splits)
        last_plan = {"mode": "scheduled", "parts": num_parts(H, q3.device)} if num_splits == 0 else {"mode": "uniform", "num_splits": num_splits}
        if need < 0:
            raise native.NativeError(f"MLA decode does not support dims qk={dim_qk} v={dim_v}")
        if need > 0 and (workspace is None or workspace.numel() * workspace.element_size() < need):
            workspace = torch.empty(need, dtype=torch.uint8, device=q3.device)
        o = torch.empty((B, H, dim_v), dtype=q3.dtype, device=q3.device)
        lse = torch.empty((B, H), dtype=torch.float32, device=q3.device)
        a = native.MlaArgs()
        a.q, a.kv = q3.data_ptr(), kv3.data_ptr()
        a.q_stride[:] = (q3.stride(0), q3.stride(1))
        a.kv_stride[:] = (kv3.stride(0), kv3.stride(1))
        if qr3 is not None:
            a.q_rope, a.kv_rope = qr3.data_ptr(), kr3.data_ptr()
            a.q_rope_stride[:] = (qr3.stride(0), qr3.stride(1))
            a.kv_rope_stride[:] = (kr3.stride(0), kr3.stride(1))
        a.o, a.lse = o.data_ptr(), lse.data_ptr()
        a.workspace = workspace.data_ptr() if need > 0 else None
        a.workspace_bytes = need
        a.shape = native.MlaShape(B, H, S, dim_qk, dim_v)
        a.num_splits = num_splits
        a.dtype = native.DTYPE_CODES[q3.dtype]
        a.scale = float(scale)
        if cache_seqlens is not None:
            a.seq_lens = cache_seqlens.data_ptr()
        if num_splits == 0 and tile_scheduler_metadata is not None:
            if num_splits_cum is None or tile_scheduler_metadata.dtype != torch.int32 or num_splits_cum.dtype != torch.int32:
                raise ValueError("tile_scheduler_metadata and num_splits_cum must be the int32 tensors of mla_schedule")
            if tile_scheduler_metadata.shape[0] != num_parts(H, q3.device) or num_splits_cum.numel() != B + 1:
                raise ValueError("the schedule was made for another batch or device")
            a.sched_meta, a.sched_num_splits = tile_scheduler_metadata.data_ptr(), num_splits_cum.data_ptr()
            a.sched_parts = tile_scheduler_metadata.shape[0]
        if block_table is not None:
            a.block_table = block_table.data_ptr()
            a.block_table_stride = block_table.stride(0)
            a.page_size, a.num_pages = page_size, num_pages
        native.check(native.load_library().attn_b200_mla_decode(C.byref(a), native.current_stream_ptr()),
                     "attn_b200_mla_decode")
    return o, lse


def build_mla_decode(engine, B, H, Hkv, Skv, D, Dv, dtype, backend):
    if Hkv != 1:
        raise NotImplementedError("MLA decode expects a single shared latent KV head")
    scale = D ** -0.5
    engine.mla_scale = scale

    if backend == "tl":
        def attention(q, q_pe, kv, k_pe):
            o, lse = mla_decode_forward(q, kv, Dv, scale, q_rope=q_pe, kv_rope=k_pe)
            engine.last_final_rowscales = {"lse": lse}
            return o.view(o.shape[0], 1, o.shape[1], o.shape[2])
        return attention

    def attention_paged(q, kv_pages):
        # identity block table over 64-token pages: the pages of one sequence are contiguous
        Bq = q.shape[0]
        kv = kv_pages.reshape(Bq, -1, kv_pages.shape[-1])
        o, lse = mla_decode_forward(q, kv, Dv, scale)
        engine.last_final_rowscales = {"lse": lse}
        return o.view(Bq, 1, o.shape[1], o.shape[2]), lse.view(Bq, lse.shape[1], 1)
    return attention_paged


def get_mla_metadata(cache_seqlens: torch.Tensor, num_heads_per_head_k: int, num_heads_k: int = 1):
    """Same call as the reference's scheduler query (cute_template_kvshared/flash_mla_interface.py:57-72): returns
    (tile_scheduler_metadata int32 [num_sm_parts, 8], num_splits int32 [batch + 1]) for these cache lengths; pass both
    on to flash_mla_with_kvcache, for every layer of a decoding step."""
    if num_heads_k != 1:
        raise NotImplementedError("MLA decode expects a single shared latent KV head")
    if cache_seqlens.dtype != torch.int32 or not cache_seqlens.is_cuda:
        raise ValueError("cache_seqlens must be a CUDA int32 tensor [batch]")
    with torch.cuda.device(cache_seqlens.device):
        return mla_schedule(cache_seqlens.contiguous(), cache_seqlens.numel(), 0x3fffffff, num_heads_per_head_k, cache_seqlens.device)


def flash_mla_with_kvcache(q, k_cache, block_table, cache_seqlens, head_dim_v, tile_scheduler_metadata=None,
                           num_splits=None, softmax_scale=None, causal=False):
    """Drop-in for the reference's paged MLA decode call
    (cute_template_kvshared/flash_mla_interface.py:74-115): q [B,1,Hq,D], k_cache [num_blocks,
    page_block_size, 1, D], block_table int32 [B, max_blocks], cache_seqlens int32 [B],
    tile_scheduler_metadata / num_splits as returned by get_mla_metadata (or None: the call makes its own schedule;
    an int num_splits asks for that many equal splits per sequence instead).
    Returns (out [B,1,Hq,head_dim_v], softmax_lse [B,Hq,1] fp32).  ``causal`` has no effect with one
    query token per sequence."""
    if q.shape[1] != 1:
        raise NotImplementedError("one query token per sequence")
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** (-0.5)
    if isinstance(num_splits, int):
        o, lse = mla_decode_forward(q, k_cache, head_dim_v, softmax_scale, num_splits=num_splits,
                                    cache_seqlens=cache_seqlens, block_table=block_table)
    else:
        o, lse = mla_decode_forward(q, k_cache, head_dim_v, softmax_scale, cache_seqlens=cache_seqlens, block_table=block_table,
                                    tile_scheduler_metadata=tile_scheduler_metadata, num_splits_cum=num_splits)
    return o.view(o.shape[0], 1, o.shape[1], o.shape[2]), lse.view(lse.shape[0], lse.shape[1], 1)
