/*
 * attn_b200.h -- C ABI of the B200-native attention backend (libattn_b200.so).
 *
 * The reference project (SJTU-IPADS/MetaAttention) has no stable C ABI: its
 * native parts are per-instantiation pybind modules generated at run time.
 * Each entry point below names the reference interface it stands in for.
 *
 * Conventions
 *   - every pointer in an *Args struct is a DEVICE pointer unless it says host;
 *   - tensors are borrowed for the duration of the call, outputs are written
 *     in place into caller-allocated buffers;
 *   - kernels are enqueued on the given stream of the CURRENT device and the
 *     call returns without synchronising;
 *   - every function returns an int status: 0 = ok, negative = error
 *     (ATTN_B200_E_*).  Nothing here exits, aborts or traps.  Device-side
 *     waits are bounded; a wait that runs out records a code that
 *     attn_b200_last_device_status() reports after the stream is synchronised;
 *   - thread-compatible: concurrent calls are fine as long as calls that
 *     target the same stream are serialised by the caller.
 */
#ifndef ATTN_B200_H_
#define ATTN_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ATTN_B200_OK 0
#define ATTN_B200_E_INVALID_ARG (-1)   /* null pointer, bad enum, negative size            */
#define ATTN_B200_E_UNSUPPORTED (-2)   /* shape / dtype / stride the kernels do not cover   */
#define ATTN_B200_E_LAUNCH (-3)        /* CUDA runtime or driver error at launch            */
#define ATTN_B200_E_DEVICE_TIMEOUT (-4)/* a bounded device-side wait ran out                */
#define ATTN_B200_E_WORKSPACE (-5)     /* workspace missing or too small                    */
#define ATTN_B200_E_SCRATCH_LIMIT (-6) /* needs more scratch than the built-in static array  */

#define ATTN_B200_DTYPE_FP16 0
#define ATTN_B200_DTYPE_BF16 1
#define ATTN_B200_DTYPE_SAME 0         /* dtype_out: the output has the dtype of the inputs */
#define ATTN_B200_DTYPE_FP32 2         /* dtype_out: fp32 output (accumulators stored unrounded) */

#define ATTN_B200_MASK_NONE 0
#define ATTN_B200_MASK_CAUSAL 1        /* keep q_idx >= kv_idx (top-left aligned)           */
#define ATTN_B200_MASK_BAND 2          /* keep q_idx - mask_left <= kv_idx <= q_idx + mask_right (sliding windows) */
#define ATTN_B200_MASK_BITS 3          /* backward entry points only: any mask that does not depend on batch or head, as
                                          keep bits (mask_bits_q / mask_bits_kv of the argument structs) */
#define ATTN_B200_MASK_OPEN 0x3fffffff /* value of mask_left / mask_right for a side without a bound */

/* Built-in functors of the parallel pattern (score_mod + online_func pairs
 * recognised by the front-end).  Anything else is compiled from the traced
 * DAG into its own library exporting attn_b200_parallel_fwd_jit. */
#define ATTN_B200_FUNCTOR_SOFTMAX 0    /* fparams[0] = scale; p = exp(scale*(s - rowmax))   */

#define ATTN_B200_MAX_CUSTOM 4
#define ATTN_B200_MAX_ROWSCALES 4

/* Arguments of the parallel-pattern forward: O = epilogue(sum_tiles P.V),
 * P = online_fwd(score_mod(mask + Q.K^T)).
 * q,k: [batch, seq, heads, dim_qk], v,o: [batch, seq, heads, dim_v] as seen
 * through the element strides (last dimension contiguous). */
typedef struct AttnB200ParallelArgs {
  const void* q;
  const void* k;
  const void* v;
  void* o;
  float* final_rowscales[ATTN_B200_MAX_ROWSCALES]; /* each [batch, heads, seq_q] fp32, or NULL */
  int32_t batch, heads, seq_q, seq_kv, dim_qk, dim_v;
  int64_t q_stride[3];   /* element strides of (batch, seq, head) */
  int64_t k_stride[3];
  int64_t v_stride[3];
  int64_t o_stride[3];
  int32_t dtype;         /* ATTN_B200_DTYPE_*  */
  int32_t mask_kind;     /* ATTN_B200_MASK_*   */
  int32_t functor;       /* ATTN_B200_FUNCTOR_* (ignored by *_jit libraries) */
  int32_t heads_kv;      /* heads of k and v: 0 or `heads` = one per query head; a divisor of `heads` = grouped
                            (query head h reads KV head h / (heads / heads_kv), attn_gqa_tl.py of the reference) */
  float fparams[8];      /* functor scalars */
  const void* custom[ATTN_B200_MAX_CUSTOM];          /* custom_fwd_inputs tensors */
  int64_t custom_stride[ATTN_B200_MAX_CUSTOM][4];    /* element strides of (batch, heads, seq_len, seq_len_kv); 0 = broadcast */
  int32_t mask_left, mask_right;   /* ATTN_B200_MASK_BAND only: tokens kept before / after the diagonal, >= 0 or
                                      ATTN_B200_MASK_OPEN; KV tiles outside the band are skipped */
  /* Split-KV (decode with few query rows and heads; the reference's split kernel + OnlineFunc.combine,
   * core/lower/lower_decode.py:287-302,375-449): 0 or 1 = off.  With num_splits > 1 the KV tiles are divided
   * among num_splits CTAs per (query tile pair, head, batch); each writes its rows after the functor's epilogue
   * and its final row scales to the workspace, and a second kernel adds the rows up with the weights the
   * functor's combine gives (built-in softmax: through the log-sum-exp; *_jit libraries: the lowered
   * OnlineFunc.combine).  Not together with block sparsity. */
  int32_t num_splits;
  int32_t reserved;
  void* workspace;                 /* attn_b200_parallel_workspace_bytes() bytes of device scratch, or NULL */
  int64_t workspace_bytes;
  /* Block sparsity (the reference's block-sparse templates, core/template/tl_template/attn/blockattn_tl.py and
   * blockattn_decode_varlen_tl.py, chosen at core/lower/lower.py:723-738): tile_keep == NULL = off.  Otherwise
   * mask_kind must be ATTN_B200_MASK_NONE and every 128-row query tile visits exactly the 128-row KV tiles whose
   * bit is set in its bitmap; tiles whose bit is also set in tile_partial get an element mask (-inf where a bit
   * is clear; applied only by functors with a -inf mask value).
   *   tile_keep, tile_partial: uint32 [sparse_batch][sparse_heads][ceil(seq_q/128)][ceil(ceil(seq_kv/128)/32)],
   *       bit (j & 31) of word j >> 5 = KV tile j; sparse_batch is 1 or batch, sparse_heads is 1, heads_kv or heads.
   *   elem_mask_rows = 128: elem_mask holds one [128 rows][4 words] slot per partial tile, in the order
   *       (sparse batch, sparse head, query tile, KV tile); tile_mask_base [sparse_batch][sparse_heads][q tiles] is
   *       the slot of each query tile's first partial tile.  Bit (c & 31) of word c >> 5 of a row = keep column c.
   *   elem_mask_rows = 0: one [4 words] column mask per (sparse batch, sparse head, KV tile), shared by all query
   *       rows (decode: kept blocks and cache length per sequence); tile_mask_base is ignored. */
  const uint32_t* tile_keep;
  const uint32_t* tile_partial;
  const int32_t* tile_mask_base;
  const uint32_t* elem_mask;
  int32_t sparse_batch, sparse_heads, elem_mask_rows, reserved2;
} AttnB200ParallelArgs;

/* Replaces the generated TileLang forward kernel and its launcher
 * (attention_engine/core/template/tl_template/attn/attn_tl.py:93-190, :656-667)
 * and the CuTe forward (core/template/cute_template/flash_api.cpp:283-460). */
int attn_b200_parallel_fwd(const AttnB200ParallelArgs* args, void* cuda_stream);

/* Bytes of scratch the forward needs for args->num_splits (0 without split-KV; -1 = bad arguments): fp32 partial
 * rows plus ATTN_B200_MAX_ROWSCALES final row scales per row and split.  Valid for *_jit libraries as well. */
int64_t attn_b200_parallel_workspace_bytes(const AttnB200ParallelArgs* args);

/* Tile bitmaps and column masks of a block-sparse, variable-length decode, built on the device from what the
 * reference's block-sparse decode kernel takes at call time (block_mask and cache_seqlens of
 * core/template/tl_template/attn/blockattn_decode_varlen_tl.py:40-75): KV position p of (sequence b, KV head g)
 * takes part when block_mask[b][g][p / block_size] != 0 and p < cache_seqlens[b].
 *   block_mask: device uint8 [batch, heads_kv, n_blocks], or NULL = every block; cache_seqlens: device int32
 *   [batch], or NULL = seq_kv for every sequence.
 *   out: attn_b200_decode_tiles_bytes() bytes of device memory (16-byte aligned), laid out as
 *     col_mask uint32 [batch][heads_kv][ceil(seq_kv/128)][4], then tile_keep and tile_partial uint32
 *     [batch][heads_kv][words], words = ceil(ceil(seq_kv/128)/32):
 *   the elem_mask (elem_mask_rows = 0), tile_keep and tile_partial of AttnB200ParallelArgs with sparse_batch = batch,
 *   sparse_heads = heads_kv and one query tile.  Enqueued on the stream; no host synchronisation. */
int64_t attn_b200_decode_tiles_bytes(int32_t batch, int32_t heads_kv, int32_t seq_kv);
int attn_b200_decode_tiles(const uint8_t* block_mask, const int32_t* cache_seqlens, int32_t batch, int32_t heads_kv,
                           int32_t n_blocks, int32_t block_size, int32_t seq_kv, void* out, int64_t out_bytes,
                           void* cuda_stream);

/* Arguments of the chunked linear-attention / retention forward
 *   h_{c+1} = h_c * exp(g_last) + (K * exp(g_last - g))^T V
 *   O       = (scale*Q h_c) * exp(g) + tril((scale*Q K^T) * exp(g_i - g_j)) V
 * with g the within-chunk inclusive cumulative sum of log_decay.
 * q,k: [batch, heads, seq, dim_qk]; v,o: [batch, heads, seq, dim_v] contiguous;
 * log_decay: [batch, heads, seq] fp32 (natural log of the per-token decay). */
typedef struct AttnB200LinearArgs {
  const void* q;
  const void* k;
  const void* v;
  const float* log_decay;
  void* o;
  int32_t batch, heads, seq, dim_qk, dim_v;
  int32_t dtype;
  int32_t normalize;     /* 0: raw output; 1: per-(token, head) group norm over dim_v, eps below, no affine */
  float q_scale;         /* q_mod of the form q * const */
  float norm_eps;
  void* workspace;       /* attn_b200_linear_workspace_bytes() bytes (only needed with normalize = 1) */
  int64_t workspace_bytes;
  int32_t dtype_out;     /* ATTN_B200_DTYPE_SAME (0): o has the dtype of q, k, v; ATTN_B200_DTYPE_FP32: o is
                            [batch, heads, seq, dim_v] fp32 -- the accumulators as they are, for callers that
                            keep the result in fp32 and for judging the kernel apart from the output rounding
                            (the reference casts its fp32 accumulators to the input dtype, linear_tl.py:398-400) */
  int32_t precise;       /* 1: the decayed scores of a block enter P V as a 16-bit value plus a 16-bit remainder (two
                            passes) instead of one 16-bit value, as the normalised output does anyway: for runs whose
                            results are subtracted from one another afterwards (the gradient of the log-decays) */
  const float* v_scale;  /* [batch, heads, seq] fp32 or NULL: a per-token factor on the rows of v, applied inside the
                            kernel where they are rescaled for the state update anyway (a v_mod of the form
                            v * t[batch, heads, seq_len], e.g. Mamba2's v * dt: the fused v_mod of the reference's
                            core/lower/lower_linear.py:211-287) */
  int32_t heads_q;       /* heads of q, 0 = `heads`: q is [batch, heads_q, seq, dim_qk], and head h of v reads q head
                            h / (heads / heads_q) (Mamba2's C and B with fewer groups than v heads) */
  int32_t heads_k;       /* the same for k */
  int32_t q_ld;          /* elements between consecutive tokens of q, 0 = dim_qk: q may be a column range of a wider
                            [batch, heads_q, seq, q_ld] tensor (pointer at the range's first column, 16-byte aligned;
                            q_ld a multiple of 8) -- the backward contracts over column ranges of dO and v in place */
  int32_t k_ld;          /* the same for k */
} AttnB200LinearArgs;

/* Bytes of scratch the linear forward needs: per-row (sum, sum of squares) fp32 when normalize = 1, else 0. */
int64_t attn_b200_linear_workspace_bytes(const AttnB200LinearArgs* args);

/* Replaces chunk_local_cumsum_scalar + chunk_fwd_h + chunk_o and their wrapper
 * (core/template/tl_template/linear/linear_tl.py:36-60, :146-223, :321-401, :1240-1268). */
int attn_b200_linear_fwd(const AttnB200LinearArgs* args, void* cuda_stream);

/* Row gathers of the linear-attention backward, which runs attn_b200_linear_fwd on time-reversed operands and on column
 * ranges of dim_v and adds up fp32 partial results (the reference's backward kernels walk the sequence backwards
 * themselves, linear_tl.py:461-975).  All tensors [outer, seq, cols] contiguous, pointers 16-byte aligned, column
 * counts and offsets multiples of 8.
 *   rows_copy16:   dst[o][s'][0:width] = src[o][s][col0:col0+width] for 16-bit elements, s' = reverse ? seq-1-s : s
 *   rows_sum_cast: dst[o][s'][:] = a[o][s][:] + b[o][s][:] (b may be NULL), fp32 -> `dtype` (fp16 / bf16) */
int attn_b200_rows_copy16(const void* src, void* dst, int64_t outer, int32_t seq, int32_t src_cols, int32_t col0, int32_t width,
                          int32_t reverse, void* cuda_stream);
int attn_b200_rows_sum_cast(const float* a, const float* b, void* dst, int32_t dtype, int64_t outer, int32_t seq, int32_t cols,
                            int32_t reverse, void* cuda_stream);

/* MLA decode problem shape: one query token per sequence, one shared latent KV head. */
typedef struct AttnB200MlaShape {
  int32_t batch, heads_q, seq_kv, dim_qk, dim_v;
} AttnB200MlaShape;

/* Plan for a batch in which every sequence has seq_kv tokens, from the shape alone (host-side, integer):
 * num_splits_out >= 1 = that many equal splits per sequence fill the sm_count SMs well; 0 = they would leave the last
 * round of clusters far from full, use the scheduled mode.  (For ragged batches always use the scheduled mode: the
 * scheduler below, which looks at the actual cache lengths, is the counterpart of the reference's get_mla_metadata.) */
int attn_b200_mla_plan(const AttnB200MlaShape* shape, int32_t sm_count, int32_t* num_splits_out);

/* Tile scheduler.  Replaces get_mla_metadata (core/template/cute_template_kvshared/flash_api.cpp:23-59,
 * kernels/get_mla_metadata.cu:8-82): from the per-sequence cache lengths ON THE DEVICE, cuts the 128-row KV tiles of
 * all sequences -- every sequence, and every piece of one, charged 4 tiles of fixed overhead -- into num_parts equal
 * payloads, one per two-SM cluster.  Enqueued on the stream, no host synchronisation.
 *   cache_seqlens: device int32 [batch], or NULL = seq_kv tokens each;
 *   num_parts: attn_b200_mla_num_parts(heads_q, SM count) = SM pairs / head blocks of 128 heads;
 *   tile_scheduler_metadata: device int32 [num_parts][8] = first sequence, first token, last sequence (inclusive),
 *     end token (exclusive), split index of the part's first piece, KV tiles of the part, 0, 0 (fields 0-4 as in
 *     the reference's record);
 *   num_splits: device int32 [batch + 1], cumulative count of pieces (= partial-result rows) per sequence. */
int32_t attn_b200_mla_num_parts(int32_t heads_q, int32_t sm_count);
int attn_b200_mla_metadata(const int32_t* cache_seqlens, int32_t batch, int32_t seq_kv, int32_t num_parts,
                           int32_t* tile_scheduler_metadata, int32_t* num_splits, void* cuda_stream);

/* Bytes of scratch the decode needs: num_splits >= 1: fp32 partial outputs + partial log-sum-exp of a uniform split;
 * num_splits = 0 (scheduled): scheduler records, split counts and up to batch + num_parts partial rows, for the
 * current device's SM count. */
int64_t attn_b200_mla_workspace_bytes(const AttnB200MlaShape* shape, int32_t num_splits);

typedef struct AttnB200MlaArgs {
  const void* q;        /* [batch, heads_q, dim_qk], or its first dim_v columns when q_rope is given      */
  const void* kv;       /* [batch, seq_kv, dim_qk] latent KV, or its first dim_v columns when kv_rope is given;
                           V = the first dim_v columns of a latent row                                    */
  const void* q_rope;   /* NULL, or the last dim_qk-dim_v query columns held in a separate tensor         */
  const void* kv_rope;  /* NULL, or the last dim_qk-dim_v latent columns held in a separate tensor        */
  int64_t q_stride[2];        /* element strides of (batch, head)  of q        */
  int64_t kv_stride[2];       /* element strides of (batch, token) of kv       */
  int64_t q_rope_stride[2];   /* same for q_rope  (ignored when q_rope  is NULL) */
  int64_t kv_rope_stride[2];  /* same for kv_rope (ignored when kv_rope is NULL) */
  void* o;              /* [batch, heads_q, dim_v] contiguous */
  float* lse;           /* [batch, heads_q] fp32 natural-log sum-exp of scaled scores, or NULL */
  void* workspace;      /* attn_b200_mla_workspace_bytes() bytes */
  int64_t workspace_bytes;
  AttnB200MlaShape shape;
  int32_t num_splits;   /* 0: scheduled -- every cluster runs the pieces the tile scheduler gives it (computed by the
                           call from seq_lens, or passed in below); >= 1: that many equal splits per sequence */
  int32_t dtype;
  float scale;          /* softmax scale, e.g. 1/sqrt(dim_qk) */
  /* Ragged and paged caches (cache_seqlens / block_table of mha_fwd_kvcache_mla,
   * core/template/cute_template_kvshared/flash_api.cpp:61-72).  All-zero fields = one dense
   * [batch, seq_kv, *] cache in which every sequence has seq_kv tokens. */
  const int32_t* seq_lens;     /* device, [batch]: tokens of each sequence, 1 <= n <= shape.seq_kv; NULL = seq_kv   */
  const int32_t* block_table;  /* device, [batch, block_table_stride]: pool page holding tokens
                                  [i*page_size, (i+1)*page_size) of the sequence; NULL = dense cache.  With a
                                  table, kv (and kv_rope) point at a page pool [num_pages, page_size, *]:
                                  kv_stride[0] is the page stride, kv_stride[1] the token stride.  Entries are
                                  read up to the page of the sequence's last token; tokens of that page past the
                                  sequence end are read but carry no weight and must be finite numbers. */
  int64_t block_table_stride;  /* elements between the tables of two sequences */
  int32_t page_size;           /* tokens per page: a multiple of 64 */
  int32_t num_pages;           /* pages in the pool */
  /* num_splits = 0 only: the output of attn_b200_mla_metadata for these cache lengths (as the reference passes
   * tile_scheduler_metadata and num_splits to its decode, flash_api.cpp:61-72), or NULL to let the call compute it. */
  const int32_t* sched_meta;        /* device, [sched_parts][8] */
  const int32_t* sched_num_splits;  /* device, [batch + 1] */
  int32_t sched_parts;
  int32_t reserved;
} AttnB200MlaArgs;

/* Split-KV decode + combine.  Replaces flash_fwd_splitkv_mla_kernel and
 * flash_fwd_mla_combine_kernel with their launcher
 * (core/template/cute_template_kvshared/kernels/splitkv_mla.cu:1061-1471,
 *  kernels/mla_combine.cu:14-203, flash_api.cpp:61-210) and the TileLang
 * variant (core/template/tl_template/attn/mla_decode_tl.py:154-303). */
int attn_b200_mla_decode(const AttnB200MlaArgs* args, void* cuda_stream);

/* MLA decode that allocates nothing.  NO COUNTERPART IN THE REFERENCE: added for hosts that cannot
 * call cudaMalloc around the decode (all device memory already owned by their own arena, or a
 * latency-critical loop that cannot take a driver allocation).  Same arguments and results as
 * attn_b200_mla_decode, except that
 *   - the split-KV scratch is a 32 MiB array inside the library's device data segment (every GPU
 *     that loads the library holds it until exit); args->workspace / workspace_bytes are ignored;
 *     a problem with attn_b200_mla_workspace_bytes() above 32 MiB returns
 *     ATTN_B200_E_SCRATCH_LIMIT and launches nothing (num_splits = 1 needs no scratch at all);
 *   - status_word is a caller-owned 4-byte DEVICE word: cleared by the call, non-zero after the
 *     stream has been synchronised iff a device-side wait ran out (100 + id of the wait);
 *   - no cudaMalloc / cudaFree / allocating library routine is called.
 * The first call made on a device looks up the array's address (once per device).  With CUDA's lazy
 * module loading that look-up, or the first launch, is also the moment the driver loads the library's
 * device code on that device and reserves the 32 MiB of the array: make this first call at start-up,
 * before any stream capture on the device and before the host's own arena claims what is left of the
 * device memory.  All calls on a device share the array and it keeps the previous call's contents
 * (no part of it needs clearing); calls that overlap on the GPU race. */
int attn_b200_mla_decode_static(const AttnB200MlaArgs* args, int32_t* status_word, void* cuda_stream);

/* Backward of softmax attention (the built-in softmax functor; mask NONE or CAUSAL; dim_qk = dim_v = 128 or 64; grouped
 * KV heads as in the forward).  Replaces the reference's generated backward kernels and their launcher
 * (attention_engine/core/template/tl_template/attn/attn_tl.py: preprocess :212-244, main :309-503, postprocess
 * :246-275, autograd wrapper :669-694; the CuTe backward behind core/template/cute_template/flash_api.cpp:462-700).
 * o and lse are the forward's results (lse = log-sum-exp of scale * q.k over the kept keys, [batch, heads, seq_q]
 * fp32); d_o is the gradient of o.  dq, dk, dv get the gradients in the dtype of q, k, v; every element inside the
 * sequence bounds is written.  All strides are element strides of (batch, seq, head) with the head dim contiguous. */
typedef struct AttnB200SoftmaxBwdArgs {
  const void* q;
  const void* k;
  const void* v;
  const void* o;
  const void* d_o;
  const float* lse;
  void* dq;
  void* dk;
  void* dv;
  int32_t batch, heads, heads_kv, seq_q, seq_kv, dim_qk, dim_v;
  int32_t dtype;       /* ATTN_B200_DTYPE_* */
  int32_t mask_kind;   /* ATTN_B200_MASK_NONE, _CAUSAL (keep kv_idx <= q_idx), _BAND or _BITS */
  float scale;         /* softmax scale */
  int64_t q_stride[3], k_stride[3], v_stride[3], o_stride[3], do_stride[3];
  int64_t dq_stride[3], dk_stride[3], dv_stride[3];
  void* workspace;     /* attn_b200_softmax_bwd_workspace_bytes() bytes of device scratch, 16-byte aligned */
  int64_t workspace_bytes;
  int32_t mask_left, mask_right;   /* ATTN_B200_MASK_BAND only, as in AttnB200ParallelArgs: tile pairs outside the band
                                      are skipped in both launches */
  /* ATTN_B200_MASK_BITS only (device, 16-byte aligned): the keep matrix of the mask and its transpose as bits, for the
   * launch that owns query rows and the one that owns KV rows.  With nq, nk = 128-row tiles of seq_q, seq_kv:
   * mask_bits_q uint32 [nq*128][nk][4]: bit (c & 31) of word c >> 5 of [q][j] = keep (q, 128 j + c);
   * mask_bits_kv uint32 [nk*128][nq][4]: bit (c & 31) of word c >> 5 of [kv][i] = keep (128 i + c, kv);
   * rows and columns past the sequence ends are 0.  (The reference's backward applies mask_mod element-wise to every
   * tile, attn_tl.py:430-461.) */
  const void* mask_bits_q;
  const void* mask_bits_kv;
  /* optional with the bits (both or neither; device): which pairs of tiles keep anything, so that the others are
   * skipped.  mask_tiles_q uint32 [nq][ceil(nk / 32)]: bit (j & 31) of word j >> 5 of row i = the pair (query tile i, KV
   * tile j) keeps something; mask_tiles_kv uint32 [nk][ceil(nq / 32)] the same matrix transposed. */
  const void* mask_tiles_q;
  const void* mask_tiles_kv;
} AttnB200SoftmaxBwdArgs;

/* Scratch the backward needs (delta = rowsum(dO o O) and the log-sum-exp in the exp2 domain, padded to whole
 * 128-row tiles); -1 = bad arguments. */
int64_t attn_b200_softmax_bwd_workspace_bytes(const AttnB200SoftmaxBwdArgs* args);

/* Three launches on `cuda_stream`: the preparation pass, dK/dV (one CTA per KV tile and KV head), dQ (one CTA per
 * query tile and head).  No atomics: results are bit-reproducible. */
int attn_b200_softmax_bwd(const AttnB200SoftmaxBwdArgs* args, void* cuda_stream);

/* Backward of an elementwise program (a lowered score_mod with no row scales: P = f(q.k), e.g. the sigmoid and relu
 * attention of the reference's examples; its gradient graph is what core/transform/core.py:119-199 and
 * core/lower/lower.py:349-436 of the reference build).  There is one entry point per functor, exported by the
 * library compiled for that functor's forward-mode derivative (`_jit/functor_*.so`), never by libattn_b200:
 *   int attn_b200_elementwise_bwd_jit(const AttnB200ElementwiseBwdArgs* args, void* cuda_stream, int32_t* device_status);
 * dV = P^T dO, dS = dP * f'(q.k), dK = dS^T Q, dQ = dS K; mask NONE or CAUSAL (masked pairs contribute nothing), grouped
 * KV heads, dim_qk = dim_v = 128 or 64.  `custom[i]` points at the i-th custom input, an fp32 scalar on the device. */
typedef struct AttnB200ElementwiseBwdArgs {
  const void* q;
  const void* k;
  const void* v;
  const void* d_o;
  void* dq;
  void* dk;
  void* dv;
  int32_t batch, heads, heads_kv, seq_q, seq_kv, dim_qk, dim_v;
  int32_t dtype;       /* ATTN_B200_DTYPE_* */
  int32_t mask_kind;   /* ATTN_B200_MASK_NONE, _CAUSAL, _BAND or _BITS */
  int32_t reserved;
  int64_t q_stride[3], k_stride[3], v_stride[3], do_stride[3];
  int64_t dq_stride[3], dk_stride[3], dv_stride[3];
  const void* custom[ATTN_B200_MAX_CUSTOM];
  int32_t mask_left, mask_right;   /* ATTN_B200_MASK_BAND only */
  const void* mask_bits_q;         /* ATTN_B200_MASK_BITS only, as in AttnB200SoftmaxBwdArgs */
  const void* mask_bits_kv;
  const void* mask_tiles_q;
  const void* mask_tiles_kv;
} AttnB200ElementwiseBwdArgs;

/* Reads and clears the device-side status word of device `device`
 * (0 = no kernel reported a problem).  Synchronises the device. */
int attn_b200_last_device_status(int32_t device, int32_t* status_out);

/* Library version, major*10000 + minor*100 + patch. */
int attn_b200_version(void);

#ifdef __cplusplus
}
#endif
#endif /* ATTN_B200_H_ */
