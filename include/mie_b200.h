/*
 * mie_b200 — C-ABI of the B200 (sm_100a) continuous-batching hot path.
 *
 * Every entry point takes plain device pointers, sizes and element strides, a
 * CUDA stream handle and (where metadata is read on the device) a pointer to
 * an int32 status word in device memory.  No entry point allocates device
 * memory unless its comment says so, none synchronises the stream, and the
 * ones whose scratch comes from the caller may be captured into a CUDA graph.
 *
 * Return value: 0 on success, a negative MIE_ERR_* code when the arguments
 * are rejected on the host (nothing was launched; mie_last_error() holds a
 * message).  Problems that only the device can see (a page id outside the
 * pool, a length that overruns its block table, a wait that ran out) never
 * trap: the offending row is skipped or clamped and a MIE_STATUS_* bit is
 * OR-ed into *status, which the caller reads back with its next device→host
 * copy.
 *
 * The reference engine has no FFI: its boundary is Python functions over
 * torch tensors (paths below are relative to the reference project).  Each
 * declaration cites the Python function whose launch it replaces; the Python
 * package mini_inference_engine_b200.engine re-exports those functions with
 * the reference's names and signatures and calls this library through ctypes.
 */
#ifndef MIE_B200_H_
#define MIE_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MIE_OK 0
#define MIE_ERR_INVALID_ARGUMENT (-1)
#define MIE_ERR_CUDA (-2)
#define MIE_ERR_UNSUPPORTED (-3)

/* Bits OR-ed into the device status word. */
#define MIE_STATUS_BAD_LENGTH 1      /* sequence length < 1 or beyond the block-table capacity */
#define MIE_STATUS_BAD_POSITION 2    /* query position outside [0, length) */
#define MIE_STATUS_BAD_PAGE 4        /* live block-table entry outside [0, num_blocks) */
#define MIE_STATUS_BAD_SEQUENCE 8    /* token_to_sequence entry outside the block-table rows */
#define MIE_STATUS_WAIT_TIMEOUT 16   /* a bounded device-side wait gave up */
#define MIE_STATUS_MAX_LENGTH 32     /* attention read length beyond max_sequence_length */
#define MIE_STATUS_CAPACITY 64       /* work plan did not fit the scratch the caller sized */
#define MIE_STATUS_NO_TOKEN 128      /* greedy sampling saw no candidate for a row; token 0 was written */

/* Element types of K/V pages, queries and activations. */
#define MIE_DTYPE_BF16 0
#define MIE_DTYPE_F16 1
#define MIE_DTYPE_F32 2

/* An int32 or int64 metadata tensor (1-D or 2-D) with element strides. */
typedef struct {
  const void* ptr;
  int32_t is64;
  int64_t stride0;
  int64_t stride1;
} mie_index_t;

/* A 4-D tensor view: base pointer and element strides. */
typedef struct {
  void* ptr;
  int64_t stride[4];
} mie_view4_t;

const char* mie_last_error(void);
int mie_version(void);
/* Number of SMs of the current device (used by callers to size scratch). */
int mie_sm_count(void);
/* Kernels this library has launched (or captured into a graph) in this process so far. */
int64_t mie_launch_count(void);

/* ------------------------------------------------------------------------
 * KV-cache scatter
 * ---------------------------------------------------------------------- */

/*
 * Replaces triton_write_decode_kv (engine/kv_cache/triton_paged_kv.py:154-223,
 * kernel :20-107): for every request b and KV head h copy the one new K and V
 * row to page block_tables[b][pos / block_size], slot pos % block_size, where
 * pos = query_positions[b] if given, else sequence_lengths[b] - 1.
 * key_states / value_states: [batch, kv_heads, 1, head_dim] with independent
 * strides.  key_blocks / value_blocks: [num_blocks, kv_heads, block_size,
 * head_dim].  A bit-exact copy.
 */
int mie_write_decode_kv(mie_view4_t key_states, mie_view4_t value_states, mie_index_t block_tables,
                        mie_index_t sequence_lengths, mie_index_t query_positions /* ptr may be NULL */,
                        mie_view4_t key_blocks, mie_view4_t value_blocks, int32_t batch, int32_t kv_heads,
                        int32_t head_dim, int32_t block_size, int32_t num_blocks, int32_t table_width,
                        int32_t elem_bytes, int32_t* status, void* stream);

/*
 * Replaces triton_write_packed_kv (engine/kv_cache/triton_packed_kv.py:146-208,
 * kernel :18-104): scatter `tokens` packed rows; row t goes to sequence
 * token_to_sequence[t], position token_positions[t], i.e. slot
 * block_tables[seq][pos / block_size] * block_size + pos % block_size.
 * key_states / value_states: [1, kv_heads, tokens, head_dim], V with strides
 * of its own.
 */
int mie_write_packed_kv(mie_view4_t key_states, mie_view4_t value_states, mie_index_t token_to_sequence,
                        mie_index_t token_positions, mie_index_t block_tables, mie_view4_t key_blocks,
                        mie_view4_t value_blocks, int32_t tokens, int32_t kv_heads, int32_t head_dim,
                        int32_t block_size, int32_t num_blocks, int32_t table_rows, int32_t table_width,
                        int32_t elem_bytes, int32_t* status, void* stream);

/*
 * Replaces PagedKvCache.gather_layer (engine/kv_cache/paged.py:910-944) and the
 * index_select gather of engine/kv_cache/qwen3_paged.py:296-312 ("block-table
 * gather"): copies the first `length` tokens of one sequence out of its pages
 * into dense [kv_heads, length, head_dim] K and V (contiguous).  Bit-exact.
 */
int mie_gather_kv(mie_view4_t key_blocks, mie_view4_t value_blocks, mie_index_t block_table_row,
                  void* key_out, void* value_out, int32_t length, int32_t kv_heads, int32_t head_dim,
                  int32_t block_size, int32_t num_blocks, int32_t elem_bytes, int32_t* status, void* stream);

/* ------------------------------------------------------------------------
 * Decode metadata validation
 * ---------------------------------------------------------------------- */

/*
 * Replaces the device half of validate_decode_metadata
 * (engine/kv_cache/decode_metadata.py:67-91).  The reference turns the checks
 * into device asserts under graph capture; here one small kernel applies the
 * same predicates and ORs MIE_STATUS_* bits into *status, so a bad replay is
 * reported without losing the context.  reserved_lengths (host array, may be
 * NULL) is only checked by the Python shim in eager mode.
 */
int mie_validate_decode_metadata(mie_index_t block_tables, mie_index_t sequence_lengths,
                                 mie_index_t query_positions /* ptr may be NULL */, int32_t batch,
                                 int32_t table_width, int32_t block_size, int32_t num_blocks,
                                 int64_t max_sequence_length /* <=0: unchecked */, int32_t* status, void* stream);

/* ------------------------------------------------------------------------
 * Paged decode attention
 * ---------------------------------------------------------------------- */

/*
 * Bytes of scratch (work plan + split-KV partials) that
 * mie_paged_decode_attention needs for a batch whose attention read lengths
 * sum to at most max_total_tokens.  Host arithmetic only.
 */
int64_t mie_decode_scratch_bytes(int32_t batch, int32_t q_heads, int32_t kv_heads, int32_t head_dim,
                                 int64_t max_total_tokens);

/*
 * Replaces triton_paged_decode_attention
 * (engine/kv_cache/triton_paged_attention.py:680-974; kernels :28, :181, :314,
 * :480) and tensor_core_decode_attention (engine/kv_cache/triton_tc_decode.py:177).
 *
 * query [batch, q_heads, 1, head_dim], out [batch, q_heads, 1, head_dim] (any
 * strides, last dim contiguous), pages [num_blocks, kv_heads, block_size,
 * head_dim].  Row b attends to the first min(len[b], pos[b]+1) tokens (len[b]
 * if query_positions.ptr is NULL).
 *
 * split_policy: 0 = one work item per (request, KV head) (no split-KV);
 *               1 = length-proportional split-KV chosen on the device from the
 *                   batch's total length (the partials are merged by a second
 *                   kernel); > 1 = fixed chunk of that many tokens (multiple of 16).
 * scratch: device buffer of at least mie_decode_scratch_bytes(...) bytes,
 * 256-byte aligned; contents need not be initialised.  plan_only / use_plan
 * let a model step build the work plan once (layer 0) and reuse it for the
 * other layers: plan_only=1 builds the plan and returns; use_plan=1 skips the
 * plan kernel and uses slot `plan_slot` (0..63) of the plan's work counters.
 * out_q8 (optional): additionally writes the output quantised for the o_proj
 * FP8 GEMM, exactly what mie_fp8_quantize would produce from `out` viewed as
 * [batch, q_heads * head_dim]: e4m3 rows of ldq8 bytes and out_scales[head *
 * out_scale_ld + request] (one 128-column group per head).
 */
int mie_paged_decode_attention(mie_view4_t query, mie_view4_t out, mie_view4_t key_blocks,
                               mie_view4_t value_blocks, mie_index_t block_tables, mie_index_t sequence_lengths,
                               mie_index_t query_positions /* ptr may be NULL */, int32_t batch, int32_t q_heads,
                               int32_t kv_heads, int32_t head_dim, int32_t block_size, int32_t num_blocks,
                               int32_t table_width, int32_t dtype, float scale, int32_t split_policy,
                               int64_t max_total_tokens, void* scratch, int64_t scratch_bytes, int32_t plan_only,
                               int32_t use_plan, int32_t plan_slot, void* out_q8 /* may be NULL */, int64_t ldq8,
                               float* out_scales, int32_t out_scale_ld, int32_t* status, void* stream);

/*
 * Has no counterpart in the reference.  The same ragged decode attention as
 * mie_paged_decode_attention, for hosts that cannot hand it a scratch buffer
 * because they have nothing to allocate device memory with: a C / Go / Java
 * binding that only owns the tensors it was given, or a server that assigned
 * all free HBM to its KV pool at start-up and keeps no allocator around.  The
 * work plan and the split-KV partials live in a 16 MiB array that is part of
 * the library image (mie_decode_builtin_scratch_bytes()); every GPU that loads
 * the library holds that array until the process exits.  The call performs no
 * device allocation and frees nothing.
 *
 * Limit: mie_decode_scratch_bytes(batch, q_heads, kv_heads, head_dim,
 * max_total_tokens) must not exceed the array (about 64 requests x 4k tokens
 * at 32 query heads); larger batches are rejected with
 * MIE_ERR_INVALID_ARGUMENT and a message, nothing is launched.  The check is
 * made on the sizes alone, so it also turns away large fp32 or odd-head_dim
 * batches that would have taken the generic kernel and never touched the array.
 *
 * The first call on each device looks the array's device address up (with that
 * device current); make that first call before any stream capture starts.
 * All calls share the one array and it keeps whatever the previous call left:
 * each call rebuilds its plan and zeroes its counters first, so stale contents
 * are harmless, but two calls that run on the GPU at the same time (different
 * streams, threads or processes' worth of overlap on one device) race on it.
 * Run them on one stream, or use mie_paged_decode_attention with separate buffers.
 */
int64_t mie_decode_builtin_scratch_bytes(void);
int mie_paged_decode_attention_static(mie_view4_t query, mie_view4_t out, mie_view4_t key_blocks,
                                      mie_view4_t value_blocks, mie_index_t block_tables,
                                      mie_index_t sequence_lengths, mie_index_t query_positions /* ptr may be NULL */,
                                      int32_t batch, int32_t q_heads, int32_t kv_heads, int32_t head_dim,
                                      int32_t block_size, int32_t num_blocks, int32_t table_width, int32_t dtype,
                                      float scale, int32_t split_policy, int64_t max_total_tokens, int32_t* status,
                                      void* stream);

/* ------------------------------------------------------------------------
 * FP8 (e4m3) KV cache: decode attention and the writer that fills it
 * ---------------------------------------------------------------------- */

/*
 * The reference keeps K/V in the model dtype; it only names an FP8 cache as the
 * next step for its HBM-bound decode (docs/phase_notes/roofline.md:76), so these
 * two entries extend mie_paged_decode_attention / mie_qkv_norm_rope_write and
 * have no reference implementation to be pinned against.
 *
 * Layout (page size 16, head_dim 128): kv_pool [num_blocks][kv_heads][2][16][128]
 * bytes - per page and KV head the 16 K rows then the 16 V rows, e4m3 - with a
 * page stride of page_stride_bytes (>= kv_heads * 4096, so one layer can be a
 * slice of a bigger pool), 1 KiB aligned; kv_scales [num_blocks][kv_heads][2][16]
 * fp32, one scale per (token, KV head) for K and for V: scale = amax / 448 of
 * the row, row / max(scale, 1e-12) rounded to e4m3 (mie_fp8_quantize's rule).
 * 2,112 bytes per token and layer at 8 KV heads instead of 4,096.
 *
 * mie_paged_decode_attention_kv8 is mie_paged_decode_attention on that pool:
 * same query / output tensors (bf16 or fp16), metadata, split policy, scratch,
 * plans and optional e4m3 output for o_proj.  Scores are (q . k8) * k_scale in
 * fp32, rounded to the query dtype like the bf16 path; the V scale of a token is
 * folded into its probability before P . V.
 */
int mie_paged_decode_attention_kv8(mie_view4_t query, mie_view4_t out, const void* kv_pool,
                                   int64_t page_stride_bytes, const float* kv_scales, mie_index_t block_tables,
                                   mie_index_t sequence_lengths, mie_index_t query_positions /* ptr may be NULL */,
                                   int32_t batch, int32_t q_heads, int32_t kv_heads, int32_t num_blocks,
                                   int32_t table_width, int32_t dtype, float scale, int32_t split_policy,
                                   void* scratch, int64_t scratch_bytes, int32_t plan_only, int32_t use_plan,
                                   int32_t plan_slot, void* out_q8 /* may be NULL */, int64_t ldq8,
                                   float* out_scales, int32_t out_scale_ld, int32_t* status, void* stream);

/*
 * mie_qkv_norm_rope_write with the K/V rows quantised into the FP8 pool above
 * instead of copied to bf16 pages (q rows, norms and RoPE are unchanged).
 */
int mie_qkv_norm_rope_write_kv8(const void* qkv, int64_t ld, const void* q_weight, const void* k_weight,
                                const void* cos_sin, int32_t max_pos, mie_index_t positions,
                                mie_index_t token_to_sequence, mie_index_t block_tables, void* q_out, void* kv_pool,
                                int64_t page_stride_bytes, float* kv_scales, int32_t tokens, int32_t q_heads,
                                int32_t kv_heads, int32_t num_blocks, int32_t table_rows, int32_t table_width,
                                float eps, int32_t* status, void* stream);

/* ------------------------------------------------------------------------
 * Chunked-prefill attention
 * ---------------------------------------------------------------------- */

/*
 * Replaces triton_flash_prefill_attention (engine/kv_cache/triton_flash_prefill.py:154-202,
 * kernel :58-151) and, through the Python shim, triton_packed_prefill_attention
 * (engine/kv_cache/triton_packed_attention.py:186-259): packed varlen causal
 * attention over K/V pages that already contain the new tokens.  query / out
 * [tokens, q_heads, head_dim] (token and head strides in elements, head_dim
 * contiguous); request r owns rows cu_seqlens[r] .. cu_seqlens[r+1] and sees
 * kv_lens[r] keys, query row i at position kv_lens[r] - q_len + i.
 * max_query_len is a host bound that sizes the grid; total_tokens is the number
 * of query rows.  head_dim 128, bf16/fp16.  GQA groups of 1/2/4/8 run the
 * tcgen05 kernel, other shapes the mma.sync kernel.
 */
int mie_flash_prefill_attention(const void* query, int64_t q_token_stride, int64_t q_head_stride,
                                int64_t total_tokens, void* out,
                                int64_t o_token_stride, int64_t o_head_stride, mie_view4_t key_blocks,
                                mie_view4_t value_blocks, mie_index_t block_tables, mie_index_t cu_seqlens,
                                mie_index_t kv_lens, int32_t requests, int32_t max_query_len, int32_t q_heads,
                                int32_t kv_heads, int32_t head_dim, int32_t block_size, int32_t num_blocks,
                                int32_t table_width, int32_t dtype, float scale, int32_t* status, void* stream);

/* ------------------------------------------------------------------------
 * FP8 128x128 block-scaled linear
 * ---------------------------------------------------------------------- */

/*
 * Replaces quantize_sm89_fp8_activation (engine/kernels/sm89_fp8.py:401-424,
 * kernel :303-332): per token and per 128-column group, scale = amax / 448 (the
 * RAW scale is stored, 0 for an all-zero group), q = x / max(scale, 1e-12)
 * rounded to e4m3.  x [m, k] (row stride ldx elements), q [m, k] bytes (row
 * stride ldq).  The scales are written K-group major: scales[group * scale_ld +
 * token], scale_ld >= m, which is the layout mie_fp8_gemm reads.
 */
int mie_fp8_quantize(const void* x, int64_t ldx, int32_t dtype, void* q, int64_t ldq, float* scales,
                     int32_t scale_ld, int32_t m, int32_t k, void* stream);

/*
 * Replaces the GEMM of sm89_fp8_linear (engine/kernels/sm89_fp8.py:444-528;
 * kernels _fp8_linear_kernel :220-300 and _fp8_split_gemm_kernel :343-398):
 *   y[m, n] = sum_kb dot(x8[m, kb], w8[n, kb]) * a_scale[kb][m] * w_scale[n / 128][kb]
 * with fp32 accumulation, y in bf16 or fp16.
 * x8 [m, k] e4m3 (row stride ldx bytes), a_scale as mie_fp8_quantize writes it,
 * w8 [n, k] e4m3 (row stride ldw bytes), w_scale [ceil(n/128), w_scale_ld].
 * Operand base pointers and row strides must be multiples of 16 bytes.
 * Up to 128 tokens (up to 256 when n <= 1536) run with the weight rows as the
 * 128 MMA rows (a weight streaming loop); more tokens run a persistent
 * 128 x 256-tile kernel.
 *
 * Summation order.  Within one CTA the K blocks are added in increasing order.
 * When a shape has fewer output tiles than SMs - or, above 128 tokens, when the
 * tiles left over after the last whole round of SMs are few - the K range of a
 * tile is cut into 2, 4 or 8 contiguous parts that run as one thread-block
 * cluster; each part is summed in increasing K order and the parts are then
 * added in part order through distributed shared memory.  That is a fixed
 * order (results never depend on timing), but it is not the single increasing
 * K order, and whether a tile is cut depends on m, n and the SM count, so a
 * token's row can differ in the last bit between batch sizes.  max_split = 1
 * never cuts: every output element is then the plain increasing-K sum,
 * independent of the batch it was computed in (the reference's row-independence
 * promise, tests/test_sm89_fp8_exact.py); max_split = 0 lets the library
 * choose, other values cap the factor.  Uses no global scratch memory.
 *
 * flags: MIE_GEMM_NO_WEIGHT_PREFETCH, or 0.  By default the weight tiles of the
 * first pipeline stages are requested while the kernel queued before this one
 * may still be running (programmatic dependent launch), so w8 must not be
 * written by that kernel; pass the flag (or set MIE_GEMM_PREFETCH=0) when it is.
 */
#define MIE_GEMM_NO_WEIGHT_PREFETCH 1
int mie_fp8_gemm(const void* x8, int64_t ldx, const float* a_scale, int32_t a_scale_ld, const void* w8,
                 int64_t ldw, const float* w_scale, int32_t w_scale_ld, void* y, int64_t ldy, int32_t out_dtype,
                 int32_t m, int32_t n, int32_t k, int32_t max_split, int32_t flags, int32_t* status, void* stream);

/* ------------------------------------------------------------------------
 * Fused memory-bound glue (bf16 activations)
 * ---------------------------------------------------------------------- */

/*
 * Replaces rms_norm (engine/kernels/fused.py:165-203, kernel :90-124) for
 * contiguous rows: out = weight * bf16(x * rsqrt(mean(x^2) + eps)) with fp32
 * math.  With `residual` the row normalised is bf16(x + residual), which is
 * also stored to `summed` (the reference's (normed, summed) pair).  When `q`
 * is given the normalised row is additionally quantised for the next FP8 GEMM
 * (e4m3 + per-128 scales in mie_fp8_quantize's layout; cols % 128 == 0) and
 * `out` may be NULL.  cols % 8 == 0, cols <= 8192.
 */
int mie_rms_norm(const void* x, int64_t ldx, const void* residual, void* summed, const void* weight, void* out,
                 void* q, int64_t ldq, float* scales, int32_t scale_ld, int32_t rows, int32_t cols, float eps,
                 void* stream);

/*
 * Replaces rms_norm on per-head strided rows (engine/kernels/fused.py:178-189:
 * q/k norm over column views of the merged qkv output).  Row r = (r / heads,
 * r % heads) starts at x + (r / heads) * outer_stride + (r % heads) *
 * head_stride; width is 128; out is contiguous [rows_total, 128].
 */
int mie_head_rms_norm(const void* x, int64_t outer_stride, int64_t head_stride, int32_t heads, const void* weight,
                      void* out, int64_t rows_total, float eps, void* stream);

/*
 * Replaces silu_mul (engine/kernels/fused.py:217-233, kernel :127-137):
 * out = bf16(bf16(silu(gate)) * up); gate/up rows share the stride ld_in (column
 * views of the merged gate_up output); out is contiguous.  Optional fused
 * quantisation as in mie_rms_norm.
 */
int mie_silu_mul(const void* gate, const void* up, int64_t ld_in, void* out, void* q, int64_t ldq, float* scales,
                 int32_t scale_ld, int32_t rows, int32_t cols, void* stream);

/*
 * Replaces _rope_kernel / apply_rotary_pos_emb (engine/kernels/fused.py:140-162,
 * :247-262): rotate-half RoPE on x [batch, heads, seq, dim] with cos/sin
 * [batch or 1, seq, dim] (cs_batch_stride 0 broadcasts), each product rounded
 * to bf16 before the add.
 */
int mie_rope(mie_view4_t x, const void* cos, const void* sin, int64_t cs_batch_stride, int64_t cs_token_stride,
             mie_view4_t out, int32_t batch, int32_t heads, int32_t seq, int32_t dim, void* stream);

/*
 * One pass over a merged qkv GEMM output [tokens, (q_heads + 2 kv_heads) * 128]
 * that replaces, for the flat-token paths of PagedQwen3Attention
 * (engine/kv_cache/qwen3_paged.py:191-219 and :244-288): q_norm / k_norm
 * (per-head RMSNorm), apply_rotary_pos_emb, and the KV-cache write
 * (triton_write_decode_kv / triton_write_packed_kv).  cos_sin is a table
 * [max_pos][2][128] (cos row, sin row) indexed by positions[t]; K and V rows go
 * to page block_tables[seq][pos / block_size], slot pos % block_size with seq =
 * token_to_sequence[t] (or t when that pointer is NULL); the normalised, rotated
 * queries go to q_out [tokens, q_heads, 128].
 */
int mie_qkv_norm_rope_write(const void* qkv, int64_t ld, const void* q_weight, const void* k_weight,
                            const void* cos_sin, int32_t max_pos, mie_index_t positions,
                            mie_index_t token_to_sequence, mie_index_t block_tables, void* q_out,
                            mie_view4_t key_blocks, mie_view4_t value_blocks, int32_t tokens, int32_t q_heads,
                            int32_t kv_heads, int32_t block_size, int32_t num_blocks, int32_t table_rows,
                            int32_t table_width, float eps, int32_t* status, void* stream);

/* ------------------------------------------------------------------------
 * lm_head + greedy sampling
 * ---------------------------------------------------------------------- */

/*
 * Replaces the last two operations of the decode step, logits = hidden @
 * lm_head^T in bf16 followed by argmax (engine/model_runner/qwen3_mixed.py:
 * 164-174, engine/serving/chunked_prefill.py:224-229), without writing the
 * [batch, vocab] logits: tokens[b] = the lowest vocabulary index whose bf16
 * logit is the largest of row b.  x [batch, k] bf16 (row stride ldx elements),
 * w [vocab, k] bf16 (row stride ldw elements; a slice of a larger table for a
 * vocabulary-sharded head, whose first row has global index vocab_offset),
 * batch <= 256.  keys: batch uint64 words of device memory owned by the
 * caller that are ZERO on entry; the call leaves them zero again (allocate and
 * clear them once).  tokens: int64 [batch], global indices.  values: NULL, or
 * int32 [batch] receiving an order-preserving key of each winning bf16 logit
 * (what ranks of a sharded head compare).  Base pointers and row strides must
 * be multiples of 16 bytes.  Two launches on the given stream.
 */
int mie_lm_head_argmax(const void* x, int64_t ldx, const void* w, int64_t ldw, int32_t batch, int32_t vocab,
                       int32_t k, int64_t vocab_offset, uint64_t* keys, int64_t* tokens, int32_t* values,
                       int32_t* status, void* stream);

/* ---------------------------------------------------------------------------
 * Tensor-parallel exchange (no counterpart in the reference, which runs on one
 * GPU; these serve the head-sharded TP = 2/4/8 decode step).
 * ------------------------------------------------------------------------- */

#define MIE_TP_MAX_RANKS 8
#define MIE_IPC_HANDLE_BYTES 64

/*
 * Sharing one device buffer between the ranks of a node.  mie_ipc_export fills
 * `handle` (MIE_IPC_HANDLE_BYTES, cudaIpcGetMemHandle of the allocation that
 * contains ptr) and the byte offset of ptr inside that allocation; the bytes
 * travel to the other processes by any host channel.  mie_ipc_open maps a
 * peer's buffer into this process with peer access enabled and returns the
 * address that corresponds to the exported ptr; mie_ipc_close unmaps it.  The
 * exporter must keep the allocation alive while it is mapped elsewhere.
 */
int mie_ipc_export(const void* ptr, uint8_t* handle, int64_t* offset);
int mie_ipc_open(const uint8_t* handle, int64_t offset, void** mapped);
int mie_ipc_close(void* mapped, int64_t offset);

/* Per-rank addresses (entry r = rank r's buffer as mapped in THIS process;
 * entry `rank` is the local buffer). */
typedef struct {
  const void* partial[MIE_TP_MAX_RANKS]; /* row-parallel GEMM output [rows, ld_partial] bf16 */
  void* q[MIE_TP_MAX_RANKS];             /* e4m3 rows [rows, ldq] for the next GEMM, or all NULL */
  float* scales[MIE_TP_MAX_RANKS];       /* their scales [cols / 128, scale_ld] */
  void* normed[MIE_TP_MAX_RANKS];        /* bf16 rows [rows, cols], or all NULL */
  uint32_t* flags[MIE_TP_MAX_RANKS];     /* 2 * MIE_TP_MAX_RANKS words per rank (epochs + a counter), zeroed once */
} mie_tp_peers_t;

/*
 * All-reduce fused into the residual add + RMSNorm (+ quantisation) that
 * follows o_proj / down_proj under tensor parallelism; replaces
 * all_reduce(partial) followed by mie_rms_norm(partial, residual, ...).
 * Rank `rank` owns rows [rank * ceil(rows / tp), ...): for those rows it sums
 * the partial rows of all ranks (fp32, rank order, rounded once to bf16),
 * adds residual (local, [rows, cols], only the owned rows are read), writes
 * the sum to summed (local, owned rows only), normalises with weight / eps
 * and stores the result into EVERY rank's q + scales and/or normed buffers.
 * The kernel first waits until every peer's partial buffer is complete and
 * returns only after every peer's rows have landed locally, so the next launch
 * on the stream may read the whole [rows, cols] result.  state: four zeroed
 * uint32 words of local device memory that belong to this set of flags
 * (epoch, arrival counter, rows landed); all ranks must make the same
 * sequence of calls with the same rows.  Waits give up
 * after max_polls polls (0 = default, about two seconds) and set
 * MIE_STATUS_WAIT_TIMEOUT; no multimem / NVLS, plain peer loads and stores.
 */
int mie_tp_reduce_rms_norm(const mie_tp_peers_t* peers, int32_t tp, int32_t rank, int64_t ld_partial,
                           const void* residual, void* summed, const void* weight, int64_t ldq, int32_t scale_ld,
                           int32_t rows, int32_t cols, float eps, uint32_t* state, uint32_t max_polls,
                           int32_t* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MIE_B200_H_ */
