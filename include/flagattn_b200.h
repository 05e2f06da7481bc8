/*
 * flagattn_b200.h -- C ABI of libflagattn_b200.so
 *
 * Hand-written sm_100a CUDA implementations of the three FlagAttention
 * operators (flash_attention fwd+bwd, piecewise_attention fwd+bwd,
 * paged_attention decode).  Every entry point
 *   - takes raw device pointers, sizes and ELEMENT strides (no torch types),
 *   - enqueues its kernels on the CUDA stream passed as `stream` (a
 *     cudaStream_t cast to void*; NULL = the legacy default stream) on the
 *     device that is current on the calling thread,
 *   - never allocates, never synchronises, never throws,
 *   - returns FA_OK (0) or a negative fa_status.
 * The caller owns all memory.  Inner-most (head_dim) stride is always 1 and
 * every row start must be 16-byte aligned (pointer % 16 == 0, all other
 * strides % 8 == 0 elements); the Python host makes a contiguous copy when a
 * tensor does not satisfy this, exactly where the reference copies when
 * stride(-1) != 1 (src/flag_attn/flash.py:14-17,44).
 *
 * Each declaration cites the reference interface it replaces, by path inside
 * the FlagOpen/FlagAttention project.
 */
#ifndef FLAGATTN_B200_H_
#define FLAGATTN_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum fa_status {
  FA_OK = 0,
  FA_ERR_BAD_ARG = -1,       /* NULL pointer, negative size, bad enum      */
  FA_ERR_UNSUPPORTED = -2,   /* head_dim / dtype / group size not built    */
  FA_ERR_ALIGNMENT = -3,     /* pointer or stride breaks the 16-byte rule  */
  FA_ERR_LAUNCH = -4,        /* cudaGetLastError() != cudaSuccess          */
  FA_ERR_WORKSPACE = -5,     /* workspace pointer missing or too small     */
  FA_ERR_TOO_LARGE = -6      /* request exceeds a fixed built-in capacity  */
} fa_status;

typedef enum fa_dtype { FA_F16 = 0, FA_BF16 = 1 } fa_dtype;

/* A (B, H, L, D) operand with arbitrary b/h/l element strides, d-stride 1.
 * Stride 0: ignored on a dimension of extent 1; on a longer dimension it is a
 * broadcast view (every index reads the same rows, e.g. one K/V head expanded
 * over the query heads, or a prefix shared by the batch) and is honoured for
 * INPUTS: such calls run on the shape-generic kernels, since a TMA tensor map
 * cannot express it.  Outputs must not overlap themselves. */
typedef struct fa_tensor4 {
  void *ptr;
  int64_t stride_b, stride_h, stride_l;
} fa_tensor4;

/* ---------------------------------------------------------------------- */
/* flash_attention                                                         */
/* ---------------------------------------------------------------------- */

/* Problem description shared by all flash entry points.
 * q:(B,H,M,D)  k,v:(B,Hk,N,D), H % Hk == 0, D in {16,32,64,128}.
 * Causal masking is bottom-right aligned: key n is visible to query m iff
 * m + (N - M) >= n  (src/flag_attn/flash.py:37,442). */
typedef struct fa_flash_shape {
  int32_t dtype;     /* fa_dtype of q,k,v,o,do,dq,dk,dv */
  int32_t B, H, Hk, M, N, D;
  int32_t causal;
  float sm_scale;
  /* Dropout on the attention probabilities (flash_attention only; 0 disables it).  Element
   * (b, h, m, n) is kept iff u > dropout_p, u = the first output of Philox-4x32 with 6 rounds,
   * key = philox_seed, counter = philox_offset + ((b*H + h)*M + m)*N + n, mapped to [0, 1);
   * kept probabilities are scaled by 1 / (1 - dropout_p).  Mirrors src/flag_attn/flash.py:52-57,
   * 454-457, 697-721, 877-880; the split-KV entry points reject dropout as the reference does. */
  float dropout_p;
  uint64_t philox_seed, philox_offset;
} fa_flash_shape;

/* Forward: o = softmax(sm_scale * q k^T [+causal]) v, lse = natural-log
 * logsumexp of the scaled masked scores, fp32 (B,H,M) contiguous; rows with
 * no visible key give o = 0, lse = -inf.
 * Replaces the launch of `_fwd_kernel` in FlashAttention.forward
 * (src/flag_attn/flash.py:64-87; kernel :325-489). */
int fa_flash_fwd(const fa_flash_shape *s, const fa_tensor4 *q, const fa_tensor4 *k,
                 const fa_tensor4 *v, const fa_tensor4 *o, float *lse, void *stream);

/* Split-KV forward for small M.  Stage 1 writes, per split, a normalised
 * fp32 partial output (B,H,S,M,D) and its fp32 log-normaliser (B,H,S,M);
 * stage 2 combines them into o and lse.  `n_split_size` keys per split, a
 * multiple of 64.
 * Replaces `_fwd_split_kv_kernel` + `_fwd_combine_kv_splits`
 * (src/flag_attn/split_kv.py:14-227; launches src/flag_attn/flash.py:88-125,
 * src/flag_attn/split_kv.py:295-328). */
int fa_splitkv_fwd(const fa_flash_shape *s, const fa_tensor4 *q, const fa_tensor4 *k,
                   const fa_tensor4 *v, int32_t num_splits, int32_t n_split_size,
                   float *o_partial, float *lse_partial, void *stream);
int fa_splitkv_combine(const fa_flash_shape *s, int32_t num_splits, const float *o_partial,
                       const float *lse_partial, const fa_tensor4 *o, float *lse, void *stream);
/* Bytes of o_partial + lse_partial for a given problem (host-only helper). */
int64_t fa_splitkv_workspace_bytes(const fa_flash_shape *s, int32_t num_splits);

/* The split-count heuristic of the reference, restated
 * (src/flag_attn/split_kv.py:234-262); host-only, no CUDA call. */
int32_t fa_num_splits_heuristic(int32_t B, int32_t H, int32_t M, int32_t N, int32_t block_m,
                                int32_t block_n, int32_t num_sms, int32_t max_splits);

/* total[b,h,n] = sum_m P[m,n] recomputed from lse, fp32 (B,H,N) contiguous.
 * Replaces `_total_attention_kernel` (src/flag_attn/total.py:50-142; launch
 * src/flag_attn/flash.py:128-140). */
int fa_total_attention(const fa_flash_shape *s, const fa_tensor4 *q, const fa_tensor4 *k,
                       const float *lse, float *total, void *stream);

/* delta[b,h,m] = sum_d o*do, fp32 (B,H,M) contiguous.
 * Replaces `_bwd_preprocess` (src/flag_attn/flash.py:522-568, launch :191-202;
 * src/flag_attn/piecewise.py:407-447). */
int fa_flash_bwd_delta(const fa_flash_shape *s, const fa_tensor4 *o, const fa_tensor4 *d_o,
                       float *delta, void *stream);

/* The same, and in the same launch `zero_bytes` bytes at `zero` are filled with zeros (16-byte
 * aligned, a multiple of 16): the workspace of fa_flash_bwd_fused, whose zero-fill is a second
 * memory-bound pass over another buffer; follow it with fa_flash_bwd_fused_stages(..., stages = 6).
 * No counterpart in the reference. */
int fa_flash_bwd_delta_zero(const fa_flash_shape *s, const fa_tensor4 *o, const fa_tensor4 *d_o,
                            float *delta, void *zero, int64_t zero_bytes, void *stream);

/* dk, dv with Hk heads: the sum over the query heads of a GQA group is taken
 * inside the kernel.  Replaces `_bwd_kv_kernel` and the host-side group sum
 * (src/flag_attn/flash.py:204-227,250-251; kernel :571-745). */
int fa_flash_bwd_dkdv(const fa_flash_shape *s, const fa_tensor4 *q, const fa_tensor4 *k,
                      const fa_tensor4 *v, const fa_tensor4 *d_o, const float *lse,
                      const float *delta, const fa_tensor4 *dk, const fa_tensor4 *dv,
                      void *stream);

/* dq, fully overwritten, no atomics.  Replaces `_bwd_q_kernel`
 * (src/flag_attn/flash.py:229-249; kernel :748-909). */
int fa_flash_bwd_dq(const fa_flash_shape *s, const fa_tensor4 *q, const fa_tensor4 *k,
                    const fa_tensor4 *v, const fa_tensor4 *d_o, const float *lse,
                    const float *delta, const fa_tensor4 *dq, void *stream);

/* dk, dv (Hk heads) and dq from ONE pass over the score tiles (head_dim 64 / 128 on the
 * tensor-core path): S and dP are computed once instead of once per kernel.  Replaces the pair
 * of launches `_bwd_kv_kernel` + `_bwd_q_kernel` (src/flag_attn/flash.py:204-249).  dq is
 * accumulated with fp32 global reductions in `workspace` (which also holds the 16 bytes of the
 * persistent kernel's work-item counter), so it is reproducible to fp32 rounding only (dk, dv
 * are bitwise reproducible).  A caller that needs bitwise reproducible
 * gradients (the `_bwd_q_kernel` contract: "no atomics") calls fa_flash_bwd_dkdv + fa_flash_bwd_dq
 * instead: which of the two a process uses is the caller's choice of entry point, nothing else
 * (the Python host chooses by torch.are_deterministic_algorithms_enabled() or
 * flagattention_b200.flash.set_backward_mode()).  A layout that a tensor map cannot express
 * (a broadcast stride) also returns FA_ERR_UNSUPPORTED here; the pair of calls then serves it.
 * fa_flash_bwd_fused_workspace_bytes returns the bytes of device memory `workspace` must hold
 * (16-byte aligned), or 0 when the shape is not covered: then call fa_flash_bwd_dkdv and
 * fa_flash_bwd_dq.  fa_flash_bwd_fused on an uncovered shape returns FA_ERR_UNSUPPORTED, with a
 * missing / short workspace FA_ERR_WORKSPACE. */
int64_t fa_flash_bwd_fused_workspace_bytes(const fa_flash_shape *s);
int fa_flash_bwd_fused(const fa_flash_shape *s, const fa_tensor4 *q, const fa_tensor4 *k,
                       const fa_tensor4 *v, const fa_tensor4 *d_o, const float *lse,
                       const float *delta, const fa_tensor4 *dq, const fa_tensor4 *dk,
                       const fa_tensor4 *dv, void *workspace, int64_t workspace_bytes,
                       void *stream);

/* Regenerates the dropout keep-mask of a flash_attention call: mask[b,h,m,n] (1 byte each,
 * contiguous) = 1 iff the element was kept.  Replaces `recompute_mask_kernel`
 * (src/flag_attn/testing/dropout.py:5-25). */
int fa_dropout_mask(int32_t B, int32_t H, int32_t M, int32_t N, float dropout_p,
                    uint64_t philox_seed, uint64_t philox_offset, uint8_t *mask, void *stream);

/* ---------------------------------------------------------------------- */
/* piecewise_attention                                                     */
/* ---------------------------------------------------------------------- */

/* Score of (m, n) is q2.k2 when (m + N - M) - n >= dist_threshold, else q1.k1
 * (src/flag_attn/piecewise.py:311,328-330).  No GQA: `s->Hk` must equal
 * `s->H`.  Same lse / empty-row conventions as fa_flash_fwd.
 * Replaces `_fwd_kernel` of piecewise (src/flag_attn/piecewise.py:54-69,
 * kernel :223-370). */
int fa_piecewise_fwd(const fa_flash_shape *s, int32_t dist_threshold, const fa_tensor4 *q1,
                     const fa_tensor4 *k1, const fa_tensor4 *q2, const fa_tensor4 *k2,
                     const fa_tensor4 *v, const fa_tensor4 *o, float *lse, void *stream);

/* Replaces piecewise `_bwd_kv_kernel` (src/flag_attn/piecewise.py:114-139,
 * kernel :450-627). */
int fa_piecewise_bwd_dkdv(const fa_flash_shape *s, int32_t dist_threshold, const fa_tensor4 *q1,
                          const fa_tensor4 *k1, const fa_tensor4 *q2, const fa_tensor4 *k2,
                          const fa_tensor4 *v, const fa_tensor4 *d_o, const float *lse,
                          const float *delta, const fa_tensor4 *dk1, const fa_tensor4 *dk2,
                          const fa_tensor4 *dv, void *stream);

/* Replaces piecewise `_bwd_q_kernel` (src/flag_attn/piecewise.py:141-164,
 * kernel :630-792). */
int fa_piecewise_bwd_dq(const fa_flash_shape *s, int32_t dist_threshold, const fa_tensor4 *q1,
                        const fa_tensor4 *k1, const fa_tensor4 *q2, const fa_tensor4 *k2,
                        const fa_tensor4 *v, const fa_tensor4 *d_o, const float *lse,
                        const float *delta, const fa_tensor4 *dq1, const fa_tensor4 *dq2,
                        void *stream);

/* The same call in parts, for callers that time or interleave them: `stages` is a bit mask of
 * 1 = zero-fill of the workspace, 2 = the kernel, 4 = scale and convert the workspace into dq;
 * they must run in that order on one stream.  fa_flash_bwd_fused(...) = stages 7. */
int fa_flash_bwd_fused_stages(const fa_flash_shape *s, const fa_tensor4 *q, const fa_tensor4 *k,
                              const fa_tensor4 *v, const fa_tensor4 *d_o, const float *lse,
                              const float *delta, const fa_tensor4 *dq, const fa_tensor4 *dk,
                              const fa_tensor4 *dv, void *workspace, int64_t workspace_bytes,
                              int32_t stages, void *stream);

/* All five gradients of piecewise_attention from ONE launch: the counterpart of
 * fa_flash_bwd_fused.  Every block of 128 keys is walked twice by the same CTA, first over the
 * query tiles that hold a near pair (q1.k1 -> dq1, dk1), then over those that hold a far pair
 * (q2.k2 -> dq2, dk2); V stays in shared memory and dV accumulates in fp32 across both walks, so
 * it is rounded once.  The workspace holds two dq accumulators:
 * fa_piecewise_bwd_fused_workspace_bytes on the same shape (0 = not covered, use
 * fa_piecewise_bwd_dkdv + fa_piecewise_bwd_dq).  Replaces the pair of launches at
 * src/flag_attn/piecewise.py:114-164.  dq1, dq2 are reproducible to fp32 rounding only. */
int64_t fa_piecewise_bwd_fused_workspace_bytes(const fa_flash_shape *s);
int fa_piecewise_bwd_fused(const fa_flash_shape *s, int32_t dist_threshold, const fa_tensor4 *q1,
                           const fa_tensor4 *k1, const fa_tensor4 *q2, const fa_tensor4 *k2,
                           const fa_tensor4 *v, const fa_tensor4 *d_o, const float *lse,
                           const float *delta, const fa_tensor4 *dq1, const fa_tensor4 *dq2,
                           const fa_tensor4 *dk1, const fa_tensor4 *dk2, const fa_tensor4 *dv,
                           void *workspace, int64_t workspace_bytes, void *stream);

/* ---------------------------------------------------------------------- */
/* paged_attention (single-token decode over a block-table KV cache)       */
/* ---------------------------------------------------------------------- */

typedef struct fa_paged_args {
  int32_t dtype;                 /* fa_dtype of query, caches and out              */
  int32_t num_seqs, num_q_heads, num_kv_heads, head_size, block_size;
  int32_t max_context_len;       /* host upper bound of context_lens               */
  int32_t block_table_is_i64;    /* 0: int32 entries, 1: int64 entries             */
  int32_t partition_size;        /* 0: one pass per (seq, kv head); else tokens    */
                                 /* per split-KV partition, a multiple of 16       */
  float attn_scale;
  const void *query;             /* [num_seqs, num_q_heads, head_size]             */
  int64_t q_stride_s, q_stride_h;
  const void *key_cache;         /* [num_blocks, num_kv_heads, block_size, head]   */
  const void *value_cache;       /* same strides as key_cache                      */
  int64_t kv_stride_b, kv_stride_h, kv_stride_t;
  const int32_t *context_lens;   /* [num_seqs]                                     */
  const void *block_tables;      /* [num_seqs, max_blocks_per_seq]                 */
  int64_t bt_stride_s;
  void *out;                     /* [num_seqs, num_q_heads, head_size]             */
  int64_t o_stride_s, o_stride_h;
  /* split-KV workspace, used only when partition_size > 0; P = number of
   * partitions = ceil(max_context_len / partition_size):                          */
  float *part_out;               /* [num_seqs, num_q_heads, P, head_size] fp32     */
  float *part_max;               /* [num_seqs, num_q_heads, P] fp32, base-2 domain */
  float *part_sum;               /* [num_seqs, num_q_heads, P] fp32                */
  /* Several query tokens per head (0 = one, the decode case of the reference).  With
   * causal_rows = Mq > 0 the query-head axis holds Mq consecutive queries of each head (index =
   * head * Mq + m; num_q_heads counts them all, and num_q_heads / num_kv_heads is a multiple of
   * Mq); they are the LAST Mq tokens of the sequence, so query m sees the tokens below
   * context_len - (Mq - 1 - m): the bottom-right aligned causal mask of fa_flash_fwd for a short
   * query block (src/flag_attn/split_kv.py:14-160 serves these shapes in the reference).  For
   * non-causal attention over several queries leave it 0 and just list the queries as heads. */
  int32_t causal_rows;
} fa_paged_args;

/* Token j of sequence i is read at
 * cache[block_tables[i, j / block_size], kv_head, j % block_size, :]; entries
 * of block_tables past ceil(context_len / block_size) are never read.
 * With partition_size == 0 writes `out`; otherwise writes the workspace for
 * every partition that starts below context_len.
 * Replaces `_paged_attn_kernel` (src/flag_attn/paged.py:56-88,112-143; kernel
 * :194-349). */
int fa_paged_decode(const fa_paged_args *a, void *stream);

/* Combines the partitions written by fa_paged_decode into `out`.
 * Replaces `_paged_attn_v2_reduce_kernel` (src/flag_attn/paged.py:145-162;
 * kernel :352-435). */
int fa_paged_reduce(const fa_paged_args *a, void *stream);

/* Bytes needed for part_out + part_max + part_sum (host-only helper). */
int64_t fa_paged_workspace_bytes(const fa_paged_args *a);

/* Partitioned paged decode that needs no workspace from the caller.  It has no
 * counterpart in the reference, whose wrapper always allocates its split-KV
 * buffers with torch.  It exists for hosts that cannot allocate: a server that
 * handed all free HBM to its KV-cache pool, or a decode loop that must never
 * enter the CUDA allocator.  The partial outputs and softmax statistics live
 * in a fixed FA_PAGED_NOALLOC_SCRATCH_BYTES array inside the library image
 * (held by every GPU that loads the library, until the process exits).
 *   - `a->partition_size` must be > 0; `a->part_out/part_max/part_sum` are
 *     ignored; inputs and `a->out` are the caller's as usual.
 *   - Requests whose workspace (fa_paged_workspace_bytes) exceeds the array
 *     return FA_ERR_TOO_LARGE: at head_size 128 that is more than 32768
 *     (sequence, query head, partition) slots.
 *   - Runs the decode kernel and the reducer on `stream`.  Calls cudaMalloc,
 *     cudaFree or any other allocating routine never.  The first call on each
 *     device resolves the array's device address (cudaGetSymbolAddress); make
 *     that first call before any stream capture begins.
 *   - All calls on a device share the one array, which keeps whatever the
 *     previous call left in it (every slot read is rewritten first, so no
 *     clearing is needed).  Two calls whose kernels overlap on the GPU (for
 *     example on different streams) race on it: serialise them. */
#define FA_PAGED_NOALLOC_SCRATCH_BYTES 17039360 /* 32768 slots x (128 fp32 + 2 fp32) */
int fa_paged_attention_noalloc(const fa_paged_args *a, void *stream);

/* Writer of the caches fa_paged_decode reads: the key / value rows of `num_tokens` new tokens,
 * (num_tokens, kv_heads, head) with element strides (src_stride_t, src_stride_h), go to
 * cache[slot / block_size, :, slot % block_size, :] with slot = slot_mapping[token] (int64);
 * tokens with a negative slot are skipped (padding).  Caches as in fa_paged_args, element
 * strides (cache_stride_b, cache_stride_h, cache_stride_t); key and value (and the two caches)
 * share strides; all strides multiples of 8, pointers 16-byte aligned, head a multiple of 8.
 * The reference only reads such caches (layout: src/flag_attn/testing/paged.py:31-37; its tests
 * and benchmark fill them with random numbers, tests/flag_attn/test_paged_attention.py:44-63);
 * this is the caller-side step that produces them in a serving loop.  Bit-exact copy. */
int fa_paged_cache_append(int32_t dtype, int32_t num_tokens, int32_t num_kv_heads,
                          int32_t head_size, int32_t block_size, const void *key,
                          const void *value, int64_t src_stride_t, int64_t src_stride_h,
                          void *key_cache, void *value_cache, int64_t cache_stride_b,
                          int64_t cache_stride_h, int64_t cache_stride_t,
                          const int64_t *slot_mapping, void *stream);

/* Test hook for "integer block-table indexing is bit-exact": writes, for
 * every (seq, logical block < ceil(context_len / block_size)), the physical
 * block id the decode kernel would gather from into visited[seq, block]
 * (int64, row stride = max_blocks), and -1 elsewhere. */
int fa_paged_trace_blocks(const fa_paged_args *a, int64_t *visited, int32_t max_blocks,
                          void *stream);

/* ---------------------------------------------------------------------- */
/* Producer of piecewise_attention's operands                               */
/* ---------------------------------------------------------------------- */

/* Two rotary position embeddings of one (B, H, L, D) tensor in one pass:
 *   out_e = rotate(x; cos_e, sin_e),  e = 1, 2,
 * where, for rotation pair i of the row at position p (column i of row p of the tables),
 *   lo' = lo * cos[p, i] - hi * sin[p, i],   hi' = hi * cos[p, i] + lo * sin[p, i],
 * and the pair is (x[i], x[i + D/2]) (interleaved = 0) or (x[2i], x[2i + 1]) (interleaved = 1).
 * Tables: fp32, `table_rows` rows of D/2 used columns, `table_stride` elements between rows
 * (a multiple of 4), 16-byte aligned.  positions: int64 (B, L) with row stride pos_stride_b
 * (0 broadcasts one row over the batch), or NULL for p = l; a position outside the tables is
 * clamped to the nearest row.  D a multiple of 16, at most 512; tensors as everywhere (unit
 * inner stride, 16-byte aligned rows).  Every product and sum is rounded to fp32 on its own
 * (no fused multiply-add) and the result rounded once to the 16-bit type, so the output is
 * bit-identical to the plain fp32 expression above.
 * The reference has no such kernel: its README describes the caller's step in prose (two
 * position embeddings applied to q and k, giving q1, q2 and k1, k2: README.md:136-138) and its
 * operator takes the four results (src/flag_attn/piecewise.py:169-191). */
int fa_rotary_pair_fwd(int32_t dtype, int32_t B, int32_t H, int32_t L, int32_t D,
                       int32_t interleaved, const fa_tensor4 *x, const float *cos1,
                       const float *sin1, const float *cos2, const float *sin2,
                       int64_t table_stride, int32_t table_rows, const int64_t *positions,
                       int64_t pos_stride_b, const fa_tensor4 *out1, const fa_tensor4 *out2,
                       void *stream);
/* Its backward: dx = R1^T g1 + R2^T g2 (the rotations by the opposite angles, summed in fp32 in
 * that order, rounded once). */
int fa_rotary_pair_bwd(int32_t dtype, int32_t B, int32_t H, int32_t L, int32_t D,
                       int32_t interleaved, const fa_tensor4 *g1, const fa_tensor4 *g2,
                       const float *cos1, const float *sin1, const float *cos2, const float *sin2,
                       int64_t table_stride, int32_t table_rows, const int64_t *positions,
                       int64_t pos_stride_b, const fa_tensor4 *dx, void *stream);

/* ---------------------------------------------------------------------- */
/* Health check of the tensor-core kernels. Every wait inside them is bounded
 * (about a second); a wait that runs out stores a code naming the wait in a
 * per-device status word, and the kernel tears down and returns instead of
 * hanging.  This call synchronises with the device, copies the word to *out
 * (0 = healthy) and optionally clears it.  The reference has no counterpart:
 * its Triton kernels contain no waits (src/flag_attn/flash.py:325-489). */
int fa_device_status(int32_t *out, int32_t clear);

/* Self-test of that mechanism, for test suites: launches one 64-thread CTA that waits for at
 * most `limit_cycles` SM clocks (1 .. 20,000,000, i.e. at most about 10 ms) on an mbarrier that
 * nobody arrives at, then gives up the way every tensor-core kernel does: status word := 990,
 * abort flag raised, normal return.  *left_flag (device int, may be NULL) is set to 1 when the
 * wait was abandoned.  Until fa_device_status(.., clear = 1) the tensor-core kernels of later
 * calls return without doing any work.  No counterpart in the reference. */
int fa_debug_wait_probe(int64_t limit_cycles, int32_t *left_flag, void *stream);

/* Kernel family used by the flash / piecewise entry points: 0 (default) = tcgen05 kernels where
 * they cover the call (head_dim 64 / 128, no dropout, layouts a tensor map can express), the
 * shape-generic mma.sync kernels elsewhere; 1 = shape-generic kernels only (what the tests use to
 * cross-check the two families); 2 = as 0, but fa_flash_fwd launches one CTA per query tile even
 * where it would run its persistent kernel (calls with more query tiles than two per SM; that
 * kernel keeps its work-item counter in a table of 64 words inside the library, one word per
 * launch in turn, so more than 64 forward launches running at the same moment on one device
 * would share a word).  Process-wide; returns the previous value.  The environment
 * variable FLAGATTN_B200_GENERIC=1 sets the initial value.  No counterpart in the reference. */
int32_t fa_set_kernel_family(int32_t family);

const char *fa_status_string(int status);
/* Library build identification: "flagattn_b200 <n> sm_100a". */
const char *fa_version(void);

#ifdef __cplusplus
}
#endif
#endif /* FLAGATTN_B200_H_ */
