/* C-ABI of libstrix_b200: the B200 (sm_100a) kernels behind libstrix's op
 * surface. Every entry point takes raw device pointers, sizes, element strides
 * and a CUDA stream; none takes a torch type, none synchronises the host and,
 * unless its comment says otherwise, none allocates (scratch is passed in by
 * the caller, sized by the matching *_workspace function).
 *
 * Return value: STRIX_OK, or an error code with a message retrievable through
 * strix_last_error() on the calling thread. A rejected geometry is an error at
 * the call, never a silent wrong answer and never a CPU fallback.
 *
 * Each declaration names the reference launcher it replaces (path inside the
 * asf0/libstrix tree, file:line). */
#ifndef STRIX_B200_H_
#define STRIX_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define STRIX_OK 0
#define STRIX_ERR_INVALID 1 /* argument / geometry check failed */
#define STRIX_ERR_CUDA 2    /* a CUDA runtime call or launch failed */

/* Opaque CUDA stream handle (cudaStream_t). */
typedef void* strix_stream_t;

/* Message of the last failed call made on this thread ("" if none). */
const char* strix_last_error(void);

/* Library version as major * 1000 + minor. */
int strix_version(void);

/* ------------------------------------------------------------------------
 * Paged decode attention, one query token per sequence.
 * Replaces strix::attn_decode_bf16 (csrc/attn/attn_decode_bf16.hip:309-430,
 * schema csrc/torch_ops.cpp:262-265).
 *
 *   q, out        bf16 [nseq, hq, head_dim], element strides (q_st, q_sh) and
 *                 (o_st, o_sh); head_dim contiguous.
 *   key_cache,
 *   value_cache   [blocks, block_size, hkv, >= head_dim] views, last dim
 *                 contiguous, element strides (k_sb, k_ss, k_sh) / (v_sb, ...).
 *                 kv_int8 != 0: int8 bytes (strides multiples of 4) with fp32
 *                 dequant scales k_scale / v_scale [blocks, block_size, hkv]
 *                 (element strides ks_* / vs_*), one per (key, head).
 *                 kv_int8 == 0: bf16 caches, the reference's native form (rows on
 *                 16-byte boundaries: strides multiples of 8; scales NULL), head_dim
 *                 64, 128, 256 or 512, with the same split-KV partials and reduce.
 *   seq_lens      int32 [nseq]; the query sits at position seq_lens[n] - 1.
 *   block_table   int32 [nseq, >= ceil(seq_len / block_size)], row stride bt_stride.
 *   sinks         optional fp32 [hq]: one extra unscaled natural-log logit per
 *                 query head that joins the softmax denominator only.
 *   window_left   >= 0: keys pos - window_left .. pos; -1: all keys.
 *   num_splits    1..64: key segments per sequence, as the reference divides
 *                 them; 0: fixed-length segments of STRIX_DECODE_AUTO_KEYS
 *                 keys (load-balanced over ragged batches; needs max_blocks).
 *   max_blocks    number of usable block_table columns (only read when
 *                 num_splits == 0).
 *   workspace     fp32 scratch of strix_attn_decode_workspace() bytes, or NULL
 *                 when that is 0. Holds un-normalised partial outputs
 *                 [nseq, hq, nseg, head_dim] followed by (m, l) pairs
 *                 [nseq, hq, nseg, 2].
 *
 * Built geometries: head_dim 128 or 256 (int8 caches), 64, 128, 256 or 512 (bf16 caches),
 * hq / hkv in 1..8, block_size a multiple of 16. Others return STRIX_ERR_INVALID.
 * ---------------------------------------------------------------------- */
#define STRIX_DECODE_AUTO_KEYS 1024

/* Number of key segments a call over nseq sequences will use (>= 1), or -1 on bad
 * arguments. num_splits 0: segments of STRIX_DECODE_AUTO_KEYS keys, of half that for
 * a batch so small (nseq x max_blocks x block_size below one wave of such segments)
 * that the SMs would otherwise stay half empty - a shard of a batch spread over
 * several GPUs. strix_attn_decode_segments is the count for a large batch. */
int64_t strix_attn_decode_segments_n(int64_t nseq, int64_t num_splits, int64_t max_blocks,
                                     int64_t block_size);
int64_t strix_attn_decode_segments(int64_t num_splits, int64_t max_blocks,
                                   int64_t block_size);

/* Scratch bytes for the given launch (0 when a single segment is used). */
int64_t strix_attn_decode_workspace(int64_t nseq, int64_t hq, int64_t head_dim,
                                    int64_t num_splits, int64_t max_blocks,
                                    int64_t block_size);

int strix_attn_decode_bf16(
    void* out, const void* q, const void* key_cache, const void* value_cache,
    const float* k_scale, const float* v_scale, const int32_t* seq_lens,
    const int32_t* block_table, const float* sinks, void* workspace,
    int64_t nseq, int64_t hq, int64_t hkv, int64_t head_dim, int64_t block_size,
    int64_t max_blocks, int64_t bt_stride,
    int64_t q_st, int64_t q_sh, int64_t o_st, int64_t o_sh,
    int64_t k_sb, int64_t k_ss, int64_t k_sh,
    int64_t v_sb, int64_t v_ss, int64_t v_sh,
    int64_t ks_sb, int64_t ks_ss, int64_t ks_sh,
    int64_t vs_sb, int64_t vs_ss, int64_t vs_sh,
    double scale, int64_t num_splits, int64_t window_left, int kv_int8,
    strix_stream_t stream);

/* ------------------------------------------------------------------------
 * MoE layer: router, permutation, activation quantisers, expert GEMMs, combine.
 * ---------------------------------------------------------------------- */

/* Router: fp32 softmax over `experts` -> top_k (ties: lower expert index) ->
 * weights p_i / sum of selected p (renormalize != 0) or p_i. Not in the
 * reference (vLLM's fused_topk on its call path, python/strix_vllm/moe.py);
 * defined by the benchmark configuration's "softmax then top-k then
 * renormalise". logits fp32 [tokens, experts] (row stride logits_stride),
 * topk_ids int32 [tokens, top_k], topk_weights fp32 [tokens, top_k]. */
int strix_moe_topk_softmax(const float* logits, int32_t* topk_ids, float* topk_weights,
                           int64_t tokens, int64_t experts, int64_t top_k,
                           int64_t logits_stride, int renormalize, strix_stream_t stream);

/* Entries sorted_ids must hold for strix_moe_align (a multiple of block_m). */
int64_t strix_moe_align_capacity(int64_t numel, int64_t experts, int64_t block_m);

/* Permutation with the moe_align_block_size contract that the reference's
 * kernels consume (csrc/moe/moe_gemm_w8a16.hip:110-123) and its tests restate
 * (tests/test_moe_gemm.py:9-31): slot ids (0 .. numel-1) grouped by expert in
 * ascending expert and ascending slot order, each expert's run padded to
 * block_m with the invalid id `numel`; experts without tokens get no block;
 * *num_post_padded = total padded length. Everything after it is filled:
 * sorted_ids with `numel`, expert_ids with -1 (a block the GEMMs skip). Ids
 * outside [0, experts) are ignored (not routed here). */
int strix_moe_align(const int32_t* topk_ids, int32_t* sorted_ids, int32_t* expert_ids,
                    int32_t* num_post_padded, int64_t numel, int64_t experts, int64_t block_m,
                    int64_t sorted_capacity, int64_t expert_capacity, strix_stream_t stream);

/* Per (row, 128-element group) symmetric int8 quantiser: s = amax / 127 (1 for
 * an all-zero group), q = clamp(rint(x * (1 / s)), +-127). Replaces
 * strix::moe_act_quant_i8 (csrc/moe/moe_gemm_w4a8.hip:283-348). x bf16 (or fp16
 * when x_is_f16) [rows, k], q int8 [rows, k], sa fp32 [rows, k / 128]. */
int strix_moe_act_quant_i8(const void* x, void* q, float* sa, int64_t rows, int64_t k,
                           int64_t x_stride, int64_t q_stride, int64_t sa_stride, int x_is_f16,
                           strix_stream_t stream);

/* As above to float8_e4m3fn: s = amax / 448 (1 for an all-zero group), q =
 * e4m3(x / s), round to nearest even. No counterpart in the reference (its FP8
 * experts take 16-bit activations); this is the activation form of the
 * benchmark's W8A8 configuration. */
int strix_moe_act_quant_fp8(const void* x, void* q, float* sa, int64_t rows, int64_t k,
                            int64_t x_stride, int64_t q_stride, int64_t sa_stride, int x_is_f16,
                            strix_stream_t stream);

/* Grouped expert GEMM over the moe_align layout. Replaces moe_gemm_bf16
 * (csrc/moe/moe_gemm_bf16.hip:298), moe_gemm_w8a16 / moe_gemm_fp8 /
 * moe_gemm_fp8_raw (csrc/moe/moe_gemm_w8a16.hip:581-623) and adds the W8A8 FP8
 * form. c[sid, :] is written only for valid sorted ids (sid < num_valid).
 *   weight_format  0 float8_e4m3fn, 1 int8, 2 bf16        w [experts, n, k]
 *   act_format     0 bf16, 1 fp16, 2 float8_e4m3fn (+ act_scales fp32 [a_rows, k/128])
 *   scale_kind     0 none, 1 per output channel [E, N], 2 block fp32 [E, N/128, K/128]
 *   scale_dtype    0 fp32, 1 bf16, 2 fp16
 *   gate_act       0: c[sid, n] = (a W^T)[n] * topk_weights[sid] (1 if NULL), c is [*, n]
 *                  1 silu / 2 gelu_tanh: W rows are [gate; up], c[sid, j] =
 *                  act(gate_j) * up_j, c is [*, n / 2]
 * Strides are in elements. k must be a multiple of 128, n of 16. */
int strix_moe_gemm(
    void* c, const void* a, const void* w, const void* scales, const float* act_scales,
    const int32_t* sorted_ids, const int32_t* expert_ids, const int32_t* num_post_padded,
    const float* topk_weights, int64_t num_valid, int64_t a_rows, int64_t experts, int64_t n,
    int64_t k, int64_t a_stride, int64_t c_stride, int64_t w_stride_e, int64_t w_stride_n,
    int64_t s_stride_e, int64_t s_stride_n, int64_t sa_stride, int64_t sorted_len,
    int64_t expert_len, int64_t top_k, int64_t block_m, int weight_format, int act_format,
    int scale_kind, int scale_dtype, int gate_act, int c_is_f16, strix_stream_t stream);

/* Combine: out[t, :] = sum over j of in[t, j, :] in fp32, one bf16 rounding
 * (vLLM's moe_sum on the reference's call path, python/strix_vllm/moe.py:1012-1014;
 * routing weights were already applied by the down GEMM). bf16 in [tokens,
 * top_k, hidden] (strides in_st, in_sj), bf16 out [tokens, hidden]. */
int strix_moe_sum(const void* in, void* out, int64_t tokens, int64_t top_k, int64_t hidden,
                  int64_t in_st, int64_t in_sj, int64_t out_st, strix_stream_t stream);

/* Layout probe of the tcgen05 path: one CTA computes D[128, n] = A[128, k] *
 * B[n, k]^T from row-major 8-bit operands (kind 0: int8 -> int32 D, bit-exact;
 * kind 1: float8_e4m3fn -> fp32 D). Plays the role of the reference's
 * _wmma_bf16_tile (csrc/testing/wmma_layout_test.hip:27, schema
 * csrc/torch_ops.cpp:183). *status (device int32, zeroed by the caller) is set
 * to 1 if a bounded wait inside the kernel ran out. */
int strix_umma_tile(void* d, const void* a, const void* b, int32_t* status, int64_t n, int64_t k,
                    int kind, strix_stream_t stream);

/* ------------------------------------------------------------------------
 * Dense quantized GEMMs.
 * ---------------------------------------------------------------------- */

/* W8A8 INT8 GEMM with per-token and per-channel scales:
 *   out[m, n] = bf16((sum_k a_q[m, k] * w[n, k]) * a_scale[m] * w_scale[n])
 * a_q int8 [m, k] (row stride a_stride), w int8 [n, k] (row stride w_stride),
 * scales fp32, out bf16 [m, n] (row stride out_stride). The sum is exact in
 * int32; acc_out, when not NULL, receives it ([m, n] int32, row stride
 * out_stride). k must be a multiple of 128. This is the per-token form of the
 * reference's w8a8_wmma_gemm (csrc/gemm/w8a8_wmma_gemm.hip:15-22, :799-918,
 * which quantises the activations per 128-wide group inside the op); runs on
 * tcgen05 kind::i8. */
int strix_w8a8_int8_gemm(void* out, int32_t* acc_out, const void* a_q, const float* a_scale,
                         const void* w, const float* w_scale, int64_t m, int64_t n, int64_t k,
                         int64_t a_stride, int64_t w_stride, int64_t out_stride,
                         strix_stream_t stream);

/* ------------------------------------------------------------------------
 * Prefill attention: causal paged flash attention over ragged sequences.
 * Replaces strix::attn_prefill_bf16 (csrc/attn/attn_prefill_bf16.hip:508-662;
 * schema csrc/torch_ops.cpp:240-244; wrapper python/strix/__init__.py:214-268).
 *   q, out        bf16 [total_q, hq, head_dim]; the queries of sequence n are
 *                 rows cu_seqlens_q[n] .. cu_seqlens_q[n + 1] and hold the LAST
 *                 q_len of its seq_lens[n] positions.
 *   key_cache, value_cache, k_scale, v_scale, block_table, sinks, window_left:
 *                 as strix_attn_decode_bf16 (int8 caches with fp32 scales per
 *                 key and head, or bf16 caches).
 *   num_splits    1..64, accepted for the reference's signature: the result
 *                 does not depend on it and this kernel always runs one pass.
 *                 sinks need num_splits == 1 (the reference's rule and message).
 * The reference's tile_offsets / max_tiles arguments are not needed: the grid is
 * sized from total_q and nseq. Built: head_dim 64, 128, 256 and 512, any hq / hkv ratio.
 * ---------------------------------------------------------------------- */
int strix_attn_prefill_bf16(void* out, const void* q, const void* key_cache,
                            const void* value_cache, const float* k_scale, const float* v_scale,
                            const int32_t* cu_seqlens_q, const int32_t* seq_lens,
                            const int32_t* block_table, const float* sinks, int64_t total_q,
                            int64_t nseq, int64_t hq, int64_t hkv, int64_t head_dim,
                            int64_t block_size, int64_t bt_stride, int64_t q_stride_t,
                            int64_t q_stride_h, int64_t out_stride_t, int64_t out_stride_h,
                            int64_t k_stride_b, int64_t k_stride_s, int64_t k_stride_h,
                            int64_t v_stride_b, int64_t v_stride_s, int64_t v_stride_h,
                            int64_t ks_stride_b, int64_t ks_stride_s, int64_t ks_stride_h,
                            int64_t vs_stride_b, int64_t vs_stride_s, int64_t vs_stride_h,
                            double scale, int64_t num_splits, int64_t window_left, int kv_int8,
                            strix_stream_t stream);

/* Decode attention through the prefill kernel, for the geometries of
 * strix_attn_decode_bf16 that have no split-KV kernel (int8 caches at head_dim 64 or
 * 512, hq / hkv above 8): same arguments as strix_attn_prefill_bf16, but the rows
 * cu_seqlens_q[n] .. cu_seqlens_q[n + 1] of sequence n are the G = hq_model / hkv query
 * heads that share one KV head, ALL at position seq_lens[n] - 1 (no causal order among
 * them). The caller regroups q and out to [nseq * G, hkv, head_dim] (row n * G + g,
 * head h = query head h * G + g) and passes hq = hkv; a KV head is then read once per
 * sequence. sinks stays fp32 [hkv * G] in query-head order. One pass, no split-KV. */
int strix_attn_decode_grouped_bf16(void* out, const void* q, const void* key_cache,
                                   const void* value_cache, const float* k_scale,
                                   const float* v_scale, const int32_t* cu_seqlens_q,
                                   const int32_t* seq_lens, const int32_t* block_table,
                                   const float* sinks, int64_t total_q, int64_t nseq, int64_t hq,
                                   int64_t hkv, int64_t head_dim, int64_t block_size,
                                   int64_t bt_stride, int64_t q_stride_t, int64_t q_stride_h,
                                   int64_t out_stride_t, int64_t out_stride_h, int64_t k_stride_b,
                                   int64_t k_stride_s, int64_t k_stride_h, int64_t v_stride_b,
                                   int64_t v_stride_s, int64_t v_stride_h, int64_t ks_stride_b,
                                   int64_t ks_stride_s, int64_t ks_stride_h, int64_t vs_stride_b,
                                   int64_t vs_stride_s, int64_t vs_stride_h, double scale,
                                   int64_t num_splits, int64_t window_left, int kv_int8,
                                   strix_stream_t stream);

/* Grouped or dense GEMM with 4-bit weights and bf16 activations, on the
 * weight-streaming kernel. Replaces moe_gemm_w4a16 (csrc/moe/moe_gemm_w4a16.hip:374),
 * w4a16_wmma_gemm, mxfp4_wmma_gemm / mxfp4_gemv (csrc/gemm/mxfp4_wmma_gemm.hip:355-372,
 * csrc/gemm/mxfp4_gemv.hip:111) and adds the grouped MXFP4 form.
 *   weight_format 3: MXFP4 - w uint8 [E, N, K/2] (byte j: k = 2j in the low
 *     nibble), scales uint8 e8m0 [E, N, K/32] (byte 0 = zero block), group 32
 *   weight_format 4: INT4 - value = nibble - 8, scales bf16 (scale_dtype 1) or
 *     fp16 (2) [E, N, K/group], group 32, 64 or 128
 * K must be a multiple of 32 (a partial last 128-block is zero-filled).
 * Routing as in strix_moe_gemm; with sorted_ids, expert_ids and
 * num_post_padded all NULL the call is a dense GEMM: slot i is row i of a (a_rows
 * = num_valid = M, experts = 1, sorted_len = M rounded up to block_m). bias (bf16,
 * bias[row * bias_stride + n], stride 0 for a per-channel bias) is added to plain
 * outputs. Strides are in elements of the tensors as stored. */
int strix_gemm_w4a16(void* c, const void* a, const void* w, const void* scales, const void* bias,
                     const int32_t* sorted_ids, const int32_t* expert_ids,
                     const int32_t* num_post_padded, const float* topk_weights, int64_t num_valid,
                     int64_t a_rows, int64_t experts, int64_t n, int64_t k, int64_t a_stride,
                     int64_t c_stride, int64_t w_stride_e, int64_t w_stride_n, int64_t s_stride_e,
                     int64_t s_stride_n, int64_t bias_stride, int64_t sorted_len,
                     int64_t expert_len, int64_t top_k, int64_t block_m, int weight_format,
                     int group, int scale_dtype, int gate_act, strix_stream_t stream);

/* Dense GEMM c = x W^T (+ bias) with 8-bit weights and 16-bit activations on the
 * weight-streaming kernel. Replaces w8a16_skinny_gemm / fp8_skinny_gemm
 * (csrc/gemm/w8a16_skinny_gemm.hip:761,768) and fp8_wmma_gemm[_raw]
 * (csrc/gemm/fp8_wmma_gemm.hip:324-344).
 *   weight_format 0 e4m3, 1 int8, 5 excess-128 bytes (value = byte - 128)
 *   act_format    0 bf16, 1 fp16 (e4m3 weights only; exact weights, scaled sums)
 *   scale_kind    1 per channel [N]; 2 fp32 blocks [ceil(N/128), K/128] (e4m3);
 *                 3 per row and K group [N, K/group]; s_stride_n = row stride
 *   group         K elements per scale for scale_kind 3: 128 (or 0), and 32 / 64 with
 *                 bf16 activations (csrc/gemm/w8a16_skinny_gemm.hip:420-426)
 * c bf16 [m, n]; K a multiple of 128, N of 16. */
int strix_dense_gemm_w8a16(void* c, const void* x, const void* w, const void* scales,
                           const void* bias, int64_t m, int64_t n, int64_t k, int64_t x_stride,
                           int64_t c_stride, int64_t w_stride, int64_t s_stride_n,
                           int64_t bias_stride, int64_t block_m, int weight_format,
                           int act_format, int scale_kind, int scale_dtype, int group, strix_stream_t stream);

/* bf16 rows into sorted order by scatter: row t of x [tokens, k] is copied to
 * the sorted positions slot_pos[t * top_k + j]; padding slots below
 * *num_post_padded get zeros. y bf16 [rows, k]. The input layout of
 * strix_moe_gemm_mxfp4_sorted. No counterpart in the reference (its kernels
 * gather token rows inside the GEMM). */
int strix_moe_permute_bf16(const void* x, void* y, const int32_t* slot_pos,
                           const int32_t* sorted_ids, const int32_t* num_post_padded,
                           int64_t tokens, int64_t rows, int64_t k, int64_t top_k,
                           int64_t x_stride, int64_t y_stride, strix_stream_t stream);

/* MXFP4 grouped expert GEMM on tcgen05 (bf16 x bf16 -> f32 MMAs over weights
 * decoded to bf16 on the way, exact) for m-blocks of 128 tokens, over bf16
 * activations in sorted order (row p of a = sorted position p). w uint8 [E, N,
 * K/2], scales e8m0 [E, N, K/32] as in strix_gemm_w4a16; epilogues, gate_act and
 * c_sorted as in strix_moe_gemm_fp8_sorted. K a multiple of 64, output width a
 * multiple of 32 (tiles of 256 weight rows, 128 + 128 under the gate; a ragged
 * last tile is zero-filled and masked); ..._covers() tells (1/0). The
 * tensor-bound form of the new moe_gemm_mxfp4 op. */
int strix_moe_gemm_mxfp4_sorted(void* c, const void* a, const void* w, const void* scales,
                                const int32_t* sorted_ids, const int32_t* expert_ids,
                                const int32_t* num_post_padded, const float* topk_weights,
                                int64_t num_valid, int64_t num_experts, int64_t n, int64_t k,
                                int64_t a_stride, int64_t c_stride, int64_t w_stride_e,
                                int64_t w_stride_n, int64_t s_stride_e, int64_t s_stride_n,
                                int64_t sorted_len, int64_t block_m, int gate_act, int c_sorted,
                                strix_stream_t stream);
int strix_moe_gemm_mxfp4_sorted_covers(int64_t n, int64_t k, int64_t block_m, int gate_act);

/* Grouped or dense GEMM with int8 activations (qa int8 [rows, k], sa fp32 [rows,
 * k/128], the output of strix_moe_act_quant_i8): s8 x s8 MMAs, sums exact in
 * int32 per 128-wide K group, folded in fp32 with sa * weight scale. Replaces
 * moe_gemm_w4a8 (csrc/moe/moe_gemm_w4a8.hip:374, kernel :57-277) and the GEMM
 * half of w8a8_wmma_gemm (csrc/gemm/w8a8_wmma_gemm.hip:799-918).
 *   weight_format 4: int4 [E, N, K/2] (nibble - 8); 5: excess-128 bytes [E, N, K]
 *   scale_kind 1: per channel [E, N]; 3: per (row, group), element strides
 *   s_stride_n over rows and s_stride_g over groups (so [N, K/128] and
 *   [K/128, N] are both taken in place); scale_dtype 0 fp32, 1 bf16, 2 fp16.
 * Routing as in strix_moe_gemm, or all three routing pointers NULL for a dense
 * GEMM (see strix_gemm_w4a16). c bf16. */
int strix_gemm_w8a8_group(void* c, const void* qa, const float* sa, const void* w,
                          const void* scales, const int32_t* sorted_ids, const int32_t* expert_ids,
                          const int32_t* num_post_padded, const float* topk_weights,
                          int64_t num_valid, int64_t a_rows, int64_t experts, int64_t n, int64_t k,
                          int64_t a_stride, int64_t c_stride, int64_t w_stride_e, int64_t w_stride_n,
                          int64_t s_stride_e, int64_t s_stride_n, int64_t s_stride_g,
                          int64_t sa_stride, int64_t sorted_len, int64_t expert_len, int64_t top_k,
                          int64_t block_m, int weight_format, int scale_kind, int scale_dtype,
                          int gate_act, strix_stream_t stream);

/* Whole-matrix decode to bf16 [n, k], byte-exact. Replaces mxfp4_dequant
 * (csrc/gemm/mxfp4_wmma_gemm.hip), w4a16_dequant and fp8_dequant
 * (csrc/gemm/fp8_dequant.hip:63). format 0 mxfp4 (w [n, k/2], scales e8m0
 * [n, k/32]), 1 int4 (scales bf16/fp16 [n, k/group]), 2 e4m3 (w [n, k], scales
 * fp32 per channel [n] = scale_kind 1, or [ceil(n/128), k/128] = scale_kind 2).
 * s_stride_n / s_stride_g: element strides of the scale tensor over rows (row
 * blocks for scale_kind 2) and K groups. */
int strix_dequant_bf16(void* out, const void* w, const void* scales, int64_t n, int64_t k,
                       int64_t w_stride, int64_t out_stride, int64_t s_stride_n, int64_t s_stride_g,
                       int format, int group, int scale_kind, int scale_dtype,
                       strix_stream_t stream);

/* Dynamic per-token int8 quantisation of activations, the input form of
 * strix_w8a8_int8_gemm: x bf16 (fp16 if in_f16) [rows, k] -> q int8 [rows, k],
 * scales fp32 [rows] with scale = absmax / 127 (1 for an all-zero row), q =
 * rint(x / scale). The reference's w8a8_wmma_gemm quantises per 128 group inside
 * its GEMM (csrc/gemm/w8a8_wmma_gemm.hip:508-529); this is the per-token rule of
 * benchmark config 2 and of vLLM's int8 scaled-MM contract. Strides in elements. */
int strix_act_quant_token_i8(const void* x, void* q, float* scales, int64_t rows, int64_t k,
                             int64_t x_stride, int64_t q_stride, int in_f16,
                             strix_stream_t stream);

/* Health of the tcgen05 kernels: *host_out = 0 while every launch so far met its
 * bounded waits, 1 after one of them gave up (its output is then incomplete: the
 * CTA stopped, waited for its own copies and MMAs in flight, freed tensor memory
 * and returned). Synchronises the device. The launches themselves never report
 * it - a caller polls this word at a point where it synchronises anyway (the
 * Python ops do so after every call when STRIX_CHECK_STATUS=1). No reference
 * counterpart. */
int strix_umma_status(int32_t* host_out);

/* The FP8 activation quantiser writing the SORTED layout the tcgen05 grouped
 * GEMM reads: output row p (p < *num_post_padded, p < rows) holds the quantised
 * input row sorted_ids[p] / top_k, or zeros with scale 1 for a padding slot
 * (sorted_ids[p] >= num_valid). With sorted_ids == NULL the rows are quantised
 * in place order (row p from row p) and only the bound by *num_post_padded
 * applies - the form used between the two GEMMs. q e4m3 [rows, k], sa fp32
 * [rows, k / 128]. No counterpart in the reference, whose kernels gather token
 * rows inside the GEMM (csrc/moe/moe_gemm_w8a16.hip:128-160). */
int strix_moe_act_quant_fp8_sorted(const void* x, void* q, float* sa, const int32_t* sorted_ids,
                                   const int32_t* num_post_padded, int64_t rows, int64_t k,
                                   int64_t top_k, int64_t num_valid, int64_t x_stride,
                                   int64_t q_stride, int64_t sa_stride, int x_is_f16,
                                   strix_stream_t stream);

/* strix_moe_align that also writes the inverse permutation: slot_pos[i] = the
 * sorted position of slot i (int32 [numel]; -1 for an id outside 0..experts-1).
 * slot_pos may be NULL. */
int strix_moe_align_pos(const int32_t* topk_ids, int32_t* sorted_ids, int32_t* expert_ids,
                        int32_t* num_post_padded, int32_t* slot_pos, int64_t numel,
                        int64_t experts, int64_t block_m, int64_t sorted_capacity,
                        int64_t expert_capacity, strix_stream_t stream);

/* strix_moe_align_counts for large batches: with a scratch of
 * strix_moe_align_scratch_bytes(numel, experts) bytes (4-byte aligned, contents
 * irrelevant) the slots are walked once per pass by one CTA per 1024 slots instead
 * of once per expert - two launches, the same output bit for bit. Falls back to the
 * one-kernel form for up to 4096 slots, more than 1024 experts or scratch == NULL. */
int64_t strix_moe_align_scratch_bytes(int64_t numel, int64_t experts);
int strix_moe_align_scratch(const int32_t* topk_ids, int32_t* sorted_ids, int32_t* expert_ids,
                            int32_t* num_post_padded, int32_t* slot_pos, int32_t* counts,
                            void* scratch, int64_t scratch_bytes, int64_t numel, int64_t experts,
                            int64_t block_m, int64_t sorted_capacity, int64_t expert_capacity,
                            strix_stream_t stream);

/* strix_moe_align_pos that also writes counts[e] = slots routed to expert e
 * (int32 [experts]; NULL to skip). With the destination rank as the "expert" and
 * block_m = 1 this is the dispatch plan of the expert-parallel path. */
int strix_moe_align_counts(const int32_t* topk_ids, int32_t* sorted_ids, int32_t* expert_ids,
                           int32_t* num_post_padded, int32_t* slot_pos, int32_t* counts,
                           int64_t numel, int64_t experts, int64_t block_m,
                           int64_t sorted_capacity, int64_t expert_capacity,
                           strix_stream_t stream);

/* Expert-parallel helpers (no counterpart in the reference, which has no EP).
 * strix_ep_pack: send[i] = x[order[i] / top_k] (bf16 rows of `hidden`), meta[i *
 * meta_stride] = (topk_ids[order[i]] % experts_per_rank as float,
 * topk_weights[order[i]]); meta_stride counts floats (2 for a dense [slots, 2]
 * array; pointing meta at the padded tail of the send rows lets one collective
 * carry both).
 * strix_moe_sum_gather: out[t] = sum_j rows[pos[t * top_k + j]] in fp32, one bf16
 * rounding (negative positions are skipped). */
int strix_ep_pack(const void* x, void* send, float* meta, const int32_t* order,
                  const int32_t* topk_ids, const float* topk_weights, int64_t slots,
                  int64_t hidden, int64_t top_k, int64_t experts_per_rank, int64_t x_stride,
                  int64_t send_stride, int64_t meta_stride, strix_stream_t stream);
int strix_moe_sum_gather(const void* rows, const int32_t* pos, void* out, int64_t tokens,
                         int64_t top_k, int64_t hidden, int64_t row_st, int64_t out_st,
                         strix_stream_t stream);

/* The sorted-layout e4m3 quantiser by scatter: token row t of x [tokens, k] is
 * quantised once and stored at the sorted positions slot_pos[t * top_k + j] of
 * its top_k slots; padding slots below *num_post_padded get zeros with scale 1.
 * Same result as strix_moe_act_quant_fp8_sorted with sorted_ids, top_k times
 * less reading and arithmetic. q e4m3 [rows, k], sa fp32 [rows, k / 128]. */
int strix_moe_act_quant_fp8_scatter(const void* x, void* q, float* sa, const int32_t* slot_pos,
                                    const int32_t* sorted_ids, const int32_t* num_post_padded,
                                    int64_t tokens, int64_t rows, int64_t k, int64_t top_k,
                                    int64_t x_stride, int64_t q_stride, int64_t sa_stride,
                                    int x_is_f16, strix_stream_t stream);

/* FP8 W8A8 grouped expert GEMM on tcgen05 over activations in sorted order
 * (row p of a / act_scales = sorted position p; see above). Arithmetic and
 * epilogues are those of strix_moe_gemm with weight_format 0, act_format 2,
 * fp32 scales (scale_kind 1 channel [E, N] or 2 block [E, N/128, K/128]);
 * gate_act 0 none (c[row, n] times topk_weights[sid] if given), 1 silu, 2
 * gelu_tanh (c is [*, n / 2]). c_sorted != 0 writes output row p for every
 * sorted position of the processed m-blocks (padding rows included), else row
 * sorted_ids[p] for valid slots only - the contract of the reference's
 * moe_gemm_fp8 (csrc/moe/moe_gemm_w8a16.hip:581-623). sorted_len counts whole
 * m-blocks; num_experts is the first extent of w (m-blocks whose expert id is
 * negative or >= num_experts are skipped). strix_moe_gemm_fp8_sorted_covers()
 * tells (1/0) whether a geometry is covered; uncovered ones are rejected. */
int strix_moe_gemm_fp8_sorted(void* c, const void* a, const float* act_scales, const void* w,
                              const float* scales, const int32_t* sorted_ids,
                              const int32_t* expert_ids, const int32_t* num_post_padded,
                              const float* topk_weights, int64_t num_valid, int64_t num_experts,
                              int64_t n, int64_t k,
                              int64_t a_stride, int64_t c_stride, int64_t w_stride_e,
                              int64_t w_stride_n, int64_t s_stride_e, int64_t s_stride_n,
                              int64_t sa_stride, int64_t sorted_len, int64_t block_m,
                              int scale_kind, int gate_act, int c_sorted, strix_stream_t stream);
int strix_moe_gemm_fp8_sorted_covers(int64_t n, int64_t k, int64_t block_m, int gate_act,
                                     int scale_kind);

/* One call for a whole FP8 W8A8 MoE layer over the sorted-layout tcgen05 kernels:
 * [router ->] permute + quantise -> gate-up GEMM with the fused gate -> quantise ->
 * down GEMM x routing weight -> sum over top-k, the sequence of the reference's
 * StrixFp8Experts.apply (python/strix_vllm/moe.py:905-1014), enqueued on `stream`
 * without allocation or synchronisation. Pass either `logits` (fp32 [tokens,
 * experts], row stride logits_stride: softmax -> top-k -> renormalise runs first)
 * or the routing itself (topk_weights fp32 / topk_ids int32, contiguous [tokens,
 * top_k]). x bf16 [tokens, hidden]; w13 e4m3 [experts, 2 inter, hidden], w2 e4m3
 * [experts, hidden, inter] with fp32 scales (scale_kind 1 channel [E, N], 2 block
 * [E, N/128, K/128]; strides in elements); out bf16 [tokens, hidden]. gate_act 1
 * silu, 2 gelu_tanh. workspace: 256-byte aligned, at least
 * strix_moe_fp8_layer_workspace(...) bytes. */
int64_t strix_moe_fp8_layer_workspace(int64_t tokens, int64_t top_k, int64_t hidden,
                                      int64_t inter, int64_t experts, int64_t block_m);
int strix_moe_fp8_layer(void* out, const void* x, const float* logits, const float* topk_weights,
                        const int32_t* topk_ids, const void* w13, const float* w13_scale,
                        const void* w2, const float* w2_scale, void* workspace,
                        int64_t workspace_bytes, int64_t tokens, int64_t hidden, int64_t inter,
                        int64_t experts, int64_t top_k, int64_t block_m, int64_t x_stride,
                        int64_t logits_stride, int64_t out_stride, int64_t w13_stride_e,
                        int64_t w13_stride_n, int64_t s13_stride_e, int64_t s13_stride_n,
                        int64_t w2_stride_e, int64_t w2_stride_n, int64_t s2_stride_e,
                        int64_t s2_stride_n, int scale_kind, int gate_act, strix_stream_t stream);

/* The experts of that layer over rows that ARRIVE quantised, with slots that may be
 * masked (expert id < 0 or >= experts): the receiving side of the expert-parallel
 * exchange below, in one call (align -> permute payload rows -> gate-up GEMM ->
 * quantise -> down GEMM x routing weight). rows_payload [rows, row_stride_bytes]:
 * hidden e4m3 bytes, then hidden / 128 fp32 scales, rows padded to 16 bytes;
 * topk_ids / topk_weights contiguous [rows, top_k]; y bf16 [rows * top_k, hidden]
 * receives the weighted rows in slot order (rows of masked slots are not written).
 * Same workspace as strix_moe_fp8_layer for tokens = rows. */
int strix_moe_fp8_experts_on_rows(void* y, const void* rows_payload, const float* topk_weights,
                                  const int32_t* topk_ids, const void* w13, const float* w13_scale,
                                  const void* w2, const float* w2_scale, void* workspace,
                                  int64_t workspace_bytes, int64_t rows, int64_t hidden,
                                  int64_t inter, int64_t experts, int64_t top_k, int64_t block_m,
                                  int64_t row_stride_bytes, int64_t y_stride, int64_t w13_stride_e,
                                  int64_t w13_stride_n, int64_t s13_stride_e, int64_t s13_stride_n,
                                  int64_t w2_stride_e, int64_t w2_stride_n, int64_t s2_stride_e,
                                  int64_t s2_stride_n, int scale_kind, int gate_act,
                                  strix_stream_t stream);

/* ---- Expert-parallel exchange over peer memory (no counterpart in the
 * reference, whose experts refuse an expert_map: python/strix_vllm/moe.py:193-210).
 * Buffers are plain device allocations that peers map through CUDA IPC:
 * strix_peer_alloc (zero-filled cudaMalloc) / _free, _export (64-byte handle) /
 * _import / _unimport. Per rank: recv [world][cap][row_bytes], meta
 * [world][cap][1 + 2 top_k] int32, counts [world], flags [world], ret
 * [world][cap][hidden] bf16, rflags [world]; `peer_*` arguments are host arrays of
 * `world` device pointers, entry d = rank d's buffer as addressable from this
 * rank. `epoch` must grow by one per layer on every rank; `ticket` is one zeroed
 * int32 of this rank. spin_limit bounds the waits (0 = about two seconds); a wait
 * that runs out raises strix_ep_status (1 dispatch, 2 return) and the kernel goes
 * on with empty input instead of hanging.
 *   strix_ep_plan      tok_pos [world][tokens] (index of token t among this rank's
 *                      tokens with a slot on rank d, or -1), counts [world]
 *   strix_ep_dispatch  payload row (row_bytes, a multiple of 16) and metadata of
 *                      every token to each rank it has a slot on, then counts and
 *                      flags (release, system scope)
 *   strix_ep_prepare   receiver: waits for all sources, writes ids int32 / weights
 *                      fp32 [world * cap, top_k] (-1 / 0 where nothing arrived) and
 *                      optionally rows_per_source [world]
 *   strix_ep_return    expert rank: y bf16 [world * cap * top_k, hidden] in slot
 *                      order -> one fp32-summed bf16 row per received token into
 *                      the source's ret region, then rflags
 *   strix_ep_combine   source: waits for all returns, out[t] = sum of the partial
 *                      rows of the ranks token t was sent to
 *   strix_moe_permute_rows  byte twin of strix_moe_permute_bf16 (rows of any
 *                      16-byte multiple, e.g. e4m3 activations followed by their
 *                      fp32 group scales) */
int strix_peer_alloc(void** ptr, int64_t bytes);
int strix_peer_free(void* ptr);
int strix_peer_export(const void* ptr, void* handle64);
int strix_peer_import(const void* handle64, void** ptr);
int strix_peer_unimport(void* ptr);
/* experts_per_rank > 0: rank r owns the experts [r * epr, (r + 1) * epr); < 0: round-robin
 * placement, expert e lives on rank e mod world as local expert e / world (-epr experts per
 * rank). `placement` (device memory, NULL for the two arithmetic forms) is a table
 * instead: int32 {global experts, row stride, then per expert a row {copies, rank << 16 |
 * local id, ... (copies entries)}}; an expert with several copies - a hot expert replicated
 * so that the ranks' loads balance - serves token t from copy t mod copies. */
int strix_ep_status(int32_t* host_out, int reset);
int strix_ep_plan(const int32_t* topk_ids, int32_t* tok_pos, int32_t* counts, int64_t tokens,
                  int64_t top_k, int64_t experts_per_rank, int64_t world, const int32_t* placement,
                  strix_stream_t stream);
int strix_ep_dispatch(const void* x, const int32_t* topk_ids, const float* topk_weights,
                      const int32_t* tok_pos, const int32_t* counts, void* const* peer_recv,
                      void* const* peer_meta, void* const* peer_counts, void* const* peer_flags,
                      int32_t* ticket, int64_t tokens, int64_t row_bytes, int64_t x_stride_bytes,
                      int64_t top_k, int64_t experts_per_rank, int64_t world, int64_t rank,
                      int64_t cap, int64_t epoch, const int32_t* placement, strix_stream_t stream);
int strix_ep_prepare(const int32_t* meta, const int32_t* counts, const int32_t* flags,
                     int32_t* ids, float* weights, int32_t* rows_per_source, int64_t world,
                     int64_t cap, int64_t top_k, int64_t epoch, int64_t spin_limit,
                     strix_stream_t stream);
int strix_ep_return(const void* y, const int32_t* ids, const int32_t* meta, const int32_t* counts,
                    void* const* peer_ret, void* const* peer_rflags, int32_t* ticket,
                    int64_t world, int64_t rank, int64_t cap, int64_t top_k, int64_t hidden,
                    int64_t y_stride, int64_t epoch, strix_stream_t stream);
int strix_ep_combine(const void* ret, const int32_t* rflags, const int32_t* tok_pos, void* out,
                     int64_t tokens, int64_t hidden, int64_t out_stride, int64_t world,
                     int64_t cap, int64_t epoch, int64_t spin_limit, strix_stream_t stream);
int strix_moe_permute_rows(const void* x, void* y, const int32_t* slot_pos,
                           const int32_t* sorted_ids, const int32_t* num_post_padded,
                           int64_t rows, int64_t sorted_rows, int64_t row_bytes, int64_t top_k,
                           int64_t x_stride_bytes, int64_t y_stride_bytes, strix_stream_t stream);

/* One call for a whole expert-parallel MoE layer over the exchange above: router ->
 * (FP8: quantise the payload) -> plan -> dispatch -> wait for the sources -> this
 * rank's experts over the received rows (sorted-layout tcgen05 kernels) -> partial
 * sums back -> wait and combine into out (bf16 [tokens, hidden]). Enqueues about
 * ten kernels on `stream`, allocates nothing, never synchronises the host. The two
 * structs carry what does not change from call to call; `epoch` must be one more
 * than at the previous call over these buffers (1 at the first). */
typedef struct strix_expert_weights {
  const void* w13;        /* MXFP4: uint8 [E, 2I, H/2]; FP8: e4m3 [E, 2I, H] */
  const void* w13_scale;  /* MXFP4: e8m0 [E, 2I, H/32]; FP8: fp32 channel [E, 2I] or block */
  const void* w2;         /* [E, H, I/2] or [E, H, I] */
  const void* w2_scale;
  int64_t w13_stride_e, w13_stride_n, s13_stride_e, s13_stride_n;   /* in elements */
  int64_t w2_stride_e, w2_stride_n, s2_stride_e, s2_stride_n;
  int64_t experts, hidden, inter;   /* experts on THIS rank */
  int32_t kind;                     /* 0 MXFP4 x bf16, 1 FP8 W8A8 channel scales, 2 block scales */
  int32_t gate_act;                 /* 1 silu, 2 gelu_tanh */
} strix_expert_weights;

typedef struct strix_ep_exchange {
  int64_t world, rank, cap, top_k, row_bytes, hidden, epoch;
  int64_t round_robin;        /* 0: contiguous expert blocks per rank, 1: expert e on rank e mod world */
  const int32_t* placement;   /* placement table (device memory) or NULL; overrides round_robin */
  int64_t experts_global;     /* router width; 0 = experts on this rank x world */
  void* const* peer_recv;     /* host arrays of `world` device addresses, own rank included */
  void* const* peer_meta;
  void* const* peer_counts;
  void* const* peer_flags;
  void* const* peer_ret;
  void* const* peer_rflags;
  int32_t* ticket;            /* 2 ints, zeroed once */
  int32_t* ids;               /* [world * cap, top_k] received routing */
  float* weights;             /* [world * cap, top_k] */
  int32_t* rows_per_source;   /* [world] */
  void* y;                    /* bf16 [world * cap * top_k, hidden] */
  int32_t* tok_pos;           /* [world, cap] */
  int32_t* counts;            /* [world] */
} strix_ep_exchange;

int64_t strix_ep_moe_layer_workspace(const strix_expert_weights* w, const strix_ep_exchange* ep,
                                     int64_t block_m);
int strix_ep_moe_layer(void* out, const void* x, const float* logits, const strix_expert_weights* w,
                       const strix_ep_exchange* ep, void* workspace, int64_t workspace_bytes,
                       int64_t tokens, int64_t x_stride, int64_t logits_stride, int64_t out_stride,
                       int64_t block_m, int64_t spin_limit, strix_stream_t stream);

/* strix_attn_prefill_bf16 on the tcgen05 tensor cores (S and O in tensor memory,
 * TMA-fed operands): same contract and arguments (attn_prefill_bf16 of the
 * reference, csrc/attn/attn_prefill_bf16.hip:508-662), for head_dim 64 / 128 with
 * 16-byte aligned q / out rows (strix_attn_prefill_umma_covers() tells, 1/0). A
 * first kernel gathers the batch's keys and values from the pages into a
 * contiguous 16-bit workspace (int8 caches dequantised with their scales, each
 * sequence padded to 128 keys); the caller provides it: `workspace` 1024-byte
 * aligned, at least strix_attn_prefill_workspace(nseq, max_blocks, block_size,
 * hkv, head_dim) bytes, where max_blocks is the block table's row length. The
 * dequantised values must fit fp16. num_splits does not apply. */
int64_t strix_attn_prefill_workspace(int64_t nseq, int64_t max_blocks, int64_t block_size,
                                     int64_t hkv, int64_t head_dim);
int strix_attn_prefill_umma_covers(int64_t head_dim, int64_t q_stride_t, int64_t q_stride_h,
                                   int64_t out_stride_t, int64_t out_stride_h, int kv_int8);
int strix_attn_prefill_umma(
    void* out, const void* q, const void* key_cache, const void* value_cache, const float* k_scale,
    const float* v_scale, const int32_t* cu_seqlens_q, const int32_t* seq_lens,
    const int32_t* block_table, const float* sinks, void* workspace, int64_t workspace_bytes,
    int64_t total_q, int64_t nseq, int64_t hq, int64_t hkv, int64_t head_dim, int64_t block_size,
    int64_t max_blocks, int64_t bt_stride, int64_t q_stride_t, int64_t q_stride_h,
    int64_t out_stride_t, int64_t out_stride_h, int64_t k_stride_b, int64_t k_stride_s,
    int64_t k_stride_h, int64_t v_stride_b, int64_t v_stride_s, int64_t v_stride_h,
    int64_t ks_stride_b, int64_t ks_stride_s, int64_t ks_stride_h, int64_t vs_stride_b,
    int64_t vs_stride_s, int64_t vs_stride_h, double scale, int64_t window_left, int kv_int8,
    strix_stream_t stream);

/* Writes new keys and values into the int8 paged KV cache with one fp32
 * dequant scale per (token, KV head) - the step before every attention call.
 * The reference leaves it to vLLM; its semantics are pinned by quantize() of
 * the reference's tests/test_attn_prefill.py:202-206 and the consumer views by
 * python/strix_vllm/attn.py:185-203. key / value: bf16 (fp16 if in_f16)
 * [tokens, hkv, head_dim] with element strides over tokens and heads;
 * slot_mapping int64 [tokens]: cache slot (block * block_size + offset) of each
 * token, negative = skip. Caches are bytes [blocks, block_size, hkv, >= head_dim]
 * with BYTE strides (multiples of 4), scales fp32 [blocks, block_size, hkv] with
 * element strides - contiguous tensors, or views into a packed cache whose head
 * rows carry the scale inline after the bytes.
 * rule 0: scale = max(absmax, 1e-8) / 127, q = clamp(rint(x / scale), +-127);
 * rule 1 (vLLM 0.22's writer): scale = max(absmax / 127, 1e-6),
 * q = trunc(clamp(x * (1 / scale), -128, 127)). */
int strix_kv_write_i8(const void* key, const void* value, void* key_cache, void* value_cache,
                      float* k_scale, float* v_scale, const int64_t* slot_mapping,
                      int64_t tokens, int64_t hkv, int64_t head_dim, int64_t block_size,
                      int64_t key_stride_t, int64_t key_stride_h, int64_t value_stride_t,
                      int64_t value_stride_h, int64_t k_stride_b, int64_t k_stride_s,
                      int64_t k_stride_h, int64_t v_stride_b, int64_t v_stride_s,
                      int64_t v_stride_h, int64_t ks_stride_b, int64_t ks_stride_s,
                      int64_t ks_stride_h, int64_t vs_stride_b, int64_t vs_stride_s,
                      int64_t vs_stride_h, int in_f16, int rule, strix_stream_t stream);

/* strix_attn_decode_bf16 without a workspace argument, for callers that cannot
 * allocate device memory: a host loop that owns nothing but the input and
 * output buffers it was given, or a process whose device memory was budgeted
 * at start-up so that a late cudaMalloc may fail or stall the GPU. It has no
 * counterpart in the reference (whose launcher allocates with torch). The
 * split-KV partials go to an array of STRIX_DECODE_STATIC_SCRATCH_BYTES built
 * into the library (held on every GPU that loads it, until exit); a launch that
 * needs more (see strix_attn_decode_workspace) is rejected with
 * STRIX_ERR_INVALID and a message that states both sizes. The call allocates and
 * frees nothing. The first call on each device looks the array's address up
 * (cudaGetSymbolAddress) - make it before any stream capture. All calls share
 * the array: calls that overlap on the GPU race on it. Arguments otherwise as
 * strix_attn_decode_bf16. */
#define STRIX_DECODE_STATIC_SCRATCH_BYTES (16 * 1024 * 1024)

int strix_attn_decode_bf16_static(
    void* out, const void* q, const void* key_cache, const void* value_cache,
    const float* k_scale, const float* v_scale, const int32_t* seq_lens,
    const int32_t* block_table, const float* sinks,
    int64_t nseq, int64_t hq, int64_t hkv, int64_t head_dim, int64_t block_size,
    int64_t max_blocks, int64_t bt_stride,
    int64_t q_st, int64_t q_sh, int64_t o_st, int64_t o_sh,
    int64_t k_sb, int64_t k_ss, int64_t k_sh,
    int64_t v_sb, int64_t v_ss, int64_t v_sh,
    int64_t ks_sb, int64_t ks_ss, int64_t ks_sh,
    int64_t vs_sb, int64_t vs_ss, int64_t vs_sh,
    double scale, int64_t num_splits, int64_t window_left, int kv_int8,
    strix_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* STRIX_B200_H_ */
