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
 *                 kv_int8 == 0: bf16 (strides multiples of 8); scales NULL.
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
 * Built geometries: head_dim 128 or 256, hq / hkv in 1..8, block_size a
 * multiple of 16. Others return STRIX_ERR_INVALID.
 * ---------------------------------------------------------------------- */
#define STRIX_DECODE_AUTO_KEYS 1024

/* Number of key segments the call will use (>= 1), or -1 on bad arguments. */
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
