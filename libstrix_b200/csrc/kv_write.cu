// Writes new keys and values into the int8 paged KV cache, one fp32 dequant
// scale per (token, KV head): the step before every attention call. The
// reference leaves it to vLLM (reshape_and_cache for int8_per_token_head); its
// semantics are pinned by quantize() of tests/test_attn_prefill.py:202-206 -
// scale = max(absmax, 1e-8) / 127, q = clamp(round(x / scale), +-127) - and the
// consumer views by python/strix_vllm/attn.py:185-203. Both cache layouts are
// served through strides: separate byte caches [blocks, block_size, Hkv, D]
// with contiguous scale tensors, and the packed layout whose head rows are D + 4
// bytes with the scale inline after the bytes (scale tensors are then strided
// views into the cache itself).
//
// One warp per (token, head, K or V): the row (D bf16/fp16 values, 256 bytes at
// D = 128) is read as 16-byte chunks, its absolute maximum reduced with
// shuffles, and the bytes written as 8-byte (4-byte where the row is only
// 4-byte aligned) stores. HBM-bound: 2 D bytes read + D + 4 written per row.
#include "common.cuh"

namespace strix {
namespace {

constexpr int kKvWarps = 8;
constexpr int kKvMaxChunks = 2;   // 16-byte chunks per lane: D <= 512

struct KvWriteArgs {
  const uint16_t* src[2];      // key, value [tokens, Hkv, D]
  uint8_t* cache[2];
  float* scale[2];
  const int64_t* slot_mapping;
  int64_t src_st[2], src_sh[2];                 // elements
  int64_t c_sb[2], c_ss[2], c_sh[2];            // bytes
  int64_t s_sb[2], s_ss[2], s_sh[2];            // elements
  int64_t tokens;
  int hkv, head_dim, block_size, in_f16, rule;
};

__global__ void __launch_bounds__(kKvWarps * 32) kv_write_i8_kernel(const KvWriteArgs p) {
  const int lane = threadIdx.x & 31;
  const int64_t row = int64_t(blockIdx.x) * kKvWarps + (threadIdx.x >> 5);
  const int64_t rows = p.tokens * p.hkv * 2;
  if (row >= rows) return;
  const int which = int(row & 1);                      // 0 key, 1 value
  const int head = int((row >> 1) % p.hkv);
  const int64_t tok = (row >> 1) / p.hkv;
  const int64_t slot = p.slot_mapping[tok];
  if (slot < 0) return;                                // a padding token writes nothing
  const int64_t blk = slot / p.block_size, in_blk = slot % p.block_size;
  const uint16_t* src = p.src[which] + tok * p.src_st[which] + head * p.src_sh[which];
  const int chunks = p.head_dim / 8;

  float v[kKvMaxChunks][8];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < kKvMaxChunks; ++i) {
    const int ch = lane + 32 * i;
    if (ch < chunks) {
      const uint4 x = *reinterpret_cast<const uint4*>(src + 8 * ch);
      const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (p.in_f16) {
          const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
          v[i][2 * j] = f.x, v[i][2 * j + 1] = f.y;
        } else {
          v[i][2 * j] = bf16_lo(w[j]), v[i][2 * j + 1] = bf16_hi(w[j]);
        }
        amax = fmaxf(amax, fmaxf(fabsf(v[i][2 * j]), fabsf(v[i][2 * j + 1])));
      }
    }
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  // rule 0 (the reference's quantize()): scale = max(absmax, 1e-8) / 127, x / scale
  // rounded to nearest even, clamped to +-127. rule 1 (vLLM 0.22's Triton writer):
  // scale = max(absmax / 127, 1e-6), x * (1 / scale) clamped to [-128, 127] and
  // converted to int8 by truncation. IEEE divisions: the build uses fast math.
  const float s = p.rule == 0 ? __fdiv_rn(fmaxf(amax, 1e-8f), 127.f)
                              : fmaxf(__fdiv_rn(amax, 127.f), 1e-6f);
  const float inv = __fdiv_rn(1.f, s);
  if (lane == 0)
    p.scale[which][blk * p.s_sb[which] + in_blk * p.s_ss[which] + int64_t(head) * p.s_sh[which]] = s;
  uint8_t* dst = p.cache[which] + blk * p.c_sb[which] + in_blk * p.c_ss[which] + int64_t(head) * p.c_sh[which];
  const bool a8 = (reinterpret_cast<uintptr_t>(dst) & 7) == 0;
#pragma unroll
  for (int i = 0; i < kKvMaxChunks; ++i) {
    const int ch = lane + 32 * i;
    if (ch < chunks) {
      int q[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (p.rule == 0) {
          q[j] = __float2int_rn(fminf(fmaxf(rintf(__fdiv_rn(v[i][j], s)), -127.f), 127.f));
        } else {
          q[j] = __float2int_rz(fminf(fmaxf(__fmul_rn(v[i][j], inv), -128.f), 127.f));
        }
      }
      const uint32_t lo = (q[0] & 255) | ((q[1] & 255) << 8) | ((q[2] & 255) << 16) | (uint32_t(q[3] & 255) << 24);
      const uint32_t hi = (q[4] & 255) | ((q[5] & 255) << 8) | ((q[6] & 255) << 16) | (uint32_t(q[7] & 255) << 24);
      if (a8) {
        *reinterpret_cast<uint2*>(dst + 8 * ch) = make_uint2(lo, hi);
      } else {
        *reinterpret_cast<uint32_t*>(dst + 8 * ch) = lo;
        *reinterpret_cast<uint32_t*>(dst + 8 * ch + 4) = hi;
      }
    }
  }
}

}  // namespace
}  // namespace strix

using namespace strix;

extern "C" int strix_kv_write_i8(
    const void* key, const void* value, void* key_cache, void* value_cache, float* k_scale,
    float* v_scale, const int64_t* slot_mapping, int64_t tokens, int64_t hkv, int64_t head_dim,
    int64_t block_size, int64_t key_stride_t, int64_t key_stride_h, int64_t value_stride_t,
    int64_t value_stride_h, int64_t k_stride_b, int64_t k_stride_s, int64_t k_stride_h,
    int64_t v_stride_b, int64_t v_stride_s, int64_t v_stride_h, int64_t ks_stride_b,
    int64_t ks_stride_s, int64_t ks_stride_h, int64_t vs_stride_b, int64_t vs_stride_s,
    int64_t vs_stride_h, int in_f16, int rule, strix_stream_t stream) {
  STRIX_CHECK(tokens >= 0 && hkv >= 1 && block_size >= 1, "bad sizes");
  STRIX_CHECK(head_dim >= 8 && head_dim % 8 == 0 && head_dim <= 256 * kKvMaxChunks,
              "head_dim must be a multiple of 8, at most %d", 256 * kKvMaxChunks);
  STRIX_CHECK(rule == 0 || rule == 1, "rule 0 (round, +-127) or 1 (truncate, [-128, 127])");
  STRIX_CHECK(key != nullptr && value != nullptr && key_cache != nullptr && value_cache != nullptr &&
                  k_scale != nullptr && v_scale != nullptr && slot_mapping != nullptr,
              "pointers must not be NULL");
  STRIX_CHECK(reinterpret_cast<uintptr_t>(key) % 16 == 0 && reinterpret_cast<uintptr_t>(value) % 16 == 0 &&
                  key_stride_t % 8 == 0 && key_stride_h % 8 == 0 && value_stride_t % 8 == 0 &&
                  value_stride_h % 8 == 0,
              "key / value rows must be 16-byte aligned");
  const int64_t cs[6] = {k_stride_b, k_stride_s, k_stride_h, v_stride_b, v_stride_s, v_stride_h};
  bool a4 = reinterpret_cast<uintptr_t>(key_cache) % 4 == 0 && reinterpret_cast<uintptr_t>(value_cache) % 4 == 0;
  for (int i = 0; i < 6; ++i) a4 = a4 && cs[i] % 4 == 0;
  STRIX_CHECK(a4, "cache rows must be 4-byte aligned");
  if (tokens == 0) return STRIX_OK;
  KvWriteArgs p;
  p.src[0] = static_cast<const uint16_t*>(key), p.src[1] = static_cast<const uint16_t*>(value);
  p.cache[0] = static_cast<uint8_t*>(key_cache), p.cache[1] = static_cast<uint8_t*>(value_cache);
  p.scale[0] = k_scale, p.scale[1] = v_scale, p.slot_mapping = slot_mapping;
  p.src_st[0] = key_stride_t, p.src_sh[0] = key_stride_h;
  p.src_st[1] = value_stride_t, p.src_sh[1] = value_stride_h;
  p.c_sb[0] = k_stride_b, p.c_ss[0] = k_stride_s, p.c_sh[0] = k_stride_h;
  p.c_sb[1] = v_stride_b, p.c_ss[1] = v_stride_s, p.c_sh[1] = v_stride_h;
  p.s_sb[0] = ks_stride_b, p.s_ss[0] = ks_stride_s, p.s_sh[0] = ks_stride_h;
  p.s_sb[1] = vs_stride_b, p.s_ss[1] = vs_stride_s, p.s_sh[1] = vs_stride_h;
  p.tokens = tokens, p.hkv = int(hkv), p.head_dim = int(head_dim), p.block_size = int(block_size);
  p.in_f16 = in_f16, p.rule = rule;
  const int64_t rows = tokens * hkv * 2;
  kv_write_i8_kernel<<<unsigned((rows + kKvWarps - 1) / kKvWarps), kKvWarps * 32, 0,
                       static_cast<cudaStream_t>(stream)>>>(p);
  return launch_status("kv_write_i8");
}
