// Grouped expert GEMM over the moe_align_block_size layout, for sm_100a: the
// weight-streaming kernel family (small and medium token counts per expert,
// where the layer is bound by reading each routed expert's weights once).
//
// Contract (all moe_gemm_* ops of the reference, csrc/moe/moe_gemm_w8a16.hip:76-404):
//   * m-block mb owns sorted ids [mb * block_m, (mb + 1) * block_m); it is
//     skipped when mb * block_m >= *num_post_padded or expert_ids[mb] < 0;
//   * a sorted id sid >= num_valid is padding: it contributes zeros and writes
//     nothing; the A row of slot sid is sid / top_k, the C row is sid;
//   * gate_mul: W rows are [gate (N/2); up (N/2)], output column j < N/2 is
//     act(sum_k A W[j]) * (sum_k A W[N/2 + j]) computed in fp32 and rounded once;
//     otherwise C[sid, n] = (sum_k ...) * topk_w[sid];
//   * block scales index [expert, global W row / 128, k / 128].
//
// Shape of the kernel: a CTA = (m-block, 4 warps); each warp owns 16 weight rows
// (8 gate rows + the 8 matching up rows under gate_mul, so the fused epilogue
// needs no exchange) and keeps them as the MMA M dimension, while the tokens of
// the m-block are the N dimension in tiles of 8 (fully padded tiles are skipped,
// so ragged experts waste no tensor work). Per 128-wide K block every thread
// copies its share of the weight rows and of the token rows into a shared-memory
// ring with 16-byte cp.async (3 blocks ahead); operands are read back as MMA
// fragments with bank-conflict-free swizzles. 8-bit x 8-bit forms run the MMA on
// the raw bytes (e4m3 x e4m3 -> f32, s8 x s8 -> s32); forms with 16-bit
// activations widen the weights exactly in registers and apply block scales to
// the fp32 partial sums of each K block.
#include <cstdlib>

#include "common.cuh"

namespace strix {
namespace {

constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr int kStages = 4;
constexpr int kKB = 128;  // K elements per pipeline step (= the scale block)

// W_INT4X (host-side only) = W_INT4 whose 32-bit words hold their eight nibbles in
// vLLM's ExLlama order (k = 0 2 4 6 1 3 5 7), the dense int4 layout of the reference
// (csrc/gemm/w8a8_wmma_gemm.hip:128-132): same kernels, words unshuffled on load
enum WFmt { W_E4M3 = 0, W_INT8 = 1, W_BF16 = 2, W_MXFP4 = 3, W_INT4 = 4, W_U8B128 = 5, W_INT4X = 6 };
constexpr bool is_w4(int wf) { return wf == W_MXFP4 || wf == W_INT4; }
enum AFmt { A_BF16 = 0, A_F16 = 1, A_E4M3 = 2, A_INT8 = 3 };
constexpr bool is_a8(int af) { return af == A_E4M3 || af == A_INT8; }
// S_GROUP: one scale per output row and 128-wide K group, [E, N, K/128]
enum ScaleKind { S_NONE = 0, S_CHANNEL = 1, S_BLOCK = 2, S_GROUP = 3 };
enum Act { ACT_NONE = 0, ACT_SILU = 1, ACT_GELU_TANH = 2 };

struct MoeArgs {
  void* c;
  const void* a;
  const void* w;
  const void* scales;
  const float* sa;  // activation scales [rows, K / 128] (A_E4M3 only)
  const int32_t* sorted_ids;
  const int32_t* expert_ids;
  const int32_t* num_post;
  const float* topk_w;
  const void* bias;  // optional bf16 added to plain outputs: bias[sid * bias_stride + n]
  int64_t bias_stride;
  int64_t num_valid;
  int64_t a_stride, c_stride, w_se, w_sn, s_se, s_sn, sa_stride;  // elements
  int64_t s_sg;       // stride of the scale tensor over 128-wide K groups (S_BLOCK, S_GROUP)
  int top_k, K, N, block_m;
  int scale_kind, scale_dtype;  // dtype: 0 fp32, 1 bf16, 2 fp16
  int c_f16;
  int tiles_per_cta;  // consecutive n-tiles one CTA streams
  int group;          // K elements per weight scale (32, 64 or 128)
  int w4_shuffled;    // int4 words in ExLlama nibble order
};

__device__ __forceinline__ float load_scale(const void* p, int64_t idx, int dtype) {
  if (dtype == 0) return static_cast<const float*>(p)[idx];
  const uint16_t h = static_cast<const uint16_t*>(p)[idx];
  if (dtype == 1) return __uint_as_float(uint32_t(h) << 16);
  return __half2float(__ushort_as_half(h));
}

__device__ __forceinline__ float apply_act(float g, int act) {
  if (act == ACT_SILU) return g / (1.f + __expf(-g));
  // GELU-tanh: 0.5 g (1 + tanh(sqrt(2/pi) (g + 0.044715 g^3)))
  const float u = 0.7978845608028654f * (g + 0.044715f * g * g * g);
  return 0.5f * g * (1.f + tanhf(u));
}

__device__ __forceinline__ void mma_e4m3_16832(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                               uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Four 8-bit weights (one 32-bit word) -> two registers of 16-bit pairs in the
// activation's format: (w0, w1) and (w2, w3). The fp16 form is exact and the
// scale goes onto the fp32 sums (the reference's "raw" kernels and their
// oracle, tests/test_moe_fp8_raw.py:17-28). The bf16 form multiplies by the
// scale first and rounds the product to bf16, which is what the reference's
// bf16 kernels stage (csrc/moe/moe_gemm_w8a16.hip:218-243) and what their
// oracle dequantises to (tests/test_moe_fp8.py:29): at these magnitudes the
// fused gate amplifies the 2^-9 rounding beyond the test tolerance otherwise.
template <int WF, int AF>
__device__ __forceinline__ void widen(uint32_t w, float scale, uint32_t& lo, uint32_t& hi) {
  uint32_t f_lo, f_hi;  // exact f16x2
  if constexpr (WF == W_E4M3) {
    asm("{\n\t.reg .b16 l, h;\n\tmov.b32 {l, h}, %2;\n\t"
        "cvt.rn.f16x2.e4m3x2 %0, l;\n\tcvt.rn.f16x2.e4m3x2 %1, h;\n\t}"
        : "=r"(f_lo), "=r"(f_hi)
        : "r"(w));
  } else {  // W_INT8: 0x6400 | (b ^ 0x80) is fp16 1024 + b + 128; excess-128 bytes are already b + 128
    const uint32_t x = WF == W_U8B128 ? w : w ^ 0x80808080u;
    f_lo = sub_f16x2(prmt(x, 0x64646464u, 0x4140), 0x64806480u);
    f_hi = sub_f16x2(prmt(x, 0x64646464u, 0x4342), 0x64806480u);
  }
  if constexpr (AF == A_F16) {
    lo = f_lo, hi = f_hi;
  } else {
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&f_lo));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&f_hi));
    lo = pack_bf16x2(a.x * scale, a.y * scale), hi = pack_bf16x2(b.x * scale, b.y * scale);
  }
}

// Eight 4-bit weights (one 32-bit word, element i in bits [4i, 4i + 4): byte j
// holds k = 2j in its low nibble, csrc/gemm/mxfp4_wmma_gemm.hip and
// tests/test_mxfp4.py:29-47) -> four registers of bf16 pairs, each value times
// `scale` and rounded to bf16 (exact for e2m1 x 2^e). MXFP4: sign, 2-bit
// exponent, 1-bit mantissa (0, .5, 1, 1.5, 2, 3, 4, 6); INT4: nibble - 8.
__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}

// An int4 word whose nibbles 0..7 hold k = 0 2 4 6 1 3 5 7 -> nibble k holds k:
// the low half carries the even elements, the high half the odd ones; interleave.
__device__ __forceinline__ uint32_t unshuffle_int4(uint32_t w) {
  uint32_t e = w & 0xffffu, o = w >> 16;
  e = (e | (e << 8)) & 0x00ff00ffu, e = (e | (e << 4)) & 0x0f0f0f0fu;
  o = (o | (o << 8)) & 0x00ff00ffu, o = (o | (o << 4)) & 0x0f0f0f0fu;
  return e | (o << 4);
}

// MXFP4 by table: the low three bits of a nibble index an 8-entry table of bf16
// bit patterns (0, .5, 1, 1.5, 2, 3, 4, 6), looked up four nibbles at a time with
// byte permutes (high bytes and low bytes apart), the sign bit moves to bit 15,
// and one bf16x2 multiply applies the power-of-two scale (exact; 2^(s - 127) has
// the bf16 pattern s << 7, and s = 0 is the zero block).
__device__ __forceinline__ void widen_mxfp4(uint32_t w, uint32_t scale2, uint32_t* out) {
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint32_t x = h == 0 ? w : w >> 16;          // nibbles 4h .. 4h + 3 in the low 16 bits
    const uint32_t sel = x & 0x7777u;
    const uint32_t hi = prmt(0x3F3F3F00u, 0x40404040u, sel);
    const uint32_t lo = prmt(0xC0800000u, 0xC0804000u, sel);
    const uint32_t p01 = prmt(lo, hi, 0x5140) | ((x & 0x8u) << 12) | ((x & 0x80u) << 24);
    const uint32_t p23 = prmt(lo, hi, 0x7362) | ((x & 0x800u) << 4) | ((x & 0x8000u) << 16);
    out[2 * h] = mul_bf16x2(p01, scale2);
    out[2 * h + 1] = mul_bf16x2(p23, scale2);
  }
}

template <int WF>
__device__ __forceinline__ void widen4(uint32_t w, float scale, uint32_t* out) {
  if constexpr (WF == W_MXFP4) {
    // `scale` is 2^(s - 127) (or 0): its upper 16 bits are the bf16 pattern
    const uint32_t sb = __float_as_uint(scale) >> 16;
    widen_mxfp4(w, sb | (sb << 16), out);
    return;
  }
  float v[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t n = (w >> (4 * i)) & 15u;
    if constexpr (WF == W_MXFP4) {
      const uint32_t e = (n >> 1) & 3u, m = n & 1u;
      const uint32_t bits = e ? (((e + 126u) << 23) | (m << 22)) : (m ? 0x3F000000u : 0u);
      v[i] = __uint_as_float(bits | ((n & 8u) << 28)) * scale;
    } else {
      v[i] = float(int(n) - 8) * scale;
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) out[i] = pack_bf16x2(v[2 * i], v[2 * i + 1]);
}

// Shared-memory row layouts of one K block. A row of 8-bit elements is 128
// bytes = 8 chunks of 16; a row of 16-bit elements is 256 bytes = 16 chunks.
// Lane c of a fragment owns elements [32c, 32c + 32) of a row: chunks 2c, 2c+1
// (8-bit) or 4c .. 4c+3 (16-bit). The physical chunk is permuted so that the 8
// lanes of each shared-memory phase (2 rows x 4 lanes) cover 8 distinct chunks
// of one 128-byte bank window.
__device__ __forceinline__ int swz8(int row, int chunk) { return chunk ^ (row & 7); }
__device__ __forceinline__ int swz16(int row, int chunk) {
  // chunk = 4c + j  ->  4j + c, then the two rows of a phase take the two halves
  return ((((chunk & 3) << 2) | (chunk >> 2)) ^ ((row & 1) << 2));
}

template <int ROWBYTES>  // bytes of a row of one K block: 64 (4-bit), 128 or 256
__device__ __forceinline__ uint32_t row_chunk_offset(int row, int chunk) {
  // 64-byte rows: a quarter-warp reads 2 rows x 4 chunks = 128 consecutive bytes as they lie
  if constexpr (ROWBYTES == 64) return uint32_t(row * 64 + (chunk << 4));
  if constexpr (ROWBYTES == 128) return uint32_t(row * 128 + (swz8(row, chunk) << 4));
  return uint32_t(row * 256 + (swz16(row, chunk) << 4));
}

template <int WF, int AF, int BMC>
struct Layout {
  static constexpr int WB = WF == W_BF16 ? 2 : 1;    // bytes per unit of the weight strides
  static constexpr int AB = is_a8(AF) ? 1 : 2;       // activation bytes / element
  static constexpr int kWRow = is_w4(WF) ? kKB / 2 : kKB * WB, kARow = kKB * AB;
  static constexpr int kWElems = kKB * 16 / kWRow;   // K elements per 16-byte weight chunk
  static constexpr int kWBytes = kWarps * 16 * kWRow;  // all warps' weight rows
  static constexpr int kABytes = BMC * kARow;
  static constexpr int kSaBytes = is_a8(AF) ? BMC * 4 : 0;
  static constexpr int kStage = kWBytes + kABytes + kSaBytes;
  static constexpr int kSmem = kStages * kStage + BMC * 8 + 16;
};

template <int WF, int AF, int BMC, int ACT>
__global__ void __launch_bounds__(kThreads) moe_gemm_stream_kernel(const MoeArgs p) {
  using L = Layout<WF, AF, BMC>;
  constexpr int NT = BMC / 8;  // token tiles of 8
  extern __shared__ __align__(16) uint8_t smem[];
  int64_t* s_arow = reinterpret_cast<int64_t*>(smem + kStages * L::kStage);  // [BMC] A row or -1

  // Without routing tensors (a dense GEMM) slot i is row i of one expert.
  const int mb = blockIdx.y;
  if (p.num_post != nullptr && mb * p.block_m >= *p.num_post) return;
  const int expert = p.expert_ids != nullptr ? p.expert_ids[mb] : 0;
  if (expert < 0) return;
  auto slot_id = [&](int pos) -> int64_t {
    return p.sorted_ids != nullptr ? int64_t(p.sorted_ids[pos]) : int64_t(pos);
  };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, c = lane & 3;
  constexpr bool kGate = ACT != ACT_NONE;
  const int half_n = p.N / 2;
  // A CTA walks `tiles_per_cta` consecutive n-tiles of its m-block as ONE flat
  // pipeline over (tile, K block). Weight rows of a warp in a tile: local row
  // r < 8 -> row_lo + r, else row_hi + r - 8.
  constexpr int kRowsPerWarp = kGate ? 8 : 16;
  const int out_rows = kGate ? half_n : p.N;
  const int n_tiles = (out_rows + kWarps * kRowsPerWarp - 1) / (kWarps * kRowsPerWarp);
  const int tile0 = blockIdx.x * p.tiles_per_cta;
  const int ntile = min(p.tiles_per_cta, n_tiles - tile0);
  const int nkb = (p.K + kKB - 1) / kKB;   // the last block may be partial: its tail is zero-filled
  const int total_it = ntile * nkb;

  const uint8_t* wbase = static_cast<const uint8_t*>(p.w) + int64_t(expert) * p.w_se * L::WB;
  const uint32_t smem_s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));

  // ---- per-thread copy plan (everything that does not depend on the K block)
  // weights: copy i of a warp covers local rows i * RPI + lane / CPW, chunk lane % CPW
  constexpr int CPW = L::kWRow / 16, RPI = 32 / CPW, NCW = 16 / RPI;
  const int w_r0 = lane / CPW, w_ch = lane % CPW;
  uint32_t w_dst[NCW];
#pragma unroll
  for (int i = 0; i < NCW; ++i)
    w_dst[i] = warp * 16 * L::kWRow + row_chunk_offset<L::kWRow>(i * RPI + w_r0, w_ch);
  // activations: copy i of a thread is chunk id = i * kThreads + tid of the BMC x CPA tile
  constexpr int CPA = L::kARow / 16, NCA = BMC * CPA / kThreads;
  static_assert(BMC * CPA % kThreads == 0, "activation tile must split evenly over the threads");
  uint32_t a_dst[NCA];
#pragma unroll
  for (int i = 0; i < NCA; ++i) {
    const int id = i * kThreads + threadIdx.x;
    a_dst[i] = L::kWBytes + row_chunk_offset<L::kARow>(id / CPA, id % CPA);
  }
  // fragment read offsets inside a stage: weights rows g, g + 8; token row 8j + g
  constexpr int WCH = L::kWRow / 64, ACH = 2 * L::AB;  // 16-byte chunks a lane owns per row
  uint32_t w_off[2][WCH], a_off[ACH];
#pragma unroll
  for (int r = 0; r < 2; ++r)
#pragma unroll
    for (int i = 0; i < WCH; ++i)
      w_off[r][i] = warp * 16 * L::kWRow + row_chunk_offset<L::kWRow>(g + 8 * r, WCH * c + i);
#pragma unroll
  for (int i = 0; i < ACH; ++i) a_off[i] = L::kWBytes + row_chunk_offset<L::kARow>(g, ACH * c + i);

  for (int tc = 0; tc < p.block_m; tc += BMC) {  // token chunks of the m-block
    __syncthreads();  // previous chunk's readers are done with s_arow and the ring
    int valid = 0;
    for (int i = threadIdx.x; i < BMC; i += kThreads) {
      const int64_t sid = tc + i < p.block_m ? slot_id(mb * p.block_m + tc + i) : p.num_valid;
      const bool ok = sid >= 0 && sid < p.num_valid;
      s_arow[i] = ok ? sid / p.top_k : -1;
      valid |= ok;
    }
    if (!__syncthreads_or(valid)) continue;  // a chunk of padding only

    // token tiles that hold at least one real token (padding sits at the end of
    // an expert's run, but a ragged middle is handled too: rows are zero-filled)
    int nt_live = 0;
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      bool any = false;
#pragma unroll
      for (int i = 0; i < 8; ++i) any |= s_arow[8 * j + i] >= 0;
      if (any) nt_live = j + 1;
    }

    // activation sources of this thread (fixed for the whole chunk)
    const uint8_t* a_src[NCA];
    bool a_ok[NCA], a_use[NCA];
#pragma unroll
    for (int i = 0; i < NCA; ++i) {
      const int id = i * kThreads + threadIdx.x, r = id / CPA;
      const int64_t arow = s_arow[r];
      a_ok[i] = arow >= 0;
      a_use[i] = r < nt_live * 8;
      a_src[i] = static_cast<const uint8_t*>(p.a) + (arow < 0 ? 0 : arow) * p.a_stride * L::AB +
                 (id % CPA) * 16;
    }
    const float* sa_src = nullptr;
    bool sa_ok = false;
    if constexpr (is_a8(AF)) {
      if (threadIdx.x < BMC) {
        const int64_t arow = s_arow[threadIdx.x];
        sa_ok = arow >= 0;
        sa_src = p.sa + (arow < 0 ? 0 : arow) * p.sa_stride;
      }
    }
    // the two token slots whose results this lane holds in tile j: 8j + 2c, + 1
    int out_sid[NT][2];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        const int slot = tc + 8 * j + 2 * c + t;
        const int64_t sid = slot < p.block_m ? slot_id(mb * p.block_m + slot) : -1;
        out_sid[j][t] = (sid >= 0 && sid < p.num_valid) ? int(sid) : -1;
      }
    // weights widened to bf16 carry their scale (see widen); other forms scale sums
    constexpr bool kPrescale = AF == A_BF16 && WF != W_BF16;

    // ---- producer side: next (tile, K block) to copy
    int it_issue = 0, ti_issue = 0, kb_issue = 0, stage_issue = 0;
    bool w_live_issue = false;
    const uint8_t* w_src[NCW];
    auto issue = [&]() {
      if (it_issue < total_it) {
        if (kb_issue == 0) {  // a new n-tile: this lane's weight row pointers
          const int nb_i = ((tile0 + ti_issue) * kWarps + warp) * kRowsPerWarp;
          w_live_issue = nb_i < out_rows;
          const int hi_i = kGate ? half_n + nb_i : nb_i + 8;
#pragma unroll
          for (int i = 0; i < NCW; ++i) {
            const int r = i * RPI + w_r0;
            const int grow = r < 8 ? nb_i + r : hi_i + r - 8;
            w_src[i] = wbase + int64_t(grow) * p.w_sn * L::WB + w_ch * 16;
          }
        }
        const uint32_t st = smem_s + stage_issue * L::kStage;
        const int k_left = p.K - kb_issue * kKB;   // elements of this K block that exist
        if (w_live_issue) {
          const bool in_k = w_ch * L::kWElems < k_left;
#pragma unroll
          for (int i = 0; i < NCW; ++i) {
            cp_async_16_zfill(st + w_dst[i], in_k ? w_src[i] : wbase, in_k);
            w_src[i] += L::kWRow;
          }
        }
        const int koff = kb_issue * kKB * L::AB;
#pragma unroll
        for (int i = 0; i < NCA; ++i) {
          if (!a_use[i]) continue;
          const int id = i * kThreads + threadIdx.x;
          const bool in_k = (id % CPA) * (16 / L::AB) < k_left;
          cp_async_16_zfill(st + a_dst[i], in_k ? a_src[i] + koff : a_src[i], a_ok[i] && in_k);
        }
        if constexpr (is_a8(AF)) {
          if (sa_src != nullptr && int(threadIdx.x) < nt_live * 8)
            cp_async_4_zfill(st + L::kWBytes + L::kABytes + threadIdx.x * 4, sa_src + kb_issue, sa_ok);
        }
        ++it_issue;
        stage_issue = stage_issue + 1 == kStages ? 0 : stage_issue + 1;
        if (++kb_issue == nkb) kb_issue = 0, ++ti_issue;
      }
      cp_async_commit();
    };

#pragma unroll
    for (int i = 0; i < kStages - 1; ++i) issue();

    // ---- consumer side
    float acc[NT][4];
    float ch0 = 1.f, ch1 = 1.f;
    int kb = 0, nb = 0, row_lo = 0, row_hi = 0, stage = 0, ti = 0;
    int64_t sc0 = 0, sc1 = 0;  // block-scale indices of the two row groups at K block 0
    bool warp_live = false;
    // 4-bit formats: this lane's 32 elements of a K block are one scale group
    // (or part of one); the scales of the next step are fetched a step ahead
    auto w4_scale = [&](int ti_, int kb_, int r) -> float {
      const int nb_ = ((tile0 + ti_) * kWarps + warp) * kRowsPerWarp;
      const int k0 = kb_ * kKB + 32 * c;
      if (ti_ >= ntile || nb_ >= out_rows || k0 >= p.K) return 0.f;
      const int row = (r == 0 ? nb_ : (kGate ? half_n + nb_ : nb_ + 8)) + g;
      const int64_t idx = int64_t(expert) * p.s_se + int64_t(row) * p.s_sn + k0 / p.group;
      if constexpr (WF == W_MXFP4)   // e8m0: 2^(byte - 127), byte 0 = the zero block
        return __uint_as_float(uint32_t(static_cast<const uint8_t*>(p.scales)[idx]) << 23);
      else
        return load_scale(p.scales, idx, p.scale_dtype);
    };
    float g4n0 = 0.f, g4n1 = 0.f;
    if constexpr (is_w4(WF) && !is_a8(AF)) g4n0 = w4_scale(0, 0, 0), g4n1 = w4_scale(0, 0, 1);
    for (int it = 0; it < total_it; ++it) {
      cp_async_wait<kStages - 2>();
      __syncthreads();          // step `it` landed for everyone; the stage of it-1 is free
      issue();
      if (kb == 0) {            // a new n-tile starts
        nb = ((tile0 + ti) * kWarps + warp) * kRowsPerWarp;
        warp_live = nb < out_rows;
        row_lo = nb, row_hi = kGate ? half_n + nb : nb + 8;
#pragma unroll
        for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
        ch0 = ch1 = 1.f;
        if (warp_live && p.scale_kind == S_CHANNEL) {
          ch0 = load_scale(p.scales, int64_t(expert) * p.s_se + row_lo + g, p.scale_dtype);
          ch1 = load_scale(p.scales, int64_t(expert) * p.s_se + row_hi + g, p.scale_dtype);
        }
        const int rdiv = p.scale_kind == S_GROUP ? 1 : 128;
        sc0 = int64_t(expert) * p.s_se + int64_t((row_lo + g) / rdiv) * p.s_sn;
        sc1 = int64_t(expert) * p.s_se + int64_t((row_hi + g) / rdiv) * p.s_sn;
      }
      const uint8_t* st = smem + stage * L::kStage;
      const bool last_kb = kb == nkb - 1;
      const int kb_now = kb;
      stage = stage + 1 == kStages ? 0 : stage + 1;
      if (last_kb) kb = 0, ++ti; else ++kb;
      const float g4_0 = g4n0, g4_1 = g4n1;
      const bool defer4 = WF == W_INT4 && p.group == 128;
      if constexpr (is_w4(WF) && !is_a8(AF)) g4n0 = w4_scale(ti, kb, 0), g4n1 = w4_scale(ti, kb, 1);
      if (!warp_live) continue;

      float sw0 = 1.f, sw1 = 1.f;
      if (p.scale_kind >= S_BLOCK) {
        // this lane's 32 elements of the K block lie in one scale group; groups finer
        // than the block (8-bit weights scaled before the MMA only) differ per lane
        const int gi = p.scale_kind == S_GROUP && p.group < kKB ? (kb_now * kKB + 32 * c) / p.group : kb_now;
        sw0 = load_scale(p.scales, sc0 + gi * p.s_sg, p.scale_dtype);
        sw1 = load_scale(p.scales, sc1 + gi * p.s_sg, p.scale_dtype);
      }

      if constexpr (is_a8(AF)) {
        // 8-bit x 8-bit on the raw bytes (e4m3 x e4m3 -> f32, s8 x s8 -> s32, exact
        // per 128-wide group): lane's 32 weights of rows g, g + 8 as bytes
        uint32_t wr[2][8];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          if constexpr (WF == W_INT4) {
            // 8 nibbles -> 8 signed bytes (nibble - 8), in element order
            const uint4 x = *reinterpret_cast<const uint4*>(st + w_off[r][0]);
            uint32_t ws[4] = {x.x, x.y, x.z, x.w};
            if (p.w4_shuffled) {
#pragma unroll
              for (int i = 0; i < 4; ++i) ws[i] = unshuffle_int4(ws[i]);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint32_t lo = ws[i] & 0x0F0F0F0Fu, hi = (ws[i] >> 4) & 0x0F0F0F0Fu;
              wr[r][2 * i] = __vsub4(prmt(lo, hi, 0x5140), 0x08080808u);
              wr[r][2 * i + 1] = __vsub4(prmt(lo, hi, 0x7362), 0x08080808u);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
              const uint4 x = *reinterpret_cast<const uint4*>(st + w_off[r][i]);
              wr[r][4 * i] = x.x, wr[r][4 * i + 1] = x.y, wr[r][4 * i + 2] = x.z, wr[r][4 * i + 3] = x.w;
            }
            if constexpr (WF == W_U8B128) {   // excess-128 bytes -> two's complement
#pragma unroll
              for (int i = 0; i < 8; ++i) wr[r][i] ^= 0x80808080u;
            }
          }
        }
        const float2* sap = reinterpret_cast<const float2*>(st + L::kWBytes + L::kABytes) + c;
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          if (j >= nt_live) break;
          uint32_t xr[8];
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            const uint4 x = *reinterpret_cast<const uint4*>(st + a_off[i] + j * 8 * L::kARow);
            xr[4 * i] = x.x, xr[4 * i + 1] = x.y, xr[4 * i + 2] = x.z, xr[4 * i + 3] = x.w;
          }
          float part[4] = {0.f, 0.f, 0.f, 0.f};
          if constexpr (AF == A_INT8) {
            int ipart[4] = {0, 0, 0, 0};
#pragma unroll
            for (int s = 0; s < 4; ++s) {
              const uint32_t a[4] = {wr[0][2 * s], wr[1][2 * s], wr[0][2 * s + 1], wr[1][2 * s + 1]};
              mma_s8s8_16832(ipart, a, xr[2 * s], xr[2 * s + 1]);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) part[i] = float(ipart[i]);
          } else {
#pragma unroll
            for (int s = 0; s < 4; ++s) {
              const uint32_t a[4] = {wr[0][2 * s], wr[1][2 * s], wr[0][2 * s + 1], wr[1][2 * s + 1]};
              mma_e4m3_16832(part, a, xr[2 * s], xr[2 * s + 1]);
            }
          }
          const float2 sa = sap[4 * j];  // scales of tokens 8j + 2c, 8j + 2c + 1
          acc[j][0] += part[0] * (sw0 * sa.x);
          acc[j][1] += part[1] * (sw0 * sa.y);
          acc[j][2] += part[2] * (sw1 * sa.x);
          acc[j][3] += part[3] * (sw1 * sa.y);
        }
      } else {
        // 16-bit activations: weights widened to the activation's format
        uint32_t wf[2][16];  // per row: 8 k-steps x (lo, hi)
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          if constexpr (WF == W_BF16) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint4 x = *reinterpret_cast<const uint4*>(st + w_off[r][i]);
              wf[r][4 * i] = x.x, wf[r][4 * i + 1] = x.y, wf[r][4 * i + 2] = x.z, wf[r][4 * i + 3] = x.w;
            }
          } else if constexpr (is_w4(WF)) {
            uint4 x = *reinterpret_cast<const uint4*>(st + w_off[r][0]);
            if (WF == W_INT4 && p.w4_shuffled)
              x.x = unshuffle_int4(x.x), x.y = unshuffle_int4(x.y), x.z = unshuffle_int4(x.z), x.w = unshuffle_int4(x.w);
            // a scale that covers the whole K block goes onto the fp32 sums and the
            // weights stay exact (the reference's deferred-scale path and its oracle,
            // tests/test_moe_wna16.py:50-62); finer groups scale the weights
            const float ws = defer4 ? 1.f : (r == 0 ? g4_0 : g4_1);
            widen4<WF>(x.x, ws, &wf[r][0]);
            widen4<WF>(x.y, ws, &wf[r][4]);
            widen4<WF>(x.z, ws, &wf[r][8]);
            widen4<WF>(x.w, ws, &wf[r][12]);
          } else {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
              const uint4 x = *reinterpret_cast<const uint4*>(st + w_off[r][i]);
              const float ws = r == 0 ? sw0 * ch0 : sw1 * ch1;
              widen<WF, AF>(x.x, ws, wf[r][8 * i], wf[r][8 * i + 1]);
              widen<WF, AF>(x.y, ws, wf[r][8 * i + 2], wf[r][8 * i + 3]);
              widen<WF, AF>(x.z, ws, wf[r][8 * i + 4], wf[r][8 * i + 5]);
              widen<WF, AF>(x.w, ws, wf[r][8 * i + 6], wf[r][8 * i + 7]);
            }
          }
        }
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          if (j >= nt_live) break;
          uint32_t xr[16];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint4 x = *reinterpret_cast<const uint4*>(st + a_off[i] + j * 8 * L::kARow);
            xr[4 * i] = x.x, xr[4 * i + 1] = x.y, xr[4 * i + 2] = x.z, xr[4 * i + 3] = x.w;
          }
          float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int s = 0; s < 8; ++s) {
            const uint32_t a[4] = {wf[0][2 * s], wf[1][2 * s], wf[0][2 * s + 1], wf[1][2 * s + 1]};
            if constexpr (AF == A_F16) mma_f16_16816(part, a, xr[2 * s], xr[2 * s + 1]);
            else mma_bf16_16816(part, a, xr[2 * s], xr[2 * s + 1]);
          }
          const float f0 = defer4 ? g4_0 : kPrescale ? 1.f : sw0, f1 = defer4 ? g4_1 : kPrescale ? 1.f : sw1;
          acc[j][0] += part[0] * f0;
          acc[j][1] += part[1] * f0;
          acc[j][2] += part[2] * f1;
          acc[j][3] += part[3] * f1;
        }
      }
      if (!last_kb) continue;

      // ---- epilogue of this n-tile: lane holds (row g | g + 8) x (tokens 2c, 2c + 1)
      const float e0 = kPrescale ? 1.f : ch0, e1 = kPrescale ? 1.f : ch1;
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        if (j >= nt_live) break;
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          const int64_t sid = out_sid[j][t];
          if (sid < 0) continue;
          const float v0 = acc[j][t] * e0, v1 = acc[j][2 + t] * e1;
          if constexpr (kGate) {
            const float o = apply_act(v0, ACT) * v1;
            const int64_t at = sid * p.c_stride + nb + g;
            if (p.c_f16) static_cast<__half*>(p.c)[at] = __float2half_rn(o);
            else static_cast<__nv_bfloat16*>(p.c)[at] = __float2bfloat16_rn(o);
          } else {
            const float tw = p.topk_w ? p.topk_w[sid] : 1.f;
            __nv_bfloat16* crow = static_cast<__nv_bfloat16*>(p.c) + sid * p.c_stride;
            float b0 = 0.f, b1 = 0.f;
            if (p.bias != nullptr) {
              const __nv_bfloat16* brow = static_cast<const __nv_bfloat16*>(p.bias) + sid * p.bias_stride;
              b0 = __bfloat162float(brow[row_lo + g]), b1 = __bfloat162float(brow[row_hi + g]);
            }
            crow[row_lo + g] = __float2bfloat16_rn(v0 * tw + b0);
            crow[row_hi + g] = __float2bfloat16_rn(v1 * tw + b1);
          }
        }
      }
    }
    cp_async_wait<0>();
  }
}

template <int WF, int AF, int BMC, int ACT>
int launch_stream(const MoeArgs& p, dim3 grid, cudaStream_t st) {
  using L = Layout<WF, AF, BMC>;
  auto kernel = moe_gemm_stream_kernel<WF, AF, BMC, ACT>;
  if (L::kSmem > 48 * 1024) {
    static bool done[64] = {};
    int dev = 0;
    STRIX_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !done[dev]) {
      STRIX_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kSmem));
      if (dev >= 0 && dev < 64) done[dev] = true;
    }
  }
  kernel<<<grid, kThreads, L::kSmem, st>>>(p);
  return launch_status("moe_gemm");
}

template <int WF, int AF, int BMC>
int launch_act(const MoeArgs& p, int act, dim3 grid, cudaStream_t st) {
  if (act == ACT_NONE) return launch_stream<WF, AF, BMC, ACT_NONE>(p, grid, st);
  if (act == ACT_SILU) return launch_stream<WF, AF, BMC, ACT_SILU>(p, grid, st);
  return launch_stream<WF, AF, BMC, ACT_GELU_TANH>(p, grid, st);
}

template <int WF, int AF>
int launch_bm(const MoeArgs& p, int act, dim3 grid, cudaStream_t st) {
  if (p.block_m <= 16) return launch_act<WF, AF, 16>(p, act, grid, st);
  if (p.block_m <= 32) return launch_act<WF, AF, 32>(p, act, grid, st);
  return launch_act<WF, AF, 64>(p, act, grid, st);
}

}  // namespace

}  // namespace strix

using namespace strix;

static int moe_gemm_impl(
    void* c, const void* a, const void* w, const void* scales, const float* act_scales,
    const int32_t* sorted_ids, const int32_t* expert_ids, const int32_t* num_post_padded,
    const float* topk_weights, int64_t num_valid, int64_t a_rows, int64_t experts, int64_t n,
    int64_t k, int64_t a_stride, int64_t c_stride, int64_t w_stride_e, int64_t w_stride_n,
    int64_t s_stride_e, int64_t s_stride_n, int64_t sa_stride, int64_t sorted_len,
    int64_t expert_len, int64_t top_k, int64_t block_m, int weight_format, int act_format,
    int scale_kind, int scale_dtype, int gate_act, int c_is_f16, strix_stream_t stream,
    const void* bias, int64_t bias_stride, int group, int64_t s_stride_g = 1) {
  STRIX_CHECK(weight_format >= W_E4M3 && weight_format <= W_INT4X, "unknown weight format");
  const int w4_shuffled = weight_format == W_INT4X;
  if (w4_shuffled) weight_format = W_INT4;
  const bool w4 = is_w4(weight_format);
  // scale groups finer than the 128-wide K block on 8-bit weights: only where the
  // weights are scaled before the MMA (bf16 activations), each lane with its own scale
  STRIX_CHECK(w4 || scale_kind != S_GROUP || group == 0 || group == 128 ||
                  ((group == 32 || group == 64) && act_format == A_BF16),
              "8-bit weights take scale groups of 128 (32 and 64 with bf16 activations)");
  STRIX_CHECK(act_format >= A_BF16 && act_format <= A_INT8, "unknown activation format");
  STRIX_CHECK(gate_act >= ACT_NONE && gate_act <= ACT_GELU_TANH,
              "activation must be silu or gelu_tanh");
  STRIX_CHECK(scale_kind >= S_NONE && scale_kind <= S_GROUP && scale_dtype >= 0 && scale_dtype <= 2,
              "scales bf16, fp16 or fp32");
  STRIX_CHECK(experts > 0 && n > 0 && k > 0 && num_valid >= 0 && a_rows >= 0, "bad ranks");
  STRIX_CHECK(w4 ? k % 32 == 0 : k % kKB == 0, "K %% 128 (K %% 32 for 4-bit weights)");
  STRIX_CHECK(!w4 || act_format == A_INT8 ||
                  (act_format == A_BF16 && (group == 32 || group == 64 || group == 128) &&
                   scales != nullptr && (weight_format != W_MXFP4 || group == 32)),
              "4-bit weights take bf16 activations and scales per 32, 64 or 128 elements (32 for MXFP4)");
  STRIX_CHECK(act_format != A_INT8 ||
                  ((weight_format == W_INT4 || weight_format == W_U8B128 || weight_format == W_INT8) &&
                   act_scales != nullptr && k % kKB == 0 &&
                   (scale_kind == S_GROUP || scale_kind == S_CHANNEL)),
              "int8 activations need int4 / int8 weights, activation scales, K %% 128 and scales "
              "per channel or per (row, 128 group)");
  STRIX_CHECK(bias == nullptr || gate_act == ACT_NONE, "bias only on plain outputs");
  STRIX_CHECK(gate_act == ACT_NONE || (n % 16 == 0 && topk_weights == nullptr),
              "silu_mul needs even N and no topk weights");
  STRIX_CHECK(gate_act != ACT_NONE || n % 16 == 0, "N %% 16");
  STRIX_CHECK(top_k >= 1 && block_m >= 1 && block_m <= 1024, "bad top_k / block_m");
  STRIX_CHECK(expert_ids == nullptr || expert_len * block_m >= sorted_len,
              "expert_ids too short for block_m %lld", (long long)block_m);
  STRIX_CHECK((sorted_ids == nullptr) == (expert_ids == nullptr) &&
                  (sorted_ids == nullptr) == (num_post_padded == nullptr),
              "routing tensors come together or not at all");
  STRIX_CHECK(act_format != A_E4M3 || (weight_format == W_E4M3 && act_scales != nullptr),
              "e4m3 activations need e4m3 weights and activation scales");
  STRIX_CHECK(weight_format != W_BF16 || (act_format == A_BF16 && scale_kind == S_NONE),
              "bf16 weights take bf16 activations and no scales");
  STRIX_CHECK(weight_format == W_BF16 || w4 || scale_kind != S_NONE, "quantized weights need scales");
  STRIX_CHECK(scale_kind != S_BLOCK || weight_format == W_E4M3,
              "block scales must be fp32 [E, N/128, K/128]");
  STRIX_CHECK(!c_is_f16 || (gate_act != ACT_NONE && act_format == A_F16),
              "fp16 output only for the fused activation of the fp16 form");
  const int wb = weight_format == W_BF16 ? 2 : 1, ab = is_a8(act_format) ? 1 : 2;
  STRIX_CHECK((a_stride * ab) % 16 == 0 && (w_stride_n * wb) % 16 == 0 && (w_stride_e * wb) % 16 == 0 &&
                  reinterpret_cast<uintptr_t>(a) % 16 == 0 && reinterpret_cast<uintptr_t>(w) % 16 == 0,
              "16-byte aligned rows required");
  if (sorted_len == 0 || num_valid == 0) return STRIX_OK;
  MoeArgs p;
  p.c = c, p.a = a, p.w = w, p.scales = scales, p.sa = act_scales;
  p.sorted_ids = sorted_ids, p.expert_ids = expert_ids, p.num_post = num_post_padded;
  p.topk_w = topk_weights;
  p.bias = bias, p.bias_stride = bias_stride, p.group = group > 0 ? group : 128;
  p.num_valid = num_valid;
  p.a_stride = a_stride, p.c_stride = c_stride, p.w_se = w_stride_e, p.w_sn = w_stride_n;
  p.s_se = s_stride_e, p.s_sn = s_stride_n, p.sa_stride = sa_stride;
  p.s_sg = s_stride_g > 0 ? s_stride_g : 1;
  p.top_k = int(top_k), p.K = int(k), p.N = int(n), p.block_m = int(block_m);
  p.scale_kind = scale_kind, p.scale_dtype = scale_dtype, p.c_f16 = c_is_f16;
  p.w4_shuffled = w4_shuffled;

  const int rows_per_cta = kWarps * (gate_act != ACT_NONE ? 8 : 16);
  const int64_t out_rows = gate_act != ACT_NONE ? n / 2 : n;
  const int64_t m_blocks = (sorted_len + block_m - 1) / block_m;
  STRIX_CHECK(m_blocks <= 65535, "too many m-blocks");
  const int64_t n_tiles = (out_rows + rows_per_cta - 1) / rows_per_cta;
  // n-tiles per CTA: enough K blocks per CTA (>= 48, i.e. 6 KB x 4 warps x 48 of
  // weights) to amortise the pipeline fill, while keeping several CTAs per
  // m-block. STRIX_MOE_TILES_PER_CTA overrides it for tuning runs.
  static const int tpc_env = [] {
    const char* e = getenv("STRIX_MOE_TILES_PER_CTA");
    return e ? atoi(e) : 0;
  }();
  const int64_t nkb = (k + kKB - 1) / kKB;
  int64_t tpc = tpc_env > 0 ? tpc_env : (48 + nkb - 1) / nkb;
  if (tpc > n_tiles) tpc = n_tiles;
  p.tiles_per_cta = int(tpc);
  const dim3 grid{unsigned((n_tiles + tpc - 1) / tpc), unsigned(m_blocks), 1u};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (weight_format == W_E4M3 && act_format == A_E4M3) return launch_bm<W_E4M3, A_E4M3>(p, gate_act, grid, st);
  if (weight_format == W_E4M3 && act_format == A_BF16) return launch_bm<W_E4M3, A_BF16>(p, gate_act, grid, st);
  if (weight_format == W_E4M3 && act_format == A_F16) return launch_bm<W_E4M3, A_F16>(p, gate_act, grid, st);
  if (weight_format == W_INT8 && act_format == A_BF16) return launch_bm<W_INT8, A_BF16>(p, gate_act, grid, st);
  if (weight_format == W_U8B128 && act_format == A_BF16) return launch_bm<W_U8B128, A_BF16>(p, gate_act, grid, st);
  if (weight_format == W_U8B128 && act_format == A_INT8) return launch_bm<W_U8B128, A_INT8>(p, gate_act, grid, st);
  if (weight_format == W_INT4 && act_format == A_INT8) return launch_bm<W_INT4, A_INT8>(p, gate_act, grid, st);
  if (weight_format == W_BF16) return launch_bm<W_BF16, A_BF16>(p, gate_act, grid, st);
  if (weight_format == W_MXFP4) return launch_bm<W_MXFP4, A_BF16>(p, gate_act, grid, st);
  if (weight_format == W_INT4) return launch_bm<W_INT4, A_BF16>(p, gate_act, grid, st);
  return fail(STRIX_ERR_INVALID, "moe_gemm: weight/activation format pair not built");
}

extern "C" int strix_moe_gemm(
    void* c, const void* a, const void* w, const void* scales, const float* act_scales,
    const int32_t* sorted_ids, const int32_t* expert_ids, const int32_t* num_post_padded,
    const float* topk_weights, int64_t num_valid, int64_t a_rows, int64_t experts, int64_t n,
    int64_t k, int64_t a_stride, int64_t c_stride, int64_t w_stride_e, int64_t w_stride_n,
    int64_t s_stride_e, int64_t s_stride_n, int64_t sa_stride, int64_t sorted_len,
    int64_t expert_len, int64_t top_k, int64_t block_m, int weight_format, int act_format,
    int scale_kind, int scale_dtype, int gate_act, int c_is_f16, strix_stream_t stream) {
  STRIX_CHECK(weight_format <= W_BF16, "unknown weight format");
  STRIX_CHECK(sorted_ids != nullptr, "routing tensors must not be NULL");
  STRIX_CHECK(scale_kind != S_BLOCK || n % 128 == 0, "block scales must be fp32 [E, N/128, K/128]");
  return moe_gemm_impl(c, a, w, scales, act_scales, sorted_ids, expert_ids, num_post_padded,
                       topk_weights, num_valid, a_rows, experts, n, k, a_stride, c_stride,
                       w_stride_e, w_stride_n, s_stride_e, s_stride_n, sa_stride, sorted_len,
                       expert_len, top_k, block_m, weight_format, act_format, scale_kind,
                       scale_dtype, gate_act, c_is_f16, stream, nullptr, 0, 0);
}

extern "C" int strix_gemm_w4a16(
    void* c, const void* a, const void* w, const void* scales, const void* bias,
    const int32_t* sorted_ids, const int32_t* expert_ids, const int32_t* num_post_padded,
    const float* topk_weights, int64_t num_valid, int64_t a_rows, int64_t experts, int64_t n,
    int64_t k, int64_t a_stride, int64_t c_stride, int64_t w_stride_e, int64_t w_stride_n,
    int64_t s_stride_e, int64_t s_stride_n, int64_t bias_stride, int64_t sorted_len,
    int64_t expert_len, int64_t top_k, int64_t block_m, int weight_format, int group,
    int scale_dtype, int gate_act, strix_stream_t stream) {
  STRIX_CHECK(weight_format == W_MXFP4 || weight_format == W_INT4 || weight_format == W_INT4X,
              "weight_format 3 (mxfp4), 4 (int4) or 6 (int4, ExLlama word order)");
  return moe_gemm_impl(c, a, w, scales, nullptr, sorted_ids, expert_ids, num_post_padded,
                       topk_weights, num_valid, a_rows, experts, n, k, a_stride, c_stride,
                       w_stride_e, w_stride_n, s_stride_e, s_stride_n, 0, sorted_len, expert_len,
                       top_k, block_m, weight_format, A_BF16, S_NONE, scale_dtype, gate_act, 0,
                       stream, bias, bias_stride, group);
}

extern "C" int strix_dense_gemm_w8a16(void* c, const void* x, const void* w, const void* scales,
                                      const void* bias, int64_t m, int64_t n, int64_t k,
                                      int64_t x_stride, int64_t c_stride, int64_t w_stride,
                                      int64_t s_stride_n, int64_t bias_stride, int64_t block_m,
                                      int weight_format, int act_format, int scale_kind,
                                      int scale_dtype, int group, strix_stream_t stream) {
  STRIX_CHECK(weight_format == W_E4M3 || weight_format == W_INT8 || weight_format == W_U8B128,
              "weight_format 0 (e4m3), 1 (int8) or 5 (excess-128 bytes)");
  STRIX_CHECK(m >= 0 && block_m >= 1, "bad M / block_m");
  const int64_t sorted_len = (m + block_m - 1) / block_m * block_m;
  return moe_gemm_impl(c, x, w, scales, nullptr, nullptr, nullptr, nullptr, nullptr, m, m, 1, n, k,
                       x_stride, c_stride, 0, w_stride, 0, s_stride_n, 0, sorted_len, 0, 1, block_m,
                       weight_format, act_format, scale_kind, scale_dtype, ACT_NONE, 0, stream, bias,
                       bias_stride, group);
}

extern "C" int strix_gemm_w8a8_group(
    void* c, const void* qa, const float* sa, const void* w, const void* scales,
    const int32_t* sorted_ids, const int32_t* expert_ids, const int32_t* num_post_padded,
    const float* topk_weights, int64_t num_valid, int64_t a_rows, int64_t experts, int64_t n,
    int64_t k, int64_t a_stride, int64_t c_stride, int64_t w_stride_e, int64_t w_stride_n,
    int64_t s_stride_e, int64_t s_stride_n, int64_t s_stride_g, int64_t sa_stride,
    int64_t sorted_len, int64_t expert_len, int64_t top_k, int64_t block_m, int weight_format,
    int scale_kind, int scale_dtype, int gate_act, strix_stream_t stream) {
  STRIX_CHECK(weight_format == W_INT4 || weight_format == W_U8B128 || weight_format == W_INT4X,
              "weight_format 4 (int4), 5 (excess-128 bytes) or 6 (int4, ExLlama word order)");
  return moe_gemm_impl(c, qa, w, scales, sa, sorted_ids, expert_ids, num_post_padded, topk_weights,
                       num_valid, a_rows, experts, n, k, a_stride, c_stride, w_stride_e, w_stride_n,
                       s_stride_e, s_stride_n, sa_stride, sorted_len, expert_len, top_k, block_m,
                       weight_format, A_INT8, scale_kind, scale_dtype, gate_act, 0, stream, nullptr, 0,
                       128, s_stride_g);
}
