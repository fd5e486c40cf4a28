// Paged decode attention (one query token per sequence) over an int8 or bf16
// KV cache, for sm_100a.
//
// Semantics follow strix::attn_decode_bf16 (csrc/attn/attn_decode_bf16.hip:28-300
// of the reference): exp2-domain online softmax, K scale multiplies the score,
// V scale multiplies P, l is the unweighted sum of p, split-KV partials
// (m, l, un-normalised O) combined by a second kernel, sinks folded after the
// combine, window_left keys to the left of the query.
//
// Design (HBM-bound: 1,056 bytes per key per sequence at 4 KV heads, D = 128):
//   * one CTA per (segment, sequence, group of KV heads); its 8 warps are split
//     over the KV heads of the group, so the warps of one CTA walk the same
//     pages at the same time and each page is fetched from DRAM once;
//   * a warp owns whole 16-key tiles: K and V bytes go global -> registers with
//     128-bit loads (a row of one head is read by 4 or 8 adjacent lanes as one
//     contiguous run), double-buffered one tile ahead, block-table entries 32
//     tiles ahead;
//   * int8 -> fp16 is exact and done with byte permutes (0x6400 | (b ^ 0x80) is
//     1024 + b + 128), which also performs the V transposition for free;
//   * scores are S^T = K Q^T with the 16 keys as the MMA M dimension and the
//     (up to) 8 query heads of the KV head as N, so no tensor-core work is
//     wasted on padding; P^T comes from the score fragment with two
//     movmatrix transposes; O^T = V^T P^T accumulates in fp32 registers;
//   * each warp keeps its own (m, l, O); warps of a head merge through shared
//     memory once, at the end.
#include <cstdlib>

#include "common.cuh"

namespace strix {
namespace {

constexpr uint32_t kMagic = 0x64646464u;   // high byte of fp16 1024 + x
// The softmax reference of a warp is renewed only when a score exceeds it by more
// than 2^kLazy: the weights then stay below 2^kLazy, and kPScale = 2^(15 - kLazy)
// keeps the V-scaled fp16 weights in range.
constexpr float kLazy = 4.f;
constexpr float kPScale = 2048.f;
constexpr float kPScaleInv = 1.f / 2048.f;

// Bytes of one ring stage: 16 K rows, 16 V rows, 16 + 16 fp32 scales.
constexpr int stage_bytes(int d) { return 2 * 16 * d + 128; }

struct DecodeArgs {
  __nv_bfloat16* out;
  const __nv_bfloat16* q;
  const void* kc;
  const void* vc;
  const float* ksc;
  const float* vsc;
  const int32_t* seq_lens;
  const int32_t* bt;
  const float* sinks;
  float* o_part;
  float* ml_part;
  int64_t bt_stride, q_st, q_sh, o_st, o_sh;
  int64_t k_sb, k_ss, k_sh, v_sb, v_ss, v_sh;
  int64_t ks_sb, ks_ss, ks_sh, vs_sb, vs_ss, vs_sh;
  int block_size, hq, hkv, g, hpc;  // hpc: KV heads per CTA
  int nseg, seg_keys, win_left;
  float scale_log2;
  int tpb_shift;  // log2(16-key tiles per page) when that is a power of two, else -1
};

// Page-table index and first row within the page of 16-key tile t: shifts for
// power-of-two pages, a division only for the others.
__device__ __forceinline__ int tile_page(const DecodeArgs& a, int t) {
  return a.tpb_shift >= 0 ? t >> a.tpb_shift : (t * 16) / a.block_size;
}
__device__ __forceinline__ int tile_row(const DecodeArgs& a, int t) {
  return a.tpb_shift >= 0 ? (t & ((1 << a.tpb_shift) - 1)) << 4 : (t * 16) % a.block_size;
}

template <int NW, bool ALIGNED>
__device__ __forceinline__ void load_words(uint32_t (&dst)[NW], const uint8_t* p) {
  if constexpr (ALIGNED) {
    static_assert(NW % 4 == 0, "vector path needs whole uint4s");
#pragma unroll
    for (int i = 0; i < NW / 4; ++i) {
      const uint4 x = ldg_stream(p + 16 * i);
      dst[4 * i] = x.x;
      dst[4 * i + 1] = x.y;
      dst[4 * i + 2] = x.z;
      dst[4 * i + 3] = x.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < NW; ++i)
      dst[i] = __ldg(reinterpret_cast<const uint32_t*>(p + 4 * i));
  }
}

// One 16-key tile of one KV head as this lane sees it. With g = lane / 4 and
// c = lane % 4: K rows g and g + 8, bytes [c * D/4, (c + 1) * D/4) of each;
// V rows 2c, 2c + 1, 2c + 8, 2c + 9, bytes [g * D/8, (g + 1) * D/8) of each.
template <int D>
struct TileQ8 {
  uint32_t k[2][D / 16];
  uint32_t v[4][D / 32];
  float ks[2], vs[2];
};

template <int D, bool ALIGNED>
__device__ __forceinline__ void load_tile(TileQ8<D>& t, const DecodeArgs& a, int blk,
                                          int off, int kvh, int g, int c) {
  const uint8_t* kb = static_cast<const uint8_t*>(a.kc) + int64_t(blk) * a.k_sb +
                      int64_t(off) * a.k_ss + int64_t(kvh) * a.k_sh + c * (D / 4);
  load_words<D / 16, ALIGNED>(t.k[0], kb + int64_t(g) * a.k_ss);
  load_words<D / 16, ALIGNED>(t.k[1], kb + int64_t(g + 8) * a.k_ss);
  const uint8_t* vb = static_cast<const uint8_t*>(a.vc) + int64_t(blk) * a.v_sb +
                      int64_t(off) * a.v_ss + int64_t(kvh) * a.v_sh + g * (D / 8);
  load_words<D / 32, ALIGNED>(t.v[0], vb + int64_t(2 * c) * a.v_ss);
  load_words<D / 32, ALIGNED>(t.v[1], vb + int64_t(2 * c + 1) * a.v_ss);
  load_words<D / 32, ALIGNED>(t.v[2], vb + int64_t(2 * c + 8) * a.v_ss);
  load_words<D / 32, ALIGNED>(t.v[3], vb + int64_t(2 * c + 9) * a.v_ss);
  const float* ksp = a.ksc + int64_t(blk) * a.ks_sb + int64_t(off) * a.ks_ss +
                     int64_t(kvh) * a.ks_sh;
  const float* vsp = a.vsc + int64_t(blk) * a.vs_sb + int64_t(off) * a.vs_ss +
                     int64_t(kvh) * a.vs_sh;
  t.ks[0] = __ldg(ksp + int64_t(g) * a.ks_ss);
  t.ks[1] = __ldg(ksp + int64_t(g + 8) * a.ks_ss);
  t.vs[0] = __ldg(vsp + int64_t(g) * a.vs_ss);
  t.vs[1] = __ldg(vsp + int64_t(g + 8) * a.vs_ss);
}

// Per-warp running softmax state for the two query heads 2c and 2c + 1 this
// lane holds scores for, and the O^T accumulator: acc[t] covers head dims
// g * D/8 + 2t (c0, c1) and + 2t + 1 (c2, c3) for heads 2c (c0, c2), 2c + 1.
template <int D>
struct WarpState {
  float m[2], l[2];
  float acc[D / 16][4];
  float wsum[4];   // sum of the fp16 weights per head (computed by the MMA): see compute_tile
};

// Query fragments for the score MMAs. The bf16 query of a head is turned into
// 16-bit fixed point against the head's absmax, q = s * (256 * hi + lo) with
// hi a signed and lo an unsigned byte (error <= absmax * 2^-16, far below
// bf16's own resolution), so that S^T = K Q^T runs as two exact int8 MMAs on
// the raw cache bytes with no widening of K at all.
template <int D>
struct QFrag {
  uint32_t hi[D / 16], lo[D / 16];
  float qs[2];  // s * softmax_scale * log2(e) for heads 2c and 2c + 1
};

// (A second instantiation without the per-key tests for tiles wholly inside
// [k_begin, k_end) was measured: it spills at the 128-register cap and is slower.)
template <int D>
__device__ __forceinline__ void compute_tile(const TileQ8<D>& t, WarpState<D>& st,
                                             const QFrag<D>& qf, int key0, int k_begin,
                                             int k_end, int g) {
  // S^T[16 keys, 8 heads] = K Q^T, int32-exact
  int sh[4] = {0, 0, 0, 0}, sl[4] = {0, 0, 0, 0};
#pragma unroll
  for (int i = 0; i < D / 32; ++i) {
    const uint32_t a[4] = {t.k[0][2 * i], t.k[1][2 * i], t.k[0][2 * i + 1], t.k[1][2 * i + 1]};
    mma_s8s8_16832(sh, a, qf.hi[2 * i], qf.hi[2 * i + 1]);
    mma_s8u8_16832(sl, a, qf.lo[2 * i], qf.lo[2 * i + 1]);
  }
  float s[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) s[i] = float(sh[i] * 256 + sl[i]);
  s[0] *= qf.qs[0];
  s[1] *= qf.qs[1];
  s[2] *= qf.qs[0];
  s[3] *= qf.qs[1];
  const int ka = key0 + g, kb = ka + 8;
  const bool va = ka >= k_begin && ka < k_end, vb = kb >= k_begin && kb < k_end;
  const float ksa = t.ks[0], ksb = t.ks[1];
  const float x0 = va ? s[0] * ksa : -INFINITY, x1 = va ? s[1] * ksa : -INFINITY;
  const float x2 = vb ? s[2] * ksb : -INFINITY, x3 = vb ? s[3] * ksb : -INFINITY;
  // The running reference is max(x + log2|v_scale|), not max(x): then the
  // V-scaled weights p * |v_scale| are bounded whatever the scale's magnitude, and
  // kPScale lifts them into fp16's normal range (tiny weights of a 65k-key
  // softmax would otherwise land in fp16 subnormals). m, l and O all use the
  // same reference, so the split-KV merge formulas are unchanged. A stale scale
  // of a masked key may be anything (NaN included): it is replaced.
  const float lva = va ? fmaxf(fast_log2(fabsf(t.vs[0])), -100.f) : 0.f;
  const float lvb = vb ? fmaxf(fast_log2(fabsf(t.vs[1])), -100.f) : 0.f;
  const float c0 = fmaxf(x0 + lva, x2 + lvb), c1 = fmaxf(x1 + lva, x3 + lvb);
  // The reference is any upper bound minus at most kLazy, the same in the eight
  // lanes that share a head: it is renewed (warp-wide maximum, accumulators
  // rescaled) only when some score outgrew it by more than 2^kLazy - after the
  // first tiles almost never, which saves the shuffles and the rescale test.
  if (__any_sync(0xffffffffu, c0 > st.m[0] + kLazy || c1 > st.m[1] + kLazy)) {
    float mx0 = c0, mx1 = c1;
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, o));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o));
    }
    const float mn0 = fmaxf(st.m[0], mx0), mn1 = fmaxf(st.m[1], mx1);
    const float al0 = mn0 == -INFINITY ? 1.f : fast_exp2(st.m[0] - mn0);
    const float al1 = mn1 == -INFINITY ? 1.f : fast_exp2(st.m[1] - mn1);
    st.m[0] = mn0;
    st.m[1] = mn1;
    st.l[0] *= al0;
    st.l[1] *= al1;
#pragma unroll
    for (int i = 0; i < D / 16; ++i) {
      st.acc[i][0] *= al0;
      st.acc[i][1] *= al1;
      st.acc[i][2] *= al0;
      st.acc[i][3] *= al1;
    }
    st.wsum[0] *= al0, st.wsum[1] *= al1, st.wsum[2] *= al0, st.wsum[3] *= al1;
  }
  const float r0 = st.m[0] == -INFINITY ? 0.f : st.m[0], r1 = st.m[1] == -INFINITY ? 0.f : st.m[1];
  const float p0 = fast_exp2(x0 - r0), p1 = fast_exp2(x1 - r1);
  const float p2 = fast_exp2(x2 - r0), p3 = fast_exp2(x3 - r1);
  st.l[0] += p0 + p2;
  st.l[1] += p1 + p3;
  const float vsa = va ? t.vs[0] * kPScale : 0.f, vsb = vb ? t.vs[1] * kPScale : 0.f;
  const uint32_t b0 = movmatrix_trans(pack_f16x2(p0 * vsa, p1 * vsa));
  const uint32_t b1 = movmatrix_trans(pack_f16x2(p2 * vsb, p3 * vsb));
  // The V bytes enter the MMA as fp16 1024 + (b + 128) - one byte permute per
  // register, no subtraction: V^T P^T then carries the offset 1152 x (sum of the
  // weights), and that sum comes out of one more MMA with an all-ones A operand
  // (exactly the fp16-rounded weights the other MMAs see), so the offset is
  // removed once per launch, in fp32, when the accumulators are merged.
  uint32_t vx[4][D / 32];
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int w = 0; w < D / 32; ++w) vx[r][w] = t.v[r][w] ^ 0x80808080u;
  {
    const uint32_t ones[4] = {0x3C003C00u, 0x3C003C00u, 0x3C003C00u, 0x3C003C00u};
    mma_f16_16816(st.wsum, ones, b0, b1);
  }
#pragma unroll
  for (int i = 0; i < D / 16; ++i) {
    const int w = i / 2;
    const uint32_t sel = (i & 1) ? 0x7362u : 0x5140u;
    const uint32_t x01 = prmt(vx[0][w], vx[1][w], sel);
    const uint32_t x23 = prmt(vx[2][w], vx[3][w], sel);
    uint32_t a[4];
    a[0] = prmt(x01, kMagic, 0x4140);
    a[1] = prmt(x01, kMagic, 0x4342);
    a[2] = prmt(x23, kMagic, 0x4140);
    a[3] = prmt(x23, kMagic, 0x4342);
    mma_f16_16816(st.acc[i], a, b0, b1);
  }
}

// STAGES == 0: tiles go global -> registers, double-buffered (any 4-byte-aligned
// layout). STAGES >= 2: each warp owns a ring of STAGES tiles in shared memory
// filled with 16-byte cp.async copies STAGES - 1 tiles ahead (rows 16-byte
// aligned); 16-byte chunks are XOR-swizzled by row so that both the K and the V
// fragment reads are bank-conflict free. No barrier or flag is shared between
// warps in the main loop.
template <int D, bool ALIGNED, int kWarps, int kMinCtas, int STAGES>
__global__ void __launch_bounds__(kWarps * 32, kMinCtas)
attn_decode_q8_kernel(const DecodeArgs a) {
  pdl_enter();
  constexpr int kThreads = kWarps * 32;
  extern __shared__ __align__(128) uint8_t dyn_smem[];
  const int seg = blockIdx.x, hgrp = blockIdx.y, n = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, c = lane & 3;
  const int hslot = warp % a.hpc;           // KV head within the CTA's group
  const int sub = warp / a.hpc;             // this warp's rank among the head's warps
  const int wph = kWarps / a.hpc;           // warps per KV head
  const int kvh = hgrp * a.hpc + hslot;
  const int G = a.g;
  const int h0 = kvh * G;

  const int kv_len = a.seq_lens[n];
  const int pos = kv_len - 1;
  const int k_lo = a.win_left >= 0 ? max(0, pos - a.win_left) : 0;
  const int seg_len = a.seg_keys > 0
                          ? a.seg_keys
                          : ((kv_len - k_lo + a.nseg - 1) / a.nseg + 15) / 16 * 16;
  const int k_begin = k_lo + seg * seg_len;
  const int k_end = min(kv_len, k_begin + seg_len);
  const bool single = a.nseg == 1;

  __shared__ float s_m[kWarps][8], s_l[kWarps][8];
  float* const s_o = reinterpret_cast<float*>(dyn_smem);  // [hpc][8][D], after the main loop

  if (k_begin >= k_end) {  // empty segment (block-uniform)
    const int heads = a.hpc * G;
    if (single) {
      for (int i = threadIdx.x; i < heads * D; i += kThreads) {
        const int h = hgrp * heads + i / D;
        a.out[int64_t(n) * a.o_st + int64_t(h) * a.o_sh + i % D] = __float2bfloat16(0.f);
      }
    } else if (threadIdx.x < heads) {
      const int h = hgrp * heads + threadIdx.x;
      float* ml = a.ml_part + ((int64_t(n) * a.hq + h) * a.nseg + seg) * 2;
      ml[0] = -INFINITY;
      ml[1] = 0.f;
    }
    return;
  }

  // Q^T fragments: head g of this KV head, dims c * D/4 + 8i .. + 7 for k-step i
  // (the same permutation of head dims that the K loads use).
  QFrag<D> qf;
  {
    float qv[D / 4];
    float amax = 0.f;
    if (g < G) {
      const __nv_bfloat16* qp =
          a.q + int64_t(n) * a.q_st + int64_t(h0 + g) * a.q_sh + c * (D / 4);
#pragma unroll
      for (int i = 0; i < D / 16; ++i) {
        const uint2 w = *reinterpret_cast<const uint2*>(qp + 4 * i);
        qv[4 * i] = bf16_lo(w.x);
        qv[4 * i + 1] = bf16_hi(w.x);
        qv[4 * i + 2] = bf16_lo(w.y);
        qv[4 * i + 3] = bf16_hi(w.y);
      }
#pragma unroll
      for (int i = 0; i < D / 4; ++i) amax = fmaxf(amax, fabsf(qv[i]));
    } else {
#pragma unroll
      for (int i = 0; i < D / 4; ++i) qv[i] = 0.f;
    }
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    const float step = amax > 0.f ? amax * (1.f / 32767.f) : 1.f;
    const float inv = 1.f / step;
#pragma unroll
    for (int i = 0; i < D / 16; ++i) {
      uint32_t hi = 0, lo = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int f = __float2int_rn(qv[4 * i + j] * inv);
        hi |= (uint32_t(f >> 8) & 0xffu) << (8 * j);
        lo |= (uint32_t(f) & 0xffu) << (8 * j);
      }
      qf.hi[i] = hi;
      qf.lo[i] = lo;
    }
    const float qs = step * a.scale_log2;
    qf.qs[0] = __shfl_sync(0xffffffffu, qs, 8 * c);
    qf.qs[1] = __shfl_sync(0xffffffffu, qs, 8 * c + 4);
  }

  WarpState<D> st;
  st.m[0] = st.m[1] = -INFINITY;
  st.l[0] = st.l[1] = 0.f;
  st.wsum[0] = st.wsum[1] = st.wsum[2] = st.wsum[3] = 0.f;
#pragma unroll
  for (int i = 0; i < D / 16; ++i)
    st.acc[i][0] = st.acc[i][1] = st.acc[i][2] = st.acc[i][3] = 0.f;

  // Tiles are aligned to 16 keys from position 0, so a tile never straddles a
  // page (block_size is a multiple of 16).
  const int t_begin = k_begin >> 4, t_end = (k_end + 15) >> 4;
  const int32_t* bt = a.bt + int64_t(n) * a.bt_stride;

  auto run_tile = [&](const TileQ8<D>& tile, int key0) {
    compute_tile<D>(tile, st, qf, key0, k_begin, k_end, g);
  };

  int my_blk = 0, nload = 0;
  // Returns the block id of this warp's nload-th tile; every 32 tiles each lane
  // fetches one entry ahead of use.
  auto next_block = [&](int tile) {
    if ((nload & 31) == 0) {
      const int tl = tile + lane * wph;
      my_blk = tl < t_end ? bt[tile_page(a, tl)] : 0;
    }
    const int blk = __shfl_sync(0xffffffffu, my_blk, nload & 31);
    ++nload;
    return blk;
  };

  if constexpr (STAGES == 0) {
    TileQ8<D> ta, tb;
    int t = t_begin + sub;
    if (t < t_end) {
      const int blk = next_block(t);
      load_tile<D, ALIGNED>(ta, a, blk, tile_row(a, t), kvh, g, c);
    }
    while (t < t_end) {
      if (t + wph < t_end) {
        const int blk = next_block(t + wph);
        load_tile<D, ALIGNED>(tb, a, blk, tile_row(a, t + wph), kvh, g, c);
      }
      run_tile(ta, t * 16);
      t += wph;
      if (t >= t_end) break;
      if (t + wph < t_end) {
        const int blk = next_block(t + wph);
        load_tile<D, ALIGNED>(ta, a, blk, tile_row(a, t + wph), kvh, g, c);
      }
      run_tile(tb, t * 16);
      t += wph;
    }
  } else {
    constexpr int kStage = stage_bytes(D);
    constexpr int CPR = D / 16;       // 16-byte chunks per row
    constexpr int RPI = 32 / CPR;     // rows one warp-wide copy instruction covers
    uint8_t* const ring = dyn_smem + warp * (STAGES * kStage);
    const uint32_t ring_s = static_cast<uint32_t>(__cvta_generic_to_shared(ring));
    const int crow = lane / CPR, cch = lane % CPR;
    const int64_t k_lane = int64_t(crow) * a.k_ss + cch * 16 + int64_t(kvh) * a.k_sh;
    const int64_t v_lane = int64_t(crow) * a.v_ss + cch * 16 + int64_t(kvh) * a.v_sh;
    const bool is_k = lane < 16;
    const float* sc_base = is_k ? a.ksc + int64_t(kvh) * a.ks_sh + int64_t(lane) * a.ks_ss
                                : a.vsc + int64_t(kvh) * a.vs_sh + int64_t(lane - 16) * a.vs_ss;
    const int64_t sc_sb = is_k ? a.ks_sb : a.vs_sb, sc_ss = is_k ? a.ks_ss : a.vs_ss;

    int t_issue = t_begin + sub, stage_issue = 0;
    auto issue_next = [&]() {
      if (t_issue < t_end) {
        const int blk = next_block(t_issue);
        const int off = tile_row(a, t_issue);
        const uint8_t* kp = static_cast<const uint8_t*>(a.kc) + int64_t(blk) * a.k_sb +
                            int64_t(off) * a.k_ss + k_lane;
        const uint8_t* vp = static_cast<const uint8_t*>(a.vc) + int64_t(blk) * a.v_sb +
                            int64_t(off) * a.v_ss + v_lane;
        const uint32_t dst = ring_s + stage_issue * kStage;
#pragma unroll
        for (int j = 0; j < 16 / RPI; ++j) {
          const int row = j * RPI + crow;
          const uint32_t d = dst + row * D + ((cch ^ (row & 7)) << 4);
          cp_async_16(d, kp + int64_t(j * RPI) * a.k_ss);
          cp_async_16(d + 16 * D, vp + int64_t(j * RPI) * a.v_ss);
        }
        cp_async_4(dst + 32 * D + lane * 4, sc_base + int64_t(blk) * sc_sb + int64_t(off) * sc_ss);
      }
      cp_async_commit();
      t_issue += wph;
      stage_issue = stage_issue + 1 == STAGES ? 0 : stage_issue + 1;
    };
#pragma unroll
    for (int i = 0; i < STAGES - 1; ++i) issue_next();
    int stage = 0;
    for (int t = t_begin + sub; t < t_end; t += wph) {
      issue_next();
      cp_async_wait<STAGES - 1>();
      __syncwarp();
      TileQ8<D> tile;
      const uint8_t* sp = ring + stage * kStage;
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const uint8_t* rowp = sp + (g + 8 * r) * D;
#pragma unroll
        for (int i = 0; i < D / 64; ++i) {
          const uint4 x = *reinterpret_cast<const uint4*>(rowp + (((c * (D / 64) + i) ^ g) << 4));
          tile.k[r][4 * i] = x.x, tile.k[r][4 * i + 1] = x.y;
          tile.k[r][4 * i + 2] = x.z, tile.k[r][4 * i + 3] = x.w;
        }
      }
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int row = 2 * c + (r & 1) + 8 * (r >> 1);
        const uint8_t* rowp = sp + 16 * D + row * D;
#pragma unroll
        for (int i = 0; i < D / 128; ++i) {
          const uint4 x =
              *reinterpret_cast<const uint4*>(rowp + (((g * (D / 128) + i) ^ (row & 7)) << 4));
          tile.v[r][4 * i] = x.x, tile.v[r][4 * i + 1] = x.y;
          tile.v[r][4 * i + 2] = x.z, tile.v[r][4 * i + 3] = x.w;
        }
      }
      const float* scp = reinterpret_cast<const float*>(sp + 32 * D);
      tile.ks[0] = scp[g], tile.ks[1] = scp[g + 8];
      tile.vs[0] = scp[16 + g], tile.vs[1] = scp[24 + g];
      run_tile(tile, t * 16);
      __syncwarp();
      stage = stage + 1 == STAGES ? 0 : stage + 1;
    }
    cp_async_wait<0>();
  }

  // ---- merge the warps of each KV head ------------------------------------
#pragma unroll
  for (int o = 4; o < 32; o <<= 1) {
    st.l[0] += __shfl_xor_sync(0xffffffffu, st.l[0], o);
    st.l[1] += __shfl_xor_sync(0xffffffffu, st.l[1], o);
  }
  if (g == 0) {
    s_m[warp][2 * c] = st.m[0];
    s_m[warp][2 * c + 1] = st.m[1];
    s_l[warp][2 * c] = st.l[0];
    s_l[warp][2 * c + 1] = st.l[1];
  }
  __syncthreads();
  float M[2] = {-INFINITY, -INFINITY}, L[2] = {0.f, 0.f};
  for (int w = hslot; w < kWarps; w += a.hpc) {
    M[0] = fmaxf(M[0], s_m[w][2 * c]);
    M[1] = fmaxf(M[1], s_m[w][2 * c + 1]);
  }
  for (int w = hslot; w < kWarps; w += a.hpc) {
    const float m0 = s_m[w][2 * c], m1 = s_m[w][2 * c + 1];
    L[0] += m0 == -INFINITY ? 0.f : s_l[w][2 * c] * fast_exp2(m0 - M[0]);
    L[1] += m1 == -INFINITY ? 0.f : s_l[w][2 * c + 1] * fast_exp2(m1 - M[1]);
  }
  {
    const float f0 = st.m[0] == -INFINITY ? 0.f : fast_exp2(st.m[0] - M[0]) * kPScaleInv;
    const float f1 = st.m[1] == -INFINITY ? 0.f : fast_exp2(st.m[1] - M[1]) * kPScaleInv;
    // the offset the unsubtracted V operand left behind: 1152 x the weights' sum
    const float off0 = 1152.f * st.wsum[0], off1 = 1152.f * st.wsum[1];
#pragma unroll
    for (int i = 0; i < D / 16; ++i) {
      st.acc[i][0] = (st.acc[i][0] - off0) * f0;
      st.acc[i][1] = (st.acc[i][1] - off1) * f1;
      st.acc[i][2] = (st.acc[i][2] - off0) * f0;
      st.acc[i][3] = (st.acc[i][3] - off1) * f1;
    }
  }
  // s_o[slot][head][d]: lane owns dims g * D/8 + 2i, + 2i + 1 of heads 2c, 2c + 1.
  float* so0 = s_o + (hslot * 8 + 2 * c) * D + g * (D / 8);
  float* so1 = so0 + D;
  for (int r = wph - 1; r >= 1; --r) {
    if (sub == r) {
#pragma unroll
      for (int i = 0; i < D / 16; ++i) {
        *reinterpret_cast<float2*>(so0 + 2 * i) = make_float2(st.acc[i][0], st.acc[i][2]);
        *reinterpret_cast<float2*>(so1 + 2 * i) = make_float2(st.acc[i][1], st.acc[i][3]);
      }
    }
    __syncthreads();
    if (sub == 0) {
#pragma unroll
      for (int i = 0; i < D / 16; ++i) {
        const float2 x = *reinterpret_cast<const float2*>(so0 + 2 * i);
        const float2 y = *reinterpret_cast<const float2*>(so1 + 2 * i);
        st.acc[i][0] += x.x;
        st.acc[i][2] += x.y;
        st.acc[i][1] += y.x;
        st.acc[i][3] += y.y;
      }
    }
    __syncthreads();
  }
  if (sub != 0) return;

  // ---- write: final rows (single segment) or partials ----------------------
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int hl = 2 * c + j;
    if (hl >= G) continue;
    const int h = h0 + hl;
    if (single) {
      float inv = L[j] > 0.f ? 1.f / L[j] : 0.f;
      if (a.sinks != nullptr) {
        const float s2 = a.sinks[h] * kLog2e;
        const float mf = fmaxf(M[j], s2);
        const float al = M[j] == -INFINITY ? 0.f : fast_exp2(M[j] - mf);
        inv = al / (L[j] * al + fast_exp2(s2 - mf));
      }
      __nv_bfloat16* op = a.out + int64_t(n) * a.o_st + int64_t(h) * a.o_sh + g * (D / 8);
#pragma unroll
      for (int i = 0; i < D / 16; ++i)
        *reinterpret_cast<uint32_t*>(op + 2 * i) =
            pack_bf16x2(st.acc[i][j] * inv, st.acc[i][2 + j] * inv);
    } else {
      const int64_t row = (int64_t(n) * a.hq + h) * a.nseg + seg;
      float* op = a.o_part + row * D + g * (D / 8);
#pragma unroll
      for (int i = 0; i < D / 16; ++i)
        *reinterpret_cast<float2*>(op + 2 * i) = make_float2(st.acc[i][j], st.acc[i][2 + j]);
      if (g == 0) {
        a.ml_part[2 * row] = M[j];
        a.ml_part[2 * row + 1] = L[j];
      }
    }
  }
}

// ---------------------------------------------------------------------------
// The same operation over a bf16 KV cache (the reference's native form). One warp
// per KV head of the CTA's group, no cross-warp merge: a warp owns 16-key tiles of
// 2 x 16 x D bf16 that arrive through a per-warp cp.async ring (3 stages, 16-byte
// chunks XOR-swizzled by row); S^T = K Q^T and O^T = V^T P^T are bf16
// mma.sync.m16n8k16 whose A fragments come from ldmatrix (transposing for V), so
// neither K nor V is touched by an ordinary instruction. Softmax, split-KV
// partials and the reduce are those of the int8 kernel.
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                               uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

constexpr int kBfStages = 3;

// SPLIT = 2 (head 512): two warps share a KV head, each owning D = 256 of its dims -
// that half of every K and V row in its own ring, that half of Q and of O. Each
// computes the score partials over its dims; the pair exchanges them through shared
// memory (two buffers by tile parity, one 64-thread named barrier per tile) and then
// holds the same scores, maxima and sums.
template <int D, int SPLIT>
__global__ void __launch_bounds__(128) attn_decode_bf16kv_kernel(const DecodeArgs a) {
  pdl_enter();
  constexpr int kRow = D * 2;                 // bytes of this warp's part of a cache row
  constexpr int kChunks = kRow / 16;          // 16-byte chunks per row
  constexpr int kTile = 16 * kRow;            // K (or V) rows of a tile
  constexpr int kStage = 2 * kTile;
  extern __shared__ __align__(128) uint8_t dyn_smem[];
  const int seg = blockIdx.x, hgrp = blockIdx.y, n = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, c = lane & 3;
  const int hslot = warp / SPLIT, half = warp % SPLIT;
  const int kvh = hgrp * a.hpc + hslot;       // blockDim.x = 32 * hpc * SPLIT
  const int d0 = half * D;                    // first head dim of this warp
  const int G = a.g;
  const int h0 = kvh * G;

  const int kv_len = a.seq_lens[n];
  const int pos = kv_len - 1;
  const int k_lo = a.win_left >= 0 ? max(0, pos - a.win_left) : 0;
  const int seg_len = a.seg_keys > 0 ? a.seg_keys
                                     : ((kv_len - k_lo + a.nseg - 1) / a.nseg + 15) / 16 * 16;
  const int k_begin = k_lo + seg * seg_len;
  const int k_end = min(kv_len, k_begin + seg_len);
  const bool single = a.nseg == 1;

  if (k_begin >= k_end) {                     // empty segment (block-uniform)
    for (int j = 0; j < 2; ++j) {
      const int hl = 2 * c + j;
      if (hl >= G) continue;
      const int h = h0 + hl;
      if (single) {
        for (int d = g; d < D; d += 8)
          a.out[int64_t(n) * a.o_st + int64_t(h) * a.o_sh + d0 + d] = __float2bfloat16(0.f);
      } else if (g == 0 && half == 0) {
        float* ml = a.ml_part + ((int64_t(n) * a.hq + h) * a.nseg + seg) * 2;
        ml[0] = -INFINITY;
        ml[1] = 0.f;
      }
    }
    return;
  }

  // Q^T fragments: b0 / b1 of k-step ks = q[head g][16 ks + 2c, + 1] / [16 ks + 8 + 2c, + 1]
  uint32_t qb[D / 16][2];
  {
    const __nv_bfloat16* qp = a.q + int64_t(n) * a.q_st + int64_t(h0 + g) * a.q_sh + d0;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      qb[ks][0] = g < G ? *reinterpret_cast<const uint32_t*>(qp + 16 * ks + 2 * c) : 0u;
      qb[ks][1] = g < G ? *reinterpret_cast<const uint32_t*>(qp + 16 * ks + 8 + 2 * c) : 0u;
    }
  }
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float acc[D / 16][4];
#pragma unroll
  for (int i = 0; i < D / 16; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;

  const int t_begin = k_begin >> 4, t_end = (k_end + 15) >> 4;
  const int32_t* bt = a.bt + int64_t(n) * a.bt_stride;
  uint8_t* const ring = dyn_smem + warp * (kBfStages * kStage);
  const uint32_t ring_s = static_cast<uint32_t>(__cvta_generic_to_shared(ring));
  const uint8_t* const kc = static_cast<const uint8_t*>(a.kc) + (int64_t(kvh) * a.k_sh + d0) * 2;
  const uint8_t* const vc = static_cast<const uint8_t*>(a.vc) + (int64_t(kvh) * a.v_sh + d0) * 2;
  // score partials of the pair: [parity][hslot][half][lane] float4, behind the rings
  float4* const xch = reinterpret_cast<float4*>(dyn_smem + a.hpc * SPLIT * (kBfStages * kStage));

  int t_issue = t_begin, stage_issue = 0;
  auto issue_next = [&]() {
    if (t_issue < t_end) {
      const int blk = bt[tile_page(a, t_issue)];
      const int off = tile_row(a, t_issue);
      const uint8_t* kp = kc + (int64_t(blk) * a.k_sb + int64_t(off) * a.k_ss) * 2;
      const uint8_t* vp = vc + (int64_t(blk) * a.v_sb + int64_t(off) * a.v_ss) * 2;
      const uint32_t dst = ring_s + stage_issue * kStage;
#pragma unroll
      for (int j = 0; j < 16 * kChunks / 32; ++j) {
        const int idx = j * 32 + lane, row = idx / kChunks, ch = idx % kChunks;
        const uint32_t d = dst + row * kRow + ((ch ^ (row & 7)) << 4);
        cp_async_16(d, kp + int64_t(row) * a.k_ss * 2 + ch * 16);
        cp_async_16(d + kTile, vp + int64_t(row) * a.v_ss * 2 + ch * 16);
      }
    }
    cp_async_commit();
    ++t_issue;
    stage_issue = stage_issue + 1 == kBfStages ? 0 : stage_issue + 1;
  };
#pragma unroll
  for (int i = 0; i < kBfStages - 1; ++i) issue_next();
  int stage = 0;
  for (int t = t_begin; t < t_end; ++t) {
    issue_next();
    cp_async_wait<kBfStages - 1>();
    __syncwarp();
    const uint32_t ks_s = ring_s + stage * kStage, vs_s = ks_s + kTile;
    const int key0 = t * 16;
    // rows of keys outside [k_begin, k_end) may hold anything (NaN bit patterns too):
    // their scores are masked below, their V rows are zeroed here
    if (key0 < k_begin || key0 + 16 > k_end) {
      for (int idx = lane; idx < 16 * kChunks; idx += 32) {
        const int row = idx / kChunks;
        const int key = key0 + row;
        if (key < k_begin || key >= k_end)
          *reinterpret_cast<uint4*>(ring + stage * kStage + kTile + idx * 16) = make_uint4(0u, 0u, 0u, 0u);
      }
      __syncwarp();
    }
    // S^T[16 keys, 8 heads] = K Q^T
    float sc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      uint32_t af[4];
      const int row = lane & 15, ch = 2 * ks + (lane >> 4);
      ldmatrix_x4(af, ks_s + row * kRow + ((ch ^ (row & 7)) << 4));
      mma_bf16_16816(sc, af, qb[ks][0], qb[ks][1]);
    }
    if constexpr (SPLIT == 2) {
      float4* const mine = xch + (((t & 1) * a.hpc + hslot) * 2 + half) * 32 + lane;
      *mine = make_float4(sc[0], sc[1], sc[2], sc[3]);
      asm volatile("bar.sync %0, 64;" ::"r"(hslot + 1) : "memory");
      const float4 other = half == 0 ? mine[32] : mine[-32];
      sc[0] += other.x, sc[1] += other.y, sc[2] += other.z, sc[3] += other.w;
    }
    const int ka = key0 + g, kb = ka + 8;
    const bool va = ka >= k_begin && ka < k_end, vb = kb >= k_begin && kb < k_end;
    const float x0 = va ? sc[0] * a.scale_log2 : -INFINITY, x1 = va ? sc[1] * a.scale_log2 : -INFINITY;
    const float x2 = vb ? sc[2] * a.scale_log2 : -INFINITY, x3 = vb ? sc[3] * a.scale_log2 : -INFINITY;
    const float c0 = fmaxf(x0, x2), c1 = fmaxf(x1, x3);
    if (__any_sync(0xffffffffu, c0 > m[0] + kLazy || c1 > m[1] + kLazy)) {
      float mx0 = c0, mx1 = c1;
#pragma unroll
      for (int o = 4; o < 32; o <<= 1) {
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, o));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o));
      }
      const float mn0 = fmaxf(m[0], mx0), mn1 = fmaxf(m[1], mx1);
      const float al0 = mn0 == -INFINITY ? 1.f : fast_exp2(m[0] - mn0);
      const float al1 = mn1 == -INFINITY ? 1.f : fast_exp2(m[1] - mn1);
      m[0] = mn0, m[1] = mn1;
      l[0] *= al0, l[1] *= al1;
#pragma unroll
      for (int i = 0; i < D / 16; ++i) {
        acc[i][0] *= al0, acc[i][1] *= al1, acc[i][2] *= al0, acc[i][3] *= al1;
      }
    }
    const float r0 = m[0] == -INFINITY ? 0.f : m[0], r1 = m[1] == -INFINITY ? 0.f : m[1];
    const float p0 = fast_exp2(x0 - r0), p1 = fast_exp2(x1 - r1);
    const float p2 = fast_exp2(x2 - r0), p3 = fast_exp2(x3 - r1);
    l[0] += p0 + p2;
    l[1] += p1 + p3;
    const uint32_t b0 = movmatrix_trans(pack_bf16x2(p0, p1));
    const uint32_t b1 = movmatrix_trans(pack_bf16x2(p2, p3));
    // O^T[D, 8 heads] += V^T P^T
#pragma unroll
    for (int i = 0; i < D / 16; ++i) {
      uint32_t af[4];
      const int key = (lane & 7) + 8 * (lane >> 4), ch = 2 * i + ((lane >> 3) & 1);
      ldmatrix_x4_trans(af, vs_s + key * kRow + ((ch ^ (key & 7)) << 4));
      mma_bf16_16816(acc[i], af, b0, b1);
    }
    __syncwarp();
    stage = stage + 1 == kBfStages ? 0 : stage + 1;
  }
  cp_async_wait<0>();

  // l is a per-lane partial over this lane's keys: the eight lanes of a head pair add up
#pragma unroll
  for (int o = 4; o < 32; o <<= 1) {
    l[0] += __shfl_xor_sync(0xffffffffu, l[0], o);
    l[1] += __shfl_xor_sync(0xffffffffu, l[1], o);
  }
  // acc[i][j]: dim 16 i + g (j = 0, 1) or 16 i + g + 8 (j = 2, 3), head 2c + (j & 1)
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int hl = 2 * c + j;
    if (hl >= G) continue;
    const int h = h0 + hl;
    if (single) {
      float inv = l[j] > 0.f ? 1.f / l[j] : 0.f;
      if (a.sinks != nullptr) {
        const float s2 = a.sinks[h] * kLog2e;
        const float mf = fmaxf(m[j], s2);
        const float al = m[j] == -INFINITY ? 0.f : fast_exp2(m[j] - mf);
        inv = al / (l[j] * al + fast_exp2(s2 - mf));
      }
      __nv_bfloat16* op = a.out + int64_t(n) * a.o_st + int64_t(h) * a.o_sh + d0;
#pragma unroll
      for (int i = 0; i < D / 16; ++i) {
        op[16 * i + g] = __float2bfloat16(acc[i][j] * inv);
        op[16 * i + g + 8] = __float2bfloat16(acc[i][2 + j] * inv);
      }
    } else {
      const int64_t row = (int64_t(n) * a.hq + h) * a.nseg + seg;
      float* op = a.o_part + row * (D * SPLIT) + d0;
#pragma unroll
      for (int i = 0; i < D / 16; ++i) {
        op[16 * i + g] = acc[i][j];
        op[16 * i + g + 8] = acc[i][2 + j];
      }
      if (g == 0 && half == 0) {
        a.ml_part[2 * row] = m[j];
        a.ml_part[2 * row + 1] = l[j];
      }
    }
  }
}

// Combines the segments of one (sequence, head): w_s = 2^(m_s - m),
// O = sum w_s O_s / sum w_s l_s; empty segments (m = -inf) weigh nothing.
// Follows attn_decode_reduce_kernel (csrc/attn/attn_decode_bf16.hip:276-300). Four
// groups of D / 2 threads take every fourth segment each (a 65,536-key row has 64
// partials: one thread walking them all is 64 dependent round trips to L2) and
// meet in shared memory.
constexpr int kReduceParts = 4;

template <int D>
__global__ void __launch_bounds__(kReduceParts * D / 2) attn_decode_reduce_kernel(
    __nv_bfloat16* __restrict__ out, const float* __restrict__ o_part,
    const float* __restrict__ ml_part, int nseg, int hq, int64_t o_st, int64_t o_sh,
    const float* __restrict__ sinks) {
  pdl_enter();
  __shared__ float s_m[kReduceParts], s_l[kReduceParts];
  __shared__ float2 s_acc[kReduceParts][D / 2];
  const int part = threadIdx.x / (D / 2), dp = threadIdx.x % (D / 2);
  const int64_t row = int64_t(blockIdx.y) * hq + blockIdx.x;
  const float* ml = ml_part + row * nseg * 2;
  float m = -INFINITY;
  for (int s = part; s < nseg; s += kReduceParts) m = fmaxf(m, ml[2 * s]);
  if (dp == 0) s_m[part] = m;
  __syncthreads();
#pragma unroll
  for (int i = 0; i < kReduceParts; ++i) m = fmaxf(m, s_m[i]);
  float l = 0.f;
  float2 acc = make_float2(0.f, 0.f);
#pragma unroll 4
  for (int s = part; s < nseg; s += kReduceParts) {
    const float ms = ml[2 * s];
    if (ms == -INFINITY) continue;
    const float w = exp2f(ms - m);
    l += w * ml[2 * s + 1];
    const float2 o = *reinterpret_cast<const float2*>(o_part + (row * nseg + s) * D + 2 * dp);
    acc.x += w * o.x;
    acc.y += w * o.y;
  }
  s_acc[part][dp] = acc;
  if (dp == 0) s_l[part] = l;
  __syncthreads();
  if (part != 0) return;
#pragma unroll
  for (int i = 1; i < kReduceParts; ++i) {
    acc.x += s_acc[i][dp].x;
    acc.y += s_acc[i][dp].y;
    l += s_l[i];
  }
  if (sinks != nullptr) {
    const float s2 = sinks[blockIdx.x] * kLog2e;
    const float mf = fmaxf(m, s2);
    const float al = m == -INFINITY ? 0.f : exp2f(m - mf);
    acc.x *= al;
    acc.y *= al;
    l = l * al + exp2f(s2 - mf);
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  *reinterpret_cast<uint32_t*>(out + int64_t(blockIdx.y) * o_st + int64_t(blockIdx.x) * o_sh + 2 * dp) =
      pack_bf16x2(acc.x * inv, acc.y * inv);
}

template <int D, bool AL, int W, int MINB, int S>
int launch_decode(dim3 grid, cudaStream_t st, const DecodeArgs& a, size_t smem) {
  auto kernel = attn_decode_q8_kernel<D, AL, W, MINB, S>;
  if (smem > 48 * 1024) {
    // per device, once: opt in to more than 48 KB of dynamic shared memory
    static bool done[64] = {};
    int dev = 0;
    STRIX_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !done[dev]) {
      STRIX_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      int(smem)));
      if (dev >= 0 && dev < 64) done[dev] = true;
    }
  }
  launch_chain(kernel, grid, W * 32, smem, st, a);
  return launch_status("attn_decode");
}

template <int D, int SPLIT>
int launch_decode_bf16kv(dim3 grid, cudaStream_t st, const DecodeArgs& a) {
  auto kernel = attn_decode_bf16kv_kernel<D, SPLIT>;
  // rings, then (SPLIT == 2) the pairs' score exchange: 2 parities x 2 halves x 32 float4
  const size_t smem = size_t(a.hpc) * SPLIT * kBfStages * 2 * 16 * D * 2 +
                      (SPLIT == 2 ? size_t(a.hpc) * 2 * 2 * 32 * 16 : 0);
  if (smem > 48 * 1024) {
    // per device, once: opt in to the largest ring this head size can ask for
    static bool done[64] = {};
    int dev = 0;
    STRIX_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !done[dev]) {
      STRIX_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (D == 256 ? 2 : 4) * kBfStages * 2 * 16 * D * 2 + 4096));
      if (dev >= 0 && dev < 64) done[dev] = true;
    }
  }
  launch_chain(kernel, grid, 32 * a.hpc * SPLIT, smem, st, a);
  return launch_status("attn_decode_bf16kv");
}

}  // namespace
}  // namespace strix

using namespace strix;

// Keys per segment in automatic mode: STRIX_DECODE_AUTO_KEYS, halved for a batch so
// small that 1,024-key segments would not even fill one wave of CTAs (a shard of 8
// long sequences: 3,360 -> 3,780 GB/s; at 16 sequences the longer segments win
// again). STRIX_DECODE_SEG_KEYS (a multiple of 16) fixes the length for tuning runs.
static int auto_seg_keys(int64_t nseq, int64_t max_keys) {
  static const int fixed = [] {
    const char* e = getenv("STRIX_DECODE_SEG_KEYS");
    const int v = e ? atoi(e) : 0;
    return (v >= 64 && v % 16 == 0) ? v : 0;
  }();
  if (fixed) return fixed;
  constexpr int64_t kWaveKeys = int64_t(148) * 4 * STRIX_DECODE_AUTO_KEYS;   // one CTA slot per segment
  return (nseq > 0 && nseq * max_keys < kWaveKeys) ? STRIX_DECODE_AUTO_KEYS / 2 : STRIX_DECODE_AUTO_KEYS;
}

extern "C" int64_t strix_attn_decode_segments_n(int64_t nseq, int64_t num_splits, int64_t max_blocks,
                                                int64_t block_size) {
  if (num_splits < 0 || num_splits > 64) return -1;
  if (num_splits > 0) return num_splits;
  if (max_blocks < 0 || block_size <= 0) return -1;
  const int64_t keys = max_blocks * block_size;
  const int64_t seg = auto_seg_keys(nseq, keys);
  const int64_t n = (keys + seg - 1) / seg;
  return n < 1 ? 1 : n;
}

extern "C" int64_t strix_attn_decode_segments(int64_t num_splits, int64_t max_blocks,
                                              int64_t block_size) {
  return strix_attn_decode_segments_n(0, num_splits, max_blocks, block_size);
}

extern "C" int64_t strix_attn_decode_workspace(int64_t nseq, int64_t hq, int64_t head_dim,
                                               int64_t num_splits, int64_t max_blocks,
                                               int64_t block_size) {
  const int64_t nseg = strix_attn_decode_segments_n(nseq, num_splits, max_blocks, block_size);
  if (nseg < 0) return -1;
  if (nseg == 1) return 0;
  return nseq * hq * nseg * (head_dim + 2) * int64_t(sizeof(float));
}

extern "C" int strix_attn_decode_bf16(
    void* out, const void* q, const void* key_cache, const void* value_cache,
    const float* k_scale, const float* v_scale, const int32_t* seq_lens,
    const int32_t* block_table, const float* sinks, void* workspace, int64_t nseq,
    int64_t hq, int64_t hkv, int64_t head_dim, int64_t block_size, int64_t max_blocks,
    int64_t bt_stride, int64_t q_st, int64_t q_sh, int64_t o_st, int64_t o_sh, int64_t k_sb,
    int64_t k_ss, int64_t k_sh, int64_t v_sb, int64_t v_ss, int64_t v_sh, int64_t ks_sb,
    int64_t ks_ss, int64_t ks_sh, int64_t vs_sb, int64_t vs_ss, int64_t vs_sh, double scale,
    int64_t num_splits, int64_t window_left, int kv_int8, strix_stream_t stream) {
  STRIX_CHECK(nseq >= 0 && hq > 0 && hkv > 0, "q [N, H, D], caches [blocks, block_size, Hkv, D]");
  STRIX_CHECK(hq % hkv == 0, "Hq %% Hkv");
  const int64_t g = hq / hkv;
  if (kv_int8) {
    STRIX_CHECK((head_dim == 128 || head_dim == 256) && g <= 8,
                "attn_decode_bf16 int8: head_dim %lld GQA %lld not built (128, 256: GQA 1-8)",
                (long long)head_dim, (long long)g);
    STRIX_CHECK(k_scale != nullptr && v_scale != nullptr, "int8 KV needs k_scale and v_scale");
    STRIX_CHECK(k_sb % 4 == 0 && k_ss % 4 == 0 && k_sh % 4 == 0 && v_sb % 4 == 0 &&
                    v_ss % 4 == 0 && v_sh % 4 == 0,
                "aligned cache rows");
    STRIX_CHECK((reinterpret_cast<uintptr_t>(key_cache) | reinterpret_cast<uintptr_t>(value_cache)) % 4 == 0,
                "aligned cache rows");
  } else {
    STRIX_CHECK((head_dim == 64 || head_dim == 128 || head_dim == 256 || head_dim == 512) && g <= 8,
                "attn_decode_bf16 bf16 KV: head_dim %lld GQA %lld not built (64, 128, 256, 512: GQA 1-8)",
                (long long)head_dim, (long long)g);
    STRIX_CHECK(k_sb % 8 == 0 && k_ss % 8 == 0 && k_sh % 8 == 0 && v_sb % 8 == 0 &&
                    v_ss % 8 == 0 && v_sh % 8 == 0 &&
                    (reinterpret_cast<uintptr_t>(key_cache) | reinterpret_cast<uintptr_t>(value_cache)) % 16 == 0,
                "bf16 cache rows must be 16-byte aligned");
  }
  STRIX_CHECK(block_size > 0 && block_size % 16 == 0, "block_size must be a multiple of 16");
  STRIX_CHECK(q_st % 4 == 0 && q_sh % 4 == 0 && reinterpret_cast<uintptr_t>(q) % 8 == 0,
              "q must be bf16 with a contiguous head_dim");
  STRIX_CHECK(o_st % 2 == 0 && o_sh % 2 == 0 && reinterpret_cast<uintptr_t>(out) % 4 == 0,
              "out must match q");
  STRIX_CHECK(num_splits >= 0 && num_splits <= 64, "num_splits in [1, 64]");
  STRIX_CHECK(window_left >= -1, "window_left >= -1");
  const int64_t nseg = strix_attn_decode_segments_n(nseq, num_splits, max_blocks, block_size);
  STRIX_CHECK(nseg >= 1 && nseg <= 65535, "segment count out of range");
  STRIX_CHECK(nseg == 1 || nseq == 0 || workspace != nullptr, "split-KV needs a workspace");
  STRIX_CHECK(nseq <= 65535, "at most 65535 sequences per call");
  if (nseq == 0) return STRIX_OK;

  DecodeArgs a;
  a.out = static_cast<__nv_bfloat16*>(out);
  a.q = static_cast<const __nv_bfloat16*>(q);
  a.kc = key_cache;
  a.vc = value_cache;
  a.ksc = k_scale;
  a.vsc = v_scale;
  a.seq_lens = seq_lens;
  a.bt = block_table;
  a.sinks = sinks;
  a.o_part = static_cast<float*>(workspace);
  a.ml_part = a.o_part ? a.o_part + nseq * hq * nseg * head_dim : nullptr;
  a.bt_stride = bt_stride;
  a.q_st = q_st, a.q_sh = q_sh, a.o_st = o_st, a.o_sh = o_sh;
  a.k_sb = k_sb, a.k_ss = k_ss, a.k_sh = k_sh;
  a.v_sb = v_sb, a.v_ss = v_ss, a.v_sh = v_sh;
  a.ks_sb = ks_sb, a.ks_ss = ks_ss, a.ks_sh = ks_sh;
  a.vs_sb = vs_sb, a.vs_ss = vs_ss, a.vs_sh = vs_sh;
  a.block_size = int(block_size);
  {
    const int tpb = int(block_size / 16);
    a.tpb_shift = -1;
    if ((tpb & (tpb - 1)) == 0)
      for (int sh = 0; sh < 31; ++sh)
        if ((1 << sh) == tpb) a.tpb_shift = sh;
  }
  a.hq = int(hq), a.hkv = int(hkv), a.g = int(g);
  a.hpc = hkv % 4 == 0 ? 4 : (hkv % 2 == 0 ? 2 : 1);
  a.nseg = int(nseg);
  a.seg_keys = num_splits == 0 ? auto_seg_keys(nseq, max_blocks * block_size) : 0;
  a.win_left = int(window_left);
  a.scale_log2 = float(scale) * kLog2e;

  if (!kv_int8) {
    // bf16 caches: one warp per KV head of the group, per-warp cp.async ring
    // (head 256: two KV heads per CTA, so that two CTAs of 96 KB share an SM; head 512:
    // one KV head per CTA, its dims split over a pair of warps)
    if (head_dim == 256 && a.hpc > 2) a.hpc = 2;
    if (head_dim == 512) a.hpc = 1;
    const dim3 bgrid{unsigned(nseg), unsigned(hkv / a.hpc), unsigned(nseq)};
    cudaStream_t bst = static_cast<cudaStream_t>(stream);
    int brc = head_dim == 512   ? launch_decode_bf16kv<256, 2>(bgrid, bst, a)
              : head_dim == 256 ? launch_decode_bf16kv<256, 1>(bgrid, bst, a)
              : head_dim == 128 ? launch_decode_bf16kv<128, 1>(bgrid, bst, a)
                                : launch_decode_bf16kv<64, 1>(bgrid, bst, a);
    if (brc != STRIX_OK) return brc;
    if (nseg > 1) {
      const dim3 rgrid{unsigned(hq), unsigned(nseq), 1u};
      if (head_dim == 512)
        launch_chain(attn_decode_reduce_kernel<512>, rgrid, kReduceParts * 256, 0, bst, a.out, a.o_part,
                     a.ml_part, a.nseg, a.hq, o_st, o_sh, sinks);
      else if (head_dim == 256)
        launch_chain(attn_decode_reduce_kernel<256>, rgrid, kReduceParts * 128, 0, bst, a.out, a.o_part,
                     a.ml_part, a.nseg, a.hq, o_st, o_sh, sinks);
      else if (head_dim == 128)
        launch_chain(attn_decode_reduce_kernel<128>, rgrid, kReduceParts * 64, 0, bst, a.out, a.o_part,
                     a.ml_part, a.nseg, a.hq, o_st, o_sh, sinks);
      else
        launch_chain(attn_decode_reduce_kernel<64>, rgrid, kReduceParts * 32, 0, bst, a.out, a.o_part,
                     a.ml_part, a.nseg, a.hq, o_st, o_sh, sinks);
      brc = launch_status("attn_decode_reduce");
    }
    return brc;
  }
  const bool aligned = (k_sb | k_ss | k_sh | v_sb | v_ss | v_sh) % 16 == 0 &&
                       (reinterpret_cast<uintptr_t>(key_cache) |
                        reinterpret_cast<uintptr_t>(value_cache)) % 16 == 0;
  const dim3 grid{unsigned(nseg), unsigned(hkv / a.hpc), unsigned(nseq)};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // Path and shape of the main kernel. Rows that are 16-byte aligned take the
  // shared-memory ring (4 warps, 3 stages, 4 CTAs per SM at head_dim 128);
  // anything else takes the register-buffered loop. STRIX_DECODE_STAGES
  // (0, 3, 4) and STRIX_DECODE_WARPS (4, 8) override the choice for tuning runs.
  static const int stages_env = [] {
    const char* e = getenv("STRIX_DECODE_STAGES");
    return e ? atoi(e) : -1;
  }();
  static const int warps_env = [] {
    const char* e = getenv("STRIX_DECODE_WARPS");
    return e ? atoi(e) : 0;
  }();
  int stages = aligned ? 3 : 0;
  if (aligned && (stages_env == 0 || stages_env == 3 || stages_env == 4)) stages = stages_env;
  const int warps = (warps_env == 4 || warps_env == 8) ? warps_env : 4;
  const size_t merge_bytes = size_t(a.hpc) * 8 * head_dim * sizeof(float);
  int rc = STRIX_OK;
#define STRIX_DECODE_CASE(D, AL, W, MINB, S)                                              \
  rc = launch_decode<D, AL, W, MINB, S>(                                                  \
      grid, st, a, S == 0 ? merge_bytes : size_t(W) * S * stage_bytes(D))
  if (head_dim == 128) {
    if (stages == 0) {
      if (warps == 8) { if (aligned) STRIX_DECODE_CASE(128, true, 8, 2, 0); else STRIX_DECODE_CASE(128, false, 8, 2, 0); }
      else { if (aligned) STRIX_DECODE_CASE(128, true, 4, 3, 0); else STRIX_DECODE_CASE(128, false, 4, 3, 0); }
    } else if (stages == 4) {
      if (warps == 8) STRIX_DECODE_CASE(128, true, 8, 1, 4); else STRIX_DECODE_CASE(128, true, 4, 3, 4);
    } else {
      if (warps == 8) STRIX_DECODE_CASE(128, true, 8, 2, 3); else STRIX_DECODE_CASE(128, true, 4, 4, 3);
    }
  } else {
    if (stages == 0) {
      if (aligned) STRIX_DECODE_CASE(256, true, 4, 2, 0); else STRIX_DECODE_CASE(256, false, 4, 2, 0);
    } else {
      STRIX_DECODE_CASE(256, true, 4, 2, 3);
    }
  }
#undef STRIX_DECODE_CASE
  if (rc != STRIX_OK) return rc;
  if (nseg > 1) {
    const dim3 rgrid{unsigned(hq), unsigned(nseq), 1u};
    if (head_dim == 128)
      launch_chain(attn_decode_reduce_kernel<128>, rgrid, kReduceParts * 64, 0, st, a.out, a.o_part,
                   a.ml_part, a.nseg, a.hq, o_st, o_sh, sinks);
    else
      launch_chain(attn_decode_reduce_kernel<256>, rgrid, kReduceParts * 128, 0, st, a.out, a.o_part,
                   a.ml_part, a.nseg, a.hq, o_st, o_sh, sinks);
    rc = launch_status("attn_decode_reduce");
  }
  return rc;
}

// ---------------------------------------------------------------------------
// Allocation-free variant of strix_attn_decode_bf16.
//
// Some hosts of this library cannot hand it scratch memory: a C or C++ serving
// loop that only owns the input and output buffers its framework gave it, or a
// process whose device memory was budgeted at start-up, where a late cudaMalloc
// may fail or stall the device. For them the split-KV partials live in the
// fixed array below instead of a caller-provided workspace. Every GPU that
// loads the library holds these STRIX_DECODE_STATIC_SCRATCH_BYTES until exit.
//
// g_decode_scratch is a device symbol: in host code its name is only a
// stand-in, never a device address, so the address handed to the kernels is
// obtained with cudaGetSymbolAddress - once per device, with that device
// current, on the first call made on it (make that first call before any
// stream capture begins). No call here allocates or frees memory.
//
// All calls share the array and it keeps the previous call's contents. Nothing
// in it has to start at zero: every (sequence, head, segment) slot's (m, l)
// pair is rewritten by each call, and a partial O row is read only when its m
// is finite, i.e. when this call wrote it. Two calls that overlap on the GPU
// (different streams, or one device used from several threads) race on it.
static __device__ __align__(256) float
    g_decode_scratch[STRIX_DECODE_STATIC_SCRATCH_BYTES / sizeof(float)];

extern "C" int strix_attn_decode_bf16_static(
    void* out, const void* q, const void* key_cache, const void* value_cache,
    const float* k_scale, const float* v_scale, const int32_t* seq_lens,
    const int32_t* block_table, const float* sinks, int64_t nseq, int64_t hq, int64_t hkv,
    int64_t head_dim, int64_t block_size, int64_t max_blocks, int64_t bt_stride, int64_t q_st,
    int64_t q_sh, int64_t o_st, int64_t o_sh, int64_t k_sb, int64_t k_ss, int64_t k_sh,
    int64_t v_sb, int64_t v_ss, int64_t v_sh, int64_t ks_sb, int64_t ks_ss, int64_t ks_sh,
    int64_t vs_sb, int64_t vs_ss, int64_t vs_sh, double scale, int64_t num_splits,
    int64_t window_left, int kv_int8, strix_stream_t stream) {
  STRIX_CHECK(nseq >= 0 && hq > 0 && head_dim > 0, "q [N, H, D], caches [blocks, block_size, Hkv, D]");
  const int64_t bytes =
      strix_attn_decode_workspace(nseq, hq, head_dim, num_splits, max_blocks, block_size);
  STRIX_CHECK(bytes >= 0, "num_splits in [1, 64]");
  STRIX_CHECK(bytes <= int64_t(STRIX_DECODE_STATIC_SCRATCH_BYTES),
              "attn_decode_bf16_static: this launch needs %lld bytes of split-KV scratch but the "
              "built-in array holds %lld; lower num_splits or the batch, or use "
              "strix_attn_decode_bf16 with a caller workspace",
              (long long)bytes, (long long)STRIX_DECODE_STATIC_SCRATCH_BYTES);
  float* scratch = nullptr;
  if (bytes > 0) {
    static float* device_address[64] = {};
    int dev = 0;
    STRIX_CUDA(cudaGetDevice(&dev));
    STRIX_CHECK(dev >= 0 && dev < 64, "device index %d out of range", dev);
    if (device_address[dev] == nullptr) {
      void* p = nullptr;
      STRIX_CUDA(cudaGetSymbolAddress(&p, g_decode_scratch));
      device_address[dev] = static_cast<float*>(p);
    }
    scratch = device_address[dev];
  }
  return strix_attn_decode_bf16(out, q, key_cache, value_cache, k_scale, v_scale, seq_lens,
                                block_table, sinks, scratch, nseq, hq, hkv, head_dim, block_size,
                                max_blocks, bt_stride, q_st, q_sh, o_st, o_sh, k_sb, k_ss, k_sh,
                                v_sb, v_ss, v_sh, ks_sb, ks_ss, ks_sh, vs_sb, vs_ss, vs_sh, scale,
                                num_splits, window_left, kv_int8, stream);
}
