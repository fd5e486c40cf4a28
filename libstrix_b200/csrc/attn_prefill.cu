// Causal paged attention for prefill (varlen, GQA, int8 or bf16 KV cache,
// sliding window, attention sinks), for sm_100a. Replaces attn_prefill_bf16
// (csrc/attn/attn_prefill_bf16.hip:508-662 of the reference; semantics pinned
// by tests/test_attn_prefill.py:31-59): the queries of sequence n are the last
// q_len of its seq_lens[n] positions, query at position p sees keys <= p (and
// >= p - window_left), the K scale multiplies the score, the V scale the
// softmax weight, a sink is one extra unscaled natural-log logit per head that
// joins only the denominator.
//
// Shape of the kernel: a CTA = 64 queries of one sequence x one query head, 4
// warps of 16 queries. Key tiles of 64 (32 above head 128): the raw cache rows of the NEXT tile are
// in flight (cp.async, double buffer) while the current one is used. int8
// caches are widened once per tile to fp16 in shared memory with byte permutes
// (exact, the scales stay out: K scale on the score, V scale on P), and the two
// contractions run as fp16 mma.sync m16n8k16 (the bf16 queries convert to fp16
// exactly); bf16 caches are copied straight into the operand tiles and use
// bf16 MMAs. Operand tiles are read with ldmatrix (V transposed) through a
// 16-byte-chunk XOR swizzle. Softmax is online, in the exp2 domain, fp32.
//
// Head 256 keeps the query tile in shared memory too (its fragments are re-read per
// key tile) and runs two CTAs of 97 KB per SM. Head 512 (SPLIT = 2) gives each group of 16 queries to a PAIR of warps,
// each owning 256 of the head's dims - that part of Q, of every K row (score
// partials, added through shared memory behind a 64-thread named barrier) and of
// every V row and O - over key tiles of 32.
#include "common.cuh"

namespace strix {
namespace {

constexpr int kBM = 64;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLift = 64.f;   // P x v_scale is lifted into fp16's normal range

struct PrefillArgs {
  __nv_bfloat16* out;
  const __nv_bfloat16* q;
  const uint8_t* kc;
  const uint8_t* vc;
  const float* ks;
  const float* vs;
  const int32_t* cu;        // [nseq + 1] query offsets
  const int32_t* seq_lens;  // [nseq]
  const int32_t* block_table;
  const float* sinks;       // optional [hq]
  int64_t q_st, q_sh, o_st, o_sh;             // elements
  int64_t k_sb, k_ss, k_sh, v_sb, v_ss, v_sh; // bytes
  int64_t ks_sb, ks_ss, ks_sh, vs_sb, vs_ss, vs_sh;  // elements
  int64_t bt_stride;
  int nseq, hq, hkv, block_size, window_left;
  int aligned16;            // cache rows start on 16-byte boundaries
  int same_pos;             // decode form: every query row of a sequence sits at its last position
  float scale;
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

// byte offset of 16-byte chunk `chunk` of key row `key` in a [rows][D] 16-bit tile
template <int D>
__device__ __forceinline__ uint32_t tile_off(int key, int chunk) {
  return uint32_t(key * (D * 2) + ((chunk ^ (key & 7)) << 4));
}

template <int D, bool Q8>
struct PfLayout {
  static constexpr int kSplit = D > 256 ? 2 : 1;                 // warps sharing 16 queries
  static constexpr int kDW = D / kSplit;                         // head dims per warp
  static constexpr int kThreads = 128 * kSplit;
  static constexpr int kBN = D > 128 ? 32 : 64;                  // keys per tile
  static constexpr int kTile = kBN * D * 2;                      // one 16-bit operand tile
  static constexpr int kRawKV = Q8 ? kBN * D : 0;                // raw int8 rows of K (or V)
  static constexpr int kRaw = Q8 ? 2 * kRawKV + 2 * kBN * 4 : 0; // K, V, k scales, v scales
  // Q8: two raw buffers + one pair of operand tiles; bf16: two pairs of operand tiles
  static constexpr int kKV = Q8 ? 2 * kRaw + 2 * kTile : 4 * kTile;
  // Head sizes above 128 keep the 64 x D query tile in shared memory as well (its
  // fragments are re-read per key tile): 64 + 128 accumulator registers leave no room
  // for D / 4 more of Q.
  static constexpr bool kQInSmem = D > 128;
  static constexpr int kQ = kQInSmem ? kBM * D * 2 : 0;
  // score partials of the warp pairs: [parity][4 query groups][2][kBN / 8][32 lanes] float4
  static constexpr int kXch = kSplit == 2 ? 2 * 4 * 2 * (kBN / 8) * 32 * 16 : 0;
  static constexpr int kSmem = kKV + kQ + kXch;
};

template <int D, bool Q8>
__global__ void __launch_bounds__(PfLayout<D, Q8>::kThreads, D <= 128 ? 3 : D == 256 ? 2 : 1)
attn_prefill_kernel(const PrefillArgs p) {
  using L = PfLayout<D, Q8>;
  constexpr bool QS = L::kQInSmem;
  constexpr int SPLIT = L::kSplit, DW = L::kDW, kBN = L::kBN;
  extern __shared__ __align__(128) uint8_t smem[];
  const int tid = threadIdx.x, lane = tid & 31;
  const int warp = (tid >> 5) / SPLIT;          // group of 16 queries
  const int half = (tid >> 5) % SPLIT;          // which DW dims of the head
  constexpr int kC0 = DW / 8;                   // 16-byte chunks of a 16-bit row per warp
  const int g = lane >> 2, c = lane & 3;
  const int head = blockIdx.y, kvh = head / (p.hq / p.hkv);

  // ---- which sequence and which 64-query tile of it
  int n = 0, tile = blockIdx.x, q_begin = 0, q_len = 0;
  for (;; ++n) {
    if (n >= p.nseq) return;
    q_begin = p.cu[n];
    q_len = p.cu[n + 1] - q_begin;
    const int tiles = (q_len + kBM - 1) / kBM;
    if (tile < tiles) {
      tile = tiles - 1 - tile;   // the last tiles see the most keys: start them first
      break;
    }
    tile -= tiles;
  }
  const int kv_len = p.seq_lens[n];
  const int row0 = tile * kBM + warp * 16;             // this warp's first query (local index)
  const int pos0 = kv_len - q_len;                     // position of local query 0
  // keys this CTA needs: up to its last query's position, from the window of its first
  // (decode form: the rows of a sequence are the query heads of one KV head, all at the
  // last position - no causal order among them)
  const bool grp = p.same_pos != 0;
  const int cta_last = min(tile * kBM + kBM, q_len) - 1;
  const int k_end = grp ? kv_len : pos0 + cta_last + 1;
  const int cta_first_pos = grp ? kv_len - 1 : pos0 + tile * kBM;
  const int k_begin = p.window_left >= 0 ? max(0, cta_first_pos - p.window_left) / kBN * kBN : 0;
  const int n_tiles = (k_end - k_begin + kBN - 1) / kBN;

  // ---- Q fragments (A operand, m16k16 per 16 dims), rows g and g + 8 of the warp
  // (QS: the same words go to this warp's 16 rows of the shared query tile instead)
  uint32_t qf[QS ? 1 : DW / 16][4];
  const uint32_t q_tile = static_cast<uint32_t>(__cvta_generic_to_shared(smem)) + L::kKV;
  {
    const int r_lo = row0 + g, r_hi = row0 + g + 8;
    const __nv_bfloat16* q_lo = p.q + int64_t(q_begin + min(r_lo, q_len - 1)) * p.q_st + head * p.q_sh + half * DW;
    const __nv_bfloat16* q_hi = p.q + int64_t(q_begin + min(r_hi, q_len - 1)) * p.q_st + head * p.q_sh + half * DW;
#pragma unroll
    for (int s = 0; s < DW / 16; ++s) {
      uint32_t w[4];
      w[0] = *reinterpret_cast<const uint32_t*>(q_lo + 16 * s + 2 * c);
      w[1] = *reinterpret_cast<const uint32_t*>(q_hi + 16 * s + 2 * c);
      w[2] = *reinterpret_cast<const uint32_t*>(q_lo + 16 * s + 8 + 2 * c);
      w[3] = *reinterpret_cast<const uint32_t*>(q_hi + 16 * s + 8 + 2 * c);
#pragma unroll
      for (int i = 0; i < 4; ++i) w[i] = Q8 ? pack_f16x2(bf16_lo(w[i]), bf16_hi(w[i])) : w[i];
      if constexpr (QS) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          *reinterpret_cast<uint32_t*>(smem + L::kKV +
                                       tile_off<D>(warp * 16 + g + 8 * (i & 1), half * kC0 + 2 * s + (i >> 1)) +
                                       4 * c) = w[i];
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) qf[s][i] = w[i];
      }
    }
    if constexpr (QS) __syncwarp();
  }
  const int qpos_lo = grp ? kv_len - 1 : pos0 + row0 + g;       // positions of the two rows
  const int qpos_hi = grp ? kv_len - 1 : qpos_lo + 8;
  const int wpos_first = grp ? kv_len - 1 : pos0 + row0;        // of the warp's first and last row
  const int wpos_last = grp ? kv_len - 1 : pos0 + row0 + 15;

  const uint32_t smem_s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  // Q8: [raw 0][raw 1][K16][V16]; bf16: [K16 0][V16 0][K16 1][V16 1]
  auto raw_base = [&](int buf) { return uint32_t(buf * L::kRaw); };
  auto k16_base = [&](int buf) { return Q8 ? uint32_t(2 * L::kRaw) : uint32_t(buf * 2 * L::kTile); };
  auto v16_base = [&](int buf) { return k16_base(buf) + L::kTile; };

  // ---- producer: key row tid / kTPR, part tid % kTPR of the row
  constexpr int kRowBytes = Q8 ? D : 2 * D;      // cache bytes per key row and head
  constexpr int kTPR = L::kThreads / kBN;        // threads per key row
  constexpr int kHalf = kRowBytes / kTPR;        // bytes this thread copies per matrix
  const int prow = tid / kTPR, ppart = tid % kTPR;
  auto issue_tile = [&](int t, int buf) {
    const int key = k_begin + t * kBN + prow;
    const bool ok = key < k_end;
    const int kk = ok ? key : k_end - 1;
    const int blk = p.block_table[int64_t(n) * p.bt_stride + kk / p.block_size];
    const int slot = kk % p.block_size;
    const uint8_t* ksrc = p.kc + int64_t(blk) * p.k_sb + int64_t(slot) * p.k_ss + int64_t(kvh) * p.k_sh + ppart * kHalf;
    const uint8_t* vsrc = p.vc + int64_t(blk) * p.v_sb + int64_t(slot) * p.v_ss + int64_t(kvh) * p.v_sh + ppart * kHalf;
    const int row = prow;
    if constexpr (Q8) {
      const uint32_t kd = smem_s + raw_base(buf) + row * D + ppart * kHalf;
      const uint32_t vd = kd + L::kRawKV;
      if (p.aligned16) {
#pragma unroll
        for (int i = 0; i < kHalf / 16; ++i) {
          cp_async_16_zfill(kd + 16 * i, ksrc + 16 * i, ok);
          cp_async_16_zfill(vd + 16 * i, vsrc + 16 * i, ok);
        }
      } else {
#pragma unroll
        for (int i = 0; i < kHalf / 4; ++i) {
          cp_async_4_zfill(kd + 4 * i, ksrc + 4 * i, ok);
          cp_async_4_zfill(vd + 4 * i, vsrc + 4 * i, ok);
        }
      }
      if (ppart == 0) {
        const uint32_t sd = smem_s + raw_base(buf) + 2 * L::kRawKV + row * 4;
        cp_async_4_zfill(sd, p.ks + int64_t(blk) * p.ks_sb + int64_t(slot) * p.ks_ss + int64_t(kvh) * p.ks_sh, ok);
        cp_async_4_zfill(sd + kBN * 4, p.vs + int64_t(blk) * p.vs_sb + int64_t(slot) * p.vs_ss + int64_t(kvh) * p.vs_sh, ok);
      }
    } else {
      // bf16: straight into the swizzled operand tiles (chunks of 8 elements)
#pragma unroll
      for (int i = 0; i < kHalf / 16; ++i) {
        const int chunk = ppart * (kHalf / 16) + i;
        cp_async_16_zfill(smem_s + k16_base(buf) + tile_off<D>(row, chunk), ksrc + 16 * i, ok);
        cp_async_16_zfill(smem_s + v16_base(buf) + tile_off<D>(row, chunk), vsrc + 16 * i, ok);
      }
    }
    cp_async_commit();
  };

  float o[DW / 8][4];
#pragma unroll
  for (int i = 0; i < DW / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
  const float sl2 = p.scale * kLog2e;

  if (n_tiles > 0) issue_tile(0, 0);
  for (int t = 0; t < n_tiles; ++t) {
    const int buf = t & 1;
    cp_async_wait<0>();
    __syncthreads();                       // tile t landed; everyone is done with tile t - 1
    if (t + 1 < n_tiles) issue_tile(t + 1, buf ^ 1);
    if constexpr (Q8) {
      // widen this thread's half rows: 0x6400 | (b ^ 0x80) is fp16 1024 + b + 128
      const int row = prow;
      const uint8_t* rk = smem + raw_base(buf) + row * D + ppart * kHalf;
#pragma unroll
      for (int m = 0; m < 2; ++m) {
        const uint8_t* src = rk + m * L::kRawKV;
        uint8_t* dst = smem + (m == 0 ? k16_base(0) : v16_base(0));
#pragma unroll
        for (int i = 0; i < kHalf / 16; ++i) {
          const uint4 x = *reinterpret_cast<const uint4*>(src + 16 * i);
          const uint32_t ws[4] = {x.x ^ 0x80808080u, x.y ^ 0x80808080u, x.z ^ 0x80808080u, x.w ^ 0x80808080u};
          uint32_t h[8];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            h[2 * j] = sub_f16x2(prmt(ws[j], 0x64646464u, 0x4140), 0x64806480u);
            h[2 * j + 1] = sub_f16x2(prmt(ws[j], 0x64646464u, 0x4342), 0x64806480u);
          }
          const int chunk = (ppart * (kHalf / 16) + i) * 2;   // 16 bytes -> two 8-element chunks
          *reinterpret_cast<uint4*>(dst + tile_off<D>(row, chunk)) = make_uint4(h[0], h[1], h[2], h[3]);
          *reinterpret_cast<uint4*>(dst + tile_off<D>(row, chunk + 1)) = make_uint4(h[4], h[5], h[6], h[7]);
        }
      }
      // the tile's scales, once: K scale x softmax scale x log2(e), V scale x lift
      if (tid < 2 * kBN) {
        float* sc = reinterpret_cast<float*>(smem + raw_base(buf) + 2 * L::kRawKV) + tid;
        *sc *= tid < kBN ? sl2 : kLift;
      }
      __syncthreads();
    }
    const uint32_t kt = smem_s + k16_base(buf), vt = smem_s + v16_base(buf);
    const int k0 = k_begin + t * kBN;

    // ---- S = Q K^T: kBN / 8 key tiles of 8 x DW / 16 steps
    // (d steps outermost: consecutive MMAs then feed eight independent accumulators)
    float s[kBN / 8][4];
#pragma unroll
    for (int j = 0; j < kBN / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
    for (int sp = 0; sp < DW / 32; ++sp) {
      uint32_t b[kBN / 8][4];
#pragma unroll
      for (int j = 0; j < kBN / 8; ++j)
        ldmatrix_x4(b[j], kt + tile_off<D>(8 * j + (lane & 7), half * kC0 + 4 * sp + (lane >> 3)));
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        if constexpr (QS)
          ldmatrix_x4(qf[0], q_tile + tile_off<D>(warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1),
                                                  half * kC0 + 2 * (2 * sp + h) + (lane >> 4)));
        const uint32_t (&qa)[4] = qf[QS ? 0 : 2 * sp + h];
#pragma unroll
        for (int j = 0; j < kBN / 8; ++j) {
          if constexpr (Q8) mma_f16_16816(s[j], qa, b[j][2 * h], b[j][2 * h + 1]);
          else mma_bf16_16816(s[j], qa, b[j][2 * h], b[j][2 * h + 1]);
        }
      }
    }

    if constexpr (SPLIT == 2) {
      // the pair adds its score partials: both warps then hold the same scores
      float4* const mine = reinterpret_cast<float4*>(smem + L::kKV + L::kQ) +
                           ((((t & 1) * 4 + warp) * 2 + half) * (kBN / 8)) * 32 + lane;
#pragma unroll
      for (int j = 0; j < kBN / 8; ++j) mine[j * 32] = make_float4(s[j][0], s[j][1], s[j][2], s[j][3]);
      asm volatile("bar.sync %0, 64;" ::"r"(warp + 1) : "memory");
      const float4* const other = half == 0 ? mine + (kBN / 8) * 32 : mine - (kBN / 8) * 32;
#pragma unroll
      for (int j = 0; j < kBN / 8; ++j) {
        const float4 x = other[j * 32];
        s[j][0] += x.x, s[j][1] += x.y, s[j][2] += x.z, s[j][3] += x.w;
      }
    }

    // ---- scale, mask, online softmax (rows g and g + 8; keys 8j + 2c, + 1)
    const float* sks = reinterpret_cast<const float*>(smem + raw_base(buf) + 2 * L::kRawKV);
    const float* svs = sks + kBN;
    float mx_lo = m_lo, mx_hi = m_hi;
    // a tile strictly inside every row's visible range needs no mask (most tiles do not):
    // all its keys at or before the warp's first query, and inside the window of its last
    const bool interior = k0 + kBN - 1 <= wpos_first &&
                          (p.window_left < 0 || wpos_last - k0 <= p.window_left);
    if (interior) {
#pragma unroll
      for (int j = 0; j < kBN / 8; ++j) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float f = Q8 ? sks[8 * j + 2 * c + e] : sl2;
          s[j][e] *= f;
          s[j][2 + e] *= f;
          mx_lo = fmaxf(mx_lo, s[j][e]);
          mx_hi = fmaxf(mx_hi, s[j][2 + e]);
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < kBN / 8; ++j) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int key = k0 + 8 * j + 2 * c + e;
          const float f = Q8 ? sks[8 * j + 2 * c + e] : sl2;
          const bool in = key < k_end;
          const bool v_lo = in && key <= qpos_lo && (p.window_left < 0 || qpos_lo - key <= p.window_left);
          const bool v_hi = in && key <= qpos_hi && (p.window_left < 0 || qpos_hi - key <= p.window_left);
          s[j][e] = v_lo ? s[j][e] * f : -INFINITY;
          s[j][2 + e] = v_hi ? s[j][2 + e] * f : -INFINITY;
          mx_lo = fmaxf(mx_lo, s[j][e]);
          mx_hi = fmaxf(mx_hi, s[j][2 + e]);
        }
      }
    }
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
    // a row that has seen no key yet keeps m = -inf; its exponent base is 0 then
    const float b_lo = mx_lo == -INFINITY ? 0.f : mx_lo, b_hi = mx_hi == -INFINITY ? 0.f : mx_hi;
    const float r_lo = fast_exp2(m_lo - b_lo), r_hi = fast_exp2(m_hi - b_hi);
    // the accumulators are rescaled only when some row's maximum moved (a warp-wide
    // decision: after the first tiles it rarely does)
    const bool moved = __any_sync(0xffffffffu, mx_lo != m_lo || mx_hi != m_hi);
    m_lo = mx_lo, m_hi = mx_hi;
    if (moved) {
      l_lo *= r_lo, l_hi *= r_hi;
#pragma unroll
      for (int i = 0; i < DW / 8; ++i) o[i][0] *= r_lo, o[i][1] *= r_lo, o[i][2] *= r_hi, o[i][3] *= r_hi;
    }

    uint32_t pf[kBN / 16][4];   // P as the A operand of P V
#pragma unroll
    for (int j = 0; j < kBN / 8; ++j) {
      float pv[4];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float p_lo = fast_exp2(s[j][e] - b_lo), p_hi = fast_exp2(s[j][2 + e] - b_hi);
        l_lo += p_lo, l_hi += p_hi;
        const float w = Q8 ? svs[8 * j + 2 * c + e] : 1.f;
        pv[e] = p_lo * w, pv[2 + e] = p_hi * w;
      }
      const int tt = j >> 1, h = (j & 1) * 2;
      pf[tt][h] = Q8 ? pack_f16x2(pv[0], pv[1]) : pack_bf16x2(pv[0], pv[1]);
      pf[tt][h + 1] = Q8 ? pack_f16x2(pv[2], pv[3]) : pack_bf16x2(pv[2], pv[3]);
    }

    // ---- O += P V: DW / 8 output tiles x kBN / 16 key steps of 16
#pragma unroll
    for (int tt = 0; tt < kBN / 16; ++tt) {
#pragma unroll
      for (int i2 = 0; i2 < DW / 16; ++i2) {
        uint32_t b[4];
        ldmatrix_x4_trans(b, vt + tile_off<D>(16 * tt + (lane & 7) + 8 * ((lane >> 3) & 1),
                                              half * kC0 + 2 * i2 + (lane >> 4)));
        if constexpr (Q8) {
          mma_f16_16816(o[2 * i2], pf[tt], b[0], b[1]);
          mma_f16_16816(o[2 * i2 + 1], pf[tt], b[2], b[3]);
        } else {
          mma_bf16_16816(o[2 * i2], pf[tt], b[0], b[1]);
          mma_bf16_16816(o[2 * i2 + 1], pf[tt], b[2], b[3]);
        }
      }
    }
  }
  cp_async_wait<0>();

  // ---- finish: row sums across the 4 lanes of a row, sinks, normalise, store
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
  const int r_lo = row0 + g, r_hi = row0 + g + 8;
  if (p.sinks != nullptr) {
    // decode form: row r of the sequence is query head head * q_len + r
    const float sk_lo = p.sinks[grp ? head * q_len + min(r_lo, q_len - 1) : head] * kLog2e;
    const float sk_hi = p.sinks[grp ? head * q_len + min(r_hi, q_len - 1) : head] * kLog2e;
    if (m_lo == -INFINITY) l_lo = 1.f; else l_lo += fast_exp2(sk_lo - m_lo);
    if (m_hi == -INFINITY) l_hi = 1.f; else l_hi += fast_exp2(sk_hi - m_hi);
  }
  const float unlift = Q8 ? 1.f / kLift : 1.f;
  const float inv_lo = l_lo > 0.f ? unlift / l_lo : 0.f, inv_hi = l_hi > 0.f ? unlift / l_hi : 0.f;
#pragma unroll
  for (int i = 0; i < DW / 8; ++i) {
    if (r_lo < q_len)
      *reinterpret_cast<uint32_t*>(p.out + int64_t(q_begin + r_lo) * p.o_st + head * p.o_sh + half * DW + 8 * i + 2 * c) =
          pack_bf16x2(o[i][0] * inv_lo, o[i][1] * inv_lo);
    if (r_hi < q_len)
      *reinterpret_cast<uint32_t*>(p.out + int64_t(q_begin + r_hi) * p.o_st + head * p.o_sh + half * DW + 8 * i + 2 * c) =
          pack_bf16x2(o[i][2] * inv_hi, o[i][3] * inv_hi);
  }
}

template <int D, bool Q8>
int launch_prefill(const PrefillArgs& p, int64_t max_tiles, cudaStream_t st) {
  using L = PfLayout<D, Q8>;
  auto kernel = attn_prefill_kernel<D, Q8>;
  static bool done[64] = {};
  int dev = 0;
  STRIX_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !done[dev]) {
    STRIX_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kSmem));
    if (dev >= 0 && dev < 64) done[dev] = true;
  }
  const dim3 grid{unsigned(max_tiles), unsigned(p.hq), 1u};
  kernel<<<grid, L::kThreads, L::kSmem, st>>>(p);
  return launch_status("attn_prefill");
}

}  // namespace
}  // namespace strix

using namespace strix;

static int prefill_impl(
    int same_pos,
    void* out, const void* q, const void* key_cache, const void* value_cache, const float* k_scale,
    const float* v_scale, const int32_t* cu_seqlens_q, const int32_t* seq_lens,
    const int32_t* block_table, const float* sinks, int64_t total_q, int64_t nseq, int64_t hq,
    int64_t hkv, int64_t head_dim, int64_t block_size, int64_t bt_stride, int64_t q_stride_t,
    int64_t q_stride_h, int64_t out_stride_t, int64_t out_stride_h, int64_t k_stride_b,
    int64_t k_stride_s, int64_t k_stride_h, int64_t v_stride_b, int64_t v_stride_s,
    int64_t v_stride_h, int64_t ks_stride_b, int64_t ks_stride_s, int64_t ks_stride_h,
    int64_t vs_stride_b, int64_t vs_stride_s, int64_t vs_stride_h, double scale,
    int64_t num_splits, int64_t window_left, int kv_int8, strix_stream_t stream) {
  STRIX_CHECK(head_dim == 64 || head_dim == 128 || head_dim == 256 || head_dim == 512,
              "head_dim 64, 128, 256 or 512 (others are not built)");
  STRIX_CHECK(hq > 0 && hkv > 0 && hq % hkv == 0 && hq <= 65535, "hq must be a multiple of hkv");
  STRIX_CHECK(block_size >= 1 && nseq >= 0 && total_q >= 0, "bad sizes");
  STRIX_CHECK(num_splits >= 1 && num_splits <= 64, "num_splits in [1, 64]");
  STRIX_CHECK(sinks == nullptr || num_splits == 1, "sinks need num_splits == 1");
  STRIX_CHECK(!kv_int8 || (k_scale != nullptr && v_scale != nullptr), "int8 KV needs k_scale and v_scale");
  const int eb = kv_int8 ? 1 : 2;
  STRIX_CHECK(q_stride_t % 2 == 0 && q_stride_h % 2 == 0 && out_stride_t % 2 == 0 && out_stride_h % 2 == 0 &&
                  reinterpret_cast<uintptr_t>(q) % 4 == 0 && reinterpret_cast<uintptr_t>(out) % 4 == 0,
              "q / out rows must be 4-byte aligned");
  const int64_t ks[6] = {k_stride_b * eb, k_stride_s * eb, k_stride_h * eb, v_stride_b * eb, v_stride_s * eb, v_stride_h * eb};
  bool a4 = reinterpret_cast<uintptr_t>(key_cache) % 4 == 0 && reinterpret_cast<uintptr_t>(value_cache) % 4 == 0;
  bool a16 = reinterpret_cast<uintptr_t>(key_cache) % 16 == 0 && reinterpret_cast<uintptr_t>(value_cache) % 16 == 0;
  for (int i = 0; i < 6; ++i) a4 = a4 && ks[i] % 4 == 0, a16 = a16 && ks[i] % 16 == 0;
  STRIX_CHECK(kv_int8 ? a4 : a16, "cache rows must be 4-byte (int8) / 16-byte (bf16) aligned");
  if (nseq == 0 || total_q == 0) return STRIX_OK;
  PrefillArgs p;
  p.out = static_cast<__nv_bfloat16*>(out), p.q = static_cast<const __nv_bfloat16*>(q);
  p.kc = static_cast<const uint8_t*>(key_cache), p.vc = static_cast<const uint8_t*>(value_cache);
  p.ks = k_scale, p.vs = v_scale, p.cu = cu_seqlens_q, p.seq_lens = seq_lens;
  p.block_table = block_table, p.sinks = sinks;
  p.q_st = q_stride_t, p.q_sh = q_stride_h, p.o_st = out_stride_t, p.o_sh = out_stride_h;
  p.k_sb = ks[0], p.k_ss = ks[1], p.k_sh = ks[2], p.v_sb = ks[3], p.v_ss = ks[4], p.v_sh = ks[5];
  p.ks_sb = ks_stride_b, p.ks_ss = ks_stride_s, p.ks_sh = ks_stride_h;
  p.vs_sb = vs_stride_b, p.vs_ss = vs_stride_s, p.vs_sh = vs_stride_h;
  p.bt_stride = bt_stride;
  p.nseq = int(nseq), p.hq = int(hq), p.hkv = int(hkv), p.block_size = int(block_size);
  p.window_left = int(window_left), p.aligned16 = a16 ? 1 : 0, p.scale = float(scale);
  p.same_pos = same_pos;
  // an upper bound on the 64-query tiles without reading the lengths on the host
  const int64_t max_tiles = (total_q + kBM - 1) / kBM + nseq;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (head_dim == 512) return kv_int8 ? launch_prefill<512, true>(p, max_tiles, st) : launch_prefill<512, false>(p, max_tiles, st);
  if (head_dim == 256) return kv_int8 ? launch_prefill<256, true>(p, max_tiles, st) : launch_prefill<256, false>(p, max_tiles, st);
  if (head_dim == 128) return kv_int8 ? launch_prefill<128, true>(p, max_tiles, st) : launch_prefill<128, false>(p, max_tiles, st);
  return kv_int8 ? launch_prefill<64, true>(p, max_tiles, st) : launch_prefill<64, false>(p, max_tiles, st);
}

#define STRIX_PREFILL_PARAMS                                                                       \
  void *out, const void *q, const void *key_cache, const void *value_cache, const float *k_scale, \
      const float *v_scale, const int32_t *cu_seqlens_q, const int32_t *seq_lens,                 \
      const int32_t *block_table, const float *sinks, int64_t total_q, int64_t nseq, int64_t hq,  \
      int64_t hkv, int64_t head_dim, int64_t block_size, int64_t bt_stride, int64_t q_stride_t,   \
      int64_t q_stride_h, int64_t out_stride_t, int64_t out_stride_h, int64_t k_stride_b,         \
      int64_t k_stride_s, int64_t k_stride_h, int64_t v_stride_b, int64_t v_stride_s,             \
      int64_t v_stride_h, int64_t ks_stride_b, int64_t ks_stride_s, int64_t ks_stride_h,          \
      int64_t vs_stride_b, int64_t vs_stride_s, int64_t vs_stride_h, double scale,                \
      int64_t num_splits, int64_t window_left, int kv_int8, strix_stream_t stream
#define STRIX_PREFILL_ARGS                                                                          \
  out, q, key_cache, value_cache, k_scale, v_scale, cu_seqlens_q, seq_lens, block_table, sinks,    \
      total_q, nseq, hq, hkv, head_dim, block_size, bt_stride, q_stride_t, q_stride_h,             \
      out_stride_t, out_stride_h, k_stride_b, k_stride_s, k_stride_h, v_stride_b, v_stride_s,      \
      v_stride_h, ks_stride_b, ks_stride_s, ks_stride_h, vs_stride_b, vs_stride_s, vs_stride_h,    \
      scale, num_splits, window_left, kv_int8, stream

extern "C" int strix_attn_prefill_bf16(STRIX_PREFILL_PARAMS) {
  return prefill_impl(0, STRIX_PREFILL_ARGS);
}

// Decode through the same kernel, for geometries without a split-KV decode kernel: the
// rows cu_seqlens_q[n] .. of sequence n are the hq / hkv query heads of one KV head (q
// and out regrouped to [nseq * G, hkv, head_dim]), all at position seq_lens[n] - 1, so a
// KV head is read once for its whole group; sinks stay [hkv * G] in query-head order.
extern "C" int strix_attn_decode_grouped_bf16(STRIX_PREFILL_PARAMS) {
  return prefill_impl(1, STRIX_PREFILL_ARGS);
}
