// Causal paged attention for prefill on the Blackwell tensor cores (tcgen05.mma
// kind::f16, S and O accumulators in tensor memory, operands fed by TMA), for
// sm_100a. Same contract as attn_prefill.cu (attn_prefill_bf16 of the reference,
// csrc/attn/attn_prefill_bf16.hip:508-662; semantics pinned by
// tests/test_attn_prefill.py:31-59): varlen, GQA, int8 or bf16 KV cache, sliding
// window, sinks. Two kernels:
//
// 1. prefill_gather_kernel: one pass over the pages of every sequence that
//    writes the keys and values the batch needs as contiguous 16-bit matrices in
//    a workspace - K' [Hkv][rows][D] (row = key) and V'^T [Hkv][D][rows] (row =
//    head dimension, keys contiguous), each sequence's keys starting on a
//    128-row boundary. int8 caches are dequantised here (fp16(byte x scale): the K
//    scale rides in K', the V scale in V'), bf16 caches are copied. All paging,
//    stride and scale-layout variants end here; it moves 3 bytes per cache byte
//    once, against T / 2 reads of every key by the attention proper.
//
// 2. attn_prefill_umma_kernel: a CTA owns 256 consecutive queries of one sequence
//    and one query head as two tiles of 128 (TMEM lanes = queries), and walks the
//    key tiles of 128 its queries can see:
//      producer (1 thread)  TMA: the two Q tiles once, then K' and V'^T tiles into a
//                           2-stage ring (128-byte-swizzled K-major operand tiles);
//      issuer (1 thread)    S_q = Q_q K'^T (8 MMAs of 128 x 128 x 16 from shared
//                           memory) and O_q += P_q V' (8 MMAs whose A operand, P,
//                           is read from TENSOR MEMORY where the softmax warps
//                           stored it over S), interleaved between the two tiles
//                           so the tensor pipe works on one tile while the softmax
//                           of the other runs;
//      softmax (2 x 8 warps) TWO threads per query row, 64 of a key tile's 128
//                           columns each (the two warps that share a TMEM lane
//                           quadrant): tcgen05.ld of the scores, online softmax
//                           in the exp2 domain, P packed to 16 bits and written
//                           back with tcgen05.st, the running sum kept per half;
//                           the halves exchange their maxima through shared
//                           memory and an mbarrier once per key tile, which also
//                           orders one half's P store after the other's S reads.
//                           O is rescaled in TMEM only when the row maximum grew
//                           by more than 2^8 (the stale maximum keeps P below
//                           256, well inside 16-bit range). Four softmax warps
//                           per scheduler instead of two hide the latencies of
//                           the dependent max / exp2 / sum chains. (One issuing
//                           thread for both tiles is deliberate: with a thread per
//                           tile the two tiles' MMAs interleave in the tensor
//                           pipe and each tile waits for both - measured 850
//                           against 1,015 TFLOP/s.)
//    TMEM: S0, S1 (128 columns each, P aliases their first 64), O0, O1 (D each).
//    Every mbarrier wait is bounded; a timeout raises the status word and the CTA
//    drains its copies and MMAs before it frees TMEM.
#include "tma.cuh"

namespace strix {

int32_t* umma_status_ptr();   // moe_gemm_umma.cu

namespace {

using namespace umma;

constexpr int kPuQ = 128, kPuKeys = 128;           // Q tile rows, key tile
constexpr int kPuHalves = 2;                       // threads per query row
constexpr int kPuCols = kPuKeys / kPuHalves;       // columns of a key tile per softmax thread
constexpr int kPuSoftmaxWarps = 2 * 4 * kPuHalves;
constexpr int kPuThreads = (2 + kPuSoftmaxWarps) * 32;   // producer, issuer, softmax warps
constexpr int kPuStages = 2;
constexpr float kPuRescale = 8.f;                  // log2 of the growth of the maximum that forces a rescale

template <int D>
struct PuLayout {
  static constexpr int kQTile = kPuQ * D * 2;                  // one Q tile, 16-bit
  static constexpr int kKTile = kPuKeys * D * 2;               // K' tile: [keys][D]
  static constexpr int kVTile = D * kPuKeys * 2;               // V'^T tile: [D][keys]
  static constexpr int kStage = kKTile + kVTile;
  static constexpr int kSmem = 1024 + 2 * kQTile + kPuStages * kStage + 256;
  static constexpr int kTmemS = 0, kTmemO = 2 * kPuKeys;       // column offsets
};

struct PuArgs {
  __nv_bfloat16* out;
  const int32_t* cu;         // [nseq + 1] query offsets
  const int32_t* seq_lens;   // [nseq]
  const float* sinks;        // optional [hq]
  int32_t* status;
  int64_t o_st, o_sh;        // elements
  int64_t q_row_bytes_h;     // bytes between heads of one query row
  int64_t cap;               // workspace rows per KV head
  int nseq, hq, hkv, window_left;
  float scale;
};

// ------------------------------------------------------------------ gather pass
struct GatherArgs {
  const uint8_t* kc;
  const uint8_t* vc;
  const float* ks;
  const float* vs;
  const int32_t* seq_lens;
  const int32_t* block_table;
  uint16_t* kp;              // K'   [hkv][cap][D]
  uint16_t* vt;              // V'^T [hkv][D][cap]
  int64_t k_sb, k_ss, k_sh, v_sb, v_ss, v_sh;          // bytes
  int64_t ks_sb, ks_ss, ks_sh, vs_sb, vs_ss, vs_sh;    // elements
  int64_t bt_stride, cap;
  int nseq, hkv, block_size, aligned16;
};

// 256 threads: key = tid / 2 of the tile, half = tid % 2 of the row.
template <int D, bool Q8>
__global__ void __launch_bounds__(256) prefill_gather_kernel(const GatherArgs p) {
  constexpr int kPad = D + 2;                        // 16-bit elements per staged V row
  __shared__ uint16_t s_v[kPuKeys * kPad];
  __shared__ int64_t s_off;
  const int tid = threadIdx.x;
  const int tile = blockIdx.x, h = blockIdx.y, n = blockIdx.z;
  const int kv_len = p.seq_lens[n];
  if (tile * kPuKeys >= kv_len) return;
  if (tid == 0) {
    int64_t off = 0;
    for (int m = 0; m < n; ++m) off += (int64_t(p.seq_lens[m]) + kPuKeys - 1) / kPuKeys * kPuKeys;
    s_off = off;
  }
  __syncthreads();
  const int64_t row0 = s_off + int64_t(tile) * kPuKeys;     // first workspace row of this tile
  if (row0 + kPuKeys > p.cap) return;                        // never: the host sized cap from the table
  const int key_l = tid >> 1, half = tid & 1;
  const int key = tile * kPuKeys + key_l;
  const bool ok = key < kv_len;
  constexpr int kHalfEl = D / 2;                             // elements this thread converts per matrix
  uint32_t kw[kHalfEl / 2], vw[kHalfEl / 2];                 // 16-bit pairs
#pragma unroll
  for (int i = 0; i < kHalfEl / 2; ++i) kw[i] = vw[i] = 0u;
  if (ok) {
    const int blk = p.block_table[int64_t(n) * p.bt_stride + key / p.block_size];
    const int slot = key % p.block_size;
    constexpr int kEb = Q8 ? 1 : 2;
    const uint8_t* ksrc = p.kc + int64_t(blk) * p.k_sb + int64_t(slot) * p.k_ss + int64_t(h) * p.k_sh + half * kHalfEl * kEb;
    const uint8_t* vsrc = p.vc + int64_t(blk) * p.v_sb + int64_t(slot) * p.v_ss + int64_t(h) * p.v_sh + half * kHalfEl * kEb;
    if constexpr (Q8) {
      const float ksc = p.ks[int64_t(blk) * p.ks_sb + int64_t(slot) * p.ks_ss + int64_t(h) * p.ks_sh];
      const float vsc = p.vs[int64_t(blk) * p.vs_sb + int64_t(slot) * p.vs_ss + int64_t(h) * p.vs_sh];
#pragma unroll
      for (int m = 0; m < 2; ++m) {
        const uint8_t* src = m == 0 ? ksrc : vsrc;
        const float sc = m == 0 ? ksc : vsc;
        uint32_t* dst = m == 0 ? kw : vw;
#pragma unroll
        for (int i = 0; i < kHalfEl / 4; ++i) {
          const uint32_t x = p.aligned16 ? reinterpret_cast<const uint32_t*>(src)[i]
                                         : *reinterpret_cast<const uint32_t*>(src + 4 * i);
          const float f0 = float(int8_t(x & 255)) * sc, f1 = float(int8_t((x >> 8) & 255)) * sc;
          const float f2 = float(int8_t((x >> 16) & 255)) * sc, f3 = float(int8_t(x >> 24)) * sc;
          dst[2 * i] = pack_f16x2(f0, f1);
          dst[2 * i + 1] = pack_f16x2(f2, f3);
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < kHalfEl / 8; ++i) {
        const uint4 a = reinterpret_cast<const uint4*>(ksrc)[i], b = reinterpret_cast<const uint4*>(vsrc)[i];
        kw[4 * i] = a.x, kw[4 * i + 1] = a.y, kw[4 * i + 2] = a.z, kw[4 * i + 3] = a.w;
        vw[4 * i] = b.x, vw[4 * i + 1] = b.y, vw[4 * i + 2] = b.z, vw[4 * i + 3] = b.w;
      }
    }
  }
  // K' row: contiguous 16-byte stores (keys past the sequence are zeros)
  uint4* kdst = reinterpret_cast<uint4*>(p.kp + ((int64_t(h) * p.cap + row0 + key_l) * D + half * kHalfEl));
#pragma unroll
  for (int i = 0; i < kHalfEl / 8; ++i) kdst[i] = make_uint4(kw[4 * i], kw[4 * i + 1], kw[4 * i + 2], kw[4 * i + 3]);
  // V: through shared memory for the transposition
  uint32_t* srow = reinterpret_cast<uint32_t*>(s_v + key_l * kPad + half * kHalfEl);
#pragma unroll
  for (int i = 0; i < kHalfEl / 2; ++i) srow[i] = vw[i];
  __syncthreads();
  // thread -> (d, half of the keys): 64 keys = 128 contiguous bytes of row d
  for (int idx = tid; idx < D * 2; idx += 256) {
    const int d = idx >> 1, kh = idx & 1;
    uint32_t w[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const uint32_t lo = s_v[(kh * 64 + 2 * i) * kPad + d], hi = s_v[(kh * 64 + 2 * i + 1) * kPad + d];
      w[i] = lo | (hi << 16);
    }
    uint4* vdst = reinterpret_cast<uint4*>(p.vt + ((int64_t(h) * D + d) * p.cap + row0 + kh * 64));
#pragma unroll
    for (int i = 0; i < 8; ++i) vdst[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
  }
}

__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// ------------------------------------------------------------------ attention
template <int D, bool Q8>
__global__ void __launch_bounds__(kPuThreads, 1) attn_prefill_umma_kernel(
    const PuArgs p, const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
    const __grid_constant__ CUtensorMap map_v) {
  using L = PuLayout<D>;
  constexpr int S = kPuStages;
  constexpr uint32_t kFmt = Q8 ? 0u : 1u;            // kind::f16 operand format: f16 / bf16
  constexpr int kSub = D / 64;                       // 128-byte column blocks of a Q or K' row
  extern __shared__ uint8_t raw_smem[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) & ~uintptr_t(1023));
  __shared__ __align__(8) uint64_t q_full, q_ready, full_bar[S], empty_bar[S], s_full[2], p_full[2], o_full, drain_bar;
  __shared__ __align__(8) uint64_t pair_bar[8];      // the two warps that share (Q tile, lane quadrant)
  __shared__ float s_xmax[2][kPuHalves][kPuQ], s_xl[2][kPuHalves][kPuQ];   // what the halves of a row exchange
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int head = blockIdx.x, kvh = head / (p.hq / p.hkv);
  int armed = 0;
  // once a bounded wait gave up somewhere the output is void anyway: the CTAs still
  // to come return at once instead of each running into its own timeouts
  if (*reinterpret_cast<const volatile int32_t*>(p.status) != 0) return;

  // ---- which sequence and which 256-query tile of it; first workspace row of its keys
  int n = 0, tile = blockIdx.y, q_begin = 0, q_len = 0;
  int64_t kv_off = 0;
  for (;; ++n) {
    if (n >= p.nseq) return;
    q_begin = p.cu[n];
    q_len = p.cu[n + 1] - q_begin;
    const int tiles = (q_len + 2 * kPuQ - 1) / (2 * kPuQ);
    if (tile < tiles) {
      tile = tiles - 1 - tile;          // the last tiles see the most keys: start them first
      break;
    }
    tile -= tiles;
    kv_off += (int64_t(p.seq_lens[n]) + kPuKeys - 1) / kPuKeys * kPuKeys;
  }
  const int kv_len = p.seq_lens[n];
  const int pos0 = kv_len - q_len;                               // position of local query 0
  const int cta_q0 = tile * 2 * kPuQ;
  const int cta_last = min(cta_q0 + 2 * kPuQ, q_len) - 1;        // last live local query
  const int k_end = min(pos0 + cta_last + 1, kv_len);
  const int k_begin = p.window_left >= 0 ? max(0, pos0 + cta_q0 - p.window_left) / kPuKeys * kPuKeys : 0;
  const int n_tiles = k_end > k_begin ? (k_end - k_begin + kPuKeys - 1) / kPuKeys : 0;

  if (n_tiles == 0) {   // no visible key at all (empty context): zeros, as a 0-weight softmax
    for (int i = tid; i < (cta_last - cta_q0 + 1) * (D / 8); i += kPuThreads) {
      const int r = cta_q0 + i / (D / 8), ch = i % (D / 8);
      if (r < q_len)
        *reinterpret_cast<uint4*>(p.out + int64_t(q_begin + r) * p.o_st + head * p.o_sh + 8 * ch) = make_uint4(0, 0, 0, 0);
    }
    return;
  }

  if (tid == 0) {
    mbar_init(&q_full, 1);
    mbar_init(&q_ready, kPuSoftmaxWarps);
    for (int i = 0; i < S; ++i) mbar_init(&full_bar[i], 1), mbar_init(&empty_bar[i], 1);
    for (int i = 0; i < 2; ++i) mbar_init(&s_full[i], 1), mbar_init(&p_full[i], 4 * kPuHalves);
    for (int i = 0; i < 8; ++i) mbar_init(&pair_bar[i], kPuHalves);
    mbar_init(&o_full, 1);
    mbar_init(&drain_bar, 1);
    s_abort = 0;
    fence_mbar_init();
  }
  if (warp == 1) tmem_alloc(&tmem_slot, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_slot;
  const uint32_t smem_s = smem_u32(smem);
  const uint32_t q_s = smem_s, ring_s = smem_s + 2 * L::kQTile;

  if (warp == 0) {
    // ------------------------------------------------------------- producer
    if (lane == 0) {
      tma::prefetch_map(&map_q);
      tma::prefetch_map(&map_k);
      tma::prefetch_map(&map_v);
      tma::mbar_expect_tx(&q_full, 2 * L::kQTile);
#pragma unroll
      for (int q = 0; q < 2; ++q)
#pragma unroll
        for (int sb = 0; sb < kSub; ++sb)
          tma::load_2d(q_s + q * L::kQTile + sb * (kPuQ * 128), &map_q,
                       int(head * p.q_row_bytes_h) + sb * 128, q_begin + cta_q0 + q * kPuQ, &q_full);
      bool dead = false;
      int t = 0;
      for (; t < n_tiles; ++t) {
        const int s = t % S;
        if (!mbar_wait(&empty_bar[s], ((t / S) & 1) ^ 1) || s_abort) {
          dead = true;
          break;
        }
        const uint32_t st = ring_s + s * L::kStage;
        const int64_t row = kv_off + k_begin + int64_t(t) * kPuKeys;
        tma::mbar_expect_tx(&full_bar[s], L::kStage);
#pragma unroll
        for (int sb = 0; sb < kSub; ++sb)
          tma::load_2d(st + sb * (kPuKeys * 128), &map_k, sb * 128, int(int64_t(kvh) * p.cap + row), &full_bar[s]);
#pragma unroll
        for (int kh = 0; kh < 2; ++kh)
          tma::load_2d(st + L::kKTile + kh * (D * 128), &map_v, int((row + kh * 64) * 2), kvh * D, &full_bar[s]);
      }
      armed = t;
      if (dead) atomicExch(p.status, 1), s_abort = 1;
    }
  } else if (warp == 1) {
    // --------------------------------------------------------------- issuer
    if (lane == 0) {
      const uint32_t idesc_s = instr_desc(D_F32, kFmt, kFmt, kPuQ, kPuKeys);
      const uint32_t idesc_o = instr_desc(D_F32, kFmt, kFmt, kPuQ, D);
      const uint32_t q_lo = smem_desc_lo(q_s), ring_lo = smem_desc_lo(ring_s);
      bool dead = false;
      auto issue_s = [&](int q, int j) {
        const uint32_t a0 = q_lo + ((q * L::kQTile) >> 4), b0 = ring_lo + (((j % S) * L::kStage) >> 4);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t o = ((kk >> 2) * (kPuQ * 128) + (kk & 3) * 32) >> 4;
          mma_ss<KIND_F16>(tmem + L::kTmemS + q * kPuKeys, desc_pack(a0 + o, kDescHiSw128),
                           desc_pack(b0 + o, kDescHiSw128), idesc_s, kk > 0 ? 1u : 0u);
        }
        mma_commit(&s_full[q]);
      };
      auto issue_pv = [&](int q, int j) {
        const uint32_t b0 = ring_lo + (((j % S) * L::kStage + L::kKTile) >> 4);
#pragma unroll
        for (int kk = 0; kk < kPuKeys / 16; ++kk) {
          const uint32_t o = ((kk >> 2) * (D * 128) + (kk & 3) * 32) >> 4;
          mma_ts_f16(tmem + L::kTmemO + q * D, tmem + L::kTmemS + q * kPuKeys + kk * 8,
                     desc_pack(b0 + o, kDescHiSw128), idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
        }
      };
      if (!mbar_wait(Q8 ? &q_ready : &q_full, 0) || !mbar_wait(&full_bar[0], 0)) dead = true;
      if (!dead) {
        tc_fence_after_sync();
        issue_s(0, 0);
        issue_s(1, 0);
      }
      for (int j = 0; j < n_tiles && !dead; ++j) {
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          if (!mbar_wait(&p_full[q], j & 1) || s_abort) {
            dead = true;
            break;
          }
          tc_fence_after_sync();
          issue_pv(q, j);
          if (q == 1) mma_commit(&empty_bar[j % S]);      // K' and V' of tile j are consumed
          if (j + 1 < n_tiles) {
            if (q == 0 && !mbar_wait(&full_bar[(j + 1) % S], ((j + 1) / S) & 1)) {
              dead = true;
              break;
            }
            tc_fence_after_sync();
            issue_s(q, j + 1);
          }
        }
      }
      if (!dead) mma_commit(&o_full);
      if (dead) atomicExch(p.status, 1), s_abort = 1;
    }
  } else if (warp >= 2) {
    // -------------------------------------------------------------- softmax
    const int sw = warp - 2;
    const int q = sw >> 3;                             // Q tile
    const int half = (sw >> 2) & 1;                    // which 64 of a key tile's columns
    const int quad = warp & 3;                         // the TMEM lane quadrant this warp may touch
    const int row = quad * 32 + lane;
    uint64_t* const pbar = &pair_bar[q * 4 + quad];
    const uint32_t lane_base = uint32_t(quad * 32) << 16;
    const uint32_t t_s = tmem + lane_base + L::kTmemS + q * kPuKeys + half * kPuCols;   // this thread's scores
    const uint32_t t_p = tmem + lane_base + L::kTmemS + q * kPuKeys + half * (kPuCols / 2);   // its share of P
    const uint32_t t_o = tmem + lane_base + L::kTmemO + q * D;
    bool dead = false;
    int px = 0;                                        // uses of the pair's barrier so far
    // Both warps of a row have passed this point and see each other's shared-memory
    // writes from before it. A bounded mbarrier wait, not bar.sync: if one warp gave
    // up on a wait and left, the other must time out too instead of hanging.
    auto pair_sync = [&]() {
      __syncwarp();
      if (lane == 0) mbar_arrive(pbar);
      const bool ok = mbar_wait(pbar, px & 1);
      ++px;
      return !__any_sync(0xffffffffu, !ok);
    };

    if constexpr (Q8) {
      // the bf16 queries become fp16 in place (element-wise, so the swizzle is untouched)
      const bool ok = mbar_wait(&q_full, 0);
      if (__any_sync(0xffffffffu, !ok)) dead = true;
      if (!dead) {
        uint4* qv = reinterpret_cast<uint4*>(smem);
        for (int i = tid - 64; i < 2 * L::kQTile / 16; i += kPuSoftmaxWarps * 32) {
          uint4 x = qv[i];
          x.x = pack_f16x2(bf16_lo(x.x), bf16_hi(x.x)), x.y = pack_f16x2(bf16_lo(x.y), bf16_hi(x.y));
          x.z = pack_f16x2(bf16_lo(x.z), bf16_hi(x.z)), x.w = pack_f16x2(bf16_lo(x.w), bf16_hi(x.w));
          qv[i] = x;
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(&q_ready);
      }
    }

    const int qi = cta_q0 + q * kPuQ + row;            // local query index of this thread's row
    const int qpos = pos0 + qi;
    const int warp_q0 = pos0 + cta_q0 + q * kPuQ + quad * 32;   // position of the warp's first row
    const float sl2 = p.scale * kLog2e;
    const float2 sl2x2 = make_float2(sl2, sl2);
    float m_ref = -INFINITY, l = 0.f;                  // l: this half's share of the row sum
    for (int j = 0; j < n_tiles && !dead; ++j) {
      const int k0 = k_begin + j * kPuKeys + half * kPuCols;   // first key of this thread's columns
      const bool ok = mbar_wait(&s_full[q], j & 1);
      if (__any_sync(0xffffffffu, !ok) || s_abort) {
        dead = true;
        break;
      }
      tc_fence_after_sync();
      // columns every row of the warp sees completely need no mask
      const bool interior = k0 + kPuCols <= k_end && k0 + kPuCols - 1 <= warp_q0 &&
                            (p.window_left < 0 || warp_q0 + 31 - k0 <= p.window_left);
      auto masked = [&](float v, int key) {
        const bool vis = key < k_end && key <= qpos && (p.window_left < 0 || qpos - key <= p.window_left);
        return vis ? v : -INFINITY;
      };
      // One pass over the scores in the common case: P = 2^(s - m_ref) against the
      // maximum carried over from the earlier tiles, the tile's own maximum taken on
      // the way (three-input max, packed two-wide multiply-add and add: about three
      // instructions per score). Only if the row's maximum exceeds m_ref by more than
      // 2^kPuRescale (or no key was seen yet) the accumulator is rescaled and the pass
      // repeated - S is still intact, because P (which overwrites its first 64
      // columns) is held in registers until both halves have decided. The scores come
      // 16 columns at a time and are not prefetched: with four softmax warps per
      // scheduler another warp covers the TMEM load, and the registers a second buffer
      // would take are what keeps the loop free of spills at the 96 registers a CTA of
      // 18 warps allows (measured at 65,536 tokens: 8-column double buffering 950
      // TFLOP/s, 16-column double buffering with spills 825, this form 1,015). Maxima
      // and sums run in four independent chains each.
      uint32_t pk[kPuCols / 2];
      float lt = 0.f;
      const bool seen = __all_sync(0xffffffffu, m_ref != -INFINITY);
#pragma unroll 1
      for (int attempt = 0; attempt < 2 && !dead; ++attempt) {
        const bool want_p = attempt == 1 || seen;   // rows without a key yet only take the maximum first
        const float nb = m_ref == -INFINITY ? 0.f : -m_ref;
        const float2 nbx2 = make_float2(nb, nb);
        float mxa[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        float2 lta[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
        uint32_t r[16];
#pragma unroll
        for (int c = 0; c < kPuCols / 16; ++c) {
          tmem_ld_32x16(t_s + c * 16, r);
          tmem_ld_wait();
          float v[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
          if (!interior) {
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = masked(v[i], k0 + c * 16 + i);
          }
#pragma unroll
          for (int i = 0; i < 16; i += 2) mxa[(i >> 1) & 3] = max3(mxa[(i >> 1) & 3], v[i], v[i + 1]);
          if (want_p) {
#pragma unroll
            for (int i = 0; i < 16; i += 2) {
              const float2 e = __ffma2_rn(make_float2(v[i], v[i + 1]), sl2x2, nbx2);
              const float2 pp = make_float2(fast_exp2(e.x), fast_exp2(e.y));
              lta[(i >> 1) & 1] = __fadd2_rn(lta[(i >> 1) & 1], pp);
              pk[c * 8 + (i >> 1)] = Q8 ? pack_f16x2(pp.x, pp.y) : pack_bf16x2(pp.x, pp.y);
            }
          }
        }
        lt = (lta[0].x + lta[0].y) + (lta[1].x + lta[1].y);
        if (attempt == 1) {
          if (!pair_sync()) dead = true;     // the other half has finished re-reading S
          break;
        }
        s_xmax[q][half][row] = fmaxf(max3(mxa[0], mxa[1], mxa[2]), mxa[3]);
        if (!pair_sync()) {                  // both halves have read S; the maxima are visible
          dead = true;
          break;
        }
        const float mx = fmaxf(s_xmax[q][0][row], s_xmax[q][1][row]);
        const float m_new = fmaxf(m_ref, mx * sl2);
        // lazy rescale: only when the maximum grew by more than 2^kPuRescale (or is the first)
        const bool need = m_new > m_ref + kPuRescale || (m_ref == -INFINITY && m_new > -INFINITY);
        const bool any_need = __any_sync(0xffffffffu, need);
        if (!any_need && seen) break;
        if (any_need) {
          const float f = need ? (m_ref == -INFINITY ? 0.f : fast_exp2(m_ref - m_new)) : 1.f;
          if (j > 0) {                       // each half rescales its half of O's columns
#pragma unroll 1
            for (int c = half * (D / 32); c < (half + 1) * (D / 32); ++c) {
              uint32_t ro[16];
              tmem_ld_32x16(t_o + c * 16, ro);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 16; ++i) ro[i] = __float_as_uint(__uint_as_float(ro[i]) * f);
              tmem_st_32x16(t_o + c * 16, ro);
            }
          }
          l *= f;
          if (need) m_ref = m_new;
        }
      }
      if (dead) break;
      l += lt;
#pragma unroll
      for (int c = 0; c < kPuCols / 32; ++c)
        tmem_st_32x16(t_p + c * 16, *reinterpret_cast<uint32_t(*)[16]>(&pk[c * 16]));
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[q]);
    }

    // ---- epilogue: the row's sum from both halves, sinks, normalise, store this half's columns
    if (!dead) {
      s_xl[q][half][row] = l;
      if (!pair_sync()) dead = true;
      l = s_xl[q][0][row] + s_xl[q][1][row];
    }
    if (!dead) {
      const bool ok = mbar_wait(&o_full, 0);
      if (__any_sync(0xffffffffu, !ok) || s_abort) dead = true;
    }
    if (!dead) {
      tc_fence_after_sync();
      if (p.sinks != nullptr) {
        const float sk = p.sinks[head] * kLog2e;
        if (m_ref == -INFINITY) l = 1.f; else l += fast_exp2(sk - m_ref);
      }
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* orow = p.out + int64_t(q_begin + min(qi, q_len - 1)) * p.o_st + head * p.o_sh;
#pragma unroll 1
      for (int c = half * (D / 32); c < (half + 1) * (D / 32); ++c) {
        uint32_t r[16];
        tmem_ld_32x16(t_o + c * 16, r);
        tmem_ld_wait();
        if (qi < q_len) {
#pragma unroll
          for (int i = 0; i < 16; i += 8) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(r[i]) * inv, __uint_as_float(r[i + 1]) * inv);
            o.y = pack_bf16x2(__uint_as_float(r[i + 2]) * inv, __uint_as_float(r[i + 3]) * inv);
            o.z = pack_bf16x2(__uint_as_float(r[i + 4]) * inv, __uint_as_float(r[i + 5]) * inv);
            o.w = pack_bf16x2(__uint_as_float(r[i + 6]) * inv, __uint_as_float(r[i + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c * 16 + i) = o;
          }
        }
      }
    }
    if (dead) atomicExch(p.status, 1), s_abort = 1;
  }

  tc_fence_before_sync();
  __syncthreads();
  if (s_abort) {   // wait for the copies and MMAs still in flight before TMEM goes
    if (tid == 0) {
      mbar_wait(&q_full, 0);
      drain_armed_loads(full_bar, S, armed);
    }
    if (warp == 1 && lane == 0) drain_issued_mmas(&drain_bar);
    tc_fence_before_sync();
    __syncthreads();
  }
  if (warp == 1) tmem_dealloc(tmem, 512);
}

template <int D, bool Q8>
int launch_umma_prefill(const PuArgs& p, const GatherArgs& g, const CUtensorMap& mq, const CUtensorMap& mk,
                        const CUtensorMap& mv, int64_t gather_tiles, int64_t q_tiles, cudaStream_t st) {
  using L = PuLayout<D>;
  auto kernel = attn_prefill_umma_kernel<D, Q8>;
  static bool done[64] = {};
  int dev = 0;
  STRIX_CUDA(cudaGetDevice(&dev));
  STRIX_CHECK(dev >= 0 && dev < 64, "device index %d out of range", dev);
  if (!done[dev]) {
    STRIX_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kSmem));
    done[dev] = true;
  }
  const dim3 ggrid{unsigned(gather_tiles), unsigned(p.hkv), unsigned(p.nseq)};
  prefill_gather_kernel<D, Q8><<<ggrid, 256, 0, st>>>(g);
  if (int rc = launch_status("prefill_gather")) return rc;
  const dim3 grid{unsigned(p.hq), unsigned(q_tiles), 1u};
  kernel<<<grid, kPuThreads, L::kSmem, st>>>(p, mq, mk, mv);
  return launch_status("attn_prefill_umma");
}

// workspace rows per KV head: every sequence padded to whole key tiles
int64_t prefill_cap(int64_t nseq, int64_t max_blocks, int64_t block_size) {
  return nseq * ((max_blocks * block_size + kPuKeys - 1) / kPuKeys * kPuKeys);
}

}  // namespace
}  // namespace strix

using namespace strix;

extern "C" int64_t strix_attn_prefill_workspace(int64_t nseq, int64_t max_blocks, int64_t block_size,
                                                int64_t hkv, int64_t head_dim) {
  if (nseq < 0 || max_blocks < 0 || block_size < 1 || hkv < 1 || head_dim < 1) return -1;
  return 2 * hkv * prefill_cap(nseq, max_blocks, block_size) * head_dim * 2;
}

extern "C" int strix_attn_prefill_umma_covers(int64_t head_dim, int64_t q_stride_t, int64_t q_stride_h,
                                              int64_t out_stride_t, int64_t out_stride_h, int kv_int8) {
  (void)kv_int8;
  return (head_dim == 64 || head_dim == 128) && q_stride_t % 8 == 0 && q_stride_h % 8 == 0 &&
         out_stride_t % 8 == 0 && out_stride_h % 8 == 0;
}

extern "C" int strix_attn_prefill_umma(
    void* out, const void* q, const void* key_cache, const void* value_cache, const float* k_scale,
    const float* v_scale, const int32_t* cu_seqlens_q, const int32_t* seq_lens,
    const int32_t* block_table, const float* sinks, void* workspace, int64_t workspace_bytes,
    int64_t total_q, int64_t nseq, int64_t hq, int64_t hkv, int64_t head_dim, int64_t block_size,
    int64_t max_blocks, int64_t bt_stride, int64_t q_stride_t, int64_t q_stride_h, int64_t out_stride_t,
    int64_t out_stride_h, int64_t k_stride_b, int64_t k_stride_s, int64_t k_stride_h,
    int64_t v_stride_b, int64_t v_stride_s, int64_t v_stride_h, int64_t ks_stride_b,
    int64_t ks_stride_s, int64_t ks_stride_h, int64_t vs_stride_b, int64_t vs_stride_s,
    int64_t vs_stride_h, double scale, int64_t window_left, int kv_int8, strix_stream_t stream) {
  STRIX_CHECK(strix_attn_prefill_umma_covers(head_dim, q_stride_t, q_stride_h, out_stride_t, out_stride_h, kv_int8) &&
                  reinterpret_cast<uintptr_t>(q) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0,
              "head_dim 64 or 128 with 16-byte aligned q / out rows");
  STRIX_CHECK(hq > 0 && hkv > 0 && hq % hkv == 0 && hq <= 65535, "hq must be a multiple of hkv");
  STRIX_CHECK(block_size >= 1 && nseq >= 0 && total_q >= 0 && max_blocks >= 0 && nseq <= 65535, "bad sizes");
  STRIX_CHECK(!kv_int8 || (k_scale != nullptr && v_scale != nullptr), "int8 KV needs k_scale and v_scale");
  const int eb = kv_int8 ? 1 : 2;
  const int64_t ks[6] = {k_stride_b * eb, k_stride_s * eb, k_stride_h * eb, v_stride_b * eb, v_stride_s * eb, v_stride_h * eb};
  bool a4 = reinterpret_cast<uintptr_t>(key_cache) % 4 == 0 && reinterpret_cast<uintptr_t>(value_cache) % 4 == 0;
  bool a16 = reinterpret_cast<uintptr_t>(key_cache) % 16 == 0 && reinterpret_cast<uintptr_t>(value_cache) % 16 == 0;
  for (int i = 0; i < 6; ++i) a4 = a4 && ks[i] % 4 == 0, a16 = a16 && ks[i] % 16 == 0;
  STRIX_CHECK(kv_int8 ? a4 : a16, "cache rows must be 4-byte (int8) / 16-byte (bf16) aligned");
  if (nseq == 0 || total_q == 0) return STRIX_OK;
  const int64_t need = strix_attn_prefill_workspace(nseq, max_blocks, block_size, hkv, head_dim);
  STRIX_CHECK(workspace != nullptr && workspace_bytes >= need && reinterpret_cast<uintptr_t>(workspace) % 1024 == 0,
              "workspace of %lld bytes (1024-byte aligned) required, got %lld", (long long)need,
              (long long)workspace_bytes);
  const int64_t cap = prefill_cap(nseq, max_blocks, block_size);
  STRIX_CHECK(hkv * cap < (int64_t(1) << 31) && cap * 2 < (int64_t(1) << 31) && total_q < (int64_t(1) << 31),
              "batch too large for 32-bit tile coordinates");

  GatherArgs g;
  g.kc = static_cast<const uint8_t*>(key_cache), g.vc = static_cast<const uint8_t*>(value_cache);
  g.ks = k_scale, g.vs = v_scale, g.seq_lens = seq_lens, g.block_table = block_table;
  g.kp = static_cast<uint16_t*>(workspace);
  g.vt = g.kp + hkv * cap * head_dim;
  g.k_sb = ks[0], g.k_ss = ks[1], g.k_sh = ks[2], g.v_sb = ks[3], g.v_ss = ks[4], g.v_sh = ks[5];
  g.ks_sb = ks_stride_b, g.ks_ss = ks_stride_s, g.ks_sh = ks_stride_h;
  g.vs_sb = vs_stride_b, g.vs_ss = vs_stride_s, g.vs_sh = vs_stride_h;
  g.bt_stride = bt_stride, g.cap = cap;
  g.nseq = int(nseq), g.hkv = int(hkv), g.block_size = int(block_size), g.aligned16 = a16 ? 1 : 0;

  PuArgs p;
  p.out = static_cast<__nv_bfloat16*>(out), p.cu = cu_seqlens_q, p.seq_lens = seq_lens, p.sinks = sinks;
  p.status = umma_status_ptr();
  STRIX_CHECK(p.status != nullptr, "status word unavailable");
  p.o_st = out_stride_t, p.o_sh = out_stride_h, p.q_row_bytes_h = q_stride_h * 2, p.cap = cap;
  p.nseq = int(nseq), p.hq = int(hq), p.hkv = int(hkv), p.window_left = int(window_left);
  p.scale = float(scale);

  CUtensorMap mq, mk, mv;
  // queries: bytes [total_q, (hq - 1) * head stride + D], boxes of 128 rows x 128 bytes
  STRIX_CHECK(tma::make_map_u8(&mq, q, uint64_t(total_q), uint64_t((hq - 1) * q_stride_h * 2 + head_dim * 2),
                               uint64_t(q_stride_t * 2), kPuQ) &&
                  tma::make_map_u8(&mk, g.kp, uint64_t(hkv * cap), uint64_t(head_dim * 2),
                                   uint64_t(head_dim * 2), kPuKeys) &&
                  tma::make_map_u8(&mv, g.vt, uint64_t(hkv * head_dim), uint64_t(cap * 2), uint64_t(cap * 2),
                                   uint32_t(head_dim)),
              "tensor map encoding failed");
  const int64_t gather_tiles = (max_blocks * block_size + kPuKeys - 1) / kPuKeys;
  const int64_t q_tiles = (total_q + 2 * kPuQ - 1) / (2 * kPuQ) + nseq;
  STRIX_CHECK(gather_tiles >= 1 && gather_tiles < (int64_t(1) << 31) && q_tiles <= 65535,
              "too many tiles for one launch");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (head_dim == 128)
    return kv_int8 ? launch_umma_prefill<128, true>(p, g, mq, mk, mv, gather_tiles, q_tiles, st)
                   : launch_umma_prefill<128, false>(p, g, mq, mk, mv, gather_tiles, q_tiles, st);
  return kv_int8 ? launch_umma_prefill<64, true>(p, g, mq, mk, mv, gather_tiles, q_tiles, st)
                 : launch_umma_prefill<64, false>(p, g, mq, mk, mv, gather_tiles, q_tiles, st);
}
