// Grouped expert GEMM for MXFP4 experts (e2m1 nibbles, e8m0 scale per 32
// elements) and bf16 activations on the Blackwell tensor cores, for sm_100a:
// the tensor-bound form (m-blocks of 128 tokens) of moe_gemm_mxfp4, over
// activations laid out by sorted position (row p of `a` = sorted position p).
//
// MXFP4 x bf16 has no native MMA kind, so the weights are decoded on the way:
//   producer (1 thread)   TMA: the m-block's 128 token rows of a 64-wide K block
//                         (bf16, 128-byte-swizzled) and the tile's 256 weight
//                         rows of the same K block as packed bytes (32 per row;
//                         a 4-d box interleaves gate and up rows);
//   transform (16 warps)  half a weight row per thread - one scale group: 32 nibbles
//                         -> 32 bf16 by a byte-permute table, times the group's e8m0
//                         scale (exact), stored as the 128-byte-swizzled B operand
//                         tile (four warps per scheduler, so that the latencies of
//                         the shared-memory round trip are covered);
//   issuer (1 thread)     four tcgen05.mma kind::f16 (bf16 x bf16 -> f32, 128 x 256
//                         x 16) per K block; the whole K accumulates in one of two
//                         256-column TMEM buffers;
//   epilogue (4 warps)    one token row per thread: act(gate) * up on adjacent
//                         columns, or x routing weight; contiguous output rows.
// The decode is the expensive part (about 200 instructions per weight row and K
// block), so a decoded tile serves TWO m-blocks where it can: consecutive
// m-blocks of one expert form a unit of 256 tokens, whose halves accumulate in
// the two 256-column TMEM buffers from the same decoded tile (a lone m-block is a
// unit of one). Two rings: three stages of (two token tiles + packed weights),
// 40 KB each, and two decoded operand tiles of 32 KB that alternate between the
// transform warps and the MMAs. A K block's single tcgen05.commit frees its stage
// for the producer and, two K blocks later, its decoded tile for the transform
// warps. Every mbarrier wait is bounded.
#include <cstdlib>

#include "tma.cuh"

namespace strix {

int32_t* umma_status_ptr();   // moe_gemm_umma.cu: the status word of the tcgen05 kernels

namespace {

using namespace umma;

constexpr int kMxTok = 128, kMxCols = 256, kMxKB = 64;       // tile: tokens x weight rows x K
constexpr int kMxTransformWarps = 16, kMxEpilogueWarps = 4;
constexpr int kMxThreads = (4 + kMxTransformWarps + kMxEpilogueWarps) * 32;
constexpr int kMxStages = 3, kMxDecoded = 2;
constexpr int kMxMaxMBlocks = 2048;

struct MxLayout {
  static constexpr int kABytes = kMxTok * kMxKB * 2;          // 16 KB of bf16 token rows
  static constexpr int kRawBytes = kMxCols * kMxKB / 2;       // 8 KB of packed weights
  static constexpr int kBBytes = kMxCols * kMxKB * 2;         // 32 KB of decoded weights
  static constexpr int kStageBytes = 2 * kABytes + kRawBytes; // what the TMA fills: two token tiles + weights
  static constexpr int kSmem = 1024 + kMxStages * kStageBytes + kMxDecoded * kBBytes + 256;
};

struct MxArgs {
  __nv_bfloat16* c;
  const uint8_t* scales;      // e8m0 [E, N, K / 32]
  const int32_t* sorted_ids;
  const int32_t* expert_ids;
  const int32_t* num_post;
  const float* topk_w;
  int32_t* status;
  int64_t num_valid, c_stride, s_se, s_sn;
  int K, N, n_tiles, gate_act, c_sorted, experts;
};

__device__ __forceinline__ uint32_t mx_mul_bf16x2(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}

// Eight nibbles (element i in bits [4i, 4i + 4)) -> four bf16 pairs times scale2
// (2^(s - 127) twice, bf16 pattern s << 7; s = 0 is the zero block). The low three
// bits of a nibble index an 8-entry table of bf16 patterns (0, .5, 1, 1.5, 2, 3,
// 4, 6) looked up by byte permutes. Bit 3 is the sign: a permute whose selector
// nibble has bit 3 set replicates the source byte's top bit, so the raw nibbles
// as selectors over bytes of 0x80 give 0xFF for a negative element and 0x80 for a
// positive one - the four sign bits of a half word cost three instructions.
__device__ __forceinline__ void mx_decode8(uint32_t w, uint32_t scale2, uint32_t* out) {
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint32_t x = h == 0 ? w : w >> 16;
    const uint32_t sel = x & 0x7777u;
    const uint32_t neg = prmt(0x80808080u, 0x80808080u, x) << 7;        // bit 7 of a byte: negative
    const uint32_t hi = prmt(0x3F3F3F00u, 0x40404040u, sel) | (neg & 0x80808080u);
    const uint32_t lo = prmt(0xC0800000u, 0xC0804000u, sel);
    out[2 * h] = mx_mul_bf16x2(prmt(lo, hi, 0x5140), scale2);
    out[2 * h + 1] = mx_mul_bf16x2(prmt(lo, hi, 0x7362), scale2);
  }
}

__device__ __forceinline__ float mx_gate(float g, int act) {
  if (act == 1) return g / (1.f + __expf(-g));
  const float u = 0.7978845608028654f * (g + 0.044715f * g * g * g);
  return 0.5f * g * (1.f + tanhf(u));
}

__global__ void __launch_bounds__(kMxThreads, 1) moe_gemm_mxfp4_umma_kernel(
    const MxArgs p, const __grid_constant__ CUtensorMap map_a,
    const __grid_constant__ CUtensorMap map_w) {
  pdl_enter();
  using L = MxLayout;
  constexpr int S = kMxStages;
  extern __shared__ uint8_t raw_smem[];
  uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) &
                                             ~uintptr_t(1023));
  __shared__ __align__(8) uint64_t full_bar[S], bready_bar[S], done_bar[S], tfull_bar, tempty_bar[2], drain_bar;
  __shared__ int s_unit[kMxMaxMBlocks];   // first m-block | (m-blocks in the unit << 16)
  __shared__ int s_units;
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int s_abort;
  __shared__ int s_expert[kMxMaxMBlocks];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int armed = 0;   // producer thread: stages it handed to the TMA (read at teardown)
  const bool gate = p.gate_act != 0;
  const int half_n = p.N / 2;
  const int nkb = p.K / kMxKB;
  const int m_blocks = *p.num_post / kMxTok;
  const int tile_rows = gate ? kMxCols / 2 : kMxCols;
  for (int i = tid; i < m_blocks && i < kMxMaxMBlocks; i += kMxThreads) {
    const int e = p.expert_ids[i];
    s_expert[i] = e < p.experts ? e : -1;   // ids past the weight tensor skip their m-block
  }
  __syncthreads();
  if (tid == 0) {
    // units: pairs of consecutive m-blocks of one expert, else single m-blocks. The
    // pairs come first in the list: items are dealt to the CTAs in a fixed stride, and
    // a pair costs twice a single, so this order keeps the CTAs' sums within one single
    // of each other instead of leaving the balance to chance.
    int n = 0;
    for (int want = 2; want >= 1; --want)
      for (int i = 0; i < m_blocks;) {
        const int e = s_expert[i];
        if (e < 0) { ++i; continue; }
        const int cnt = (i + 1 < m_blocks && s_expert[i + 1] == e) ? 2 : 1;
        if (cnt == want) s_unit[n++] = i | (cnt << 16);
        i += cnt;
      }
    s_units = n;
  }
  if (tid == 0) {
    for (int i = 0; i < S; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&bready_bar[i], kMxTransformWarps);
      mbar_init(&done_bar[i], 1);
    }
    mbar_init(&tfull_bar, 1);
    mbar_init(&drain_bar, 1);
    for (int i = 0; i < 2; ++i) mbar_init(&tempty_bar[i], kMxEpilogueWarps);
    s_abort = 0;
    fence_mbar_init();
  }
  if (warp == 1) tmem_alloc(&tmem_slot, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_slot;
  const uint32_t ring_s = smem_u32(ring);
  const int total_items = s_units * p.n_tiles;

  if (warp == 0) {
    // ------------------------------------------------------------- producer
    if (lane == 0) {
      tma::prefetch_map(&map_a);
      tma::prefetch_map(&map_w);
      int t = 0;
      bool dead = false;
      for (int item = blockIdx.x; item < total_items && !dead; item += gridDim.x) {
        const int unit = s_unit[item / p.n_tiles], nt = item % p.n_tiles;
        const int mb = unit & 0xffff, cnt = unit >> 16;
        const int expert = s_expert[mb];
        for (int kb = 0; kb < nkb; ++kb, ++t) {
          const int s = t % S;
          if (!mbar_wait(&done_bar[s], ((t / S) & 1) ^ 1) || s_abort) {
            dead = true;
            break;
          }
          const uint32_t st = ring_s + s * L::kStageBytes;
          tma::mbar_expect_tx(&full_bar[s], cnt * L::kABytes + L::kRawBytes);
          tma::load_2d(st, &map_a, kb * kMxKB * 2, mb * kMxTok, &full_bar[s]);
          if (cnt == 2)
            tma::load_2d(st + L::kABytes, &map_a, kb * kMxKB * 2, (mb + 1) * kMxTok, &full_bar[s]);
          tma::load_4d(st + 2 * L::kABytes, &map_w, kb * (kMxKB / 2), 0, nt * tile_rows, expert,
                       &full_bar[s]);
        }
      }
      armed = t;
      if (dead) atomicExch(p.status, 1), s_abort = 1;
    }
  } else if (warp == 1) {
    // --------------------------------------------------------------- issuer
    if (lane == 0) {
      const uint32_t idesc = instr_desc(D_F32, 1, 1, kMxTok, kMxCols);   // bf16 x bf16 -> f32
      const uint32_t lo0 = smem_desc_lo(ring_s);
      int t = 0, li = 0;
      bool dead = false;
      for (int item = blockIdx.x; item < total_items && !dead; item += gridDim.x, ++li) {
        const int cnt = s_unit[item / p.n_tiles] >> 16;
        // both accumulators belong to this item: the epilogue must have drained them
        if (!mbar_wait(&tempty_bar[0], (li & 1) ^ 1) || !mbar_wait(&tempty_bar[1], (li & 1) ^ 1)) {
          dead = true;
          break;
        }
        for (int kb = 0; kb < nkb; ++kb, ++t) {
          const int s = t % S;
          if (!mbar_wait(&bready_bar[s], (t / S) & 1) || s_abort) {   // tokens landed, weights decoded
            dead = true;
            break;
          }
          tc_fence_after_sync();
          const uint32_t b_lo = lo0 + ((S * L::kStageBytes + (t % kMxDecoded) * L::kBBytes) >> 4);
          for (int h = 0; h < cnt; ++h) {             // the unit's m-blocks share the decoded tile
            const uint32_t a_lo = lo0 + ((s * L::kStageBytes + h * L::kABytes) >> 4);
            const uint32_t d = tmem + h * kMxCols;
            if (kb == 0) mma_ss_lo<KIND_F16, false>(d, a_lo, b_lo, idesc);
            else mma_ss_lo<KIND_F16, true>(d, a_lo, b_lo, idesc);
            mma_ss_lo<KIND_F16, true>(d, a_lo + 2, b_lo + 2, idesc);
            mma_ss_lo<KIND_F16, true>(d, a_lo + 4, b_lo + 4, idesc);
            mma_ss_lo<KIND_F16, true>(d, a_lo + 6, b_lo + 6, idesc);
          }
          mma_commit(&done_bar[s]);
        }
        if (!dead) mma_commit(&tfull_bar);
      }
      if (dead) atomicExch(p.status, 1), s_abort = 1;
    }
  } else if (warp >= 4 && warp < 4 + kMxTransformWarps) {
    // ------------------------------------------------------------ transform
    const int r = (tid - 128) >> 1;                   // row of the tile, 0..255
    const int th = (tid - 128) & 1;                   // which 32 of the K block's 64 elements
    int t = 0;
    bool dead = false;
    for (int item = blockIdx.x; item < total_items && !dead; item += gridDim.x) {
      const int nt = item % p.n_tiles;
      const int expert = s_expert[s_unit[item / p.n_tiles] & 0xffff];
      // a ragged last tile: rows past the matrix arrive as zeros (TMA) and take scale 0
      const int orow = nt * tile_rows + (gate ? (r >> 1) : r);
      const bool row_ok = orow < (gate ? half_n : p.N);
      const int wrow = gate && (r & 1) ? half_n + orow : orow;
      const uint8_t* sc = p.scales + int64_t(expert) * p.s_se + int64_t(row_ok ? wrow : 0) * p.s_sn + th;
      uint32_t sc_next = row_ok ? uint32_t(sc[0]) : 0u;
      for (int kb = 0; kb < nkb && !dead; ++kb, ++t) {
        const int s = t % S;
        const uint32_t scb = sc_next;               // the scale byte of this thread's group
        if (kb + 1 < nkb && row_ok) sc_next = uint32_t(sc[2 * kb + 2]);
        bool ok = mbar_wait(&full_bar[s], (t / S) & 1);
        // the decoded tile t % 2 was last read by the MMAs of K block t - 2
        if (t >= kMxDecoded) {
          const int u = t - kMxDecoded;
          ok = mbar_wait(&done_bar[u % S], (u / S) & 1) && ok;
        }
        if (__any_sync(0xffffffffu, !ok || s_abort != 0)) {
          dead = true;
          break;
        }
        const uint8_t* st = ring + s * L::kStageBytes;
        const uint4 x = *reinterpret_cast<const uint4*>(st + 2 * L::kABytes + r * (kMxKB / 2) + th * 16);
        uint8_t* dst = ring + S * L::kStageBytes + (t % kMxDecoded) * L::kBBytes;
        const uint32_t sb = scb << 7;
        const uint32_t s2 = sb | (sb << 16);
        const uint32_t ws[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint32_t o[4];
          mx_decode8(ws[i], s2, o);
          const int chunk = 4 * th + i;              // 8 elements = 16 bytes
          *reinterpret_cast<uint4*>(dst + r * 128 + ((chunk ^ (r & 7)) << 4)) =
              make_uint4(o[0], o[1], o[2], o[3]);
        }
        fence_proxy_async();                          // generic-proxy stores -> the MMA's async proxy
        __syncwarp();
        if (lane == 0) mbar_arrive(&bready_bar[s]);
      }
    }
    if (dead) atomicExch(p.status, 1), s_abort = 1;
  } else if (warp >= 4 + kMxTransformWarps) {
    // ------------------------------------------------------------- epilogue
    const int tok = (warp & 3) * 32 + lane;
    const uint32_t lane_base = uint32_t((warp & 3) * 32) << 16;
    int li = 0;
    bool dead = false;
    for (int item = blockIdx.x; item < total_items && !dead; item += gridDim.x, ++li) {
      const int unit = s_unit[item / p.n_tiles], nt = item % p.n_tiles;
      const int mb0 = unit & 0xffff, cnt = unit >> 16;
      int sid[2], crow[2];
      float tw[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int64_t raw = h < cnt ? p.sorted_ids[(mb0 + h) * kMxTok + tok] : -1;
        sid[h] = (raw >= 0 && raw < p.num_valid) ? int(raw) : -1;
        tw[h] = (sid[h] >= 0 && p.topk_w != nullptr) ? p.topk_w[sid[h]] : 1.f;
        crow[h] = h < cnt ? (p.c_sorted ? (mb0 + h) * kMxTok + tok : sid[h]) : -1;
      }
      const bool ok = mbar_wait(&tfull_bar, li & 1);
      if (__any_sync(0xffffffffu, !ok || s_abort != 0)) {
        dead = true;
        break;
      }
      tc_fence_after_sync();
#pragma unroll 1
      for (int h = 0; h < 2; ++h) {
        __nv_bfloat16* cptr = p.c + int64_t(crow[h] < 0 ? 0 : crow[h]) * p.c_stride + nt * tile_rows;
        if (h >= cnt) {            // a unit of one: the second accumulator was not used
          __syncwarp();
          if (lane == 0) mbar_arrive(&tempty_bar[h]);
          continue;
        }
#pragma unroll 1
        for (int c0 = 0; c0 < kMxCols; c0 += 32) {
          uint32_t rr[32];
          tmem_ld_32x32(tmem + lane_base + h * kMxCols + c0, rr);
          tmem_ld_wait();
          if (c0 + 32 == kMxCols) {
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tempty_bar[h]);
          }
          // output columns of this chunk: 16 under the gate, else 32; past the matrix: nothing
          const int out_col = nt * tile_rows + (gate ? c0 / 2 : c0);
          if (crow[h] < 0 || out_col >= (gate ? half_n : p.N)) continue;
          if (gate) {
            uint32_t o[8];
#pragma unroll
            for (int i = 0; i < 16; i += 2) {
              const float v0 = mx_gate(__uint_as_float(rr[2 * i]), p.gate_act) * __uint_as_float(rr[2 * i + 1]);
              const float v1 = mx_gate(__uint_as_float(rr[2 * i + 2]), p.gate_act) * __uint_as_float(rr[2 * i + 3]);
              o[i >> 1] = pack_bf16x2(v0, v1);
            }
            uint4* dstp = reinterpret_cast<uint4*>(cptr + c0 / 2);
            dstp[0] = make_uint4(o[0], o[1], o[2], o[3]);
            dstp[1] = make_uint4(o[4], o[5], o[6], o[7]);
          } else {
            uint32_t o[16];
#pragma unroll
            for (int i = 0; i < 32; i += 2)
              o[i >> 1] = pack_bf16x2(__uint_as_float(rr[i]) * tw[h], __uint_as_float(rr[i + 1]) * tw[h]);
            uint4* dstp = reinterpret_cast<uint4*>(cptr + c0);
#pragma unroll
            for (int i = 0; i < 4; ++i) dstp[i] = make_uint4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
          }
        }
      }
    }
    if (dead) atomicExch(p.status, 1), s_abort = 1;
  }

  tc_fence_before_sync();
  __syncthreads();
  if (s_abort) {   // wait for the copies and MMAs still in flight before TMEM goes
    if (tid == 0) drain_armed_loads(full_bar, S, armed);
    if (warp == 1 && lane == 0) drain_issued_mmas(&drain_bar);
    tc_fence_before_sync();
    __syncthreads();
  }
  if (warp == 1) tmem_dealloc(tmem, 512);
}

// bf16 rows into sorted order by scatter: token row t goes to the sorted
// positions of its top_k slots; padding slots below *num_post get zeros.
__global__ void __launch_bounds__(256) permute_rows_kernel(
    const uint4* __restrict__ x, int64_t x_stride16, uint4* __restrict__ y, int64_t y_stride16,
    int64_t tokens, int chunks, int top_k, const int32_t* __restrict__ slot_pos,
    const int32_t* __restrict__ sorted_ids, const int32_t* __restrict__ num_post, int64_t rows_cap,
    int64_t num_valid) {
  pdl_enter();
  const int64_t idx = int64_t(blockIdx.x) * 256 + threadIdx.x;
  const int64_t row = idx / chunks;
  const int ch = int(idx % chunks);
  if (row < tokens) {
    const uint4 v = x[row * x_stride16 + ch];
    for (int j = 0; j < top_k; ++j) {
      const int pos = slot_pos[row * top_k + j];
      if (pos >= 0 && pos < rows_cap) y[int64_t(pos) * y_stride16 + ch] = v;
    }
    return;
  }
  const int64_t r = row - tokens;
  if (r >= rows_cap || r >= *num_post) return;
  const int64_t sid = sorted_ids[r];
  if (sid >= 0 && sid < num_valid) return;
  y[r * y_stride16 + ch] = make_uint4(0u, 0u, 0u, 0u);
}

}  // namespace
}  // namespace strix

using namespace strix;

extern "C" int strix_moe_permute_bf16(const void* x, void* y, const int32_t* slot_pos,
                                      const int32_t* sorted_ids, const int32_t* num_post_padded,
                                      int64_t tokens, int64_t rows, int64_t k, int64_t top_k,
                                      int64_t x_stride, int64_t y_stride, strix_stream_t stream) {
  STRIX_CHECK(slot_pos != nullptr && sorted_ids != nullptr && num_post_padded != nullptr,
              "slot_pos, sorted_ids and num_post_padded must not be NULL");
  STRIX_CHECK(tokens >= 0 && rows >= 0 && k > 0 && k % 8 == 0 && top_k >= 1, "K must be a multiple of 8");
  STRIX_CHECK(x_stride % 8 == 0 && y_stride % 8 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 &&
                  reinterpret_cast<uintptr_t>(y) % 16 == 0, "16-byte aligned rows required");
  if (tokens + rows == 0) return STRIX_OK;
  const int chunks = int(k / 8);
  const int64_t threads = (tokens + rows) * chunks;
  launch_chain(permute_rows_kernel, unsigned((threads + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream), 
      static_cast<const uint4*>(x), x_stride / 8, static_cast<uint4*>(y), y_stride / 8, tokens, chunks,
      int(top_k), slot_pos, sorted_ids, num_post_padded, rows, tokens * top_k);
  return launch_status("moe_permute_bf16");
}

extern "C" int strix_moe_gemm_mxfp4_sorted_covers(int64_t n, int64_t k, int64_t block_m, int gate_act) {
  const int64_t out_rows = gate_act ? n / 2 : n;
  const int tile = gate_act ? kMxCols / 2 : kMxCols;
  (void)tile;   // a ragged last tile is allowed: its rows are zero-filled and its columns masked
  return block_m == kMxTok && n > 0 && n % 2 == 0 && out_rows % 32 == 0 && k > 0 && k % kMxKB == 0;
}

extern "C" int strix_moe_gemm_mxfp4_sorted(
    void* c, const void* a, const void* w, const void* scales, const int32_t* sorted_ids,
    const int32_t* expert_ids, const int32_t* num_post_padded, const float* topk_weights,
    int64_t num_valid, int64_t num_experts, int64_t n, int64_t k, int64_t a_stride, int64_t c_stride,
    int64_t w_stride_e, int64_t w_stride_n, int64_t s_stride_e, int64_t s_stride_n, int64_t sorted_len,
    int64_t block_m, int gate_act, int c_sorted, strix_stream_t stream) {
  STRIX_CHECK(gate_act >= 0 && gate_act <= 2, "activation must be none, silu or gelu_tanh");
  STRIX_CHECK(num_experts >= 1 && num_experts <= (int64_t(1) << 24), "num_experts out of range");
  STRIX_CHECK(strix_moe_gemm_mxfp4_sorted_covers(n, k, block_m, gate_act),
              "geometry not covered: block_m 128, K %% 64, output width %% 32");
  STRIX_CHECK(sorted_len % block_m == 0 && sorted_len / block_m <= kMxMaxMBlocks,
              "sorted_len must be whole m-blocks, at most %d of them", kMxMaxMBlocks);
  STRIX_CHECK(gate_act == 0 || topk_weights == nullptr, "the fused gate takes no routing weights");
  STRIX_CHECK(w_stride_n % 16 == 0 && w_stride_e % 16 == 0 && (a_stride * 2) % 16 == 0 &&
                  c_stride % 8 == 0 && reinterpret_cast<uintptr_t>(w) % 16 == 0 &&
                  reinterpret_cast<uintptr_t>(a) % 16 == 0 && reinterpret_cast<uintptr_t>(c) % 16 == 0,
              "16-byte aligned rows required");
  if (sorted_len == 0 || num_valid == 0) return STRIX_OK;
  const int64_t out_rows = gate_act ? n / 2 : n;
  const int tile = gate_act ? kMxCols / 2 : kMxCols;
  MxArgs p;
  p.c = static_cast<__nv_bfloat16*>(c), p.scales = static_cast<const uint8_t*>(scales);
  p.sorted_ids = sorted_ids, p.expert_ids = expert_ids, p.num_post = num_post_padded;
  p.topk_w = topk_weights, p.status = umma_status_ptr();
  STRIX_CHECK(p.status != nullptr, "status word unavailable");
  p.num_valid = num_valid, p.c_stride = c_stride, p.s_se = s_stride_e, p.s_sn = s_stride_n;
  p.K = int(k), p.N = int(n), p.n_tiles = int((out_rows + tile - 1) / tile), p.gate_act = gate_act;
  p.c_sorted = c_sorted, p.experts = int(num_experts);
  // activations: bytes [sorted rows, 2K], boxes of 128 rows x 128 bytes, swizzled
  CUtensorMap map_a, map_w;
  STRIX_CHECK(tma::make_map_u8(&map_a, a, uint64_t(sorted_len), uint64_t(2 * k), uint64_t(2 * a_stride), kMxTok),
              "tensor map encoding failed (activations)");
  // packed weights: bytes (k / 2, half, row, expert), boxes of 32 bytes x halves x rows, not swizzled
  const uint64_t halves = gate_act ? 2 : 1, rows = uint64_t(out_rows);
  const uint64_t dims[4] = {uint64_t(k / 2), halves, rows, uint64_t(num_experts)};
  const uint64_t strides[3] = {uint64_t(w_stride_n) * rows, uint64_t(w_stride_n), uint64_t(w_stride_e)};
  const uint32_t box[4] = {kMxKB / 2, uint32_t(halves), uint32_t(tile), 1};
  STRIX_CHECK(tma::make_map_u8_nd(&map_w, w, 4, dims, strides, box, /*swizzle128=*/false),
              "tensor map encoding failed (weights)");
  static bool done[64] = {};
  static int sms[64] = {};
  int dev = 0;
  STRIX_CUDA(cudaGetDevice(&dev));
  STRIX_CHECK(dev >= 0 && dev < 64, "device index %d out of range", dev);
  if (!done[dev]) {
    STRIX_CUDA(cudaFuncSetAttribute(moe_gemm_mxfp4_umma_kernel,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, MxLayout::kSmem));
    STRIX_CUDA(cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev));
    done[dev] = true;
  }
  launch_chain(moe_gemm_mxfp4_umma_kernel, sms[dev], kMxThreads, MxLayout::kSmem, static_cast<cudaStream_t>(stream), 
      p, map_a, map_w);
  return launch_status("moe_gemm_mxfp4_umma");
}
