// Grouped expert GEMM for FP8 W8A8 experts on the Blackwell tensor cores
// (tcgen05.mma kind::f8f6f4, accumulators in TMEM), for sm_100a.
//
// Same contract as moe_gemm.cu (moe_align_block_size layout, fused gate
// epilogue, routing weight on the down GEMM; csrc/moe/moe_gemm_w8a16.hip:76-404
// of the reference). What differs is the machine mapping:
//
//   * operands swap roles: a tile of 128 expert-weight rows is the MMA's A (M =
//     128) and the m-block's tokens are B (N = block_m, 16..128), so a ragged
//     expert with 16 tokens still fills the tensor core's M dimension and the
//     weights - the bytes that bound the layer at small token counts - are read
//     exactly once per m-block, straight from shared memory, with no widening;
//   * one persistent CTA per SM walks work items (m-block, 128-row weight tile)
//     in a fixed stride; three roles run decoupled through mbarriers:
//       producers (4 warps)  cp.async weight rows and gathered token rows into an
//                            8..5-stage ring, in the 128-byte-swizzled K-major
//                            layout the MMA descriptors expect;
//       issuer (1 thread)    four K=32 MMAs per 128-wide K block into one of the
//                            TMEM accumulator buffers, then tcgen05.commit to
//                            free the ring stage and to publish the buffer;
//       consumers (4 warps)  tcgen05.ld the K block's partial sums and fold them
//                            into fp32 registers with the block's weight scale
//                            times the token's activation scale (the scales are
//                            not powers of two, so they cannot ride the MMA);
//   * under the fused gate the tile's rows alternate gate row i / up row i, so
//     act(gate) * up is one lane shuffle in the epilogue;
//   * every mbarrier wait is bounded; on a timeout the CTA sets *status, stops
//     issuing, drains its copies, frees TMEM and returns.
#include <cstdlib>
#include <type_traits>

#include "umma.cuh"

namespace strix {
namespace {

using namespace umma;

constexpr int kProducerWarps = 4, kConsumerWarps = 4;
constexpr int kThreadsU = (kProducerWarps + kConsumerWarps + 1) * 32;  // + issuer warp
constexpr int kTileM = 128;   // weight rows per tile (TMEM lanes)
constexpr int kKBlock = 128;  // K bytes per pipeline step = the scale block
constexpr int kMaxMBlocks = 2048;  // m-blocks whose expert ids are cached in shared memory

struct UmmaMoeArgs {
  void* c;
  const uint8_t* a;        // e4m3 [rows, K]
  const uint8_t* w;        // e4m3 [E, N, K]
  const float* scales;     // block [E, N/128, K/128] or channel [E, N] fp32
  const float* sa;         // [rows, K/128]
  const int32_t* sorted_ids;
  const int32_t* expert_ids;
  const int32_t* num_post;
  const float* topk_w;
  int32_t* status;
  long long* prof;         // optional cycle counters of CTA 0 (tuning aid), or NULL
  int64_t num_valid;
  int64_t a_stride, c_stride, w_se, w_sn, s_se, s_sn, sa_stride;
  int top_k, K, N, block_m;
  int scale_kind;  // 1 channel, 2 block
  int gate_act;    // 0 none, 1 silu, 2 gelu_tanh
  int n_tiles;     // weight tiles per m-block
};

template <int NTOK>
struct UmmaLayout {
  static constexpr int kABytes = kTileM * kKBlock;      // 16 KB of weights
  static constexpr int kBBytes = NTOK * kKBlock;        // token rows
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = NTOK <= 32 ? 8 : NTOK <= 64 ? 7 : 5;
  // TMEM accumulator buffers: as many as fit (the issuer then runs that many K
  // blocks ahead of the consumers, which covers their per-item epilogue)
  static constexpr int kAccBufs = 512 / NTOK < 8 ? 512 / NTOK : 8;
  static constexpr int kTmemCols = NTOK * kAccBufs < 32 ? 32 : NTOK * kAccBufs;
  static constexpr int kMaxKBlocks = NTOK <= 64 ? 64 : 32;  // K <= 8192 (4096 at 128 tokens)
  static constexpr int kSaFloats = kMaxKBlocks * NTOK;      // one item's activation scales
  static constexpr int kMetaBytes = 2 * (kSaFloats * 4 + NTOK * 4);  // double-buffered per item
  static constexpr int kSmem = 1024 + kStages * kStageBytes + kMetaBytes + 1024;
};

__device__ __forceinline__ float gate_fn(float g, int act) {
  if (act == 1) return g / (1.f + __expf(-g));
  const float u = 0.7978845608028654f * (g + 0.044715f * g * g * g);
  return 0.5f * g * (1.f + tanhf(u));
}

// Row of the expert's weight matrix held by TMEM lane `lane` of tile `nt`.
__device__ __forceinline__ int tile_row(int nt, int lane, bool gate, int half_n) {
  if (!gate) return nt * kTileM + lane;
  const int i = nt * (kTileM / 2) + (lane >> 1);
  return (lane & 1) ? half_n + i : i;
}

template <int NTOK>
__global__ void __launch_bounds__(kThreadsU, 1) moe_gemm_umma_kernel(const UmmaMoeArgs p) {
  using L = UmmaLayout<NTOK>;
  constexpr int S = L::kStages, NB = L::kAccBufs;
  extern __shared__ uint8_t raw_smem[];
  uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) &
                                             ~uintptr_t(1023));
  // per-item metadata, double-buffered: activation scales [kb][NTOK] and the
  // tokens' slot ids (-1 = padding); written by the producers one item ahead
  float* s_sa = reinterpret_cast<float*>(ring + S * L::kStageBytes);      // [2][kSaFloats]
  int* s_sid = reinterpret_cast<int*>(s_sa + 2 * L::kSaFloats);           // [2][NTOK]
  __shared__ __align__(8) uint64_t full_bar[S], empty_bar[S], tfull_bar[NB], tempty_bar[NB];
  __shared__ __align__(8) uint64_t meta_empty_bar[2], meta_full_bar[2], landed_bar[S];
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const long long kernel_t0 = clock64();
  const bool gate = p.gate_act != 0;
  const int half_n = p.N / 2;
  const int nkb = p.K / kKBlock;
  const int m_blocks = *p.num_post / p.block_m;
  const int total_items = m_blocks * p.n_tiles;
  // expert of every m-block, once, so that no role pays a global-memory round
  // trip per work item for it
  __shared__ int s_expert[kMaxMBlocks];
  for (int i = tid; i < m_blocks && i < kMaxMBlocks; i += kThreadsU) s_expert[i] = p.expert_ids[i];

  if (tid == 0) {
    for (int i = 0; i < S; ++i) {
      mbar_init(&full_bar[i], kProducerWarps);       // one arrive per producer warp
      mbar_init(&empty_bar[i], 1);
      mbar_init(&landed_bar[i], kProducerWarps * 32);
    }
    for (int i = 0; i < NB; ++i) {
      mbar_init(&tfull_bar[i], 1);
      mbar_init(&tempty_bar[i], kConsumerWarps);
    }
    mbar_init(&meta_empty_bar[0], kConsumerWarps);
    mbar_init(&meta_empty_bar[1], kConsumerWarps);
    mbar_init(&meta_full_bar[0], kProducerWarps);
    mbar_init(&meta_full_bar[1], kProducerWarps);
    s_abort = 0;
    fence_mbar_init();
  }
  if (warp == kProducerWarps + kConsumerWarps) tmem_alloc(&tmem_slot, L::kTmemCols);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_slot;
  const uint32_t ring_s = smem_u32(ring);

  if (warp < kProducerWarps) {
    // ------------------------------------------------------------ producers
    // A non-blocking loop with two duties, so that neither can starve the other:
    //   issue    when the next ring stage is free (its MMAs retired), copy the next
    //            K block into it; the copies report to the stage's `landed`
    //            barrier by themselves (cp.async.mbarrier.arrive);
    //   publish  when the oldest unpublished stage has landed, make its bytes
    //            visible to the tensor core's async proxy and arrive on `full`.
    const int ch = tid & 7, r0 = tid >> 3;                    // chunk, first row (0..15)
    const uint32_t dst0 = uint32_t(r0 * 128 + ((ch ^ (r0 & 7)) << 4));  // rows r0 + 16 i: + 2048 i
    constexpr int NCB = NTOK * 8 / 128 > 0 ? NTOK * 8 / 128 : 1;
    // Slot ids of the rows this thread copies (and of token tid % NTOK for the
    // metadata) are fetched one item ahead: a global-memory round trip per item
    // on the producers' critical path would drain the ring between items.
    int pre_rows[NCB], pre_tok = -1;
    auto prefetch_ids = [&](int item) {
      const int mb = item / p.n_tiles;
#pragma unroll
      for (int i = 0; i < NCB; ++i) {
        const int r = r0 + 16 * i;
        pre_rows[i] = (item < total_items && r < NTOK && r < p.block_m)
                          ? p.sorted_ids[mb * p.block_m + r] : -1;
      }
      const int j = tid % NTOK;
      pre_tok = (item < total_items && j < p.block_m) ? p.sorted_ids[mb * p.block_m + j] : -1;
    };
    // next valid item at or after `item` (items of skipped m-blocks are passed over)
    auto next_valid = [&](int item) {
      while (item < total_items && s_expert[item / p.n_tiles] < 0) item += gridDim.x;
      return item;
    };

    int item = next_valid(blockIdx.x);   // item being issued
    prefetch_ids(item);
    int kb = nkb;                        // K block to issue next; nkb = "open the item first"
    int issued = 0, pub = 0, li = 0;     // steps issued / published, items opened
    const uint8_t* wsrc[8];
    const uint8_t* asrc[NCB];
    bool aok[NCB];
    bool dead = false;
    uint32_t idle = 0;
    while (!dead && (item < total_items || pub < issued)) {
      bool progressed = false;
      // ---- open the next item: pointers + metadata (needs a free metadata buffer)
      if (item < total_items && kb == nkb) {
        const int buf = li & 1;
        if (__all_sync(0xffffffffu, mbar_test(&meta_empty_bar[buf], ((li >> 1) & 1) ^ 1))) {
          const int mb = item / p.n_tiles, nt = item - mb * p.n_tiles;
          const int expert = s_expert[mb];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int row = tile_row(nt, r0 + 16 * i, gate, half_n);
            wsrc[i] = p.w + int64_t(expert) * p.w_se + int64_t(row) * p.w_sn + ch * 16;
          }
#pragma unroll
          for (int i = 0; i < NCB; ++i) {
            const int64_t sid = pre_rows[i];
            aok[i] = sid >= 0 && sid < p.num_valid;
            asrc[i] = p.a + (aok[i] ? sid / p.top_k : 0) * p.a_stride + ch * 16;
          }
          // metadata for the consumers; it rides the item's first copy group
          const int j = tid % NTOK;
          const int64_t sid = pre_tok;
          const bool ok = sid >= 0 && sid < p.num_valid;
          if (tid < NTOK) s_sid[buf * NTOK + j] = ok ? int(sid) : -1;
          const float* sap = p.sa + (ok ? sid / p.top_k : 0) * p.sa_stride;
          const uint32_t sa_dst = smem_u32(s_sa + buf * L::kSaFloats);
          for (int k2 = tid / NTOK; k2 < nkb; k2 += 128 / NTOK)
            cp_async_4_zfill(sa_dst + (k2 * NTOK + j) * 4, sap + k2, ok);
          prefetch_ids(next_valid(item + gridDim.x));
          kb = 0;
          ++li;
          progressed = true;
        }
      }
      // ---- issue one K block
      if (item < total_items && kb < nkb) {
        const int s = issued % S;
        if (__all_sync(0xffffffffu, mbar_test(&empty_bar[s], ((issued / S) & 1) ^ 1))) {
          const uint32_t st = ring_s + s * L::kStageBytes;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            cp_async_16(st + dst0 + 2048 * i, wsrc[i]);
            wsrc[i] += kKBlock;
          }
#pragma unroll
          for (int i = 0; i < NCB; ++i) {
            if (r0 + 16 * i < NTOK)
              cp_async_16_zfill(st + L::kABytes + dst0 + 2048 * i, asrc[i] + kb * kKBlock, aok[i]);
          }
          mbar_arrive_cp_async(&landed_bar[s]);   // fires when this thread's copies land
          ++issued;
          if (++kb == nkb) item = next_valid(item + gridDim.x);
          progressed = true;
        }
      }
      // ---- publish the oldest stage whose copies (all 128 threads') have landed
      if (pub < issued) {
        const int s = pub % S;
        if (__all_sync(0xffffffffu, mbar_test(&landed_bar[s], (pub / S) & 1))) {
          fence_proxy_async();     // each thread fences its own copies ...
          __syncwarp();            // ... then one lane arrives for the warp: 128
          if (lane == 0) {         // arrives on one shared word would serialise
            mbar_arrive(&full_bar[s]);
            // every item has nkb steps, so step u opens item u / nkb: its metadata landed too
            if (pub % nkb == 0) mbar_arrive(&meta_full_bar[(pub / nkb) & 1]);
          }
          ++pub;
          progressed = true;
        }
      }
      if (progressed) {
        idle = 0;
      } else {
        __nanosleep(200);   // leave the issue slots to the consumer warps
        // warp-uniform, like every other decision in this loop (it holds warp votes)
        if (__any_sync(0xffffffffu, ++idle > (kSpinLimit >> 4) || s_abort != 0)) dead = true;
      }
    }
    cp_async_wait<0>();
    if (dead) atomicExch(p.status, 1), s_abort = 1;
  } else if (warp == kProducerWarps + kConsumerWarps) {
    // --------------------------------------------------------------- issuer
    if (lane == 0) {
      const uint32_t idesc = instr_desc(D_F32, 0, 0, kTileM, NTOK);
      int t = 0;
      bool dead = false;
      for (int item = blockIdx.x; item < total_items && !dead; item += gridDim.x) {
        const int mb = item / p.n_tiles;
        if (s_expert[mb] < 0) continue;
        for (int kb = 0; kb < nkb; ++kb, ++t) {
          const int s = t % S, b = t % NB;
          const long long c0 = clock64();
          const bool ok_full = mbar_wait(&full_bar[s], (t / S) & 1);
          const long long c1 = clock64();
          const bool ok_acc = mbar_wait(&tempty_bar[b], ((t / NB) & 1) ^ 1);
          const long long c2 = clock64();
          if (p.prof != nullptr && blockIdx.x == 0) {
            p.prof[0] += c1 - c0;   // cycles waiting for data
            p.prof[1] += c2 - c1;   // cycles waiting for a free accumulator
            p.prof[2] += 1;         // steps
          }
          if (!ok_full || !ok_acc || s_abort) {
            dead = true;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa_addr = ring_s + s * L::kStageBytes, sb_addr = sa_addr + L::kABytes;
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4)
            mma_ss<KIND_F8F6F4>(tmem + b * NTOK, smem_desc_sw128(sa_addr, 32 * k4),
                                smem_desc_sw128(sb_addr, 32 * k4), idesc, k4 > 0 ? 1u : 0u);
          mma_commit(&empty_bar[s]);   // the stage may be refilled
          mma_commit(&tfull_bar[b]);   // the partial sums are ready
        }
      }
      if (dead) atomicExch(p.status, 1), s_abort = 1;
    }
  } else {
    // ------------------------------------------------------------ consumers
    const int ctid = tid - kProducerWarps * 32;      // 0..127 = TMEM lane = tile row
    const uint32_t lane_base = uint32_t((warp & 3) * 32) << 16;
    constexpr int CH = NTOK < 32 ? NTOK : 32;        // columns per tcgen05.ld
    int t = 0, li = 0;
    bool dead = false;
    for (int item = blockIdx.x; item < total_items && !dead; item += gridDim.x) {
      const int mb = item / p.n_tiles, nt = item - mb * p.n_tiles;
      const int expert = s_expert[mb];
      if (expert < 0) continue;
      // this row's scales: the loads are in flight while the item's data arrives
      const int row = tile_row(nt, ctid, gate, half_n);
      const float* swp = p.scales + int64_t(expert) * p.s_se + int64_t(row / 128) * p.s_sn;
      float sw_next = p.scale_kind == 2 ? swp[0] : 1.f;
      const float chs = p.scale_kind == 1 ? p.scales[int64_t(expert) * p.s_se + row] : 1.f;
      // the producers wrote this item's token ids and activation scales
      const int buf = li & 1;
      const long long m0 = clock64();
      const bool meta_ok = mbar_wait(&meta_full_bar[buf], (li >> 1) & 1);
      if (p.prof != nullptr && blockIdx.x == 0 && ctid == 0) p.prof[6] += clock64() - m0;
      if (__any_sync(0xffffffffu, !meta_ok) || s_abort) {
        dead = true;
        break;
      }
      const float* sa_item = s_sa + buf * L::kSaFloats;
      const int* sid_item = s_sid + buf * NTOK;
      float acc[NTOK];
#pragma unroll
      for (int j = 0; j < NTOK; ++j) acc[j] = 0.f;
      // The K blocks' partial sums are read as a stream of (step, chunk of CH
      // columns) units through two register buffers: the TMEM load (and, at a
      // step's first chunk, the wait for its MMAs) of the next unit is issued
      // before the multiply-adds of the current one, so neither latency sits
      // on this warp's critical path.
      constexpr int NCH = NTOK / CH;
      uint32_t R[2][CH];
      const int t0 = t;
      auto issue_ld = [&](int kb, int c, uint32_t (&r)[CH]) {
        const int ts = t0 + kb, b = ts % NB;
        if (c == 0) {
          const long long w0 = clock64();
          const bool ok = mbar_wait(&tfull_bar[b], (ts / NB) & 1);
          if (p.prof != nullptr && blockIdx.x == 0 && ctid == 0) p.prof[3] += clock64() - w0;
          if (__any_sync(0xffffffffu, !ok)) {   // warp-uniform: the epilogue shuffles
            dead = true;
            return;
          }
          tc_fence_after_sync();
        }
        if constexpr (CH == 32) tmem_ld_32x32(tmem + lane_base + b * NTOK + c * CH, r);
        else tmem_ld_32x16(tmem + lane_base + b * NTOK + c * CH, r);
      };
      auto landed = [&](int kb, int c) {   // after the wait for unit (kb, c)
        if (c == NCH - 1) {                // the step's last chunk: hand the buffer back
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tempty_bar[(t0 + kb) % NB]);
        }
      };
      issue_ld(0, 0, R[0]);
      if (!dead) {
        tmem_ld_wait();
        landed(0, 0);
      }
      for (int kb2 = 0; kb2 < nkb && !dead; kb2 += 2) {
        auto step = [&](auto par) {
          constexpr int PAR = decltype(par)::value;
          const int kb = kb2 + PAR;
          if (kb >= nkb || dead) return;
          const float sw = sw_next;
          if (p.scale_kind == 2 && kb + 1 < nkb) sw_next = swp[kb + 1];
          const float* sak = sa_item + kb * NTOK;
          auto chunk = [&](auto cc) {
            constexpr int C = decltype(cc)::value;
            constexpr int BUF = NCH == 1 ? PAR : (C & 1);
            if (dead) return;
            const bool last = C == NCH - 1;
            const int nkb_ = last ? kb + 1 : kb, nc = last ? 0 : C + 1;
            const bool more = nkb_ < nkb;
            if (more) issue_ld(nkb_, nc, R[BUF ^ 1]);
#pragma unroll
            for (int j = 0; j < CH; j += 4) {
              const float4 s4 = *reinterpret_cast<const float4*>(sak + C * CH + j);
              acc[C * CH + j] = fmaf(__uint_as_float(R[BUF][j]), sw * s4.x, acc[C * CH + j]);
              acc[C * CH + j + 1] = fmaf(__uint_as_float(R[BUF][j + 1]), sw * s4.y, acc[C * CH + j + 1]);
              acc[C * CH + j + 2] = fmaf(__uint_as_float(R[BUF][j + 2]), sw * s4.z, acc[C * CH + j + 2]);
              acc[C * CH + j + 3] = fmaf(__uint_as_float(R[BUF][j + 3]), sw * s4.w, acc[C * CH + j + 3]);
            }
            if (more && !dead) {
              const long long w0 = clock64();
              tmem_ld_wait();
              if (p.prof != nullptr && blockIdx.x == 0 && ctid == 0) p.prof[4] += clock64() - w0;
              landed(nkb_, nc);
            }
          };
          chunk(std::integral_constant<int, 0>{});
          if constexpr (NCH > 1) chunk(std::integral_constant<int, 1>{});
          if constexpr (NCH > 2) {
            chunk(std::integral_constant<int, 2>{});
            chunk(std::integral_constant<int, 3>{});
          }
        };
        step(std::integral_constant<int, 0>{});
        step(std::integral_constant<int, 1>{});
      }
      t = t0 + nkb;
      if (dead) break;

      // ---- epilogue of the item: this thread owns weight row `row`, all tokens
      const long long ep0 = clock64();
      if (gate) {
        __nv_bfloat16* cbase = static_cast<__nv_bfloat16*>(p.c) + nt * (kTileM / 2) + (ctid >> 1);
#pragma unroll
        for (int j = 0; j < NTOK; ++j) {
          const float v = acc[j] * chs;
          const float other = __shfl_xor_sync(0xffffffffu, v, 1);  // even lane: gate, odd: up
          const int sid = sid_item[j];
          if (sid >= 0 && (ctid & 1) == 0)
            cbase[int64_t(sid) * p.c_stride] = __float2bfloat16_rn(gate_fn(v, p.gate_act) * other);
        }
      } else {
        __nv_bfloat16* cbase = static_cast<__nv_bfloat16*>(p.c) + row;
        // routing weights first (independent loads in flight together), stores after
#pragma unroll
        for (int j = 0; j < NTOK; ++j) {
          const int sid = sid_item[j];
          const float tw = (sid >= 0 && p.topk_w) ? __ldg(p.topk_w + sid) : 1.f;
          acc[j] *= chs * tw;
        }
#pragma unroll
        for (int j = 0; j < NTOK; ++j) {
          const int sid = sid_item[j];
          if (sid >= 0) cbase[int64_t(sid) * p.c_stride] = __float2bfloat16_rn(acc[j]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&meta_empty_bar[buf]);   // the producers may reuse this buffer
      if (p.prof != nullptr && blockIdx.x == 0 && ctid == 0) p.prof[5] += clock64() - ep0;
      ++li;
    }
    if (dead) atomicExch(p.status, 1), s_abort = 1;
  }

  if (p.prof != nullptr && blockIdx.x == 0 && tid == 0) p.prof[7] += clock64() - kernel_t0;
  // ---- teardown: all roles meet, then the allocating warp frees TMEM
  tc_fence_before_sync();
  __syncthreads();
  if (warp == kProducerWarps + kConsumerWarps) tmem_dealloc(tmem, L::kTmemCols);
}

// Status word the kernels raise when a bounded wait runs out (0 = healthy).
__device__ int32_t g_umma_status = 0;
// Cycle counters of CTA 0, filled only while STRIX_UMMA_PROF is set: [0] issuer
// waiting for data, [1] issuer waiting for an accumulator, [2] steps, [3]
// consumer waiting for MMAs, [4] consumer waiting for TMEM loads, [5] consumer
// epilogues, [6] consumer waiting for metadata, [7] kernel cycles.
__device__ long long g_umma_prof[8] = {};

template <int NTOK>
int launch_umma(const UmmaMoeArgs& p, cudaStream_t st) {
  using L = UmmaLayout<NTOK>;
  auto kernel = moe_gemm_umma_kernel<NTOK>;
  static bool done[64] = {};
  static int sms[64] = {};
  int dev = 0;
  STRIX_CUDA(cudaGetDevice(&dev));
  STRIX_CHECK(dev >= 0 && dev < 64, "device index %d out of range", dev);
  if (!done[dev]) {
    STRIX_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kSmem));
    STRIX_CUDA(cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev));
    done[dev] = true;
  }
  kernel<<<sms[dev], kThreadsU, L::kSmem, st>>>(p);
  return launch_status("moe_gemm_umma");
}

}  // namespace

// Device address of the status word shared by every tcgen05 kernel of the library.
int32_t* umma_status_ptr() {
  void* addr = nullptr;
  return cudaGetSymbolAddress(&addr, g_umma_status) == cudaSuccess ? static_cast<int32_t*>(addr)
                                                                    : nullptr;
}

// Widest m-block the tcgen05 kernel takes (wider ones go to the streaming kernel).
int g_umma_max_block_m = [] {
  const char* e = getenv("STRIX_MOE_UMMA_MAX_BLOCK_M");
  return e ? atoi(e) : 32;
}();

// FP8 W8A8 grouped GEMM on tcgen05. Returns -1 when the geometry is not covered
// (the caller then takes the mma.sync weight-streaming kernel), else a status.
int moe_gemm_fp8_umma(void* c, const void* a, const void* w, const float* scales,
                      const float* act_scales, const int32_t* sorted_ids,
                      const int32_t* expert_ids, const int32_t* num_post, const float* topk_w,
                      int64_t num_valid, int64_t n, int64_t k, int64_t a_stride, int64_t c_stride,
                      int64_t w_se, int64_t w_sn, int64_t s_se, int64_t s_sn, int64_t sa_stride,
                      int64_t sorted_len, int64_t top_k, int64_t block_m, int scale_kind,
                      int scale_is_f32, int gate_act, cudaStream_t st) {
  static const bool disabled = getenv("STRIX_MOE_NO_UMMA") != nullptr;
  // Measured on B200 (256 and 4,096 tokens, 128 experts, top-8): with the fp32
  // promotion of every K block the consumer warps, not the tensor core, set the
  // pace; up to 32 tokens per m-block this kernel matches the mma.sync streaming
  // kernel, beyond that the streaming kernel is ahead, so wider blocks go there
  // unless STRIX_MOE_UMMA_MAX_BLOCK_M raises the limit.
  if (block_m > g_umma_max_block_m) return -1;
  const int64_t out_rows = gate_act ? n / 2 : n;
  const int tile_out = gate_act ? kTileM / 2 : kTileM;
  if (disabled || !scale_is_f32 || block_m < 16 || block_m > 128 || block_m % 16 != 0 ||
      out_rows % tile_out != 0 || k % kKBlock != 0 || k > (block_m > 64 ? 32 : 64) * kKBlock ||
      (scale_kind == 2 && gate_act && (n / 2) % 128 != 0) || sorted_len < block_m ||
      sorted_len / block_m > kMaxMBlocks)
    return -1;
  UmmaMoeArgs p;
  p.c = c, p.a = static_cast<const uint8_t*>(a), p.w = static_cast<const uint8_t*>(w);
  p.scales = scales, p.sa = act_scales;
  p.sorted_ids = sorted_ids, p.expert_ids = expert_ids, p.num_post = num_post, p.topk_w = topk_w;
  void* status_addr = nullptr;
  STRIX_CUDA(cudaGetSymbolAddress(&status_addr, g_umma_status));
  p.status = static_cast<int32_t*>(status_addr);
  static const bool profiling = getenv("STRIX_UMMA_PROF") != nullptr;
  p.prof = nullptr;
  if (profiling) {
    void* prof_addr = nullptr;
    STRIX_CUDA(cudaGetSymbolAddress(&prof_addr, g_umma_prof));
    p.prof = static_cast<long long*>(prof_addr);
  }
  p.num_valid = num_valid;
  p.a_stride = a_stride, p.c_stride = c_stride, p.w_se = w_se, p.w_sn = w_sn;
  p.s_se = s_se, p.s_sn = s_sn, p.sa_stride = sa_stride;
  p.top_k = int(top_k), p.K = int(k), p.N = int(n), p.block_m = int(block_m);
  p.scale_kind = scale_kind, p.gate_act = gate_act;
  p.n_tiles = int(out_rows / tile_out);
  if (block_m <= 16) return launch_umma<16>(p, st);
  if (block_m <= 32) return launch_umma<32>(p, st);
  if (block_m <= 64) return launch_umma<64>(p, st);
  return launch_umma<128>(p, st);
}

}  // namespace strix

// 0 while every tcgen05 kernel launched so far met its waits; 1 after one of
// them gave up on a bounded wait (its output is then incomplete). Synchronises
// the device; meant for tests and debugging.
extern "C" int strix_moe_set_umma_max_block_m(int block_m) {
  STRIX_CHECK(block_m >= 0 && block_m <= 128, "block_m limit must be in 0..128");
  strix::g_umma_max_block_m = block_m;
  return STRIX_OK;
}

extern "C" int strix_umma_prof(int64_t* host_out8, int reset) {
  STRIX_CHECK(host_out8 != nullptr, "host_out8 must not be NULL");
  STRIX_CUDA(cudaMemcpyFromSymbol(host_out8, strix::g_umma_prof, 8 * sizeof(long long)));
  if (reset) {
    const long long zeros[8] = {};
    STRIX_CUDA(cudaMemcpyToSymbol(strix::g_umma_prof, zeros, sizeof(zeros)));
  }
  return STRIX_OK;
}

extern "C" int strix_umma_status(int32_t* host_out) {
  STRIX_CHECK(host_out != nullptr, "host_out must not be NULL");
  STRIX_CUDA(cudaMemcpyFromSymbol(host_out, strix::g_umma_status, sizeof(int32_t)));
  return STRIX_OK;
}
