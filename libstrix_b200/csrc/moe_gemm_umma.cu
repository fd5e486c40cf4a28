// Grouped expert GEMM for FP8 W8A8 experts on the Blackwell tensor cores
// (tcgen05.mma kind::f8f6f4, accumulators in TMEM), for sm_100a.
//
// Same arithmetic as the FP8 W8A8 form of moe_gemm.cu (moe_align_block_size
// layout, fused gate epilogue, routing weight on the down GEMM;
// csrc/moe/moe_gemm_w8a16.hip:76-404 of the reference), but over activations
// that are already laid out in sorted order: row p of `a` (and of its scales)
// belongs to sorted position p, so an m-block's tokens are block_m consecutive
// rows and one TMA box fetches them. The quantiser writes that layout
// (strix_moe_act_quant_fp8_scatter / _sorted), the gate-up GEMM can write its
// output in it too, and the down GEMM scatters to slot order for the combine.
// Two kernels: this one for m-blocks of 16..64 tokens (the weight stream sets the
// pace), and the wide-tile kernel further down for m-blocks of 128 tokens. What
// differs from moe_gemm.cu is the machine mapping:
//
//   * operands swap roles: a tile of 128 expert-weight rows is the MMA's A (M =
//     128) and the m-block's tokens are B (N = block_m, 16..128), so a ragged
//     expert with 16 tokens still fills the tensor core's M dimension and the
//     weights - the bytes that bound the layer at small token counts - are read
//     exactly once per m-block, straight from shared memory, with no widening;
//   * one persistent CTA per SM walks work items (m-block, 128-row weight tile)
//     in a fixed stride; three roles run decoupled through mbarriers:
//       producer (1 thread)  two TMA boxes per K block - 128 weight rows (a 4-d
//                            box, which also interleaves the gate and up rows)
//                            and the m-block's token rows - into a ring of up to
//                            12 stages (what shared memory and TMEM leave) in
//                            the 128-byte-swizzled K-major layout the MMA
//                            descriptors expect; they complete the stage's
//                            barrier by byte count;
//       metadata (1 warp)    a few items ahead: the tokens' slot ids, routing
//                            weights and activation scales and the tile's weight
//                            block scales, into shared memory;
//       issuers (2 threads, alternate K blocks) four K=32 MMAs per 128-wide K block into the ring
//                            position's TMEM accumulator, then ONE tcgen05.commit
//                            that frees the stage and publishes the sums;
//       consumers (8-16 warps, 2-4 per TMEM lane quadrant, each a share of the
//                            tokens) tcgen05.ld the K block's partial sums and fold them
//                            into fp32 registers with the block's weight scale
//                            times the token's activation scale (the scales are
//                            not powers of two, so they cannot ride the MMA);
//   * under the fused gate the tile's rows alternate gate row i / up row i, so
//     act(gate) * up is one lane shuffle in the epilogue;
//   * every mbarrier wait is bounded; on a timeout the CTA sets *status, stops
//     issuing, waits (bounded) for the copies and MMAs it has in flight, frees
//     TMEM and returns.
#include <cstdlib>
#include <type_traits>

#include "tma.cuh"

namespace strix {
namespace {

using namespace umma;

// warps 0..3: producer, metadata, issuer, spare; then G consumer warps per TMEM
// lane quadrant, each folding 1/G of the m-block's tokens (8 at least)
constexpr int kProducerWarps = 4;
// (measured: 4 groups pay at 64 tokens; at 32 the extra warps only add barrier traffic,
// at 128 they push the kernel into register spills)
constexpr int column_groups(int ntok) { return ntok == 64 ? 4 : 2; }
constexpr int umma_threads(int ntok) { return (kProducerWarps + 4 * column_groups(ntok)) * 32; }
constexpr int kIssuerWarp = 2;
constexpr int kTileM = 128;   // weight rows per tile (TMEM lanes)
constexpr int kKBlock = 128;  // K bytes per pipeline step = the scale block
constexpr int kMaxMBlocks = 2048;  // m-blocks whose expert ids are cached in shared memory

struct UmmaMoeArgs {
  void* c;
  const float* scales;     // block [E, N/128, K/128] or channel [E, N] fp32
  const float* sa;         // [sorted rows, K/128]
  const int32_t* sorted_ids;
  const int32_t* expert_ids;
  const int32_t* num_post;
  const float* topk_w;
  int32_t* status;
  int64_t num_valid;
  int64_t c_stride, s_se, s_sn, sa_stride;
  int K, N, block_m;
  int experts;     // expert ids outside [0, experts) skip their m-block
  int scale_kind;  // 1 channel, 2 block
  int gate_act;    // 0 none, 1 silu, 2 gelu_tanh
  int n_tiles;     // weight tiles per m-block
  int c_sorted;    // 1: c rows are sorted positions, 0: slot ids (padding skipped)
  int prefetch;    // K blocks of weights requested into L2 ahead of the ring
};

// KBMAX bounds the K blocks of an item (16: K <= 2048, 64: K <= 8192); it sizes
// the per-item scale buffers, and what they leave goes to the ring.
template <int NTOK, int KBMAX>
struct UmmaLayout {
  static constexpr int kABytes = kTileM * kKBlock;      // 16 KB of weights
  static constexpr int kBBytes = NTOK * kKBlock;        // token rows
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kMaxKBlocks = KBMAX;
  static constexpr int kSaFloats = kMaxKBlocks * NTOK;      // one item's activation scales
  static constexpr int kSwFloats = kMaxKBlocks * 2;         // weight block scales (gate / up row block)
  // per item, kMetaBufs deep: activation scales, block scales, slot ids, routing weights
  static constexpr int kMetaBufs = NTOK <= 32 ? 4 : 2;
  static constexpr int kMetaBytes = kMetaBufs * (kSaFloats * 4 + kSwFloats * 4 + NTOK * 4 + NTOK * 4);
  // One ring position = a stage of operands + a TMEM accumulator: the MMAs of a
  // K block then finish with ONE tcgen05.commit, which both frees the stage for
  // the producer and publishes the partial sums to the consumers (a commit costs
  // the issuing thread about as much as three MMAs). The ring takes the shared
  // memory the metadata leaves (bytes in flight are what covers the memory
  // latency), up to the 512 TMEM columns.
  static constexpr int kBudget = 227 * 1024 - 10 * 1024 - 2048;   // static arrays, alignment slack
  static constexpr int kFit = (kBudget - kMetaBytes) / kStageBytes;
  static constexpr int kTmemFit = 512 / NTOK;
  static constexpr int kStages = kFit < kTmemFit ? (kFit < 12 ? kFit : 12) : (kTmemFit < 12 ? kTmemFit : 12);
  static constexpr int kAccBufs = kStages;
  static constexpr int kTmemUsed = NTOK * kAccBufs;   // the allocation is a power of two >= 32
  static constexpr int kTmemCols = kTmemUsed <= 32 ? 32 : kTmemUsed <= 64 ? 64 : kTmemUsed <= 128 ? 128 : kTmemUsed <= 256 ? 256 : 512;
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

template <int NTOK, int KBMAX>
__global__ void __launch_bounds__(umma_threads(NTOK), 1) moe_gemm_umma_kernel(const UmmaMoeArgs p,
                                                                    const __grid_constant__ CUtensorMap map_w,
                                                                    const __grid_constant__ CUtensorMap map_a) {
  pdl_enter();
  using L = UmmaLayout<NTOK, KBMAX>;
  constexpr int S = L::kStages, NB = L::kAccBufs;
  constexpr int kColumnGroups = column_groups(NTOK), kConsumerWarps = 4 * kColumnGroups;
  constexpr int kThreadsU = umma_threads(NTOK);
  extern __shared__ uint8_t raw_smem[];
  uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) &
                                             ~uintptr_t(1023));
  // per-item metadata, MB buffers deep: activation scales [kb][NTOK], weight
  // block scales, routing weights and the tokens' slot ids (-1 = padding);
  // written by the metadata warp ahead of the consumers
  constexpr int MB = L::kMetaBufs;
  float* s_sa = reinterpret_cast<float*>(ring + S * L::kStageBytes);      // [MB][kSaFloats]
  float* s_sw = s_sa + MB * L::kSaFloats;                                 // [MB][kb][gate|up]
  float* s_tw = s_sw + MB * L::kSwFloats;                                 // [MB][NTOK] routing weights
  int* s_sid = reinterpret_cast<int*>(s_tw + MB * NTOK);                  // [MB][NTOK]
  __shared__ __align__(8) uint64_t full_bar[S], empty_bar[S], tempty_bar[NB];
  __shared__ __align__(8) uint64_t meta_empty_bar[MB], meta_full_bar[MB], drain_bar[2];
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int armed = 0;   // producer thread: stages it handed to the TMA (read at teardown)
  const bool gate = p.gate_act != 0;
  const int half_n = p.N / 2;
  const int nkb = p.K / kKBlock;
  const int m_blocks = *p.num_post / p.block_m;
  const int total_items = m_blocks * p.n_tiles;
  // expert of every m-block, once, so that no role pays a global-memory round
  // trip per work item for it
  __shared__ int s_expert[kMaxMBlocks];
  for (int i = tid; i < m_blocks && i < kMaxMBlocks; i += kThreadsU) {
    const int e = p.expert_ids[i];
    s_expert[i] = e < p.experts ? e : -1;
  }

  if (tid == 0) {
    for (int i = 0; i < S; ++i) {
      mbar_init(&full_bar[i], 1);    // the producer's arrive, which announces the stage's bytes
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < NB; ++i) {
      mbar_init(&tempty_bar[i], kConsumerWarps);
    }
    for (int i = 0; i < MB; ++i) {
      mbar_init(&meta_empty_bar[i], kConsumerWarps);
      mbar_init(&meta_full_bar[i], 1);
    }
    mbar_init(&drain_bar[0], 1), mbar_init(&drain_bar[1], 1);
    s_abort = 0;
    fence_mbar_init();
  }
  if (warp == kIssuerWarp) tmem_alloc(&tmem_slot, L::kTmemCols);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_slot;
  const uint32_t ring_s = smem_u32(ring);

  // next valid item at or after `item` (items of skipped m-blocks are passed over)
  auto next_valid = [&](int item) {
    while (item < total_items && s_expert[item / p.n_tiles] < 0) item += gridDim.x;
    return item;
  };

  if (warp == 0) {
    // ------------------------------------------------------------- producer
    if (lane == 0) {
      tma::prefetch_map(&map_w);
      tma::prefetch_map(&map_a);
      int t = 0;
      bool dead = false;
      // A second cursor runs p.prefetch K blocks ahead of the loads and asks for
      // the weights in L2 only: the ring holds too few bytes to cover the memory
      // latency at full bandwidth, L2 has room for the rest.
      int pf_item = next_valid(blockIdx.x), pf_kb = 0;
      auto prefetch_one = [&]() {
        if (pf_item >= total_items) return;
        const int mb = pf_item / p.n_tiles, nt = pf_item - mb * p.n_tiles;
        tma::prefetch_l2_4d(&map_w, pf_kb * kKBlock, 0, nt * (gate ? kTileM / 2 : kTileM),
                            s_expert[mb]);
        if (++pf_kb == nkb) pf_kb = 0, pf_item = next_valid(pf_item + gridDim.x);
      };
      for (int i = 0; i < p.prefetch; ++i) prefetch_one();
      for (int item = next_valid(blockIdx.x); item < total_items && !dead;
           item = next_valid(item + gridDim.x)) {
        const int mb = item / p.n_tiles, nt = item - mb * p.n_tiles;
        const int expert = s_expert[mb];
        const int w_row = nt * (gate ? kTileM / 2 : kTileM);
        for (int kb = 0; kb < nkb; ++kb, ++t) {
          if (p.prefetch > 0) prefetch_one();
          const int s = t % S;
          if (!mbar_wait(&empty_bar[s], ((t / S) & 1) ^ 1) || s_abort) {   // its MMAs retired
            dead = true;
            break;
          }
          const uint32_t st = ring_s + s * L::kStageBytes;
          tma::mbar_expect_tx(&full_bar[s], L::kStageBytes);
          tma::load_4d(st, &map_w, kb * kKBlock, 0, w_row, expert, &full_bar[s]);
          tma::load_2d(st + L::kABytes, &map_a, kb * kKBlock, mb * NTOK, &full_bar[s]);
        }
      }
      armed = t;
      if (dead) atomicExch(p.status, 1), s_abort = 1;
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- metadata
    int pre_sid[NTOK / 32 > 0 ? NTOK / 32 : 1];
    constexpr int NR = NTOK / 32 > 0 ? NTOK / 32 : 1;
    auto fetch_ids = [&](int item) {
      const int mb = item / p.n_tiles;
#pragma unroll
      for (int i = 0; i < NR; ++i) {
        const int r = lane + 32 * i;
        pre_sid[i] = (item < total_items && r < NTOK && r < p.block_m)
                         ? p.sorted_ids[mb * p.block_m + r] : -1;
      }
    };
    int item = next_valid(blockIdx.x), li = 0;
    fetch_ids(item);
    bool dead = false;
    while (item < total_items && !dead) {
      const int buf = li % MB;
      const bool free_ok = mbar_wait(&meta_empty_bar[buf], ((li / MB) & 1) ^ 1);
      if (__any_sync(0xffffffffu, !free_ok || s_abort != 0)) {
        dead = true;
        break;
      }
      const int mb = item / p.n_tiles, nt = item - mb * p.n_tiles;
      const int expert = s_expert[mb];
      const uint32_t sa_dst = smem_u32(s_sa + buf * L::kSaFloats);
#pragma unroll
      for (int i = 0; i < NR; ++i) {
        const int j = lane + 32 * i;
        if (j >= NTOK) continue;
        const int64_t sid = pre_sid[i];
        const bool ok = sid >= 0 && sid < p.num_valid;
        s_sid[buf * NTOK + j] = ok ? int(sid) : -1;
        if (p.topk_w != nullptr)
          cp_async_4_zfill(smem_u32(s_tw + buf * NTOK + j), p.topk_w + (ok ? sid : 0), ok);
        else
          s_tw[buf * NTOK + j] = 1.f;
        const float* sap = p.sa + (int64_t(mb) * NTOK + j) * p.sa_stride;
        for (int k2 = 0; k2 < nkb; ++k2) cp_async_4(sa_dst + (k2 * NTOK + j) * 4, sap + k2);
      }
      // the tile's weight block scales, one per K block and per row block (the
      // gate rows and the up rows of a tile lie in two different 128-row blocks)
      if (p.scale_kind == 2) {
        for (int i = lane; i < 2 * nkb; i += 32) {
          const int k2 = i >> 1, par = i & 1;
          const int blk = gate ? ((par ? half_n : 0) + nt * (kTileM / 2)) / 128 : nt;
          cp_async_4(smem_u32(s_sw + buf * L::kSwFloats + i),
                     p.scales + int64_t(expert) * p.s_se + int64_t(blk) * p.s_sn + k2);
        }
      }
      item = next_valid(item + gridDim.x);
      fetch_ids(item);            // in flight while this item's copies land
      cp_async_commit();
      cp_async_wait<0>();
      __syncwarp();
      if (lane == 0) mbar_arrive(&meta_full_bar[buf]);
      ++li;
    }
    if (dead && lane == 0) atomicExch(p.status, 1), s_abort = 1;
  } else if (warp == kIssuerWarp || warp == kIssuerWarp + 1) {
    // -------------------------------------------------------------- issuers
    // Two issuing threads take the K blocks alternately (each block has its own
    // stage and accumulator, so they are independent): a block costs one thread
    // two waits, four MMAs and a commit in program order, which at full weight
    // bandwidth is most of a block's time (measured: 0.205 -> 0.188 ms per 256-token
    // layer, 0.186 -> 0.154 ms at 64 tokens).
    const int parity = warp - kIssuerWarp;
    if (lane == 0) {
      const uint32_t idesc = instr_desc(D_F32, 0, 0, kTileM, NTOK);
      const uint32_t a_lo0 = smem_desc_lo(ring_s);
      int t = 0;
      bool dead = false;
      for (int item = blockIdx.x; item < total_items && !dead; item += gridDim.x) {
        const int mb = item / p.n_tiles;
        if (s_expert[mb] < 0) continue;
        for (int kb = 0; kb < nkb; ++kb, ++t) {
          if ((t & 1) != parity) continue;
          const int s = t % S, b = t % NB;
          const bool ok_full = mbar_wait(&full_bar[s], (t / S) & 1);
          const bool ok_acc = mbar_wait(&tempty_bar[b], ((t / NB) & 1) ^ 1);
          if (!ok_full || !ok_acc || s_abort) {
            dead = true;
            break;
          }
          tc_fence_after_sync();
          // one add per operand and MMA: the issuing thread runs in order
          const uint32_t a_lo = a_lo0 + s * (L::kStageBytes >> 4), b_lo = a_lo + (L::kABytes >> 4);
          const uint32_t d = tmem + b * NTOK;
          mma_ss_lo<KIND_F8F6F4, false>(d, a_lo, b_lo, idesc);
          mma_ss_lo<KIND_F8F6F4, true>(d, a_lo + 2, b_lo + 2, idesc);
          mma_ss_lo<KIND_F8F6F4, true>(d, a_lo + 4, b_lo + 4, idesc);
          mma_ss_lo<KIND_F8F6F4, true>(d, a_lo + 6, b_lo + 6, idesc);
          mma_commit(&empty_bar[s]);   // the stage may be refilled, the partial sums are ready
        }
      }
      if (dead) atomicExch(p.status, 1), s_abort = 1;
    }
  } else if (warp >= kProducerWarps) {
    // ------------------------------------------------------------ consumers
    const int ctid = (warp & 3) * 32 + lane;         // 0..127 = TMEM lane = tile row
    const int cg = (warp - kProducerWarps) >> 2;     // which half of the tokens
    constexpr int NT2 = NTOK / kColumnGroups;        // tokens per consumer thread
    const uint32_t lane_base = uint32_t((warp & 3) * 32) << 16;
    constexpr int CH = NT2 < 32 ? NT2 : 32;          // columns per tcgen05.ld
    int t = 0, li = 0;
    bool dead = false;
    for (int item = blockIdx.x; item < total_items && !dead; item += gridDim.x) {
      const int mb = item / p.n_tiles, nt = item - mb * p.n_tiles;
      const int expert = s_expert[mb];
      if (expert < 0) continue;
      // this row's scales: the loads are in flight while the item's data arrives
      const int row = tile_row(nt, ctid, gate, half_n);
      const float chs = p.scale_kind == 1 ? p.scales[int64_t(expert) * p.s_se + row] : 1.f;
      // the producers wrote this item's token ids and activation scales
      const int buf = li % MB;
      const bool meta_ok = mbar_wait(&meta_full_bar[buf], (li / MB) & 1);
      if (__any_sync(0xffffffffu, !meta_ok) || s_abort) {
        dead = true;
        break;
      }
      const float* sa_item = s_sa + buf * L::kSaFloats;
      const int* sid_item = s_sid + buf * NTOK;
      const float* sw_item = s_sw + buf * L::kSwFloats + (gate ? (ctid & 1) : 0);
      const float* tw_item = s_tw + buf * NTOK;
      float acc[NT2];
#pragma unroll
      for (int j = 0; j < NT2; ++j) acc[j] = 0.f;
      // The K blocks' partial sums are read as a stream of (step, chunk of CH
      // columns) units through two register buffers: the TMEM load (and, at a
      // step's first chunk, the wait for its MMAs) of the next unit is issued
      // before the multiply-adds of the current one, so neither latency sits
      // on this warp's critical path.
      constexpr int NCH = NT2 / CH;
      uint32_t R[2][CH];
      const int t0 = t;
      auto issue_ld = [&](int kb, int c, uint32_t (&r)[CH]) {
        const int ts = t0 + kb, b = ts % NB;
        if (c == 0) {
          const bool ok = mbar_wait(&empty_bar[b], (ts / NB) & 1);
          if (__any_sync(0xffffffffu, !ok)) {   // warp-uniform: the epilogue shuffles
            dead = true;
            return;
          }
          tc_fence_after_sync();
        }
        const uint32_t src = tmem + lane_base + b * NTOK + cg * NT2 + c * CH;
        if constexpr (CH == 32) tmem_ld_32x32(src, r);
        else if constexpr (CH == 16) tmem_ld_32x16(src, r);
        else tmem_ld_32x8(src, r);
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
          const float sw = p.scale_kind == 2 ? sw_item[2 * kb] : 1.f;
          const float* sak = sa_item + kb * NTOK + cg * NT2;
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
              tmem_ld_wait();
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
      if (gate) {
        __nv_bfloat16* cbase = static_cast<__nv_bfloat16*>(p.c) + nt * (kTileM / 2) + (ctid >> 1);
#pragma unroll
        for (int j = 0; j < NT2; ++j) {
          const float v = acc[j] * chs;
          const float other = __shfl_xor_sync(0xffffffffu, v, 1);  // even lane: gate, odd: up
          const int crow = p.c_sorted ? mb * NTOK + cg * NT2 + j : sid_item[cg * NT2 + j];
          if (crow >= 0 && (ctid & 1) == 0)
            cbase[int64_t(crow) * p.c_stride] = __float2bfloat16_rn(gate_fn(v, p.gate_act) * other);
        }
      } else {
        __nv_bfloat16* cbase = static_cast<__nv_bfloat16*>(p.c) + row;
#pragma unroll
        for (int j = 0; j < NT2; ++j) {
          const int crow = p.c_sorted ? mb * NTOK + cg * NT2 + j : sid_item[cg * NT2 + j];
          if (crow >= 0)
            cbase[int64_t(crow) * p.c_stride] = __float2bfloat16_rn(acc[j] * chs * tw_item[cg * NT2 + j]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&meta_empty_bar[buf]);   // the producers may reuse this buffer
      ++li;
    }
    if (dead) atomicExch(p.status, 1), s_abort = 1;
  }

  // ---- teardown: all roles meet; after an abort the copies and MMAs still in
  // flight are waited for; then the allocating warp frees TMEM
  tc_fence_before_sync();
  __syncthreads();
  if (s_abort) {
    if (tid == 0) drain_armed_loads(full_bar, S, armed);
    if ((warp == kIssuerWarp || warp == kIssuerWarp + 1) && lane == 0)
      drain_issued_mmas(&drain_bar[warp - kIssuerWarp]);
    tc_fence_before_sync();
    __syncthreads();
  }
  if (warp == kIssuerWarp) tmem_dealloc(tmem, L::kTmemCols);
}

// ===================================================================== wide tiles
// The same GEMM for m-blocks of 128 tokens, where the tensor core, not the weight
// stream, sets the pace: the operands keep their natural roles - the m-block's
// 128 tokens are the MMA's A (M = 128, one TMEM lane per token) and 256 weight
// rows its B (N = 256; under the fused gate 128 gate rows interleaved with the
// 128 matching up rows) - so one MMA does 128 x 256 x 32 multiply-adds and a K
// block of 128 costs four of them. A consumer thread owns one token and 128 of
// the 256 columns: the fold needs one scalar per thread and K block (the
// token's activation scale times one of two weight-block scales), the gate
// pairs adjacent columns in the thread's own registers, and an output row is
// written as 128 or 256 contiguous bytes. Two 256-column accumulators fill TMEM;
// a ring position's single commit frees its operand stage and publishes the sums.
constexpr int kWideTok = 128, kWideCols = 256, kWideKbMax = 16;
constexpr int kWideConsumerWarps = 8;                       // 2 per TMEM lane quadrant
constexpr int kWideThreads = (kProducerWarps + kWideConsumerWarps) * 32;
struct WideLayout {
  static constexpr int kABytes = kWideTok * kKBlock;        // 16 KB of token rows
  static constexpr int kBBytes = kWideCols * kKBlock;       // 32 KB of weight rows
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = 4, kAccBufs = 2, kMetaBufs = 2;
  static constexpr int kSaFloats = kWideKbMax * kWideTok, kSwFloats = kWideKbMax * 2;
  static constexpr int kMetaBytes = kMetaBufs * (kSaFloats * 4 + kSwFloats * 4 + kWideTok * 8);
  static constexpr int kSmem = 1024 + kStages * kStageBytes + kMetaBytes + 256;
};

__global__ void __launch_bounds__(kWideThreads, 1) moe_gemm_umma_wide_kernel(
    const UmmaMoeArgs p, const __grid_constant__ CUtensorMap map_w,
    const __grid_constant__ CUtensorMap map_a) {
  pdl_enter();
  using L = WideLayout;
  constexpr int S = L::kStages, NB = L::kAccBufs, MB = L::kMetaBufs;
  extern __shared__ uint8_t raw_smem[];
  uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) &
                                             ~uintptr_t(1023));
  float* s_sa = reinterpret_cast<float*>(ring + S * L::kStageBytes);      // [MB][kb][token]
  float* s_sw = s_sa + MB * L::kSaFloats;                                 // [MB][kb][2]
  float* s_tw = s_sw + MB * L::kSwFloats;                                 // [MB][token]
  int* s_sid = reinterpret_cast<int*>(s_tw + MB * kWideTok);              // [MB][token]
  __shared__ __align__(8) uint64_t full_bar[S], done_bar[S], tempty_bar[NB];
  __shared__ __align__(8) uint64_t meta_empty_bar[MB], meta_full_bar[MB], drain_bar[2];
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int s_abort;
  __shared__ int s_expert[kMaxMBlocks];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int armed = 0;   // producer thread: stages it handed to the TMA (read at teardown)
  const bool gate = p.gate_act != 0;
  const int half_n = p.N / 2;
  const int nkb = p.K / kKBlock;
  const int m_blocks = *p.num_post / kWideTok;
  const int total_items = m_blocks * p.n_tiles;
  const int tile_rows = gate ? kWideCols / 2 : kWideCols;   // output rows (per half) of a tile
  for (int i = tid; i < m_blocks && i < kMaxMBlocks; i += kWideThreads) {
    const int e = p.expert_ids[i];
    s_expert[i] = e < p.experts ? e : -1;
  }
  if (tid == 0) {
    for (int i = 0; i < S; ++i) mbar_init(&full_bar[i], 1), mbar_init(&done_bar[i], 1);
    for (int i = 0; i < NB; ++i) mbar_init(&tempty_bar[i], kWideConsumerWarps);
    for (int i = 0; i < MB; ++i) mbar_init(&meta_empty_bar[i], kWideConsumerWarps), mbar_init(&meta_full_bar[i], 1);
    mbar_init(&drain_bar[0], 1), mbar_init(&drain_bar[1], 1);
    s_abort = 0;
    fence_mbar_init();
  }
  if (warp == kIssuerWarp) tmem_alloc(&tmem_slot, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_slot;
  const uint32_t ring_s = smem_u32(ring);
  auto next_valid = [&](int item) {
    while (item < total_items && s_expert[item / p.n_tiles] < 0) item += gridDim.x;
    return item;
  };


  if (warp == 0) {
    // ------------------------------------------------------------- producer
    if (lane == 0) {
      tma::prefetch_map(&map_w);
      tma::prefetch_map(&map_a);
      int t = 0;
      bool dead = false;
      for (int item = next_valid(blockIdx.x); item < total_items && !dead;
           item = next_valid(item + gridDim.x)) {
        const int mb = item / p.n_tiles, nt = item - mb * p.n_tiles;
        const int expert = s_expert[mb];
        for (int kb = 0; kb < nkb; ++kb, ++t) {
          const int s = t % S;
          if (!mbar_wait(&done_bar[s], ((t / S) & 1) ^ 1) || s_abort) {   // its MMAs retired
            dead = true;
            break;
          }
          const uint32_t st = ring_s + s * L::kStageBytes;
          tma::mbar_expect_tx(&full_bar[s], L::kStageBytes);
          tma::load_2d(st, &map_a, kb * kKBlock, mb * kWideTok, &full_bar[s]);
          tma::load_4d(st + L::kABytes, &map_w, kb * kKBlock, 0, nt * tile_rows, expert, &full_bar[s]);
        }
      }
      armed = t;
      if (dead) atomicExch(p.status, 1), s_abort = 1;
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- metadata
    int li = 0;
    bool dead = false;
    for (int item = next_valid(blockIdx.x); item < total_items && !dead;
         item = next_valid(item + gridDim.x), ++li) {
      const int buf = li % MB;
      const bool free_ok = mbar_wait(&meta_empty_bar[buf], ((li / MB) & 1) ^ 1);
      if (__any_sync(0xffffffffu, !free_ok || s_abort != 0)) {
        dead = true;
        break;
      }
      const int mb = item / p.n_tiles, nt = item - mb * p.n_tiles;
      const int expert = s_expert[mb];
      const uint32_t sa_dst = smem_u32(s_sa + buf * L::kSaFloats);
#pragma unroll
      for (int i = 0; i < kWideTok / 32; ++i) {
        const int j = lane + 32 * i;
        const int64_t sid = p.sorted_ids[mb * kWideTok + j];
        const bool ok = sid >= 0 && sid < p.num_valid;
        s_sid[buf * kWideTok + j] = ok ? int(sid) : -1;
        if (p.topk_w != nullptr)
          cp_async_4_zfill(smem_u32(s_tw + buf * kWideTok + j), p.topk_w + (ok ? sid : 0), ok);
        else
          s_tw[buf * kWideTok + j] = 1.f;
        const float* sap = p.sa + (int64_t(mb) * kWideTok + j) * p.sa_stride;
        for (int k2 = 0; k2 < nkb; ++k2) cp_async_4(sa_dst + (k2 * kWideTok + j) * 4, sap + k2);
      }
      if (p.scale_kind == 2) {
        // the tile's two 128-row blocks: gate / up rows, or the lower / upper half
        for (int i = lane; i < 2 * nkb; i += 32) {
          const int k2 = i >> 1, par = i & 1;
          const int blk = gate ? ((par ? half_n : 0) + nt * tile_rows) / 128 : nt * 2 + par;
          cp_async_4(smem_u32(s_sw + buf * L::kSwFloats + i),
                     p.scales + int64_t(expert) * p.s_se + int64_t(blk) * p.s_sn + k2);
        }
      }
      cp_async_commit();
      cp_async_wait<0>();
      __syncwarp();
      if (lane == 0) mbar_arrive(&meta_full_bar[buf]);
    }
    if (dead && lane == 0) atomicExch(p.status, 1), s_abort = 1;
  } else if (warp == kIssuerWarp || warp == kIssuerWarp + 1) {
    // -------------------------------------------------------------- issuers
    // two threads on alternate K blocks (= alternate accumulators; measured 0.539 ->
    // 0.528 ms per 4096-token layer)
    const int parity = warp - kIssuerWarp;
    if (lane == 0) {
      const uint32_t idesc = instr_desc(D_F32, 0, 0, kWideTok, kWideCols);
      const uint32_t a_lo0 = smem_desc_lo(ring_s);
      int t = 0;
      bool dead = false;
      for (int item = next_valid(blockIdx.x); item < total_items && !dead;
           item = next_valid(item + gridDim.x)) {
        for (int kb = 0; kb < nkb; ++kb, ++t) {
          if ((t & 1) != parity) continue;
          const int s = t % S, b = t % NB;
          const bool ok_full = mbar_wait(&full_bar[s], (t / S) & 1);
          const bool ok_acc = mbar_wait(&tempty_bar[b], ((t / NB) & 1) ^ 1);
          if (!ok_full || !ok_acc || s_abort) {
            dead = true;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_lo = a_lo0 + s * (L::kStageBytes >> 4), b_lo = a_lo + (L::kABytes >> 4);
          const uint32_t d = tmem + b * kWideCols;
          mma_ss_lo<KIND_F8F6F4, false>(d, a_lo, b_lo, idesc);
          mma_ss_lo<KIND_F8F6F4, true>(d, a_lo + 2, b_lo + 2, idesc);
          mma_ss_lo<KIND_F8F6F4, true>(d, a_lo + 4, b_lo + 4, idesc);
          mma_ss_lo<KIND_F8F6F4, true>(d, a_lo + 6, b_lo + 6, idesc);
          mma_commit(&done_bar[s]);   // the stage may be refilled, the sums are ready
        }
      }
      if (dead) atomicExch(p.status, 1), s_abort = 1;
    }
  } else if (warp >= kProducerWarps) {
    // ------------------------------------------------------------ consumers
    const int tok = (warp & 3) * 32 + lane;           // TMEM lane = token of the m-block
    const int cg = (warp - kProducerWarps) >> 2;      // which 128 of the 256 columns
    const uint32_t lane_base = uint32_t((warp & 3) * 32) << 16;
    constexpr int NC = kWideCols / 2;                 // columns per thread
    int t = 0, li = 0;
    bool dead = false;
    for (int item = next_valid(blockIdx.x); item < total_items && !dead;
         item = next_valid(item + gridDim.x), ++li) {
      const int mb = item / p.n_tiles, nt = item - mb * p.n_tiles;
      const int expert = s_expert[mb];
      const int buf = li % MB;
      const bool meta_ok = mbar_wait(&meta_full_bar[buf], (li / MB) & 1);
      if (__any_sync(0xffffffffu, !meta_ok) || s_abort) {
        dead = true;
        break;
      }
      const float* sa_item = s_sa + buf * L::kSaFloats + tok;
      const float* sw_item = s_sw + buf * L::kSwFloats;
      float acc[NC];
#pragma unroll
      for (int j = 0; j < NC; ++j) acc[j] = 0.f;
      for (int kb = 0; kb < nkb && !dead; ++kb, ++t) {
        const int s = t % S, b = t % NB;
        const bool ok = mbar_wait(&done_bar[s], (t / S) & 1);
        if (__any_sync(0xffffffffu, !ok)) {
          dead = true;
          break;
        }
        tc_fence_after_sync();
        const float sa = sa_item[kb * kWideTok];
        // gate: even columns are gate rows, odd ones up rows; else one block per column group
        float f_even = sa, f_odd = sa;
        if (p.scale_kind == 2) {
          f_even *= gate ? sw_item[2 * kb] : sw_item[2 * kb + cg];
          f_odd *= gate ? sw_item[2 * kb + 1] : sw_item[2 * kb + cg];
        }
        const uint32_t src = tmem + lane_base + b * kWideCols + cg * NC;
        // (measured on the 4096-token gate-up GEMM: 32-column loads with scalar FMAs,
        // 198 us, beat 16-column loads with packed fma.f32x2, 224 us; with neither
        // folds nor epilogue the launch takes 147 us, without MMAs as well 118 us)
        uint32_t r[16];
#pragma unroll
        for (int ch = 0; ch < NC / 16; ++ch) {
          tmem_ld_32x16(src + ch * 16, r);
          tmem_ld_wait();
          if (ch + 1 == NC / 16) {       // everything read: hand the accumulator back
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tempty_bar[b]);
          }
#pragma unroll
          for (int j = 0; j < 16; j += 2) {
            const float2 a2 = __ffma2_rn(make_float2(__uint_as_float(r[j]), __uint_as_float(r[j + 1])),
                                         make_float2(f_even, f_odd),
                                         make_float2(acc[ch * 16 + j], acc[ch * 16 + j + 1]));
            acc[ch * 16 + j] = a2.x, acc[ch * 16 + j + 1] = a2.y;
          }
        }
      }
      if (dead) break;

      // ---- epilogue: this thread's token row, its 128 columns
      const int sid = s_sid[buf * kWideTok + tok];
      const int crow = p.c_sorted ? mb * kWideTok + tok : sid;
      __nv_bfloat16* cptr = static_cast<__nv_bfloat16*>(p.c) + int64_t(crow < 0 ? 0 : crow) * p.c_stride;
      if (gate) {
        // columns 2i, 2i + 1 of the tile = gate row, up row  nt * 128 + cg * 64 + i
        const int out0 = nt * tile_rows + cg * (NC / 2);
        const float* chp = p.scales + int64_t(expert) * p.s_se;
#pragma unroll
        for (int i = 0; i < NC / 2; i += 8) {
          uint32_t o[4];
#pragma unroll
          for (int u = 0; u < 8; u += 2) {
            float v[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              float gv = acc[2 * (i + u + e)], uv = acc[2 * (i + u + e) + 1];
              if (p.scale_kind == 1) gv *= __ldg(chp + out0 + i + u + e), uv *= __ldg(chp + half_n + out0 + i + u + e);
              v[e] = gate_fn(gv, p.gate_act) * uv;
            }
            o[u >> 1] = pack_bf16x2(v[0], v[1]);
          }
          if (crow >= 0) *reinterpret_cast<uint4*>(cptr + out0 + i) = make_uint4(o[0], o[1], o[2], o[3]);
        }
      } else {
        const int out0 = nt * tile_rows + cg * NC;
        const float tw = s_tw[buf * kWideTok + tok];
        const float* chp = p.scales + int64_t(expert) * p.s_se + out0;
#pragma unroll
        for (int i = 0; i < NC; i += 8) {
          uint32_t o[4];
#pragma unroll
          for (int u = 0; u < 8; u += 2) {
            float v0 = acc[i + u] * tw, v1 = acc[i + u + 1] * tw;
            if (p.scale_kind == 1) v0 *= __ldg(chp + i + u), v1 *= __ldg(chp + i + u + 1);
            o[u >> 1] = pack_bf16x2(v0, v1);
          }
          if (crow >= 0) *reinterpret_cast<uint4*>(cptr + out0 + i) = make_uint4(o[0], o[1], o[2], o[3]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&meta_empty_bar[buf]);
    }
    if (dead) atomicExch(p.status, 1), s_abort = 1;
  }

  tc_fence_before_sync();
  __syncthreads();
  if (s_abort) {
    if (tid == 0) drain_armed_loads(full_bar, S, armed);
    if ((warp == kIssuerWarp || warp == kIssuerWarp + 1) && lane == 0)
      drain_issued_mmas(&drain_bar[warp - kIssuerWarp]);
    tc_fence_before_sync();
    __syncthreads();
  }
  if (warp == kIssuerWarp) tmem_dealloc(tmem, 512);
}

// Status word the kernels raise when a bounded wait runs out (0 = healthy).
__device__ int32_t g_umma_status = 0;

template <int NTOK, int KBMAX>
int launch_umma(const UmmaMoeArgs& p, const CUtensorMap& map_w, const CUtensorMap& map_a,
                cudaStream_t st) {
  using L = UmmaLayout<NTOK, KBMAX>;
  auto kernel = moe_gemm_umma_kernel<NTOK, KBMAX>;
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
  launch_chain(kernel, sms[dev], umma_threads(NTOK), L::kSmem, st, p, map_w, map_a);
  return launch_status("moe_gemm_umma");
}

int launch_umma_wide(const UmmaMoeArgs& p, const CUtensorMap& map_w, const CUtensorMap& map_a,
                     cudaStream_t st) {
  static bool done[64] = {};
  static int sms[64] = {};
  int dev = 0;
  STRIX_CUDA(cudaGetDevice(&dev));
  STRIX_CHECK(dev >= 0 && dev < 64, "device index %d out of range", dev);
  if (!done[dev]) {
    STRIX_CUDA(cudaFuncSetAttribute(moe_gemm_umma_wide_kernel,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, WideLayout::kSmem));
    STRIX_CUDA(cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev));
    done[dev] = true;
  }
  launch_chain(moe_gemm_umma_wide_kernel, sms[dev], kWideThreads, WideLayout::kSmem, st, p, map_w, map_a);
  return launch_status("moe_gemm_umma_wide");
}

}  // namespace

// Device address of the status word shared by every tcgen05 kernel of the library.
int32_t* umma_status_ptr() {
  void* addr = nullptr;
  return cudaGetSymbolAddress(&addr, g_umma_status) == cudaSuccess ? static_cast<int32_t*>(addr)
                                                                    : nullptr;
}

// Whether the tcgen05 kernel covers a geometry (the entry point below rejects the rest).
static bool sorted_covers(int64_t n, int64_t k, int64_t block_m, int gate_act, int scale_kind) {
  const int64_t out_rows = gate_act ? n / 2 : n;
  const int tile_out = gate_act ? kTileM / 2 : kTileM;
  return (block_m == 16 || block_m == 32 || block_m == 64 || block_m == 128) && n > 0 && k > 0 &&
         n % 2 == 0 && out_rows % tile_out == 0 && k % kKBlock == 0 &&
         k <= (block_m > 64 ? 32 : 64) * kKBlock && (scale_kind == 1 || scale_kind == 2) &&
         !(scale_kind == 2 && gate_act && (n / 2) % 128 != 0);
}

}  // namespace strix

using namespace strix;

extern "C" int strix_moe_gemm_fp8_sorted_covers(int64_t n, int64_t k, int64_t block_m, int gate_act,
                                                int scale_kind) {
  return sorted_covers(n, k, block_m, gate_act, scale_kind) ? 1 : 0;
}

extern "C" int strix_moe_gemm_fp8_sorted(
    void* c, const void* a, const float* act_scales, const void* w, const float* scales,
    const int32_t* sorted_ids, const int32_t* expert_ids, const int32_t* num_post_padded,
    const float* topk_weights, int64_t num_valid, int64_t num_experts, int64_t n, int64_t k,
    int64_t a_stride, int64_t c_stride, int64_t w_stride_e, int64_t w_stride_n, int64_t s_stride_e,
    int64_t s_stride_n, int64_t sa_stride, int64_t sorted_len, int64_t block_m, int scale_kind,
    int gate_act, int c_sorted, strix_stream_t stream) {
  STRIX_CHECK(gate_act >= 0 && gate_act <= 2, "activation must be none, silu or gelu_tanh");
  STRIX_CHECK(num_experts >= 1 && num_experts <= (int64_t(1) << 24), "num_experts out of range");
  STRIX_CHECK(sorted_covers(n, k, block_m, gate_act, scale_kind),
              "geometry not covered: block_m in 16/32/64/128, K %% 128, K <= 8192 (4096 at 128 "
              "tokens), whole 128-row weight tiles, channel or 128x128 block scales");
  STRIX_CHECK(sorted_len % block_m == 0 && sorted_len / block_m <= kMaxMBlocks,
              "sorted_len must be whole m-blocks, at most %d of them", kMaxMBlocks);
  STRIX_CHECK(gate_act == 0 || topk_weights == nullptr, "the fused gate takes no routing weights");
  STRIX_CHECK(w_stride_n % 16 == 0 && w_stride_e % 16 == 0 && a_stride % 16 == 0 &&
                  reinterpret_cast<uintptr_t>(w) % 16 == 0 && reinterpret_cast<uintptr_t>(a) % 16 == 0,
              "16-byte aligned rows required");
  STRIX_CHECK(sa_stride >= k / kKBlock, "act_scales must be [sorted_len, K / 128]");
  if (sorted_len == 0 || num_valid == 0) return STRIX_OK;
  const int64_t out_rows = gate_act ? n / 2 : n;
  // m-blocks of 128 tokens take the wide-tile kernel (tokens as the MMA's M, 256
  // weight rows as its N) where its tile divides the problem
  static const bool no_wide = getenv("STRIX_MOE_NO_WIDE") != nullptr;
  const int wide_out = gate_act ? kWideCols / 2 : kWideCols;
  const bool wide = !no_wide && block_m == kWideTok && k <= kWideKbMax * kKBlock &&
                    out_rows % wide_out == 0;
  const int tile_out = wide ? wide_out : gate_act ? kTileM / 2 : kTileM;
  UmmaMoeArgs p;
  p.c = c, p.scales = scales, p.sa = act_scales;
  p.sorted_ids = sorted_ids, p.expert_ids = expert_ids, p.num_post = num_post_padded;
  p.topk_w = topk_weights;
  p.status = umma_status_ptr();
  STRIX_CHECK(p.status != nullptr, "status word unavailable");
  p.num_valid = num_valid;
  p.c_stride = c_stride, p.s_se = s_stride_e, p.s_sn = s_stride_n, p.sa_stride = sa_stride;
  p.K = int(k), p.N = int(n), p.block_m = int(block_m), p.experts = int(num_experts);
  p.scale_kind = scale_kind, p.gate_act = gate_act, p.c_sorted = c_sorted;
  p.n_tiles = int(out_rows / tile_out);
  static const int prefetch = [] { const char* e = getenv("STRIX_UMMA_PREFETCH"); return e ? atoi(e) : 0; }();
  p.prefetch = prefetch < 0 ? 0 : prefetch > 256 ? 256 : prefetch;
  // Weights as a 4-d byte tensor (k, half, row, expert): under the fused gate
  // `half` steps from the gate rows to the up rows, so a box of 2 x 64 rows lands
  // as gate row i / up row i alternating; otherwise it has extent 1.
  const uint64_t halves = gate_act ? 2 : 1, rows = uint64_t(out_rows);
  const uint64_t dims[4] = {uint64_t(k), halves, rows, uint64_t(num_experts)};
  const uint64_t strides[3] = {uint64_t(w_stride_n) * rows, uint64_t(w_stride_n), uint64_t(w_stride_e)};
  const uint32_t box[4] = {128, uint32_t(halves), uint32_t(tile_out), 1};
  CUtensorMap map_w, map_a;
  STRIX_CHECK(tma::make_map_u8_nd(&map_w, w, 4, dims, strides, box) &&
                  tma::make_map_u8(&map_a, a, uint64_t(sorted_len), uint64_t(k), uint64_t(a_stride),
                                   uint32_t(block_m)),
              "tensor map encoding failed");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (wide) return launch_umma_wide(p, map_w, map_a, st);
  const bool short_k = k <= 16 * kKBlock;
  if (block_m == 16) return short_k ? launch_umma<16, 16>(p, map_w, map_a, st) : launch_umma<16, 64>(p, map_w, map_a, st);
  if (block_m == 32) return short_k ? launch_umma<32, 16>(p, map_w, map_a, st) : launch_umma<32, 64>(p, map_w, map_a, st);
  if (block_m == 64) return short_k ? launch_umma<64, 16>(p, map_w, map_a, st) : launch_umma<64, 64>(p, map_w, map_a, st);
  return short_k ? launch_umma<128, 16>(p, map_w, map_a, st) : launch_umma<128, 32>(p, map_w, map_a, st);
}

extern "C" int strix_umma_status(int32_t* host_out) {
  STRIX_CHECK(host_out != nullptr, "host_out must not be NULL");
  STRIX_CUDA(cudaMemcpyFromSymbol(host_out, strix::g_umma_status, sizeof(int32_t)));
  return STRIX_OK;
}
