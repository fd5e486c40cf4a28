// The small kernels around the expert GEMMs of a MoE layer, for sm_100a:
// router (softmax -> top-k -> renormalise), token permutation
// (moe_align_block_size contract), per-(row, 128-group) activation quantisers
// (e4m3 and int8) and the top-k combine.
//
// The reference takes the router, the permutation and the combine from vLLM
// (python/strix_vllm/moe.py:959-961, 1012-1014 call moe_align_block_size and
// moe_sum); the permutation contract is the one its tests restate
// (tests/test_moe_gemm.py:9-31). moe_act_quant_i8 follows
// csrc/moe/moe_gemm_w4a8.hip:283-316.
#include "common.cuh"

namespace strix {
namespace {

// ------------------------------------------------------------------ router
// One warp per token. Selection is on the logits (softmax is monotonic), ties
// go to the lower expert index; weights are p_i / sum of the selected p.
template <int VPL>  // values per lane: experts <= 32 * VPL
__global__ void __launch_bounds__(128) topk_softmax_kernel(
    const float* __restrict__ logits, int64_t l_stride, int32_t* __restrict__ ids,
    float* __restrict__ weights, int tokens, int experts, int top_k, int renorm) {
  pdl_enter();
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (t >= tokens) return;
  const float* row = logits + int64_t(t) * l_stride;
  float v[VPL];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int e = lane + 32 * i;
    v[i] = e < experts ? row[e] : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) sum += v[i] == -INFINITY ? 0.f : expf(v[i] - mx);
#pragma unroll
  for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  float my_w = 0.f, wsum = 0.f;   // lane j keeps the j-th selection
  int my_id = 0;
  for (int j = 0; j < top_k; ++j) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int e = lane + 32 * i;
      if (e < experts && (v[i] > best || (v[i] == best && e < bi)) && v[i] != -INFINITY) {
        best = v[i];
        bi = e;
      }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) {
        best = ob;
        bi = oi;
      }
    }
    // every lane now agrees on (best, bi); its owner retires the value
    if (bi != 0x7fffffff && (bi & 31) == lane) {
#pragma unroll
      for (int i = 0; i < VPL; ++i)
        if (i == (bi >> 5)) v[i] = -INFINITY;
    }
    const float p = bi == 0x7fffffff ? 0.f : __fdiv_rn(expf(best - mx), sum);
    wsum += p;
    if (lane == j) {
      my_w = p;
      my_id = bi == 0x7fffffff ? 0 : bi;
    }
  }
  if (lane < top_k) {
    ids[int64_t(t) * top_k + lane] = my_id;
    weights[int64_t(t) * top_k + lane] = renorm ? __fdiv_rn(my_w, wsum) : my_w;
  }
}

// ------------------------------------------------------------------- align
// CTA e < experts places the slots routed to expert e; CTA `experts` writes
// num_post_padded and fills everything past it. Each CTA histograms all slots
// itself (one pass over the ids, served by L2), so there is no inter-CTA
// dependency and a single launch suffices. Order inside an expert is ascending
// slot id (a stable partition), which makes the result unique and comparable
// bit for bit. Every warp owns one contiguous eighth of the slots: the histogram
// pass also counts the warp's hits for expert e, one barrier turns the counts
// into offsets, and the placement pass runs on warp ballots alone - no barrier
// inside either pass, whatever the number of slots.
constexpr int kAlignThreads = 256, kAlignWarps = kAlignThreads / 32;

__global__ void __launch_bounds__(kAlignThreads) moe_align_kernel(
    const int32_t* __restrict__ topk_ids, int32_t* __restrict__ sorted_ids,
    int32_t* __restrict__ expert_ids, int32_t* __restrict__ num_post, int numel, int experts,
    int block_m, int cap, int cap_blocks, int32_t* __restrict__ slot_pos,
    int32_t* __restrict__ counts) {
  pdl_enter();
  extern __shared__ int s_count[];            // [experts]
  __shared__ int s_warp[kAlignWarps];
  __shared__ int s_base;
  const int e = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (int i = tid; i < experts; i += kAlignThreads) s_count[i] = 0;
  __syncthreads();
  // this warp's slots: [lo, hi), a multiple of 32 long except at the end
  const int per_warp = ((numel + kAlignWarps - 1) / kAlignWarps + 31) / 32 * 32;
  const int lo = min(warp * per_warp, numel), hi = min(lo + per_warp, numel);
  int mine = 0;                                // hits for expert e in this warp's slots
  for (int i = lo + lane; i - lane < hi; i += 32) {
    const int id = i < hi ? topk_ids[i] : -1;
    if (id >= 0 && id < experts) atomicAdd(&s_count[id], 1);
    mine += __popc(__ballot_sync(0xffffffffu, id == e));
  }
  if (lane == 0) s_warp[warp] = mine;
  __syncthreads();
  // padded slots before expert e (or the grand total for the last CTA)
  int part = 0;
  const int upto = e < experts ? e : experts;
  for (int i = tid; i < upto; i += kAlignThreads)
    part += (s_count[i] + block_m - 1) / block_m * block_m;
#pragma unroll
  for (int o = 16; o; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
  int before = 0;                              // hits of the warps in front of this one
#pragma unroll
  for (int w = 0; w < kAlignWarps; ++w) before += w < warp ? s_warp[w] : 0;
  __syncthreads();                             // s_warp is reused for the partial sums
  if (lane == 0) s_warp[warp] = part;
  __syncthreads();
  if (tid == 0) {
    int t = 0;
    for (int i = 0; i < kAlignWarps; ++i) t += s_warp[i];
    s_base = t;
  }
  __syncthreads();
  const int base = s_base;
  if (e == experts) {
    if (tid == 0) num_post[0] = base;
    // slots whose id names no expert (masked, -1) have no position
    if (slot_pos != nullptr)
      for (int i = tid; i < numel; i += kAlignThreads) {
        const int id = topk_ids[i];
        if (id < 0 || id >= experts) slot_pos[i] = -1;
      }
    for (int i = base + tid; i < cap; i += kAlignThreads) sorted_ids[i] = numel;
    for (int i = base / block_m + tid; i < cap_blocks; i += kAlignThreads) expert_ids[i] = -1;
    return;
  }
  const int count = s_count[e];
  if (counts != nullptr && tid == 0) counts[e] = count;
  const int padded = (count + block_m - 1) / block_m * block_m;
  for (int i = tid; i < padded / block_m; i += kAlignThreads)
    if (base / block_m + i < cap_blocks) expert_ids[base / block_m + i] = e;
  for (int i = count + tid; i < padded; i += kAlignThreads)
    if (base + i < cap) sorted_ids[base + i] = numel;
  if (count == 0) return;
  // ordered compaction of the slots whose id == e
  int placed = base + before;
  for (int i = lo + lane; i - lane < hi; i += 32) {
    const bool hit = i < hi && topk_ids[i] == e;
    const unsigned bal = __ballot_sync(0xffffffffu, hit);
    if (hit) {
      const int pos = placed + __popc(bal & ((1u << lane) - 1u));
      if (pos < cap) sorted_ids[pos] = i;
      if (slot_pos != nullptr) slot_pos[i] = pos < cap ? pos : -1;   // the inverse permutation
    }
    placed += __popc(bal);
  }
}

// ------------------------------------------------ the same, for many slots
// moe_align_kernel lets every expert's CTA walk all the slots: fine up to a few
// thousand, 67 us at 32,768. The two-level form walks them once per pass:
//   hist   one CTA per chunk of 1024 consecutive slots counts its slots per expert
//          into hist[chunk][expert] (global scratch from the caller);
//   place  the same CTAs sum the columns of hist (the expert's total, and the slots
//          of earlier chunks - which, in slot order, come first), scan the padded
//          totals, rank their own slots (a warp owns 128 consecutive slots; ranks
//          inside a warp from match masks, warps ordered through shared memory) and
//          write sorted_ids / slot_pos; paddings, expert_ids and the tail are split
//          over the CTAs.
// Same output, bit for bit, as moe_align_kernel.
constexpr int kChunkSlots = 1024, kPlaceThreads = 256, kPlaceWarps = 8, kPlaceMaxExperts = 1024;

__global__ void __launch_bounds__(kPlaceThreads) moe_align_hist_kernel(
    const int32_t* __restrict__ topk_ids, int32_t* __restrict__ hist, int numel, int experts) {
  pdl_enter();
  extern __shared__ int s_cnt[];
  for (int i = threadIdx.x; i < experts; i += kPlaceThreads) s_cnt[i] = 0;
  __syncthreads();
  const int base = blockIdx.x * kChunkSlots;
#pragma unroll
  for (int j = 0; j < kChunkSlots / kPlaceThreads; ++j) {
    const int i = base + j * kPlaceThreads + threadIdx.x;
    const int id = i < numel ? topk_ids[i] : -1;
    if (id >= 0 && id < experts) atomicAdd(&s_cnt[id], 1);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < experts; i += kPlaceThreads) hist[blockIdx.x * experts + i] = s_cnt[i];
}

__global__ void __launch_bounds__(kPlaceThreads) moe_align_place_kernel(
    const int32_t* __restrict__ topk_ids, const int32_t* __restrict__ hist,
    int32_t* __restrict__ sorted_ids, int32_t* __restrict__ expert_ids, int32_t* __restrict__ num_post,
    int numel, int experts, int block_m, int cap, int cap_blocks, int chunks,
    int32_t* __restrict__ slot_pos, int32_t* __restrict__ counts) {
  pdl_enter();
  extern __shared__ int s_dyn[];
  int* s_tot = s_dyn;                       // [experts] slots of the expert
  int* s_base = s_tot + experts;            // [experts] first sorted position of the expert
  int* s_off = s_base + experts;            // [experts] its slots in earlier chunks
  int* s_w = s_off + experts;               // [warps][experts] running rank within this chunk
  __shared__ int s_scan[kPlaceWarps];
  __shared__ int s_total;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, chunk = blockIdx.x;
  for (int e = tid; e < experts; e += kPlaceThreads) {
    int tot = 0, off = 0;
    for (int c = 0; c < chunks; ++c) {
      const int h = hist[c * experts + e];
      tot += h;
      off += c < chunk ? h : 0;
    }
    s_tot[e] = tot, s_off[e] = off;
  }
  for (int i = tid; i < kPlaceWarps * experts; i += kPlaceThreads) s_w[i] = 0;
  __syncthreads();
  // exclusive scan of the padded totals: thread t owns experts [t * per, t * per + per)
  const int per = (experts + kPlaceThreads - 1) / kPlaceThreads;
  int mine = 0;
  for (int j = 0; j < per; ++j) {
    const int e = tid * per + j;
    if (e < experts) mine += (s_tot[e] + block_m - 1) / block_m * block_m;
  }
  int incl = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int v = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += v;
  }
  if (lane == 31) s_scan[warp] = incl;
  __syncthreads();
  int before = 0;
#pragma unroll
  for (int w = 0; w < kPlaceWarps; ++w) before += w < warp ? s_scan[w] : 0;
  if (tid == kPlaceThreads - 1) s_total = before + incl;
  int run = before + incl - mine;
  for (int j = 0; j < per; ++j) {
    const int e = tid * per + j;
    if (e < experts) {
      s_base[e] = run;
      run += (s_tot[e] + block_m - 1) / block_m * block_m;
    }
  }
  // this warp's 128 slots: counts per expert, then the warps in slot order
  const int w0 = chunk * kChunkSlots + warp * (kChunkSlots / kPlaceWarps);
  int ids[kChunkSlots / kPlaceWarps / 32];
#pragma unroll
  for (int j = 0; j < kChunkSlots / kPlaceWarps / 32; ++j) {
    const int i = w0 + j * 32 + lane;
    const int id = i < numel ? topk_ids[i] : -1;
    ids[j] = (id >= 0 && id < experts) ? id : -1;
    if (ids[j] >= 0) atomicAdd(&s_w[warp * experts + ids[j]], 1);
  }
  __syncthreads();
  for (int e = tid; e < experts; e += kPlaceThreads) {
    int acc = 0;
#pragma unroll
    for (int w = 0; w < kPlaceWarps; ++w) {
      const int t = s_w[w * experts + e];
      s_w[w * experts + e] = acc;
      acc += t;
    }
  }
  __syncthreads();
  const int total = s_total;
  if (chunk < chunks) {
#pragma unroll
    for (int j = 0; j < kChunkSlots / kPlaceWarps / 32; ++j) {
      const int i = w0 + j * 32 + lane;
      const int id = ids[j];
      // lanes without an expert get keys of their own, so that they match nobody
      const unsigned peers = __match_any_sync(0xffffffffu, id >= 0 ? id : experts + lane);
      if (id >= 0) {
        const int rank = __popc(peers & ((1u << lane) - 1u));
        const int pos = s_base[id] + s_off[id] + s_w[warp * experts + id] + rank;
        if (pos < cap) sorted_ids[pos] = i;
        if (slot_pos != nullptr) slot_pos[i] = pos < cap ? pos : -1;
      } else if (slot_pos != nullptr && i < numel) {
        slot_pos[i] = -1;
      }
      __syncwarp();
      if (id >= 0 && (peers & ((1u << lane) - 1u)) == 0) s_w[warp * experts + id] += __popc(peers);
      __syncwarp();
    }
  }
  // paddings and block ids of the experts e = blockIdx.x, + gridDim.x, ...; the tail in slices
  for (int e = blockIdx.x; e < experts; e += gridDim.x) {
    const int count = s_tot[e], padded = (count + block_m - 1) / block_m * block_m, base = s_base[e];
    if (counts != nullptr && tid == 0) counts[e] = count;
    for (int i = tid; i < padded / block_m; i += kPlaceThreads)
      if (base / block_m + i < cap_blocks) expert_ids[base / block_m + i] = e;
    for (int i = count + tid; i < padded; i += kPlaceThreads)
      if (base + i < cap) sorted_ids[base + i] = numel;
  }
  if (blockIdx.x == 0 && tid == 0) num_post[0] = total;
  {
    const int tail = cap - total, slice = (tail + int(gridDim.x) - 1) / int(gridDim.x);
    const int lo = total + blockIdx.x * slice, hi = min(lo + slice, cap);
    for (int i = lo + tid; i < hi; i += kPlaceThreads) sorted_ids[i] = numel;
    const int b0 = total / block_m, btail = cap_blocks - b0, bslice = (btail + int(gridDim.x) - 1) / int(gridDim.x);
    const int blo = b0 + blockIdx.x * bslice, bhi = min(blo + bslice, cap_blocks);
    for (int i = blo + tid; i < bhi; i += kPlaceThreads) expert_ids[i] = -1;
  }
}

// ------------------------------------------------------- activation quantisers
// 16 lanes share one 128-element group (8 elements = 16 bytes each).
// With `row_map` (the sorted ids of moe_align_block_size) output row r is the
// quantised input row row_map[r] / top_k - the activations in sorted order, a
// row of zeros (scale 1) for a padding slot; `row_limit` (the padded slot count,
// on the device) bounds the rows that are written at all.
template <bool FP8, bool IN_F16>
__global__ void __launch_bounds__(256) act_quant_kernel(
    const uint16_t* __restrict__ x, int64_t x_stride, uint8_t* __restrict__ q, int64_t q_stride,
    float* __restrict__ sa, int64_t sa_stride, int64_t rows, int groups,
    const int32_t* __restrict__ row_map, const int32_t* __restrict__ row_limit, int top_k,
    int64_t num_valid) {
  pdl_enter();
  int64_t team = (int64_t(blockIdx.x) * 256 + threadIdx.x) >> 4;
  const int sub = threadIdx.x & 15;
  // out-of-range teams redo the last group and skip the stores, so every lane
  // of the warp stays in the shuffles below
  bool live = team < rows * groups;
  if (!live) team = rows * groups - 1;
  const int64_t r = team / groups;
  const int gi = int(team % groups);
  if (row_limit != nullptr && r >= *row_limit) live = false;
  int64_t src = r;
  bool filled = true;
  if (row_map != nullptr) {
    const int64_t sid = live ? row_map[r] : -1;
    filled = sid >= 0 && sid < num_valid;
    src = filled ? sid / top_k : 0;
  } else if (!live) {
    src = 0;
  }
  uint4 w = make_uint4(0u, 0u, 0u, 0u);
  if (filled) w = *reinterpret_cast<const uint4*>(x + src * x_stride + gi * 128 + sub * 8);
  const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
  float v[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (IN_F16) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&ws[i]));
      v[2 * i] = f.x, v[2 * i + 1] = f.y;
    } else {
      v[2 * i] = bf16_lo(ws[i]), v[2 * i + 1] = bf16_hi(ws[i]);
    }
  }
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
  for (int o = 8; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o, 16));
  uint2 packed;
  float s;
  if (FP8) {
    s = amax > 0.f ? __fdiv_rn(amax, 448.f) : 1.f;
    uint32_t h[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float a = __fdiv_rn(v[2 * i], s), b = __fdiv_rn(v[2 * i + 1], s);
      uint16_t o;
      asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(o) : "f"(b), "f"(a));
      h[i] = o;
    }
    packed.x = h[0] | (h[1] << 16);
    packed.y = h[2] | (h[3] << 16);
  } else {
    // s = amax / 127 (1 for an all-zero group), q = clamp(rint(x * (1 / s)), +-127):
    // csrc/moe/moe_gemm_w4a8.hip:305-312
    s = amax > 0.f ? __fdiv_rn(amax, 127.f) : 1.f;
    const float inv = __fdiv_rn(1.f, s);
    uint32_t b[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int qi = max(-127, min(127, __float2int_rn(v[i] * inv)));
      b[i] = uint32_t(qi) & 0xffu;
    }
    packed.x = b[0] | (b[1] << 8) | (b[2] << 16) | (b[3] << 24);
    packed.y = b[4] | (b[5] << 8) | (b[6] << 16) | (b[7] << 24);
  }
  if (!live) return;
  *reinterpret_cast<uint2*>(q + r * q_stride + gi * 128 + sub * 8) = packed;
  if (sub == 0) sa[r * sa_stride + gi] = s;
}

// e4m3 quantiser that writes the sorted layout by SCATTER: a 16-lane team
// quantises one (token, 128 group) once and stores it at the sorted positions of
// the token's top_k slots (slot_pos = the inverse permutation from moe_align), so
// a token is read and quantised once instead of top_k times. Teams past the
// tokens cover the sorted positions: a padding slot inside the padded range gets
// a row of zeros with scale 1.
template <bool IN_F16>
__global__ void __launch_bounds__(256) act_quant_scatter_kernel(
    const uint16_t* __restrict__ x, int64_t x_stride, uint8_t* __restrict__ q, int64_t q_stride,
    float* __restrict__ sa, int64_t sa_stride, int64_t tokens, int groups, int top_k,
    const int32_t* __restrict__ slot_pos, const int32_t* __restrict__ sorted_ids,
    const int32_t* __restrict__ num_post, int64_t rows_cap, int64_t num_valid) {
  pdl_enter();
  const int64_t team = (int64_t(blockIdx.x) * 256 + threadIdx.x) >> 4;
  const int sub = threadIdx.x & 15;
  const int64_t token_teams = tokens * groups;
  if (team >= token_teams) {
    // ---- padding rows (a whole 16-lane team takes this branch together)
    const int64_t pt = team - token_teams;
    const int64_t r = pt / groups;
    const int gi = int(pt % groups);
    if (r >= rows_cap || r >= *num_post) return;
    const int64_t sid = sorted_ids[r];
    if (sid >= 0 && sid < num_valid) return;
    *reinterpret_cast<uint2*>(q + r * q_stride + gi * 128 + sub * 8) = make_uint2(0u, 0u);
    if (sub == 0) sa[r * sa_stride + gi] = 1.f;
    return;
  }
  const int64_t r = team / groups;
  const int gi = int(team % groups);
  const uint4 w = *reinterpret_cast<const uint4*>(x + r * x_stride + gi * 128 + sub * 8);
  const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
  float v[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (IN_F16) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&ws[i]));
      v[2 * i] = f.x, v[2 * i + 1] = f.y;
    } else {
      v[2 * i] = bf16_lo(ws[i]), v[2 * i + 1] = bf16_hi(ws[i]);
    }
  }
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
  // only this team's 16 lanes take part: the other half of the warp may be a padding team
  const unsigned team_mask = 0xffffu << (threadIdx.x & 16);
#pragma unroll
  for (int o = 8; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(team_mask, amax, o, 16));
  const float s = amax > 0.f ? __fdiv_rn(amax, 448.f) : 1.f;
  uint32_t h[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float a = __fdiv_rn(v[2 * i], s), b = __fdiv_rn(v[2 * i + 1], s);
    uint16_t o;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(o) : "f"(b), "f"(a));
    h[i] = o;
  }
  const uint2 packed = make_uint2(h[0] | (h[1] << 16), h[2] | (h[3] << 16));
  for (int j = 0; j < top_k; ++j) {
    const int pos = slot_pos[r * top_k + j];
    if (pos < 0 || pos >= rows_cap) continue;
    *reinterpret_cast<uint2*>(q + int64_t(pos) * q_stride + gi * 128 + sub * 8) = packed;
    if (sub == 0) sa[int64_t(pos) * sa_stride + gi] = s;
  }
}

// -------------------------------------------------------------------- combine
// out[t, h] = sum_j in[t, j, h] in fp32 (j ascending), one bf16 rounding.
__global__ void __launch_bounds__(256) moe_sum_kernel(
    const uint16_t* __restrict__ in, int64_t in_st, int64_t in_sj, uint16_t* __restrict__ out,
    int64_t out_st, int tokens, int top_k, int hidden8) {
  pdl_enter();
  const int64_t idx = int64_t(blockIdx.x) * 256 + threadIdx.x;
  if (idx >= int64_t(tokens) * hidden8) return;
  const int64_t t = idx / hidden8;
  const int h = int(idx % hidden8) * 8;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int j = 0; j < top_k; ++j) {
    const uint4 w = *reinterpret_cast<const uint4*>(in + t * in_st + j * in_sj + h);
    const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      acc[2 * i] += bf16_lo(ws[i]);
      acc[2 * i + 1] += bf16_hi(ws[i]);
    }
  }
  uint4 o;
  o.x = pack_bf16x2(acc[0], acc[1]);
  o.y = pack_bf16x2(acc[2], acc[3]);
  o.z = pack_bf16x2(acc[4], acc[5]);
  o.w = pack_bf16x2(acc[6], acc[7]);
  *reinterpret_cast<uint4*>(out + t * out_st + h) = o;
}

// out[t, h] = sum_j rows[pos[t * top_k + j], h]: the combine over rows that lie in
// another order (expert-parallel: the order the result rows came back in).
__global__ void __launch_bounds__(256) moe_sum_gather_kernel(
    const uint16_t* __restrict__ rows, int64_t row_st, const int32_t* __restrict__ pos,
    uint16_t* __restrict__ out, int64_t out_st, int tokens, int top_k, int hidden8) {
  const int64_t idx = int64_t(blockIdx.x) * 256 + threadIdx.x;
  if (idx >= int64_t(tokens) * hidden8) return;
  const int64_t t = idx / hidden8;
  const int h = int(idx % hidden8) * 8;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int j = 0; j < top_k; ++j) {
    const int64_t r = pos[t * top_k + j];
    if (r < 0) continue;
    const uint4 w = *reinterpret_cast<const uint4*>(rows + r * row_st + h);
    const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      acc[2 * i] += bf16_lo(ws[i]);
      acc[2 * i + 1] += bf16_hi(ws[i]);
    }
  }
  uint4 o;
  o.x = pack_bf16x2(acc[0], acc[1]);
  o.y = pack_bf16x2(acc[2], acc[3]);
  o.z = pack_bf16x2(acc[4], acc[5]);
  o.w = pack_bf16x2(acc[6], acc[7]);
  *reinterpret_cast<uint4*>(out + t * out_st + h) = o;
}

// Expert-parallel dispatch buffers: row i of the send buffer is the token row of
// slot order[i]; meta[i] = (expert id modulo experts_per_rank, routing weight).
__global__ void __launch_bounds__(256) ep_pack_kernel(
    const uint4* __restrict__ x, int64_t x_st16, uint4* __restrict__ send, int64_t send_st16,
    float2* __restrict__ meta, const int32_t* __restrict__ order, const int32_t* __restrict__ topk_ids,
    const float* __restrict__ topk_w, int64_t slots, int chunks, int top_k, int experts_per_rank,
    int64_t meta_st2) {
  const int64_t idx = int64_t(blockIdx.x) * 256 + threadIdx.x;
  const int64_t i = idx / chunks;
  if (i >= slots) return;
  const int ch = int(idx % chunks);
  const int slot = order[i];
  if (slot < 0 || slot >= slots) return;   // a position no valid slot was sorted into
  send[i * send_st16 + ch] = x[int64_t(slot / top_k) * x_st16 + ch];
  if (ch == 0) meta[i * meta_st2] = make_float2(float(topk_ids[slot] % experts_per_rank), topk_w[slot]);
}

}  // namespace
}  // namespace strix

using namespace strix;

extern "C" int strix_moe_sum_gather(const void* rows, const int32_t* pos, void* out, int64_t tokens,
                                    int64_t top_k, int64_t hidden, int64_t row_st, int64_t out_st,
                                    strix_stream_t stream) {
  STRIX_CHECK(tokens >= 0 && top_k >= 1 && hidden > 0 && hidden % 8 == 0,
              "hidden must be a multiple of 8");
  STRIX_CHECK(row_st % 8 == 0 && out_st % 8 == 0 && reinterpret_cast<uintptr_t>(rows) % 16 == 0 &&
                  reinterpret_cast<uintptr_t>(out) % 16 == 0 && pos != nullptr,
              "16-byte aligned rows required");
  if (tokens == 0) return STRIX_OK;
  const int64_t work = tokens * (hidden / 8);
  moe_sum_gather_kernel<<<unsigned((work + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint16_t*>(rows), row_st, pos, static_cast<uint16_t*>(out), out_st,
      int(tokens), int(top_k), int(hidden / 8));
  return launch_status("moe_sum_gather");
}

extern "C" int strix_ep_pack(const void* x, void* send, float* meta, const int32_t* order,
                             const int32_t* topk_ids, const float* topk_weights, int64_t slots,
                             int64_t hidden, int64_t top_k, int64_t experts_per_rank,
                             int64_t x_stride, int64_t send_stride, int64_t meta_stride,
                             strix_stream_t stream) {
  STRIX_CHECK(meta_stride >= 2 && meta_stride % 2 == 0, "meta_stride counts floats, even, >= 2");
  STRIX_CHECK(slots >= 0 && hidden > 0 && hidden % 8 == 0 && top_k >= 1 && experts_per_rank >= 1,
              "hidden must be a multiple of 8");
  STRIX_CHECK(x_stride % 8 == 0 && send_stride % 8 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 &&
                  reinterpret_cast<uintptr_t>(send) % 16 == 0 &&
                  reinterpret_cast<uintptr_t>(meta) % 8 == 0,
              "16-byte aligned rows required");
  if (slots == 0) return STRIX_OK;
  const int chunks = int(hidden / 8);
  const int64_t work = slots * chunks;
  ep_pack_kernel<<<unsigned((work + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(x), x_stride / 8, static_cast<uint4*>(send), send_stride / 8,
      reinterpret_cast<float2*>(meta), order, topk_ids, topk_weights, slots, chunks, int(top_k),
      int(experts_per_rank), meta_stride / 2);
  return launch_status("ep_pack");
}

extern "C" int strix_moe_topk_softmax(const float* logits, int32_t* topk_ids, float* topk_weights,
                                      int64_t tokens, int64_t experts, int64_t top_k,
                                      int64_t logits_stride, int renormalize,
                                      strix_stream_t stream) {
  STRIX_CHECK(tokens >= 0 && experts >= 1 && experts <= 1024, "experts must be in 1..1024");
  STRIX_CHECK(top_k >= 1 && top_k <= 32 && top_k <= experts, "top_k must be in 1..min(32, experts)");
  STRIX_CHECK(logits_stride >= experts, "logits rows must not overlap");
  if (tokens == 0) return STRIX_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = unsigned((tokens + 3) / 4);
#define STRIX_TOPK(V)                                                                        \
  launch_chain(topk_softmax_kernel<V>, grid, 128, 0, st, logits, logits_stride, topk_ids, topk_weights, \
               int(tokens), int(experts), int(top_k), renormalize)
  if (experts <= 32) STRIX_TOPK(1);
  else if (experts <= 64) STRIX_TOPK(2);
  else if (experts <= 128) STRIX_TOPK(4);
  else if (experts <= 256) STRIX_TOPK(8);
  else if (experts <= 512) STRIX_TOPK(16);
  else STRIX_TOPK(32);
#undef STRIX_TOPK
  return launch_status("moe_topk_softmax");
}

extern "C" int64_t strix_moe_align_capacity(int64_t numel, int64_t experts, int64_t block_m) {
  if (numel < 0 || experts < 1 || block_m < 1) return -1;
  // every routed expert wastes at most block_m - 1 slots; at most min(numel, experts) are routed
  const int64_t routed = numel < experts ? numel : experts;
  const int64_t cap = numel + routed * (block_m - 1);
  return (cap + block_m - 1) / block_m * block_m;
}

extern "C" int strix_moe_align_pos(const int32_t* topk_ids, int32_t* sorted_ids,
                                   int32_t* expert_ids, int32_t* num_post_padded,
                                   int32_t* slot_pos, int64_t numel, int64_t experts,
                                   int64_t block_m, int64_t sorted_capacity,
                                   int64_t expert_capacity, strix_stream_t stream) {
  return strix_moe_align_counts(topk_ids, sorted_ids, expert_ids, num_post_padded, slot_pos, nullptr,
                                numel, experts, block_m, sorted_capacity, expert_capacity, stream);
}

extern "C" int strix_moe_align_counts(const int32_t* topk_ids, int32_t* sorted_ids,
                                      int32_t* expert_ids, int32_t* num_post_padded,
                                      int32_t* slot_pos, int32_t* counts, int64_t numel,
                                      int64_t experts, int64_t block_m, int64_t sorted_capacity,
                                      int64_t expert_capacity, strix_stream_t stream) {
  STRIX_CHECK(numel >= 0 && numel < (int64_t(1) << 30), "too many routed slots");
  STRIX_CHECK(experts >= 1 && experts <= 8192, "experts must be in 1..8192");
  STRIX_CHECK(block_m >= 1 && block_m <= 1024, "block_m must be in 1..1024");
  STRIX_CHECK(sorted_capacity >= strix_moe_align_capacity(numel, experts, block_m),
              "sorted_ids too short: needs strix_moe_align_capacity() entries");
  STRIX_CHECK(expert_capacity * block_m >= sorted_capacity,
              "expert_ids too short for block_m %lld", (long long)block_m);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  launch_chain(moe_align_kernel, unsigned(experts + 1), kAlignThreads, size_t(experts) * sizeof(int), st,
      topk_ids, sorted_ids, expert_ids, num_post_padded, int(numel), int(experts), int(block_m),
      int(sorted_capacity), int(expert_capacity), slot_pos, counts);
  return launch_status("moe_align");
}

extern "C" int64_t strix_moe_align_scratch_bytes(int64_t numel, int64_t experts) {
  if (numel < 0 || experts < 1) return -1;
  return ((numel + kChunkSlots - 1) / kChunkSlots) * experts * int64_t(sizeof(int32_t));
}

extern "C" int strix_moe_align_scratch(const int32_t* topk_ids, int32_t* sorted_ids,
                                       int32_t* expert_ids, int32_t* num_post_padded,
                                       int32_t* slot_pos, int32_t* counts, void* scratch,
                                       int64_t scratch_bytes, int64_t numel, int64_t experts,
                                       int64_t block_m, int64_t sorted_capacity,
                                       int64_t expert_capacity, strix_stream_t stream) {
  // few slots, or more experts than the ranking tables hold: the one-kernel form
  if (numel <= 4 * kChunkSlots || experts > kPlaceMaxExperts || scratch == nullptr)
    return strix_moe_align_counts(topk_ids, sorted_ids, expert_ids, num_post_padded, slot_pos, counts,
                                  numel, experts, block_m, sorted_capacity, expert_capacity, stream);
  STRIX_CHECK(numel < (int64_t(1) << 30), "too many routed slots");
  STRIX_CHECK(block_m >= 1 && block_m <= 1024, "block_m must be in 1..1024");
  STRIX_CHECK(sorted_capacity >= strix_moe_align_capacity(numel, experts, block_m),
              "sorted_ids too short: needs strix_moe_align_capacity() entries");
  STRIX_CHECK(expert_capacity * block_m >= sorted_capacity,
              "expert_ids too short for block_m %lld", (long long)block_m);
  STRIX_CHECK(scratch_bytes >= strix_moe_align_scratch_bytes(numel, experts) &&
                  reinterpret_cast<uintptr_t>(scratch) % 4 == 0, "scratch too small");
  const int chunks = int((numel + kChunkSlots - 1) / kChunkSlots);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int32_t* hist = static_cast<int32_t*>(scratch);
  launch_chain(moe_align_hist_kernel, unsigned(chunks), kPlaceThreads, size_t(experts) * sizeof(int), st,
      topk_ids, hist, int(numel), int(experts));
  if (int rc = launch_status("moe_align_hist")) return rc;
  const size_t smem = size_t(3 + kPlaceWarps) * size_t(experts) * sizeof(int);
  launch_chain(moe_align_place_kernel, unsigned(chunks), kPlaceThreads, smem, st,
      topk_ids, hist, sorted_ids, expert_ids, num_post_padded, int(numel), int(experts), int(block_m),
      int(sorted_capacity), int(expert_capacity), chunks, slot_pos, counts);
  return launch_status("moe_align_place");
}

extern "C" int strix_moe_align(const int32_t* topk_ids, int32_t* sorted_ids, int32_t* expert_ids,
                               int32_t* num_post_padded, int64_t numel, int64_t experts,
                               int64_t block_m, int64_t sorted_capacity, int64_t expert_capacity,
                               strix_stream_t stream) {
  return strix_moe_align_pos(topk_ids, sorted_ids, expert_ids, num_post_padded, nullptr, numel,
                             experts, block_m, sorted_capacity, expert_capacity, stream);
}

extern "C" int strix_moe_act_quant_fp8_scatter(const void* x, void* q, float* sa,
                                               const int32_t* slot_pos, const int32_t* sorted_ids,
                                               const int32_t* num_post_padded, int64_t tokens,
                                               int64_t rows, int64_t k, int64_t top_k,
                                               int64_t x_stride, int64_t q_stride,
                                               int64_t sa_stride, int x_is_f16,
                                               strix_stream_t stream) {
  STRIX_CHECK(slot_pos != nullptr && sorted_ids != nullptr && num_post_padded != nullptr,
              "slot_pos, sorted_ids and num_post_padded must not be NULL");
  STRIX_CHECK(tokens >= 0 && rows >= 0 && k > 0 && k % 128 == 0 && top_k >= 1,
              "K must be a multiple of 128");
  STRIX_CHECK(x_stride % 8 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 && q_stride % 8 == 0 &&
                  reinterpret_cast<uintptr_t>(q) % 8 == 0 && sa_stride >= k / 128,
              "16-byte aligned rows required");
  if (tokens == 0 && rows == 0) return STRIX_OK;
  const int groups = int(k / 128);
  const int64_t teams = (tokens + rows) * groups;
  const unsigned grid = unsigned((teams * 16 + 255) / 256);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto xp = static_cast<const uint16_t*>(x);
  auto qp = static_cast<uint8_t*>(q);
  const int64_t num_valid = tokens * top_k;
  if (x_is_f16)
    launch_chain(act_quant_scatter_kernel<true>, grid, 256, 0, st, xp, x_stride, qp, q_stride, sa, sa_stride, tokens, groups, int(top_k), slot_pos, sorted_ids, num_post_padded, rows, num_valid);
  else
    launch_chain(act_quant_scatter_kernel<false>, grid, 256, 0, st, xp, x_stride, qp, q_stride, sa, sa_stride, tokens, groups, int(top_k), slot_pos, sorted_ids, num_post_padded, rows, num_valid);
  return launch_status("moe_act_quant_scatter");
}

static int act_quant_common(const void* x, void* q, float* sa, int64_t rows, int64_t k,
                            int64_t x_stride, int64_t q_stride, int64_t sa_stride, int x_is_f16,
                            bool fp8, strix_stream_t stream, const int32_t* row_map = nullptr,
                            const int32_t* row_limit = nullptr, int top_k = 1,
                            int64_t num_valid = 0) {
  STRIX_CHECK(rows >= 0 && k > 0 && k % 128 == 0, "K must be a multiple of 128");
  STRIX_CHECK(x_stride % 8 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 &&
                  q_stride % 8 == 0 && reinterpret_cast<uintptr_t>(q) % 8 == 0,
              "16-byte aligned rows required");
  STRIX_CHECK(sa_stride >= k / 128, "sa must be [rows, K / 128]");
  if (rows == 0) return STRIX_OK;
  const int groups = int(k / 128);
  const int64_t teams = rows * groups;
  const unsigned grid = unsigned((teams * 16 + 255) / 256);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto xp = static_cast<const uint16_t*>(x);
  auto qp = static_cast<uint8_t*>(q);
  if (fp8) {
    if (x_is_f16) launch_chain(act_quant_kernel<true, true>, grid, 256, 0, st, xp, x_stride, qp, q_stride, sa, sa_stride, rows, groups, row_map, row_limit, top_k, num_valid);
    else launch_chain(act_quant_kernel<true, false>, grid, 256, 0, st, xp, x_stride, qp, q_stride, sa, sa_stride, rows, groups, row_map, row_limit, top_k, num_valid);
  } else {
    if (x_is_f16) launch_chain(act_quant_kernel<false, true>, grid, 256, 0, st, xp, x_stride, qp, q_stride, sa, sa_stride, rows, groups, row_map, row_limit, top_k, num_valid);
    else launch_chain(act_quant_kernel<false, false>, grid, 256, 0, st, xp, x_stride, qp, q_stride, sa, sa_stride, rows, groups, row_map, row_limit, top_k, num_valid);
  }
  return launch_status("moe_act_quant");
}

extern "C" int strix_moe_act_quant_i8(const void* x, void* q, float* sa, int64_t rows, int64_t k,
                                      int64_t x_stride, int64_t q_stride, int64_t sa_stride,
                                      int x_is_f16, strix_stream_t stream) {
  return act_quant_common(x, q, sa, rows, k, x_stride, q_stride, sa_stride, x_is_f16, false, stream);
}

extern "C" int strix_moe_act_quant_fp8(const void* x, void* q, float* sa, int64_t rows, int64_t k,
                                       int64_t x_stride, int64_t q_stride, int64_t sa_stride,
                                       int x_is_f16, strix_stream_t stream) {
  return act_quant_common(x, q, sa, rows, k, x_stride, q_stride, sa_stride, x_is_f16, true, stream);
}

extern "C" int strix_moe_act_quant_fp8_sorted(const void* x, void* q, float* sa,
                                              const int32_t* sorted_ids,
                                              const int32_t* num_post_padded, int64_t rows,
                                              int64_t k, int64_t top_k, int64_t num_valid,
                                              int64_t x_stride, int64_t q_stride,
                                              int64_t sa_stride, int x_is_f16,
                                              strix_stream_t stream) {
  STRIX_CHECK(num_post_padded != nullptr, "num_post_padded must not be NULL");
  STRIX_CHECK(top_k >= 1 && num_valid >= 0, "bad top_k / num_valid");
  return act_quant_common(x, q, sa, rows, k, x_stride, q_stride, sa_stride, x_is_f16, true, stream,
                          sorted_ids, num_post_padded, int(top_k), num_valid);
}

extern "C" int strix_moe_sum(const void* in, void* out, int64_t tokens, int64_t top_k,
                             int64_t hidden, int64_t in_st, int64_t in_sj, int64_t out_st,
                             strix_stream_t stream) {
  STRIX_CHECK(tokens >= 0 && top_k >= 1 && hidden > 0 && hidden % 8 == 0,
              "hidden must be a multiple of 8");
  STRIX_CHECK(in_st % 8 == 0 && in_sj % 8 == 0 && out_st % 8 == 0 &&
                  reinterpret_cast<uintptr_t>(in) % 16 == 0 &&
                  reinterpret_cast<uintptr_t>(out) % 16 == 0,
              "16-byte aligned rows required");
  if (tokens == 0) return STRIX_OK;
  const int64_t work = tokens * (hidden / 8);
  launch_chain(moe_sum_kernel, unsigned((work + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream),
      static_cast<const uint16_t*>(in), in_st, in_sj, static_cast<uint16_t*>(out), out_st,
      int(tokens), int(top_k), int(hidden / 8));
  return launch_status("moe_sum");
}
