// Expert-parallel token exchange over peer memory (NVLink), for sm_100a: the
// dispatch and combine of an MoE layer whose experts are sharded over the GPUs of
// one node, written as this library's own kernels instead of collective calls.
// The reference has no expert parallelism (its experts refuse an expert_map,
// python/strix_vllm/moe.py:193-210), so there is no counterpart to cite; the
// layer semantics are those of the single-GPU path (router -> experts -> sum).
//
// Every rank owns a set of buffers that its peers can address (CUDA IPC
// mappings of plain cudaMalloc memory; the kernels use ordinary st.global /
// ld.global on the mapped addresses - no multicast, no collective library):
//   recv   [world][cap][row_bytes]  payload rows, one region per source rank
//   meta   [world][cap][1 + 2 top_k] int32: source token, then per routed slot
//                                   (local expert id or -1, routing weight bits)
//   counts [world], flags [world]   rows written by each source, its epoch stamp
//   ret    [world][cap][hidden]     bf16 partial sums coming back, one region per
//                                   expert rank, indexed by the source's token
//   rflags [world]                  epoch stamp of each expert rank's return
// One layer = five kernels around the local expert GEMMs:
//   ep_plan      per destination rank, the tokens that have a slot there, in token
//                order (a token travels ONCE per destination however many of its
//                top-k experts live there) and their count;
//   ep_dispatch  copies each token's payload row (bf16 activations, or e4m3 bytes
//                plus per-128 scales when the layer quantises before dispatch)
//                and its metadata into every destination's recv / meta; the last
//                CTA publishes counts and flags (release, system scope);
//   ep_prepare   (receiver) waits for every source's flag - bounded, with a status
//                word - and lays out expert ids and weights per (row, slot), -1
//                past each source's count, ready for moe_align_block_size;
//   ep_return    (expert rank) sums a received token's result rows (its slots on
//                this rank, already weighted) in fp32 and writes one bf16 row into
//                the source's ret region; the last CTA publishes rflags;
//   ep_combine   (source) waits for every rank's return flag and sums a token's
//                partial rows over the ranks it was sent to.
// Flags carry a per-layer epoch that only grows, so nothing is reset between
// layers; a region is rewritten only after its reader has signalled (a rank
// starts layer L + 1 after its combine of layer L, which needs every peer's
// return of L, issued after that peer's last read of what layer L delivered).
#include <cstring>

#include "common.cuh"

namespace strix {
namespace {

constexpr int kEpMaxWorld = 16;
constexpr uint32_t kEpSpinDefault = 1u << 22;   // polls of ~0.5 us: about two seconds

struct EpPeers {
  uint8_t* recv[kEpMaxWorld];
  int32_t* meta[kEpMaxWorld];
  int32_t* counts[kEpMaxWorld];
  int32_t* flags[kEpMaxWorld];
  uint8_t* ret[kEpMaxWorld];
  int32_t* rflags[kEpMaxWorld];
};

__device__ int32_t g_ep_status = 0;    // 0 healthy, 1 a dispatch wait gave up, 2 a return wait

__device__ __forceinline__ int32_t ld_acquire_sys(const int32_t* p) {
  int32_t v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(int32_t* p, int32_t v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Waits until *flag >= epoch; false when the limit ran out.
__device__ __forceinline__ bool wait_epoch(const int32_t* flag, int32_t epoch, uint32_t limit) {
  for (uint32_t i = 0; i < limit; ++i) {
    if (ld_acquire_sys(flag) - epoch >= 0) return true;
    __nanosleep(200);
  }
  return false;
}

// Which rank owns global expert e, and under which local index. experts_per_rank > 0:
// contiguous blocks (rank r owns [r * epr, (r + 1) * epr)); < 0: round-robin (expert e
// lives on rank e mod world as local expert e / world, -epr experts per rank), which
// spreads a load that is skewed along the expert index evenly over the ranks.
// With a placement table (device memory: [0] = global experts, [1] = row stride, then
// per expert a row {copies, rank << 16 | local id, ...}) the owner is looked up, and an
// expert that has several copies (a hot expert replicated to balance the ranks) serves
// token t from copy t mod copies. Returns rank << 16 | local id, or -1.
__device__ __forceinline__ int ep_where(int e, int t, int epr, int world, const int32_t* __restrict__ table) {
  if (e < 0) return -1;
  if (table != nullptr) {
    if (e >= table[0]) return -1;
    const int32_t* row = table + 2 + int64_t(e) * table[1];
    const int copies = row[0];
    return copies > 0 ? row[1 + t % copies] : -1;
  }
  if (epr > 0) return e / epr < world ? ((e / epr) << 16) | (e % epr) : -1;
  return e < -epr * world ? ((e % world) << 16) | (e / world) : -1;
}

// One CTA per destination rank: tok_pos[d][t] = index of token t among this
// rank's tokens with a slot on rank d (token order), or -1; counts[d].
__global__ void __launch_bounds__(256) ep_plan_kernel(const int32_t* __restrict__ topk_ids,
                                                      int32_t* __restrict__ tok_pos,
                                                      int32_t* __restrict__ counts, int tokens,
                                                      int top_k, int experts_per_rank, int world,
                                                      const int32_t* __restrict__ placement) {
  pdl_enter();
  __shared__ int s_warp[8];
  const int d = blockIdx.x, tid = threadIdx.x;
  int placed = 0;
  for (int start = 0; start < tokens; start += 256) {
    const int t = start + tid;
    bool hit = false;
    if (t < tokens)
      for (int j = 0; j < top_k; ++j) {
        const int e = topk_ids[t * top_k + j];
        const int w = ep_where(e, t, experts_per_rank, world, placement);
        hit = hit || (w >= 0 && (w >> 16) == d);
      }
    const unsigned bal = __ballot_sync(0xffffffffu, hit);
    __syncthreads();
    if ((tid & 31) == 0) s_warp[tid >> 5] = __popc(bal);
    __syncthreads();
    int before = 0, total = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      const int c = s_warp[w];
      before += w < (tid >> 5) ? c : 0;
      total += c;
    }
    if (t < tokens)
      tok_pos[int64_t(d) * tokens + t] = hit ? placed + before + __popc(bal & ((1u << (tid & 31)) - 1u)) : -1;
    placed += total;
  }
  if (tid == 0) counts[d] = placed;
}

// Raises this grid's flags once every CTA has passed: a CTA's stores are ordered
// before its ticket by a barrier and ONE system-scope fence of thread 0 (fences are
// cumulative over what the barrier made visible to that thread), and the CTA that
// draws the last ticket publishes.
template <class Publish>
__device__ __forceinline__ void publish_when_last(int32_t* ticket, Publish publish) {
  __shared__ int s_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    s_last = atomicAdd(ticket, 1) == int(gridDim.x) - 1;
  }
  __syncthreads();
  if (!s_last) return;
  if (threadIdx.x == 0) __threadfence_system();
  __syncthreads();
  publish();
  if (threadIdx.x == 0) *ticket = 0;
}

constexpr int kEpWarps = 8;   // warps per CTA of the row-copy kernels (a warp = one row at a time)

// A warp = one token at a time: its payload row goes to every destination the token
// has a slot on (16-byte chunks, lane-strided); lane 0 also writes the row's metadata.
__global__ void __launch_bounds__(kEpWarps * 32) ep_dispatch_kernel(
    const uint4* __restrict__ x, int64_t x_st16, const int32_t* __restrict__ topk_ids,
    const float* __restrict__ topk_w, const int32_t* __restrict__ tok_pos,
    const int32_t* __restrict__ counts, const EpPeers peers, int32_t* __restrict__ ticket,
    int tokens, int chunks, int top_k, int experts_per_rank, int world, int rank, int64_t cap,
    const int32_t* __restrict__ placement,
    int32_t epoch) {
  pdl_enter();
  const int lane = threadIdx.x & 31;
  const int warps = gridDim.x * kEpWarps;
  const int meta_st = 1 + 2 * top_k;
  for (int t = blockIdx.x * kEpWarps + (threadIdx.x >> 5); t < tokens; t += warps) {
    for (int d = 0; d < world; ++d) {
      const int pos = tok_pos[int64_t(d) * tokens + t];
      if (pos < 0 || pos >= cap) continue;
      const int64_t row = int64_t(rank) * cap + pos;
      uint4* dst = reinterpret_cast<uint4*>(peers.recv[d]) + row * chunks;
      const uint4* src = x + int64_t(t) * x_st16;
      for (int ch = lane; ch < chunks; ch += 32) dst[ch] = src[ch];
      if (lane <= top_k) {
        int32_t* m = peers.meta[d] + row * meta_st;
        if (lane == 0) {
          m[0] = t;
        } else {
          const int j = lane - 1;
          const int e = topk_ids[t * top_k + j];
          const int w = ep_where(e, t, experts_per_rank, world, placement);
          m[1 + 2 * j] = (w >= 0 && (w >> 16) == d) ? (w & 0xffff) : -1;
          m[2 + 2 * j] = __float_as_int(topk_w[t * top_k + j]);
        }
      }
    }
  }
  publish_when_last(ticket, [&] {
    if (threadIdx.x < world) {
      const int d = threadIdx.x;
      peers.counts[d][rank] = min(counts[d], int(cap));
      __threadfence_system();
      st_release_sys(peers.flags[d] + rank, epoch);
    }
  });
}

// Receiver: ids / weights per (row, slot) for the rows that arrived, -1 elsewhere.
// (meta and counts are written by the peers while this kernel waits: they are read
// with ld.global.cg after the flag, never through the non-coherent path)
__global__ void __launch_bounds__(256) ep_prepare_kernel(
    const int32_t* meta, const int32_t* counts, const int32_t* flags, int32_t* __restrict__ ids,
    float* __restrict__ wts,
    int32_t* __restrict__ rows_out, int world, int64_t cap, int top_k, int32_t epoch,
    uint32_t spin_limit) {
  pdl_enter();
  __shared__ int s_ok;
  const int64_t first = int64_t(blockIdx.x) * 256, total = int64_t(world) * cap * top_k;
  if (threadIdx.x == 0) {
    const int64_t last = min(first + 255, total - 1);
    bool ok = true;
    for (int s = int(first / (cap * top_k)); s <= int(last / (cap * top_k)); ++s)
      ok = wait_epoch(flags + s, epoch, spin_limit) && ok;
    if (!ok) atomicExch(&g_ep_status, 1);
    s_ok = ok;
  }
  __syncthreads();
  const int64_t idx = first + threadIdx.x;
  if (idx >= total) return;
  const int64_t row = idx / top_k;
  const int j = int(idx % top_k);
  const int src = int(row / cap), pos = int(row % cap);
  const int n = s_ok ? __ldcg(counts + src) : 0;
  const int32_t* m = meta + row * (1 + 2 * top_k);
  const bool live = pos < n;
  ids[idx] = live ? __ldcg(m + 1 + 2 * j) : -1;
  wts[idx] = live ? __int_as_float(__ldcg(m + 2 + 2 * j)) : 0.f;
  if (rows_out != nullptr && pos == 0 && j == 0) rows_out[src] = n;
}

// Expert rank: one bf16 row per received token = the fp32 sum of its result rows
// here, written into the source rank's ret region at the source's token index.
// A warp = one received row at a time (rows nothing arrived in cost one compare).
__global__ void __launch_bounds__(kEpWarps * 32) ep_return_kernel(
    const uint16_t* __restrict__ y, int64_t y_st, const int32_t* __restrict__ ids,
    const int32_t* __restrict__ meta, const int32_t* __restrict__ counts, const EpPeers peers,
    int32_t* __restrict__ ticket, int world, int rank, int64_t cap, int top_k, int hidden8,
    int32_t epoch) {
  pdl_enter();
  const int lane = threadIdx.x & 31;
  const int warps = gridDim.x * kEpWarps;
  const int64_t rows = int64_t(world) * cap;
  for (int64_t row = blockIdx.x * kEpWarps + (threadIdx.x >> 5); row < rows; row += warps) {
    const int src = int(row / cap), pos = int(row % cap);
    if (pos >= counts[src]) continue;
    const int tok = meta[row * (1 + 2 * top_k)];
    uint16_t* dst = reinterpret_cast<uint16_t*>(peers.ret[src]) + (int64_t(rank) * cap + tok) * (int64_t(hidden8) * 8);
    for (int c = lane; c < hidden8; c += 32) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int j = 0; j < top_k; ++j) {
        if (ids[row * top_k + j] < 0) continue;
        const uint4 w = *reinterpret_cast<const uint4*>(y + (row * top_k + j) * y_st + c * 8);
        const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[2 * i] += bf16_lo(ws[i]), acc[2 * i + 1] += bf16_hi(ws[i]);
      }
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]), o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]), o.w = pack_bf16x2(acc[6], acc[7]);
      *reinterpret_cast<uint4*>(dst + c * 8) = o;
    }
  }
  publish_when_last(ticket, [&] {
    if (threadIdx.x < world) st_release_sys(peers.rflags[threadIdx.x] + rank, epoch);
  });
}

// Source rank: out[t] = sum over the ranks token t was sent to of their partial rows.
// A warp = one token at a time. (ret is written by the peers while this kernel waits:
// it is read with ld.global.cg after the flags, never through the non-coherent path.)
__global__ void __launch_bounds__(kEpWarps * 32) ep_combine_kernel(
    const uint16_t* ret, const int32_t* rflags, const int32_t* __restrict__ tok_pos,
    uint16_t* __restrict__ out, int64_t out_st, int tokens, int hidden8, int world, int64_t cap,
    int32_t epoch, uint32_t spin_limit) {
  pdl_enter();
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    bool ok = true;
    for (int d = 0; d < world; ++d) ok = wait_epoch(rflags + d, epoch, spin_limit) && ok;
    if (!ok) atomicExch(&g_ep_status, 2);
    s_ok = ok;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int warps = gridDim.x * kEpWarps;
  for (int t = blockIdx.x * kEpWarps + (threadIdx.x >> 5); t < tokens; t += warps) {
    unsigned from = 0;
    if (s_ok)
      for (int d = 0; d < world; ++d) from |= tok_pos[int64_t(d) * tokens + t] >= 0 ? 1u << d : 0u;
    for (int c = lane; c < hidden8; c += 32) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int d = 0; d < world; ++d) {
        if (!(from >> d & 1)) continue;
        const uint4 w = __ldcg(reinterpret_cast<const uint4*>(ret + (int64_t(d) * cap + t) * (int64_t(hidden8) * 8) + c * 8));
        const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[2 * i] += bf16_lo(ws[i]), acc[2 * i + 1] += bf16_hi(ws[i]);
      }
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]), o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]), o.w = pack_bf16x2(acc[6], acc[7]);
      *reinterpret_cast<uint4*>(out + int64_t(t) * out_st + c * 8) = o;
    }
  }
}

// Byte rows into sorted order by scatter (the byte twin of moe_permute_bf16):
// row r goes to the sorted positions of its top_k slots; padding positions below
// *num_post get zeros.
__global__ void __launch_bounds__(256) permute_byte_rows_kernel(
    const uint4* __restrict__ x, int64_t x_st16, uint4* __restrict__ y, int64_t y_st16, int64_t rows,
    int chunks, int top_k, const int32_t* __restrict__ slot_pos, const int32_t* __restrict__ sorted_ids,
    const int32_t* __restrict__ num_post, int64_t rows_cap, int64_t num_valid) {
  pdl_enter();
  const int64_t idx = int64_t(blockIdx.x) * 256 + threadIdx.x;
  const int64_t row = idx / chunks;
  const int ch = int(idx % chunks);
  if (row < rows) {
    bool any = false;
    for (int j = 0; j < top_k; ++j) any = any || slot_pos[row * top_k + j] >= 0;
    if (!any) return;                      // rows nobody routed here are not even read
    const uint4 v = x[row * x_st16 + ch];
    for (int j = 0; j < top_k; ++j) {
      const int pos = slot_pos[row * top_k + j];
      if (pos >= 0 && pos < rows_cap) y[int64_t(pos) * y_st16 + ch] = v;
    }
    return;
  }
  const int64_t r = row - rows;
  if (r >= rows_cap || r >= *num_post) return;
  const int64_t sid = sorted_ids[r];
  if (sid >= 0 && sid < num_valid) return;
  y[r * y_st16 + ch] = make_uint4(0u, 0u, 0u, 0u);
}

// CTAs of a row-copy kernel: enough warps for the rows, at most eight CTAs per SM
unsigned row_grid(int64_t rows) {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      sms = 148;
  }
  const int64_t want = (rows + kEpWarps - 1) / kEpWarps;
  return unsigned(want < 1 ? 1 : want > int64_t(sms) * 8 ? int64_t(sms) * 8 : want);
}

int fill_peers(EpPeers* p, void* const* recv, void* const* meta, void* const* counts, void* const* flags,
               void* const* ret, void* const* rflags, int64_t world) {
  STRIX_CHECK(world >= 1 && world <= kEpMaxWorld, "world size must be in 1..%d", kEpMaxWorld);
  for (int i = 0; i < world; ++i) {
    STRIX_CHECK((recv == nullptr || recv[i]) && (meta == nullptr || meta[i]) &&
                    (counts == nullptr || counts[i]) && (flags == nullptr || flags[i]) &&
                    (ret == nullptr || ret[i]) && (rflags == nullptr || rflags[i]),
                "peer pointer %d is NULL", i);
    p->recv[i] = recv ? static_cast<uint8_t*>(recv[i]) : nullptr;
    p->meta[i] = meta ? static_cast<int32_t*>(meta[i]) : nullptr;
    p->counts[i] = counts ? static_cast<int32_t*>(counts[i]) : nullptr;
    p->flags[i] = flags ? static_cast<int32_t*>(flags[i]) : nullptr;
    p->ret[i] = ret ? static_cast<uint8_t*>(ret[i]) : nullptr;
    p->rflags[i] = rflags ? static_cast<int32_t*>(rflags[i]) : nullptr;
  }
  return STRIX_OK;
}

}  // namespace
}  // namespace strix

using namespace strix;

// ------------------------------------------------------------ peer memory
extern "C" int strix_peer_alloc(void** ptr, int64_t bytes) {
  STRIX_CHECK(ptr != nullptr && bytes > 0, "bad arguments");
  STRIX_CUDA(cudaMalloc(ptr, size_t(bytes)));
  STRIX_CUDA(cudaMemset(*ptr, 0, size_t(bytes)));
  STRIX_CUDA(cudaDeviceSynchronize());
  return STRIX_OK;
}

extern "C" int strix_peer_free(void* ptr) {
  if (ptr != nullptr) STRIX_CUDA(cudaFree(ptr));
  return STRIX_OK;
}

extern "C" int strix_peer_export(const void* ptr, void* handle64) {
  STRIX_CHECK(ptr != nullptr && handle64 != nullptr, "bad arguments");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handles are 64 bytes");
  STRIX_CUDA(cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(handle64), const_cast<void*>(ptr)));
  return STRIX_OK;
}

extern "C" int strix_peer_import(const void* handle64, void** ptr) {
  STRIX_CHECK(ptr != nullptr && handle64 != nullptr, "bad arguments");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  STRIX_CUDA(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return STRIX_OK;
}

extern "C" int strix_peer_unimport(void* ptr) {
  if (ptr != nullptr) STRIX_CUDA(cudaIpcCloseMemHandle(ptr));
  return STRIX_OK;
}

extern "C" int strix_ep_status(int32_t* host_out, int reset) {
  STRIX_CHECK(host_out != nullptr, "host_out must not be NULL");
  STRIX_CUDA(cudaMemcpyFromSymbol(host_out, strix::g_ep_status, sizeof(int32_t)));
  if (reset) {
    const int32_t zero = 0;
    STRIX_CUDA(cudaMemcpyToSymbol(strix::g_ep_status, &zero, sizeof(zero)));
  }
  return STRIX_OK;
}

// ------------------------------------------------------------------ kernels
extern "C" int strix_ep_plan(const int32_t* topk_ids, int32_t* tok_pos, int32_t* counts, int64_t tokens,
                             int64_t top_k, int64_t experts_per_rank, int64_t world,
                             const int32_t* placement, strix_stream_t stream) {
  STRIX_CHECK(counts != nullptr && (tokens == 0 || (topk_ids != nullptr && tok_pos != nullptr)),
              "pointers must not be NULL");
  STRIX_CHECK(tokens >= 0 && top_k >= 1 && experts_per_rank != 0 && world >= 1 && world <= kEpMaxWorld,
              "bad sizes");
  launch_chain(ep_plan_kernel, unsigned(world), 256, 0, static_cast<cudaStream_t>(stream), 
      topk_ids, tok_pos, counts, int(tokens), int(top_k), int(experts_per_rank), int(world), placement);
  return launch_status("ep_plan");
}

extern "C" int strix_ep_dispatch(const void* x, const int32_t* topk_ids, const float* topk_weights,
                                 const int32_t* tok_pos, const int32_t* counts, void* const* peer_recv,
                                 void* const* peer_meta, void* const* peer_counts, void* const* peer_flags,
                                 int32_t* ticket, int64_t tokens, int64_t row_bytes, int64_t x_stride_bytes,
                                 int64_t top_k, int64_t experts_per_rank, int64_t world, int64_t rank,
                                 int64_t cap, int64_t epoch, const int32_t* placement,
                                 strix_stream_t stream) {
  STRIX_CHECK(counts != nullptr && ticket != nullptr &&
                  (tokens == 0 || (x != nullptr && topk_ids != nullptr && topk_weights != nullptr &&
                                   tok_pos != nullptr)), "pointers must not be NULL");
  STRIX_CHECK(row_bytes > 0 && row_bytes % 16 == 0 && x_stride_bytes % 16 == 0 &&
                  reinterpret_cast<uintptr_t>(x) % 16 == 0, "payload rows must be whole 16-byte chunks");
  STRIX_CHECK(tokens >= 0 && tokens <= cap && rank >= 0 && rank < world && top_k >= 1 && top_k <= 31,
              "tokens must fit the buffer capacity");
  EpPeers peers;
  if (int rc = fill_peers(&peers, peer_recv, peer_meta, peer_counts, peer_flags, nullptr, nullptr, world)) return rc;
  const int chunks = int(row_bytes / 16);
  // an empty rank still raises its flags
  const unsigned grid = row_grid(tokens);
  launch_chain(ep_dispatch_kernel, grid, kEpWarps * 32, 0, static_cast<cudaStream_t>(stream), 
      static_cast<const uint4*>(x), x_stride_bytes / 16, topk_ids, topk_weights, tok_pos, counts, peers,
      ticket, int(tokens), chunks, int(top_k), int(experts_per_rank), int(world), int(rank), cap,
      placement, int32_t(epoch));
  return launch_status("ep_dispatch");
}

extern "C" int strix_ep_prepare(const int32_t* meta, const int32_t* counts, const int32_t* flags,
                                int32_t* ids, float* weights, int32_t* rows_per_source, int64_t world,
                                int64_t cap, int64_t top_k, int64_t epoch, int64_t spin_limit,
                                strix_stream_t stream) {
  STRIX_CHECK(meta != nullptr && counts != nullptr && flags != nullptr && ids != nullptr && weights != nullptr,
              "pointers must not be NULL");
  STRIX_CHECK(world >= 1 && world <= kEpMaxWorld && cap >= 1 && top_k >= 1, "bad sizes");
  const int64_t total = world * cap * top_k;
  launch_chain(ep_prepare_kernel, unsigned((total + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream), 
      meta, counts, flags, ids, weights, rows_per_source, int(world), cap, int(top_k), int32_t(epoch),
      spin_limit > 0 ? uint32_t(spin_limit) : kEpSpinDefault);
  return launch_status("ep_prepare");
}

extern "C" int strix_ep_return(const void* y, const int32_t* ids, const int32_t* meta, const int32_t* counts,
                               void* const* peer_ret, void* const* peer_rflags, int32_t* ticket,
                               int64_t world, int64_t rank, int64_t cap, int64_t top_k, int64_t hidden,
                               int64_t y_stride, int64_t epoch, strix_stream_t stream) {
  STRIX_CHECK(y != nullptr && ids != nullptr && meta != nullptr && counts != nullptr && ticket != nullptr,
              "pointers must not be NULL");
  STRIX_CHECK(hidden > 0 && hidden % 8 == 0 && y_stride % 8 == 0 && reinterpret_cast<uintptr_t>(y) % 16 == 0,
              "hidden must be a multiple of 8");
  EpPeers peers;
  if (int rc = fill_peers(&peers, nullptr, nullptr, nullptr, nullptr, peer_ret, peer_rflags, world)) return rc;
  STRIX_CHECK(rank >= 0 && rank < world && cap >= 1, "bad rank");
  launch_chain(ep_return_kernel, row_grid(world * cap), kEpWarps * 32, 0, static_cast<cudaStream_t>(stream), 
      static_cast<const uint16_t*>(y), y_stride, ids, meta, counts, peers, ticket, int(world), int(rank),
      cap, int(top_k), int(hidden / 8), int32_t(epoch));
  return launch_status("ep_return");
}

extern "C" int strix_ep_combine(const void* ret, const int32_t* rflags, const int32_t* tok_pos, void* out,
                                int64_t tokens, int64_t hidden, int64_t out_stride, int64_t world,
                                int64_t cap, int64_t epoch, int64_t spin_limit, strix_stream_t stream) {
  STRIX_CHECK(ret != nullptr && rflags != nullptr && (tokens == 0 || (tok_pos != nullptr && out != nullptr)),
              "pointers must not be NULL");
  STRIX_CHECK(hidden > 0 && hidden % 8 == 0 && out_stride % 8 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0,
              "hidden must be a multiple of 8");
  STRIX_CHECK(tokens >= 0 && tokens <= cap && world >= 1 && world <= kEpMaxWorld, "bad sizes");
  launch_chain(ep_combine_kernel, row_grid(tokens), kEpWarps * 32, 0, static_cast<cudaStream_t>(stream), 
      static_cast<const uint16_t*>(ret), rflags, tok_pos, static_cast<uint16_t*>(out), out_stride, int(tokens),
      int(hidden / 8), int(world), cap, int32_t(epoch), spin_limit > 0 ? uint32_t(spin_limit) : kEpSpinDefault);
  return launch_status("ep_combine");
}

extern "C" int strix_moe_permute_rows(const void* x, void* y, const int32_t* slot_pos,
                                      const int32_t* sorted_ids, const int32_t* num_post_padded,
                                      int64_t rows, int64_t sorted_rows, int64_t row_bytes, int64_t top_k,
                                      int64_t x_stride_bytes, int64_t y_stride_bytes, strix_stream_t stream) {
  STRIX_CHECK(slot_pos != nullptr && sorted_ids != nullptr && num_post_padded != nullptr,
              "slot_pos, sorted_ids and num_post_padded must not be NULL");
  STRIX_CHECK(rows >= 0 && sorted_rows >= 0 && row_bytes > 0 && row_bytes % 16 == 0 && top_k >= 1,
              "rows must be whole 16-byte chunks");
  STRIX_CHECK(x_stride_bytes % 16 == 0 && y_stride_bytes % 16 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 &&
                  reinterpret_cast<uintptr_t>(y) % 16 == 0, "16-byte aligned rows required");
  if (rows + sorted_rows == 0) return STRIX_OK;
  const int chunks = int(row_bytes / 16);
  const int64_t threads = (rows + sorted_rows) * chunks;
  launch_chain(permute_byte_rows_kernel, unsigned((threads + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream), 
      static_cast<const uint4*>(x), x_stride_bytes / 16, static_cast<uint4*>(y), y_stride_bytes / 16, rows,
      chunks, int(top_k), slot_pos, sorted_ids, num_post_padded, sorted_rows, rows * top_k);
  return launch_status("moe_permute_rows");
}
