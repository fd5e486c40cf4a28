// Dense W8A8 INT8 GEMM on the Blackwell tensor cores (tcgen05.mma kind::i8,
// int32 accumulators in TMEM), for sm_100a:
//
//     out[m, n] = bf16( (sum_k a[m, k] * w[n, k]) * a_scale[m] * w_scale[n] )
//
// with int8 activations a [M, K] (one fp32 scale per token), int8 weights
// w [N, K] (one fp32 scale per output channel) and an int32-exact sum. This is
// the per-token form of the reference's w8a8_wmma_gemm
// (csrc/gemm/w8a8_wmma_gemm.hip:15-22, which quantises per 128-wide group
// inside the op); the int32 accumulators can be written out as well, so tests
// can compare them bit for bit.
//
// Both operands are K-major row matrices, so one kernel serves two
// orientations of the 128 x NB accumulator tile:
//   * M >= 128: A = 128 tokens, B = 256 weight rows; a thread of the epilogue
//     owns one token and writes 256 consecutive outputs;
//   * small M (decode): the operands swap - A = 128 weight rows (they fill the
//     MMA's M dimension whatever the batch), B = the tokens padded to 16/32/64;
//     the kernel is then a pure weight stream (HBM-bound).
// One persistent CTA per SM: one producing thread (TMA boxes of 128 bytes x
// rows with the 128-byte swizzle into a ring of stages), one issuing thread,
// 4 epilogue warps; two TMEM accumulators so a tile's epilogue overlaps the
// next tile's MMAs. Every mbarrier wait is bounded.
#include <cstdlib>

#include "tma.cuh"

namespace strix {
namespace {

using namespace umma;

constexpr int kGEpilogueWarps = 4;             // warps 2..5; warp 0 produces, warp 1 issues
constexpr int kGThreads = (kGEpilogueWarps + 2) * 32;
constexpr int kGKBlock = 128;

struct GemmArgs {
  __nv_bfloat16* out;      // [M, N]
  int32_t* acc_out;        // optional [M, N] int32 accumulators, or NULL
  const float* a_scale;    // per A row
  const float* b_scale;    // per B row
  int32_t* status;
  int64_t out_stride;
  int a_rows, b_rows, K;
  int a_tiles, b_tiles;
  int swap;                // 1: A rows are output columns (weights), B rows are tokens
};

template <int NB>
struct GemmLayout {
  static constexpr int kABytes = 128 * kGKBlock;
  static constexpr int kBBytes = NB * kGKBlock;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (208 * 1024) / kStageBytes > 12 ? 12 : (208 * 1024) / kStageBytes;
  static constexpr int kTmemCols = 2 * NB < 32 ? 32 : 2 * NB;
  static constexpr int kSmem = 1024 + kStages * kStageBytes + 256;
};

template <int NB>
__global__ void __launch_bounds__(kGThreads, 1) gemm_w8a8_umma_kernel(const GemmArgs p,
                                                                     const __grid_constant__ CUtensorMap map_a,
                                                                     const __grid_constant__ CUtensorMap map_b) {
  using L = GemmLayout<NB>;
  constexpr int S = L::kStages;
  extern __shared__ uint8_t raw_smem[];
  uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) &
                                             ~uintptr_t(1023));
  __shared__ __align__(8) uint64_t full_bar[S], empty_bar[S], tfull_bar[2], tempty_bar[2], drain_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int armed = 0;   // producer thread: stages it handed to the TMA (read at teardown)
  const int nkb = p.K / kGKBlock;
  const int total_items = p.a_tiles * p.b_tiles;

  if (tid == 0) {
    for (int i = 0; i < S; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull_bar[i], 1);
      mbar_init(&tempty_bar[i], kGEpilogueWarps);
    }
    mbar_init(&drain_bar, 1);
    s_abort = 0;
    fence_mbar_init();
  }
  if (warp == 1) tmem_alloc(&tmem_slot, L::kTmemCols);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_slot;
  const uint32_t ring_s = smem_u32(ring);

  if (warp == 0) {
    // ------------------------------------------------------------- producer
    if (lane == 0) {
      tma::prefetch_map(&map_a);
      tma::prefetch_map(&map_b);
      bool dead = false;
      int t = 0;
      for (int item = blockIdx.x; item < total_items && !dead; item += gridDim.x) {
        const int bt = item / p.a_tiles, at = item - bt * p.a_tiles;
        for (int kb = 0; kb < nkb; ++kb, ++t) {
          const int s = t % S;
          if (!mbar_wait(&empty_bar[s], ((t / S) & 1) ^ 1) || s_abort) {   // the MMAs have read it
            dead = true;
            break;
          }
          const uint32_t st = ring_s + s * L::kStageBytes;
          tma::mbar_expect_tx(&full_bar[s], L::kStageBytes);
          tma::load_2d(st, &map_a, kb * kGKBlock, at * 128, &full_bar[s]);
          tma::load_2d(st + L::kABytes, &map_b, kb * kGKBlock, bt * NB, &full_bar[s]);
        }
      }
      armed = t;
      if (dead) atomicExch(p.status, 1), s_abort = 1;
    }
  } else if (warp == 1) {
    // --------------------------------------------------------------- issuer
    if (lane == 0) {
      const uint32_t idesc = instr_desc(D_S32, 1, 1, 128, NB);
      const uint32_t a_lo0 = smem_desc_lo(ring_s);
      int t = 0, li = 0;
      bool dead = false;
      for (int item = blockIdx.x; item < total_items && !dead; item += gridDim.x, ++li) {
        const int buf = li & 1;
        if (!mbar_wait(&tempty_bar[buf], ((li >> 1) & 1) ^ 1)) {  // epilogue drained it
          dead = true;
          break;
        }
        for (int kb = 0; kb < nkb; ++kb, ++t) {
          const int s = t % S;
          if (!mbar_wait(&full_bar[s], (t / S) & 1) || s_abort) {
            dead = true;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_lo = a_lo0 + s * (L::kStageBytes >> 4), b_lo = a_lo + (L::kABytes >> 4);
          const uint32_t d = tmem + buf * NB;
          if (kb == 0) mma_ss_lo<KIND_I8, false>(d, a_lo, b_lo, idesc);
          else mma_ss_lo<KIND_I8, true>(d, a_lo, b_lo, idesc);
          mma_ss_lo<KIND_I8, true>(d, a_lo + 2, b_lo + 2, idesc);
          mma_ss_lo<KIND_I8, true>(d, a_lo + 4, b_lo + 4, idesc);
          mma_ss_lo<KIND_I8, true>(d, a_lo + 6, b_lo + 6, idesc);
          mma_commit(&empty_bar[s]);
        }
        if (!dead) mma_commit(&tfull_bar[buf]);   // the tile's sums are complete
      }
      if (dead) atomicExch(p.status, 1), s_abort = 1;
    }
  } else {
    // ------------------------------------------------------------- epilogue
    const int ctid = (warp & 3) * 32 + lane;              // TMEM lane = A row of the tile
    const uint32_t lane_base = uint32_t((warp & 3) * 32) << 16;
    constexpr int CH = NB < 32 ? NB : 32;
    int li = 0;
    bool dead = false;
    for (int item = blockIdx.x; item < total_items && !dead; item += gridDim.x, ++li) {
      const int bt = item / p.a_tiles, at = item - bt * p.a_tiles;
      const int buf = li & 1;
      const int row_a = at * 128 + ctid;
      const bool row_ok = row_a < p.a_rows;
      const float sa = row_ok ? __ldg(p.a_scale + row_a) : 0.f;
      const bool ok = mbar_wait(&tfull_bar[buf], (li >> 1) & 1);
      if (__any_sync(0xffffffffu, !ok) || s_abort) {
        dead = true;
        break;
      }
      tc_fence_after_sync();
#pragma unroll 1
      for (int c0 = 0; c0 < NB; c0 += CH) {
        __syncwarp();
        uint32_t r[CH];
        if constexpr (CH == 32) tmem_ld_32x32(tmem + lane_base + buf * NB + c0, r);
        else tmem_ld_32x16(tmem + lane_base + buf * NB + c0, r);
        tmem_ld_wait();
        if (c0 + CH >= NB) {   // everything read: the issuer may reuse this accumulator
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tempty_bar[buf]);
        }
        const int col0 = bt * NB + c0;
        if (!row_ok) {
          // a padding row of the tile: nothing to write (the warp stays together
          // for the next chunk's collective TMEM load)
        } else if (p.swap) {
          // A rows are output columns: out[token = col0 + j][n = row_a]
#pragma unroll
          for (int j = 0; j < CH; ++j) {
            const int tok = col0 + j;
            if (tok >= p.b_rows) continue;
            // (sum * token scale) * channel scale, the order of the other orientation
            const float v = float(int(r[j])) * __ldg(p.b_scale + tok) * sa;
            p.out[int64_t(tok) * p.out_stride + row_a] = __float2bfloat16_rn(v);
            if (p.acc_out) p.acc_out[int64_t(tok) * p.out_stride + row_a] = int(r[j]);
          }
        } else {
          // A rows are tokens: this thread writes CH consecutive outputs of its row
          __nv_bfloat16* orow = p.out + int64_t(row_a) * p.out_stride + col0;
          if (col0 + CH <= p.b_rows) {
#pragma unroll
            for (int j = 0; j < CH; j += 8) {
              const float4 s0 = __ldg(reinterpret_cast<const float4*>(p.b_scale + col0 + j));
              const float4 s1 = __ldg(reinterpret_cast<const float4*>(p.b_scale + col0 + j + 4));
              uint4 o;
              o.x = pack_bf16x2(float(int(r[j])) * sa * s0.x, float(int(r[j + 1])) * sa * s0.y);
              o.y = pack_bf16x2(float(int(r[j + 2])) * sa * s0.z, float(int(r[j + 3])) * sa * s0.w);
              o.z = pack_bf16x2(float(int(r[j + 4])) * sa * s1.x, float(int(r[j + 5])) * sa * s1.y);
              o.w = pack_bf16x2(float(int(r[j + 6])) * sa * s1.z, float(int(r[j + 7])) * sa * s1.w);
              *reinterpret_cast<uint4*>(orow + j) = o;
            }
          } else {
#pragma unroll
            for (int j = 0; j < CH; ++j)
              if (col0 + j < p.b_rows)
                orow[j] = __float2bfloat16_rn(float(int(r[j])) * sa * __ldg(p.b_scale + col0 + j));
          }
          if (p.acc_out) {
            int32_t* arow = p.acc_out + int64_t(row_a) * p.out_stride + col0;
#pragma unroll
            for (int j = 0; j < CH; ++j)
              if (col0 + j < p.b_rows) arow[j] = int(r[j]);
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
  if (warp == 1) tmem_dealloc(tmem, L::kTmemCols);
}

// Dynamic per-token int8 quantisation of the activations (the input form of the
// GEMM above; vLLM's scaled_int8_quant rule for symmetric dynamic activations):
// scale = absmax / 127 (1 for an all-zero row), q = rint(x / scale). One CTA per
// row: a pass for the maximum, a pass to write (the row is served by L1 / L2).
__global__ void __launch_bounds__(256) act_quant_token_i8_kernel(
    const uint16_t* __restrict__ x, int64_t x_st, int8_t* __restrict__ q, int64_t q_st,
    float* __restrict__ scales, int k8, int in_f16) {
  __shared__ float s_red[8];
  const int64_t row = blockIdx.x;
  const uint4* src = reinterpret_cast<const uint4*>(x + row * x_st);
  auto unpack = [&](const uint4& w, float* v) {
    const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (in_f16) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&ws[i]));
        v[2 * i] = f.x, v[2 * i + 1] = f.y;
      } else {
        v[2 * i] = bf16_lo(ws[i]), v[2 * i + 1] = bf16_hi(ws[i]);
      }
    }
  };
  float amax = 0.f;
  for (int c = threadIdx.x; c < k8; c += 256) {
    float v[8];
    unpack(src[c], v);
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = s_red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) amax = fmaxf(amax, s_red[i]);
  const float s = amax > 0.f ? __fdiv_rn(amax, 127.f) : 1.f;
  if (threadIdx.x == 0) scales[row] = s;
  uint2* dst = reinterpret_cast<uint2*>(q + row * q_st);
  for (int c = threadIdx.x; c < k8; c += 256) {
    float v[8];
    unpack(src[c], v);
    int b[8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
      b[i] = __float2int_rn(fminf(fmaxf(rintf(__fdiv_rn(v[i], s)), -127.f), 127.f)) & 255;
    dst[c] = make_uint2(b[0] | (b[1] << 8) | (b[2] << 16) | (b[3] << 24),
                        b[4] | (b[5] << 8) | (b[6] << 16) | (b[7] << 24));
  }
}

template <int NB>
int launch_gemm(const GemmArgs& p, const void* a_mat, int64_t a_stride, const void* b_mat,
                int64_t b_stride, cudaStream_t st) {
  using L = GemmLayout<NB>;
  auto kernel = gemm_w8a8_umma_kernel<NB>;
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
  CUtensorMap map_a, map_b;
  STRIX_CHECK(tma::make_map_u8(&map_a, a_mat, uint64_t(p.a_rows), uint64_t(p.K), uint64_t(a_stride), 128) &&
                  tma::make_map_u8(&map_b, b_mat, uint64_t(p.b_rows), uint64_t(p.K), uint64_t(b_stride), NB),
              "tensor map encoding failed");
  const int items = p.a_tiles * p.b_tiles;
  kernel<<<items < sms[dev] ? items : sms[dev], kGThreads, L::kSmem, st>>>(p, map_a, map_b);
  return launch_status("w8a8_int8_gemm");
}

}  // namespace

int32_t* umma_status_ptr();  // moe_gemm_umma.cu: device address of the shared status word

}  // namespace strix

using namespace strix;

extern "C" int strix_w8a8_int8_gemm(void* out, int32_t* acc_out, const void* a_q,
                                    const float* a_scale, const void* w, const float* w_scale,
                                    int64_t m, int64_t n, int64_t k, int64_t a_stride,
                                    int64_t w_stride, int64_t out_stride, strix_stream_t stream) {
  STRIX_CHECK(m >= 0 && n > 0 && k > 0, "bad shapes");
  STRIX_CHECK(k % 128 == 0, "K must be a multiple of 128");
  STRIX_CHECK(a_stride % 16 == 0 && w_stride % 16 == 0 && out_stride % 8 == 0 &&
                  reinterpret_cast<uintptr_t>(a_q) % 16 == 0 && reinterpret_cast<uintptr_t>(w) % 16 == 0 &&
                  reinterpret_cast<uintptr_t>(out) % 16 == 0 && reinterpret_cast<uintptr_t>(w_scale) % 16 == 0,
              "16-byte aligned rows required");
  STRIX_CHECK(n < (int64_t(1) << 31) && m < (int64_t(1) << 31), "matrix too large");
  if (m == 0) return STRIX_OK;
  GemmArgs p;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.acc_out = acc_out;
  p.status = umma_status_ptr();
  STRIX_CHECK(p.status != nullptr, "status word unavailable");
  p.out_stride = out_stride;
  p.K = int(k);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (m <= 64) {
    // decode: weights fill the MMA's M dimension, the tokens are the N dimension
    p.swap = 1;
    p.a_scale = w_scale, p.b_scale = a_scale;
    p.a_rows = int(n), p.b_rows = int(m);
    p.a_tiles = int((n + 127) / 128), p.b_tiles = 1;
    if (m <= 16) return launch_gemm<16>(p, w, w_stride, a_q, a_stride, st);
    if (m <= 32) return launch_gemm<32>(p, w, w_stride, a_q, a_stride, st);
    return launch_gemm<64>(p, w, w_stride, a_q, a_stride, st);
  }
  p.swap = 0;
  p.a_scale = a_scale, p.b_scale = w_scale;
  p.a_rows = int(m), p.b_rows = int(n);
  p.a_tiles = int((m + 127) / 128), p.b_tiles = int((n + 255) / 256);
  return launch_gemm<256>(p, a_q, a_stride, w, w_stride, st);
}

extern "C" int strix_act_quant_token_i8(const void* x, void* q, float* scales, int64_t rows, int64_t k,
                                        int64_t x_stride, int64_t q_stride, int in_f16,
                                        strix_stream_t stream) {
  STRIX_CHECK(x != nullptr && q != nullptr && scales != nullptr, "pointers must not be NULL");
  STRIX_CHECK(rows >= 0 && k > 0 && k % 8 == 0 && x_stride % 8 == 0 && q_stride % 8 == 0 &&
                  reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(q) % 8 == 0,
              "K must be a multiple of 8 with 16-byte aligned rows");
  if (rows == 0) return STRIX_OK;
  act_quant_token_i8_kernel<<<unsigned(rows), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint16_t*>(x), x_stride, static_cast<int8_t*>(q), q_stride, scales, int(k / 8),
      in_f16);
  return launch_status("act_quant_token_i8");
}
