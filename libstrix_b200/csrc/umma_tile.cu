// One-CTA tcgen05 tile product, D[128, N] = A[128, K] * B[N, K]^T, for int8
// (s32 accumulate, bit-exact) and e4m3 (f32 accumulate).
//
// This is the layout probe of the sm_100a build: it pins, against a CPU matmul,
// everything the production kernels rely on - the shared-memory descriptor of a
// K-major 128-byte-swizzled tile, the K advance inside the swizzle span, the
// instruction descriptor, the row <-> TMEM lane and column <-> TMEM column
// mapping of the accumulator, and the commit / mbarrier hand-off. It plays the
// role of the reference's _wmma_bf16_tile (csrc/testing/wmma_layout_test.hip:27),
// which pins the gfx11 WMMA fragment layout the same way.
#include "umma.cuh"

namespace strix {
namespace {

using namespace umma;

template <int KIND>
__global__ void __launch_bounds__(128) umma_tile_kernel(void* __restrict__ d,
                                                        const uint8_t* __restrict__ a,
                                                        const uint8_t* __restrict__ b, int n, int k,
                                                        int* __restrict__ status) {
  extern __shared__ uint8_t raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sa = tiles;               // 128 rows x 128 bytes
  uint8_t* sb = tiles + 128 * 128;   // n rows x 128 bytes
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t tmem_slot;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t cols = n <= 32 ? 32 : n <= 64 ? 64 : n <= 128 ? 128 : 256;

  if (warp == 0) tmem_alloc(&tmem_slot, cols);
  if (tid == 0) {
    mbar_init(&bar, 1);
    fence_mbar_init();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_slot;
  const uint32_t idesc = KIND == KIND_I8 ? instr_desc(D_S32, 1, 1, 128, n)
                                         : instr_desc(D_F32, 0, 0, 128, n);
  uint32_t phase = 0;
  bool ok = true;
  for (int kb = 0; kb < k / 128 && ok; ++kb) {
    for (int id = tid; id < 128 * 8; id += 128) {
      const int r = id >> 3, ch = id & 7;
      *reinterpret_cast<uint4*>(sa + sw128_offset(r, ch)) =
          *reinterpret_cast<const uint4*>(a + int64_t(r) * k + kb * 128 + ch * 16);
    }
    for (int id = tid; id < n * 8; id += 128) {
      const int r = id >> 3, ch = id & 7;
      *reinterpret_cast<uint4*>(sb + sw128_offset(r, ch)) =
          *reinterpret_cast<const uint4*>(b + int64_t(r) * k + kb * 128 + ch * 16);
    }
    fence_proxy_async();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after_sync();
#pragma unroll
      for (int s = 0; s < 4; ++s)
        mma_ss<KIND>(tmem, smem_desc_sw128(smem_u32(sa), 32 * s), smem_desc_sw128(smem_u32(sb), 32 * s),
                     idesc, (kb > 0 || s > 0) ? 1u : 0u);
      mma_commit(&bar);
    }
    ok = mbar_wait(&bar, phase);  // the MMAs have read the tiles: they may be refilled
    phase ^= 1;
  }
  if (!ok && lane == 0) atomicExch(status, 1);
  tc_fence_after_sync();
  if (ok) {
    // accumulator row m lives in TMEM lane m, column j in TMEM column j
    const int row = warp * 32 + lane;
    for (int c0 = 0; c0 < n; c0 += 16) {
      uint32_t r[16];
      tmem_ld_32x16(tmem + (uint32_t(warp * 32) << 16) + c0, r);
      tmem_ld_wait();
      uint32_t* out = static_cast<uint32_t*>(d) + int64_t(row) * n + c0;
#pragma unroll
      for (int i = 0; i < 16; ++i) out[i] = r[i];
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, cols);
}

}  // namespace
}  // namespace strix

using namespace strix;

extern "C" int strix_umma_tile(void* d, const void* a, const void* b, int32_t* status, int64_t n,
                               int64_t k, int kind, strix_stream_t stream) {
  STRIX_CHECK(n >= 16 && n <= 256 && n % 16 == 0, "N must be a multiple of 16 in 16..256");
  STRIX_CHECK(k >= 128 && k % 128 == 0, "K must be a multiple of 128");
  STRIX_CHECK(kind == 0 || kind == 1, "kind: 0 int8, 1 e4m3");
  STRIX_CHECK(reinterpret_cast<uintptr_t>(a) % 16 == 0 && reinterpret_cast<uintptr_t>(b) % 16 == 0,
              "16-byte aligned rows required");
  const size_t smem = 1024 + 128 * 128 + size_t(n) * 128;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto pa = static_cast<const uint8_t*>(a), pb = static_cast<const uint8_t*>(b);
  if (kind == 0) {
    STRIX_CUDA(cudaFuncSetAttribute(umma_tile_kernel<umma::KIND_I8>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    umma_tile_kernel<umma::KIND_I8><<<1, 128, smem, st>>>(d, pa, pb, int(n), int(k), status);
  } else {
    STRIX_CUDA(cudaFuncSetAttribute(umma_tile_kernel<umma::KIND_F8F6F4>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    umma_tile_kernel<umma::KIND_F8F6F4><<<1, 128, smem, st>>>(d, pa, pb, int(n), int(k), status);
  }
  return launch_status("umma_tile");
}
