// Tensor Memory Accelerator helpers for sm_100a: host-side tensor maps over
// row matrices of bytes, device-side bulk tensor loads that complete on an
// mbarrier. Loads only, never multicast; every load lands in the issuing CTA's
// own shared memory.
//
// A map describes a K-major matrix [rows, row_bytes] with a row stride, read in
// boxes of `box_rows` rows x 128 bytes with the 128-byte swizzle, so a box lands
// in exactly the layout the tcgen05 shared-memory descriptors of umma.cuh read
// (row r at r * 128, 16-byte chunk c at position c ^ (r & 7)). Rows or bytes
// outside the matrix arrive as zeros and still count toward the box's bytes.
#pragma once

#include <cuda.h>

#include "umma.cuh"

namespace strix {
namespace tma {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver's encoder, looked up through the runtime (no link against the driver library).
inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// Map over bytes [rows, row_bytes] at `base` (16-byte aligned, stride a multiple
// of 16), boxes of box_rows x 128 bytes, 128-byte swizzle. Returns false on failure.
inline bool make_map_u8(CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_bytes,
                        uint64_t stride_bytes, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {row_bytes, rows};
  const cuuint64_t strides[1] = {stride_bytes};
  const cuuint32_t box[2] = {128, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box,
            estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Map over bytes with up to 4 dimensions: dims[0] = bytes per row (stride 1),
// dims[i] with byte strides[i - 1] for i >= 1 (multiples of 16, in any order of
// magnitude, which lets a box interleave rows of two regions); box[0] = 128 with
// the 128-byte swizzle, or any multiple of 16 bytes without swizzle.
inline bool make_map_u8_nd(CUtensorMap* map, const void* base, int rank, const uint64_t* dims,
                           const uint64_t* strides, const uint32_t* box, bool swizzle128 = true) {
  EncodeTiledFn fn = encode_fn();
  if (!fn || rank < 2 || rank > 4) return false;
  cuuint64_t d[4], st[3];
  cuuint32_t b[4], estr[4];
  for (int i = 0; i < rank; ++i) d[i] = dims[i], b[i] = box[i], estr[i] = 1;
  for (int i = 0; i + 1 < rank; ++i) st[i] = strides[i];
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, cuuint32_t(rank), const_cast<void*>(base), d, st, b,
            estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

__device__ __forceinline__ void prefetch_map(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// One arrival on `bar` that also announces `bytes` of asynchronous copies.
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(umma::smem_u32(bar)),
               "r"(bytes)
               : "memory");
}

// Box at (byte x, row y) -> shared memory; completes `bar` by the box's bytes.
// x must be a multiple of 16.
__device__ __forceinline__ void load_2d(uint32_t smem_dst, const CUtensorMap* map, int x, int y,
                                        uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(umma::smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void load_4d(uint32_t smem_dst, const CUtensorMap* map, int c0, int c1,
                                        int c2, int c3, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(
          smem_dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(umma::smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2),
      "r"(c3)
      : "memory");
}

// Asks the TMA to bring a box into L2 only: no shared memory, no barrier. Bytes
// a CTA will need later than its ring of stages can hold are put in flight this
// way, so that the load proper finds them at L2 latency.
__device__ __forceinline__ void prefetch_l2_4d(const CUtensorMap* map, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.prefetch.tensor.4d.L2.global.tile [%0, {%1, %2, %3, %4}];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}
__device__ __forceinline__ void prefetch_l2_2d(const CUtensorMap* map, int x, int y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(x), "r"(y)
               : "memory");
}

}  // namespace tma
}  // namespace strix
