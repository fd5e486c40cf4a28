// Whole-matrix decoders of the quantized weight formats to bf16, for sm_100a:
// what a caller feeds a library GEMM at prefill sizes, and the byte-exact
// statement of each format's decode rule.
//   mxfp4  e2m1 nibbles (byte j: k = 2j low, 2j + 1 high) x e8m0 scale per 32
//          elements, a scale byte of 0 is the zero block
//          (csrc/gemm/mxfp4_wmma_gemm.hip, tests/test_mxfp4.py:29-47, :112-127)
//   int4   (nibble - 8) x 16-bit scale per group (tests/test_moe_wna16.py:48-62)
//   e4m3   x fp32 scale per 128 x 128 block or per output channel
//          (csrc/gemm/fp8_dequant.hip:63)
// One thread decodes 8 consecutive K elements of one row and stores 16 bytes.
#include "common.cuh"

namespace strix {
namespace {

// DQ_INT4X = int4 whose 32-bit words hold their nibbles in vLLM's ExLlama order
// (k = 0 2 4 6 1 3 5 7), the dense layout of w4a16_dequant in the reference
enum DqFmt { DQ_MXFP4 = 0, DQ_INT4 = 1, DQ_E4M3 = 2, DQ_INT4X = 3 };

__device__ __forceinline__ float e2m1(uint32_t n) {
  const uint32_t e = (n >> 1) & 3u, m = n & 1u;
  const uint32_t bits = e ? (((e + 126u) << 23) | (m << 22)) : (m ? 0x3F000000u : 0u);
  return __uint_as_float(bits | ((n & 8u) << 28));
}

template <int FMT>
__global__ void __launch_bounds__(256) dequant_kernel(const uint8_t* __restrict__ w, int64_t w_stride,
                                                      const void* __restrict__ scales,
                                                      int64_t s_stride_n, int64_t s_stride_g,
                                                      __nv_bfloat16* __restrict__ out,
                                                      int64_t out_stride, int64_t n, int64_t k,
                                                      int group, int scale_kind, int scale_dtype) {
  const int64_t idx = int64_t(blockIdx.x) * 256 + threadIdx.x;
  const int64_t k8 = k / 8;
  if (idx >= n * k8) return;
  const int64_t row = idx / k8;
  const int64_t k0 = (idx % k8) * 8;
  float v[8];
  float s = 1.f;
  if constexpr (FMT == DQ_E4M3) {
    const uint2 x = *reinterpret_cast<const uint2*>(w + row * w_stride + k0);
    const uint32_t ws[2] = {x.x, x.y};
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      uint32_t lo, hi;
      asm("{\n\t.reg .b16 l, h;\n\tmov.b32 {l, h}, %2;\n\t"
          "cvt.rn.f16x2.e4m3x2 %0, l;\n\tcvt.rn.f16x2.e4m3x2 %1, h;\n\t}"
          : "=r"(lo), "=r"(hi)
          : "r"(ws[i]));
      const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&lo));
      const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&hi));
      v[4 * i] = a.x, v[4 * i + 1] = a.y, v[4 * i + 2] = b.x, v[4 * i + 3] = b.y;
    }
    // scale_kind 1: per channel [N]; 2: block [ceil(N/128), K/128]
    const float* sp = static_cast<const float*>(scales);
    s = scale_kind == 1 ? sp[row * s_stride_n] : sp[(row / 128) * s_stride_n + (k0 / 128) * s_stride_g];
  } else {
    const uint32_t x = *reinterpret_cast<const uint32_t*>(w + row * w_stride + k0 / 2);
    const int64_t si = row * s_stride_n + (k0 / group) * s_stride_g;
    if constexpr (FMT == DQ_MXFP4) {
      s = __uint_as_float(uint32_t(static_cast<const uint8_t*>(scales)[si]) << 23);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = e2m1((x >> (4 * i)) & 15u);
    } else {
      const uint16_t h = static_cast<const uint16_t*>(scales)[si];
      s = scale_dtype == 1 ? __uint_as_float(uint32_t(h) << 16) : __half2float(__ushort_as_half(h));
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        // element i sits in nibble i, or (shuffled words) evens in the low half, odds in the high
        const int nib = FMT == DQ_INT4X ? (i >> 1) + 4 * (i & 1) : i;
        v[i] = float(int((x >> (4 * nib)) & 15u) - 8);
      }
    }
  }
  uint4 o;
  o.x = pack_bf16x2(v[0] * s, v[1] * s);
  o.y = pack_bf16x2(v[2] * s, v[3] * s);
  o.z = pack_bf16x2(v[4] * s, v[5] * s);
  o.w = pack_bf16x2(v[6] * s, v[7] * s);
  *reinterpret_cast<uint4*>(out + row * out_stride + k0) = o;
}

}  // namespace
}  // namespace strix

using namespace strix;

extern "C" int strix_dequant_bf16(void* out, const void* w, const void* scales, int64_t n, int64_t k,
                                  int64_t w_stride, int64_t out_stride, int64_t s_stride_n,
                                  int64_t s_stride_g, int format, int group, int scale_kind,
                                  int scale_dtype, strix_stream_t stream) {
  STRIX_CHECK(format >= DQ_MXFP4 && format <= DQ_INT4X, "format 0 mxfp4, 1 int4, 2 e4m3, 3 int4 (ExLlama order)");
  STRIX_CHECK(n >= 0 && k > 0 && k % 8 == 0, "K must be a multiple of 8");
  STRIX_CHECK(out_stride % 8 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0 &&
                  reinterpret_cast<uintptr_t>(w) % 8 == 0 &&
                  w_stride % (format == DQ_E4M3 ? 8 : 4) == 0,
              "aligned rows required");
  if (format == DQ_MXFP4) STRIX_CHECK(group == 32 && k % 32 == 0, "mxfp4 scales cover 32 elements");
  if (format == DQ_INT4 || format == DQ_INT4X)
    STRIX_CHECK((group == 32 || group == 64 || group == 128) && k % group == 0 &&
                    (scale_dtype == 1 || scale_dtype == 2),
                "int4 scales are bf16 or fp16 per 32, 64 or 128 elements");
  if (format == DQ_E4M3)
    STRIX_CHECK((scale_kind == 1 || (scale_kind == 2 && k % 128 == 0)) && scale_dtype == 0,
                "e4m3 scales are fp32 per channel or per 128 x 128 block");
  if (n == 0) return STRIX_OK;
  const int64_t threads = n * (k / 8);
  const unsigned grid = unsigned((threads + 255) / 256);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto wp = static_cast<const uint8_t*>(w);
  auto op = static_cast<__nv_bfloat16*>(out);
  if (format == DQ_MXFP4)
    dequant_kernel<DQ_MXFP4><<<grid, 256, 0, st>>>(wp, w_stride, scales, s_stride_n, s_stride_g, op,
                                                   out_stride, n, k, group, scale_kind, scale_dtype);
  else if (format == DQ_INT4)
    dequant_kernel<DQ_INT4><<<grid, 256, 0, st>>>(wp, w_stride, scales, s_stride_n, s_stride_g, op,
                                                  out_stride, n, k, group, scale_kind, scale_dtype);
  else if (format == DQ_INT4X)
    dequant_kernel<DQ_INT4X><<<grid, 256, 0, st>>>(wp, w_stride, scales, s_stride_n, s_stride_g, op,
                                                   out_stride, n, k, group, scale_kind, scale_dtype);
  else
    dequant_kernel<DQ_E4M3><<<grid, 256, 0, st>>>(wp, w_stride, scales, s_stride_n, s_stride_g, op,
                                                  out_stride, n, k, group, scale_kind, scale_dtype);
  return launch_status("dequant_bf16");
}
