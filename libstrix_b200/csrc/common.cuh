// Shared device/host helpers for the sm_100a kernels of libstrix_b200.
//
// Everything in csrc/ is plain CUDA behind an extern "C" boundary: no torch
// types, raw pointers and sizes only. Argument validation mirrors the
// TORCH_CHECKs of the reference launchers; a failed check records a message
// (strix_last_error) and returns STRIX_ERR_INVALID instead of throwing.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdlib>
#include <cstdio>

#include "../../include/strix_b200.h"

namespace strix {

// Thread-local message of the last failed call on this thread.
char* error_buffer();
int fail(int code, const char* fmt, ...);

#define STRIX_CHECK(cond, ...)                                  \
  do {                                                          \
    if (!(cond)) return ::strix::fail(STRIX_ERR_INVALID, __VA_ARGS__); \
  } while (0)

#define STRIX_CUDA(expr)                                                     \
  do {                                                                       \
    cudaError_t err__ = (expr);                                              \
    if (err__ != cudaSuccess)                                                \
      return ::strix::fail(STRIX_ERR_CUDA, "%s: %s", #expr,                  \
                           cudaGetErrorString(err__));                       \
  } while (0)

inline int launch_status(const char* what) {
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess)
    return fail(STRIX_ERR_CUDA, "%s launch: %s", what, cudaGetErrorString(err));
  return STRIX_OK;
}

// Programmatic dependent launch: the kernels of a layer are enqueued back to back
// and each one begins with pdl_enter(), which lets the NEXT kernel of the stream be
// launched right away (its CTAs become resident as resources allow) and then waits
// until every kernel before it has completed and its writes are visible. A kernel
// does nothing before that wait, so the order of all memory effects is that of
// ordinary stream order; what is saved is the launch latency and scheduling gap
// between kernels (a few microseconds each, a tenth of a 256-token MoE layer).
// STRIX_PDL=0 launches the plain way.
inline bool pdl_enabled() {
  static const bool on = [] {
    const char* v = getenv("STRIX_PDL");
    return v == nullptr || v[0] != '0';
  }();
  return on;
}

template <typename... P, typename... A>
inline void launch_chain(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                         A&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = st;
  cudaLaunchAttribute attr{};
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  cudaLaunchKernelEx(&cfg, kernel, P(static_cast<A&&>(args))...);
}

// ---------------------------------------------------------------- device side

// First statement of a kernel launched with launch_chain (see there).
__device__ __forceinline__ void pdl_enter() {
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}

__device__ __forceinline__ uint32_t sub_f16x2(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}

// Two fp32 -> packed f16x2 (lo in the low half), round to nearest even.
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

__device__ __forceinline__ float fast_exp2(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

__device__ __forceinline__ float fast_log2(float x) {
  float r;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

// 128-bit streaming load that does not allocate in L1 (single-use KV / weights).
__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

// Asynchronous global -> shared copies (LDGSTS). The 16-byte form bypasses L1.
__device__ __forceinline__ void cp_async_16(uint32_t smem_addr, const void* gptr) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr), "l"(gptr));
}
__device__ __forceinline__ void cp_async_4(uint32_t smem_addr, const void* gptr) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_addr), "l"(gptr));
}
// As above, but the destination is filled with zeros when `valid` is false
// (src-size 0); the source address must still be a mapped one.
__device__ __forceinline__ void cp_async_16_zfill(uint32_t smem_addr, const void* gptr, bool valid) {
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr), "l"(gptr), "r"(n));
}
__device__ __forceinline__ void cp_async_4_zfill(uint32_t smem_addr, const void* gptr, bool valid) {
  const int n = valid ? 4 : 0;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(smem_addr), "l"(gptr), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// D(16x8,f32) += A(16x16,f16,row) * B(16x8,f16,col)
__device__ __forceinline__ void mma_f16_16816(float (&d)[4], const uint32_t (&a)[4],
                                              uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4],
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// D(16x8,s32) += A(16x32,s8,row) * B(32x8,s8 or u8,col)
__device__ __forceinline__ void mma_s8s8_16832(int (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                               uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void mma_s8u8_16832(int (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                               uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.u8.s32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Transposes an 8x8 matrix of 16-bit elements held one row-pair per lane.
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
  uint32_t r;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(x));
  return r;
}

}  // namespace strix
