// Blackwell (sm_100a) tensor-core plumbing: tcgen05 MMA with accumulators in
// tensor memory (TMEM), shared-memory operand descriptors, mbarriers with
// bounded waits. Inline PTX only; nothing here depends on a library.
//
// Conventions used by every kernel in this directory:
//   * operands are K-major tiles of 128 bytes of K per row, rows grouped by 8
//     (a 1,024-byte swizzle atom), in the 128-byte swizzle: the 16-byte chunk c
//     of row r is stored at chunk c ^ (r & 7). Tiles start on 1,024-byte
//     boundaries. This is the layout a TMA copy with 128-byte swizzle writes,
//     and the kernels that gather rows write the same layout with cp.async;
//   * every wait on an mbarrier is bounded: after kSpinLimit polls the waiter
//     gives up, records a status word and raises the CTA's abort flag; every role
//     then leaves its loop, the producer waits for the copies it armed and the
//     issuers for the MMAs they issued (drain_armed_loads / drain_issued_mmas),
//     and only then is TMEM freed, so a protocol bug can never hang the device.
#pragma once

#include "common.cuh"

namespace strix {
namespace umma {

constexpr uint32_t kSpinLimit = 1u << 24;  // polls before a wait gives up (~ 1 s)

// ----------------------------------------------------------------- mbarrier
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Arrive that fires once all cp.async copies this thread issued so far landed.
__device__ __forceinline__ void mbar_arrive_cp_async(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// Polls the phase with the given parity; false if the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = smem_u32(bar);
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}

// One poll of the phase with the given parity (no waiting).
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}

__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// Makes shared-memory writes of the generic proxy (st.shared, cp.async)
// visible to the async proxy that tcgen05.mma reads operands through.
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// --------------------------------------------------------------------- TMEM
// One full warp allocates `cols` (power of two, 32..512) columns and writes the
// TMEM base address to *slot (shared memory); the same warp frees them.
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(slot)),
               "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols)
               : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// mbarrier arrive when every MMA this thread issued so far has completed.
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}

// 32 lanes x 32 columns of 32-bit: thread i of warp w reads TMEM lane
// 32 * (w % 4) + i, columns [col, col + 32) of `taddr`.
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_ld_32x8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7])
      : "r"(taddr)
      : "memory");
}

// The mirror of tmem_ld_32x16 / tmem_ld_32x32: thread i of warp w writes columns
// [col, col + n) of TMEM lane 32 * (w % 4) + i.
__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
        "r"(r[14]), "r"(r[15])
      : "memory");
}

__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
        "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
        "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
        "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// -------------------------------------------------------------- descriptors
// Shared-memory matrix descriptor of a K-major, 128-byte-swizzled operand tile
// whose 8-row groups are 1,024 bytes apart. Fields (64 bits): start address
// >> 4 in [0,14); leading byte offset >> 4 in [16,30) (not used by swizzled
// K-major tiles, set to 1); stride byte offset >> 4 in [32,46) = distance
// between 8-row groups; descriptor version 1 in [46,48); layout type in
// [61,64), 2 = 128-byte swizzle. `byte_offset` (a multiple of 32, < 128) selects
// the K slice of one MMA inside the 128-byte row.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t tile_smem_addr, uint32_t byte_offset = 0) {
  uint64_t d = 0;
  d |= uint64_t(((tile_smem_addr + byte_offset) & 0x3ffffu) >> 4);
  d |= uint64_t(1) << 16;                 // LBO = 16 bytes (ignored)
  d |= uint64_t(1024 >> 4) << 32;         // SBO = 1,024 bytes
  d |= uint64_t(1) << 46;                 // version
  d |= uint64_t(2) << 61;                 // SWIZZLE_128B
  return d;
}

// The same descriptor as two 32-bit words, for issue loops: the high word is a
// constant, and advancing the tile address by `bytes` (a multiple of 16) adds
// bytes >> 4 to the low word, so the issuing thread spends one add per operand.
constexpr uint32_t kDescHiSw128 = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t smem_desc_lo(uint32_t tile_smem_addr) {
  return ((tile_smem_addr & 0x3ffffu) >> 4) | (1u << 16);
}
__device__ __forceinline__ uint64_t desc_pack(uint32_t lo, uint32_t hi) {
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
  return d;
}

// Instruction descriptor (32 bits) of a dense tcgen05.mma with K-major A and B:
// D format in [4,6) (1 = f32, 2 = s32); A format in [7,10), B format in
// [10,13) (kind::f8f6f4: 0 = e4m3, 1 = e5m2; kind::i8: 0 = u8, 1 = s8;
// kind::f16: 0 = f16, 1 = bf16); N >> 3 in [17,23); M >> 4 in [24,29).
enum DFormat : uint32_t { D_F16 = 0, D_F32 = 1, D_S32 = 2 };
__host__ __device__ constexpr uint32_t instr_desc(uint32_t d_fmt, uint32_t a_fmt, uint32_t b_fmt,
                                                  uint32_t m, uint32_t n) {
  return (d_fmt << 4) | (a_fmt << 7) | (b_fmt << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

enum Kind { KIND_F16 = 0, KIND_F8F6F4 = 1, KIND_I8 = 2 };

// D[tmem] (+)= A[smem] * B[smem]^T; one thread issues. `accumulate` = 0 overwrites D.
template <int KIND>
__device__ __forceinline__ void mma_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                       uint32_t idesc, uint32_t accumulate) {
  if constexpr (KIND == KIND_F8F6F4) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else if constexpr (KIND == KIND_I8) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}

// D[tmem] (+)= A[tmem] * B[smem]^T, kind::f16: the A operand (M = 128 rows on the
// 128 lanes, 16-bit elements packed two per 32-bit column, element k of a row in
// column k / 2, low half first) is read from tensor memory at `tmem_a`.
__device__ __forceinline__ void mma_ts_f16(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc,
                                           uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// As mma_ss with the operands' low descriptor words and a compile-time
// accumulate flag: the shortest issue sequence (the issuing thread runs in
// order, so every instruction around the MMA adds to the time between MMAs).
template <int KIND, bool ACC>
__device__ __forceinline__ void mma_ss_lo(uint32_t tmem_d, uint32_t a_lo, uint32_t b_lo, uint32_t idesc) {
  const uint64_t adesc = desc_pack(a_lo, kDescHiSw128), bdesc = desc_pack(b_lo, kDescHiSw128);
  if constexpr (KIND == KIND_F8F6F4) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "n"(ACC ? 1 : 0)
        : "memory");
  } else if constexpr (KIND == KIND_I8) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "n"(ACC ? 1 : 0)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "n"(ACC ? 1 : 0)
        : "memory");
  }
}

// Teardown after a bounded wait gave up (a role set the CTA's abort flag). A CTA
// must not free TMEM or exit while bulk copies it armed can still write its
// shared memory or MMAs it issued can still write TMEM, so before the final
// barrier the producing thread waits (bounded again) for the last `stages`
// stages it armed, and every issuing thread commits to a barrier of its own and
// waits for it: tcgen05.commit arrives once all MMAs that thread issued retired.
__device__ __forceinline__ void drain_armed_loads(uint64_t* full_bar, int stages, int armed) {
  const int n = armed < stages ? armed : stages;
  for (int i = 0; i < n; ++i) {
    const int t = armed - 1 - i;
    mbar_wait(&full_bar[t % stages], (t / stages) & 1);
  }
}
__device__ __forceinline__ void drain_issued_mmas(uint64_t* drain_bar) {
  mma_commit(drain_bar);
  mbar_wait(drain_bar, 0);
}

// Byte offset of 16-byte chunk `chunk` of row `row` inside a swizzled tile.
__device__ __forceinline__ uint32_t sw128_offset(int row, int chunk) {
  return uint32_t(row * 128 + ((chunk ^ (row & 7)) << 4));
}

}  // namespace umma
}  // namespace strix
