// Blackwell (sm_100a) building blocks in inline PTX: mbarriers with bounded
// waits, TMA tile loads, tensor memory (TMEM) allocation, tcgen05 matrix
// multiply-accumulate with shared-memory operand descriptors, and the loads
// that bring accumulators back from TMEM.
//
// Every wait has a time limit. A wait that runs out records a code in the
// library's device error word and makes the kernel wind down: nothing spins
// for ever, and nothing traps.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace tc {

// Codes in the device error word.
enum : int { ERR_NONE = 0, ERR_WAIT_FULL = 1, ERR_WAIT_EMPTY = 2, ERR_WAIT_ACCUM = 3, ERR_WAIT_DRAIN = 4 };

constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;  // 2 s

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// ------------------------------------------------------------------ mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Waits for the phase with the given parity to complete. False after WAIT_LIMIT_NS.
// The clock is read only once in a few thousand polls: reading it costs far more than a
// poll, and a waiter that is busy reading the clock wakes up late.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity,
                                          unsigned long long limit_ns = WAIT_LIMIT_NS) {
  if (mbar_try_wait(bar, parity)) return true;
  unsigned long long t0 = 0;
  uint32_t polls = 0;
#pragma unroll 1
  while (!mbar_try_wait(bar, parity)) {
    if ((++polls & 0xFFFu) == 0) {
      const unsigned long long now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > limit_ns) return false;
    }
  }
  return true;
}

// ------------------------------------------------------------------ TMA
// One box of a 2-D tensor map into shared memory; completion is counted in
// bytes on `bar`. c0 is the coordinate along the contiguous dimension (its
// byte offset must be a multiple of 16), c1 the row. No multicast.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
// Four-dimensional variant (pages of the cache: [page, head, position, channel]).
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1,
                                            int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ------------------------------------------------------------------ clusters
__device__ __forceinline__ void cluster_arrive_wait() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The address, in the cluster's shared window, of `local` in the CTA of rank `rank`.
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
  return r;
}

// Four bytes into the shared memory of another CTA of the cluster; they are counted on that CTA's
// mbarrier when they have landed.
__device__ __forceinline__ void st_async_f32(uint32_t remote_addr, uint32_t remote_bar, float v) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %2, [%1];"
               ::"r"(remote_addr), "r"(remote_bar), "r"(__float_as_uint(v))
               : "memory");
}


// ------------------------------------------------------------------ CTA pairs (cta_group::2)
// Two CTAs of a cluster (ranks 2i and 2i + 1) can run one matrix product together: the product is
// issued by one thread of the even CTA, reads the operands' halves from both CTAs' shared memory at
// the same offsets, and leaves each CTA's 128 rows of the result in that CTA's tensor memory.
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// A TMA load into this CTA's shared memory whose bytes are counted on a barrier of the pair's
// even CTA (`bar`: that barrier's address in the cluster's shared window). No multicast.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
// An arrival on a barrier of another CTA of the cluster.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Both CTAs of the pair execute these with one warp each.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// D[tmem of both CTAs] (+)= A * B^T with M = 256 (128 rows per CTA); issued by one thread of the even CTA.
__device__ __forceinline__ void mma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                              bool accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"((uint32_t)accumulate)
      : "memory");
}
// Makes the barrier at `bar`'s offset in both CTAs of the pair (mask 0b11: cluster ranks 0 and 1)
// complete a phase once every product issued so far by this thread has finished.
__device__ __forceinline__ void mma_commit_pair(uint32_t bar, uint16_t cta_mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"(cta_mask)
               : "memory");
}

// ------------------------------------------------------------------ TMEM
// Allocation is done by one whole warp; the base address lands in shared memory.
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ------------------------------------------------------------------ MMA
// Shared-memory operand descriptor for a K-major tile whose rows are 128 bytes
// (64 bf16) stored with the 128-byte swizzle that TMA writes: start address
// (>>4) in bits 0-13, leading byte offset (unused for this layout, set to 1) in
// 16-29, stride byte offset (8 rows * 128 B = 1024, >>4) in 32-45, descriptor
// version 1 in 46-47, layout type 2 (128-byte swizzle) in 61-63.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// The same for an operand whose contraction dimension is NOT the contiguous one ("MN-major": for
// V of attention, [keys][channels] with keys contracted). Rows of 128 bytes (64 channels) with the
// 128-byte swizzle; eight rows (keys) are one 1024-byte group, and the stride byte offset is the
// distance between such groups along the contraction. The leading byte offset (between blocks of
// 64 channels) is not used with 64 channels.
__device__ __forceinline__ uint64_t smem_desc_sw128_mn(uint32_t smem_addr) { return smem_desc_sw128(smem_addr); }
// With more than 64 channels: blocks of 64 channels lie `block_bytes` apart (the leading byte offset).
__device__ __forceinline__ uint64_t smem_desc_sw128_mn(uint32_t smem_addr, uint32_t block_bytes) {
  uint64_t d = smem_desc_sw128(smem_addr);
  d &= ~((uint64_t)0x3FFF << 16);
  d |= (uint64_t)((block_bytes >> 4) & 0x3FFF) << 16;
  return d;
}

// Instruction descriptor, kind::f16: D format f32 (1) in bits 4-5, A and B
// format bf16 (1) in 7-9 and 10-12, both K-major (bits 15, 16 clear), N >> 3 in
// 17-22, M >> 4 in 24-28.
__host__ __device__ constexpr uint32_t instr_desc_bf16(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
// Bit 16: the B operand is MN-major (see smem_desc_sw128_mn).
constexpr uint32_t INSTR_B_MN_MAJOR = 1u << 16;

// D[tmem] (+)= A[smem] * B[smem]^T; issued by one thread.
__device__ __forceinline__ void mma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                         bool accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"((uint32_t)accumulate)
      : "memory");
}
// Four products in a row onto one accumulator, the first overwriting it: the k steps of a 64-deep
// block whose operand descriptors advance by a fixed step (in descriptor units of 16 bytes). One
// predicate set-up for all four, and nothing between them for the issuing thread to wait on.
__device__ __forceinline__ void mma_bf16_x4(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                            uint32_t step_a, uint32_t step_b) {
  const uint64_t a1 = desc_a + step_a, a2 = desc_a + 2 * step_a, a3 = desc_a + 3 * step_a;
  const uint64_t b1 = desc_b + step_b, b2 = desc_b + 2 * step_b, b3 = desc_b + 3 * step_b;
  asm volatile(
      "{\n\t.reg .pred p0, p1;\n\t"
      "setp.ne.b32 p0, 0, 0;\n\t"
      "setp.eq.b32 p1, 0, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %5, %9, p0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %2, %6, %9, p1;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %3, %7, %9, p1;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %4, %8, %9, p1;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(a1), "l"(a2), "l"(a3), "l"(desc_b), "l"(b1), "l"(b2), "l"(b3), "r"(idesc)
      : "memory");
}
// The same with a choice for the first product: it overwrites the accumulator or adds to it.
__device__ __forceinline__ void mma_bf16_x4(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                            uint32_t step_a, uint32_t step_b, bool first_accumulates) {
  const uint64_t a1 = desc_a + step_a, a2 = desc_a + 2 * step_a, a3 = desc_a + 3 * step_a;
  const uint64_t b1 = desc_b + step_b, b2 = desc_b + 2 * step_b, b3 = desc_b + 3 * step_b;
  asm volatile(
      "{\n\t.reg .pred p0, p1;\n\t"
      "setp.ne.b32 p0, %10, 0;\n\t"
      "setp.eq.b32 p1, 0, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %5, %9, p0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %2, %6, %9, p1;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %3, %7, %9, p1;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %4, %8, %9, p1;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(a1), "l"(a2), "l"(a3), "l"(desc_b), "l"(b1), "l"(b2), "l"(b3), "r"(idesc),
        "r"((uint32_t)first_accumulates)
      : "memory");
}
// Four products whose A operand lies in tensor memory: 128 lanes (rows), per product 8 columns of
// 32 bits, each holding two consecutive elements of the contraction in bf16 (the lower index in the
// lower half). B comes from shared memory as above.
__device__ __forceinline__ void mma_bf16_ts_x4(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                               uint32_t step_b, bool first_accumulates) {
  const uint64_t b1 = desc_b + step_b, b2 = desc_b + 2 * step_b, b3 = desc_b + 3 * step_b;
  asm volatile(
      "{\n\t.reg .pred p0, p1;\n\t"
      "setp.ne.b32 p0, %10, 0;\n\t"
      "setp.eq.b32 p1, 0, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %5, %9, p0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%2], %6, %9, p1;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%3], %7, %9, p1;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%4], %8, %9, p1;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "r"(tmem_a + 8), "r"(tmem_a + 16), "r"(tmem_a + 24), "l"(desc_b), "l"(b1), "l"(b2),
        "l"(b3), "r"(idesc), "r"((uint32_t)first_accumulates)
      : "memory");
}
// The same for two products.
__device__ __forceinline__ void mma_bf16_ts_x2(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                               uint32_t step_b, bool first_accumulates) {
  const uint64_t b1 = desc_b + step_b;
  asm volatile(
      "{\n\t.reg .pred p0, p1;\n\t"
      "setp.ne.b32 p0, %6, 0;\n\t"
      "setp.eq.b32 p1, 0, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %3, %5, p0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%2], %4, %5, p1;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "r"(tmem_a + 8), "l"(desc_b), "l"(b1), "r"(idesc), "r"((uint32_t)first_accumulates)
      : "memory");
}
template <int STEPS>
__device__ __forceinline__ void mma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                            uint32_t step_b, bool first_accumulates) {
  static_assert(STEPS == 2 || STEPS == 4, "two or four products");
  if (STEPS == 2) mma_bf16_ts_x2(tmem_d, tmem_a, desc_b, idesc, step_b, first_accumulates);
  else mma_bf16_ts_x4(tmem_d, tmem_a, desc_b, idesc, step_b, first_accumulates);
}
// Makes `bar` complete once every MMA issued so far by this thread has finished.
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}

// 16 consecutive 32-bit columns of this thread's TMEM lane (lane = 32 * warp + laneid).
__device__ __forceinline__ void tmem_ld_16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
// 32 consecutive columns.
__device__ __forceinline__ void tmem_ld_32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// The other way: 32 registers into 32 consecutive columns of this thread's lane.
__device__ __forceinline__ void tmem_st_32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
// 16 registers into 16 consecutive columns.
__device__ __forceinline__ void tmem_st_16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st(uint32_t taddr, const uint32_t (&r)[32]) { tmem_st_32(taddr, r); }
__device__ __forceinline__ void tmem_st(uint32_t taddr, const uint32_t (&r)[16]) { tmem_st_16(taddr, r); }
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

}  // namespace tc
