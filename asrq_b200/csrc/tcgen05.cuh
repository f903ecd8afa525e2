// Blackwell (sm_100a) primitives used by the tensor-core kernels: mbarrier with
// bounded waits, TMA tile loads, TMEM allocation, tcgen05.mma / commit / ld and the
// shared-memory and instruction descriptors they take.
#pragma once

#include <cuda.h>  // CUtensorMap (types only; the encoder is fetched at run time)

#include "common.cuh"

namespace asrq {
namespace tc {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier ----------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}
// Two barriers tested by back-to-back try_waits whose results are read together: bit 0 = first, bit 1 = second.
__device__ __forceinline__ uint32_t mbar_try_wait2(uint32_t bar_a, uint32_t parity_a, uint32_t bar_b, uint32_t parity_b) {
  uint32_t got;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t.reg .u32 x, y;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 q, [%3], %4;\n\t"
      "selp.u32 x, 1, 0, p;\n\t"
      "selp.u32 y, 2, 0, q;\n\t"
      "or.b32 %0, x, y;\n\t}"
      : "=r"(got)
      : "r"(bar_a), "r"(parity_a), "r"(bar_b), "r"(parity_b)
      : "memory");
  return got;
}
__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
// Non-suspending poll, for the one thread whose wake-up latency is on the critical path.
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}

// Every wait in these kernels is bounded: after kWaitCycles SM clocks without the
// barrier completing, the waiter records where it gave up in the status block
// (word 0 = 1, word 1 = site) and returns false; the caller then leaves its loop
// and the block tears down normally.  The host reads the block with
// asrq_check_status.
constexpr long long kWaitCycles = 400000000ll;  // ~0.2 s at 1.9 GHz

// Same bound, polling without suspension (test_wait): lower wake-up latency, costs issue slots.
__device__ __forceinline__ bool mbar_wait_spin(uint32_t bar, uint32_t parity, unsigned* status, unsigned site) {
  if (mbar_test_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i)
      if (mbar_test_wait(bar, parity)) return true;
    if (clock64() - t0 > kWaitCycles) {
      if (atomicCAS(status, 0u, 1u) == 0u) status[1] = site;
      return false;
    }
  }
}

// Acquire at cluster scope: pairs with mbarrier.arrive.release.cluster from the other CTA of a pair.
__device__ __forceinline__ bool mbar_test_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}
__device__ __forceinline__ bool mbar_wait_spin_cluster(uint32_t bar, uint32_t parity, unsigned* status, unsigned site) {
  if (mbar_test_wait_cluster(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i)
      if (mbar_test_wait_cluster(bar, parity)) return true;
    if (clock64() - t0 > kWaitCycles) {
      if (atomicCAS(status, 0u, 1u) == 0u) status[1] = site;
      return false;
    }
  }
}

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, unsigned* status, unsigned site) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (clock64() - t0 > kWaitCycles) {
      if (atomicCAS(status, 0u, 1u) == 0u) status[1] = site;
      return false;
    }
  }
}

__device__ __forceinline__ long long globaltimer_ns() {
  long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)::"memory");
  return t;
}

// ---- TMA -----------------------------------------------------------------------------
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 2-D tile load global -> shared, completion counted in bytes on `bar`.
// c0 is the innermost coordinate; c0 * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* m, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(c0), "r"(c1), "r"(bar)
      : "memory");
}

// ---- TMEM ----------------------------------------------------------------------------
// Whole-warp operations.
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
__device__ __forceinline__ void fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---- descriptors -----------------------------------------------------------------------
// Shared-memory operand, K-major, 128-byte swizzle: rows of 128 bytes, groups of 8 rows
// 1024 bytes apart (stride byte offset), 16-byte chunk index XOR (row & 7) inside a
// row.  The tile base must be 1024-byte aligned; a K step of 32 bytes inside the row
// is taken by advancing the start address.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
  uint64_t d = 0;
  d |= uint64_t((addr & 0x3ffffu) >> 4);  // start address, 16-byte units
  d |= uint64_t(1) << 16;                 // leading byte offset (unused for swizzled K-major)
  d |= uint64_t(1024 >> 4) << 32;         // stride byte offset
  d |= uint64_t(1) << 46;                 // descriptor version (sm_100)
  d |= uint64_t(2) << 61;                 // SWIZZLE_128B
  return d;
}

// Instruction descriptor.  D format: 1 = f32, 2 = s32.  A/B format for kind::f16:
// 0 = f16, 1 = bf16; for kind::i8: 0 = u8, 1 = s8; for kind::f8f6f4: 0 = e4m3, 1 = e5m2.  Both operands K-major.
__device__ __forceinline__ uint32_t instr_desc(uint32_t dfmt, uint32_t abfmt, uint32_t m, uint32_t n) {
  return (dfmt << 4) | (abfmt << 7) | (abfmt << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// ---- MMA (single thread) -----------------------------------------------------------------
// One lane of a converged warp.  A role loop that the whole warp runs, with only the tcgen05
// instructions under this predicate, keeps its counters, addresses and descriptors warp-uniform.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.b32 %0, 1, 0, P;\n\t}" : "=r"(pred));
  return pred != 0;
}
__device__ __forceinline__ void mma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_i8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// kind::f8f6f4 with 8-bit operands (instruction descriptor A/B format 0 = e4m3, 1 = e5m2), f32 accumulation;
// K = 32 per instruction like kind::i8.
__device__ __forceinline__ void mma_f8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Same with the A operand in tensor memory (lane = row, 32-bit column c = elements 2c and 2c+1 of a
// 16-bit type): a K step of 16 elements is 8 columns.
__device__ __forceinline__ void mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives once on `bar` when every MMA issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}

// ---- two-CTA (cta_group::2) forms ----------------------------------------------------------
// A pair of CTAs of one cluster works on one MMA: each holds 128 of the 256 A rows and half of the B
// rows in its own shared memory at the same offsets, each gets its 128 accumulator lanes in its own
// tensor memory; one thread of the even CTA (rank 0) issues, and its commits can signal barriers of
// both CTAs.
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Execution barrier only: the arrival does not wait for this thread's earlier global stores to become visible
// (the release form does, which at the end of a kernel means waiting for the output tile to drain).
__device__ __forceinline__ void cluster_sync_relaxed() {
  asm volatile("barrier.cluster.arrive.relaxed.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of the same shared-memory offset in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
// fp32 load from the shared memory of another CTA of the cluster (address from mapa)
__device__ __forceinline__ float ld_dsmem_f32(uint32_t cluster_addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(cluster_addr) : "memory");
  return v;
}
// Without release semantics: for hand-offs whose data never went through memory (a tensor-memory buffer
// already read into registers).  A release at cluster scope stalls the arriving warp for ~1000 cycles.
__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// 2-D tile load into this CTA's shared memory, completion counted on a barrier that may live in the
// other CTA of the pair (shared::cluster address).  No multicast.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* m, int c0, int c1, uint32_t bar_cluster) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(c0), "r"(c1), "r"(bar_cluster)
      : "memory");
}
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
__device__ __forceinline__ void mma_f16_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
template <bool F8>
__device__ __forceinline__ void mma_8bit_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                              uint32_t accumulate) {
  if (F8) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
// Arrives once on the barrier at this offset in every CTA of `cta_mask` when the MMAs issued so far complete.
__device__ __forceinline__ void mma_commit_pair(uint32_t bar, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
      "h"(cta_mask)
      : "memory");
}

// One K block of a CTA pair's fp16/bf16 GEMM in a single instruction stream: tests of two barriers of the NEXT
// block (parity `parity`), then - in the lane with el != 0 - four MMAs over consecutive 16-element K steps (the
// descriptors advance by 32 bytes = 2 address units) and a commit to `commit_bar` in both CTAs.  The tests' results
// are read after the MMAs have been issued, so their latency is not added to the issuing warp's critical path.
// Returns 1 when both probed barriers had completed that phase.
__device__ __forceinline__ uint32_t mma4_commit_probe_pair(uint32_t el, uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                                           uint32_t idesc, uint32_t accumulate, uint32_t commit_bar,
                                                           uint32_t probe_a, uint32_t probe_b, uint32_t parity) {
  uint32_t ready;
  asm volatile(
      "{\n\t"
      ".reg .pred pe, pacc, pt, p1, p2;\n\t"
      ".reg .b64 a1, b1, a2, b2, a3, b3;\n\t"
      ".reg .b16 m;\n\t"
      "setp.ne.b32 pe, %1, 0;\n\t"
      "setp.ne.b32 pacc, %6, 0;\n\t"
      "setp.eq.b32 pt, %1, %1;\n\t"
      "mov.b16 m, 3;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p1, [%8], %10;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p2, [%9], %10;\n\t"
      "add.s64 a1, %3, 2;\n\tadd.s64 b1, %4, 2;\n\t"
      "add.s64 a2, %3, 4;\n\tadd.s64 b2, %4, 4;\n\t"
      "add.s64 a3, %3, 6;\n\tadd.s64 b3, %4, 6;\n\t"
      "@pe tcgen05.mma.cta_group::2.kind::f16 [%2], %3, %4, %5, pacc;\n\t"
      "@pe tcgen05.mma.cta_group::2.kind::f16 [%2], a1, b1, %5, pt;\n\t"
      "@pe tcgen05.mma.cta_group::2.kind::f16 [%2], a2, b2, %5, pt;\n\t"
      "@pe tcgen05.mma.cta_group::2.kind::f16 [%2], a3, b3, %5, pt;\n\t"
      "@pe tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%7], m;\n\t"
      "and.pred p1, p1, p2;\n\t"
      "selp.u32 %0, 1, 0, p1;\n\t"
      "}"
      : "=r"(ready)
      : "r"(el), "r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(commit_bar), "r"(probe_a),
        "r"(probe_b), "r"(parity)
      : "memory");
  return ready;
}

// ---- TMEM -> registers: lane = 32*(warp%4) + laneid, 32 consecutive 32-bit columns ------------
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
        "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
        "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
        "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
// Same, 16 columns.
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
// registers -> TMEM, same shape: 32 lanes of the warp's quadrant x 32 columns.
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

}  // namespace tc

// ---- host: tensor maps ----------------------------------------------------------------------
// 2-D row-major tensor of `rows` x `inner` elements of `elem_bytes` bytes (1 or 2),
// box `box_inner` x `box_rows`.  swizzle128: 128-byte swizzle (box_inner*elem_bytes == 128)
// or none.  Returns 0 or a negative ASRQ status.
int make_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, bool bf16, uint64_t inner, uint64_t rows,
                 uint32_t box_inner, uint32_t box_rows, bool swizzle128);

}  // namespace asrq
