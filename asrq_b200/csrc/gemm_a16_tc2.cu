// Prefill / encoder path on CTA pairs: y[M,N] = x[M,K] . dequant(W)[N,K]^T (+ bias) for large M.
//
// Same roles as gemm_a16_tc.cu, but two CTAs of a cluster share one MMA (tcgen05 cta_group::2,
// M = 256): CTA r of the pair dequantises feature tile 2j + r (its 128 A rows) into its own shared
// memory and loads HALF of the activation tile (BT/2 token rows) by TMA; one thread of CTA 0 issues
// 128x(2)xBTx16 MMAs that read A from both CTAs and B halves from both, and each CTA gets its own
// feature tile's accumulators in its own tensor memory.  Per SM and K block that halves the
// activation rows the TMA unit has to fetch and the number of MMA instructions to issue, which is
// what bounds the one-CTA kernel.
//
// Barriers (all in shared memory, same offsets in both CTAs):
//   wfull[w]   local    packed weights of slot w landed (this CTA's own TMA; the weight ring is separate from the
//                       activation stages, so weights run ahead of the MMAs by up to eight K blocks)
//   wfree[w]   local    slot w unpacked by the four warps of a dequant group
//   full[s]    CTA 0    both halves of the activation tile landed (TMA of both CTAs, byte count)
//   deq[a]     CTA 0    A slot a written in BOTH CTAs (256 arrivals, CTA 1's come over the cluster)
//   afree[a]   both     A slot a and activation stage a consumed (multicast tcgen05.commit of CTA 0's issuer; the
//                       two rings have the same depth, so one commit per K block serves both)
//   accf[b]    both     accumulator buffer b complete (multicast commit)
//   acce[b]    CTA 0    buffer b drained by both CTAs' epilogues (256 arrivals)
// Every barrier has one consumer that sees each phase in order.  No TMA multicast.  Every wait is bounded.
#include <algorithm>
#include <cstdlib>

#include "dequant.cuh"
#include "tcgen05.cuh"

namespace asrq {

int ensure_dynamic_smem(const void* kernel, size_t bytes);

namespace {

struct GemmTc2Params {
  const __half* scales;
  const __half* zeros;
  const __half* bias;
  uint16_t* y;
  unsigned* status;
  int M, N, K, group_size, groups_per_row, bt, nstages, n_fpairs, n_ttiles;
  int release_arrive;  // 1: the peer CTA's "A slot written" arrivals carry release semantics at cluster scope
  long long* trace;    // builds with -DASRQ_TRACE: clock marks of one block (4 roles x 64 events x 4 marks), else NULL
  int trace_block;
  long long* gtrace;   // same builds: globaltimer marks of every block (entry, set-up, released, loads issued, exit)
};

#ifdef ASRQ_TRACE
#define T2_MARK(role, idx, m)                                                                          \
  do {                                                                                                 \
    if (p.trace && int(blockIdx.x) == p.trace_block && lane == 0 && (idx) < 64)                        \
      p.trace[((role) * 64 + (idx)) * 4 + (m)] = clock64();                                            \
  } while (0)
#else
#define T2_MARK(role, idx, m) do { } while (0)
#endif

constexpr int kT2Groups = 3;
constexpr int kT2Slots = 6;  // A slots: two per dequant group (slot = K-block count % 6, group = count % 3), so that a
                             // group need not wait for the MMAs of its previous block before starting the next
constexpr int kT2Warps = 20;
constexpr int kT2Threads = 32 * kT2Warps;
// Roles by warp: 0 TMA producer of activations, 1 MMA issuer, 2 TMA producer of packed weights, 3 none, 4-15 dequant (group g = warps 4+4g .. 7+4g: one warp
// on each of the SM's four schedulers, three dequant warps per scheduler), 16-19 epilogue (lane quadrant warp % 4).
constexpr int kT2MmaWarp = 1, kT2ProducerWarp = 0, kT2WeightWarp = 2;
constexpr int kT2FirstDequantWarp = 4, kT2FirstEpilogueWarp = 16;
constexpr int kT2Drainers = 4;  // warps per lane quadrant that drain the last unit: the epilogue warp and one per group
constexpr int kT2MaxStages = 8;
constexpr uint32_t kT2ATileBytes = 128 * 128;  // one dequantised A slot: 128 rows x 64 16-bit elements
constexpr uint32_t kT2WSlotBytes = 4096;       // packed weights of one K block (<= 128 x 32 B)
constexpr int kT2WSlots = 8;                    // ring of packed-weight slots, independent of the activation stages

// y = accumulator + bias for chunks ch0, ch0 + step, ... (32 tokens each) of one accumulator tile, for the calling
// warp's 32 features (one per lane). Not inlined: it is called from three roles, and its 32 accumulator registers
// must not add to the dequant warps' live set.
template <bool BF16>
__device__ __noinline__ void t2_drain(uint16_t* y, int N, int rows_left, int chunks, float bias, uint32_t taddr,
                                      int ch0, int step) {
  for (int ch = ch0; ch < chunks; ch += step) {
    // one output column (token) per register: the warp's 32 lanes write 32 consecutive features
    uint16_t* yp = y + size_t(ch) * 32 * N;
    uint32_t r[32];
    tc::tmem_ld_32x32(taddr + ch * 32, r);
    tc::tmem_ld_wait();
    if (rows_left >= (ch + 1) * 32) {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        *yp = float_to_out16(__uint_as_float(r[j]) + bias, BF16);
        yp += N;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if (ch * 32 + j < rows_left) *yp = float_to_out16(__uint_as_float(r[j]) + bias, BF16);
        yp += N;
      }
    }
  }
}

template <int BITS, bool BF16>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kT2Threads, 1)
gemm_a16_tc2_kernel(const __grid_constant__ CUtensorMap tmx, const __grid_constant__ CUtensorMap tmw,
                    const GemmTc2Params p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[2 * kT2MaxStages + 2 * kT2WSlots + 2 * kT2Slots + 5];
  __shared__ uint32_t tmem_slot;

  // the next kernel on the stream may begin its set-up and weight fetch on SMs this grid leaves idle
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#ifdef ASRQ_TRACE
  if (p.gtrace && threadIdx.x == 0) p.gtrace[blockIdx.x * 8 + 0] = tc::globaltimer_ns();
#endif
  const uint32_t raw_addr = tc::smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  const uint32_t xbytes = uint32_t(p.bt / 2) * 128u;  // this CTA's half of the activation tile
  constexpr uint32_t a_ring_bytes = kT2Slots * kT2ATileBytes;
  constexpr uint32_t wbytes = 128u * 8u * BITS;
  const int nst = p.nstages;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = tc::cluster_ctarank();  // 0: issues the MMAs and owns the shared barriers
  const int cluster = blockIdx.x >> 1, nclusters = gridDim.x >> 1;
  const uint32_t bar0 = tc::smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  constexpr int kB0 = 2 * kT2MaxStages + 2 * kT2WSlots;
  auto wfull_bar = [&](int s) { return bar0 + 8u * (2 * kT2MaxStages + s); };
  auto wfree_bar = [&](int s) { return bar0 + 8u * (2 * kT2MaxStages + kT2WSlots + s); };
  auto deq_bar = [&](int a) { return bar0 + 8u * (kB0 + a); };
  auto afree_bar = [&](int a) { return bar0 + 8u * (kB0 + kT2Slots + a); };
  auto accf_bar = [&](int b) { return bar0 + 8u * (kB0 + 2 * kT2Slots + b); };
  auto acce_bar = [&](int b) { return bar0 + 8u * (kB0 + 2 * kT2Slots + 2 + b); };
  const uint32_t fin_bar = bar0 + 8u * (kB0 + 2 * kT2Slots + 4);  // the last unit's accumulator is complete
  const uint32_t x_ring = a_ring_bytes, w_ring = a_ring_bytes + uint32_t(nst) * xbytes;  // offsets from base
  // One arrival per warp on a barrier of CTA 0, from either CTA, after every lane has made its writes
  // visible to the async proxy (fence.proxy.async) and the warp has synchronised.
  // "Accumulator drained" carries no data through memory (the values are in registers), so its remote
  // arrival is relaxed.  "A slot written" hands over shared-memory contents of the peer CTA that the
  // pair's MMA then reads: `release` selects mbarrier.arrive.release.cluster for it (the memory model's
  // release/acquire edge; it stalls the arriving warp ~1000 cycles).  The relaxed form relies on the
  // hardware performing a CTA's own shared-memory stores, and the proxy fence after them, before a later
  // remote arrival of the same thread leaves the SM; tests/test_gpu_a16.py repeats large shapes and
  // compares both forms bit for bit with the one-CTA kernel.
  auto arrive_on_leader = [&](uint32_t bar, bool release) {
    __syncwarp();
    if (lane == 0) {
      if (rank == 0) {
        tc::mbar_arrive(bar);
      } else if (release) {
        tc::mbar_arrive_cluster(tc::mapa(bar, 0));
      } else {
        tc::mbar_arrive_cluster_relaxed(tc::mapa(bar, 0));
      }
    }
  };

  {
    // one barrier per thread: expected arrivals by position in the array
    constexpr int kNBars = kB0 + 2 * kT2Slots + 5;
    const int i = threadIdx.x;
    if (i < kNBars) {
      uint32_t count = 1;                                                         // full, wfull, afree, accf, fin
      if (i >= 2 * kT2MaxStages + kT2WSlots && i < kB0) count = 4;               // wfree: the four warps of a dequant group
      if (i >= kB0 && i < kB0 + kT2Slots) count = 8;                             // deq: four dequant warps of each CTA
      if (i >= kB0 + 2 * kT2Slots + 2 && i < kB0 + 2 * kT2Slots + 4) count = 8;  // acce: four epilogue warps of each CTA
      tc::mbar_init(bar0 + 8u * i, count);
      tc::fence_barrier_init();
      tc::fence_proxy_async_smem();
    }
    if (threadIdx.x == 32 * kT2ProducerWarp) tc::prefetch_tmap(&tmx);
    if (threadIdx.x == 32 * kT2WeightWarp) tc::prefetch_tmap(&tmw);
  }
  if (warp == kT2MmaWarp) {
    tc::tmem_alloc_pair(tc::smem_u32(&tmem_slot), 512);
    tc::tmem_relinquish_pair();
  }
  tc::fence_before_sync();
  __syncthreads();
#ifdef ASRQ_TRACE
  if (p.gtrace && threadIdx.x == 0) p.gtrace[blockIdx.x * 8 + 5] = tc::globaltimer_ns();
#endif
  // The peer's barriers are initialised before anything arrives on them.  (Splitting this barrier - arrive here,
  // wait where a role first touches the other CTA, so that the first weight blocks are fetched and unpacked
  // meanwhile - measured 0.3 us slower per launch than the plain barrier.)
  tc::cluster_sync();
  tc::fence_after_sync();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&tmem_slot);
#ifdef ASRQ_TRACE
  if (p.gtrace && threadIdx.x == 0) p.gtrace[blockIdx.x * 8 + 1] = tc::globaltimer_ns();
#endif

  const int nunits = p.n_fpairs * p.n_ttiles;  // a unit: feature tiles 2j, 2j+1 of token tile tt
  const int nkb = p.K / 64;
  // position among the twelve dequant warps, -1: not a dequant warp
  const int dpos = (warp >= kT2FirstDequantWarp && warp < kT2FirstEpilogueWarp) ? warp - kT2FirstDequantWarp : -1;
  // The last unit of this pair: nothing runs under its epilogue, so the drain of its accumulator is shared
  // by four warps per lane quadrant (the epilogue warp plus the dequant warps of that quadrant, idle by then).
  const int my_units = (nunits - cluster + nclusters - 1) / nclusters;
  const int last_unit = cluster + (my_units - 1) * nclusters;
  const int helper = dpos >= 0 ? 1 + (dpos >> 2) : (warp >= kT2FirstEpilogueWarp ? 0 : -1);  // position among the drainers
  // y = accumulator + bias for chunks ch0, ch0 + step, ... (32 tokens each) of `unit`'s tile, this warp's 32 features
  auto drain = [&](int unit, uint32_t buf, int ch0, int step) {
    __syncwarp();  // the tensor-memory loads are warp-wide instructions: the lanes come out of a polling loop
    const int fp = unit % p.n_fpairs, tt = unit / p.n_fpairs;
    const int f = (2 * fp + int(rank)) * 128 + (warp & 3) * 32 + lane;
    t2_drain<BF16>(p.y + size_t(tt) * p.bt * p.N + f, p.N, p.M - tt * p.bt, p.bt / 32,
                   p.bias ? __half2float(__ldg(p.bias + f)) : 0.f,
                   tmem_base + (uint32_t((warp & 3) * 32) << 16) + buf * 256u, ch0, step);
  };
  // a helper that is not an epilogue warp: wait for the last unit's accumulator, drain its share
  auto help_drain = [&]() {
    if (helper > 0 && __all_sync(0xffffffffu, tc::mbar_wait(fin_bar, 0u, p.status, 8))) {
      tc::fence_after_sync();
      drain(last_unit, uint32_t(my_units - 1) & 1u, helper, kT2Drainers);
    }
  };

  if (warp == kT2ProducerWarp) {
    // ------------------------------ TMA producer of activations (both CTAs) ------------------------------
    // Launched with programmatic stream serialisation: activations may be written by the kernel before this one
    // on the stream, so their loads start after griddepcontrol.wait.
    if (lane == 0) {
      const uint32_t full0 = tc::mapa(full_bar(0), 0);  // CTA 0's full barriers, as seen from here
      asm volatile("griddepcontrol.wait;" ::: "memory");
#ifdef ASRQ_TRACE
      if (p.gtrace) p.gtrace[blockIdx.x * 8 + 2] = tc::globaltimer_ns();
#endif
      uint32_t ph = 0;
      int s = 0, step = 0;
      (void)step;
      bool ok = true;
      for (int unit = cluster; unit < nunits && ok; unit += nclusters) {
        const int tt = unit / p.n_fpairs;
        const int row_x = tt * p.bt + int(rank) * (p.bt / 2);
        for (int kb = 0; kb < nkb; ++kb, ++step) {
          T2_MARK(3, step, 0);
          if (!tc::mbar_wait(afree_bar(s), ph ^ 1u, p.status, 1)) { ok = false; break; }
          T2_MARK(3, step, 1);
          if (rank == 0) tc::mbar_arrive_expect_tx(full_bar(s), 2u * xbytes);
          tc::tma_load_2d_pair(base + x_ring + s * xbytes, &tmx, kb * 64, row_x, full0 + 8u * s);
          if (++s == nst) { s = 0; ph ^= 1u; }
        }
      }
    }
  } else if (warp == kT2WeightWarp) {
    // ------------------------------ TMA producer of packed weights (both CTAs) ------------------------------
    // Packed weights are constants, so this warp does not wait for the stream dependency: it runs up to
    // kT2WSlots K blocks ahead of the dequant warps, which unpack the first blocks into the A slots while the
    // kernel before this one on the stream is still finishing.  A slot is free again when the four warps of the
    // dequant group that read it have arrived on wfree.
    if (lane == 0) {
      uint32_t ph = 0;
      int s = 0, step = 0;
      (void)step;
      bool ok = true;
      for (int unit = cluster; unit < nunits && ok; unit += nclusters) {
        const int row_w = (2 * (unit % p.n_fpairs) + int(rank)) * 128;
        for (int kb = 0; kb < nkb; ++kb, ++step) {
          if (!tc::mbar_wait(wfree_bar(s), ph ^ 1u, p.status, 9)) { ok = false; break; }
          tc::mbar_arrive_expect_tx(wfull_bar(s), wbytes);
          tc::tma_load_2d(base + w_ring + s * kT2WSlotBytes, &tmw, kb * 8 * BITS, row_w, wfull_bar(s));
          if (++s == kT2WSlots) { s = 0; ph ^= 1u; }
        }
      }
    }
  } else if (warp == kT2MmaWarp) {
    // ------------------------------ MMA issuer (CTA 0 only) ------------------------------
    // Run by the whole warp (counters and descriptors stay warp-uniform), tcgen05 instructions in one elected lane.
    // The warp's own instruction latency is the critical path of the kernel (a barrier test costs 100 - 200 clocks,
    // the MMAs of a K block run 512), so the tests for the NEXT block's two barriers are issued ahead of this
    // block's MMAs and read after them; the waiting loop runs only when that probe found a barrier incomplete.
    if (rank == 0) {
      const uint32_t el = tc::elect_one() ? 1u : 0u;
      const uint32_t idesc = tc::instr_desc(1u, BF16 ? 1u : 0u, 256u, uint32_t(p.bt));
      uint32_t dph = 0, ucount = 0, ready = 0;
      int a = 0;  // A slot and activation stage of the current K block (the two rings have the same depth)
      int tstep = 0;
      (void)tstep;
      bool ok = true;
      for (int unit = cluster; unit < nunits && ok; unit += nclusters, ++ucount) {
        const uint32_t buf = ucount & 1u;
        const uint32_t d_tmem = tmem_base + buf * 256u;
        // the accumulator buffer must have been drained by both CTAs
        ok = tc::mbar_wait_spin(acce_bar(buf), ((ucount >> 1) & 1u) ^ 1u, p.status, 2);
        for (int kb = 0; kb < nkb && ok; ++kb, ++tstep) {
          T2_MARK(0, tstep, 0);
          if (!ready || p.release_arrive) {
            ok = (p.release_arrive ? tc::mbar_wait_spin_cluster(deq_bar(a), dph, p.status, 4)
                                   : tc::mbar_wait_spin(deq_bar(a), dph, p.status, 4)) &&
                 tc::mbar_wait_spin(full_bar(a), dph, p.status, 3);
            if (!ok) break;
          }
          T2_MARK(0, tstep, 2);
          tc::fence_after_sync();
          int an = a + 1;
          uint32_t dphn = dph;
          if (an == kT2Slots) { an = 0; dphn ^= 1u; }
          // the four MMAs of the block (a K step of 16 elements = 32 bytes = +2 in the descriptors' 16-byte address
          // field), one commit that frees the A slot and the activation stage in both CTAs, and the probe
          ready = tc::mma4_commit_probe_pair(el, d_tmem, tc::smem_desc_sw128(base + a * kT2ATileBytes),
                                             tc::smem_desc_sw128(base + x_ring + a * xbytes), idesc, uint32_t(kb != 0),
                                             afree_bar(a), deq_bar(an), full_bar(an), dphn);
          if (el && kb + 1 == nkb) {
            tc::mma_commit_pair(accf_bar(buf), 3);
            if (unit == last_unit) tc::mma_commit_pair(fin_bar, 3);
          }
          T2_MARK(0, tstep, 3);
          a = an;
          dph = dphn;
        }
      }
    }
  } else if (dpos >= 0) {
    // ------------------------------ dequant (both CTAs) ------------------------------
    const int t = (dpos & 3) * 32 + lane;  // weight row inside the tile
    const int dgroup = dpos >> 2;          // this warp group takes K blocks dgroup, dgroup+3, ... and owns A slot dgroup
    int unit = cluster, kb = dgroup;
    while (kb >= nkb && unit < nunits) { kb -= nkb; unit += nclusters; }
    int s = dgroup;  // packed-weight slot of the current K block (count % kT2WSlots) and the parity of its use count
    uint32_t ph = 0;
    static_assert(kT2Groups <= kT2WSlots, "the first block of every group starts in the ring's first pass");
    int a = dgroup;    // A slot of the current K block (count % kT2Slots) and the parity of its use count
    uint32_t aph = 0;
    const int kbpg = p.group_size / 64;  // K blocks per weight group
    // Scale and zero of this thread's row for K block k of unit u, fetched one iteration (three K blocks) ahead.
    // Volatile asm: the loads are issued here, not moved down to their first use.
    int sz_unit = -1;
    size_t sz_row = 0;
    auto load_sz = [&](int u, int k) -> uint32_t {
      if (u != sz_unit) {
        sz_unit = u;
        sz_row = (size_t(2 * (u % p.n_fpairs) + int(rank)) * 128 + t) * p.groups_per_row;
      }
      const int gi = kbpg == 1 ? k : (kbpg == 2 ? (k >> 1) : k / kbpg);
      uint16_t sv, zv;
      asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(sv) : "l"(p.scales + sz_row + gi));
      asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(zv) : "l"(p.zeros + sz_row + gi));
      return uint32_t(sv) | (uint32_t(zv) << 16);
    };
    uint32_t sz_next = unit < nunits ? load_sz(unit, kb) : 0u;
    int titer = 0;
    (void)titer;
    while (unit < nunits) {
      const uint32_t sz = sz_next;
      int nunit = unit, nk = kb + kT2Groups;
      while (nk >= nkb && nunit < nunits) { nk -= nkb; nunit += nclusters; }
      if (nunit < nunits) sz_next = load_sz(nunit, nk);  // consumed three K blocks from now
      const __half sh = __ushort_as_half(uint16_t(sz & 0xffffu)), zh = __ushort_as_half(uint16_t(sz >> 16));
      uint32_t s2, z2;
      if (BF16) {
        s2 = __float_as_uint(__half2float(sh));
        z2 = __float_as_uint(__half2float(zh));
      } else {
        s2 = h2_as_u32(__half2half2(sh));
        z2 = h2_as_u32(__half2half2(zh));
      }
      // the A slot must have been consumed by the MMAs of the K block that used it last (six blocks ago):
      // their commit arrived on the slot's barrier in both CTAs.  Both barriers are tested in one go, the A slot's
      // first.  The packed-weight slot's barrier is shared by the three groups in turn, and a parity test can only
      // tell a phase from its neighbours: while the slot's PREVIOUS pass (eight K blocks ago, another group's) has not
      // landed, the test for this pass reads "complete".  That pass has landed once this block's A slot is free (the
      // MMAs of the block two after it are done), so the weight slot's test counts only if it was made after the A
      // slot's test succeeded; otherwise it is made again.
      if (dpos == 0) T2_MARK(1, titer, 0);
      {
        const uint32_t got = tc::mbar_try_wait2(afree_bar(a), aph ^ 1u, wfull_bar(s), ph);
        bool okw = true;
        if (!(got & 1u)) {
          okw = tc::mbar_wait(afree_bar(a), aph ^ 1u, p.status, 7) && tc::mbar_wait(wfull_bar(s), ph, p.status, 5);
        } else if (!(got & 2u)) {
          okw = tc::mbar_wait(wfull_bar(s), ph, p.status, 5);
        }
        // one decision for the warp: a wait that gave up ends the loop for all its lanes (the warp barriers below
        // need every lane).  Nothing below assumes that the lanes run in step after this vote.
        if (!__all_sync(0xffffffffu, okw)) break;
      }
      if (dpos == 0) T2_MARK(1, titer, 2);
      constexpr int NV = BITS / 2;  // 16-byte vectors of packed weights per row per K block
      uint4 qv[NV];
#pragma unroll
      for (int v = 0; v < NV; ++v) qv[v] = tc::ld_shared_v4(base + w_ring + s * kT2WSlotBytes + t * (8 * BITS) + v * 16);
      // 128-byte swizzle: 16-byte chunk c of row t lives at chunk position c ^ (t % 8); the row start is 128-byte
      // aligned, so the position is an XOR on the address
      const uint32_t arow = (base + a * kT2ATileBytes + t * 128) | uint32_t((t & 7) << 4);
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        const uint32_t qw[4] = {qv[v].x, qv[v].y, qv[v].z, qv[v].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          constexpr int PW = 32 / BITS / 2;  // output pairs per word: 4 or 8
          uint32_t o[PW];
          dequant_word<BITS, BF16>(qw[j], s2, z2, o);
#pragma unroll
          for (int cc = 0; cc < PW / 4; ++cc) {
            const int chunk = (v * 4 + j) * (PW / 4) + cc;  // 16-byte chunk (8 elements) in the row
            tc::st_shared_v4(arow ^ uint32_t(chunk << 4), o[4 * cc], o[4 * cc + 1], o[4 * cc + 2], o[4 * cc + 3]);
          }
        }
      }
      tc::fence_proxy_async_smem();
      // The packed-weight slot is released only here, after the stores that consumed its words and behind a warp
      // barrier: every lane has finished with the slot, whatever the lanes' relative progress was.  (Released right
      // after the loads by lane 0, even behind a warp-wide reduction over the loaded words, the next TMA write into
      // the slot was seen to land between the two 16-byte loads of lanes that ran behind lane 0: one K block of a few
      // weight rows then held the codes of the block eight further on, once in some thousand launches.)
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(wfree_bar(s));
      arrive_on_leader(deq_bar(a), p.release_arrive != 0);
      if (dpos == 0) T2_MARK(1, titer, 3);
      ++titer;
      unit = nunit;
      kb = nk;
      s += kT2Groups;
      if (s >= kT2WSlots) { s -= kT2WSlots; ph ^= 1u; }
      a += kT2Groups;
      if (a >= kT2Slots) { a -= kT2Slots; aph ^= 1u; }
    }
    help_drain();
  } else if (warp >= kT2FirstEpilogueWarp) {
    // ------------------------------ epilogue (both CTAs) ------------------------------
    uint32_t ucount = 0;
    bool ok = true;
    for (int unit = cluster; unit < nunits && ok; unit += nclusters, ++ucount) {
      const uint32_t buf = ucount & 1u, aph = (ucount >> 1) & 1u;
      if (warp == kT2FirstEpilogueWarp) T2_MARK(2, ucount, 0);
      if (!__all_sync(0xffffffffu, tc::mbar_wait(accf_bar(buf), aph, p.status, 6))) { ok = false; break; }
      if (warp == kT2FirstEpilogueWarp) T2_MARK(2, ucount, 1);
      tc::fence_after_sync();
      if (unit == last_unit) {
        drain(unit, buf, 0, kT2Drainers);  // shared with the dequant warps of the same lane quadrant
      } else {
        drain(unit, buf, 0, 1);
      }
      tc::fence_before_sync();
      // Nobody waits for the last unit's "drained", and it must not be sent: the closing barrier over the pair is an
      // execution barrier only, so a remote arrival still in flight could land in shared memory that the leader
      // CTA has already handed to the next kernel's block.
      if (unit != last_unit) arrive_on_leader(acce_bar(buf), false);
      if (warp == kT2FirstEpilogueWarp) T2_MARK(2, ucount, 2);
    }
#ifdef ASRQ_TRACE
    if (p.gtrace && warp == kT2FirstEpilogueWarp && lane == 0) p.gtrace[blockIdx.x * 8 + 7] = tc::globaltimer_ns();
#endif
  }

#ifdef ASRQ_TRACE
  if (p.gtrace && threadIdx.x == 0) p.gtrace[blockIdx.x * 8 + 3] = tc::globaltimer_ns();
#endif
  __syncwarp();
  tc::fence_before_sync();
  __syncthreads();
  // neither CTA leaves while the other may still signal its barriers or read its memory; an execution barrier is
  // enough (nothing is handed over through memory here), and it does not wait for the output stores to drain
  tc::cluster_sync_relaxed();
#ifdef ASRQ_TRACE
  if (p.gtrace && threadIdx.x == 0) p.gtrace[blockIdx.x * 8 + 6] = tc::globaltimer_ns();
#endif
  if (warp == kT2MmaWarp) {
    tc::fence_after_sync();
    tc::tmem_dealloc_pair(tmem_base, 512);
  }
#ifdef ASRQ_TRACE
  if (p.gtrace && threadIdx.x == 32 * kT2MmaWarp) p.gtrace[blockIdx.x * 8 + 4] = tc::globaltimer_ns();
#endif
}

// Token-tile width: the multiple of 32 (<= 256, <= M) that minimises rounds over the CTA pairs x
// (tile width + fixed per-tile overhead).
int pick_bt(int64_t M, int64_t npairs, int nclusters) {
  const int forced = option(kOptTcBt);  // tuning knob: force the token-tile width
  if (forced >= 32 && forced <= 256 && forced % 32 == 0) return forced;
  int best = 32;
  double best_cost = 1e30;
  for (int bt = 32; bt <= 256; bt += 32) {
    if (bt > M && bt != 32) break;
    const int64_t units = npairs * ((M + bt - 1) / bt);
    const int64_t rounds = (units + nclusters - 1) / nclusters;
    // a K block costs its MMAs (2 clocks per token column on a pair) or the fixed work beside them (dequantising a
    // 128 x 64 weight tile, the issuing warp's own loop: about 540 clocks measured), whichever is longer
    const double cost = double(rounds) * std::max(2.0 * bt, 540.0) + 1e-3 * double(units);
    if (cost <= best_cost) {
      best_cost = cost;
      best = bt;
    }
  }
  return best;
}

template <int BITS, bool BF16>
int launch_tc2(const CUtensorMap& tmx, const CUtensorMap& tmw, const GemmTc2Params& p, int grid, size_t smem,
               cudaStream_t stream) {
  auto kern = gemm_a16_tc2_kernel<BITS, BF16>;
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem)) return rc;
  cudaLaunchConfig_t cfg = {};  // the cluster shape comes from __cluster_dims__
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kT2Threads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = option(kOptNoPdl) ? 0 : 1;
  ASRQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, tmx, tmw, p));
  return ASRQ_OK;
}

}  // namespace

// The pair kernel needs an even number of feature tiles and enough work for the CTA pairs.
bool gemm_a16_tc2_supports(int64_t M, int64_t N, int64_t K, int group_size) {
  return M >= 64 && N % 256 == 0 && K % 64 == 0 && group_size > 0 && group_size % 64 == 0 && K % group_size == 0;
}

int gemm_a16_tc2(int bits, const void* x, const uint8_t* w, const void* scales, const void* zeros, const void* bias,
                 void* y, int64_t M, int64_t N, int64_t K, int group_size, int dtype, void* workspace,
                 size_t workspace_bytes, int sm_count, cudaStream_t stream) {
  if (!gemm_a16_tc2_supports(M, N, K, group_size))
    return fail(ASRQ_ERR_SHAPE, "w%da16 gemm (pair): unsupported shape N=%lld K=%lld g=%d", bits, (long long)N,
                (long long)K, group_size);
  if (M > (1ll << 30) || N > (1ll << 30) || K > (1ll << 24)) return fail(ASRQ_ERR_LIMIT, "w%da16 gemm: size", bits);
  if (workspace_bytes < kStatusBytes) return fail(ASRQ_ERR_WORKSPACE, "w%da16 gemm: workspace too small", bits);
  if (!aligned16(x) || !aligned16(w)) return fail(ASRQ_ERR_ALIGN, "w%da16 gemm: x and w must be 16-byte aligned", bits);

  GemmTc2Params p;
  p.scales = static_cast<const __half*>(scales);
  p.zeros = static_cast<const __half*>(zeros);
  p.bias = static_cast<const __half*>(bias);
  p.y = static_cast<uint16_t*>(y);
  p.status = static_cast<unsigned*>(workspace);
  p.M = int(M);
  p.N = int(N);
  p.K = int(K);
  p.group_size = group_size;
  p.groups_per_row = int(K / group_size);
  p.n_fpairs = int(N / 256);
  p.release_arrive = option(kOptTcPairRelease);
  p.trace = nullptr;
  p.gtrace = nullptr;
  p.trace_block = 0;
#ifdef ASRQ_TRACE
  if (option(kOptTrace) && workspace_bytes >= (8u << 20)) {
    static unsigned launch_no = 0;  // consecutive launches alternate between two mark blocks
    p.trace = reinterpret_cast<long long*>(static_cast<char*>(workspace) + (4u << 20)) + size_t(launch_no & 1u) * 1024;
    p.gtrace = reinterpret_cast<long long*>(static_cast<char*>(workspace) + (5u << 20)) + size_t(launch_no & 7u) * 148 * 8;
    ++launch_no;
    p.trace_block = option(kOptTraceBlock);
  }
#endif
  const int max_clusters = sm_count / 2;
  p.bt = pick_bt(M, p.n_fpairs, max_clusters);
  p.n_ttiles = int((M + p.bt - 1) / p.bt);
  const size_t stage_bytes = size_t(p.bt / 2) * 128;  // one CTA's half of an activation tile
  const size_t fixed = kT2Slots * kT2ATileBytes + kT2WSlots * kT2WSlotBytes;
  const size_t budget = 227 * 1024 - 1024 - 512 - fixed;
  p.nstages = kT2Slots;  // the activation ring is as deep as the A ring: one barrier frees both
  if (size_t(p.nstages) * stage_bytes > budget) return fail(ASRQ_ERR_LIMIT, "w%da16 gemm (pair): shared memory", bits);
  const size_t smem = 1024 + fixed + p.nstages * stage_bytes;

  const bool bf16 = dtype == ASRQ_BF16;
  CUtensorMap tmx, tmw;
  int rc = make_tmap_2d(&tmx, x, 2, bf16, uint64_t(K), uint64_t(M), 64, uint32_t(p.bt / 2), true);
  if (rc) return rc;
  rc = make_tmap_2d(&tmw, w, 1, false, uint64_t(K) * bits / 8, uint64_t(N), uint32_t(8 * bits), 128, false);
  if (rc) return rc;
  const int nclusters = int(std::min<int64_t>(int64_t(p.n_fpairs) * p.n_ttiles, max_clusters));
  const int grid = 2 * nclusters;
  if (bits == 4)
    return bf16 ? launch_tc2<4, true>(tmx, tmw, p, grid, smem, stream) : launch_tc2<4, false>(tmx, tmw, p, grid, smem, stream);
  return bf16 ? launch_tc2<2, true>(tmx, tmw, p, grid, smem, stream) : launch_tc2<2, false>(tmx, tmw, p, grid, smem, stream);
}

}  // namespace asrq
