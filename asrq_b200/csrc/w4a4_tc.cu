// W4A4 GEMM on tcgen05 kind::i8: exact int32 group sums in TMEM, fused dequant.
//
// Two steps per call, both on the caller's stream:
//
//  1. expand: packed signed nibbles -> int8 holding 16x the value, natural k order
//     ((q << 4) & 0xf0f0f0f0 gives the even k, q & 0xf0f0f0f0 the odd k, one byte permute
//     interleaves them).  Weights N x K and activations M x K go to the caller's workspace;
//     the fused LinearQQ entry skips the activation pass because its prologue writes this
//     format directly.  A product is 256x the true one; the factor is folded into the
//     weight scale (an exact power of two).
//
//  2. GEMM: one persistent block per SM.  Weight tile = MMA A operand (128 features = TMEM
//     lanes), activation tile = B operand (BT tokens = TMEM columns), both int8 K-major with
//     128-byte swizzle, loaded by TMA; a K block is 128 = one row of 128 bytes = 4 MMAs of
//     K = 32.  Every weight group (group_size / 128 K blocks) gets a fresh int32 accumulator
//     buffer in TMEM (two buffers, ping-pong); twelve drain warps read it back, convert and
//     add float(acc) * sW[feature, group] into fp32 registers while the next group is
//     multiplied.  After the last group: * sA[token] + bias, convert, store.
//
//   warp 0      TMA producer        warps 1, 2  MMA issuers, one per accumulator buffer (warp 1 owns TMEM)
//   warps 4-15  drain + epilogue: warp w reads TMEM lanes 32*(w%4).., column third (w-4)/4.
//               Three warps per scheduler: the drain (one int->float convert and one FMA per
//               output per group) needs about as many issue slots as the MMAs need cycles, so
//               it only keeps up if its instruction latencies are hidden.
#include <algorithm>
#include <cstdlib>

#include "tcgen05.cuh"

namespace asrq {

int ensure_dynamic_smem(const void* kernel, size_t bytes);

__global__ void __launch_bounds__(256)
expand_int4_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, size_t n_vec) {
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < n_vec; i += size_t(gridDim.x) * blockDim.x) {
    const uint4 q = __ldg(src + i);
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
    uint32_t o[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t e = (w[j] << 4) & 0xf0f0f0f0u;  // 16 * (k0, k2, k4, k6)
      const uint32_t d = w[j] & 0xf0f0f0f0u;         // 16 * (k1, k3, k5, k7)
      o[2 * j] = prmt(e, d, 0x5140);                 // k0 k1 k2 k3
      o[2 * j + 1] = prmt(e, d, 0x7362);             // k4 k5 k6 k7
    }
    dst[2 * i] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[2 * i + 1] = make_uint4(o[4], o[5], o[6], o[7]);
  }
}

// Packed signed nibbles -> one FP8 (e4m3) byte per code, natural k order.  -8..7 are exact in e4m3
// (1 = 0x38, 2 = 0x40, 3 = 0x44, 4 = 0x48, 5 = 0x4a, 6 = 0x4c, 7 = 0x4e, 8 = 0x50, sign = 0x80).
__device__ __forceinline__ uint32_t e4m3_of_nibble(uint32_t c) {  // c = two's-complement nibble 0..15
  const uint32_t neg = c >> 3, mag = neg ? 16u - c : c;           // magnitude 0..8
  // 0, 1, 2, 3 | 4, 5, 6, 7 | 8 as bytes of two table words and a constant
  const uint32_t lo = 0x44403800u, hi = 0x4e4c4a48u;
  const uint32_t e = mag == 8u ? 0x50u : (((mag & 4u) ? hi : lo) >> (8u * (mag & 3u))) & 0xffu;
  return e | (neg << 7);
}
__global__ void __launch_bounds__(256)
expand_int4_f8_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, size_t n_vec) {
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < n_vec; i += size_t(gridDim.x) * blockDim.x) {
    const uint4 q = __ldg(src + i);
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
    uint32_t o[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t r = 0;
#pragma unroll
        for (int e = 0; e < 4; ++e) r |= e4m3_of_nibble((w[j] >> (16 * h + 4 * e)) & 0xfu) << (8 * e);
        o[2 * j + h] = r;
      }
    }
    dst[2 * i] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[2 * i + 1] = make_uint4(o[4], o[5], o[6], o[7]);
  }
}

struct W4A4TcParams {
  const float* sa;
  const __half* sw;
  const __half* bias;
  uint16_t* y;
  int32_t* acc_dump;
  unsigned* status;
  long long* trace;  // builds with -DASRQ_TRACE: when not NULL, block `trace_block` records clock64() at pipeline milestones
  int M, N, K, groups, blocks_per_group, bt, nbuf, nstages, n_ftiles, n_ttiles, bf16, trace_block;
};

constexpr int kW4A4MaxBufs = 4;
constexpr int kW4A4MaxStages = 8;
// The CTA-pair kernel is parity-green and measures 10-15 % slower than one CTA per tile on M=6000 K=4096
// N=1024 at every tile width tried (45.6 against 40.1 us at BT=192): both are paced by the round trip of
// the two accumulator buffers, not by operand delivery.  It runs only on request.  (It was 1.8-2x
// slower until the cross-CTA arrivals lost their release semantics: a release at cluster scope stalls
// the arriving warp for ~1000 cycles, once per drain warp per group and once per stage in the relay.)
constexpr bool kW4A4PairDefault = false;
constexpr int w4a4_threads(int cg) { return 32 * (4 + 4 * cg); }  // producer, two MMA issuers, one idle, drain
constexpr uint32_t kW8TileBytes = 128 * 128;

// F8 = false: operands are int8 holding 16x the code, kind::i8, int32 sums in TMEM (256x the true sum).
// F8 = true: operands are e4m3 bytes holding the code, kind::f8f6f4, fp32 sums in TMEM: a group sum is
// an integer of magnitude <= 128 * 64, so it is exact, and the drain needs no int->float conversion.
// CG: column groups of the drain (4 * CG drain warps); NCH: 16-column chunks a drain warp handles at most.
// PAIR: two CTAs of a cluster work on one 256-feature x BT-token tile with tcgen05 cta_group::2 MMAs.
// Each CTA loads its own 128 weight rows and HALF of the activation rows of a K block (the MMA reads
// the other half from the peer's shared memory), which cuts the bytes an SM takes in per MMA cycle
// from 16 KB + BT*128 to 16 KB + BT*64 per K block.  CTA 0 issues for both, its full[] barriers count
// the bytes of both CTAs' loads, commits are multicast to both CTAs' empty[]/accf[] barriers, and the
// drain warps of both CTAs arrive on CTA 0's acce[] barriers.
template <bool DUMP, bool F8, int CG, int NCH, bool PAIR>
__device__ __forceinline__ void w4a4_tc_body(const CUtensorMap* tmw_p, const CUtensorMap* tma_p, const W4A4TcParams& p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[3 * kW4A4MaxStages + 2 * kW4A4MaxBufs];
  __shared__ uint32_t tmem_slot;

  const uint32_t raw_addr = tc::smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  const uint32_t bbytes = uint32_t(PAIR ? p.bt / 2 : p.bt) * 128u;  // this CTA's activation rows of a K block
  const uint32_t stage_bytes = kW8TileBytes + bbytes;
  const uint32_t rank = PAIR ? tc::cluster_ctarank() : 0u;
  const int worker = PAIR ? int(blockIdx.x >> 1) : int(blockIdx.x);     // tile-loop start and stride:
  const int nworkers = PAIR ? int(gridDim.x >> 1) : int(gridDim.x);     // CTAs, or CTA pairs
  const int nst = p.nstages;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t bar0 = tc::smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (kW4A4MaxStages + s); };
  auto accf_bar = [&](int b) { return bar0 + 8u * (2 * kW4A4MaxStages + b); };
  auto acce_bar = [&](int b) { return bar0 + 8u * (2 * kW4A4MaxStages + kW4A4MaxBufs + b); };
  // PAIR, CTA 0: "the peer's tiles of stage s have landed" (one remote arrival per stage by the peer's relay thread)
  auto pfull_bar = [&](int s) { return bar0 + 8u * (2 * kW4A4MaxStages + 2 * kW4A4MaxBufs + s); };

  if (threadIdx.x == 0) {
    for (int s = 0; s < nst; ++s) {
      tc::mbar_init(full_bar(s), 1);
      tc::mbar_init(empty_bar(s), 1);
      tc::mbar_init(pfull_bar(s), 1);
    }
    for (int b = 0; b < p.nbuf; ++b) {
      tc::mbar_init(accf_bar(b), 1);
      tc::mbar_init(acce_bar(b), PAIR ? 2 * 4 * CG : 32 * 4 * CG);  // per drain warp of both CTAs / per drain thread
    }
    tc::fence_barrier_init();
    tc::fence_proxy_async_smem();
    tc::prefetch_tmap(tmw_p);
    tc::prefetch_tmap(tma_p);
  }
  if (warp == 1) {
    if (PAIR) {
      tc::tmem_alloc_pair(tc::smem_u32(&tmem_slot), 512);
      tc::tmem_relinquish_pair();
    } else {
      tc::tmem_alloc(tc::smem_u32(&tmem_slot), 512);
      tc::tmem_relinquish();
    }
  }
  tc::fence_before_sync();
  __syncthreads();
  if (PAIR) tc::cluster_sync();  // the peer's barriers are initialised before anything arrives on them
  tc::fence_after_sync();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&tmem_slot);
  // Launched with programmatic stream serialisation: everything above (barriers, tensor memory,
  // descriptor prefetch) may overlap the tail of the kernel before; the activation operand, the
  // token scales and the output belong to this kernel only from here on.
  asm volatile("griddepcontrol.wait;" ::: "memory");

  // PAIR: a "tile" is the feature-tile pair (2j, 2j+1) of a token tile; this CTA owns feature tile 2j + rank
  const int n_ft = PAIR ? p.n_ftiles / 2 : p.n_ftiles;
  const int ntiles = n_ft * p.n_ttiles;
  const int nkb = p.K / 128;
#ifdef ASRQ_TRACE
  const bool tr = p.trace != nullptr && int(blockIdx.x) == p.trace_block;
  auto mark = [&](int role, uint32_t i, int slot) {
    if (tr && i < 512) p.trace[(role * 512 + i) * 2 + slot] = clock64();
  };
#else
  auto mark = [](int, uint32_t, int) {};  // the shipped kernels carry no trace branches
#endif

  // Ring positions are (index, phase) counters: no integer division inside the role loops.
  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0, ph = 0;
      int s = 0;
      bool ok = true;
      for (int tile = worker; tile < ntiles && ok; tile += nworkers) {
        const int ft = PAIR ? 2 * (tile % n_ft) + int(rank) : tile % n_ft, tt = tile / n_ft;
        const int row_w = ft * 128, row_a = tt * p.bt + (PAIR ? int(rank) * (p.bt / 2) : 0);
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          if (!tc::mbar_wait(empty_bar(s), ph ^ 1u, p.status, 11)) { ok = false; break; }
          mark(0, it, 0);
          const uint32_t sb = base + s * stage_bytes;
          // every CTA's loads complete on its own barrier (a load that counts its bytes on the peer's
          // barrier measured far slower); the peer's relay thread forwards "landed" once per stage
          tc::mbar_arrive_expect_tx(full_bar(s), kW8TileBytes + bbytes);
          tc::tma_load_2d(sb, tmw_p, kb * 128, row_w, full_bar(s));
          tc::tma_load_2d(sb + kW8TileBytes, tma_p, kb * 128, row_a, full_bar(s));
          mark(0, it, 1);
          if (++s == nst) { s = 0; ph ^= 1u; }
        }
      }
    }
  } else if (warp == 1 || warp == 2) {
    // Two MMA issuers.  Every tcgen05.mma / commit / barrier poll costs its issuing thread tens of
    // cycles, more when heavy ALU warps (the drain) share its scheduler, and one thread alone cannot
    // keep the pipe fed.  The groups of a tile alternate between the two TMEM accumulator buffers,
    // so issuer w-1 takes the groups that land in buffer w-1: the two threads never touch the same
    // accumulator, each commit tracks only its own thread's MMAs, and shared-memory stages are
    // consumed independently, so they need no ordering between them.
    // The loop is run by the whole warp (counters, addresses and descriptors stay warp-uniform); only the
    // tcgen05 instructions are under an elected lane.
    if (rank == 0) {
      const bool el = tc::elect_one();
      const uint32_t me = uint32_t(warp - 1);
      const uint32_t mrows = PAIR ? 256u : 128u;
      const uint32_t idesc = F8 ? tc::instr_desc(1u, 0u, mrows, uint32_t(p.bt)) : tc::instr_desc(2u, 1u, mrows, uint32_t(p.bt));
      uint32_t it = 0, ac = 0, ph = 0;  // K block, group and stage phase, counted over ALL groups
      uint32_t buf = 0, bph = 0;        // accumulator buffer of group ac and the parity of its use count
      int s = 0, gb = 0;
      bool ok = true;
      for (int tile = worker; tile < ntiles && ok; tile += nworkers) {
        for (int kb = 0; kb < nkb && ok; ++kb, ++it) {
          // Both issuers observe every phase of every stage barrier, also for the other one's K blocks:
          // a waiter that skipped a phase could mistake an older, still incomplete phase of the same
          // parity for the one it wants.  (Accumulator buffers never change hands: their number is even.)
          ok = tc::mbar_wait_spin(full_bar(s), ph, p.status, 13);
          if (PAIR && ok) {
            ok = tc::mbar_wait_spin(pfull_bar(s), ph, p.status, 15);
          }
          if (!ok) break;
          if ((ac & 1u) == me) {
            if (gb == 0) {  // fresh accumulator: its previous contents must have been drained
              ok = tc::mbar_wait_spin(acce_bar(buf), bph ^ 1u, p.status, 12);
              if (!ok) break;
            }
            tc::fence_after_sync();
            mark(1, it, 0);
            const uint32_t sb = base + s * stage_bytes;
            const uint32_t d_tmem = tmem_base + buf * uint32_t(p.bt);
            // a K step of 32 bytes = +2 in the descriptor's 16-byte address field
            const uint64_t da = tc::smem_desc_sw128(sb), db = tc::smem_desc_sw128(sb + kW8TileBytes);
            if (el) {
              if (PAIR) {
                tc::mma_8bit_pair<F8>(d_tmem, da, db, idesc, uint32_t(gb != 0));
                tc::mma_8bit_pair<F8>(d_tmem, da + 2, db + 2, idesc, 1u);
                tc::mma_8bit_pair<F8>(d_tmem, da + 4, db + 4, idesc, 1u);
                tc::mma_8bit_pair<F8>(d_tmem, da + 6, db + 6, idesc, 1u);
              } else if (F8) {
                tc::mma_f8(d_tmem, da, db, idesc, uint32_t(gb != 0));
                tc::mma_f8(d_tmem, da + 2, db + 2, idesc, 1u);
                tc::mma_f8(d_tmem, da + 4, db + 4, idesc, 1u);
                tc::mma_f8(d_tmem, da + 6, db + 6, idesc, 1u);
              } else {
                tc::mma_i8(d_tmem, da, db, idesc, uint32_t(gb != 0));
                tc::mma_i8(d_tmem, da + 2, db + 2, idesc, 1u);
                tc::mma_i8(d_tmem, da + 4, db + 4, idesc, 1u);
                tc::mma_i8(d_tmem, da + 6, db + 6, idesc, 1u);
              }
              if (PAIR) {
                tc::mma_commit_pair(empty_bar(s), 3);
                if (gb + 1 == p.blocks_per_group) tc::mma_commit_pair(accf_bar(buf), 3);
              } else {
                tc::mma_commit(empty_bar(s));
                if (gb + 1 == p.blocks_per_group) tc::mma_commit(accf_bar(buf));
              }
            }
          }
          if (++s == nst) { s = 0; ph ^= 1u; }
          if (++gb == p.blocks_per_group) {
            gb = 0;
            ++ac;
            if (++buf == uint32_t(p.nbuf)) { buf = 0; bph ^= 1u; }
          }
        }
      }
    }
  } else if (warp == 3) {
    // PAIR, CTA 1: relay.  Waits for each stage of this CTA to land and tells CTA 0's issuers.
    if (PAIR && rank == 1 && lane == 0) {
      const uint32_t pfull0 = tc::mapa(pfull_bar(0), 0);
      uint32_t ph = 0;
      int s = 0;
      bool ok = true;
      for (int tile = worker; tile < ntiles && ok; tile += nworkers) {
        for (int kb = 0; kb < nkb; ++kb) {
          if (!tc::mbar_wait(full_bar(s), ph, p.status, 16)) { ok = false; break; }
          tc::mbar_arrive_cluster_relaxed(pfull0 + 8u * s);
          if (++s == nst) { s = 0; ph ^= 1u; }
        }
      }
    }
  } else if (warp >= 4) {
    const int qd = warp & 3;           // TMEM lane quadrant this warp may read
    const int cg = (warp - 4) >> 2;    // column group 0..2
    const int wcols = p.bt / CG;       // columns this warp drains (multiple of 16, at most 16 * NCH)
    const int nch = wcols >> 4;        // 16-column chunks: 1..NCH
    uint32_t ac = 0, buf = 0, aph = 0;
    bool ok = true;
    for (int tile = worker; tile < ntiles && ok; tile += nworkers) {
      const int ft = PAIR ? 2 * (tile % n_ft) + int(rank) : tile % n_ft, tt = tile / n_ft;
      const int f = ft * 128 + qd * 32 + lane;
      const __half* swrow = p.sw + size_t(f) * p.groups;
      float2 accf[8 * NCH];  // running fp32 sums, two columns per register pair (packed fp32 FMA)
#pragma unroll
      for (int i = 0; i < 8 * NCH; ++i) accf[i] = make_float2(0.f, 0.f);
      const int tok0 = tt * p.bt + cg * wcols;
      __half s_next = __ldg(swrow);
      for (int gi = 0; gi < p.groups && ok; ++gi, ++ac) {
        const float s = __half2float(s_next) * (F8 ? 1.0f : 1.0f / 256.0f);  // int8 operands hold 16x the codes
        if (gi + 1 < p.groups) s_next = __ldg(swrow + gi + 1);
        if (!tc::mbar_wait(accf_bar(buf), aph, p.status, 14)) { ok = false; break; }
        tc::fence_after_sync();
        if (threadIdx.x == 128) mark(2, ac, 0);
        const uint32_t taddr = tmem_base + (uint32_t(qd * 32) << 16) + buf * uint32_t(p.bt) + uint32_t(cg * wcols);
        uint32_t r[2][16];
        tc::tmem_ld_32x16(taddr, r[0]);
#pragma unroll
        for (int ch = 0; ch < NCH; ++ch) {
          if (ch < nch) {
            tc::tmem_ld_wait();
            if (ch + 1 < nch) {
              tc::tmem_ld_32x16(taddr + (ch + 1) * 16, r[(ch + 1) & 1]);
            } else {  // buffer fully read: hand it back before the math
              // PAIR: one arrival per warp (an arrival from the peer CTA is a remote shared-memory operation)
              tc::fence_before_sync();
              if (PAIR) {
                __syncwarp();
                if (lane == 0) {
                  if (rank != 0) {
                    tc::mbar_arrive_cluster_relaxed(tc::mapa(acce_bar(buf), 0));
                  } else {
                    tc::mbar_arrive(acce_bar(buf));
                  }
                }
              } else {
                tc::mbar_arrive(acce_bar(buf));
              }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const uint32_t u0 = r[ch & 1][2 * j], u1 = r[ch & 1][2 * j + 1];
              const float2 g2 = F8 ? make_float2(__uint_as_float(u0), __uint_as_float(u1))
                                   : make_float2(__int2float_rn(int(u0)), __int2float_rn(int(u1)));
              // one fma.rn.f32x2 for two outputs: same bits as two scalar FMAs, half the issue slots
              accf[ch * 8 + j] = __ffma2_rn(g2, make_float2(s, s), accf[ch * 8 + j]);
              if (DUMP) {
                const int tok = tok0 + ch * 16 + 2 * j;
                const int v0 = F8 ? __float2int_rn(g2.x) : int(u0) >> 8, v1 = F8 ? __float2int_rn(g2.y) : int(u1) >> 8;
                if (tok < p.M) p.acc_dump[(size_t(tok) * p.N + f) * p.groups + gi] = v0;
                if (tok + 1 < p.M) p.acc_dump[(size_t(tok + 1) * p.N + f) * p.groups + gi] = v1;
              }
            }
          }
        }
        if (threadIdx.x == 128) mark(2, ac, 1);
        if (++buf == uint32_t(p.nbuf)) { buf = 0; aph ^= 1u; }
      }
      if (!ok) break;
      const float bias = p.bias ? __half2float(__ldg(p.bias + f)) : 0.f;
#pragma unroll
      for (int ch = 0; ch < NCH; ++ch) {
        if (ch < nch) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int tok = tok0 + ch * 16 + j;
            const float a = (j & 1) ? accf[ch * 8 + (j >> 1)].y : accf[ch * 8 + (j >> 1)].x;
            if (tok < p.M) p.y[size_t(tok) * p.N + f] = float_to_out16(a * __ldg(p.sa + tok) + bias, p.bf16);
          }
        }
      }
    }
  }

  __syncwarp();
  tc::fence_before_sync();
  __syncthreads();
  if (PAIR) tc::cluster_sync();  // neither CTA leaves while the other may still signal its barriers or read its memory
  if (warp == 1) {
    tc::fence_after_sync();
    if (PAIR) {
      tc::tmem_dealloc_pair(tmem_base, 512);
    } else {
      tc::tmem_dealloc(tmem_base, 512);
    }
  }
}

template <bool DUMP, bool F8, int CG, int NCH>
__global__ void __launch_bounds__(w4a4_threads(CG), 1)
w4a4_tc_kernel(const __grid_constant__ CUtensorMap tmw, const __grid_constant__ CUtensorMap tma,
               const W4A4TcParams p) {
  w4a4_tc_body<DUMP, F8, CG, NCH, false>(&tmw, &tma, p);
}
template <bool DUMP, bool F8, int CG, int NCH>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(w4a4_threads(CG), 1)
w4a4_tc_pair_kernel(const __grid_constant__ CUtensorMap tmw, const __grid_constant__ CUtensorMap tma,
                    const W4A4TcParams p) {
  w4a4_tc_body<DUMP, F8, CG, NCH, true>(&tmw, &tma, p);
}

// Token-tile width.  Two drain geometries: three column groups (BT a multiple of 48, up to 192, up to
// four 16-column chunks per warp) or four (BT a multiple of 64, up to 128, two chunks per warp, 16 drain
// warps).  The accumulator buffers fill tensor memory: min(4, 512 / BT) of them.
struct W4A4Tile {
  int bt, cg;
};
// `N` and `sm_count` are halved by the caller for the CTA-pair kernel (feature-tile pairs over CTA pairs).
static W4A4Tile w4a4_pick_tile(int64_t M, int64_t N, int sm_count) {
  const int bt_env = option(kOptW4a4Bt);  // tuning knob
  if (bt_env > 0 && bt_env <= 192 && (bt_env % 48 == 0 || bt_env % 64 == 0))
    return {bt_env, bt_env % 48 == 0 ? 3 : 4};
  W4A4Tile best = {48, 3};
  double best_cost = 1e30;
  const int64_t nft = N / 128;
  for (int bt = 48; bt <= 192; bt += 48) {
    const int64_t tiles = nft * ((M + bt - 1) / bt);
    const int64_t rounds = (tiles + sm_count - 1) / sm_count;
    const double cost = double(rounds) * (bt + 16);
    if (cost <= best_cost) {
      best_cost = cost;
      best = {bt, 3};
    }
  }
  return best;
}

bool w4a4_gemm_tc_supports(int64_t M, int64_t N, int64_t K, int group_size) {
  return M >= 64 && N % 128 == 0 && K % 128 == 0 && group_size > 0 && group_size % 128 == 0 && K % group_size == 0 &&
         group_size <= 4096;
}

size_t w4a4_tc_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  return 1024 + size_t(N) * K + ((size_t(M) * K + 255) & ~size_t(255)) + size_t(M) * sizeof(float) + 256;
}

// fmt: 1 = int8 holding 16x the code, 2 = e4m3 holding the code
int expand_int4(const uint8_t* src, uint8_t* dst, size_t n_elems, int fmt, int sm_count, cudaStream_t stream) {
  const size_t nvec = n_elems / 32;
  const int blocks = int(std::max<size_t>(1, std::min<size_t>(size_t(sm_count) * 8, (nvec + 255) / 256)));
  if (fmt == 2)
    expand_int4_f8_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const uint4*>(src), reinterpret_cast<uint4*>(dst), nvec);
  else
    expand_int4_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const uint4*>(src), reinterpret_cast<uint4*>(dst), nvec);
  ASRQ_CUDA_TRY(cudaGetLastError());
  return ASRQ_OK;
}

// GEMM proper on 8-bit operands already in global memory (fmt as in expand_int4).
int w4a4_gemm_int8(const uint8_t* w8, const uint8_t* a8, const float* sa, const void* sw, const void* bias,
                   void* y, int32_t* acc_dump, int64_t M, int64_t N, int64_t K, int group_size, int dtype, int fmt,
                   void* workspace, size_t workspace_bytes, int sm_count, cudaStream_t stream) {
  W4A4TcParams p;
  p.sa = sa;
  p.sw = static_cast<const __half*>(sw);
  p.bias = static_cast<const __half*>(bias);
  p.y = static_cast<uint16_t*>(y);
  p.acc_dump = acc_dump;
  p.status = static_cast<unsigned*>(workspace);
  // diagnostic timeline (3 roles x 512 events x 2 clocks), only on request and only if the workspace has room
  p.trace = nullptr;
  p.trace_block = 0;
#ifdef ASRQ_TRACE
  if (option(kOptTrace) && workspace_bytes >= (1u << 20) + 3 * 512 * 2 * 8)
    p.trace = reinterpret_cast<long long*>(static_cast<char*>(workspace) + (1u << 20));
  p.trace_block = option(kOptTraceBlock);
#endif
  p.M = int(M);
  p.N = int(N);
  p.K = int(K);
  p.groups = int(K / group_size);
  p.blocks_per_group = group_size / 128;
  // CTA pairs (tcgen05 cta_group::2) halve the activation bytes an SM takes in per MMA; they need an even
  // number of feature tiles.  Option "w4a4_pair" = 0 / 1 forces the choice (tuning knob).
  const int pair_env = option(kOptW4a4Pair);
  const bool pair = (N / 128) % 2 == 0 && sm_count >= 2 && pair_env != 0 && (pair_env == 1 || kW4A4PairDefault);
  const W4A4Tile tile = pair ? w4a4_pick_tile(M, N / 2, sm_count / 2) : w4a4_pick_tile(M, N, sm_count);
  p.bt = tile.bt;
  p.nbuf = 512 / p.bt >= 4 ? 4 : 2;  // even, so that a buffer always belongs to the same issuer
  p.n_ftiles = int(N / 128);
  p.n_ttiles = int((M + p.bt - 1) / p.bt);
  p.bf16 = dtype == ASRQ_BF16;
  const size_t stage_bytes = kW8TileBytes + size_t(pair ? p.bt / 2 : p.bt) * 128;
  const size_t budget = 227 * 1024 - 1024 - 512;
  p.nstages = int(std::min<size_t>(kW4A4MaxStages, budget / stage_bytes));
  const size_t smem = 1024 + p.nstages * stage_bytes;

  CUtensorMap tmw, tma;
  int rc = make_tmap_2d(&tmw, w8, 1, false, uint64_t(K), uint64_t(N), 128, 128, true);
  if (rc) return rc;
  rc = make_tmap_2d(&tma, a8, 1, false, uint64_t(K), uint64_t(M), 128, uint32_t(pair ? p.bt / 2 : p.bt), true);
  if (rc) return rc;
  const int grid = pair ? 2 * int(std::min<int64_t>(int64_t(p.n_ftiles / 2) * p.n_ttiles, sm_count / 2))
                        : int(std::min<int64_t>(int64_t(p.n_ftiles) * p.n_ttiles, sm_count));
  void (*kern)(const CUtensorMap, const CUtensorMap, const W4A4TcParams);
  if (pair) {
    if (tile.cg == 3)
      kern = fmt == 2 ? (acc_dump ? w4a4_tc_pair_kernel<true, true, 3, 4> : w4a4_tc_pair_kernel<false, true, 3, 4>)
                      : (acc_dump ? w4a4_tc_pair_kernel<true, false, 3, 4> : w4a4_tc_pair_kernel<false, false, 3, 4>);
    else
      kern = fmt == 2 ? (acc_dump ? w4a4_tc_pair_kernel<true, true, 4, 2> : w4a4_tc_pair_kernel<false, true, 4, 2>)
                      : (acc_dump ? w4a4_tc_pair_kernel<true, false, 4, 2> : w4a4_tc_pair_kernel<false, false, 4, 2>);
  } else if (tile.cg == 3)
    kern = fmt == 2 ? (acc_dump ? w4a4_tc_kernel<true, true, 3, 4> : w4a4_tc_kernel<false, true, 3, 4>)
                    : (acc_dump ? w4a4_tc_kernel<true, false, 3, 4> : w4a4_tc_kernel<false, false, 3, 4>);
  else
    kern = fmt == 2 ? (acc_dump ? w4a4_tc_kernel<true, true, 4, 2> : w4a4_tc_kernel<false, true, 4, 2>)
                    : (acc_dump ? w4a4_tc_kernel<true, false, 4, 2> : w4a4_tc_kernel<false, false, 4, 2>);
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem)) return rc;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(w4a4_threads(tile.cg));
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = option(kOptNoPdl) ? 0 : 1;
  ASRQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, tmw, tma, p));
  return ASRQ_OK;
}

// workspace: [0,1024) status | W8 (N*K) | A8 (M*K) | sA (M floats, fused entry only)
int w4a4_gemm_tc(const uint8_t* qa, const float* sa, const uint8_t* qw, const void* sw, const void* bias, void* y,
                 int32_t* acc_dump, int64_t M, int64_t N, int64_t K, int group_size, int dtype, void* workspace,
                 size_t workspace_bytes, int sm_count, cudaStream_t stream) {
  if (workspace_bytes < w4a4_tc_workspace_bytes(M, N, K))
    return fail(ASRQ_ERR_WORKSPACE, "w4a4 gemm: workspace %zu < %zu bytes", workspace_bytes,
                w4a4_tc_workspace_bytes(M, N, K));
  if (M > (1ll << 30) || N > (1ll << 30) || K > (1ll << 24)) return fail(ASRQ_ERR_LIMIT, "w4a4 gemm: size");
  uint8_t* w8 = static_cast<uint8_t*>(workspace) + 1024;
  uint8_t* a8 = w8 + size_t(N) * K;
  int rc = expand_int4(qw, w8, size_t(N) * K, 1, sm_count, stream);
  if (rc) return rc;
  if ((rc = expand_int4(qa, a8, size_t(M) * K, 1, sm_count, stream))) return rc;
  return w4a4_gemm_int8(w8, a8, sa, sw, bias, y, acc_dump, M, N, K, group_size, dtype, 1, workspace, kStatusBytes, sm_count, stream);
}

int hadamard_quant_int4(const void* x, uint8_t* qa, float* sa, int64_t M, int64_t K, int hadamard, int dtype,
                        int out_int8, cudaStream_t stream);

// LinearQQ.forward in one call: the prologue writes int8 activations straight into the workspace.
int w4a4_linear_tc(const void* x, const uint8_t* qw, const void* sw, const void* bias, void* y, int64_t M, int64_t N,
                   int64_t K, int group_size, int hadamard, int dtype, void* workspace, size_t workspace_bytes,
                   int sm_count, cudaStream_t stream) {
  if (workspace_bytes < w4a4_tc_workspace_bytes(M, N, K))
    return fail(ASRQ_ERR_WORKSPACE, "w4a4 linear: workspace %zu < %zu bytes", workspace_bytes,
                w4a4_tc_workspace_bytes(M, N, K));
  if (M > (1ll << 30) || N > (1ll << 30) || K > (1ll << 24)) return fail(ASRQ_ERR_LIMIT, "w4a4 linear: size");
  uint8_t* w8 = static_cast<uint8_t*>(workspace) + 1024;
  uint8_t* a8 = w8 + size_t(N) * K;
  float* sa = reinterpret_cast<float*>(a8 + ((size_t(M) * K + 255) & ~size_t(255)));
  int rc = hadamard_quant_int4(x, a8, sa, M, K, hadamard, dtype, 1, stream);
  if (rc) return rc;
  if ((rc = expand_int4(qw, w8, size_t(N) * K, 1, sm_count, stream))) return rc;
  return w4a4_gemm_int8(w8, a8, sa, sw, bias, y, nullptr, M, N, K, group_size, dtype, 1, workspace, kStatusBytes, sm_count, stream);
}

}  // namespace asrq
