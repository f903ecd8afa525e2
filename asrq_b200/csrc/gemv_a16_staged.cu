// Decode path, staged variant: y[M,N] = x[M,K] . dequant(W)[N,K]^T (+ bias) for M <= 32 per launch.
//
// A chain of decode layers is bound by what sits between two dependent launches, not by bytes: a 1-7 MB
// layer is ~1 us of HBM time, and a kernel that issues its loads, waits one DRAM round trip, computes and
// exits has no steady state.  This variant takes the weight stream off that critical path:
//
//   * one block per SM owns a contiguous strip of 16-row tiles (all of K).  Packed rows, scales and
//     zeros of the strip are contiguous in global memory; they are brought into shared memory with
//     plain bulk copies (cp.async.bulk, this GPU's memory, no multicast) on one mbarrier, each row at
//     a pitch of row bytes + 64 / (groups per step), which makes the fragment loads of a warp (128-, 64-
//     or 32-bit per lane, rows g and g+8) fall on distinct banks in every phase;
//   * the copies are issued BEFORE griddepcontrol.wait, and the block triggers its dependents as its
//     first instruction.  Blocks are sized (<= half the registers and shared memory of an SM) so that
//     the next launches of the stream become resident while this one computes: their weights stream
//     in under this launch's arithmetic, and when they pass their wait the operands are in shared
//     memory already;
//   * after the wait only the activations are fetched: one bulk copy per token brings the block's whole
//     activation matrix (or, when it is larger than its share of shared memory, one K chunk of it at a
//     time) into shared memory, so a warp pays ONE L2 round trip instead of one per quantisation group
//     (measured: with fragment loads straight from L2, a warp's chain of 8 groups took 3.4 us of a
//     4.9 us launch); the arithmetic is the masked-field
//     mma.sync scheme of gemv_a16.cu (a packed field left in the low mantissa bits of an fp16 number is
//     the code times a power of two; scale and zero applied once per group in fp32).
//
// Measured on B200 (CUDA-graph chains of 40 launches over distinct weights, W4 g64 2048 -> 6144, one token):
// 4.4 us per launch against 4.1 us for the strip-per-block kernel of gemv_a16.cu, and no faster with the
// weights resident in L2 -- neither kernel is bound by bytes.  Timeline of a launch in the chain: the wait
// is released 0.5 us after the last block of the launch before exits, the operands are in shared memory
// by then (0.2 us), the activations arrive 0.6 us later, the arithmetic takes 2.4 us (the legacy mma.sync
// pipe issues one m16n8k16 per ~13 clocks per scheduler; 16 of them per kilobyte of 4-bit weights with the
// activation sums), reduction and stores 0.6 us.  The strip-per-block kernel therefore stays the default;
// this variant runs on request (option "gemv_kernel" = 3).
//
// Work split inside a block: unit = (tile, token group of 8*MH); the block's warps are divided among
// the units and split K between them; partial tiles are added through shared memory in a fixed order.
// Up to 32 tokens per launch (two token groups of 16), so a decode batch of 32 reads the weights once.
#include <algorithm>

#include "tcgen05.cuh"

namespace asrq {

namespace {

// warps per block: twelve at 80 registers for up to 8 tokens, eight at 128 registers for 16-token units
// (two blocks of either shape share an SM)
__host__ __device__ constexpr int st_warps(int mh) { return mh == 1 ? 12 : 8; }
constexpr int kStHeader = 128;                 // mbarrier + padding in front of the staged rows
constexpr size_t kStSmemBudget = 100 * 1024;   // strip + tables + partial sums of a block
constexpr size_t kStSmemPair = 113 * 1024;     // a block this small shares its SM with the next launch's block
constexpr size_t kStSmemSolo = 200 * 1024;     // above that a block has the SM to itself

struct StagedParams {
  const uint16_t* x;
  const uint8_t* w;
  const __half* scales;
  const __half* zeros;
  const __half* bias;
  uint16_t* y;
  unsigned* status;
  int M, N, K, groups_per_row, bf16;
  int tiles_total;   // N / 16
  int tab_offset;    // byte offset of the staged scales inside shared memory (zeros follow at tab_offset + tab_max)
  int tab_max;       // bytes reserved for each of the two tables
  int red_offset;    // byte offset of the partial-sum area
  int x_offset;      // XS: byte offset of the staged activations
  int x_pitch;       // XS: bytes per staged token row (chunk bytes + 16: eight tokens fall on distinct banks)
  int kchunk;        // XS: k per staged chunk (a multiple of the step; K when the whole matrix fits)
  unsigned long long* trace;  // builds with -DASRQ_TRACE: 8 globaltimer marks per block, NULL otherwise
};

#ifdef ASRQ_TRACE
#define ST_MARK(i)                                                                       \
  do {                                                                                   \
    if (p.trace && threadIdx.x == 0) {                                                   \
      unsigned long long t__;                                                            \
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t__)::"memory");                  \
      p.trace[size_t(blockIdx.x) * 8 + (i)] = t__;                                       \
    }                                                                                    \
  } while (0)
#else
#define ST_MARK(i) do { } while (0)
#endif

__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

__device__ __forceinline__ void st_mma_acc(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                           uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void st_mma_new(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                           uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}

__device__ __forceinline__ uint32_t st_bf16x2_to_f16x2_sat(uint32_t v) {
  float lo = __uint_as_float(v << 16);
  float hi = __uint_as_float(v & 0xffff0000u);
  lo = fminf(fmaxf(lo, -65504.f), 65504.f);
  hi = fminf(fmaxf(hi, -65504.f), 65504.f);
  return h2_as_u32(__floats2half2_rn(lo, hi));
}

// BITS: 4 or 2.  MH: token halves per unit (1: 8 tokens, 2: 16 tokens).  GPS: quantisation groups per
// step of 64 bytes per row (1, 2 or 4: group size 128 / 64 / 32 for 4-bit, 256 / 128 / 64 for 2-bit).
// XS: activations staged in shared memory (else fragment loads go to L2 directly).
template <int BITS, int MH, int GPS, bool XS>
__global__ void __launch_bounds__(32 * st_warps(MH), 2) gemv_a16_staged_kernel(const StagedParams p) {
  constexpr int kStWarps = st_warps(MH);
  constexpr int kStThreads = 32 * kStWarps;
  constexpr int CPWORD = 32 / BITS;   // codes per 32-bit word (8 / 16)
  constexpr int STEPK = 16 * CPWORD;  // k per step (128 / 256)
  constexpr int NT = 8 / BITS;        // field positions inside a byte = accumulator types (2 / 4)
  constexpr int WPC = 4 / GPS;        // consecutive words a lane owns per group
  constexpr int G = STEPK / GPS;      // group size
  constexpr int XR = CPWORD / 2;      // 32-bit activation registers per word (4 / 8)
  constexpr int FR = 4 * MH;          // output registers per lane
  constexpr uint32_t FIELD = (1u << BITS) - 1u;
  constexpr uint32_t MASK0 = FIELD | (FIELD << 16);
  constexpr uint32_t ONES = 0x3c003c00u;  // (1.0, 1.0)

  extern __shared__ __align__(128) uint8_t smem[];
  // the next kernels on the stream may start now: they prefetch their weights while this one works
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  ST_MARK(0);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, c = lane & 3;
  // this block's strip of 16-row tiles: contiguous, sizes differ by at most one over the grid
  const int nb = gridDim.x, bq = p.tiles_total / nb, br = p.tiles_total % nb, b = blockIdx.x;
  const int tile0 = b * bq + min(b, br);
  const int T = bq + (b < br ? 1 : 0);
  const int rows = T * 16;
  const int row_bytes = p.K * BITS / 8, pitch = row_bytes + 64 / GPS;
  const int gpr = p.groups_per_row;
  uint8_t* wsm = smem + kStHeader;
  const __half* ssm = reinterpret_cast<const __half*>(smem + p.tab_offset);
  const __half* zsm = reinterpret_cast<const __half*>(smem + p.tab_offset + p.tab_max);
  float* red = reinterpret_cast<float*>(smem + p.red_offset);
  const uint32_t bar = tc::smem_u32(smem), xbar = bar + 8;
  const uint8_t* xsm = smem + p.x_offset;

  if (tid == 0) {
    tc::mbar_init(bar, 1);
    tc::mbar_init(xbar, 1);
    tc::fence_barrier_init();
    tc::fence_proxy_async_smem();
  }
  __syncthreads();
  if (warp == 0) {
    const uint32_t tab_bytes = uint32_t(rows) * gpr * 2;
    if (lane == 0) tc::mbar_arrive_expect_tx(bar, uint32_t(rows) * row_bytes + 2 * tab_bytes);
    __syncwarp();
    const uint8_t* src = p.w + size_t(tile0) * 16 * row_bytes;
    for (int rr = lane; rr < rows; rr += 32)
      bulk_g2s(tc::smem_u32(wsm + rr * pitch), src + size_t(rr) * row_bytes, uint32_t(row_bytes), bar);
    if (lane == 0) {
      bulk_g2s(tc::smem_u32(ssm), p.scales + size_t(tile0) * 16 * gpr, tab_bytes, bar);
      bulk_g2s(tc::smem_u32(zsm), p.zeros + size_t(tile0) * 16 * gpr, tab_bytes, bar);
    }
  }
  ST_MARK(1);
  // activations and output belong to this kernel only once its predecessor on the stream is complete
  asm volatile("griddepcontrol.wait;" ::: "memory");
  ST_MARK(2);

  const int TG = (p.M + 8 * MH - 1) / (8 * MH);  // token groups
  const int S = p.K / STEPK;                     // steps per row
  const int units = T * TG;
  int KQ = kStWarps / units;
  KQ = KQ < 1 ? 1 : (KQ > S ? S : KQ);
  const int nslots = units * KQ;

  // wait for the staged operands (bounded: a waiter that gives up records it and the block leaves)
  const bool staged = tc::mbar_wait(bar, 0u, p.status, 21);
  ST_MARK(3);

  // XS: the K range is walked in chunks whose activations fit the staging area (one chunk = all of K
  // when they fit); a warp keeps its slot's sums in registers across chunks (the host picks XS with
  // several chunks only when every warp has at most one slot).
  const int kchunk = XS ? p.kchunk : p.K;
  const int nchunks = p.K / kchunk;
  const int steps_per_chunk = kchunk / STEPK;
  float yv[MH][4];
  bool x_ok = true;
  for (int chunk = 0; staged && x_ok && chunk < nchunks; ++chunk) {
    if (XS) {
      if (chunk > 0) __syncthreads();  // every warp is done with the previous chunk's activations
      if (warp == 0) {
        const uint32_t row_b = uint32_t(kchunk) * 2;
        if (lane == 0) tc::mbar_arrive_expect_tx(xbar, uint32_t(p.M) * row_b);
        __syncwarp();
        for (int m = lane; m < p.M; m += 32)
          bulk_g2s(tc::smem_u32(xsm + m * p.x_pitch), p.x + size_t(m) * p.K + size_t(chunk) * kchunk, row_b, xbar);
      }
      x_ok = tc::mbar_wait(xbar, uint32_t(chunk & 1), p.status, 22);
      if (!x_ok) break;
      if (chunk == 0) ST_MARK(7);
    }
    const int cs0 = chunk * steps_per_chunk;  // first step of this chunk
  for (int slot = warp; slot < nslots; slot += kStWarps) {
    const int unit = slot / KQ, kq = slot - unit * KQ;
    const int tl = unit / TG, tg = unit - tl * TG;
    // this warp's groups of the row: its share of the chunk's steps
    const int ws0 = cs0 + kq * steps_per_chunk / KQ, ws1 = cs0 + (kq + 1) * steps_per_chunk / KQ;
    const int gfirst = ws0 * GPS, glast = ws1 * GPS;
    const int mbase = tg * 8 * MH;
    const uint8_t* w0 = wsm + (tl * 16 + g) * pitch + c * (16 / GPS);
    const uint8_t* w1 = w0 + 8 * pitch;
    const __half* s0p = ssm + (tl * 16 + g) * gpr;
    const __half* z0p = zsm + (tl * 16 + g) * gpr;
    if (chunk == 0 || nslots > kStWarps) {
#pragma unroll
      for (int mh = 0; mh < MH; ++mh)
#pragma unroll
        for (int i = 0; i < 4; ++i) yv[mh][i] = 0.f;
    }

    // activations of token mbase + g (+8) for the k of this lane's WPC words of group gi, natural order
    auto load_x = [&](int gi, uint32_t (&dst)[MH][WPC][XR]) {
      const int kbase = gi * G + c * (G / 4);
#pragma unroll
      for (int mh = 0; mh < MH; ++mh) {
        const int m = mbase + g + 8 * mh;
        const uint4* xp = XS ? reinterpret_cast<const uint4*>(xsm + m * p.x_pitch + (kbase - chunk * kchunk) * 2)
                             : reinterpret_cast<const uint4*>(p.x + size_t(m) * p.K + kbase);
#pragma unroll
        for (int v = 0; v < WPC * XR / 4; ++v) {
          uint4 u = make_uint4(0, 0, 0, 0);
          if (m < p.M) {
            u = XS ? xp[v] : __ldcg(xp + v);  // not XS: L2 (written by the kernel before this one on the stream)
            if (p.bf16) {
              u.x = st_bf16x2_to_f16x2_sat(u.x); u.y = st_bf16x2_to_f16x2_sat(u.y);
              u.z = st_bf16x2_to_f16x2_sat(u.z); u.w = st_bf16x2_to_f16x2_sat(u.w);
            }
          }
          dst[mh][(4 * v) / XR][(4 * v) % XR + 0] = u.x; dst[mh][(4 * v) / XR][(4 * v) % XR + 1] = u.y;
          dst[mh][(4 * v) / XR][(4 * v) % XR + 2] = u.z; dst[mh][(4 * v) / XR][(4 * v) % XR + 3] = u.w;
        }
      }
    };
    // one quantisation group: packed words from shared memory, fields times activations, then scale and zero
    auto do_group = [&](int gi, const uint32_t (&xr)[MH][WPC][XR]) {
      const int boff = (gi / GPS) * 64 + (gi % GPS) * (64 / GPS);  // byte offset of the group inside the row
      uint32_t qa[WPC], qb[WPC];
      if constexpr (WPC == 4) {
        const uint4 a = *reinterpret_cast<const uint4*>(w0 + boff), bb = *reinterpret_cast<const uint4*>(w1 + boff);
        qa[0] = a.x; qa[1] = a.y; qa[2] = a.z; qa[3] = a.w;
        qb[0] = bb.x; qb[1] = bb.y; qb[2] = bb.z; qb[3] = bb.w;
      } else if constexpr (WPC == 2) {
        const uint2 a = *reinterpret_cast<const uint2*>(w0 + boff), bb = *reinterpret_cast<const uint2*>(w1 + boff);
        qa[0] = a.x; qa[1] = a.y; qb[0] = bb.x; qb[1] = bb.y;
      } else {
        qa[0] = *reinterpret_cast<const uint32_t*>(w0 + boff);
        qb[0] = *reinterpret_cast<const uint32_t*>(w1 + boff);
      }
      const float sc0 = __half2float(s0p[gi]) * 16777216.f, sc1 = __half2float(s0p[8 * gpr + gi]) * 16777216.f;
      const float zr0 = __half2float(z0p[gi]), zr1 = __half2float(z0p[8 * gpr + gi]);
      float acc[MH][NT][4], accx[MH][4];
#pragma unroll
      for (int t = 0; t < WPC; ++t) {
        const uint32_t q0 = qa[t], q1 = qb[t];
        const uint32_t q0h = q0 >> 8, q1h = q1 >> 8;
#pragma unroll
        for (int ty = 0; ty < NT; ++ty) {
          const uint32_t mask = MASK0 << (BITS * ty);
          const uint32_t a0 = q0 & mask, a1 = q1 & mask, a2 = q0h & mask, a3 = q1h & mask;
#pragma unroll
          for (int mh = 0; mh < MH; ++mh) {
            // element a of the word pairs with element a + CPWORD/2: codes e_a and e_(a + CPWORD/2) share a field
            // position in the two halves of the word
            const uint32_t* xw = xr[mh][t];
            const uint32_t sel = (ty & 1) ? 0x7632u : 0x5410u;
            const uint32_t b0 = prmt(xw[ty / 2], xw[(ty + CPWORD / 2) / 2], sel);
            const uint32_t b1 = prmt(xw[(ty + NT) / 2], xw[(ty + NT + CPWORD / 2) / 2], sel);
            if (t == 0) {
              st_mma_new(acc[mh][ty], a0, a1, a2, a3, b0, b1);
            } else {
              st_mma_acc(acc[mh][ty], a0, a1, a2, a3, b0, b1);
            }
            // sums of the activations over the group: one more MMA, against ones
            if (t == 0 && ty == 0) {
              st_mma_new(accx[mh], ONES, ONES, ONES, ONES, b0, b1);
            } else {
              st_mma_acc(accx[mh], ONES, ONES, ONES, ONES, b0, b1);
            }
          }
        }
      }
      // combine the types (a field at bit BITS*ty carries 2^(BITS*ty) times its code; a code in the lowest field is
      // code * 2^-24 as an fp16 number), scale, add zero * sum(x)
#pragma unroll
      for (int mh = 0; mh < MH; ++mh) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          float tsum = acc[mh][NT - 1][r];
#pragma unroll
          for (int ty = NT - 2; ty >= 0; --ty) tsum = fmaf(tsum, 1.f / float(1 << BITS), acc[mh][ty][r]);
          yv[mh][r] = fmaf(tsum, r < 2 ? sc0 : sc1, yv[mh][r]);
          yv[mh][r] = fmaf(accx[mh][r & 1], r < 2 ? zr0 : zr1, yv[mh][r]);
        }
      }
    };

    // fragment loads from L2: where registers allow, the next group's activations are fetched while this
    // group's MMAs run (from shared memory there is nothing to hide)
    constexpr bool PF = !XS && MH * WPC * XR <= 16;
    if (gfirst >= glast) {
      // more warps than steps in this chunk: nothing to add
    } else if (PF) {
      uint32_t xa[MH][WPC][XR], xb[MH][WPC][XR];
      load_x(gfirst, xa);
      for (int gi = gfirst; gi < glast; gi += 2) {
        if (gi + 1 < glast) load_x(gi + 1, xb);
        do_group(gi, xa);
        if (gi + 1 < glast) {
          if (gi + 2 < glast) load_x(gi + 2, xa);
          do_group(gi + 1, xb);
        }
      }
    } else {
      uint32_t xa[MH][WPC][XR];
      for (int gi = gfirst; gi < glast; ++gi) {
        load_x(gi, xa);
        do_group(gi, xa);
      }
    }
    if (chunk + 1 == nchunks || nslots > kStWarps) {
#pragma unroll
      for (int mh = 0; mh < MH; ++mh)
#pragma unroll
        for (int r = 0; r < 4; ++r) red[(slot * FR + mh * 4 + r) * 32 + lane] = yv[mh][r];
    }
  }
  }  // chunks
  ST_MARK(4);
  __syncthreads();
  ST_MARK(5);
  if (!staged || !x_ok) return;

  // ---- add the KQ partial tiles of every unit in K order and write the strip ----------------------------
  // register f = mh*4 + r of lane (g, c): weight row g + 8*(r>>1) of the tile, token 8*mh + 2c + (r&1) of the group
  const int per_unit = FR * 32;
  for (int i = tid; i < units * per_unit; i += kStThreads) {
    const int unit = i / per_unit, rem = i - unit * per_unit;
    const int f = rem >> 5, ln = rem & 31;
    float v = 0.f;
    for (int q = 0; q < KQ; ++q) v += red[((unit * KQ + q) * FR + f) * 32 + ln];
    const int tl = unit / TG, tg = unit - tl * TG;
    const int n = (tile0 + tl) * 16 + (ln >> 2) + ((f >> 1) & 1) * 8;
    const int m = tg * 8 * MH + 8 * (f >> 2) + 2 * (ln & 3) + (f & 1);
    if (m < p.M) {
      if (p.bias) v += __half2float(__ldg(p.bias + n));
      p.y[size_t(m) * p.N + n] = float_to_out16(v, p.bf16);
    }
  }
  ST_MARK(6);
}

using StagedKernel = void (*)(const StagedParams);

template <int BITS, int MH>
StagedKernel staged_kernel_for(int gps, bool xs) {
  switch (gps) {
    case 1: return xs ? gemv_a16_staged_kernel<BITS, MH, 1, true> : gemv_a16_staged_kernel<BITS, MH, 1, false>;
    case 2: return xs ? gemv_a16_staged_kernel<BITS, MH, 2, true> : gemv_a16_staged_kernel<BITS, MH, 2, false>;
    case 4: return xs ? gemv_a16_staged_kernel<BITS, MH, 4, true> : gemv_a16_staged_kernel<BITS, MH, 4, false>;
    default: return nullptr;
  }
}

}  // namespace

int ensure_dynamic_smem(const void* kernel, size_t bytes);

// Whether the staged kernel takes this call; fills the launch geometry.  It needs the whole strip of a
// block (weights at their padded pitch, both tables, the partial-sum area) inside its shared-memory
// budget, 1, 2 or 4 groups per 64-byte step, and 16-byte aligned tables.
struct StagedPlan {
  int grid, tab_offset, tab_max, red_offset, x_offset, x_pitch, kchunk;
  bool xs;
  size_t smem;
};
static bool staged_plan(int bits, int64_t M, int64_t N, int64_t K, int group_size, int sm_count, StagedPlan* plan) {
  const int chunk = (128 / bits) * 4;  // k per step
  if (M < 1 || M > 32 || N % 16 || K % chunk || group_size <= 0 || chunk % group_size || K % group_size) return false;
  const int gps = chunk / group_size;
  if (gps != 1 && gps != 2 && gps != 4) return false;
  const int64_t tiles = N / 16;
  const int grid = int(std::min<int64_t>(sm_count, tiles));
  const int64_t tmax = (tiles + grid - 1) / grid;
  const int64_t row_bytes = K * bits / 8, gpr = K / group_size;
  const int mh = M <= 8 ? 1 : 2;
  const int64_t tg = (M + 8 * mh - 1) / (8 * mh);
  const int64_t units = tmax * tg, steps = K / chunk;
  const int64_t slots = std::max<int64_t>(units, st_warps(mh));  // a block with fewer tiles splits K further, up to one slot per warp
  const int64_t wbytes = tmax * 16 * (row_bytes + 64 / gps);
  const int64_t tab = (tmax * 16 * gpr * 2 + 127) & ~int64_t(127);
  const int64_t red = slots * (4 * mh) * 32 * 4;
  const int64_t base = kStHeader + wbytes + 2 * tab + red;
  if (base > int64_t(kStSmemBudget)) return false;
  plan->grid = grid;
  plan->tab_offset = int(kStHeader + wbytes);
  plan->tab_max = int(tab);
  plan->red_offset = int(kStHeader + wbytes + 2 * tab);
  // Activations in shared memory: the whole matrix if it fits beside the strip inside the two-blocks-per-SM
  // budget, else inside one block's maximum, else the largest K chunk (a divisor of K in whole steps) that
  // fits -- chunks only when every warp has a single slot, because sums stay in registers across chunks.
  plan->xs = false;
  plan->x_offset = int((base + 127) & ~int64_t(127));
  plan->x_pitch = 0;
  plan->kchunk = int(K);
  plan->smem = size_t(base);
  const int64_t pair_room = int64_t(kStSmemPair) - plan->x_offset, solo_room = int64_t(kStSmemSolo) - plan->x_offset;
  auto x_bytes = [&](int64_t kc) { return M * (kc * 2 + 16); };
  int64_t kc = 0;
  if (x_bytes(K) <= pair_room || x_bytes(K) <= solo_room) {
    kc = K;
  }
  // (The kernel can also walk K in chunks whose activations fit; every chunk then costs a block-wide barrier
  // and an L2 round trip, and 8 chunks of a 5120-wide layer at 32 tokens measured 26 us against 15 us with
  // fragment loads straight from L2, so chunking is not planned.)
  (void)steps;
  if (kc > 0 && option(kOptGemvXStage) != 0) {
    plan->xs = true;
    plan->kchunk = int(kc);
    plan->x_pitch = int(kc * 2 + 16);
    plan->smem = size_t(plan->x_offset + x_bytes(kc));
  }
  return true;
}

bool gemv_a16_staged_supports(int bits, int64_t M, int64_t N, int64_t K, int group_size, int sm_count) {
  StagedPlan plan;
  return staged_plan(bits, M, N, K, group_size, sm_count, &plan);
}

// One launch (M <= 32).  The caller has checked pointers, alignment of x / w / y and the workspace.
int gemv_a16_staged(int bits, const void* x, const uint8_t* w, const void* scales, const void* zeros, const void* bias,
                    void* y, int64_t M, int64_t N, int64_t K, int group_size, int dtype, void* workspace, int sm_count,
                    cudaStream_t stream) {
  StagedPlan plan;
  if (!staged_plan(bits, M, N, K, group_size, sm_count, &plan))
    return fail(ASRQ_ERR_SHAPE, "w%da16 gemv (staged): unsupported shape M=%lld N=%lld K=%lld g=%d", bits, (long long)M,
                (long long)N, (long long)K, group_size);
  const int gps = (128 / bits) * 4 / group_size;
  const int mh = M <= 8 ? 1 : 2;
  StagedKernel kern = bits == 4 ? (mh == 1 ? staged_kernel_for<4, 1>(gps, plan.xs) : staged_kernel_for<4, 2>(gps, plan.xs))
                                : (mh == 1 ? staged_kernel_for<2, 1>(gps, plan.xs) : staged_kernel_for<2, 2>(gps, plan.xs));
  if (!kern) return fail(ASRQ_ERR_SHAPE, "w%da16 gemv (staged): no kernel for %d groups per step", bits, gps);
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), plan.smem)) return rc;
  StagedParams p;
  p.x = static_cast<const uint16_t*>(x);
  p.w = w;
  p.scales = static_cast<const __half*>(scales);
  p.zeros = static_cast<const __half*>(zeros);
  p.bias = static_cast<const __half*>(bias);
  p.y = static_cast<uint16_t*>(y);
  p.status = static_cast<unsigned*>(workspace);
  p.M = int(M);
  p.N = int(N);
  p.K = int(K);
  p.groups_per_row = int(K / group_size);
  p.bf16 = dtype == ASRQ_BF16;
  p.tiles_total = int(N / 16);
  p.tab_offset = plan.tab_offset;
  p.tab_max = plan.tab_max;
  p.red_offset = plan.red_offset;
  p.x_offset = plan.x_offset;
  p.x_pitch = plan.x_pitch;
  p.kchunk = plan.kchunk;
  p.trace = nullptr;
#ifdef ASRQ_TRACE
  if (option(kOptTrace)) {  // marks of launch number trace_block (counted from the option's last change) go to the workspace
    static int launch_no = 0;
    static unsigned gen = 0;
    if (gen != options_generation()) { gen = options_generation(); launch_no = 0; }
    p.trace = reinterpret_cast<unsigned long long*>(static_cast<char*>(workspace) + kPartialOffset) + size_t(launch_no % 64) * 148 * 8;
    ++launch_no;
  }
#endif
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(plan.grid);
  cfg.blockDim = dim3(32 * st_warps(mh));
  cfg.dynamicSmemBytes = plan.smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = option(kOptNoPdl) ? 0 : 1;
  ASRQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, p));
  return ASRQ_OK;
}

}  // namespace asrq
