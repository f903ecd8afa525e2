// Decode path: y[M,N] = x[M,K] . dequant(W)[N,K]^T for M <= 16 per launch.
//
// HBM-bound skinny GEMM whose second limit is the instruction issue rate (at 6.5 TB/s an SM
// receives a kilobyte of packed weights every ~44 clocks), so the weights are never turned into
// scaled fp16 values one by one.  A packed word is only masked (one LOP3 per two codes): a 4-bit
// or 2-bit field left in the low mantissa bits of an fp16 number is that code times a power of
// two (a subnormal), which mma.sync.m16n8k16 multiplies exactly with the fp16 activations and
// accumulates in fp32.  Fields at different bit positions ("types") go to different accumulators
// and are combined, scaled by the group's scale and offset by zero * sum(x) once per quantisation
// group in fp32; sum(x) over the group comes from one more MMA against a matrix of ones.
//
// Work split: a warp owns a strip of 16 weight rows (rows g and g+8 per lane, g = lane/4) over one
// to four "steps" (a step = 64 bytes of a row per lane quad = 128 k for 4-bit, 256 k for 2-bit),
// loaded with all its 128-bit (or, for small groups, narrower) loads in flight at once before the
// kernel waits for its predecessor on the stream.  The KQ <= 16 warps of a block share the row
// strip and split K; their partial tiles are added through shared memory in a fixed order, so the
// result never depends on scheduling and no workspace is touched.  Shapes outside this kernel's
// menu (group sizes other than 1, 1/2 or 1/4 step, very long K, unaligned scale tables) go to the
// split-K kernel in gemv_a16_splitk.cu.
#include <algorithm>
#include <cstdlib>
#include <mutex>
#include <vector>

#include "common.cuh"

namespace asrq {

int gemv_a16_splitk(int bits, const void* x, const uint8_t* w, const void* scales, const void* zeros,
                    const void* bias, void* y, int64_t M, int64_t N, int64_t K, int group_size, int dtype,
                    void* workspace, size_t workspace_bytes, int sm_count, cudaStream_t stream, int max_split);
size_t gemv_workspace_bytes(int64_t N, int max_split);
bool gemv_a16_staged_supports(int bits, int64_t M, int64_t N, int64_t K, int group_size, int sm_count);
int gemv_a16_staged(int bits, const void* x, const uint8_t* w, const void* scales, const void* zeros, const void* bias,
                    void* y, int64_t M, int64_t N, int64_t K, int group_size, int dtype, void* workspace, int sm_count,
                    cudaStream_t stream);

namespace {

struct GemvParams {
  const uint16_t* x;
  const uint8_t* w;
  const __half* scales;
  const __half* zeros;
  const __half* bias;
  uint16_t* y;
  int M, N, K, groups_per_row, KQ, CPW, bf16;  // CPW repeats the kernel's template argument
  int R;                                       // rounds (LOOP variants): a warp takes R runs of CPW steps, KQ * CPW steps apart
  unsigned long long* trace;  // builds with -DASRQ_TRACE: per-warp clock marks (8 words per warp), NULL otherwise
};

constexpr int kGemvMaxWarps = 16;
constexpr int kGemvMaxSteps = 4;

// d = a * b (+ c): m16n8k16, fp16 operands, fp32 accumulation
__device__ __forceinline__ void mma_acc(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_new(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%10,%10,%10,%10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}

__device__ __forceinline__ uint32_t bf16x2_to_f16x2_sat(uint32_t v) {
  float lo = __uint_as_float(v << 16);
  float hi = __uint_as_float(v & 0xffff0000u);
  lo = fminf(fmaxf(lo, -65504.f), 65504.f);
  hi = fminf(fmaxf(hi, -65504.f), 65504.f);
  return h2_as_u32(__floats2half2_rn(lo, hi));
}

// streaming loads of W words (never re-read by this kernel: keep them out of L1)
template <int WORDS>
__device__ __forceinline__ void ldg_stream_words(const uint8_t* p, uint32_t* out) {
  if (WORDS == 4) {
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(out[0]), "=r"(out[1]), "=r"(out[2]), "=r"(out[3])
                 : "l"(p));
  } else if (WORDS == 2) {
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(out[0]), "=r"(out[1]) : "l"(p));
  } else {
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(out[0]) : "l"(p));
  }
}

// NG consecutive halves (NG in {1,2,4,8}) of one row of the scale or zero table into packed pairs
template <int NG>
__device__ __forceinline__ void load_group_table(const __half* p, uint32_t (&out)[4]) {
  if (NG == 1) {
    out[0] = __ldg(reinterpret_cast<const unsigned short*>(p));
  } else if (NG == 2) {
    out[0] = __ldg(reinterpret_cast<const unsigned*>(p));
  } else if (NG == 4) {
    const uint2 v = __ldg(reinterpret_cast<const uint2*>(p));
    out[0] = v.x; out[1] = v.y;
  } else {
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(p));
    out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
  }
}
__device__ __forceinline__ float table_entry(const uint32_t (&t)[4], int idx) {  // idx is a compile-time value
  const uint32_t w = t[idx >> 1];
  return __half2float(__ushort_as_half((unsigned short)((idx & 1) ? (w >> 16) : (w & 0xffffu))));
}

__device__ __forceinline__ unsigned long long gemv_clock() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%clock64;" : "=l"(t)::"memory");
  return t;
}
__device__ __forceinline__ unsigned long long gemv_clock_after(uint32_t dep) {  // waits for dep to be loaded
  unsigned long long t;
  asm volatile("mov.u64 %0, %%clock64;" : "=l"(t) : "r"(dep) : "memory");
  return t;
}
__device__ __forceinline__ unsigned long long gemv_globaltimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)::"memory");
  return t;
}

// BITS: 4 or 2.  MH: token halves (1: M <= 8, 2: M <= 16).  GPS: quantisation groups per step
// (1, 2 or 4; the group size is 128/GPS k for 4-bit and 256/GPS k for 2-bit).  CPW: steps per warp
// (1, 2 or 4, CPW * GPS <= 8).  XC: M <= 2, the activation sums are made on the CUDA cores instead of
// by an MMA against ones (the legacy MMA pipe is this kernel's second bottleneck).
// LOOP: layers too large for one resident wave.  Blocks are small (a few warps), several share an SM
// at different points of their lives, and a warp walks K in R rounds, so that loads of one block
// are in flight while another computes.  (Measured on 32-128 MB layers at M=1: 2.7-3.4 TB/s against
// 2.0-2.5 for one round per warp.  Requesting the next round's words before this round's arithmetic,
// in registers or through a cp.async ring in shared memory, measured slower: the variant is bound by
// per-warp latency with 12-16 warps per SM at 128 registers, not by bytes in flight.)
template <int BITS, int MH, int GPS, int CPW, bool XC, bool TRACE, bool LOOP = false>
__global__ void __launch_bounds__(kGemvMaxWarps * 32, (CPW == 1 && MH == 1 && BITS == 4 && !LOOP) ? 3 : 1)
gemv_a16_kernel(const GemvParams p) {
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

  __shared__ float red[kGemvMaxWarps * FR * 32];
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;  // warp = K part inside the block
  const int g = lane >> 2, c = lane & 3;
  const int n_base = blockIdx.x * 16;
  const int r0 = n_base + g;
  unsigned long long* tr = nullptr;
  if (TRACE) {
    tr = p.trace + (size_t(blockIdx.x) * kGemvMaxWarps + warp) * 8;
    if (lane == 0) {
      tr[0] = gemv_globaltimer();
      tr[1] = gemv_clock();
    }
  }
  constexpr int NG = CPW * GPS;       // groups per warp
  const size_t row_bytes = size_t(p.K) * BITS / 8;
  float yv[MH][4];
#pragma unroll
  for (int mh = 0; mh < MH; ++mh)
#pragma unroll
    for (int i = 0; i < 4; ++i) yv[mh][i] = 0.f;
  // Let the next kernel on the stream start, and start streaming weights before this kernel's
  // own predecessor has finished: weights, scales and zeros are constants; only the activations
  // and the output depend on earlier kernels.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int rounds = LOOP ? p.R : 1;
  // word (j, t) of step i sits at byte i*64 + j*(64/GPS) + c*(16/GPS) + 4*t of the warp's row span
  auto row_ptr = [&](int step0) { return p.w + size_t(r0) * row_bytes + size_t(step0) * 64 + c * (16 / GPS); };
  // scale and zero of the warp's NG = CPW * GPS groups of a round, rows g and g+8
  auto load_tables = [&](int step0, uint32_t (&s0)[4], uint32_t (&z0)[4], uint32_t (&s1)[4], uint32_t (&z1)[4]) {
    const size_t o0 = size_t(r0) * p.groups_per_row + size_t(step0) * GPS;
    const size_t o1 = o0 + size_t(8) * p.groups_per_row;
    load_group_table<NG>(p.scales + o0, s0);
    load_group_table<NG>(p.zeros + o0, z0);
    load_group_table<NG>(p.scales + o1, s1);
    load_group_table<NG>(p.zeros + o1, z1);
  };
  uint32_t qa[CPW][4], qb[CPW][4], ts0[4], tz0[4], ts1[4], tz1[4];
#pragma unroll 1
  for (int rd = 0; rd < rounds; ++rd) {
  const int step0 = (rd * p.KQ + warp) * CPW;
  {
    const uint8_t* w0 = row_ptr(step0);
    const uint8_t* w1 = w0 + 8 * row_bytes;
#pragma unroll
    for (int i = 0; i < CPW; ++i) {
#pragma unroll
      for (int j = 0; j < GPS; ++j) {
        ldg_stream_words<WPC>(w0 + i * 64 + j * (64 / GPS), &qa[i][j * WPC]);
        ldg_stream_words<WPC>(w1 + i * 64 + j * (64 / GPS), &qb[i][j * WPC]);
      }
    }
    load_tables(step0, ts0, tz0, ts1, tz1);
  }
  if (rd == 0) asm volatile("griddepcontrol.wait;" ::: "memory");
  if (TRACE && lane == 0) tr[2] = gemv_clock();

  // XC: sum of x over each of the warp's groups for tokens 0 and 1, the same in every lane.  The
  // warp's k span is cut into 32 runs, one per lane; a group is 32/NG consecutive lanes.  The loads
  // go out here, next to the first group's activation loads; the sums are made when first needed.
  constexpr int HPL = CPW * STEPK / 32;  // halves per lane: 4, 8, 16, 32 or 64
  constexpr int LPG = 32 / NG;           // lanes per group
  float xs[2][NG];
  uint2 xu[2][HPL / 4];
  if (XC) {
#pragma unroll
    for (int tok = 0; tok < 2; ++tok) {
      const uint16_t* xp = p.x + size_t(tok) * p.K + step0 * STEPK + lane * HPL;
#pragma unroll
      for (int v = 0; v < HPL / 4; ++v)
        xu[tok][v] = tok < p.M ? __ldg(reinterpret_cast<const uint2*>(xp) + v) : make_uint2(0, 0);
    }
  }

  // activations of token g (+8) for the k of this lane's WPC words of group gi, natural order;
  // where registers allow, the next group's are fetched while this group's MMAs run
  constexpr bool PF = MH * WPC * XR <= 16;
  uint32_t xbuf[PF ? 2 : 1][MH][WPC][XR];
  auto load_x = [&](int gi, uint32_t (&dst)[MH][WPC][XR]) {
    const int kbase = (step0 + gi / GPS) * STEPK + (gi % GPS) * G + c * (G / 4);
#pragma unroll
    for (int mh = 0; mh < MH; ++mh) {
      const int m = g + 8 * mh;
      const uint4* xp = reinterpret_cast<const uint4*>(p.x + size_t(m) * p.K + kbase);
#pragma unroll
      for (int v = 0; v < WPC * XR / 4; ++v) {
        uint4 u = make_uint4(0, 0, 0, 0);
        if (m < p.M) {
          u = __ldg(xp + v);
          if (p.bf16) {
            u.x = bf16x2_to_f16x2_sat(u.x); u.y = bf16x2_to_f16x2_sat(u.y);
            u.z = bf16x2_to_f16x2_sat(u.z); u.w = bf16x2_to_f16x2_sat(u.w);
          }
        }
        dst[mh][(4 * v) / XR][(4 * v) % XR + 0] = u.x; dst[mh][(4 * v) / XR][(4 * v) % XR + 1] = u.y;
        dst[mh][(4 * v) / XR][(4 * v) % XR + 2] = u.z; dst[mh][(4 * v) / XR][(4 * v) % XR + 3] = u.w;
      }
    }
  };
  if (PF) load_x(0, xbuf[0]);

#pragma unroll
  for (int i = 0; i < CPW; ++i) {
    {
#pragma unroll
      for (int j = 0; j < GPS; ++j) {
        const int gcur = i * GPS + j;
        if (PF) {
          if (gcur + 1 < NG) load_x(gcur + 1, xbuf[(gcur + 1) & 1]);
        } else {
          load_x(gcur, xbuf[0]);
        }
        uint32_t (&xr)[MH][WPC][XR] = xbuf[PF ? (gcur & 1) : 0];
        if (TRACE && i == 0 && j == 0 && lane == 0) {
          tr[3] = gemv_clock_after(xr[0][0][0]);
          tr[4] = gemv_clock_after(qa[0][0] ^ qb[0][0]);
        }
        // raw fields times activations: acc[mh][type], and the plain activation sums accx[mh]
        float acc[MH][NT][4], accx[MH][4];
#pragma unroll
        for (int t = 0; t < WPC; ++t) {
          const uint32_t q0 = qa[i][j * WPC + t], q1 = qb[i][j * WPC + t];
          const uint32_t q0h = q0 >> 8, q1h = q1 >> 8;
#pragma unroll
          for (int ty = 0; ty < NT; ++ty) {
            const uint32_t mask = MASK0 << (BITS * ty);
            const uint32_t a0 = q0 & mask, a1 = q1 & mask, a2 = q0h & mask, a3 = q1h & mask;
#pragma unroll
            for (int mh = 0; mh < MH; ++mh) {
              // element a of the word pairs with element a + CPWORD/2: codes e_a and e_(a + CPWORD/2)
              // share a field position in the two halves of the word
              const uint32_t* xw = xr[mh][t];
              const uint32_t sel = (ty & 1) ? 0x7632u : 0x5410u;
              const uint32_t b0 = prmt(xw[ty / 2], xw[(ty + CPWORD / 2) / 2], sel);
              const uint32_t b1 = prmt(xw[(ty + NT) / 2], xw[(ty + NT + CPWORD / 2) / 2], sel);
              if (t == 0) {
                mma_new(acc[mh][ty], a0, a1, a2, a3, b0, b1);
              } else {
                mma_acc(acc[mh][ty], a0, a1, a2, a3, b0, b1);
              }
              if (!XC) {
                if (t == 0 && ty == 0) {
                  mma_new(accx[mh], ONES, ONES, ONES, ONES, b0, b1);
                } else {
                  mma_acc(accx[mh], ONES, ONES, ONES, ONES, b0, b1);
                }
              }
            }
          }
        }
        if (XC && i == 0 && j == 0) {
#pragma unroll
          for (int tok = 0; tok < 2; ++tok) {
            float sum = 0.f;
#pragma unroll
            for (int v = 0; v < HPL / 4; ++v) {
              uint2 u = xu[tok][v];
              if (p.bf16) {
                u.x = bf16x2_to_f16x2_sat(u.x);
                u.y = bf16x2_to_f16x2_sat(u.y);
              }
              const float2 f0 = __half22float2(u32_as_h2(u.x)), f1 = __half22float2(u32_as_h2(u.y));
              sum += f0.x; sum += f0.y; sum += f1.x; sum += f1.y;
            }
#pragma unroll
            for (int o = LPG / 2; o >= 1; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
#pragma unroll
            for (int gi = 0; gi < NG; ++gi) xs[tok][gi] = __shfl_sync(0xffffffffu, sum, gi * LPG);
          }
        }
        // once per group: combine the types (a field at bit BITS*ty carries 2^(BITS*ty) times its code;
        // a code in the lowest field is code * 2^-24 as an fp16 number), scale, add zero * sum(x)
        const int gidx = i * GPS + j;
        const float s0 = table_entry(ts0, gidx) * 16777216.f, s1 = table_entry(ts1, gidx) * 16777216.f;
        const float z0 = table_entry(tz0, gidx), z1 = table_entry(tz1, gidx);
#pragma unroll
        for (int mh = 0; mh < MH; ++mh)
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            float tsum = acc[mh][NT - 1][r];
#pragma unroll
            for (int ty = NT - 2; ty >= 0; --ty) tsum = fmaf(tsum, 1.f / float(1 << BITS), acc[mh][ty][r]);
            yv[mh][r] = fmaf(tsum, r < 2 ? s0 : s1, yv[mh][r]);
            const float xsum = XC ? xs[r & 1][gidx] : accx[mh][r & 1];
            yv[mh][r] = fmaf(xsum, r < 2 ? z0 : z1, yv[mh][r]);
          }
      }
    }
  }
  }  // rounds
  if (TRACE && lane == 0) tr[5] = gemv_clock_after(__float_as_uint(yv[0][0]));

  // ---- add the KQ partial tiles through shared memory (fixed order) and write the strip ---------
  // yv[mh][r] of lane (g, c): weight row n_base + g + 8*(r>>1), token 8*mh + 2c + (r&1).
  if (p.KQ > 1) {
#pragma unroll
    for (int mh = 0; mh < MH; ++mh)
#pragma unroll
      for (int r = 0; r < 4; ++r) red[(warp * FR + mh * 4 + r) * 32 + lane] = yv[mh][r];
    __syncthreads();
    if (TRACE && lane == 0) tr[6] = gemv_clock();
    for (int f = warp; f < FR; f += p.KQ) {  // warp f adds register f of every warp, in warp order
      float v = 0.f;
      for (int q = 0; q < p.KQ; ++q) v += red[(q * FR + f) * 32 + lane];
      const int n = n_base + g + ((f >> 1) & 1) * 8, m = 8 * (f >> 2) + 2 * c + (f & 1);
      if (m < p.M) {
        if (p.bias) v += __half2float(__ldg(p.bias + n));
        p.y[size_t(m) * p.N + n] = float_to_out16(v, p.bf16);
      }
    }
  } else {
#pragma unroll
    for (int mh = 0; mh < MH; ++mh)
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int n = n_base + g + (r >> 1) * 8, m = 8 * mh + 2 * c + (r & 1);
        if (m < p.M) {
          float v = yv[mh][r];
          if (p.bias) v += __half2float(__ldg(p.bias + n));
          p.y[size_t(m) * p.N + n] = float_to_out16(v, p.bf16);
        }
      }
  }
  if (TRACE && lane == 0) tr[7] = gemv_globaltimer();
}

using GemvKernel = void (*)(const GemvParams);

template <int BITS, int MH, int GPS, int CPW>
GemvKernel kernel_for(bool xc, bool trace) {
#ifdef ASRQ_TRACE
  if (trace) {
    if (MH == 1 && xc) return gemv_a16_kernel<BITS, 1, GPS, CPW, true, true>;
    return gemv_a16_kernel<BITS, MH, GPS, CPW, false, true>;
  }
#endif
  (void)trace;  // the shipped library holds no trace variants
  if (MH == 1 && xc) return gemv_a16_kernel<BITS, 1, GPS, CPW, true, false>;
  return gemv_a16_kernel<BITS, MH, GPS, CPW, false, false>;
}
template <int BITS, int MH>
GemvKernel kernel_for(int gps, int cpw, bool xc, bool trace) {
  switch (gps * 8 + cpw) {
    case 1 * 8 + 1: return kernel_for<BITS, MH, 1, 1>(xc, trace);
    case 1 * 8 + 2: return kernel_for<BITS, MH, 1, 2>(xc, trace);
    case 1 * 8 + 4: return kernel_for<BITS, MH, 1, 4>(xc, trace);
    case 2 * 8 + 1: return kernel_for<BITS, MH, 2, 1>(xc, trace);
    case 2 * 8 + 2: return kernel_for<BITS, MH, 2, 2>(xc, trace);
    case 2 * 8 + 4: return kernel_for<BITS, MH, 2, 4>(xc, trace);
    case 4 * 8 + 1: return kernel_for<BITS, MH, 4, 1>(xc, trace);
    case 4 * 8 + 2: return kernel_for<BITS, MH, 4, 2>(xc, trace);
    default: return nullptr;
  }
}
// LOOP variants: the most steps per round the group table allows (CPW * GPS <= 8), no trace build
template <int BITS, int MH>
GemvKernel loop_kernel_for(int gps, bool xc, int* cpw) {
  *cpw = gps == 4 ? 2 : 4;
  if (MH == 1 && xc) {
    switch (gps) {
      case 1: return gemv_a16_kernel<BITS, 1, 1, 4, true, false, true>;
      case 2: return gemv_a16_kernel<BITS, 1, 2, 4, true, false, true>;
      case 4: return gemv_a16_kernel<BITS, 1, 4, 2, true, false, true>;
      default: return nullptr;
    }
  }
  switch (gps) {
    case 1: return gemv_a16_kernel<BITS, MH, 1, 4, false, false, true>;
    case 2: return gemv_a16_kernel<BITS, MH, 2, 4, false, false, true>;
    case 4: return gemv_a16_kernel<BITS, MH, 4, 2, false, false, true>;
    default: return nullptr;
  }
}
GemvKernel loop_kernel_for(int bits, int mh, int gps, bool xc, int* cpw) {
  if (bits == 4) return mh == 1 ? loop_kernel_for<4, 1>(gps, xc, cpw) : loop_kernel_for<4, 2>(gps, xc, cpw);
  return mh == 1 ? loop_kernel_for<2, 1>(gps, xc, cpw) : loop_kernel_for<2, 2>(gps, xc, cpw);
}

GemvKernel kernel_for(int bits, int mh, int gps, int cpw, bool xc, bool trace) {
  if (bits == 4) return mh == 1 ? kernel_for<4, 1>(gps, cpw, xc, trace) : kernel_for<4, 2>(gps, cpw, xc, trace);
  return mh == 1 ? kernel_for<2, 1>(gps, cpw, xc, trace) : kernel_for<2, 2>(gps, cpw, xc, trace);
}

// How one launch splits K inside a block: a warp takes CPW steps (1, 2 or 4) and KQ warps (1..16)
// share the row strip, KQ * CPW = steps.  The pair is chosen so that the whole grid is resident at
// once if possible (fewest waves, from the occupancy of the kernel variant), then for the most
// warps: all loads of the layer go out together and the per-warp instruction streams are short.
struct GemvSplit {
  int KQ, CPW;
  GemvKernel kern;
  int R = 1;        // rounds per warp (LOOP variants)
};

GemvSplit gemv_pick_split(int bits, int mh, int gps, bool xc, bool trace, int64_t N, int64_t K, int sm_count) {
  const int stepk = bits == 4 ? 128 : 256;
  const int steps = int(K / stepk);
  const int cpw_env = option(kOptGemvCpw);  // tuning knob
  GemvSplit best;
  best.KQ = best.CPW = 0;
  best.kern = nullptr;
  long best_waves = 0;
  for (int cpw = 1; cpw <= kGemvMaxSteps; cpw *= 2) {
    if (steps % cpw || steps / cpw > kGemvMaxWarps || cpw * gps > 8) continue;
    if (cpw_env && cpw != cpw_env) continue;
    const int kq = steps / cpw;
    GemvKernel k = kernel_for(bits, mh, gps, cpw, xc, trace);
    if (!k) continue;
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k, 32 * kq, 0) != cudaSuccess || per_sm < 1) {
      cudaGetLastError();
      continue;
    }
    const long slots = long(per_sm) * sm_count;
    const long waves = (long(N / 16) + slots - 1) / slots;
    // Fewest waves first.  Among those, 8 to 12 warps per block measured fastest on the decode
    // shapes (16 warps pay more for the shared-memory reduction and the block-wide barrier, 4 to 6
    // leave too few loads in flight): the largest count up to 12, else the smallest above.
    auto rank = [](int q) { return q <= 12 ? 100 - q : 100 + q; };
    if (!best.kern || waves < best_waves || (waves == best_waves && rank(kq) < rank(best.KQ))) {
      best.KQ = kq;
      best.CPW = cpw;
      best.kern = k;
      best_waves = waves;
    }
  }
  // Layers that do not fit one resident wave (or whose K is longer than 16 warps x 4 steps): small
  // blocks that walk K in rounds, so that the blocks sharing an SM overlap loads and arithmetic.
  const int loop_env = option(kOptGemvLoop);  // tuning knob
  const bool large = N * K * bits / 8 >= (int64_t(16) << 20);
  if (!trace && loop_env != 0 && (!best.kern || (best_waves > 1 && (large || loop_env == 1)))) {
    int cpw = 0;
    GemvKernel k = loop_kernel_for(bits, mh, gps, xc, &cpw);
    static const int kq_order[] = {4, 8, 2, 16, 1};
    for (int kq : kq_order) {
      if (!k || steps % (kq * cpw)) continue;
      GemvSplit sp;
      sp.KQ = kq;
      sp.CPW = cpw;
      sp.kern = k;
      sp.R = steps / (kq * cpw);
      return sp;
    }
  }
  return best;
}

// the choice costs a few occupancy queries: keep it per (bits, class, groups per step, N, K, device SMs)
GemvSplit cached_split(int bits, int cls, int gps, bool trace, int64_t N, int64_t K, int sm_count) {
  struct Entry {
    uint64_t key;
    GemvSplit sp;
  };
  static std::mutex mu;
  static std::vector<Entry> cache;
  static unsigned cache_generation = 0;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (cache_generation != options_generation()) {  // a tuning option changed: choose again
      cache.clear();
      cache_generation = options_generation();
    }
  }
  const uint64_t key = (uint64_t(N) << 40) ^ (uint64_t(K) << 16) ^ (uint64_t(sm_count) << 6) ^ (uint64_t(gps) << 3) ^
                       (uint64_t(cls) << 1) ^ uint64_t(bits == 4);
  {
    std::lock_guard<std::mutex> lock(mu);
    for (const Entry& e : cache)
      if (e.key == key) return e.sp;
  }
  const GemvSplit sp = gemv_pick_split(bits, cls == 2 ? 2 : 1, gps, cls == 0, trace, N, K, sm_count);
  std::lock_guard<std::mutex> lock(mu);
  if (cache.size() < 4096) cache.push_back({key, sp});
  return sp;
}

int launch_gemv(const GemvSplit& sp, const GemvParams& p, cudaStream_t stream) {
  // Programmatic dependent launch: consecutive decode kernels overlap their weight fetch with the
  // predecessor's tail (the kernel orders itself with griddepcontrol.wait).
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.N / 16);
  cfg.blockDim = dim3(32 * p.KQ);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  const bool pdl = option(kOptNoPdl) == 0;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  ASRQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, sp.kern, p));
  return ASRQ_OK;
}

}  // namespace

int gemv_a16(int bits, const void* x, const uint8_t* w, const void* scales, const void* zeros,
             const void* bias, void* y, int64_t M, int64_t N, int64_t K, int group_size, int dtype,
             void* workspace, size_t workspace_bytes, int sm_count, cudaStream_t stream, int max_split) {
  const int chunk = (128 / bits) * 4;
  if (N % 16 || K % chunk || group_size <= 0 || K % group_size || group_size % (128 / bits))
    return fail(ASRQ_ERR_SHAPE,
                "w%da16 gemv: need N%%16==0, K%%%d==0, group_size%%%d==0, K%%group_size==0 "
                "(N=%lld K=%lld g=%d)", bits, chunk, 128 / bits, (long long)N, (long long)K, group_size);
  if (N > int64_t(4096) * 16 || K > (1 << 20))
    return fail(ASRQ_ERR_LIMIT, "w%da16 gemv: N > 65536 or K > 2^20", bits);
  // the workspace contract is the same whichever kernel runs
  if (workspace_bytes < gemv_workspace_bytes(N, max_split))
    return fail(ASRQ_ERR_WORKSPACE, "w%da16 gemv: workspace %zu < %zu bytes", bits, workspace_bytes,
                gemv_workspace_bytes(N, max_split));
  const int gps = chunk % group_size == 0 ? chunk / group_size : 0;  // groups per step: 1, 2 or 4
  // Staged variant (gemv_a16_staged.cu): weights prefetched into shared memory ahead of the stream dependency,
  // up to 32 tokens per launch.  Measured no faster than the kernel below, so it runs only on request.
  const int which = option(kOptGemvKernel);
  if (which == 3 && aligned16(scales) && aligned16(zeros) &&
      gemv_a16_staged_supports(bits, std::min<int64_t>(M, 32), N, K, group_size, sm_count)) {
    for (int64_t m0 = 0; m0 < M; m0 += 32) {
      const int64_t mb = std::min<int64_t>(32, M - m0);
      const int rc = gemv_a16_staged(bits, static_cast<const uint16_t*>(x) + m0 * K, w, scales, zeros, bias,
                                     static_cast<uint16_t*>(y) + m0 * N, mb, N, K, group_size, dtype, workspace, sm_count,
                                     stream);
      if (rc) return rc;
    }
    return ASRQ_OK;
  }
  const bool force_splitk = which == 2;
#ifdef ASRQ_TRACE
  const bool trace = option(kOptTrace) != 0;
#else
  const bool trace = false;
#endif
  if (force_splitk || (gps != 1 && gps != 2 && gps != 4) || !aligned16(scales) || !aligned16(zeros))
    return gemv_a16_splitk(bits, x, w, scales, zeros, bias, y, M, N, K, group_size, dtype, workspace,
                           workspace_bytes, sm_count, stream, max_split);
  // one split per token-count class (the kernel variant, hence its occupancy, depends on it):
  // 0: M <= 2, 1: M <= 8, 2: M <= 16; remembered per layer shape
  GemvSplit split[3];
  for (int cls = 0; cls < 3; ++cls) {
    const bool needed = cls == 2 ? M > 8 : (cls == 1 ? (M % 16 > 2 && M % 16 <= 8) : (M % 16 >= 1 && M % 16 <= 2));
    if (!needed) continue;
    split[cls] = cached_split(bits, cls, gps, trace, N, K, sm_count);
    if (!split[cls].kern)
      return gemv_a16_splitk(bits, x, w, scales, zeros, bias, y, M, N, K, group_size, dtype, workspace,
                             workspace_bytes, sm_count, stream, max_split);
  }
  GemvParams p;
  p.w = w;
  p.scales = static_cast<const __half*>(scales);
  p.zeros = static_cast<const __half*>(zeros);
  p.bias = static_cast<const __half*>(bias);
  p.N = int(N);
  p.K = int(K);
  p.groups_per_row = int(K / group_size);
  p.bf16 = dtype == ASRQ_BF16;
  // diagnostic marks go to the (otherwise unused) partial-sum area of the workspace
  p.trace = trace ? reinterpret_cast<unsigned long long*>(static_cast<char*>(workspace) + kPartialOffset) : nullptr;
  for (int64_t m0 = 0; m0 < M; m0 += 16) {
    const int mb = int(std::min<int64_t>(16, M - m0));
    p.x = static_cast<const uint16_t*>(x) + m0 * K;
    p.y = static_cast<uint16_t*>(y) + m0 * N;
    p.M = mb;
    const GemvSplit& sp = split[mb <= 2 ? 0 : (mb <= 8 ? 1 : 2)];
    p.KQ = sp.KQ;
    p.CPW = sp.CPW;
    p.R = sp.R;
    const int rc = launch_gemv(sp, p, stream);
    if (rc) return rc;
  }
  return ASRQ_OK;
}

}  // namespace asrq
