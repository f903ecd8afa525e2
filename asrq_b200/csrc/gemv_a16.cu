// Decode path: y[M,N] = x[M,K] . dequant(W)[N,K]^T for M <= 16 per launch.
//
// HBM-bound skinny GEMM, organised so that every weight byte of the layer is requested within
// the first microsecond and no warp has a long instruction stream: a warp owns a strip of 16
// weight rows over a short K span of one to four "steps" (a step = one 128-bit load per lane
// per row = 128 k for 4-bit, 256 k for 2-bit).  Each lane streams 128-bit words of packed
// weights for two rows (rows g and g+8, g = lane/4), turns them into fp16 in registers (exact
// integer code, then one fused multiply-add with the group scale and offset) and uses them as
// the A operand of mma.sync.m16n8k16; the activations (B operand, up to 16 tokens) are read
// straight from global memory (they are tiny and L1-resident) and permuted in registers to the
// element order the unpacking produces.
//
// The KQ warps of a block share a row strip and split K between them; their partial tiles are
// added through shared memory in a fixed order, so the result never depends on scheduling and
// no workspace is touched.  Layers too long for 16 warps x 4 steps go to the split-K kernel in
// gemv_a16_splitk.cu, which splits K across blocks through the caller's workspace.
#include <algorithm>
#include <cstdlib>

#include "common.cuh"

namespace asrq {

int gemv_a16_splitk(int bits, const void* x, const uint8_t* w, const void* scales, const void* zeros,
                    const void* bias, void* y, int64_t M, int64_t N, int64_t K, int group_size, int dtype,
                    void* workspace, size_t workspace_bytes, int sm_count, cudaStream_t stream, int max_split);
size_t gemv_workspace_bytes(int64_t N, int max_split);

namespace {

struct GemvParams {
  const uint16_t* x;
  const uint8_t* w;
  const __half* scales;
  const __half* zeros;
  const __half* bias;
  uint16_t* y;
  int M, N, K, group_size, groups_per_row, KQ, CPW, bf16;
  unsigned long long* trace;  // diagnostic: per-warp clock marks (8 words per warp), NULL normally
};

constexpr int kGemvMaxWarps = 16;
constexpr int kGemvMaxSteps = 4;

__device__ __forceinline__ void mma_m16n8k16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                             uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t bf16x2_to_f16x2_sat(uint32_t v) {
  float lo = __uint_as_float(v << 16);
  float hi = __uint_as_float(v & 0xffff0000u);
  lo = fminf(fmaxf(lo, -65504.f), 65504.f);
  hi = fminf(fmaxf(hi, -65504.f), 65504.f);
  return h2_as_u32(__floats2half2_rn(lo, hi));
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

template <int BITS, int MH, bool TRACE>
__global__ void __launch_bounds__(kGemvMaxWarps * 32) gemv_a16_kernel(const GemvParams p) {
  constexpr int KPT = 128 / BITS;    // k handled by one lane per 128-bit load
  constexpr int CHUNK = KPT * 4;     // k handled by a warp per step
  constexpr int UPT = KPT / 8;       // 8-element activation units per lane per step
  constexpr int NH = 32 / BITS / 2;  // half2 values per 32-bit weight word
  constexpr int FR = 4 * MH;         // accumulator registers per lane

  __shared__ float red[kGemvMaxWarps * FR * 32];
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;  // warp = K part inside the block
  const int g = lane >> 2, c = lane & 3;
  const int n_base = blockIdx.x * 16;
  unsigned long long* tr = nullptr;
  if (TRACE) {
    tr = p.trace + (size_t(blockIdx.x) * kGemvMaxWarps + warp) * 8;
    if (lane == 0) {
      tr[0] = gemv_globaltimer();
      tr[1] = gemv_clock();
    }
  }
  const int r0 = n_base + g, r1 = r0 + 8;
  const int kw = warp * (p.CPW * CHUNK) + c * KPT;  // first k of this lane
  const size_t row_bytes = size_t(p.K) * BITS / 8;
  const uint8_t* w0 = p.w + size_t(r0) * row_bytes + size_t(kw) * BITS / 8;
  const uint8_t* w1 = p.w + size_t(r1) * row_bytes + size_t(kw) * BITS / 8;
  const __half* sc0 = p.scales + size_t(r0) * p.groups_per_row;
  const __half* sc1 = p.scales + size_t(r1) * p.groups_per_row;
  const __half* zr0 = p.zeros + size_t(r0) * p.groups_per_row;
  const __half* zr1 = p.zeros + size_t(r1) * p.groups_per_row;

  // Let the next kernel on the stream start, and start streaming weights before this kernel's
  // own predecessor has finished: weights, scales and zeros are constants; only the activations
  // and the output depend on earlier kernels.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  uint4 qa[kGemvMaxSteps], qb[kGemvMaxSteps];
  __half sa[kGemvMaxSteps], sb[kGemvMaxSteps], za[kGemvMaxSteps], zb[kGemvMaxSteps];
#pragma unroll
  for (int i = 0; i < kGemvMaxSteps; ++i) {
    if (i < p.CPW) {
      qa[i] = ldg_stream_v4(w0 + size_t(i) * (CHUNK * BITS / 8));
      qb[i] = ldg_stream_v4(w1 + size_t(i) * (CHUNK * BITS / 8));
      const int gi = (kw + i * CHUNK) / p.group_size;
      sa[i] = __ldg(sc0 + gi);
      za[i] = __ldg(zr0 + gi);
      sb[i] = __ldg(sc1 + gi);
      zb[i] = __ldg(zr1 + gi);
    }
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (TRACE && lane == 0) tr[2] = gemv_clock();

  float acc[MH][4];
#pragma unroll
  for (int mh = 0; mh < MH; ++mh)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[mh][i] = 0.f;

#pragma unroll
  for (int i = 0; i < kGemvMaxSteps; ++i) {
    if (i < p.CPW) {
      // activations of token g (and g+8) for this lane's KPT k: natural order from global memory,
      // then paired (e, e+4) within each 8 for 4-bit, (e, e+8) within each 16 for 2-bit
      uint32_t xb[MH][UPT][4];
#pragma unroll
      for (int mh = 0; mh < MH; ++mh) {
        const int m = g + 8 * mh;
        uint4 u[UPT];
#pragma unroll
        for (int t = 0; t < UPT; ++t) {
          u[t] = make_uint4(0, 0, 0, 0);
          if (m < p.M) {
            u[t] = __ldg(reinterpret_cast<const uint4*>(p.x + size_t(m) * p.K + kw + i * CHUNK) + t);
            if (p.bf16) {
              u[t].x = bf16x2_to_f16x2_sat(u[t].x); u[t].y = bf16x2_to_f16x2_sat(u[t].y);
              u[t].z = bf16x2_to_f16x2_sat(u[t].z); u[t].w = bf16x2_to_f16x2_sat(u[t].w);
            }
          }
        }
        if (BITS == 4) {
#pragma unroll
          for (int t = 0; t < UPT; ++t) {
            xb[mh][t][0] = prmt(u[t].x, u[t].z, 0x5410); xb[mh][t][1] = prmt(u[t].x, u[t].z, 0x7632);
            xb[mh][t][2] = prmt(u[t].y, u[t].w, 0x5410); xb[mh][t][3] = prmt(u[t].y, u[t].w, 0x7632);
          }
        } else {
#pragma unroll
          for (int t = 0; t + 1 < UPT; t += 2) {
            const uint4 lo = u[t], hi = u[t + 1];
            xb[mh][t][0] = prmt(lo.x, hi.x, 0x5410); xb[mh][t][1] = prmt(lo.x, hi.x, 0x7632);
            xb[mh][t][2] = prmt(lo.y, hi.y, 0x5410); xb[mh][t][3] = prmt(lo.y, hi.y, 0x7632);
            xb[mh][t + 1][0] = prmt(lo.z, hi.z, 0x5410); xb[mh][t + 1][1] = prmt(lo.z, hi.z, 0x7632);
            xb[mh][t + 1][2] = prmt(lo.w, hi.w, 0x5410); xb[mh][t + 1][3] = prmt(lo.w, hi.w, 0x7632);
          }
        }
      }
      if (TRACE && i == 0 && lane == 0) {
        tr[3] = gemv_clock_after(xb[0][0][0]);
        tr[4] = gemv_clock_after(qa[0].x ^ qb[0].x);
      }
      const __half2 s0 = __half2half2(sa[i]), z0 = __half2half2(za[i]);
      const __half2 s1 = __half2half2(sb[i]), z1 = __half2half2(zb[i]);
      const uint32_t wa[4] = {qa[i].x, qa[i].y, qa[i].z, qa[i].w};
      const uint32_t wb[4] = {qb[i].x, qb[i].y, qb[i].z, qb[i].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        __half2 ha[NH], hb[NH];
        unpack_codes_f16<BITS>(wa[j], ha);
        unpack_codes_f16<BITS>(wb[j], hb);
#pragma unroll
        for (int q = 0; q < NH; ++q) {
          ha[q] = __hfma2(ha[q], s0, z0);
          hb[q] = __hfma2(hb[q], s1, z1);
        }
#pragma unroll
        for (int mh = 0; mh < MH; ++mh) {
#pragma unroll
          for (int t = 0; t < NH / 4; ++t) {
            const uint32_t* xv = xb[mh][j * (NH / 4) + t];
            mma_m16n8k16(acc[mh], h2_as_u32(ha[4 * t]), h2_as_u32(hb[4 * t]), h2_as_u32(ha[4 * t + 1]),
                         h2_as_u32(hb[4 * t + 1]), xv[0], xv[1]);
            mma_m16n8k16(acc[mh], h2_as_u32(ha[4 * t + 2]), h2_as_u32(hb[4 * t + 2]), h2_as_u32(ha[4 * t + 3]),
                         h2_as_u32(hb[4 * t + 3]), xv[2], xv[3]);
          }
        }
      }
    }
  }

  if (TRACE && lane == 0) tr[5] = gemv_clock_after(__float_as_uint(acc[0][0]));
  // ---- add the KQ partial tiles through shared memory (fixed order) ----------------------------
  // acc[mh][i] of lane (g, c): weight row n_base + g + 8*(i>>1), token 8*mh + 2c + (i&1).
  if (p.KQ > 1) {
#pragma unroll
    for (int mh = 0; mh < MH; ++mh)
#pragma unroll
      for (int i = 0; i < 4; ++i) red[(warp * FR + mh * 4 + i) * 32 + lane] = acc[mh][i];
    __syncthreads();
    if (TRACE && lane == 0) tr[6] = gemv_clock();
    if (warp != 0) return;
#pragma unroll
    for (int mh = 0; mh < MH; ++mh)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float v = 0.f;
        for (int q = 0; q < p.KQ; ++q) v += red[(q * FR + mh * 4 + i) * 32 + lane];
        acc[mh][i] = v;
      }
  }
  // warp 0 now holds the block's 16 x (8*MH) tile
#pragma unroll
  for (int mh = 0; mh < MH; ++mh)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int n = n_base + g + (i >> 1) * 8, m = 8 * mh + 2 * c + (i & 1);
      if (m < p.M) {
        float v = acc[mh][i];
        if (p.bias) v += __half2float(__ldg(p.bias + n));
        p.y[size_t(m) * p.N + n] = float_to_out16(v, p.bf16);
      }
    }
  if (TRACE && lane == 0) tr[7] = gemv_globaltimer();
}

// How one launch splits K inside a block: a warp takes CPW steps (1..4) and KQ warps (1..16)
// share the row strip, KQ * CPW = steps.  KQ is chosen among the divisors of the step count so
// that the grid has about 20 warps per SM (enough bytes in flight, short per-warp instruction
// streams).  ok = false when no divisor fits.
struct GemvSplit {
  int KQ, CPW;
  bool ok;
};

GemvSplit gemv_pick_split(int bits, int64_t N, int64_t K, int sm_count) {
  const int chunk = (128 / bits) * 4;
  const int nchunks = int(K / chunk);
  const double want = double(sm_count) * 20.0;
  GemvSplit r = {1, nchunks, false};
  double best_cost = 1e30;
  for (int kq = 1; kq <= std::min(nchunks, kGemvMaxWarps); ++kq) {
    if (nchunks % kq || nchunks / kq > kGemvMaxSteps) continue;
    const double warps = double(N / 16) * kq;
    const double cost = warps < want ? want / warps : warps / want;  // distance from the target, as a ratio
    if (cost < best_cost) {
      best_cost = cost;
      r = {kq, nchunks / kq, true};
    }
  }
  return r;
}

template <int BITS, int MH>
int launch_gemv(const GemvParams& p, cudaStream_t stream) {
  auto kern = p.trace ? gemv_a16_kernel<BITS, MH, true> : gemv_a16_kernel<BITS, MH, false>;
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
  static const bool pdl = getenv("ASRQ_B200_NO_PDL") == nullptr;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  ASRQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, p));
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
  const GemvSplit sp = gemv_pick_split(bits, N, K, sm_count);
  static const bool force_splitk = getenv("ASRQ_B200_GEMV_SPLITK") != nullptr;
  if (!sp.ok || force_splitk)
    return gemv_a16_splitk(bits, x, w, scales, zeros, bias, y, M, N, K, group_size, dtype, workspace,
                           workspace_bytes, sm_count, stream, max_split);
  GemvParams p;
  p.w = w;
  p.scales = static_cast<const __half*>(scales);
  p.zeros = static_cast<const __half*>(zeros);
  p.bias = static_cast<const __half*>(bias);
  p.N = int(N);
  p.K = int(K);
  p.group_size = group_size;
  p.groups_per_row = int(K / group_size);
  p.bf16 = dtype == ASRQ_BF16;
  p.KQ = sp.KQ;
  p.CPW = sp.CPW;
  // diagnostic marks go to the (otherwise unused) partial-sum area of the workspace
  p.trace = getenv("ASRQ_B200_TRACE")
                ? reinterpret_cast<unsigned long long*>(static_cast<char*>(workspace) + kPartialOffset)
                : nullptr;
  for (int64_t m0 = 0; m0 < M; m0 += 16) {
    const int mb = int(std::min<int64_t>(16, M - m0));
    const int mh = mb > 8 ? 2 : 1;
    p.x = static_cast<const uint16_t*>(x) + m0 * K;
    p.y = static_cast<uint16_t*>(y) + m0 * N;
    p.M = mb;
    int rc;
    if (bits == 4)
      rc = mh == 1 ? launch_gemv<4, 1>(p, stream) : launch_gemv<4, 2>(p, stream);
    else
      rc = mh == 1 ? launch_gemv<2, 1>(p, stream) : launch_gemv<2, 2>(p, stream);
    if (rc) return rc;
  }
  return ASRQ_OK;
}

}  // namespace asrq
