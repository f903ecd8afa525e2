// Decode path: y[M,N] = x[M,K] . dequant(W)[N,K]^T for M <= 16 per launch.
//
// HBM-bound skinny GEMM.  A warp owns a strip of 16 weight rows over one K slice:
// each lane streams 128-bit words of packed weights for two rows (rows g and g+8,
// g = lane/4), turns them into fp16 in registers (exact integer code, then one
// fused multiply-add with the group scale and offset) and uses them as the A
// operand of mma.sync.m16n8k16; the activations (B operand, up to 16 tokens) sit
// in shared memory in the element order the unpacking produces, so no shuffles are
// needed.  K is split across gridDim.y; partial sums go to the caller's workspace
// and the last block to arrive for a row tile adds them in slice order, so the
// result does not depend on scheduling.
#include <algorithm>

#include "common.cuh"

namespace asrq {

struct GemvParams {
  const uint16_t* x;
  const uint8_t* w;
  const __half* scales;
  const __half* zeros;
  const __half* bias;
  uint16_t* y;
  float* partials;
  unsigned* counters;
  int M, N, K, group_size, groups_per_row, S, kslice, bf16;
};

constexpr int kGemvWarps = 8;
constexpr int kGemvRows = kGemvWarps * 16;  // weight rows per block

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

template <int BITS, int MH>
__global__ void __launch_bounds__(kGemvWarps * 32) gemv_a16_kernel(const GemvParams p) {
  constexpr int KPT = 128 / BITS;    // k handled by one lane per 128-bit load
  constexpr int CHUNK = KPT * 4;     // k handled by a warp per step
  constexpr int UPT = KPT / 8;       // 16-byte activation units per lane per step
  constexpr int NH = 32 / BITS / 2;  // half2 values per 32-bit weight word
  constexpr int MR = 8 * MH;         // token rows held in shared memory

  extern __shared__ uint4 xs[];
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, c = lane & 3;
  const int k_begin = blockIdx.y * p.kslice;
  const int row_units = p.kslice / 8 + 4;  // +64 B: rows g and g+1 land on different banks

  // ---- stage the activation slice, re-ordered to the unpacking order -------------
  {
    const int blocks16 = p.kslice / 16;
    for (int i = tid; i < MR * blocks16; i += blockDim.x) {
      const int m = i / blocks16, b = i - m * blocks16;
      uint4 lo = make_uint4(0, 0, 0, 0), hi = lo;
      if (m < p.M) {
        const uint4* src = reinterpret_cast<const uint4*>(p.x + size_t(m) * p.K + k_begin + b * 16);
        lo = __ldg(src);
        hi = __ldg(src + 1);
        if (p.bf16) {
          lo.x = bf16x2_to_f16x2_sat(lo.x); lo.y = bf16x2_to_f16x2_sat(lo.y);
          lo.z = bf16x2_to_f16x2_sat(lo.z); lo.w = bf16x2_to_f16x2_sat(lo.w);
          hi.x = bf16x2_to_f16x2_sat(hi.x); hi.y = bf16x2_to_f16x2_sat(hi.y);
          hi.z = bf16x2_to_f16x2_sat(hi.z); hi.w = bf16x2_to_f16x2_sat(hi.w);
        }
      }
      uint4 o0, o1;
      if (BITS == 4) {  // within each 8: (0,4)(1,5)(2,6)(3,7)
        o0.x = prmt(lo.x, lo.z, 0x5410); o0.y = prmt(lo.x, lo.z, 0x7632);
        o0.z = prmt(lo.y, lo.w, 0x5410); o0.w = prmt(lo.y, lo.w, 0x7632);
        o1.x = prmt(hi.x, hi.z, 0x5410); o1.y = prmt(hi.x, hi.z, 0x7632);
        o1.z = prmt(hi.y, hi.w, 0x5410); o1.w = prmt(hi.y, hi.w, 0x7632);
      } else {  // within each 16: (0,8)(1,9)...(7,15)
        o0.x = prmt(lo.x, hi.x, 0x5410); o0.y = prmt(lo.x, hi.x, 0x7632);
        o0.z = prmt(lo.y, hi.y, 0x5410); o0.w = prmt(lo.y, hi.y, 0x7632);
        o1.x = prmt(lo.z, hi.z, 0x5410); o1.y = prmt(lo.z, hi.z, 0x7632);
        o1.z = prmt(lo.w, hi.w, 0x5410); o1.w = prmt(lo.w, hi.w, 0x7632);
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int kb = 2 * b + h;  // 8-element block inside the slice
        const int chunk = kb / (CHUNK / 8);
        const int r = kb - chunk * (CHUNK / 8);
        const int cc = r / UPT, blk = r - cc * UPT;
        xs[m * row_units + (chunk * UPT + blk) * 4 + cc] = h ? o1 : o0;
      }
    }
  }
  __syncthreads();

  const int n_base = blockIdx.x * kGemvRows + warp * 16;
  float acc[MH][4];
#pragma unroll
  for (int mh = 0; mh < MH; ++mh)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[mh][i] = 0.f;

  if (n_base < p.N) {
    const int r0 = n_base + g, r1 = r0 + 8;
    const size_t row_bytes = size_t(p.K) * BITS / 8;
    const uint8_t* w0 = p.w + r0 * row_bytes + size_t(k_begin + c * KPT) * BITS / 8;
    const uint8_t* w1 = p.w + r1 * row_bytes + size_t(k_begin + c * KPT) * BITS / 8;
    const __half* sc0 = p.scales + size_t(r0) * p.groups_per_row;
    const __half* sc1 = p.scales + size_t(r1) * p.groups_per_row;
    const __half* zr0 = p.zeros + size_t(r0) * p.groups_per_row;
    const __half* zr1 = p.zeros + size_t(r1) * p.groups_per_row;
    const int nchunks = p.kslice / CHUNK;
    constexpr int PF = 2;  // chunks of weights in flight ahead of the math
    uint4 qa[PF + 1], qb[PF + 1];
#pragma unroll
    for (int i = 0; i < PF; ++i) {
      if (i < nchunks) {
        qa[i] = ldg_stream_v4(w0 + size_t(i) * (CHUNK * BITS / 8));
        qb[i] = ldg_stream_v4(w1 + size_t(i) * (CHUNK * BITS / 8));
      }
    }
    for (int chunk0 = 0; chunk0 < nchunks; chunk0 += PF + 1) {
#pragma unroll
      for (int u = 0; u < PF + 1; ++u) {
        const int chunk = chunk0 + u;
        if (chunk < nchunks) {
          const int nxt = chunk + PF;
          if (nxt < nchunks) {
            qa[(u + PF) % (PF + 1)] = ldg_stream_v4(w0 + size_t(nxt) * (CHUNK * BITS / 8));
            qb[(u + PF) % (PF + 1)] = ldg_stream_v4(w1 + size_t(nxt) * (CHUNK * BITS / 8));
          }
          const int gi = (k_begin + chunk * CHUNK + c * KPT) / p.group_size;
          const __half2 s0 = __half2half2(__ldg(sc0 + gi)), z0 = __half2half2(__ldg(zr0 + gi));
          const __half2 s1 = __half2half2(__ldg(sc1 + gi)), z1 = __half2half2(__ldg(zr1 + gi));
          const uint32_t wa[4] = {qa[u].x, qa[u].y, qa[u].z, qa[u].w};
          const uint32_t wb[4] = {qb[u].x, qb[u].y, qb[u].z, qb[u].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            __half2 ha[NH], hb[NH];
            unpack_codes_f16<BITS>(wa[j], ha);
            unpack_codes_f16<BITS>(wb[j], hb);
#pragma unroll
            for (int i = 0; i < NH; ++i) {
              ha[i] = __hfma2(ha[i], s0, z0);
              hb[i] = __hfma2(hb[i], s1, z1);
            }
#pragma unroll
            for (int mh = 0; mh < MH; ++mh) {
#pragma unroll
              for (int t = 0; t < NH / 4; ++t) {
                const uint4 xb =
                    xs[(g + 8 * mh) * row_units + (chunk * UPT + j * (NH / 4) + t) * 4 + c];
                mma_m16n8k16(acc[mh], h2_as_u32(ha[4 * t]), h2_as_u32(hb[4 * t]),
                             h2_as_u32(ha[4 * t + 1]), h2_as_u32(hb[4 * t + 1]), xb.x, xb.y);
                mma_m16n8k16(acc[mh], h2_as_u32(ha[4 * t + 2]), h2_as_u32(hb[4 * t + 2]),
                             h2_as_u32(ha[4 * t + 3]), h2_as_u32(hb[4 * t + 3]), xb.z, xb.w);
              }
            }
          }
        }
      }
    }
  }

  // ---- epilogue --------------------------------------------------------------------
  // acc[mh][0..1]: weight row n_base+g, tokens 8*mh+2c, +1;  acc[mh][2..3]: row n_base+g+8.
  if (p.S == 1) {
    if (n_base < p.N) {
#pragma unroll
      for (int mh = 0; mh < MH; ++mh)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int n = n_base + g + (i >> 1) * 8;
          const int m = 8 * mh + 2 * c + (i & 1);
          if (m < p.M) {
            float v = acc[mh][i];
            if (p.bias) v += __half2float(__ldg(p.bias + n));
            p.y[size_t(m) * p.N + n] = float_to_out16(v, p.bf16);
          }
        }
    }
    return;
  }

  if (n_base < p.N) {
    float* dst = p.partials + size_t(blockIdx.y) * MR * p.N;
#pragma unroll
    for (int mh = 0; mh < MH; ++mh)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int n = n_base + g + (i >> 1) * 8;
        const int m = 8 * mh + 2 * c + (i & 1);
        if (m < p.M) __stcg(dst + size_t(m) * p.N + n, acc[mh][i]);
      }
  }
  __threadfence();
  __syncthreads();
  __shared__ unsigned is_last;
  if (tid == 0) {
    const unsigned ticket = atomicAdd(p.counters + blockIdx.x, 1u);
    is_last = (ticket == unsigned(p.S) - 1u);
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  const int n0 = blockIdx.x * kGemvRows;
  const int ncols = min(kGemvRows, p.N - n0);
  for (int i = tid; i < p.M * kGemvRows; i += blockDim.x) {
    const int m = i / kGemvRows, nn = i - m * kGemvRows;
    if (nn < ncols) {
      const int n = n0 + nn;
      float v = 0.f;
      for (int s = 0; s < p.S; ++s) v += __ldcg(p.partials + (size_t(s) * MR + m) * p.N + n);
      if (p.bias) v += __half2float(__ldg(p.bias + n));
      p.y[size_t(m) * p.N + n] = float_to_out16(v, p.bf16);
    }
  }
  if (tid == 0) p.counters[blockIdx.x] = 0;
}

// Number of K slices for one launch: enough blocks to cover the SMs about twice, a
// slice no longer than 2048 (shared-memory footprint), partial-sum traffic at most a
// quarter of the weight bytes, and a divisor of the number of 128-bit steps.
int gemv_pick_split(int bits, int mrows, int64_t N, int64_t K, int sm_count) {
  const int chunk = (128 / bits) * 4;
  const int nchunks = int(K / chunk);
  const int ntiles = int((N + kGemvRows - 1) / kGemvRows);
  int want = (2 * sm_count + ntiles - 1) / ntiles;
  const int traffic_cap = int(std::max<int64_t>(1, K * bits / (128 * int64_t(mrows))));
  want = std::min(want, traffic_cap);
  want = std::min(want, std::min(nchunks, kGemvMaxSplit));
  const int need = int((K + 2047) / 2048);
  want = std::max(want, need);
  int s = std::max(1, want);
  while (s < nchunks && nchunks % s) ++s;
  if (s > kGemvMaxSplit) {  // fall back to the largest divisor within the limit
    s = kGemvMaxSplit;
    while (s > 1 && nchunks % s) --s;
  }
  return s;
}

size_t gemv_workspace_bytes(int64_t N) {
  return kPartialOffset + size_t(kGemvMaxSplit) * 16 * size_t(N) * sizeof(float);
}

template <int BITS, int MH>
static int launch_gemv(const GemvParams& p, int ntiles, cudaStream_t stream) {
  const size_t smem = size_t(8 * MH) * (p.kslice / 8 + 4) * 16;
  auto kern = gemv_a16_kernel<BITS, MH>;
  static thread_local size_t configured[4] = {0, 0, 0, 0};
  size_t& cfg = configured[(BITS == 4 ? 0 : 2) + (MH - 1)];
  if (smem > 48 * 1024 && smem > cfg) {
    ASRQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    cfg = smem;
  }
  kern<<<dim3(ntiles, p.S), kGemvWarps * 32, smem, stream>>>(p);
  ASRQ_CUDA_TRY(cudaGetLastError());
  return ASRQ_OK;
}

int gemv_a16(int bits, const void* x, const uint8_t* w, const void* scales, const void* zeros,
             const void* bias, void* y, int64_t M, int64_t N, int64_t K, int group_size, int dtype,
             void* workspace, size_t workspace_bytes, int sm_count, cudaStream_t stream) {
  const int chunk = (128 / bits) * 4;
  if (N % 16 || K % chunk || group_size <= 0 || K % group_size || group_size % (128 / bits))
    return fail(ASRQ_ERR_SHAPE,
                "w%da16 gemv: need N%%16==0, K%%%d==0, group_size%%%d==0, K%%group_size==0 "
                "(N=%lld K=%lld g=%d)", bits, chunk, 128 / bits, (long long)N, (long long)K, group_size);
  if (N > int64_t(4096) * kGemvRows || K > (1 << 20))
    return fail(ASRQ_ERR_LIMIT, "w%da16 gemv: N or K too large", bits);
  if (workspace_bytes < gemv_workspace_bytes(N))
    return fail(ASRQ_ERR_WORKSPACE, "w%da16 gemv: workspace %zu < %zu bytes", bits, workspace_bytes,
                gemv_workspace_bytes(N));
  GemvParams p;
  p.w = w;
  p.scales = static_cast<const __half*>(scales);
  p.zeros = static_cast<const __half*>(zeros);
  p.bias = static_cast<const __half*>(bias);
  p.partials = reinterpret_cast<float*>(static_cast<char*>(workspace) + kPartialOffset);
  p.counters = reinterpret_cast<unsigned*>(static_cast<char*>(workspace) + kStatusBytes);
  p.N = int(N);
  p.K = int(K);
  p.group_size = group_size;
  p.groups_per_row = int(K / group_size);
  p.bf16 = dtype == ASRQ_BF16;
  const int ntiles = int((N + kGemvRows - 1) / kGemvRows);
  for (int64_t m0 = 0; m0 < M; m0 += 16) {
    const int mb = int(std::min<int64_t>(16, M - m0));
    const int mh = mb > 8 ? 2 : 1;
    p.x = static_cast<const uint16_t*>(x) + m0 * K;
    p.y = static_cast<uint16_t*>(y) + m0 * N;
    p.M = mb;
    p.S = gemv_pick_split(bits, 8 * mh, N, K, sm_count);
    p.kslice = int(K / p.S);
    int rc;
    if (bits == 4)
      rc = mh == 1 ? launch_gemv<4, 1>(p, ntiles, stream) : launch_gemv<4, 2>(p, ntiles, stream);
    else
      rc = mh == 1 ? launch_gemv<2, 1>(p, ntiles, stream) : launch_gemv<2, 2>(p, ntiles, stream);
    if (rc) return rc;
  }
  return ASRQ_OK;
}

}  // namespace asrq
