// W4A4 GEMM, register-tile variant (mma.sync.m16n8k32 s8): used for shapes the
// tcgen05 kernel does not take (ragged N tiles, small M) and as its cross-check.
//
// Both operands are packed signed nibbles.  A nibble pair word q is split into
// E = (q << 4) & 0xf0f0f0f0 (even k) and O = q & 0xf0f0f0f0 (odd k): each byte is
// then 16x the signed value, so a product is 256x the true one and the exact group
// sum is (acc >> 8).  The k order inside a lane's 32-k span is the same for both
// operands, which is all a contraction needs.
//
// Per 128-k step (one weight group) the int32 tile is scaled by sW[n, group] and
// added to an fp32 running sum; the per-token scale and the bias come last.
#include "common.cuh"

namespace asrq {

struct W4A4Params {
  const uint8_t* qa;
  const float* sa;
  const uint8_t* qw;
  const __half* sw;
  const __half* bias;
  uint16_t* y;
  int32_t* acc_dump;
  int M, N, K, group_size, groups, bf16;
};

__device__ __forceinline__ void mma_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// block: 4 warps as 2(m) x 2(n); warp tile 32(m) x 32(n); block tile 64 x 64.
__global__ void __launch_bounds__(128) w4a4_mma_kernel(const W4A4Params p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, c = lane & 3;
  const int m_base = blockIdx.y * 64 + (warp >> 1) * 32;
  const int n_base = blockIdx.x * 64 + (warp & 1) * 32;
  const size_t row_bytes = size_t(p.K) / 2;
  const int steps_per_group = p.group_size / 128;

  float accf[2][4][4];
  int acc[2][4][4];
#pragma unroll
  for (int a = 0; a < 2; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        accf[a][b][i] = 0.f;
        acc[a][b][i] = 0;
      }

  const int nsteps = p.K / 128;
  for (int step = 0; step < nsteps; ++step) {
    const size_t koff = size_t(step) * 64 + c * 16;  // bytes
    uint4 ar[2][2], br[4];
#pragma unroll
    for (int f = 0; f < 2; ++f)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int m = m_base + 16 * f + 8 * h + g;
        ar[f][h] = m < p.M ? __ldg(reinterpret_cast<const uint4*>(p.qa + m * row_bytes + koff))
                           : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
    for (int f = 0; f < 4; ++f) {
      const int n = n_base + 8 * f + g;
      br[f] = __ldg(reinterpret_cast<const uint4*>(p.qw + n * row_bytes + koff));
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t ae[2][2], ao[2][2], be[4], bo[4];
#pragma unroll
      for (int f = 0; f < 2; ++f)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const uint32_t q = (&ar[f][h].x)[j];
          ae[f][h] = (q << 4) & 0xf0f0f0f0u;
          ao[f][h] = q & 0xf0f0f0f0u;
        }
#pragma unroll
      for (int f = 0; f < 4; ++f) {
        const uint32_t q = (&br[f].x)[j];
        be[f] = (q << 4) & 0xf0f0f0f0u;
        bo[f] = q & 0xf0f0f0f0u;
      }
#pragma unroll
      for (int fm = 0; fm < 2; ++fm)
#pragma unroll
        for (int fn = 0; fn < 4; ++fn)
          mma_s8(acc[fm][fn], ae[fm][0], ae[fm][1], ao[fm][0], ao[fm][1], be[fn], bo[fn]);
    }
    if ((step + 1) % steps_per_group == 0) {
      const int gi = step / steps_per_group;
#pragma unroll
      for (int fn = 0; fn < 4; ++fn) {
        const int n0 = n_base + 8 * fn + 2 * c;
        const float s0 = __half2float(__ldg(p.sw + size_t(n0) * p.groups + gi));
        const float s1 = __half2float(__ldg(p.sw + size_t(n0 + 1) * p.groups + gi));
#pragma unroll
        for (int fm = 0; fm < 2; ++fm)
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int v = acc[fm][fn][i] >> 8;
            accf[fm][fn][i] += float(v) * ((i & 1) ? s1 : s0);
            if (p.acc_dump) {
              const int m = m_base + 16 * fm + 8 * (i >> 1) + g;
              if (m < p.M) p.acc_dump[(size_t(m) * p.N + n0 + (i & 1)) * p.groups + gi] = v;
            }
            acc[fm][fn][i] = 0;
          }
      }
    }
  }
#pragma unroll
  for (int fm = 0; fm < 2; ++fm)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int m = m_base + 16 * fm + 8 * h + g;
      if (m >= p.M) continue;
      const float s = __ldg(p.sa + m);
#pragma unroll
      for (int fn = 0; fn < 4; ++fn) {
        const int n0 = n_base + 8 * fn + 2 * c;
        float v0 = accf[fm][fn][2 * h] * s, v1 = accf[fm][fn][2 * h + 1] * s;
        if (p.bias) {
          v0 += __half2float(__ldg(p.bias + n0));
          v1 += __half2float(__ldg(p.bias + n0 + 1));
        }
        const uint32_t o = uint32_t(float_to_out16(v0, p.bf16)) | (uint32_t(float_to_out16(v1, p.bf16)) << 16);
        *reinterpret_cast<uint32_t*>(p.y + size_t(m) * p.N + n0) = o;
      }
    }
}

int w4a4_gemm_mma(const uint8_t* qa, const float* sa, const uint8_t* qw, const void* sw, const void* bias,
                  void* y, int32_t* acc_dump, int64_t M, int64_t N, int64_t K, int group_size, int dtype,
                  cudaStream_t stream) {
  if (group_size <= 0 || N % 64 || K % 128 || group_size % 128 || K % group_size)
    return fail(ASRQ_ERR_SHAPE,
                "w4a4 gemm: need N%%64==0, K%%128==0, group_size%%128==0, K%%group_size==0 "
                "(N=%lld K=%lld g=%d)", (long long)N, (long long)K, group_size);
  if (M <= 0) return ASRQ_OK;
  W4A4Params p;
  p.qa = qa; p.sa = sa; p.qw = qw;
  p.sw = static_cast<const __half*>(sw);
  p.bias = static_cast<const __half*>(bias);
  p.y = static_cast<uint16_t*>(y);
  p.acc_dump = acc_dump;
  p.M = int(M); p.N = int(N); p.K = int(K);
  p.group_size = group_size;
  p.groups = int(K / group_size);
  p.bf16 = dtype == ASRQ_BF16;
  dim3 grid(unsigned(N / 64), unsigned((M + 63) / 64));
  w4a4_mma_kernel<<<grid, 128, 0, stream>>>(p);
  ASRQ_CUDA_TRY(cudaGetLastError());
  return ASRQ_OK;
}

}  // namespace asrq
