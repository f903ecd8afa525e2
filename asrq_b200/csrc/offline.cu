// Model preparation on the device: the two offline steps between a float checkpoint and the packed buffers.
//
//   rtn_pack        round-to-nearest codes on the reference's uniform grid (asrq/quantizers/base.py:58-77,
//                   asrq/quantizers/rtn.py:32-46) and their packing (asrq/core/linear.py:43-52 for the LinearQ layout,
//                   asrq/matmulq/test.py:141-142 for signed nibbles), one warp per (row, group).  Every operation is
//                   rounded to the weight's own type, as the reference's tensor expressions round it, so the codes,
//                   scales and zeros are the bits the host-side packer (asrq_b200/packing.py) produces.
//   hadamard_fold   W' = hadU(W) along K in fp32 (the butterfly order of matmul_hadU,
//                   asrq/transforms/rotation/hadamard_utils.py:64-81), one block per row: the rotation a W4A4 layer
//                   applies online to its input, folded into the weight before it is quantised.
#include <algorithm>

#include "common.cuh"

namespace asrq {

namespace {

enum { kT16 = 0, kTBf16 = 1, kT32 = 2 };

// a value of the weight's type, held as float; rnd() rounds an fp32 intermediate back to that type
template <int T>
__device__ __forceinline__ float load_as_float(const void* p, size_t i) {
  if (T == kT32) return static_cast<const float*>(p)[i];
  const uint16_t b = static_cast<const uint16_t*>(p)[i];
  return T == kTBf16 ? bf16_bits_to_float(b) : __half2float(__ushort_as_half(b));
}
template <int T>
__device__ __forceinline__ float rnd(float v) {
  if (T == kT32) return v;
  if (T == kTBf16) return __bfloat162float(__float2bfloat16_rn(v));
  return __half2float(__float2half_rn(v));
}

// layout 0: unsigned codes in LinearQ's byte layout plus fp16 scales and zeros (a symmetric grid is shifted by
// 2^(bits-1) with zeros = -2^(bits-1) * scale); layout 1: two's-complement nibbles (symmetric, 4 bits), scales only
template <int T, int BITS>
__global__ void __launch_bounds__(256)
rtn_pack_kernel(const void* __restrict__ w, uint8_t* __restrict__ out, __half* __restrict__ scales, __half* __restrict__ zeros,
                int64_t n_groups_total, int K, int g, int symmetric, int layout) {
  const int lane = threadIdx.x & 31;
  const int64_t grp = int64_t(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (grp >= n_groups_total) return;
  const int gpr = K / g;
  const int64_t row = grp / gpr;
  const int gi = int(grp - row * gpr);
  const size_t base = size_t(row) * K + size_t(gi) * g;
  float mx = -INFINITY, mn = INFINITY;
  for (int e = lane; e < g; e += 32) {
    const float v = load_as_float<T>(w, base + e);
    mx = fmaxf(mx, symmetric ? fabsf(v) : v);
    mn = fminf(mn, v);
  }
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) {
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
  }
  const float maxq = symmetric ? float((1 << (BITS - 1)) - 1) : float((1 << BITS) - 1);
  const float minq = symmetric ? -maxq : 0.f;
  float scale, zero;
  if (symmetric) {
    scale = rnd<T>(mx / maxq);
    zero = 0.f;
  } else {
    scale = rnd<T>(rnd<T>(mx - mn) / maxq);
    zero = mn;
  }
  if (lane == 0) {
    const size_t si = size_t(row) * gpr + gi;
    scales[si] = __float2half_rn(scale);
    if (layout == 0) zeros[si] = __float2half_rn(symmetric ? rnd<T>(-float(1 << (BITS - 1)) * scale) : zero);
  }
  constexpr int PER_BYTE = 8 / BITS;
  const int off = (symmetric && layout == 0) ? (1 << (BITS - 1)) : 0;
  // eight consecutive elements per lane and step: 4 (4-bit) or 2 (2-bit) bytes
  for (int e0 = lane * 8; e0 < g; e0 += 256) {
    uint32_t packed = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float v = load_as_float<T>(w, base + e0 + j);
      float q = symmetric ? rnd<T>(v / scale) : rnd<T>(rnd<T>(v - zero) / scale);
      q = fminf(fmaxf(rintf(q), minq), maxq);
      if (!(q == q)) q = 0.f;  // 0/0 in a group of zeros: the code is arbitrary (it decodes to the same value), zero here
      const int c = (int(q) + off) & ((1 << BITS) - 1);
      packed |= uint32_t(c) << (BITS * j);
    }
    uint8_t* o = out + (base + e0) / PER_BYTE;
    if (BITS == 4) {
      *reinterpret_cast<uint32_t*>(o) = packed;
    } else {
      *reinterpret_cast<uint16_t*>(o) = uint16_t(packed);
    }
  }
}

// one block per row; K floats in shared memory, log2(K) butterfly stages
template <int T>
__global__ void __launch_bounds__(256)
hadamard_fold_kernel(const void* __restrict__ w, float* __restrict__ out, int K) {
  extern __shared__ float row[];
  const size_t base = size_t(blockIdx.x) * K;
  for (int e = threadIdx.x; e < K; e += blockDim.x) row[e] = load_as_float<T>(w, base + e);
  __syncthreads();
  for (int h = 1; h < K; h <<= 1) {
    for (int p = threadIdx.x; p < K / 2; p += blockDim.x) {
      const int j = ((p / h) * 2 * h) + (p % h);  // pair (j, j + h)
      const float a = row[j], b = row[j + h];
      row[j] = a + b;
      row[j + h] = a - b;
    }
    __syncthreads();
  }
  const float s = sqrtf(float(K));
  for (int e = threadIdx.x; e < K; e += blockDim.x) out[base + e] = row[e] / s;
}

}  // namespace

int rtn_pack(const void* w, int w_dtype, int bits, int group_size, int symmetric, int layout, uint8_t* weight, void* scales,
             void* zeros, int64_t N, int64_t K, cudaStream_t stream) {
  const int64_t groups = N * (K / group_size);
  const unsigned blocks = unsigned((groups + 7) / 8);
  auto sp = static_cast<__half*>(scales), zp = static_cast<__half*>(zeros);
#define ASRQ_RTN_LAUNCH(T, B) \
  rtn_pack_kernel<T, B><<<blocks, 256, 0, stream>>>(w, weight, sp, zp, groups, int(K), group_size, symmetric, layout)
  if (bits == 4) {
    if (w_dtype == kT16) ASRQ_RTN_LAUNCH(kT16, 4);
    else if (w_dtype == kTBf16) ASRQ_RTN_LAUNCH(kTBf16, 4);
    else ASRQ_RTN_LAUNCH(kT32, 4);
  } else {
    if (w_dtype == kT16) ASRQ_RTN_LAUNCH(kT16, 2);
    else if (w_dtype == kTBf16) ASRQ_RTN_LAUNCH(kTBf16, 2);
    else ASRQ_RTN_LAUNCH(kT32, 2);
  }
#undef ASRQ_RTN_LAUNCH
  ASRQ_CUDA_TRY(cudaGetLastError());
  return ASRQ_OK;
}

int hadamard_fold(const void* w, int w_dtype, float* out, int64_t N, int64_t K, cudaStream_t stream) {
  const size_t smem = size_t(K) * sizeof(float);
  if (w_dtype == kT16) hadamard_fold_kernel<kT16><<<unsigned(N), 256, smem, stream>>>(w, out, int(K));
  else if (w_dtype == kTBf16) hadamard_fold_kernel<kTBf16><<<unsigned(N), 256, smem, stream>>>(w, out, int(K));
  else hadamard_fold_kernel<kT32><<<unsigned(N), 256, smem, stream>>>(w, out, int(K));
  ASRQ_CUDA_TRY(cudaGetLastError());
  return ASRQ_OK;
}

}  // namespace asrq
