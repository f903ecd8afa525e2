// W4A4 prologue: optional online Hadamard rotation + per-token symmetric int4
// quantisation, one warp per token, everything in fp32 registers.
//
// The rotation is the normalised Walsh-Hadamard transform computed as butterflies
// with strides 1, 2, 4, ... K/2 in that order, (a, b) -> (a + b, a - b), followed by
// a division by sqrt(K).  Each output of a stage is a single fp32 add or subtract of
// two values of the previous stage, so the result is bit-identical to any other
// evaluation that keeps the stage order, however the butterflies are spread over
// lanes.  A lane holds V = K/32 consecutive elements: the strides below V are
// register-to-register, the five strides V..16V are warp shuffles.
//
// Quantisation: s = absmax/7 (0 -> 1e-3), q = rint(v/s) with IEEE division and
// round-half-even, packed two's-complement nibbles, even k in the low nibble.
#include "common.cuh"

namespace asrq {

constexpr int kQuantWarps = 4;

__device__ __forceinline__ float in16_to_float(uint16_t b, bool bf16) {
  return bf16 ? bf16_bits_to_float(b) : __half2float(__ushort_as_half(b));
}

__device__ __forceinline__ uint32_t pack8_int4(const float* v, float s) {
  uint32_t w = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float q = rintf(__fdiv_rn(v[i], s));
    q = fminf(fmaxf(q, -7.f), 7.f);
    w |= (uint32_t(int(q)) & 0xFu) << (4 * i);
  }
  return w;
}

template <int V>
__global__ void __launch_bounds__(kQuantWarps * 32)
hadamard_quant_kernel(const uint16_t* __restrict__ x, uint8_t* __restrict__ qa,
                      float* __restrict__ sa, int M, int K, int bf16) {
  const int lane = threadIdx.x & 31;
  const int token = blockIdx.x * kQuantWarps + (threadIdx.x >> 5);
  if (token >= M) return;
  float v[V];
  const uint4* src = reinterpret_cast<const uint4*>(x + size_t(token) * K + lane * V);
#pragma unroll
  for (int i = 0; i < V / 8; ++i) {
    const uint4 u = __ldg(src + i);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      v[8 * i + 2 * j] = in16_to_float(uint16_t(w[j] & 0xffffu), bf16);
      v[8 * i + 2 * j + 1] = in16_to_float(uint16_t(w[j] >> 16), bf16);
    }
  }
  // strides 1 .. V/2: inside the lane
#pragma unroll
  for (int h = 1; h < V; h <<= 1) {
#pragma unroll
    for (int j = 0; j < V; ++j) {
      if ((j & h) == 0) {
        const float a = v[j], b = v[j + h];
        v[j] = a + b;
        v[j + h] = a - b;
      }
    }
  }
  // strides V .. 16V: across lanes
#pragma unroll
  for (int mask = 1; mask < 32; mask <<= 1) {
    const bool upper = (lane & mask) != 0;
#pragma unroll
    for (int j = 0; j < V; ++j) {
      const float o = __shfl_xor_sync(0xffffffffu, v[j], mask);
      v[j] = upper ? (o - v[j]) : (v[j] + o);
    }
  }
  const float root = sqrtf(float(K));
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < V; ++j) {
    v[j] = __fdiv_rn(v[j], root);
    amax = fmaxf(amax, fabsf(v[j]));
  }
#pragma unroll
  for (int mask = 16; mask > 0; mask >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, mask));
  float s = __fdiv_rn(amax, 7.f);
  if (s == 0.f) s = 1e-3f;
  if (lane == 0) sa[token] = s;
  uint32_t* dst = reinterpret_cast<uint32_t*>(qa + size_t(token) * (K / 2) + lane * (V / 2));
  if (V >= 32) {
#pragma unroll
    for (int i = 0; i < V / 32; ++i) {
      uint4 o;
      o.x = pack8_int4(v + 32 * i, s);
      o.y = pack8_int4(v + 32 * i + 8, s);
      o.z = pack8_int4(v + 32 * i + 16, s);
      o.w = pack8_int4(v + 32 * i + 24, s);
      reinterpret_cast<uint4*>(dst)[i] = o;
    }
  } else {
#pragma unroll
    for (int i = 0; i < V / 8; ++i) dst[i] = pack8_int4(v + 8 * i, s);
  }
}

// No rotation: any K that is a multiple of 8.  Two passes over the token (the second
// one hits L1/L2).
__global__ void __launch_bounds__(kQuantWarps * 32)
quant_int4_kernel(const uint16_t* __restrict__ x, uint8_t* __restrict__ qa, float* __restrict__ sa,
                  int M, int K, int bf16) {
  const int lane = threadIdx.x & 31;
  const int token = blockIdx.x * kQuantWarps + (threadIdx.x >> 5);
  if (token >= M) return;
  const uint4* src = reinterpret_cast<const uint4*>(x + size_t(token) * K);
  const int units = K / 8;
  float amax = 0.f;
  for (int i = lane; i < units; i += 32) {
    const uint4 u = __ldg(src + i);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      amax = fmaxf(amax, fabsf(in16_to_float(uint16_t(w[j] & 0xffffu), bf16)));
      amax = fmaxf(amax, fabsf(in16_to_float(uint16_t(w[j] >> 16), bf16)));
    }
  }
#pragma unroll
  for (int mask = 16; mask > 0; mask >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, mask));
  float s = __fdiv_rn(amax, 7.f);
  if (s == 0.f) s = 1e-3f;
  if (lane == 0) sa[token] = s;
  uint32_t* dst = reinterpret_cast<uint32_t*>(qa + size_t(token) * (K / 2));
  for (int i = lane; i < units; i += 32) {
    const uint4 u = __ldg(src + i);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
    float v[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      v[2 * j] = in16_to_float(uint16_t(w[j] & 0xffffu), bf16);
      v[2 * j + 1] = in16_to_float(uint16_t(w[j] >> 16), bf16);
    }
    dst[i] = pack8_int4(v, s);
  }
}

int hadamard_quant_int4(const void* x, uint8_t* qa, float* sa, int64_t M, int64_t K, int hadamard,
                        int dtype, cudaStream_t stream) {
  if (M <= 0) return ASRQ_OK;
  const uint16_t* xp = static_cast<const uint16_t*>(x);
  const int blocks = int((M + kQuantWarps - 1) / kQuantWarps);
  const int bf16 = dtype == ASRQ_BF16;
  if (!hadamard) {
    if (K % 8 || K <= 0) return fail(ASRQ_ERR_SHAPE, "quant_int4: K %% 8 != 0 (K=%lld)", (long long)K);
    quant_int4_kernel<<<blocks, kQuantWarps * 32, 0, stream>>>(xp, qa, sa, int(M), int(K), bf16);
  } else {
    switch (K) {
      case 256: hadamard_quant_kernel<8><<<blocks, kQuantWarps * 32, 0, stream>>>(xp, qa, sa, int(M), int(K), bf16); break;
      case 512: hadamard_quant_kernel<16><<<blocks, kQuantWarps * 32, 0, stream>>>(xp, qa, sa, int(M), int(K), bf16); break;
      case 1024: hadamard_quant_kernel<32><<<blocks, kQuantWarps * 32, 0, stream>>>(xp, qa, sa, int(M), int(K), bf16); break;
      case 2048: hadamard_quant_kernel<64><<<blocks, kQuantWarps * 32, 0, stream>>>(xp, qa, sa, int(M), int(K), bf16); break;
      case 4096: hadamard_quant_kernel<128><<<blocks, kQuantWarps * 32, 0, stream>>>(xp, qa, sa, int(M), int(K), bf16); break;
      default:
        return fail(ASRQ_ERR_SHAPE, "hadamard_quant_int4: K must be 256, 512, 1024, 2048 or 4096 (K=%lld)",
                    (long long)K);
    }
  }
  ASRQ_CUDA_TRY(cudaGetLastError());
  return ASRQ_OK;
}

}  // namespace asrq
