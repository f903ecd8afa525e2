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

// Per-token scale and its reciprocal.
struct QScale {
  float s, inv;
};

// rint(v / s) with IEEE division, bit for bit, without a division per element: r = v * (1/s) is
// within 1.3e-6 of the correctly rounded quotient (|r| <= 7), so both round to the same integer
// unless r lies within 1e-5 of a tie; only then is the true quotient computed.  Rounding to
// nearest-even is done by adding 1.5 * 2^23, which also leaves the two's-complement code in the
// low mantissa bits, so there is no float->int conversion either.  |code| <= 7 by construction
// (s = absmax / 7), as in the reference formula, which has no clamp.
__device__ __forceinline__ int quant1(float v, QScale qs) {
  const float magic = 12582912.f;
  const float r = __fmul_rn(v, qs.inv);
  float t = __fadd_rn(r, magic);
  const float d = fabsf(__fsub_rn(r, __fsub_rn(t, magic)));
  if (d > 0.49999f) t = __fadd_rn(rintf(__fdiv_rn(v, qs.s)), magic);
  return __float_as_int(t) - 0x4B400000;
}

__device__ __forceinline__ QScale make_qscale(float amax) {
  QScale q;
  q.s = __fdiv_rn(amax, 7.f);
  if (q.s == 0.f) q.s = 1e-3f;
  q.inv = __fdiv_rn(1.f, q.s);
  return q;
}

__device__ __forceinline__ uint32_t pack8_int4(const float* v, QScale s) {
  uint32_t w = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) w |= (uint32_t(quant1(v[i], s)) & 0xFu) << (4 * i);
  return w;
}

// Four codes as int8 bytes holding 16x the value (the operand format of the tcgen05 W4A4 GEMM).
__device__ __forceinline__ uint32_t pack4_int8x16(const float* v, QScale s) {
  uint32_t w = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) w |= ((uint32_t(quant1(v[i], s)) << 4) & 0xFFu) << (8 * i);
  return w;
}

// OUT = 0: packed nibbles (K/2 bytes per token); OUT = 1: int8 holding 16*q (K bytes per token).
template <int V, int OUT>
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
  const QScale s = make_qscale(amax);
  if (lane == 0) sa[token] = s.s;
  if (OUT == 1) {
    uint32_t* d8 = reinterpret_cast<uint32_t*>(qa + size_t(token) * K + lane * V);
    if (V >= 16) {
#pragma unroll
      for (int i = 0; i < V / 16; ++i)
        reinterpret_cast<uint4*>(d8)[i] = make_uint4(pack4_int8x16(v + 16 * i, s), pack4_int8x16(v + 16 * i + 4, s),
                                                     pack4_int8x16(v + 16 * i + 8, s), pack4_int8x16(v + 16 * i + 12, s));
    } else {
#pragma unroll
      for (int i = 0; i < V / 4; ++i) d8[i] = pack4_int8x16(v + 4 * i, s);
    }
    return;
  }
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
template <int OUT>
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
  const QScale s = make_qscale(amax);
  if (lane == 0) sa[token] = s.s;
  uint32_t* dst = reinterpret_cast<uint32_t*>(qa + size_t(token) * (OUT == 1 ? K : K / 2));
  for (int i = lane; i < units; i += 32) {
    const uint4 u = __ldg(src + i);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
    float v[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      v[2 * j] = in16_to_float(uint16_t(w[j] & 0xffffu), bf16);
      v[2 * j + 1] = in16_to_float(uint16_t(w[j] >> 16), bf16);
    }
    if (OUT == 1) {
      reinterpret_cast<uint2*>(dst)[i] = make_uint2(pack4_int8x16(v, s), pack4_int8x16(v + 4, s));
    } else {
      dst[i] = pack8_int4(v, s);
    }
  }
}

// K = 4096 specialisation.  The five butterfly strides that cross lanes in the generic kernel
// (640 shuffles per lane) are replaced by one transpose through shared memory:
//   phase A  lane L owns elements L*128 .. L*128+127 (index bits 0-6 private): strides 1..64;
//   phase B  lane L owns elements o*128 + L*4 + c, o = 0..31, c = 0..3 (bits 0-1 and 7-11 private):
//            strides 128..2048, and the four consecutive elements pack into one store.
// A lane's private elements live in a per-warp shared-memory array of 16-byte slots,
// slot(owner, g) = g*32 + (owner ^ g) for the four elements 4g..4g+3: conflict-free both when every
// lane touches its own group g and when lane L reads group L of every owner (the transpose).
// Phase A and the quantisation are ROLLED loops over small register tiles: a fully unrolled
// version (3600 instructions of straight-line code per warp) measured 57 us for 6000 tokens with
// "no instruction" (instruction-fetch) as its dominant stall.
constexpr int kHad4096Warps = 3;
constexpr int kHad4096WarpBytes = 8192 + 16384;  // fp16 staging + fp32 private array

template <int OUT>
__global__ void __launch_bounds__(kHad4096Warps * 32)
hadamard4096_quant_kernel(const uint16_t* __restrict__ x, uint8_t* __restrict__ qa, float* __restrict__ sa,
                          int M, int bf16) {
  extern __shared__ uint4 smem4[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int token = blockIdx.x * kHad4096Warps + warp;
  if (token >= M) return;  // warp-uniform; only warp-level synchronisation below
  uint4* stg = smem4 + warp * (kHad4096WarpBytes / 16);  // 512 slots of 8 fp16
  float4* pv = reinterpret_cast<float4*>(stg + 512);     // 1024 slots of 4 fp32
  // coalesced global load, each 16-byte unit handed to the lane that owns it in phase A
  const uint4* src = reinterpret_cast<const uint4*>(x + size_t(token) * 4096);
#pragma unroll
  for (int jj = 0; jj < 16; ++jj) {
    const int u = jj * 32 + lane;
    const int owner = u >> 4, j = u & 15;
    stg[owner * 16 + (j ^ (owner & 15))] = __ldg(src + u);
  }
  __syncwarp();
  // phase A1: strides 1, 2, 4, 8 on blocks of 16 elements
#pragma unroll 1
  for (int b = 0; b < 8; ++b) {
    float v[16];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint4 u = stg[lane * 16 + ((2 * b + h) ^ (lane & 15))];
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        v[8 * h + 2 * e] = in16_to_float(uint16_t(w[e] & 0xffffu), bf16);
        v[8 * h + 2 * e + 1] = in16_to_float(uint16_t(w[e] >> 16), bf16);
      }
    }
#pragma unroll
    for (int h = 1; h < 16; h <<= 1)
#pragma unroll
      for (int j = 0; j < 16; ++j)
        if ((j & h) == 0) {
          const float a = v[j], c = v[j + h];
          v[j] = a + c;
          v[j + h] = a - c;
        }
#pragma unroll
    for (int gq = 0; gq < 4; ++gq) {
      const int g = 4 * b + gq;
      pv[g * 32 + (lane ^ g)] = make_float4(v[4 * gq], v[4 * gq + 1], v[4 * gq + 2], v[4 * gq + 3]);
    }
  }
  // phase A2: strides 16, 32, 64 = bits 2, 3, 4 of the group index g
#pragma unroll 1
  for (int gl = 0; gl < 4; ++gl) {
    float4 w[8];
#pragma unroll
    for (int m = 0; m < 8; ++m) w[m] = pv[(gl + 4 * m) * 32 + (lane ^ (gl + 4 * m))];
#pragma unroll
    for (int h = 1; h < 8; h <<= 1)
#pragma unroll
      for (int m = 0; m < 8; ++m)
        if ((m & h) == 0) {
          const float4 a = w[m], c = w[m + h];
          w[m] = make_float4(a.x + c.x, a.y + c.y, a.z + c.z, a.w + c.w);
          w[m + h] = make_float4(a.x - c.x, a.y - c.y, a.z - c.z, a.w - c.w);
        }
#pragma unroll
    for (int m = 0; m < 8; ++m) pv[(gl + 4 * m) * 32 + (lane ^ (gl + 4 * m))] = w[m];
  }
  __syncwarp();
  // phase B: transpose (lane L takes group L of every owner o), strides 128..2048 over o, in registers
  float4 z[32];
#pragma unroll
  for (int o = 0; o < 32; ++o) z[o] = pv[lane * 32 + (o ^ lane)];
#pragma unroll
  for (int h = 1; h < 32; h <<= 1)
#pragma unroll
    for (int o = 0; o < 32; ++o)
      if ((o & h) == 0) {
        const float4 a = z[o], c = z[o + h];
        z[o] = make_float4(a.x + c.x, a.y + c.y, a.z + c.z, a.w + c.w);
        z[o + h] = make_float4(a.x - c.x, a.y - c.y, a.z - c.z, a.w - c.w);
      }
  float amax = 0.f;
  __syncwarp();  // every lane has read the transposed view before the slots are reused below
#pragma unroll
  for (int o = 0; o < 32; ++o) {
    // / sqrt(4096): exact, same bits as the division
    z[o] = make_float4(z[o].x * 0.015625f, z[o].y * 0.015625f, z[o].z * 0.015625f, z[o].w * 0.015625f);
    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(z[o].x), fabsf(z[o].y)), fmaxf(fabsf(z[o].z), fabsf(z[o].w))));
    pv[o * 32 + lane] = z[o];  // lane-private, conflict-free: parked for the rolled quantisation loop
  }
#pragma unroll
  for (int mask = 16; mask > 0; mask >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, mask));
  const QScale s = make_qscale(amax);
  if (lane == 0) sa[token] = s.s;
  // element index of (o, lane, c) is o*128 + lane*4 + c: one 32-bit (int8) or 16-bit (packed) store per o
  uint32_t* d8 = reinterpret_cast<uint32_t*>(qa + size_t(token) * 4096);
  uint16_t* d4 = reinterpret_cast<uint16_t*>(qa + size_t(token) * 2048);
#pragma unroll 4
  for (int o = 0; o < 32; ++o) {
    const float4 f = pv[o * 32 + lane];
    const float v4[4] = {f.x, f.y, f.z, f.w};
    if (OUT == 1) {
      d8[o * 32 + lane] = pack4_int8x16(v4, s);
    } else {
      uint32_t w = 0;
#pragma unroll
      for (int c = 0; c < 4; ++c) w |= (uint32_t(quant1(v4[c], s)) & 0xFu) << (4 * c);
      d4[o * 32 + lane] = uint16_t(w);
    }
  }
}

template <int OUT>
static int launch_quant(const uint16_t* xp, uint8_t* qa, float* sa, int64_t M, int64_t K, int hadamard, int bf16,
                        cudaStream_t stream) {
  const int blocks = int((M + kQuantWarps - 1) / kQuantWarps);
  const int thr = kQuantWarps * 32;
  if (!hadamard) {
    if (K % 8 || K <= 0) return fail(ASRQ_ERR_SHAPE, "quant_int4: K %% 8 != 0 (K=%lld)", (long long)K);
    quant_int4_kernel<OUT><<<blocks, thr, 0, stream>>>(xp, qa, sa, int(M), int(K), bf16);
  } else {
    switch (K) {
      case 256: hadamard_quant_kernel<8, OUT><<<blocks, thr, 0, stream>>>(xp, qa, sa, int(M), int(K), bf16); break;
      case 512: hadamard_quant_kernel<16, OUT><<<blocks, thr, 0, stream>>>(xp, qa, sa, int(M), int(K), bf16); break;
      case 1024: hadamard_quant_kernel<32, OUT><<<blocks, thr, 0, stream>>>(xp, qa, sa, int(M), int(K), bf16); break;
      case 2048: hadamard_quant_kernel<64, OUT><<<blocks, thr, 0, stream>>>(xp, qa, sa, int(M), int(K), bf16); break;
      case 4096: {
        const int smem = kHad4096Warps * kHad4096WarpBytes;
        ASRQ_CUDA_TRY(cudaFuncSetAttribute(hadamard4096_quant_kernel<OUT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        hadamard4096_quant_kernel<OUT><<<int((M + kHad4096Warps - 1) / kHad4096Warps), kHad4096Warps * 32, smem, stream>>>(
            xp, qa, sa, int(M), bf16);
        break;
      }
      default:
        return fail(ASRQ_ERR_SHAPE, "hadamard_quant_int4: K must be 256, 512, 1024, 2048 or 4096 (K=%lld)",
                    (long long)K);
    }
  }
  ASRQ_CUDA_TRY(cudaGetLastError());
  return ASRQ_OK;
}

// out_int8 = 0: qa receives packed nibbles (M x K/2); 1: int8 holding 16*q (M x K).
int hadamard_quant_int4(const void* x, uint8_t* qa, float* sa, int64_t M, int64_t K, int hadamard, int dtype,
                        int out_int8, cudaStream_t stream) {
  if (M <= 0) return ASRQ_OK;
  const uint16_t* xp = static_cast<const uint16_t*>(x);
  const int bf16 = dtype == ASRQ_BF16;
  return out_int8 ? launch_quant<1>(xp, qa, sa, M, K, hadamard, bf16, stream)
                  : launch_quant<0>(xp, qa, sa, M, K, hadamard, bf16, stream);
}

}  // namespace asrq
