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
#include <cuda_fp8.h>

#include "common.cuh"

namespace asrq {

int ensure_dynamic_smem(const void* kernel, size_t bytes);

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
// Four codes as FP8 e4m3 bytes holding the value itself (the operand format of the kind::f8f6f4 GEMM).
__device__ __forceinline__ uint32_t e4m3x2(float a, float b) {
  return uint32_t(__nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3));
}
__device__ __forceinline__ uint32_t pack4_e4m3(const float* v, QScale s) {
  return e4m3x2(float(quant1(v[0], s)), float(quant1(v[1], s))) |
         (e4m3x2(float(quant1(v[2], s)), float(quant1(v[3], s))) << 16);
}
template <int OUT>
__device__ __forceinline__ uint32_t pack4_operand(const float* v, QScale s) {
  return OUT == 2 ? pack4_e4m3(v, s) : pack4_int8x16(v, s);
}

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
  if (OUT >= 1) {
    uint32_t* d8 = reinterpret_cast<uint32_t*>(qa + size_t(token) * K + lane * V);
    if (V >= 16) {
#pragma unroll
      for (int i = 0; i < V / 16; ++i)
        reinterpret_cast<uint4*>(d8)[i] = make_uint4(pack4_operand<OUT>(v + 16 * i, s), pack4_operand<OUT>(v + 16 * i + 4, s),
                                                     pack4_operand<OUT>(v + 16 * i + 8, s), pack4_operand<OUT>(v + 16 * i + 12, s));
    } else {
#pragma unroll
      for (int i = 0; i < V / 4; ++i) d8[i] = pack4_operand<OUT>(v + 4 * i, s);
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
  uint32_t* dst = reinterpret_cast<uint32_t*>(qa + size_t(token) * (OUT >= 1 ? K : K / 2));
  for (int i = lane; i < units; i += 32) {
    const uint4 u = __ldg(src + i);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
    float v[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      v[2 * j] = in16_to_float(uint16_t(w[j] & 0xffffu), bf16);
      v[2 * j + 1] = in16_to_float(uint16_t(w[j] >> 16), bf16);
    }
    if (OUT >= 1) {
      reinterpret_cast<uint2*>(dst)[i] = make_uint2(pack4_operand<OUT>(v, s), pack4_operand<OUT>(v + 4, s));
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
// A lane's 128 values live in registers as 64 pairs of neighbouring elements (e_2j, e_2j+1), in
// both phases, so every butterfly except stride 1 is one packed fp32 add and one packed fp32
// subtract (add.f32x2 / fma.f32x2) on two pairs.  The transpose goes through a per-warp
// shared-memory array of 16-byte slots, slot(owner, g) = g*32 + (owner ^ g) for the four elements
// 4g..4g+3: conflict-free both when every lane writes its own groups and when lane L reads group L
// of every owner.
// The division by sqrt(4096) = 64 is exact and is applied to the scale only: rint((v/64) / (s/64))
// is rint(v/s) bit for bit.
// Quantisation without a division per element: t_lo = fma(v, inv_lo, magic), t_hi = fma(v, inv_hi,
// magic) with inv_lo < 1/s < inv_hi (2^-22 apart) bracket the exact quotient, and adding 1.5*2^23
// rounds to nearest-even and leaves the two's-complement code in the low mantissa bits; where the
// two agree (all but a few elements in a million) that is rint(v/s); where they differ the true
// quotient is computed.
constexpr int kHad4096Warps = 3;
constexpr int kHad4096WarpBytes = 16384;  // fp32 transpose array; the fp16 staging area is overlaid on its first half

__device__ __forceinline__ float2 sub2(float2 a, float2 c) { return __ffma2_rn(c, make_float2(-1.f, -1.f), a); }

// The rare path of quant4_bytes, out of line so that its 32 call sites do not double the size of the
// kernel (inlined, the kernel was 66 KB of code against 41 KB and took 31 us against 24.5 us for 6000
// tokens: its hot path is ~2000 instructions of straight-line code per token, fetched once per warp):
// IEEE division and round-half-even, as magic + code.
__device__ __noinline__ float4 quant4_exact(float2 v01, float2 v23, float s) {
  return make_float4(__fadd_rn(rintf(__fdiv_rn(v01.x, s)), 12582912.f), __fadd_rn(rintf(__fdiv_rn(v01.y, s)), 12582912.f),
                     __fadd_rn(rintf(__fdiv_rn(v23.x, s)), 12582912.f), __fadd_rn(rintf(__fdiv_rn(v23.y, s)), 12582912.f));
}

// codes of four values: OUT 0 and 1 as bytes b0..b3 = low byte of each t (t = magic + code), OUT 2 as e4m3 bytes
template <int OUT>
__device__ __forceinline__ uint32_t quant4_bytes(float2 v01, float2 v23, float2 inv_lo, float2 inv_hi, float s) {
  const float2 magic = make_float2(12582912.f, 12582912.f);
  float2 a = __ffma2_rn(v01, inv_lo, magic), b = __ffma2_rn(v23, inv_lo, magic);
  const float2 a2 = __ffma2_rn(v01, inv_hi, magic), b2 = __ffma2_rn(v23, inv_hi, magic);
  const uint32_t diff = (__float_as_uint(a.x) ^ __float_as_uint(a2.x)) | (__float_as_uint(a.y) ^ __float_as_uint(a2.y)) |
                        (__float_as_uint(b.x) ^ __float_as_uint(b2.x)) | (__float_as_uint(b.y) ^ __float_as_uint(b2.y));
  if (diff != 0) {  // an element within 4e-6 of a rounding boundary: IEEE division
    const float4 e = quant4_exact(v01, v23, s);
    a = make_float2(e.x, e.y);
    b = make_float2(e.z, e.w);
  }
  if (OUT == 2) {
    const float2 nm = make_float2(-12582912.f, -12582912.f);
    a = __fadd2_rn(a, nm);  // exact: the code as a float
    b = __fadd2_rn(b, nm);
    return e4m3x2(a.x, a.y) | (e4m3x2(b.x, b.y) << 16);
  }
  const uint32_t p01 = prmt(__float_as_uint(a.x), __float_as_uint(a.y), 0x0040u);
  const uint32_t p23 = prmt(__float_as_uint(b.x), __float_as_uint(b.y), 0x0040u);
  return prmt(p01, p23, 0x5410u);
}

template <int OUT, bool BF16>
__global__ void __launch_bounds__(kHad4096Warps * 32, 3)
hadamard4096_quant_kernel(const uint16_t* __restrict__ x, uint8_t* __restrict__ qa, float* __restrict__ sa, int M) {
  extern __shared__ uint4 smem4[];
  // A GEMM launched behind this kernel with programmatic stream serialisation may be scheduled once
  // every block of this grid has started, and set itself up on SMs the last wave leaves idle; it
  // orders itself with griddepcontrol.wait before it touches this kernel's output.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int token = blockIdx.x * kHad4096Warps + warp;
  if (token >= M) return;  // warp-uniform; only warp-level synchronisation below
  uint4* stg = smem4 + warp * (kHad4096WarpBytes / 16);  // 512 slots of 8 fp16, dead once phase A has loaded them
  float4* pv = reinterpret_cast<float4*>(stg);           // 1024 slots of 4 fp32
  // coalesced global load, each 16-byte unit handed to the lane that owns it in phase A
  const uint4* src = reinterpret_cast<const uint4*>(x + size_t(token) * 4096);
#pragma unroll
  for (int jj = 0; jj < 16; ++jj) {
    const int u = jj * 32 + lane;
    const int owner = u >> 4, j = u & 15;
    stg[owner * 16 + (j ^ (owner & 15))] = __ldg(src + u);
  }
  __syncwarp();
  // phase A: 64 pairs (e_2j, e_2j+1) of this lane's 128 consecutive elements
  float2 P[64];
#pragma unroll
  for (int u = 0; u < 16; ++u) {
    const uint4 q = stg[lane * 16 + (u ^ (lane & 15))];
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int e = 0; e < 4; ++e)
      P[4 * u + e] = BF16 ? make_float2(__uint_as_float(w[e] << 16), __uint_as_float(w[e] & 0xffff0000u))
                          : __half22float2(u32_as_h2(w[e]));
  }
  __syncwarp();  // every lane has read its staging row: pv may overwrite the area
#pragma unroll
  for (int j = 0; j < 64; ++j) {  // stride 1: inside the pair
    const float a = P[j].x, c = P[j].y;
    P[j] = make_float2(a + c, a - c);
  }
#pragma unroll
  for (int h = 1; h < 64; h <<= 1)  // strides 2..64: pair j with pair j + h
#pragma unroll
    for (int j = 0; j < 64; ++j)
      if ((j & h) == 0) {
        const float2 a = P[j], c = P[j + h];
        P[j] = __fadd2_rn(a, c);
        P[j + h] = sub2(a, c);
      }
#pragma unroll
  for (int g = 0; g < 32; ++g) pv[g * 32 + (lane ^ g)] = make_float4(P[2 * g].x, P[2 * g].y, P[2 * g + 1].x, P[2 * g + 1].y);
  __syncwarp();
  // phase B: transpose (lane L takes group L of every owner o), strides 128..2048 over o
#pragma unroll
  for (int o = 0; o < 32; ++o) {
    const float4 z = pv[lane * 32 + (o ^ lane)];
    P[2 * o] = make_float2(z.x, z.y);
    P[2 * o + 1] = make_float2(z.z, z.w);
  }
#pragma unroll
  for (int h = 2; h < 64; h <<= 1)
#pragma unroll
    for (int j = 0; j < 64; ++j)
      if ((j & h) == 0) {
        const float2 a = P[j], c = P[j + h];
        P[j] = __fadd2_rn(a, c);
        P[j + h] = sub2(a, c);
      }
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 64; ++j) amax = fmaxf(amax, fmaxf(fabsf(P[j].x), fabsf(P[j].y)));
#pragma unroll
  for (int mask = 16; mask > 0; mask >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, mask));
  // scale of the unnormalised values; the token's scale is that / 64 (exact)
  float s = __fdiv_rn(amax, 7.f);
  const bool zero = s == 0.f;
  if (lane == 0) sa[token] = zero ? 1e-3f : s * 0.015625f;
  if (zero) s = 1.f;  // every value is 0: any scale gives code 0
  const float inv = __fdiv_rn(1.f, s);
  const float il = inv * (1.f - 2.384185791015625e-07f), ih = inv * (1.f + 2.384185791015625e-07f);  // 2^-22
  const float2 inv_lo = make_float2(il, il), inv_hi = make_float2(ih, ih);
  // element index of (o, lane, c) is o*128 + lane*4 + c: one 32-bit (int8) or 16-bit (packed) store per o
  uint32_t* d8 = reinterpret_cast<uint32_t*>(qa + size_t(token) * 4096);
  uint16_t* d4 = reinterpret_cast<uint16_t*>(qa + size_t(token) * 2048);
#pragma unroll
  for (int o = 0; o < 32; ++o) {
    const uint32_t b = quant4_bytes<OUT>(P[2 * o], P[2 * o + 1], inv_lo, inv_hi, s);
    if (OUT == 2) {
      d8[o * 32 + lane] = b;
    } else if (OUT == 1) {
      d8[o * 32 + lane] = (b << 4) & 0xf0f0f0f0u;
    } else {
      const uint32_t n = b & 0x0f0f0f0fu;  // four nibbles in four bytes -> 16 bits, element 0 lowest
      const uint32_t m = n | (n >> 4);     // bytes 0 and 2 now hold two nibbles each
      d4[o * 32 + lane] = uint16_t((m & 0xffu) | ((m >> 8) & 0xff00u));
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
        auto kern = bf16 ? hadamard4096_quant_kernel<OUT, true> : hadamard4096_quant_kernel<OUT, false>;
        if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), size_t(smem))) return rc;
        kern<<<int((M + kHad4096Warps - 1) / kHad4096Warps), kHad4096Warps * 32, smem, stream>>>(xp, qa, sa, int(M));
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

// out_fmt = 0: qa receives packed nibbles (M x K/2); 1: int8 holding 16*q (M x K); 2: e4m3 holding q (M x K).
int hadamard_quant_int4(const void* x, uint8_t* qa, float* sa, int64_t M, int64_t K, int hadamard, int dtype,
                        int out_fmt, cudaStream_t stream) {
  if (M <= 0) return ASRQ_OK;
  const uint16_t* xp = static_cast<const uint16_t*>(x);
  const int bf16 = dtype == ASRQ_BF16;
  if (out_fmt == 2) return launch_quant<2>(xp, qa, sa, M, K, hadamard, bf16, stream);
  return out_fmt ? launch_quant<1>(xp, qa, sa, M, K, hadamard, bf16, stream)
                 : launch_quant<0>(xp, qa, sa, M, K, hadamard, bf16, stream);
}

}  // namespace asrq
