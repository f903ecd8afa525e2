// Shared host/device helpers of the asrq_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>
#include <string>

#include "../../include/asrq_b200.h"

namespace asrq {

// ---- host: per-thread error text ------------------------------------------------
std::string& last_error();
int fail(int code, const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);

#define ASRQ_CUDA_TRY(expr)                                  \
  do {                                                       \
    cudaError_t e__ = (expr);                                \
    if (e__ != cudaSuccess) return asrq::cuda_fail(e__, #expr); \
  } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---- host: tuning and test switches (asrq_set_option / asrq_get_option) ------------------
// Process-wide integers.  Each takes its default from the environment variable ASRQ_B200_<NAME>
// (upper case) read ONCE, when the library is loaded; afterwards only asrq_set_option changes it.
// No launch path calls getenv.
enum Option {
  kOptNoPdl = 0,     // 1: launch without programmatic dependent launch
  kOptMidKernel,     // 17..64 tokens: 0 auto (chain-oriented tensor-core kernel where it fits), 1 the decode / prefill kernels
  kOptGemvKernel,    // decode kernel: 0 auto, 1 strip-per-block (registers), 2 split-K (workspace), 3 staged (shared memory)
  kOptGemvCpw,       // strip-per-block decode kernel: steps per warp (0 auto)
  kOptGemvXStage,    // staged decode kernel: 0 = fragment loads of the activations straight from L2 (no staging in shared memory)
  kOptGemvLoop,      // strip-per-block decode kernel, rounds variant: -1 auto, 0 never, 1 whenever a layer needs > 1 wave
  kOptTcSplit,       // prefill kernel: 1 disables split K
  kOptTcBt,          // prefill kernels: token-tile width (0 auto)
  kOptTcPair,        // prefill: -1 auto, 0 one CTA per tile, 1 CTA pairs
  kOptTcPairRelease, // CTA-pair prefill: 1 = release-ordered cross-CTA arrivals (one per dequant warp), 0 = relaxed
  kOptW4a4Bt,        // W4A4 GEMM: token-tile width (0 auto)
  kOptW4a4Pair,      // W4A4 GEMM: -1 auto, 0 one CTA per tile, 1 CTA pairs
  kOptTrace,         // builds with -DASRQ_TRACE only: 1 records pipeline clock marks into the workspace
  kOptTraceBlock,    // builds with -DASRQ_TRACE only: which block records
  kOptCount
};
int option(Option o);
unsigned options_generation();  // bumped by every asrq_set_option: caches of derived choices compare it

// ---- workspace layout --------------------------------------------------------------
// [0,256)            status block: word 0 = error flag (0 ok), word 1 = where a wait gave up
// [256, 256+16384)   4096 tile counters (zero between calls)
// [16640, ...)       fp32 split-K partial sums
constexpr size_t kStatusBytes = 256;
constexpr size_t kCounterBytes = 4096 * sizeof(unsigned);
constexpr size_t kPartialOffset = kStatusBytes + kCounterBytes;
constexpr int kGemvMaxSplit = 32;

// ---- device helpers ----------------------------------------------------------------
__device__ __forceinline__ uint32_t lop3_and_or(uint32_t x, uint32_t mask, uint32_t orv) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xea;" : "=r"(r) : "r"(x), "r"(mask), "r"(orv));  // (x & mask) | orv
  return r;
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}

__device__ __forceinline__ uint4 ldg_stream_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }

// Convert one 32-bit word of packed weights into fp16 pairs of exact integer codes.
// 4-bit: out[i] = (e_i, e_{i+4}), i = 0..3.   2-bit: out[i] = (e_i, e_{i+8}), i = 0..7.
// The caller pairs them with activations stored in the same (i, i+4) / (i, i+8) order.
template <int BITS>
__device__ __forceinline__ void unpack_codes_f16(uint32_t q, __half2* out) {
  const uint32_t magic = 0x64006400u;  // 1024.0 in both halves
  if (BITS == 4) {
    const __half2 k1024 = __half2half2(__ushort_as_half(0x6400));
    const __half2 k16th = __half2half2(__ushort_as_half(0x2c00));  // 1/16
    const __half2 km64 = __half2half2(__ushort_as_half(0xd400));   // -64
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      uint32_t lo = lop3_and_or(q, 0x000f000fu, magic);
      uint32_t hi = lop3_and_or(q, 0x00f000f0u, magic);
      out[2 * j] = __hsub2(u32_as_h2(lo), k1024);
      out[2 * j + 1] = __hfma2(u32_as_h2(hi), k16th, km64);
      q >>= 8;
    }
  } else {
    const __half2 k1024 = __half2half2(__ushort_as_half(0x6400));
    const __half2 k4th = __half2half2(__ushort_as_half(0x3400));    // 1/4
    const __half2 km256 = __half2half2(__ushort_as_half(0xdc00));   // -256
    const __half2 k16th = __half2half2(__ushort_as_half(0x2c00));   // 1/16
    const __half2 km64 = __half2half2(__ushort_as_half(0xd400));    // -64
    const __half2 k64th = __half2half2(__ushort_as_half(0x2400));   // 1/64
    const __half2 km16 = __half2half2(__ushort_as_half(0xcc00));    // -16
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      uint32_t f0 = lop3_and_or(q, 0x00030003u, magic);
      uint32_t f1 = lop3_and_or(q, 0x000c000cu, magic);
      uint32_t f2 = lop3_and_or(q, 0x00300030u, magic);
      uint32_t f3 = lop3_and_or(q, 0x00c000c0u, magic);
      out[4 * j] = __hsub2(u32_as_h2(f0), k1024);
      out[4 * j + 1] = __hfma2(u32_as_h2(f1), k4th, km256);
      out[4 * j + 2] = __hfma2(u32_as_h2(f2), k16th, km64);
      out[4 * j + 3] = __hfma2(u32_as_h2(f3), k64th, km16);
      q >>= 8;
    }
  }
}

__device__ __forceinline__ float bf16_bits_to_float(uint16_t b) { return __uint_as_float(uint32_t(b) << 16); }

__device__ __forceinline__ uint16_t float_to_out16(float v, bool bf16) {
  if (bf16) {
    __nv_bfloat16 b = __float2bfloat16_rn(v);
    return *reinterpret_cast<uint16_t*>(&b);
  }
  __half h = __float2half_rn(v);
  return *reinterpret_cast<uint16_t*>(&h);
}

// ---- fused epilogue of a quantized layer -----------------------------------------------------------
// What may follow y = x . W^T + bias inside the same kernel: an activation, or the addition of a residual
// stream.  Both act on the 16-bit-rounded layer output, exactly as the unfused sequence of modules does
// (the layer returns a 16-bit tensor; GELU, or the residual add, reads it and rounds again).
constexpr int kActNone = 0, kActGelu = 1;  // GELU: x * Phi(x) with the exact erf form
struct Epilogue {
  const void* residual = nullptr;  // same shape and type as y, or NULL
  int act = kActNone;
};
__device__ __forceinline__ float out16_to_float(uint16_t b, bool bf16) {
  return bf16 ? bf16_bits_to_float(b) : __half2float(__ushort_as_half(b));
}
__device__ __forceinline__ uint16_t epilogue16(uint16_t y16, int act, bool has_res, uint16_t res16, bool bf16) {
  float r = out16_to_float(y16, bf16);
  if (act == kActGelu) y16 = float_to_out16(0.5f * r * (1.f + erff(r * 0.70710678118654752440f)), bf16);
  if (has_res) y16 = float_to_out16(out16_to_float(res16, bf16) + out16_to_float(y16, bf16), bf16);
  return y16;
}
// ---- layer norm of a row held by one warp as VEC 16-byte vectors per lane (dim = 256 * VEC) --------------------
// raw[i] holds elements (i * 32 + lane) * 8 .. + 7 of the row; statistics in fp32, two passes.
template <int VEC>
__device__ __forceinline__ void ln_row_stats(const uint4 (&raw)[VEC], int dim, float eps, bool bf16, float& mean, float& rstd) {
  auto val = [&](int i, int e) {
    const uint32_t w = e < 2 ? raw[i].x : (e < 4 ? raw[i].y : (e < 6 ? raw[i].z : raw[i].w));
    const uint16_t h = uint16_t((e & 1) ? (w >> 16) : (w & 0xffffu));
    return out16_to_float(h, bf16);
  };
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < VEC; ++i)
#pragma unroll
    for (int e = 0; e < 8; ++e) sum += val(i, e);
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  mean = sum / float(dim);
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < VEC; ++i)
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float d = val(i, e) - mean;
      sq = fmaf(d, d, sq);
    }
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
  rstd = rsqrtf(sq / float(dim) + eps);
}
__device__ __forceinline__ float ln_apply(float v, float mean, float rstd, float g, float b) {
  return fmaf((v - mean) * rstd, g, b);
}

// the fp32 result of a layer (bias already added) through rounding and the epilogue
__device__ __forceinline__ uint16_t finish16(float v, int act, const uint16_t* residual, size_t idx, bool bf16) {
  const uint16_t y16 = float_to_out16(v, bf16);
  if (act == kActNone && residual == nullptr) return y16;
  return epilogue16(y16, act, residual != nullptr, residual ? residual[idx] : uint16_t(0), bf16);
}

}  // namespace asrq
