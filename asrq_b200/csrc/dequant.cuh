// Dequantisation of one packed word for the tcgen05 prefill kernels.
#pragma once

#include "common.cuh"

namespace asrq {

// One 32-bit word of packed weights -> 16-bit floats in natural k order, scaled.
// out holds 32/BITS/2 packed pairs.
template <int BITS, bool BF16>
__device__ __forceinline__ void dequant_word(uint32_t q, uint32_t s2, uint32_t z2, uint32_t* out) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t t = prmt(q, q, 0x1111u * j);  // byte j replicated
    if (!BF16) {
      const uint32_t magic = 0x64006400u;  // 1024 | field
      if (BITS == 4) {
        const uint32_t v = lop3_and_or(t, 0x00f0000fu, magic);  // (1024+e0, 1024+16*e1)
        const __half2 c = __hfma2(u32_as_h2(v), u32_as_h2(0x2c003c00u), u32_as_h2(0xd400e400u));
        out[j] = h2_as_u32(__hfma2(c, u32_as_h2(s2), u32_as_h2(z2)));
      } else {
        const uint32_t v0 = lop3_and_or(t, 0x000c0003u, magic);  // (1024+e0, 1024+4*e1)
        const uint32_t v1 = lop3_and_or(t, 0x00c00030u, magic);  // (1024+16*e2, 1024+64*e3)
        const __half2 c0 = __hfma2(u32_as_h2(v0), u32_as_h2(0x34003c00u), u32_as_h2(0xdc00e400u));
        const __half2 c1 = __hfma2(u32_as_h2(v1), u32_as_h2(0x24002c00u), u32_as_h2(0xcc00d400u));
        out[2 * j] = h2_as_u32(__hfma2(c0, u32_as_h2(s2), u32_as_h2(z2)));
        out[2 * j + 1] = h2_as_u32(__hfma2(c1, u32_as_h2(s2), u32_as_h2(z2)));
      }
    } else {
      // bf16 activations: exact codes via the fp16 trick, q*scale+zero in fp32, one rounding to bf16
      // (s2, z2 carry the fp32 scale and zero bit patterns in this mode).
      const uint32_t magic = 0x64006400u;
      const float sf = __uint_as_float(s2), zf = __uint_as_float(z2);
      if (BITS == 4) {
        const uint32_t v = lop3_and_or(t, 0x00f0000fu, magic);
        const float2 c = __half22float2(__hfma2(u32_as_h2(v), u32_as_h2(0x2c003c00u), u32_as_h2(0xd400e400u)));
        const __nv_bfloat162 w = __floats2bfloat162_rn(fmaf(c.x, sf, zf), fmaf(c.y, sf, zf));
        out[j] = *reinterpret_cast<const uint32_t*>(&w);
      } else {
        const uint32_t v0 = lop3_and_or(t, 0x000c0003u, magic);
        const uint32_t v1 = lop3_and_or(t, 0x00c00030u, magic);
        const float2 c0 = __half22float2(__hfma2(u32_as_h2(v0), u32_as_h2(0x34003c00u), u32_as_h2(0xdc00e400u)));
        const float2 c1 = __half22float2(__hfma2(u32_as_h2(v1), u32_as_h2(0x24002c00u), u32_as_h2(0xcc00d400u)));
        const __nv_bfloat162 w0 = __floats2bfloat162_rn(fmaf(c0.x, sf, zf), fmaf(c0.y, sf, zf));
        const __nv_bfloat162 w1 = __floats2bfloat162_rn(fmaf(c1.x, sf, zf), fmaf(c1.y, sf, zf));
        out[2 * j] = *reinterpret_cast<const uint32_t*>(&w0);
        out[2 * j + 1] = *reinterpret_cast<const uint32_t*>(&w1);
      }
    }
  }
}

}  // namespace asrq
