// The steps either side of a quantized layer in a decoder block, as kernels of their own:
//
//   add_layernorm   x' = x + delta (optional), h = LayerNorm(x') * gamma + beta, one warp per row, fp32
//                   statistics on the 16-bit-rounded x' (what the unfused sequence "add, then layer_norm"
//                   computes), 16-bit in and out;
//   add_rmsnorm     x' = x + delta (optional), h = (x' / rms(x')) rounded to 16 bits, then * gamma: the RMS norm of
//                   the Qwen3 decoder blocks (statistics in fp32, the normalised value rounded before the weight
//                   multiplies it, as the module does);
//   silu_mul        out[m, i] = silu(gu[m, i]) * gu[m, I + i] on the output of a fused gate/up projection, each
//                   factor rounded to 16 bits as the unfused sequence rounds them;
//   qk_norm_rope    what sits between a fused q/k/v projection and the attention of a Qwen3 block, in one launch: the
//                   per-head RMS norm of queries and keys, the rotary embedding, and the write of the new keys and
//                   values into the caches at the sequence position (read from device memory when decoding under a
//                   graph), every step rounded to 16 bits where the module sequence rounds it;
//   decode_self_attention   one new token per sequence against its own cache (multi-head, one warp per sequence and
//                   head): the new key and value are written at the position read from device memory, then
//                   softmax(q . K^T) . V over positions 0..pos in fp32 -- the cache write and the attention of a
//                   decoder step's self-attention in one launch of this library's chain;
//   epilogue16      y = act(y) or y = residual + y on an already written output: the fall-back for
//                   layers whose kernel does not fuse the epilogue.
//
// All open with griddepcontrol.launch_dependents / .wait and are launched with programmatic stream
// serialisation, so in a chain of this library's kernels (a decoder step replayed as a CUDA graph)
// consecutive launches overlap their ramp-up with the predecessor's tail.
#include <algorithm>

#include "common.cuh"

namespace asrq {

namespace {

__device__ __forceinline__ float in16(uint16_t b, bool bf16) {
  return bf16 ? bf16_bits_to_float(b) : __half2float(__ushort_as_half(b));
}

constexpr int kLnWarps = 8;

// VEC: 16-byte vectors per lane (dim = 256 * VEC); generic dims take the strided loop with VEC = 0
template <int VEC>
__global__ void __launch_bounds__(32 * kLnWarps)
add_layernorm_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ delta, const uint16_t* __restrict__ gamma,
                     const uint16_t* __restrict__ beta, float eps, uint16_t* __restrict__ x_out, uint16_t* __restrict__ h_out,
                     int rows, int dim, int bf16) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * kLnWarps + (threadIdx.x >> 5);
  // the norm's weight and bias are constants: fetched ahead of the stream dependency (vector path)
  uint4 gpre[VEC > 0 ? VEC : 1], bpre[VEC > 0 ? VEC : 1];
  if constexpr (VEC > 0) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const int e = (i * 32 + lane) * 8;
      gpre[i] = __ldg(reinterpret_cast<const uint4*>(gamma + e));
      bpre[i] = __ldg(reinterpret_cast<const uint4*>(beta + e));
    }
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (row >= rows) return;
  const size_t off = size_t(row) * dim;
  if constexpr (VEC > 0) {
    uint4 xr[VEC > 0 ? VEC : 1];  // the row (after the add, rounded to 16 bits), as the statistics see it
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const int e = (i * 32 + lane) * 8;
      const uint4 a = *reinterpret_cast<const uint4*>(x + off + e);
      if (delta) {
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
        const uint4 d = *reinterpret_cast<const uint4*>(delta + off + e);
        const uint32_t dw[4] = {d.x, d.y, d.z, d.w};
        uint32_t ow[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float lo = in16(uint16_t(aw[j] & 0xffffu), bf16) + in16(uint16_t(dw[j] & 0xffffu), bf16);
          const float hi = in16(uint16_t(aw[j] >> 16), bf16) + in16(uint16_t(dw[j] >> 16), bf16);
          ow[j] = uint32_t(float_to_out16(lo, bf16)) | (uint32_t(float_to_out16(hi, bf16)) << 16);
        }
        xr[i] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
      } else {
        xr[i] = a;
      }
      if (x_out) *reinterpret_cast<uint4*>(x_out + off + e) = xr[i];
    }
    float mean, rstd;
    ln_row_stats<(VEC > 0 ? VEC : 1)>(xr, dim, eps, bf16 != 0, mean, rstd);
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const int e = (i * 32 + lane) * 8;
      const uint4 g = gpre[i], b = bpre[i];
      const uint32_t xw[4] = {xr[i].x, xr[i].y, xr[i].z, xr[i].w};
      const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, bw[4] = {b.x, b.y, b.z, b.w};
      uint32_t ow[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float lo = ln_apply(in16(uint16_t(xw[j] & 0xffffu), bf16), mean, rstd, in16(uint16_t(gw[j] & 0xffffu), bf16),
                                  in16(uint16_t(bw[j] & 0xffffu), bf16));
        const float hi = ln_apply(in16(uint16_t(xw[j] >> 16), bf16), mean, rstd, in16(uint16_t(gw[j] >> 16), bf16),
                                  in16(uint16_t(bw[j] >> 16), bf16));
        ow[j] = uint32_t(float_to_out16(lo, bf16)) | (uint32_t(float_to_out16(hi, bf16)) << 16);
      }
      *reinterpret_cast<uint4*>(h_out + off + e) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
  } else {
    // any dimension: three passes over the row (the second and third hit L1/L2)
    float sum = 0.f;
    for (int e = lane; e < dim; e += 32) {
      float a = in16(x[off + e], bf16);
      if (delta) a += in16(delta[off + e], bf16);
      const uint16_t a16 = float_to_out16(a, bf16);
      if (x_out) x_out[off + e] = a16;
      sum += in16(a16, bf16);
    }
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float mean = sum / float(dim);
    float sq = 0.f;
    for (int e = lane; e < dim; e += 32) {
      float a = in16(x[off + e], bf16);
      if (delta) a += in16(delta[off + e], bf16);
      const float d = in16(float_to_out16(a, bf16), bf16) - mean;
      sq = fmaf(d, d, sq);
    }
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
    const float rstd = rsqrtf(sq / float(dim) + eps);
    for (int e = lane; e < dim; e += 32) {
      float a = in16(x[off + e], bf16);
      if (delta) a += in16(delta[off + e], bf16);
      const float c = in16(float_to_out16(a, bf16), bf16);
      h_out[off + e] = float_to_out16((c - mean) * rstd * in16(gamma[e], bf16) + in16(beta[e], bf16), bf16);
    }
  }
}

// One warp per row; VEC 16-byte vectors per lane when dim == 256 * VEC, else (VEC = 0) a strided loop.
template <int VEC>
__global__ void __launch_bounds__(32 * kLnWarps)
add_rmsnorm_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ delta, const uint16_t* __restrict__ gamma,
                   float eps, uint16_t* __restrict__ x_out, uint16_t* __restrict__ h_out, int rows, int dim, int bf16) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * kLnWarps + (threadIdx.x >> 5);
  if (row >= rows) return;
  const size_t off = size_t(row) * dim;
  if constexpr (VEC > 0) {
    float v[VEC > 0 ? VEC * 8 : 1];
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const int e = (i * 32 + lane) * 8;
      const uint4 a = *reinterpret_cast<const uint4*>(x + off + e);
      const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
      uint32_t dw[4] = {0, 0, 0, 0};
      if (delta) {
        const uint4 d = *reinterpret_cast<const uint4*>(delta + off + e);
        dw[0] = d.x; dw[1] = d.y; dw[2] = d.z; dw[3] = d.w;
      }
      uint32_t ow[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float lo = in16(uint16_t(aw[j] & 0xffffu), bf16), hi = in16(uint16_t(aw[j] >> 16), bf16);
        if (delta) {
          lo += in16(uint16_t(dw[j] & 0xffffu), bf16);
          hi += in16(uint16_t(dw[j] >> 16), bf16);
        }
        const uint16_t lo16 = float_to_out16(lo, bf16), hi16 = float_to_out16(hi, bf16);
        ow[j] = uint32_t(lo16) | (uint32_t(hi16) << 16);
        const float l = in16(lo16, bf16), h = in16(hi16, bf16);
        v[i * 8 + 2 * j] = l;
        v[i * 8 + 2 * j + 1] = h;
        sq = fmaf(l, l, sq);
        sq = fmaf(h, h, sq);
      }
      if (x_out) *reinterpret_cast<uint4*>(x_out + off + e) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
    const float rs = rsqrtf(sq / float(dim) + eps);
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const int e = (i * 32 + lane) * 8;
      const uint4 g = __ldg(reinterpret_cast<const uint4*>(gamma + e));
      const uint32_t gw[4] = {g.x, g.y, g.z, g.w};
      uint32_t ow[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float lo = in16(float_to_out16(v[i * 8 + 2 * j] * rs, bf16), bf16) * in16(uint16_t(gw[j] & 0xffffu), bf16);
        const float hi = in16(float_to_out16(v[i * 8 + 2 * j + 1] * rs, bf16), bf16) * in16(uint16_t(gw[j] >> 16), bf16);
        ow[j] = uint32_t(float_to_out16(lo, bf16)) | (uint32_t(float_to_out16(hi, bf16)) << 16);
      }
      *reinterpret_cast<uint4*>(h_out + off + e) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
  } else {
    float sq = 0.f;
    for (int e = lane; e < dim; e += 32) {
      float a = in16(x[off + e], bf16);
      if (delta) a += in16(delta[off + e], bf16);
      const uint16_t a16 = float_to_out16(a, bf16);
      if (x_out) x_out[off + e] = a16;
      const float c = in16(a16, bf16);
      sq = fmaf(c, c, sq);
    }
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
    const float rs = rsqrtf(sq / float(dim) + eps);
    for (int e = lane; e < dim; e += 32) {
      float a = in16(x[off + e], bf16);
      if (delta) a += in16(delta[off + e], bf16);
      const float c = in16(float_to_out16(a, bf16), bf16);
      h_out[off + e] = float_to_out16(in16(float_to_out16(c * rs, bf16), bf16) * in16(gamma[e], bf16), bf16);
    }
  }
}

// gu: rows x 2*inter (gate columns first, then up), out: rows x inter; eight elements per thread
__global__ void __launch_bounds__(256)
silu_mul_kernel(const uint16_t* __restrict__ gu, uint16_t* __restrict__ out, int rows, int inter, int bf16) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int vpr = inter / 8;  // vectors per output row
  const size_t n_vec = size_t(rows) * vpr;
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < n_vec; i += size_t(gridDim.x) * blockDim.x) {
    const size_t r = i / vpr, c = (i - r * vpr) * 8;
    const uint4 g = *reinterpret_cast<const uint4*>(gu + r * 2 * inter + c);
    const uint4 u = *reinterpret_cast<const uint4*>(gu + r * 2 * inter + inter + c);
    const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
    uint32_t ow[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint16_t o2[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const float gv = in16(uint16_t(gw[j] >> (16 * h)), bf16), uv = in16(uint16_t(uw[j] >> (16 * h)), bf16);
        const float sv = in16(float_to_out16(gv / (1.f + expf(-gv)), bf16), bf16);  // silu, rounded as the module rounds it
        o2[h] = float_to_out16(sv * uv, bf16);
      }
      ow[j] = uint32_t(o2[0]) | (uint32_t(o2[1]) << 16);
    }
    *reinterpret_cast<uint4*>(out + r * inter + c) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
  }
}

// qkv: rows x (nq + 2 nkv) x hd, a row = sequence b, step t (rows = B * T).  One warp per (row, head); E = hd / 32
// elements per lane; the rotary partner of element i is i +- hd / 2, i.e. the same slot of lane ^ 16.
// q_out: B x nq x T x hd; caches: B x nkv x max_len x hd, written at position pos0 + t.
template <int E>
__global__ void __launch_bounds__(256)
qk_norm_rope_kernel(const uint16_t* __restrict__ qkv, const uint16_t* __restrict__ qw, const uint16_t* __restrict__ kw,
                    const uint16_t* __restrict__ cos_t, const uint16_t* __restrict__ sin_t, const long long* __restrict__ pos_dev,
                    long long pos_host, uint16_t* __restrict__ q_out, uint16_t* __restrict__ k_cache, uint16_t* __restrict__ v_cache,
                    int rows, int T, int nq, int nkv, int max_len, float eps, int bf16) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  constexpr int hd = 32 * E;
  const int lane = threadIdx.x & 31;
  const int heads = nq + 2 * nkv;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (long long)rows * heads) return;
  const int row = int(item / heads), head = int(item - (long long)row * heads);
  const int b = row / T, t = row - b * T;
  const long long pos = (pos_dev ? *pos_dev : pos_host) + t;
  const uint16_t* src = qkv + (size_t(row) * heads + head) * hd + lane * E;
  uint16_t v16[E];
  if (E == 4) {
    const uint2 u = *reinterpret_cast<const uint2*>(src);
    v16[0] = uint16_t(u.x & 0xffffu); v16[1] = uint16_t(u.x >> 16); v16[2 % E] = uint16_t(u.y & 0xffffu); v16[3 % E] = uint16_t(u.y >> 16);
  } else {
    const uint32_t u = *reinterpret_cast<const uint32_t*>(src);
    v16[0] = uint16_t(u & 0xffffu); v16[1] = uint16_t(u >> 16);
  }
  uint16_t* dst;
  if (head < nq) {
    dst = q_out + ((size_t(b) * nq + head) * T + t) * hd + lane * E;
  } else if (head < nq + nkv) {
    dst = k_cache + ((size_t(b) * nkv + (head - nq)) * max_len + size_t(pos)) * hd + lane * E;
  } else {
    dst = v_cache + ((size_t(b) * nkv + (head - nq - nkv)) * max_len + size_t(pos)) * hd + lane * E;
  }
  if (head < nq + nkv) {  // queries and keys: norm over the head, weight, rotary embedding
    const uint16_t* w = (head < nq ? qw : kw) + lane * E;
    float f[E], sq = 0.f;
#pragma unroll
    for (int i = 0; i < E; ++i) {
      f[i] = in16(v16[i], bf16);
      sq = fmaf(f[i], f[i], sq);
    }
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
    const float rs = rsqrtf(sq / float(hd) + eps);
#pragma unroll
    for (int i = 0; i < E; ++i) {
      const float n = in16(float_to_out16(f[i] * rs, bf16), bf16);
      const float y = in16(float_to_out16(in16(w[i], bf16) * n, bf16), bf16);
      const float partner = __shfl_xor_sync(0xffffffffu, y, 16);
      const float rot = lane < 16 ? -partner : partner;
      const size_t ci = size_t(pos) * hd + lane * E + i;
      const float a = in16(float_to_out16(y * in16(cos_t[ci], bf16), bf16), bf16);
      const float c = in16(float_to_out16(rot * in16(sin_t[ci], bf16), bf16), bf16);
      v16[i] = float_to_out16(a + c, bf16);
    }
  }
  if (E == 4) {
    *reinterpret_cast<uint2*>(dst) = make_uint2(uint32_t(v16[0]) | (uint32_t(v16[1]) << 16), uint32_t(v16[2 % E]) | (uint32_t(v16[3 % E]) << 16));
  } else {
    *reinterpret_cast<uint32_t*>(dst) = uint32_t(v16[0]) | (uint32_t(v16[1]) << 16);
  }
}

// qkv: B rows of [q | k | v], each H * hd wide.  kv: (2, B, H, max_len, hd) keys then values.  out: B x (H * hd).
// E = hd / 32 elements per lane.  Scores: lane j takes keys j, j + 32, ... (q from shared memory); output: lane owns E
// consecutive elements of the head, probabilities broadcast by shuffle.
template <int E>
__global__ void __launch_bounds__(128)
decode_self_attention_kernel(const uint16_t* __restrict__ qkv, uint16_t* __restrict__ kv, const long long* __restrict__ pos_dev,
                             uint16_t* __restrict__ out, int B, int H, int max_len, float scale, int bf16) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  constexpr int hd = 32 * E;
  constexpr int kWarps = 4;
  constexpr int kMaxKeysPerLane = 16;  // max_len <= 512
  __shared__ float qs[kWarps][hd];
  __shared__ float ps[kWarps][32 * kMaxKeysPerLane + 16];  // probabilities by key; the tail stays zero
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const int item = blockIdx.x * kWarps + wib;
  if (item >= B * H) return;
  const int b = item / H, h = item - b * H;
  const int pos = int(*pos_dev);
  const size_t d = size_t(H) * hd;
  const uint16_t* row = qkv + size_t(b) * 3 * d + size_t(h) * hd;
  uint16_t* kc = kv + ((size_t(b) * H + h) * max_len) * hd;
  uint16_t* vc = kc + size_t(B) * H * max_len * hd;
  // the new key and value into the cache, the query (scaled) into shared memory
#pragma unroll
  for (int i = 0; i < E; ++i) {
    const int e = lane * E + i;
    qs[wib][e] = in16(row[e], bf16) * scale;
    kc[size_t(pos) * hd + e] = row[d + e];
    vc[size_t(pos) * hd + e] = row[2 * d + e];
  }
  __syncwarp();
  // scores of this lane's keys
  float sc[kMaxKeysPerLane];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < kMaxKeysPerLane; ++j) {
    const int t = lane + 32 * j;
    sc[j] = -INFINITY;
    if (t <= pos) {
      const uint4* kr = reinterpret_cast<const uint4*>(kc + size_t(t) * hd);
      float acc = 0.f;
#pragma unroll
      for (int c = 0; c < hd / 8; ++c) {
        const uint4 u = kr[c];
        const uint32_t w4[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int m = 0; m < 4; ++m) {
          acc = fmaf(qs[wib][c * 8 + 2 * m], in16(uint16_t(w4[m] & 0xffffu), bf16), acc);
          acc = fmaf(qs[wib][c * 8 + 2 * m + 1], in16(uint16_t(w4[m] >> 16), bf16), acc);
        }
      }
      sc[j] = acc;
      mx = fmaxf(mx, acc);
    }
  }
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < kMaxKeysPerLane; ++j) {
    sc[j] = (lane + 32 * j <= pos) ? __expf(sc[j] - mx) : 0.f;
    sum += sc[j];
  }
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float inv = 1.f / sum;
  // output: probabilities through shared memory (read as broadcasts), every lane accumulates its E elements of the head;
  // sixteen value rows are requested before the first is used, so their latencies overlap
#pragma unroll
  for (int j = 0; j < kMaxKeysPerLane; ++j) ps[wib][lane + 32 * j] = sc[j];
  __syncwarp();
  if (lane < 16) ps[wib][32 * kMaxKeysPerLane + lane] = 0.f;
  __syncwarp();
  float o_acc[E];
#pragma unroll
  for (int i = 0; i < E; ++i) o_acc[i] = 0.f;
  for (int t0 = 0; t0 <= pos; t0 += 16) {  // warp-uniform
    uint32_t vv[16][E / 2];
#pragma unroll
    for (int u = 0; u < 16; ++u) {
      const int t = min(t0 + u, pos);  // rows past the position repeat the last one; their probability is zero
      const uint32_t* vr = reinterpret_cast<const uint32_t*>(vc + size_t(t) * hd + lane * E);
#pragma unroll
      for (int i = 0; i < E / 2; ++i) vv[u][i] = vr[i];
    }
#pragma unroll
    for (int u = 0; u < 16; ++u) {
      const float pr = ps[wib][t0 + u];
#pragma unroll
      for (int i = 0; i < E / 2; ++i) {
        o_acc[2 * i] = fmaf(pr, in16(uint16_t(vv[u][i] & 0xffffu), bf16), o_acc[2 * i]);
        o_acc[2 * i + 1] = fmaf(pr, in16(uint16_t(vv[u][i] >> 16), bf16), o_acc[2 * i + 1]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < E; ++i) out[size_t(b) * d + size_t(h) * hd + lane * E + i] = float_to_out16(o_acc[i] * inv, bf16);
}

__global__ void __launch_bounds__(256)
epilogue16_kernel(uint16_t* __restrict__ y, const uint16_t* __restrict__ residual, size_t n_vec, int act, int bf16) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < n_vec; i += size_t(gridDim.x) * blockDim.x) {
    uint4 a = reinterpret_cast<uint4*>(y)[i];
    uint32_t aw[4] = {a.x, a.y, a.z, a.w}, rw[4] = {0, 0, 0, 0};
    if (residual) {
      const uint4 r = reinterpret_cast<const uint4*>(residual)[i];
      rw[0] = r.x; rw[1] = r.y; rw[2] = r.z; rw[3] = r.w;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint16_t lo = epilogue16(uint16_t(aw[j] & 0xffffu), act, residual != nullptr, uint16_t(rw[j] & 0xffffu), bf16 != 0);
      const uint16_t hi = epilogue16(uint16_t(aw[j] >> 16), act, residual != nullptr, uint16_t(rw[j] >> 16), bf16 != 0);
      aw[j] = uint32_t(lo) | (uint32_t(hi) << 16);
    }
    reinterpret_cast<uint4*>(y)[i] = make_uint4(aw[0], aw[1], aw[2], aw[3]);
  }
}

template <typename K, typename... Args>
int launch_pdl(K kern, dim3 grid, dim3 block, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = option(kOptNoPdl) ? 0 : 1;
  ASRQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, args...));
  return ASRQ_OK;
}

}  // namespace

int add_layernorm(const void* x, const void* delta, const void* gamma, const void* beta, float eps, void* x_out, void* h_out,
                  int64_t rows, int64_t dim, int dtype, cudaStream_t stream) {
  const int bf16 = dtype == ASRQ_BF16;
  const dim3 grid(unsigned((rows + kLnWarps - 1) / kLnWarps)), block(32 * kLnWarps);
  auto xp = static_cast<const uint16_t*>(x), dp = static_cast<const uint16_t*>(delta);
  auto gp = static_cast<const uint16_t*>(gamma), bp = static_cast<const uint16_t*>(beta);
  auto xo = static_cast<uint16_t*>(x_out), ho = static_cast<uint16_t*>(h_out);
  const bool vec_ok = aligned16(x) && aligned16(h_out) && aligned16(gamma) && aligned16(beta) && (!delta || aligned16(delta)) &&
                      (!x_out || aligned16(x_out));
  if (vec_ok && dim == 1280) return launch_pdl(add_layernorm_kernel<5>, grid, block, stream, xp, dp, gp, bp, eps, xo, ho, int(rows), int(dim), bf16);
  if (vec_ok && dim == 1024) return launch_pdl(add_layernorm_kernel<4>, grid, block, stream, xp, dp, gp, bp, eps, xo, ho, int(rows), int(dim), bf16);
  if (vec_ok && dim == 2048) return launch_pdl(add_layernorm_kernel<8>, grid, block, stream, xp, dp, gp, bp, eps, xo, ho, int(rows), int(dim), bf16);
  if (vec_ok && dim == 256) return launch_pdl(add_layernorm_kernel<1>, grid, block, stream, xp, dp, gp, bp, eps, xo, ho, int(rows), int(dim), bf16);
  return launch_pdl(add_layernorm_kernel<0>, grid, block, stream, xp, dp, gp, bp, eps, xo, ho, int(rows), int(dim), bf16);
}

int add_rmsnorm(const void* x, const void* delta, const void* gamma, float eps, void* x_out, void* h_out, int64_t rows,
                int64_t dim, int dtype, cudaStream_t stream) {
  const int bf16 = dtype == ASRQ_BF16;
  const dim3 grid(unsigned((rows + kLnWarps - 1) / kLnWarps)), block(32 * kLnWarps);
  auto xp = static_cast<const uint16_t*>(x), dp = static_cast<const uint16_t*>(delta);
  auto gp = static_cast<const uint16_t*>(gamma);
  auto xo = static_cast<uint16_t*>(x_out), ho = static_cast<uint16_t*>(h_out);
  const bool vec_ok = aligned16(x) && aligned16(h_out) && aligned16(gamma) && (!delta || aligned16(delta)) && (!x_out || aligned16(x_out));
  if (vec_ok && dim == 2048) return launch_pdl(add_rmsnorm_kernel<8>, grid, block, stream, xp, dp, gp, eps, xo, ho, int(rows), int(dim), bf16);
  if (vec_ok && dim == 1024) return launch_pdl(add_rmsnorm_kernel<4>, grid, block, stream, xp, dp, gp, eps, xo, ho, int(rows), int(dim), bf16);
  if (vec_ok && dim == 256) return launch_pdl(add_rmsnorm_kernel<1>, grid, block, stream, xp, dp, gp, eps, xo, ho, int(rows), int(dim), bf16);
  return launch_pdl(add_rmsnorm_kernel<0>, grid, block, stream, xp, dp, gp, eps, xo, ho, int(rows), int(dim), bf16);
}

int silu_mul(const void* gu, void* out, int64_t rows, int64_t inter, int dtype, int sm_count, cudaStream_t stream) {
  const size_t n_vec = size_t(rows) * size_t(inter) / 8;
  const unsigned blocks = unsigned(std::max<size_t>(1, std::min<size_t>(size_t(sm_count) * 8, (n_vec + 255) / 256)));
  return launch_pdl(silu_mul_kernel, dim3(blocks), dim3(256), stream, static_cast<const uint16_t*>(gu), static_cast<uint16_t*>(out),
                    int(rows), int(inter), int(dtype == ASRQ_BF16));
}

int qk_norm_rope(const void* qkv, const void* qw, const void* kw, const void* cos_t, const void* sin_t, const long long* pos_dev,
                 long long pos_host, void* q_out, void* k_cache, void* v_cache, int64_t B, int64_t T, int nq, int nkv, int hd,
                 int64_t max_len, float eps, int dtype, cudaStream_t stream) {
  const int64_t items = B * T * (nq + 2 * nkv);
  const dim3 grid(unsigned((items + 7) / 8)), block(256);
  auto p = [](const void* v) { return static_cast<const uint16_t*>(v); };
  auto o = [](void* v) { return static_cast<uint16_t*>(v); };
  const int bf16 = dtype == ASRQ_BF16;
  if (hd == 128)
    return launch_pdl(qk_norm_rope_kernel<4>, grid, block, stream, p(qkv), p(qw), p(kw), p(cos_t), p(sin_t), pos_dev, pos_host, o(q_out),
                      o(k_cache), o(v_cache), int(B * T), int(T), nq, nkv, int(max_len), eps, bf16);
  return launch_pdl(qk_norm_rope_kernel<2>, grid, block, stream, p(qkv), p(qw), p(kw), p(cos_t), p(sin_t), pos_dev, pos_host, o(q_out),
                    o(k_cache), o(v_cache), int(B * T), int(T), nq, nkv, int(max_len), eps, bf16);
}

int decode_self_attention(const void* qkv, void* kv, const long long* pos_dev, void* out, int64_t B, int H, int hd, int64_t max_len,
                          float scale, int dtype, cudaStream_t stream) {
  const dim3 grid(unsigned((B * H + 3) / 4)), block(128);
  const int bf16 = dtype == ASRQ_BF16;
  if (hd == 64)
    return launch_pdl(decode_self_attention_kernel<2>, grid, block, stream, static_cast<const uint16_t*>(qkv), static_cast<uint16_t*>(kv),
                      pos_dev, static_cast<uint16_t*>(out), int(B), H, int(max_len), scale, bf16);
  return launch_pdl(decode_self_attention_kernel<4>, grid, block, stream, static_cast<const uint16_t*>(qkv), static_cast<uint16_t*>(kv),
                    pos_dev, static_cast<uint16_t*>(out), int(B), H, int(max_len), scale, bf16);
}

// y = act(y) / y = residual + y over M x N 16-bit elements (M*N a multiple of 8, pointers 16-byte aligned)
int epilogue16_apply(void* y, const void* residual, int64_t M, int64_t N, int act, int dtype, int sm_count, cudaStream_t stream) {
  const size_t n_vec = size_t(M) * size_t(N) / 8;
  const unsigned blocks = unsigned(std::max<size_t>(1, std::min<size_t>(size_t(sm_count) * 8, (n_vec + 255) / 256)));
  return launch_pdl(epilogue16_kernel, dim3(blocks), dim3(256), stream, static_cast<uint16_t*>(y),
                    static_cast<const uint16_t*>(residual), n_vec, act, int(dtype == ASRQ_BF16));
}

}  // namespace asrq
