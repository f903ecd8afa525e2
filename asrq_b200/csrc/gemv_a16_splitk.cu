// Decode path, split-K variant: y[M,N] = x[M,K] . dequant(W)[N,K]^T for M <= 16 per launch.
//
// Used where the strip-per-block kernel of gemv_a16.cu does not apply (layers longer than 16
// warps x 4 steps) and by the entry point with built-in scratch.  A warp owns a strip of 16
// weight rows over one K span: each lane streams 128-bit words of packed weights for two rows
// (rows g and g+8, g = lane/4), turns them into fp16 in registers (exact integer code, then one
// fused multiply-add with the group scale and offset) and uses them as the A operand of
// mma.sync.m16n8k16; the activations (B operand, up to 16 tokens) sit in shared memory in the
// element order the unpacking produces, so no shuffles are needed.
//
// K is split twice: KQ warps of a block share a row strip and each take a part of the block's K
// slice, their partial tiles are added through shared memory in a fixed order; and, where the
// layer has too few rows to fill the SMs, gridDim.y blocks split K further through the caller's
// workspace, the last block to arrive for a row tile adding the slices in slice order.  The
// result never depends on scheduling.
#include <algorithm>
#include <cstdlib>

#include "common.cuh"

namespace asrq {
namespace splitk {

struct GemvParams {
  const uint16_t* x;
  const uint8_t* w;
  const __half* scales;
  const __half* zeros;
  const __half* bias;
  uint16_t* y;
  float* partials;
  unsigned* counters;
  int M, N, K, group_size, groups_per_row, S, kslice, KQ, bf16;
};

constexpr int kGemvWarps = 8;

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
  constexpr int PF = 3;              // steps of weights in flight ahead of the math
  constexpr int FR = 4 * MH;         // accumulator registers per lane

  extern __shared__ uint4 xs[];
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, c = lane & 3;
  const int KQ = p.KQ;
  const int strips = kGemvWarps / KQ;  // row strips per block
  const int strip = warp / KQ, kq = warp - strip * KQ;
  const int rows_per_block = strips * 16;
  const int k_begin = blockIdx.y * p.kslice;  // block's K slice
  const int wslice = p.kslice / KQ;           // this warp's span inside it
  const int row_units = p.kslice / 8 + 4;     // +64 B: rows g and g+1 land on different banks
  const int n_base = blockIdx.x * rows_per_block + strip * 16;
  const bool active = n_base < p.N;
  const int nchunks = wslice / CHUNK;
  const int chunk0 = kq * nchunks;  // first step of this warp inside the block's slice

  // ---- weights, scales and zeros first: they do not depend on the staged activations ----------
  const int r0 = n_base + g, r1 = r0 + 8;
  const size_t row_bytes = size_t(p.K) * BITS / 8;
  const int kw = k_begin + kq * wslice + c * KPT;  // first k of this lane
  const uint8_t* w0 = p.w + size_t(r0) * row_bytes + size_t(kw) * BITS / 8;
  const uint8_t* w1 = p.w + size_t(r1) * row_bytes + size_t(kw) * BITS / 8;
  const __half* sc0 = p.scales + size_t(r0) * p.groups_per_row;
  const __half* sc1 = p.scales + size_t(r1) * p.groups_per_row;
  const __half* zr0 = p.zeros + size_t(r0) * p.groups_per_row;
  const __half* zr1 = p.zeros + size_t(r1) * p.groups_per_row;
  uint4 qa[PF + 1], qb[PF + 1];
  __half sa[PF + 1], sb[PF + 1], za[PF + 1], zb[PF + 1];
  auto issue = [&](int chunk, int slot) {
    qa[slot] = ldg_stream_v4(w0 + size_t(chunk) * (CHUNK * BITS / 8));
    qb[slot] = ldg_stream_v4(w1 + size_t(chunk) * (CHUNK * BITS / 8));
    const int gi = (kw + chunk * CHUNK) / p.group_size;
    sa[slot] = __ldg(sc0 + gi);
    za[slot] = __ldg(zr0 + gi);
    sb[slot] = __ldg(sc1 + gi);
    zb[slot] = __ldg(zr1 + gi);
  };
  // Let the next kernel on the stream start as early as possible, and start streaming weights
  // before this one's own predecessor has finished: weights, scales and zeros are constants,
  // only the activations, the output and the workspace depend on earlier kernels.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (active) {
#pragma unroll
    for (int i = 0; i < PF; ++i)
      if (i < nchunks) issue(i, i);
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");

  // ---- stage the block's activation slice, re-ordered to the unpacking order ------------------
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

  float acc[MH][4];
#pragma unroll
  for (int mh = 0; mh < MH; ++mh)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[mh][i] = 0.f;

  if (active) {
    for (int cbase = 0; cbase < nchunks; cbase += PF + 1) {
#pragma unroll
      for (int u = 0; u < PF + 1; ++u) {
        const int chunk = cbase + u;
        if (chunk < nchunks) {
          if (chunk + PF < nchunks) issue(chunk + PF, (u + PF) % (PF + 1));
          const __half2 s0 = __half2half2(sa[u]), z0 = __half2half2(za[u]);
          const __half2 s1 = __half2half2(sb[u]), z1 = __half2half2(zb[u]);
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
                const uint4 xb = xs[(g + 8 * mh) * row_units + ((chunk0 + chunk) * UPT + j * (NH / 4) + t) * 4 + c];
                mma_m16n8k16(acc[mh], h2_as_u32(ha[4 * t]), h2_as_u32(hb[4 * t]), h2_as_u32(ha[4 * t + 1]),
                             h2_as_u32(hb[4 * t + 1]), xb.x, xb.y);
                mma_m16n8k16(acc[mh], h2_as_u32(ha[4 * t + 2]), h2_as_u32(hb[4 * t + 2]), h2_as_u32(ha[4 * t + 3]),
                             h2_as_u32(hb[4 * t + 3]), xb.z, xb.w);
              }
            }
          }
        }
      }
    }
  }

  // ---- add the KQ partial tiles of each strip through shared memory (fixed order) --------------
  // acc[mh][i] of lane (g, c): weight row strip*16 + g + 8*(i>>1), token 8*mh + 2c + (i&1).
  __syncthreads();  // everyone is done reading xs
  float* red = reinterpret_cast<float*>(xs);
#pragma unroll
  for (int mh = 0; mh < MH; ++mh)
#pragma unroll
    for (int i = 0; i < 4; ++i) red[(warp * FR + mh * 4 + i) * 32 + lane] = acc[mh][i];
  __syncthreads();

  const int per_strip = FR * 32;
  const int n_out = strips * per_strip;  // values this block owns
  __shared__ unsigned is_last;
  for (int o = tid; o < n_out; o += blockDim.x) {
    const int st = o / per_strip, rem = o - st * per_strip;
    float v = 0.f;
    for (int q = 0; q < KQ; ++q) v += red[(st * KQ + q) * per_strip + rem];
    const int fi = rem >> 5, l = rem & 31;
    const int n = blockIdx.x * rows_per_block + st * 16 + (l >> 2) + ((fi >> 1) & 1) * 8;
    const int m = 8 * (fi >> 2) + 2 * (l & 3) + (fi & 1);
    if (n < p.N && m < p.M) {
      if (p.S == 1) {
        if (p.bias) v += __half2float(__ldg(p.bias + n));
        p.y[size_t(m) * p.N + n] = float_to_out16(v, p.bf16);
      } else {
        __stcg(p.partials + (size_t(blockIdx.y) * MR + m) * p.N + n, v);
      }
    }
  }
  if (p.S == 1) return;

  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned ticket = atomicAdd(p.counters + blockIdx.x, 1u);
    is_last = (ticket == unsigned(p.S) - 1u);
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  const int n0 = blockIdx.x * rows_per_block;
  const int ncols = min(rows_per_block, p.N - n0);
  for (int i = tid; i < p.M * rows_per_block; i += blockDim.x) {
    const int m = i / rows_per_block, nn = i - m * rows_per_block;
    if (nn < ncols) {
      const int n = n0 + nn;
      const float* src = p.partials + size_t(m) * p.N + n;
      const size_t sstride = size_t(MR) * p.N;
      float v = 0.f;
      int s = 0;
      for (; s + 4 <= p.S; s += 4) {  // four independent loads, added in slice order
        const float a0 = __ldcg(src + (s + 0) * sstride), a1 = __ldcg(src + (s + 1) * sstride);
        const float a2 = __ldcg(src + (s + 2) * sstride), a3 = __ldcg(src + (s + 3) * sstride);
        v += a0; v += a1; v += a2; v += a3;
      }
      for (; s < p.S; ++s) v += __ldcg(src + s * sstride);
      if (p.bias) v += __half2float(__ldg(p.bias + n));
      p.y[size_t(m) * p.N + n] = float_to_out16(v, p.bf16);
    }
  }
  if (tid == 0) p.counters[blockIdx.x] = 0;
}

// How one launch splits K.  T = S * KQ spans per row strip, chosen as the smallest divisor of
// the number of 128-bit steps such that (a) a warp has at most four steps, so all its loads
// are in flight at once, and (b) the grid has at least one block per SM.  KQ of them (at
// most 4, fewer for larger M so that re-staging the activations stays cheap) are taken
// inside a block; the remaining S go through the workspace.
struct GemvSplit {
  int S, KQ;
};

GemvSplit gemv_pick_split(int bits, int m, int64_t N, int64_t K, int sm_count, int max_split) {
  const int chunk = (128 / bits) * 4;
  const int nchunks = int(K / chunk);
  const int64_t strips = (N + 15) / 16;
  int t_min = std::max((nchunks + 3) / 4, int((int64_t(sm_count) * kGemvWarps + strips - 1) / strips));
  t_min = std::min(std::max(t_min, 1), nchunks);
  int T = t_min;
  while (T < nchunks && nchunks % T) ++T;
  const int kq_cap = m <= 4 ? 4 : (m <= 8 ? 2 : 1);
  int KQ = 1;
  for (int q = kq_cap; q >= 1; q >>= 1)
    if (T % q == 0) {
      KQ = q;
      break;
    }
  int S = T / KQ;
  // the block's slice is staged in shared memory: keep it at or below 2048
  while (K / S > 2048 && S < nchunks) {
    ++S;
    while (S < nchunks && (nchunks % S || (nchunks / S) % KQ)) ++S;
  }
  if (S > max_split || (nchunks % S) || (nchunks / S) % KQ) {  // fall back to the plainest legal split
    KQ = 1;
    S = std::min(max_split, nchunks);
    while (S > 1 && nchunks % S) --S;
  }
  return {S, KQ};
}

}  // namespace splitk

size_t gemv_workspace_bytes(int64_t N, int max_split) {
  return kPartialOffset + size_t(max_split) * 16 * size_t(N) * sizeof(float);
}
size_t gemv_workspace_bytes(int64_t N) { return gemv_workspace_bytes(N, kGemvMaxSplit); }

namespace splitk {

template <int BITS, int MH>
static int launch_gemv(const GemvParams& p, cudaStream_t stream) {
  const size_t xs_bytes = size_t(8 * MH) * (p.kslice / 8 + 4) * 16;
  const size_t red_bytes = size_t(kGemvWarps) * 4 * MH * 32 * sizeof(float);
  const size_t smem = std::max(xs_bytes, red_bytes);
  auto kern = gemv_a16_kernel<BITS, MH>;
  if (smem > 48 * 1024)
    ASRQ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
  const int rows_per_block = (kGemvWarps / p.KQ) * 16;
  const int ntiles = (p.N + rows_per_block - 1) / rows_per_block;
  // Programmatic dependent launch: consecutive decode kernels overlap their weight fetch with the
  // predecessor's tail (the kernel orders itself with griddepcontrol.wait).
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(ntiles, p.S);
  cfg.blockDim = dim3(kGemvWarps * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  const bool pdl = option(kOptNoPdl) == 0;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  ASRQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, p));
  return ASRQ_OK;
}

}  // namespace splitk

int gemv_a16_splitk(int bits, const void* x, const uint8_t* w, const void* scales, const void* zeros,
             const void* bias, void* y, int64_t M, int64_t N, int64_t K, int group_size, int dtype,
             void* workspace, size_t workspace_bytes, int sm_count, cudaStream_t stream, int max_split) {
  const int chunk = (128 / bits) * 4;
  if (N % 16 || K % chunk || group_size <= 0 || K % group_size || group_size % (128 / bits))
    return fail(ASRQ_ERR_SHAPE,
                "w%da16 gemv: need N%%16==0, K%%%d==0, group_size%%%d==0, K%%group_size==0 "
                "(N=%lld K=%lld g=%d)", bits, chunk, 128 / bits, (long long)N, (long long)K, group_size);
  if (N > int64_t(4096) * 16 || K > (1 << 20))
    return fail(ASRQ_ERR_LIMIT, "w%da16 gemv: N > 65536 or K > 2^20", bits);
  if (workspace_bytes < gemv_workspace_bytes(N, max_split))
    return fail(ASRQ_ERR_WORKSPACE, "w%da16 gemv: workspace %zu < %zu bytes", bits, workspace_bytes,
                gemv_workspace_bytes(N, max_split));
  using namespace splitk;
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
  for (int64_t m0 = 0; m0 < M; m0 += 16) {
    const int mb = int(std::min<int64_t>(16, M - m0));
    const int mh = mb > 8 ? 2 : 1;
    p.x = static_cast<const uint16_t*>(x) + m0 * K;
    p.y = static_cast<uint16_t*>(y) + m0 * N;
    p.M = mb;
    const GemvSplit sp = gemv_pick_split(bits, mb, N, K, sm_count, max_split);
    p.S = sp.S;
    p.KQ = sp.KQ;
    p.kslice = int(K / p.S);
    if (p.kslice > 4096) return fail(ASRQ_ERR_LIMIT, "w%da16 gemv: K slice %d too long", bits, p.kslice);
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

// ---------------------------------------------------------------------------------------------
// asrq_w4a16_gemv_static: the W4A16 decode kernel for callers that cannot allocate device memory.
//
// Some hosts of this library have no way to obtain a workspace: a plugin that is handed input and
// output buffers by an inference server and is forbidden to call cudaMalloc on the request path, a
// real-time audio callback, or code that runs after the application has frozen its memory pools.
// For them the split-K scratch (status block, tile counters, fp32 partial sums) lives in a
// file-scope device array that every GPU loading the library holds until the process exits.
//
// The array's name is only a host-side handle: its device address is fetched once per device with
// cudaGetSymbolAddress (by the first call made with that device current -- make that first call
// before any stream capture) and that address is what the kernel receives.  The entry point calls
// no cudaMalloc, cudaFree or any other allocating routine.  All calls on a device share the one
// array: the counters and the status block are cleared on the stream at the start of every call,
// and two calls that overlap on the GPU (different streams) race on it -- serialise them.
// Limits: N <= 8192 and at most 8 K slices, which bounds the array at 16 640 + 4 Mi bytes.
// ---------------------------------------------------------------------------------------------
#include <mutex>

namespace asrq {

int check_a16_common(const char* who, const void* x, const uint8_t* w, const void* scales, const void* zeros, void* y,
                     int64_t M, int64_t N, int64_t K, int dtype, void* workspace);
int current_device_sm_count(int* sm_count);

constexpr int64_t kStaticMaxN = 8192;
constexpr int kStaticMaxSplit = 8;
constexpr size_t kStaticScratchBytes = kPartialOffset + size_t(kStaticMaxSplit) * 16 * kStaticMaxN * sizeof(float);

static __device__ __align__(256) unsigned char g_gemv_scratch[kStaticScratchBytes];

static std::mutex g_scratch_mutex;
static void* g_scratch_ptr[64];  // device address of g_gemv_scratch, per device ordinal

static int static_scratch(void** out) {
  int dev = 0;
  ASRQ_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(ASRQ_ERR_DEVICE, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (!g_scratch_ptr[dev]) {
    void* p = nullptr;
    ASRQ_CUDA_TRY(cudaGetSymbolAddress(&p, g_gemv_scratch));
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return ASRQ_OK;
}

}  // namespace asrq

#pragma GCC visibility push(default)
extern "C" int asrq_w4a16_gemv_static(const void* x, const uint8_t* w, const void* scales, const void* zeros,
                                      const void* bias, void* y, int64_t M, int64_t N, int64_t K, int group_size,
                                      int dtype, void* stream) {
  using namespace asrq;
  last_error().clear();
  int rc = check_a16_common("asrq_w4a16_gemv_static", x, w, scales, zeros, y, M, N, K, dtype,
                            /*workspace placeholder, checked non-NULL only*/ const_cast<void*>(x));
  if (rc) return rc;
  if (N > kStaticMaxN)
    return fail(ASRQ_ERR_LIMIT,
                "asrq_w4a16_gemv_static: N=%lld exceeds the built-in scratch (N <= %lld); use asrq_w4a16_gemv with a "
                "caller-provided workspace", (long long)N, (long long)kStaticMaxN);
  int sms = 0;
  if ((rc = current_device_sm_count(&sms))) return rc;
  if (M == 0) return ASRQ_OK;
  void* scratch = nullptr;
  if ((rc = static_scratch(&scratch))) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // the array keeps whatever the previous call left: status block and tile counters must start at zero
  ASRQ_CUDA_TRY(cudaMemsetAsync(scratch, 0, kPartialOffset, st));
  return gemv_a16_splitk(4, x, w, scales, zeros, bias, y, M, N, K, group_size, dtype, scratch, kStaticScratchBytes, sms, st,
                  kStaticMaxSplit);
}
#pragma GCC visibility pop
