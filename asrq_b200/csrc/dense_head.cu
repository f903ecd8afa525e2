// The floating-point output head of a decoding step: y[M, N] = x[M, K] . W[N, K]^T for M <= 32 tokens and a
// vocabulary-sized N (Whisper's proj_out 1280 -> 51 866, Qwen3's lm_head 2048 -> 151 936; the reference keeps
// these layers as nn.Linear: asrq/models/transformers/whisper.py:268, asrq/models/nemo/canary_qwen.py:179).
//
// Bound: HBM (the weight is read once: 133 MB and 622 MB for the two heads above, against a few hundred KB of
// activations and logits).  The decode kernel's skeleton without the unpacking: a warp owns 16 weight rows, every
// lane reads 16 bytes of rows g and g + 8 per 32-wide K step straight from global memory (its own fragment of
// mma.sync.m16n8k16 under a fixed permutation of k inside the step, which the activation fragments follow), the
// activations sit in shared memory for the whole block, accumulation in fp32.  Four steps of loads are in flight
// per warp before the first is used.
#include <algorithm>

#include "common.cuh"

namespace asrq {

int ensure_dynamic_smem(const void* kernel, size_t bytes);

namespace {

constexpr int kHeadWarps = 12;
constexpr int kHeadTokens = 32;  // per launch: four token tiles of eight
constexpr int kHeadAhead = 4;    // K steps of weight loads in flight per warp

__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1, bool bf16) {
  if (bf16) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}

__device__ __forceinline__ uint4 ldg_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// x: M x K, w: N x K, y: M x N, all 16-bit of one type; K a multiple of 32; shared memory: dense_head_smem(K) bytes
template <bool BF16>
__global__ void __launch_bounds__(32 * kHeadWarps, 2)
dense_head_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ w, uint16_t* __restrict__ y, int M, int N, int K) {
  extern __shared__ __align__(16) uint16_t xs[];
  // row pitch = 64 bytes modulo 128: the eight lanes of a quarter warp (two token rows x four 16-byte pieces) then
  // read eight distinct 16-byte bank groups
  const int pitch = K + ((K & 63) ? 0 : 32);
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int n_tiles = (N + 15) / 16;
  const int steps = K / 32;
  int tile = blockIdx.x * kHeadWarps + warp;
  const int tile_stride = gridDim.x * kHeadWarps;

  // the weights do not depend on the kernel before this one on the stream: the first loads go out before the wait
  uint4 wa[kHeadAhead], wb[kHeadAhead];
  auto rows_of = [&](int tl, const uint16_t*& ra, const uint16_t*& rb) {
    const int r0 = tl * 16 + g, r1 = r0 + 8;
    ra = w + size_t(min(r0, N - 1)) * K + 8 * t;  // rows past the end read the last row; their results are not stored
    rb = w + size_t(min(r1, N - 1)) * K + 8 * t;
  };
  const uint16_t *ra = w, *rb = w;
  if (tile < n_tiles) {
    rows_of(tile, ra, rb);
#pragma unroll
    for (int i = 0; i < kHeadAhead; ++i) {
      if (i < steps) {
        wa[i] = ldg_stream16(ra + 32 * i);
        wb[i] = ldg_stream16(rb + 32 * i);
      }
    }
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
  // activations -> shared memory (rows beyond M are zero)
  for (int i = threadIdx.x; i < kHeadTokens * (K / 8); i += blockDim.x) {
    const int r = i / (K / 8), c = (i - r * (K / 8)) * 8;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < M) v = *reinterpret_cast<const uint4*>(x + size_t(r) * K + c);
    *reinterpret_cast<uint4*>(xs + r * pitch + c) = v;
  }
  __syncthreads();

  for (; tile < n_tiles; tile += tile_stride) {
    float acc[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;
    for (int s0 = 0; s0 < steps; s0 += kHeadAhead) {
#pragma unroll
      for (int i = 0; i < kHeadAhead; ++i) {
        const int s = s0 + i;
        if (s < steps) {
          const uint4 a = wa[i], b = wb[i];
          if (s + kHeadAhead < steps) {  // refill this slot with the step four ahead
            wa[i] = ldg_stream16(ra + 32 * (s + kHeadAhead));
            wb[i] = ldg_stream16(rb + 32 * (s + kHeadAhead));
          }
          // k slots (2t, 2t+1 | 2t+8, 2t+9) of the two MMAs of this step hold actual k = 8t + (0,1 | 2,3) and 8t + (4,5 | 6,7)
          const uint32_t a0[4] = {a.x, b.x, a.y, b.y}, a1[4] = {a.z, b.z, a.w, b.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint4 xv = *reinterpret_cast<const uint4*>(xs + (8 * j + g) * pitch + 32 * s + 8 * t);
            mma16816(acc[j], a0, xv.x, xv.y, BF16);
            mma16816(acc[j], a1, xv.z, xv.w, BF16);
          }
        }
      }
    }
    // the next tile's first loads go out before this tile's stores
    const int next = tile + tile_stride;
    if (next < n_tiles) {
      rows_of(next, ra, rb);
#pragma unroll
      for (int i = 0; i < kHeadAhead; ++i) {
        if (i < steps) {
          wa[i] = ldg_stream16(ra + 32 * i);
          wb[i] = ldg_stream16(rb + 32 * i);
        }
      }
    }
    const int r0 = tile * 16 + g, r1 = r0 + 8;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int m0 = 8 * j + 2 * t, m1 = m0 + 1;
      if (m0 < M) {
        if (r0 < N) y[size_t(m0) * N + r0] = float_to_out16(acc[j][0], BF16);
        if (r1 < N) y[size_t(m0) * N + r1] = float_to_out16(acc[j][2], BF16);
      }
      if (m1 < M) {
        if (r0 < N) y[size_t(m1) * N + r0] = float_to_out16(acc[j][1], BF16);
        if (r1 < N) y[size_t(m1) * N + r1] = float_to_out16(acc[j][3], BF16);
      }
    }
  }
}

}  // namespace

size_t dense_head_smem(int64_t K) { return size_t(kHeadTokens) * size_t(K + ((K & 63) ? 0 : 32)) * 2; }

int dense_head(const void* x, const void* w, void* y, int64_t M, int64_t N, int64_t K, int dtype, int sm_count, cudaStream_t stream) {
  const size_t smem = dense_head_smem(K);
  const bool bf16 = dtype == ASRQ_BF16;
  auto kern = bf16 ? dense_head_kernel<true> : dense_head_kernel<false>;
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem)) return rc;
  const int blocks_per_sm = smem <= 100 * 1024 ? 2 : 1;
  const int64_t n_tiles = (N + 15) / 16;
  const int grid = int(std::min<int64_t>(int64_t(sm_count) * blocks_per_sm, (n_tiles + kHeadWarps - 1) / kHeadWarps));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(32 * kHeadWarps);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = option(kOptNoPdl) ? 0 : 1;
  ASRQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, static_cast<const uint16_t*>(x), static_cast<const uint16_t*>(w),
                                   static_cast<uint16_t*>(y), int(M), int(N), int(K)));
  return ASRQ_OK;
}

}  // namespace asrq
