// Decode batches on the tensor cores: y[M,N] = x[M,K] . dequant(W)[N,K]^T (+ bias) for 17 <= M <= 64.
//
// At these token counts the mma.sync decode kernel is bound by the legacy MMA pipe (one m16n8k16 per ~13
// clocks per scheduler, one per 8 tokens per 256 codes), and the persistent prefill kernel by its fixed
// costs (set-up, first TMA and first dequantisation pass before the first MMA, an epilogue nothing
// overlaps): 10-15 us for a 1-3 MB layer either way.  This kernel is built for a CHAIN of such layers:
//
//   * a block owns ONE work item -- a 128-feature tile and a part of K of at most 12 blocks of 64 -- so all
//     of its packed weights (<= 48 KB) and all of its activation tiles fit shared memory at once;
//   * it triggers its dependents as its first instruction and is small enough (448 threads, <= 73
//     registers, < 113 KB) for two launches to share an SM.  Packed weights are fetched by TMA and the
//     first three K blocks are dequantised BEFORE griddepcontrol.wait: weights do not depend on the
//     kernel before, so the next launch's weight traffic and unpacking run under this launch's tail;
//   * after the wait only the activation tiles (tokens as the MMA's N dimension: 32 or 64 TMEM columns)
//     are fetched, all at once; tcgen05.mma kind::f16 128 x BT x 16, fp32 accumulator in tensor memory;
//   * K parts of a tile meet through the workspace: fp32 partial tiles and one arrival counter per tile.
//     The last BLOCK to arrive adds the parts in part order (results do not depend on timing) with all
//     of its threads, every thread's loads of all parts in flight together, adds the bias, converts,
//     stores, and leaves the counter at zero.  (With one warp per lane quadrant doing this, one L2 round
//     trip per part in turn, the reduction took 8 of a launch's 9.6 us.)
//
// Roles (14 warps): warp 0 TMA producer, warp 1 MMA issuer (owns the tensor-memory allocation), warps
// 2-13 three dequant groups of 128 threads (one weight row per thread, group d takes K blocks d, d+3, ...
// and owns A slot d); the first group (warps 2-5, one per TMEM lane quadrant) then runs the epilogue.
// No TMA multicast.  Every wait is bounded.
#include <algorithm>

#include "dequant.cuh"
#include "tcgen05.cuh"

namespace asrq {

int ensure_dynamic_smem(const void* kernel, size_t bytes);

namespace {

constexpr int kSkWarps = 14;
constexpr int kSkThreads = 32 * kSkWarps;
constexpr int kSkMaxKb = 12;                    // K blocks of 64 per work item
constexpr int kSkMaxSplit = 8;
constexpr uint32_t kSkATile = 128 * 128;        // one dequantised A slot: 128 rows x 64 16-bit elements
constexpr uint32_t kSkWSlot = 4096;             // packed weights of one K block (<= 128 x 32 B)

struct SkinnyParams {
  const __half* scales;
  const __half* zeros;
  const __half* bias;
  const uint16_t* residual;  // fused epilogue: y = residual + layer output (NULL: none)
  int act;                   // fused epilogue: activation on the layer output (kActNone / kActGelu)
  uint16_t* y;
  unsigned* status;
  float* partials;     // [tile][part][bt tokens][128 features]
  unsigned* counters;  // one per tile, zero between launches
  int M, N, K, group_size, groups_per_row, bt, ksplit, nkb, kbmax;
  unsigned long long* trace;  // builds with -DASRQ_TRACE: 8 globaltimer marks per block, NULL otherwise
};

#ifdef ASRQ_TRACE
#define SK_MARK(i)                                                                   \
  do {                                                                               \
    if (p.trace) {                                                                   \
      unsigned long long t__;                                                        \
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t__)::"memory");              \
      p.trace[size_t(blockIdx.x) * 8 + (i)] = t__;                                   \
    }                                                                                \
  } while (0)
#else
#define SK_MARK(i) do { } while (0)
#endif

template <int BITS, bool BF16>
__global__ void __launch_bounds__(kSkThreads, 2)
gemm_a16_skinny_kernel(const __grid_constant__ CUtensorMap tmx, const __grid_constant__ CUtensorMap tmw,
                       const SkinnyParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[kSkMaxKb + 8];
  __shared__ int is_last;
  __shared__ uint32_t tmem_slot;
  // the next launch on the stream may start its own set-up, weight fetch and first dequantisation now
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (threadIdx.x == 0) SK_MARK(0);
  const uint32_t raw_addr = tc::smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw_addr);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // work item: feature tile ft, K part ks (parts of a tile on neighbouring blocks)
  const int ks = blockIdx.x % p.ksplit, ft = blockIdx.x / p.ksplit;
  const int kb0 = ks * p.nkb / p.ksplit, kb1 = (ks + 1) * p.nkb / p.ksplit, kbn = kb1 - kb0;
  const uint32_t xbytes = uint32_t(p.bt) * 128u;
  // [A slot x 3] [activation tile x kbmax] [packed weights x kbmax]
  const uint32_t x_base = 3 * kSkATile, w_base = x_base + uint32_t(p.kbmax) * xbytes;
  constexpr uint32_t wbytes = 128u * 8u * BITS;
  const uint32_t bar0 = tc::smem_u32(bars);
  auto w_bar = [&](int kb) { return bar0 + 8u * kb; };
  const uint32_t x_bar = bar0 + 8u * kSkMaxKb, accf_bar = x_bar + 8u;
  auto deq_bar = [&](int a) { return x_bar + 16u + 8u * a; };
  auto afree_bar = [&](int a) { return x_bar + 40u + 8u * a; };
  const uint32_t tmem_cols = p.bt <= 32 ? 32u : 64u;

  if (threadIdx.x == 0) {
    for (int kb = 0; kb < kSkMaxKb; ++kb) tc::mbar_init(w_bar(kb), 1);
    tc::mbar_init(x_bar, 1);
    tc::mbar_init(accf_bar, 1);
    for (int a = 0; a < 3; ++a) {
      tc::mbar_init(deq_bar(a), 128);
      tc::mbar_init(afree_bar(a), 1);
    }
    tc::fence_barrier_init();
    tc::fence_proxy_async_smem();
    tc::prefetch_tmap(&tmx);
    tc::prefetch_tmap(&tmw);
  }
  if (warp == 1) {
    tc::tmem_alloc(tc::smem_u32(&tmem_slot), tmem_cols);
    tc::tmem_relinquish();
  }
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&tmem_slot);
  if (threadIdx.x == 0) SK_MARK(1);

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      for (int kb = 0; kb < kbn; ++kb) {  // weights: constants, fetched ahead of the stream dependency
        tc::mbar_arrive_expect_tx(w_bar(kb), wbytes);
        tc::tma_load_2d(base + w_base + kb * kSkWSlot, &tmw, (kb0 + kb) * 8 * BITS, ft * 128, w_bar(kb));
      }
      SK_MARK(2);
      // activations belong to this kernel only once its predecessor on the stream is complete
      asm volatile("griddepcontrol.wait;" ::: "memory");
      SK_MARK(3);
      tc::mbar_arrive_expect_tx(x_bar, uint32_t(kbn) * xbytes);
      for (int kb = 0; kb < kbn; ++kb) tc::tma_load_2d(base + x_base + kb * xbytes, &tmx, (kb0 + kb) * 64, 0, x_bar);
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    const bool el = tc::elect_one();
    const uint32_t idesc = tc::instr_desc(1u, BF16 ? 1u : 0u, 128u, uint32_t(p.bt));
    bool ok = tc::mbar_wait_spin(x_bar, 0u, p.status, 31);
    if (lane == 0) SK_MARK(4);
    for (int kb = 0; kb < kbn && ok; ++kb) {
      const int a = kb % 3;
      ok = tc::mbar_wait_spin(deq_bar(a), uint32_t(kb / 3) & 1u, p.status, 32);
      if (!ok) break;
      tc::fence_after_sync();
      const uint64_t da = tc::smem_desc_sw128(base + a * kSkATile);
      const uint64_t db = tc::smem_desc_sw128(base + x_base + kb * xbytes);
      if (el) {
        tc::mma_f16(tmem_base, da, db, idesc, uint32_t(kb != 0));
        tc::mma_f16(tmem_base, da + 2, db + 2, idesc, 1u);
        tc::mma_f16(tmem_base, da + 4, db + 4, idesc, 1u);
        tc::mma_f16(tmem_base, da + 6, db + 6, idesc, 1u);
        tc::mma_commit(afree_bar(a));
        if (kb + 1 == kbn) tc::mma_commit(accf_bar);
      }
    }
    if (lane == 0) SK_MARK(5);
  } else {
    // ------------------------------ dequant (three groups) ------------------------------
    const int dgroup = (warp - 2) >> 2;
    const int t = ((warp - 2) & 3) * 32 + lane;  // weight row inside the tile
    const int kbpg = p.group_size / 64;
    bool ok = true;
    for (int kb = dgroup; kb < kbn && ok; kb += 3) {
      const int gi = (kb0 + kb) / kbpg;
      const size_t idx = (size_t(ft) * 128 + t) * p.groups_per_row + gi;
      const __half sh = __ldg(p.scales + idx), zh = __ldg(p.zeros + idx);
      uint32_t s2, z2;
      if (BF16) {
        s2 = __float_as_uint(__half2float(sh));
        z2 = __float_as_uint(__half2float(zh));
      } else {
        s2 = h2_as_u32(__half2half2(sh));
        z2 = h2_as_u32(__half2half2(zh));
      }
      // the slot's previous K block (three back) must have been consumed by its MMAs
      if (kb >= 3) ok = tc::mbar_wait(afree_bar(dgroup), uint32_t(kb / 3 - 1) & 1u, p.status, 33);
      ok = ok && tc::mbar_wait(w_bar(kb), 0u, p.status, 34);
      if (!ok) break;
      const uint4* wp = reinterpret_cast<const uint4*>(smem + w_base + kb * kSkWSlot + t * (8 * BITS));
      uint8_t* arow = smem + dgroup * kSkATile + t * 128;
      constexpr int NV = BITS / 2;  // 16-byte vectors of packed weights per row per K block
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        const uint4 qv = wp[v];
        const uint32_t qw[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          constexpr int PW = 32 / BITS / 2;  // output pairs per word: 4 or 8
          uint32_t o[PW];
          dequant_word<BITS, BF16>(qw[j], s2, z2, o);
#pragma unroll
          for (int cc = 0; cc < PW / 4; ++cc) {
            const int chunk = (v * 4 + j) * (PW / 4) + cc;  // 16-byte chunk (8 elements) in the row
            *reinterpret_cast<uint4*>(arow + ((chunk ^ (t & 7)) << 4)) =
                make_uint4(o[4 * cc], o[4 * cc + 1], o[4 * cc + 2], o[4 * cc + 3]);
          }
        }
      }
      tc::fence_proxy_async_smem();
      tc::mbar_arrive(deq_bar(dgroup));
    }
    ok = __all_sync(0xffffffffu, ok);  // a wait that gave up in any lane ends the warp's work
    if (dgroup == 0 && ok) {
      // ------------------------------ epilogue (warps 2-5: lane quadrants 2, 3, 0, 1) ------------------------------
      const int qd = warp & 3;
      const int f = ft * 128 + qd * 32 + lane;
      const float bias = p.bias ? __half2float(__ldg(p.bias + f)) : 0.f;
      // one decision for the warp, and the lanes together again after the polling loop: the tensor-memory loads
      // below are warp-wide instructions
      if (__all_sync(0xffffffffu, tc::mbar_wait(accf_bar, 0u, p.status, 35))) {
        __syncwarp();
        tc::fence_after_sync();
        if (warp == 2 && lane == 0) SK_MARK(6);
        const uint32_t taddr = tmem_base + (uint32_t(qd * 32) << 16);
        if (p.ksplit == 1) {
          for (int ch = 0; ch < p.bt / 32; ++ch) {
            uint32_t r[32];
            tc::tmem_ld_32x32(taddr + ch * 32, r);
            tc::tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (ch * 32 + j < p.M) {
                const size_t idx = size_t(ch * 32 + j) * p.N + f;
                p.y[idx] = finish16(__uint_as_float(r[j]) + bias, p.act, p.residual, idx, BF16);
              }
          }
        } else {
          // this block's part of the tile, fp32 [token][128 features]: a warp writes 128 contiguous bytes per token
          float* part = p.partials + (size_t(ft) * p.ksplit + ks) * size_t(p.bt) * 128 + qd * 32 + lane;
          for (int ch = 0; ch < p.bt / 32; ++ch) {
            uint32_t r[32];
            tc::tmem_ld_32x32(taddr + ch * 32, r);
            tc::tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) __stcg(part + size_t(ch * 32 + j) * 128, __uint_as_float(r[j]));
          }
        }
      }
    }
  }

  __syncwarp();
  tc::fence_before_sync();
  __syncthreads();
  if (p.ksplit > 1) {
    // the block that arrives last for its tile adds the parts; which block that is depends on timing, the
    // order of the additions does not.  Ordering as in a grid-wide barrier: the block's stores are ordered before
    // thread 0's fence by the block barrier above, the fence is cumulative, and the last block's loads follow
    // thread 0's second fence through the barrier below -- one thread fences, not 448 (1.5 % of a decode step).
    if (threadIdx.x == 0) {
      __threadfence();
      is_last = atomicAdd(p.counters + ft, 1u) == unsigned(p.ksplit - 1);
      __threadfence();
    }
    __syncthreads();
    if (is_last) {
      const int total = p.bt * 128;
      const float* part0 = p.partials + size_t(ft) * p.ksplit * total;
      // four features per thread and step, all parts' loads of a step in flight together: the reduction costs
      // three L2 round trips (one load at a time per part it cost nine, 6 us)
      for (int o4 = threadIdx.x; o4 < total / 4; o4 += kSkThreads) {
        float4 a[kSkMaxSplit];
#pragma unroll
        for (int s = 0; s < kSkMaxSplit; ++s)
          if (s < p.ksplit) a[s] = __ldcg(reinterpret_cast<const float4*>(part0 + size_t(s) * total) + o4);
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int s = 0; s < kSkMaxSplit; ++s)
          if (s < p.ksplit) {
            v.x += a[s].x; v.y += a[s].y; v.z += a[s].z; v.w += a[s].w;
          }
        const int tok = o4 >> 5, f = ft * 128 + (o4 & 31) * 4;
        if (tok < p.M) {
          if (p.bias) {
            const uint2 b = __ldg(reinterpret_cast<const uint2*>(p.bias + f));
            const float2 b01 = __half22float2(u32_as_h2(b.x)), b23 = __half22float2(u32_as_h2(b.y));
            v.x += b01.x; v.y += b01.y; v.z += b23.x; v.w += b23.y;
          }
          const size_t idx = size_t(tok) * p.N + f;
          uint2 out;
          out.x = uint32_t(finish16(v.x, p.act, p.residual, idx, BF16)) | (uint32_t(finish16(v.y, p.act, p.residual, idx + 1, BF16)) << 16);
          out.y = uint32_t(finish16(v.z, p.act, p.residual, idx + 2, BF16)) | (uint32_t(finish16(v.w, p.act, p.residual, idx + 3, BF16)) << 16);
          *reinterpret_cast<uint2*>(p.y + idx) = out;
        }
      }
      if (threadIdx.x == 0) p.counters[ft] = 0u;
    }
  }
  if (threadIdx.x == 0) SK_MARK(7);
  if (warp == 1) {
    tc::fence_after_sync();
    tc::tmem_dealloc(tmem_base, tmem_cols);
  }
}

struct SkinnyPlan {
  int bt, ksplit, nkb, kbmax, grid;
  size_t smem;
};

bool skinny_plan(int64_t M, int64_t N, int64_t K, int group_size, int sm_count, size_t workspace_bytes, SkinnyPlan* pl) {
  if (M < 1 || M > 64 || N % 128 || K % 64 || group_size <= 0 || group_size % 64 || K % group_size) return false;
  if (workspace_bytes < kStatusBytes) return false;
  const int64_t tiles = N / 128, nkb = K / 64;
  const int bt = M <= 32 ? 32 : 64;
  // parts of K: as many as fill the machine in one wave, at most 8, at least enough for kSkMaxKb K blocks per part
  int64_t split = std::max<int64_t>((nkb + kSkMaxKb - 1) / kSkMaxKb, std::min<int64_t>(sm_count / tiles, kSkMaxSplit));
  split = std::max<int64_t>(1, std::min<int64_t>(split, nkb));
  if (split > kSkMaxSplit || tiles * split > sm_count) return false;
  if (tiles > int64_t(kCounterBytes / sizeof(unsigned))) return false;
  if (split > 1 && workspace_bytes < kPartialOffset + size_t(4) * N * bt * split) return false;
  pl->bt = bt;
  pl->ksplit = int(split);
  pl->nkb = int(nkb);
  pl->kbmax = int((nkb + split - 1) / split);
  pl->grid = int(tiles * split);
  pl->smem = 1024 + 3 * kSkATile + size_t(pl->kbmax) * (size_t(bt) * 128 + kSkWSlot);
  return pl->smem <= 200 * 1024;
}

template <int BITS, bool BF16>
int launch_skinny(const CUtensorMap& tmx, const CUtensorMap& tmw, const SkinnyParams& p, int grid, size_t smem,
                  cudaStream_t stream) {
  auto kern = gemm_a16_skinny_kernel<BITS, BF16>;
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem)) return rc;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kSkThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = option(kOptNoPdl) ? 0 : 1;
  ASRQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, tmx, tmw, p));
  return ASRQ_OK;
}

}  // namespace

bool gemm_a16_skinny_supports(int64_t M, int64_t N, int64_t K, int group_size, int sm_count, size_t workspace_bytes) {
  SkinnyPlan pl;
  return skinny_plan(M, N, K, group_size, sm_count, workspace_bytes, &pl);
}

int gemm_a16_skinny(int bits, const void* x, const uint8_t* w, const void* scales, const void* zeros, const void* bias,
                    void* y, int64_t M, int64_t N, int64_t K, int group_size, int dtype, void* workspace,
                    size_t workspace_bytes, int sm_count, cudaStream_t stream, const Epilogue& ep) {
  SkinnyPlan pl;
  if (!skinny_plan(M, N, K, group_size, sm_count, workspace_bytes, &pl))
    return fail(ASRQ_ERR_SHAPE, "w%da16 skinny gemm: unsupported shape M=%lld N=%lld K=%lld g=%d", bits, (long long)M,
                (long long)N, (long long)K, group_size);
  if (!aligned16(x) || !aligned16(w)) return fail(ASRQ_ERR_ALIGN, "w%da16 skinny gemm: x and w must be 16-byte aligned", bits);
  SkinnyParams p;
  p.scales = static_cast<const __half*>(scales);
  p.zeros = static_cast<const __half*>(zeros);
  p.bias = static_cast<const __half*>(bias);
  p.residual = static_cast<const uint16_t*>(ep.residual);
  p.act = ep.act;
  p.y = static_cast<uint16_t*>(y);
  p.status = static_cast<unsigned*>(workspace);
  p.partials = reinterpret_cast<float*>(static_cast<char*>(workspace) + kPartialOffset);
  p.counters = reinterpret_cast<unsigned*>(static_cast<char*>(workspace) + kStatusBytes);
  p.M = int(M);
  p.N = int(N);
  p.K = int(K);
  p.group_size = group_size;
  p.groups_per_row = int(K / group_size);
  p.bt = pl.bt;
  p.ksplit = pl.ksplit;
  p.nkb = pl.nkb;
  p.kbmax = pl.kbmax;
  p.trace = nullptr;
#ifdef ASRQ_TRACE
  if (option(kOptTrace) && workspace_bytes >= (8u << 20)) {  // marks of the launches since the option last changed
    static int launch_no = 0;
    static unsigned gen = 0;
    if (gen != options_generation()) { gen = options_generation(); launch_no = 0; }
    p.trace = reinterpret_cast<unsigned long long*>(static_cast<char*>(workspace) + (4u << 20)) + size_t(launch_no % 64) * 148 * 8;
    ++launch_no;
  }
#endif
  const bool bf16 = dtype == ASRQ_BF16;
  CUtensorMap tmx, tmw;
  int rc = make_tmap_2d(&tmx, x, 2, bf16, uint64_t(K), uint64_t(M), 64, uint32_t(pl.bt), true);
  if (rc) return rc;
  rc = make_tmap_2d(&tmw, w, 1, false, uint64_t(K) * bits / 8, uint64_t(N), uint32_t(8 * bits), 128, false);
  if (rc) return rc;
  if (bits == 4)
    return bf16 ? launch_skinny<4, true>(tmx, tmw, p, pl.grid, pl.smem, stream)
                : launch_skinny<4, false>(tmx, tmw, p, pl.grid, pl.smem, stream);
  return bf16 ? launch_skinny<2, true>(tmx, tmw, p, pl.grid, pl.smem, stream)
              : launch_skinny<2, false>(tmx, tmw, p, pl.grid, pl.smem, stream);
}

}  // namespace asrq
