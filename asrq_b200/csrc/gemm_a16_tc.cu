// Prefill / encoder path: y[M,N] = x[M,K] . dequant(W)[N,K]^T (+ bias) for large M.
//
// The weight tile is the MMA "A" operand (128 output features = 128 TMEM lanes), the
// activation tile is the "B" operand (BT tokens = BT TMEM columns, BT <= 256 chosen by the
// host).  One persistent block per SM, twenty warps (see kTcDequantPos for who is who):
//
//   1 warp      TMA producer: per 64-wide K block, one tile of activations
//               (BT x 64, 128-byte swizzle) and one tile of packed weights (128 rows).
//   1 warp      MMA issuer: tcgen05.mma kind::f16, 4 x (128 x BT x 16) per K block, fp32
//               accumulators in TMEM (two buffers of 256 columns).
//   12 warps    dequant, three groups of four warps; group d takes the K blocks with
//               index % 3 == d and owns A slot d, one weight row per thread: packed words ->
//               fp16/bf16 in registers -> q*scale+zero -> the swizzled K-major slot in shared
//               memory.  Three slots keep the chain "MMA of block i done -> slot free ->
//               dequant of block i+3 -> MMA of block i+3" two MMA blocks slack.  (A variant with
//               the A operand written to tensor memory by tcgen05.st measured the same speed but
//               leaves room for only two slots beside 2 x 224 accumulator columns.)
//   4 warps     epilogue: tcgen05.ld of the previous tile's accumulator, + bias,
//               convert, store, while the next tile's main loop runs.
//
// Rings: full[s] (TMA landed) -> deq[a] (A slot written) -> MMA -> empty[s] (TMA stage
// reusable) and afree[a] (A slot reusable); accf[b]/acce[b] hand the accumulator buffers
// back and forth.  Every wait is bounded (tcgen05.cuh).
#include <algorithm>
#include <cstdlib>

#include "dequant.cuh"
#include "tcgen05.cuh"

namespace asrq {

int ensure_dynamic_smem(const void* kernel, size_t bytes);

struct GemmTcParams {
  const __half* scales;
  const __half* zeros;
  const __half* bias;
  uint16_t* y;
  unsigned* status;
  long long* trace;  // builds with -DASRQ_TRACE: when not NULL, block 0 records clock64() at pipeline milestones
  float* partials;    // split-K: fp32 partial tiles [tile][split][bt tokens][128 features]
  unsigned* counters; // split-K: one arrival counter per (tile, lane quadrant), zero between launches
  int M, N, K, group_size, groups_per_row, bt, nstages, n_ftiles, n_ttiles;
  int ksplit;         // parts the K blocks of a tile are divided into (1: no split)
};

// One unit of work of a block: the K blocks [kb0, kb1) of output tile (ft, tt).  Items are numbered
// with the split index fastest, so the parts of a tile run on neighbouring blocks at the same time.
struct TcItem {
  int ft, tt, ks, kb0, kb1;
};
__device__ __forceinline__ TcItem tc_item(const GemmTcParams& p, int w, int nkb) {
  TcItem it;
  if (p.ksplit == 1) {
    it.ks = 0;
    it.kb0 = 0;
    it.kb1 = nkb;
  } else {
    it.ks = w % p.ksplit;
    w /= p.ksplit;
    it.kb0 = it.ks * nkb / p.ksplit;
    it.kb1 = (it.ks + 1) * nkb / p.ksplit;
  }
  it.ft = w % p.n_ftiles;
  it.tt = w / p.n_ftiles;
  return it;
}

constexpr int kTcDequantGroups = 3;
constexpr int kTcWarps = 20;
constexpr int kTcThreads = 32 * kTcWarps;
// Warp roles.  A warp with index w issues on scheduler w % 4.  The MMA thread's instruction stream
// is the critical path of the kernel (every tcgen05.mma / commit / barrier poll costs it 40-100
// cycles), so scheduler 1 hosts only warp 1 (MMA), the light TMA producer (warp 9) and the one
// epilogue warp that must live there to read TMEM lanes 32-63 (warp 5); warps 13 and 17 idle.
constexpr int kTcMmaWarp = 1, kTcProducerWarp = 9;
// position of a warp among the twelve dequant warps (-1: not a dequant warp)
__constant__ int8_t kTcDequantPos[kTcWarps] = {0, -1, -1, -1, -1, -1, 1, 2, 3, -1, 4, 5, 6, -1, 7, 8, 9, -1, 10, 11};
constexpr int kTcMaxStages = 8;
constexpr int64_t kTcMaxSplit = 8;  // the last block to arrive reads every part: one trip to L2 each
constexpr uint32_t kATileBytes = 128 * 128;  // one dequantised A slot: 128 rows x 64 16-bit elements
constexpr uint32_t kWSlotBytes = 4096;       // packed weights of one K block (<= 128 x 32 B)

template <int BITS, bool BF16>
__global__ void __launch_bounds__(kTcThreads, 1)
gemm_a16_tc_kernel(const __grid_constant__ CUtensorMap tmx, const __grid_constant__ CUtensorMap tmw,
                   const GemmTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[2 * kTcMaxStages + 2 * kTcDequantGroups + 4];
  __shared__ uint32_t tmem_slot;

  const uint32_t raw_addr = tc::smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw_addr);
  const uint32_t xbytes = uint32_t(p.bt) * 128u;
  // [A slot x kTcDequantGroups] [TMA stage: activations (bt x 128 B) + packed weights] x nstages
  constexpr uint32_t a_ring_bytes = kTcDequantGroups * kATileBytes;
  const uint32_t stage_bytes = xbytes + kWSlotBytes;
  constexpr uint32_t wbytes = 128u * 8u * BITS;
  const int nst = p.nstages;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t bar0 = tc::smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (kTcMaxStages + s); };
  auto deq_bar = [&](int a) { return bar0 + 8u * (2 * kTcMaxStages + a); };                       // A slot written
  auto afree_bar = [&](int a) { return bar0 + 8u * (2 * kTcMaxStages + kTcDequantGroups + a); };  // A slot consumed
  auto accf_bar = [&](int b) { return bar0 + 8u * (2 * kTcMaxStages + 2 * kTcDequantGroups + b); };
  auto acce_bar = [&](int b) { return bar0 + 8u * (2 * kTcMaxStages + 2 * kTcDequantGroups + 2 + b); };

  if (threadIdx.x == 0) {
    for (int s = 0; s < nst; ++s) {
      tc::mbar_init(full_bar(s), 1);
      tc::mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < kTcDequantGroups; ++a) {
      tc::mbar_init(deq_bar(a), 128);
      tc::mbar_init(afree_bar(a), 1);
    }
    for (int b = 0; b < 2; ++b) {
      tc::mbar_init(accf_bar(b), 1);
      tc::mbar_init(acce_bar(b), 128);
    }
    tc::fence_barrier_init();
    tc::fence_proxy_async_smem();
    tc::prefetch_tmap(&tmx);
    tc::prefetch_tmap(&tmw);
  }
  if (warp == kTcMmaWarp) {
    tc::tmem_alloc(tc::smem_u32(&tmem_slot), 512);
    tc::tmem_relinquish();
  }
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&tmem_slot);
  // Launched with programmatic stream serialisation: the set-up above may overlap the tail of the
  // kernel before; activations, workspace and output are touched only from here on.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");

  const int nkb = p.K / 64;
  const int nitems = p.n_ftiles * p.n_ttiles * p.ksplit;
#ifdef ASRQ_TRACE
  const bool tr = p.trace != nullptr && blockIdx.x == 0;
  auto mark = [&](int role, uint32_t i, int slot) {
    if (tr && i < 512) p.trace[(role * 512 + i) * 2 + slot] = clock64();
  };
#else
  auto mark = [](int, uint32_t, int) {};  // the shipped kernels carry no trace branches
#endif

  // Ring positions are carried as (index, phase) counters: the role loops below run on one
  // thread (or one warp per scheduler), where every integer division costs ~150 cycles of
  // dependent latency.
  const int dpos = kTcDequantPos[warp];
  if (warp == kTcProducerWarp) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      uint32_t it = 0, ph = 0;
      int s = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < nitems && ok; w += gridDim.x) {
        const TcItem item = tc_item(p, w, nkb);
        const int row_x = item.tt * p.bt, row_w = item.ft * 128;
        for (int kb = item.kb0; kb < item.kb1; ++kb, ++it) {
          if (!tc::mbar_wait(empty_bar(s), ph ^ 1u, p.status, 1)) { ok = false; break; }
          mark(0, it, 0);
          const uint32_t sb = base + a_ring_bytes + s * stage_bytes;
          tc::mbar_arrive_expect_tx(full_bar(s), xbytes + wbytes);
          tc::tma_load_2d(sb, &tmx, kb * 64, row_x, full_bar(s));
          tc::tma_load_2d(sb + xbytes, &tmw, kb * 8 * BITS, row_w, full_bar(s));
          mark(0, it, 1);
          if (++s == nst) { s = 0; ph ^= 1u; }
        }
      }
    }
  } else if (warp == kTcMmaWarp) {
    // ------------------------------ MMA issuer ------------------------------
    // tcgen05.mma issue is paced by execution (the queue is about one instruction deep), so the
    // pipe starves unless the next issue follows within one MMA time (~110 cycles, ~15 dependent
    // instructions of this lone thread).  All bookkeeping for the NEXT K block -- ring counters,
    // barrier waits -- is therefore placed between the four issues of the current one.
    {
      const bool el = tc::elect_one();
      const uint32_t idesc = tc::instr_desc(1u, BF16 ? 1u : 0u, 128u, uint32_t(p.bt));
      uint32_t it = 0, tcount = 0, ph = 0, dph = 0;
      int s = 0, a = 0;
      bool ok = nitems > int(blockIdx.x);
      if (ok) {
        ok = tc::mbar_wait_spin(acce_bar(0), 1u, p.status, 2) && tc::mbar_wait_spin(deq_bar(0), 0u, p.status, 4);
        tc::fence_after_sync();
      }
      for (int w = blockIdx.x; w < nitems && ok; w += gridDim.x, ++tcount) {
        const TcItem item = tc_item(p, w, nkb);
        const uint32_t buf = tcount & 1u;
        const uint32_t d_tmem = tmem_base + buf * 256u;
        const bool more_tiles = w + int(gridDim.x) < nitems;
        for (int kb = item.kb0; kb < item.kb1; ++kb, ++it) {
          mark(1, it, 0);
          // a K step of 16 elements = 32 bytes = +2 in the descriptors' 16-byte address field
          const uint64_t da = tc::smem_desc_sw128(base + a * kATileBytes);
          const uint64_t db = tc::smem_desc_sw128(base + a_ring_bytes + s * stage_bytes);
          if (el) tc::mma_f16(d_tmem, da, db, idesc, uint32_t(kb != item.kb0));
          // next K block's ring positions
          int s1 = s + 1, a1 = a + 1;
          uint32_t ph1 = ph, dph1 = dph;
          if (s1 == nst) { s1 = 0; ph1 ^= 1u; }
          if (a1 == kTcDequantGroups) { a1 = 0; dph1 ^= 1u; }
          const bool last_kb = kb + 1 == item.kb1;
          const bool have_next = !last_kb || more_tiles;
          if (el) tc::mma_f16(d_tmem, da + 2, db + 2, idesc, 1u);
          if (el) tc::mma_f16(d_tmem, da + 4, db + 4, idesc, 1u);
          // deq[a1] completing implies full[s1]: the dequant group of the next block waited for that
          // stage's TMA before it wrote the A slot and arrived (release), and this wait acquires it
          if (have_next) ok = tc::mbar_wait_spin(deq_bar(a1), dph1, p.status, 4);
          if (el) tc::mma_f16(d_tmem, da + 6, db + 6, idesc, 1u);
          // one commit frees both the TMA stage (producer) and the A slot (dequant group waits on
          // the empty barrier of the stage its previous block used)
          if (el) {
            tc::mma_commit(empty_bar(s));
            if (last_kb) tc::mma_commit(accf_bar(buf));
          }
          if (have_next && last_kb && ok) {  // the next tile's accumulator buffer must have been drained
            const uint32_t nt = tcount + 1;
            ok = tc::mbar_wait_spin(acce_bar(nt & 1u), ((nt >> 1) & 1u) ^ 1u, p.status, 2);
          }
          tc::fence_after_sync();
          s = s1; ph = ph1; a = a1; dph = dph1;
          if (!ok) break;
        }
      }
    }
  } else if (dpos >= 0) {
    // ------------------------------ dequant ------------------------------
    const int t = (dpos & 3) * 32 + lane;  // weight row inside the tile
    const int dgroup = dpos >> 2;          // this warp group takes K blocks dgroup, dgroup+3, ...
    constexpr int NDG = kTcDequantGroups;
    // position (item, K block) of the block being processed; `advance` moves a position NDG blocks
    // along this block's sequence of items (an item has at least one K block)
    int w = blockIdx.x;
    TcItem item = tc_item(p, w < nitems ? w : 0, nkb);
    int kb = item.kb0;
    auto advance = [&](int& aw, TcItem& ai, int& ak, int by) {
      ak += by;
      while (aw < nitems && ak >= ai.kb1) {
        const int over = ak - ai.kb1;
        aw += gridDim.x;
        if (aw < nitems) {
          ai = tc_item(p, aw, nkb);
          ak = ai.kb0 + over;
        }
      }
    };
    advance(w, item, kb, dgroup);
    int s = dgroup % nst;
    uint32_t ph = (dgroup / nst) & 1u, dph = 0, it = dgroup;
    const int kbpg = p.group_size / 64;  // K blocks per weight group
    auto load_sz = [&](int f, int k) -> uint32_t {
      const int gi = kbpg == 1 ? k : (kbpg == 2 ? (k >> 1) : k / kbpg);
      const size_t idx = (size_t(f) * 128 + t) * p.groups_per_row + gi;
      return uint32_t(__half_as_ushort(__ldg(p.scales + idx))) | (uint32_t(__half_as_ushort(__ldg(p.zeros + idx))) << 16);
    };
    uint32_t sz_next = w < nitems ? load_sz(item.ft, kb) : 0u;
    bool ok = true, first = true;
    int s_prev = 0;
    uint32_t ph_prev = 0;
    while (w < nitems && ok) {
      const uint32_t sz = sz_next;
      int nw = w, nk = kb;
      TcItem nitem = item;
      advance(nw, nitem, nk, NDG);
      if (nw < nitems) sz_next = load_sz(nitem.ft, nk);  // consumed three K blocks from now
      const __half sh = __ushort_as_half(uint16_t(sz & 0xffffu)), zh = __ushort_as_half(uint16_t(sz >> 16));
      uint32_t s2, z2;
      if (BF16) {
        s2 = __float_as_uint(__half2float(sh));
        z2 = __float_as_uint(__half2float(zh));
      } else {
        s2 = h2_as_u32(__half2half2(sh));
        z2 = h2_as_u32(__half2half2(zh));
      }
      // this group's A slot must have been consumed by the MMAs of its previous K block: their
      // commit arrived on the empty barrier of the stage that block used (s_prev, phase ph_prev).
      // That barrier cannot advance a second time before this wait: its next completion needs the
      // MMAs of a later block, which need this block's slot.
      if ((!first && !tc::mbar_wait(empty_bar(s_prev), ph_prev, p.status, 7)) ||
          !tc::mbar_wait(full_bar(s), ph, p.status, 5)) {
        ok = false;
        break;
      }
      first = false;
      s_prev = s;
      ph_prev = ph;
      if (t == 0) mark(2, it, 0);
      const uint4* wp = reinterpret_cast<const uint4*>(smem + a_ring_bytes + s * stage_bytes + xbytes + t * (8 * BITS));
      uint8_t* arow = smem + dgroup * kATileBytes + t * 128;
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
      if (t == 0) mark(2, it, 1);
      w = nw;
      item = nitem;
      kb = nk;
      it += NDG;
      dph ^= 1u;
      s += NDG;
      if (s >= nst) { s -= nst; ph ^= 1u; }
    }
  } else if (warp >= 2 && warp <= 5) {
    // ------------------------------ epilogue ------------------------------
    const int qd = warp & 3;
    uint32_t tcount = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < nitems && ok; w += gridDim.x, ++tcount) {
      const TcItem item = tc_item(p, w, nkb);
      const int ft = item.ft, tt = item.tt;
      const uint32_t buf = tcount & 1u, aph = (tcount >> 1) & 1u;
      const int f = ft * 128 + qd * 32 + lane;
      const float bias = p.bias ? __half2float(__ldg(p.bias + f)) : 0.f;
      // one decision for the warp, and the lanes together again after the polling loop: the tensor-memory loads
      // below are warp-wide instructions
      if (!__all_sync(0xffffffffu, tc::mbar_wait(accf_bar(buf), aph, p.status, 6))) { ok = false; break; }
      __syncwarp();
      tc::fence_after_sync();
      if (warp == 4 && lane == 0) mark(3, tcount, 0);
      const uint32_t taddr = tmem_base + (uint32_t(qd * 32) << 16) + buf * 256u;
      // one output column (token) per register: the warp's 32 lanes write 32 consecutive features
      // (64 contiguous bytes) of that token's row; the row pointer advances by N per column
      uint16_t* yp = p.y + size_t(tt) * p.bt * p.N + f;
      const int rows_left = p.M - tt * p.bt;  // tokens of this tile that exist
      if (p.ksplit > 1) {
        // Split K: this block's part of the tile goes to the workspace as fp32 ([token][feature], a
        // warp writes 128 contiguous bytes per token); the warp that arrives last for its 32
        // features adds the parts in split order (so the result does not depend on timing), adds
        // the bias, converts and stores.  Each lane quadrant synchronises by itself through its own
        // counter, which the last warp leaves at zero for the next launch.
        const int tile = tt * p.n_ftiles + ft;
        const size_t part_elems = size_t(p.bt) * 128;
        float* part0 = p.partials + size_t(tile) * p.ksplit * part_elems + qd * 32 + lane;
        float* mine = part0 + size_t(item.ks) * part_elems;
        for (int ch = 0; ch < p.bt / 32; ++ch) {
          uint32_t r[32];
          tc::tmem_ld_32x32(taddr + ch * 32, r);
          tc::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) __stcg(mine + size_t(ch * 32 + j) * 128, __uint_as_float(r[j]));
        }
        tc::fence_before_sync();
        tc::mbar_arrive(acce_bar(buf));
        __threadfence();
        __syncwarp();
        unsigned prev = 0;
        if (lane == 0) prev = atomicAdd(p.counters + tile * 4 + qd, 1u);
        prev = __shfl_sync(0xffffffffu, prev, 0);
        if (prev == unsigned(p.ksplit - 1)) {
          __threadfence();
          // 32 tokens at a time, one load per token in flight per lane: a part costs one trip to L2
          for (int ch = 0; ch * 32 < rows_left && ch < p.bt / 32; ++ch) {
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = 0.f;
            const float* src = part0 + size_t(ch) * 32 * 128;
            for (int ks = 0; ks < p.ksplit; ++ks, src += part_elems) {
              float a[32];
#pragma unroll
              for (int j = 0; j < 32; ++j) a[j] = __ldcg(src + j * 128);
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] += a[j];
            }
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (ch * 32 + j < rows_left) *yp = float_to_out16(v[j] + bias, BF16);
              yp += p.N;
            }
          }
          if (lane == 0) p.counters[tile * 4 + qd] = 0u;
        }
        if (warp == 4 && lane == 0) mark(3, tcount, 1);
        continue;
      }
      for (int ch = 0; ch < p.bt / 32; ++ch) {
        uint32_t r[32];
        tc::tmem_ld_32x32(taddr + ch * 32, r);
        tc::tmem_ld_wait();
        if (rows_left >= (ch + 1) * 32) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            *yp = float_to_out16(__uint_as_float(r[j]) + bias, BF16);
            yp += p.N;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (ch * 32 + j < rows_left) *yp = float_to_out16(__uint_as_float(r[j]) + bias, BF16);
            yp += p.N;
          }
        }
      }
      tc::fence_before_sync();
      tc::mbar_arrive(acce_bar(buf));
      if (warp == 4 && lane == 0) mark(3, tcount, 1);
    }
  }

  __syncwarp();
  tc::fence_before_sync();
  __syncthreads();
  if (warp == kTcMmaWarp) {
    tc::fence_after_sync();
    tc::tmem_dealloc(tmem_base, 512);
  }
}

// Token-tile width: the multiple of 32 (<= 256, <= M) that minimises
// rounds-over-the-SMs x (tile width + fixed per-tile overhead).
int gemm_tc_pick_bt(int64_t M, int64_t N, int sm_count) {
  const int forced = option(kOptTcBt);  // tuning knob: force the token-tile width
  if (forced >= 32 && forced <= 256 && forced % 32 == 0) return forced;
  int best = 32;
  double best_cost = 1e30;
  const int64_t nft = N / 128;
  for (int bt = 32; bt <= 256; bt += 32) {
    if (bt > M && bt != 32) break;
    const int64_t tiles = nft * ((M + bt - 1) / bt);
    const int64_t rounds = (tiles + sm_count - 1) / sm_count;
    const double cost = double(rounds) * (bt + 24);
    if (cost <= best_cost) {
      best_cost = cost;
      best = bt;
    }
  }
  return best;
}

// Split K (mid-size M): with few output tiles most SMs would idle while each busy one walks the
// whole K range, so the K blocks of a tile are divided among `split` blocks.  Bounded by the SM
// count, by two K blocks per part, and by the partial-sum area the workspace contract provides
// (split x padded M <= 512, the skinny kernel's 2048 bytes per output feature).
int gemm_tc_pick_split(int64_t M, int64_t N, int64_t K, int bt, int sm_count) {
  if (option(kOptTcSplit) == 1) return 1;  // tuning knob: 1 disables
  const int64_t n_tt = (M + bt - 1) / bt, tiles = (N / 128) * n_tt, nkb = K / 64;
  int64_t split = std::min<int64_t>({int64_t(sm_count) / tiles, nkb / 2, 512 / (n_tt * bt), kTcMaxSplit});
  return int(std::max<int64_t>(split, 1));
}
size_t gemm_tc_workspace_bytes(int64_t M, int64_t N) {
  return M <= 256 ? kPartialOffset + size_t(2048) * size_t(N) : kStatusBytes;
}

template <int BITS, bool BF16>
static int launch_tc(const CUtensorMap& tmx, const CUtensorMap& tmw, const GemmTcParams& p, int grid, size_t smem,
                     cudaStream_t stream) {
  auto kern = gemm_a16_tc_kernel<BITS, BF16>;
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem)) return rc;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kTcThreads);
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

bool gemm_a16_tc2_supports(int64_t M, int64_t N, int64_t K, int group_size);
int gemm_a16_tc2(int bits, const void* x, const uint8_t* w, const void* scales, const void* zeros, const void* bias,
                 void* y, int64_t M, int64_t N, int64_t K, int group_size, int dtype, void* workspace,
                 size_t workspace_bytes, int sm_count, cudaStream_t stream);

// `ep`: an epilogue the caller would like fused; *fused says whether the kernel that ran applied it.  Neither
// persistent kernel does: their four epilogue warps run under the next tile's main loop and have no slack for an
// erf per output or a strided read of the residual (with both fused into the CTA-pair kernel a Whisper encoder
// pass went from 95 to 195 ms, and the mere test for an epilogue per output cost the GEMM a quarter of its rate).
int gemm_a16_tc(int bits, const void* x, const uint8_t* w, const void* scales, const void* zeros, const void* bias,
                void* y, int64_t M, int64_t N, int64_t K, int group_size, int dtype, void* workspace,
                size_t workspace_bytes, int sm_count, cudaStream_t stream, const Epilogue& ep, bool* fused) {
  *fused = false;
  // The CTA-pair kernel (gemm_a16_tc2.cu, tcgen05 cta_group::2: half the activation rows per SM per
  // MMA) takes large M where the shape allows (20.9 us against 23.1 us on M=1500 K=1280 N=5120); M <= 256
  // stays here for the K split.  Option "tc_pair" = 1 / 0 forces / forbids it.
  const int pair_opt = option(kOptTcPair);
  const bool want_pair = pair_opt >= 0 ? pair_opt != 0 : M > 256;
  (void)ep;
  if (want_pair && gemm_a16_tc2_supports(M, N, K, group_size))
    return gemm_a16_tc2(bits, x, w, scales, zeros, bias, y, M, N, K, group_size, dtype, workspace, workspace_bytes,
                        sm_count, stream);
  if (N % 128 || K % 64 || group_size <= 0 || group_size % 64 || K % group_size)
    return fail(ASRQ_ERR_SHAPE,
                "w%da16 gemm: need N%%128==0, K%%64==0, group_size%%64==0, K%%group_size==0 "
                "(N=%lld K=%lld g=%d)", bits, (long long)N, (long long)K, group_size);
  if (M < 32) return fail(ASRQ_ERR_SHAPE, "w%da16 gemm: M=%lld < 32 (use the gemv entry point)", bits, (long long)M);
  if (M > (1ll << 30) || N > (1ll << 30) || K > (1ll << 24)) return fail(ASRQ_ERR_LIMIT, "w%da16 gemm: size", bits);
  if (workspace_bytes < kStatusBytes) return fail(ASRQ_ERR_WORKSPACE, "w%da16 gemm: workspace too small", bits);
  if (!aligned16(x) || !aligned16(w)) return fail(ASRQ_ERR_ALIGN, "w%da16 gemm: x and w must be 16-byte aligned", bits);

  GemmTcParams p;
  p.scales = static_cast<const __half*>(scales);
  p.zeros = static_cast<const __half*>(zeros);
  p.bias = static_cast<const __half*>(bias);
  p.y = static_cast<uint16_t*>(y);
  p.status = static_cast<unsigned*>(workspace);
  // diagnostic timeline (4 roles x 512 events x 2 clocks), only on request and only if the workspace has room
  p.trace = nullptr;
#ifdef ASRQ_TRACE
  if (option(kOptTrace) && workspace_bytes >= (1u << 20) + 4 * 512 * 2 * 8)
    p.trace = reinterpret_cast<long long*>(static_cast<char*>(workspace) + (1u << 20));
#endif
  p.M = int(M);
  p.N = int(N);
  p.K = int(K);
  p.group_size = group_size;
  p.groups_per_row = int(K / group_size);
  p.bt = gemm_tc_pick_bt(M, N, sm_count);
  p.n_ftiles = int(N / 128);
  p.n_ttiles = int((M + p.bt - 1) / p.bt);
  const size_t stage_bytes = size_t(p.bt) * 128 + kWSlotBytes;
  const size_t budget = 227 * 1024 - 1024 - 512 - kTcDequantGroups * kATileBytes;
  p.nstages = int(std::min<size_t>(kTcMaxStages, budget / stage_bytes));
  const size_t smem = 1024 + kTcDequantGroups * kATileBytes + p.nstages * stage_bytes;

  const bool bf16 = dtype == ASRQ_BF16;
  CUtensorMap tmx, tmw;
  int rc = make_tmap_2d(&tmx, x, 2, bf16, uint64_t(K), uint64_t(M), 64, uint32_t(p.bt), true);
  if (rc) return rc;
  rc = make_tmap_2d(&tmw, w, 1, false, uint64_t(K) * bits / 8, uint64_t(N), uint32_t(8 * bits), 128, false);
  if (rc) return rc;
  p.ksplit = gemm_tc_pick_split(M, N, K, p.bt, sm_count);
  if (p.ksplit > 1 && (workspace_bytes < kPartialOffset + size_t(4) * N * p.n_ttiles * p.bt * p.ksplit ||
                       p.n_ftiles * p.n_ttiles * 4 > int(kCounterBytes / sizeof(unsigned))))
    p.ksplit = 1;
  p.partials = reinterpret_cast<float*>(static_cast<char*>(workspace) + kPartialOffset);
  p.counters = reinterpret_cast<unsigned*>(static_cast<char*>(workspace) + kStatusBytes);
  const int grid = int(std::min<int64_t>(int64_t(p.n_ftiles) * p.n_ttiles * p.ksplit, sm_count));
  if (bits == 4)
    return bf16 ? launch_tc<4, true>(tmx, tmw, p, grid, smem, stream) : launch_tc<4, false>(tmx, tmw, p, grid, smem, stream);
  return bf16 ? launch_tc<2, true>(tmx, tmw, p, grid, smem, stream) : launch_tc<2, false>(tmx, tmw, p, grid, smem, stream);
}

}  // namespace asrq
