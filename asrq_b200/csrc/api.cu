// extern "C" entry points declared in include/asrq_b200.h: argument checks on the host,
// per-device facts cached once, dispatch to the kernels.  Nothing here allocates device
// memory or synchronises (asrq_check_status excepted, which says so).
#include <algorithm>
#include <atomic>
#include <cctype>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "tcgen05.cuh"

namespace asrq {

// kernels (one translation unit each)
int gemv_a16(int bits, const void* x, const uint8_t* w, const void* scales, const void* zeros, const void* bias,
             void* y, int64_t M, int64_t N, int64_t K, int group_size, int dtype, void* workspace,
             size_t workspace_bytes, int sm_count, cudaStream_t stream, int max_split);
size_t gemv_workspace_bytes(int64_t N);
size_t gemm_tc_workspace_bytes(int64_t M, int64_t N);
int gemm_a16_tc(int bits, const void* x, const uint8_t* w, const void* scales, const void* zeros, const void* bias,
                void* y, int64_t M, int64_t N, int64_t K, int group_size, int dtype, void* workspace,
                size_t workspace_bytes, int sm_count, cudaStream_t stream, const Epilogue& ep, bool* fused);
int add_layernorm(const void* x, const void* delta, const void* gamma, const void* beta, float eps, void* x_out, void* h_out,
                  int64_t rows, int64_t dim, int dtype, cudaStream_t stream);
int epilogue16_apply(void* y, const void* residual, int64_t M, int64_t N, int act, int dtype, int sm_count, cudaStream_t stream);
int add_rmsnorm(const void* x, const void* delta, const void* gamma, float eps, void* x_out, void* h_out, int64_t rows,
                int64_t dim, int dtype, cudaStream_t stream);
int silu_mul(const void* gu, void* out, int64_t rows, int64_t inter, int dtype, int sm_count, cudaStream_t stream);
int rtn_pack(const void* w, int w_dtype, int bits, int group_size, int symmetric, int layout, uint8_t* weight, void* scales,
             void* zeros, int64_t N, int64_t K, cudaStream_t stream);
int hadamard_fold(const void* w, int w_dtype, float* out, int64_t N, int64_t K, cudaStream_t stream);
int qk_norm_rope(const void* qkv, const void* qw, const void* kw, const void* cos_t, const void* sin_t, const long long* pos_dev,
                 long long pos_host, void* q_out, void* k_cache, void* v_cache, int64_t B, int64_t T, int nq, int nkv, int hd,
                 int64_t max_len, float eps, int dtype, cudaStream_t stream);
int decode_self_attention(const void* qkv, void* kv, const long long* pos_dev, void* out, int64_t B, int H, int hd, int64_t max_len,
                          float scale, int dtype, cudaStream_t stream);
int dense_head(const void* x, const void* w, void* y, int64_t M, int64_t N, int64_t K, int dtype, int sm_count, cudaStream_t stream);
int hadamard_quant_int4(const void* x, uint8_t* qa, float* sa, int64_t M, int64_t K, int hadamard, int dtype,
                        int out_int8, cudaStream_t stream);
int w4a4_linear_tc(const void* x, const uint8_t* qw, const void* sw, const void* bias, void* y, int64_t M, int64_t N,
                   int64_t K, int group_size, int hadamard, int dtype, void* workspace, size_t workspace_bytes,
                   int sm_count, cudaStream_t stream);
int w4a4_gemm_mma(const uint8_t* qa, const float* sa, const uint8_t* qw, const void* sw, const void* bias, void* y,
                  int32_t* acc_dump, int64_t M, int64_t N, int64_t K, int group_size, int dtype,
                  cudaStream_t stream);
int w4a4_gemm_tc(const uint8_t* qa, const float* sa, const uint8_t* qw, const void* sw, const void* bias, void* y,
                 int32_t* acc_dump, int64_t M, int64_t N, int64_t K, int group_size, int dtype, void* workspace,
                 size_t workspace_bytes, int sm_count, cudaStream_t stream);
bool w4a4_gemm_tc_supports(int64_t M, int64_t N, int64_t K, int group_size);
int expand_int4(const uint8_t* src, uint8_t* dst, size_t n_elems, int fmt, int sm_count, cudaStream_t stream);
int w4a4_gemm_int8(const uint8_t* w8, const uint8_t* a8, const float* sa, const void* sw, const void* bias, void* y,
                   int32_t* acc_dump, int64_t M, int64_t N, int64_t K, int group_size, int dtype, int fmt,
                   void* workspace, size_t workspace_bytes, int sm_count, cudaStream_t stream);
size_t w4a4_tc_workspace_bytes(int64_t M, int64_t N, int64_t K);
bool gemm_a16_skinny_supports(int64_t M, int64_t N, int64_t K, int group_size, int sm_count, size_t workspace_bytes);
int gemm_a16_skinny(int bits, const void* x, const uint8_t* w, const void* scales, const void* zeros, const void* bias,
                    void* y, int64_t M, int64_t N, int64_t K, int group_size, int dtype, void* workspace,
                    size_t workspace_bytes, int sm_count, cudaStream_t stream, const Epilogue& ep);

// ---- errors -----------------------------------------------------------------------------
std::string& last_error() {
  static thread_local std::string s;
  return s;
}

int fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  last_error() = buf;
  return code;
}

int cuda_fail(cudaError_t e, const char* what) {
  char buf[512];
  snprintf(buf, sizeof(buf), "CUDA error %d (%s) at %s", int(e), cudaGetErrorString(e), what);
  last_error() = buf;
  return int(e) > 0 ? int(e) : 1;
}

// ---- options ------------------------------------------------------------------------------
namespace {
struct OptionDef {
  const char* name;
  int def;
};
const OptionDef kOptionDefs[kOptCount] = {
    {"no_pdl", 0},      {"mid_kernel", 0}, {"gemv_kernel", 0}, {"gemv_cpw", 0},  {"gemv_xstage", 1}, {"gemv_loop", -1},   {"tc_split", 0},   {"tc_bt", 0},
    {"tc_pair", -1},    {"tc_pair_release", 0}, {"w4a4_bt", 0}, {"w4a4_pair", -1}, {"trace", 0},      {"trace_block", 0},
};
struct OptionTable {
  std::atomic<int> v[kOptCount];
  std::atomic<unsigned> generation{0};
  OptionTable() {
    for (int i = 0; i < kOptCount; ++i) {
      std::string env = "ASRQ_B200_";
      for (const char* c = kOptionDefs[i].name; *c; ++c) env.push_back(char(toupper(*c)));
      const char* e = getenv(env.c_str());
      v[i].store(e && *e ? atoi(e) : kOptionDefs[i].def);
    }
  }
};
OptionTable& option_table() {
  static OptionTable t;  // environment read once, at first use
  return t;
}
int find_option(const char* name) {
  if (!name) return -1;
  for (int i = 0; i < kOptCount; ++i)
    if (!strcmp(name, kOptionDefs[i].name)) return i;
  return -1;
}
}  // namespace

int option(Option o) { return option_table().v[o].load(std::memory_order_relaxed); }
unsigned options_generation() { return option_table().generation.load(std::memory_order_relaxed); }

// ---- per-device facts ---------------------------------------------------------------------
struct DeviceFacts {
  std::once_flag once;
  int status = ASRQ_ERR_DEVICE;
  int sm_count = 0;
  int cc_major = 0;
};
static DeviceFacts g_dev[64];

static int device_facts(const DeviceFacts** out) {
  int dev = 0;
  ASRQ_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(ASRQ_ERR_DEVICE, "device index %d out of range", dev);
  DeviceFacts& f = g_dev[dev];
  std::call_once(f.once, [&] {
    int major = 0, sms = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return;
    f.cc_major = major;
    f.sm_count = sms;
    f.status = (major == 10) ? ASRQ_OK : ASRQ_ERR_DEVICE;
  });
  if (f.status != ASRQ_OK)
    return fail(ASRQ_ERR_DEVICE, "device %d has compute capability %d.x; this library is built for sm_100a only", dev,
                f.cc_major);
  *out = &f;
  return ASRQ_OK;
}

// ---- tensor maps ----------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// Encoding a tensor map costs a driver call of a few microseconds, as much as a short kernel runs; a
// decode or prefill loop calls with the same buffers over and over, so the last maps are remembered.
namespace {
struct TmapKey {
  const void* base;
  uint64_t inner, rows;
  uint32_t box_inner, box_rows;
  int elem_bytes, flags;
  bool operator==(const TmapKey& o) const {
    return base == o.base && inner == o.inner && rows == o.rows && box_inner == o.box_inner && box_rows == o.box_rows &&
           elem_bytes == o.elem_bytes && flags == o.flags;
  }
};
struct TmapEntry {
  TmapKey key;
  CUtensorMap map;
  bool used = false;
};
constexpr int kTmapCache = 64;
std::mutex g_tmap_mutex;
TmapEntry g_tmap_cache[kTmapCache];
int g_tmap_next = 0;
}  // namespace

int make_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, bool bf16, uint64_t inner, uint64_t rows,
                 uint32_t box_inner, uint32_t box_rows, bool swizzle128) {
  const TmapKey key = {base, inner, rows, box_inner, box_rows, elem_bytes, (bf16 ? 1 : 0) | (swizzle128 ? 2 : 0)};
  {
    std::lock_guard<std::mutex> lock(g_tmap_mutex);
    for (const TmapEntry& e : g_tmap_cache)
      if (e.used && e.key == key) {
        *out = e.map;
        return ASRQ_OK;
      }
  }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(ASRQ_ERR_DEVICE, "cuTensorMapEncodeTiled is not available from this driver");
  const CUtensorMapDataType dt = elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                 : bf16          ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const cuuint64_t dims[2] = {inner, rows};
  const cuuint64_t strides[1] = {inner * uint64_t(elem_bytes)};
  const cuuint32_t box[2] = {box_inner, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  if (strides[0] % 16) return fail(ASRQ_ERR_ALIGN, "row pitch %llu is not a multiple of 16 bytes", (unsigned long long)strides[0]);
  const CUresult r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(ASRQ_ERR_SHAPE, "cuTensorMapEncodeTiled failed with CUresult %d", int(r));
  std::lock_guard<std::mutex> lock(g_tmap_mutex);
  TmapEntry& e = g_tmap_cache[g_tmap_next];
  g_tmap_next = (g_tmap_next + 1) % kTmapCache;
  e.key = key;
  e.map = *out;
  e.used = true;
  return ASRQ_OK;
}

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) once per (kernel, device) and size, not once per launch.
int ensure_dynamic_smem(const void* kernel, size_t bytes) {
  struct Seen {
    const void* kernel;
    int device;
    size_t bytes;
  };
  static std::mutex mu;
  static std::vector<Seen> seen;
  int dev = 0;
  ASRQ_CUDA_TRY(cudaGetDevice(&dev));
  {
    std::lock_guard<std::mutex> lock(mu);
    for (const Seen& s : seen)
      if (s.kernel == kernel && s.device == dev && s.bytes >= bytes) return ASRQ_OK;
  }
  ASRQ_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(bytes)));
  std::lock_guard<std::mutex> lock(mu);
  seen.push_back({kernel, dev, bytes});
  return ASRQ_OK;
}

int check_a16_common(const char* who, const void* x, const uint8_t* w, const void* scales, const void* zeros,
                            void* y, int64_t M, int64_t N, int64_t K, int dtype, void* workspace) {
  if (!x || !w || !scales || !zeros || !y) return fail(ASRQ_ERR_NULL, "%s: x, w, scales, zeros and y must not be NULL", who);
  if (!workspace) return fail(ASRQ_ERR_WORKSPACE, "%s: workspace must not be NULL", who);
  if (dtype != ASRQ_F16 && dtype != ASRQ_BF16) return fail(ASRQ_ERR_DTYPE, "%s: dtype %d", who, dtype);
  if (M < 0 || N <= 0 || K <= 0) return fail(ASRQ_ERR_SHAPE, "%s: M=%lld N=%lld K=%lld", who, (long long)M, (long long)N, (long long)K);
  if (!aligned16(x) || !aligned16(w) || !aligned16(y) || !aligned16(workspace))
    return fail(ASRQ_ERR_ALIGN, "%s: x, w, y and workspace must be 16-byte aligned", who);
  return ASRQ_OK;
}

// SM count of the current device (checked to be sm_100), for code outside this file.
int current_device_sm_count(int* sm_count) {
  const DeviceFacts* f;
  const int rc = device_facts(&f);
  if (rc) return rc;
  *sm_count = f->sm_count;
  return ASRQ_OK;
}

// M at or below which LinearQ.forward goes to the skinny kernel.
constexpr int64_t kGemvMaxM = 32;

}  // namespace asrq

using namespace asrq;

#pragma GCC visibility push(default)
extern "C" {

int asrq_version(void) { return 100; }

const char* asrq_last_error_string(void) { return last_error().c_str(); }

size_t asrq_workspace_bytes(int kind, int64_t M, int64_t N, int64_t K) {
  switch (kind) {
    case ASRQ_WS_A16_GEMV:
    case ASRQ_WS_LINEARQ:
      return gemv_workspace_bytes(N);
    case ASRQ_WS_A16_GEMM:
      return gemm_tc_workspace_bytes(M, N);
    case ASRQ_WS_W4A4_GEMM:
      return w4a4_tc_workspace_bytes(M, N, K);
    default:
      return 0;
  }
}

static int a16_gemv(int bits, const void* x, const uint8_t* w, const void* scales, const void* zeros, const void* bias,
                    void* y, int64_t M, int64_t N, int64_t K, int group_size, int dtype, void* workspace,
                    size_t workspace_bytes, void* stream) {
  last_error().clear();
  int rc = check_a16_common(bits == 4 ? "asrq_w4a16_gemv" : "asrq_w2a16_gemv", x, w, scales, zeros, y, M, N, K, dtype,
                            workspace);
  if (rc) return rc;
  const DeviceFacts* f;
  if ((rc = device_facts(&f))) return rc;
  if (M == 0) return ASRQ_OK;
  return gemv_a16(bits, x, w, scales, zeros, bias, y, M, N, K, group_size, dtype, workspace, workspace_bytes,
                  f->sm_count, static_cast<cudaStream_t>(stream), kGemvMaxSplit);
}

static int a16_gemm(int bits, const void* x, const uint8_t* w, const void* scales, const void* zeros, const void* bias,
                    void* y, int64_t M, int64_t N, int64_t K, int group_size, int dtype, void* workspace,
                    size_t workspace_bytes, void* stream, const Epilogue& ep = Epilogue(), bool* fused = nullptr) {
  last_error().clear();
  bool fused_here = false;
  if (!fused) fused = &fused_here;
  *fused = false;
  int rc = check_a16_common(bits == 4 ? "asrq_w4a16_gemm" : "asrq_w2a16_gemm", x, w, scales, zeros, y, M, N, K, dtype,
                            workspace);
  if (rc) return rc;
  const DeviceFacts* f;
  if ((rc = device_facts(&f))) return rc;
  if (M == 0) return ASRQ_OK;
  // decode batches (17..64 tokens): the chain-oriented tensor-core kernel where its one-wave grid fits
  if (M <= 64 && option(kOptMidKernel) != 1 && (reinterpret_cast<uintptr_t>(bias) & 7u) == 0 &&
      gemm_a16_skinny_supports(M, N, K, group_size, f->sm_count, workspace_bytes)) {
    *fused = true;
    return gemm_a16_skinny(bits, x, w, scales, zeros, bias, y, M, N, K, group_size, dtype, workspace, workspace_bytes,
                           f->sm_count, static_cast<cudaStream_t>(stream), ep);
  }
  return gemm_a16_tc(bits, x, w, scales, zeros, bias, y, M, N, K, group_size, dtype, workspace, workspace_bytes,
                     f->sm_count, static_cast<cudaStream_t>(stream), ep, fused);
}

int asrq_w4a16_gemv(const void* x, const uint8_t* w, const void* scales, const void* zeros, const void* bias, void* y,
                    int64_t M, int64_t N, int64_t K, int group_size, int dtype, void* workspace,
                    size_t workspace_bytes, void* stream) {
  return a16_gemv(4, x, w, scales, zeros, bias, y, M, N, K, group_size, dtype, workspace, workspace_bytes, stream);
}
int asrq_w2a16_gemv(const void* x, const uint8_t* w, const void* scales, const void* zeros, const void* bias, void* y,
                    int64_t M, int64_t N, int64_t K, int group_size, int dtype, void* workspace,
                    size_t workspace_bytes, void* stream) {
  return a16_gemv(2, x, w, scales, zeros, bias, y, M, N, K, group_size, dtype, workspace, workspace_bytes, stream);
}
int asrq_w4a16_gemm(const void* x, const uint8_t* w, const void* scales, const void* zeros, const void* bias, void* y,
                    int64_t M, int64_t N, int64_t K, int group_size, int dtype, void* workspace,
                    size_t workspace_bytes, void* stream) {
  return a16_gemm(4, x, w, scales, zeros, bias, y, M, N, K, group_size, dtype, workspace, workspace_bytes, stream);
}
int asrq_w2a16_gemm(const void* x, const uint8_t* w, const void* scales, const void* zeros, const void* bias, void* y,
                    int64_t M, int64_t N, int64_t K, int group_size, int dtype, void* workspace,
                    size_t workspace_bytes, void* stream) {
  return a16_gemm(2, x, w, scales, zeros, bias, y, M, N, K, group_size, dtype, workspace, workspace_bytes, stream);
}

static int linearq_a16(int bits, const void* x, const uint8_t* w, const void* scales, const void* zeros,
                       const void* bias, void* y, int64_t M, int64_t N, int64_t K, int group_size, int dtype,
                       void* workspace, size_t workspace_bytes, void* stream, const Epilogue& ep) {
  if (bits != 2 && bits != 4) {
    last_error().clear();
    return fail(ASRQ_ERR_SHAPE, "asrq_linearq_a16: bits must be 2 or 4 (got %d)", bits);
  }
  const bool want_ep = ep.act != kActNone || ep.residual != nullptr;
  if (ep.act != kActNone && ep.act != kActGelu) return fail(ASRQ_ERR_SHAPE, "asrq_linearq_a16_fused: act %d", ep.act);
  if (want_ep && ((M * N) % 8 || !aligned16(y) || !aligned16(ep.residual)))
    return fail(ASRQ_ERR_ALIGN, "asrq_linearq_a16_fused: y and residual must be 16-byte aligned and M*N a multiple of 8");
  const bool tc_ok = N % 128 == 0 && K % 64 == 0 && group_size > 0 && group_size % 64 == 0 && K % group_size == 0;
  bool fused = false;
  int rc;
  // 17..32 tokens: the tensor cores (gemm_a16_skinny.cu) unless switched off; the mma.sync decode kernel is bound
  // by the legacy MMA pipe there
  bool mid = false;
  if (M > 16 && M <= kGemvMaxM && tc_ok && option(kOptMidKernel) != 1 && workspace) {
    int sms = 0;
    mid = current_device_sm_count(&sms) == ASRQ_OK && gemm_a16_skinny_supports(M, N, K, group_size, sms, workspace_bytes);
  }
  if (mid || (M > kGemvMaxM && tc_ok))
    rc = a16_gemm(bits, x, w, scales, zeros, bias, y, M, N, K, group_size, dtype, workspace, workspace_bytes, stream,
                  ep, &fused);
  else
    rc = a16_gemv(bits, x, w, scales, zeros, bias, y, M, N, K, group_size, dtype, workspace, workspace_bytes, stream);
  if (rc || !want_ep || fused || M == 0) return rc;
  // the kernel that ran does not fuse the epilogue: one more pass over the output
  const DeviceFacts* f;
  if ((rc = device_facts(&f))) return rc;
  return epilogue16_apply(y, ep.residual, M, N, ep.act, dtype, f->sm_count, static_cast<cudaStream_t>(stream));
}

int asrq_linearq_a16(int bits, const void* x, const uint8_t* w, const void* scales, const void* zeros,
                     const void* bias, void* y, int64_t M, int64_t N, int64_t K, int group_size, int dtype,
                     void* workspace, size_t workspace_bytes, void* stream) {
  return linearq_a16(bits, x, w, scales, zeros, bias, y, M, N, K, group_size, dtype, workspace, workspace_bytes, stream,
                     Epilogue());
}

int asrq_linearq_a16_fused(int bits, const void* x, const uint8_t* w, const void* scales, const void* zeros,
                           const void* bias, const void* residual, void* y, int64_t M, int64_t N, int64_t K,
                           int group_size, int dtype, int act, void* workspace, size_t workspace_bytes, void* stream) {
  Epilogue ep;
  ep.residual = residual;
  ep.act = act;
  return linearq_a16(bits, x, w, scales, zeros, bias, y, M, N, K, group_size, dtype, workspace, workspace_bytes, stream, ep);
}

int asrq_add_layernorm(const void* x, const void* delta, const void* gamma, const void* beta, float eps, void* x_out,
                       void* h_out, int64_t rows, int64_t dim, int dtype, void* stream) {
  last_error().clear();
  if (!x || !gamma || !beta || !h_out) return fail(ASRQ_ERR_NULL, "asrq_add_layernorm: x, gamma, beta and h_out must not be NULL");
  if (dtype != ASRQ_F16 && dtype != ASRQ_BF16) return fail(ASRQ_ERR_DTYPE, "asrq_add_layernorm: dtype %d", dtype);
  if (rows < 0 || dim <= 0 || dim > (1 << 20) || rows > (int64_t(1) << 31) - 64)
    return fail(ASRQ_ERR_SHAPE, "asrq_add_layernorm: rows=%lld dim=%lld", (long long)rows, (long long)dim);
  const DeviceFacts* f;
  int rc;
  if ((rc = device_facts(&f))) return rc;
  if (rows == 0) return ASRQ_OK;
  return add_layernorm(x, delta, gamma, beta, eps, x_out, h_out, rows, dim, dtype, static_cast<cudaStream_t>(stream));
}

int asrq_add_rmsnorm(const void* x, const void* delta, const void* gamma, float eps, void* x_out, void* h_out, int64_t rows,
                     int64_t dim, int dtype, void* stream) {
  last_error().clear();
  if (!x || !gamma || !h_out) return fail(ASRQ_ERR_NULL, "asrq_add_rmsnorm: x, gamma and h_out must not be NULL");
  if (dtype != ASRQ_F16 && dtype != ASRQ_BF16) return fail(ASRQ_ERR_DTYPE, "asrq_add_rmsnorm: dtype %d", dtype);
  if (rows < 0 || dim <= 0 || dim > (1 << 20) || rows > (int64_t(1) << 31) - 64)
    return fail(ASRQ_ERR_SHAPE, "asrq_add_rmsnorm: rows=%lld dim=%lld", (long long)rows, (long long)dim);
  const DeviceFacts* f;
  int rc;
  if ((rc = device_facts(&f))) return rc;
  if (rows == 0) return ASRQ_OK;
  return add_rmsnorm(x, delta, gamma, eps, x_out, h_out, rows, dim, dtype, static_cast<cudaStream_t>(stream));
}

int asrq_silu_mul(const void* gate_up, void* out, int64_t rows, int64_t inter, int dtype, void* stream) {
  last_error().clear();
  if (!gate_up || !out) return fail(ASRQ_ERR_NULL, "asrq_silu_mul: gate_up and out must not be NULL");
  if (dtype != ASRQ_F16 && dtype != ASRQ_BF16) return fail(ASRQ_ERR_DTYPE, "asrq_silu_mul: dtype %d", dtype);
  if (rows < 0 || inter <= 0 || inter % 8 != 0 || rows > (int64_t(1) << 31) - 64 || inter > (1 << 24))
    return fail(ASRQ_ERR_SHAPE, "asrq_silu_mul: rows=%lld inter=%lld (a multiple of 8)", (long long)rows, (long long)inter);
  if (!aligned16(gate_up) || !aligned16(out)) return fail(ASRQ_ERR_ALIGN, "asrq_silu_mul: gate_up and out must be 16-byte aligned");
  const DeviceFacts* f;
  int rc;
  if ((rc = device_facts(&f))) return rc;
  if (rows == 0) return ASRQ_OK;
  return silu_mul(gate_up, out, rows, inter, dtype, f->sm_count, static_cast<cudaStream_t>(stream));
}

int asrq_qk_norm_rope(const void* qkv, const void* q_weight, const void* k_weight, const void* cos_table, const void* sin_table,
                      const int64_t* pos_device, int64_t pos, void* q_out, void* k_cache, void* v_cache, int64_t B, int64_t T,
                      int n_q_heads, int n_kv_heads, int head_dim, int64_t max_len, float eps, int dtype, void* stream) {
  last_error().clear();
  if (!qkv || !q_weight || !k_weight || !cos_table || !sin_table || !q_out || !k_cache || !v_cache)
    return fail(ASRQ_ERR_NULL, "asrq_qk_norm_rope: only pos_device may be NULL");
  if (dtype != ASRQ_F16 && dtype != ASRQ_BF16) return fail(ASRQ_ERR_DTYPE, "asrq_qk_norm_rope: dtype %d", dtype);
  if (B < 0 || T <= 0 || n_q_heads <= 0 || n_kv_heads <= 0 || (head_dim != 64 && head_dim != 128) || max_len <= 0 ||
      (!pos_device && (pos < 0 || pos + T > max_len)) || B * T > (int64_t(1) << 30))
    return fail(ASRQ_ERR_SHAPE, "asrq_qk_norm_rope: B=%lld T=%lld heads=%d/%d head_dim=%d (64 or 128) max_len=%lld pos=%lld", (long long)B,
                (long long)T, n_q_heads, n_kv_heads, head_dim, (long long)max_len, (long long)pos);
  if (reinterpret_cast<uintptr_t>(qkv) % 8 || reinterpret_cast<uintptr_t>(q_out) % 8 || reinterpret_cast<uintptr_t>(k_cache) % 8 ||
      reinterpret_cast<uintptr_t>(v_cache) % 8)
    return fail(ASRQ_ERR_ALIGN, "asrq_qk_norm_rope: qkv, q_out and the caches must be 8-byte aligned");
  const DeviceFacts* f;
  int rc;
  if ((rc = device_facts(&f))) return rc;
  if (B == 0) return ASRQ_OK;
  return qk_norm_rope(qkv, q_weight, k_weight, cos_table, sin_table, reinterpret_cast<const long long*>(pos_device), (long long)pos, q_out,
                      k_cache, v_cache, B, T, n_q_heads, n_kv_heads, head_dim, max_len, eps, dtype, static_cast<cudaStream_t>(stream));
}

int asrq_decode_self_attention(const void* qkv, void* kv_cache, const int64_t* pos_device, void* out, int64_t B, int n_heads,
                               int head_dim, int64_t max_len, float scale, int dtype, void* stream) {
  last_error().clear();
  if (!qkv || !kv_cache || !pos_device || !out) return fail(ASRQ_ERR_NULL, "asrq_decode_self_attention: no argument may be NULL");
  if (dtype != ASRQ_F16 && dtype != ASRQ_BF16) return fail(ASRQ_ERR_DTYPE, "asrq_decode_self_attention: dtype %d", dtype);
  if (B < 0 || n_heads <= 0 || (head_dim != 64 && head_dim != 128) || max_len <= 0 || max_len > 512 || B * n_heads > (int64_t(1) << 28))
    return fail(ASRQ_ERR_SHAPE, "asrq_decode_self_attention: B=%lld heads=%d head_dim=%d (64 or 128) max_len=%lld (at most 512)",
                (long long)B, n_heads, head_dim, (long long)max_len);
  if (!aligned16(kv_cache)) return fail(ASRQ_ERR_ALIGN, "asrq_decode_self_attention: kv_cache must be 16-byte aligned");
  const DeviceFacts* f;
  int rc;
  if ((rc = device_facts(&f))) return rc;
  if (B == 0) return ASRQ_OK;
  return decode_self_attention(qkv, kv_cache, reinterpret_cast<const long long*>(pos_device), out, B, n_heads, head_dim, max_len, scale,
                               dtype, static_cast<cudaStream_t>(stream));
}

int asrq_dense_head(const void* x, const void* w, void* y, int64_t M, int64_t N, int64_t K, int dtype, void* stream) {
  last_error().clear();
  if (!x || !w || !y) return fail(ASRQ_ERR_NULL, "asrq_dense_head: x, w and y must not be NULL");
  if (dtype != ASRQ_F16 && dtype != ASRQ_BF16) return fail(ASRQ_ERR_DTYPE, "asrq_dense_head: dtype %d", dtype);
  if (M < 0 || M > 32 || N <= 0 || K <= 0 || K % 32 != 0 || K > 3200 || N > (int64_t(1) << 30))
    return fail(ASRQ_ERR_SHAPE, "asrq_dense_head: M=%lld (at most 32) N=%lld K=%lld (a multiple of 32, at most 3200)", (long long)M,
                (long long)N, (long long)K);
  if (!aligned16(x) || !aligned16(w)) return fail(ASRQ_ERR_ALIGN, "asrq_dense_head: x and w must be 16-byte aligned");
  const DeviceFacts* f;
  int rc;
  if ((rc = device_facts(&f))) return rc;
  if (M == 0) return ASRQ_OK;
  return dense_head(x, w, y, M, N, K, dtype, f->sm_count, static_cast<cudaStream_t>(stream));
}

int asrq_rtn_pack(const void* w, int w_dtype, int bits, int group_size, int symmetric, int layout, uint8_t* weight,
                  void* scales, void* zeros, int64_t N, int64_t K, void* stream) {
  last_error().clear();
  if (!w || !weight || !scales || (layout == 0 && !zeros)) return fail(ASRQ_ERR_NULL, "asrq_rtn_pack: w, weight, scales (and zeros for layout 0) must not be NULL");
  if (w_dtype != ASRQ_F16 && w_dtype != ASRQ_BF16 && w_dtype != ASRQ_F32) return fail(ASRQ_ERR_DTYPE, "asrq_rtn_pack: w_dtype %d", w_dtype);
  if ((bits != 2 && bits != 4) || (layout != 0 && layout != 1) || (layout == 1 && (bits != 4 || !symmetric)))
    return fail(ASRQ_ERR_SHAPE, "asrq_rtn_pack: bits=%d layout=%d symmetric=%d (layout 1 is signed 4-bit, symmetric)", bits, layout, symmetric);
  if (N < 0 || K <= 0 || group_size < 8 || group_size % 8 != 0 || K % group_size != 0 || N > (int64_t(1) << 31) || K > (1 << 24))
    return fail(ASRQ_ERR_SHAPE, "asrq_rtn_pack: N=%lld K=%lld group_size=%d (a multiple of 8 that divides K)", (long long)N, (long long)K, group_size);
  if (reinterpret_cast<uintptr_t>(weight) % 4 != 0) return fail(ASRQ_ERR_ALIGN, "asrq_rtn_pack: weight must be 4-byte aligned");
  const DeviceFacts* f;
  int rc;
  if ((rc = device_facts(&f))) return rc;
  if (N == 0) return ASRQ_OK;
  return rtn_pack(w, w_dtype, bits, group_size, symmetric != 0, layout, weight, scales, zeros, N, K, static_cast<cudaStream_t>(stream));
}

int asrq_hadamard_fold(const void* w, int w_dtype, float* out, int64_t N, int64_t K, void* stream) {
  last_error().clear();
  if (!w || !out) return fail(ASRQ_ERR_NULL, "asrq_hadamard_fold: w and out must not be NULL");
  if (w_dtype != ASRQ_F16 && w_dtype != ASRQ_BF16 && w_dtype != ASRQ_F32) return fail(ASRQ_ERR_DTYPE, "asrq_hadamard_fold: w_dtype %d", w_dtype);
  if (N < 0 || K < 2 || K > 8192 || (K & (K - 1)) != 0 || N > (int64_t(1) << 31) - 1)
    return fail(ASRQ_ERR_SHAPE, "asrq_hadamard_fold: N=%lld K=%lld (K a power of two, 2..8192)", (long long)N, (long long)K);
  const DeviceFacts* f;
  int rc;
  if ((rc = device_facts(&f))) return rc;
  if (N == 0) return ASRQ_OK;
  return hadamard_fold(w, w_dtype, out, N, K, static_cast<cudaStream_t>(stream));
}

int asrq_hadamard_quant_int4(const void* x, uint8_t* qa, float* sa, int64_t M, int64_t K, int hadamard, int dtype,
                             void* stream) {
  last_error().clear();
  if (!x || !qa || !sa) return fail(ASRQ_ERR_NULL, "asrq_hadamard_quant_int4: x, qa and sa must not be NULL");
  if (dtype != ASRQ_F16 && dtype != ASRQ_BF16) return fail(ASRQ_ERR_DTYPE, "asrq_hadamard_quant_int4: dtype %d", dtype);
  if (M < 0 || K <= 0) return fail(ASRQ_ERR_SHAPE, "asrq_hadamard_quant_int4: M=%lld K=%lld", (long long)M, (long long)K);
  if (!aligned16(x) || !aligned16(qa)) return fail(ASRQ_ERR_ALIGN, "asrq_hadamard_quant_int4: x and qa must be 16-byte aligned");
  const DeviceFacts* f;
  int rc;
  if ((rc = device_facts(&f))) return rc;
  return hadamard_quant_int4(x, qa, sa, M, K, hadamard, dtype, 0, static_cast<cudaStream_t>(stream));
}

int asrq_w4a4_gemm(const uint8_t* qa, const float* sa, const uint8_t* qw, const void* sw, const void* bias, void* y,
                   int32_t* acc_dump, int64_t M, int64_t N, int64_t K, int group_size, int dtype, void* workspace,
                   size_t workspace_bytes, void* stream) {
  last_error().clear();
  if (!qa || !sa || !qw || !sw || !y) return fail(ASRQ_ERR_NULL, "asrq_w4a4_gemm: qa, sa, qw, sw and y must not be NULL");
  if (!workspace || workspace_bytes < kStatusBytes) return fail(ASRQ_ERR_WORKSPACE, "asrq_w4a4_gemm: workspace");
  if (dtype != ASRQ_F16 && dtype != ASRQ_BF16) return fail(ASRQ_ERR_DTYPE, "asrq_w4a4_gemm: dtype %d", dtype);
  if (M < 0 || N <= 0 || K <= 0 || group_size <= 0)
    return fail(ASRQ_ERR_SHAPE, "asrq_w4a4_gemm: M=%lld N=%lld K=%lld group_size=%d", (long long)M, (long long)N,
                (long long)K, group_size);
  if (!aligned16(qa) || !aligned16(qw) || !aligned16(y) || !aligned16(workspace))
    return fail(ASRQ_ERR_ALIGN, "asrq_w4a4_gemm: qa, qw, y and workspace must be 16-byte aligned");
  const DeviceFacts* f;
  int rc;
  if ((rc = device_facts(&f))) return rc;
  if (M == 0) return ASRQ_OK;
  if (w4a4_gemm_tc_supports(M, N, K, group_size))
    return w4a4_gemm_tc(qa, sa, qw, sw, bias, y, acc_dump, M, N, K, group_size, dtype, workspace, workspace_bytes,
                        f->sm_count, static_cast<cudaStream_t>(stream));
  return w4a4_gemm_mma(qa, sa, qw, sw, bias, y, acc_dump, M, N, K, group_size, dtype,
                       static_cast<cudaStream_t>(stream));
}

int asrq_w4a4_linear(const void* x, const uint8_t* qw, const void* sw, const void* bias, void* y, int64_t M, int64_t N,
                     int64_t K, int group_size, int hadamard, int dtype, void* workspace, size_t workspace_bytes,
                     void* stream) {
  last_error().clear();
  if (!x || !qw || !sw || !y) return fail(ASRQ_ERR_NULL, "asrq_w4a4_linear: x, qw, sw and y must not be NULL");
  if (!workspace) return fail(ASRQ_ERR_WORKSPACE, "asrq_w4a4_linear: workspace must not be NULL");
  if (dtype != ASRQ_F16 && dtype != ASRQ_BF16) return fail(ASRQ_ERR_DTYPE, "asrq_w4a4_linear: dtype %d", dtype);
  if (M < 0 || N <= 0 || K <= 0) return fail(ASRQ_ERR_SHAPE, "asrq_w4a4_linear: M=%lld N=%lld K=%lld", (long long)M, (long long)N, (long long)K);
  if (!aligned16(x) || !aligned16(qw) || !aligned16(y) || !aligned16(workspace))
    return fail(ASRQ_ERR_ALIGN, "asrq_w4a4_linear: x, qw, y and workspace must be 16-byte aligned");
  if (!w4a4_gemm_tc_supports(std::max<int64_t>(M, 64), N, K, group_size))
    return fail(ASRQ_ERR_SHAPE,
                "asrq_w4a4_linear: need N%%128==0, K%%128==0, group_size%%128==0, K%%group_size==0 "
                "(N=%lld K=%lld g=%d)", (long long)N, (long long)K, group_size);
  const DeviceFacts* f;
  int rc;
  if ((rc = device_facts(&f))) return rc;
  if (M == 0) return ASRQ_OK;
  return w4a4_linear_tc(x, qw, sw, bias, y, M, N, K, group_size, hadamard, dtype, workspace, workspace_bytes,
                        f->sm_count, static_cast<cudaStream_t>(stream));
}

// fmt: 1 = int8 holding 16x the code (kind::i8), 2 = e4m3 holding the code (kind::f8f6f4)
static int prepare_weight(const char* who, const uint8_t* qw, uint8_t* w8, int64_t N, int64_t K, int fmt, void* stream) {
  last_error().clear();
  if (!qw || !w8) return fail(ASRQ_ERR_NULL, "%s: qw and w8 must not be NULL", who);
  if (N <= 0 || K <= 0 || (N * K) % 32) return fail(ASRQ_ERR_SHAPE, "%s: N*K must be a positive multiple of 32", who);
  if (!aligned16(qw) || !aligned16(w8)) return fail(ASRQ_ERR_ALIGN, "%s: qw and w8 must be 16-byte aligned", who);
  const DeviceFacts* f;
  int rc;
  if ((rc = device_facts(&f))) return rc;
  return expand_int4(qw, w8, size_t(N) * size_t(K), fmt, f->sm_count, static_cast<cudaStream_t>(stream));
}

static int quant_operand(const char* who, const void* x, uint8_t* a8, float* sa, int64_t M, int64_t K, int hadamard,
                         int dtype, int fmt, void* stream) {
  last_error().clear();
  if (!x || !a8 || !sa) return fail(ASRQ_ERR_NULL, "%s: x, a8 and sa must not be NULL", who);
  if (dtype != ASRQ_F16 && dtype != ASRQ_BF16) return fail(ASRQ_ERR_DTYPE, "%s: dtype %d", who, dtype);
  if (M < 0 || K <= 0) return fail(ASRQ_ERR_SHAPE, "%s: M=%lld K=%lld", who, (long long)M, (long long)K);
  if (!aligned16(x) || !aligned16(a8)) return fail(ASRQ_ERR_ALIGN, "%s: x and a8 must be 16-byte aligned", who);
  const DeviceFacts* f;
  int rc;
  if ((rc = device_facts(&f))) return rc;
  return hadamard_quant_int4(x, a8, sa, M, K, hadamard, dtype, fmt, static_cast<cudaStream_t>(stream));
}

static int gemm_operand(const char* who, const uint8_t* a8, const float* sa, const uint8_t* w8, const void* sw,
                        const void* bias, void* y, int32_t* acc_dump, int64_t M, int64_t N, int64_t K, int group_size,
                        int dtype, int fmt, void* workspace, size_t workspace_bytes, void* stream) {
  last_error().clear();
  if (!a8 || !sa || !w8 || !sw || !y) return fail(ASRQ_ERR_NULL, "%s: a8, sa, w8, sw and y must not be NULL", who);
  if (!workspace || workspace_bytes < kStatusBytes) return fail(ASRQ_ERR_WORKSPACE, "%s: workspace", who);
  if (dtype != ASRQ_F16 && dtype != ASRQ_BF16) return fail(ASRQ_ERR_DTYPE, "%s: dtype %d", who, dtype);
  if (M < 0 || N <= 0 || K <= 0) return fail(ASRQ_ERR_SHAPE, "%s: M=%lld N=%lld K=%lld", who, (long long)M, (long long)N, (long long)K);
  if (!aligned16(a8) || !aligned16(w8) || !aligned16(y) || !aligned16(workspace))
    return fail(ASRQ_ERR_ALIGN, "%s: a8, w8, y and workspace must be 16-byte aligned", who);
  if (!w4a4_gemm_tc_supports(std::max<int64_t>(M, 64), N, K, group_size))
    return fail(ASRQ_ERR_SHAPE,
                "%s: need N%%128==0, K%%128==0, group_size%%128==0, K%%group_size==0 "
                "(N=%lld K=%lld g=%d)", who, (long long)N, (long long)K, group_size);
  if (M > (1ll << 30) || N > (1ll << 30) || K > (1ll << 24)) return fail(ASRQ_ERR_LIMIT, "%s: size", who);
  const DeviceFacts* f;
  int rc;
  if ((rc = device_facts(&f))) return rc;
  if (M == 0) return ASRQ_OK;
  return w4a4_gemm_int8(w8, a8, sa, sw, bias, y, acc_dump, M, N, K, group_size, dtype, fmt, workspace, workspace_bytes,
                        f->sm_count, static_cast<cudaStream_t>(stream));
}

int asrq_w4a4_prepare_weight(const uint8_t* qw, uint8_t* w8, int64_t N, int64_t K, void* stream) {
  return prepare_weight("asrq_w4a4_prepare_weight", qw, w8, N, K, 1, stream);
}
int asrq_w4a4_prepare_weight_f8(const uint8_t* qw, uint8_t* w8, int64_t N, int64_t K, void* stream) {
  return prepare_weight("asrq_w4a4_prepare_weight_f8", qw, w8, N, K, 2, stream);
}
int asrq_hadamard_quant_int8(const void* x, uint8_t* a8, float* sa, int64_t M, int64_t K, int hadamard, int dtype,
                             void* stream) {
  return quant_operand("asrq_hadamard_quant_int8", x, a8, sa, M, K, hadamard, dtype, 1, stream);
}
int asrq_hadamard_quant_f8(const void* x, uint8_t* a8, float* sa, int64_t M, int64_t K, int hadamard, int dtype,
                           void* stream) {
  return quant_operand("asrq_hadamard_quant_f8", x, a8, sa, M, K, hadamard, dtype, 2, stream);
}
int asrq_w4a4_gemm_int8(const uint8_t* a8, const float* sa, const uint8_t* w8, const void* sw, const void* bias,
                        void* y, int32_t* acc_dump, int64_t M, int64_t N, int64_t K, int group_size, int dtype,
                        void* workspace, size_t workspace_bytes, void* stream) {
  return gemm_operand("asrq_w4a4_gemm_int8", a8, sa, w8, sw, bias, y, acc_dump, M, N, K, group_size, dtype, 1,
                      workspace, workspace_bytes, stream);
}
int asrq_w4a4_gemm_f8(const uint8_t* a8, const float* sa, const uint8_t* w8, const void* sw, const void* bias,
                      void* y, int32_t* acc_dump, int64_t M, int64_t N, int64_t K, int group_size, int dtype,
                      void* workspace, size_t workspace_bytes, void* stream) {
  return gemm_operand("asrq_w4a4_gemm_f8", a8, sa, w8, sw, bias, y, acc_dump, M, N, K, group_size, dtype, 2,
                      workspace, workspace_bytes, stream);
}

int asrq_set_option(const char* name, int value) {
  last_error().clear();
  const int i = find_option(name);
  if (i < 0) return fail(ASRQ_ERR_SHAPE, "asrq_set_option: unknown option '%s'", name ? name : "(null)");
  option_table().v[i].store(value);
  option_table().generation.fetch_add(1);
  return ASRQ_OK;
}

int asrq_get_option(const char* name, int* value) {
  last_error().clear();
  const int i = find_option(name);
  if (i < 0 || !value) return fail(ASRQ_ERR_SHAPE, "asrq_get_option: unknown option '%s' or NULL result", name ? name : "(null)");
  *value = option_table().v[i].load();
  return ASRQ_OK;
}

int asrq_check_status(void* workspace, void* stream) {
  last_error().clear();
  if (!workspace) return fail(ASRQ_ERR_NULL, "asrq_check_status: workspace is NULL");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  unsigned host[2] = {0, 0};
  ASRQ_CUDA_TRY(cudaMemcpyAsync(host, workspace, sizeof(host), cudaMemcpyDeviceToHost, st));
  ASRQ_CUDA_TRY(cudaStreamSynchronize(st));
  if (host[0] == 0) return ASRQ_OK;
  ASRQ_CUDA_TRY(cudaMemsetAsync(workspace, 0, sizeof(host), st));
  ASRQ_CUDA_TRY(cudaStreamSynchronize(st));
  return fail(ASRQ_ERR_TIMEOUT, "a device-side wait gave up at site %u", host[1]);
}

int asrq_device_info_query(int device, asrq_device_info* out) {
  last_error().clear();
  if (!out) return fail(ASRQ_ERR_NULL, "asrq_device_info_query: out is NULL");
  cudaDeviceProp prop;
  ASRQ_CUDA_TRY(cudaGetDeviceProperties(&prop, device));
  std::memset(out, 0, sizeof(*out));
  std::strncpy(out->name, prop.name, sizeof(out->name) - 1);
  out->cc_major = prop.major;
  out->cc_minor = prop.minor;
  out->sm_count = prop.multiProcessorCount;
  out->max_smem_per_block_optin = int(prop.sharedMemPerBlockOptin);
  out->l2_bytes = prop.l2CacheSize;
  int v = 0;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrClockRate, device) == cudaSuccess) out->clock_khz = v;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrMemoryClockRate, device) == cudaSuccess) out->mem_clock_khz = v;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrGlobalMemoryBusWidth, device) == cudaSuccess) out->mem_bus_bits = v;
  out->total_mem = prop.totalGlobalMem;
  return ASRQ_OK;
}

}  // extern "C"
#pragma GCC visibility pop
