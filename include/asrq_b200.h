/*
 * asrq_b200 -- C ABI of the B200 (sm_100a) quantized-linear kernels.
 *
 * This is the native boundary behind the reference's `LinearQ` Python module
 * (asrq/core/linear.py:8-66).  It replaces the torch-C++/pybind11 extension of
 * the reference (asrq/matmulq/csrc/bindings.cpp:805-896, built at import by
 * asrq/matmulq/base.py:102-110).  Conventions, chosen against the reference's:
 *
 *   - plain C: raw DEVICE pointers, int64 sizes, the CUDA stream as `void*`
 *     (a cudaStream_t; the reference takes at::cuda::getCurrentCUDAStream(),
 *     bindings.cpp:188);
 *   - every function returns an int status: 0 = ok, negative = argument error
 *     found on the host before any launch, positive = a cudaError_t.  Nothing
 *     here calls exit() (the reference's CUDA_CHECK does, csrc/cuda/common.h:5-12);
 *   - the caller owns all memory, including the scratch `workspace`
 *     (size from asrq_workspace_bytes); no entry point allocates, frees or
 *     synchronises, so all of them are safe on any stream;
 *   - the buffers' device must be the CURRENT device of the calling thread (the library reads
 *     cudaGetDevice for its per-device facts and launches there);
 *   - constant operands (packed weights, scales, zeros, bias; a layer norm's weight and bias; the
 *     output head's matrix) must be complete in memory before the call is ENQUEUED, not merely
 *     ordered before it on the stream: the kernels are launched with programmatic dependent launch
 *     and fetch these operands before they wait for the preceding kernel on the stream.  After writing or repacking weights on a stream,
 *     synchronise that stream once (or set option "no_pdl") before the first call that uses them.
 *     Activations, outputs and the workspace carry ordinary stream ordering;
 *   - all matrices are row-major and contiguous.  `dtype` selects the 16-bit
 *     activation / output format (ASRQ_F16 or ASRQ_BF16); scales, zeros and bias
 *     are always fp16, as LinearQ registers them (linear.py:18-25).
 *
 * Packed weight layout (defined by LinearQ.dequantize_weight, linear.py:33-54):
 *   4-bit: byte j of a row holds k=2j in bits[0,3] and k=2j+1 in bits[4,7];
 *   2-bit: byte j of a row holds k=4j+e in bits[2e,2e+1];
 *   W[n,k] = q[n,k]*scales[n,k/g] + zeros[n,k/g], q unsigned, zeros an additive
 *   fp16 offset.  The W4A4 path instead uses two's-complement signed nibbles in
 *   the same positions (asrq/matmulq/test.py:141-142) and scales only.
 */
#ifndef ASRQ_B200_H_
#define ASRQ_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ASRQ_F16 0
#define ASRQ_BF16 1
#define ASRQ_F32 2 /* accepted only where a function says so (the offline steps) */

/* status codes (negative: rejected on the host, nothing was launched) */
#define ASRQ_OK 0
#define ASRQ_ERR_NULL (-1)      /* a required pointer is NULL */
#define ASRQ_ERR_SHAPE (-2)     /* M/N/K/group_size outside what the kernel supports */
#define ASRQ_ERR_ALIGN (-3)     /* a pointer is not 16-byte aligned */
#define ASRQ_ERR_WORKSPACE (-4) /* workspace missing or smaller than asrq_workspace_bytes */
#define ASRQ_ERR_DTYPE (-5)     /* dtype is neither ASRQ_F16 nor ASRQ_BF16 */
#define ASRQ_ERR_DEVICE (-6)    /* current device is not sm_100 */
#define ASRQ_ERR_TIMEOUT (-7)   /* a bounded device-side wait gave up (see asrq_check_status) */
#define ASRQ_ERR_LIMIT (-8)     /* size beyond a fixed built-in maximum */

/* workspace kinds for asrq_workspace_bytes */
#define ASRQ_WS_A16_GEMV 1
#define ASRQ_WS_A16_GEMM 2
#define ASRQ_WS_W4A4_GEMM 3
#define ASRQ_WS_LINEARQ 4 /* max over everything asrq_linearq_a16 may dispatch to */

/*
 * Bytes of scratch the caller must pass as `workspace` for one call of the
 * given kind and shape.  The first 16640 bytes of every workspace (a 256-byte
 * status block, then 4096 tile counters where the workspace is that large) must
 * be zero before the first use (cudaMemset once); the kernels leave them zero
 * after every call that completes.  Counterpart of mymatmul_workspace_sizes
 * (asrq/matmulq/csrc/bindings.cpp:17-22,192-198), which sized the reference's
 * stream-K workspace and lock array.
 */
size_t asrq_workspace_bytes(int kind, int64_t M, int64_t N, int64_t K);

/*
 * y[M,N] = x[M,K] . dequant(w)[N,K]^T (+ bias[N]) for 4-bit / 2-bit weights, small M
 * (the decode path): split-K skinny GEMM bound by HBM bandwidth.  Any M >= 1 is
 * accepted (row blocks of 16 are streamed one after the other).
 * Requires N % 16 == 0, group_size % 32 == 0 (4-bit) or % 64 == 0 (2-bit),
 * K % 128 == 0 (4-bit) or K % 256 == 0 (2-bit), K % group_size == 0.
 * Replaces the declared-but-sourceless matmul_f16xint4 / matmul_f16xint2 /
 * matmul_w4a16_sym of the reference for M <= 64
 * (asrq/matmulq/csrc/bindings.cpp:44-57, 607-650, 705-747, 773-781).
 */
int asrq_w4a16_gemv(const void* x, const uint8_t* w, const void* scales, const void* zeros,
                    const void* bias, void* y, int64_t M, int64_t N, int64_t K, int group_size,
                    int dtype, void* workspace, size_t workspace_bytes, void* stream);
int asrq_w2a16_gemv(const void* x, const uint8_t* w, const void* scales, const void* zeros,
                    const void* bias, void* y, int64_t M, int64_t N, int64_t K, int group_size,
                    int dtype, void* workspace, size_t workspace_bytes, void* stream);

/*
 * asrq_w4a16_gemv for callers that cannot allocate device memory (a plugin that is only handed
 * input and output buffers, a real-time callback, code running after memory pools are frozen):
 * the scratch lives in a static device array inside the library (16 640 + 4 Mi bytes per GPU,
 * held until exit), so there is no workspace argument and the call allocates nothing.
 * Limits: N <= 8192 (ASRQ_ERR_LIMIT beyond).  The first call on a device looks the array's device
 * address up (make it before any stream capture).  All calls on a device share the array; calls
 * that overlap on the GPU race on it.  Same results as asrq_w4a16_gemv within its tolerance (the
 * K split may differ).  No counterpart in the reference.
 */
int asrq_w4a16_gemv_static(const void* x, const uint8_t* w, const void* scales, const void* zeros,
                           const void* bias, void* y, int64_t M, int64_t N, int64_t K,
                           int group_size, int dtype, void* stream);

/*
 * Same contraction for large M (the prefill / encoder path): weights are unpacked
 * and scaled in registers, staged to shared memory and fed to tcgen05 kind::f16
 * MMAs with TMEM accumulators; activations arrive by TMA.
 * Requires M >= 32, N % 128 == 0, K % 64 == 0, group_size % 64 == 0, K % group_size == 0.
 * For M <= 256 the K range of an output tile may be divided among several blocks
 * (fp32 parts in the workspace, added in a fixed order); with a workspace smaller
 * than asrq_workspace_bytes(ASRQ_WS_A16_GEMM, M, N, K) but at least 256 bytes the
 * call still runs, unsplit.
 * Replaces matmul_f16xint4 / matmul_f16xint2 for M > 64
 * (asrq/matmulq/csrc/bindings.cpp:44-57, 607-650, 705-747).
 */
int asrq_w4a16_gemm(const void* x, const uint8_t* w, const void* scales, const void* zeros,
                    const void* bias, void* y, int64_t M, int64_t N, int64_t K, int group_size,
                    int dtype, void* workspace, size_t workspace_bytes, void* stream);
int asrq_w2a16_gemm(const void* x, const uint8_t* w, const void* scales, const void* zeros,
                    const void* bias, void* y, int64_t M, int64_t N, int64_t K, int group_size,
                    int dtype, void* workspace, size_t workspace_bytes, void* stream);

/*
 * LinearQ.forward (asrq/core/linear.py:56-66) for bits in {2,4}: dispatches on M
 * between the two kernels above, the way the reference's matmul_w4ax switches
 * at M = 64 (asrq/matmulq/csrc/bindings.cpp:749-803).
 */
int asrq_linearq_a16(int bits, const void* x, const uint8_t* w, const void* scales,
                     const void* zeros, const void* bias, void* y, int64_t M, int64_t N,
                     int64_t K, int group_size, int dtype, void* workspace,
                     size_t workspace_bytes, void* stream);

/*
 * The same layer with what follows it in a transformer block fused into the kernel's epilogue:
 *   act = ASRQ_ACT_GELU   y = gelu(layer(x))            (exact erf form; Whisper's fc1)
 *   residual != NULL      y = residual + layer(x)       (residual: M x N, the type of y; out_proj, fc2)
 * Both act on the layer output ROUNDED to the 16-bit type, i.e. they give the bits of the unfused module
 * sequence (LinearQ returns a 16-bit tensor; the activation or the add reads that and rounds again).
 * The tcgen05 kernels (M > 16 on shapes they take) fuse the epilogue; on other paths the library runs
 * one extra elementwise pass over y, so the call is valid for every shape asrq_linearq_a16 takes.
 * y and residual 16-byte aligned, M*N a multiple of 8.  residual may alias y.
 * The reference has no fused form: its model classes call LinearQ, then the activation / the add
 * (asrq/models/transformers/whisper.py:100-125 through the stock encoder / decoder layer forward).
 */
#define ASRQ_ACT_NONE 0
#define ASRQ_ACT_GELU 1
int asrq_linearq_a16_fused(int bits, const void* x, const uint8_t* w, const void* scales, const void* zeros,
                           const void* bias, const void* residual, void* y, int64_t M, int64_t N, int64_t K,
                           int group_size, int dtype, int act, void* workspace, size_t workspace_bytes,
                           void* stream);

/*
 * x' = x + delta (delta may be NULL), h = LayerNorm(x') * gamma + beta over the last dimension.
 * x, delta, x_out (optional; may alias x), h_out: rows x dim in the 16-bit type `dtype`; gamma, beta: dim
 * values of that type.  Statistics in fp32 on the 16-bit-rounded x' (what "add, then layer_norm" computes).
 * The pre-norm residual blocks of the decoder spend as many launches on these two steps as on the
 * quantized layers; the reference leaves them to torch (nn.LayerNorm in its model classes,
 * asrq/models/transformers/whisper.py:119,125).
 */
int asrq_add_layernorm(const void* x, const void* delta, const void* gamma, const void* beta, float eps, void* x_out,
                       void* h_out, int64_t rows, int64_t dim, int dtype, void* stream);

/*
 * x' = x + delta (delta may be NULL), h = RMSNorm(x') * gamma over the last dimension, with the rounding of
 * the Qwen3 decoder's norm module: x' / sqrt(mean(x'^2) + eps) in fp32, rounded to `dtype`, then multiplied by
 * gamma and rounded again.  Same arguments as asrq_add_layernorm without beta.  The reference leaves the step
 * to the stock module (Qwen3RMSNorm in asrq/models/nemo/canary_qwen.py:117-118,131-132).
 */
int asrq_add_rmsnorm(const void* x, const void* delta, const void* gamma, float eps, void* x_out, void* h_out,
                     int64_t rows, int64_t dim, int dtype, void* stream);

/*
 * out[m, i] = silu(gate_up[m, i]) * gate_up[m, inter + i]: the gated activation between a fused gate/up
 * projection (one LinearQ call over 2*inter output features) and the down projection
 * (act_fn(gate_proj(x)) * up_proj(x) of Qwen3MLPQ, asrq/models/nemo/canary_qwen.py:70-86).  silu is rounded to
 * `dtype` before the product, as the unfused sequence rounds it.  gate_up: rows x 2*inter, out: rows x inter,
 * inter a multiple of 8, both 16-byte aligned.
 */
int asrq_silu_mul(const void* gate_up, void* out, int64_t rows, int64_t inter, int dtype, void* stream);

/*
 * Between a fused q/k/v projection and the attention of a Qwen3 decoder block, in one launch: per-head RMS norm of queries
 * and keys (weights q_weight, k_weight of head_dim values), rotary embedding from cos_table / sin_table (max_len x
 * head_dim), and the write of the new keys and values into the caches.  Every step is rounded to `dtype` where the
 * module sequence rounds it (Qwen3AttentionQ.forward of asrq/models/nemo/canary_qwen.py:89-120 runs the stock modules:
 * norm in fp32 then cast, times weight, q * cos + rotate_half(q) * sin).
 *   qkv      B*T rows of (n_q_heads + 2 n_kv_heads) * head_dim: queries, keys, values of one sequence position each;
 *   q_out    B x n_q_heads x T x head_dim;
 *   k_cache, v_cache   B x n_kv_heads x max_len x head_dim; row t of sequence b goes to position pos + t, where pos is
 *            read from pos_device when that is not NULL (a decoding step replayed as a CUDA graph) and is the argument
 *            otherwise.
 * head_dim 64 or 128; qkv, q_out and the caches 8-byte aligned.
 */
int asrq_qk_norm_rope(const void* qkv, const void* q_weight, const void* k_weight, const void* cos_table, const void* sin_table,
                      const int64_t* pos_device, int64_t pos, void* q_out, void* k_cache, void* v_cache, int64_t B, int64_t T,
                      int n_q_heads, int n_kv_heads, int head_dim, int64_t max_len, float eps, int dtype, void* stream);

/*
 * The self-attention of one decoding step (multi-head, one new token per sequence), cache write included: for every
 * sequence b and head h the new key and value (from the fused projection's output row) are stored at position *pos_device
 * of the cache, then out = softmax(scale * q . K[0..pos]^T) . V[0..pos] with fp32 scores, softmax and accumulation.
 * In the reference this is the stock attention module behind WhisperAttentionQ's projections plus its cache update
 * (asrq/models/transformers/whisper.py:38-97 runs the parent class's forward).
 *   qkv       B rows of [q | k | v], each n_heads * head_dim wide, type `dtype`;
 *   kv_cache  (2, B, n_heads, max_len, head_dim): keys, then values; 16-byte aligned; max_len <= 512;
 *   out       B x (n_heads * head_dim);  head_dim 64 or 128;  pos_device: one int64 in device memory, < max_len.
 */
int asrq_decode_self_attention(const void* qkv, void* kv_cache, const int64_t* pos_device, void* out, int64_t B, int n_heads,
                               int head_dim, int64_t max_len, float scale, int dtype, void* stream);

/*
 * The floating-point output head of a decoding step: y[M, N] = x[M, K] . w[N, K]^T, all of the 16-bit type `dtype`,
 * fp32 accumulation, for M <= 32 tokens and a vocabulary-sized N (any N >= 1).  The reference keeps these layers as
 * nn.Linear (proj_out, asrq/models/transformers/whisper.py:268; lm_head, asrq/models/nemo/canary_qwen.py:179); after
 * the 4-bit layers they are the largest read of a decoding step.  K a multiple of 32, at most 3200; x and w 16-byte
 * aligned; w must not be written by work in flight on the stream (it is read ahead of the stream dependency).
 */
int asrq_dense_head(const void* x, const void* w, void* y, int64_t M, int64_t N, int64_t K, int dtype, void* stream);

/*
 * Offline step: round-to-nearest codes of a float weight on the reference's uniform grid, packed, on the device.
 * Per (row, group of group_size inputs): asymmetric scale = (max - min) / (2^bits - 1), zero = min,
 * code = clamp(round((w - zero) / scale), 0, 2^bits - 1); symmetric scale = max|w| / (2^(bits-1) - 1),
 * code = clamp(round(w / scale), -(2^(bits-1) - 1), 2^(bits-1) - 1); round is half-to-even and every operation
 * is rounded to the weight's own type w_dtype (ASRQ_F16, ASRQ_BF16 or ASRQ_F32), as the reference's tensor
 * expressions round it (asrq/quantizers/base.py:61-77, asrq/quantizers/rtn.py:32-46).  The reference stops at
 * fake-quantised floats; this also does the packing it lacks:
 *   layout 0  LinearQ's buffers (asrq/core/linear.py:16-25,43-52): weight uint8 (N, K*bits/8), scales and zeros
 *             fp16 (N, K/group_size); a symmetric grid is stored shifted (code + 2^(bits-1),
 *             zero = -2^(bits-1) * scale) because LinearQ decodes unsigned codes;
 *   layout 1  the W4A4 weight operand (asrq/matmulq/test.py:141-142): two's-complement nibbles (N, K/2), scales only;
 *             bits must be 4 and the grid symmetric; zeros may be NULL.
 * group_size a multiple of 8 that divides K; weight 4-byte aligned.
 */
int asrq_rtn_pack(const void* w, int w_dtype, int bits, int group_size, int symmetric, int layout, uint8_t* weight,
                  void* scales, void* zeros, int64_t N, int64_t K, void* stream);

/*
 * Offline step: out = hadU(w) along K in fp32, the normalised Walsh-Hadamard transform in the butterfly order of
 * matmul_hadU (asrq/transforms/rotation/hadamard_utils.py:64-81; strides 1, 2, ... K/2, then / sqrt(K)), K a power of
 * two up to 8192.  It folds into a weight the rotation that asrq_hadamard_quant_* applies online to the
 * activations (x . W^T == hadU(x) . hadU(W)^T), as the reference's offline fusion does for its rotations
 * (asrq/transforms/rotation/utils.py:382-428).  w: N x K of w_dtype (ASRQ_F16, ASRQ_BF16 or ASRQ_F32), out: N x K fp32.
 */
int asrq_hadamard_fold(const void* w, int w_dtype, float* out, int64_t N, int64_t K, void* stream);

/*
 * W4A4 prologue: optional online Hadamard rotation over K (normalised
 * Walsh-Hadamard, butterflies with strides 1,2,4..K/2 then /sqrt(K), in fp32:
 * asrq/transforms/rotation/hadamard_utils.py:60-81) followed by per-token
 * symmetric int4 quantisation  s = absmax/7 (0 -> 1e-3),  q = rint(v/s)  with
 * IEEE fp32 division (asrq/quantizers/activation.py:26-28, asrq/core/linear.py:77-82).
 * Writes qa[M,K/2] (signed nibbles, even k low) and sa[M] (fp32).
 * hadamard != 0 requires K in {256, 512, 1024, 2048, 4096}; otherwise K % 8 == 0.
 * Replaces per_token_quant_int4 (asrq/matmulq/csrc/bindings.cpp:69-72).
 */
int asrq_hadamard_quant_int4(const void* x, uint8_t* qa, float* sa, int64_t M, int64_t K,
                             int hadamard, int dtype, void* stream);

/*
 * W4A4 GEMM with fused dequant epilogue:
 *   acc[m,n,g] = sum_{k in group g} qa[m,k]*qw[n,k]           (exact int32)
 *   y[m,n]     = sa[m] * sum_g float(acc[m,n,g]) * sw[n,g]  (+ bias[n])
 * qa[M,K/2], qw[N,K/2] signed-nibble packed; sw[N,K/group_size] fp16; sa[M] fp32.
 * If acc_dump is not NULL the int32 group sums are also written to
 * acc_dump[M,N,K/group_size] (for exactness checks).
 * Requires N % 64 == 0, K % 128 == 0, group_size % 128 == 0, K % group_size == 0; the tcgen05
 * kernel takes M >= 64 and N % 128 == 0, other shapes run on a register-tile kernel.
 * Workspace: asrq_workspace_bytes(ASRQ_WS_W4A4_GEMM, M, N, K) (holds the int8 operands).
 * Replaces matmul_wxax / matmul_w4a4 / matmul_int4_rescale
 * (asrq/matmulq/csrc/bindings.cpp:29-43, 552-605, 652-703).
 */
int asrq_w4a4_gemm(const uint8_t* qa, const float* sa, const uint8_t* qw, const void* sw,
                   const void* bias, void* y, int32_t* acc_dump, int64_t M, int64_t N, int64_t K,
                   int group_size, int dtype, void* workspace, size_t workspace_bytes,
                   void* stream);

/*
 * LinearQQ.forward in one call: the prologue above (writing int8 activations straight into the
 * workspace instead of packed nibbles) followed by the GEMM above.  Same integer codes, same
 * int32 group sums and therefore the same output bits as the two-call sequence.
 * x[M,K] fp16/bf16; qw[N,K/2] signed nibbles; sw[N,K/group_size] fp16; y[M,N].
 * Requires N % 128 == 0, K % 128 == 0, group_size % 128 == 0; with hadamard != 0, K in
 * {256, 512, 1024, 2048, 4096}.  Workspace: asrq_workspace_bytes(ASRQ_WS_W4A4_GEMM, M, N, K).
 * Replaces matmul_wxax, which likewise took f16 activations and quantised them into scratch
 * (asrq/matmulq/csrc/bindings.cpp:37-43, 552-605).
 */
int asrq_w4a4_linear(const void* x, const uint8_t* qw, const void* sw, const void* bias, void* y,
                     int64_t M, int64_t N, int64_t K, int group_size, int hadamard, int dtype,
                     void* workspace, size_t workspace_bytes, void* stream);

/*
 * The three steps of asrq_w4a4_linear as separate calls, for callers that keep the expanded
 * weight resident (it depends only on the weights) or want to time the steps:
 *   asrq_w4a4_prepare_weight  qw[N,K/2] signed nibbles -> w8[N,K] int8 holding 16x the value, natural
 *                             k order: the operand format of the tcgen05 kind::i8 kernel.  Done once
 *                             per layer; counterpart of unpack_int4_to_int8 (bindings.cpp:79-80, 373-400).
 *   asrq_hadamard_quant_int8  the prologue, writing a8[M,K] in that same format plus sa[M].
 *                             Same codes as asrq_hadamard_quant_int4 (a8 byte = 16 * code).
 *   asrq_w4a4_gemm_int8       the GEMM on operands in that format; arguments otherwise as
 *                             asrq_w4a4_gemm; workspace >= 256 bytes (status block only).
 *                             Requires N % 128 == 0, K % 128 == 0, group_size % 128 == 0.
 */
int asrq_w4a4_prepare_weight(const uint8_t* qw, uint8_t* w8, int64_t N, int64_t K, void* stream);
int asrq_hadamard_quant_int8(const void* x, uint8_t* a8, float* sa, int64_t M, int64_t K,
                             int hadamard, int dtype, void* stream);
int asrq_w4a4_gemm_int8(const uint8_t* a8, const float* sa, const uint8_t* w8, const void* sw,
                        const void* bias, void* y, int32_t* acc_dump, int64_t M, int64_t N,
                        int64_t K, int group_size, int dtype, void* workspace,
                        size_t workspace_bytes, void* stream);

/*
 * The same three steps with the 8-bit operands in FP8 (e4m3) instead of int8: a byte holds the code
 * itself (-8..7 are exact in e4m3), the GEMM is tcgen05 kind::f8f6f4 with fp32 accumulators in tensor
 * memory.  A group sum is an integer of magnitude <= 128 * 64 and therefore exact in fp32, so results
 * are bit-identical to the int8 path (acc_dump receives the same integers); the drain saves the
 * int->float conversion per output per group.  Operands of the two families do not mix.
 * No counterpart in the reference (its W4A4 declarations are integer-only, bindings.cpp:29-43).
 */
int asrq_w4a4_prepare_weight_f8(const uint8_t* qw, uint8_t* w8, int64_t N, int64_t K, void* stream);
int asrq_hadamard_quant_f8(const void* x, uint8_t* a8, float* sa, int64_t M, int64_t K,
                           int hadamard, int dtype, void* stream);
int asrq_w4a4_gemm_f8(const uint8_t* a8, const float* sa, const uint8_t* w8, const void* sw,
                      const void* bias, void* y, int32_t* acc_dump, int64_t M, int64_t N,
                      int64_t K, int group_size, int dtype, void* workspace,
                      size_t workspace_bytes, void* stream);

/*
 * Tuning and test switches, process-wide integers.  Each option takes its default from the
 * environment variable ASRQ_B200_<NAME IN UPPER CASE>, read once when the library is first used;
 * afterwards only asrq_set_option changes it (no call path reads the environment).  Options:
 *   no_pdl (0)            1: launch every kernel without programmatic dependent launch
 *   mid_kernel (0)        17..64 tokens: 0 = the chain-oriented tensor-core kernel where its grid fits one wave,
 *                         1 = the decode kernel (<= 32 tokens) / the prefill kernel instead
 *   gemv_kernel (0)       decode kernel: 0 auto (strip per block, split K for shapes outside its menu),
 *                         1 strip per block, 2 split K through the workspace, 3 weights staged in
 *                         shared memory ahead of the stream dependency (measured no faster; opt-in)
 *   gemv_xstage (1)       staged decode kernel: 0 = activations read from L2 per fragment, not staged
 *   gemv_cpw (0), gemv_loop (-1)   strip-per-block decode kernel: steps per warp, rounds variant
 *   tc_split (0)          1: no split K in the prefill kernel
 *   tc_bt (0), w4a4_bt (0)         token-tile width of the tcgen05 kernels (0 auto)
 *   tc_pair (-1), w4a4_pair (-1)   CTA-pair variants: -1 auto, 0 off, 1 on
 *   tc_pair_release (0)   CTA-pair prefill kernel: 1 = release/acquire at cluster scope on the
 *                         cross-CTA "operand written" hand-off (slower), 0 = relaxed arrival
 *   trace (0), trace_block (0)     only in builds with -DASRQ_TRACE: pipeline clock marks
 * Returns ASRQ_ERR_SHAPE for an unknown name.  No counterpart in the reference.
 */
int asrq_set_option(const char* name, int value);
int asrq_get_option(const char* name, int* value);

/*
 * Reads the workspace status block back (this one DOES synchronise the stream).
 * Returns ASRQ_OK, or ASRQ_ERR_TIMEOUT when a kernel's bounded wait gave up; the
 * block is cleared on return.  No reference counterpart (its kernels spin unbounded,
 * asrq/matmulq/csrc/cuda/asrq.cu:17-41).
 */
int asrq_check_status(void* workspace, void* stream);

/* Text of the last error raised on the calling thread ("" if none). */
const char* asrq_last_error_string(void);

typedef struct asrq_device_info {
  char name[128];
  int cc_major, cc_minor;
  int sm_count;
  int max_smem_per_block_optin;
  int l2_bytes;
  int clock_khz;
  int mem_clock_khz;
  int mem_bus_bits;
  size_t total_mem;
} asrq_device_info;

/* Properties of `device`; counterpart of get_gpu_metrics (bindings.cpp:101-134). */
int asrq_device_info_query(int device, asrq_device_info* out);

/* Library version, e.g. 100 = 0.1.0. */
int asrq_version(void);

#ifdef __cplusplus
}
#endif
#endif /* ASRQ_B200_H_ */
