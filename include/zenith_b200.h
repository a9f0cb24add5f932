/*
 * zenith_b200 — C ABI of the B200 (sm_100a) transformer-encoder kernels.
 *
 * Conventions (all entry points):
 *   - plain C types only; every pointer is a DEVICE pointer unless the name ends in _host;
 *   - buffers are caller-owned; nothing here allocates device memory and nothing synchronises
 *     the device (the two zen_device_status_* calls excepted);
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream);
 *   - the return value is 0 (ZEN_OK) or a ZEN_ERR_* code; nothing throws, nothing prints;
 *   - a kernel-side wait that ran out (ZEN_ERR_TIMEOUT) is reported asynchronously through the
 *     device status word, read with zen_device_status_read().
 *
 * Each declaration names the interface of the reference project (vibeswithkk/ZENITH, paths
 * relative to that project) that it replaces.
 */
#ifndef ZENITH_B200_H_
#define ZENITH_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ZEN_VERSION 100

/* status codes */
#define ZEN_OK 0
#define ZEN_ERR_INVALID_ARG 1   /* null pointer, non-positive extent, bad enum */
#define ZEN_ERR_UNSUPPORTED 2   /* shape / alignment / stride the kernels do not cover */
#define ZEN_ERR_LAUNCH 3        /* cudaGetLastError() after the launch was not cudaSuccess */
#define ZEN_ERR_TIMEOUT 4       /* a bounded device-side wait ran out (device status word) */
#define ZEN_ERR_DRIVER 5        /* tensor-map encoding entry point unavailable or failed */
#define ZEN_ERR_TOO_LARGE 6     /* request exceeds a fixed capacity of the entry point */

/* element types of GEMM outputs */
#define ZEN_DT_S32 0
#define ZEN_DT_F32 1
#define ZEN_DT_F16 2
#define ZEN_DT_S8 3

/* activation fused into a GEMM epilogue */
#define ZEN_ACT_NONE 0
#define ZEN_ACT_GELU 1 /* tanh form: 0.5 x (1 + tanh(0.7978845608 (x + 0.044715 x^3))) */
#define ZEN_ACT_RELU 2

/* rounding used when a value is quantized to int8 */
#define ZEN_ROUND_NEAREST_EVEN 0 /* rint: zenith/optimization/qat.py:267, core/src/cuda_kernels.cu:926 */
#define ZEN_ROUND_TRUNC 1        /* toward zero: zenith/optimization/quantization.py:49-53 */

int zen_version(void);
const char* zen_status_string(int status);

/* Device status word: 0 or the first ZEN_ERR_* recorded by a kernel since the last clear.
 * Both calls synchronise the current device. */
int zen_device_status_read(int* status_host);
int zen_device_status_clear(void);

/* Stream-ordered copy by a copy engine (cudaMemcpyAsync, kind inferred from the pointers): device memory of this or
 * of a peer GPU, a CUDA IPC mapping of another process's buffer, or pinned host memory, in either direction.  No
 * kernel runs, so the copy never takes an SM from the persistent GEMM kernels it overlaps; the multi-GPU gather of
 * the encoder outputs is built on it.  The reference has no multi-GPU data path
 * (benchmarks/mlperf_suite.py:750-850 runs independent replicas). */
int zen_memcpy_async(void* dst, const void* src, size_t bytes, void* stream);

/* Self-test of the wait limit: one small CTA waits on a barrier that nothing signals, in a build of the wait
 * loop whose limit is 1 ms.  The wait gives up by itself, the kernel returns normally and leaves
 * ZEN_ERR_TIMEOUT in the device status word (read it with zen_device_status_read, reset it with
 * zen_device_status_clear).  result3 (device, 3 x uint64, may be NULL): [0] = 1 if the first wait gave up,
 * [1] = 1 if a second waiter of the same CTA left because the abort flag was up, [2] = nanoseconds spent.
 * The reference has host-side fault injectors only (tests/chaos/gpu_chaos.py:143-250). */
int zen_selftest_wait_limit(unsigned long long* result3, void* stream);

/* ------------------------------------------------------------------------------------------
 * W8A8 Linear:  acc[m,n] = sum_k xq[m,k] * wq[n,k]   (int32, exact, tcgen05 kind::i8)
 *   out_dtype S32 : out = acc
 *   otherwise     : y = (float(acc) * x_scale) * w_scale[n] + bias[n]; y = act(y);
 *                   F32: out = y;  F16: out = half(y);
 *                   S8 : out = clamp(round(y / out_scale), -128, 127)
 * xq [M,K] row-major (row stride ldx bytes == elements), wq [N,K] row-major (ldw), out row
 * stride ldo elements.  w_scale may be NULL (treated as 1.0 for every n), bias may be NULL.
 * K, ldx and ldw must be multiples of 16; xq, wq 16-byte aligned.
 * Replaces core/src/cuda_kernels.cu:963-1049 (int8_matmul_kernel, fused_int8_linear_kernel),
 * :918-958 (quantize / dequantize) and core/src/fused_kernels.cu:47-62,317-330 (bias+GELU
 * epilogues that ran as separate kernels).
 * ------------------------------------------------------------------------------------------ */
int zen_linear_i8(const int8_t* xq, int64_t ldx, const int8_t* wq, int64_t ldw, int M, int N, int K, float x_scale,
                  const float* w_scale, const float* bias, int act, int out_dtype, float out_scale, int round_mode,
                  void* out, int64_t ldo, void* stream);

/* zen_linear_i8 plus an L2 prefetch hint: while its CTAs wait for their own operands the kernel asks the
 * memory system to bring up to two read-only ranges into L2 (typically the weights of the GEMMs that
 * follow; a pass's weights do not stay in L2 beside the activations, so each GEMM otherwise starts on
 * HBM-cold weights).  The ranges are only hinted at, never read: results are those of zen_linear_i8.
 * A range with 0 bytes is ignored.  No counterpart in the reference. */
int zen_linear_i8_prefetch(const int8_t* xq, int64_t ldx, const int8_t* wq, int64_t ldw, int M, int N, int K,
                           float x_scale, const float* w_scale, const float* bias, int act, int out_dtype,
                           float out_scale, int round_mode, void* out, int64_t ldo, const void* next0,
                           size_t next0_bytes, const void* next1, size_t next1_bytes, void* stream);

/* W8A8 Linear + residual add + LayerNorm in one kernel, for projections whose output width is the hidden
 * size (attention output, FFN2):
 *   t = (float(acc) * x_scale) * w_scale[n] + bias[n] + residual[m,n];   y = LayerNorm_n(t) * gamma + beta
 * y is written as fp16 [M,N] (contiguous) and, if yq != NULL, also as int8 clamp(round(y / out_scale)) of
 * the fp16 value.  residual fp16 [M,N] (row stride ldr), gamma / beta fp16 [N].  Statistics in fp32 over
 * the un-rounded t (pairwise-combined mean / M2).  N must be 768 or 1024 (four CTAs of a cluster, 192 or 256
 * columns each, share a row through distributed shared memory); other widths: zen_linear_i8 followed by zen_add_layernorm_f16.
 * Replaces the sequence linear -> fused_add_layernorm of the reference's encoder drivers
 * (benchmarks/bert_hybrid.py:121-145; core/src/fused_kernels.cu:145-221). */
int zen_linear_i8_add_layernorm(const int8_t* xq, int64_t ldx, const int8_t* wq, int64_t ldw, int M, int N, int K,
                                float x_scale, const float* w_scale, const float* bias, const void* residual,
                                int64_t ldr, const void* gamma, const void* beta, float eps, void* y, int8_t* yq,
                                float out_scale, int round_mode, void* stream);

/* The same kernel with fp16 operands (fp32 accumulation, no scales): y = LayerNorm(x . w^T + bias + residual),
 * x fp16 [M, K], w fp16 [N, K], N = 768 or 1024, K a multiple of 8.  Replaces linear_fp16 + add_fp16 +
 * layernorm_fp16 (core/src/fp16_kernels.cu:92-122, 154-279). */
int zen_linear_f16_add_layernorm(const void* x, int64_t ldx, const void* w, int64_t ldw, int M, int N, int K,
                                 const float* bias, const void* residual, int64_t ldr, const void* gamma,
                                 const void* beta, float eps, void* y, int8_t* yq, float out_scale, int round_mode,
                                 void* stream);

/* Per-call options: the `flags` argument of the *_ex entry points (0 = the behaviour of the plain forms).
 * The library keeps no process-wide switches; every option travels with the call it applies to.
 *   ZEN_GEMM_CONST_WEIGHTS  promise that the weight operand (wq / w) of THIS call is a constant: not written by
 *                           any work that may still be running on the device when the call is made.  The kernel
 *                           then requests the first weight tiles of each CTA before it waits for the kernel ahead
 *                           of it in the stream (programmatic dependent launch), hiding their latency behind that
 *                           kernel's tail.  Without the flag every operand is read after that wait, so a weight
 *                           matrix produced by the preceding kernel in the stream is safe.  Applies to the int8 and
 *                           the fp16 forms alike.
 *   ZEN_GEMM_TILE_N(bn)     force the tile width (64, 128, 192 or 256; a width the kernel family lacks is ignored);
 *                           a tuning hook for benchmarks.  Not accepted by the *_add_layernorm_ex forms.
 *   ZEN_GEMM_PAIR / _NO_PAIR force or forbid the CTA-pair kernel, which the library otherwise chooses by shape;
 *                           results are identical either way.  Tuning / test hook.
 * None of this has a counterpart in the reference. */
#define ZEN_GEMM_CONST_WEIGHTS 0x1u
#define ZEN_GEMM_NO_PAIR 0x2u /* never run this GEMM on CTA pairs (one CTA per 128-row tile) */
#define ZEN_GEMM_PAIR 0x4u    /* always run it on CTA pairs (two CTAs per 256-row tile, tcgen05 cta_group::2) */
#define ZEN_GEMM_TILE_N(bn) ((unsigned)(bn) << 8)

/* zen_linear_i8_prefetch with per-call options. */
int zen_linear_i8_ex(const int8_t* xq, int64_t ldx, const int8_t* wq, int64_t ldw, int M, int N, int K, float x_scale,
                     const float* w_scale, const float* bias, int act, int out_dtype, float out_scale, int round_mode,
                     void* out, int64_t ldo, const void* next0, size_t next0_bytes, const void* next1,
                     size_t next1_bytes, unsigned flags, void* stream);

/* zen_linear_i8_add_layernorm / zen_linear_f16_add_layernorm with per-call options (ZEN_GEMM_CONST_WEIGHTS). */
int zen_linear_i8_add_layernorm_ex(const int8_t* xq, int64_t ldx, const int8_t* wq, int64_t ldw, int M, int N, int K,
                                   float x_scale, const float* w_scale, const float* bias, const void* residual,
                                   int64_t ldr, const void* gamma, const void* beta, float eps, void* y, int8_t* yq,
                                   float out_scale, int round_mode, unsigned flags, void* stream);
int zen_linear_f16_add_layernorm_ex(const void* x, int64_t ldx, const void* w, int64_t ldw, int M, int N, int K,
                                    const float* bias, const void* residual, int64_t ldr, const void* gamma,
                                    const void* beta, float eps, void* y, int8_t* yq, float out_scale, int round_mode,
                                    unsigned flags, void* stream);

/* FP16 Linear: y = x[M,K] . w[N,K]^T (+ bias[n], fp32) ; act ; out F16 or F32.  fp32 accumulate,
 * tcgen05 kind::f16.  K, ldx, ldw multiples of 8.
 * Replaces core/src/fp16_kernels.cu:92-122 (linear_fp16 = cublasGemmEx + add_bias_fp16_kernel)
 * and zenith/runtime/triton_kernels.py:118-207 (fused Linear+GELU). */
int zen_linear_f16(const void* x, int64_t ldx, const void* w, int64_t ldw, int M, int N, int K, const float* bias,
                   int act, int out_dtype, void* out, int64_t ldo, void* stream);
/* ... with per-call options (see ZEN_GEMM_CONST_WEIGHTS, ZEN_GEMM_TILE_N). */
int zen_linear_f16_ex(const void* x, int64_t ldx, const void* w, int64_t ldw, int M, int N, int K, const float* bias,
                      int act, int out_dtype, void* out, int64_t ldo, unsigned flags, void* stream);

/* FP32 Linear on the tensor cores in TF32: y = act(x[M,K] . w[N,K]^T + bias), fp32 in and out.
 * K, ldx, ldw multiples of 4.  Replaces cuda.linear_gpu = cublasSgemm (TF32 math mode) +
 * add_bias_kernel, python/src/bindings.cpp:1454-1496, core/include/zenith/cublas_ops.hpp:133-156. */
int zen_linear_f32(const float* x, int64_t ldx, const float* w, int64_t ldw, int M, int N, int K, const float* bias,
                   int act, float* out, int64_t ldo, void* stream);

/* C f32[M,N] = A f16[M,K] . B f16[K,N], all row-major contiguous (B is [K,N], not a [N,K] weight).
 * N and K multiples of 8.  Replaces zenith::cuda_kernels::wmma_matmul_f16,
 * core/src/cuda_kernels.cu:698-767 (bound as zenith_cuda.wmma_matmul,
 * core/bindings/cuda_bindings.cpp:110-132). */
int zen_wmma_matmul_f16(const void* A, const void* B, float* C, int M, int N, int K, void* stream);

/* C f32[M,N] = A f32[M,K] . B f32[K,N] on the tensor cores in TF32 (the reference's cuBLAS
 * handle runs in TF32 math mode, core/include/zenith/cublas_ops.hpp:51).  B is first transposed
 * into `workspace` (at least zen_matmul_f32_workspace_bytes(N, K) bytes of device memory, 16-byte
 * aligned, caller-owned), then multiplied as a K-major operand.  K a multiple of 4.
 * Replaces zenith::cuda_kernels::matmul_f32, core/src/cuda_kernels.cu:297-336 (zenith_cuda.matmul). */
size_t zen_matmul_f32_workspace_bytes(int N, int K);
int zen_matmul_f32(const float* A, const float* B, float* C, int M, int N, int K, void* workspace,
                   size_t workspace_bytes, void* stream);

/* The same product as zen_matmul_f32 for callers that have no way to provide a workspace.  It has no
 * counterpart in the reference.  Who needs it: code that runs where device memory cannot be obtained —
 * inside a stream capture (cudaMalloc is not allowed there), in a serving loop that must not hit the
 * allocator's implicit device synchronisation, or behind a dispatcher that hands a kernel nothing but
 * its inputs and outputs.  The transposed copy of B goes to a fixed array that lives in the library
 * image on every GPU that loads it (ZEN_MATMUL_STATIC_MAX_ELEMS floats = 4 MiB per device, held until
 * the process exits); N * K may not exceed that count (ZEN_ERR_TOO_LARGE otherwise).  Nothing is
 * allocated or freed, here or in anything this calls.
 * The first call on each device looks the array's address up (cudaGetSymbolAddress, with that device
 * current); make that first call outside any stream capture.  All calls on a device share the one
 * array: two calls whose kernels may overlap on the GPU (different streams without an ordering
 * between them) race on it and must be serialised by the caller.  The array keeps the previous call's
 * contents; this entry point overwrites every element it later reads, so no clearing is needed. */
#define ZEN_MATMUL_STATIC_MAX_ELEMS (1 << 20)
int zen_matmul_f32_static(const float* A, const float* B, float* C, int M, int N, int K, void* stream);

/* Elementwise.  n = element count.
 * gelu: core/src/cuda_kernels.cu:115-126,559-562 (gelu_f32), core/src/fp16_kernels.cu:128-147.
 * relu: core/src/cuda_kernels.cu relu_f32 (zenith_cuda.relu). */
int zen_gelu_f32(const float* x, float* y, int64_t n, void* stream);
int zen_gelu_f16(const void* x, void* y, int64_t n, void* stream);
int zen_relu_f32(const float* x, float* y, int64_t n, void* stream);
/* tanh, the activation of the BERT pooler (the HuggingFace BertModel the reference measures itself against keeps
 * one: benchmarks/bert_hybrid.py:188-196); the reference's own kernel set has none. */
int zen_tanh_f32(const float* x, float* y, int64_t n, void* stream);
int zen_tanh_f16(const void* x, void* y, int64_t n, void* stream);

/* bias + GELU over [rows, features]: core/src/fused_kernels.cu:47-62,347-353 (fused_bias_gelu). */
int zen_bias_gelu_f32(const float* x, const float* bias, float* y, int rows, int features, void* stream);

/* LayerNorm over the last dim of [rows, hidden]; biased variance, two-pass, fp32 statistics.
 * core/src/cuda_kernels.cu:132-184,564-575 (layernorm_f32); core/src/fp16_kernels.cu:154-261. */
int zen_layernorm_f32(const float* x, const float* gamma, const float* beta, float* y, int rows, int hidden, float eps,
                      void* stream);
int zen_layernorm_f16(const void* x, const void* gamma, const void* beta, void* y, int rows, int hidden, float eps,
                      void* stream);

/* y = LayerNorm(x + residual).  The f16 form can also emit yq = quantize(y, out_scale) as int8
 * (yq may be NULL).  core/src/fused_kernels.cu:145-221,393-399 (fused_add_layernorm);
 * core/src/cuda_kernels.cu:778-859 (fused_residual_layernorm_f32). */
int zen_add_layernorm_f32(const float* x, const float* residual, const float* gamma, const float* beta, float* y,
                          int rows, int hidden, float eps, void* stream);
int zen_add_layernorm_f16(const void* x, const void* residual, const void* gamma, const void* beta, void* y,
                          int8_t* yq, float out_scale, int round_mode, int rows, int hidden, float eps, void* stream);

/* q = clamp(round(x / scale) + zero_point, -128, 127);  x = (q - zero_point) * scale.
 * core/src/cuda_kernels.cu:918-958 (quantize_f32_to_int8, dequantize_int8_to_f32). */
int zen_quantize_f32(const float* x, int8_t* q, int64_t n, float scale, int zero_point, int round_mode, void* stream);
int zen_quantize_f16(const void* x, int8_t* q, int64_t n, float scale, int zero_point, int round_mode, void* stream);
int zen_dequantize_f32(const int8_t* q, float* x, int64_t n, float scale, int zero_point, void* stream);

/* FP8 (e4m3) linear: out = act((float(xq . wq^T) * x_scale) * w_scale[n] + bias[n]) with xq [M,K], wq [N,K] holding
 * e4m3 bit patterns (x / x_scale and w / w_scale[n] rounded to e4m3), products accumulated in fp32 on the tensor
 * cores (tcgen05 kind::f8f6f4); out fp32 or fp16.  A tolerance path like the fp16 GEMM: the accumulation order of
 * the hardware is not specified.  K, ldx, ldw multiples of 16.  flags: ZEN_GEMM_CONST_WEIGHTS, ZEN_GEMM_TILE_N.
 * zen_quantize_e4m3_*: q = e4m3(x / scale), round to nearest even, saturating at +-448.
 * The reference has no FP8 kernel; its roadmap sketches one (docs/SPEEDUP_ROADMAP.md:201-210). */
int zen_linear_f8(const uint8_t* xq, int64_t ldx, const uint8_t* wq, int64_t ldw, int M, int N, int K, float x_scale,
                  const float* w_scale, const float* bias, int act, int out_dtype, void* out, int64_t ldo, unsigned flags,
                  void* stream);
int zen_quantize_e4m3_f32(const float* x, uint8_t* q, int64_t n, float scale, void* stream);
int zen_quantize_e4m3_f16(const void* x, uint8_t* q, int64_t n, float scale, void* stream);

/* Attention forward, O = softmax(scale * Q K^T  [masked]) V, fp16 in / fp16 out, fp32 softmax.
 * Element (b,h,s,d) of Q sits at q + b*q_sb + h*q_sh + s*q_ss + d (strides in elements, d
 * contiguous; strides multiples of 8) and likewise for K, V, O.  kv_lens[b] (NULL = S for all)
 * masks keys >= kv_lens[b]; a row with no valid key yields zeros.  causal keeps key <= query.
 * If oq != NULL the int8 copy clamp(round(o / o_scale)) is written with the O strides as well.
 * head_dim 64 or 128.
 * Replaces core/src/flash_attention.cu:55-355 (tiled_attention_kernel, fp16 twin),
 * core/src/flash_attention_v2.cu:121-462 (causal), core/src/fp16_kernels.cu:416-456 (cuBLAS path). */
int zen_flash_attention_f16(const void* q, const void* k, const void* v, void* o, int8_t* oq, float o_scale, int B,
                            int H, int S, int D, int64_t q_sb, int64_t q_sh, int64_t q_ss, int64_t k_sb, int64_t k_sh,
                            int64_t k_ss, int64_t v_sb, int64_t v_sh, int64_t v_ss, int64_t o_sb, int64_t o_sh,
                            int64_t o_ss, const int32_t* kv_lens, int causal, float scale, void* stream);

/* W8A8 QKV projection and attention of an encoder layer in ONE kernel, for sequences of at most 128 tokens and head
 * size 64:  [Q | K | V] = half((float(xq . wqkv^T) * x_scale) * w_scale[n] + bias[n]) per token, then per (sequence,
 * head)  ctx = softmax(scale * Q K^T [keys >= kv_lens[b] masked]) V.
 * xq int8 [B * S, K] (row stride ldx); wqkv int8 [3 * heads * 64, K] (ldw), rows ordered Q | K | V, each head's 64 rows
 * together; w_scale / bias fp32 [3 * heads * 64] (may be NULL); ctx fp16 [B * S, heads * 64], ctxq (may be NULL) its
 * int8 copy clamp(round(ctx / ctx_scale)); qkv_out (may be NULL) receives the fp16 projection [B * S, 3 * heads * 64].
 * The results equal, bit for bit, zen_linear_i8 (fp16 output) followed by zen_flash_attention_f16 on column slices
 * of that output; the projection never leaves the chip.  next0 / next1: L2 prefetch hints as in
 * zen_linear_i8_prefetch; flags: ZEN_GEMM_CONST_WEIGHTS.  S > 128 returns ZEN_ERR_UNSUPPORTED (use the two calls).
 * Replaces linear_gpu x3 + transposes + attention of the reference's encoder drivers
 * (benchmarks/bert_hybrid.py:96-120) and core/src/flash_attention.cu:194-340. */
int zen_qkv_attention_i8(const int8_t* xq, int64_t ldx, const int8_t* wqkv, int64_t ldw, int B, int S, int heads, int K,
                         float x_scale, const float* w_scale, const float* bias, const int32_t* kv_lens, float scale,
                         void* ctx, int8_t* ctxq, float ctx_scale, void* qkv_out, const void* next0, size_t next0_bytes,
                         const void* next1, size_t next1_bytes, unsigned flags, void* stream);

/* Unpadded batches.  The reference's encoder drivers pad every sequence to the batch's length and spend GEMM work
 * on the padding (benchmarks/bert_hybrid.py:88-120 reshapes [B, S, H] to [B * S, H] for every projection).  Here the
 * valid tokens are packed back to back, sequence b in rows cu_seqlens[b] .. cu_seqlens[b + 1] - 1, every row-wise
 * kernel and GEMM runs on the packed rows as it is, and attention takes its sequences from the offsets.
 *
 * zen_pack_tokens_i32: from padded ids [B, S] (+ optional type ids) and key lengths kv_lens[B] (clamped to [0, S]) to
 *   cu_seqlens[B + 1], ids_packed / pos_packed / type_packed (may be NULL) of `capacity` rows: a sequence's valid
 *   tokens with their positions; rows between the total and the capacity get id 0, position 0 (defined values:
 *   their results are never read).  Rows that would not fit the capacity are dropped.
 * zen_embed_layernorm_unpadded_f16: zen_embed_layernorm_f16 with the position of each row read from pos_packed.
 * zen_qkv_attention_unpadded_i8: zen_qkv_attention_i8 on `rows` packed rows; sequences of at most 128 tokens (a
 *   longer one is cut to its first 128 keys and ZEN_ERR_UNSUPPORTED is recorded in the device status word).  Every
 *   valid row's result equals, bit for bit, the padded call's result for that token.
 * zen_unpad_rows_f16: padded[b * S + s] = packed[cu_seqlens[b] + s] for valid positions, zeros for padding.
 * No counterpart in the reference (its roadmap lists variable-length batching as future work). */
/* zen_flash_attention_unpadded_f16: zen_flash_attention_f16 on packed tensors: token t of Q sits at q + t*q_st + h*q_sh + d
 * (likewise K, V, O), sequence b owns tokens cu_seqlens[b] .. cu_seqlens[b + 1] - 1 (cut at `rows`; at most max_seqlen
 * each: a longer one is cut to its first max_seqlen tokens), causal counts positions within the sequence.  Any
 * sequence length; rows that belong to no sequence are left unwritten. */
int zen_flash_attention_unpadded_f16(const void* q, const void* k, const void* v, void* o, int8_t* oq, float o_scale, int B,
                                     int H, int max_seqlen, int D, int64_t rows, int64_t q_st, int64_t q_sh, int64_t k_st,
                                     int64_t k_sh, int64_t v_st, int64_t v_sh, int64_t o_st, int64_t o_sh,
                                     const int32_t* cu_seqlens, int causal, float scale, void* stream);
int zen_pack_tokens_i32(const int32_t* ids, const int32_t* type_ids, const int32_t* kv_lens, int B, int S, int capacity,
                        int32_t* cu_seqlens, int32_t* ids_packed, int32_t* pos_packed, int32_t* type_packed, void* stream);
int zen_embed_layernorm_unpadded_f16(const int32_t* ids_packed, const int32_t* pos_packed, const int32_t* type_packed,
                                     const void* word, const void* pos, const void* type, const void* gamma,
                                     const void* beta, void* y, int8_t* yq, float out_scale, int round_mode, int rows,
                                     int max_pos, int hidden, int vocab, float eps, void* stream);
int zen_qkv_attention_unpadded_i8(const int8_t* xq, int64_t ldx, const int8_t* wqkv, int64_t ldw, int B, int64_t rows,
                                  const int32_t* cu_seqlens, int heads, int K, float x_scale, const float* w_scale,
                                  const float* bias, float scale, void* ctx, int8_t* ctxq, float ctx_scale, void* qkv_out,
                                  const void* next0, size_t next0_bytes, const void* next1, size_t next1_bytes,
                                  unsigned flags, void* stream);
int zen_unpad_rows_f16(const void* packed, const int32_t* cu_seqlens, int B, int S, int hidden, int capacity, void* padded,
                       void* stream);

/* f32 <-> f16 converts (core/src/fp16_kernels.cu:53-77). */
int zen_convert_f32_to_f16(const float* x, void* y, int64_t n, void* stream);
int zen_convert_f16_to_f32(const void* x, float* y, int64_t n, void* stream);

/* Calibration reductions on the device (a calibration pass then needs no host read-back per tensor).
 *
 * zen_minmax_*: running range of an activation tensor: minmax[0] = min(minmax[0], min x),
 *   minmax[1] = max(minmax[1], max x); minmax is fp32[2] in device memory, initialised by the caller
 *   (+inf, -inf); NaNs are skipped.  Two launches, no atomics; `workspace` (device, 8-byte aligned) must
 *   hold zen_minmax_workspace_bytes().  Replaces TensorStats.update (zenith/optimization/quantization.py:
 *   69-72) and the min / max observer kernels (core/src/qat_cuda.cu:146-227).
 * zen_absmax_rows_f32: out[r] = max_c |w[r, c]|, the per-output-channel observer
 *   (zenith/optimization/qat.py:195-199).
 * zen_quantize_rows_f32: q[r, c] = clamp(round(w[r, c] / scale[r]), -128, 127), per-channel int8 weights
 *   (the int8 form of core/src/qat_cuda.cu:90-114).
 * zen_histogram_*: hist[i] += number of x in bin i of `bins` equal bins over [minmax[0], minmax[1]] (device fp32[2],
 *   read by the kernel: run zen_minmax_* first and the range is the running one, with no host read-back), binned
 *   exactly as numpy.histogram bins a float32 array; hist is int64[bins] in device memory, bins <= 4096.  The running
 *   histogram of TensorStats.update (zenith/optimization/quantization.py:69-83), which the percentile and entropy
 *   calibrators read (:119-214); replaces nothing on the device: the reference's observers are host numpy. */
size_t zen_minmax_workspace_bytes(void);
int zen_minmax_f32(const float* x, int64_t n, float* minmax, void* workspace, size_t workspace_bytes, void* stream);
int zen_minmax_f16(const void* x, int64_t n, float* minmax, void* workspace, size_t workspace_bytes, void* stream);
int zen_histogram_f32(const float* x, int64_t n, const float* minmax, int bins, long long* hist, void* stream);
int zen_histogram_f16(const void* x, int64_t n, const float* minmax, int bins, long long* hist, void* stream);
int zen_absmax_rows_f32(const float* w, int rows, int cols, int64_t ld, float* out, void* stream);
int zen_quantize_rows_f32(const float* w, const float* scale, int rows, int cols, int64_t ldw, int8_t* q, int64_t ldq,
                          int round_mode, void* stream);

/* out[t,:] = LayerNorm(word[ids[t]] + pos[t % seq] + type[type_ids[t]]) in fp16, plus optional
 * int8 copy.  ids/type_ids int32 [tokens]; type_ids may be NULL (row 0 of the type table).
 * core/src/transformer_kernels.cu:236-262 (embedding_f32: word-table gather only). */
int zen_embed_layernorm_f16(const int32_t* ids, const int32_t* type_ids, const void* word, const void* pos,
                            const void* type, const void* gamma, const void* beta, void* y, int8_t* yq,
                            float out_scale, int round_mode, int tokens, int seq, int hidden, int vocab, float eps,
                            void* stream);

#ifdef __cplusplus
}
#endif
#endif /* ZENITH_B200_H_ */
