/*
 * CPU oracle for the zenith_b200 kernels — TEST INFRASTRUCTURE, NOT PRODUCT.
 *
 * Plain C restatement of the reference's (vibeswithkk/ZENITH) arithmetic for the transformer-
 * encoder inference path.  Only tests, the smoke check and the benchmark's CPU-baseline leg may
 * link or call this file; the product never does.  Each function cites the reference lines it
 * follows (paths relative to the reference project).
 *
 * Build: gcc -O2 -ffp-contract=off -shared -fPIC (see oracle/build.py).  -ffp-contract=off is
 * required: the float steps before an int8 rounding must be the same individually rounded IEEE
 * operations as on the GPU (zenith_b200/csrc/det_math.h holds that shared definition).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "../zenith_b200/csrc/det_math.h"

/* acc[m,n] = sum_k A[m,k] * W[n,k], int32.
 * core/src/cuda_kernels.cu:963-978 (int8_matmul_kernel: int32 sum of int8 products) and
 * benchmarks/int8_bench.py:42-45 (a.astype(int32) @ b.astype(int32)); the weight is held as
 * [N,K] (Linear layout, zenith/optimization/qat.py:751-776 multiplies by weight.T). */
void orc_gemm_s8s8_s32(const int8_t* A, const int8_t* W, int32_t* acc, int M, int N, int K) {
  for (int m = 0; m < M; ++m) {
    const int8_t* a = A + (size_t)m * K;
    for (int n = 0; n < N; ++n) {
      const int8_t* w = W + (size_t)n * K;
      int32_t s = 0;
      for (int k = 0; k < K; ++k) s += (int32_t)a[k] * (int32_t)w[k];
      acc[(size_t)m * N + n] = s;
    }
  }
}

/* y = act((float(acc) * x_scale) * w_scale[n] + bias[n])
 * core/src/cuda_kernels.cu:1035-1036 (dequant order), core/src/fused_kernels.cu:47-62 (bias then
 * GELU).  w_scale / bias may be NULL (1 / 0). */
void orc_epilogue_f32(const int32_t* acc, float* y, int M, int N, float x_scale, const float* w_scale,
                      const float* bias, int act) {
  for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) {
      const float v = zen_det_dequant(acc[(size_t)m * N + n], x_scale, w_scale ? w_scale[n] : 1.0f,
                                      bias ? bias[n] : 0.0f);
      y[(size_t)m * N + n] = zen_det_act(v, act);
    }
}

/* q = clamp(round(x / scale + zero_point), -128, 127)
 * core/src/cuda_kernels.cu:918-929 (nearest-even via __float2int_rn), zenith/optimization/qat.py:267
 * (np.round), zenith/optimization/quantization.py:49-53 (round_mode 1: truncation by astype). */
void orc_quantize_f32(const float* x, int8_t* q, size_t n, float scale, int zero_point, int round_mode) {
  for (size_t i = 0; i < n; ++i)
    q[i] = (int8_t)zen_det_round_clamp_i8(ZEN_ADD(ZEN_DIV(x[i], scale), (float)zero_point), round_mode);
}

/* x = (q - zero_point) * scale — core/src/cuda_kernels.cu:941-950. */
void orc_dequantize_f32(const int8_t* q, float* x, size_t n, float scale, int zero_point) {
  for (size_t i = 0; i < n; ++i) x[i] = ZEN_MUL(ZEN_SUB((float)q[i], (float)zero_point), scale);
}

/* tanh-form GELU — core/src/cuda_kernels.cu:115-126. */
void orc_gelu_f32(const float* x, float* y, size_t n) {
  for (size_t i = 0; i < n; ++i) y[i] = zen_det_gelu(x[i]);
}

/* The same GELU with libm tanhf, exactly as the reference writes it; used to measure how far the
 * deterministic evaluation is from it. */
void orc_gelu_libm_f32(const float* x, float* y, size_t n) {
  for (size_t i = 0; i < n; ++i) {
    const float v = x[i];
    const float inner = 0.7978845608028654f * (v + 0.044715f * v * v * v);
    y[i] = 0.5f * v * (1.0f + tanhf(inner));
  }
}

/* tanh as the device evaluates it (det_math.h) and with libm, for the pooler head
 * (HuggingFace BertPooler, the FP reference of benchmarks/bert_hybrid.py:188-196). */
void orc_tanh_f32(const float* x, float* y, size_t n) {
  for (size_t i = 0; i < n; ++i) y[i] = zen_det_tanh(x[i]);
}
void orc_tanh_libm_f32(const float* x, float* y, size_t n) {
  for (size_t i = 0; i < n; ++i) y[i] = tanhf(x[i]);
}

/* y = LayerNorm(x [+ residual]) * gamma + beta, two-pass, biased variance, fp32.
 * core/src/cuda_kernels.cu:132-184 (layernorm_parallel_kernel) and
 * python/src/features_bindings.hpp:116-171 (fused_add_layernorm_cpu). */
void orc_add_layernorm_f32(const float* x, const float* residual, const float* gamma, const float* beta, float* y,
                           int rows, int hidden, float eps) {
  float* v = (float*)malloc(sizeof(float) * (size_t)hidden);
  for (int r = 0; r < rows; ++r) {
    const float* xr = x + (size_t)r * hidden;
    const float* rr = residual ? residual + (size_t)r * hidden : NULL;
    float sum = 0.0f;
    for (int c = 0; c < hidden; ++c) {
      v[c] = rr ? xr[c] + rr[c] : xr[c];
      sum += v[c];
    }
    const float mean = sum / (float)hidden;
    float sq = 0.0f;
    for (int c = 0; c < hidden; ++c) {
      const float d = v[c] - mean;
      sq += d * d;
    }
    const float rstd = 1.0f / sqrtf(sq / (float)hidden + eps);
    for (int c = 0; c < hidden; ++c) y[(size_t)r * hidden + c] = (v[c] - mean) * rstd * gamma[c] + beta[c];
  }
  free(v);
}

/* O = softmax(scale * Q K^T) V per (batch, head), fp32, [B,H,S,D] contiguous.
 * core/src/flash_attention.cu:194-321 (tiled_attention_kernel; scale 1/sqrt(D), output divided by
 * the row sum, nothing stored when the sum is 0), causal j <= i from
 * core/src/flash_attention_v2.cu:362-414, key-padding mask with zeros for a fully masked row from
 * zenith/jax/primitives.py:302-310.  kv_lens may be NULL. */
void orc_attention_f32(const float* Q, const float* K, const float* V, float* O, int B, int H, int S, int D,
                       const int32_t* kv_lens, int causal, float scale) {
  double* p = (double*)malloc(sizeof(double) * (size_t)S);
  for (int b = 0; b < B; ++b) {
    int kvl = kv_lens ? kv_lens[b] : S;
    if (kvl < 0) kvl = 0;
    if (kvl > S) kvl = S;
    for (int h = 0; h < H; ++h) {
      const size_t base = ((size_t)b * H + h) * (size_t)S * D;
      for (int i = 0; i < S; ++i) {
        int lim = kvl;
        if (causal && i + 1 < lim) lim = i + 1;
        double mx = -INFINITY;
        for (int j = 0; j < lim; ++j) {
          double s = 0.0;
          for (int d = 0; d < D; ++d) s += (double)Q[base + (size_t)i * D + d] * (double)K[base + (size_t)j * D + d];
          p[j] = s * (double)scale;
          if (p[j] > mx) mx = p[j];
        }
        double l = 0.0;
        for (int j = 0; j < lim; ++j) {
          p[j] = exp(p[j] - mx);
          l += p[j];
        }
        for (int d = 0; d < D; ++d) {
          double o = 0.0;
          for (int j = 0; j < lim; ++j) o += p[j] * (double)V[base + (size_t)j * D + d];
          O[base + (size_t)i * D + d] = l > 0.0 ? (float)(o / l) : 0.0f;
        }
      }
    }
  }
  free(p);
}

/* orc_attention_f32 for a subset of the query rows: O_rows[b,h,r,:] is row rows[r] of the full result (the same
 * arithmetic, same reference lines); lets a test check long sequences on sampled rows in seconds. */
void orc_attention_rows_f32(const float* Q, const float* K, const float* V, float* O_rows, int B, int H, int S, int D,
                            const int32_t* kv_lens, int causal, float scale, const int32_t* rows, int n_rows) {
  double* p = (double*)malloc(sizeof(double) * (size_t)S);
  for (int b = 0; b < B; ++b) {
    int kvl = kv_lens ? kv_lens[b] : S;
    if (kvl < 0) kvl = 0;
    if (kvl > S) kvl = S;
    for (int h = 0; h < H; ++h) {
      const size_t base = ((size_t)b * H + h) * (size_t)S * D;
      for (int r = 0; r < n_rows; ++r) {
        const int i = rows[r];
        int lim = kvl;
        if (causal && i + 1 < lim) lim = i + 1;
        double mx = -INFINITY;
        for (int j = 0; j < lim; ++j) {
          double s = 0.0;
          for (int d = 0; d < D; ++d) s += (double)Q[base + (size_t)i * D + d] * (double)K[base + (size_t)j * D + d];
          p[j] = s * (double)scale;
          if (p[j] > mx) mx = p[j];
        }
        double l = 0.0;
        for (int j = 0; j < lim; ++j) {
          p[j] = exp(p[j] - mx);
          l += p[j];
        }
        float* out = O_rows + (((size_t)b * H + h) * (size_t)n_rows + (size_t)r) * D;
        for (int d = 0; d < D; ++d) {
          double o = 0.0;
          for (int j = 0; j < lim; ++j) o += p[j] * (double)V[base + (size_t)j * D + d];
          out[d] = l > 0.0 ? (float)(o / l) : 0.0f;
        }
      }
    }
  }
  free(p);
}

/* C[M,N] = A[M,K] . W[N,K]^T in fp32 with double accumulation (checker for the fp16 / TF32 GEMMs). */
void orc_gemm_f32_nt(const float* A, const float* W, float* C, int M, int N, int K) {
  for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) {
      double s = 0.0;
      for (int k = 0; k < K; ++k) s += (double)A[(size_t)m * K + k] * (double)W[(size_t)n * K + k];
      C[(size_t)m * N + n] = (float)s;
    }
}
