/*
 * Deterministic fp32 arithmetic shared by device code (nvcc) and host code (gcc).
 *
 * A requantized int8 output can only be bit-identical on the GPU and on a CPU checker if every
 * float operation before the rounding step is the same correctly-rounded IEEE operation on both
 * sides.  libm tanhf / expf and CUDA's tanhf / expf differ in the last bits, so GELU is DEFINED
 * here from fma / mul / add / div / rint only, each spelled explicitly so that neither compiler
 * may contract or reassociate.  The formula is the reference's tanh-form GELU
 * (core/src/cuda_kernels.cu:115-126, core/src/fused_kernels.cu:47-62):
 *     gelu(x) = 0.5 x (1 + tanh(0.7978845608 (x + 0.044715 x^3)))
 * evaluated as x / (1 + exp(-2u)), the same function written with the logistic identity
 * 0.5 (1 + tanh u) = 1 / (1 + exp(-2u)); exp is 2^n * p(f) with a degree-6 polynomial.
 *
 * Host builds must use -ffp-contract=off.
 */
#ifndef ZEN_DET_MATH_H_
#define ZEN_DET_MATH_H_

#include <stdint.h>

#if defined(__CUDACC__)
#define ZEN_DM_FN __host__ __device__ __forceinline__
#else
#define ZEN_DM_FN static inline
#endif

#if defined(__CUDA_ARCH__)
#define ZEN_FMA(a, b, c) __fmaf_rn((a), (b), (c))
#define ZEN_MUL(a, b) __fmul_rn((a), (b))
#define ZEN_ADD(a, b) __fadd_rn((a), (b))
#define ZEN_SUB(a, b) __fsub_rn((a), (b))
#define ZEN_DIV(a, b) __fdiv_rn((a), (b))
#define ZEN_RINT(a) rintf(a)
#define ZEN_F2I_RN(a) __float2int_rn(a)
#define ZEN_F2I_RZ(a) __float2int_rz(a)
#define ZEN_BITS_TO_F(i) __int_as_float(i)
#define ZEN_F_TO_BITS(f) __float_as_int(f)
#else
#include <math.h>
#include <string.h>
#define ZEN_FMA(a, b, c) fmaf((a), (b), (c))
#define ZEN_MUL(a, b) ((a) * (b))
#define ZEN_ADD(a, b) ((a) + (b))
#define ZEN_SUB(a, b) ((a) - (b))
#define ZEN_DIV(a, b) ((a) / (b))
#define ZEN_RINT(a) rintf(a)
#define ZEN_F2I_RN(a) ((int)lrintf(a))
#define ZEN_F2I_RZ(a) ((int)(a))
static inline float zen_bits_to_f_(int32_t i) {
  float f;
  memcpy(&f, &i, sizeof f);
  return f;
}
#define ZEN_BITS_TO_F(i) zen_bits_to_f_(i)
static inline int32_t zen_f_to_bits_(float f) {
  int32_t i;
  memcpy(&i, &f, sizeof i);
  return i;
}
#define ZEN_F_TO_BITS(f) zen_f_to_bits_(f)
#endif

/* 2^z for z clamped to [-126, 126]: 2^n * p(f), n = rint(z), f = z - n in [-0.5, 0.5],
 * p a degree-6 fit of 2^f (max relative error 8e-8).  NaN maps to 2^-126. */
ZEN_DM_FN float zen_det_exp2(float z) {
  z = z > -126.0f ? z : -126.0f;
  z = z < 126.0f ? z : 126.0f;
  const float n = ZEN_RINT(z);
  const float f = ZEN_SUB(z, n); /* exact */
  float p = 0.00015337577497120947f;
  p = ZEN_FMA(p, f, 0.0013399859890341759f);
  p = ZEN_FMA(p, f, 0.009618519805371761f);
  p = ZEN_FMA(p, f, 0.05550329014658928f);
  p = ZEN_FMA(p, f, 0.24022646248340607f);
  p = ZEN_FMA(p, f, 0.6931471824645996f);
  p = ZEN_FMA(p, f, 1.0f);
  /* p in [0.70, 1.42]; adding n to its exponent field cannot leave the normal range */
  return ZEN_BITS_TO_F(ZEN_F_TO_BITS(p) + ZEN_F2I_RN(n) * 8388608);
}

/* gelu(x) = 0.5 x (1 + tanh(u)), u = 0.7978845608 (x + 0.044715 x^3), evaluated in the
 * algebraically identical logistic form x / (1 + exp(-2u)), which needs one exponential and
 * one division and has no cancellation for small |u|. */
ZEN_DM_FN float zen_det_gelu(float x) {
  const float x2 = ZEN_MUL(x, x);
  const float w = ZEN_FMA(0.044715f, x2, 1.0f);
  const float v = ZEN_MUL(x, w);                       /* x + 0.044715 x^3 */
  const float e = zen_det_exp2(ZEN_MUL(v, -2.302208198144325f)); /* exp(-2u), -2 * 0.79788456 * log2(e) folded */
  return ZEN_DIV(x, ZEN_ADD(1.0f, e));
}

/* tanh(x) = 2 / (1 + exp(-2x)) - 1 with the exponential above (absolute error below 2e-7; the pooler's activation). */
ZEN_DM_FN float zen_det_tanh(float x) {
  const float e = zen_det_exp2(ZEN_MUL(x, -2.885390081777927f)); /* exp(-2x): -2 log2(e) folded */
  return ZEN_SUB(ZEN_DIV(2.0f, ZEN_ADD(1.0f, e)), 1.0f);
}

/* clamp(round(v), -128, 127); mode 0 = nearest-even, 1 = toward zero.  NaN maps to -128. */
ZEN_DM_FN int zen_det_round_clamp_i8(float v, int round_mode) {
  v = v > -128.0f ? v : -128.0f;
  v = v < 127.0f ? v : 127.0f;
  return round_mode == 0 ? ZEN_F2I_RN(v) : ZEN_F2I_RZ(v);
}

/* The W8A8 epilogue, in the order the reference's fused kernel multiplies
 * (core/src/cuda_kernels.cu:1035-1036): (float(acc) * s_x) * s_w, then + bias. */
ZEN_DM_FN float zen_det_dequant(int32_t acc, float x_scale, float w_scale, float bias) {
  const float y = ZEN_MUL(ZEN_MUL((float)acc, x_scale), w_scale);
  return ZEN_ADD(y, bias);
}

ZEN_DM_FN float zen_det_act(float y, int act) {
  if (act == 1) return zen_det_gelu(y);
  if (act == 2) return y > 0.0f ? y : 0.0f;
  return y;
}

#endif /* ZEN_DET_MATH_H_ */
