// Persistent, warp-specialised tcgen05 GEMM for sm_100a:  D[M,N] = A[M,K] . B^T  with a fused
// epilogue.  One kernel template serves the int8 (kind::i8, s32 accumulators), fp16
// (kind::f16, f32 accumulators) and fp32-as-TF32 (kind::tf32) paths.
//
//   warp 0      : TMA producer  — 128-byte-swizzled tiles of A and B into a STAGES-deep ring
//   warp 1      : allocates TMEM, issues tcgen05.mma (one lane), commits stage / accumulator barriers
//   warps 2..17 : epilogue — four warps per 32-lane TMEM quadrant, each owning one 64-column slab of the
//                 tile: tcgen05.ld in 16-column steps, dequant / bias / activation / requant, then the
//                 32 x 64 block is staged in swizzled shared memory and written by one TMA store
//                 (full 128-byte lines; edges clipped by the tensor map).  fp32 / int32 outputs and
//                 unaligned outputs use per-thread 16-byte global stores instead.
//
// TMEM holds two accumulators (2 x BN columns) so the epilogue of tile i overlaps the MMAs of
// tile i+1.  CTAs are persistent: tile t = blockIdx.x + i * gridDim.x, M-fastest.
//
// A is always K-major ([M,K] row-major).  B is K-major ([N,K] row-major, a Linear weight) or,
// with B_MN, MN-major ([K,N] row-major, the right operand of a plain matmul).
// Out-of-range rows / columns / K are zero-filled by TMA on load and masked on store.
#pragma once
#include "zen_common.cuh"
#include "det_math.h"

namespace zen {

enum { KIND_I8 = 0, KIND_F16 = 1, KIND_TF32 = 2, KIND_F8 = 3 };  // F8: e4m3 operands, fp32 accumulation

struct GemmParams {
  int M, N, K;
  int tiles_m, tiles_n, num_k_blocks;
  void* out;
  int64_t ldo;
  int out_dtype;
  int act;
  int round_mode;
  float x_scale;
  float out_scale;
  const float* w_scale;
  const float* bias;
  int staged_store;  // 1: fp16 / int8 output leaves through shared memory and TMA stores
  // L2 prefetch hint: read-only ranges (16-byte aligned, sizes multiples of 16) that later kernels will
  // read, e.g. the next GEMMs' weights; every CTA asks for its slice while it waits for its own operands
  const uint8_t* pf_ptr[2];
  uint64_t pf_bytes[2];
  // 1: B is constant (weights): its first tiles may be requested before the kernel waits for its predecessor
  int early_b;
};

// One CTA's share of an L2 prefetch range, in requests of at most 32 KB (a hint: nothing waits on it).
__device__ __forceinline__ void prefetch_slice_l2(const uint8_t* ptr, uint64_t bytes, uint32_t cta, uint32_t n_ctas) {
  const uint64_t per = ((bytes + n_ctas - 1) / n_ctas + 127u) & ~uint64_t(127);
  const uint64_t lo = uint64_t(cta) * per;
  if (lo >= bytes) return;
  const uint64_t hi = lo + per < bytes ? lo + per : bytes;
  for (uint64_t off = lo; off < hi; off += 32768u) {
    const uint32_t sz = uint32_t(hi - off < 32768u ? hi - off : 32768u);
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(ptr + off), "r"(sz) : "memory");
  }
}

template <int KIND>
struct GemmKind;
template <>
struct GemmKind<KIND_I8> {
  static constexpr int ELEM = 1;
};
template <>
struct GemmKind<KIND_F16> {
  static constexpr int ELEM = 2;
};
template <>
struct GemmKind<KIND_TF32> {
  static constexpr int ELEM = 4;
};
template <>
struct GemmKind<KIND_F8> {
  static constexpr int ELEM = 1;
};

constexpr int GEMM_BM = 128;
constexpr int GEMM_EPI_WARPS = 16;
constexpr int GEMM_THREADS = 64 + 32 * GEMM_EPI_WARPS;

template <int BN>
__host__ __device__ constexpr uint32_t gemm_tmem_cols() {
  return 2 * BN <= 32 ? 32u : 2 * BN <= 64 ? 64u : 2 * BN <= 128 ? 128u : 2 * BN <= 256 ? 256u : 512u;
}

template <int BN, int STAGES>
__host__ __device__ constexpr size_t gemm_smem_bytes() {
  // ring + output staging (4 KB per active epilogue warp) + barriers/flags (256 B) + per-epilogue-warp
  // scale and bias entries + alignment slack
  return size_t(STAGES) * (GEMM_BM * 128 + BN * 128) + size_t((BN + 63) / 64) * 4 * 4096 + 256 +
         size_t(GEMM_EPI_WARPS) * 3 * 64 * 4 + 1024;
}

template <int KIND>
__device__ __forceinline__ void issue_mma(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
  if constexpr (KIND == KIND_I8) mma_i8_ss(d, a, b, idesc, acc);
  else if constexpr (KIND == KIND_F16) mma_f16_ss(d, a, b, idesc, acc);
  else if constexpr (KIND == KIND_F8) mma_f8_ss(d, a, b, idesc, acc);
  else mma_tf32_ss(d, a, b, idesc, acc);
}

// 16-byte stores of NW consecutive 32-bit words (dst 16-byte aligned)
template <int NW>
__device__ __forceinline__ void store_words(void* dst, const uint32_t* w) {
  uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
  for (int i = 0; i < NW / 4; ++i) d4[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float rcp_approx(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// GELU through the hardware exp2 / reciprocal units.  Same formula and same argument of the
// exponential (bit for bit) as zen_det_gelu; differs from it by less than 1e-6 relative.
__device__ __forceinline__ float gelu_fast(float x) {
  const float x2 = ZEN_MUL(x, x);
  const float w = ZEN_FMA(0.044715f, x2, 1.0f);
  const float v = ZEN_MUL(x, w);
  const float e = ex2_approx(ZEN_MUL(v, -2.302208198144325f));
  return x * rcp_approx(1.0f + e);
}

constexpr int GEMM_CW = 16;  // accumulator columns per epilogue step (kept small: the step is the unrolled unit)

// Requantisation to int8 with the exact result of  clamp(round(act(y) / out_scale))  at a fraction of
// its cost.  y is exact; the quotient t is formed with approximate arithmetic (hardware exp2 /
// reciprocal, reciprocal multiply): relative error below 1e-6, i.e. below 1e-6 |t| of an int8 step.
// Unless t lies within 4e-6 |t| + 2e-6 of a rounding boundary its rounding is already the exact
// answer; the rare elements that do are recomputed with the individually rounded IEEE operations of
// det_math.h, so the output is bit-identical to the CPU definition everywhere.  Nearest-even rounding uses the 1.5 * 2^23 constant (exact rint for
// |t| < 2^22, the integer falls out of the mantissa), which keeps the conversion units free.
template <int ACT>
__device__ __forceinline__ uint32_t requant_fast(const float (&yfast)[GEMM_CW], float inv_scale, int round_mode,
                                                 int (&q)[GEMM_CW]) {
  constexpr float MAGIC = 12582912.0f;  // 1.5 * 2^23
  uint32_t risky = 0;
  if (round_mode == 0) {
#pragma unroll
    for (int j = 0; j < GEMM_CW; ++j) {
      float g = yfast[j];
      if constexpr (ACT == ZEN_ACT_GELU) g = gelu_fast(g);
      if constexpr (ACT == ZEN_ACT_RELU) g = fmaxf(g, 0.0f);
      const float tc = fminf(fmaxf(g * inv_scale, -128.0f), 127.0f);  // NaN -> -128, as in the exact definition
      const float m = tc + MAGIC;
      q[j] = __float_as_int(m) - 0x4B400000;
      // |tc - rint(tc)| close to 0.5 <=> close to a rounding boundary (a clamped value has distance 0)
      if (fabsf(tc - (m - MAGIC)) > fmaf(fabsf(tc), -4e-6f, 0.5f - 2e-6f)) risky |= 1u << j;
    }
  } else {
#pragma unroll
    for (int j = 0; j < GEMM_CW; ++j) {
      float g = yfast[j];
      if constexpr (ACT == ZEN_ACT_GELU) g = gelu_fast(g);
      if constexpr (ACT == ZEN_ACT_RELU) g = fmaxf(g, 0.0f);
      const float t = g * inv_scale;
      q[j] = __float2int_rz(fminf(fmaxf(t, -128.0f), 127.0f));
      if (fabsf(t - rintf(t)) < 1e-3f && fabsf(t) < 130.0f) risky |= 1u << j;  // boundaries are the integers
    }
  }
  return risky;
}

__device__ __forceinline__ void pack_q(const int (&q)[GEMM_CW], uint32_t (&packed)[GEMM_CW / 4]) {
#pragma unroll
  for (int j = 0; j < GEMM_CW / 4; ++j)
    packed[j] = (uint32_t(q[4 * j]) & 0xffu) | ((uint32_t(q[4 * j + 1]) & 0xffu) << 8) |
                ((uint32_t(q[4 * j + 2]) & 0xffu) << 16) | ((uint32_t(q[4 * j + 3]) & 0xffu) << 24);
}

// One GEMM_CW-column step of one accumulator row: dequant / bias / activation / conversion / store.
// OUT and ACT are compile-time so that the independent element chains carry no branches and the
// compiler can interleave them.
// `stage` != nullptr: this lane's row of the warp's staging block (fp16: 128-byte rows, 128B swizzle;
// int8: 64-byte rows, 64B swizzle — the layouts the output tensor map expects); `istep` is the
// position of the step inside the 64-column slab.
template <int KIND, int OUT, int ACT>
__device__ __forceinline__ void epilogue_chunk(const uint32_t (&r)[GEMM_CW], const float* sc, const float* bi,
                                               const GemmParams& p, int row, int col0, bool full, float inv_scale,
                                               uint8_t* stage, int lane, int istep) {
  constexpr int CW = GEMM_CW;
  const int nvalid = p.N - col0;  // >= 1
  if constexpr (OUT == ZEN_DT_S32) {
    int32_t* o = static_cast<int32_t*>(p.out) + int64_t(row) * p.ldo + col0;
    if (full) store_words<CW>(o, r);
    else {
#pragma unroll
      for (int j = 0; j < CW; ++j)
        if (j < nvalid) o[j] = int32_t(r[j]);
    }
    return;
  } else {
    float y[CW];
#pragma unroll
    for (int j4 = 0; j4 < CW / 4; ++j4) {
      const float4 s4 = reinterpret_cast<const float4*>(sc)[j4];
      const float4 b4 = reinterpret_cast<const float4*>(bi)[j4];
      const float ss[4] = {s4.x, s4.y, s4.z, s4.w};
      const float bb[4] = {b4.x, b4.y, b4.z, b4.w};
      if constexpr (KIND == KIND_I8) {
        // zen_det_dequant on column pairs: packed fp32x2 products, each rounded before the bias add
        const float2 xs2 = make_float2(p.x_scale, p.x_scale);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int j = 4 * j4 + 2 * h;
          const float2 a = make_float2(float(int32_t(r[j])), float(int32_t(r[j + 1])));
          const float2 v = f2mul_then_add(f2mul(a, xs2), make_float2(ss[2 * h], ss[2 * h + 1]),
                                          make_float2(bb[2 * h], bb[2 * h + 1]));
          y[j] = v.x;
          y[j + 1] = v.y;
        }
      } else if constexpr (KIND == KIND_F8) {
        // operands were scaled into the e4m3 range: (acc * x_scale) * w_scale[n] + bias, as on the int8 path
        const float2 xs2 = make_float2(p.x_scale, p.x_scale);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int j = 4 * j4 + 2 * h;
          const float2 a = make_float2(__uint_as_float(r[j]), __uint_as_float(r[j + 1]));
          const float2 v = f2mul_then_add(f2mul(a, xs2), make_float2(ss[2 * h], ss[2 * h + 1]),
                                          make_float2(bb[2 * h], bb[2 * h + 1]));
          y[j] = v.x;
          y[j + 1] = v.y;
        }
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) y[4 * j4 + e] = ZEN_ADD(__uint_as_float(r[4 * j4 + e]), bb[e]);
      }
    }
    if constexpr (OUT == ZEN_DT_S8) {
      uint32_t w[CW / 4];
      int q[CW];
      const uint32_t risky = requant_fast<ACT>(y, inv_scale, p.round_mode, q);
      if (risky) {
#pragma unroll
        for (int j = 0; j < CW; ++j)
          if (risky & (1u << j))
            q[j] = zen_det_round_clamp_i8(ZEN_DIV(zen_det_act(y[j], ACT), p.out_scale), p.round_mode);
      }
      pack_q(q, w);
      if (stage != nullptr) {
        *reinterpret_cast<uint4*>(stage + lane * 64 + ((istep ^ ((lane >> 1) & 3)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
        return;
      }
      int8_t* o = static_cast<int8_t*>(p.out) + int64_t(row) * p.ldo + col0;
      if (full) store_words<CW / 4>(o, w);
      else {
#pragma unroll
        for (int j = 0; j < CW; ++j)
          if (j < nvalid) o[j] = int8_t((w[j >> 2] >> (8 * (j & 3))) & 0xffu);
      }
    } else {
      // int8 GEMMs keep the bit-exact activation; the fp16 / TF32 GEMMs are tolerance paths and use
      // the hardware exp2 / reciprocal form
#pragma unroll
      for (int j = 0; j < CW; ++j) {
        if constexpr (ACT == ZEN_ACT_GELU) y[j] = (KIND == KIND_I8) ? zen_det_gelu(y[j]) : gelu_fast(y[j]);
        if constexpr (ACT == ZEN_ACT_RELU) y[j] = y[j] > 0.0f ? y[j] : 0.0f;
      }
      if constexpr (OUT == ZEN_DT_F32) {
        float* o = static_cast<float*>(p.out) + int64_t(row) * p.ldo + col0;
        if (full) store_words<CW>(o, reinterpret_cast<const uint32_t*>(y));
        else {
#pragma unroll
          for (int j = 0; j < CW; ++j)
            if (j < nvalid) o[j] = y[j];
        }
      } else {
        __half* o = static_cast<__half*>(p.out) + int64_t(row) * p.ldo + col0;
        uint32_t w[CW / 2];
#pragma unroll
        for (int j = 0; j < CW / 2; ++j) {
          const __half2 h = __floats2half2_rn(y[2 * j], y[2 * j + 1]);
          w[j] = *reinterpret_cast<const uint32_t*>(&h);
        }
        if (stage != nullptr) {
          uint8_t* srow = stage + lane * 128;
          *reinterpret_cast<uint4*>(srow + (((2 * istep) ^ (lane & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
          *reinterpret_cast<uint4*>(srow + (((2 * istep + 1) ^ (lane & 7)) << 4)) = make_uint4(w[4], w[5], w[6], w[7]);
          return;
        }
        if (full) store_words<CW / 2>(o, w);
        else {
#pragma unroll
          for (int j = 0; j < CW; ++j)
            if (j < nvalid) o[j] = __ushort_as_half((unsigned short)((w[j >> 1] >> (16 * (j & 1))) & 0xffffu));
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// int8 accumulators -> int8 outputs, nearest-even: the FFN1 epilogue, which is bound by instruction
// issue and by the conversion / special-function unit, not by memory.  Differences from the generic
// step: (1) the s32 -> f32 conversion goes through the 1.5 * 2^23 constant on the integer and FP32
// pipes (exact for |acc| < 2^22; anything larger is caught by `span` and takes the exact path), which
// leaves the conversion unit to the exponential and the reciprocal; (2) the exact recomputation is a
// rolled out-of-line loop over the flagged columns that reads the accumulators again from tensor
// memory, so the straight-line step body stays small.  Returns the mask of this lane's elements that
// must be recomputed.
// ---------------------------------------------------------------------------------------------
// The FP32 arithmetic runs on column pairs with the packed fp32x2 instructions of sm_100 (individually
// rounded, so bit-identical to the scalar forms): one issue slot for two operations.
// The fast path differs from the definition in two places, both covered by the boundary test:
// * it dequantises with ONE fused multiply-add, y' = fl(acc * c + b), c = fl(x_scale * w_scale[n]), instead of the
//   definition's three rounded operations y = fl(fl(fl(acc * x_scale) * w_scale) + b): with u = 2^-24,
//   |y' - y| <= 3u |acc x_scale w_scale| + 2u |y| <= 3.0e-7 |y| + 1.8e-7 |b|; through the activation (|gelu'| <= 1.13,
//   |y gelu'(y)| <= 0.2 for y < 0, |y| <= gelu(y) + 0.17 for y > 0) and the output scale that is at most
//   3.4e-7 |t| + inv_scale (6e-8 + 2.1e-7 |b|) in t = act(y) / out_scale.  The test flags every element whose t lies
//   within 5e-6 |t| + 2e-6 + inv_scale (1.6e-7 + 4.2e-7 max|b|) of a rounding boundary (the first two terms cover the
//   approximate exponential / reciprocal and the reciprocal multiply; the last is the bound above, doubled);
// * it does not clamp in floating point: the rounded integers are saturated when they are packed.  rint(t) through
//   the 1.5 * 2^23 constant is exact for |t| < 2^22, and any larger |t| fails the test (5e-6 |t| alone exceeds 0.5
//   from |t| = 100000 on), as does a NaN (the comparison counts an unordered result as "near a boundary").  Values far
//   outside the int8 range are flagged more often than values inside it: a cost only for an output scale chosen far
//   too small.
// Flagged elements are recomputed with the definition itself (requant_i8_fixup).
//
template <int ACT>
__device__ __forceinline__ uint32_t requant_i8_step(const uint32_t (&r)[GEMM_CW], const float* fold, const float* bi,
                                                    float risk_thr, float inv_scale, uint32_t (&w)[GEMM_CW / 4]) {
  constexpr float MAGIC = 12582912.0f;  // 1.5 * 2^23
  const float2 neg_magic = make_float2(-MAGIC, -MAGIC);
  const float2 pos_magic = make_float2(MAGIC, MAGIC);
  const float2 inv2 = make_float2(inv_scale, inv_scale);
  uint32_t span = 0;
  uint32_t risky = 0;
#pragma unroll
  for (int j4 = 0; j4 < GEMM_CW / 4; ++j4) {
    const float4 s4 = reinterpret_cast<const float4*>(fold)[j4];
    const float4 b4 = reinterpret_cast<const float4*>(bi)[j4];
    uint32_t mb[4];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int j = 4 * j4 + 2 * h;
      const uint32_t t0 = r[j] + 0x4B400000u;  // bits of the float 1.5 * 2^23 + acc while |acc| < 2^22
      const uint32_t t1 = r[j + 1] + 0x4B400000u;
      span |= (t0 ^ 0x4B000000u) | (t1 ^ 0x4B000000u);  // any bit >= 23 set: acc outside that range
      const float2 a = f2add(make_float2(__uint_as_float(t0), __uint_as_float(t1)), neg_magic);  // == float(acc), exact
      const float2 ss = h ? make_float2(s4.z, s4.w) : make_float2(s4.x, s4.y);
      const float2 bb = h ? make_float2(b4.z, b4.w) : make_float2(b4.x, b4.y);
      float2 g = f2fma(a, ss, bb);  // one rounding instead of zen_det_dequant's three
      if constexpr (ACT == ZEN_ACT_GELU) {
        // gelu_fast on both halves: x / (1 + 2^(x (c + 0.044715 c x^2))), c = -2 * 0.79788456 * log2(e) folded into
        // the polynomial's coefficients
        const float2 x2 = f2mul(g, g);
        const float2 wv = f2fma(make_float2(-0.10294324f, -0.10294324f), x2, make_float2(-2.3022082f, -2.3022082f));
        const float2 arg = f2mul(g, wv);
        const float2 den = f2add(make_float2(1.0f, 1.0f), make_float2(ex2_approx(arg.x), ex2_approx(arg.y)));
        g = f2mul(g, make_float2(rcp_approx(den.x), rcp_approx(den.y)));
      }
      if constexpr (ACT == ZEN_ACT_RELU) g = make_float2(fmaxf(g.x, 0.0f), fmaxf(g.y, 0.0f));
      const float2 t = f2mul(g, inv2);
      // NaN -> -128, as in the exact definition
      const float2 m = f2add(t, pos_magic);  // mantissa == 2^22 + rint(t) in two's complement
      const float2 d = f2fma(f2add(m, neg_magic), make_float2(-1.0f, -1.0f), t);  // t - rint(t), exact
      // |t - rint(t)| close to 0.5 <=> close to a rounding boundary
      if (!(fmaf(fabsf(t.x), 5e-6f, fabsf(d.x)) <= risk_thr)) risky |= 1u << j;
      if (!(fmaf(fabsf(t.y), 5e-6f, fabsf(d.y)) <= risk_thr)) risky |= 1u << (j + 1);
      mb[2 * h] = __float_as_uint(m.x) - 0x4B400000u;  // rint(t) as a 32-bit integer
      mb[2 * h + 1] = __float_as_uint(m.y) - 0x4B400000u;
    }
    w[j4] = pack_sat_s8x4(mb[0], mb[1], mb[2], mb[3]);
  }
  return span >= 0x00800000u ? (1u << GEMM_CW) - 1u : risky;
}

// The exact definition for the columns flagged in `any` (the union of the lanes' masks), one column
// per iteration, starting at tensor-memory address `taddr` (the whole warp must call this: the loads
// are warp-collective).  Each lane overwrites the output bytes at `dst` that its own mask flags.
template <int ACT>
__device__ __noinline__ void requant_i8_fixup(uint32_t taddr, const float* sc, const float* bi, float x_scale,
                                              float out_scale, uint32_t any, uint32_t mine, int8_t* dst) {
  while (any != 0) {
    const int j = __ffs(int(any)) - 1;
    any &= any - 1u;
    uint32_t v;
    tmem_ld_32x1(taddr + uint32_t(j), v);
    tmem_wait_ld();
    if (mine & (1u << j)) {
      const float y = zen_det_dequant(int32_t(v), x_scale, sc[j], bi[j]);
      dst[j] = int8_t(zen_det_round_clamp_i8(ZEN_DIV(zen_det_act(y, ACT), out_scale), 0));
    }
    __syncwarp();
  }
}

// One step of the int8 -> int8 nearest-even epilogue (all 32 lanes must call it).
template <int ACT>
__device__ __forceinline__ void epilogue_step_s8(const uint32_t (&r)[GEMM_CW], uint32_t taddr, const float* sc,
                                                 const float* bi, const float* fold, float risk_thr, const GemmParams& p,
                                                 int row, int col0, bool row_ok, bool vec_ok, float inv_scale,
                                                 uint8_t* stage, int lane, int istep) {
  uint32_t w[GEMM_CW / 4];
  uint32_t redo = requant_i8_step<ACT>(r, fold, bi, risk_thr, inv_scale, w);
  const int nvalid = p.N - col0;
  int8_t* dst;
  bool live;
  if (stage != nullptr) {
    dst = reinterpret_cast<int8_t*>(stage + lane * 64 + ((istep ^ ((lane >> 1) & 3)) << 4));
    live = true;
    *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
  } else {
    dst = static_cast<int8_t*>(p.out) + int64_t(row) * p.ldo + col0;
    live = row_ok && nvalid > 0;
    if (live) {
      if (vec_ok && nvalid >= GEMM_CW) store_words<GEMM_CW / 4>(dst, w);
      else {
#pragma unroll
        for (int j = 0; j < GEMM_CW; ++j)
          if (j < nvalid) dst[j] = int8_t((w[j >> 2] >> (8 * (j & 3))) & 0xffu);
      }
    }
  }
  if (!live) redo = 0;
  else if (stage == nullptr && nvalid < GEMM_CW) redo &= (1u << nvalid) - 1u;
  const uint32_t any = __reduce_or_sync(0xffffffffu, redo);
  if (any != 0) requant_i8_fixup<ACT>(taddr, sc, bi, p.x_scale, p.out_scale, any, redo, dst);
}

template <int KIND, int OUT>
__device__ __forceinline__ void epilogue_chunk_act(const uint32_t (&r)[GEMM_CW], const float* sc, const float* bi,
                                                   const GemmParams& p, int row, int col0, bool full, float inv_scale,
                                                   uint8_t* stage, int lane, int istep) {
  if (p.act == ZEN_ACT_GELU)
    epilogue_chunk<KIND, OUT, ZEN_ACT_GELU>(r, sc, bi, p, row, col0, full, inv_scale, stage, lane, istep);
  else if (p.act == ZEN_ACT_RELU)
    epilogue_chunk<KIND, OUT, ZEN_ACT_RELU>(r, sc, bi, p, row, col0, full, inv_scale, stage, lane, istep);
  else
    epilogue_chunk<KIND, OUT, ZEN_ACT_NONE>(r, sc, bi, p, row, col0, full, inv_scale, stage, lane, istep);
}

// ---------------------------------------------------------------------------------------------
// Epilogue role of the persistent GEMM kernels (warps 2..17 of a CTA), shared by the one-CTA kernel below and
// the CTA-pair kernel of gemm_pair.cuh.  The calling CTA owns 128 rows of every tile it works on:
//   tile t (t = first_tile, first_tile + tile_step, ...) covers rows (t % p.tiles_m) * TILE_M + row_off .. + 127
//   and columns (t / p.tiles_m) * BN .. + BN - 1,
// with TILE_M = 128 (one CTA per tile, row_off = 0) or 256 (a CTA pair per tile, row_off = 128 * rank).
// `tempty` releases an accumulator to the MMA issuer: a local barrier on which every epilogue thread arrives
// (one CTA), or the cluster address of the leader CTA's barrier on which one lane per warp arrives (pair).
// ---------------------------------------------------------------------------------------------
struct TmemEmptySignal {
  uint64_t* local;        // one-CTA kernel: tempty_bar[2] of this CTA (count = epilogue threads)
  uint32_t cluster_addr;  // pair kernel: shared::cluster address of the leader's tempty_bar[0] (count = warps of both CTAs)
};

template <bool PAIR>
__device__ __forceinline__ void release_accumulator(const TmemEmptySignal& sig, int acc, int lane) {
  if constexpr (PAIR) {
    __syncwarp();
    if (lane == 0) mbar_arrive_remote(sig.cluster_addr + uint32_t(acc) * 8u);
  } else {
    mbar_arrive(&sig.local[acc]);
  }
}

template <int KIND, int BN, bool PAIR>
__device__ __forceinline__ void gemm_epilogue_role(const GemmParams& p, const CUtensorMap& tmap_c, uint32_t tmem_base,
                                                   uint8_t* out_stage, float* epi_rows, uint64_t* tfull_bar,
                                                   const TmemEmptySignal& tempty, volatile int* abort_flag, int warp,
                                                   int lane, int first_tile, int tile_step, int num_tiles, int row_off) {
  constexpr int TILE_M = PAIR ? 2 * GEMM_BM : GEMM_BM;
  const int quad = warp & 3;        // TMEM lane quadrant this warp may read: rows quad*32 .. +31 of the CTA's 128
  const int sub = (warp - 2) >> 2;  // 64-column slab of the tile owned by this warp
  constexpr int STEPS = 64 / GEMM_CW;
  if (sub * 64 < BN) {
    float* s_scale = epi_rows + (warp - 2) * 3 * 64;
    float* s_bias = s_scale + 64;
    float* s_fold = s_bias + 64;  // fl(x_scale * w_scale[n]): the one-multiply form of the int8 -> int8 fast path
    const int slab_cols = (BN - sub * 64) < 64 ? (BN - sub * 64) : 64;
    const int elem = p.out_dtype == ZEN_DT_S8 ? 1 : p.out_dtype == ZEN_DT_F16 ? 2 : 4;
    const bool vec_ok = (reinterpret_cast<uintptr_t>(p.out) % 16 == 0) && ((p.ldo * elem) % 16 == 0);
    const bool staged = p.staged_store != 0;
    uint8_t* stage = staged ? out_stage + size_t(sub * 4 + quad) * 4096 : nullptr;
    const float inv_scale = ZEN_DIV(1.0f, p.out_scale);
    int acc = 0;
    uint32_t acc_phase = 0;
    // Per-column scale and bias of the slab: lane l holds columns l and l + 32.  The values of the
    // next tile are fetched while the current tile's steps run, so that no tile starts on a global load.
    auto fetch_cols = [&](int tile, float (&sv)[2], float (&bv)[2]) {
      const int nn = (tile / p.tiles_m) * BN + sub * 64;
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int col = nn + lane + 32 * u;
        // predicated loads with no dependent instruction behind them: the warp issues in order and
        // would otherwise sit on the load until it returns
        sv[u] = 1.0f;
        bv[u] = 0.0f;
        if (p.w_scale != nullptr && col < p.N) sv[u] = __ldg(p.w_scale + col);
        if (p.bias != nullptr && col < p.N) bv[u] = __ldg(p.bias + col);
      }
    };
    float sv[2] = {1.0f, 1.0f}, bv[2] = {0.0f, 0.0f};
    if (first_tile < num_tiles) fetch_cols(first_tile, sv, bv);
    for (int tile = first_tile; tile < num_tiles; tile += tile_step) {
      const int m0 = (tile % p.tiles_m) * TILE_M + row_off;
      const int n0 = (tile / p.tiles_m) * BN + sub * 64;
      __syncwarp();
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        s_scale[lane + 32 * u] = sv[u];
        s_bias[lane + 32 * u] = bv[u];
        s_fold[lane + 32 * u] = ZEN_MUL(p.x_scale, sv[u]);
      }
      // Rounding-boundary test of the int8 -> int8 fast path (see requant_i8_step): the largest |bias| of the slab
      // (non-negative floats order like their bit patterns) bounds what the folded dequantisation can be off by.
      const float bmax = __int_as_float(__reduce_max_sync(0xffffffffu, max(__float_as_int(fabsf(bv[0])), __float_as_int(fabsf(bv[1])))));
      const float risk_thr = 0.5f - 2e-6f - inv_scale * fmaf(4.2e-7f, bmax, 1.6e-7f);
      if (tile + tile_step < num_tiles) fetch_cols(tile + tile_step, sv, bv);
      if (staged) {
        if (lane == 0) tma_store_wait_read();  // the previous tile's store has finished reading the block
      }
      __syncwarp();
      if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_flag)) break;
      tc_fence_after_sync();
      const int row = m0 + quad * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t tacc = tmem_base + (uint32_t(quad * 32) << 16) + uint32_t(acc * BN + sub * 64);
      // The loop is kept rolled: the step body (above all the GELU + requant one) is large, and
      // unrolling it made instruction fetch the bottleneck.  (Requesting the columns of step i + 1
      // before working on step i was tried twice and lost both times: 16 more live registers.)
#pragma unroll 1
      for (int i = 0; i < STEPS; ++i) {
        if (i * GEMM_CW >= slab_cols) break;
        uint32_t r[GEMM_CW];
        __syncwarp();
        tmem_ld_32x16(tacc + uint32_t(i * GEMM_CW), r);
        tmem_wait_ld();
        const int col0 = n0 + i * GEMM_CW;
        if constexpr (KIND == KIND_I8) {
          if (p.out_dtype == ZEN_DT_S8 && p.round_mode == 0) {
            const float* sc = s_scale + i * GEMM_CW;
            const float* bi = s_bias + i * GEMM_CW;
            const float* fo = s_fold + i * GEMM_CW;
            const uint32_t ta = tacc + uint32_t(i * GEMM_CW);
            if (p.act == ZEN_ACT_GELU)
              epilogue_step_s8<ZEN_ACT_GELU>(r, ta, sc, bi, fo, risk_thr, p, row, col0, row_ok, vec_ok, inv_scale, stage, lane, i);
            else if (p.act == ZEN_ACT_RELU)
              epilogue_step_s8<ZEN_ACT_RELU>(r, ta, sc, bi, fo, risk_thr, p, row, col0, row_ok, vec_ok, inv_scale, stage, lane, i);
            else
              epilogue_step_s8<ZEN_ACT_NONE>(r, ta, sc, bi, fo, risk_thr, p, row, col0, row_ok, vec_ok, inv_scale, stage, lane, i);
            continue;
          }
        }
        if (!staged && (!row_ok || col0 >= p.N)) continue;
        const bool full = vec_ok && (col0 + GEMM_CW <= p.N);
        const float* sc = s_scale + i * GEMM_CW;
        const float* bi = s_bias + i * GEMM_CW;
        if constexpr (KIND == KIND_I8) {
          switch (p.out_dtype) {
            case ZEN_DT_S32:
              epilogue_chunk<KIND, ZEN_DT_S32, ZEN_ACT_NONE>(r, sc, bi, p, row, col0, full, inv_scale, stage, lane, i);
              break;
            case ZEN_DT_F32: epilogue_chunk_act<KIND, ZEN_DT_F32>(r, sc, bi, p, row, col0, full, inv_scale, stage, lane, i); break;
            case ZEN_DT_F16: epilogue_chunk_act<KIND, ZEN_DT_F16>(r, sc, bi, p, row, col0, full, inv_scale, stage, lane, i); break;
            default: epilogue_chunk_act<KIND, ZEN_DT_S8>(r, sc, bi, p, row, col0, full, inv_scale, stage, lane, i); break;
          }
        } else {
          if (p.out_dtype == ZEN_DT_F32)
            epilogue_chunk_act<KIND, ZEN_DT_F32>(r, sc, bi, p, row, col0, full, inv_scale, stage, lane, i);
          else
            epilogue_chunk_act<KIND, ZEN_DT_F16>(r, sc, bi, p, row, col0, full, inv_scale, stage, lane, i);
        }
      }
      __syncwarp();
      tc_fence_before_sync();
      release_accumulator<PAIR>(tempty, acc, lane);  // the accumulator is free as soon as it has been read
      if (staged) {
        fence_proxy_async_smem();  // this lane's writes to the block -> visible to the TMA engine
        __syncwarp();
        if (lane == 0 && n0 < p.N && m0 + quad * 32 < p.M) {
          tma_store_2d(&tmap_c, stage, n0, m0 + quad * 32);
          tma_store_commit();
        }
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
    if (staged && lane == 0) tma_store_wait_all();
  } else {
    // no slab for this warp at this tile width: it still owes its arrivals on the accumulator barriers
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int tile = first_tile; tile < num_tiles; tile += tile_step) {
      if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_flag)) break;
      tc_fence_before_sync();
      release_accumulator<PAIR>(tempty, acc, lane);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }
}

template <int KIND, int BN, int STAGES, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const __grid_constant__ CUtensorMap tmap_c, const GemmParams p) {
  constexpr int ELEM = GemmKind<KIND>::ELEM;
  constexpr int BK = 128 / ELEM;  // elements per 128-byte swizzle row == K extent of one stage
  constexpr int UK = 32 / ELEM;   // K extent of one tcgen05.mma
  constexpr int A_BYTES = GEMM_BM * 128;
  constexpr int B_BYTES = BN * 128;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t TMEM_COLS = gemm_tmem_cols<BN>();
  constexpr uint32_t IDESC =
      KIND == KIND_I8 ? make_idesc(IDESC_C_S32, IDESC_S8, IDESC_S8, 0, B_MN ? 1 : 0, GEMM_BM, BN)
      : KIND == KIND_F16 ? make_idesc(IDESC_C_F32, IDESC_F16, IDESC_F16, 0, B_MN ? 1 : 0, GEMM_BM, BN)
      : KIND == KIND_F8  ? make_idesc(IDESC_C_F32, IDESC_E4M3, IDESC_E4M3, 0, B_MN ? 1 : 0, GEMM_BM, BN)
                         : make_idesc(IDESC_C_F32, IDESC_TF32, IDESC_TF32, 0, B_MN ? 1 : 0, GEMM_BM, BN);
  static_assert(BN % 32 == 0 && BN >= 32 && BN <= 256, "BN");
  static_assert(!B_MN || BN % BK == 0, "MN-major B is loaded in 128-byte wide boxes");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  constexpr int SLABS = (BN + 63) / 64;  // 64-column slabs of the tile, one per epilogue warp of a quadrant
  uint8_t* out_stage = smem + size_t(STAGES) * STAGE_BYTES;  // [SLABS][4 quadrants][4 KB], 1024-byte aligned
  uint8_t* ctrl = out_stage + size_t(SLABS) * 4 * 4096;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(ctrl);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* epi_rows = reinterpret_cast<float*>(ctrl + 256);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int nkb = p.num_k_blocks;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    if (p.staged_store) tma_prefetch_desc(&tmap_c);
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull_bar[i], 1);
      mbar_init(&tempty_bar[i], GEMM_EPI_WARPS * 32);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 1) {
    // constants of later kernels: safe to ask for before the previous kernel has finished
#pragma unroll
    for (int i = 0; i < 2; ++i)
      if (p.pf_bytes[i] != 0) prefetch_slice_l2(p.pf_ptr[i], p.pf_bytes[i], blockIdx.x, gridDim.x);
  }
  grid_launch_dependents();
  // Constant weights: the B tiles of the first tile's first k-blocks are requested now, while the previous
  // kernel may still be running (this CTA became resident when that kernel's CTA left the SM); only the A
  // tiles, which the previous kernel may be writing, wait.  `pre` lives in the producer thread.
  int pre = 0;
  if constexpr (!B_MN) {
    if (threadIdx.x == 0 && p.early_b && int(blockIdx.x) < num_tiles) {
      const int n0 = (int(blockIdx.x) / p.tiles_m) * BN;
      pre = nkb < STAGES ? nkb : STAGES;
      for (int kb = 0; kb < pre; ++kb) {
        mbar_arrive_expect_tx(&full_bar[kb], STAGE_BYTES);
        tma_load_2d(smem + size_t(kb) * STAGE_BYTES + A_BYTES, &tmap_b, &full_bar[kb], kb * BK, n0);
      }
    }
  }
  grid_dependency_wait();  // operands and output buffers may belong to the previous kernel until here

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile % p.tiles_m) * GEMM_BM;
        const int n0 = (tile / p.tiles_m) * BN;
        for (int kb = 0; kb < nkb; ++kb) {
          uint8_t* sa = smem + size_t(stage) * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          if (tile == int(blockIdx.x) && kb < pre) {
            // stage kb: fresh, its barrier already expects the bytes and its B tile is on the way
            tma_load_2d(sa, &tmap_a, &full_bar[stage], kb * BK, m0);
            if (++stage == STAGES) {
              stage = 0;
              phase ^= 1u;
            }
            continue;
          }
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&full_bar[stage], STAGE_BYTES);
          tma_load_2d(sa, &tmap_a, &full_bar[stage], kb * BK, m0);
          if constexpr (!B_MN) {
            tma_load_2d(sb, &tmap_b, &full_bar[stage], kb * BK, n0);
          } else {
#pragma unroll
            for (int c = 0; c < BN / BK; ++c)
              tma_load_2d(sb + c * (BK * 128), &tmap_b, &full_bar[stage], n0 + c * BK, kb * BK);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) {
        // give copies already in flight time to land before the CTA's shared memory is released
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1u, abort_flag)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + uint32_t(acc * BN);
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smem + size_t(stage) * STAGE_BYTES);
          const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UK; ++k) {
            const uint64_t a_desc = make_smem_desc_sw128(a_addr + k * 32, 1024, 16);
            const uint64_t b_desc = B_MN ? make_smem_desc_sw128(b_addr + k * (UK * 128), 1024, BK * 128)
                                         : make_smem_desc_sw128(b_addr + k * 32, 1024, 16);
            issue_mma<KIND>(d_tmem, a_desc, b_desc, IDESC, (kb | k) != 0 ? 1u : 0u);
          }
          tc_commit(&empty_bar[stage]);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) tc_commit(&tfull_bar[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const TmemEmptySignal tempty{tempty_bar, 0u};
    gemm_epilogue_role<KIND, BN, false>(p, tmap_c, tmem_base, out_stage, epi_rows, tfull_bar, tempty, abort_flag, warp, lane,
                                        int(blockIdx.x), int(gridDim.x), num_tiles, 0);
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

}  // namespace zen
