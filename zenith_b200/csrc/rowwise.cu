// HBM-bound kernels: LayerNorm, residual-add + LayerNorm (+ int8 copy), embedding + LayerNorm,
// GELU / ReLU / bias+GELU, quantize / dequantize, fp32 <-> fp16 converts.
//
// Row kernels: one warp owns one row, keeps it in registers as 16-byte vectors (a single read of
// every input), reduces with warp shuffles (two-pass variance in fp32) and writes 16-byte vectors.
// Elementwise kernels: 16-byte vectors, grid-stride, grid = SM count x 8.
#include "zen_common.cuh"
#include "det_math.h"
#include "tma_host.cuh"
#include <cuda_fp8.h>
#include <type_traits>

namespace zen {

// ------------------------------------------------------------------------------------------
// 16-byte vector access for half / float rows
// ------------------------------------------------------------------------------------------
template <typename T>
struct Vec16;
template <>
struct Vec16<__half> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const __half* p, float (&v)[8]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(h[i]);
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  }
  static __device__ __forceinline__ void store(__half* p, const float (&v)[8]) {
    uint4 u;
    __half2* h = reinterpret_cast<__half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = u;
  }
  // the value a later reader of the stored row will see
  static __device__ __forceinline__ float stored(float v) { return __half2float(__float2half_rn(v)); }
  // column pairs (for the packed fp32x2 arithmetic of the row kernels)
  static __device__ __forceinline__ void load2(const __half* p, float2 (&v)[4]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = __half22float2(h[i]);
  }
  // stores the row piece and returns, in `seen`, the values a later reader of it will see
  static __device__ __forceinline__ void store2(__half* p, const float2 (&v)[4], float2 (&seen)[4]) {
    uint4 u;
    __half2* h = reinterpret_cast<__half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      h[i] = __floats2half2_rn(v[i].x, v[i].y);
      seen[i] = __half22float2(h[i]);
    }
    *reinterpret_cast<uint4*>(p) = u;
  }
};
template <>
struct Vec16<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
    const float4 f = *reinterpret_cast<const float4*>(p);
    v[0] = f.x;
    v[1] = f.y;
    v[2] = f.z;
    v[3] = f.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
  static __device__ __forceinline__ float stored(float v) { return v; }
  static __device__ __forceinline__ void load2(const float* p, float2 (&v)[2]) {
    const float4 f = *reinterpret_cast<const float4*>(p);
    v[0] = make_float2(f.x, f.y);
    v[1] = make_float2(f.z, f.w);
  }
  static __device__ __forceinline__ void store2(float* p, const float2 (&v)[2], float2 (&seen)[2]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0].x, v[0].y, v[1].x, v[1].y);
    seen[0] = v[0];
    seen[1] = v[1];
  }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ int quantize_value(float x, float scale, int zero_point, int round_mode) {
  // core/src/cuda_kernels.cu:925-927: x / scale + zero_point, round, clamp
  return zen_det_round_clamp_i8(ZEN_ADD(ZEN_DIV(x, scale), float(zero_point)), round_mode);
}

template <int N>
__device__ __forceinline__ void store_q(int8_t* p, const float (&v)[N], float scale, float inv_scale, int round_mode) {
  int q[N];
  if (round_mode == 0) {
    const uint32_t risky = quantize_fast_rn<N>(v, inv_scale, q);
    if (risky) {
#pragma unroll
      for (int j = 0; j < N; ++j)
        if (risky & (1u << j)) q[j] = zen_det_round_clamp_i8(ZEN_DIV(v[j], scale), 0);
    }
  } else {
#pragma unroll
    for (int j = 0; j < N; ++j) q[j] = zen_det_round_clamp_i8(ZEN_DIV(v[j], scale), round_mode);
  }
  uint32_t w[N / 4];
#pragma unroll
  for (int i = 0; i < N / 4; ++i)
    w[i] = (uint32_t(q[4 * i]) & 0xffu) | ((uint32_t(q[4 * i + 1]) & 0xffu) << 8) |
           ((uint32_t(q[4 * i + 2]) & 0xffu) << 16) | ((uint32_t(q[4 * i + 3]) & 0xffu) << 24);
  if constexpr (N == 8) *reinterpret_cast<uint2*>(p) = make_uint2(w[0], w[1]);
  else *reinterpret_cast<uint32_t*>(p) = w[0];
}

// int8 copy of N values held as column pairs (nearest-even on the packed path, truncation by division)
template <int N>
__device__ __forceinline__ void store_q_pairs(int8_t* p, const float2 (&v)[N / 2], float scale, float inv_scale, int round_mode) {
  uint32_t w[N / 4];
  if (round_mode == 0) {
    const uint32_t risky = quantize_pairs_rn<N>(v, inv_scale, w);
    if (risky) {
#pragma unroll
      for (int j = 0; j < N; ++j)
        if (risky & (1u << j)) patch_q_byte(w, j, zen_det_round_clamp_i8(ZEN_DIV((j & 1) ? v[j >> 1].y : v[j >> 1].x, scale), 0));
    }
  } else {
#pragma unroll
    for (int i = 0; i < N / 4; ++i) {
      uint32_t acc = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = 4 * i + e;
        acc |= (uint32_t(zen_det_round_clamp_i8(ZEN_DIV((j & 1) ? v[j >> 1].y : v[j >> 1].x, scale), round_mode)) & 0xffu) << (8 * e);
      }
      w[i] = acc;
    }
  }
  if constexpr (N == 8) *reinterpret_cast<uint2*>(p) = make_uint2(w[0], w[1]);
  else *reinterpret_cast<uint32_t*>(p) = w[0];
}

// ------------------------------------------------------------------------------------------
// LayerNorm family.  SRC: 0 = x, 1 = x + residual, 2 = word[id] + pos[t % seq] + type[tid]
// ------------------------------------------------------------------------------------------
struct RowParams {
  const void* x;
  const void* residual;
  const void* gamma;
  const void* beta;
  void* y;
  int8_t* yq;
  float q_scale;
  int round_mode;
  int rows, hidden;
  float eps;
  // embedding source
  const int32_t* ids;
  const int32_t* type_ids;
  const int32_t* pos_ids;  // position of each row in its sequence; null: row % seq
  const void* pos;
  const void* type;
  int seq, vocab;
};

constexpr int ROW_WARPS = 4;

template <typename T, int VPL, int SRC>
__global__ void __launch_bounds__(ROW_WARPS * 32) ln_warp_kernel(const RowParams p) {
  constexpr int N = Vec16<T>::N;
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * ROW_WARPS + (threadIdx.x >> 5);
  grid_launch_dependents();
  grid_dependency_wait();  // inputs and outputs may belong to the previous kernel until here
  if (row >= p.rows) return;
  const int H = p.hidden;
  const T* x = static_cast<const T*>(p.x);
  const T* pos = nullptr;
  const T* typ = nullptr;
  if constexpr (SRC == 2) {
    int id = p.ids[row];
    id = id < 0 ? 0 : (id >= p.vocab ? p.vocab - 1 : id);
    x += int64_t(id) * H;
    pos = static_cast<const T*>(p.pos) + int64_t(p.pos_ids ? min(max(p.pos_ids[row], 0), p.seq - 1) : row % p.seq) * H;
    const int tid = p.type_ids ? p.type_ids[row] : 0;
    typ = static_cast<const T*>(p.type) + int64_t(tid != 0 ? 1 : 0) * H;
  } else {
    x += int64_t(row) * H;
  }
  const T* res = SRC == 1 ? static_cast<const T*>(p.residual) + int64_t(row) * H : nullptr;

  // The row lives in registers as column pairs; sums, deviations and the normalisation run on the
  // packed fp32x2 instructions (the kernel is bound by instruction issue, not by HBM).
  constexpr int P = N / 2;
  float2 v[VPL][P];
  float2 sum2 = make_float2(0.f, 0.f);
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int c = (i * 32 + lane) * N;
    if (c < H) {
      Vec16<T>::load2(x + c, v[i]);
      if constexpr (SRC == 1) {
        float2 r[P];
        Vec16<T>::load2(res + c, r);
#pragma unroll
        for (int j = 0; j < P; ++j) v[i][j] = f2add(v[i][j], r[j]);
      }
      if constexpr (SRC == 2) {
        float2 r[P];
        Vec16<T>::load2(pos + c, r);
#pragma unroll
        for (int j = 0; j < P; ++j) v[i][j] = f2add(v[i][j], r[j]);
        Vec16<T>::load2(typ + c, r);
#pragma unroll
        for (int j = 0; j < P; ++j) v[i][j] = f2add(v[i][j], r[j]);
      }
#pragma unroll
      for (int j = 0; j < P; ++j) sum2 = f2add(sum2, v[i][j]);
    } else {
#pragma unroll
      for (int j = 0; j < P; ++j) v[i][j] = make_float2(0.f, 0.f);
    }
  }
  const float mean = warp_sum(sum2.x + sum2.y) / float(H);
  const float2 nmean = make_float2(-mean, -mean);
  float2 sq2 = make_float2(0.f, 0.f);
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int c = (i * 32 + lane) * N;
    if (c < H) {
#pragma unroll
      for (int j = 0; j < P; ++j) {
        const float2 d = f2add(v[i][j], nmean);
        sq2 = f2fma(d, d, sq2);
      }
    }
  }
  const float rstd = rsqrtf(warp_sum(sq2.x + sq2.y) / float(H) + p.eps);
  const float2 rstd2 = make_float2(rstd, rstd);
  const float inv_q_scale = ZEN_DIV(1.0f, p.q_scale);
  const T* gamma = static_cast<const T*>(p.gamma);
  const T* beta = static_cast<const T*>(p.beta);
  T* y = static_cast<T*>(p.y) + int64_t(row) * H;
  int8_t* yq = p.yq ? p.yq + int64_t(row) * H : nullptr;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int c = (i * 32 + lane) * N;
    if (c < H) {
      float2 g[P], b[P], o[P], seen[P];
      Vec16<T>::load2(gamma + c, g);
      Vec16<T>::load2(beta + c, b);
#pragma unroll
      for (int j = 0; j < P; ++j) o[j] = f2fma(f2mul(f2add(v[i][j], nmean), rstd2), g[j], b[j]);
      Vec16<T>::store2(y + c, o, seen);
      if (yq) {
        // quantize the value that was stored, so that yq == quantize(y) exactly
        store_q_pairs<N>(yq + c, seen, p.q_scale, inv_q_scale, p.round_mode);
      }
    }
  }
}

// Fallback for rows that do not fit the register kernel (hidden not a multiple of the vector
// width, or wider than 32 lanes x 8 vectors): one CTA per row, three passes.
template <typename T, int SRC>
__global__ void __launch_bounds__(256) ln_block_kernel(const RowParams p) {
  __shared__ float red[8];
  __shared__ float bc;
  const int row = blockIdx.x;
  const int H = p.hidden;
  const T* x = static_cast<const T*>(p.x);
  const T* pos = nullptr;
  const T* typ = nullptr;
  if constexpr (SRC == 2) {
    int id = p.ids[row];
    id = id < 0 ? 0 : (id >= p.vocab ? p.vocab - 1 : id);
    x += int64_t(id) * H;
    pos = static_cast<const T*>(p.pos) + int64_t(p.pos_ids ? min(max(p.pos_ids[row], 0), p.seq - 1) : row % p.seq) * H;
    const int tid = p.type_ids ? p.type_ids[row] : 0;
    typ = static_cast<const T*>(p.type) + int64_t(tid != 0 ? 1 : 0) * H;
  } else {
    x += int64_t(row) * H;
  }
  const T* res = SRC == 1 ? static_cast<const T*>(p.residual) + int64_t(row) * H : nullptr;
  auto value = [&](int c) -> float {
    float a = float(x[c]);
    if constexpr (SRC == 1) a += float(res[c]);
    if constexpr (SRC == 2) a += float(pos[c]) + float(typ[c]);
    return a;
  };
  auto block_sum = [&](float s) -> float {
    s = warp_sum(s);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x < 32) {
      float t = threadIdx.x < 8 ? red[threadIdx.x] : 0.f;
      t = warp_sum(t);
      if (threadIdx.x == 0) bc = t;
    }
    __syncthreads();
    const float r = bc;
    __syncthreads();
    return r;
  };
  float s = 0.f;
  for (int c = threadIdx.x; c < H; c += 256) s += value(c);
  const float mean = block_sum(s) / float(H);
  float sq = 0.f;
  for (int c = threadIdx.x; c < H; c += 256) {
    const float d = value(c) - mean;
    sq += d * d;
  }
  const float rstd = rsqrtf(block_sum(sq) / float(H) + p.eps);
  const T* gamma = static_cast<const T*>(p.gamma);
  const T* beta = static_cast<const T*>(p.beta);
  T* y = static_cast<T*>(p.y) + int64_t(row) * H;
  for (int c = threadIdx.x; c < H; c += 256) {
    const float o = (value(c) - mean) * rstd * float(gamma[c]) + float(beta[c]);
    y[c] = T(o);
    if (p.yq) p.yq[int64_t(row) * H + c] = int8_t(quantize_value(float(y[c]), p.q_scale, 0, p.round_mode));
  }
}

template <typename T, int SRC>
static int launch_ln(const RowParams& p, cudaStream_t s) {
  constexpr int N = Vec16<T>::N;
  const int H = p.hidden;
  const bool aligned = (H % N == 0) && (reinterpret_cast<uintptr_t>(p.x) % 16 == 0) &&
                       (reinterpret_cast<uintptr_t>(p.y) % 16 == 0) &&
                       (reinterpret_cast<uintptr_t>(p.gamma) % 16 == 0) &&
                       (reinterpret_cast<uintptr_t>(p.beta) % 16 == 0) &&
                       (reinterpret_cast<uintptr_t>(p.residual) % 16 == 0) &&
                       (reinterpret_cast<uintptr_t>(p.pos) % 16 == 0) &&
                       (reinterpret_cast<uintptr_t>(p.type) % 16 == 0) &&
                       (reinterpret_cast<uintptr_t>(p.yq) % 8 == 0);
  const int vecs = (H + N * 32 - 1) / (N * 32);
  const int grid = (p.rows + ROW_WARPS - 1) / ROW_WARPS;
  if (aligned && vecs <= 8) {
    switch (vecs) {
      case 1: return launch_pdl(PDL_ROW, ln_warp_kernel<T, 1, SRC>, dim3(grid), dim3(ROW_WARPS * 32), 0, s, p);
      case 2: return launch_pdl(PDL_ROW, ln_warp_kernel<T, 2, SRC>, dim3(grid), dim3(ROW_WARPS * 32), 0, s, p);
      case 3: return launch_pdl(PDL_ROW, ln_warp_kernel<T, 3, SRC>, dim3(grid), dim3(ROW_WARPS * 32), 0, s, p);
      case 4: return launch_pdl(PDL_ROW, ln_warp_kernel<T, 4, SRC>, dim3(grid), dim3(ROW_WARPS * 32), 0, s, p);
      case 5:
      case 6: return launch_pdl(PDL_ROW, ln_warp_kernel<T, 6, SRC>, dim3(grid), dim3(ROW_WARPS * 32), 0, s, p);
      default: return launch_pdl(PDL_ROW, ln_warp_kernel<T, 8, SRC>, dim3(grid), dim3(ROW_WARPS * 32), 0, s, p);
    }
  } else {
    ln_block_kernel<T, SRC><<<p.rows, 256, 0, s>>>(p);
  }
  return cudaGetLastError() == cudaSuccess ? ZEN_OK : ZEN_ERR_LAUNCH;
}

// ------------------------------------------------------------------------------------------
// elementwise
// ------------------------------------------------------------------------------------------
enum { EW_GELU = 0, EW_RELU = 1, EW_BIAS_GELU = 2, EW_QUANT = 3, EW_DEQUANT = 4, EW_CONVERT = 5, EW_TANH = 6, EW_QUANT_F8 = 7 };

struct EwParams {
  const void* x;
  void* y;
  const float* bias;
  int64_t n;
  int features;
  float scale;
  int zero_point;
  int round_mode;
};

template <int OP, typename TI, typename TO>
__device__ __forceinline__ TO ew_apply(TI xin, const EwParams& p, int64_t idx) {
  if constexpr (OP == EW_DEQUANT) {
    return TO(ZEN_MUL(ZEN_SUB(float(xin), float(p.zero_point)), p.scale));
  } else {
    const float x = float(xin);
    if constexpr (OP == EW_GELU) return TO(zen_det_gelu(x));
    else if constexpr (OP == EW_RELU) return TO(x > 0.f ? x : 0.f);
    else if constexpr (OP == EW_TANH) return TO(zen_det_tanh(x));
    else if constexpr (OP == EW_BIAS_GELU) return TO(zen_det_gelu(ZEN_ADD(x, __ldg(p.bias + (idx % p.features)))));
    else if constexpr (OP == EW_QUANT) return TO(quantize_value(x, p.scale, p.zero_point, p.round_mode));
    // e4m3 bits of x / scale: round to nearest even, saturate to +-448 (NaN stays NaN)
    else if constexpr (OP == EW_QUANT_F8) return TO(__nv_cvt_float_to_fp8(ZEN_DIV(x, p.scale), __NV_SATFINITE, __NV_E4M3));
    else return TO(x);
  }
}

// Unsigned type of exactly BYTES bytes: the unit one thread moves per step.
template <int BYTES> struct EwWord;
template <> struct EwWord<1> { using type = uint8_t; };
template <> struct EwWord<2> { using type = uint16_t; };
template <> struct EwWord<4> { using type = uint32_t; };
template <> struct EwWord<8> { using type = uint2; };
template <> struct EwWord<16> { using type = uint4; };

// Each thread handles VEC consecutive elements per step (16 bytes of the wider side).  VEC == 1 is the
// form for pointers that are not 16-byte aligned: plain element accesses, which need only the natural
// alignment of the element type.
template <int OP, typename TI, typename TO, int VEC>
__global__ void __launch_bounds__(256) ew_kernel(const EwParams p) {
  const TI* x = static_cast<const TI*>(p.x);
  TO* y = static_cast<TO*>(p.y);
  const int64_t nvec = p.n / VEC;
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  if constexpr (VEC == 1) {
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < p.n; i += stride)
      y[i] = ew_apply<OP, TI, TO>(x[i], p, i);
  } else {
    using VI = typename EwWord<sizeof(TI) * VEC>::type;
    using VO = typename EwWord<sizeof(TO) * VEC>::type;
    static_assert(sizeof(VI) == sizeof(TI) * VEC && sizeof(VO) == sizeof(TO) * VEC, "vector width");
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += stride) {
      union { VI v; TI e[VEC]; } in;
      union { VO v; TO e[VEC]; } out;
      in.v = reinterpret_cast<const VI*>(x)[i];
#pragma unroll
      for (int j = 0; j < VEC; ++j) out.e[j] = ew_apply<OP, TI, TO>(in.e[j], p, i * VEC + j);
      reinterpret_cast<VO*>(y)[i] = out.v;
    }
    // tail
    const int64_t tail0 = nvec * VEC;
    for (int64_t i = tail0 + int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < p.n; i += stride)
      y[i] = ew_apply<OP, TI, TO>(x[i], p, i);
  }
}

template <int OP, typename TI, typename TO>
static int launch_ew(const EwParams& p, cudaStream_t s) {
  if (p.n <= 0) return ZEN_OK;
  constexpr int VEC = 16 / (sizeof(TI) > sizeof(TO) ? sizeof(TI) : sizeof(TO));
  const bool aligned = (reinterpret_cast<uintptr_t>(p.x) % 16 == 0) && (reinterpret_cast<uintptr_t>(p.y) % 16 == 0);
  int64_t work = aligned ? (p.n + VEC - 1) / VEC : p.n;
  int64_t blocks = (work + 255) / 256;
  const int64_t cap = int64_t(num_sms()) * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  if (aligned) ew_kernel<OP, TI, TO, VEC><<<int(blocks), 256, 0, s>>>(p);
  else ew_kernel<OP, TI, TO, 1><<<int(blocks), 256, 0, s>>>(p);
  return cudaGetLastError() == cudaSuccess ? ZEN_OK : ZEN_ERR_LAUNCH;
}


// ------------------------------------------------------------------------------------------
// Unpadded batches: the valid tokens of a padded [B, S] batch packed back to back
// ------------------------------------------------------------------------------------------
// Block b < B: the offset of sequence b (sum of the clamped lengths before it), then its ids / positions / types.
// Block B: the total, and defined values (id 0, position 0) for the rows between the total and the capacity.
__global__ void __launch_bounds__(128) pack_tokens_kernel(const int32_t* __restrict__ ids, const int32_t* __restrict__ type_ids,
                                                          const int32_t* __restrict__ kv_lens, int B, int S, int capacity,
                                                          int32_t* __restrict__ cu_seqlens, int32_t* __restrict__ ids_packed,
                                                          int32_t* __restrict__ pos_packed, int32_t* __restrict__ type_packed) {
  __shared__ int red[4];
  const int b = blockIdx.x;
  int part = 0;
  for (int i = threadIdx.x; i < b; i += blockDim.x) part += min(max(kv_lens[i], 0), S);
  part = __reduce_add_sync(0xffffffffu, part);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = part;
  __syncthreads();
  const int start = red[0] + red[1] + red[2] + red[3];
  if (b < B) {
    const int len = min(max(kv_lens[b], 0), S);
    if (threadIdx.x == 0) cu_seqlens[b] = start;
    for (int s = threadIdx.x; s < len; s += blockDim.x) {
      const int dst = start + s;
      if (dst < capacity) {
        ids_packed[dst] = ids[int64_t(b) * S + s];
        pos_packed[dst] = s;
        if (type_packed) type_packed[dst] = type_ids ? type_ids[int64_t(b) * S + s] : 0;
      }
    }
  } else {
    if (threadIdx.x == 0) cu_seqlens[B] = start;
    for (int t = start + int(threadIdx.x); t < capacity; t += blockDim.x) {
      ids_packed[t] = 0;
      pos_packed[t] = 0;
      if (type_packed) type_packed[t] = 0;
    }
  }
}

// One warp per padded row: its packed row, or zeros for a padding position.
template <typename T>
__global__ void __launch_bounds__(ROW_WARPS * 32) unpad_rows_kernel(const T* __restrict__ packed, const int32_t* __restrict__ cu_seqlens,
                                                                   int B, int S, int hidden, int capacity, T* __restrict__ padded) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * ROW_WARPS + (threadIdx.x >> 5);
  grid_launch_dependents();
  grid_dependency_wait();
  if (row >= B * S) return;
  const int b = row / S, s = row - b * S;
  const int start = cu_seqlens[b];
  const int len = cu_seqlens[b + 1] - start;
  const bool valid = s < len && start + s < capacity;
  constexpr int N = 16 / int(sizeof(T));
  const uint4* src = reinterpret_cast<const uint4*>(packed + int64_t(valid ? start + s : 0) * hidden);
  uint4* dst = reinterpret_cast<uint4*>(padded + int64_t(row) * hidden);
  for (int c = lane; c < hidden / N; c += 32) dst[c] = valid ? src[c] : make_uint4(0u, 0u, 0u, 0u);
}

}  // namespace zen

using namespace zen;

ZEN_DEFINE_TU_STATUS(rowwise)

extern "C" {

int zen_gelu_f32(const float* x, float* y, int64_t n, void* stream) {
  if (n < 0 || (n > 0 && (!x || !y))) return ZEN_ERR_INVALID_ARG;
  EwParams p{x, y, nullptr, n, 1, 1.f, 0, 0};
  return launch_ew<EW_GELU, float, float>(p, static_cast<cudaStream_t>(stream));
}
int zen_gelu_f16(const void* x, void* y, int64_t n, void* stream) {
  if (n < 0 || (n > 0 && (!x || !y))) return ZEN_ERR_INVALID_ARG;
  EwParams p{x, y, nullptr, n, 1, 1.f, 0, 0};
  return launch_ew<EW_GELU, __half, __half>(p, static_cast<cudaStream_t>(stream));
}
int zen_tanh_f32(const float* x, float* y, int64_t n, void* stream) {
  if (n < 0 || (n > 0 && (!x || !y))) return ZEN_ERR_INVALID_ARG;
  EwParams p{x, y, nullptr, n, 1, 1.f, 0, 0};
  return launch_ew<EW_TANH, float, float>(p, static_cast<cudaStream_t>(stream));
}
int zen_tanh_f16(const void* x, void* y, int64_t n, void* stream) {
  if (n < 0 || (n > 0 && (!x || !y))) return ZEN_ERR_INVALID_ARG;
  EwParams p{x, y, nullptr, n, 1, 1.f, 0, 0};
  return launch_ew<EW_TANH, __half, __half>(p, static_cast<cudaStream_t>(stream));
}
int zen_relu_f32(const float* x, float* y, int64_t n, void* stream) {
  if (n < 0 || (n > 0 && (!x || !y))) return ZEN_ERR_INVALID_ARG;
  EwParams p{x, y, nullptr, n, 1, 1.f, 0, 0};
  return launch_ew<EW_RELU, float, float>(p, static_cast<cudaStream_t>(stream));
}
int zen_bias_gelu_f32(const float* x, const float* bias, float* y, int rows, int features, void* stream) {
  if (rows < 0 || features <= 0 || !bias || (rows > 0 && (!x || !y))) return ZEN_ERR_INVALID_ARG;
  EwParams p{x, y, bias, int64_t(rows) * features, features, 1.f, 0, 0};
  return launch_ew<EW_BIAS_GELU, float, float>(p, static_cast<cudaStream_t>(stream));
}
int zen_quantize_f32(const float* x, int8_t* q, int64_t n, float scale, int zero_point, int round_mode, void* stream) {
  if (n < 0 || (n > 0 && (!x || !q)) || !(scale > 0.f) || (round_mode != 0 && round_mode != 1))
    return ZEN_ERR_INVALID_ARG;
  EwParams p{x, q, nullptr, n, 1, scale, zero_point, round_mode};
  return launch_ew<EW_QUANT, float, int8_t>(p, static_cast<cudaStream_t>(stream));
}
int zen_quantize_f16(const void* x, int8_t* q, int64_t n, float scale, int zero_point, int round_mode, void* stream) {
  if (n < 0 || (n > 0 && (!x || !q)) || !(scale > 0.f) || (round_mode != 0 && round_mode != 1))
    return ZEN_ERR_INVALID_ARG;
  EwParams p{x, q, nullptr, n, 1, scale, zero_point, round_mode};
  return launch_ew<EW_QUANT, __half, int8_t>(p, static_cast<cudaStream_t>(stream));
}
int zen_quantize_e4m3_f32(const float* x, uint8_t* q, int64_t n, float scale, void* stream) {
  if (n < 0 || (n > 0 && (!x || !q)) || !(scale > 0.f)) return ZEN_ERR_INVALID_ARG;
  EwParams p{x, q, nullptr, n, 1, scale, 0, 0};
  return launch_ew<EW_QUANT_F8, float, uint8_t>(p, static_cast<cudaStream_t>(stream));
}
int zen_quantize_e4m3_f16(const void* x, uint8_t* q, int64_t n, float scale, void* stream) {
  if (n < 0 || (n > 0 && (!x || !q)) || !(scale > 0.f)) return ZEN_ERR_INVALID_ARG;
  EwParams p{x, q, nullptr, n, 1, scale, 0, 0};
  return launch_ew<EW_QUANT_F8, __half, uint8_t>(p, static_cast<cudaStream_t>(stream));
}
int zen_dequantize_f32(const int8_t* q, float* x, int64_t n, float scale, int zero_point, void* stream) {
  if (n < 0 || (n > 0 && (!x || !q))) return ZEN_ERR_INVALID_ARG;
  EwParams p{q, x, nullptr, n, 1, scale, zero_point, 0};
  return launch_ew<EW_DEQUANT, int8_t, float>(p, static_cast<cudaStream_t>(stream));
}
int zen_convert_f32_to_f16(const float* x, void* y, int64_t n, void* stream) {
  if (n < 0 || (n > 0 && (!x || !y))) return ZEN_ERR_INVALID_ARG;
  EwParams p{x, y, nullptr, n, 1, 1.f, 0, 0};
  return launch_ew<EW_CONVERT, float, __half>(p, static_cast<cudaStream_t>(stream));
}
int zen_convert_f16_to_f32(const void* x, float* y, int64_t n, void* stream) {
  if (n < 0 || (n > 0 && (!x || !y))) return ZEN_ERR_INVALID_ARG;
  EwParams p{x, y, nullptr, n, 1, 1.f, 0, 0};
  return launch_ew<EW_CONVERT, __half, float>(p, static_cast<cudaStream_t>(stream));
}

static int check_ln(const void* x, const void* g, const void* b, const void* y, int rows, int hidden) {
  if (rows < 0 || hidden <= 0) return ZEN_ERR_INVALID_ARG;
  if (rows > 0 && (!x || !g || !b || !y)) return ZEN_ERR_INVALID_ARG;
  return ZEN_OK;
}

int zen_layernorm_f32(const float* x, const float* gamma, const float* beta, float* y, int rows, int hidden, float eps,
                      void* stream) {
  int st = check_ln(x, gamma, beta, y, rows, hidden);
  if (st != ZEN_OK || rows == 0) return st;
  RowParams p{};
  p.x = x; p.gamma = gamma; p.beta = beta; p.y = y; p.rows = rows; p.hidden = hidden; p.eps = eps;
  return launch_ln<float, 0>(p, static_cast<cudaStream_t>(stream));
}
int zen_layernorm_f16(const void* x, const void* gamma, const void* beta, void* y, int rows, int hidden, float eps,
                      void* stream) {
  int st = check_ln(x, gamma, beta, y, rows, hidden);
  if (st != ZEN_OK || rows == 0) return st;
  RowParams p{};
  p.x = x; p.gamma = gamma; p.beta = beta; p.y = y; p.rows = rows; p.hidden = hidden; p.eps = eps;
  return launch_ln<__half, 0>(p, static_cast<cudaStream_t>(stream));
}
int zen_add_layernorm_f32(const float* x, const float* residual, const float* gamma, const float* beta, float* y,
                          int rows, int hidden, float eps, void* stream) {
  int st = check_ln(x, gamma, beta, y, rows, hidden);
  if (st == ZEN_OK && rows > 0 && !residual) st = ZEN_ERR_INVALID_ARG;
  if (st != ZEN_OK || rows == 0) return st;
  RowParams p{};
  p.x = x; p.residual = residual; p.gamma = gamma; p.beta = beta; p.y = y; p.rows = rows; p.hidden = hidden;
  p.eps = eps;
  return launch_ln<float, 1>(p, static_cast<cudaStream_t>(stream));
}
int zen_add_layernorm_f16(const void* x, const void* residual, const void* gamma, const void* beta, void* y,
                          int8_t* yq, float out_scale, int round_mode, int rows, int hidden, float eps, void* stream) {
  int st = check_ln(x, gamma, beta, y, rows, hidden);
  if (st == ZEN_OK && rows > 0 && !residual) st = ZEN_ERR_INVALID_ARG;
  if (st == ZEN_OK && yq && (!(out_scale > 0.f) || (round_mode != 0 && round_mode != 1))) st = ZEN_ERR_INVALID_ARG;
  if (st != ZEN_OK || rows == 0) return st;
  RowParams p{};
  p.x = x; p.residual = residual; p.gamma = gamma; p.beta = beta; p.y = y; p.yq = yq; p.q_scale = out_scale;
  p.round_mode = round_mode; p.rows = rows; p.hidden = hidden; p.eps = eps;
  return launch_ln<__half, 1>(p, static_cast<cudaStream_t>(stream));
}
int zen_embed_layernorm_f16(const int32_t* ids, const int32_t* type_ids, const void* word, const void* pos,
                            const void* type, const void* gamma, const void* beta, void* y, int8_t* yq,
                            float out_scale, int round_mode, int tokens, int seq, int hidden, int vocab, float eps,
                            void* stream) {
  int st = check_ln(word, gamma, beta, y, tokens, hidden);
  if (st == ZEN_OK && (seq <= 0 || vocab <= 0)) st = ZEN_ERR_INVALID_ARG;
  if (st == ZEN_OK && tokens > 0 && (!ids || !pos || !type)) st = ZEN_ERR_INVALID_ARG;
  if (st == ZEN_OK && yq && (!(out_scale > 0.f) || (round_mode != 0 && round_mode != 1))) st = ZEN_ERR_INVALID_ARG;
  if (st != ZEN_OK || tokens == 0) return st;
  RowParams p{};
  p.x = word; p.pos = pos; p.type = type; p.ids = ids; p.type_ids = type_ids; p.gamma = gamma; p.beta = beta;
  p.y = y; p.yq = yq; p.q_scale = out_scale; p.round_mode = round_mode; p.rows = tokens; p.hidden = hidden;
  p.eps = eps; p.seq = seq; p.vocab = vocab;
  return launch_ln<__half, 2>(p, static_cast<cudaStream_t>(stream));
}

int zen_pack_tokens_i32(const int32_t* ids, const int32_t* type_ids, const int32_t* kv_lens, int B, int S, int capacity,
                        int32_t* cu_seqlens, int32_t* ids_packed, int32_t* pos_packed, int32_t* type_packed, void* stream) {
  if (B < 0 || S <= 0 || capacity < 0) return ZEN_ERR_INVALID_ARG;
  if (B == 0) return ZEN_OK;
  if (!ids || !kv_lens || !cu_seqlens || !ids_packed || !pos_packed) return ZEN_ERR_INVALID_ARG;
  if (int64_t(B) * S >= (int64_t(1) << 31) || B > 65535) return ZEN_ERR_UNSUPPORTED;
  pack_tokens_kernel<<<B + 1, 128, 0, static_cast<cudaStream_t>(stream)>>>(ids, type_ids, kv_lens, B, S, capacity, cu_seqlens,
                                                                            ids_packed, pos_packed, type_packed);
  return cudaGetLastError() == cudaSuccess ? ZEN_OK : ZEN_ERR_LAUNCH;
}

int zen_unpad_rows_f16(const void* packed, const int32_t* cu_seqlens, int B, int S, int hidden, int capacity, void* padded,
                       void* stream) {
  if (B < 0 || S <= 0 || hidden <= 0 || capacity < 0) return ZEN_ERR_INVALID_ARG;
  if (B == 0) return ZEN_OK;
  if (!packed || !cu_seqlens || !padded) return ZEN_ERR_INVALID_ARG;
  if (hidden % 8 || reinterpret_cast<uintptr_t>(packed) % 16 || reinterpret_cast<uintptr_t>(padded) % 16) return ZEN_ERR_UNSUPPORTED;
  const int64_t rows = int64_t(B) * S;
  if (rows > (int64_t(1) << 30)) return ZEN_ERR_UNSUPPORTED;
  const int grid = int((rows + ROW_WARPS - 1) / ROW_WARPS);
  return launch_pdl(PDL_ROW, unpad_rows_kernel<__half>, dim3(grid), dim3(ROW_WARPS * 32), 0, static_cast<cudaStream_t>(stream),
                    static_cast<const __half*>(packed), cu_seqlens, B, S, hidden, capacity, static_cast<__half*>(padded));
}

int zen_embed_layernorm_unpadded_f16(const int32_t* ids_packed, const int32_t* pos_packed, const int32_t* type_packed,
                                     const void* word, const void* pos, const void* type, const void* gamma,
                                     const void* beta, void* y, int8_t* yq, float out_scale, int round_mode, int rows,
                                     int max_pos, int hidden, int vocab, float eps, void* stream) {
  int st = check_ln(word, gamma, beta, y, rows, hidden);
  if (st == ZEN_OK && (max_pos <= 0 || vocab <= 0)) st = ZEN_ERR_INVALID_ARG;
  if (st == ZEN_OK && rows > 0 && (!ids_packed || !pos_packed || !pos || !type)) st = ZEN_ERR_INVALID_ARG;
  if (st == ZEN_OK && yq && (!(out_scale > 0.f) || (round_mode != 0 && round_mode != 1))) st = ZEN_ERR_INVALID_ARG;
  if (st != ZEN_OK || rows == 0) return st;
  RowParams p{};
  p.x = word; p.pos = pos; p.type = type; p.ids = ids_packed; p.pos_ids = pos_packed; p.type_ids = type_packed;
  p.gamma = gamma; p.beta = beta; p.y = y; p.yq = yq; p.q_scale = out_scale; p.round_mode = round_mode; p.rows = rows;
  p.hidden = hidden; p.eps = eps; p.seq = max_pos; p.vocab = vocab;
  return launch_ln<__half, 2>(p, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
