// Calibration reductions on the device: running min / max of an activation tensor (per-tensor observer),
// per-row absmax of a weight matrix (per-output-channel observer) and per-row int8 conversion.
//
// They replace the reference's observer kernels (core/src/qat_cuda.cu:146-227: block reductions merged with
// atomicMin / atomicMax on the raw float bits, which orders negative values the wrong way round) and its
// per-channel fake-quant kernel (core/src/qat_cuda.cu:90-114), and keep a calibration pass on the device:
// no host read-back per tensor.  All three are bandwidth-bound, deterministic (no atomics) and exact:
// min / max / absmax select among the inputs, the int8 conversion divides and rounds with IEEE operations
// (det_math.h), so the scales and weights derived from them are bit-identical to what the numpy front-end
// (zenith/optimization/quantization.py:69-72, zenith/optimization/qat.py:195-228) computes from the same data.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "det_math.h"
#include "tma_host.cuh"
#include "zenith_b200.h"

namespace zen {

constexpr int MM_THREADS = 256;
constexpr int MM_MAX_CTAS = 1024;  // partial (min, max) pairs in the workspace

__device__ __forceinline__ float lanes_min(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float lanes_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// CTA-wide (min, max); valid in thread 0.  fminf / fmaxf drop NaN operands, as np.nanmin would; a tensor
// of NaNs only leaves the running values untouched.
__device__ __forceinline__ void cta_minmax(float& mn, float& mx) {
  __shared__ float s_mn[MM_THREADS / 32], s_mx[MM_THREADS / 32];
  mn = lanes_min(mn);
  mx = lanes_max(mx);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    s_mn[warp] = mn;
    s_mx[warp] = mx;
  }
  __syncthreads();
  if (warp == 0) {
    mn = lane < MM_THREADS / 32 ? s_mn[lane] : INFINITY;
    mx = lane < MM_THREADS / 32 ? s_mx[lane] : -INFINITY;
    mn = lanes_min(mn);
    mx = lanes_max(mx);
  }
}

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }

// phase 1: every CTA reduces a grid-strided share of x (16-byte vectors when x is 16-byte aligned)
template <typename T>
__global__ void __launch_bounds__(MM_THREADS) minmax_partial_kernel(const T* __restrict__ x, int64_t n, float2* __restrict__ partial) {
  constexpr int VEC = 16 / sizeof(T);
  float mn = INFINITY, mx = -INFINITY;
  const int64_t tid = int64_t(blockIdx.x) * MM_THREADS + threadIdx.x;
  const int64_t nthreads = int64_t(gridDim.x) * MM_THREADS;
  int64_t done = 0;
  if (reinterpret_cast<uintptr_t>(x) % 16 == 0) {
    const int64_t nvec = n / VEC;
    const uint4* xv = reinterpret_cast<const uint4*>(x);
    for (int64_t i = tid; i < nvec; i += nthreads) {
      const uint4 raw = __ldg(xv + i);
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        const float v = to_f32<T>(e[j]);
        mn = fminf(mn, v);
        mx = fmaxf(mx, v);
      }
    }
    done = nvec * VEC;
  }
  for (int64_t i = done + tid; i < n; i += nthreads) {
    const float v = to_f32<T>(x[i]);
    mn = fminf(mn, v);
    mx = fmaxf(mx, v);
  }
  cta_minmax(mn, mx);
  if (threadIdx.x == 0) partial[blockIdx.x] = make_float2(mn, mx);
}

// phase 2: one CTA folds the partials into the running pair
__global__ void __launch_bounds__(MM_THREADS) minmax_merge_kernel(const float2* __restrict__ partial, int count, float* __restrict__ minmax) {
  float mn = INFINITY, mx = -INFINITY;
  for (int i = threadIdx.x; i < count; i += MM_THREADS) {
    const float2 v = partial[i];
    mn = fminf(mn, v.x);
    mx = fmaxf(mx, v.y);
  }
  cta_minmax(mn, mx);
  if (threadIdx.x == 0) {
    minmax[0] = fminf(minmax[0], mn);
    minmax[1] = fmaxf(minmax[1], mx);
  }
}

template <typename T>
static int run_minmax(const T* x, int64_t n, float* minmax, void* workspace, size_t workspace_bytes, cudaStream_t s) {
  if (n < 0 || !minmax) return ZEN_ERR_INVALID_ARG;
  if (n == 0) return ZEN_OK;
  if (!x || !workspace) return ZEN_ERR_INVALID_ARG;
  if (workspace_bytes < size_t(MM_MAX_CTAS) * sizeof(float2) || reinterpret_cast<uintptr_t>(workspace) % 8) return ZEN_ERR_INVALID_ARG;
  constexpr int VEC = 16 / sizeof(T);
  int64_t want = (n / VEC + MM_THREADS * 4 - 1) / (MM_THREADS * 4);  // about four vectors per thread
  const int cap = min(MM_MAX_CTAS, num_sms() * 4);
  const int ctas = int(want < 1 ? 1 : (want > cap ? cap : want));
  float2* partial = static_cast<float2*>(workspace);
  minmax_partial_kernel<T><<<ctas, MM_THREADS, 0, s>>>(x, n, partial);
  minmax_merge_kernel<<<1, MM_THREADS, 0, s>>>(partial, ctas, minmax);
  return cudaGetLastError() == cudaSuccess ? ZEN_OK : ZEN_ERR_LAUNCH;
}

// one warp per row: absmax over the row's columns
__global__ void __launch_bounds__(256) absmax_rows_kernel(const float* __restrict__ w, int rows, int cols, int64_t ld, float* __restrict__ out) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const float* wr = w + int64_t(row) * ld;
  float m = 0.0f;
  int done = 0;
  if (reinterpret_cast<uintptr_t>(wr) % 16 == 0) {
    const int nvec = cols / 4;
    const float4* wv = reinterpret_cast<const float4*>(wr);
    for (int i = lane; i < nvec; i += 32) {
      const float4 v = __ldg(wv + i);
      m = fmaxf(m, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
    }
    done = nvec * 4;
  }
  for (int i = done + lane; i < cols; i += 32) m = fmaxf(m, fabsf(wr[i]));
  m = lanes_max(m);
  if (lane == 0) out[row] = m;
}

// q[r, c] = clamp(rint(w[r, c] / scale[r]), -128, 127)
__global__ void __launch_bounds__(256) quantize_rows_kernel(const float* __restrict__ w, const float* __restrict__ scale, int rows, int cols, int64_t ldw,
                                                            int8_t* __restrict__ q, int64_t ldq, int round_mode) {
  const int row = blockIdx.y;
  const float s = scale[row];
  const float* wr = w + int64_t(row) * ldw;
  int8_t* qr = q + int64_t(row) * ldq;
  for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < cols; c += gridDim.x * blockDim.x)
    qr[c] = int8_t(zen_det_round_clamp_i8(ZEN_DIV(wr[c], s), round_mode));
}

// ------------------------------------------------------------------------------------------------
// histogram of an activation tensor over the running range, as TensorStats.update keeps it
// (zenith/optimization/quantization.py:69-83: np.histogram(tensor, bins, range=(min, max)) added to the running
// histogram, the range being the running one AFTER this tensor's min / max went into it).
// Bin of a value, as numpy's uniform-bin path computes it for a float32 array:
//   edges[i] = float32(i * step + lo)  with step = (hi - lo) / bins in float64 (np.linspace), edges[bins] = hi
//   i = trunc(((x - lo) / float32(hi - lo)) * bins)   in float32;  i == bins -> bins - 1
//   x <  edges[i]                        -> i - 1
//   x >= edges[i + 1] and i != bins - 1  -> i + 1
// Values outside [lo, hi] (and NaNs) are not counted.  lo >= hi: the range (0, 1), as the reference does.
// Counts are integers: the result does not depend on the order of the atomic additions.
// ------------------------------------------------------------------------------------------------
constexpr int HIST_THREADS = 256;
constexpr int HIST_MAX_BINS = 4096;

template <typename T>
__global__ void __launch_bounds__(HIST_THREADS) histogram_kernel(const T* __restrict__ x, int64_t n, const float* __restrict__ minmax,
                                                                  int bins, unsigned long long* __restrict__ hist) {
  extern __shared__ unsigned char hist_smem[];
  float* edges = reinterpret_cast<float*>(hist_smem);                    // [bins + 1]
  unsigned int* local = reinterpret_cast<unsigned int*>(edges + bins + 1);  // [bins]
  float lo = minmax[0], hi = minmax[1];
  if (!(lo < hi)) {
    lo = 0.0f;
    hi = 1.0f;
  }
  const double step = __ddiv_rn(__dsub_rn(double(hi), double(lo)), double(bins));
  for (int i = threadIdx.x; i <= bins; i += HIST_THREADS) {
    edges[i] = i == bins ? hi : float(__dadd_rn(__dmul_rn(double(i), step), double(lo)));
    if (i < bins) local[i] = 0u;
  }
  __syncthreads();
  const float denom = float(__dsub_rn(double(hi), double(lo)));
  const float fbins = float(bins);
  const int64_t nthreads = int64_t(gridDim.x) * HIST_THREADS;
  for (int64_t k = int64_t(blockIdx.x) * HIST_THREADS + threadIdx.x; k < n; k += nthreads) {
    const float v = to_f32<T>(x[k]);
    if (!(v >= lo && v <= hi)) continue;
    int i = int(ZEN_MUL(ZEN_DIV(ZEN_SUB(v, lo), denom), fbins));
    if (i == bins) i = bins - 1;
    if (i < 0 || i >= bins) continue;  // cannot happen for v in [lo, hi]; guards the table accesses below
    if (v < edges[i]) {
      if (i == 0) continue;
      i -= 1;
    }
    if (i != bins - 1 && v >= edges[i + 1]) i += 1;
    atomicAdd(&local[i], 1u);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < bins; i += HIST_THREADS)
    if (local[i] != 0u) atomicAdd(&hist[i], static_cast<unsigned long long>(local[i]));
}

template <typename T>
static int run_histogram(const T* x, int64_t n, const float* minmax, int bins, long long* hist, cudaStream_t s) {
  if (n < 0 || bins <= 0 || bins > HIST_MAX_BINS || !minmax || !hist) return ZEN_ERR_INVALID_ARG;
  if (n == 0) return ZEN_OK;
  if (!x) return ZEN_ERR_INVALID_ARG;
  int64_t want = (n + HIST_THREADS * 16 - 1) / (HIST_THREADS * 16);
  const int cap = num_sms() * 4;
  const int ctas = int(want < 1 ? 1 : (want > cap ? cap : want));
  const size_t smem = size_t(2 * bins + 1) * 4;
  histogram_kernel<T><<<ctas, HIST_THREADS, smem, s>>>(x, n, minmax, bins, reinterpret_cast<unsigned long long*>(hist));
  return cudaGetLastError() == cudaSuccess ? ZEN_OK : ZEN_ERR_LAUNCH;
}

}  // namespace zen

using namespace zen;

extern "C" int zen_histogram_f32(const float* x, int64_t n, const float* minmax, int bins, long long* hist, void* stream) {
  return run_histogram<float>(x, n, minmax, bins, hist, static_cast<cudaStream_t>(stream));
}

extern "C" int zen_histogram_f16(const void* x, int64_t n, const float* minmax, int bins, long long* hist, void* stream) {
  return run_histogram<__half>(static_cast<const __half*>(x), n, minmax, bins, hist, static_cast<cudaStream_t>(stream));
}

extern "C" size_t zen_minmax_workspace_bytes(void) { return size_t(MM_MAX_CTAS) * sizeof(float2); }

extern "C" int zen_minmax_f32(const float* x, int64_t n, float* minmax, void* workspace, size_t workspace_bytes, void* stream) {
  return run_minmax<float>(x, n, minmax, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

extern "C" int zen_minmax_f16(const void* x, int64_t n, float* minmax, void* workspace, size_t workspace_bytes, void* stream) {
  return run_minmax<__half>(static_cast<const __half*>(x), n, minmax, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

extern "C" int zen_absmax_rows_f32(const float* w, int rows, int cols, int64_t ld, float* out, void* stream) {
  if (rows < 0 || cols < 0 || ld < cols) return ZEN_ERR_INVALID_ARG;
  if (rows == 0) return ZEN_OK;
  if (!w || !out) return ZEN_ERR_INVALID_ARG;
  absmax_rows_kernel<<<(rows + 7) / 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(w, rows, cols, ld, out);
  return cudaGetLastError() == cudaSuccess ? ZEN_OK : ZEN_ERR_LAUNCH;
}

extern "C" int zen_quantize_rows_f32(const float* w, const float* scale, int rows, int cols, int64_t ldw, int8_t* q, int64_t ldq,
                                     int round_mode, void* stream) {
  if (rows < 0 || cols < 0 || ldw < cols || ldq < cols) return ZEN_ERR_INVALID_ARG;
  if (round_mode != ZEN_ROUND_NEAREST_EVEN && round_mode != ZEN_ROUND_TRUNC) return ZEN_ERR_INVALID_ARG;
  if (rows == 0 || cols == 0) return ZEN_OK;
  if (!w || !scale || !q) return ZEN_ERR_INVALID_ARG;
  if (rows > 65535) return ZEN_ERR_UNSUPPORTED;
  dim3 grid(min((cols + 255) / 256, 64), rows);
  quantize_rows_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(w, scale, rows, cols, ldw, q, ldq, round_mode);
  return cudaGetLastError() == cudaSuccess ? ZEN_OK : ZEN_ERR_LAUNCH;
}
