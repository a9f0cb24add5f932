// Host side of the tcgen05 GEMMs: tile selection, tensor maps, launches, C ABI.
#include "gemm_tc.cuh"
#include "gemm_pair.cuh"
#include "tma_host.cuh"
#include <map>
#include <mutex>

namespace zen {

// Smallest estimated time: waves of persistent CTAs x (tile width + fixed per-tile cost).  `flags` may carry a
// forced width (ZEN_GEMM_TILE_N); a width the kernel family does not have is ignored.
static int pick_bn(int M, int N, const int* allowed, int n_allowed, unsigned flags) {
  const int forced = int((flags >> 8) & 0x3ffu);
  if (forced) {
    for (int i = 0; i < n_allowed; ++i)
      if (allowed[i] == forced) return forced;
  }
  const int sms = num_sms();
  const int tiles_m = (M + GEMM_BM - 1) / GEMM_BM;
  long best_cost = -1;
  int best = allowed[0];
  for (int i = 0; i < n_allowed; ++i) {
    const int bn = allowed[i];
    const long tiles = long(tiles_m) * ((N + bn - 1) / bn);
    const long waves = (tiles + sms - 1) / sms;
    const long cost = waves * (bn + 24);
    if (best_cost < 0 || cost < best_cost) {
      best_cost = cost;
      best = bn;
    }
  }
  return best;
}

template <int KIND, int BN, int STAGES, bool B_MN>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, GemmParams p,
                       cudaStream_t stream) {
  auto kernel = gemm_tc_kernel<KIND, BN, STAGES, B_MN>;
  constexpr size_t smem = gemm_smem_bytes<BN, STAGES>();
  if (int st = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), smem); st != ZEN_OK) return st;
  p.tiles_m = (p.M + GEMM_BM - 1) / GEMM_BM;
  p.tiles_n = (p.N + BN - 1) / BN;
  const int tiles = p.tiles_m * p.tiles_n;
  const int grid = tiles < num_sms() ? tiles : num_sms();
  return launch_pdl(PDL_GEMM, kernel, dim3(grid), dim3(GEMM_THREADS), smem, stream, ta, tb, tc, p);
}

// Pairs of CTAs that can be resident at once for a pair kernel (SMs of a GPC come in odd numbers on some
// parts, so this may be below half the SM count); asked of the runtime once per (kernel, device).
static int max_resident_pairs(const void* kernel, size_t smem) {
  static std::mutex mu;
  static std::map<std::pair<const void*, int>, int> cache;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    return num_sms() / 2;
  }
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find({kernel, dev});
  if (it != cache.end()) return it->second;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(unsigned(num_sms() / 2 * 2));
  cfg.blockDim = dim3(GEMM_THREADS);
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n <= 0) {
    cudaGetLastError();
    n = num_sms() / 2;
  }
  cache[{kernel, dev}] = n;
  return n;
}

template <int KIND, int BN, int STAGES>
static int launch_gemm_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, GemmParams p,
                            cudaStream_t stream) {
  auto kernel = gemm_pair_kernel<KIND, BN, STAGES>;
  constexpr size_t smem = gemm_pair_smem_bytes<BN, STAGES>();
  if (int st = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), smem); st != ZEN_OK) return st;
  p.tiles_m = (p.M + 2 * GEMM_BM - 1) / (2 * GEMM_BM);  // 256-row blocks
  p.tiles_n = (p.N + BN - 1) / BN;
  const int tiles = p.tiles_m * p.tiles_n;
  const int resident = max_resident_pairs(reinterpret_cast<const void*>(kernel), smem);
  const int pairs = tiles < resident ? tiles : resident;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(unsigned(2 * pairs));
  cfg.blockDim = dim3(GEMM_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (pdl_mask() & PDL_GEMM) ? 2 : 1;
  if (cudaLaunchKernelEx(&cfg, kernel, ta, tb, tc, p) != cudaSuccess) {
    cudaGetLastError();
    return ZEN_ERR_LAUNCH;
  }
  return ZEN_OK;
}

template <int KIND>
static CUtensorMapDataType tmap_dtype() {
  return (KIND == KIND_I8 || KIND == KIND_F8) ? CU_TENSOR_MAP_DATA_TYPE_UINT8
         : KIND == KIND_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                            : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
}

// A [M,K] (row stride lda elements); B K-major [N,K] (ldb) or MN-major [K,N] (ldb).
// PAIR: the CTA-pair kernel (gemm_pair.cuh); each CTA then copies BN / 2 rows of B per k-block.
template <int KIND, int BN, int STAGES, bool B_MN, bool PAIR = false>
static int run_gemm(const void* A, int64_t lda, const void* B, int64_t ldb, GemmParams p, cudaStream_t stream) {
  static_assert(!(PAIR && B_MN), "the pair kernel takes K-major B only");
  constexpr int ELEM = GemmKind<KIND>::ELEM;
  constexpr int BK = 128 / ELEM;
  CUtensorMap ta, tb;
  int st = encode_tmap_2d(&ta, tmap_dtype<KIND>(), A, uint64_t(p.K), uint64_t(p.M), uint64_t(lda) * ELEM, BK, GEMM_BM);
  if (st != ZEN_OK) return st;
  if (!B_MN) st = encode_tmap_2d(&tb, tmap_dtype<KIND>(), B, uint64_t(p.K), uint64_t(p.N), uint64_t(ldb) * ELEM, BK, PAIR ? BN / 2 : BN);
  else st = encode_tmap_2d(&tb, tmap_dtype<KIND>(), B, uint64_t(p.N), uint64_t(p.K), uint64_t(ldb) * ELEM, BK, BK);
  if (st != ZEN_OK) return st;
  p.num_k_blocks = (p.K + BK - 1) / BK;
  // fp16 / int8 outputs with 16-byte aligned rows leave through shared memory and TMA stores of
  // 32-row x 64-column blocks; anything else is stored by the epilogue threads directly
  CUtensorMap tc = ta;
  p.staged_store = 0;
  const int oelem = p.out_dtype == ZEN_DT_S8 ? 1 : p.out_dtype == ZEN_DT_F16 ? 2 : 4;
  if ((p.out_dtype == ZEN_DT_F16 || p.out_dtype == ZEN_DT_S8) && reinterpret_cast<uintptr_t>(p.out) % 16 == 0 &&
      (p.ldo * oelem) % 16 == 0) {
    st = encode_tmap_2d(&tc, p.out_dtype == ZEN_DT_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8,
                        p.out, uint64_t(p.N), uint64_t(p.M), uint64_t(p.ldo) * oelem, 64, 32,
                        p.out_dtype == ZEN_DT_F16 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B);
    if (st != ZEN_OK) return st;
    p.staged_store = 1;
  }
  if constexpr (PAIR) return launch_gemm_pair<KIND, BN, STAGES>(ta, tb, tc, p, stream);
  else return launch_gemm<KIND, BN, STAGES, B_MN>(ta, tb, tc, p, stream);
}

// Whether a GEMM of this shape runs on CTA pairs.  ZEN_GEMM_PAIR / ZEN_GEMM_NO_PAIR force the choice.  A pair
// moves a third fewer operand bytes per operation but starts and ends more slowly (cluster scheduling, two
// cluster-wide rendezvous), and it does nothing for the epilogue: it pays when the main loop dominates, i.e. for
// large products, and for the GELU + requantisation epilogue only with a deep K (measured on 11 shapes: wins of
// 8 - 17 % above the thresholds, losses of 3 - 9 % below them).
static bool use_pair(int M, int N, int K, bool heavy_epilogue, unsigned flags) {
  if (flags & ZEN_GEMM_NO_PAIR) return false;
  if (flags & ZEN_GEMM_PAIR) return true;
  const double work = double(M) * double(N) * double(K);
  return M >= 1024 && work >= 34359738368.0 /* 2^35 */ && (!heavy_epilogue || K >= 4096);
}

// Pair tile width: fewest rounds of the resident pairs, wider tiles preferred on a tie (less traffic per operation).
static int pick_bn_pair(int M, int N, unsigned flags) {
  static const int allowed[] = {256, 192, 128};
  const int forced = int((flags >> 8) & 0x3ffu);
  for (int bn : allowed)
    if (bn == forced) return bn;
  const int pairs = num_sms() / 2;
  const int tiles_m = (M + 2 * GEMM_BM - 1) / (2 * GEMM_BM);
  long best_cost = -1;
  int best = allowed[0];
  for (int bn : allowed) {
    const long tiles = long(tiles_m) * ((N + bn - 1) / bn);
    const long rounds = (tiles + pairs - 1) / pairs;
    const long cost = rounds * (bn + 24);
    if (best_cost < 0 || cost < best_cost) {
      best_cost = cost;
      best = bn;
    }
  }
  return best;
}

// out[c, r] = in[r, c] for a row-major [rows, cols] fp32 matrix, 32 x 32 tiles through shared memory.
__global__ void __launch_bounds__(256) transpose_f32_kernel(const float* __restrict__ in, float* __restrict__ out,
                                                            int rows, int cols) {
  __shared__ float tile[32][33];
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int i = ty; i < 32; i += 8) {
    const int r = r0 + i, c = c0 + tx;
    if (r < rows && c < cols) tile[i][tx] = in[size_t(r) * cols + c];
  }
  __syncthreads();
  for (int i = ty; i < 32; i += 8) {
    const int c = c0 + i, r = r0 + tx;
    if (r < rows && c < cols) out[size_t(c) * rows + r] = tile[tx][i];
  }
}

static int launch_transpose_f32(const float* in, float* out, int rows, int cols, cudaStream_t s) {
  dim3 grid((cols + 31) / 32, (rows + 31) / 32);
  if (grid.y > 65535) return ZEN_ERR_UNSUPPORTED;
  transpose_f32_kernel<<<grid, 256, 0, s>>>(in, out, rows, cols);
  return cudaGetLastError() == cudaSuccess ? ZEN_OK : ZEN_ERR_LAUNCH;
}

}  // namespace zen

using namespace zen;

ZEN_DEFINE_TU_STATUS(gemm)

extern "C" {

int zen_version(void) { return ZEN_VERSION; }

const char* zen_status_string(int s) {
  switch (s) {
    case ZEN_OK: return "ok";
    case ZEN_ERR_INVALID_ARG: return "invalid argument";
    case ZEN_ERR_UNSUPPORTED: return "unsupported shape, stride or alignment";
    case ZEN_ERR_LAUNCH: return "kernel launch failed";
    case ZEN_ERR_TIMEOUT: return "a bounded device-side wait ran out";
    case ZEN_ERR_DRIVER: return "tensor-map encoding unavailable or failed";
    case ZEN_ERR_TOO_LARGE: return "request exceeds a fixed capacity";
    default: return "unknown status";
  }
}

static bool flags_ok(unsigned flags) {
  const unsigned bn = (flags >> 8) & 0x3ffu;
  if (flags & ~(ZEN_GEMM_CONST_WEIGHTS | ZEN_GEMM_PAIR | ZEN_GEMM_NO_PAIR | (0x3ffu << 8))) return false;
  if ((flags & ZEN_GEMM_PAIR) && (flags & ZEN_GEMM_NO_PAIR)) return false;
  return bn == 0 || bn == 64 || bn == 128 || bn == 192 || bn == 256;
}

int zen_linear_i8(const int8_t* xq, int64_t ldx, const int8_t* wq, int64_t ldw, int M, int N, int K, float x_scale,
                  const float* w_scale, const float* bias, int act, int out_dtype, float out_scale, int round_mode,
                  void* out, int64_t ldo, void* stream) {
  return zen_linear_i8_ex(xq, ldx, wq, ldw, M, N, K, x_scale, w_scale, bias, act, out_dtype, out_scale, round_mode, out,
                          ldo, nullptr, 0, nullptr, 0, 0u, stream);
}

int zen_linear_i8_prefetch(const int8_t* xq, int64_t ldx, const int8_t* wq, int64_t ldw, int M, int N, int K,
                           float x_scale, const float* w_scale, const float* bias, int act, int out_dtype,
                           float out_scale, int round_mode, void* out, int64_t ldo, const void* next0,
                           size_t next0_bytes, const void* next1, size_t next1_bytes, void* stream) {
  return zen_linear_i8_ex(xq, ldx, wq, ldw, M, N, K, x_scale, w_scale, bias, act, out_dtype, out_scale, round_mode, out,
                          ldo, next0, next0_bytes, next1, next1_bytes, 0u, stream);
}

int zen_linear_i8_ex(const int8_t* xq, int64_t ldx, const int8_t* wq, int64_t ldw, int M, int N, int K, float x_scale,
                     const float* w_scale, const float* bias, int act, int out_dtype, float out_scale, int round_mode,
                     void* out, int64_t ldo, const void* next0, size_t next0_bytes, const void* next1,
                     size_t next1_bytes, unsigned flags, void* stream) {
  if (!xq || !wq || !out || M <= 0 || N <= 0 || K <= 0 || !flags_ok(flags)) return ZEN_ERR_INVALID_ARG;
  if ((next0_bytes != 0 && !next0) || (next1_bytes != 0 && !next1)) return ZEN_ERR_INVALID_ARG;
  if (out_dtype < ZEN_DT_S32 || out_dtype > ZEN_DT_S8 || act < ZEN_ACT_NONE || act > ZEN_ACT_RELU)
    return ZEN_ERR_INVALID_ARG;
  if (round_mode != ZEN_ROUND_NEAREST_EVEN && round_mode != ZEN_ROUND_TRUNC) return ZEN_ERR_INVALID_ARG;
  if (out_dtype == ZEN_DT_S8 && !(out_scale > 0.0f)) return ZEN_ERR_INVALID_ARG;
  if (K % 16 || ldx % 16 || ldw % 16 || ldx < K || ldw < K || ldo < N) return ZEN_ERR_UNSUPPORTED;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.out = out; p.ldo = ldo; p.out_dtype = out_dtype; p.act = act; p.round_mode = round_mode;
  p.x_scale = x_scale; p.out_scale = out_scale; p.w_scale = w_scale; p.bias = bias;
  p.early_b = (flags & ZEN_GEMM_CONST_WEIGHTS) ? 1 : 0;
  const void* next[2] = {next0, next1};
  const size_t next_bytes[2] = {next0_bytes, next1_bytes};
  for (int i = 0; i < 2; ++i) {
    // whole 16-byte units only: a hint may skip the ragged ends
    const uintptr_t lo = (reinterpret_cast<uintptr_t>(next[i]) + 15u) & ~uintptr_t(15);
    const uintptr_t hi = (reinterpret_cast<uintptr_t>(next[i]) + next_bytes[i]) & ~uintptr_t(15);
    if (next_bytes[i] != 0 && hi > lo) {
      p.pf_ptr[i] = reinterpret_cast<const uint8_t*>(lo);
      p.pf_bytes[i] = uint64_t(hi - lo);
    }
  }
  static const int allowed[] = {64, 128, 192, 256};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (use_pair(M, N, K, out_dtype == ZEN_DT_S8 && act == ZEN_ACT_GELU, flags)) {
    switch (pick_bn_pair(M, N, flags)) {
      case 128: return run_gemm<KIND_I8, 128, 6, false, true>(xq, ldx, wq, ldw, p, s);
      case 192: return run_gemm<KIND_I8, 192, 5, false, true>(xq, ldx, wq, ldw, p, s);
      default: return run_gemm<KIND_I8, 256, 4, false, true>(xq, ldx, wq, ldw, p, s);
    }
  }
  switch (pick_bn(M, N, allowed, 4, flags)) {
    case 64: return run_gemm<KIND_I8, 64, 7, false>(xq, ldx, wq, ldw, p, s);
    case 128: return run_gemm<KIND_I8, 128, 5, false>(xq, ldx, wq, ldw, p, s);
    case 192: return run_gemm<KIND_I8, 192, 4, false>(xq, ldx, wq, ldw, p, s);
    default: return run_gemm<KIND_I8, 256, 3, false>(xq, ldx, wq, ldw, p, s);
  }
}

int zen_linear_f16(const void* x, int64_t ldx, const void* w, int64_t ldw, int M, int N, int K, const float* bias,
                   int act, int out_dtype, void* out, int64_t ldo, void* stream) {
  return zen_linear_f16_ex(x, ldx, w, ldw, M, N, K, bias, act, out_dtype, out, ldo, 0u, stream);
}

int zen_linear_f16_ex(const void* x, int64_t ldx, const void* w, int64_t ldw, int M, int N, int K, const float* bias,
                      int act, int out_dtype, void* out, int64_t ldo, unsigned flags, void* stream) {
  if (!x || !w || !out || M <= 0 || N <= 0 || K <= 0 || !flags_ok(flags)) return ZEN_ERR_INVALID_ARG;
  if ((out_dtype != ZEN_DT_F32 && out_dtype != ZEN_DT_F16) || act < ZEN_ACT_NONE || act > ZEN_ACT_RELU)
    return ZEN_ERR_INVALID_ARG;
  if (K % 8 || ldx % 8 || ldw % 8 || ldx < K || ldw < K || ldo < N) return ZEN_ERR_UNSUPPORTED;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.out = out; p.ldo = ldo; p.out_dtype = out_dtype; p.act = act;
  p.x_scale = 1.0f; p.out_scale = 1.0f; p.w_scale = nullptr; p.bias = bias;
  p.early_b = (flags & ZEN_GEMM_CONST_WEIGHTS) ? 1 : 0;
  static const int allowed[] = {64, 128, 192, 256};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (use_pair(M, N, 2 * K /* fp16 operands: twice the bytes per element */, false, flags)) {
    switch (pick_bn_pair(M, N, flags)) {
      case 128: return run_gemm<KIND_F16, 128, 6, false, true>(x, ldx, w, ldw, p, s);
      case 192: return run_gemm<KIND_F16, 192, 5, false, true>(x, ldx, w, ldw, p, s);
      default: return run_gemm<KIND_F16, 256, 4, false, true>(x, ldx, w, ldw, p, s);
    }
  }
  switch (pick_bn(M, N, allowed, 4, flags)) {
    case 64: return run_gemm<KIND_F16, 64, 7, false>(x, ldx, w, ldw, p, s);
    case 128: return run_gemm<KIND_F16, 128, 5, false>(x, ldx, w, ldw, p, s);
    case 192: return run_gemm<KIND_F16, 192, 4, false>(x, ldx, w, ldw, p, s);
    default: return run_gemm<KIND_F16, 256, 3, false>(x, ldx, w, ldw, p, s);
  }
}

int zen_linear_f8(const uint8_t* xq, int64_t ldx, const uint8_t* wq, int64_t ldw, int M, int N, int K, float x_scale,
                  const float* w_scale, const float* bias, int act, int out_dtype, void* out, int64_t ldo, unsigned flags,
                  void* stream) {
  if (!xq || !wq || !out || M <= 0 || N <= 0 || K <= 0) return ZEN_ERR_INVALID_ARG;
  if (!flags_ok(flags) || (flags & ZEN_GEMM_PAIR)) return ZEN_ERR_INVALID_ARG;
  if ((out_dtype != ZEN_DT_F32 && out_dtype != ZEN_DT_F16) || act < ZEN_ACT_NONE || act > ZEN_ACT_RELU)
    return ZEN_ERR_INVALID_ARG;
  if (K % 16 || ldx % 16 || ldw % 16 || ldx < K || ldw < K || ldo < N) return ZEN_ERR_UNSUPPORTED;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.out = out; p.ldo = ldo; p.out_dtype = out_dtype; p.act = act;
  p.x_scale = x_scale; p.out_scale = 1.0f; p.w_scale = w_scale; p.bias = bias;
  p.early_b = (flags & ZEN_GEMM_CONST_WEIGHTS) ? 1 : 0;
  static const int allowed[] = {64, 128, 192, 256};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (pick_bn(M, N, allowed, 4, flags)) {
    case 64: return run_gemm<KIND_F8, 64, 7, false>(xq, ldx, wq, ldw, p, s);
    case 128: return run_gemm<KIND_F8, 128, 5, false>(xq, ldx, wq, ldw, p, s);
    case 192: return run_gemm<KIND_F8, 192, 4, false>(xq, ldx, wq, ldw, p, s);
    default: return run_gemm<KIND_F8, 256, 3, false>(xq, ldx, wq, ldw, p, s);
  }
}

int zen_linear_f32(const float* x, int64_t ldx, const float* w, int64_t ldw, int M, int N, int K, const float* bias,
                   int act, float* out, int64_t ldo, void* stream) {
  if (!x || !w || !out || M <= 0 || N <= 0 || K <= 0) return ZEN_ERR_INVALID_ARG;
  if (act < ZEN_ACT_NONE || act > ZEN_ACT_RELU) return ZEN_ERR_INVALID_ARG;
  if (K % 4 || ldx % 4 || ldw % 4 || ldx < K || ldw < K || ldo < N) return ZEN_ERR_UNSUPPORTED;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.out = out; p.ldo = ldo; p.out_dtype = ZEN_DT_F32; p.act = act;
  p.x_scale = 1.0f; p.out_scale = 1.0f; p.w_scale = nullptr; p.bias = bias;
  static const int allowed[] = {64, 128, 256};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (pick_bn(M, N, allowed, 3, 0u)) {
    case 64: return run_gemm<KIND_TF32, 64, 7, false>(x, ldx, w, ldw, p, s);
    case 128: return run_gemm<KIND_TF32, 128, 5, false>(x, ldx, w, ldw, p, s);
    default: return run_gemm<KIND_TF32, 256, 3, false>(x, ldx, w, ldw, p, s);
  }
}

int zen_wmma_matmul_f16(const void* A, const void* B, float* C, int M, int N, int K, void* stream) {
  if (!A || !B || !C || M <= 0 || N <= 0 || K <= 0) return ZEN_ERR_INVALID_ARG;
  if (K % 8 || N % 8) return ZEN_ERR_UNSUPPORTED;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.out = C; p.ldo = N; p.out_dtype = ZEN_DT_F32; p.act = ZEN_ACT_NONE;
  p.x_scale = 1.0f; p.out_scale = 1.0f;
  static const int allowed[] = {64, 128, 256};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (pick_bn(M, N, allowed, 3, 0u)) {
    case 64: return run_gemm<KIND_F16, 64, 7, true>(A, K, B, N, p, s);
    case 128: return run_gemm<KIND_F16, 128, 5, true>(A, K, B, N, p, s);
    default: return run_gemm<KIND_F16, 256, 3, true>(A, K, B, N, p, s);
  }
}

size_t zen_matmul_f32_workspace_bytes(int N, int K) {
  if (N <= 0 || K <= 0) return 0;
  return size_t(N) * size_t(K) * sizeof(float);
}

int zen_matmul_f32(const float* A, const float* B, float* C, int M, int N, int K, void* workspace,
                   size_t workspace_bytes, void* stream) {
  if (!A || !B || !C || !workspace || M <= 0 || N <= 0 || K <= 0) return ZEN_ERR_INVALID_ARG;
  if (K % 4) return ZEN_ERR_UNSUPPORTED;
  if (workspace_bytes < zen_matmul_f32_workspace_bytes(N, K) || reinterpret_cast<uintptr_t>(workspace) % 16)
    return ZEN_ERR_INVALID_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  float* Bt = static_cast<float*>(workspace);
  int st = launch_transpose_f32(B, Bt, K, N, s);
  if (st != ZEN_OK) return st;
  return zen_linear_f32(A, K, Bt, K, M, N, K, nullptr, ZEN_ACT_NONE, C, N, stream);
}

// ------------------------------------------------------------------------------------------------
// zen_matmul_f32 without a caller workspace
// ------------------------------------------------------------------------------------------------
// Scratch for the transposed B operand, resident in every device that loads this library for as long
// as the process lives.  In host code the NAME below is only a stand-in for the symbol: it is not a
// device address and must never be handed to a kernel.  The address valid on a given device is
// obtained once per device with cudaGetSymbolAddress (scratch_for_current_device) and that pointer is
// what the kernels receive.
static __device__ __align__(256) float g_matmul_static_scratch[ZEN_MATMUL_STATIC_MAX_ELEMS];

static int scratch_for_current_device(float** out) {
  constexpr int kMaxDevices = 64;
  static std::mutex mu;
  static float* per_device[kMaxDevices] = {};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    cudaGetLastError();
    return ZEN_ERR_LAUNCH;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (per_device[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_matmul_static_scratch) != cudaSuccess || p == nullptr) {
      cudaGetLastError();
      return ZEN_ERR_LAUNCH;
    }
    per_device[dev] = static_cast<float*>(p);
  }
  *out = per_device[dev];
  return ZEN_OK;
}

int zen_matmul_f32_static(const float* A, const float* B, float* C, int M, int N, int K, void* stream) {
  if (!A || !B || !C || M <= 0 || N <= 0 || K <= 0) return ZEN_ERR_INVALID_ARG;
  if (K % 4) return ZEN_ERR_UNSUPPORTED;
  if (size_t(N) * size_t(K) > size_t(ZEN_MATMUL_STATIC_MAX_ELEMS)) return ZEN_ERR_TOO_LARGE;
  float* Bt = nullptr;
  int st = scratch_for_current_device(&Bt);
  if (st != ZEN_OK) return st;
  // every element of Bt that the GEMM reads is written by the transpose first: nothing needs clearing
  st = launch_transpose_f32(B, Bt, K, N, static_cast<cudaStream_t>(stream));
  if (st != ZEN_OK) return st;
  return zen_linear_f32(A, K, Bt, K, M, N, K, nullptr, ZEN_ACT_NONE, C, N, stream);
}

}  // extern "C"
