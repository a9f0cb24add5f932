// W8A8 Linear + residual add + LayerNorm (+ int8 copy) in ONE kernel:
//     y   = (float(acc) * s_x) * s_w[n] + b[n] + residual[m, n]        acc = xq . wq^T  (int32, tcgen05 kind::i8)
//     out = (y - mean_m) * rstd_m * gamma[n] + beta[n]   -> fp16, and clamp(round(out / out_scale)) -> int8
// for the two projections of an encoder layer whose output width is the hidden size (attention
// output and FFN2).  The row statistics need all N columns of a row; a CTA holds only BN = N / 4 of
// them in TMEM, so four CTAs form a thread-block cluster along N.  Each of the 16 epilogue warps of a
// CTA owns 32 rows x BN / 4 columns and keeps its values in REGISTERS from the accumulator load to the
// stores: one pass over tensor memory, (mean, M2) of the thread's columns, published to all four CTAs
// through distributed shared memory (remote st.shared::cluster + one remote mbarrier arrival per warp),
// then the 16 partials of the row are merged (equal counts: mean of the means, M2 = sum of M2 + n *
// sum of squared mean deviations, as robust as the two-pass form of the stand-alone kernel), the row
// is normalised in registers and written to global memory directly.  No cluster-wide barrier inside
// the tile loop, so the TMA / MMA warps keep running the next tile underneath, and the accumulator is
// released as soon as it has been read.  (An earlier form made two passes over tensor memory with a
// CTA-level reduction between them and staged the output for TMA stores: 5.3 us on top of the plain
// GEMM for one tile per CTA.)
//
// Main loop, warp roles and TMEM double buffering are those of gemm_tc.cuh.
#include "gemm_tc.cuh"
#include "tma_host.cuh"

namespace zen {

struct GemmLnParams {
  int M, N, K;
  int tiles_m, num_k_blocks;
  float x_scale, out_scale, eps;
  int round_mode;
  const float* w_scale;
  const float* bias;
  const __half* residual;  // [M, N], row stride ldr
  int64_t ldr;
  const __half* gamma;
  const __half* beta;
  __half* y;   // [M, N] fp16 output (row stride N)
  int8_t* yq;  // its int8 copy, or null
  int emit_q;  // write the int8 copy
  int early_b;  // 1: the weights are constant: their first tiles may be requested before the dependency wait
};

constexpr int LN_CLUSTER = 4;

__device__ __forceinline__ void st_cluster_f32x2(uint32_t cluster_addr, float a, float b) {
  asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};" ::"r"(cluster_addr), "f"(a), "f"(b) : "memory");
}

// (n_a, mean_a, m2_a) <- merge with (n_b, mean_b, m2_b)
__device__ __forceinline__ void chan_merge(float& n_a, float& mean_a, float& m2_a, float n_b, float mean_b, float m2_b) {
  const float n = n_a + n_b;
  const float delta = mean_b - mean_a;
  const float f = n_b / n;
  mean_a = fmaf(delta, f, mean_a);
  m2_a = m2_a + m2_b + delta * delta * n_a * f;
  n_a = n;
}

constexpr int LN_PARTS = LN_CLUSTER * 4;  // partial statistics per row: 4 CTAs x 4 column groups

template <int BN, int STAGES>
constexpr size_t gemm_ln_smem_bytes() {
  // ring + cluster statistics (2 tiles in flight x 16 partials x 128 rows, float2) + control (256 B) + per-warp
  // rows (scale, bias, gamma, beta x 64 floats for 16 warps) + alignment slack
  return size_t(STAGES) * (GEMM_BM * 128 + BN * 128) + 2 * size_t(LN_PARTS) * 128 * 8 + 256 +
         size_t(GEMM_EPI_WARPS) * 4 * 64 * 4 + 1024;
}

// KIND_I8: int8 operands, s32 accumulators, dequantised with x_scale * w_scale[n]; KIND_F16: fp16 operands, fp32
// accumulators (the scale row holds ones).  Everything after the accumulator is shared.
template <int KIND, int BN, int STAGES>
__device__ __forceinline__ void gemm_ln_body(const CUtensorMap& tmap_a, const CUtensorMap& tmap_b, const GemmLnParams& p) {
  constexpr int ELEM = GemmKind<KIND>::ELEM;
  constexpr int BK = 128 / ELEM, UK = 32 / ELEM;
  constexpr int A_BYTES = GEMM_BM * 128;
  constexpr int B_BYTES = BN * 128;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int COLS = BN / 4;  // columns of a row held by one epilogue thread (48 or 64)
  constexpr uint32_t TMEM_COLS = gemm_tmem_cols<BN>();
  constexpr uint32_t IDESC = KIND == KIND_I8 ? make_idesc(IDESC_C_S32, IDESC_S8, IDESC_S8, 0, 0, GEMM_BM, BN)
                                             : make_idesc(IDESC_C_F32, IDESC_F16, IDESC_F16, 0, 0, GEMM_BM, BN);
  constexpr int STEPS = COLS / GEMM_CW;
  static_assert(BN % 64 == 0 && BN <= 256 && COLS % GEMM_CW == 0, "BN");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  float2* xstats = reinterpret_cast<float2*>(smem + size_t(STAGES) * STAGE_BYTES);  // [2][4 ranks x 4 column groups][128]
  uint8_t* ctrl = reinterpret_cast<uint8_t*>(xstats + 2 * LN_PARTS * 128);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(ctrl);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint64_t* stats_bar = tempty_bar + 2;  // [2] cluster-wide: the 16 partials of every row have arrived
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(stats_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* epi_rows = reinterpret_cast<float*>(ctrl + 256);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int cluster_id = blockIdx.x / LN_CLUSTER;
  const int num_clusters = gridDim.x / LN_CLUSTER;
  const int nkb = p.num_k_blocks;
  const int n_base = int(rank) * BN;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull_bar[i], 1);
      mbar_init(&tempty_bar[i], GEMM_EPI_WARPS * 32);
      mbar_init(&stats_bar[i], LN_CLUSTER * GEMM_EPI_WARPS);  // one arrival per epilogue warp of each CTA of the cluster
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
  cluster_sync_all();  // every CTA's barriers exist before any peer arrives on them
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  grid_launch_dependents();
  // constant weights: request the first weight tiles while the previous kernel may still be running
  // (see gemm_tc_kernel); `pre` lives in the producer thread
  int pre = 0;
  if (threadIdx.x == 0 && p.early_b && cluster_id < p.tiles_m) {
    pre = nkb < STAGES ? nkb : STAGES;
    for (int kb = 0; kb < pre; ++kb) {
      mbar_arrive_expect_tx(&full_bar[kb], STAGE_BYTES);
      tma_load_2d(smem + size_t(kb) * STAGE_BYTES + A_BYTES, &tmap_b, &full_bar[kb], kb * BK, n_base);
    }
  }
  grid_dependency_wait();

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int mt = cluster_id; mt < p.tiles_m && ok; mt += num_clusters) {
        const int m0 = mt * GEMM_BM;
        for (int kb = 0; kb < nkb; ++kb) {
          uint8_t* sa = smem + size_t(stage) * STAGE_BYTES;
          if (mt == cluster_id && kb < pre) {
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
          tma_load_2d(sa + A_BYTES, &tmap_b, &full_bar[stage], kb * BK, n_base);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) {
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
      for (int mt = cluster_id; mt < p.tiles_m && ok; mt += num_clusters) {
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
          for (int k = 0; k < BK / UK; ++k)
            issue_mma<KIND>(d_tmem, make_smem_desc_sw128(a_addr + k * 32, 1024, 16),
                            make_smem_desc_sw128(b_addr + k * 32, 1024, 16), IDESC, (kb | k) != 0 ? 1u : 0u);
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
    const int quad = warp & 3;         // TMEM lane quadrant
    const int cg = (warp - 2) >> 2;    // column group of the CTA's BN columns
    const int r = quad * 32 + lane;    // row of the tile owned by this thread
    const int ew = cg * 4 + quad;      // index among the epilogue warps
    float* s_scale = epi_rows + ew * 4 * 64;
    float* s_bias = s_scale + 64;
    float* s_gamma = s_bias + 64;
    float* s_beta = s_gamma + 64;
    const int n0 = n_base + cg * COLS;  // first column of this warp's group (the same for every tile)
    for (int i = lane; i < COLS; i += 32) {
      const int col = n0 + i;
      // LayerNorm is a tolerance path: the two dequantisation scales are folded into one factor
      s_scale[i] = p.x_scale * (p.w_scale != nullptr ? __ldg(p.w_scale + col) : 1.0f);
      s_bias[i] = p.bias != nullptr ? __ldg(p.bias + col) : 0.0f;
      s_gamma[i] = __half2float(p.gamma[col]);
      s_beta[i] = __half2float(p.beta[col]);
    }
    __syncwarp();
    const float inv_q = ZEN_DIV(1.0f, p.out_scale);
    const float inv_n = 1.0f / float(p.N);
    int acc = 0;
    uint32_t acc_phase = 0;
    int it = 0;
    for (int mt = cluster_id; mt < p.tiles_m; mt += num_clusters, ++it) {
      const int row = mt * GEMM_BM + r;
      const bool row_ok = row < p.M;
      const int par = it & 1;
      // this thread's piece of the residual row, requested before the accumulator is waited for
      uint4 rr[COLS / 8];
      {
        const uint4* src = reinterpret_cast<const uint4*>(p.residual + int64_t(row_ok ? row : 0) * p.ldr + n0);
#pragma unroll
        for (int c = 0; c < COLS / 8; ++c) rr[c] = row_ok ? __ldg(src + c) : make_uint4(0u, 0u, 0u, 0u);
      }
      if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_flag)) break;
      tc_fence_after_sync();
      const uint32_t tacc = tmem_base + (uint32_t(quad * 32) << 16) + uint32_t(acc * BN + cg * COLS);
      // ---- y = dequant + bias + residual for this thread's COLS values of its row.  64 columns per thread are
      //      fetched in two halves (accumulators + residual + y would not fit the 96 registers a thread has).
      constexpr int PHASES = COLS > 48 ? 2 : 1;
      constexpr int PSTEPS = STEPS / PHASES;
      float2 y[COLS / 2];
      float2 s2 = make_float2(0.f, 0.f);
      const __half2* rh = reinterpret_cast<const __half2*>(rr);
#pragma unroll
      for (int ph = 0; ph < PHASES; ++ph) {
        uint32_t a[PSTEPS][GEMM_CW];
#pragma unroll
        for (int i = 0; i < PSTEPS; ++i) tmem_ld_32x16(tacc + uint32_t((ph * PSTEPS + i) * GEMM_CW), a[i]);
        tmem_wait_ld();
        if (ph == PHASES - 1) {
          tc_fence_before_sync();
          mbar_arrive(&tempty_bar[acc]);  // the accumulator has been read: the next tile's products may overwrite it
        }
#pragma unroll
        for (int ii = 0; ii < PSTEPS; ++ii) {
          const int i = ph * PSTEPS + ii;
#pragma unroll
          for (int j4 = 0; j4 < GEMM_CW / 4; ++j4) {
            const float4 c4 = reinterpret_cast<const float4*>(s_scale + i * GEMM_CW)[j4];
            const float4 b4 = reinterpret_cast<const float4*>(s_bias + i * GEMM_CW)[j4];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int e = 4 * j4 + 2 * h;          // element of the step
              const int j = (i * GEMM_CW + e) >> 1;  // column pair of the thread
              const float2 af = KIND == KIND_I8 ? make_float2(float(int32_t(a[ii][e])), float(int32_t(a[ii][e + 1])))
                                                : make_float2(__uint_as_float(a[ii][e]), __uint_as_float(a[ii][e + 1]));
              y[j] = f2add(f2fma(af, h ? make_float2(c4.z, c4.w) : make_float2(c4.x, c4.y),
                                 h ? make_float2(b4.z, b4.w) : make_float2(b4.x, b4.y)),
                           __half22float2(rh[j]));
              s2 = f2add(s2, y[j]);
            }
          }
        }
      }
      const float mean_t = (s2.x + s2.y) * (1.0f / COLS);
      float m2_t;
      {
        const float2 nmu = make_float2(-mean_t, -mean_t);
        float2 q22 = make_float2(0.f, 0.f);
#pragma unroll
        for (int j = 0; j < COLS / 2; ++j) {
          const float2 d = f2add(y[j], nmu);
          q22 = f2fma(d, d, q22);
        }
        m2_t = q22.x + q22.y;
      }
      // ---- publish to all four CTAs of the cluster; one release per warp: the 32 lanes' stores are ordered
      //      before lane 0's fence by the warp barrier, the fence before its arrivals
      {
        const uint32_t slot = smem_u32(&xstats[(par * LN_PARTS + int(rank) * 4 + cg) * 128 + r]);
        const uint32_t bar = smem_u32(&stats_bar[par]);
#pragma unroll
        for (uint32_t dst = 0; dst < LN_CLUSTER; ++dst) st_cluster_f32x2(map_to_cta(slot, dst), mean_t, m2_t);
        __syncwarp();
        if (lane == 0) {
          fence_acq_rel_cluster();
#pragma unroll
          for (uint32_t dst = 0; dst < LN_CLUSTER; ++dst) mbar_arrive_remote(map_to_cta(bar, dst));
        }
      }
      // ---- all 16 partials of every row have arrived (phase of stats_bar[par] flips every 2 tiles)
      if (!mbar_wait_cluster(&stats_bar[par], uint32_t(it >> 1) & 1u, abort_flag)) break;
      float mu, q2;
      {
        // equal counts: the row mean is the mean of the partial means, M2 = sum M2_k + COLS * sum (mean_k - mean)^2
        // (the partial means are read twice rather than held: the thread's registers are full of y)
        const float2* part = xstats + par * LN_PARTS * 128 + r;
        float sm = 0.f, sq = 0.f;
#pragma unroll
        for (int k = 0; k < LN_PARTS; ++k) {
          const float2 o = part[k * 128];
          sm += o.x;
          sq += o.y;
        }
        mu = sm * (1.0f / LN_PARTS);
        float dev = 0.f;
#pragma unroll
        for (int k = 0; k < LN_PARTS; ++k) {
          const float d = part[k * 128].x - mu;
          dev = fmaf(d, d, dev);
        }
        q2 = fmaf(dev, float(COLS), sq);
      }
      const float rstd = rsqrtf(q2 * inv_n + p.eps);

      // ---- normalise in registers, write fp16 (+ int8 copy of the values that were stored)
      const float2 nmu = make_float2(-mu, -mu);
      const float2 rstd2 = make_float2(rstd, rstd);
      __half* yrow = p.y + int64_t(row_ok ? row : 0) * p.N + n0;
      int8_t* qrow = p.yq + int64_t(row_ok ? row : 0) * p.N + n0;
#pragma unroll
      for (int i = 0; i < STEPS; ++i) {
        uint32_t w[GEMM_CW / 2];
        float2 of[GEMM_CW / 2];
#pragma unroll
        for (int j4 = 0; j4 < GEMM_CW / 4; ++j4) {
          const float4 g4 = reinterpret_cast<const float4*>(s_gamma + i * GEMM_CW)[j4];
          const float4 b4 = reinterpret_cast<const float4*>(s_beta + i * GEMM_CW)[j4];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int e = 4 * j4 + 2 * h;
            const float2 o = f2fma(f2mul(f2add(y[(i * GEMM_CW + e) >> 1], nmu), rstd2),
                                   h ? make_float2(g4.z, g4.w) : make_float2(g4.x, g4.y),
                                   h ? make_float2(b4.z, b4.w) : make_float2(b4.x, b4.y));
            const __half2 hv = __floats2half2_rn(o.x, o.y);
            w[e >> 1] = *reinterpret_cast<const uint32_t*>(&hv);
            of[e >> 1] = __half22float2(hv);
          }
        }
        if (row_ok) {
          uint4* dst = reinterpret_cast<uint4*>(yrow + i * GEMM_CW);
          dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
          dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
        }
        if (p.emit_q) {
          // branch-free fast rounding of all 16 values, exact recomputation only for the flagged ones
          uint32_t qw[GEMM_CW / 4];
          if (p.round_mode == 0) {
            const uint32_t risky = quantize_pairs_rn<GEMM_CW>(of, inv_q, qw);
            if (risky) {
#pragma unroll
              for (int j = 0; j < GEMM_CW; ++j)
                if (risky & (1u << j))
                  patch_q_byte(qw, j, zen_det_round_clamp_i8(ZEN_DIV((j & 1) ? of[j >> 1].y : of[j >> 1].x, p.out_scale), 0));
            }
          } else {
            int q[GEMM_CW];
#pragma unroll
            for (int j = 0; j < GEMM_CW; ++j)
              q[j] = zen_det_round_clamp_i8(ZEN_DIV((j & 1) ? of[j >> 1].y : of[j >> 1].x, p.out_scale), p.round_mode);
            pack_q(q, qw);
          }
          if (row_ok) *reinterpret_cast<uint4*>(qrow + i * GEMM_CW) = make_uint4(qw[0], qw[1], qw[2], qw[3]);
        }
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // no CTA leaves while a peer may still store into its shared memory
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_i8_ln_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const GemmLnParams p) {
  gemm_ln_body<KIND_I8, BN, STAGES>(tmap_a, tmap_b, p);
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_f16_ln_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const GemmLnParams p) {
  gemm_ln_body<KIND_F16, BN, STAGES>(tmap_a, tmap_b, p);
}

template <int KIND, int BN, int STAGES>
static int launch_gemm_ln(const CUtensorMap& ta, const CUtensorMap& tb, const GemmLnParams& p, cudaStream_t stream) {
  auto kernel = KIND == KIND_I8 ? gemm_i8_ln_kernel<BN, STAGES> : gemm_f16_ln_kernel<BN, STAGES>;
  constexpr size_t smem = gemm_ln_smem_bytes<BN, STAGES>();
  if (int st = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), smem); st != ZEN_OK) return st;
  int clusters = num_sms() / LN_CLUSTER;
  if (clusters > p.tiles_m) clusters = p.tiles_m;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(clusters * LN_CLUSTER);
  cfg.blockDim = dim3(GEMM_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = LN_CLUSTER;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (pdl_mask() & PDL_GEMM) ? 2 : 1;
  if (cudaLaunchKernelEx(&cfg, kernel, ta, tb, p) != cudaSuccess) {
    cudaGetLastError();
    return ZEN_ERR_LAUNCH;
  }
  return ZEN_OK;
}

}  // namespace zen

using namespace zen;

ZEN_DEFINE_TU_STATUS(gemm_ln)

template <int KIND>
static int run_linear_add_layernorm(const void* x, int64_t ldx, const void* w, int64_t ldw, int M, int N, int K, float x_scale,
                                    const float* w_scale, const float* bias, const void* residual, int64_t ldr,
                                    const void* gamma, const void* beta, float eps, void* y, int8_t* yq, float out_scale,
                                    int round_mode, unsigned flags, void* stream) {
  constexpr int ELEM = GemmKind<KIND>::ELEM;  // bytes per operand element
  constexpr int KA = 16 / ELEM;               // elements per 16 bytes: the unit K and the row strides must be a multiple of
  if (!x || !w || !residual || !gamma || !beta || !y || M <= 0 || N <= 0 || K <= 0) return ZEN_ERR_INVALID_ARG;
  if (round_mode != ZEN_ROUND_NEAREST_EVEN && round_mode != ZEN_ROUND_TRUNC) return ZEN_ERR_INVALID_ARG;
  if (flags & ~unsigned(ZEN_GEMM_CONST_WEIGHTS)) return ZEN_ERR_INVALID_ARG;
  if (yq && !(out_scale > 0.0f)) return ZEN_ERR_INVALID_ARG;
  if (N != 768 && N != 1024) return ZEN_ERR_UNSUPPORTED;  // four CTAs x 192 (or 256) columns hold one row
  if (K % KA || ldx % KA || ldw % KA || ldx < K || ldw < K || ldr % 8 || ldr < N) return ZEN_ERR_UNSUPPORTED;
  if (reinterpret_cast<uintptr_t>(y) % 16 || reinterpret_cast<uintptr_t>(yq) % 16 ||
      reinterpret_cast<uintptr_t>(residual) % 16)
    return ZEN_ERR_UNSUPPORTED;
  const int BN = N / LN_CLUSTER;
  constexpr int BK = 128 / ELEM;
  GemmLnParams p{};
  p.M = M; p.N = N; p.K = K;
  p.tiles_m = (M + GEMM_BM - 1) / GEMM_BM;
  p.num_k_blocks = (K + BK - 1) / BK;
  p.x_scale = x_scale; p.out_scale = yq ? out_scale : 1.0f; p.eps = eps; p.round_mode = round_mode;
  p.w_scale = w_scale; p.bias = bias;
  p.residual = static_cast<const __half*>(residual); p.ldr = ldr;
  p.gamma = static_cast<const __half*>(gamma); p.beta = static_cast<const __half*>(beta);
  p.y = static_cast<__half*>(y); p.yq = yq;
  p.emit_q = yq ? 1 : 0;
  p.early_b = (flags & ZEN_GEMM_CONST_WEIGHTS) ? 1 : 0;
  const CUtensorMapDataType dt = KIND == KIND_I8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUtensorMap ta, tb;
  int st = encode_tmap_2d(&ta, dt, x, uint64_t(K), uint64_t(M), uint64_t(ldx) * ELEM, BK, GEMM_BM);
  if (st == ZEN_OK) st = encode_tmap_2d(&tb, dt, w, uint64_t(K), uint64_t(N), uint64_t(ldw) * ELEM, BK, BN);
  if (st != ZEN_OK) return st;
  if (BN == 192) return launch_gemm_ln<KIND, 192, 4>(ta, tb, p, static_cast<cudaStream_t>(stream));
  return launch_gemm_ln<KIND, 256, 3>(ta, tb, p, static_cast<cudaStream_t>(stream));
}

extern "C" int zen_linear_i8_add_layernorm_ex(const int8_t* xq, int64_t ldx, const int8_t* wq, int64_t ldw, int M, int N,
                                              int K, float x_scale, const float* w_scale, const float* bias,
                                              const void* residual, int64_t ldr, const void* gamma, const void* beta,
                                              float eps, void* y, int8_t* yq, float out_scale, int round_mode,
                                              unsigned flags, void* stream) {
  return run_linear_add_layernorm<KIND_I8>(xq, ldx, wq, ldw, M, N, K, x_scale, w_scale, bias, residual, ldr, gamma, beta, eps,
                                           y, yq, out_scale, round_mode, flags, stream);
}

extern "C" int zen_linear_i8_add_layernorm(const int8_t* xq, int64_t ldx, const int8_t* wq, int64_t ldw, int M, int N,
                                           int K, float x_scale, const float* w_scale, const float* bias,
                                           const void* residual, int64_t ldr, const void* gamma, const void* beta,
                                           float eps, void* y, int8_t* yq, float out_scale, int round_mode,
                                           void* stream) {
  return run_linear_add_layernorm<KIND_I8>(xq, ldx, wq, ldw, M, N, K, x_scale, w_scale, bias, residual, ldr, gamma, beta, eps,
                                           y, yq, out_scale, round_mode, 0u, stream);
}

extern "C" int zen_linear_f16_add_layernorm_ex(const void* x, int64_t ldx, const void* w, int64_t ldw, int M, int N, int K,
                                               const float* bias, const void* residual, int64_t ldr, const void* gamma,
                                               const void* beta, float eps, void* y, int8_t* yq, float out_scale,
                                               int round_mode, unsigned flags, void* stream) {
  return run_linear_add_layernorm<KIND_F16>(x, ldx, w, ldw, M, N, K, 1.0f, nullptr, bias, residual, ldr, gamma, beta, eps, y,
                                            yq, out_scale, round_mode, flags, stream);
}

extern "C" int zen_linear_f16_add_layernorm(const void* x, int64_t ldx, const void* w, int64_t ldw, int M, int N, int K,
                                            const float* bias, const void* residual, int64_t ldr, const void* gamma,
                                            const void* beta, float eps, void* y, int8_t* yq, float out_scale,
                                            int round_mode, void* stream) {
  return run_linear_add_layernorm<KIND_F16>(x, ldx, w, ldw, M, N, K, 1.0f, nullptr, bias, residual, ldr, gamma, beta, eps, y,
                                            yq, out_scale, round_mode, 0u, stream);
}
