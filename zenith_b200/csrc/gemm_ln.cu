// W8A8 Linear + residual add + LayerNorm (+ int8 copy) in ONE kernel:
//     y   = (float(acc) * s_x) * s_w[n] + b[n] + residual[m, n]        acc = xq . wq^T  (int32, tcgen05 kind::i8)
//     out = (y - mean_m) * rstd_m * gamma[n] + beta[n]   -> fp16, and clamp(round(out / out_scale)) -> int8
// for the two projections of an encoder layer whose output width is the hidden size (attention
// output and FFN2).  The row statistics need all N columns of a row; a CTA holds only BN = N / 4 of
// them in TMEM, so four CTAs form a thread-block cluster along N, each reduces its BN columns per
// row and the four partial (mean, M2) pairs are exchanged through distributed shared memory:
// remote st.shared::cluster + remote mbarrier arrive, no cluster-wide barrier inside the tile loop,
// so the TMA / MMA warps keep running the next tile underneath.  Variances are combined with the
// pairwise (Chan) update, which is as robust as the two-pass form of the stand-alone kernel.
//
// Main loop, warp roles, TMEM double buffering and the TMA-store epilogue are those of
// gemm_tc.cuh; the epilogue makes two passes over tensor memory: the first replaces each accumulator
// by y (fp32) and reduces the statistics, the second normalises.
//
// A one-pass form was built and timed against this one (16 epilogue warps x BN / 4 columns held in registers, with
// registers moved from the producer / MMA warp group by setmaxnreg; statistics published as 256-byte bulk copies
// into the peers' shared memory; rows in and out through per-warp staging): 11.8 / 17.3 us for the two BERT-base
// projections at 4096 tokens against 11.4 / 16.6 us for this form.  Timestamps showed why: after the accumulator
// is complete the epilogue is bound by instruction issue (about 14 instructions per output at 0.45 per clock and
// scheduler: dequantise + residual + statistics 1.0 us, normalise + requantise 2.8 us, stores 1.3 us), not by the
// second trip through tensor memory, which overlaps that arithmetic here.
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

template <int BN, int STAGES>
constexpr size_t gemm_ln_smem_bytes() {
  constexpr int SLABS = BN / 64;
  // ring + fp16 staging (4 KB / warp) + int8 staging (2 KB / warp) + cluster statistics (2 x 4 x 128 float2)
  // + slab statistics (SLABS x 128 float2) + control (256 B) + per-warp rows (scale, bias, gamma, beta x 64)
  // + alignment slack
  return size_t(STAGES) * (GEMM_BM * 128 + BN * 128) + size_t(SLABS) * 4 * (4096 + 2048) + 2 * 4 * 128 * 8 +
         size_t(SLABS) * 128 * 8 + 256 + size_t(SLABS) * 4 * 4 * 64 * 4 + 1024;
}

// KIND_I8: int8 operands, s32 accumulators, dequantised with x_scale * w_scale[n]; KIND_F16: fp16 operands, fp32
// accumulators (the scale row holds ones).  Everything after the accumulator is shared.
template <int KIND, int BN, int STAGES>
__device__ __forceinline__ void gemm_ln_body(const CUtensorMap& tmap_a, const CUtensorMap& tmap_b, const CUtensorMap& tmap_y,
                                             const CUtensorMap& tmap_q, const CUtensorMap& tmap_r, const GemmLnParams& p) {
  constexpr int ELEM = GemmKind<KIND>::ELEM;
  constexpr int BK = 128 / ELEM, UK = 32 / ELEM;
  constexpr int A_BYTES = GEMM_BM * 128;
  constexpr int B_BYTES = BN * 128;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int SLABS = BN / 64;
  constexpr int EPI_ACTIVE = SLABS * 4 * 32;  // epilogue threads that own a slab
  constexpr uint32_t TMEM_COLS = gemm_tmem_cols<BN>();
  constexpr uint32_t IDESC = KIND == KIND_I8 ? make_idesc(IDESC_C_S32, IDESC_S8, IDESC_S8, 0, 0, GEMM_BM, BN)
                                             : make_idesc(IDESC_C_F32, IDESC_F16, IDESC_F16, 0, 0, GEMM_BM, BN);
  constexpr int STEPS = 64 / GEMM_CW;
  static_assert(BN % 64 == 0 && BN <= 256, "BN");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* stage_y = smem + size_t(STAGES) * STAGE_BYTES;       // [SLABS*4][4 KB]
  uint8_t* stage_q = stage_y + size_t(SLABS) * 4 * 4096;        // [SLABS*4][2 KB]
  float2* xstats = reinterpret_cast<float2*>(stage_q + size_t(SLABS) * 4 * 2048);  // [2][4 ranks][128]
  float2* pstats = xstats + 2 * LN_CLUSTER * 128;               // [SLABS][128]
  uint8_t* ctrl = reinterpret_cast<uint8_t*>(pstats + SLABS * 128);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(ctrl);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint64_t* stats_bar = tempty_bar + 2;  // [2] cluster-wide: the four partials of every row have arrived
  uint64_t* slab_bar = stats_bar + 2;    // CTA-local: the SLABS partials of every row are in pstats
  uint64_t* res_bar = slab_bar + 1;      // [SLABS * 4] per warp: its 32 x 64 residual block has landed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(res_bar + SLABS * 4);
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
    tma_prefetch_desc(&tmap_y);
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_r);
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull_bar[i], 1);
      mbar_init(&tempty_bar[i], GEMM_EPI_WARPS * 32);
      mbar_init(&stats_bar[i], LN_CLUSTER * 4);  // one arrival per row-owning warp of each CTA of the cluster
    }
    mbar_init(slab_bar, EPI_ACTIVE);
    for (int i = 0; i < SLABS * 4; ++i) mbar_init(&res_bar[i], 1);
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
    const int quad = warp & 3;
    const int sub = (warp - 2) >> 2;
    const int r = quad * 32 + lane;  // row of the tile owned by this thread
    if (sub < SLABS) {
      const int ew = sub * 4 + quad;  // index among the slab-owning warps
      float* s_scale = epi_rows + ew * 4 * 64;
      float* s_bias = s_scale + 64;
      float* s_gamma = s_bias + 64;
      float* s_beta = s_gamma + 64;
      uint8_t* sty = stage_y + size_t(ew) * 4096;
      uint8_t* stq = stage_q + size_t(ew) * 2048;
      const int n0 = n_base + sub * 64;  // first column of this warp's slab (the same for every tile)
      for (int i = lane; i < 64; i += 32) {
        const int col = n0 + i;
        const bool in = col < p.N;
        // LayerNorm is a tolerance path: the two dequantisation scales are folded into one factor
        s_scale[i] = p.x_scale * ((p.w_scale != nullptr && in) ? __ldg(p.w_scale + col) : 1.0f);
        s_bias[i] = (p.bias != nullptr && in) ? __ldg(p.bias + col) : 0.0f;
        s_gamma[i] = in ? __half2float(p.gamma[col]) : 0.0f;
        s_beta[i] = in ? __half2float(p.beta[col]) : 0.0f;
      }
      __syncwarp();
      const float inv_q = ZEN_DIV(1.0f, p.out_scale);
      const float inv_n = 1.0f / float(p.N);
      int acc = 0;
      uint32_t acc_phase = 0;
      int it = 0;
      bool ok = true;
      for (int mt = cluster_id; mt < p.tiles_m; mt += num_clusters, ++it) {
        const int m0 = mt * GEMM_BM;
        const int par = it & 1;
        // The 32 x 64 residual block of this warp is fetched by TMA into the fp16 staging block (same
        // swizzled layout as the output block that later overwrites it in place, row by row).
        if (lane == 0) {
          tma_store_wait_read();  // the previous tile's stores have finished reading the blocks
          mbar_arrive_expect_tx(&res_bar[ew], 4096);
          tma_load_2d(sty, &tmap_r, &res_bar[ew], n0, m0 + quad * 32);
        }
        __syncwarp();
        if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_flag)) { ok = false; break; }
        if (!mbar_wait(&res_bar[ew], uint32_t(it) & 1u, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t tacc = tmem_base + (uint32_t(quad * 32) << 16) + uint32_t(acc * BN + sub * 64);

        // ---- pass A: y = dequant + bias + residual for this thread's 64 values of its row, written
        //      back over the accumulator (fp32 bits) for pass B, and their (mean, M2)
        float mean = 0.f, m2 = 0.f;
#pragma unroll 1
        for (int i = 0; i < STEPS; ++i) {
          uint32_t a[GEMM_CW];
          __syncwarp();
          tmem_ld_32x16(tacc + uint32_t(i * GEMM_CW), a);
          uint4 rr[2];
          rr[0] = *reinterpret_cast<const uint4*>(sty + lane * 128 + (((2 * i) ^ (lane & 7)) << 4));
          rr[1] = *reinterpret_cast<const uint4*>(sty + lane * 128 + (((2 * i + 1) ^ (lane & 7)) << 4));
          float cs[GEMM_CW], bs[GEMM_CW];
#pragma unroll
          for (int j4 = 0; j4 < GEMM_CW / 4; ++j4) {
            *reinterpret_cast<float4*>(cs + 4 * j4) = reinterpret_cast<const float4*>(s_scale + i * GEMM_CW)[j4];
            *reinterpret_cast<float4*>(bs + 4 * j4) = reinterpret_cast<const float4*>(s_bias + i * GEMM_CW)[j4];
          }
          tmem_wait_ld();
          const __half2* rh = reinterpret_cast<const __half2*>(rr);
          // column pairs on the packed fp32x2 instructions (one issue slot for two operations)
          float2 y[GEMM_CW / 2];
          float2 s2 = make_float2(0.f, 0.f);
#pragma unroll
          for (int j = 0; j < GEMM_CW / 2; ++j) {
            const float2 af = KIND == KIND_I8 ? make_float2(float(int32_t(a[2 * j])), float(int32_t(a[2 * j + 1])))
                                              : make_float2(__uint_as_float(a[2 * j]), __uint_as_float(a[2 * j + 1]));
            y[j] = f2add(f2fma(af, make_float2(cs[2 * j], cs[2 * j + 1]), make_float2(bs[2 * j], bs[2 * j + 1])),
                              __half22float2(rh[j]));
            s2 = f2add(s2, y[j]);
          }
          uint32_t yb[GEMM_CW];
#pragma unroll
          for (int j = 0; j < GEMM_CW / 2; ++j) {
            yb[2 * j] = __float_as_uint(y[j].x);
            yb[2 * j + 1] = __float_as_uint(y[j].y);
          }
          tmem_st_32x16(tacc + uint32_t(i * GEMM_CW), yb);
          const float mu = (s2.x + s2.y) * (1.0f / GEMM_CW);
          const float2 nmu = make_float2(-mu, -mu);
          float2 q22 = make_float2(0.f, 0.f);
#pragma unroll
          for (int j = 0; j < GEMM_CW / 2; ++j) {
            const float2 d = f2add(y[j], nmu);
            q22 = f2fma(d, d, q22);
          }
          const float q2 = q22.x + q22.y;
          if (i == 0) {
            mean = mu;
            m2 = q2;
          } else {
            // pairwise update with n_a = 16 i, n_b = 16: n_b / n = 1 / (i + 1)
            const float f = i == 1 ? 0.5f : i == 2 ? (1.0f / 3.0f) : i == 3 ? 0.25f : 1.0f / float(i + 1);
            const float delta = mu - mean;
            mean = fmaf(delta, f, mean);
            m2 = m2 + q2 + delta * delta * (float(GEMM_CW * i) * f);
          }
        }
        tmem_wait_st();
        pstats[sub * 128 + r] = make_float2(mean, m2);
        mbar_arrive(slab_bar);
        if (sub == 0) {
          if (!mbar_wait(slab_bar, uint32_t(it) & 1u, abort_flag)) { ok = false; break; }
          // one thread per row: this CTA's BN columns, published to all four CTAs of the cluster
          float c = 64.f, mu = mean, q2 = m2;
#pragma unroll
          for (int s = 1; s < SLABS; ++s) {
            const float2 o = pstats[s * 128 + r];
            chan_merge(c, mu, q2, 64.f, o.x, o.y);
          }
          const uint32_t slot = smem_u32(&xstats[(par * LN_CLUSTER + int(rank)) * 128 + r]);
          const uint32_t bar = smem_u32(&stats_bar[par]);
#pragma unroll
          for (uint32_t dst = 0; dst < LN_CLUSTER; ++dst) st_cluster_f32x2(map_to_cta(slot, dst), mu, q2);
          // one release per warp instead of one per row: the 32 lanes' stores are ordered before lane
          // 0's fence by the warp barrier, the fence before its arrivals
          __syncwarp();
          if (lane == 0) {
            fence_acq_rel_cluster();
#pragma unroll
            for (uint32_t dst = 0; dst < LN_CLUSTER; ++dst) mbar_arrive_remote(map_to_cta(bar, dst));
          }
        }
        // ---- all four partials of every row have arrived (phase of stats_bar[par] flips every 2 tiles)
        if (!mbar_wait_cluster(&stats_bar[par], uint32_t(it >> 1) & 1u, abort_flag)) { ok = false; break; }
        float c = float(BN), mu, q2;
        {
          const float2 o0 = xstats[(par * LN_CLUSTER + 0) * 128 + r];
          mu = o0.x;
          q2 = o0.y;
#pragma unroll
          for (int k = 1; k < LN_CLUSTER; ++k) {
            const float2 o = xstats[(par * LN_CLUSTER + k) * 128 + r];
            chan_merge(c, mu, q2, float(BN), o.x, o.y);
          }
        }
        const float rstd = rsqrtf(q2 * inv_n + p.eps);

        // ---- pass B: normalise y (read back from tensor memory), stage fp16 (+ int8), TMA stores
#pragma unroll 1
        for (int i = 0; i < STEPS; ++i) {
          uint32_t yb[GEMM_CW];
          __syncwarp();
          tmem_ld_32x16(tacc + uint32_t(i * GEMM_CW), yb);
          float gs[GEMM_CW], bs[GEMM_CW];
#pragma unroll
          for (int j4 = 0; j4 < GEMM_CW / 4; ++j4) {
            *reinterpret_cast<float4*>(gs + 4 * j4) = reinterpret_cast<const float4*>(s_gamma + i * GEMM_CW)[j4];
            *reinterpret_cast<float4*>(bs + 4 * j4) = reinterpret_cast<const float4*>(s_beta + i * GEMM_CW)[j4];
          }
          tmem_wait_ld();
          uint32_t w[GEMM_CW / 2];
          float2 of[GEMM_CW / 2];  // the values that are stored: the int8 copy quantizes these
          const float2 nmu = make_float2(-mu, -mu);
          const float2 rstd2 = make_float2(rstd, rstd);
#pragma unroll
          for (int j = 0; j < GEMM_CW; j += 2) {
            const float2 yv = make_float2(__uint_as_float(yb[j]), __uint_as_float(yb[j + 1]));
            const float2 o = f2fma(f2mul(f2add(yv, nmu), rstd2), make_float2(gs[j], gs[j + 1]),
                                   make_float2(bs[j], bs[j + 1]));
            const __half2 h = __floats2half2_rn(o.x, o.y);
            w[j >> 1] = *reinterpret_cast<const uint32_t*>(&h);
            of[j >> 1] = __half22float2(h);
          }
          uint8_t* srow = sty + lane * 128;
          *reinterpret_cast<uint4*>(srow + (((2 * i) ^ (lane & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
          *reinterpret_cast<uint4*>(srow + (((2 * i + 1) ^ (lane & 7)) << 4)) = make_uint4(w[4], w[5], w[6], w[7]);
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
            *reinterpret_cast<uint4*>(stq + lane * 64 + ((i ^ ((lane >> 1) & 3)) << 4)) = make_uint4(qw[0], qw[1], qw[2], qw[3]);
          }
        }
        __syncwarp();
        tc_fence_before_sync();
        mbar_arrive(&tempty_bar[acc]);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0 && n0 < p.N && m0 + quad * 32 < p.M) {
          tma_store_2d(&tmap_y, sty, n0, m0 + quad * 32);
          if (p.emit_q) tma_store_2d(&tmap_q, stq, n0, m0 + quad * 32);
          tma_store_commit();
        }
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
      if (lane == 0) tma_store_wait_all();
      (void)ok;
    } else {
      // no slab for this warp at this tile width: it still owes its arrivals on the accumulator barriers
      int acc = 0;
      uint32_t acc_phase = 0;
      for (int mt = cluster_id; mt < p.tiles_m; mt += num_clusters) {
        if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_flag)) break;
        mbar_arrive(&tempty_bar[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  // No cluster-wide rendezvous here: the only accesses a peer makes to this CTA's shared memory are the partial
  // statistics of a tile and the arrival that follows them, and this CTA has waited for all of them (stats_bar of
  // its last tile) before it got here; a peer publishes nothing after its last tile.
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_i8_ln_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                  const __grid_constant__ CUtensorMap tmap_y, const __grid_constant__ CUtensorMap tmap_q,
                  const __grid_constant__ CUtensorMap tmap_r, const GemmLnParams p) {
  gemm_ln_body<KIND_I8, BN, STAGES>(tmap_a, tmap_b, tmap_y, tmap_q, tmap_r, p);
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_f16_ln_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                   const __grid_constant__ CUtensorMap tmap_y, const __grid_constant__ CUtensorMap tmap_q,
                   const __grid_constant__ CUtensorMap tmap_r, const GemmLnParams p) {
  gemm_ln_body<KIND_F16, BN, STAGES>(tmap_a, tmap_b, tmap_y, tmap_q, tmap_r, p);
}

template <int KIND, int BN, int STAGES>
static int launch_gemm_ln(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& ty, const CUtensorMap& tq,
                          const CUtensorMap& tr, const GemmLnParams& p, cudaStream_t stream) {
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
  if (cudaLaunchKernelEx(&cfg, kernel, ta, tb, ty, tq, tr, p) != cudaSuccess) {
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
  p.emit_q = yq ? 1 : 0;
  p.early_b = (flags & ZEN_GEMM_CONST_WEIGHTS) ? 1 : 0;
  const CUtensorMapDataType dt = KIND == KIND_I8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUtensorMap ta, tb, ty, tq, tr;
  int st = encode_tmap_2d(&ta, dt, x, uint64_t(K), uint64_t(M), uint64_t(ldx) * ELEM, BK, GEMM_BM);
  if (st == ZEN_OK) st = encode_tmap_2d(&tb, dt, w, uint64_t(K), uint64_t(N), uint64_t(ldw) * ELEM, BK, BN);
  if (st == ZEN_OK)
    st = encode_tmap_2d(&ty, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, y, uint64_t(N), uint64_t(M), uint64_t(N) * 2, 64, 32,
                        CU_TENSOR_MAP_SWIZZLE_128B);
  tq = ty;
  if (st == ZEN_OK && yq)
    st = encode_tmap_2d(&tq, CU_TENSOR_MAP_DATA_TYPE_UINT8, yq, uint64_t(N), uint64_t(M), uint64_t(N), 64, 32,
                        CU_TENSOR_MAP_SWIZZLE_64B);
  if (st == ZEN_OK)
    st = encode_tmap_2d(&tr, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, residual, uint64_t(N), uint64_t(M), uint64_t(ldr) * 2, 64, 32,
                        CU_TENSOR_MAP_SWIZZLE_128B);
  if (st != ZEN_OK) return st;
  if (BN == 192) return launch_gemm_ln<KIND, 192, 3>(ta, tb, ty, tq, tr, p, static_cast<cudaStream_t>(stream));
  return launch_gemm_ln<KIND, 256, 2>(ta, tb, ty, tq, tr, p, static_cast<cudaStream_t>(stream));
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
