// CTA-pair form of the persistent tcgen05 GEMM of gemm_tc.cuh:  D[M,N] = A[M,K] . B[N,K]^T  with the same fused
// epilogue, for int8 and fp16 operands (K-major B only).
//
// Two CTAs of a cluster (ranks 0 = leader and 1) share every 256 x BN tile: tcgen05.mma.cta_group::2 with
// M = 256.  Each CTA loads only ITS 128 rows of A and ITS BN / 2 rows of B per k-block (32 KB at BN = 256,
// where the one-CTA kernel pulls 48 KB for half the work), which is what the main loop of these GEMMs is bound
// by: the rate at which L2 feeds an SM's shared memory.  The smaller stages also buy a deeper ring.
// No TMA multicast: every copy lands in the issuing CTA's own shared memory.
//
//   warp 0      : TMA producer of its CTA.  Both producers count their bytes on the LEADER's full barrier.
//   warp 1      : allocates / frees TMEM (both CTAs, cta_group::2); in the leader one lane issues the MMAs and
//                 commits: stage-free barriers and accumulator-full barriers of BOTH CTAs (commit with a CTA mask).
//   warps 2..17 : epilogue of the CTA's own 128 accumulator rows (gemm_epilogue_role); one lane per warp
//                 releases the accumulator on the leader's barrier (a remote arrival for the peer CTA).
//
// Tile t = pair + i * num_pairs, row blocks fastest; CTA `rank` owns rows rank * 128 .. + 127 of the tile.
#pragma once
#include "gemm_tc.cuh"

namespace zen {

template <int BN, int STAGES>
__host__ __device__ constexpr size_t gemm_pair_smem_bytes() {
  // ring (A 16 KB + B BN/2 x 128 B per stage) + output staging (4 KB per active epilogue warp) + barriers / flags
  // (256 B) + per-epilogue-warp scale and bias entries + alignment slack
  return size_t(STAGES) * (GEMM_BM * 128 + (BN / 2) * 128) + size_t((BN + 63) / 64) * 4 * 4096 + 256 +
         size_t(GEMM_EPI_WARPS) * 3 * 64 * 4 + 1024;
}

template <int KIND>
__device__ __forceinline__ void issue_mma_pair(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
  if constexpr (KIND == KIND_I8) mma_i8_ss_pair(d, a, b, idesc, acc);
  else mma_f16_ss_pair(d, a, b, idesc, acc);
}

template <int KIND, int BN, int STAGES>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_c, const GemmParams p) {
  static_assert(KIND == KIND_I8 || KIND == KIND_F16, "operand kinds of the pair kernel");
  constexpr int ELEM = GemmKind<KIND>::ELEM;
  constexpr int BK = 128 / ELEM;  // elements per 128-byte swizzle row == K extent of one stage
  constexpr int UK = 32 / ELEM;   // K extent of one tcgen05.mma
  constexpr int HALF_N = BN / 2;  // B rows held by each CTA
  constexpr int A_BYTES = GEMM_BM * 128;
  constexpr int B_BYTES = HALF_N * 128;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;  // per CTA; the leader's barrier expects twice this
  constexpr uint32_t TMEM_COLS = gemm_tmem_cols<BN>();
  constexpr uint32_t IDESC = KIND == KIND_I8 ? make_idesc(IDESC_C_S32, IDESC_S8, IDESC_S8, 0, 0, 2 * GEMM_BM, BN)
                                             : make_idesc(IDESC_C_F32, IDESC_F16, IDESC_F16, 0, 0, 2 * GEMM_BM, BN);
  static_assert(BN % 64 == 0 && BN >= 64 && BN <= 256, "BN");
  static_assert(HALF_N % 8 == 0, "each CTA's B rows come in whole 8-row swizzle groups");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  constexpr int SLABS = (BN + 63) / 64;
  uint8_t* out_stage = smem + size_t(STAGES) * STAGE_BYTES;  // [SLABS][4 quadrants][4 KB], 1024-byte aligned
  uint8_t* ctrl = out_stage + size_t(SLABS) * 4 * 4096;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(ctrl);  // used in the leader only
  uint64_t* empty_bar = full_bar + STAGES;                  // one set per CTA, signalled by the leader's commits
  uint64_t* tfull_bar = empty_bar + STAGES;                 // one set per CTA, signalled by the leader's commits
  uint64_t* tempty_bar = tfull_bar + 2;                     // used in the leader only: epilogue warps of both CTAs
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* epi_rows = reinterpret_cast<float*>(ctrl + 256);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0: leader
  const bool leader = rank == 0;
  const int pair = int(blockIdx.x) >> 1;
  const int num_pairs = int(gridDim.x) >> 1;
  const int num_tiles = p.tiles_m * p.tiles_n;  // p.tiles_m counts 256-row blocks here
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
      mbar_init(&tempty_bar[i], 2 * GEMM_EPI_WARPS);  // one arrival per epilogue warp of both CTAs
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before a copy or an arrival of the peer can reach them
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // shared::cluster addresses of the leader's barriers (the local ones when this CTA is the leader)
  const uint32_t full_bar_leader = map_to_cta(smem_u32(full_bar), 0);
  const uint32_t tempty_bar_leader = map_to_cta(smem_u32(tempty_bar), 0);
  if (threadIdx.x == 1) {
#pragma unroll
    for (int i = 0; i < 2; ++i)
      if (p.pf_bytes[i] != 0) prefetch_slice_l2(p.pf_ptr[i], p.pf_bytes[i], blockIdx.x, gridDim.x);
  }
  grid_launch_dependents();
  // Constant weights: the B tiles of the first tile's first k-blocks are requested before the dependency wait
  // (see gemm_tc_kernel); the leader announces the bytes of the whole stage (both CTAs, A and B).
  int pre = 0;
  if (threadIdx.x == 0 && p.early_b && pair < num_tiles) {
    const int n0 = (pair / p.tiles_m) * BN + int(rank) * HALF_N;
    pre = nkb < STAGES ? nkb : STAGES;
    for (int kb = 0; kb < pre; ++kb) {
      if (leader) mbar_arrive_expect_tx(&full_bar[kb], 2 * STAGE_BYTES);
      tma_load_2d_pair(smem + size_t(kb) * STAGE_BYTES + A_BYTES, &tmap_b, full_bar_leader + uint32_t(kb) * 8u, kb * BK, n0);
    }
  }
  grid_dependency_wait();  // operands and output buffers may belong to the previous kernel until here

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (each CTA: its own halves)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        const int m0 = (tile % p.tiles_m) * (2 * GEMM_BM) + int(rank) * GEMM_BM;
        const int n0 = (tile / p.tiles_m) * BN + int(rank) * HALF_N;
        for (int kb = 0; kb < nkb; ++kb) {
          uint8_t* sa = smem + size_t(stage) * STAGE_BYTES;
          const uint32_t bar = full_bar_leader + uint32_t(stage) * 8u;
          if (tile == pair && kb < pre) {
            // stage kb: fresh, the leader's barrier already expects the bytes and the B half is on the way
            tma_load_2d_pair(sa, &tmap_a, bar, kb * BK, m0);
          } else {
            if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) {
              ok = false;
              break;
            }
            if (leader) mbar_arrive_expect_tx(&full_bar[stage], 2 * STAGE_BYTES);
            tma_load_2d_pair(sa, &tmap_a, bar, kb * BK, m0);
            tma_load_2d_pair(sa + A_BYTES, &tmap_b, bar, kb * BK, n0);
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
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && leader) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        if (!mbar_wait_cluster(&tempty_bar[acc], acc_phase ^ 1u, abort_flag)) break;
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
            issue_mma_pair<KIND>(d_tmem, make_smem_desc_sw128(a_addr + k * 32, 1024, 16),
                                 make_smem_desc_sw128(b_addr + k * 32, 1024, 16), IDESC, (kb | k) != 0 ? 1u : 0u);
          tc_commit_pair(&empty_bar[stage], 0x3);  // the stage is free in both CTAs
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) tc_commit_pair(&tfull_bar[acc], 0x3);  // both CTAs' halves of the accumulator are complete
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (own 128 rows of each tile)
    const TmemEmptySignal tempty{nullptr, tempty_bar_leader};
    gemm_epilogue_role<KIND, BN, true>(p, tmap_c, tmem_base, out_stage, epi_rows, tfull_bar, tempty, abort_flag, warp, lane,
                                       pair, num_pairs, num_tiles, int(rank) * GEMM_BM);
  }

  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // neither CTA leaves (or frees TMEM) while the pair's MMAs, copies or arrivals may still touch it
  if (warp == 1) tmem_dealloc_pair(tmem_base, TMEM_COLS);
}

}  // namespace zen
