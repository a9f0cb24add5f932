// Flash-attention forward for sequences longer than one key block: two 128-query tiles per CTA.
//
//   warp 0      : TMA producer — both Q tiles once, then K and V tiles of 128 keys (ring of KV_STAGES)
//   warp 1      : TMEM owner and tcgen05.mma issuer for both tiles
//   warps 2..5  : softmax group A (query rows 0..127 of the CTA), one thread per row
//   warps 6..9  : softmax group B (query rows 128..255)
//
// K and V are loaded once for 256 queries, and while one group runs its softmax the tensor core
// works for the other (S = Q K^T of the next block, O += P V of the current one).  A softmax thread
// takes its whole row of S (128 values) into registers in one trip through tensor memory and
// releases the S columns at once, so that Q K^T of the group's next block runs under the softmax
// of this one; the issuer serves both groups' events (S read, P ready) in the order they occur.
// Moving a share of the exponentials from the special-function unit to a cubic on the FMA / integer pipes
// (round-to-nearest split, 2^f on [-0.5, 0.5], exponent add: about ten issue slots per column pair against
// two) was measured at 25 / 50 / 75 / 100 % of the pairs and lost at every share (head size 64, S = 8192:
// 563 TFLOP/s without it, 533 / 545 / 457 / 409 with it): with two softmax warps per scheduler the loop is
// bound by instruction issue and dependent-instruction latency, not by the unit's 16 results per clock.
// Two threads per row (16 softmax warps per CTA, block maximum and row sum exchanged through shared memory,
// as in the fused QKV + attention kernel) was also built and measured: 561 / 957 TFLOP/s at head size 64 /
// 128 against 563 / 1002 with one thread per row; profiler counters of that form: issue slots 48 % busy,
// special-function unit 50 %, ALU 47 %, tensor pipe 24 %, 7.7 thread-instructions per score.  O accumulates in
// TMEM across key blocks (tcgen05.mma with the accumulate flag); the running maximum used for
// scaling is only moved, and O rescaled in TMEM by tcgen05.ld / st, when the row maximum has grown
// by more than 2^8 since the last move, so that the rescale is rare after the first blocks and P
// stays below 256 in fp16.  TMEM: S_A, S_B (128 columns each), O_A, O_B (D columns each).
#pragma once
#include "zen_common.cuh"

namespace zen {

constexpr int FAP_THREADS = 320;

template <int D, int KV_STAGES>
constexpr size_t fap_smem_bytes() {
  // 2 Q tiles + KV_STAGES x (K + V) tiles (128 x D fp16 each) + 2 P tiles (128 x 128 fp16) + control + slack
  return size_t(2 + 2 * KV_STAGES) * 128 * D * 2 + 2 * 128 * 128 * 2 + 256 + 1024;
}

template <int D, int KV_STAGES>
__global__ void __launch_bounds__(FAP_THREADS, 1)
flash_attn_pipe_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                       const __grid_constant__ CUtensorMap tmap_v, const FaParams p) {
  constexpr int DC = D / 64;
  constexpr int TILE_BYTES = 128 * D * 2;
  constexpr int CHUNK_BYTES = 128 * 128;
  constexpr int P_BYTES = 128 * 128 * 2;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t IDESC_QK = make_idesc(IDESC_C_F32, IDESC_F16, IDESC_F16, 0, 0, 128, 128);
  constexpr uint32_t IDESC_PV = make_idesc(IDESC_C_F32, IDESC_F16, IDESC_F16, 0, 1, 128, D);
  constexpr float RESCALE_THRESHOLD = 8.0f;  // log2 units

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* sQ = smem;                              // [2][TILE]
  uint8_t* sK = sQ + 2 * TILE_BYTES;               // [KV_STAGES][TILE]
  uint8_t* sV = sK + KV_STAGES * TILE_BYTES;       // [KV_STAGES][TILE]
  uint8_t* sP = sV + KV_STAGES * TILE_BYTES;       // [2][P]
  uint8_t* ctrl = sP + 2 * P_BYTES;
  uint64_t* q_full = reinterpret_cast<uint64_t*>(ctrl);
  uint64_t* k_full = q_full + 1;                   // [KV_STAGES]
  uint64_t* k_empty = k_full + KV_STAGES;
  uint64_t* v_full = k_empty + KV_STAGES;
  uint64_t* v_empty = v_full + KV_STAGES;
  uint64_t* s_full = v_empty + KV_STAGES;          // [2] per group
  uint64_t* p_full = s_full + 2;                   // [2]
  uint64_t* o_full = p_full + 2;                   // [2]
  uint64_t* s_free = o_full + 2;                   // [2] the group has taken S into registers
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_free + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * 256;
  const int h = blockIdx.y;
  const int b = blockIdx.z;

  // see flash_attn_kernel: the key length is read after the dependency wait when this family launches early
  int kv_len = p.S;
  if constexpr (!kAttentionLaunchesEarly) {
    if (p.kv_lens) kv_len = p.kv_lens[b];
  }

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
    mbar_init(q_full, 1);
    for (int i = 0; i < KV_STAGES; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
    }
    for (int g = 0; g < 2; ++g) {
      mbar_init(&s_full[g], 1);
      mbar_init(&p_full[g], 128);
      mbar_init(&o_full[g], 1);
      mbar_init(&s_free[g], 128);
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
  grid_launch_dependents();
  grid_dependency_wait();
  if constexpr (kAttentionLaunchesEarly) {
    if (p.kv_lens) kv_len = p.kv_lens[b];
  }
  // Unpadded batches: the sequences lie back to back in one [rows, ...] tensor, sequence b in rows cu_seqlens[b] ..
  // cu_seqlens[b + 1] - 1 (cut at the tensor's rows).  A tile then starts at the sequence's first row and may run on
  // into the next sequence's rows: as keys they lie beyond the key length and are masked like padding, as queries
  // their rows are not stored.  The tensor maps see one batch of `rows` tokens.
  int row_base = 0;  // first row of this sequence in the packed tensors
  int tma_b = b;
  if (p.cu_seqlens != nullptr) {
    const int lo = p.cu_seqlens[b], hi = p.cu_seqlens[b + 1];
    kv_len = lo < 0 ? 0 : (hi < p.rows ? hi : p.rows) - lo;
    row_base = lo < 0 ? 0 : lo;
    tma_b = 0;
  }
  kv_len = kv_len < 0 ? 0 : (kv_len > p.S ? p.S : kv_len);
  const int q_len = p.cu_seqlens != nullptr ? kv_len : p.S;  // query rows of this sequence
  // key blocks needed by each group (group B has no rows if the sequence ends before its tile)
  int nblk[2];
#pragma unroll
  for (int g = 0; g < 2; ++g) {
    int end = kv_len;
    if (p.causal && q0 + g * 128 + 128 < end) end = q0 + g * 128 + 128;
    nblk[g] = (q0 + g * 128 < q_len) ? (end + 127) / 128 : 0;
  }
  const int n_blocks = nblk[0] > nblk[1] ? nblk[0] : nblk[1];

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0 && n_blocks > 0) {
      bool ok = true;
      mbar_arrive_expect_tx(q_full, 2 * TILE_BYTES);
#pragma unroll
      for (int g = 0; g < 2; ++g)
#pragma unroll
        for (int dc = 0; dc < DC; ++dc)
          fa_tma_tile(sQ + g * TILE_BYTES + dc * CHUNK_BYTES, &tmap_q, q_full, p.q_perm, dc * 64, row_base + q0 + g * 128, h, tma_b);
      for (int j = 0; j < n_blocks && ok; ++j) {
        const int st = j % KV_STAGES;
        const uint32_t ph = (j / KV_STAGES) & 1;
        if (!mbar_wait(&k_empty[st], ph ^ 1u, abort_flag)) { ok = false; break; }
        mbar_arrive_expect_tx(&k_full[st], TILE_BYTES);
#pragma unroll
        for (int dc = 0; dc < DC; ++dc)
          fa_tma_tile(sK + st * TILE_BYTES + dc * CHUNK_BYTES, &tmap_k, &k_full[st], p.k_perm, dc * 64, row_base + j * 128, h, tma_b);
        if (!mbar_wait(&v_empty[st], ph ^ 1u, abort_flag)) { ok = false; break; }
        mbar_arrive_expect_tx(&v_full[st], TILE_BYTES);
#pragma unroll
        for (int dc = 0; dc < DC; ++dc)
          fa_tma_tile(sV + st * TILE_BYTES + dc * CHUNK_BYTES, &tmap_v, &v_full[st], p.v_perm, dc * 64, row_base + j * 128, h, tma_b);
      }
      if (!ok) {
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0 && n_blocks > 0) {
      auto issue_qk = [&](int g, int j) {
        const uint32_t qa = smem_u32(sQ + g * TILE_BYTES);
        const uint32_t ka = smem_u32(sK + (j % KV_STAGES) * TILE_BYTES);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = (ks / 4) * CHUNK_BYTES + (ks % 4) * 32;
          mma_f16_ss(tmem_base + uint32_t(g * 128), make_smem_desc_sw128(qa + off, 1024, 16),
                     make_smem_desc_sw128(ka + off, 1024, 16), IDESC_QK, ks != 0 ? 1u : 0u);
        }
        tc_commit(&s_full[g]);
      };
      auto issue_pv = [&](int g, int j) {
        const uint32_t pa = smem_u32(sP + g * P_BYTES);
        const uint32_t va = smem_u32(sV + (j % KV_STAGES) * TILE_BYTES);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          mma_f16_ss(tmem_base + uint32_t(256 + g * D),
                     make_smem_desc_sw128(pa + (ks / 4) * CHUNK_BYTES + (ks % 4) * 32, 1024, 16),
                     make_smem_desc_sw128(va + ks * (16 * 128), 1024, CHUNK_BYTES), IDESC_PV, (j | ks) != 0 ? 1u : 0u);
        tc_commit(&o_full[g]);
      };
      bool ok = mbar_wait(q_full, 0, abort_flag);
      if (ok) ok = mbar_wait(&k_full[0], 0, abort_flag);
      if (ok) {
        tc_fence_after_sync();
        if (nblk[0] > 0) issue_qk(0, 0);
        if (nblk[1] > 0) issue_qk(1, 0);
        tc_commit(&k_empty[0]);
      }
      // Both groups' events are served in the order they occur: "S(j) has been read" lets Q K^T of block j + 1 go
      // (its K tile permitting), "P(j) is ready" lets P V of block j go (its V tile permitting).  A K / V stage is
      // released when every group that needs the block has issued its product.
      int qk_next[2] = {1, 1};  // block whose Q K^T is issued next (block 0 went out above)
      int pv_next[2] = {0, 0};
      uint32_t qk_half = 0, pv_half = 0;  // bit (j & 3): one of the two groups that need block j has been served
      auto needed = [&](int j) { return (j < nblk[0] ? 1 : 0) + (j < nblk[1] ? 1 : 0); };
      // true when every group that needs block j has been served (the groups never drift 4 blocks apart: a K / V
      // stage is refilled only after both have used it)
      auto all_served = [&](uint32_t& mask, int j) -> bool {
        if (needed(j) == 1) return true;
        const uint32_t bit = 1u << (j & 3);
        mask ^= bit;
        return (mask & bit) == 0;
      };
      uint64_t t_last = global_timer_ns();  // time of the last product issued: the wait for the next event is bounded
      uint32_t spins = 0;
      while (ok && (pv_next[0] < nblk[0] || pv_next[1] < nblk[1])) {
        bool progress = false;
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          const int jn = qk_next[g];
          if (jn < nblk[g] && mbar_try_wait(&s_free[g], (jn - 1) & 1) &&
              mbar_try_wait(&k_full[jn % KV_STAGES], (jn / KV_STAGES) & 1)) {
            tc_fence_after_sync();
            issue_qk(g, jn);
            qk_next[g] = jn + 1;
            if (all_served(qk_half, jn)) tc_commit(&k_empty[jn % KV_STAGES]);  // K(jn) consumed by every group that needs it
            progress = true;
          }
          const int jp = pv_next[g];
          if (jp < nblk[g] && mbar_try_wait(&p_full[g], jp & 1) &&
              mbar_try_wait(&v_full[jp % KV_STAGES], (jp / KV_STAGES) & 1)) {
            // P_g(jp) is in shared memory; O_g has been rescaled if it had to be
            tc_fence_after_sync();
            issue_pv(g, jp);
            pv_next[g] = jp + 1;
            if (all_served(pv_half, jp)) tc_commit(&v_empty[jp % KV_STAGES]);  // V(jp) consumed
            progress = true;
          }
        }
        if (progress) {
          t_last = global_timer_ns();
          spins = 0;
        } else if ((++spins & 0x3f) == 0) {
          if (*abort_flag) ok = false;
          else if (global_timer_ns() - t_last > ZEN_WAIT_LIMIT_NS) {
            *abort_flag = 1;
            record_status(ZEN_ERR_TIMEOUT);
            ok = false;
          }
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax groups
    const int g = (warp - 2) >> 2;
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const int q = q0 + g * 128 + r;
    const uint32_t lane_sel = uint32_t(quad * 32) << 16;
    const uint32_t tmem_s = tmem_base + uint32_t(g * 128);
    const uint32_t tmem_o = tmem_base + uint32_t(256 + g * D);
    uint8_t* myP = sP + g * P_BYTES;
    const int nb = nblk[g];
    float m_ref = -INFINITY;  // the maximum the stored probabilities and O are scaled with (log2 units)
    float l_run = 0.f;
    bool ok = true;

    for (int j = 0; j < nb && ok; ++j) {
      if (!mbar_wait(&s_full[g], j & 1, abort_flag)) { ok = false; break; }
      tc_fence_after_sync();
      const int key0 = j * 128;
      int lim = kv_len - key0;
      if (p.causal && q + 1 - key0 < lim) lim = q + 1 - key0;
      // the whole row of S in registers, in one trip through tensor memory; the S columns are then free for
      // Q K^T of the group's next block
      const bool full_blk = lim >= 128;
      uint32_t sv[4][32];
      __syncwarp();
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32(tmem_s + lane_sel + c * 32, sv[c]);
      tmem_wait_ld();
      tc_fence_before_sync();
      mbar_arrive(&s_free[g]);
      // row maximum of this block (four independent chains; no predicates when the block is entirely valid)
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (full_blk) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sv[c][i]));
      } else {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c * 32 + i < lim) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sv[c][i]));
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      const float m_blk = mx * p.scale_log2;
      // move the reference maximum only when this row has outgrown it by more than the threshold
      const bool grow = m_blk > m_ref + RESCALE_THRESHOLD || (m_ref == -INFINITY && m_blk != -INFINITY);
      const float m_new = grow ? m_blk : m_ref;
      const float alpha = (grow && m_ref != -INFINITY) ? fast_exp2(m_ref - m_new) : 1.0f;
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      if (j > 0) {
        // P V of the previous block has completed: P may be overwritten, O may be rescaled
        if (!mbar_wait(&o_full[g], (j - 1) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        if (__any_sync(0xffffffffu, alpha != 1.0f)) {
          // (16 columns at a time: the row of S occupies most of the thread's registers)
#pragma unroll 1
          for (int c = 0; c < D / 16; ++c) {
            uint32_t ov[16];
            __syncwarp();
            tmem_ld_32x16(tmem_o + lane_sel + c * 16, ov);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 16; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
            tmem_st_32x16(tmem_o + lane_sel + c * 16, ov);
          }
          tmem_wait_st();
          l_run *= alpha;
        }
      }
      m_ref = m_new;
      // probabilities -> shared memory (fp16, swizzled K-major), row sum; column pairs on the packed fp32x2
      // instructions
      float2 rs2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
      const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
      const float2 nm2 = make_float2(-m_use, -m_use);
#pragma unroll
      for (int hc = 0; hc < 8; ++hc) {  // 16 columns (8 pairs, two 16-byte units of the P row) at a time
        const int c = hc >> 1;          // 32-column chunk of S
        uint32_t pk[8];
#pragma unroll
        for (int ii = 0; ii < 8; ++ii) {
          const int i = (hc & 1) * 8 + ii;  // pair within the chunk
          const float2 x = f2fma(make_float2(__uint_as_float(sv[c][2 * i]), __uint_as_float(sv[c][2 * i + 1])), sc2, nm2);
          float2 e = make_float2(fast_exp2(x.x), fast_exp2(x.y));
          if (!full_blk) {
            e.x = (c * 32 + 2 * i < lim) ? e.x : 0.f;
            e.y = (c * 32 + 2 * i + 1 < lim) ? e.y : 0.f;
          }
          rs2[i & 1] = f2add(rs2[i & 1], e);
          const __half2 hh = __floats2half2_rn(e.x, e.y);
          pk[ii] = *reinterpret_cast<const uint32_t*>(&hh);
        }
        uint8_t* prow = myP + (c >> 1) * CHUNK_BYTES + r * 128;
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int unit = ((c & 1) * 4 + (hc & 1) * 2 + u) ^ (r & 7);
          *reinterpret_cast<uint4*>(prow + unit * 16) = make_uint4(pk[4 * u], pk[4 * u + 1], pk[4 * u + 2], pk[4 * u + 3]);
        }
      }
      const float rs4[4] = {rs2[0].x, rs2[0].y, rs2[1].x, rs2[1].y};
      const float rowsum = (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
      l_run += rowsum;
      tc_fence_before_sync();
      fence_proxy_async_smem();
      mbar_arrive(&p_full[g]);
    }

    if (ok && nb > 0) {
      if (!mbar_wait(&o_full[g], (nb - 1) & 1, abort_flag)) ok = false;
      tc_fence_after_sync();
    }
    if (ok) {
      // every lane takes part in the TMEM loads; only rows inside the sequence are stored
      const bool row_ok = q < q_len;
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      const int64_t off = p.cu_seqlens != nullptr ? int64_t(h) * p.o_sh + (int64_t(row_base) + q) * p.o_ss
                                                    : int64_t(b) * p.o_sb + int64_t(h) * p.o_sh + int64_t(q) * p.o_ss;
      __half* orow = static_cast<__half*>(p.o) + off;
      const float inv_o_scale = p.oq ? ZEN_DIV(1.0f, p.o_scale) : 1.0f;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t ov[32];
        __syncwarp();
        if (nb > 0) {
          tmem_ld_32x32(tmem_o + lane_sel + c * 32, ov);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) ov[i] = 0;
        }
        uint32_t w[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const __half2 hh = __floats2half2_rn(__uint_as_float(ov[2 * i]) * inv, __uint_as_float(ov[2 * i + 1]) * inv);
          w[i] = *reinterpret_cast<const uint32_t*>(&hh);
        }
        if (!row_ok) continue;
#pragma unroll
        for (int i = 0; i < 4; ++i)
          reinterpret_cast<uint4*>(orow + c * 32)[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
        if (p.oq) {
          // the int8 copy quantizes the fp16 values that were stored (branch-free rounding, exact
          // division only next to a rounding boundary)
          uint32_t qw[8];
#pragma unroll
          for (int g = 0; g < 2; ++g) {
            float2 val[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) val[e] = __half22float2(*reinterpret_cast<const __half2*>(&w[8 * g + e]));
            uint32_t q4[4];
            const uint32_t risky = quantize_pairs_rn<16>(val, inv_o_scale, q4);
            if (risky) {
#pragma unroll
              for (int e = 0; e < 16; ++e)
                if (risky & (1u << e))
                  patch_q_byte(q4, e, zen_det_round_clamp_i8(ZEN_DIV((e & 1) ? val[e >> 1].y : val[e >> 1].x, p.o_scale), 0));
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) qw[4 * g + e] = q4[e];
          }
          int8_t* qrow = p.oq + off + c * 32;
          reinterpret_cast<uint4*>(qrow)[0] = make_uint4(qw[0], qw[1], qw[2], qw[3]);
          reinterpret_cast<uint4*>(qrow)[1] = make_uint4(qw[4], qw[5], qw[6], qw[7]);
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

}  // namespace zen
