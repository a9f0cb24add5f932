// W8A8 QKV projection + attention in ONE persistent kernel, for sequences of at most 128 tokens and head size 64
// (the encoder's case).  With S <= 128 one 128-row GEMM tile IS one sequence, and the 192 output columns
// {Q_h, K_h, V_h} of one head are everything attention needs for (sequence b, head h).  A work item is therefore
// (b, h):
//
//   acc[128, 192] = xq[b] . {Wq_h, Wk_h, Wv_h}^T                  int8 tcgen05, s32 in TMEM       (GEMM issuer)
//   Q, K, V       = half((float(acc) * s_x) * s_w[n] + bias[n])    written to shared memory as MMA operands
//   S = Q K^T  ->  P = exp2(scale * S - max)  ->  O = P V          as in flash_attn_kernel (same arithmetic)
//   ctx[b, :, h]  = half(O / rowsum)  (+ int8 copy)                TMA stores
//
// so the fp16 QKV tensor never travels to L2 / HBM and back, one kernel boundary and the attention kernel's load
// latency disappear, and the projection of item i + 1 runs under the attention of item i.
//
//   warp 0       TMA producer of the GEMM operand ring
//   warp 1       GEMM MMA issuer (one lane)
//   warps 2, 3   attention MMA issuers (one lane each) for the items of buffer set 0 / 1
//   warps 4..11  work group 0: TWO threads per row (each half of the columns / keys); projection epilogue, softmax,
//                output of the items of set 0.  One thread per row ran its 3000-instruction chain at 0.4 instructions
//                per clock (7 us per item, measured with timestamps); splitting a row over two warps halves it.
//   warps 12..19 work group 1: the same for set 1
// A buffer set = 192 TMEM columns (accumulators, then S over the first 128, O over the last 64) + 48 KB of shared
// memory (Q, K, V tiles; P later overwrites Q + K, the output staging overwrites them again).  Items alternate
// between the sets, so two items are in flight per CTA besides the one whose operands are being loaded.
//
// Results are bit-identical to zen_linear_i8 (fp16 output) followed by zen_flash_attention_f16.
//
// PACKED form (unpadded batches): the valid tokens of all sequences lie back to back, sequence b in rows
// cu_seqlens[b] .. cu_seqlens[b + 1] - 1.  The 128-row activation tile of an item starts at the sequence's first row
// and runs on into its successors' rows (or past the end of the tensor, which reads as zero): those rows are keys
// beyond the key length (masked as padding is) and queries whose outputs are never written, because the outputs go
// from registers to global memory with a row guard instead of through box-shaped TMA stores.
#pragma once
#include "gemm_tc.cuh"

namespace zen {

constexpr int QA_THREADS = 640;
constexpr int QA_WG_THREADS = 256;  // one work group: 8 warps, two per TMEM lane quadrant
constexpr int QA_STAGES = 3;
constexpr int QA_BN = 192;                                    // Q, K, V columns of one head
constexpr int QA_STAGE_BYTES = GEMM_BM * 128 + QA_BN * 128;  // 16 KB of activations + 24 KB of weights per k-block
constexpr int QA_TILE_BYTES = 128 * 128;                     // one Q / K / V tile: 128 rows x 64 fp16
constexpr int QA_SET_BYTES = 3 * QA_TILE_BYTES;

struct QkvAttnParams {
  int B, S, heads, K;  // K: input width of the projection (the hidden size); output width 3 * heads * 64
  int num_k_blocks;
  float x_scale;
  const float* w_scale;  // [3 * heads * 64] or null
  const float* bias;     // [3 * heads * 64] or null
  const int32_t* kv_lens;
  const int32_t* cu_seqlens;  // PACKED: [B + 1] row offsets; the key length of sequence b is their difference
  int rows;                   // PACKED: rows of the packed tensors; offsets beyond it are cut (nothing is stored there)
  __half* ctx;                // PACKED: output rows are written with plain stores (ld = heads * 64)
  float scale_log2;  // softmax scale * log2(e)
  int8_t* ctxq;      // int8 copy of the output (may be null)
  float ctx_scale;
  __half* qkv_out;  // optional fp16 [B * S, 3 * heads * 64] copy of the projection (tests / calibration), may be null
  int o_perm[3];    // position of (seq, head, batch) in the rank-4 output maps
  const uint8_t* pf_ptr[2];
  uint64_t pf_bytes[2];
  int early_b;
};

constexpr size_t qkv_attn_smem_bytes() {
  // ring + two buffer sets + scale / bias rows (2 sets x 2 x 192 floats) + row maxima and sums exchanged between the
  // two threads of a row (2 sets x 5 x 128 floats) + barriers and flags + alignment slack
  return size_t(QA_STAGES) * QA_STAGE_BYTES + 2 * size_t(QA_SET_BYTES) + 2 * 2 * QA_BN * 4 + 2 * 5 * 128 * 4 + 512 + 1024;
}

__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

template <bool PACKED>
__global__ void __launch_bounds__(QA_THREADS, 1)
qkv_attn_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                const __grid_constant__ CUtensorMap tmap_o, const __grid_constant__ CUtensorMap tmap_oq,
                const QkvAttnParams p) {
  constexpr int BK = 128, UK = 32;  // int8: 128 elements per swizzle row, 32 per MMA
  constexpr int A_BYTES = GEMM_BM * 128;
  constexpr uint32_t TMEM_COLS = 512;  // 2 x 192 used
  constexpr uint32_t IDESC_PROJ = make_idesc(IDESC_C_S32, IDESC_S8, IDESC_S8, 0, 0, GEMM_BM, QA_BN);
  constexpr uint32_t IDESC_QK = make_idesc(IDESC_C_F32, IDESC_F16, IDESC_F16, 0, 0, 128, 128);
  constexpr uint32_t IDESC_PV = make_idesc(IDESC_C_F32, IDESC_F16, IDESC_F16, 0, 1, 128, 64);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* sets = smem + size_t(QA_STAGES) * QA_STAGE_BYTES;  // [2][Q | K | V], 1024-byte aligned
  float* col_rows = reinterpret_cast<float*>(sets + 2 * QA_SET_BYTES);  // [2 sets][scale 192 | bias 192]
  float* xch = col_rows + 2 * 2 * QA_BN;                                // [2 sets][max half 0 | max half 1 | sums x 3][128 rows]
  uint8_t* ctrl = reinterpret_cast<uint8_t*>(xch + 2 * 5 * 128);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(ctrl);
  uint64_t* empty_bar = full_bar + QA_STAGES;
  uint64_t* acc_full = empty_bar + QA_STAGES;  // [2] projection accumulators of the set are complete
  uint64_t* acc_empty = acc_full + 2;          // [2] the work group has finished with the set's TMEM columns
  uint64_t* qkv_ready = acc_empty + 2;         // [2] Q, K, V of the set are in shared memory
  uint64_t* s_full = qkv_ready + 2;            // [2] S = Q K^T is complete
  uint64_t* p_ready = s_full + 2;              // [2] P is in shared memory and S has been read
  uint64_t* o_full = p_ready + 2;              // [2] O = P V is complete
  uint64_t* wg_bar = o_full + 2;               // [2] work-group-wide rendezvous (a bounded wait, unlike bar.sync)
  uint64_t* pair_bar = wg_bar + 2;             // [2 sets][4 quadrants][3 uses per item] the two warps that share 32 rows
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pair_bar + 24);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int items = p.B * p.heads;
  const int nkb = p.num_k_blocks;
  const int hidden = p.heads * 64;
  // items of this CTA: blockIdx.x + j * gridDim.x, j = 0 .. n_mine - 1; item -> (sequence, head), heads fastest,
  // so that neighbouring CTAs read the same activation rows at the same time
  const int n_mine = int(blockIdx.x) < items ? (items - 1 - int(blockIdx.x)) / int(gridDim.x) + 1 : 0;
  // first row of sequence b in a packed batch; key length of sequence b (clamped to what one tile holds)
  auto first_row = [&](int b) -> int { return PACKED ? p.cu_seqlens[b] : b * p.S; };
  auto key_len = [&](int b) -> int {
    int n = p.S;
    if (PACKED) {
      // a sequence that runs past the end of the packed tensors (offsets that exceed the row capacity) is cut there
      const int lo = p.cu_seqlens[b], hi = p.cu_seqlens[b + 1];
      n = lo < 0 ? 0 : (hi < p.rows ? hi : p.rows) - lo;
    } else if (p.kv_lens) {
      n = p.kv_lens[b];
    }
    return n < 0 ? 0 : (n > p.S ? p.S : n);
  };

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    if (!PACKED) {
      tma_prefetch_desc(&tmap_o);
      if (p.ctxq) tma_prefetch_desc(&tmap_oq);
    }
    for (int i = 0; i < QA_STAGES; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], QA_WG_THREADS);
      mbar_init(&qkv_ready[i], QA_WG_THREADS);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_ready[i], QA_WG_THREADS);
      mbar_init(&o_full[i], 1);
      mbar_init(&wg_bar[i], QA_WG_THREADS);
    }
    for (int i = 0; i < 24; ++i) mbar_init(&pair_bar[i], 64);
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
#pragma unroll
    for (int i = 0; i < 2; ++i)
      if (p.pf_bytes[i] != 0) prefetch_slice_l2(p.pf_ptr[i], p.pf_bytes[i], blockIdx.x, gridDim.x);
  }
  grid_launch_dependents();
  // constant weights: the weight tiles of the first item's first k-blocks are requested before the dependency wait
  int pre = 0;
  if (threadIdx.x == 0 && p.early_b && n_mine > 0) {
    const int h = int(blockIdx.x) % p.heads;
    pre = nkb < QA_STAGES ? nkb : QA_STAGES;
    for (int kb = 0; kb < pre; ++kb) {
      mbar_arrive_expect_tx(&full_bar[kb], QA_STAGE_BYTES);
      uint8_t* sb = smem + size_t(kb) * QA_STAGE_BYTES + A_BYTES;
#pragma unroll
      for (int t = 0; t < 3; ++t) tma_load_2d(sb + t * (64 * 128), &tmap_b, &full_bar[kb], kb * BK, t * hidden + h * 64);
    }
  }
  grid_dependency_wait();  // activations, key lengths and output buffers may belong to the previous kernel until here

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int j = 0; j < n_mine && ok; ++j) {
        const int item = int(blockIdx.x) + j * int(gridDim.x);
        const int b = item / p.heads, h = item % p.heads;
        const int row0 = PACKED ? first_row(b) : 0;
        auto load_a = [&](uint8_t* dst, uint64_t* bar, int kb) {
          if (PACKED) tma_load_2d(dst, &tmap_a, bar, kb * BK, row0);
          else tma_load_3d(dst, &tmap_a, bar, kb * BK, 0, b);
        };
        for (int kb = 0; kb < nkb; ++kb) {
          uint8_t* sa = smem + size_t(stage) * QA_STAGE_BYTES;
          if (j == 0 && kb < pre) {
            load_a(sa, &full_bar[stage], kb);
          } else {
            if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) {
              ok = false;
              break;
            }
            mbar_arrive_expect_tx(&full_bar[stage], QA_STAGE_BYTES);
            load_a(sa, &full_bar[stage], kb);
#pragma unroll
            for (int t = 0; t < 3; ++t)
              tma_load_2d(sa + A_BYTES + t * (64 * 128), &tmap_b, &full_bar[stage], kb * BK, t * hidden + h * 64);
          }
          if (++stage == QA_STAGES) {
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
    // ------------------------------------------------------------------ projection MMA issuer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int j = 0; j < n_mine && ok; ++j) {
        const int set = j & 1;
        const uint32_t it = uint32_t(j >> 1);
        if (!mbar_wait(&acc_empty[set], (it & 1u) ^ 1u, abort_flag)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + uint32_t(set * QA_BN);
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smem + size_t(stage) * QA_STAGE_BYTES);
          const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UK; ++k)
            mma_i8_ss(d_tmem, make_smem_desc_sw128(a_addr + k * 32, 1024, 16), make_smem_desc_sw128(b_addr + k * 32, 1024, 16),
                      IDESC_PROJ, (kb | k) != 0 ? 1u : 0u);
          tc_commit(&empty_bar[stage]);
          if (++stage == QA_STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) tc_commit(&acc_full[set]);
      }
    }
  } else if (warp < 4) {
    // ------------------------------------------------------------------ attention MMA issuer of one buffer set
    if (lane == 0) {
      const int set = warp - 2;
      const uint32_t region = tmem_base + uint32_t(set * QA_BN);
      const uint32_t qa = smem_u32(sets + size_t(set) * QA_SET_BYTES);
      const uint32_t ka = qa + QA_TILE_BYTES;
      const uint32_t va = ka + QA_TILE_BYTES;
      uint32_t it = 0;
      for (int j = set; j < n_mine; j += 2, ++it) {
        const int item = int(blockIdx.x) + j * int(gridDim.x);
        const int kv_len = key_len(item / p.heads);
        const int k_cols = ((kv_len + 15) / 16) * 16;
        if (!mbar_wait(&qkv_ready[set], it & 1u, abort_flag)) break;
        tc_fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          mma_f16_ss(region, make_smem_desc_sw128(qa + ks * 32, 1024, 16), make_smem_desc_sw128(ka + ks * 32, 1024, 16), IDESC_QK,
                     ks != 0 ? 1u : 0u);
        tc_commit(&s_full[set]);
        if (!mbar_wait(&p_ready[set], it & 1u, abort_flag)) break;
        tc_fence_after_sync();
        // keys at and beyond kv_len carry no probability mass: only the 16-key steps below it are multiplied
#pragma unroll 1
        for (int ks = 0; ks < k_cols / 16; ++ks)
          mma_f16_ss(region + 128u, make_smem_desc_sw128(qa + (ks / 4) * QA_TILE_BYTES + (ks % 4) * 32, 1024, 16),
                     make_smem_desc_sw128(va + ks * (16 * 128), 1024, QA_TILE_BYTES), IDESC_PV, ks != 0 ? 1u : 0u);
        tc_commit(&o_full[set]);
      }
    }
  } else {
    // ------------------------------------------------------------------ work groups: two threads per row
    const int wgw = warp - 4;          // 0 .. 15
    const int set = wgw >> 3;
    const int half = (wgw >> 2) & 1;   // which half of the row's columns / keys this thread handles
    const int quad = warp & 3;         // TMEM lane quadrant (== wgw & 3)
    const int r = quad * 32 + lane;    // row of the tile == TMEM lane == token of the sequence
    const uint32_t lane_sel = uint32_t(quad * 32) << 16;
    const uint32_t region = tmem_base + lane_sel + uint32_t(set * QA_BN);
    uint8_t* sQ = sets + size_t(set) * QA_SET_BYTES;
    uint8_t* sK = sQ + QA_TILE_BYTES;
    float* s_scale = col_rows + set * 2 * QA_BN;
    float* s_bias = s_scale + QA_BN;
    float* x_max = xch + set * 5 * 128;  // [2 halves][128]
    float* x_sum = x_max + 2 * 128;      // [3][128]: half 0's two chunks added, half 1's chunk 2, half 1's chunk 3
    uint64_t* my_pair = pair_bar + (set * 4 + quad) * 3;
    const int gt = int(threadIdx.x) - 128 - set * QA_WG_THREADS;  // 0 .. 255 within the work group
    const float inv_o_scale = p.ctxq ? ZEN_DIV(1.0f, p.ctx_scale) : 1.0f;
    const float2 xs2 = make_float2(p.x_scale, p.x_scale);
    uint32_t it = 0;
    for (int j = set; j < n_mine; j += 2, ++it) {
      const int item = int(blockIdx.x) + j * int(gridDim.x);
      const int b = item / p.heads, h = item % p.heads;
      const int kv_len = key_len(b);
      if (PACKED && gt == 0 && p.cu_seqlens[b + 1] - p.cu_seqlens[b] > p.S) record_status(ZEN_ERR_UNSUPPORTED);  // longer than a tile
      const int64_t grow = int64_t(first_row(b)) + r;  // this thread's row of the global tensors
      const bool row_live = PACKED ? r < kv_len : r < p.S;
      const int k_cols = ((kv_len + 15) / 16) * 16;
      // Per-column scale and bias of this head's 192 columns (thread gt < 192: column gt).  The rows can be
      // rewritten at once: no thread is still reading the previous item's (its Q K^T product needed every
      // thread's arrival after the projection epilogue, and this thread has waited for that product).
      {
        if (gt < QA_BN) {
          const int c = (gt >> 6) * hidden + h * 64 + (gt & 63);
          s_scale[gt] = p.w_scale != nullptr ? __ldg(p.w_scale + c) : 1.0f;
          s_bias[gt] = p.bias != nullptr ? __ldg(p.bias + c) : 0.0f;
        }
        // the previous item of this set: its stores (issued by lane 0 of the half-0 warps) have finished reading
        // the staging rows of the Q / K tiles before any thread of the group writes Q / K / P rows again
        if (!PACKED && half == 0 && lane == 0) tma_store_wait_read();
        mbar_arrive(&wg_bar[set]);
        if (!mbar_wait(&wg_bar[set], it & 1u, abort_flag)) break;
      }
      // ---- projection epilogue: this thread's 96 of the row's 192 accumulators -> fp16 Q, K, V in shared memory
      if (!mbar_wait(&acc_full[set], it & 1u, abort_flag)) break;
      tc_fence_after_sync();
#pragma unroll 1
      for (int k = 0; k < 6; ++k) {
        const int i = half * 6 + k;  // 16-column step of the row: tile i / 4 (Q, K, V), units 2 (i % 4) and + 1
        uint32_t a[16];
        __syncwarp();
        tmem_ld_32x16(region + uint32_t(i * 16), a);
        tmem_wait_ld();
        uint32_t w[8];
#pragma unroll
        for (int j4 = 0; j4 < 4; ++j4) {
          const float4 s4 = reinterpret_cast<const float4*>(s_scale + i * 16)[j4];
          const float4 b4 = reinterpret_cast<const float4*>(s_bias + i * 16)[j4];
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            const int e = 4 * j4 + 2 * hh;
            const float2 av = make_float2(float(int32_t(a[e])), float(int32_t(a[e + 1])));
            // zen_det_dequant on a column pair: each product rounded before the bias is added
            const float2 v = f2mul_then_add(f2mul(av, xs2), hh ? make_float2(s4.z, s4.w) : make_float2(s4.x, s4.y),
                                            hh ? make_float2(b4.z, b4.w) : make_float2(b4.x, b4.y));
            const __half2 hv = __floats2half2_rn(v.x, v.y);
            w[e >> 1] = *reinterpret_cast<const uint32_t*>(&hv);
          }
        }
        uint8_t* trow = sQ + (i >> 2) * QA_TILE_BYTES + r * 128;  // 128-byte swizzle
        *reinterpret_cast<uint4*>(trow + (((2 * (i & 3)) ^ (r & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
        *reinterpret_cast<uint4*>(trow + (((2 * (i & 3) + 1) ^ (r & 7)) << 4)) = make_uint4(w[4], w[5], w[6], w[7]);
        if (p.qkv_out != nullptr && row_live) {
          uint4* dst = reinterpret_cast<uint4*>(p.qkv_out + grow * (3 * hidden) + (i >> 2) * hidden + h * 64 + (i & 3) * 16);
          dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
          dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
        }
      }
      tc_fence_before_sync();
      fence_proxy_async_smem();
      mbar_arrive(&qkv_ready[set]);

      // ---- softmax (the arithmetic of flash_attn_kernel): this thread's 64 of the row's 128 keys
      if (!mbar_wait(&s_full[set], it & 1u, abort_flag)) break;
      tc_fence_after_sync();
      const int lim = kv_len;
      float mx = -INFINITY;
#pragma unroll 1
      for (int cc = 0; cc < 2; ++cc) {
        const int c = 2 * half + cc;
        const int rem = lim - c * 32;
        if (rem <= 0) break;  // uniform: the key length is the same for every row of the sequence
        uint32_t sv[32];
        __syncwarp();
        tmem_ld_32x32(region + uint32_t(c * 32), sv);
        tmem_wait_ld();
        if (rem >= 32) {
#pragma unroll
          for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(sv[i]));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (i < rem) mx = fmaxf(mx, __uint_as_float(sv[i]));
        }
      }
      x_max[half * 128 + r] = mx;
      mbar_arrive(&my_pair[0]);
      if (!mbar_wait(&my_pair[0], it & 1u, abort_flag)) break;
      mx = fmaxf(mx, x_max[(half ^ 1) * 128 + r]);  // the row maximum over all valid keys, as one thread would find it
      const float m_use = mx == -INFINITY ? 0.f : mx * p.scale_log2;
      float csum[2] = {0.f, 0.f};  // this thread's two 32-key chunks
#pragma unroll 1
      for (int cc = 0; cc < 2; ++cc) {
        const int c = 2 * half + cc;
        if (c * 32 >= k_cols) break;
        const int rem = lim - c * 32;
        uint32_t pk[16];
        if (rem <= 0) {
#pragma unroll
          for (int i = 0; i < 16; ++i) pk[i] = 0u;
        } else {
          uint32_t sv[32];
          __syncwarp();
          tmem_ld_32x32(region + uint32_t(c * 32), sv);
          tmem_wait_ld();
          float rs0 = 0.f, rs1 = 0.f;
          if (rem >= 32) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float e0 = fast_exp2(fmaf(__uint_as_float(sv[2 * i]), p.scale_log2, -m_use));
              const float e1 = fast_exp2(fmaf(__uint_as_float(sv[2 * i + 1]), p.scale_log2, -m_use));
              rs0 += e0;
              rs1 += e1;
              const __half2 hv = __floats2half2_rn(e0, e1);
              pk[i] = *reinterpret_cast<const uint32_t*>(&hv);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float e0 = (2 * i < rem) ? fast_exp2(fmaf(__uint_as_float(sv[2 * i]), p.scale_log2, -m_use)) : 0.f;
              const float e1 = (2 * i + 1 < rem) ? fast_exp2(fmaf(__uint_as_float(sv[2 * i + 1]), p.scale_log2, -m_use)) : 0.f;
              rs0 += e0;
              rs1 += e1;
              const __half2 hv = __floats2half2_rn(e0, e1);
              pk[i] = *reinterpret_cast<const uint32_t*>(&hv);
            }
          }
          csum[cc] = rs0 + rs1;
        }
        // P[row, 32 keys of chunk c]: the Q tile holds keys 0..63, the K tile keys 64..127 (both dead by now)
        uint8_t* prow = sQ + (c >> 1) * QA_TILE_BYTES + r * 128;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int unit = ((c & 1) * 4 + u) ^ (r & 7);
          *reinterpret_cast<uint4*>(prow + unit * 16) = make_uint4(pk[4 * u], pk[4 * u + 1], pk[4 * u + 2], pk[4 * u + 3]);
        }
      }
      // The row sum in the order one thread would add it, ((c0 + c1) + c2) + c3: half 0 publishes c0 + c1, half 1
      // its two chunks separately (a chunk without valid keys is 0; adding 0 changes nothing).
      if (half == 0) {
        x_sum[r] = csum[0] + csum[1];
      } else {
        x_sum[128 + r] = csum[0];
        x_sum[256 + r] = csum[1];
      }
      tc_fence_before_sync();
      fence_proxy_async_smem();
      mbar_arrive(&p_ready[set]);
      mbar_arrive(&my_pair[1]);

      // ---- output: O / rowsum -> fp16 (+ int8 copy) for this thread's 32 of the 64 columns, staged in the rows of
      //      the Q / K tiles that belong to this pair of warps
      if (!mbar_wait(&o_full[set], it & 1u, abort_flag)) break;
      tc_fence_after_sync();
      if (!mbar_wait(&my_pair[1], it & 1u, abort_flag)) break;
      const float l_sum = (x_sum[r] + x_sum[128 + r]) + x_sum[256 + r];
      const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
      uint8_t* sty = sQ + quad * 4096;  // 32 rows x 128 B, 128-byte swizzle
      uint8_t* stq = sK + quad * 4096;  // 32 rows x 64 B, 64-byte swizzle
#pragma unroll 1
      for (int k = 0; k < 2; ++k) {
        const int g = 2 * half + k;  // 16-column step of the output row
        uint32_t ov[16];
        if (kv_len > 0) {
          __syncwarp();
          tmem_ld_32x16(region + 128u + uint32_t(g * 16), ov);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) ov[i] = 0u;  // a sequence without keys yields zeros
        }
        uint32_t w[8];
        float2 val[8];  // the fp16 values that are stored: the int8 copy quantizes these
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const __half2 hv = __floats2half2_rn(__uint_as_float(ov[2 * i]) * inv, __uint_as_float(ov[2 * i + 1]) * inv);
          w[i] = *reinterpret_cast<const uint32_t*>(&hv);
          val[i] = __half22float2(hv);
        }
        uint8_t* srow = sty + lane * 128;
        *reinterpret_cast<uint4*>(srow + (((2 * g) ^ (lane & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
        *reinterpret_cast<uint4*>(srow + (((2 * g + 1) ^ (lane & 7)) << 4)) = make_uint4(w[4], w[5], w[6], w[7]);
        if (p.ctxq) {
          uint32_t qw[4];
          const uint32_t risky = quantize_pairs_rn<16>(val, inv_o_scale, qw);
          if (risky) {
#pragma unroll
            for (int e = 0; e < 16; ++e)
              if (risky & (1u << e))
                patch_q_byte(qw, e, zen_det_round_clamp_i8(ZEN_DIV((e & 1) ? val[e >> 1].y : val[e >> 1].x, p.ctx_scale), 0));
          }
          *reinterpret_cast<uint4*>(stq + lane * 64 + ((g ^ ((lane >> 1) & 3)) << 4)) = make_uint4(qw[0], qw[1], qw[2], qw[3]);
        }
      }
      tc_fence_before_sync();
      mbar_arrive(&acc_empty[set]);  // the set's TMEM columns may receive the next projection
      fence_proxy_async_smem();      // this thread's staged bytes -> visible to the TMA engine
      mbar_arrive(&my_pair[2]);
      if (half == 0) {
        // both warps of the pair have staged their halves of the 32 rows
        if (!mbar_wait(&my_pair[2], it & 1u, abort_flag)) break;
        if (PACKED) {
          // Box-shaped stores would write the rows of the next sequence: the valid rows leave with plain stores,
          // consecutive lanes taking consecutive 16-byte pieces of a row (whole 128-byte lines per row).
          const int live = kv_len - quad * 32;  // rows of this quadrant that belong to the sequence
          const int64_t base_row = int64_t(first_row(b)) + quad * 32;
#pragma unroll 2
          for (int idx = lane; idx < 32 * 8; idx += 32) {
            const int rw = idx >> 3, c = idx & 7;
            if (rw < live)
              *(reinterpret_cast<uint4*>(p.ctx + (base_row + rw) * hidden + h * 64) + c) =
                  *reinterpret_cast<const uint4*>(sty + rw * 128 + ((c ^ (rw & 7)) << 4));
          }
          if (p.ctxq) {
#pragma unroll 2
            for (int idx = lane; idx < 32 * 4; idx += 32) {
              const int rw = idx >> 2, c = idx & 3;
              if (rw < live)
                *(reinterpret_cast<uint4*>(p.ctxq + (base_row + rw) * hidden + h * 64) + c) =
                    *reinterpret_cast<const uint4*>(stq + rw * 64 + ((c ^ ((rw >> 1) & 3)) << 4));
            }
          }
        } else if (lane == 0 && quad * 32 < p.S) {
          int c[4];
          c[0] = 0;
          c[p.o_perm[0]] = quad * 32;
          c[p.o_perm[1]] = h;
          c[p.o_perm[2]] = b;
          tma_store_4d(&tmap_o, sty, 0, c[1], c[2], c[3]);
          if (p.ctxq) tma_store_4d(&tmap_oq, stq, 0, c[1], c[2], c[3]);
          tma_store_commit();
        }
      }
    }
    if (!PACKED && half == 0 && lane == 0) tma_store_wait_all();
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

}  // namespace zen
