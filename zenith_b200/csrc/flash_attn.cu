// Flash-attention forward for sm_100a: O = softmax(scale * Q K^T [key-padding / causal mask]) V.
// fp16 operands, fp32 accumulation.  Two kernels:
//   * flash_attn_kernel (this file): sequences of at most 128 keys, one CTA per (head, batch):
//       warp 0      : TMA producer - the Q, K and V tiles
//       warp 1      : TMEM owner and tcgen05.mma issuer:  S = Q K^T (kind::f16, K-major x K-major),
//                     O = P V (A = P from shared memory, B = V as an MN-major operand, so V is
//                     consumed in its natural [key, d] layout without a transpose)
//       warps 2..5  : one thread per query row: tcgen05.ld of S, softmax in registers (exp2 with the
//                     scale folded in), P written to shared memory as fp16 in the 128-byte-swizzled
//                     K-major layout, 1/l normalisation of O, outputs staged and sent by TMA stores.
//   * flash_attn_pipe_kernel (flash_attn_pipe.cuh): longer sequences, two query tiles per CTA with
//     an online softmax.
//
// Q, K, V, O are addressed through (batch, head, seq) strides with d contiguous, so both the
// reference's [B, heads, S, d] tensors and column slices of a fused [tokens, 3*hidden] QKV
// projection are read in place by rank-4 tensor maps.  Rows / keys beyond S read as zero.
#include "zen_common.cuh"
#include "det_math.h"
#include "tma_host.cuh"

namespace zen {

constexpr int FA_BQ = 128;
constexpr int FA_BKV = 128;
constexpr int FA_THREADS = 192;

struct FaParams {
  void* o;
  int8_t* oq;
  float o_scale;
  int B, H, S;
  int64_t o_sb, o_sh, o_ss;
  const int32_t* kv_lens;
  const int32_t* cu_seqlens;  // unpadded batches (long-sequence kernel only): [B + 1] row offsets, null otherwise
  int rows;                   // ... rows of the packed tensors
  int causal;
  float scale_log2;  // softmax scale * log2(e)
  // position of the (seq, head, batch) coordinates in each rank-4 tensor map (dim 0 is d)
  int q_perm[3], k_perm[3], v_perm[3];
  int o_perm[3];  // the same for the output maps of the single-block kernel (o and its int8 copy share strides)
};

template <int D>
constexpr size_t fa_smem_bytes() {
  // Q, K, V tiles (128 x D fp16 each; P later reuses Q + K, the output staging reuses them again)
  // + control + alignment slack
  return size_t(3) * FA_BQ * D * 2 + 256 + 1024;
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void fa_tma_tile(uint8_t* dst, const CUtensorMap* map, uint64_t* bar, const int (&perm)[3],
                                            int d0, int s, int h, int b) {
  int c[4];
  c[0] = d0;
  c[perm[0]] = s;
  c[perm[1]] = h;
  c[perm[2]] = b;
  tma_load_4d(dst, map, bar, c[0], c[1], c[2], c[3]);
}

}  // namespace zen
#include "flash_attn_pipe.cuh"
#include "qkv_attn.cuh"
namespace zen {

// Sequences of at most one key block (S <= 128, the encoder's case).  P reuses the Q / K tiles and
// O reuses the TMEM columns of S, so that four CTAs fit on an SM (one wave for 32 x 12 heads on 148
// SMs) and one CTA's softmax overlaps the others' loads and MMAs.  Every CTA executes its code once,
// so the kernel is as much bound by instruction fetch as by anything else: all per-column work sits
// in rolled loops over 32- or 16-column chunks.
template <int D>
__global__ void __launch_bounds__(FA_THREADS, D == 64 ? 4 : 1)
flash_attn_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                  const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_o,
                  const __grid_constant__ CUtensorMap tmap_oq, const FaParams p) {
  constexpr int DC = D / 64;                 // 128-byte column chunks per row
  constexpr int TILE_BYTES = FA_BQ * D * 2;  // one Q / K / V tile
  constexpr int CHUNK_BYTES = FA_BQ * 128;   // one 64-column chunk of a tile
  constexpr uint32_t TMEM_COLS = 128;        // S: 128 columns; O: its first D columns once P is in shared memory
  constexpr uint32_t IDESC_QK = make_idesc(IDESC_C_F32, IDESC_F16, IDESC_F16, 0, 0, FA_BQ, FA_BKV);
  constexpr uint32_t IDESC_PV = make_idesc(IDESC_C_F32, IDESC_F16, IDESC_F16, 0, 1, FA_BQ, D);
  static_assert(2 * TILE_BYTES >= FA_BQ * FA_BKV * 2, "P must fit in the Q + K tiles");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + TILE_BYTES;
  uint8_t* sV = sK + TILE_BYTES;
  uint8_t* sP = sQ;  // 2 chunks of 64 keys
  uint8_t* ctrl = sV + TILE_BYTES;
  uint64_t* qk_full = reinterpret_cast<uint64_t*>(ctrl);
  uint64_t* v_full = qk_full + 1;
  uint64_t* s_full = v_full + 1;
  uint64_t* p_full = s_full + 1;
  uint64_t* o_full = p_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * FA_BQ;  // 0: the grid has one query tile
  const int h = blockIdx.y;
  const int b = blockIdx.z;

  // The key length may be produced by the kernel ahead in the stream.  When this kernel family is launched
  // with programmatic dependent launch it is therefore read after the dependency wait; otherwise the launch
  // itself orders it and the load is issued here, where the set-up below hides its latency.
  int kv_len = p.S;
  if constexpr (!kAttentionLaunchesEarly) {
    if (p.kv_lens) kv_len = p.kv_lens[b];
  }

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
    tma_prefetch_desc(&tmap_o);
    if (p.oq) tma_prefetch_desc(&tmap_oq);
    mbar_init(qk_full, 1);
    mbar_init(v_full, 1);
    mbar_init(s_full, 1);
    mbar_init(p_full, 128);
    mbar_init(o_full, 1);
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
  const uint32_t tmem_s = *tmem_slot;
  const uint32_t tmem_o = tmem_s;
  grid_launch_dependents();
  grid_dependency_wait();  // Q, K, V and the output buffers may belong to the previous kernel until here
  if constexpr (kAttentionLaunchesEarly) {
    if (p.kv_lens) kv_len = p.kv_lens[b];
  }
  kv_len = kv_len < 0 ? 0 : (kv_len > p.S ? p.S : kv_len);
  int kv_end = kv_len;
  if (p.causal && q0 + FA_BQ < kv_end) kv_end = q0 + FA_BQ;
  const bool any_keys = kv_end > 0;
  const int k_cols = ((min(kv_end, FA_BKV) + 15) / 16) * 16;  // columns of P the P V product reads

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0 && any_keys) {
      mbar_arrive_expect_tx(qk_full, 2 * TILE_BYTES);
#pragma unroll
      for (int dc = 0; dc < DC; ++dc) {
        fa_tma_tile(sQ + dc * CHUNK_BYTES, &tmap_q, qk_full, p.q_perm, dc * 64, q0, h, b);
        fa_tma_tile(sK + dc * CHUNK_BYTES, &tmap_k, qk_full, p.k_perm, dc * 64, 0, h, b);
      }
      mbar_arrive_expect_tx(v_full, TILE_BYTES);
#pragma unroll
      for (int dc = 0; dc < DC; ++dc) fa_tma_tile(sV + dc * CHUNK_BYTES, &tmap_v, v_full, p.v_perm, dc * 64, 0, h, b);
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0 && any_keys) {
      bool ok = mbar_wait(qk_full, 0, abort_flag);
      if (ok) {
        tc_fence_after_sync();
        const uint32_t qa = smem_u32(sQ);
        const uint32_t ka = smem_u32(sK);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = (ks / 4) * CHUNK_BYTES + (ks % 4) * 32;
          mma_f16_ss(tmem_s, make_smem_desc_sw128(qa + off, 1024, 16), make_smem_desc_sw128(ka + off, 1024, 16),
                     IDESC_QK, ks != 0 ? 1u : 0u);
        }
        tc_commit(s_full);
        // P is in shared memory and S has been read by every softmax thread
        ok = mbar_wait(p_full, 0, abort_flag) && mbar_wait(v_full, 0, abort_flag);
      }
      if (ok) {
        tc_fence_after_sync();
        const uint32_t pa = smem_u32(sP);
        const uint32_t va = smem_u32(sV);
        // keys at and beyond kv_end carry no probability mass: only the 16-key steps below it are
        // multiplied (the softmax warps do not write the columns of P beyond them)
#pragma unroll 1
        for (int ks = 0; ks < k_cols / 16; ++ks) {
          const uint64_t a_desc = make_smem_desc_sw128(pa + (ks / 4) * CHUNK_BYTES + (ks % 4) * 32, 1024, 16);
          const uint64_t b_desc = make_smem_desc_sw128(va + ks * (16 * 128), 1024, CHUNK_BYTES);
          mma_f16_ss(tmem_o, a_desc, b_desc, IDESC_PV, ks != 0 ? 1u : 0u);
        }
        tc_commit(o_full);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax, normalisation, output
    const int quad = warp & 3;
    const int r = quad * 32 + lane;  // row within the query tile == TMEM lane
    const int q = q0 + r;
    const uint32_t lane_sel = uint32_t(quad * 32) << 16;
    float l_sum = 0.f;
    bool ok = true;

    if (any_keys) {
      ok = mbar_wait(s_full, 0, abort_flag);
      tc_fence_after_sync();
      int lim = kv_len;  // keys [0, lim) are valid for this row
      if (p.causal && q + 1 < lim) lim = q + 1;
      // Masking is decided per 32-key chunk and per warp: a chunk whose keys are valid for all 32 rows
      // runs without per-element tests, one that is valid for none is skipped (or zero-filled when the
      // P V product still reads it for other rows' sake), only a chunk that holds a boundary tests each key.
      // pass 1: row maximum
      float mx = -INFINITY;
      if (__all_sync(0xffffffffu, ok)) {
#pragma unroll 1
        for (int c = 0; c < FA_BKV / 32; ++c) {
          const int rem = lim - c * 32;
          if (__all_sync(0xffffffffu, rem <= 0)) break;  // the valid keys are a prefix: later chunks are empty too
          uint32_t sv[32];
          __syncwarp();
          tmem_ld_32x32(tmem_s + lane_sel + c * 32, sv);
          tmem_wait_ld();
          if (__all_sync(0xffffffffu, rem >= 32)) {
#pragma unroll
            for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(sv[i]));
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (i < rem) mx = fmaxf(mx, __uint_as_float(sv[i]));
          }
        }
        const float m_use = mx == -INFINITY ? 0.f : mx * p.scale_log2;
        // pass 2: probabilities -> shared memory (fp16, swizzled K-major), row sum
#pragma unroll 1
        for (int c = 0; c < FA_BKV / 32; ++c) {
          if (c * 32 >= k_cols) break;
          const int rem = lim - c * 32;
          uint32_t pk[16];
          if (__all_sync(0xffffffffu, rem <= 0)) {
#pragma unroll
            for (int i = 0; i < 16; ++i) pk[i] = 0u;
          } else {
            uint32_t sv[32];
            __syncwarp();
            tmem_ld_32x32(tmem_s + lane_sel + c * 32, sv);
            tmem_wait_ld();
            float rs0 = 0.f, rs1 = 0.f;
            if (__all_sync(0xffffffffu, rem >= 32)) {
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                const float a = fast_exp2(fmaf(__uint_as_float(sv[2 * i]), p.scale_log2, -m_use));
                const float bq = fast_exp2(fmaf(__uint_as_float(sv[2 * i + 1]), p.scale_log2, -m_use));
                rs0 += a;
                rs1 += bq;
                const __half2 hh = __floats2half2_rn(a, bq);
                pk[i] = *reinterpret_cast<const uint32_t*>(&hh);
              }
            } else {
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                const float a = (2 * i < rem) ? fast_exp2(fmaf(__uint_as_float(sv[2 * i]), p.scale_log2, -m_use)) : 0.f;
                const float bq = (2 * i + 1 < rem) ? fast_exp2(fmaf(__uint_as_float(sv[2 * i + 1]), p.scale_log2, -m_use)) : 0.f;
                rs0 += a;
                rs1 += bq;
                const __half2 hh = __floats2half2_rn(a, bq);
                pk[i] = *reinterpret_cast<const uint32_t*>(&hh);
              }
            }
            l_sum += rs0 + rs1;
          }
          uint8_t* prow = sP + (c >> 1) * CHUNK_BYTES + r * 128;
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int unit = ((c & 1) * 4 + u) ^ (r & 7);
            *reinterpret_cast<uint4*>(prow + unit * 16) = make_uint4(pk[4 * u], pk[4 * u + 1], pk[4 * u + 2], pk[4 * u + 3]);
          }
        }
        tc_fence_before_sync();
        fence_proxy_async_smem();
        mbar_arrive(p_full);
        ok = mbar_wait(o_full, 0, abort_flag);
        tc_fence_after_sync();
      }
    }

    // Output: every warp stages its 32 rows in shared memory (the Q / K tiles are dead once the P V
    // product has completed) in the swizzled layouts of the output tensor maps and one lane sends them
    // with TMA stores; rows beyond S are clipped by the map.  (Per-thread row stores - 32 different
    // 128-byte lines per instruction - took 4 of this kernel's 10 microseconds.)  A sequence without
    // keys stores zeros.
    if (__all_sync(0xffffffffu, ok)) {
      const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
      const float inv_o_scale = p.oq ? ZEN_DIV(1.0f, p.o_scale) : 1.0f;
      uint8_t* sty = sQ + quad * 4096;  // [dc][4 warps][32 rows x 128 B], 128-byte swizzle
      uint8_t* stq = sK + quad * 2048;  // [dc][4 warps][32 rows x 64 B], 64-byte swizzle
#pragma unroll 1
      for (int g = 0; g < D / 16; ++g) {
        uint32_t ov[16];
        if (any_keys) {
          __syncwarp();
          tmem_ld_32x16(tmem_o + lane_sel + g * 16, ov);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) ov[i] = 0u;
        }
        uint32_t w[8];
        float2 val[8];  // the fp16 values that are stored: the int8 copy quantizes these
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const __half2 hh = __floats2half2_rn(__uint_as_float(ov[2 * i]) * inv, __uint_as_float(ov[2 * i + 1]) * inv);
          w[i] = *reinterpret_cast<const uint32_t*>(&hh);
          val[i] = __half22float2(hh);
        }
        // 16 columns = two 16-byte units (2g, 2g+1) of the row's 128-byte chunk g / 4
        uint8_t* srow = sty + (g / 4) * (4 * 4096) + lane * 128;
        *reinterpret_cast<uint4*>(srow + ((((2 * g) & 7) ^ (lane & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
        *reinterpret_cast<uint4*>(srow + ((((2 * g + 1) & 7) ^ (lane & 7)) << 4)) = make_uint4(w[4], w[5], w[6], w[7]);
        if (p.oq) {
          // branch-free fast rounding, exact division only for the few values next to a rounding boundary
          uint32_t qw[4];
          const uint32_t risky = quantize_pairs_rn<16>(val, inv_o_scale, qw);
          if (risky) {
#pragma unroll
            for (int e = 0; e < 16; ++e)
              if (risky & (1u << e))
                patch_q_byte(qw, e, zen_det_round_clamp_i8(ZEN_DIV((e & 1) ? val[e >> 1].y : val[e >> 1].x, p.o_scale), 0));
          }
          // 16 values = 16-byte unit g % 4 of the row's 64-byte chunk g / 4
          *reinterpret_cast<uint4*>(stq + (g / 4) * (4 * 2048) + lane * 64 + (((g % 4) ^ ((lane >> 1) & 3)) << 4)) =
              make_uint4(qw[0], qw[1], qw[2], qw[3]);
        }
      }
      tc_fence_before_sync();
      fence_proxy_async_smem();  // this lane's writes to the blocks -> visible to the TMA engine
      __syncwarp();
      const int row0 = q0 + quad * 32;
      if (lane == 0 && row0 < p.S) {
        int c[4];
        c[p.o_perm[0]] = row0;
        c[p.o_perm[1]] = h;
        c[p.o_perm[2]] = b;
#pragma unroll
        for (int dc = 0; dc < DC; ++dc) {
          tma_store_4d(&tmap_o, sty + dc * (4 * 4096), dc * 64, c[1], c[2], c[3]);
          if (p.oq) tma_store_4d(&tmap_oq, stq + dc * (4 * 2048), dc * 64, c[1], c[2], c[3]);
        }
        tma_store_commit();
        tma_store_wait_all();  // shared memory is released when the CTA exits
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_s, TMEM_COLS);
}

// Rank-4 map over (d, seq, head, batch) with the three outer dims ordered by ascending stride.
// `elem_bytes` 2: fp16 with 128-byte swizzle (64-column boxes); 1: int8 with 64-byte swizzle.
static int encode_qkv_map(CUtensorMap* map, const void* base, int B, int H, int S, int D, int64_t sb, int64_t sh,
                          int64_t ss, int (&perm)[3], uint32_t box_rows = FA_BQ, int elem_bytes = 2) {
  struct Dim {
    uint64_t extent;
    int64_t stride;
    uint32_t box;
    int id;
  } dims[3] = {{uint64_t(S), ss, box_rows, 0}, {uint64_t(H), sh, 1u, 1}, {uint64_t(B), sb, 1u, 2}};
  // the stride of an extent-1 dim is never used to form an address: give it a valid, outermost value
  int64_t span = 8;
  for (int i = 0; i < 3; ++i)
    if (dims[i].extent > 1 && int64_t(dims[i].extent) * dims[i].stride > span) span = int64_t(dims[i].extent) * dims[i].stride;
  for (int i = 0; i < 3; ++i)
    if (dims[i].extent == 1) dims[i].stride = (span + 7) / 8 * 8;
  for (int i = 0; i < 3; ++i)
    for (int j = i + 1; j < 3; ++j)
      if (dims[j].stride < dims[i].stride) {
        Dim t = dims[i];
        dims[i] = dims[j];
        dims[j] = t;
      }
  uint64_t gd[4] = {uint64_t(D), 0, 0, 0};
  uint64_t gs[3];
  uint32_t bx[4] = {64u, 0, 0, 0};
  for (int i = 0; i < 3; ++i) {
    gd[i + 1] = dims[i].extent;
    gs[i] = uint64_t(dims[i].stride) * uint64_t(elem_bytes);
    bx[i + 1] = dims[i].box;
    perm[dims[i].id] = i + 1;
    if (dims[i].stride <= 0 || dims[i].stride % (16 / elem_bytes)) return ZEN_ERR_UNSUPPORTED;
  }
  if (elem_bytes == 1)
    return encode_tmap(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, base, gd, gs, bx, CU_TENSOR_MAP_SWIZZLE_64B);
  return encode_tmap(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, base, gd, gs, bx);
}

template <int D>
static int launch_fa(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, FaParams p, cudaStream_t s) {
  // output maps: 32-row boxes, one per softmax warp
  CUtensorMap to, toq;
  int perm_q[3];
  if (int st = encode_qkv_map(&to, p.o, p.B, p.H, p.S, D, p.o_sb, p.o_sh, p.o_ss, p.o_perm, 32u, 2); st != ZEN_OK) return st;
  toq = to;
  if (p.oq)
    if (int st = encode_qkv_map(&toq, p.oq, p.B, p.H, p.S, D, p.o_sb, p.o_sh, p.o_ss, perm_q, 32u, 1); st != ZEN_OK) return st;
  auto kernel = flash_attn_kernel<D>;
  constexpr size_t smem = fa_smem_bytes<D>();
  if (int st = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), smem); st != ZEN_OK) return st;
  dim3 grid((p.S + FA_BQ - 1) / FA_BQ, p.H, p.B);
  return launch_pdl(PDL_ATTENTION, kernel, grid, dim3(FA_THREADS), smem, s, tq, tk, tv, to, toq, p);
}

template <int D, int KV_STAGES>
static int launch_fa_pipe(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const FaParams& p,
                          cudaStream_t s) {
  auto kernel = flash_attn_pipe_kernel<D, KV_STAGES>;
  constexpr size_t smem = fap_smem_bytes<D, KV_STAGES>();
  if (int st = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), smem); st != ZEN_OK) return st;
  dim3 grid((p.S + 255) / 256, p.H, p.B);
  return launch_pdl(PDL_ATTENTION, kernel, grid, dim3(FAP_THREADS), smem, s, tq, tk, tv, p);
}

}  // namespace zen

using namespace zen;

ZEN_DEFINE_TU_STATUS(flash_attn)

extern "C" int zen_flash_attention_f16(const void* q, const void* k, const void* v, void* o, int8_t* oq, float o_scale,
                                       int B, int H, int S, int D, int64_t q_sb, int64_t q_sh, int64_t q_ss,
                                       int64_t k_sb, int64_t k_sh, int64_t k_ss, int64_t v_sb, int64_t v_sh,
                                       int64_t v_ss, int64_t o_sb, int64_t o_sh, int64_t o_ss, const int32_t* kv_lens,
                                       int causal, float scale, void* stream) {
  if (!q || !k || !v || !o || B <= 0 || H <= 0 || S <= 0) return ZEN_ERR_INVALID_ARG;
  if (D != 64 && D != 128) return ZEN_ERR_UNSUPPORTED;
  if (H > 65535 || B > 65535) return ZEN_ERR_UNSUPPORTED;
  if (oq && !(o_scale > 0.f)) return ZEN_ERR_INVALID_ARG;
  if (reinterpret_cast<uintptr_t>(o) % 16 || o_sb % 8 || o_sh % 8 || o_ss % 8) return ZEN_ERR_UNSUPPORTED;
  if (oq && (reinterpret_cast<uintptr_t>(oq) % 16 || o_sb % 16 || o_sh % 16 || o_ss % 16)) return ZEN_ERR_UNSUPPORTED;
  FaParams p{};
  p.o = o; p.oq = oq; p.o_scale = o_scale; p.B = B; p.H = H; p.S = S;
  p.o_sb = o_sb; p.o_sh = o_sh; p.o_ss = o_ss; p.kv_lens = kv_lens; p.causal = causal ? 1 : 0;
  p.scale_log2 = scale * 1.4426950408889634f;
  CUtensorMap tq, tk, tv;
  int st = encode_qkv_map(&tq, q, B, H, S, D, q_sb, q_sh, q_ss, p.q_perm);
  if (st == ZEN_OK) st = encode_qkv_map(&tk, k, B, H, S, D, k_sb, k_sh, k_ss, p.k_perm);
  if (st == ZEN_OK) st = encode_qkv_map(&tv, v, B, H, S, D, v_sb, v_sh, v_ss, p.v_perm);
  if (st != ZEN_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (S <= FA_BKV) return D == 64 ? launch_fa<64>(tq, tk, tv, p, s) : launch_fa<128>(tq, tk, tv, p, s);
  return D == 64 ? launch_fa_pipe<64, 2>(tq, tk, tv, p, s) : launch_fa_pipe<128, 1>(tq, tk, tv, p, s);
}

extern "C" int zen_flash_attention_unpadded_f16(const void* q, const void* k, const void* v, void* o, int8_t* oq, float o_scale,
                                                int B, int H, int max_seqlen, int D, int64_t rows, int64_t q_st, int64_t q_sh,
                                                int64_t k_st, int64_t k_sh, int64_t v_st, int64_t v_sh, int64_t o_st,
                                                int64_t o_sh, const int32_t* cu_seqlens, int causal, float scale,
                                                void* stream) {
  if (!q || !k || !v || !o || !cu_seqlens || B <= 0 || H <= 0 || max_seqlen <= 0 || rows <= 0) return ZEN_ERR_INVALID_ARG;
  if (D != 64 && D != 128) return ZEN_ERR_UNSUPPORTED;
  if (H > 65535 || B > 65535 || rows >= (int64_t(1) << 31)) return ZEN_ERR_UNSUPPORTED;
  if (oq && !(o_scale > 0.f)) return ZEN_ERR_INVALID_ARG;
  if (reinterpret_cast<uintptr_t>(o) % 16 || o_sh % 8 || o_st % 8) return ZEN_ERR_UNSUPPORTED;
  if (oq && (reinterpret_cast<uintptr_t>(oq) % 16 || o_sh % 16 || o_st % 16)) return ZEN_ERR_UNSUPPORTED;
  FaParams p{};
  p.o = o; p.oq = oq; p.o_scale = o_scale; p.B = B; p.H = H; p.S = max_seqlen;
  p.o_sb = 0; p.o_sh = o_sh; p.o_ss = o_st; p.kv_lens = nullptr; p.cu_seqlens = cu_seqlens; p.rows = int(rows);
  p.causal = causal ? 1 : 0;
  p.scale_log2 = scale * 1.4426950408889634f;
  // the packed tensors as ONE batch of `rows` tokens: a tile may start at any row
  CUtensorMap tq, tk, tv;
  const int R = int(rows);
  int st = encode_qkv_map(&tq, q, 1, H, R, D, int64_t(R) * q_st, q_sh, q_st, p.q_perm);
  if (st == ZEN_OK) st = encode_qkv_map(&tk, k, 1, H, R, D, int64_t(R) * k_st, k_sh, k_st, p.k_perm);
  if (st == ZEN_OK) st = encode_qkv_map(&tv, v, 1, H, R, D, int64_t(R) * v_st, v_sh, v_st, p.v_perm);
  if (st != ZEN_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return D == 64 ? launch_fa_pipe<64, 2>(tq, tk, tv, p, s) : launch_fa_pipe<128, 1>(tq, tk, tv, p, s);
}

// Shared body of the padded and the packed entry points.  Padded: S tokens per sequence, kv_lens optional.
// Packed: `rows` valid tokens back to back, cu_seqlens[B + 1] on the device, sequences of at most 128 tokens.
static int qkv_attention_launch(bool packed, const int8_t* xq, int64_t ldx, const int8_t* wqkv, int64_t ldw, int B, int S,
                                int64_t rows, int heads, int K, float x_scale, const float* w_scale, const float* bias,
                                const int32_t* kv_lens, const int32_t* cu_seqlens, float scale, void* ctx, int8_t* ctxq,
                                float ctx_scale, void* qkv_out, const void* next0, size_t next0_bytes, const void* next1,
                                size_t next1_bytes, unsigned flags, void* stream) {
  if (!xq || !wqkv || !ctx || B <= 0 || S <= 0 || heads <= 0 || K <= 0 || rows <= 0) return ZEN_ERR_INVALID_ARG;
  if (packed && !cu_seqlens) return ZEN_ERR_INVALID_ARG;
  if ((next0_bytes != 0 && !next0) || (next1_bytes != 0 && !next1)) return ZEN_ERR_INVALID_ARG;
  if (flags & ~unsigned(ZEN_GEMM_CONST_WEIGHTS)) return ZEN_ERR_INVALID_ARG;
  if (ctxq && !(ctx_scale > 0.f)) return ZEN_ERR_INVALID_ARG;
  if (S > 128 || B > 65535 || heads > 65535) return ZEN_ERR_UNSUPPORTED;  // longer sequences: zen_linear_i8 + zen_flash_attention_f16
  if (rows >= (int64_t(1) << 31)) return ZEN_ERR_UNSUPPORTED;
  if (K % 16 || ldx % 16 || ldw % 16 || ldx < K || ldw < K) return ZEN_ERR_UNSUPPORTED;
  const int hidden = heads * 64;
  if (reinterpret_cast<uintptr_t>(ctx) % 16 || reinterpret_cast<uintptr_t>(ctxq) % 16 ||
      reinterpret_cast<uintptr_t>(qkv_out) % 16)
    return ZEN_ERR_UNSUPPORTED;
  QkvAttnParams p{};
  p.B = B; p.S = S; p.heads = heads; p.K = K;
  p.num_k_blocks = (K + 127) / 128;
  p.x_scale = x_scale; p.w_scale = w_scale; p.bias = bias; p.kv_lens = kv_lens;
  p.cu_seqlens = cu_seqlens; p.ctx = static_cast<__half*>(ctx); p.rows = int(rows);
  p.scale_log2 = scale * 1.4426950408889634f;
  p.ctxq = ctxq; p.ctx_scale = ctxq ? ctx_scale : 1.0f;
  p.qkv_out = static_cast<__half*>(qkv_out);
  p.early_b = (flags & ZEN_GEMM_CONST_WEIGHTS) ? 1 : 0;
  const void* next[2] = {next0, next1};
  const size_t next_bytes[2] = {next0_bytes, next1_bytes};
  for (int i = 0; i < 2; ++i) {
    const uintptr_t lo = (reinterpret_cast<uintptr_t>(next[i]) + 15u) & ~uintptr_t(15);
    const uintptr_t hi = (reinterpret_cast<uintptr_t>(next[i]) + next_bytes[i]) & ~uintptr_t(15);
    if (next_bytes[i] != 0 && hi > lo) {
      p.pf_ptr[i] = reinterpret_cast<const uint8_t*>(lo);
      p.pf_bytes[i] = uint64_t(hi - lo);
    }
  }
  CUtensorMap ta, tb, to, toq;
  if (packed) {
    // activations as (k, row of the packed batch): a tile starts at any row; rows past the end read as zero
    if (int st = encode_tmap_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, xq, uint64_t(K), uint64_t(rows), uint64_t(ldx), 128, 128);
        st != ZEN_OK)
      return st;
  } else {
    // activations as (k, token of the sequence, sequence): rows beyond S read as zero, so a tile never holds a
    // neighbouring sequence's tokens
    const uint64_t dims[3] = {uint64_t(K), uint64_t(S), uint64_t(B)};
    const uint64_t str[2] = {uint64_t(ldx), uint64_t(ldx) * uint64_t(S)};
    const uint32_t box[3] = {128u, 128u, 1u};
    if (int st = encode_tmap(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, xq, dims, str, box); st != ZEN_OK) return st;
  }
  if (int st = encode_tmap_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, wqkv, uint64_t(K), uint64_t(3) * hidden, uint64_t(ldw), 128, 64);
      st != ZEN_OK)
    return st;
  to = ta;  // the packed form stores without tensor maps
  toq = ta;
  if (!packed) {
    // outputs: ctx[b * S + s, h * 64 + d] seen as (d, seq, head, batch), 32-row boxes (one per softmax warp)
    int perm_q[3];
    if (int st = encode_qkv_map(&to, ctx, B, heads, S, 64, int64_t(S) * hidden, 64, hidden, p.o_perm, 32u, 2); st != ZEN_OK)
      return st;
    toq = to;
    if (ctxq)
      if (int st = encode_qkv_map(&toq, ctxq, B, heads, S, 64, int64_t(S) * hidden, 64, hidden, perm_q, 32u, 1); st != ZEN_OK)
        return st;
  }
  constexpr size_t smem = qkv_attn_smem_bytes();
  const int items = B * heads;
  const int grid = items < num_sms() ? items : num_sms();
  if (packed) {
    if (int st = ensure_dynamic_smem(reinterpret_cast<const void*>(qkv_attn_kernel<true>), smem); st != ZEN_OK) return st;
    return launch_pdl(PDL_GEMM, qkv_attn_kernel<true>, dim3(grid), dim3(QA_THREADS), smem, static_cast<cudaStream_t>(stream), ta,
                      tb, to, toq, p);
  }
  if (int st = ensure_dynamic_smem(reinterpret_cast<const void*>(qkv_attn_kernel<false>), smem); st != ZEN_OK) return st;
  return launch_pdl(PDL_GEMM, qkv_attn_kernel<false>, dim3(grid), dim3(QA_THREADS), smem, static_cast<cudaStream_t>(stream), ta,
                    tb, to, toq, p);
}

extern "C" int zen_qkv_attention_i8(const int8_t* xq, int64_t ldx, const int8_t* wqkv, int64_t ldw, int B, int S, int heads,
                                    int K, float x_scale, const float* w_scale, const float* bias,
                                    const int32_t* kv_lens, float scale, void* ctx, int8_t* ctxq, float ctx_scale,
                                    void* qkv_out, const void* next0, size_t next0_bytes, const void* next1,
                                    size_t next1_bytes, unsigned flags, void* stream) {
  return qkv_attention_launch(false, xq, ldx, wqkv, ldw, B, S, int64_t(B) * S, heads, K, x_scale, w_scale, bias, kv_lens,
                              nullptr, scale, ctx, ctxq, ctx_scale, qkv_out, next0, next0_bytes, next1, next1_bytes, flags,
                              stream);
}

extern "C" int zen_qkv_attention_unpadded_i8(const int8_t* xq, int64_t ldx, const int8_t* wqkv, int64_t ldw, int B,
                                             int64_t rows, const int32_t* cu_seqlens, int heads, int K, float x_scale,
                                             const float* w_scale, const float* bias, float scale, void* ctx, int8_t* ctxq,
                                             float ctx_scale, void* qkv_out, const void* next0, size_t next0_bytes,
                                             const void* next1, size_t next1_bytes, unsigned flags, void* stream) {
  return qkv_attention_launch(true, xq, ldx, wqkv, ldw, B, 128, rows, heads, K, x_scale, w_scale, bias, nullptr, cu_seqlens,
                              scale, ctx, ctxq, ctx_scale, qkv_out, next0, next0_bytes, next1, next1_bytes, flags, stream);
}
