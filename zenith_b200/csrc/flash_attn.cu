// Flash-attention forward for sm_100a: O = softmax(scale * Q K^T [key-padding / causal mask]) V.
//
// One CTA per (128-query tile, head, batch).  fp16 operands, fp32 accumulation.
//   warp 0      : TMA producer — Q once, then K and V tiles of 128 keys into two-deep rings
//   warp 1      : TMEM owner and tcgen05.mma issuer:  S = Q K^T (kind::f16, K-major x K-major),
//                 O_blk = P V (A = P from shared memory, B = V as an MN-major operand, so V is
//                 consumed in its natural [key, d] layout without a transpose)
//   warps 2..5  : one thread per query row: tcgen05.ld of S, online softmax in registers
//                 (running max / sum, exp2 with the scale folded in), P written to shared memory
//                 as fp16 in the 128-byte-swizzled K-major layout, O accumulated in registers
//                 from the per-block P V product, final 1/l normalisation and 16-byte stores.
// QK^T of block j+1 is issued before P V of block j so that the tensor core works while the
// softmax threads fold O_blk(j) into their accumulators.
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
  int causal;
  float scale_log2;  // softmax scale * log2(e)
  // position of the (seq, head, batch) coordinates in each rank-4 tensor map (dim 0 is d)
  int q_perm[3], k_perm[3], v_perm[3];
};

template <int D, int KV_STAGES>
constexpr size_t fa_smem_bytes() {
  // Q + KV_STAGES x (K + V) tiles (128 x D fp16 each) + P (128 x 128 fp16) + control + alignment slack;
  // with a single key block P reuses the Q and K tiles, which are dead once S = Q K^T has completed
  return size_t(1 + 2 * KV_STAGES) * FA_BQ * D * 2 + (KV_STAGES == 1 ? 0 : FA_BQ * FA_BKV * 2) + 256 + 1024;
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
namespace zen {

// KV_STAGES = 2 double-buffers K and V for long sequences; KV_STAGES = 1 serves sequences of at most
// one key block (S <= 128, the encoder's case): P reuses the Q / K tiles and O_blk reuses the TMEM
// columns of S, so that four CTAs fit on an SM (one wave for 32 x 12 heads on 148 SMs) and one CTA's
// softmax overlaps the others' loads and MMAs.
template <int D, int KV_STAGES>
__global__ void __launch_bounds__(FA_THREADS, (D == 64 && KV_STAGES == 1) ? 4 : 1)
flash_attn_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                  const __grid_constant__ CUtensorMap tmap_v, const FaParams p) {
  constexpr int DC = D / 64;                 // 128-byte column chunks per row
  constexpr int TILE_BYTES = FA_BQ * D * 2;  // one Q / K / V tile
  constexpr int CHUNK_BYTES = FA_BQ * 128;   // one 64-column chunk of a tile
  constexpr uint32_t TMEM_COLS = KV_STAGES == 1 ? 128 : 256;  // S: 128 columns; O_blk: D columns (aliased on S
                                                              // when there is a single key block)
  constexpr uint32_t IDESC_QK = make_idesc(IDESC_C_F32, IDESC_F16, IDESC_F16, 0, 0, FA_BQ, FA_BKV);
  constexpr uint32_t IDESC_PV = make_idesc(IDESC_C_F32, IDESC_F16, IDESC_F16, 0, 1, FA_BQ, D);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + TILE_BYTES;              // KV_STAGES stages
  uint8_t* sV = sK + KV_STAGES * TILE_BYTES;  // KV_STAGES stages
  uint8_t* sP = KV_STAGES == 1 ? sQ : sV + KV_STAGES * TILE_BYTES;  // 2 chunks of 64 keys
  uint8_t* ctrl = sV + KV_STAGES * TILE_BYTES + (KV_STAGES == 1 ? 0 : FA_BQ * FA_BKV * 2);
  static_assert(KV_STAGES != 1 || 2 * TILE_BYTES >= FA_BQ * FA_BKV * 2, "P must fit in the Q + K tiles");
  uint64_t* q_full = reinterpret_cast<uint64_t*>(ctrl);
  uint64_t* k_full = q_full + 1;    // [2]
  uint64_t* k_empty = k_full + 2;   // [2]
  uint64_t* v_full = k_empty + 2;   // [2]
  uint64_t* v_empty = v_full + 2;   // [2]
  uint64_t* s_full = v_empty + 2;
  uint64_t* p_full = s_full + 1;
  uint64_t* o_full = p_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * FA_BQ;
  const int h = blockIdx.y;
  const int b = blockIdx.z;

  int kv_len = p.kv_lens ? p.kv_lens[b] : p.S;
  kv_len = kv_len < 0 ? 0 : (kv_len > p.S ? p.S : kv_len);
  int kv_end = kv_len;
  if (p.causal && q0 + FA_BQ < kv_end) kv_end = q0 + FA_BQ;
  const int n_blocks = (kv_end + FA_BKV - 1) / FA_BKV;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
    }
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
  const uint32_t tmem_base = *tmem_slot;
  grid_launch_dependents();
  grid_dependency_wait();  // Q, K, V and the output buffers may belong to the previous kernel until here
  const uint32_t tmem_s = tmem_base;
  const uint32_t tmem_o = KV_STAGES == 1 ? tmem_base : tmem_base + 128;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0 && n_blocks > 0) {
      bool ok = true;
      mbar_arrive_expect_tx(q_full, TILE_BYTES);
#pragma unroll
      for (int dc = 0; dc < DC; ++dc) fa_tma_tile(sQ + dc * CHUNK_BYTES, &tmap_q, q_full, p.q_perm, dc * 64, q0, h, b);
      for (int j = 0; j < n_blocks && ok; ++j) {
        const int st = j % KV_STAGES;
        const uint32_t ph = (j / KV_STAGES) & 1;
        if (!mbar_wait(&k_empty[st], ph ^ 1u, abort_flag)) { ok = false; break; }
        mbar_arrive_expect_tx(&k_full[st], TILE_BYTES);
#pragma unroll
        for (int dc = 0; dc < DC; ++dc)
          fa_tma_tile(sK + st * TILE_BYTES + dc * CHUNK_BYTES, &tmap_k, &k_full[st], p.k_perm, dc * 64, j * FA_BKV, h, b);
        if (!mbar_wait(&v_empty[st], ph ^ 1u, abort_flag)) { ok = false; break; }
        mbar_arrive_expect_tx(&v_full[st], TILE_BYTES);
#pragma unroll
        for (int dc = 0; dc < DC; ++dc)
          fa_tma_tile(sV + st * TILE_BYTES + dc * CHUNK_BYTES, &tmap_v, &v_full[st], p.v_perm, dc * 64, j * FA_BKV, h, b);
      }
      if (!ok) {
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0 && n_blocks > 0) {
      auto issue_qk = [&](int j) -> bool {
        const int st = j % KV_STAGES;
        if (!mbar_wait(&k_full[st], (j / KV_STAGES) & 1, abort_flag)) return false;
        tc_fence_after_sync();
        const uint32_t qa = smem_u32(sQ);
        const uint32_t ka = smem_u32(sK + st * TILE_BYTES);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = (ks / 4) * CHUNK_BYTES + (ks % 4) * 32;
          mma_f16_ss(tmem_s, make_smem_desc_sw128(qa + off, 1024, 16), make_smem_desc_sw128(ka + off, 1024, 16),
                     IDESC_QK, ks != 0 ? 1u : 0u);
        }
        tc_commit(&k_empty[st]);
        tc_commit(s_full);
        return true;
      };
      bool ok = mbar_wait(q_full, 0, abort_flag);
      if (ok) ok = issue_qk(0);
      for (int j = 0; j < n_blocks && ok; ++j) {
        const int st = j % KV_STAGES;
        // P(j) is in shared memory, S(j) and O_blk(j-1) have been read by every softmax thread
        if (!mbar_wait(p_full, j & 1, abort_flag)) break;
        tc_fence_after_sync();
        if (j + 1 < n_blocks && !issue_qk(j + 1)) break;
        if (!mbar_wait(&v_full[st], (j / KV_STAGES) & 1, abort_flag)) break;
        tc_fence_after_sync();
        const uint32_t pa = smem_u32(sP);
        const uint32_t va = smem_u32(sV + st * TILE_BYTES);
#pragma unroll
        for (int ks = 0; ks < FA_BKV / 16; ++ks) {
          const uint64_t a_desc = make_smem_desc_sw128(pa + (ks / 4) * CHUNK_BYTES + (ks % 4) * 32, 1024, 16);
          const uint64_t b_desc = make_smem_desc_sw128(va + ks * (16 * 128), 1024, CHUNK_BYTES);
          mma_f16_ss(tmem_o, a_desc, b_desc, IDESC_PV, ks != 0 ? 1u : 0u);
        }
        tc_commit(&v_empty[st]);
        tc_commit(o_full);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax + accumulate
    const int quad = warp & 3;
    const int r = quad * 32 + lane;  // row within the query tile == TMEM lane
    const int q = q0 + r;
    const uint32_t lane_sel = uint32_t(quad * 32) << 16;
    float m_run = -INFINITY;
    float l_run = 0.f;
    float o_acc[D];
#pragma unroll
    for (int i = 0; i < D; ++i) o_acc[i] = 0.f;
    bool ok = true;

    for (int j = 0; j < n_blocks && ok; ++j) {
      if (!mbar_wait(s_full, j & 1, abort_flag)) { ok = false; break; }
      tc_fence_after_sync();
      const int key0 = j * FA_BKV;
      int lim = kv_len - key0;  // keys [0, lim) of this block are valid for this row
      if (p.causal && q + 1 - key0 < lim) lim = q + 1 - key0;
      // pass 1: row maximum
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < FA_BKV / 32; ++c) {
        uint32_t sv[32];
        __syncwarp();
        tmem_ld_32x32(tmem_s + lane_sel + c * 32, sv);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (c * 32 + i < lim) mx = fmaxf(mx, __uint_as_float(sv[i]));
      }
      const float m_new = fmaxf(m_run, mx * p.scale_log2);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = fast_exp2(m_run - m_use);
      // pass 2: probabilities -> shared memory (fp16, swizzled K-major), row sum
      float rowsum = 0.f;
#pragma unroll 1
      for (int c = 0; c < FA_BKV / 32; ++c) {
        uint32_t sv[32];
        __syncwarp();
        tmem_ld_32x32(tmem_s + lane_sel + c * 32, sv);
        tmem_wait_ld();
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float a = (c * 32 + 2 * i < lim) ? fast_exp2(__uint_as_float(sv[2 * i]) * p.scale_log2 - m_use) : 0.f;
          const float bq = (c * 32 + 2 * i + 1 < lim) ? fast_exp2(__uint_as_float(sv[2 * i + 1]) * p.scale_log2 - m_use) : 0.f;
          rowsum += a + bq;
          const __half2 hh = __floats2half2_rn(a, bq);
          pk[i] = *reinterpret_cast<const uint32_t*>(&hh);
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

      l_run = l_run * alpha + rowsum;
      m_run = m_new;
      if constexpr (KV_STAGES != 1) {
        if (alpha != 1.f) {
#pragma unroll
          for (int i = 0; i < D; ++i) o_acc[i] *= alpha;
        }
        if (!mbar_wait(o_full, j & 1, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t ov[32];
          __syncwarp();
          tmem_ld_32x32(tmem_o + lane_sel + c * 32, ov);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) o_acc[c * 32 + i] += __uint_as_float(ov[i]);
        }
        tc_fence_before_sync();
      }
    }
    if constexpr (KV_STAGES == 1) {
      // a single key block: O is the one P V product, read straight from TMEM
      if (ok && n_blocks > 0) {
        if (!mbar_wait(o_full, 0, abort_flag)) ok = false;
        tc_fence_after_sync();
        if (ok) {
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t ov[32];
            __syncwarp();
            tmem_ld_32x32(tmem_o + lane_sel + c * 32, ov);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o_acc[c * 32 + i] = __uint_as_float(ov[i]);
          }
        }
        tc_fence_before_sync();
      }
    }

    if (ok && q < p.S) {
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      const int64_t off = int64_t(b) * p.o_sb + int64_t(h) * p.o_sh + int64_t(q) * p.o_ss;
      __half* orow = static_cast<__half*>(p.o) + off;
      uint32_t w[D / 2];
#pragma unroll
      for (int i = 0; i < D / 2; ++i) {
        const __half2 hh = __floats2half2_rn(o_acc[2 * i] * inv, o_acc[2 * i + 1] * inv);
        w[i] = *reinterpret_cast<const uint32_t*>(&hh);
      }
#pragma unroll
      for (int i = 0; i < D / 8; ++i)
        reinterpret_cast<uint4*>(orow)[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
      if (p.oq) {
        const float inv_o_scale = ZEN_DIV(1.0f, p.o_scale);
        int8_t* qrow = p.oq + off;
        uint32_t qw[D / 4];
#pragma unroll
        for (int i = 0; i < D / 4; ++i) {
          uint32_t pk = 0;
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const __half2 hh = *reinterpret_cast<const __half2*>(&w[(4 * i + e) / 2]);
            const float val = (e & 1) ? __high2float(hh) : __low2float(hh);
            pk |= (uint32_t(quantize_exact(val, p.o_scale, inv_o_scale, 0)) & 0xffu) << (8 * e);
          }
          qw[i] = pk;
        }
#pragma unroll
        for (int i = 0; i < D / 16; ++i)
          reinterpret_cast<uint4*>(qrow)[i] = make_uint4(qw[4 * i], qw[4 * i + 1], qw[4 * i + 2], qw[4 * i + 3]);
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// Rank-4 map over (d, seq, head, batch) with the three outer dims ordered by ascending stride.
static int encode_qkv_map(CUtensorMap* map, const void* base, int B, int H, int S, int D, int64_t sb, int64_t sh,
                          int64_t ss, int (&perm)[3]) {
  struct Dim {
    uint64_t extent;
    int64_t stride;
    uint32_t box;
    int id;
  } dims[3] = {{uint64_t(S), ss, uint32_t(FA_BQ), 0}, {uint64_t(H), sh, 1u, 1}, {uint64_t(B), sb, 1u, 2}};
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
    gs[i] = uint64_t(dims[i].stride) * 2;
    bx[i + 1] = dims[i].box;
    perm[dims[i].id] = i + 1;
    if (dims[i].stride <= 0 || dims[i].stride % 8) return ZEN_ERR_UNSUPPORTED;
  }
  return encode_tmap(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, base, gd, gs, bx);
}

template <int D, int KV_STAGES>
static int launch_fa(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const FaParams& p,
                     cudaStream_t s) {
  auto kernel = flash_attn_kernel<D, KV_STAGES>;
  constexpr size_t smem = fa_smem_bytes<D, KV_STAGES>();
  if (int st = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), smem); st != ZEN_OK) return st;
  dim3 grid((p.S + FA_BQ - 1) / FA_BQ, p.H, p.B);
  return launch_pdl(PDL_ATTENTION, kernel, grid, dim3(FA_THREADS), smem, s, tq, tk, tv, p);
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
  if (S <= FA_BKV) return D == 64 ? launch_fa<64, 1>(tq, tk, tv, p, s) : launch_fa<128, 1>(tq, tk, tv, p, s);
  static const bool simple = []() {
    const char* e = getenv("ZEN_ATTENTION_SIMPLE");  // 1: the one-tile-per-CTA kernel also for long sequences
    return e && e[0] == '1';
  }();
  if (simple) return D == 64 ? launch_fa<64, 2>(tq, tk, tv, p, s) : launch_fa<128, 2>(tq, tk, tv, p, s);
  return D == 64 ? launch_fa_pipe<64, 2>(tq, tk, tv, p, s) : launch_fa_pipe<128, 1>(tq, tk, tv, p, s);
}
