// Flash attention forward for sm_100a (head_dim 128, GQA, causal + column-wise "masked from row" document masks).
//
// One CTA = one 128-row query tile of one head. S = Q K^T and O_tile = P V run on tcgen05 with accumulators in TMEM;
// four softmax warps own one query row per thread (online softmax in registers, exp2 domain); one control thread
// issues TMA loads and MMAs. P is written back into the TMEM columns of S as bf16 and used as the A operand of the
// second MMA (or staged through swizzled shared memory when P_TMEM is false). Two CTAs fit per SM (96 KB smem,
// 256 TMEM columns) so one CTA's softmax overlaps the other's MMAs.
//
// Mask semantics follow the reference's FlashMask lower-triangular start rows
// (paddleformers/utils/masking_utils.py:24-113): key column j is visible to query row i iff j <= i and i < kend[j];
// document-causal packing sets kend[j] to the end of the document that contains j
// (paddleformers/datasets/collate.py:1185-1215). Call site replaced: paddleformers/nn/attention/flashmask_attention.py:24-76.
#pragma once
#include "sm100_common.cuh"

namespace pfb {

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

constexpr int ATT_BQ = 128;
constexpr int ATT_BKV = 128;
constexpr int ATT_D = 128;
constexpr int ATT_THREADS = 160;  // warps 0-3 softmax, warp 4 control

struct AttnFwdParams {
  __nv_bfloat16* O;       // [B*S, Hq, D], row stride o_row_stride
  float* lse;             // [B, Hq, S]
  const int* kend;        // [B, S] first masked row per key column (nullptr: plain causal)
  const int* tile_min_end;  // [B, kv_tiles] min of kend per kv tile (nullptr with kend == nullptr)
  const int* tile_max_end;  // [B, kv_tiles]
  long long o_row_stride;
  int S, Hq, Hkv;
  float scale_log2;       // softmax scale * log2(e)
  int causal;
  int* status;
};

// DQK is the width of queries and keys (128, or 192 for multi-head latent attention whose values stay 128 wide: the
// reference's call sites are paddleformers/transformers/deepseek_v3/modeling.py:542-801); Q and K tiles are stored as
// DQK / 64 slabs of [128 rows x 64 columns] (128-byte swizzle), V as two.
template <bool P_TMEM, int DQK = ATT_D>
struct AttnFwdSmem {
  static constexpr int TILE = ATT_BQ * ATT_D * 2;      // 32 KB: V, P
  static constexpr int SLAB = ATT_BQ * 64 * 2;         // 16 KB
  static constexpr int QK_TILE = (DQK / 64) * SLAB;
  static constexpr int Q_OFF = 0, K_OFF = QK_TILE, V_OFF = 2 * QK_TILE, P_OFF = 2 * QK_TILE + TILE;
  static constexpr int AUX_OFF = P_TMEM ? P_OFF : P_OFF + TILE;
  static constexpr int TOTAL = AUX_OFF + 2048 + 256 + 1024;
};

template <bool P_TMEM, int DQK = ATT_D>
__global__ void __launch_bounds__(ATT_THREADS, (P_TMEM && DQK == ATT_D) ? 2 : 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const AttnFwdParams p) {
  using SM = AttnFwdSmem<P_TMEM, DQK>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + SM::Q_OFF; uint8_t* sK = smem + SM::K_OFF; uint8_t* sV = smem + SM::V_OFF;
  uint8_t* sP = smem + SM::P_OFF;
  int* s_kend_all = reinterpret_cast<int*>(smem + SM::AUX_OFF);        // [4 warps][128]: private copy per warp
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::AUX_OFF + 2048);
  uint64_t* bar_q = bars; uint64_t* bar_k = bars + 1; uint64_t* bar_v = bars + 2; uint64_t* bar_s = bars + 3;
  uint64_t* bar_p = bars + 4; uint64_t* bar_o = bars + 5;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 6);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = gridDim.x - 1 - blockIdx.x;  // heavy (late) causal tiles first
  const int head = blockIdx.y, b = blockIdx.z;
  const int kvh = head / (p.Hq / p.Hkv);
  const int q0 = qt * ATT_BQ;
  const int row_base = b * p.S;

  if (threadIdx.x == 0) {
    mbar_init(bar_q, 1); mbar_init(bar_k, 1); mbar_init(bar_v, 1); mbar_init(bar_s, 1);
    mbar_init(bar_p, 4); mbar_init(bar_o, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 4) { tmem_alloc(tmem_slot, 256); tmem_relinquish(); tc_fence_before(); }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base, tO = tmem_base + 128;

  // kv tile range [j_lo, j_hi]
  const int kv_tiles = (p.S + ATT_BKV - 1) / ATT_BKV;
  int j_hi = p.causal ? min(kv_tiles - 1, (q0 + ATT_BQ - 1) / ATT_BKV) : kv_tiles - 1;
  int j_lo = 0;
  if (p.kend) {
    // keys whose masked-from row is <= q0 are invisible to the whole tile
    const int* tmax = p.tile_max_end + b * kv_tiles;
    while (j_lo < j_hi && tmax[j_lo] <= q0) ++j_lo;
  }

  if (warp == 4) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc(ATT_BQ, ATT_BKV, false, false, 1);
      constexpr uint32_t idesc_o = make_idesc(ATT_BQ, ATT_D, false, true, 1);
      mbar_expect_tx(bar_q, SM::QK_TILE);
      #pragma unroll
      for (int sl = 0; sl < DQK / 64; ++sl) tma_load_3d(sQ + sl * SM::SLAB, &tmQ, bar_q, 64 * sl, head, row_base + q0);
      mbar_expect_tx(bar_k, SM::QK_TILE);
      #pragma unroll
      for (int sl = 0; sl < DQK / 64; ++sl) tma_load_3d(sK + sl * SM::SLAB, &tmK, bar_k, 64 * sl, kvh, row_base + j_lo * ATT_BKV);
      mbar_expect_tx(bar_v, SM::TILE);
      tma_load_3d(sV, &tmV, bar_v, 0, kvh, row_base + j_lo * ATT_BKV);
      tma_load_3d(sV + SM::TILE / 2, &tmV, bar_v, 64, kvh, row_base + j_lo * ATT_BKV);
      bool ok = mbar_wait(bar_q, 0, abort_flag, p.status, PFB_ERR_WAIT_FULL);
      uint32_t ph = 0;
      for (int j = j_lo; j <= j_hi && ok; ++j, ph ^= 1) {
        if (!mbar_wait(bar_k, ph, abort_flag, p.status, PFB_ERR_WAIT_FULL)) break;
        tc_fence_after();
        #pragma unroll
        for (int k = 0; k < DQK / 16; ++k) {
          const uint32_t off = (k >> 2) * SM::SLAB + (k & 3) * 32;
          tc_mma_f16_ss(tS, make_smem_desc_sw128(smem_u32(sQ) + off, 16, 1024),
                        make_smem_desc_sw128(smem_u32(sK) + off, 16, 1024), idesc_s, k != 0);
        }
        tc_commit(bar_s);
        if (!mbar_wait(bar_s, ph, abort_flag, p.status, PFB_ERR_WAIT_TMEM_FULL)) break;
        if (j < j_hi) {
          mbar_expect_tx(bar_k, SM::QK_TILE);
          #pragma unroll
          for (int sl = 0; sl < DQK / 64; ++sl) tma_load_3d(sK + sl * SM::SLAB, &tmK, bar_k, 64 * sl, kvh, row_base + (j + 1) * ATT_BKV);
        }
        if (!mbar_wait(bar_p, ph, abort_flag, p.status, PFB_ERR_WAIT_TMEM_EMPTY)) break;
        if (!mbar_wait(bar_v, ph, abort_flag, p.status, PFB_ERR_WAIT_FULL)) break;
        tc_fence_after();
        #pragma unroll
        for (int k = 0; k < ATT_BKV / 16; ++k) {
          const uint64_t dv = make_smem_desc_sw128(smem_u32(sV) + k * 16 * 128, SM::TILE / 2, 1024);
          if constexpr (P_TMEM) {
            tc_mma_f16_ts(tO, tS + k * 8, dv, idesc_o, k != 0);
          } else {
            const uint32_t off = (k >> 2) * (SM::TILE / 2) + (k & 3) * 32;
            tc_mma_f16_ss(tO, make_smem_desc_sw128(smem_u32(sP) + off, 16, 1024), dv, idesc_o, k != 0);
          }
        }
        tc_commit(bar_o);
        if (!mbar_wait(bar_o, ph, abort_flag, p.status, PFB_ERR_WAIT_TMEM_FULL)) break;
        if (j < j_hi) {
          mbar_expect_tx(bar_v, SM::TILE);
          tma_load_3d(sV, &tmV, bar_v, 0, kvh, row_base + (j + 1) * ATT_BKV);
          tma_load_3d(sV + SM::TILE / 2, &tmV, bar_v, 64, kvh, row_base + (j + 1) * ATT_BKV);
        }
      }
    }
  } else {
    // ---------------- softmax: thread r owns query row q0 + r ----------------
    const int r = threadIdx.x;
    const int qi = q0 + r;
    const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;
    int* s_kend = s_kend_all + warp * 128;
    float m = -INFINITY, l = 0.f;
    float o[ATT_D];
    #pragma unroll
    for (int i = 0; i < ATT_D; ++i) o[i] = 0.f;
    uint32_t ph = 0;
    bool ok = true;
    for (int j = j_lo; j <= j_hi; ++j, ph ^= 1) {
      const int k0 = j * ATT_BKV;
      bool need_mask = (p.causal && k0 + ATT_BKV - 1 > q0) || (k0 + ATT_BKV > p.S);
      const bool need_kend = p.kend && p.tile_min_end[b * kv_tiles + j] < q0 + ATT_BQ;
      if (need_kend) {
        // each warp stages its own copy, so no cross-warp barrier is needed
        __syncwarp();
        #pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int kk = lane + 32 * i;
          s_kend[kk] = (k0 + kk < p.S) ? p.kend[b * p.S + k0 + kk] : 0;
        }
        __syncwarp();
        need_mask = true;
      }
      if (!mbar_wait(bar_s, ph, abort_flag, p.status, PFB_ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      // pass 1: row max
      float mx = -INFINITY;
      #pragma unroll 1
      for (int c = 0; c < ATT_BKV; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(tS + lane_off + c, v);
        tmem_ld_wait();
        if (need_mask) {
          #pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int kj = k0 + c + i;
            bool vis = kj < p.S && (!p.causal || kj <= qi);
            if (need_kend) vis = vis && qi < s_kend[c + i];
            mx = vis ? fmaxf(mx, __uint_as_float(v[i])) : mx;
          }
        } else {
          #pragma unroll
          for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(v[i]));
        }
      }
      const float m_new = fmaxf(m, mx * p.scale_log2);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = fast_exp2(m - m_use);  // m = -inf -> 0
      float lt = 0.f;
      // pass 2: probabilities -> bf16 P
      #pragma unroll 1
      for (int c = 0; c < ATT_BKV; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(tS + lane_off + c, v);
        tmem_ld_wait();
        uint32_t pk[16];
        #pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float p0 = fast_exp2(__uint_as_float(v[i]) * p.scale_log2 - m_use);
          float p1 = fast_exp2(__uint_as_float(v[i + 1]) * p.scale_log2 - m_use);
          if (need_mask) {
            const int kj = k0 + c + i;
            bool v0 = kj < p.S && (!p.causal || kj <= qi);
            bool v1 = kj + 1 < p.S && (!p.causal || kj + 1 <= qi);
            if (need_kend) { v0 = v0 && qi < s_kend[c + i]; v1 = v1 && qi < s_kend[c + i + 1]; }
            p0 = v0 ? p0 : 0.f; p1 = v1 ? p1 : 0.f;
          }
          lt += p0 + p1;
          pk[i >> 1] = pack_bf16x2(p0, p1);
        }
        if constexpr (P_TMEM) {
          tmem_st_32x16(tS + lane_off + (c >> 1), pk);
        } else {
          // K-major swizzled A tile: slab (c / 64), row r, 16-byte chunk index XOR (r % 8)
          uint8_t* slab = sP + (c >> 6) * (SM::TILE / 2) + r * 128;
          #pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int chunk = ((c & 63) >> 3) + q;
            *reinterpret_cast<uint4*>(slab + ((chunk ^ (r & 7)) << 4)) = make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
          }
        }
      }
      if constexpr (P_TMEM) tmem_st_wait(); else fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_p);
      l = l * alpha + lt;
      m = m_new;
      if (!mbar_wait(bar_o, ph, abort_flag, p.status, PFB_ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      #pragma unroll
      for (int c = 0; c < ATT_D; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(tO + lane_off + c, v);
        tmem_ld_wait();
        #pragma unroll
        for (int i = 0; i < 32; ++i) o[c + i] = o[c + i] * alpha + __uint_as_float(v[i]);
      }
      tc_fence_before();
    }
    if (ok && qi < p.S) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* dst = p.O + static_cast<long long>(row_base + qi) * p.o_row_stride + head * ATT_D;
      #pragma unroll
      for (int c = 0; c < ATT_D; c += 8) {
        uint4 w = make_uint4(pack_bf16x2(o[c] * inv, o[c + 1] * inv), pack_bf16x2(o[c + 2] * inv, o[c + 3] * inv),
                             pack_bf16x2(o[c + 4] * inv, o[c + 5] * inv), pack_bf16x2(o[c + 6] * inv, o[c + 7] * inv));
        *reinterpret_cast<uint4*>(dst + c) = w;
      }
      p.lse[(static_cast<long long>(b) * p.Hq + head) * p.S + qi] =
          l > 0.f ? (m + log2f(l)) * 0.6931471805599453f : -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 4) { tc_fence_after(); tmem_dealloc(tmem_base, 256); }
}

// ------------------------------------------------------------------------------------------------------------------
// Two-tile ("ping-pong") forward, the default. One CTA owns two consecutive 128-row query tiles of one head, so that
// the tensor pipe always has the other tile's product to run while one tile is in its softmax:
//
//   warp 8      TMA loader: both Q tiles once, K and V tiles through two-stage rings
//   warp 9      MMA issuer:  S_t = Q_t K_j^T and O_t += P_t V_j for t = 0, 1, the S product of step j+1 issued right after
//               the PV product of step j of the same tile (the pipe executes in order, so it cannot overtake the read of P)
//   warps 0-3   softmax of tile 0, warps 4-7 softmax of tile 1: ONE pass over S (the 128 scores of a row stay in
//               registers), P written back over S as bf16. O stays in TMEM for the whole walk: it is rescaled only when
//               a row maximum has grown by more than 2^8 since the scale last used (the lazy rescale), which after the
//               first tiles is rare; the final 1/l normalisation absorbs the stale scale exactly.
//
// TMEM: S_0, S_1, O_0, O_1 at 128 columns each (all 512). Same masks, layouts and outputs as attn_fwd_kernel.
constexpr int AF2_THREADS = 320;
constexpr float AF2_RESCALE_LOG2 = 8.f;

struct AttnFwd2Smem {
  static constexpr int TILE = ATT_BQ * ATT_D * 2;  // 32 KB
  static constexpr int Q_OFF = 0;                  // 2 tiles
  static constexpr int K_OFF = 2 * TILE;           // 2 stages
  static constexpr int V_OFF = 4 * TILE;           // 2 stages
  static constexpr int KEND_OFF = 6 * TILE;        // per softmax warp: 128 ints
  static constexpr int BAR_OFF = KEND_OFF + 8 * 128 * 4;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

static __global__ void __launch_bounds__(AF2_THREADS, 1)
attn_fwd2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const AttnFwdParams p) {
  using SM = AttnFwd2Smem;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::BAR_OFF);
  uint64_t* q_full = bars;          // 1
  uint64_t* k_full = bars + 1;      // [2]
  uint64_t* k_empty = bars + 3;     // [2]
  uint64_t* v_full = bars + 5;      // [2]
  uint64_t* v_empty = bars + 7;     // [2]
  uint64_t* s_full = bars + 9;      // [2] per tile
  uint64_t* p_full = bars + 11;     // [2] per tile
  uint64_t* o_full = bars + 13;     // [2] per tile
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pair = gridDim.x - 1 - blockIdx.x;     // heavy (late) causal tiles first
  const int head = blockIdx.y, b = blockIdx.z;
  const int kvh = head / (p.Hq / p.Hkv);
  const int q0 = pair * 2 * ATT_BQ;
  const int row_base = b * p.S;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
      mbar_init(&s_full[s], 1); mbar_init(&p_full[s], 4); mbar_init(&o_full[s], 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 9) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); tc_fence_before(); }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // kv tile ranges: common lower end, one upper end per query tile
  const int kv_tiles = (p.S + ATT_BKV - 1) / ATT_BKV;
  int j_lo = 0;
  if (p.kend) {
    const int* tmax = p.tile_max_end + b * kv_tiles;
    const int top = p.causal ? min(kv_tiles - 1, (q0 + ATT_BQ - 1) / ATT_BKV) : kv_tiles - 1;
    while (j_lo < top && tmax[j_lo] <= q0) ++j_lo;
  }
  int n_t[2];
  #pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int qt0 = q0 + t * ATT_BQ;
    const int j_hi = p.causal ? min(kv_tiles - 1, (qt0 + ATT_BQ - 1) / ATT_BKV) : kv_tiles - 1;
    n_t[t] = qt0 < p.S ? max(j_hi - j_lo + 1, 0) : 0;
  }
  const int n = max(n_t[0], n_t[1]);

  if (warp == 8) {
    // ------------------------------------------------------------ TMA loader
    if (lane == 0 && n > 0) {
      uint8_t* sQ = smem + SM::Q_OFF;
      mbar_expect_tx(q_full, 2 * SM::TILE);
      #pragma unroll
      for (int t = 0; t < 2; ++t) {
        tma_load_3d(sQ + t * SM::TILE, &tmQ, q_full, 0, head, row_base + q0 + t * ATT_BQ);
        tma_load_3d(sQ + t * SM::TILE + SM::TILE / 2, &tmQ, q_full, 64, head, row_base + q0 + t * ATT_BQ);
      }
      for (int jj = 0; jj < n; ++jj) {
        const int st = jj & 1;
        const uint32_t ph = (jj >> 1) & 1;
        const int row = row_base + (j_lo + jj) * ATT_BKV;
        if (!mbar_wait(&k_empty[st], ph ^ 1, abort_flag, p.status, PFB_ERR_WAIT_EMPTY)) break;
        uint8_t* sK = smem + SM::K_OFF + st * SM::TILE;
        mbar_expect_tx(&k_full[st], SM::TILE);
        tma_load_3d(sK, &tmK, &k_full[st], 0, kvh, row);
        tma_load_3d(sK + SM::TILE / 2, &tmK, &k_full[st], 64, kvh, row);
        if (!mbar_wait(&v_empty[st], ph ^ 1, abort_flag, p.status, PFB_ERR_WAIT_EMPTY)) break;
        uint8_t* sV = smem + SM::V_OFF + st * SM::TILE;
        mbar_expect_tx(&v_full[st], SM::TILE);
        tma_load_3d(sV, &tmV, &v_full[st], 0, kvh, row);
        tma_load_3d(sV + SM::TILE / 2, &tmV, &v_full[st], 64, kvh, row);
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0 && n > 0) {
      constexpr uint32_t idesc_s = make_idesc(ATT_BQ, ATT_BKV, false, false, 1);
      constexpr uint32_t idesc_o = make_idesc(ATT_BQ, ATT_D, false, true, 1);
      auto issue_s = [&](int t, int jj) {
        const uint32_t sq = smem_u32(smem + SM::Q_OFF + t * SM::TILE);
        const uint32_t sk = smem_u32(smem + SM::K_OFF + (jj & 1) * SM::TILE);
        #pragma unroll
        for (int k = 0; k < ATT_D / 16; ++k) {
          const uint32_t off = (k >> 2) * (SM::TILE / 2) + (k & 3) * 32;
          tc_mma_f16_ss(tmem_base + t * 128, make_smem_desc_sw128(sq + off, 16, 1024), make_smem_desc_sw128(sk + off, 16, 1024),
                        idesc_s, k != 0);
        }
        tc_commit(&s_full[t]);
      };
      auto issue_pv = [&](int t, int jj) {
        const uint32_t sv = smem_u32(smem + SM::V_OFF + (jj & 1) * SM::TILE);
        #pragma unroll
        for (int k = 0; k < ATT_BKV / 16; ++k)
          tc_mma_f16_ts(tmem_base + 256 + t * 128, tmem_base + t * 128 + k * 8,
                        make_smem_desc_sw128(sv + k * 16 * 128, SM::TILE / 2, 1024), idesc_o, (jj | k) != 0);
        tc_commit(&o_full[t]);
      };
      bool ok = mbar_wait(q_full, 0, abort_flag, p.status, PFB_ERR_WAIT_FULL);
      ok = ok && mbar_wait(&k_full[0], 0, abort_flag, p.status, PFB_ERR_WAIT_FULL);
      if (ok) {
        tc_fence_after();
        if (n_t[0] > 0) issue_s(0, 0);
        if (n_t[1] > 0) issue_s(1, 0);
        tc_commit(&k_empty[0]);
      }
      for (int jj = 0; jj < n && ok; ++jj) {
        const uint32_t ph = jj & 1, ph2 = (jj >> 1) & 1, ph2n = ((jj + 1) >> 1) & 1;
        if (!mbar_wait(&v_full[jj & 1], ph2, abort_flag, p.status, PFB_ERR_WAIT_FULL)) break;
        const bool more = jj + 1 < n;
        if (more && !mbar_wait(&k_full[(jj + 1) & 1], ph2n, abort_flag, p.status, PFB_ERR_WAIT_FULL)) break;
        #pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (jj < n_t[t]) {
            if (!mbar_wait(&p_full[t], ph, abort_flag, p.status, PFB_ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
            tc_fence_after();
            issue_pv(t, jj);
          }
          if (jj + 1 < n_t[t]) issue_s(t, jj + 1);
        }
        if (!ok) break;
        tc_commit(&v_empty[jj & 1]);
        if (more) tc_commit(&k_empty[(jj + 1) & 1]);
      }
    }
  } else {
    // ------------------------------------------------------------ softmax: warps 0-3 tile 0, warps 4-7 tile 1
    const int t = warp >> 2;
    const int r = threadIdx.x & 127;
    const int qt0 = q0 + t * ATT_BQ;
    const int qi = qt0 + r;
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tS = tmem_base + t * 128 + lane_off, tO = tmem_base + 256 + t * 128 + lane_off;
    int* s_kend = reinterpret_cast<int*>(smem + SM::KEND_OFF) + warp * 128;
    const int nt = n_t[t];
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int jj = 0; jj < nt; ++jj) {
      const uint32_t ph = jj & 1;
      const int j = j_lo + jj;
      const int k0 = j * ATT_BKV;
      bool need_mask = (p.causal && k0 + ATT_BKV - 1 > qt0) || (k0 + ATT_BKV > p.S);
      const bool need_kend = p.kend && p.tile_min_end[b * kv_tiles + j] < qt0 + ATT_BQ;
      if (need_kend) {
        __syncwarp();
        #pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int kk = lane + 32 * i;
          s_kend[kk] = (k0 + kk < p.S) ? p.kend[b * p.S + k0 + kk] : 0;
        }
        __syncwarp();
        need_mask = true;
      }
      if (!mbar_wait(&s_full[t], ph, abort_flag, p.status, PFB_ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      uint32_t v[128];
      #pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32(tS + 32 * c, *reinterpret_cast<uint32_t(*)[32]>(&v[32 * c]));
      tmem_ld_wait();
      // four independent running maxima (and sums below): one serial chain over 128 values would leave this warp
      // waiting on its own ALU latency most of the time
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (need_mask) {
        #pragma unroll
        for (int i = 0; i < 128; ++i) {
          const int kj = k0 + i;
          bool vis = kj < p.S && (!p.causal || kj <= qi);
          if (need_kend) vis = vis && qi < s_kend[i];
          const float x = vis ? __uint_as_float(v[i]) : -INFINITY;
          v[i] = __float_as_uint(x);
          mx4[i & 3] = fmaxf(mx4[i & 3], x);
        }
      } else {
        #pragma unroll
        for (int i = 0; i < 128; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(v[i]));
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      const float m_new = fmaxf(m_used, mx * p.scale_log2);
      // lazy rescale: keep the old reference maximum unless some row of this warp has outgrown it by 2^8
      const bool grow = m_new > m_used + AF2_RESCALE_LOG2 || (m_used == -INFINITY && m_new != -INFINITY);
      if (__any_sync(0xffffffffu, grow)) {
        const float alpha = (m_new == -INFINITY) ? 1.f : fast_exp2(m_used - m_new);   // m_used = -inf -> 0
        if (jj > 0) {
          // O of this tile holds sums scaled by the old reference: wait for the last PV product, then rescale in place
          if (!mbar_wait(&o_full[t], (jj - 1) & 1, abort_flag, p.status, PFB_ERR_WAIT_TMEM_FULL)) { ok = false; break; }
          tc_fence_after();
          #pragma unroll 1
          for (int c = 0; c < ATT_D; c += 32) {
            uint32_t o[32];
            tmem_ld_32x32(tO + c, o);
            tmem_ld_wait();
            #pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x16(tO + c, *reinterpret_cast<uint32_t(*)[16]>(&o[0]));
            tmem_st_32x16(tO + c + 16, *reinterpret_cast<uint32_t(*)[16]>(&o[16]));
          }
        }
        l *= alpha;
        m_used = m_new;
      }
      const float m_sub = m_used == -INFINITY ? 0.f : m_used;
      float lt4[4] = {0.f, 0.f, 0.f, 0.f};
      #pragma unroll
      for (int c = 0; c < 128; c += 32) {
        uint32_t pk[16];
        #pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float p0 = fast_exp2(__uint_as_float(v[c + i]) * p.scale_log2 - m_sub);     // masked: exp2(-inf) = 0
          const float p1 = fast_exp2(__uint_as_float(v[c + i + 1]) * p.scale_log2 - m_sub);
          lt4[(i >> 1) & 3] += p0 + p1;
          pk[i >> 1] = pack_bf16x2(p0, p1);
        }
        tmem_st_32x16(tS + (c >> 1), pk);
      }
      const float lt = (lt4[0] + lt4[1]) + (lt4[2] + lt4[3]);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[t]);
      l += lt;
    }
    if (ok && nt > 0) ok = mbar_wait(&o_full[t], (nt - 1) & 1, abort_flag, p.status, PFB_ERR_WAIT_TMEM_FULL);
    if (ok && qt0 < p.S) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* dst = p.O + static_cast<long long>(row_base + qi) * p.o_row_stride + head * ATT_D;
      #pragma unroll 1
      for (int c = 0; c < ATT_D; c += 32) {
        uint32_t o[32];
        if (nt > 0) { tmem_ld_32x32(tO + c, o); tmem_ld_wait(); }
        else {
          #pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0u;
        }
        if (qi < p.S) {
          #pragma unroll
          for (int i = 0; i < 32; i += 8)
            *reinterpret_cast<uint4*>(dst + c + i) = make_uint4(
                pack_bf16x2(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv),
                pack_bf16x2(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv),
                pack_bf16x2(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv),
                pack_bf16x2(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv));
        }
      }
      if (qi < p.S)
        p.lse[(static_cast<long long>(b) * p.Hq + head) * p.S + qi] =
            l > 0.f ? (m_used + log2f(l)) * 0.6931471805599453f : -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 9) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

}  // namespace pfb
