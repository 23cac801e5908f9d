// Flash attention backward for sm_100a (head_dim 128, GQA, causal + document masks), tcgen05 + TMEM.
//
// One CTA owns one 128-key tile and one query head and walks over that head's query tiles (64 rows); with grouped
// queries the G heads of a KV head run as G CTAs whose fp32 dK / dV partials are summed by a small second kernel, so
// that the grid stays large when tensor parallelism leaves a rank a single KV head. All five products of the backward pass run on the tensor cores with the key dimension on the TMEM lanes:
//
//   S^T  = K  Q^T            (128 keys x 64 queries, fp32 in TMEM)
//   dP^T = V  dO^T
//   dV  += P^T  dO           (P^T  written back to TMEM as bf16, used as the A operand)
//   dK  += dS^T Q            (dS^T written back to TMEM as bf16, used as the A operand)
//   dQ^T = K^T dS^T          (128 head dims x 64 queries; dS^T also staged in swizzled smem as the B operand)
//
// dK and dV accumulate in TMEM over the whole walk and are written once; dQ^T is added to an fp32 accumulator with
// red.global (consecutive threads hit consecutive addresses). Thread r of the four compute warps owns key row r of
// the tile, so the causal / document mask is two integer compares per element against per-thread constants.
// Replaces the reference's flash-attention backward call sites (paddleformers/nn/attention/sink_impl.py:129-220,
// paddleformers/cli/train/deepseek_v3_pretrain/modeling.py:2520-2638).
#pragma once
#include "attention_sm100.cuh"

namespace pfb {

__device__ __forceinline__ void fence_proxy_async_all_bwd() { asm volatile("fence.proxy.async;" ::: "memory"); }

constexpr int ATTB_BKV = 128;
constexpr int ATTB_BQ = 64;
constexpr int ATTB_THREADS = 160;

struct AttnBwdParams {
  const float* lse;      // [B, Hq, S] natural log
  const float* delta;    // [B, Hq, S] rowsum(dO * O)
  float* dq_acc;         // [B*S, Hq, 128] fp32, zero-initialised
  __nv_bfloat16* dk;     // [B*S, Hkv, 128] views (row strides below, head stride 128)
  __nv_bfloat16* dv;
  float* dk_part;        // [B*S, Hq, 128] fp32 per-query-head partials (nullptr when Hq == Hkv)
  float* dv_part;
  long long dk_row_stride, dv_row_stride;
  const int* kend;           // [B, S] or nullptr
  const int* tile_min_end;   // [B, kv_tiles]
  const int* tile_max_end;
  int S, Hq, Hkv;
  float scale, scale_log2;
  int causal;
  int* status;
};

// DQK: width of queries / keys (128, or 192 for multi-head latent attention; values and dO stay 128 wide).
template <int DQK>
struct AttnBwdSmemT {
  static constexpr int KSLABS = DQK == 128 ? 2 : 4;       // 192: a fourth, zero-filled slab pads K^T to 256 rows for dQ^T
  static constexpr int K_SLAB = ATTB_BKV * 64 * 2;        // 16 KB: [128 keys x 64 columns]
  static constexpr int Q_SLAB = ATTB_BQ * 64 * 2;         // 8 KB:  [64 queries x 64 columns]
  static constexpr int K_TILE = KSLABS * K_SLAB;
  static constexpr int V_TILE = 2 * K_SLAB;
  static constexpr int Q_TILE = (DQK / 64) * Q_SLAB;
  static constexpr int DO_TILE = 2 * Q_SLAB;
  static constexpr int K_OFF = 0, V_OFF = K_TILE;
  static constexpr int Q_OFF = K_TILE + V_TILE;            // 2 stages x (Q, dO)
  static constexpr int DS_OFF = Q_OFF + 2 * (Q_TILE + DO_TILE);   // dS^T [128 keys x 64 q] bf16 = 16 KB
  static constexpr int STAT_OFF = DS_OFF + ATTB_BKV * ATTB_BQ * 2;  // per-warp lse / delta copies: 4 x 2 x 64 floats
  static constexpr int BAR_OFF = STAT_OFF + 4 * 2 * 64 * 4;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};
using AttnBwdSmem = AttnBwdSmemT<128>;

// One tile at a time (no overlap between the products and the element-wise work): the simple schedule. It is the only
// kernel for DQK = 192, where dK alone takes 192 TMEM columns and no second [S^T | dP^T] stage fits.
// TMEM: [S^T 0-63][dP^T 64-127][dQ^T(d < 128) 128-191][dV 192-319][dK 320-...]; P^T (bf16) over S^T columns 0-31, dS^T
// (bf16) over dP^T columns 96-127; for DQK = 192 the second half of dQ^T (head dims 128-191, computed as a 128-row
// product against the zero-padded K^T) goes to the dead columns 32-95 in between.
template <int DQK>
__global__ void __launch_bounds__(ATTB_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                const AttnBwdParams p) {
  using SM = AttnBwdSmemT<DQK>;
  constexpr bool MLA = DQK != 128;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem + SM::K_OFF; uint8_t* sV = smem + SM::V_OFF;
  uint8_t* sdS = smem + SM::DS_OFF;
  float* s_stat_all = reinterpret_cast<float*>(smem + SM::STAT_OFF);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::BAR_OFF);
  uint64_t* bar_kv = bars; uint64_t* bar_q = bars + 1;  // [2]
  uint64_t* bar_s = bars + 3; uint64_t* bar_p = bars + 4; uint64_t* bar_ds = bars + 5;
  uint64_t* bar_dq = bars + 6; uint64_t* bar_dqread = bars + 7;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int jt = blockIdx.x, head = blockIdx.y, b = blockIdx.z;
  const int G = p.Hq / p.Hkv;
  const int kvh = head / G;
  const int k0 = jt * ATTB_BKV;
  const int row_base = b * p.S;
  const int kv_tiles = (p.S + ATTB_BKV - 1) / ATTB_BKV;

  if (threadIdx.x == 0) {
    mbar_init(bar_kv, 1); mbar_init(&bar_q[0], 1); mbar_init(&bar_q[1], 1);
    mbar_init(bar_s, 1); mbar_init(bar_p, 4); mbar_init(bar_ds, 4); mbar_init(bar_dq, 1); mbar_init(bar_dqread, 4);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 4) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); tc_fence_before(); }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base, tdP = tmem_base + 64, tdQ = tmem_base + 128, tdV = tmem_base + 192, tdK = tmem_base + 320;
  const uint32_t tdQb = tmem_base + 32;     // DQK = 192 only

  // query tile range visible to this key tile
  const int q_tiles = (p.S + ATTB_BQ - 1) / ATTB_BQ;
  int i_lo = p.causal ? k0 / ATTB_BQ : 0;
  int i_hi = q_tiles - 1;
  int tmin_end = 0x7fffffff;
  if (p.kend) {
    const int tmax = p.tile_max_end[b * kv_tiles + jt];
    tmin_end = p.tile_min_end[b * kv_tiles + jt];
    i_hi = min(i_hi, (tmax - 1) / ATTB_BQ);
  }
  const int n_q = max(i_hi - i_lo + 1, 0);
  const int n_it = n_q;

  if (warp == 4) {
    if (lane == 0 && n_it > 0) {
      constexpr uint32_t idesc_s = make_idesc(128, ATTB_BQ, false, false, 1);   // K-major x K-major
      constexpr uint32_t idesc_dv = make_idesc(128, ATT_D, false, true, 1);      // TMEM A x MN-major B
      constexpr uint32_t idesc_dk = make_idesc(128, DQK, false, true, 1);
      constexpr uint32_t idesc_dq = make_idesc(128, ATTB_BQ, true, true, 1);     // MN-major x MN-major
      auto load_q = [&](int it) {
        const int i = i_lo + it;
        const int st = it & 1;
        uint8_t* sq = smem + SM::Q_OFF + st * (SM::Q_TILE + SM::DO_TILE);
        uint8_t* sdo = sq + SM::Q_TILE;
        mbar_expect_tx(&bar_q[st], SM::Q_TILE + SM::DO_TILE);
        #pragma unroll
        for (int sl = 0; sl < DQK / 64; ++sl) tma_load_3d(sq + sl * SM::Q_SLAB, &tmQ, &bar_q[st], 64 * sl, head, row_base + i * ATTB_BQ);
        tma_load_3d(sdo, &tmdO, &bar_q[st], 0, head, row_base + i * ATTB_BQ);
        tma_load_3d(sdo + SM::Q_SLAB, &tmdO, &bar_q[st], 64, head, row_base + i * ATTB_BQ);
      };
      mbar_expect_tx(bar_kv, SM::K_TILE + SM::V_TILE);
      #pragma unroll
      for (int sl = 0; sl < SM::KSLABS; ++sl)       // a slab that starts at or beyond column DQK reads as zeros
        tma_load_3d(sK + sl * SM::K_SLAB, &tmK, bar_kv, 64 * sl, kvh, row_base + k0);
      tma_load_3d(sV, &tmV, bar_kv, 0, kvh, row_base + k0);
      tma_load_3d(sV + SM::K_SLAB, &tmV, bar_kv, 64, kvh, row_base + k0);
      load_q(0);
      bool ok = mbar_wait(bar_kv, 0, abort_flag, p.status, PFB_ERR_WAIT_FULL);
      for (int it = 0; it < n_it && ok; ++it) {
        const int st = it & 1;
        const uint32_t ph = it & 1, qph = (it >> 1) & 1;
        const uint32_t sq = smem_u32(smem + SM::Q_OFF + st * (SM::Q_TILE + SM::DO_TILE));
        const uint32_t sdo = sq + SM::Q_TILE;
        if (!mbar_wait(&bar_q[st], qph, abort_flag, p.status, PFB_ERR_WAIT_FULL)) break;
        if constexpr (MLA) {
          // the second half of dQ^T of the previous tile sits in columns that S^T / dP^T are about to overwrite
          if (it > 0 && !mbar_wait(bar_dqread, (it - 1) & 1, abort_flag, p.status, PFB_ERR_WAIT_TMEM_EMPTY)) break;
        }
        tc_fence_after();
        #pragma unroll
        for (int k = 0; k < DQK / 16; ++k) {
          const uint32_t offk = (k >> 2) * SM::K_SLAB + (k & 3) * 32;
          const uint32_t offq = (k >> 2) * SM::Q_SLAB + (k & 3) * 32;
          tc_mma_f16_ss(tS, make_smem_desc_sw128(smem_u32(sK) + offk, 16, 1024), make_smem_desc_sw128(sq + offq, 16, 1024),
                        idesc_s, k != 0);
        }
        #pragma unroll
        for (int k = 0; k < ATT_D / 16; ++k) {
          const uint32_t offk = (k >> 2) * SM::K_SLAB + (k & 3) * 32;
          const uint32_t offq = (k >> 2) * SM::Q_SLAB + (k & 3) * 32;
          tc_mma_f16_ss(tdP, make_smem_desc_sw128(smem_u32(sV) + offk, 16, 1024), make_smem_desc_sw128(sdo + offq, 16, 1024),
                        idesc_s, k != 0);
        }
        tc_commit(bar_s);
        if (it > 0) {
          // stage st^1 was read by the MMAs of iteration it-1: free once they have completed
          if (!mbar_wait(bar_dq, (it - 1) & 1, abort_flag, p.status, PFB_ERR_WAIT_TMEM_FULL)) break;
        }
        if (it + 1 < n_it) load_q(it + 1);
        if (!mbar_wait(bar_p, ph, abort_flag, p.status, PFB_ERR_WAIT_TMEM_EMPTY)) break;
        tc_fence_after();
        #pragma unroll
        for (int k = 0; k < ATTB_BQ / 16; ++k)
          tc_mma_f16_ts(tdV, tS + k * 8, make_smem_desc_sw128(sdo + k * 16 * 128, SM::Q_SLAB, 1024), idesc_dv, (it | k) != 0);
        if (!mbar_wait(bar_ds, ph, abort_flag, p.status, PFB_ERR_WAIT_TMEM_EMPTY)) break;
        tc_fence_after();
        #pragma unroll
        for (int k = 0; k < ATTB_BQ / 16; ++k)
          tc_mma_f16_ts(tdK, tdP + 32 + k * 8, make_smem_desc_sw128(sq + k * 16 * 128, SM::Q_SLAB, 1024), idesc_dk, (it | k) != 0);
        if (it > 0) {
          if (!mbar_wait(bar_dqread, (it - 1) & 1, abort_flag, p.status, PFB_ERR_WAIT_TMEM_EMPTY)) break;
          tc_fence_after();
        }
        #pragma unroll
        for (int k = 0; k < ATTB_BKV / 16; ++k)
          tc_mma_f16_ss(tdQ, make_smem_desc_sw128(smem_u32(sK) + k * 16 * 128, SM::K_SLAB, 1024),
                        make_smem_desc_sw128(smem_u32(sdS) + k * 16 * 128, 16, 1024), idesc_dq, k != 0);
        if constexpr (MLA) {
          // head dims 128-255 of K^T (192-255 are the zero slab): its own 128-row product into the dead columns
          #pragma unroll
          for (int k = 0; k < ATTB_BKV / 16; ++k)
            tc_mma_f16_ss(tdQb, make_smem_desc_sw128(smem_u32(sK) + 2 * SM::K_SLAB + k * 16 * 128, SM::K_SLAB, 1024),
                          make_smem_desc_sw128(smem_u32(sdS) + k * 16 * 128, 16, 1024), idesc_dq, k != 0);
        }
        tc_commit(bar_dq);
      }
    }
  } else {
    // ---------------- compute warps: thread r owns key row k0 + r ----------------
    const int r = threadIdx.x;
    const int kj = k0 + r;
    const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;
    float* s_lse = s_stat_all + warp * 128;
    float* s_delta = s_lse + 64;
    const int my_kend = (p.kend && kj < p.S) ? p.kend[b * p.S + kj] : 0x7fffffff;
    bool ok = true;
    for (int it = 0; it < n_it; ++it) {
      const uint32_t ph = it & 1;
      const int i = i_lo + it;
      const int q0 = i * ATTB_BQ;
      // stage this tile's lse (in log2 units) and delta: every warp keeps a private copy
      __syncwarp();
      {
        const long long base = (static_cast<long long>(b) * p.Hq + head) * p.S;
        #pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int qi = q0 + lane + 32 * c;
          s_lse[lane + 32 * c] = qi < p.S ? p.lse[base + qi] * 1.4426950408889634f : 0.f;
          s_delta[lane + 32 * c] = qi < p.S ? p.delta[base + qi] : 0.f;
        }
      }
      __syncwarp();
      const bool need_mask = (p.causal && q0 < k0 + ATTB_BKV) || (q0 + ATTB_BQ > p.S) || (k0 + ATTB_BKV > p.S) ||
                             (q0 + ATTB_BQ > tmin_end);
      if (!mbar_wait(bar_s, ph, abort_flag, p.status, PFB_ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      float pv[ATTB_BQ];
      #pragma unroll
      for (int c = 0; c < ATTB_BQ; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(tS + lane_off + c, v);
        tmem_ld_wait();
        #pragma unroll
        for (int x = 0; x < 32; x += 2) {
          float p0 = fast_exp2(__uint_as_float(v[x]) * p.scale_log2 - s_lse[c + x]);
          float p1 = fast_exp2(__uint_as_float(v[x + 1]) * p.scale_log2 - s_lse[c + x + 1]);
          if (need_mask) {
            const int qi = q0 + c + x;
            const bool v0 = qi < p.S && kj < p.S && (!p.causal || kj <= qi) && qi < my_kend;
            const bool v1 = qi + 1 < p.S && kj < p.S && (!p.causal || kj <= qi + 1) && qi + 1 < my_kend;
            p0 = v0 ? p0 : 0.f; p1 = v1 ? p1 : 0.f;
          }
          pv[c + x] = p0; pv[c + x + 1] = p1;
        }
      }
      #pragma unroll
      for (int c = 0; c < ATTB_BQ; c += 32) {       // after ALL raw scores of this lane have been read
        uint32_t pk[16];
        #pragma unroll
        for (int x = 0; x < 32; x += 2) pk[x >> 1] = pack_bf16x2(pv[c + x], pv[c + x + 1]);
        tmem_st_32x16(tS + lane_off + (c >> 1), pk);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_p);
      // dS^T = P^T * (dP^T - delta) * scale
      uint32_t dsk[ATTB_BQ / 2];
      #pragma unroll
      for (int c = 0; c < ATTB_BQ; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(tdP + lane_off + c, v);
        tmem_ld_wait();
        #pragma unroll
        for (int x = 0; x < 32; x += 2) {
          const float d0 = pv[c + x] * (__uint_as_float(v[x]) - s_delta[c + x]) * p.scale;
          const float d1 = pv[c + x + 1] * (__uint_as_float(v[x + 1]) - s_delta[c + x + 1]) * p.scale;
          dsk[(c + x) >> 1] = pack_bf16x2(d0, d1);
        }
      }
      uint8_t* rowp = sdS + r * 128;
      #pragma unroll
      for (int c = 0; c < ATTB_BQ; c += 32) {
        uint32_t pk[16];
        #pragma unroll
        for (int x = 0; x < 16; ++x) pk[x] = dsk[(c >> 1) + x];
        tmem_st_32x16(tdP + lane_off + 32 + (c >> 1), pk);
        #pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const int chunk = (c >> 3) + q4;
          *reinterpret_cast<uint4*>(rowp + ((chunk ^ (r & 7)) << 4)) = make_uint4(pk[4 * q4], pk[4 * q4 + 1], pk[4 * q4 + 2], pk[4 * q4 + 3]);
        }
      }
      tmem_st_wait();
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_ds);
      // dQ^T tile(s): lane (TMEM) index = head dim, columns = the 64 queries
      if (!mbar_wait(bar_dq, ph, abort_flag, p.status, PFB_ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const long long qstride = static_cast<long long>(p.Hq) * DQK;
      #pragma unroll 1
      for (int hb = 0; hb < (MLA ? 2 : 1); ++hb) {
        uint32_t dq0[32], dq1[32];
        const uint32_t src = hb == 0 ? tdQ : tdQb;
        tmem_ld_32x32(src + lane_off, dq0);
        tmem_ld_32x32(src + lane_off + 32, dq1);
        tmem_ld_wait();
        const int d = hb * 128 + r;
        if (d < DQK) {
          float* acc = p.dq_acc + (static_cast<long long>(row_base + q0) * p.Hq + head) * DQK + d;
          #pragma unroll
          for (int x = 0; x < 32; ++x)
            if (q0 + x < p.S) atomicAdd(acc + x * qstride, __uint_as_float(dq0[x]));
          #pragma unroll
          for (int x = 0; x < 32; ++x)
            if (q0 + 32 + x < p.S) atomicAdd(acc + (32 + x) * qstride, __uint_as_float(dq1[x]));
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_dqread);
    }
    // dK, dV: one key row per thread
    if (ok) {
      if (n_it > 0) tc_fence_after();
      __nv_bfloat16* dkp = p.dk + static_cast<long long>(row_base + kj) * p.dk_row_stride + kvh * DQK;
      __nv_bfloat16* dvp = p.dv + static_cast<long long>(row_base + kj) * p.dv_row_stride + kvh * ATT_D;
      #pragma unroll 1
      for (int c = 0; c < DQK; c += 32) {
        uint32_t a[32], bb[32];
        const bool has_v = c < ATT_D;
        if (n_it > 0) {
          tmem_ld_32x32(tdK + lane_off + c, a);
          if (has_v) tmem_ld_32x32(tdV + lane_off + c, bb);
          tmem_ld_wait();
        } else {
          #pragma unroll
          for (int x = 0; x < 32; ++x) { a[x] = 0u; bb[x] = 0u; }
        }
        if (kj < p.S && p.dk_part != nullptr) {
          float* pk = p.dk_part + (static_cast<long long>(row_base + kj) * p.Hq + head) * DQK + c;
          #pragma unroll
          for (int x = 0; x < 32; x += 4)
            *reinterpret_cast<float4*>(pk + x) = make_float4(__uint_as_float(a[x]), __uint_as_float(a[x + 1]), __uint_as_float(a[x + 2]), __uint_as_float(a[x + 3]));
          if (has_v) {
            float* pv2 = p.dv_part + (static_cast<long long>(row_base + kj) * p.Hq + head) * ATT_D + c;
            #pragma unroll
            for (int x = 0; x < 32; x += 4)
              *reinterpret_cast<float4*>(pv2 + x) = make_float4(__uint_as_float(bb[x]), __uint_as_float(bb[x + 1]), __uint_as_float(bb[x + 2]), __uint_as_float(bb[x + 3]));
          }
        } else if (kj < p.S) {
          #pragma unroll
          for (int x = 0; x < 32; x += 8)
            *reinterpret_cast<uint4*>(dkp + c + x) = make_uint4(
                pack_bf16x2(__uint_as_float(a[x]), __uint_as_float(a[x + 1])), pack_bf16x2(__uint_as_float(a[x + 2]), __uint_as_float(a[x + 3])),
                pack_bf16x2(__uint_as_float(a[x + 4]), __uint_as_float(a[x + 5])), pack_bf16x2(__uint_as_float(a[x + 6]), __uint_as_float(a[x + 7])));
          if (has_v) {
            #pragma unroll
            for (int x = 0; x < 32; x += 8)
              *reinterpret_cast<uint4*>(dvp + c + x) = make_uint4(
                  pack_bf16x2(__uint_as_float(bb[x]), __uint_as_float(bb[x + 1])), pack_bf16x2(__uint_as_float(bb[x + 2]), __uint_as_float(bb[x + 3])),
                  pack_bf16x2(__uint_as_float(bb[x + 4]), __uint_as_float(bb[x + 5])), pack_bf16x2(__uint_as_float(bb[x + 6]), __uint_as_float(bb[x + 7])));
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 4) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

// ------------------------------------------------------------------------------------------------------------------
// Pipelined backward (the default). Same mathematics and operand layouts as attn_bwd_kernel above, but the work of a
// query tile is spread over four roles that run concurrently on several tiles:
//
//   warp 12    TMA loader: K, V once; Q / dO tiles through a three-stage ring
//   warp 13    MMA issuer: S^T and dP^T run TWO tiles ahead of the dV / dK / dQ products, so the tensor pipe always has
//              queued work while the compute warps handle a tile, and no product waits for a round trip through
//              another warp except dP^T(i+2), which needs the dQ warps to have emptied the columns it reuses
//   warps 0-7  compute: P^T = exp2(S^T - lse), dS^T = P^T (dP^T - delta) scale; both are written back to TMEM as bf16
//              (A operands of the dV / dK products) and dS^T also to swizzled shared memory (B operand of dQ^T).
//              Two warps share a TMEM lane quadrant (32 key rows) and split the 64 query columns, so that every
//              scheduler has two compute warps to interleave: one warp per scheduler leaves the ALU latencies exposed
//   warps 8-11 dQ: read dQ^T from TMEM, transpose through shared memory, and add it to the fp32 accumulator with one
//              TMA reduce-add per 32 query rows (instead of per-element atomics). With `deterministic` the adds of one
//              query tile happen in a fixed order (descending key tile): every CTA takes its turn on a per-tile counter.
//
// TMEM (512 columns): two stages of [S^T 64 | dP^T 64], dV 128, dK 128. Each half-warp group overwrites its OWN 32 raw
// score columns: P^T (bf16) the first 16 of them, dS^T (bf16) the last 16, so the two groups never touch each other's
// columns and need no barrier; the dP^T columns 64-127 are dead once dS^T exists and receive dQ^T, so no separate dQ accumulator is needed, and S^T(i+2) can be issued into columns 0-63 as
// soon as the products that read P^T(i) / dS^T(i) have been issued (the tensor pipe executes in order).
// With `heads_per_cta` = G the CTA walks all query heads of its KV head and dK / dV accumulate over them in TMEM (no
// fp32 partials); with 1 it owns one query head (keeps the grid large when a rank has few KV heads).
constexpr int AB2_THREADS = 448;
constexpr int AB2_QSTAGES = 3;

struct AttnBwd2Params {
  AttnBwdParams base;
  int heads_per_cta;     // Hq / Hkv, or 1
  int deterministic;     // 1: ordered dQ accumulation
  int* dq_turn;          // [B, Hq, q_tiles] zero-initialised counters (deterministic mode)
};

struct AttnBwd2Smem {
  static constexpr int KV_TILE = ATTB_BKV * ATT_D * 2;   // 32 KB
  static constexpr int Q_TILE = ATTB_BQ * ATT_D * 2;     // 16 KB
  static constexpr int K_OFF = 0, V_OFF = KV_TILE;
  static constexpr int Q_OFF = 2 * KV_TILE;                               // QSTAGES x (Q, dO)
  static constexpr int DS_OFF = Q_OFF + AB2_QSTAGES * 2 * Q_TILE;         // 2 x dS^T [128 keys x 64 q] bf16
  static constexpr int DQ_OFF = DS_OFF + 2 * ATTB_BKV * ATTB_BQ * 2;      // fp32 [32 q x 128 d] staging for the reduce-add
  static constexpr int STAT_OFF = DQ_OFF + 32 * ATT_D * 4;                // per compute warp: lse[32], delta[32]
  static constexpr int BAR_OFF = STAT_OFF + 8 * 2 * 32 * 4;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

__device__ __forceinline__ void tma_reduce_add_3d(const CUtensorMap* m, const void* smem_src, int c0, int c1, int c2) {
  asm volatile("cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}
__device__ __forceinline__ void named_bar_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__global__ void __launch_bounds__(AB2_THREADS, 1)
attn_bwd2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                 const __grid_constant__ CUtensorMap tmdQ, const AttnBwd2Params pp) {
  using SM = AttnBwd2Smem;
  const AttnBwdParams& p = pp.base;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem + SM::K_OFF; uint8_t* sV = smem + SM::V_OFF;
  float* sDQ = reinterpret_cast<float*>(smem + SM::DQ_OFF);
  float* s_stat_all = reinterpret_cast<float*>(smem + SM::STAT_OFF);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::BAR_OFF);
  uint64_t* bar_kv = bars;                 // 1
  uint64_t* q_full = bars + 1;             // [3]
  uint64_t* q_empty = bars + 4;            // [3]
  uint64_t* bar_s = bars + 7;              // [2]
  uint64_t* bar_dp = bars + 9;             // [2]
  uint64_t* bar_p = bars + 11;             // [2]
  uint64_t* bar_ds = bars + 13;            // [2]
  uint64_t* bar_dq = bars + 15;            // [2]
  uint64_t* dq_read = bars + 17;           // [2]
  uint64_t* bar_done = bars + 19;          // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 20);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kv_tiles = (p.S + ATTB_BKV - 1) / ATTB_BKV;
  // deterministic mode: a CTA waits for the CTA of the next key tile, which must therefore have the lower block index;
  // otherwise the heavy (early) key tiles of a causal mask start first
  const int jt = pp.deterministic ? kv_tiles - 1 - static_cast<int>(blockIdx.x) : static_cast<int>(blockIdx.x);
  const int b = blockIdx.z;
  const int G = p.Hq / p.Hkv;
  const int HPC = pp.heads_per_cta;
  const int head0 = HPC == 1 ? static_cast<int>(blockIdx.y) : static_cast<int>(blockIdx.y) * G;
  const int kvh = head0 / G;
  const int k0 = jt * ATTB_BKV;
  const int row_base = b * p.S;

  if (threadIdx.x == 0) {
    mbar_init(bar_kv, 1);
    for (int s = 0; s < AB2_QSTAGES; ++s) { mbar_init(&q_full[s], 1); mbar_init(&q_empty[s], 1); }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bar_s[s], 1); mbar_init(&bar_dp[s], 1); mbar_init(&bar_p[s], 8); mbar_init(&bar_ds[s], 8);
      mbar_init(&bar_dq[s], 1); mbar_init(&dq_read[s], 4);
    }
    mbar_init(bar_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 13) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); tc_fence_before(); }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tdV = tmem_base + 256, tdK = tmem_base + 384;

  // query tile range visible to this key tile
  const int q_tiles = (p.S + ATTB_BQ - 1) / ATTB_BQ;
  const int i_lo = p.causal ? k0 / ATTB_BQ : 0;
  int i_hi = q_tiles - 1;
  int tmin_end = 0x7fffffff;
  if (p.kend) {
    const int tmax = p.tile_max_end[b * kv_tiles + jt];
    tmin_end = p.tile_min_end[b * kv_tiles + jt];
    i_hi = min(i_hi, (tmax - 1) / ATTB_BQ);
  }
  const int n_q = max(i_hi - i_lo + 1, 0);
  const int n_it = n_q * HPC;

  if (warp == 12) {
    // ------------------------------------------------------------ TMA loader
    if (lane == 0 && n_it > 0) {
      mbar_expect_tx(bar_kv, 2 * SM::KV_TILE);
      tma_load_3d(sK, &tmK, bar_kv, 0, kvh, row_base + k0);
      tma_load_3d(sK + SM::KV_TILE / 2, &tmK, bar_kv, 64, kvh, row_base + k0);
      tma_load_3d(sV, &tmV, bar_kv, 0, kvh, row_base + k0);
      tma_load_3d(sV + SM::KV_TILE / 2, &tmV, bar_kv, 64, kvh, row_base + k0);
      int st = 0; uint32_t ph = 0;
      for (int it = 0; it < n_it; ++it) {
        const int g = it / n_q, i = i_lo + (it - g * n_q);
        if (!mbar_wait(&q_empty[st], ph ^ 1, abort_flag, p.status, PFB_ERR_WAIT_EMPTY)) break;
        uint8_t* sq = smem + SM::Q_OFF + st * 2 * SM::Q_TILE;
        uint8_t* sdo = sq + SM::Q_TILE;
        mbar_expect_tx(&q_full[st], 2 * SM::Q_TILE);
        tma_load_3d(sq, &tmQ, &q_full[st], 0, head0 + g, row_base + i * ATTB_BQ);
        tma_load_3d(sq + SM::Q_TILE / 2, &tmQ, &q_full[st], 64, head0 + g, row_base + i * ATTB_BQ);
        tma_load_3d(sdo, &tmdO, &q_full[st], 0, head0 + g, row_base + i * ATTB_BQ);
        tma_load_3d(sdo + SM::Q_TILE / 2, &tmdO, &q_full[st], 64, head0 + g, row_base + i * ATTB_BQ);
        if (++st == AB2_QSTAGES) { st = 0; ph ^= 1; }
      }
    }
  } else if (warp == 13) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0 && n_it > 0) {
      constexpr uint32_t idesc_s = make_idesc(128, ATTB_BQ, false, false, 1);   // K-major x K-major
      constexpr uint32_t idesc_dkv = make_idesc(128, ATT_D, false, true, 1);     // TMEM A x MN-major B
      constexpr uint32_t idesc_dq = make_idesc(128, ATTB_BQ, true, true, 1);     // MN-major x MN-major
      bool ok = mbar_wait(bar_kv, 0, abort_flag, p.status, PFB_ERR_WAIT_FULL);
      auto issue_s = [&](int it) -> bool {
        const int qs = it % AB2_QSTAGES, st = it & 1;
        if (!mbar_wait(&q_full[qs], (it / AB2_QSTAGES) & 1, abort_flag, p.status, PFB_ERR_WAIT_FULL)) return false;
        tc_fence_after();
        const uint32_t sq = smem_u32(smem + SM::Q_OFF + qs * 2 * SM::Q_TILE);
        #pragma unroll
        for (int k = 0; k < ATT_D / 16; ++k) {
          const uint32_t offk = (k >> 2) * (SM::KV_TILE / 2) + (k & 3) * 32;
          const uint32_t offq = (k >> 2) * (SM::Q_TILE / 2) + (k & 3) * 32;
          tc_mma_f16_ss(tmem_base + st * 128, make_smem_desc_sw128(smem_u32(sK) + offk, 16, 1024),
                        make_smem_desc_sw128(sq + offq, 16, 1024), idesc_s, k != 0);
        }
        tc_commit(&bar_s[st]);
        return true;
      };
      auto issue_dp = [&](int it) {
        const int qs = it % AB2_QSTAGES, st = it & 1;
        const uint32_t sdo = smem_u32(smem + SM::Q_OFF + qs * 2 * SM::Q_TILE) + SM::Q_TILE;
        #pragma unroll
        for (int k = 0; k < ATT_D / 16; ++k) {
          const uint32_t offk = (k >> 2) * (SM::KV_TILE / 2) + (k & 3) * 32;
          const uint32_t offq = (k >> 2) * (SM::Q_TILE / 2) + (k & 3) * 32;
          tc_mma_f16_ss(tmem_base + st * 128 + 64, make_smem_desc_sw128(smem_u32(sV) + offk, 16, 1024),
                        make_smem_desc_sw128(sdo + offq, 16, 1024), idesc_s, k != 0);
        }
        tc_commit(&bar_dp[st]);
      };
      // both stages start empty: the first two tiles' S^T / dP^T need no hand-shake
      for (int it = 0; it < 2 && it < n_it && ok; ++it) {
        ok = issue_s(it);
        if (ok) issue_dp(it);
      }
      for (int it = 0; it < n_it && ok; ++it) {
        const int st = it & 1, qs = it % AB2_QSTAGES;
        const uint32_t ph2 = (it >> 1) & 1;
        const uint32_t stage = tmem_base + st * 128;
        const uint32_t sq = smem_u32(smem + SM::Q_OFF + qs * 2 * SM::Q_TILE);
        const uint32_t sdo = sq + SM::Q_TILE;
        if (!mbar_wait(&bar_p[st], ph2, abort_flag, p.status, PFB_ERR_WAIT_TMEM_EMPTY)) break;
        tc_fence_after();
        #pragma unroll
        for (int k = 0; k < ATTB_BQ / 16; ++k)
          tc_mma_f16_ts(tdV, stage + (k >> 1) * 32 + (k & 1) * 8, make_smem_desc_sw128(sdo + k * 16 * 128, SM::Q_TILE / 2, 1024), idesc_dkv,
                        (it | k) != 0);
        if (!mbar_wait(&bar_ds[st], ph2, abort_flag, p.status, PFB_ERR_WAIT_TMEM_EMPTY)) break;
        tc_fence_after();
        // dQ^T first: its consumers (the dQ warps) get a head start while dK runs
        const uint32_t sds = smem_u32(smem + SM::DS_OFF + st * (ATTB_BKV * ATTB_BQ * 2));
        #pragma unroll
        for (int k = 0; k < ATTB_BKV / 16; ++k)
          tc_mma_f16_ss(stage + 64, make_smem_desc_sw128(smem_u32(sK) + k * 16 * 128, SM::KV_TILE / 2, 1024),
                        make_smem_desc_sw128(sds + k * 16 * 128, 16, 1024), idesc_dq, k != 0);
        tc_commit(&bar_dq[st]);
        #pragma unroll
        for (int k = 0; k < ATTB_BQ / 16; ++k)
          tc_mma_f16_ts(tdK, stage + (k >> 1) * 32 + 16 + (k & 1) * 8, make_smem_desc_sw128(sq + k * 16 * 128, SM::Q_TILE / 2, 1024), idesc_dkv,
                        (it | k) != 0);
        tc_commit(&q_empty[qs]);   // Q / dO of this tile are no longer read once everything issued so far has run
        if (it + 2 < n_it) {
          // columns 0-63 of this stage: P^T / dS^T of tile it are read by products issued above (in-order pipe)
          if (!issue_s(it + 2)) break;
          // columns 64-127 hold dQ^T of tile it until the dQ warps have read it
          if (!mbar_wait(&dq_read[st], ph2, abort_flag, p.status, PFB_ERR_WAIT_TMEM_EMPTY)) break;
          tc_fence_after();
          issue_dp(it + 2);
        }
      }
      tc_commit(bar_done);
    }
  } else if (warp < 8) {
    // ------------------------------------------------------------ compute warps: thread owns key row k0 + r and the
    // 32 query columns of its half
    const int quad = warp & 3, half = warp >> 2;
    const int r = quad * 32 + lane;
    const int kj = k0 + r;
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    float* s_lse = s_stat_all + warp * 64;
    float* s_delta = s_lse + 32;
    const int my_kend = (p.kend && kj < p.S) ? p.kend[b * p.S + kj] : 0x7fffffff;
    bool ok = true;
    // statistics of the first tile; those of tile it+1 are fetched while tile it is being processed
    float nl, nd;
    auto fetch_stats = [&](int it) {
      const int g = it / n_q, i = i_lo + (it - g * n_q);
      const long long base = (static_cast<long long>(b) * p.Hq + head0 + g) * p.S;
      const int qi = i * ATTB_BQ + half * 32 + lane;
      nl = qi < p.S ? p.lse[base + qi] * 1.4426950408889634f : 0.f;
      nd = qi < p.S ? p.delta[base + qi] : 0.f;
    };
    if (n_it > 0) fetch_stats(0);
    for (int it = 0; it < n_it; ++it) {
      const int st = it & 1;
      const uint32_t ph2 = (it >> 1) & 1;
      const int g = it / n_q, i = i_lo + (it - g * n_q);
      const int q0 = i * ATTB_BQ + half * 32;            // first query of this thread's 32 columns
      const uint32_t tS = tmem_base + st * 128 + half * 32 + lane_off, tdP = tS + 64;
      __syncwarp();
      s_lse[lane] = nl;
      s_delta[lane] = nd;
      __syncwarp();
      if (it + 1 < n_it) fetch_stats(it + 1);
      const bool need_mask = (p.causal && q0 < k0 + ATTB_BKV) || (q0 + 32 > p.S) || (k0 + ATTB_BKV > p.S) || (q0 + 32 > tmin_end);
      // the row statistics go to registers with a few vector loads before the wait: while the tensor pipe streams its
      // operands out of shared memory, scalar shared-memory reads inside the loops below would queue behind them
      float ls[32];
      #pragma unroll
      for (int x = 0; x < 32; x += 4) {
        const float4 t4 = *reinterpret_cast<const float4*>(s_lse + x);
        ls[x] = t4.x; ls[x + 1] = t4.y; ls[x + 2] = t4.z; ls[x + 3] = t4.w;
      }
      if (!mbar_wait(&bar_s[st], ph2, abort_flag, p.status, PFB_ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      float pv[32];
      {
        uint32_t v[32];
        tmem_ld_32x32(tS, v);
        tmem_ld_wait();
        #pragma unroll
        for (int x = 0; x < 32; x += 2) {
          float p0 = fast_exp2(__uint_as_float(v[x]) * p.scale_log2 - ls[x]);
          float p1 = fast_exp2(__uint_as_float(v[x + 1]) * p.scale_log2 - ls[x + 1]);
          if (need_mask) {
            const int qi = q0 + x;
            const bool v0 = qi < p.S && kj < p.S && (!p.causal || kj <= qi) && qi < my_kend;
            const bool v1 = qi + 1 < p.S && kj < p.S && (!p.causal || kj <= qi + 1) && qi + 1 < my_kend;
            p0 = v0 ? p0 : 0.f; p1 = v1 ? p1 : 0.f;
          }
          pv[x] = p0; pv[x + 1] = p1;
        }
      }
      {
        // the 32 raw scores of this thread have been read: P^T (bf16) overwrites the first 16 of their columns
        uint32_t pk[16];
        #pragma unroll
        for (int x = 0; x < 32; x += 2) pk[x >> 1] = pack_bf16x2(pv[x], pv[x + 1]);
        tmem_st_32x16(tS, pk);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar_p[st]);
      // dS^T = P^T * (dP^T - delta) * scale
      #pragma unroll
      for (int x = 0; x < 32; x += 4) {
        const float4 t4 = *reinterpret_cast<const float4*>(s_delta + x);
        ls[x] = t4.x; ls[x + 1] = t4.y; ls[x + 2] = t4.z; ls[x + 3] = t4.w;
      }
      if (!mbar_wait(&bar_dp[st], ph2, abort_flag, p.status, PFB_ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      uint32_t pk[16];
      {
        uint32_t v[32];
        tmem_ld_32x32(tdP, v);
        tmem_ld_wait();
        #pragma unroll
        for (int x = 0; x < 32; x += 2) {
          const float d0 = pv[x] * (__uint_as_float(v[x]) - ls[x]) * p.scale;
          const float d1 = pv[x + 1] * (__uint_as_float(v[x + 1]) - ls[x + 1]) * p.scale;
          pk[x >> 1] = pack_bf16x2(d0, d1);
        }
      }
      tmem_st_32x16(tS + 16, pk);       // dS^T: the last 16 of this thread's raw score columns
      uint8_t* rowp = smem + SM::DS_OFF + st * (ATTB_BKV * ATTB_BQ * 2) + r * 128;
      #pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        const int chunk = half * 4 + q4;
        *reinterpret_cast<uint4*>(rowp + ((chunk ^ (r & 7)) << 4)) = make_uint4(pk[4 * q4], pk[4 * q4 + 1], pk[4 * q4 + 2], pk[4 * q4 + 3]);
      }
      tmem_st_wait();
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar_ds[st]);
    }
    // dK, dV: one key row per thread, the two halves take 64 head dims each
    if (ok && n_it > 0) ok = mbar_wait(bar_done, 0, abort_flag, p.status, PFB_ERR_WAIT_TMEM_FULL);
    if (ok) {
      if (n_it > 0) tc_fence_after();
      const bool partial = p.dk_part != nullptr && HPC == 1;
      __nv_bfloat16* dkp = p.dk + static_cast<long long>(row_base + kj) * p.dk_row_stride + kvh * ATT_D;
      __nv_bfloat16* dvp = p.dv + static_cast<long long>(row_base + kj) * p.dv_row_stride + kvh * ATT_D;
      #pragma unroll 1
      for (int c = half * 64; c < half * 64 + 64; c += 32) {
        uint32_t a[32], bb[32];
        if (n_it > 0) {
          tmem_ld_32x32(tdK + lane_off + c, a);
          tmem_ld_32x32(tdV + lane_off + c, bb);
          tmem_ld_wait();
        } else {
          #pragma unroll
          for (int x = 0; x < 32; ++x) { a[x] = 0u; bb[x] = 0u; }
        }
        if (kj < p.S && partial) {
          float* pk = p.dk_part + (static_cast<long long>(row_base + kj) * p.Hq + head0) * ATT_D + c;
          float* pv2 = p.dv_part + (static_cast<long long>(row_base + kj) * p.Hq + head0) * ATT_D + c;
          #pragma unroll
          for (int x = 0; x < 32; x += 4) {
            *reinterpret_cast<float4*>(pk + x) = make_float4(__uint_as_float(a[x]), __uint_as_float(a[x + 1]), __uint_as_float(a[x + 2]), __uint_as_float(a[x + 3]));
            *reinterpret_cast<float4*>(pv2 + x) = make_float4(__uint_as_float(bb[x]), __uint_as_float(bb[x + 1]), __uint_as_float(bb[x + 2]), __uint_as_float(bb[x + 3]));
          }
        } else if (kj < p.S) {
          #pragma unroll
          for (int x = 0; x < 32; x += 8) {
            *reinterpret_cast<uint4*>(dkp + c + x) = make_uint4(
                pack_bf16x2(__uint_as_float(a[x]), __uint_as_float(a[x + 1])), pack_bf16x2(__uint_as_float(a[x + 2]), __uint_as_float(a[x + 3])),
                pack_bf16x2(__uint_as_float(a[x + 4]), __uint_as_float(a[x + 5])), pack_bf16x2(__uint_as_float(a[x + 6]), __uint_as_float(a[x + 7])));
            *reinterpret_cast<uint4*>(dvp + c + x) = make_uint4(
                pack_bf16x2(__uint_as_float(bb[x]), __uint_as_float(bb[x + 1])), pack_bf16x2(__uint_as_float(bb[x + 2]), __uint_as_float(bb[x + 3])),
                pack_bf16x2(__uint_as_float(bb[x + 4]), __uint_as_float(bb[x + 5])), pack_bf16x2(__uint_as_float(bb[x + 6]), __uint_as_float(bb[x + 7])));
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------ dQ warps (8-11): thread d owns head dim d of dQ^T
    const int d = threadIdx.x - 256;
    const uint32_t lane_off = static_cast<uint32_t>((warp - 8) * 32) << 16;
    const bool leader = d == 0;
    bool ok = true;
    for (int it = 0; it < n_it && ok; ++it) {
      const int st = it & 1;
      const uint32_t ph2 = (it >> 1) & 1;
      const int g = it / n_q, i = i_lo + (it - g * n_q);
      const int q0 = i * ATTB_BQ;
      if (!mbar_wait(&bar_dq[st], ph2, abort_flag, p.status, PFB_ERR_WAIT_TMEM_FULL)) break;
      tc_fence_after();
      uint32_t dq0[32], dq1[32];
      tmem_ld_32x32(tmem_base + st * 128 + 64 + lane_off, dq0);
      tmem_ld_32x32(tmem_base + st * 128 + 96 + lane_off, dq1);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&dq_read[st]);
      int my_turn = 0;
      if (pp.deterministic && warp == 8) {
        // contributors of this query tile are taken in descending key-tile order: count those above this CTA's tile
        const int j_top = p.causal ? min(kv_tiles - 1, (q0 + ATTB_BQ - 1) / ATTB_BKV) : kv_tiles - 1;
        int cnt = 0;
        for (int j2 = jt + 1 + lane; j2 <= j_top; j2 += 32)
          cnt += (p.kend == nullptr || p.tile_max_end[b * kv_tiles + j2] > q0) ? 1 : 0;
        #pragma unroll
        for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
        my_turn = cnt;
      }
      #pragma unroll 1
      for (int half = 0; half < 2; ++half) {
        // the previous reduce-add has finished reading the staging tile
        if (leader) tma_store_wait_read<0>();
        named_bar_sync(1, 128);
        const uint32_t* src = half == 0 ? dq0 : dq1;
        #pragma unroll
        for (int x = 0; x < 32; ++x) sDQ[x * ATT_D + d] = __uint_as_float(src[x]);
        fence_proxy_async_smem();
        named_bar_sync(1, 128);
        if (leader) {
          int* turn = pp.dq_turn + (static_cast<long long>(b) * p.Hq + head0 + g) * q_tiles + i;
          if (pp.deterministic && half == 0) {
            const long long t0 = global_ns(), budget = wait_budget_ns(p.status);
            while (*reinterpret_cast<volatile int*>(turn) < my_turn) {
              if (*abort_flag) { ok = false; break; }
              if (global_ns() - t0 > budget) { *abort_flag = 1; atomicCAS(p.status, 0, PFB_ERR_WAIT_PEER); ok = false; break; }
            }
            __threadfence();
          }
          if (ok) {
            tma_reduce_add_3d(&tmdQ, sDQ, 0, head0 + g, row_base + q0 + half * 32);
            tma_store_commit();
            if (pp.deterministic && half == 1) {
              tma_store_wait<0>();          // both halves are in memory: pass the turn on
              fence_proxy_async_all_bwd();
              __threadfence();
              atomicExch(turn, my_turn + 1);
            }
          }
        }
      }
      ok = ok && !*abort_flag;
    }
    if (leader) tma_store_wait<0>();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 13) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

// delta[b, h, s] = sum_d dO * O ; one warp per (token, head).
__global__ void attn_bwd_delta_kernel(const __nv_bfloat16* __restrict__ dO, const __nv_bfloat16* __restrict__ O,
                                      float* __restrict__ delta, int B, int S, int Hq) {
  const long long w = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= static_cast<long long>(B) * S * Hq) return;
  const long long t = w / Hq;
  const int h = static_cast<int>(w - t * Hq);
  const uint2 a = reinterpret_cast<const uint2*>(dO + w * ATT_D)[lane];
  const uint2 o = reinterpret_cast<const uint2*>(O + w * ATT_D)[lane];
  const __nv_bfloat162* ab = reinterpret_cast<const __nv_bfloat162*>(&a);
  const __nv_bfloat162* ob = reinterpret_cast<const __nv_bfloat162*>(&o);
  float s = 0.f;
  #pragma unroll
  for (int j = 0; j < 2; ++j) {
    const float2 fa = __bfloat1622float2(ab[j]), fo = __bfloat1622float2(ob[j]);
    s += fa.x * fo.x + fa.y * fo.y;
  }
  #pragma unroll
  for (int o2 = 16; o2 > 0; o2 >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o2);
  const long long b = t / S, si = t - b * S;
  if (lane == 0) delta[(b * Hq + h) * S + si] = s;
}

// dk / dv (bf16, strided rows) = sum over the G query heads of a group of the fp32 partials [T, Hq, 128]
__global__ void attn_bwd_dkv_reduce_kernel(const float* __restrict__ part, __nv_bfloat16* __restrict__ out, long long T,
                                           int Hq, int Hkv, long long out_row_stride) {
  const int G = Hq / Hkv;
  const int nv = Hkv * (ATT_D / 4);
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < T * nv;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = idx / nv;
    const int r = static_cast<int>(idx - t * nv);
    const int kvh = r / (ATT_D / 4), d4 = r - kvh * (ATT_D / 4);
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int g = 0; g < G; ++g) {
      const float4 v = reinterpret_cast<const float4*>(part + (t * Hq + kvh * G + g) * ATT_D)[d4];
      s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
    }
    uint2 o;
    o.x = pack_bf16x2(s.x, s.y);
    o.y = pack_bf16x2(s.z, s.w);
    reinterpret_cast<uint2*>(out + t * out_row_stride + kvh * ATT_D)[d4] = o;
  }
}

// dq (bf16, strided rows) = dq_acc (fp32, contiguous [T, Hq*128])
__global__ void attn_bwd_dq_convert_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, long long T,
                                           int width, long long dq_row_stride) {
  const int nv = width >> 2;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < T * nv;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = idx / nv;
    const int c = static_cast<int>(idx - t * nv);
    const float4 v = reinterpret_cast<const float4*>(acc + t * width)[c];
    uint2 o;
    o.x = pack_bf16x2(v.x, v.y);
    o.y = pack_bf16x2(v.z, v.w);
    reinterpret_cast<uint2*>(dq + t * dq_row_stride)[c] = o;
  }
}

}  // namespace pfb
