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

struct AttnBwdSmem {
  static constexpr int KV_TILE = ATTB_BKV * ATT_D * 2;   // 32 KB
  static constexpr int Q_TILE = ATTB_BQ * ATT_D * 2;     // 16 KB
  static constexpr int K_OFF = 0, V_OFF = KV_TILE;
  static constexpr int Q_OFF = 2 * KV_TILE;               // 2 stages x (Q, dO)
  static constexpr int DS_OFF = Q_OFF + 4 * Q_TILE;       // dS^T [128 keys x 64 q] bf16 = 16 KB
  static constexpr int STAT_OFF = DS_OFF + ATTB_BKV * ATTB_BQ * 2;  // per-warp lse / delta copies: 4 x 2 x 64 floats
  static constexpr int BAR_OFF = STAT_OFF + 4 * 2 * 64 * 4;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

__global__ void __launch_bounds__(ATTB_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                const AttnBwdParams p) {
  using SM = AttnBwdSmem;
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
  const uint32_t tS = tmem_base, tdP = tmem_base + 64, tdV = tmem_base + 128, tdK = tmem_base + 256, tdQ = tmem_base + 384;

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
      constexpr uint32_t idesc_dkv = make_idesc(128, ATT_D, false, true, 1);     // TMEM A x MN-major B
      constexpr uint32_t idesc_dq = make_idesc(128, ATTB_BQ, true, true, 1);     // MN-major x MN-major
      auto load_q = [&](int it) {
        const int i = i_lo + it;
        const int st = it & 1;
        uint8_t* sq = smem + SM::Q_OFF + st * 2 * SM::Q_TILE;
        uint8_t* sdo = sq + SM::Q_TILE;
        mbar_expect_tx(&bar_q[st], 2 * SM::Q_TILE);
        tma_load_3d(sq, &tmQ, &bar_q[st], 0, head, row_base + i * ATTB_BQ);
        tma_load_3d(sq + SM::Q_TILE / 2, &tmQ, &bar_q[st], 64, head, row_base + i * ATTB_BQ);
        tma_load_3d(sdo, &tmdO, &bar_q[st], 0, head, row_base + i * ATTB_BQ);
        tma_load_3d(sdo + SM::Q_TILE / 2, &tmdO, &bar_q[st], 64, head, row_base + i * ATTB_BQ);
      };
      mbar_expect_tx(bar_kv, 2 * SM::KV_TILE);
      tma_load_3d(sK, &tmK, bar_kv, 0, kvh, row_base + k0);
      tma_load_3d(sK + SM::KV_TILE / 2, &tmK, bar_kv, 64, kvh, row_base + k0);
      tma_load_3d(sV, &tmV, bar_kv, 0, kvh, row_base + k0);
      tma_load_3d(sV + SM::KV_TILE / 2, &tmV, bar_kv, 64, kvh, row_base + k0);
      load_q(0);
      bool ok = mbar_wait(bar_kv, 0, abort_flag, p.status, PFB_ERR_WAIT_FULL);
      for (int it = 0; it < n_it && ok; ++it) {
        const int st = it & 1;
        const uint32_t ph = it & 1, qph = (it >> 1) & 1;
        const uint32_t sq = smem_u32(smem + SM::Q_OFF + st * 2 * SM::Q_TILE);
        const uint32_t sdo = sq + SM::Q_TILE;
        if (!mbar_wait(&bar_q[st], qph, abort_flag, p.status, PFB_ERR_WAIT_FULL)) break;
        tc_fence_after();
        #pragma unroll
        for (int k = 0; k < ATT_D / 16; ++k) {
          const uint32_t offk = (k >> 2) * (SM::KV_TILE / 2) + (k & 3) * 32;
          const uint32_t offq = (k >> 2) * (SM::Q_TILE / 2) + (k & 3) * 32;
          tc_mma_f16_ss(tS, make_smem_desc_sw128(smem_u32(sK) + offk, 16, 1024), make_smem_desc_sw128(sq + offq, 16, 1024),
                        idesc_s, k != 0);
        }
        #pragma unroll
        for (int k = 0; k < ATT_D / 16; ++k) {
          const uint32_t offk = (k >> 2) * (SM::KV_TILE / 2) + (k & 3) * 32;
          const uint32_t offq = (k >> 2) * (SM::Q_TILE / 2) + (k & 3) * 32;
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
          tc_mma_f16_ts(tdV, tS + k * 8, make_smem_desc_sw128(sdo + k * 16 * 128, SM::Q_TILE / 2, 1024), idesc_dkv,
                        (it | k) != 0);
        if (!mbar_wait(bar_ds, ph, abort_flag, p.status, PFB_ERR_WAIT_TMEM_EMPTY)) break;
        tc_fence_after();
        #pragma unroll
        for (int k = 0; k < ATTB_BQ / 16; ++k)
          tc_mma_f16_ts(tdK, tdP + k * 8, make_smem_desc_sw128(sq + k * 16 * 128, SM::Q_TILE / 2, 1024), idesc_dkv,
                        (it | k) != 0);
        if (it > 0) {
          if (!mbar_wait(bar_dqread, (it - 1) & 1, abort_flag, p.status, PFB_ERR_WAIT_TMEM_EMPTY)) break;
          tc_fence_after();
        }
        #pragma unroll
        for (int k = 0; k < ATTB_BKV / 16; ++k)
          tc_mma_f16_ss(tdQ, make_smem_desc_sw128(smem_u32(sK) + k * 16 * 128, SM::KV_TILE / 2, 1024),
                        make_smem_desc_sw128(smem_u32(sdS) + k * 16 * 128, 16, 1024), idesc_dq, k != 0);
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
        uint32_t pk[16];
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
          pk[x >> 1] = pack_bf16x2(p0, p1);
        }
        tmem_st_32x16(tS + lane_off + (c >> 1), pk);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_p);
      // dS^T = P^T * (dP^T - delta) * scale
      #pragma unroll
      for (int c = 0; c < ATTB_BQ; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(tdP + lane_off + c, v);
        tmem_ld_wait();
        uint32_t pk[16];
        #pragma unroll
        for (int x = 0; x < 32; x += 2) {
          const float d0 = pv[c + x] * (__uint_as_float(v[x]) - s_delta[c + x]) * p.scale;
          const float d1 = pv[c + x + 1] * (__uint_as_float(v[x + 1]) - s_delta[c + x + 1]) * p.scale;
          pk[x >> 1] = pack_bf16x2(d0, d1);
        }
        tmem_st_32x16(tdP + lane_off + (c >> 1), pk);
        uint8_t* rowp = sdS + r * 128;
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
      // dQ^T tile: lane (TMEM) index = head dim r, columns = the 64 queries
      if (!mbar_wait(bar_dq, ph, abort_flag, p.status, PFB_ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      uint32_t dq0[32], dq1[32];
      tmem_ld_32x32(tdQ + lane_off, dq0);
      tmem_ld_32x32(tdQ + lane_off + 32, dq1);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_dqread);
      float* acc = p.dq_acc + (static_cast<long long>(row_base + q0) * p.Hq + head) * ATT_D + r;
      const long long qstride = static_cast<long long>(p.Hq) * ATT_D;
      #pragma unroll
      for (int x = 0; x < 32; ++x)
        if (q0 + x < p.S) atomicAdd(acc + x * qstride, __uint_as_float(dq0[x]));
      #pragma unroll
      for (int x = 0; x < 32; ++x)
        if (q0 + 32 + x < p.S) atomicAdd(acc + (32 + x) * qstride, __uint_as_float(dq1[x]));
    }
    // dK, dV: one key row per thread
    if (ok) {
      if (n_it > 0) tc_fence_after();
      __nv_bfloat16* dkp = p.dk + static_cast<long long>(row_base + kj) * p.dk_row_stride + kvh * ATT_D;
      __nv_bfloat16* dvp = p.dv + static_cast<long long>(row_base + kj) * p.dv_row_stride + kvh * ATT_D;
      #pragma unroll 1
      for (int c = 0; c < ATT_D; c += 32) {
        uint32_t a[32], bb[32];
        if (n_it > 0) {
          tmem_ld_32x32(tdK + lane_off + c, a);
          tmem_ld_32x32(tdV + lane_off + c, bb);
          tmem_ld_wait();
        } else {
          #pragma unroll
          for (int x = 0; x < 32; ++x) { a[x] = 0u; bb[x] = 0u; }
        }
        if (kj < p.S && p.dk_part != nullptr) {
          float* pk = p.dk_part + (static_cast<long long>(row_base + kj) * p.Hq + head) * ATT_D + c;
          float* pv2 = p.dv_part + (static_cast<long long>(row_base + kj) * p.Hq + head) * ATT_D + c;
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
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 4) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
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
