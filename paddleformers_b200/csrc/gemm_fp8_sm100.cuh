// Block-scaled fp8 (e4m3) GEMM for sm_100a and the quantisation kernels that feed it.
//
//   D[M,N] (bf16) = sum over 128-wide K blocks kb of
//                   sa[m, kb] * sb[n / 128, kb] * ( Aq[m, kb-block] . Bq[n, kb-block] )
//
// Aq: [M, K] e4m3 with one fp32 scale per 1x128 block, stored transposed as sa_t[K/128, M] so that the 32 lanes of
// an epilogue warp read consecutive floats. Bq: [N, K] e4m3 (E stacked matrices in the grouped variant) with one fp32
// scale per 128x128 block, sb[N/128, K/128].
//
// Structure: the persistent TMA / MMA / epilogue split of the bf16 kernel with 128 x 128 x 128 tiles. Each K block is
// multiplied into a FRESH TMEM accumulator (four 128-column buffers rotate), committed to the epilogue warps, and
// (eight of them: two per TMEM lane quadrant, 64 columns each) read it back with tcgen05.ld, multiply by the block's
// scale product and add into fp32 registers: the
// promotion that a 1x128 / 128x128 scaled format needs, with the tensor core never waiting for it as long as the
// epilogue keeps up (four buffers of slack).
//
// Counterparts in the reference: deep_gemm.fp8_gemm_nt / m_grouped_fp8_gemm_nt_contiguous call sites
// (paddleformers/transformers/fp8_utils.py:35-46, 187, 278, 949, 1002), the Triton specification of the math
// (paddleformers/cli/train/deepseek_v3_pretrain/kernel.py:129-219) and fp8_quant_blockwise (fp8_utils.py:112-131).
#pragma once
#include <cuda_fp8.h>

#include "sm100_common.cuh"

namespace pfb {

constexpr int F8_BM = 128, F8_BN = 128, F8_BK = 128;   // 128 e4m3 = one 128-byte swizzle row
constexpr int F8_UMMA_K = 32;
constexpr int F8_ACC_BUFS = 4;
constexpr int F8_EPI_WARPS = 8;            // two warps per TMEM lane quadrant, 64 accumulator columns each
constexpr int F8_THREADS = 64 + 32 * F8_EPI_WARPS;

struct Fp8GemmParams {
  int M, N, K;
  __nv_bfloat16* D;
  long long ldd;
  const float* sa_t;        // [K/128, sa_ld]
  long long sa_ld;
  const float* sb;          // [rows_b/128, K/128]
  int m_blocks, n_blocks, k_blocks, group_m;
  const int* block_expert;  // grouped: expert per 128-row block of A (-1 = skip)
  int n_per_expert;         // grouped: rows of B per expert (multiple of 128)
  int* status;
};

template <int STAGES>
struct Fp8Smem {
  static constexpr int A_BYTES = F8_BM * F8_BK;
  static constexpr int B_BYTES = F8_BN * F8_BK;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + 256 + 1024;
};

template <int STAGES, bool GROUPED>
__global__ void __launch_bounds__(F8_THREADS, 1)
gemm_fp8_blockscaled_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                            const Fp8GemmParams p) {
  using S = Fp8Smem<STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;          // [F8_ACC_BUFS]
  uint64_t* tempty_bar = tfull_bar + F8_ACC_BUFS;    // [F8_ACC_BUFS]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + F8_ACC_BUFS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr uint32_t TMEM_COLS = F8_ACC_BUFS * F8_BN;   // 512

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < F8_ACC_BUFS; ++a) { mbar_init(&tfull_bar[a], 1); mbar_init(&tempty_bar[a], F8_EPI_WARPS); }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); tc_fence_before(); }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int num_tiles = p.m_blocks * p.n_blocks;
  const int tiles_per_group = p.group_m * p.n_blocks;
  auto tile_coords = [&](int t, int& mb, int& nb) {
    int g = t / tiles_per_group;
    int r = t - g * tiles_per_group;
    int gsz = min(p.group_m, p.m_blocks - g * p.group_m);
    mb = g * p.group_m + (r % gsz);
    nb = r / gsz;
  };

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int mb, nb; tile_coords(t, mb, nb);
        int b_row0 = nb * F8_BN;
        if constexpr (GROUPED) {
          const int e = p.block_expert[mb];
          if (e < 0) continue;
          b_row0 += e * p.n_per_expert;
        }
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, PFB_ERR_WAIT_EMPTY)) { ok = false; break; }
          uint8_t* sa = smem + stage * S::STAGE_BYTES;
          mbar_expect_tx(&full_bar[stage], S::STAGE_BYTES);
          tma_load_2d(sa, &tmA, &full_bar[stage], kb * F8_BK, mb * F8_BM);
          tma_load_2d(sa + S::A_BYTES, &tmB, &full_bar[stage], kb * F8_BK, b_row0);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(F8_BM, F8_BN, false, false, 0);   // e4m3 x e4m3 -> fp32
      int stage = 0; uint32_t phase = 0;
      int buf = 0; uint32_t buf_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        if constexpr (GROUPED) {
          int mb, nb; tile_coords(t, mb, nb);
          if (p.block_expert[mb] < 0) continue;
        }
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(&tempty_bar[buf], buf_phase ^ 1, abort_flag, p.status, PFB_ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, PFB_ERR_WAIT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * S::STAGE_BYTES);
          const uint32_t sb = sa + S::A_BYTES;
          const uint32_t d_tmem = tmem_base + buf * F8_BN;
          #pragma unroll
          for (int k = 0; k < F8_BK / F8_UMMA_K; ++k) {
            const uint64_t da = make_smem_desc_sw128(sa + k * F8_UMMA_K, 16, 1024);
            const uint64_t db = make_smem_desc_sw128(sb + k * F8_UMMA_K, 16, 1024);
            tc_mma_f8_ss(d_tmem, da, db, idesc, k != 0 ? 1u : 0u);
          }
          tc_commit(&empty_bar[stage]);
          tc_commit(&tfull_bar[buf]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
          if (++buf == F8_ACC_BUFS) { buf = 0; buf_phase ^= 1; }
        }
      }
    }
  } else {
    const int quad = warp & 3;                 // TMEM lanes this warp may read
    const int half = (warp - 2) >> 2;          // which 64 of the tile's 128 columns it accumulates
    constexpr int COLS = F8_BN / 2;
    int buf = 0; uint32_t buf_phase = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      int mb, nb; tile_coords(t, mb, nb);
      int sb_row = nb;
      if constexpr (GROUPED) {
        const int e = p.block_expert[mb];
        if (e < 0) continue;
        sb_row += e * (p.n_per_expert / F8_BN);
      }
      const int row = mb * F8_BM + quad * 32 + lane;
      const int row_c = min(row, p.M - 1);
      const float* sa_col = p.sa_t + row_c;
      const float* sb_rowp = p.sb + static_cast<long long>(sb_row) * p.k_blocks;
      float acc[COLS];
      #pragma unroll
      for (int j = 0; j < COLS; ++j) acc[j] = 0.f;
      float s_ring[4];
      #pragma unroll
      for (int u = 0; u < 4; ++u)
        s_ring[u] = u < p.k_blocks ? sa_col[static_cast<long long>(u) * p.sa_ld] * sb_rowp[u] : 0.f;
      for (int kb0 = 0; kb0 < p.k_blocks && ok; kb0 += 4) {
        #pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int kb = kb0 + u;
          if (kb >= p.k_blocks) break;
          const float s = s_ring[u];
          if (kb + 4 < p.k_blocks)   // prefetch the scale product four K blocks ahead
            s_ring[u] = sa_col[static_cast<long long>(kb + 4) * p.sa_ld] * sb_rowp[kb + 4];
          if (!mbar_wait(&tfull_bar[buf], buf_phase, abort_flag, p.status, PFB_ERR_WAIT_TMEM_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * F8_BN + half * COLS;
          uint32_t v0[32], v1[32];
          tmem_ld_32x32(taddr, v0);
          tmem_ld_32x32(taddr + 32, v1);
          tmem_ld_wait();
          // the partial sums are in registers: hand the buffer back before the arithmetic
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tempty_bar[buf]);
          #pragma unroll
          for (int j = 0; j < 32; ++j) acc[j] = fmaf(s, __uint_as_float(v0[j]), acc[j]);
          #pragma unroll
          for (int j = 0; j < 32; ++j) acc[32 + j] = fmaf(s, __uint_as_float(v1[j]), acc[32 + j]);
          if (++buf == F8_ACC_BUFS) { buf = 0; buf_phase ^= 1; }
        }
      }
      if (!ok) break;
      if (row < p.M) {
        __nv_bfloat16* drow = p.D + static_cast<long long>(row) * p.ldd;
        #pragma unroll
        for (int c = 0; c < COLS / 32; ++c) {
          const int col = nb * F8_BN + half * COLS + c * 32;
          if (col + 32 <= p.N) {
            #pragma unroll
            for (int j = 0; j < 4; ++j)
              reinterpret_cast<uint4*>(drow + col)[j] = make_uint4(
                  pack_bf16x2(acc[c * 32 + 8 * j], acc[c * 32 + 8 * j + 1]), pack_bf16x2(acc[c * 32 + 8 * j + 2], acc[c * 32 + 8 * j + 3]),
                  pack_bf16x2(acc[c * 32 + 8 * j + 4], acc[c * 32 + 8 * j + 5]), pack_bf16x2(acc[c * 32 + 8 * j + 6], acc[c * 32 + 8 * j + 7]));
          } else {
            #pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col + j < p.N) drow[col + j] = __float2bfloat16(acc[c * 32 + j]);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }
}

// ---------------------------------------------------------------------------------------------------------------
// quantisation
// ---------------------------------------------------------------------------------------------------------------
// One warp per (row, 128-column block): q[T, K] e4m3 and scales stored transposed, s_t[K/128, T].
__global__ void fp8_quant_act_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, uint8_t* __restrict__ q,
                                     float* __restrict__ s_t, int T, int K, bool ue8m0) {
  const int lane = threadIdx.x & 31;
  const int nb = K / 128;
  const long long units = static_cast<long long>(T) * nb;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long u = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; u < units; u += warps) {
    const int kb = static_cast<int>(u % nb);
    const long long t = u / nb;
    const uint2 raw = *reinterpret_cast<const uint2*>(x + t * ldx + kb * 128 + lane * 4);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    float amax = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y)));
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float scale = fp8_block_scale(amax, ue8m0);
    const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a.x / scale, a.y / scale), __NV_SATFINITE, __NV_E4M3);
    const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(b.x / scale, b.y / scale), __NV_SATFINITE, __NV_E4M3);
    *reinterpret_cast<uint32_t*>(q + t * K + kb * 128 + lane * 4) = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
    if (lane == 0) s_t[static_cast<long long>(kb) * T + t] = scale;
  }
}

// One CTA of 256 threads per 128x128 block of w[N, K]: q[N, K] e4m3, s[ceil(N/128), K/128].
__global__ void fp8_quant_weight_kernel(const __nv_bfloat16* __restrict__ w, long long ldw, uint8_t* __restrict__ q,
                                        float* __restrict__ s, int N, int K, bool ue8m0) {
  __shared__ float red[8];
  __shared__ float s_scale;
  const int kb = blockIdx.x, nb = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // thread -> (row r0 + 16 * i, 8 columns): 16 threads cover one 128-column row segment, 16 rows per pass, 8 passes
  const int c8 = (tid & 15) * 8, r0 = tid >> 4;
  uint4 vals[8];
  float amax = 0.f;
  #pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int row = nb * 128 + r0 + 16 * i;
    vals[i] = make_uint4(0u, 0u, 0u, 0u);
    if (row < N) vals[i] = *reinterpret_cast<const uint4*>(w + static_cast<long long>(row) * ldw + kb * 128 + c8);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&vals[i]);
    #pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(h[j]);
      amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
  #pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if (lane == 0) red[warp] = amax;
  __syncthreads();
  if (tid == 0) {
    float m = red[0];
    #pragma unroll
    for (int i = 1; i < 8; ++i) m = fmaxf(m, red[i]);
    s_scale = fp8_block_scale(m, ue8m0);
    s[static_cast<long long>(nb) * gridDim.x + kb] = s_scale;
  }
  __syncthreads();
  const float scale = s_scale;
  #pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int row = nb * 128 + r0 + 16 * i;
    if (row >= N) continue;
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&vals[i]);
    uint32_t out[2];
    #pragma unroll
    for (int j = 0; j < 2; ++j) {
      const float2 f0 = __bfloat1622float2(h[2 * j]);
      const float2 f1 = __bfloat1622float2(h[2 * j + 1]);
      const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(f0.x / scale, f0.y / scale), __NV_SATFINITE, __NV_E4M3);
      const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(f1.x / scale, f1.y / scale), __NV_SATFINITE, __NV_E4M3);
      out[j] = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
    }
    *reinterpret_cast<uint2*>(q + static_cast<long long>(row) * K + kb * 128 + c8) = make_uint2(out[0], out[1]);
  }
}

}  // namespace pfb
