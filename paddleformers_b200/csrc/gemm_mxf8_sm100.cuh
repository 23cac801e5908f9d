// Block-scaled fp8 (e4m3) GEMM on the tensor core's own scaling path: tcgen05.mma.kind::mxf8f6f4.block_scale.
//
//   D[M,N] = sum over 128-wide K blocks kb of  2^ea[m,kb] * 2^eb[n,kb] * ( Aq[m, kb-block] . Bq[n, kb-block] )
//
// The 1x128 / 128x128 scaled format of gemm_fp8_sm100.cuh needs one multiply per accumulator element and K block when
// the scales are arbitrary floats, and that promotion (tcgen05.ld + FMA in the epilogue warps) is what bounds that
// kernel at bf16 speed. When every scale is a power of two (the UE8M0 option of the quantisation kernels) the tensor
// core can apply it itself: the instruction takes one 8-bit exponent per operand row and 32-element K group from
// tensor memory. A 128-wide block is four such groups that share one exponent, so all four K=32 instructions of a
// block select the same byte. The whole K extent then accumulates in ONE TMEM accumulator, exactly as in the bf16
// kernel, and the epilogue reads it once per tile.
//
// Scale operands. One 32-bit word per operand row holds the exponent bytes of four consecutive K blocks (byte kb % 4);
// the instruction descriptor's scale-id fields pick the byte. The words of a 128-row group are stored as 32 rows of
// 16 bytes, row l holding the words of operand rows l, 32 + l, 64 + l, 96 + l; tcgen05.cp (32x128b, warpx4) copies
// that into four TMEM columns of every lane quadrant. mx_pack_scales_kernel writes this order directly, per tile, so
// the kernel moves 512 bytes per 128 rows and four K blocks with one bulk copy and no shuffle.
//
// Structure: persistent CTAs, warp 0 TMA producer, warp 1 MMA issuer, warps 2-9 epilogue (two per TMEM lane quadrant).
// Tiles are 128 x BN with BN in {128, 192, 240}: two accumulators of up to 240 columns plus the 12 scale columns fit
// the 512 columns of tensor memory, which a 256-wide double-buffered tile would not.
//
// Counterparts in the reference: deep_gemm.fp8_gemm_nt / m_grouped_fp8_gemm_nt_contiguous call sites
// (paddleformers/transformers/fp8_utils.py:35-46, 187, 278, 949, 1002).
#pragma once
#include <cuda_fp8.h>

#include "sm100_common.cuh"

namespace pfb {

constexpr int MX_BM = 128, MX_BK = 128, MX_UMMA_K = 32;
constexpr int MX_EPI_WARPS = 8;
constexpr int MX_THREADS = 64 + 32 * MX_EPI_WARPS;
constexpr uint32_t MX_TMEM_COLS = 512;
constexpr uint32_t MX_SFA_COL = 496, MX_SFB_COL = 500;   // accumulators at columns 0 and 256 (each at most 240 wide)

struct MxGemmParams {
  int M, N, K;
  __nv_bfloat16* D;         // bf16 output, or nullptr when Dacc is set
  float* Dacc;              // fp32 output that the product is ADDED to (weight gradients)
  long long ldd;
  const uint32_t* sfa;      // [m_blocks][k_groups][128]
  const uint32_t* sfb;      // [b_tiles][k_groups][SFB_ROWS]
  int m_blocks, n_blocks, k_blocks, k_groups, group_m;
  const int* block_expert;  // grouped: expert per 128-row block of A (-1 = skip)
  int n_per_expert;         // grouped: rows of B per expert
  int* status;
};

template <int BN, int STAGES>
struct MxSmem {
  static constexpr int A_BYTES = MX_BM * MX_BK;
  static constexpr int B_BYTES = BN * MX_BK;                       // a multiple of 1024 for BN % 8 == 0
  static constexpr int SFB_ROWS = (BN + 127) / 128 * 128;
  static constexpr int SF_BYTES = 512 + SFB_ROWS * 4;
  static constexpr int SF_SLOT = 2048;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SF_SLOT;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + 256 + 1024;
  static_assert(B_BYTES % 1024 == 0 && SF_BYTES <= SF_SLOT, "stage layout");
};

// global -> shared bulk copy (no multicast), completion on an mbarrier; both addresses and the size multiples of 16
__device__ __forceinline__ void mx_bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// 32 rows x 16 bytes of shared memory -> 4 TMEM columns, replicated into all four lane quadrants
__device__ __forceinline__ void tc_cp_32x128b_warpx4(uint32_t tmem_dst, uint64_t smem_desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_dst), "l"(smem_desc) : "memory");
}
// un-swizzled descriptor of a 32 x 16-byte scale slab: 8-row atoms 128 bytes apart
__device__ __forceinline__ uint64_t make_sf_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>(128 >> 4) << 32;   // stride byte offset
  d |= 1ull << 46;                              // descriptor version
  return d;
}
// e4m3 x e4m3 with UE8M0 block scales; sf ids select the exponent byte of the 32-bit scale words
__device__ __forceinline__ uint32_t make_idesc_mx(int M, int N, uint32_t a_sf_id, uint32_t b_sf_id) {
  return (b_sf_id << 4) | (1u << 23) | (static_cast<uint32_t>(N >> 3) << 17) | (static_cast<uint32_t>(M >> 4) << 24) |
         (a_sf_id << 29);
}
__device__ __forceinline__ void tc_mma_mxf8_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                               uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
      : "memory");
}

template <int BN, int STAGES, bool GROUPED>
__global__ void __launch_bounds__(MX_THREADS, 1)
gemm_mxf8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const MxGemmParams p) {
  using S = MxSmem<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;     // [2]
  uint64_t* tempty_bar = tfull_bar + 2;         // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tfull_bar[a], 1); mbar_init(&tempty_bar[a], MX_EPI_WARPS); }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, MX_TMEM_COLS); tmem_relinquish(); tc_fence_before(); }
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
        int b_row0 = nb * BN;
        int b_tile = nb;
        if constexpr (GROUPED) {
          const int e = p.block_expert[mb];
          if (e < 0) continue;
          b_row0 += e * p.n_per_expert;
          b_tile += e * p.n_blocks;
        }
        const uint32_t* sfa = p.sfa + static_cast<long long>(mb) * p.k_groups * 128;
        const uint32_t* sfb = p.sfb + static_cast<long long>(b_tile) * p.k_groups * S::SFB_ROWS;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, PFB_ERR_WAIT_EMPTY)) { ok = false; break; }
          uint8_t* sa = smem + stage * S::STAGE_BYTES;
          const bool with_sf = (kb & 3) == 0;
          mbar_expect_tx(&full_bar[stage], S::A_BYTES + S::B_BYTES + (with_sf ? S::SF_BYTES : 0));
          tma_load_2d(sa, &tmA, &full_bar[stage], kb * MX_BK, mb * MX_BM);
          tma_load_2d(sa + S::A_BYTES, &tmB, &full_bar[stage], kb * MX_BK, b_row0);
          if (with_sf) {
            uint8_t* sf = sa + S::A_BYTES + S::B_BYTES;
            mx_bulk_load(sf, sfa + (kb >> 2) * 128, 512, &full_bar[stage]);
            mx_bulk_load(sf + 512, sfb + (kb >> 2) * S::SFB_ROWS, S::SFB_ROWS * 4, &full_bar[stage]);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      int buf = 0; uint32_t buf_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        if constexpr (GROUPED) {
          int mb, nb; tile_coords(t, mb, nb);
          if (p.block_expert[mb] < 0) continue;
        }
        if (!mbar_wait(&tempty_bar[buf], buf_phase ^ 1, abort_flag, p.status, PFB_ERR_WAIT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * 256;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, PFB_ERR_WAIT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * S::STAGE_BYTES);
          const uint32_t sb = sa + S::A_BYTES;
          if ((kb & 3) == 0) {
            const uint32_t sf = sb + S::B_BYTES;
            tc_cp_32x128b_warpx4(tmem_base + MX_SFA_COL, make_sf_desc(sf));
            #pragma unroll
            for (int i = 0; i < S::SFB_ROWS / 128; ++i)
              tc_cp_32x128b_warpx4(tmem_base + MX_SFB_COL + 4 * i, make_sf_desc(sf + 512 + 512 * i));
          }
          const uint32_t idesc = make_idesc_mx(MX_BM, BN, kb & 3, kb & 3);
          #pragma unroll
          for (int k = 0; k < MX_BK / MX_UMMA_K; ++k) {
            const uint64_t da = make_smem_desc_sw128(sa + k * MX_UMMA_K, 16, 1024);
            const uint64_t db = make_smem_desc_sw128(sb + k * MX_UMMA_K, 16, 1024);
            tc_mma_mxf8_ss(d_tmem, da, db, idesc, tmem_base + MX_SFA_COL, tmem_base + MX_SFB_COL, (kb | k) != 0 ? 1u : 0u);
          }
          tc_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        tc_commit(&tfull_bar[buf]);
        if (++buf == 2) { buf = 0; buf_phase ^= 1; }
      }
    }
  } else {
    const int quad = warp & 3;                 // TMEM lanes this warp may read
    const int half = (warp - 2) >> 2;          // first or second part of the tile's columns
    constexpr int SPLIT = BN == 128 ? 64 : 128;
    const int c_begin = half ? SPLIT : 0, c_end = half ? BN : SPLIT;
    int buf = 0; uint32_t buf_phase = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      int mb, nb; tile_coords(t, mb, nb);
      if constexpr (GROUPED) {
        if (p.block_expert[mb] < 0) continue;
      }
      if (!mbar_wait(&tfull_bar[buf], buf_phase, abort_flag, p.status, PFB_ERR_WAIT_TMEM_FULL)) break;
      tc_fence_after();
      const int row = mb * MX_BM + quad * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * 256;
      for (int c = c_begin; c < c_end; c += 32) {
        uint32_t v0[16], v1[16];
        const bool two = c + 16 < c_end;
        tmem_ld_32x16(taddr + c, v0);
        if (two) tmem_ld_32x16(taddr + c + 16, v1);
        tmem_ld_wait();
        if (row < p.M) {
          #pragma unroll
          for (int h = 0; h < 2; ++h) {
            if (h == 1 && !two) break;
            const uint32_t* v = h ? v1 : v0;
            const int col = nb * BN + c + 16 * h;
            if (p.Dacc != nullptr) {
              float* drow = p.Dacc + static_cast<long long>(row) * p.ldd + col;
              if (col + 16 <= p.N) {
                #pragma unroll
                for (int j = 0; j < 4; ++j) {
                  float4 o = reinterpret_cast<float4*>(drow)[j];
                  o.x += __uint_as_float(v[4 * j]); o.y += __uint_as_float(v[4 * j + 1]);
                  o.z += __uint_as_float(v[4 * j + 2]); o.w += __uint_as_float(v[4 * j + 3]);
                  reinterpret_cast<float4*>(drow)[j] = o;
                }
              } else {
                #pragma unroll
                for (int j = 0; j < 16; ++j)
                  if (col + j < p.N) drow[j] += __uint_as_float(v[j]);
              }
            } else {
              __nv_bfloat16* drow = p.D + static_cast<long long>(row) * p.ldd + col;
              if (col + 16 <= p.N) {
                #pragma unroll
                for (int j = 0; j < 2; ++j)
                  reinterpret_cast<uint4*>(drow)[j] = make_uint4(
                      pack_bf16x2(__uint_as_float(v[8 * j]), __uint_as_float(v[8 * j + 1])),
                      pack_bf16x2(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3])),
                      pack_bf16x2(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5])),
                      pack_bf16x2(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7])));
              } else {
                #pragma unroll
                for (int j = 0; j < 16; ++j)
                  if (col + j < p.N) drow[j] = __float2bfloat16(__uint_as_float(v[j]));
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[buf]);
      if (++buf == 2) { buf = 0; buf_phase ^= 1; }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, MX_TMEM_COLS); }
}

// Exponent words in the order the kernel copies to tensor memory. One thread per (tile, K group of four blocks, row).
//   mode 0: scale(row, kb) = src[kb * ld + row]            (activations, transposed scales [K/128, rows])
//   mode 1: scale(row, kb) = src[(row / 128) * ld + kb]    (weights, one scale per 128 x 128 block, ld = K/128)
// rows_per_group rows form one matrix (one expert); tiles of `bt` rows never straddle two matrices. A scale that is not
// a power of two records PFB_ERR_SCALE_NOT_POW2 in the status word (its mantissa would be dropped silently otherwise).
__global__ void mx_pack_scales_kernel(const float* __restrict__ src, long long ld, int mode, uint32_t* __restrict__ out,
                                      int rows_per_group, int groups, int bt, int k_blocks, int* not_pow2) {
  const int sfr = (bt + 127) / 128 * 128;
  const int tiles_per_group = (rows_per_group + bt - 1) / bt;
  const int k_groups = (k_blocks + 3) / 4;
  const long long total = static_cast<long long>(groups) * tiles_per_group * k_groups * sfr;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(i % sfr);
    const long long tg = i / sfr;
    const int g = static_cast<int>(tg % k_groups);
    const long long tile = tg / k_groups;
    const int grp = static_cast<int>(tile / tiles_per_group), tj = static_cast<int>(tile % tiles_per_group);
    const int local = tj * bt + r;
    uint32_t word = 0;
    #pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      const int kb = 4 * g + kk;
      uint32_t e = 127;
      if (kb < k_blocks && r < bt && local < rows_per_group) {
        const long long row = static_cast<long long>(grp) * rows_per_group + local;
        const float s = mode == 0 ? src[static_cast<long long>(kb) * ld + row] : src[(row / 128) * ld + kb];
        const uint32_t bits = __float_as_uint(s);
        if (bits & 0x807FFFFFu) atomicCAS(not_pow2, 0, PFB_ERR_SCALE_NOT_POW2);
        e = (bits >> 23) & 0xFFu;
      }
      word |= e << (8 * kk);
    }
    out[(tile * k_groups + g) * sfr + (r / 128) * 128 + (r % 32) * 4 + ((r % 128) / 32)] = word;
  }
}

}  // namespace pfb
