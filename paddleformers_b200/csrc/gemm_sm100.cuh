// Persistent warp-specialised bf16 GEMM for sm_100a: TMA -> 128B-swizzled smem ring -> tcgen05.mma
// (accumulators in TMEM, double buffered) -> tcgen05.ld epilogue.
//
//   D[M,N] = A[M,K] * B[N,K]^T        (fp32 accumulation)
//
// A and B may each be K-major (row-major [rows, K]) or MN-major (row-major [K, rows]), which covers
// the forward (x W^T), dgrad (dy W) and wgrad (dy^T x) products of a linear layer without any
// transposed copy. The grouped variant treats B as E stacked [N,K] matrices and picks the matrix of
// each 128-row block of A from a device-side table (ragged experts padded to 128 rows).
//
// Plays the role of the library GEMMs behind the reference's linear layers
// (paddleformers/nn/linear.py:29-93, paddleformers/transformers/tensor_parallel_utils.py:87-96) and of
// the M-grouped expert GEMM (paddleformers/transformers/fp8_utils.py:913-1009).
#pragma once
#include "sm100_common.cuh"

namespace pfb {

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;       // 64 bf16 = one 128-byte swizzle row
constexpr int GEMM_UMMA_K = 16;
constexpr int GEMM_THREADS = 192; // warp0 TMA, warp1 MMA, warps2-5 epilogue

enum GemmEpilogue : int {
  EPI_STORE_BF16 = 0,   // D(bf16) = acc
  EPI_STORE_F32 = 1,    // D(fp32) = acc
  EPI_ACCUM_F32 = 2,    // D(fp32) += acc            (wgrad into fp32 main_grad)
  EPI_SWIGLU_BF16 = 3,  // D(bf16)[.., N/2]: silu(acc[:, j]) * acc[:, j + BN/2] per tile (gate|up interleaved by tile)
  EPI_ACCUM_BF16 = 4,   // D(bf16) = D + acc          (residual add fused)
  EPI_REDUCE_F32 = 5,   // D(fp32) += acc through TMA reduce-add (CTA-pair kernel only): the add happens in L2, nothing is read back
};

struct GemmParams {
  int M, N, K;
  void* D;
  long long ldd;            // row stride of D in elements
  void* D2;                 // SwiGLU epilogue: optional raw [M,N] bf16 copy of gate|up (nullptr = not stored)
  long long ldd2;
  int m_blocks, n_blocks, k_blocks;
  int group_m;              // rasterisation group (m-blocks per group)
  const int* block_expert;  // grouped: expert id per 128-row block of A (-1 = skip); else nullptr
  int n_per_expert;         // grouped: rows of B per expert
  const int* expert_rows;   // k-grouped (wgrad): [E, 2] = (first row, row count) of each expert's segment, counts % 64 == 0
  int tiles_per_expert;     // k-grouped: m_blocks * n_blocks of one expert's [N, K] gradient
  long long d_expert_stride;  // k-grouped: elements between consecutive experts in D
  int* status;              // error word (0 = ok)
  int split_tail = 0;       // CTA-pair kernel: this many tiles at the end of the tile list are computed as two 128-column halves
};

template <int BN, int STAGES>
struct GemmSmem {
  static constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;
  static constexpr int B_BYTES = BN * GEMM_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + 256 + 1024;  // barriers + alignment slack
};

// Epilogue of one accumulator tile: the calling thread owns TMEM lane (row) `row` of a 128 x BN fp32 tile at `taddr`
// and writes / accumulates its BN columns into D (see GemmEpilogue). Shared by the one-CTA and the CTA-pair kernels.
template <int BN, int EPI>
__device__ __forceinline__ void gemm_store_tile(uint32_t taddr, int row, int nb, const GemmParams& p, long long d_off) {
  if constexpr (EPI == EPI_SWIGLU_BF16) {
    // tile columns [0,BN/2) hold gate, [BN/2,BN) hold up for output columns nb*BN/2 ...
    __nv_bfloat16* Dp = reinterpret_cast<__nv_bfloat16*>(p.D);
    const int n_out = p.N / 2;
    #pragma unroll 1
    for (int c = 0; c < BN / 2; c += 32) {
      uint32_t g[32], u[32];
      tmem_ld_32x32(taddr + c, g);
      tmem_ld_32x32(taddr + BN / 2 + c, u);
      tmem_ld_wait();
      const int col = nb * (BN / 2) + c;
      if (row < p.M && p.D2 != nullptr && col < n_out) {
        __nv_bfloat16* r0 = reinterpret_cast<__nv_bfloat16*>(p.D2) + static_cast<long long>(row) * p.ldd2 + col;
        __nv_bfloat16* r1 = r0 + n_out;
        if (col + 32 <= n_out) {
          #pragma unroll
          for (int j = 0; j < 4; ++j) {
            reinterpret_cast<uint4*>(r0)[j] = make_uint4(pack_bf16x2(__uint_as_float(g[8 * j]), __uint_as_float(g[8 * j + 1])),
                pack_bf16x2(__uint_as_float(g[8 * j + 2]), __uint_as_float(g[8 * j + 3])),
                pack_bf16x2(__uint_as_float(g[8 * j + 4]), __uint_as_float(g[8 * j + 5])),
                pack_bf16x2(__uint_as_float(g[8 * j + 6]), __uint_as_float(g[8 * j + 7])));
            reinterpret_cast<uint4*>(r1)[j] = make_uint4(pack_bf16x2(__uint_as_float(u[8 * j]), __uint_as_float(u[8 * j + 1])),
                pack_bf16x2(__uint_as_float(u[8 * j + 2]), __uint_as_float(u[8 * j + 3])),
                pack_bf16x2(__uint_as_float(u[8 * j + 4]), __uint_as_float(u[8 * j + 5])),
                pack_bf16x2(__uint_as_float(u[8 * j + 6]), __uint_as_float(u[8 * j + 7])));
          }
        } else {
          for (int j = 0; j < 32 && col + j < n_out; ++j) {
            r0[j] = __float2bfloat16(__uint_as_float(g[j]));
            r1[j] = __float2bfloat16(__uint_as_float(u[j]));
          }
        }
      }
      if (row < p.M && col < n_out) {
        uint32_t o[16];
        #pragma unroll
        for (int j = 0; j < 16; ++j) {
          float g0 = __uint_as_float(g[2 * j]), g1 = __uint_as_float(g[2 * j + 1]);
          float u0 = __uint_as_float(u[2 * j]), u1 = __uint_as_float(u[2 * j + 1]);
          float a0 = __fdividef(g0, 1.f + __expf(-g0)) * u0;     // fast division: the epilogue warps are latency-bound
          float a1 = __fdividef(g1, 1.f + __expf(-g1)) * u1;
          o[j] = pack_bf16x2(a0, a1);
        }
        __nv_bfloat16* dst = Dp + static_cast<long long>(row) * p.ldd + col;
        if (col + 32 <= n_out) {
          #pragma unroll
          for (int j = 0; j < 4; ++j)
            reinterpret_cast<uint4*>(dst)[j] = make_uint4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
        } else {
          for (int j = 0; j < 32 && col + j < n_out; ++j)
            dst[j] = reinterpret_cast<__nv_bfloat16*>(o)[j];
        }
      }
    }
  } else {
    #pragma unroll 1
    for (int c = 0; c < BN; c += 32) {
      uint32_t v[32];
      tmem_ld_32x32(taddr + c, v);
      tmem_ld_wait();
      const int col = nb * BN + c;
      if (row < p.M && col < p.N) {
        if constexpr (EPI == EPI_STORE_BF16 || EPI == EPI_ACCUM_BF16) {
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.D) + static_cast<long long>(row) * p.ldd + col;
          if (col + 32 <= p.N) {
            #pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 o;
              if constexpr (EPI == EPI_ACCUM_BF16) {
                uint4 old = reinterpret_cast<const uint4*>(dst)[j];
                const __nv_bfloat162* ob = reinterpret_cast<const __nv_bfloat162*>(&old);
                uint32_t* oo = reinterpret_cast<uint32_t*>(&o);
                #pragma unroll
                for (int q = 0; q < 4; ++q) {
                  float2 f = __bfloat1622float2(ob[q]);
                  oo[q] = pack_bf16x2(__uint_as_float(v[8 * j + 2 * q]) + f.x, __uint_as_float(v[8 * j + 2 * q + 1]) + f.y);
                }
              } else {
                o = make_uint4(pack_bf16x2(__uint_as_float(v[8 * j]), __uint_as_float(v[8 * j + 1])),
                               pack_bf16x2(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3])),
                               pack_bf16x2(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5])),
                               pack_bf16x2(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7])));
              }
              reinterpret_cast<uint4*>(dst)[j] = o;
            }
          } else {
            for (int j = 0; j < 32 && col + j < p.N; ++j) {
              float x = __uint_as_float(v[j]);
              if constexpr (EPI == EPI_ACCUM_BF16) x += __bfloat162float(dst[j]);
              dst[j] = __float2bfloat16(x);
            }
          }
        } else {
          float* dst = reinterpret_cast<float*>(p.D) + d_off + static_cast<long long>(row) * p.ldd + col;
          if (col + 32 <= p.N) {
            #pragma unroll
            for (int j = 0; j < 8; ++j) {
              float4 o = make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                     __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
              if constexpr (EPI == EPI_ACCUM_F32) {
                float4 old = reinterpret_cast<const float4*>(dst)[j];
                o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
              }
              reinterpret_cast<float4*>(dst)[j] = o;
            }
          } else {
            for (int j = 0; j < 32 && col + j < p.N; ++j) {
              float x = __uint_as_float(v[j]);
              if constexpr (EPI == EPI_ACCUM_F32) x += dst[j];
              dst[j] = x;
            }
          }
        }
      }
    }
  }
}

template <int BN, int STAGES, bool A_MN, bool B_MN, int EPI, bool GROUPED, bool KGROUPED = false>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const GemmParams p) {
  using S = GemmSmem<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;  // [2]
  uint64_t* tempty_bar = tfull_bar + 2;      // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr uint32_t TMEM_COLS = (2 * BN <= 32) ? 32 : (2 * BN <= 64) ? 64 : (2 * BN <= 128) ? 128 : (2 * BN <= 256) ? 256 : 512;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tfull_bar[a], 1); mbar_init(&tempty_bar[a], 4); }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); tc_fence_before(); }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int num_tiles = KGROUPED ? p.tiles_per_expert * p.n_per_expert /* = E */ : p.m_blocks * p.n_blocks;
  const int tiles_per_group = p.group_m * p.n_blocks;

  auto tile_coords = [&](int t, int& mb, int& nb) {
    if constexpr (KGROUPED) t = t % p.tiles_per_expert;
    int g = t / tiles_per_group;
    int r = t - g * tiles_per_group;
    int gsz = min(p.group_m, p.m_blocks - g * p.group_m);
    mb = g * p.group_m + (r % gsz);
    nb = r / gsz;
  };

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int mb, nb; tile_coords(t, mb, nb);
        int b_row0 = nb * BN;
        int k_row0 = 0, k_blocks = p.k_blocks;
        if constexpr (GROUPED) {
          int e = p.block_expert[mb];
          if (e < 0) continue;
          if constexpr (B_MN) k_row0 = e * p.K;   // stacked [E*K, N] operand: the expert offset is on the K rows
          else b_row0 += e * p.n_per_expert;
        }
        if constexpr (KGROUPED) {
          const int e = t / p.tiles_per_expert;
          k_row0 = p.expert_rows[2 * e];
          k_blocks = p.expert_rows[2 * e + 1] / GEMM_BK;
          if (k_blocks == 0) continue;
        }
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, PFB_ERR_WAIT_EMPTY)) { ok = false; break; }
          uint8_t* sa = smem + stage * S::STAGE_BYTES;
          uint8_t* sb = sa + S::A_BYTES;
          mbar_expect_tx(&full_bar[stage], S::STAGE_BYTES);
          if constexpr (!A_MN) {
            tma_load_2d(sa, &tmA, &full_bar[stage], kb * GEMM_BK, mb * GEMM_BM);
          } else {
            #pragma unroll
            for (int j = 0; j < GEMM_BM / 64; ++j)
              tma_load_2d(sa + j * (GEMM_BK * 128), &tmA, &full_bar[stage], mb * GEMM_BM + j * 64,
                          (KGROUPED ? k_row0 : 0) + kb * GEMM_BK);
          }
          if constexpr (EPI == EPI_SWIGLU_BF16) {
            // gate rows and up rows of the stacked [gate; up] weight land side by side in one tile
            static_assert(!(EPI == EPI_SWIGLU_BF16 && B_MN), "SwiGLU epilogue needs a K-major B");
            const int half0 = (GROUPED ? b_row0 - nb * BN : 0) + nb * (BN / 2);
            const int n_half = (GROUPED ? p.n_per_expert : p.N) / 2;
            tma_load_2d(sb, &tmB, &full_bar[stage], kb * GEMM_BK, half0);
            tma_load_2d(sb + (BN / 2) * 128, &tmB, &full_bar[stage], kb * GEMM_BK, half0 + n_half);
          } else if constexpr (!B_MN) {
            tma_load_2d(sb, &tmB, &full_bar[stage], kb * GEMM_BK, b_row0);
          } else {
            #pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * (GEMM_BK * 128), &tmB, &full_bar[stage], b_row0 + j * 64, k_row0 + kb * GEMM_BK);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(GEMM_BM, BN, A_MN, B_MN, 1);
      int stage = 0; uint32_t phase = 0;
      int acc = 0; uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int k_blocks = p.k_blocks;
        if constexpr (GROUPED) {
          int mb, nb; tile_coords(t, mb, nb);
          if (p.block_expert[mb] < 0) continue;
        }
        if constexpr (KGROUPED) {
          k_blocks = p.expert_rows[2 * (t / p.tiles_per_expert) + 1] / GEMM_BK;
          if (k_blocks == 0) continue;
        }
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag, p.status, PFB_ERR_WAIT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, PFB_ERR_WAIT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * S::STAGE_BYTES);
          const uint32_t sb = sa + S::A_BYTES;
          #pragma unroll
          for (int k = 0; k < GEMM_BK / GEMM_UMMA_K; ++k) {
            uint64_t da, db;
            if constexpr (!A_MN) da = make_smem_desc_sw128(sa + k * GEMM_UMMA_K * 2, 16, 1024);
            else da = make_smem_desc_sw128(sa + k * GEMM_UMMA_K * 128, GEMM_BK * 128, 1024);
            if constexpr (!B_MN) db = make_smem_desc_sw128(sb + k * GEMM_UMMA_K * 2, 16, 1024);
            else db = make_smem_desc_sw128(sb + k * GEMM_UMMA_K * 128, GEMM_BK * 128, 1024);
            tc_mma_f16_ss(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          tc_commit(&empty_bar[stage]);  // frees the smem stage once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) tc_commit(&tfull_bar[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ---------------- epilogue (4 warps, one TMEM lane quadrant each) ----------------
    const int quad = warp & 3;
    int acc = 0; uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      int mb, nb; tile_coords(t, mb, nb);
      if constexpr (GROUPED) { if (p.block_expert[mb] < 0) continue; }
      long long d_off = 0;
      if constexpr (KGROUPED) {
        const int e = t / p.tiles_per_expert;
        if (p.expert_rows[2 * e + 1] / GEMM_BK == 0) continue;
        d_off = e * p.d_expert_stride;
      }
      if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_flag, p.status, PFB_ERR_WAIT_TMEM_FULL)) break;
      tc_fence_after();
      const int row = mb * GEMM_BM + quad * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN;
      gemm_store_tile<BN, EPI>(taddr, row, nb, p, d_off);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }
}

}  // namespace pfb
