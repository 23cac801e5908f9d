// CTA-pair bf16 GEMM for sm_100a: one 256 x 256 output tile per cluster of two CTAs (tcgen05 cta_group::2).
//
//   D[M,N] = A[M,K] * B[N,K]^T        (fp32 accumulation; A / B each K-major or MN-major as in gemm_sm100.cuh)
//
// Each CTA of the pair loads ITS OWN 128 rows of A and ITS OWN 128 rows of B (plain per-CTA TMA loads, no multicast);
// the leader CTA's single MMA thread issues 256 x 256 x 16 products that read both CTAs' shared memory and write each
// CTA's 128 accumulator rows into that CTA's TMEM. Per k-block a CTA therefore moves 32 KB through shared memory for
// 128 x 256 x 64 of its own output, against 48 KB in the one-CTA kernel: operand delivery, not the tensor pipe, is what
// limits the one-CTA kernel. Six stages of 32 KB; two 256-column accumulators per CTA (epilogue of tile i under the
// main loop of tile i + 1); epilogues shared with the one-CTA kernel.
//
// Synchronisation between the two CTAs:
//   * data ready:   the TMA loads of BOTH CTAs complete on the LEADER's mbarrier of the stage (cta_group::2 form of the
//                   load, which may signal a barrier in the peer CTA); the leader's producer arms it with the byte count
//                   of both halves, so the MMA thread waits on one barrier and no relay hop sits in the ring's latency;
//   * stage free /  tcgen05.commit (cta_group::2) towards the leader's own barrier and, separately, towards the peer's
//     tile done:    barrier at the same offset (its cluster address), so no multicast form is needed;
//   * accumulator   the four epilogue warps of BOTH CTAs arrive on the leader's barrier (the peer's remotely).
//     drained:
// Every wait is bounded; a CTA that gives up still takes part in the closing cluster barrier, so its peer never
// signals into shared memory of a CTA that has exited.
#pragma once
#include "gemm_sm100.cuh"

namespace pfb {

constexpr int G2_STAGES = 7;          // six when the epilogue stages its tiles in shared memory (EPI_REDUCE_F32)
constexpr int G2_STAGING_BYTES = 4 * 2 * 4096;   // per epilogue warp: two 32-row x 128-byte slabs
constexpr int G2_BN = 256;            // accumulator columns per CTA (= tile N)
constexpr int G2_HALF = 128;          // B rows loaded by each CTA

template <int STAGES, int STAGING>
struct Gemm2SmemT {
  static constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;     // 16 KB
  static constexpr int B_BYTES = G2_HALF * GEMM_BK * 2;     // 16 KB
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGING_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int BAR_OFFSET = STAGING_OFFSET + STAGING;
  static constexpr int TOTAL = BAR_OFFSET + 512 + 1024;
};
template <int EPI>
using Gemm2SmemFor = Gemm2SmemT<(EPI == EPI_REDUCE_F32 ? G2_STAGES - 1 : G2_STAGES), (EPI == EPI_REDUCE_F32 ? G2_STAGING_BYTES : 0)>;
using Gemm2Smem = Gemm2SmemFor<EPI_STORE_BF16>;

__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* m, const void* smem_src, int c0, int c1) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1)
               : "memory");
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(addr), "r"(rank));
  return out;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait with cluster-scope acquire (the arrival may come from the peer CTA).
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status, int err_code) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  const long long t0 = global_ns();
  const long long budget = wait_budget_ns(status);
  while (true) {
    #pragma unroll 1
    for (int i = 0; i < 64; ++i)
      if (mbar_try_wait_cluster(bar, parity)) return true;
    if (*abort_flag) return false;
    if (global_ns() - t0 > budget) {
      *abort_flag = 1;
      if (status) atomicCAS(status, 0, err_code);
      return false;
    }
  }
}
// 2-D tiled load whose completion is signalled on the mbarrier at a CLUSTER address (the leader CTA's barrier).
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster_addr, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// Arrive on the mbarrier at a cluster address once all tcgen05.mma issued so far by this thread have completed.
__device__ __forceinline__ void tc_commit2(uint32_t cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tc_mma2_f16_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

template <bool A_MN, bool B_MN, int EPI>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm2_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const __grid_constant__ CUtensorMap tmD, const GemmParams p) {
  using S = Gemm2SmemFor<EPI>;
  constexpr int STAGES = (EPI == EPI_REDUCE_F32) ? G2_STAGES - 1 : G2_STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::BAR_OFFSET);   // [STAGES] leader only: both CTAs' loads have landed
  uint64_t* empty_bar = full_bar + STAGES;                               // [STAGES] the products that read a stage are done
  uint64_t* tfull_bar = empty_bar + STAGES;                              // [2] accumulator complete
  uint64_t* tempty_bar = tfull_bar + 2;                                     // [2] leader only: drained by both CTAs
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();          // 0 = leader
  const bool leader = cta == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tfull_bar[a], 1); mbar_init(&tempty_bar[a], 8); }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) { tmem_alloc2(tmem_slot, 512); tmem_relinquish2(); tc_fence_before(); }
  __syncthreads();
  cluster_sync_all();               // both CTAs' barriers are initialised before anybody signals across
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // tiles: 256-row block pairs x 256-column blocks, walked in groups for L2 reuse
  const int m_pairs = (p.M + 2 * GEMM_BM - 1) / (2 * GEMM_BM);
  const int n_blocks = p.n_blocks;
  const int num_tiles = m_pairs * n_blocks;
  const int n_clusters = gridDim.x >> 1;
  const int my_cluster = blockIdx.x >> 1;
  const int tiles_per_group = p.group_m * n_blocks;
  auto tile_coords = [&](int t, int& mp, int& nb) {
    int g = t / tiles_per_group;
    int r = t - g * tiles_per_group;
    int gsz = min(p.group_m, m_pairs - g * p.group_m);
    mp = g * p.group_m + (r % gsz);
    nb = r / gsz;
  };
  // Wave quantisation: with T tiles on C clusters the last round keeps only T mod C clusters busy. When that remainder is
  // at most C / 2 the host asks for those tiles to be computed as two 128-column halves each (a unit of work half as
  // long), so the last round takes half the time. Units [0, n_whole) are whole tiles, the rest are halves.
  const int n_whole = num_tiles - p.split_tail;
  const int num_units = n_whole + 2 * p.split_tail;
  auto unit_coords = [&](int v, int& mp, int& nb, int& half) {
    int t = v;
    half = -1;
    if (v >= n_whole) { const int h = v - n_whole; t = n_whole + (h >> 1); half = h & 1; }
    tile_coords(t, mp, nb);
  };

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs, each for its own halves) ----------------
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      const uint32_t leader_full0 = mapa_shared(smem_u32(&full_bar[0]), 0);
      for (int t = my_cluster; t < num_units && ok; t += n_clusters) {
        int mp, nb, half; unit_coords(t, mp, nb, half);
        const int a_row0 = mp * 2 * GEMM_BM + static_cast<int>(cta) * GEMM_BM;
        const int nbox = half >= 0 ? 1 : 2;                    // 64-row boxes of B per CTA and stage
        int b_row0;
        if constexpr (EPI == EPI_SWIGLU_BF16)                  // leader: gate rows, peer: up rows
          b_row0 = nb * G2_HALF + (half > 0 ? 64 : 0) + static_cast<int>(cta) * (p.N / 2);
        else
          b_row0 = nb * G2_BN + (half >= 0 ? half * G2_HALF + static_cast<int>(cta) * 64 : static_cast<int>(cta) * G2_HALF);
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait_cluster(&empty_bar[stage], phase ^ 1, abort_flag, p.status, PFB_ERR_WAIT_EMPTY)) { ok = false; break; }
          uint8_t* sa = smem + stage * S::STAGE_BYTES;
          uint8_t* sb = sa + S::A_BYTES;
          const uint32_t fb = leader_full0 + stage * 8;
          if (leader) mbar_expect_tx(&full_bar[stage], 2 * (S::A_BYTES + nbox * (S::B_BYTES / 2)));   // this CTA's bytes and the peer's
          if constexpr (!A_MN) {
            tma_load_2d_pair(sa, &tmA, fb, kb * GEMM_BK, a_row0);
          } else {
            #pragma unroll
            for (int j = 0; j < GEMM_BM / 64; ++j)
              tma_load_2d_pair(sa + j * (GEMM_BK * 128), &tmA, fb, a_row0 + j * 64, kb * GEMM_BK);
          }
          for (int j = 0; j < nbox; ++j) {
            if constexpr (!B_MN) tma_load_2d_pair(sb + j * (64 * 128), &tmB, fb, kb * GEMM_BK, b_row0 + j * 64);
            else tma_load_2d_pair(sb + j * (GEMM_BK * 128), &tmB, fb, b_row0 + j * 64, kb * GEMM_BK);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      if (leader) {
        // ---------------- leader: MMA issuer for the pair ----------------
        constexpr uint32_t idesc_whole = make_idesc(2 * GEMM_BM, G2_BN, A_MN, B_MN, 1);
        constexpr uint32_t idesc_half = make_idesc(2 * GEMM_BM, G2_HALF, A_MN, B_MN, 1);
        const uint32_t peer_empty0 = mapa_shared(smem_u32(&empty_bar[0]), 1);
        const uint32_t peer_tfull0 = mapa_shared(smem_u32(&tfull_bar[0]), 1);
        int acc = 0; uint32_t acc_phase = 0;
        for (int t = my_cluster; t < num_units && ok; t += n_clusters) {
          const uint32_t idesc = t >= n_whole ? idesc_half : idesc_whole;
          if (!mbar_wait_cluster(&tempty_bar[acc], acc_phase ^ 1, abort_flag, p.status, PFB_ERR_WAIT_TMEM_EMPTY)) break;
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + acc * G2_BN;
          for (int kb = 0; kb < p.k_blocks; ++kb) {
            if (!mbar_wait_cluster(&full_bar[stage], phase, abort_flag, p.status, PFB_ERR_WAIT_FULL)) { ok = false; break; }
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
              tc_mma2_f16_ss(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
            }
            // the stage is free in BOTH CTAs once these products have read it
            tc_commit2(smem_u32(&empty_bar[stage]));
            tc_commit2(peer_empty0 + stage * 8);
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
          if (ok) { tc_commit2(smem_u32(&tfull_bar[acc])); tc_commit2(peer_tfull0 + acc * 8); }
          if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        }
      }
    }
  } else {
    // ---------------- epilogue (4 warps per CTA, one TMEM lane quadrant each) ----------------
    const int quad = warp & 3;
    const uint32_t leader_tempty0 = mapa_shared(smem_u32(&tempty_bar[0]), 0);
    int acc = 0; uint32_t acc_phase = 0;
    for (int t = my_cluster; t < num_units; t += n_clusters) {
      int mp, nb, half; unit_coords(t, mp, nb, half);
      if (!mbar_wait_cluster(&tfull_bar[acc], acc_phase, abort_flag, p.status, PFB_ERR_WAIT_TMEM_FULL)) break;
      tc_fence_after();
      const int row = mp * 2 * GEMM_BM + static_cast<int>(cta) * GEMM_BM + quad * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * G2_BN;
      if constexpr (EPI == EPI_REDUCE_F32) {
        // each warp moves its 32 rows through two private 4 KB slabs (32 fp32 columns = one 128-byte swizzle row per
        // row) and hands them to the TMA unit as reduce-add operations: D += tile is formed in L2
        uint8_t* my_stg = smem + S::STAGING_OFFSET + (warp - 2) * 8192;
        const int row0 = row - lane;
        const int width = half >= 0 ? G2_HALF : G2_BN;
        const int col0 = nb * G2_BN + (half > 0 ? G2_HALF : 0);
        #pragma unroll 1
        for (int c = 0; c < width; c += 32) {
          uint32_t v[32];
          tmem_ld_32x32(taddr + c, v);
          tmem_ld_wait();
          uint8_t* slab = my_stg + ((c >> 5) & 1) * 4096;
          if (lane == 0) tma_store_wait_read<1>();   // the slab used two steps ago has been read out
          __syncwarp();
          uint8_t* rowp = slab + lane * 128;
          #pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<uint4*>(rowp + ((j ^ (lane & 7)) << 4)) = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0 && row0 < p.M && col0 + c < p.N) {
            tma_reduce_add_2d(&tmD, slab, col0 + c, row0);
            tma_store_commit();
          }
        }
      } else if (half >= 0) {
        gemm_store_tile<G2_HALF, EPI>(taddr, row, 2 * nb + half, p, 0);
      } else {
        gemm_store_tile<G2_BN, EPI>(taddr, row, nb, p, 0);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(leader_tempty0 + acc * 8);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
    if constexpr (EPI == EPI_REDUCE_F32) {
      if (lane == 0) tma_store_wait<0>();      // the staging slabs stay valid until the last reduction has read them
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();               // nobody signals into a CTA that has left
  if (warp == 1) { tc_fence_after(); tmem_dealloc2(tmem_base, 512); }
}

}  // namespace pfb
