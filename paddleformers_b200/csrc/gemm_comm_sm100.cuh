// Tensor-parallel GEMMs fused with their collective over NVLink peer memory (sm_100a).
//
//   MODE_AG  (all-gather -> GEMM, column-parallel linear with sequence-parallel input):
//     every rank owns R rows of the activation A[T, K] inside a symmetric buffer G. A few "copy" CTAs pull the other
//     ranks' row blocks into the local G with bulk async copies (cp.async.bulk, no multicast) staged through a ring in
//     shared memory (192 KB in flight per CTA, which is what it takes to cover the link latency) and publish one flag
//     per 128-row block; the GEMM CTAs walk the row blocks starting with the local ones and their TMA producer waits
//     for the flag of a block before loading it, so the transfer of block i+1 overlaps the tensor-core work on block i.
//     The gathered A stays in G for the weight-gradient GEMM of the backward pass. (A variant in which every rank
//     pushed its rows into all peers' buffers, with bulk stores or with plain vector stores from the copy CTAs,
//     measured 1.5-2.5x slower on two GPUs: a handful of CTAs keeps too few posted bytes in flight, and every
//     completion wait before a flag costs a link round trip.)
//
//   MODE_RS  (GEMM -> reduce-scatter, row-parallel linear with sequence-parallel output), two transports:
//     push (default): the epilogue TMA-stores each bf16 partial tile into the OWNER's staging slot [src_rank][R][N] with
//       peer stores and bumps a per-source counter at the owner (release, system scope); tiles of remote owners are
//       computed first. When a CTA runs out of tiles it waits (bounded) for all sources' counters and sums the tp staging
//       slots of its share of the local rows in fp32 (fixed order: deterministic). The transfer overlaps the tensor work.
//     pull (PFB_RS_PULL=1): the tile goes into THIS rank's staging, slot [owner][R][N]; the owner reads slot [its rank]
//       of every peer's staging with plain 16-byte peer loads (all tp loads of a vector in flight together) and sums in
//       rank order. The transfer starts only after the producers' tiles are done: on two GPUs, where the GEMMs are
//       long (K = 2048 ... 7168 per rank), it measured 236 / 344 us per call against 176 / 294 us for push.
//
// Flags and counters are epoch-valued and never reset. Every wait is bounded and reports PFB_ERR_WAIT_PEER.
// Dataflow precedent in the reference: Flux all_gather_gemm / gemm_reduce_scatter
// (paddleformers/cli/train/ernie_pretrain/models/sequence_parallel_utils.py:179-236).
#pragma once
#include "gemm_sm100.cuh"

namespace pfb {

constexpr int COMM_MAX_RANKS = 8;
enum { MODE_AG = 1, MODE_RS = 2 };

struct CommParams {
  int mode, rank, tp, rows_per_rank;  // rows_per_rank % 128 == 0
  const int* epoch_ptr;  // device word holding the epoch of this call (bumped by the caller on the same stream before
                         // the launch, so that a captured CUDA graph advances it on every replay)
  int n_copy_ctas;
  // AG
  const __nv_bfloat16* peer_G[COMM_MAX_RANKS];  // every rank's gathered buffer [T, K]
  __nv_bfloat16* G;                              // local one
  int* peer_ready[COMM_MAX_RANKS];               // ready pads [tp] at every rank (slot = source rank)
  int* ready;                                    // local ready pad
  int* blk_flags;                                // local [m_blocks]
  long long row_bytes;                           // K * 2
  // RS
  __nv_bfloat16* peer_stage[COMM_MAX_RANKS];     // staging [tp][R][N] at every rank
  int* peer_count[COMM_MAX_RANKS];               // counters [tp] at every rank (slot = source rank)
  int* count;                                    // local counters
  __nv_bfloat16* stage;                          // local staging
  __nv_bfloat16* out;                            // local result [R, N]
  int tiles_per_source;                          // (R / 128) * n_blocks
  int pull;                                      // RS: 1 = partial tiles stay in the producer's staging and the owner reads them
};

__device__ __forceinline__ void st_release_sys_i32(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_release_gpu_i32(int* p, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys_i32(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ld_acquire_gpu_i32(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_sys_add(int* p, int v) {
  asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// Spin until *p >= value (acquire at system or gpu scope); false + status on timeout.
template <bool SYS>
__device__ __forceinline__ bool wait_flag_ge(const int* p, int value, volatile int* abort_flag, int* status) {
  const long long t0 = global_ns();
  const long long budget = wait_budget_ns(status);
  while (true) {
    const int v = SYS ? ld_acquire_sys_i32(p) : ld_acquire_gpu_i32(p);
    if (v >= value) return true;
    if (*abort_flag) return false;
    if (global_ns() - t0 > budget) {
      *abort_flag = 1;
      if (status) atomicCAS(status, 0, PFB_ERR_WAIT_PEER);
      return false;
    }
    __nanosleep(64);
  }
}

// global (possibly peer) -> shared, completion on an mbarrier
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// shared -> global
__device__ __forceinline__ void bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(smem_src)), "r"(bytes)
               : "memory");
}

constexpr int COPY_CHUNK = 32768;  // bytes per bulk copy
constexpr int COPY_STAGES = 6;
constexpr int COPY_AHEAD = 5;        // loads in flight per copy CTA (160 KB)

struct StageMaps { CUtensorMap m[COMM_MAX_RANKS]; };  // RS: one store map per owner rank's staging buffer [tp*R, N]
constexpr int RS_STAGING_BYTES = 4 * 2 * 4096;      // per epilogue warp: two 32-row x 128-byte slabs

template <int BN, int STAGES, bool B_MN, int EPI, int MODE>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_comm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ StageMaps stage_maps, const GemmParams p, const CommParams c) {
  using S = GemmSmem<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* rs_staging = smem + S::BAR_OFFSET;         // MODE_RS only (the barriers then follow it)
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::BAR_OFFSET + (MODE == MODE_RS ? RS_STAGING_BYTES : 0));
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint64_t* copy_bar = reinterpret_cast<uint64_t*>(tmem_slot + 2);  // [COPY_STAGES], 8-byte aligned (tmem_slot + 2 ints)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t TMEM_COLS = (2 * BN <= 256) ? 256 : 512;
  const bool is_copy_cta = MODE == MODE_AG && static_cast<int>(blockIdx.x) < c.n_copy_ctas;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tfull_bar[a], 1); mbar_init(&tempty_bar[a], 4); }
    for (int s = 0; s < COPY_STAGES; ++s) mbar_init(&copy_bar[s], 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1 && !is_copy_cta) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); tc_fence_before(); }
  __syncthreads();
  tc_fence_after();

  const int blocks_per_rank = c.rows_per_rank / GEMM_BM;
  const int epoch = *c.epoch_ptr;

  if (is_copy_cta) {
    // ------------------------------------------------------------------ all-gather copy CTAs
    if (threadIdx.x == 0) {
      if (blockIdx.x == 0) {
        // this rank's own slice of G was written by earlier work on this stream: tell everyone
        __threadfence_system();
        for (int q = 0; q < c.tp; ++q) st_release_sys_i32(c.peer_ready[q] + c.rank, epoch);
      }
      const long long blk_bytes = static_cast<long long>(GEMM_BM) * c.row_bytes;
      const int chunks_per_blk = static_cast<int>(blk_bytes / COPY_CHUNK);  // row_bytes*128 is a multiple of 32 KB for K % 128 == 0
      int issue_stage = 0, done_stage = 0;
      uint32_t done_phase = 0;
      bool ok = true;
      int item = 0;
      for (int d = 1; d < c.tp && ok; ++d) {
        const int src = (c.rank + d) % c.tp;
        for (int b = 0; b < blocks_per_rank && ok; ++b, ++item) {
          if (item % c.n_copy_ctas != static_cast<int>(blockIdx.x)) continue;
          if (!wait_flag_ge<true>(c.ready + src, epoch, abort_flag, p.status)) { ok = false; break; }
          const int mb = src * blocks_per_rank + b;
          const uint8_t* gsrc = reinterpret_cast<const uint8_t*>(c.peer_G[src]) + mb * blk_bytes;
          uint8_t* gdst = reinterpret_cast<uint8_t*>(c.G) + mb * blk_bytes;
          int issued = 0, stored = 0;
          while (stored < chunks_per_blk && ok) {
            // keep up to COPY_AHEAD loads in flight. The slot of load n held chunk n - COPY_STAGES; at least
            // n - COPY_AHEAD + 1 stores have been committed by now, so that chunk's store is followed by at most
            // COPY_STAGES - COPY_AHEAD newer ones: waiting until no more than that many are still reading frees it
            while (issued < chunks_per_blk && issued - stored < COPY_AHEAD) {
              tma_store_wait_read<COPY_STAGES - COPY_AHEAD>();
              mbar_expect_tx(&copy_bar[issue_stage], COPY_CHUNK);
              bulk_load(smem + issue_stage * COPY_CHUNK, gsrc + static_cast<long long>(issued) * COPY_CHUNK, COPY_CHUNK,
                        &copy_bar[issue_stage]);
              issue_stage = (issue_stage + 1) % COPY_STAGES;
              ++issued;
            }
            if (!mbar_wait(&copy_bar[done_stage], done_phase, abort_flag, p.status, PFB_ERR_WAIT_PEER)) { ok = false; break; }
            bulk_store(gdst + static_cast<long long>(stored) * COPY_CHUNK, smem + done_stage * COPY_CHUNK, COPY_CHUNK);
            tma_store_commit();
            if (++done_stage == COPY_STAGES) { done_stage = 0; done_phase ^= 1; }
            ++stored;
          }
          if (ok) {
            tma_store_wait<0>();          // the block is in local memory
            fence_proxy_async_all();
            __threadfence();
            st_release_gpu_i32(c.blk_flags + mb, epoch);
          }
        }
      }
      tma_store_wait<0>();
    }
    return;  // copy CTAs allocate no TMEM
  }

  const uint32_t tmem_base = *tmem_slot;
  const int first_cta = MODE == MODE_AG ? c.n_copy_ctas : 0;
  const int n_ctas = gridDim.x - first_cta;
  const int my_cta = blockIdx.x - first_cta;
  const int num_tiles = p.m_blocks * p.n_blocks;
  const int tiles_per_group = p.group_m * p.n_blocks;
  // AG walks row blocks starting at this rank's own rows; RS starts with the next rank's rows (own rows last)
  const int m_shift = (MODE == MODE_AG ? c.rank : (c.rank + 1) % c.tp) * blocks_per_rank;

  auto tile_coords = [&](int t, int& mb, int& nb) {
    int g = t / tiles_per_group;
    int r = t - g * tiles_per_group;
    int gsz = min(p.group_m, p.m_blocks - g * p.group_m);
    int mlog = g * p.group_m + (r % gsz);
    mb = (mlog + m_shift) % p.m_blocks;
    nb = r / gsz;
  };

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (int t = my_cta; t < num_tiles && ok; t += n_ctas) {
        int mb, nb; tile_coords(t, mb, nb);
        if constexpr (MODE == MODE_AG) {
          if (mb / blocks_per_rank != c.rank) {
            if (!wait_flag_ge<false>(c.blk_flags + mb, epoch, abort_flag, p.status)) break;
            fence_proxy_async_all();
          }
        }
        const int b_row0 = nb * BN;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, PFB_ERR_WAIT_EMPTY)) { ok = false; break; }
          uint8_t* sa = smem + stage * S::STAGE_BYTES;
          uint8_t* sb = sa + S::A_BYTES;
          mbar_expect_tx(&full_bar[stage], S::STAGE_BYTES);
          tma_load_2d(sa, &tmA, &full_bar[stage], kb * GEMM_BK, mb * GEMM_BM);
          if constexpr (EPI == EPI_SWIGLU_BF16) {
            const int half0 = nb * (BN / 2);
            tma_load_2d(sb, &tmB, &full_bar[stage], kb * GEMM_BK, half0);
            tma_load_2d(sb + (BN / 2) * 128, &tmB, &full_bar[stage], kb * GEMM_BK, half0 + p.N / 2);
          } else if constexpr (!B_MN) {
            tma_load_2d(sb, &tmB, &full_bar[stage], kb * GEMM_BK, b_row0);
          } else {
            #pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * (GEMM_BK * 128), &tmB, &full_bar[stage], b_row0 + j * 64, kb * GEMM_BK);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(GEMM_BM, BN, false, B_MN, 1);
      int stage = 0; uint32_t phase = 0;
      int acc = 0; uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = my_cta; t < num_tiles && ok; t += n_ctas) {
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag, p.status, PFB_ERR_WAIT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, PFB_ERR_WAIT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * S::STAGE_BYTES);
          const uint32_t sb = sa + S::A_BYTES;
          #pragma unroll
          for (int k = 0; k < GEMM_BK / GEMM_UMMA_K; ++k) {
            const uint64_t da = make_smem_desc_sw128(sa + k * GEMM_UMMA_K * 2, 16, 1024);
            uint64_t db;
            if constexpr (!B_MN) db = make_smem_desc_sw128(sb + k * GEMM_UMMA_K * 2, 16, 1024);
            else db = make_smem_desc_sw128(sb + k * GEMM_UMMA_K * 128, GEMM_BK * 128, 1024);
            tc_mma_f16_ss(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          tc_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) tc_commit(&tfull_bar[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    const int quad = warp & 3;
    int acc = 0; uint32_t acc_phase = 0;
    bool ok = true;
    int rs_prev_owner = -1;
    for (int t = my_cta; t < num_tiles; t += n_ctas) {
      int mb, nb; tile_coords(t, mb, nb);
      if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_flag, p.status, PFB_ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int row = mb * GEMM_BM + quad * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN;
      if constexpr (MODE == MODE_RS) {
        // Each warp moves its 32 rows through two private 4 KB swizzled slabs and TMA-stores them into the owner's
        // staging slot (full 128-byte lines over NVLink); only __syncwarp is needed, never a cross-warp barrier.
        const int owner = mb / blocks_per_rank;
        const int slot_idx = c.pull ? owner : c.rank;            // slot inside the staging buffer that receives the tile
        const int srow0 = slot_idx * c.rows_per_rank + (mb * GEMM_BM + quad * 32 - owner * c.rows_per_rank);
        const CUtensorMap* store_map = &stage_maps.m[c.pull ? c.rank : owner];
        uint8_t* my_stg = rs_staging + (warp - 2) * 8192;
        #pragma unroll 1
        for (int cc = 0; cc < BN; cc += 64) {
          uint32_t v0[32], v1[32];
          tmem_ld_32x32(taddr + cc, v0);
          tmem_ld_32x32(taddr + cc + 32, v1);
          tmem_ld_wait();
          uint8_t* slab = my_stg + ((cc >> 6) & 1) * 4096;
          if (lane == 0) tma_store_wait_read<1>();   // the slab used two steps ago has been read out
          __syncwarp();
          uint8_t* rowp = slab + lane * 128;
          #pragma unroll
          for (int j = 0; j < 4; ++j) {
            *reinterpret_cast<uint4*>(rowp + ((j ^ (lane & 7)) << 4)) = make_uint4(
                pack_bf16x2(__uint_as_float(v0[8 * j]), __uint_as_float(v0[8 * j + 1])),
                pack_bf16x2(__uint_as_float(v0[8 * j + 2]), __uint_as_float(v0[8 * j + 3])),
                pack_bf16x2(__uint_as_float(v0[8 * j + 4]), __uint_as_float(v0[8 * j + 5])),
                pack_bf16x2(__uint_as_float(v0[8 * j + 6]), __uint_as_float(v0[8 * j + 7])));
            *reinterpret_cast<uint4*>(rowp + (((j + 4) ^ (lane & 7)) << 4)) = make_uint4(
                pack_bf16x2(__uint_as_float(v1[8 * j]), __uint_as_float(v1[8 * j + 1])),
                pack_bf16x2(__uint_as_float(v1[8 * j + 2]), __uint_as_float(v1[8 * j + 3])),
                pack_bf16x2(__uint_as_float(v1[8 * j + 4]), __uint_as_float(v1[8 * j + 5])),
                pack_bf16x2(__uint_as_float(v1[8 * j + 6]), __uint_as_float(v1[8 * j + 7])));
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0 && nb * BN + cc < p.N) {
            tma_store_2d(store_map, slab, nb * BN + cc, srow0);
            tma_store_commit();
          }
        }
        // publish the PREVIOUS tile of this warp (its stores are complete once at most this tile's groups are pending)
        if (lane == 0) {
          if (rs_prev_owner >= 0) {
            tma_store_wait<BN / 64>();
            fence_proxy_async_all();
            __threadfence_system();
            red_release_sys_add(c.peer_count[rs_prev_owner] + c.rank, 1);
          }
          rs_prev_owner = owner;
        }
      } else if constexpr (EPI == EPI_SWIGLU_BF16) {
        __nv_bfloat16* Dp = reinterpret_cast<__nv_bfloat16*>(p.D);
        const int n_out = p.N / 2;
        #pragma unroll 1
        for (int cc = 0; cc < BN / 2; cc += 32) {
          uint32_t g[32], u[32];
          tmem_ld_32x32(taddr + cc, g);
          tmem_ld_32x32(taddr + BN / 2 + cc, u);
          tmem_ld_wait();
          const int col = nb * (BN / 2) + cc;
          if (row < p.M && col < n_out) {
            __nv_bfloat16* r0 = reinterpret_cast<__nv_bfloat16*>(p.D2) + static_cast<long long>(row) * p.ldd2 + col;
            __nv_bfloat16* r1 = r0 + n_out;
            __nv_bfloat16* dst = Dp + static_cast<long long>(row) * p.ldd + col;
            if (col + 32 <= n_out) {
              #pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint32_t o[4];
                #pragma unroll
                for (int q = 0; q < 4; ++q) {
                  const float g0 = __uint_as_float(g[8 * j + 2 * q]), g1 = __uint_as_float(g[8 * j + 2 * q + 1]);
                  const float u0 = __uint_as_float(u[8 * j + 2 * q]), u1 = __uint_as_float(u[8 * j + 2 * q + 1]);
                  o[q] = pack_bf16x2(__fdividef(g0, 1.f + __expf(-g0)) * u0, __fdividef(g1, 1.f + __expf(-g1)) * u1);
                }
                reinterpret_cast<uint4*>(dst)[j] = make_uint4(o[0], o[1], o[2], o[3]);
                if (p.D2) {
                  reinterpret_cast<uint4*>(r0)[j] = make_uint4(pack_bf16x2(__uint_as_float(g[8 * j]), __uint_as_float(g[8 * j + 1])),
                      pack_bf16x2(__uint_as_float(g[8 * j + 2]), __uint_as_float(g[8 * j + 3])),
                      pack_bf16x2(__uint_as_float(g[8 * j + 4]), __uint_as_float(g[8 * j + 5])),
                      pack_bf16x2(__uint_as_float(g[8 * j + 6]), __uint_as_float(g[8 * j + 7])));
                  reinterpret_cast<uint4*>(r1)[j] = make_uint4(pack_bf16x2(__uint_as_float(u[8 * j]), __uint_as_float(u[8 * j + 1])),
                      pack_bf16x2(__uint_as_float(u[8 * j + 2]), __uint_as_float(u[8 * j + 3])),
                      pack_bf16x2(__uint_as_float(u[8 * j + 4]), __uint_as_float(u[8 * j + 5])),
                      pack_bf16x2(__uint_as_float(u[8 * j + 6]), __uint_as_float(u[8 * j + 7])));
                }
              }
            } else {
              for (int j = 0; j < 32 && col + j < n_out; ++j) {
                const float g0 = __uint_as_float(g[j]), u0 = __uint_as_float(u[j]);
                dst[j] = __float2bfloat16(g0 / (1.f + __expf(-g0)) * u0);
                if (p.D2) { r0[j] = __float2bfloat16(g0); r1[j] = __float2bfloat16(u0); }
              }
            }
          }
        }
      } else {
        #pragma unroll 1
        for (int cc = 0; cc < BN; cc += 32) {
          uint32_t v[32];
          tmem_ld_32x32(taddr + cc, v);
          tmem_ld_wait();
          const int col = nb * BN + cc;
          if (row < p.M && col < p.N) {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.D) + static_cast<long long>(row) * p.ldd + col;
            if (col + 32 <= p.N) {
              #pragma unroll
              for (int j = 0; j < 4; ++j)
                reinterpret_cast<uint4*>(dst)[j] = make_uint4(
                    pack_bf16x2(__uint_as_float(v[8 * j]), __uint_as_float(v[8 * j + 1])),
                    pack_bf16x2(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3])),
                    pack_bf16x2(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5])),
                    pack_bf16x2(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7])));
            } else {
              for (int j = 0; j < 32 && col + j < p.N; ++j) dst[j] = __float2bfloat16(__uint_as_float(v[j]));
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }

    if constexpr (MODE == MODE_RS) {
      if (lane == 0) {
        tma_store_wait<0>();
        if (rs_prev_owner >= 0) {
          fence_proxy_async_all();
          __threadfence_system();
          red_release_sys_add(c.peer_count[rs_prev_owner] + c.rank, 1);
        }
      }
      __syncwarp();
      // ---------------------------------------------------------------- reduce the tp staging slots of the local rows
      // 128 epilogue threads per CTA; CTA i handles 8-element column vectors i, i + n_ctas, ... of the [R, N] result.
      if (ok) {
        const int target = epoch * c.tiles_per_source * 4;
        bool ready = true;
        for (int q = 0; q < c.tp && ready; ++q) ready = wait_flag_ge<true>(c.count + q, target, abort_flag, p.status);
        if (ready) {
          const long long nvec = static_cast<long long>(c.rows_per_rank) * p.N / 8;
          const long long slot = static_cast<long long>(c.rows_per_rank) * p.N;
          const int tid = (warp - 2) * 32 + lane;
          const long long stride = static_cast<long long>(n_ctas) * 128;
          if (c.pull) {
            // two vectors per thread and iteration, the tp loads of both issued before any is used: 2 * tp peer loads
            // (16 bytes each) in flight per thread cover the link latency
            const long long mine = static_cast<long long>(c.rank) * slot;
            for (long long i0 = static_cast<long long>(my_cta) * 128 + tid; i0 < nvec; i0 += 2 * stride) {
              const long long i1 = i0 + stride;
              uint4 ra[COMM_MAX_RANKS], rb[COMM_MAX_RANKS];
              #pragma unroll
              for (int q = 0; q < COMM_MAX_RANKS; ++q) {
                ra[q] = make_uint4(0, 0, 0, 0); rb[q] = make_uint4(0, 0, 0, 0);
                if (q < c.tp) {
                  const __nv_bfloat16* src = c.peer_stage[q] + mine;
                  ra[q] = *reinterpret_cast<const uint4*>(src + i0 * 8);
                  if (i1 < nvec) rb[q] = *reinterpret_cast<const uint4*>(src + i1 * 8);
                }
              }
              float sa[8], sb[8];
              #pragma unroll
              for (int j = 0; j < 8; ++j) { sa[j] = 0.f; sb[j] = 0.f; }
              #pragma unroll
              for (int q = 0; q < COMM_MAX_RANKS; ++q) {
                const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&ra[q]);
                const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&rb[q]);
                #pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float2 fa = __bfloat1622float2(ha[j]), fb = __bfloat1622float2(hb[j]);
                  sa[2 * j] += fa.x; sa[2 * j + 1] += fa.y; sb[2 * j] += fb.x; sb[2 * j + 1] += fb.y;
                }
              }
              *reinterpret_cast<uint4*>(c.out + i0 * 8) = make_uint4(pack_bf16x2(sa[0], sa[1]), pack_bf16x2(sa[2], sa[3]),
                                                                     pack_bf16x2(sa[4], sa[5]), pack_bf16x2(sa[6], sa[7]));
              if (i1 < nvec)
                *reinterpret_cast<uint4*>(c.out + i1 * 8) = make_uint4(pack_bf16x2(sb[0], sb[1]), pack_bf16x2(sb[2], sb[3]),
                                                                       pack_bf16x2(sb[4], sb[5]), pack_bf16x2(sb[6], sb[7]));
            }
          } else {
          // four independent vectors per thread and iteration: tp * 4 loads in flight hide the DRAM latency
          for (long long i0 = static_cast<long long>(my_cta) * 128 + tid; i0 < nvec; i0 += 4 * stride) {
            float accv[4][8];
            #pragma unroll
            for (int u = 0; u < 4; ++u)
              #pragma unroll
              for (int j = 0; j < 8; ++j) accv[u][j] = 0.f;
            for (int q = 0; q < c.tp; ++q) {
              uint4 raw[4];
              #pragma unroll
              for (int u = 0; u < 4; ++u) {
                const long long i = i0 + u * stride;
                raw[u] = i < nvec ? *reinterpret_cast<const uint4*>(c.stage + q * slot + i * 8) : make_uint4(0, 0, 0, 0);
              }
              #pragma unroll
              for (int u = 0; u < 4; ++u) {
                const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[u]);
                #pragma unroll
                for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h[j]); accv[u][2 * j] += f.x; accv[u][2 * j + 1] += f.y; }
              }
            }
            #pragma unroll
            for (int u = 0; u < 4; ++u) {
              const long long i = i0 + u * stride;
              if (i < nvec)
                *reinterpret_cast<uint4*>(c.out + i * 8) = make_uint4(pack_bf16x2(accv[u][0], accv[u][1]), pack_bf16x2(accv[u][2], accv[u][3]),
                                                                     pack_bf16x2(accv[u][4], accv[u][5]), pack_bf16x2(accv[u][6], accv[u][7]));
            }
          }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }
}

}  // namespace pfb
