// Large-M kernel, two-SM form: a cluster of two CTAs owns a 256 x 256 output
// tile and drives it with tcgen05.mma.cta_group::2 (UMMA M = 256, N = 256).
// CTA r of the pair holds rows [128 r, 128 r + 128) of the tile: it loads those
// 128 rows of A and 128 of the tile's 256 weight rows per k-block (32 KiB per
// stage instead of 48 KiB, so the ring is six deep and the shared-memory and
// L2 traffic per flop drop by a third), keeps its 128 x 256 accumulator in its
// own TMEM and stores its own half of C.  Only the leader CTA issues MMAs.
//
// Cross-CTA signalling, all without multicast:
//   * both CTAs' TMA loads complete their bytes on the LEADER's full barrier
//     (the .cta_group::2 form of the load allows the barrier to live in the
//     peer CTA);
//   * the leader frees a stage / publishes an accumulator with two
//     tcgen05.commit, one per CTA's barrier;
//   * the follower's epilogue warps hand the accumulator back with a remote
//     mbarrier.arrive on the leader's barrier.
#pragma once
#include "gemm_kernels.cuh"

namespace flyb200 {

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_id_x() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t num_clusters_x() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%nclusterid.x;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t mapa_u32(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_barrier_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// arrive on an mbarrier that may live in the peer CTA (shared::cluster address)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_alloc_2sm(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_2sm() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_2sm(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// TMA loads whose completion bytes are credited to a barrier given as a
// shared::cluster address (the leader's), no multicast.
__device__ __forceinline__ void tma_load_2d_2sm(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster, int x, int y,
                                                uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%3, %4}], [%2], %5;" ::"r"(dst),
      "l"(map), "r"(bar_cluster), "r"(x), "r"(y), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d_2sm(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster, int x, int y,
                                                int z, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%3, %4, %5}], [%2], %6;" ::"r"(dst),
      "l"(map), "r"(bar_cluster), "r"(x), "r"(y), "r"(z), "l"(policy)
      : "memory");
}
template <int KIND>
__device__ __forceinline__ void umma_ss_2sm(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
  if constexpr (KIND == KIND_F8) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else if constexpr (KIND == KIND_I8) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
// completion of all MMAs issued so far by this thread -> one arrival on the
// barrier at `bar_cluster` (own CTA or the peer)
__device__ __forceinline__ void umma_commit_2sm(uint32_t bar_cluster) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster)
               : "memory");
}

template <int STAGES>
struct Rows2Smem {
  static constexpr int A_STAGE = BLOCK_ROWS * KBLOCK_BYTES;  // this CTA's 128 rows of A
  static constexpr int B_STAGE = BLOCK_ROWS * KBLOCK_BYTES;  // this CTA's 128 of the tile's 256 weight rows
  static constexpr int C_BUF = 32 * 128;
  static constexpr int OFF_A = 0;
  static constexpr int OFF_B = OFF_A + STAGES * A_STAGE;
  static constexpr int OFF_C = OFF_B + STAGES * B_STAGE;
  static constexpr int OFF_BAR = OFF_C + 4 * 2 * C_BUF;  // full[S], empty[S], tfull[2], tempty[2]
  static constexpr int OFF_MISC = OFF_BAR + 8 * (2 * STAGES + 4);
  static constexpr int TOTAL = OFF_MISC + 16;
};

template <int KIND, int STAGES, int OUTMODE>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_rows2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW,
                  const __grid_constant__ CUtensorMap tmC, const GemmParams p) {
  using L = Rows2Smem<STAGES>;
  using KT = KindTraits<KIND>;
  constexpr int BN = 256;        // tile columns (UMMA N)
  constexpr int TILE_ROWS = 256; // tile rows of the CTA pair (UMMA M)
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t smem_base = smem_u32(smem_raw);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_raw + L::OFF_MISC + 4);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_raw + L::OFF_MISC);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();  // 0 = leader
  const uint32_t bar_full = smem_base + L::OFF_BAR;
  const uint32_t bar_empty = bar_full + 8 * STAGES;
  const uint32_t bar_tfull = bar_empty + 8 * STAGES;
  const uint32_t bar_tempty = bar_tfull + 16;

  if ((smem_base & 1023u) != 0) {  // same answer in every CTA of the grid
    if (threadIdx.x == 0) atomicCAS(p.status, 0, ST_SMEM_ALIGN);
    return;
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);   // leader: its own expect_tx arrival; bytes come from both CTAs
      mbar_init(bar_empty + 8 * s, 1);  // one tcgen05.commit from the leader
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_tfull + 8 * s, 1);   // one tcgen05.commit from the leader
      mbar_init(bar_tempty + 8 * s, 8);  // four epilogue warps of each CTA (used in the leader only)
    }
    abort_flag[0] = 0;
    abort_flag[1] = 0;
    fence_mbar_init();
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmW);
    if (OUTMODE != OUT_RAW32) prefetch_tensormap(&tmC);
  }
  constexpr uint32_t TMEM_COLS = 512;
  if (warp == 1) {
    tmem_alloc_2sm(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish_2sm();
  }
  tc_fence_before();
  cluster_barrier_all();  // barriers of both CTAs initialised, TMEM of the pair allocated
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int num_m = (p.M + TILE_ROWS - 1) / TILE_ROWS;
  const int num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = p.K_bytes / KBLOCK_BYTES;
  const int gm_full = p.group_m;
  const int first_tile = static_cast<int>(cluster_id_x());
  const int tile_step = static_cast<int>(num_clusters_x());

  auto tile_coords = [&](int t, int& m_blk, int& n_blk) {
    const int per_group = gm_full * num_n;
    const int g = t / per_group;
    const int first_m = g * gm_full;
    const int gm = min(gm_full, num_m - first_m);
    const int r = t - g * per_group;
    m_blk = first_m + r % gm;
    n_blk = r / gm;
  };

  if (warp == 0) {
    // ---------------- producer (both CTAs): own A rows, own half of the weight rows ----------------
    if (lane == 0) {
      const uint64_t pol = l2_policy_evict_last();
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = first_tile; t < num_tiles && ok; t += tile_step) {
        int m_blk, n_blk;
        tile_coords(t, m_blk, n_blk);
        const int m0 = m_blk * TILE_ROWS + static_cast<int>(rank) * BLOCK_ROWS;
        const int n0 = n_blk * BN + static_cast<int>(rank) * BLOCK_ROWS;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag)) {
            report_failure(p.status, ST_TIMEOUT, abort_flag);
            ok = false;
            break;
          }
          const uint32_t fb_leader = mapa_u32(bar_full + 8 * stage, 0);
          if (rank == 0) mbar_expect_tx(bar_full + 8 * stage, 2 * (L::A_STAGE + L::B_STAGE));
          tma_load_2d_2sm(smem_base + L::OFF_A + stage * L::A_STAGE, &tmA, fb_leader, kb * KBLOCK_BYTES, m0, pol);
          tma_load_3d_2sm(smem_base + L::OFF_B + stage * L::B_STAGE, &tmW, fb_leader, 0, n0, kb, pol);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issue (leader only) ----------------
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = umma_idesc(KT::dfmt, KT::abfmt, TILE_ROWS, BN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = first_tile; t < num_tiles && ok; t += tile_step) {
        if (!mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1u, abort_flag)) {
          report_failure(p.status, ST_TIMEOUT, abort_flag);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag)) {
            report_failure(p.status, ST_TIMEOUT, abort_flag);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t adesc = umma_desc_sw128_kmajor(smem_base + L::OFF_A + stage * L::A_STAGE);
          const uint64_t bdesc = umma_desc_sw128_kmajor(smem_base + L::OFF_B + stage * L::B_STAGE);
#pragma unroll
          for (int k = 0; k < KBLOCK_BYTES / UMMA_K_BYTES; ++k) {
            umma_ss_2sm<KIND>(d_tmem, adesc + static_cast<uint64_t>(k * (UMMA_K_BYTES >> 4)),
                              bdesc + static_cast<uint64_t>(k * (UMMA_K_BYTES >> 4)), idesc, (kb | k) != 0 ? 1u : 0u);
          }
          // the stage is free in both CTAs once these MMAs have read it
          umma_commit_2sm(bar_empty + 8 * stage);
          umma_commit_2sm(mapa_u32(bar_empty + 8 * stage, 1));
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit_2sm(bar_tfull + 8 * acc);
        umma_commit_2sm(mapa_u32(bar_tfull + 8 * acc, 1));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
    __syncwarp();
  } else {
    // ---------------- epilogue (both CTAs): own 128 rows x 256 columns ----------------
    const int q = warp & 3;
    const int ew = warp - 2;
    const uint32_t stage_c = smem_base + L::OFF_C + ew * 2 * L::C_BUF;
    int acc = 0;
    uint32_t acc_phase = 0;
    int cbuf = 0;
    for (int t = first_tile; t < num_tiles; t += tile_step) {
      int m_blk, n_blk;
      tile_coords(t, m_blk, n_blk);
      const int m0 = m_blk * TILE_ROWS + static_cast<int>(rank) * BLOCK_ROWS + q * 32;
      const int n0 = n_blk * BN;
      if (!mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag)) {
        if (lane == 0) report_failure(p.status, ST_TIMEOUT, abort_flag);
        break;
      }
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * BN);
      const uint32_t tempty_leader = mapa_u32(bar_tempty + 8 * acc, 0);
      epilogue_warp_tile<KIND, OUTMODE>(p, &tmC, 1, 0, t_row, m0, n0, BN, lane, stage_c, cbuf, [&]() {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(tempty_leader);
      });
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
    if (lane == 0) bulk_wait_group<0>();
    __syncwarp();
  }

  // Nobody leaves while the peer may still signal one of its barriers or the
  // leader's MMAs may still read its shared memory.  All waits above are
  // bounded, so every thread of both CTAs arrives here.
  tc_fence_before();
  cluster_barrier_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_2sm(tmem_base, TMEM_COLS);
  }
}

}  // namespace flyb200
