// Large-M kernel, tall form: one CTA owns a 256 x bn output tile (bn <= 256)
// and drives it as two 128-row halves, each with its own TMEM accumulator, that
// share the weight tile of every k-block.  Per k-block and SM that is 32 KiB of
// activations + up to 32 KiB of weights for twice the flops of a 128 x 256 tile
// (48 KiB): a third fewer bytes into the SM per flop, which is what bounds the
// 128-row form at full clocks.  Unlike the CTA-pair form (rows2_kernel.cuh) the
// MMAs stay tcgen05.mma.cta_group::1, which one thread issues three times as
// fast.  The price: both accumulators (2 x 256 columns = all of TMEM) belong to
// the tile in flight, so the epilogue does not overlap the next tile's
// mainloop; eight epilogue warps (one set of four per half) keep it short, and
// the ring is three stages of up to 64 KiB.
#pragma once
#include "gemm_kernels.cuh"

namespace flyb200 {

constexpr int TALL_ROWS = 2 * BLOCK_ROWS;
constexpr int TALL_THREADS = 320;  // warp 0 producer, warp 1 MMA issue, warps 2..9 epilogue
constexpr int TALL_STAGES = 3;

struct TallLayout {
  int a_stage, b_stage, off_b, off_c, off_bar, off_misc, total;
};
__host__ __device__ inline TallLayout rows_tall_layout(int bn, int stages) {
  TallLayout l;
  l.a_stage = TALL_ROWS * KBLOCK_BYTES;
  l.b_stage = bn * KBLOCK_BYTES;
  l.off_b = stages * l.a_stage;
  l.off_c = l.off_b + stages * l.b_stage;  // 8 warps x 1 staging buffer
  l.off_bar = l.off_c + 8 * ROWS_C_BUF;    // full[S], empty[S], tfull, tempty
  l.off_misc = l.off_bar + 8 * (2 * stages + 2);
  l.total = l.off_misc + 16;
  return l;
}

template <int KIND, int OUTMODE>
__global__ void __launch_bounds__(TALL_THREADS, 1)
gemm_rows_tall_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmC,
                      const GemmParams p) {
  using KT = KindTraits<KIND>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t smem_base = smem_u32(smem_raw);
  const int BN = p.bn;
  const int STAGES = p.rows_stages;
  const TallLayout L = rows_tall_layout(BN, STAGES);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_raw + L.off_misc + 4);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_raw + L.off_misc);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t bar_full = smem_base + L.off_bar;
  const uint32_t bar_empty = bar_full + 8 * STAGES;
  const uint32_t bar_tfull = bar_empty + 8 * STAGES;
  const uint32_t bar_tempty = bar_tfull + 8;

  if ((smem_base & 1023u) != 0) {  // uniform over the CTA: the swizzle atoms need 1024-byte alignment
    if (threadIdx.x == 0) atomicCAS(p.status, 0, ST_SMEM_ALIGN);
    return;
  }
  // programmatic dependent launch: set-up below overlaps the previous kernel's tail; no global access before the wait
  if (p.pdl) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    mbar_init(bar_tfull, 1);
    mbar_init(bar_tempty, 8);  // every epilogue warp, once its half of the accumulators is read
    abort_flag[0] = 0;
    abort_flag[1] = 0;  // stays zero: lets the drain below wait on time alone
    fence_mbar_init();
    prefetch_tensormap(&tmA);
    if (OUTMODE != OUT_RAW32) prefetch_tensormap(&tmC);
  }
  constexpr uint32_t TMEM_COLS = 512;  // two halves x up to 256 columns
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (p.pdl) asm volatile("griddepcontrol.wait;" ::: "memory");  // the previous kernel has completed

  const int num_m = (p.M + TALL_ROWS - 1) / TALL_ROWS;
  const int num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = p.K_bytes / KBLOCK_BYTES;
  const int gm_full = p.group_m;  // in 256-row tiles

  // groups of row tiles; the row tile changes fastest, every second group walks the channels backwards
  auto tile_coords = [&](int t, int& m_blk, int& n_blk) {
    const int per_group = gm_full * num_n;
    const int g = t / per_group;
    const int first_m = g * gm_full;
    const int gm = min(gm_full, num_m - first_m);
    const int r = t - g * per_group;
    m_blk = first_m + r % gm;
    n_blk = r / gm;
    if (g & 1) n_blk = num_n - 1 - n_blk;
  };

  if (warp == 0) {
    // ------------------------------ producer ------------------------------
    if (lane == 0) {
      const uint64_t pol = l2_policy_evict_last();
      int stage = 0;
      uint32_t phase = 0;
      int issued = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int m_blk, n_blk;
        tile_coords(t, m_blk, n_blk);
        const int n0 = n_blk * BN;
        const uint32_t w_bytes = static_cast<uint32_t>(min(BN, p.N - n0)) * KBLOCK_BYTES;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag)) {
            report_failure(p.status, ST_TIMEOUT, abort_flag);
            ok = false;
            break;
          }
          const uint32_t fb = bar_full + 8 * stage;
          mbar_expect_tx(fb, L.a_stage + w_bytes);
          // 256 rows of activations as one box (rows past M arrive as zeros), then the weight block
          tma_load_2d(smem_base + stage * L.a_stage, &tmA, fb, kb * KBLOCK_BYTES, m_blk * TALL_ROWS, pol);
          bulk_load_1d(smem_base + L.off_b + stage * L.b_stage, p.w + (static_cast<size_t>(kb) * p.N + n0) * KBLOCK_BYTES,
                       w_bytes, fb, pol);
          ++issued;
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok || *abort_flag) {
        // wait (bounded) for copies still in flight so none lands after the CTA is gone
        const int pending = min(issued, STAGES);
        for (int i = 0; i < pending; ++i) {
          int s = stage - 1 - i;
          uint32_t ph = phase;
          if (s < 0) {
            s += STAGES;
            ph ^= 1u;
          }
          mbar_wait(bar_full + 8 * s, ph, abort_flag + 1);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issue -----------------------------
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(KT::dfmt, KT::abfmt, BLOCK_ROWS, static_cast<uint32_t>(BN));
      int stage = 0;
      uint32_t phase = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        // both accumulators have been read by the epilogue of the previous tile
        if (!mbar_wait(bar_tempty, acc_phase ^ 1u, abort_flag)) {
          report_failure(p.status, ST_TIMEOUT, abort_flag);
          break;
        }
        tc_fence_after();
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag)) {
            report_failure(p.status, ST_TIMEOUT, abort_flag);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t bdesc = umma_desc_sw128_kmajor(smem_base + L.off_b + stage * L.b_stage);
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint64_t adesc = umma_desc_sw128_kmajor(smem_base + stage * L.a_stage + h * BLOCK_ROWS * KBLOCK_BYTES);
            const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(h * ROWS_ACC_COLS);
#pragma unroll
            for (int k = 0; k < KBLOCK_BYTES / UMMA_K_BYTES; ++k) {
              umma_ss<KIND>(d_tmem, adesc + static_cast<uint64_t>(k * (UMMA_K_BYTES >> 4)),
                            bdesc + static_cast<uint64_t>(k * (UMMA_K_BYTES >> 4)), idesc, (kb | k) != 0 ? 1u : 0u);
            }
          }
          umma_commit(bar_empty + 8 * stage);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit(bar_tfull);
        acc_phase ^= 1u;
      }
    }
  } else {
    // ------------------------------ epilogue ------------------------------
    const int q = warp & 3;         // TMEM lane quadrant this warp may read
    const int ew = warp - 2;        // 0..7: staging buffer owner
    const int half = ew >> 2;       // which 128-row half of the tile
    const uint32_t stage_c = smem_base + L.off_c + ew * ROWS_C_BUF;
    uint32_t acc_phase = 0;
    int cbuf = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      int m_blk, n_blk;
      tile_coords(t, m_blk, n_blk);
      const int m0 = m_blk * TALL_ROWS + half * BLOCK_ROWS + q * 32;
      const int n0 = n_blk * BN;
      if (!mbar_wait(bar_tfull, acc_phase, abort_flag)) {
        if (lane == 0) report_failure(p.status, ST_TIMEOUT, abort_flag);
        break;
      }
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(half * ROWS_ACC_COLS);
      epilogue_warp_tile<KIND, OUTMODE, 1>(p, &tmC, 1, 0, t_row, m0, n0, BN, lane, stage_c, cbuf, [&]() {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_tempty);
      });
      acc_phase ^= 1u;
    }
    if (lane == 0) bulk_wait_group<0>();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace flyb200
