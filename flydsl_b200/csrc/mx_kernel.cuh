// MXFP8 GEMM: E4M3 codes with one E8M0 (power-of-two) scale per 32 elements
// of K on BOTH operands, multiplied with the block-scaled tensor-core
// instruction
//
//   tcgen05.mma.kind::mxf8f6f4.block_scale   D[tmem] (+)= (A . sfA) x (B . sfB)^T
//
// which reads the scale factors from tensor memory.  c[M, N] = bf16/fp16 of
// sum_k a[m, k] 2^(sa[m, k/32] - 127) w[n, k] 2^(sw[n, k/32] - 127).
//
// Data layout.  Codes: activations row-major [M, K]; weights in the same
// preshuffled image as the per-channel-scaled GEMM ([K/128][N][128 B swizzled]).
// Scales: "scale image" [K/128][rows/128][512 B]: one 512-byte atom per 128 rows
// and 128-element k-block, byte (r % 32) * 16 + (r / 32) * 4 + j = scale of row r
// of the tile for the j-th 32-element block.  An atom is what one
// tcgen05.cp.32x128b.warpx4 moves from shared memory into four TMEM columns
// (lane r % 32 of every 32-lane quarter, column r / 32, byte j), the arrangement
// the instruction expects; j is selected per instruction by the scale-factor id
// fields of the instruction descriptor.
//
// Kernel: persistent, tokens on the UMMA M side (128 per tile), BN output
// channels on the N side, a ring of {A tile, W tile, scale atom of A, scale
// atoms of W}, a rotating set of TMEM columns for the scale atoms of the stages
// in flight.  Two shapes: BN = 128 with two TMEM accumulators (the epilogue of
// tile i overlaps the mainloop of tile i + 1; 6 stages), and BN = 256 with one
// accumulator (the wider MMA needs fewer operand bytes per flop, but 2 x 256
// accumulator columns plus scale columns exceed the 512 columns of TMEM, so the
// epilogue is exposed; 4 stages) for long K, where the epilogue is a small part
// of a tile.  Threads as in the large-M kernel: warp 0 producer, warp 1 MMA
// (copies the two scale atoms to TMEM, then issues the four MMAs of a k-block),
// warps 2..5 epilogue (thread = token row, 64 contiguous output bytes per chunk).
#pragma once
#include "moe_kernel.cuh"

namespace flyb200 {


struct MxParams {
  const uint8_t* w;    // weight codes, preshuffled image
  const uint8_t* sfa;  // scale image of the activations, [K/128][ceil(M/128)][512]
  const uint8_t* sfw;  // scale image of the weights, [K/128][N/128][512]
  void* c;
  int M, N, K_bytes;
  int group_m;
  uint32_t fmt_bits;   // operand formats of kind::mxf8f6f4 as instruction-descriptor bits: (A format << 7) | (B format << 10)
  int* status;
};

// FP4: the codes are E2M1, two per byte.  A 128-byte k-block then holds 256
// elements = eight scale blocks per row: two scale atoms per 128 rows instead of
// one (atom h covers elements [128 h, 128 h + 128) of the k-block), everything
// else - operand tiles, ring, swizzle - is the same bytes as for 8-bit codes.
template <int BN, bool FP4 = false>
struct MxSmem {
  static constexpr int STAGES = BN == 128 ? 6 : 4;
  static constexpr int NACC = BN == 128 ? 2 : 1;          // TMEM accumulators
  static constexpr int HALVES = FP4 ? 2 : 1;              // scale atoms per 128 rows and k-block
  static constexpr int SFB_ATOMS = BN / 128;
  static constexpr int A_STAGE = BLOCK_ROWS * KBLOCK_BYTES;
  static constexpr int B_STAGE = BN * KBLOCK_BYTES;
  static constexpr int SFA_STAGE = HALVES * MX_SF_ATOM;
  static constexpr int SFB_HALF = SFB_ATOMS * MX_SF_ATOM;
  static constexpr int SFB_STAGE = HALVES * SFB_HALF;
  static constexpr int OFF_A = 0;
  static constexpr int OFF_B = OFF_A + STAGES * A_STAGE;
  static constexpr int OFF_SFA = OFF_B + STAGES * B_STAGE;
  static constexpr int OFF_SFB = OFF_SFA + STAGES * SFA_STAGE;
  static constexpr int OFF_BAR = OFF_SFB + STAGES * SFB_STAGE;  // full[S], empty[S], tfull[2], tempty[2]
  static constexpr int OFF_MISC = OFF_BAR + 8 * (2 * STAGES + 4);
  static constexpr int TOTAL = OFF_MISC + 16;
};

template <int OUTMODE, int BN, bool FP4 = false>
__global__ void __launch_bounds__(NUM_THREADS, 1) mx_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const MxParams p) {
  using L = MxSmem<BN, FP4>;
  constexpr int STAGES = L::STAGES;
  constexpr int NACC = L::NACC;
  constexpr int HALVES = L::HALVES;
  // TMEM columns of the scale atoms of one stage: per half, 4 for A then 4 per 128 channels for W
  constexpr int SFA_COLS = 4 * HALVES;
  constexpr int SF_COLS = SFA_COLS + 4 * L::SFB_ATOMS * HALVES;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t smem_base = smem_u32(smem_raw);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_raw + L::OFF_MISC + 4);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_raw + L::OFF_MISC);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t bar_full = smem_base + L::OFF_BAR;
  const uint32_t bar_empty = bar_full + 8 * STAGES;
  const uint32_t bar_tfull = bar_empty + 8 * STAGES;
  const uint32_t bar_tempty = bar_tfull + 16;

  if ((smem_base & 1023u) != 0) {
    if (threadIdx.x == 0) atomicCAS(p.status, 0, ST_SMEM_ALIGN);
    return;
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_tfull + 8 * s, 1);
      mbar_init(bar_tempty + 8 * s, 4);
    }
    abort_flag[0] = 0;
    abort_flag[1] = 0;
    fence_mbar_init();
    prefetch_tensormap(&tmA);
  }
  // TMEM: columns [0, 256) the accumulator(s), then per stage in flight the scale
  // atoms (4 columns for A, 4 per 128 channels for W)
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t SF_COL0 = NACC * BN;
  static_assert(SF_COL0 + STAGES * SF_COLS <= TMEM_COLS, "accumulators and scale columns must fit TMEM");
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int num_m = (p.M + BLOCK_ROWS - 1) / BLOCK_ROWS;
  const int num_n = p.N / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = p.K_bytes / KBLOCK_BYTES;
  auto tile_coords = [&](int t, int& m_blk, int& n_blk) {
    const int per_group = p.group_m * num_n;
    const int g = t / per_group;
    const int first_m = g * p.group_m;
    const int gm = min(p.group_m, num_m - first_m);
    const int r = t - g * per_group;
    m_blk = first_m + r % gm;
    n_blk = r / gm;
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
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag)) {
            report_failure(p.status, ST_TIMEOUT, abort_flag);
            ok = false;
            break;
          }
          const uint32_t fb = bar_full + 8 * stage;
          mbar_expect_tx(fb, L::A_STAGE + L::B_STAGE + L::SFA_STAGE + L::SFB_STAGE);
          tma_load_2d(smem_base + L::OFF_A + stage * L::A_STAGE, &tmA, fb, kb * KBLOCK_BYTES, m_blk * BLOCK_ROWS, pol);
          bulk_load_1d(smem_base + L::OFF_B + stage * L::B_STAGE,
                       p.w + (static_cast<size_t>(kb) * p.N + n_blk * BN) * KBLOCK_BYTES, L::B_STAGE, fb, pol);
          // the scale images are indexed by 128-ELEMENT k-blocks: HALVES of them per 128-byte k-block
#pragma unroll
          for (int h = 0; h < HALVES; ++h) {
            const size_t ekb = static_cast<size_t>(kb) * HALVES + h;
            bulk_load_1d(smem_base + L::OFF_SFA + stage * L::SFA_STAGE + h * MX_SF_ATOM,
                         p.sfa + (ekb * num_m + m_blk) * MX_SF_ATOM, MX_SF_ATOM, fb, pol);
            bulk_load_1d(smem_base + L::OFF_SFB + stage * L::SFB_STAGE + h * L::SFB_HALF,
                         p.sfw + (ekb * (p.N / 128) + n_blk * L::SFB_ATOMS) * MX_SF_ATOM, L::SFB_HALF, fb, pol);
          }
          ++issued;
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok || *abort_flag) {
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
      // 8-bit containers: E4M3 unless the caller names other formats (E2M3 / E2M1 codes padded to a byte)
      const uint32_t idesc = FP4 ? umma_idesc_mxf4(BLOCK_ROWS, BN) : (umma_idesc_mxf8(BLOCK_ROWS, BN) | p.fmt_bits);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
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
          // scale atoms of this stage: shared memory -> their TMEM columns
          const uint32_t sfa_t = tmem_base + SF_COL0 + static_cast<uint32_t>(stage * SF_COLS);
          const uint32_t sfb_t = sfa_t + SFA_COLS;
#pragma unroll
          for (int h = 0; h < HALVES; ++h) {
            tmem_cp_sf(sfa_t + 4 * h, sf_smem_desc(smem_base + L::OFF_SFA + stage * L::SFA_STAGE + h * MX_SF_ATOM));
#pragma unroll
            for (int at = 0; at < L::SFB_ATOMS; ++at)
              tmem_cp_sf(sfb_t + 4 * (h * L::SFB_ATOMS + at),
                         sf_smem_desc(smem_base + L::OFF_SFB + stage * L::SFB_STAGE + h * L::SFB_HALF + at * MX_SF_ATOM));
          }
          const uint64_t adesc = umma_desc_sw128_kmajor(smem_base + L::OFF_A + stage * L::A_STAGE);
          const uint64_t bdesc = umma_desc_sw128_kmajor(smem_base + L::OFF_B + stage * L::B_STAGE);
#pragma unroll
          for (int k = 0; k < KBLOCK_BYTES / UMMA_K_BYTES; ++k) {
            if constexpr (FP4) {
              // 32 bytes = 64 elements = scale blocks 2k and 2k+1 of the k-block: atom k/2, bytes 2(k%2) and 2(k%2)+1
              const uint32_t sf_id = static_cast<uint32_t>((k & 1) * 2);
              const uint32_t id = idesc | (sf_id << 4) | (sf_id << 29);
              umma_mxf4(d_tmem, adesc + static_cast<uint64_t>(k * (UMMA_K_BYTES >> 4)),
                        bdesc + static_cast<uint64_t>(k * (UMMA_K_BYTES >> 4)), id, sfa_t + 4 * (k >> 1),
                        sfb_t + 4 * L::SFB_ATOMS * (k >> 1), (kb | k) != 0 ? 1u : 0u);
            } else {
              // the k-th 32-element block uses byte k of the scale columns: scale-factor id k for both operands
              const uint32_t id = idesc | (static_cast<uint32_t>(k) << 4) | (static_cast<uint32_t>(k) << 29);
              umma_mxf8(d_tmem, adesc + static_cast<uint64_t>(k * (UMMA_K_BYTES >> 4)),
                        bdesc + static_cast<uint64_t>(k * (UMMA_K_BYTES >> 4)), id, sfa_t, sfb_t, (kb | k) != 0 ? 1u : 0u);
            }
          }
          umma_commit(bar_empty + 8 * stage);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit(bar_tfull + 8 * acc);
        acc = (acc + 1) % NACC;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    // ------------------------------ epilogue ------------------------------
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      int m_blk, n_blk;
      tile_coords(t, m_blk, n_blk);
      const int row = m_blk * BLOCK_ROWS + q * 32 + lane;
      if (!mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag)) {
        if (lane == 0) report_failure(p.status, ST_TIMEOUT, abort_flag);
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * BN);
      // 64 columns per TMEM wait, and each lane then writes one full 128-byte line of its output row
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 64) {
        uint32_t r0[32], r1[32];
        tmem_ld_x32(t_row + c0, r0);
        tmem_ld_x32(t_row + c0 + 32, r1);
        tmem_ld_wait();
        if (c0 + 64 >= BN) {  // last read of this accumulator: hand it back to the MMA warp
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_tempty + 8 * acc);
        }
        if (row < p.M) {
          float y[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) y[j] = __uint_as_float(r0[j]);
          moe_store_row32<OUTMODE, false>(p.c, static_cast<size_t>(row) * p.N + n_blk * BN + c0, y, 32);
#pragma unroll
          for (int j = 0; j < 32; ++j) y[j] = __uint_as_float(r1[j]);
          moe_store_row32<OUTMODE, false>(p.c, static_cast<size_t>(row) * p.N + n_blk * BN + c0 + 32, y, 32);
        }
      }
      acc = (acc + 1) % NACC;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// Scale image from row-major scales [rows, K/32] (uint8): see the layout above.
// One thread per byte of the image; rows past `rows` read as zero.
static __global__ void mx_scale_image_kernel(uint8_t* __restrict__ dst, const uint8_t* __restrict__ src, int rows, int kb32,
                                      int row_tiles) {
  const long long total = static_cast<long long>(kb32 / 4) * row_tiles * MX_SF_ATOM;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int in_atom = static_cast<int>(i % MX_SF_ATOM);
    const long long atom = i / MX_SF_ATOM;
    const int tile = static_cast<int>(atom % row_tiles);
    const int kblk = static_cast<int>(atom / row_tiles);
    const int r = tile * 128 + (in_atom >> 4) + 32 * ((in_atom >> 2) & 3);
    const int j = in_atom & 3;
    dst[i] = r < rows ? __ldg(src + static_cast<size_t>(r) * kb32 + kblk * 4 + j) : 0;
  }
}

}  // namespace flyb200
