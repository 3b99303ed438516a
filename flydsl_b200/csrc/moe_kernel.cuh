// Grouped (mixture-of-experts) A8W8 GEMMs on the preshuffled weight image.
//
// The routing step has sorted the (token, top-k slot) pairs by expert and padded
// every expert's list to a multiple of tile_m, so that "routing block" b (rows
// [b * tile_m, (b + 1) * tile_m) of the sorted list) belongs to one expert,
// expert_ids[b].  Both stages run the same kernel:
//
//   stage 1 (gate-up):  out[token, slot, n] = silu(g) * u  with
//                       g = x . Wgate[e, n, :], u = x . Wup[e, n, :]
//   stage 2 (down):     out[token, :] (+)= (a2[token, slot, :] . W2[e, :, :]^T) * routed weight
//
// Layout of one CTA: a routing block on the UMMA N side (BN >= tile_m token
// rows, read with one TMA box from the activation rows gathered into sorted
// order), two 128-channel weight tiles of the block's expert on the UMMA M side
// (stage 1: the gate tile and the matching up tile; stage 2: two neighbouring
// tiles), each tile with its own MMA-issuing warp and its own TMEM accumulator.
// Every expert has its own weight image [K/128][rows_per_expert][128 B], one
// after the other, so a tile of any expert is one contiguous 16 KiB burst per
// k-block.
//
// Threads: warp 0 producer (TMA), warp 1 MMA issuer of tile A, warps 2..5
// epilogue, warp 6 MMA issuer of tile B.  Every wait is bounded.
#pragma once
#include "gemm_kernels.cuh"
#include <type_traits>

namespace flyb200 {

enum : int { MOE_OUT_BF16 = 0, MOE_OUT_FP16 = 1, MOE_OUT_F32 = 2 };
constexpr int MOE_THREADS = 224;

struct MoeParams {
  const uint8_t* w;        // weight images, one per expert, back to back
  const float* sa;         // [P] activation scale per sorted row (0 on padding rows)
  const float* sw;         // [experts * n_expert] weight scale per channel
  const int* sorted_ids;   // [P] (slot << 24) | token; padding rows hold token >= tokens
  const int* expert_ids;   // [blocks] expert of each routing block
  const float* sorted_w;   // [P] routed weight per sorted row
  const int* num_valid;    // [1] rows of the sorted list in use (a multiple of tile_m)
  void* out;
  int tokens, topk, experts;
  int n_expert;            // weight rows per expert (stage 1: 2 * inter_dim, stage 2: model_dim)
  int n_out;               // length of an output row (stage 1: inter_dim, stage 2: model_dim)
  int K_bytes;
  int tile_m;              // routing block size (<= BN)
  int stages;              // ring depth
  int doweight;            // multiply by the routed weight in this stage
  int pdl;                 // launched as a programmatic dependent of the gather pass that writes a_sorted and sa
  int* status;
};

struct MoeLayout {
  int off_w, off_a, off_bar, off_misc, off_row, off_sa, off_tw, total;
};
__host__ __device__ inline MoeLayout moe_layout(int bn, int stages) {
  MoeLayout l;
  l.off_w = 0;  // per stage: tile A (16 KiB), tile B (16 KiB)
  l.off_a = stages * 2 * BLOCK_ROWS * KBLOCK_BYTES;
  l.off_bar = l.off_a + stages * bn * KBLOCK_BYTES;
  l.off_misc = (l.off_bar + 8 * (2 * stages + 1) + 15) & ~15;
  l.off_row = l.off_misc + 32;
  l.off_sa = l.off_row + bn * 4;
  l.off_tw = l.off_sa + bn * 4;
  l.total = l.off_tw + bn * 4;
  return l;
}

// x * sigmoid(x), with the fast exponential and reciprocal as in the reference's
// epilogue (exp2 and rcp, kernels/moe/moe_gemm_2stage/layout_helpers.py:247-248)
__device__ __forceinline__ float silu_f32(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

// Two neighbouring channels (lo at `col`, hi at `col + 1`) of one output row.
template <int OUTMODE, bool ACCUM>
__device__ __forceinline__ void moe_store_pair(void* out, size_t elem, float lo, float hi) {
  if constexpr (OUTMODE == MOE_OUT_BF16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    __nv_bfloat162* dst = reinterpret_cast<__nv_bfloat162*>(static_cast<__nv_bfloat16*>(out) + elem);
    if constexpr (ACCUM) {
      atomicAdd(dst, v);
    } else {
      *dst = v;
    }
  } else if constexpr (OUTMODE == MOE_OUT_FP16) {
    __half2 v = __floats2half2_rn(lo, hi);
    __half2* dst = reinterpret_cast<__half2*>(static_cast<__half*>(out) + elem);
    if constexpr (ACCUM) {
      atomicAdd(dst, v);
    } else {
      *dst = v;
    }
  } else {
    float* dst = static_cast<float*>(out) + elem;
    if constexpr (ACCUM) {
      atomicAdd(dst, lo);
      atomicAdd(dst + 1, hi);
    } else {
      *reinterpret_cast<float2*>(dst) = make_float2(lo, hi);
    }
  }
}

// Sixteen tokens (registers) of one channel (this lane) -> memory.  Neighbouring
// lanes swap every other token so that a lane holds two neighbouring channels of
// one token and writes them as one packed element: even lanes take the even
// tokens of the pair of channels, odd lanes the odd tokens.
// `ch`: this lane's channel inside the tile; `n_valid`: channels of the tile that exist (even).
template <int OUTMODE, bool ACCUM>
__device__ __forceinline__ void moe_emit16(void* out, const float (&v)[16], const int* row_s, int c0, int tile_m, int ch,
                                           int n_valid, int col0, int n_out) {
  const bool odd = (ch & 1) != 0;
  const int col = col0 + (ch & ~1);
#pragma unroll
  for (int j = 0; j < 16; j += 2) {
    const float send = odd ? v[j] : v[j + 1];
    const float recv = __shfl_xor_sync(0xffffffffu, send, 1);
    const int t = c0 + j + (odd ? 1 : 0);
    const float lo = odd ? recv : v[j];
    const float hi = odd ? v[j + 1] : recv;
    if (t < tile_m && ch < n_valid) {
      const int row = row_s[t];
      if (row >= 0) moe_store_pair<OUTMODE, ACCUM>(out, static_cast<size_t>(row) * n_out + col, lo, hi);
    }
  }
}

// STAGE 1: gate-up with silu; STAGE 2: down projection.
template <int KIND, int BN, int STAGE, int OUTMODE, bool ACCUM>
__global__ void __launch_bounds__(MOE_THREADS) moe_gemm_kernel(const __grid_constant__ CUtensorMap tmA,
                                                            const MoeParams p) {
  static_assert(STAGE == 1 || STAGE == 2, "two stages");
  static_assert(STAGE == 2 || !ACCUM, "only the down projection accumulates");
  using KT = KindTraits<KIND>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t smem_base = smem_u32(smem_raw);
  const int stages = p.stages;
  const MoeLayout L = moe_layout(BN, stages);
  constexpr int W_TILE = BLOCK_ROWS * KBLOCK_BYTES;
  constexpr int W_STAGE = 2 * W_TILE;
  constexpr int A_STAGE = BN * KBLOCK_BYTES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_raw + L.off_misc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_raw + L.off_misc + 4);
  int* row_s = reinterpret_cast<int*>(smem_raw + L.off_row);
  float* sa_s = reinterpret_cast<float*>(smem_raw + L.off_sa);
  float* tw_s = reinterpret_cast<float*>(smem_raw + L.off_tw);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t bar_full = smem_base + L.off_bar;
  const uint32_t bar_empty = bar_full + 8 * stages;
  const uint32_t bar_tfull = bar_empty + 8 * stages;

  // Blocks past the end of the sorted list, and blocks without an expert, have no work.
  const int blk = blockIdx.x;
  const int row0 = blk * p.tile_m;  // first sorted row of the block
  if (row0 >= __ldg(p.num_valid)) return;
  const int expert = __ldg(p.expert_ids + blk);
  if (expert < 0 || expert >= p.experts) return;
  if ((smem_base & 1023u) != 0) {
    if (threadIdx.x == 0) atomicCAS(p.status, 0, ST_SMEM_ALIGN);
    return;
  }

  // The two weight tiles of this CTA: first row in the expert's image, channels that exist, output column.
  int w_row[2], n_valid[2], col0[2];
  if constexpr (STAGE == 1) {
    const int inter = p.n_out;
    const int c = blockIdx.y * BLOCK_ROWS;
    w_row[0] = c;
    w_row[1] = inter + c;
    n_valid[0] = n_valid[1] = min(BLOCK_ROWS, inter - c);
    col0[0] = col0[1] = c;
  } else {
    const int c = blockIdx.y * 2 * BLOCK_ROWS;
    w_row[0] = c;
    w_row[1] = c + BLOCK_ROWS;
    n_valid[0] = min(BLOCK_ROWS, p.n_out - c);
    n_valid[1] = max(0, min(BLOCK_ROWS, p.n_out - c - BLOCK_ROWS));
    col0[0] = c;
    col0[1] = c + BLOCK_ROWS;
  }
  const bool has_b = n_valid[1] > 0;
  const int num_kb = p.K_bytes / KBLOCK_BYTES;
  const uint8_t* w_expert = p.w + static_cast<size_t>(expert) * p.n_expert * p.K_bytes;
  const float* sw_expert = p.sw + static_cast<size_t>(expert) * p.n_expert;
  const uint32_t w_bytes0 = static_cast<uint32_t>(n_valid[0]) * KBLOCK_BYTES;
  const uint32_t w_bytes1 = static_cast<uint32_t>(n_valid[1]) * KBLOCK_BYTES;
  bool ok = true;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, has_b ? 2 : 1);  // one commit per issuer
    }
    mbar_init(bar_tfull, has_b ? 2 : 1);
    abort_flag[0] = 0;
    abort_flag[1] = 0;  // stays zero: lets the drain below wait on time alone
    fence_mbar_init();
    prefetch_tensormap(&tmA);
  }
  constexpr uint32_t TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ producer ------------------------------
    if (lane == 0) {
      const uint64_t pol_a = l2_policy_evict_last();
      const uint64_t pol_w = l2_policy_evict_normal();  // other blocks of the same expert read the same tiles
      int stage = 0;
      uint32_t phase = 0;
      int issued = 0;
      auto load_weights = [&](int kb, int st, uint32_t fb) {
        mbar_expect_tx(fb, A_STAGE + w_bytes0 + w_bytes1);
        const uint32_t wdst = smem_base + L.off_w + st * W_STAGE;
        bulk_load_1d(wdst, w_expert + (static_cast<size_t>(kb) * p.n_expert + w_row[0]) * KBLOCK_BYTES, w_bytes0, fb,
                     pol_w);
        if (has_b)
          bulk_load_1d(wdst + W_TILE, w_expert + (static_cast<size_t>(kb) * p.n_expert + w_row[1]) * KBLOCK_BYTES,
                       w_bytes1, fb, pol_w);
      };
      // As a programmatic dependent of the gather pass the kernel may run before
      // the gathered activations exist.  The weights are model state: the ring is
      // filled with them first; everything the gather pass writes is touched only
      // after griddepcontrol.wait.
      const int pre = p.pdl ? min(stages, num_kb) : 0;
      for (int i = 0; i < pre; ++i) load_weights(i, i, bar_full + 8 * i);
      if (p.pdl) asm volatile("griddepcontrol.wait;" ::: "memory");
      for (int i = 0; i < pre; ++i)
        tma_load_2d(smem_base + L.off_a + i * A_STAGE, &tmA, bar_full + 8 * i, i * KBLOCK_BYTES, row0, pol_a);
      issued = pre;
      if (pre == stages) phase = 1u; else stage = pre;
      for (int kb = pre; kb < num_kb; ++kb) {
        if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag)) {
          report_failure(p.status, ST_TIMEOUT, abort_flag);
          ok = false;
          break;
        }
        const uint32_t fb = bar_full + 8 * stage;
        load_weights(kb, stage, fb);
        tma_load_2d(smem_base + L.off_a + stage * A_STAGE, &tmA, fb, kb * KBLOCK_BYTES, row0, pol_a);
        ++issued;
        if (++stage == stages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (!ok || *abort_flag) {
        // wait (bounded) for copies still in flight so none lands after the CTA is gone
        const int pending = min(issued, stages);
        for (int i = 0; i < pending; ++i) {
          int s = stage - 1 - i;
          uint32_t ph = phase;
          if (s < 0) {
            s += stages;
            ph ^= 1u;
          }
          mbar_wait(bar_full + 8 * s, ph, abort_flag + 1);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1 || warp == 6) {
    // ------------------------------ MMA issue -----------------------------
    const int which = warp == 1 ? 0 : 1;  // tile A / tile B
    if (lane == 0 && (which == 0 || has_b)) {
      constexpr uint32_t idesc = umma_idesc(KT::dfmt, KT::abfmt, BLOCK_ROWS, BN);
      const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(which * BN);
      int stage = 0;
      uint32_t phase = 0;
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag)) {
          report_failure(p.status, ST_TIMEOUT, abort_flag);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint64_t wdesc = umma_desc_sw128_kmajor(smem_base + L.off_w + stage * W_STAGE + which * W_TILE);
        const uint64_t adesc = umma_desc_sw128_kmajor(smem_base + L.off_a + stage * A_STAGE);
#pragma unroll
        for (int k = 0; k < KBLOCK_BYTES / UMMA_K_BYTES; ++k) {
          umma_ss<KIND>(d_tmem, wdesc + static_cast<uint64_t>(k * (UMMA_K_BYTES >> 4)),
                        adesc + static_cast<uint64_t>(k * (UMMA_K_BYTES >> 4)), idesc, (kb != 0 || k != 0) ? 1u : 0u);
        }
        umma_commit(bar_empty + 8 * stage);
        if (++stage == stages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (ok) umma_commit(bar_tfull);
    }
    __syncwarp();
  } else {
    // ------------------------------ epilogue -------------------------------
    // thread <-> channel (TMEM lane), registers <-> tokens of the block
    const int q = warp & 3;
    const int ch = q * 32 + lane;
    const int et = threadIdx.x - 64;
    const int n_rows = __ldg(p.num_valid);
    if (p.pdl) asm volatile("griddepcontrol.wait;" ::: "memory");  // p.sa is written by the gather pass
    for (int i = et; i < BN; i += 128) {
      int row = -1;
      float sa = 0.0f, tw = 1.0f;
      if (i < p.tile_m && row0 + i < n_rows) {
        const int id = __ldg(p.sorted_ids + row0 + i);
        const int tok = id & 0xFFFFFF;
        const int slot = static_cast<int>(static_cast<uint32_t>(id) >> 24);
        if (tok < p.tokens && slot < p.topk) {
          row = (STAGE == 2 && ACCUM) ? tok : tok * p.topk + slot;
          sa = __ldg(p.sa + row0 + i);
          if (p.doweight) tw = __ldg(p.sorted_w + row0 + i);
        }
      }
      row_s[i] = row;
      sa_s[i] = sa;
      tw_s[i] = tw;
    }
    const float sw0 = ch < n_valid[0] ? __ldg(sw_expert + w_row[0] + ch) : 0.0f;
    const float sw1 = ch < n_valid[1] ? __ldg(sw_expert + w_row[1] + ch) : 0.0f;
    named_bar_sync(1, 128);

    ok = mbar_wait(bar_tfull, 0, abort_flag);
    if (!ok && lane == 0) report_failure(p.status, ST_TIMEOUT, abort_flag);
    ok = named_bar_and(1, 128, ok);
    if (ok) {
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 16) {
        if (c0 >= p.tile_m) break;
        uint32_t ra[16], rb[16];
        tmem_ld_x16(t_row + c0, ra);
        if (has_b) tmem_ld_x16(t_row + BN + c0, rb);
        tmem_ld_wait();
        float va[16], vb[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float sa = sa_s[c0 + j];
          const float a = KT::is_int ? static_cast<float>(static_cast<int32_t>(ra[j])) : __uint_as_float(ra[j]);
          const float b = !has_b ? 0.0f : KT::is_int ? static_cast<float>(static_cast<int32_t>(rb[j])) : __uint_as_float(rb[j]);
          // the reference's order: accumulator times weight scale, then times activation scale
          const float fa = (a * sw0) * sa;
          const float fb = (b * sw1) * sa;
          if constexpr (STAGE == 1) {
            float y = silu_f32(fa) * fb;
            if (p.doweight) y *= tw_s[c0 + j];
            va[j] = y;
          } else {
            const float tw = tw_s[c0 + j];
            va[j] = p.doweight ? fa * tw : fa;
            vb[j] = p.doweight ? fb * tw : fb;
          }
        }
        moe_emit16<OUTMODE, ACCUM>(p.out, va, row_s, c0, p.tile_m, ch, n_valid[0], col0[0], p.n_out);
        if constexpr (STAGE == 2) {
          if (has_b) moe_emit16<OUTMODE, ACCUM>(p.out, vb, row_s, c0, p.tile_m, ch, n_valid[1], col0[1], p.n_out);
        }
      }
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

// ---------------------------------------------------------------------------
// Large routing blocks (tile_m a multiple of 128, or 64): persistent form
// ---------------------------------------------------------------------------
// Tokens on the UMMA M side (128 sorted rows per work item), the two weight
// tiles side by side on the N side (256 channels: stage 1 gate | up, stage 2 two
// neighbouring tiles), one CTA per SM walking the (row block, channel pair)
// items, a shared-memory ring that keeps streaming across items and two TMEM
// accumulators so that the epilogue of an item overlaps the mainloop of the
// next.  A thread of the epilogue owns one token row: it reads the gate and up
// columns of the same channel from its own TMEM lane and writes 64 contiguous
// bytes of its output row per 32-channel chunk.
constexpr int MOE_ROWS_STAGES = 4;
constexpr int MOE_ROWS_BN = 2 * BLOCK_ROWS;
constexpr int MOE_ROWS_GROUP = 32;  // row blocks per rasterisation group (16 MiB of activations at K = 4096)

struct MoeRowsSmem {
  static constexpr int A_STAGE = BLOCK_ROWS * KBLOCK_BYTES;
  static constexpr int B_STAGE = MOE_ROWS_BN * KBLOCK_BYTES;
  static constexpr int OFF_A = 0;
  static constexpr int OFF_B = OFF_A + MOE_ROWS_STAGES * A_STAGE;
  static constexpr int OFF_SW = OFF_B + MOE_ROWS_STAGES * B_STAGE;   // 4 warps x 256 weight scales
  static constexpr int OFF_BAR = OFF_SW + 4 * MOE_ROWS_BN * 4;       // full[S], empty[S], tfull[2], tempty[2]
  static constexpr int OFF_MISC = OFF_BAR + 8 * (2 * MOE_ROWS_STAGES + 4);
  static constexpr int TOTAL = OFF_MISC + 16;
};

template <int OUTMODE, bool ACCUM>
__device__ __forceinline__ void moe_store_row32(void* out, size_t elem, const float (&y)[32], int n_ok) {
  // 32 consecutive channels of one output row; n_ok (a multiple of 16) of them exist
  if constexpr (!ACCUM && OUTMODE != MOE_OUT_F32) {
    uint32_t pk[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      if constexpr (OUTMODE == MOE_OUT_BF16) {
        __nv_bfloat162 h = __floats2bfloat162_rn(y[2 * i], y[2 * i + 1]);
        pk[i] = *reinterpret_cast<uint32_t*>(&h);
      } else {
        __half2 h = __floats2half2_rn(y[2 * i], y[2 * i + 1]);
        pk[i] = *reinterpret_cast<uint32_t*>(&h);
      }
    }
    uint4* dst = reinterpret_cast<uint4*>(static_cast<uint16_t*>(out) + elem);
#pragma unroll
    for (int v = 0; v < 4; ++v)
      if (8 * v < n_ok) dst[v] = make_uint4(pk[4 * v], pk[4 * v + 1], pk[4 * v + 2], pk[4 * v + 3]);
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i)
      if (2 * i < n_ok) moe_store_pair<OUTMODE, ACCUM>(out, elem + 2 * i, y[2 * i], y[2 * i + 1]);
  }
}

template <int KIND, int STAGE, int OUTMODE, bool ACCUM>
__global__ void __launch_bounds__(NUM_THREADS, 1) moe_rows_kernel(const __grid_constant__ CUtensorMap tmA,
                                                                  const MoeParams p) {
  static_assert(STAGE == 2 || !ACCUM, "only the down projection accumulates");
  using L = MoeRowsSmem;
  using KT = KindTraits<KIND>;
  constexpr int STAGES = MOE_ROWS_STAGES;
  constexpr int BN = MOE_ROWS_BN;
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
  constexpr uint32_t TMEM_COLS = 512;
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // Work items: (row block of 128 sorted rows, channel pair).  Row blocks run
  // fastest, so CTAs working side by side share the weight tiles of an expert,
  // and they are taken in groups of MOE_ROWS_GROUP whose activation rows stay in
  // L2 while the group walks all channel pairs.
  const int n_rows = __ldg(p.num_valid);
  const int row_blocks = (n_rows + BLOCK_ROWS - 1) / BLOCK_ROWS;
  const int pairs = STAGE == 1 ? (p.n_out + BLOCK_ROWS - 1) / BLOCK_ROWS : (p.n_out + BN - 1) / BN;
  // Routing blocks of 64 rows: a 128-row block holds two of them.  Where both have
  // the same expert they are one item; where the expert changes inside the 128
  // rows the block is worked on twice ("passes"), once per expert, each pass
  // storing only its own 64 rows.  That happens once per expert boundary.
  const int passes = p.tile_m == 64 ? 2 : 1;
  const int items = row_blocks * pairs * passes;
  const int num_kb = p.K_bytes / KBLOCK_BYTES;
  auto item_coords = [&](int t, int& rb, int& pair) {
    const int per_group = MOE_ROWS_GROUP * pairs;
    const int g = t / per_group;
    const int first = g * MOE_ROWS_GROUP;
    const int gm = min(MOE_ROWS_GROUP, row_blocks - first);
    const int r = t - g * per_group;
    rb = first + r % gm;
    pair = r / gm;
  };
  // expert of the routing block that starts at sorted row `row`, or -1 when there is none
  auto expert_at = [&](int row) {
    if (row >= n_rows) return -1;
    const int e = __ldg(p.expert_ids + row / p.tile_m);
    return (e < 0 || e >= p.experts) ? -1 : e;
  };
  // Item t -> row block, channel pair, expert (-1: nothing to do) and the rows [lo, hi) it stores.
  auto item_of = [&](int t, int& rb, int& pair, int& lo, int& hi) {
    // all first passes come before the (few) second passes, so that the CTAs share the real work evenly
    const int base = row_blocks * pairs;
    item_coords(t % base, rb, pair);
    lo = 0;
    hi = BLOCK_ROWS;
    if (passes == 1) return expert_at(rb * BLOCK_ROWS);
    const int ea = expert_at(rb * BLOCK_ROWS), eb = expert_at(rb * BLOCK_ROWS + 64);
    if (t < base) {
      if (eb != ea) hi = 64;
      return ea;
    }
    lo = 64;
    return eb == ea ? -1 : eb;
  };
  // rows of the image and channels that exist for the two tiles of a pair
  auto tiles_of = [&](int pair, int (&w_row)[2], int (&n_valid)[2]) {
    if constexpr (STAGE == 1) {
      const int c = pair * BLOCK_ROWS;
      w_row[0] = c;
      w_row[1] = p.n_out + c;
      n_valid[0] = n_valid[1] = min(BLOCK_ROWS, p.n_out - c);
    } else {
      const int c = pair * BN;
      w_row[0] = c;
      w_row[1] = c + BLOCK_ROWS;
      n_valid[0] = min(BLOCK_ROWS, p.n_out - c);
      n_valid[1] = max(0, min(BLOCK_ROWS, p.n_out - c - BLOCK_ROWS));
    }
  };

  if (warp == 0) {
    // ------------------------------ producer ------------------------------
    if (lane == 0) {
      const uint64_t pol = l2_policy_evict_last();
      int stage = 0;
      uint32_t phase = 0;
      int issued = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < items && ok; t += gridDim.x) {
        int rb, pair, lo, hi;
        const int expert = item_of(t, rb, pair, lo, hi);
        if (expert < 0) continue;
        int w_row[2], n_valid[2];
        tiles_of(pair, w_row, n_valid);
        const uint8_t* w_expert = p.w + static_cast<size_t>(expert) * p.n_expert * p.K_bytes;
        const uint32_t b0 = static_cast<uint32_t>(n_valid[0]) * KBLOCK_BYTES, b1 = static_cast<uint32_t>(n_valid[1]) * KBLOCK_BYTES;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag)) {
            report_failure(p.status, ST_TIMEOUT, abort_flag);
            ok = false;
            break;
          }
          const uint32_t fb = bar_full + 8 * stage;
          mbar_expect_tx(fb, L::A_STAGE + b0 + b1);
          tma_load_2d(smem_base + L::OFF_A + stage * L::A_STAGE, &tmA, fb, kb * KBLOCK_BYTES, rb * BLOCK_ROWS, pol);
          const uint32_t bdst = smem_base + L::OFF_B + stage * L::B_STAGE;
          bulk_load_1d(bdst, w_expert + (static_cast<size_t>(kb) * p.n_expert + w_row[0]) * KBLOCK_BYTES, b0, fb, pol);
          if (b1)
            bulk_load_1d(bdst + BLOCK_ROWS * KBLOCK_BYTES,
                         w_expert + (static_cast<size_t>(kb) * p.n_expert + w_row[1]) * KBLOCK_BYTES, b1, fb, pol);
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
      constexpr uint32_t idesc = umma_idesc(KT::dfmt, KT::abfmt, BLOCK_ROWS, BN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < items && ok; t += gridDim.x) {
        int rb, pair, lo, hi;
        if (item_of(t, rb, pair, lo, hi) < 0) continue;
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
            umma_ss<KIND>(d_tmem, adesc + static_cast<uint64_t>(k * (UMMA_K_BYTES >> 4)),
                          bdesc + static_cast<uint64_t>(k * (UMMA_K_BYTES >> 4)), idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(bar_empty + 8 * stage);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit(bar_tfull + 8 * acc);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    // ------------------------------ epilogue ------------------------------
    const int q = warp & 3;  // TMEM lane quadrant this warp may read
    float* sw_s = reinterpret_cast<float*>(smem_raw + L::OFF_SW) + (warp - 2) * BN;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < items && ok; t += gridDim.x) {
      int rb, pair, lo, hi;
      const int expert = item_of(t, rb, pair, lo, hi);
      if (expert < 0) continue;
      int w_row[2], n_valid[2];
      tiles_of(pair, w_row, n_valid);
      // this thread's token row
      const int trow = q * 32 + lane;
      const int srow = rb * BLOCK_ROWS + trow;
      long long orow = -1;
      float sa = 0.0f, tw = 1.0f;
      if (srow < n_rows && trow >= lo && trow < hi) {
        const int id = __ldg(p.sorted_ids + srow);
        const int tok = id & 0xFFFFFF;
        const int slot = static_cast<int>(static_cast<uint32_t>(id) >> 24);
        if (tok < p.tokens && slot < p.topk) {
          orow = (STAGE == 2 && ACCUM) ? tok : static_cast<long long>(tok) * p.topk + slot;
          sa = __ldg(p.sa + srow);
          if (p.doweight) tw = __ldg(p.sorted_w + srow);
        }
      }
      // weight scales of the 256 columns, one copy per warp
      const float* sw_expert = p.sw + static_cast<size_t>(expert) * p.n_expert;
      __syncwarp();
#pragma unroll
      for (int i = 0; i < BN / 32; ++i) {
        const int c = i * 32 + lane;
        const int h = c >> 7, cc = c & 127;
        sw_s[c] = cc < n_valid[h] ? __ldg(sw_expert + w_row[h] + cc) : 0.0f;
      }
      __syncwarp();
      if (!mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag)) {
        if (lane == 0) report_failure(p.status, ST_TIMEOUT, abort_flag);
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * BN);
      auto to_f = [](uint32_t r) { return KT::is_int ? static_cast<float>(static_cast<int32_t>(r)) : __uint_as_float(r); };
      if constexpr (STAGE == 1) {
        const int col0 = pair * BLOCK_ROWS;
#pragma unroll 1
        for (int c0 = 0; c0 < BLOCK_ROWS; c0 += 32) {
          uint32_t rg[32], ru[32];
          tmem_ld_x32(t_row + c0, rg);
          tmem_ld_x32(t_row + BLOCK_ROWS + c0, ru);
          tmem_ld_wait();
          if (c0 + 32 >= BLOCK_ROWS) {  // last read of this accumulator: hand it back to the MMA warp
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_tempty + 8 * acc);
          }
          float y[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float g = (to_f(rg[j]) * sw_s[c0 + j]) * sa;
            const float u = (to_f(ru[j]) * sw_s[BLOCK_ROWS + c0 + j]) * sa;
            float v = silu_f32(g) * u;
            if (p.doweight) v *= tw;
            y[j] = v;
          }
          const int n_ok = min(32, n_valid[0] - c0);
          if (orow >= 0 && n_ok > 0)
            moe_store_row32<OUTMODE, ACCUM>(p.out, static_cast<size_t>(orow) * p.n_out + col0 + c0, y, n_ok);
        }
      } else {
        const int col0 = pair * BN;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          uint32_t ra[32];
          tmem_ld_x32(t_row + c0, ra);
          tmem_ld_wait();
          if (c0 + 32 >= BN) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_tempty + 8 * acc);
          }
          float y[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float v = (to_f(ra[j]) * sw_s[c0 + j]) * sa;
            y[j] = p.doweight ? v * tw : v;
          }
          const int h = c0 >> 7;
          const int n_ok = min(32, n_valid[h] - (c0 & 127));
          if (orow >= 0 && n_ok > 0)
            moe_store_row32<OUTMODE, ACCUM>(p.out, static_cast<size_t>(orow) * p.n_out + col0 + c0, y, n_ok);
        }
      }
      acc ^= 1;
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

// Gather the activation rows (and their scales) into sorted order:
//   dst[p, :] = src[row(p), :], dst_scale[p] = src_scale[row(p)]
// with row(p) = token (by_slot == 0, stage 1), token * topk + slot (by_slot == 1,
// stage 2) or slot * tokens + token (by_slot == 2: slot-major activations, the
// reference's "int8smooth" stage 1); rows that are padding, or past num_valid,
// become zero with scale zero.
// One warp per row, 16 bytes per lane and step.
static __global__ void moe_gather_rows_kernel(uint8_t* __restrict__ dst, float* __restrict__ dst_scale,
                                       const uint8_t* __restrict__ src, const float* __restrict__ src_scale,
                                       const int* __restrict__ sorted_ids, const int* __restrict__ num_valid, int tokens,
                                       int topk, int by_slot, int K_bytes, int rows) {
  // a GEMM launched as programmatic dependent may start its weight stream now
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_valid = __ldg(num_valid);
  for (int r = blockIdx.x * warps_per_block + (threadIdx.x >> 5); r < rows; r += gridDim.x * warps_per_block) {
    long long srow = -1;
    if (r < n_valid) {
      const int id = __ldg(sorted_ids + r);
      const int tok = id & 0xFFFFFF;
      const int slot = static_cast<int>(static_cast<uint32_t>(id) >> 24);
      if (tok < tokens && slot < topk)
        srow = by_slot == 1 ? static_cast<long long>(tok) * topk + slot
                            : by_slot == 2 ? static_cast<long long>(slot) * tokens + tok : tok;
    }
    uint4* d = reinterpret_cast<uint4*>(dst + static_cast<size_t>(r) * K_bytes);
    if (srow >= 0) {
      const uint4* s = reinterpret_cast<const uint4*>(src + static_cast<size_t>(srow) * K_bytes);
      for (int i = lane; i < K_bytes / 16; i += 32) d[i] = __ldg(s + i);
      if (lane == 0) dst_scale[r] = __ldg(src_scale + srow);
    } else {
      for (int i = lane; i < K_bytes / 16; i += 32) d[i] = make_uint4(0, 0, 0, 0);
      if (lane == 0) dst_scale[r] = 0.0f;
    }
  }
}

// ---------------------------------------------------------------------------
// Routing table (the layout tests/kernels/test_moe_gemm_2stage.py:99-137 of the
// reference describes): counting sort of the (token, slot) pairs by expert,
// stable, every expert's run padded to a multiple of block_size.
// ---------------------------------------------------------------------------
// Pass 1: fill the outputs with their padding values and count the pairs of every expert
// (`counts` must be zero on entry).
static __global__ void moe_sort_count_kernel(const int* __restrict__ topk_ids, int n_pairs, int experts, int* __restrict__ counts,
                                      int* __restrict__ sorted_ids, float* __restrict__ sorted_weights, int max_padded,
                                      int* __restrict__ sorted_expert_ids, int max_blocks, int sentinel) {
  const int stride = gridDim.x * blockDim.x;
  const int t0 = blockIdx.x * blockDim.x + threadIdx.x;
  for (int i = t0; i < max_padded; i += stride) {
    sorted_ids[i] = sentinel;
    sorted_weights[i] = 0.0f;
  }
  for (int i = t0; i < max_blocks; i += stride) sorted_expert_ids[i] = -1;
  for (int i = t0; i < n_pairs; i += stride) {
    const int e = __ldg(topk_ids + i);
    if (e >= 0 && e < experts) atomicAdd(counts + e, 1);
  }
}

// Pass 2: one CTA per expert walks the pairs in order and writes its run.
constexpr int MOE_SORT_THREADS = 256;
static __global__ void __launch_bounds__(MOE_SORT_THREADS)
moe_sort_place_kernel(const int* __restrict__ topk_ids, const float* __restrict__ topk_weights, int n_pairs, int topk,
                      int tokens, int experts, int block_size, const int* __restrict__ counts,
                      int* __restrict__ sorted_ids, float* __restrict__ sorted_weights,
                      int* __restrict__ sorted_expert_ids, int* __restrict__ post_pad) {
  __shared__ int warp_sums[MOE_SORT_THREADS / 32];
  __shared__ int s_start;
  const int e = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // first row of this expert: padded sizes of the experts before it
  int part = 0;
  for (int i = tid; i < e; i += MOE_SORT_THREADS) {
    const int c = __ldg(counts + i);
    part += (c + block_size - 1) / block_size * block_size;
  }
  for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
  if (lane == 0) warp_sums[warp] = part;
  __syncthreads();
  if (tid == 0) {
    int t = 0;
    for (int w = 0; w < MOE_SORT_THREADS / 32; ++w) t += warp_sums[w];
    s_start = t;
  }
  __syncthreads();
  const int start = s_start;
  const int mine = __ldg(counts + e);
  const int n_blk = (mine + block_size - 1) / block_size;
  for (int i = tid; i < n_blk; i += MOE_SORT_THREADS) sorted_expert_ids[start / block_size + i] = e;
  if (e == experts - 1 && tid == 0) {
    post_pad[0] = start + n_blk * block_size;
    post_pad[1] = tokens;
  }
  int base = 0;  // pairs of this expert seen so far
  for (int c0 = 0; c0 < n_pairs && base < mine; c0 += MOE_SORT_THREADS) {
    const int i = c0 + tid;
    const bool hit = i < n_pairs && __ldg(topk_ids + i) == e;
    const unsigned ballot = __ballot_sync(0xffffffffu, hit);
    const int in_warp = __popc(ballot & ((1u << lane) - 1u));
    __syncthreads();  // warp_sums of the previous chunk have been read
    if (lane == 0) warp_sums[warp] = __popc(ballot);
    __syncthreads();
    int before = 0, total = 0;
    for (int w = 0; w < MOE_SORT_THREADS / 32; ++w) {
      const int v = warp_sums[w];
      if (w < warp) before += v;
      total += v;
    }
    if (hit) {
      const int dst = start + base + before + in_warp;
      sorted_ids[dst] = ((i % topk) << 24) | (i / topk);
      sorted_weights[dst] = __ldg(topk_weights + i);
    }
    base += total;
  }
}

// y[t, :] = sum over the top-k slots of x[t, slot, :] (fp32 sum, one rounding).
// With a mask, slot k of token t counts only if expert_mask[topk_ids[t, k]] != 0
// (the expert-parallel validity mask of kernels/moe/moe_gemm_2stage/moe_reduce.py:3-7
// in the reference): rows of routes that another rank serves are never read.
template <typename T>
__global__ void moe_reduce_kernel(T* __restrict__ y, const T* __restrict__ x, int tokens, int topk, int dim,
                                  const int* __restrict__ expert_mask, const int* __restrict__ topk_ids, int num_experts) {
  const long long total = static_cast<long long>(tokens) * dim / 2;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = (i * 2) / dim;
    const long long c = (i * 2) % dim;
    float lo = 0.0f, hi = 0.0f;
    for (int s = 0; s < topk; ++s) {
      if (expert_mask != nullptr) {
        const int e = __ldg(topk_ids + t * topk + s);
        if (e < 0 || e >= num_experts || __ldg(expert_mask + e) == 0) continue;
      }
      const T* src = x + (t * topk + s) * dim + c;
      if constexpr (sizeof(T) == 2) {
        if constexpr (std::is_same<T, __nv_bfloat16>::value) {
          const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src));
          lo += f.x;
          hi += f.y;
        } else {
          const float2 f = __half22float2(*reinterpret_cast<const __half2*>(src));
          lo += f.x;
          hi += f.y;
        }
      }
    }
    if constexpr (std::is_same<T, __nv_bfloat16>::value) {
      *reinterpret_cast<__nv_bfloat162*>(y + t * dim + c) = __floats2bfloat162_rn(lo, hi);
    } else {
      *reinterpret_cast<__half2*>(y + t * dim + c) = __floats2half2_rn(lo, hi);
    }
  }
}

}  // namespace flyb200
