// A8W8 preshuffle GEMM kernels for sm_100a.
//
//   C[M,N] = epilogue( (A[M,K] . W[N,K]^T) * sa[m] * sb[n] )
//
// A (activations) is row-major 8-bit; W (weights) is in the preshuffled image
// [K/128][N][128 B, 128-byte swizzled]: one k-block of any run of rows is a
// contiguous burst that is already the shared-memory image the tensor core
// wants.  Two kernels share one pipeline skeleton (TMA producer warp -> mbarrier
// ring -> single-thread tcgen05.mma issue -> accumulators in TMEM -> epilogue
// warps):
//
//   gemm_rows_kernel   tokens on the UMMA M side (128 per tile), weights on the
//                      N side (BN per tile).  Persistent, grouped rasterisation,
//                      two TMEM accumulator buffers so the epilogue of tile i
//                      overlaps the mainloop of tile i+1, bf16 tiles leave
//                      through swizzled shared memory and TMA stores.
//   gemm_decode_kernel weights on the UMMA M side (128 channels per CTA), the
//                      few tokens on the N side (BN = 16..256), optional split-K
//                      with a ticket so the last CTA of a channel tile reduces
//                      the partials in a fixed order.  HBM-bound weight stream.
#pragma once
#include "ptx.cuh"
#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace flyb200 {

enum : int { OUT_BF16 = 0, OUT_FP16 = 1, OUT_RAW32 = 2 };
enum : int { EPI_NONE = 0, EPI_BIAS = 1, EPI_BIAS_RELU = 2, EPI_BIAS_SILU = 3, EPI_BIAS_GELU = 4 };

constexpr int BLOCK_ROWS = 128;   // UMMA M
constexpr int KBLOCK_BYTES = 128; // one swizzle row: 128 fp8/int8 or 64 half elements
constexpr int UMMA_K_BYTES = 32;  // bytes of K consumed by one tcgen05.mma
constexpr int NUM_THREADS = 192;  // warp 0 producer, warp 1 MMA, warps 2..5 epilogue

struct GemmParams {
  const uint8_t* w;      // preshuffled weights
  const float* sa;       // [M] per-token scale or nullptr
  const float* sb;       // [N] per-channel scale or nullptr
  const void* bias;      // [N] in the output type or nullptr
  void* c;               // output (bf16/fp16 [M,N], or 32-bit raw accumulators)
  int M, N, K_bytes;     // K in bytes (= elements for 8-bit inputs)
  int epilogue;
  int group_m;           // rasterisation group (row tiles per group)
  int split_k;           // decode kernel: number of K splits
  int kb_per_split;      // decode kernel: k-blocks per split
  int reduce_mode;       // decode kernel: how the K splits are combined (REDUCE_*)
  int stages;            // decode kernel: depth of the shared-memory ring
  int pdl;               // decode kernel: launched with programmatic stream serialisation
  int prefetch;          // k-blocks of weights requested into L2 ahead of the shared-memory ring (0 = none)
  float* ws_partials;    // decode kernel, REDUCE_WORKSPACE
  int* ws_tickets;       // decode kernel, REDUCE_WORKSPACE (zero before first use; self-resetting)
  int token_blocks;      // decode kernel: grid.z, blocks of BN tokens
  const uint8_t* sf_w;   // decode kernel, MX kind: scale image of the weights [K/128][N/128][512]
  const uint8_t* sf_a;   // decode kernel, MX kind: scale image of the activations [K/128][sf_a_tiles][512]
  int sf_a_tiles;        // ceil(M / 128)
  int bn;                // large-M kernel: output channels per tile (multiple of 32, 32..256)
  int rows_stages;       // large-M kernel: depth of the shared-memory ring
  int n_dst;             // scatter kernel: number of output buffers
  int dst_first;         // scatter kernel: buffer stored to first
  int* status;           // device status word (first failure wins)
#ifdef FLYB200_PROFILE
  unsigned long long* prof;  // [16] time stamps (profiling builds only)
#endif
};

template <int KIND>
struct KindTraits;
template <>
struct KindTraits<KIND_F8> {
  static constexpr uint32_t dfmt = 1, abfmt = 0;
  static constexpr bool is_int = false;
};
template <>
struct KindTraits<KIND_I8> {
  static constexpr uint32_t dfmt = 2, abfmt = 1;
  static constexpr bool is_int = true;
};
template <>
struct KindTraits<KIND_MXF8> {  // E4M3 codes with E8M0 block scales: fp32 accumulators, scaled inside the MMA
  static constexpr uint32_t dfmt = 1, abfmt = 0;
  static constexpr bool is_int = false;
};
template <>
struct KindTraits<KIND_MXF4> {  // packed E2M1 codes with E8M0 block scales
  static constexpr uint32_t dfmt = 1, abfmt = 1;
  static constexpr bool is_int = false;
};
template <>
struct KindTraits<KIND_F16> {
  static constexpr uint32_t dfmt = 1, abfmt = 0;
  static constexpr bool is_int = false;
};
template <>
struct KindTraits<KIND_BF16> {
  static constexpr uint32_t dfmt = 1, abfmt = 1;
  static constexpr bool is_int = false;
};

__device__ __forceinline__ void report_failure(int* status, int code, volatile int* abort_flag) {
  *abort_flag = 1;
  atomicCAS(status, 0, code);
}

// acc (raw 32-bit from TMEM) -> scaled/activated fp32, in the reference's
// operation order: float(acc); (v * sa[row]) * sb[col]; + bias; activation.
template <bool IS_INT>
__device__ __forceinline__ float epilogue_value(uint32_t raw, float sa, float sb, float bias, int epi, bool scaled) {
  float v = IS_INT ? static_cast<float>(static_cast<int32_t>(raw)) : __uint_as_float(raw);
  if (scaled) v = (v * sa) * sb;
  if (epi != EPI_NONE) {
    v = v + bias;
    if (epi == EPI_BIAS_RELU) {
      v = fmaxf(v, 0.0f);
    } else if (epi == EPI_BIAS_SILU) {
      v = v * (1.0f / (1.0f + __expf(-v)));
    } else if (epi == EPI_BIAS_GELU) {
      float y = 0.7978845608f * (v + 0.044715f * (v * v * v));
      float e = __expf(-2.0f * fabsf(y));
      float num = (y > 0.0f) ? 2.0f : 2.0f * e;
      v = 0.5f * v * (num * (1.0f / (1.0f + e)));
    }
  }
  return v;
}

template <int OUTMODE>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if constexpr (OUTMODE == OUT_FP16) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  } else {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  }
}
template <int OUTMODE>
__device__ __forceinline__ uint16_t pack1(float v) {
  if constexpr (OUTMODE == OUT_FP16) {
    __half h = __float2half_rn(v);
    return *reinterpret_cast<uint16_t*>(&h);
  } else {
    __nv_bfloat16 h = __float2bfloat16_rn(v);
    return *reinterpret_cast<uint16_t*>(&h);
  }
}
template <int OUTMODE>
__device__ __forceinline__ float load_bias(const void* bias, int col) {
  if constexpr (OUTMODE == OUT_FP16) {
    return __half2float(reinterpret_cast<const __half*>(bias)[col]);
  } else {
    return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(bias)[col]);
  }
}

// One warp's share (32 rows x BN columns) of an accumulator tile: TMEM ->
// registers -> scale / bias / activation -> bf16|fp16 -> 128-byte-swizzled
// staging buffer -> TMA store (clipped at M and N), or raw 32-bit stores.
// `release_tmem()` is called once, as soon as the accumulator has been read.
// `tmC` points to `n_dst` tensor maps: the staged chunk is stored through each
// of them (the caller's own output, or the same window of the output buffers of
// several GPUs), starting with map `dst_first` (+ a per-tile, per-warp rotation)
// so that neither the ranks nor the tiles of one rank all hit the same peer at
// the same time.
// CBUFS: staging buffers of this warp at `stage_c` (two: the store of one chunk overlaps the
// conversion of the next; one: where shared memory is short).
template <int KIND, int OUTMODE, int CBUFS = 2, typename ReleaseFn>
__device__ __forceinline__ void epilogue_warp_tile(const GemmParams& p, const CUtensorMap* tmC, int n_dst, int dst_first,
                                                   uint32_t t_row, int m0, int n0, int BN, int lane, uint32_t stage_c,
                                                   int& cbuf, ReleaseFn release_tmem) {
  using KT = KindTraits<KIND>;
  constexpr int C_BUF = 32 * 128;
  const bool scaled = (p.sa != nullptr) && (p.sb != nullptr);
  const int row = m0 + lane;
  const float sa_v = (scaled && row < p.M) ? __ldg(p.sa + row) : 0.0f;
  if constexpr (OUTMODE == OUT_RAW32) {
    uint32_t* out = reinterpret_cast<uint32_t*>(p.c);
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += 32) {
      uint32_t r[32];
      tmem_ld_x32(t_row + c0, r);
      tmem_ld_wait();
      if (row < p.M) {
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          const int col = n0 + c0 + j;
          if (col + 3 < p.N) {
            *reinterpret_cast<uint4*>(out + static_cast<size_t>(row) * p.N + col) =
                make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
          } else {
            for (int e = 0; e < 4; ++e)
              if (col + e < p.N) out[static_cast<size_t>(row) * p.N + col + e] = r[j + e];
          }
        }
      }
    }
    release_tmem();
  } else {
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += 64) {
      if (c0 + 64 > BN) {
        // Last 32 columns of a tile whose width is not a multiple of 64: a
        // 64-column TMA box would reach into the neighbouring tile, so these
        // leave the registers directly (64 contiguous bytes per row).
        uint32_t r[32];
        tmem_ld_x32(t_row + c0, r);
        tmem_ld_wait();
        release_tmem();
        if (row < p.M) {
          uint16_t* out_row = reinterpret_cast<uint16_t*>(p.c) + static_cast<size_t>(row) * p.N;
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            const int col = n0 + c0 + j;
            if (col < p.N) {  // N is a multiple of 16: eight columns are in or out together
              uint32_t pk[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int ce = col + 2 * e;
                const float s0 = scaled ? __ldg(p.sb + ce) : 0.0f, s1 = scaled ? __ldg(p.sb + ce + 1) : 0.0f;
                const float b0 = p.epilogue != EPI_NONE ? load_bias<OUTMODE>(p.bias, ce) : 0.0f;
                const float b1 = p.epilogue != EPI_NONE ? load_bias<OUTMODE>(p.bias, ce + 1) : 0.0f;
                pk[e] = pack2<OUTMODE>(epilogue_value<KT::is_int>(r[j + 2 * e], sa_v, s0, b0, p.epilogue, scaled),
                                       epilogue_value<KT::is_int>(r[j + 2 * e + 1], sa_v, s1, b1, p.epilogue, scaled));
              }
              *reinterpret_cast<uint4*>(out_row + col) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            }
          }
        }
        break;
      }
      uint32_t r0[32], r1[32];
      tmem_ld_x32(t_row + c0, r0);
      tmem_ld_x32(t_row + c0 + 32, r1);
      tmem_ld_wait();
      if (c0 + 64 >= BN) release_tmem();  // accumulator fully read: hand the TMEM buffer back
      // the store that last used this buffer (two chunks ago with two buffers) has to be done reading it
      if (lane == 0) bulk_wait_group_read<CBUFS - 1>();
      __syncwarp();
      const uint32_t cdst = stage_c + cbuf * C_BUF + lane * 128;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t(&r)[32] = h == 0 ? r0 : r1;
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          const int col = n0 + c0 + h * 32 + j;
          float sbv[8], bv[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const bool in = (col + e) < p.N;
            sbv[e] = (scaled && in) ? __ldg(p.sb + col + e) : 0.0f;
            bv[e] = (p.epilogue != EPI_NONE && in) ? load_bias<OUTMODE>(p.bias, col + e) : 0.0f;
          }
          uint32_t pk[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float lo = epilogue_value<KT::is_int>(r[j + 2 * e], sa_v, sbv[2 * e], bv[2 * e], p.epilogue, scaled);
            float hi =
                epilogue_value<KT::is_int>(r[j + 2 * e + 1], sa_v, sbv[2 * e + 1], bv[2 * e + 1], p.epilogue, scaled);
            pk[e] = pack2<OUTMODE>(lo, hi);
          }
          const int chunk = (h * 32 + j) >> 3;  // 16-byte chunk index inside the 128-byte row
          const uint32_t addr = cdst + static_cast<uint32_t>(((chunk ^ (lane & 7)) << 4));
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(pk[0]), "r"(pk[1]), "r"(pk[2]),
                       "r"(pk[3])
                       : "memory");
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        if (m0 < p.M && (n0 + c0) < p.N) {
          for (int d = 0; d < n_dst; ++d) {
            int which = (dst_first + d) % n_dst;
            tma_store_2d(tmC + which, stage_c + cbuf * C_BUF, n0 + c0, m0);
          }
        }
        bulk_commit_group();
      }
      cbuf = (cbuf + 1) % CBUFS;
    }
  }
}

// ===========================================================================
// Large-M kernel
// ===========================================================================
// Shared-memory carve-up of the large-M kernel for a tile width `bn` and a ring
// depth `stages` (computed identically on host and device).
struct RowsLayout {
  int a_stage, b_stage, off_b, off_c, off_bar, off_misc, total;
};
constexpr int ROWS_C_BUF = 32 * 128;  // staging buffer: 32 rows x 64 two-byte columns
constexpr int ROWS_ACC_COLS = 256;    // TMEM columns between the two accumulator buffers
__host__ __device__ inline RowsLayout rows_layout(int bn, int stages) {
  RowsLayout l;
  l.a_stage = BLOCK_ROWS * KBLOCK_BYTES;
  l.b_stage = bn * KBLOCK_BYTES;
  l.off_b = stages * l.a_stage;
  l.off_c = l.off_b + stages * l.b_stage;       // 4 warps x 2 buffers
  l.off_bar = l.off_c + 4 * 2 * ROWS_C_BUF;     // full[S], empty[S], tfull[2], tempty[2]
  l.off_misc = l.off_bar + 8 * (2 * stages + 4);
  l.total = l.off_misc + 16;
  return l;
}

constexpr int MAX_DESTINATIONS = 8;
struct OutputMaps {
  CUtensorMap m[MAX_DESTINATIONS];
};

// Body shared by the two entry kernels below: `tmC` points to `n_dst` output
// tensor maps (kernel parameters of the caller).  The tile width (p.bn, a
// multiple of 32 up to 256) and the ring depth (p.rows_stages) are run-time
// values: the host picks the width that fills the SMs in whole waves.
template <int KIND, int OUTMODE>
__device__ __forceinline__ void gemm_rows_body(const CUtensorMap& tmA, const CUtensorMap* tmC_ptr, int n_dst,
                                               int dst_first, const GemmParams& p) {
  const CUtensorMap& tmC = *tmC_ptr;
#ifdef FLYB200_PROFILE
  long long prof_wait[4] = {0, 0, 0, 0};  // producer:empty, mma:tempty, mma:full, epilogue:tfull
  const long long prof_begin = clock64();
#endif
  using KT = KindTraits<KIND>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t smem_base = smem_u32(smem_raw);
  const int BN = p.bn;
  const int STAGES = p.rows_stages;
  const RowsLayout L = rows_layout(BN, STAGES);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_raw + L.off_misc + 4);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_raw + L.off_misc);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t bar_full = smem_base + L.off_bar;
  const uint32_t bar_empty = bar_full + 8 * STAGES;
  const uint32_t bar_tfull = bar_empty + 8 * STAGES;
  const uint32_t bar_tempty = bar_tfull + 16;

  if ((smem_base & 1023u) != 0) {  // uniform over the CTA: the swizzle atoms need 1024-byte alignment
    if (threadIdx.x == 0) atomicCAS(p.status, 0, ST_SMEM_ALIGN);
    return;
  }
  // Programmatic dependent launch (p.pdl != 0): the next kernel on the stream may be scheduled onto
  // SMs as this one frees them, and this one runs its set-up (barriers, TMEM) while the previous
  // kernel finishes; no global memory is read or written before griddepcontrol.wait below.
  if (p.pdl) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

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
    abort_flag[1] = 0;  // stays zero: lets the drain below wait on time alone
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    prefetch_tensormap(&tmA);
    if (OUTMODE != OUT_RAW32) prefetch_tensormap(&tmC);
  }
  constexpr uint32_t TMEM_COLS = 512;  // two accumulator buffers of up to 256 columns
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (p.pdl) asm volatile("griddepcontrol.wait;" ::: "memory");  // the previous kernel has completed

  const int num_m = (p.M + BLOCK_ROWS - 1) / BLOCK_ROWS;
  const int num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = p.K_bytes / KBLOCK_BYTES;
  const int gm_full = p.group_m;

  // Tile order: groups of `group_m` row tiles; inside a group the row tile
  // changes fastest and the channel tiles are walked once, so the group's
  // activations stay in L2 while the weights stream through.  Odd groups walk
  // the channels backwards: the weight tiles that the previous group touched
  // last are the first ones the next group asks for.
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
      const uint64_t pol_a = l2_policy_evict_last();
      const uint64_t pol_w = l2_policy_evict_last();
      int stage = 0;
      uint32_t phase = 0;
      int issued = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int m_blk, n_blk;
        tile_coords(t, m_blk, n_blk);
        const int n0 = n_blk * BN;
        const uint32_t w_rows = static_cast<uint32_t>(min(BN, p.N - n0));
        const uint32_t w_bytes = w_rows * KBLOCK_BYTES;
        // The ring holds a few k-blocks; the weights of the next `prefetch`
        // k-blocks are already on their way from DRAM into L2, so the depth
        // of the ring only has to cover the L2 latency.
        const int ahead = min(p.prefetch, num_kb);
        for (int kb = 0; kb < ahead; ++kb)
          bulk_prefetch_l2(p.w + (static_cast<size_t>(kb) * p.N + n0) * KBLOCK_BYTES, w_bytes);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (ahead > 0 && kb + ahead < num_kb)
            bulk_prefetch_l2(p.w + (static_cast<size_t>(kb + ahead) * p.N + n0) * KBLOCK_BYTES, w_bytes);
          if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag FLYB200_PROF_ARG(&prof_wait[0]))) {
            report_failure(p.status, ST_TIMEOUT, abort_flag);
            ok = false;
            break;
          }
          const uint32_t fb = bar_full + 8 * stage;
          mbar_expect_tx(fb, L.a_stage + w_bytes);
          tma_load_2d(smem_base + stage * L.a_stage, &tmA, fb, kb * KBLOCK_BYTES, m_blk * BLOCK_ROWS, pol_a);
          bulk_load_1d(smem_base + L.off_b + stage * L.b_stage,
                       p.w + (static_cast<size_t>(kb) * p.N + n0) * KBLOCK_BYTES, w_bytes, fb, pol_w);
          ++issued;
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok || *abort_flag) {
        // Drain: wait (bounded) for the copies this thread still has in flight
        // so that none lands in shared memory after the CTA has gone.
        const int pending = min(issued, STAGES);
        for (int i = 0; i < pending; ++i) {
          int s = stage - 1 - i;
          uint32_t ph = phase;
          if (s < 0) {
            s += STAGES;
            ph ^= 1u;
          }
          mbar_wait(bar_full + 8 * s, ph, abort_flag + 1 /* never set: wait on time only */);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issue -----------------------------
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(KT::dfmt, KT::abfmt, BLOCK_ROWS, static_cast<uint32_t>(BN));
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        if (!mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1u, abort_flag FLYB200_PROF_ARG(&prof_wait[1]))) {
          report_failure(p.status, ST_TIMEOUT, abort_flag);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * ROWS_ACC_COLS);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag FLYB200_PROF_ARG(&prof_wait[2]))) {
            report_failure(p.status, ST_TIMEOUT, abort_flag);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t adesc = umma_desc_sw128_kmajor(smem_base + stage * L.a_stage);
          const uint64_t bdesc = umma_desc_sw128_kmajor(smem_base + L.off_b + stage * L.b_stage);
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
    const int ew = warp - 2; // staging buffer owner
    const uint32_t stage_c = smem_base + L.off_c + ew * 2 * ROWS_C_BUF;
    int acc = 0;
    uint32_t acc_phase = 0;
    int cbuf = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      int m_blk, n_blk;
      tile_coords(t, m_blk, n_blk);
      const int m0 = m_blk * BLOCK_ROWS + q * 32;
      const int n0 = n_blk * BN;
      if (!mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag FLYB200_PROF_ARG(&prof_wait[3]))) {
        if (lane == 0) report_failure(p.status, ST_TIMEOUT, abort_flag);
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t t_row =
          tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * ROWS_ACC_COLS);
      // own buffer first for the first tile; every further tile and warp starts one destination later
      const int first = n_dst > 1 ? (dst_first + (t / static_cast<int>(gridDim.x)) + ew) % n_dst : 0;
      epilogue_warp_tile<KIND, OUTMODE>(p, tmC_ptr, n_dst, first, t_row, m0, n0, BN, lane, stage_c, cbuf, [&]() {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_tempty + 8 * acc);
      });
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
    if (lane == 0) bulk_wait_group<0>();
  }

#ifdef FLYB200_PROFILE
  if (lane == 0) {
    const long long total = clock64() - prof_begin;
    if (warp == 0) {
      atomicAdd(p.prof + 0, static_cast<unsigned long long>(prof_wait[0]));
      atomicAdd(p.prof + 4, static_cast<unsigned long long>(total));
    } else if (warp == 1) {
      atomicAdd(p.prof + 1, static_cast<unsigned long long>(prof_wait[1]));
      atomicAdd(p.prof + 2, static_cast<unsigned long long>(prof_wait[2]));
    } else if (warp == 2) {
      atomicAdd(p.prof + 3, static_cast<unsigned long long>(prof_wait[3]));
      atomicAdd(p.prof + 5, static_cast<unsigned long long>(total));
    }
  }
#endif
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// One output buffer (the regular GEMM).
template <int KIND, int OUTMODE>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_rows_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmC,
                 const GemmParams p) {
  gemm_rows_body<KIND, OUTMODE>(tmA, &tmC, 1, 0, p);
}

// Every output tile is stored into the same window of up to eight buffers, e.g.
// the full-width output of each GPU of a column-parallel group (peer-mapped
// memory; plain TMA stores, per CTA, no multicast): the all-gather of the
// shards happens tile by tile inside the GEMM.
template <int KIND, int OUTMODE>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_rows_scatter_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ OutputMaps outs,
                         const GemmParams p) {
  gemm_rows_body<KIND, OUTMODE>(tmA, outs.m, p.n_dst, p.dst_first, p);
}

}  // namespace flyb200
