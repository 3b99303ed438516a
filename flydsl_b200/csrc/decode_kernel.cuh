// Small-M ("decode") kernel: weights on the UMMA M side (128 output channels
// per CTA), the few tokens on the N side (BN = 16..256), K optionally split
// over several CTAs.  The kernel is a weight stream: every byte of the
// preshuffled weights is read once, in 16 KiB bursts, through a deep TMA ring;
// the tensor core is nearly idle and HBM bandwidth is the bound.
//
// How the K splits of one channel tile are combined (GemmParams::reduce_mode):
//   REDUCE_NONE       one CTA owns the whole K range.
//   REDUCE_CLUSTER    the splits of a tile form a thread-block cluster; every
//                     CTA parks its partial tile in its own shared memory, and
//                     after a cluster barrier each CTA sums a slice of the
//                     tokens over all peers through distributed shared memory
//                     (fixed order s = 0..S-1) and writes that slice of C.  No
//                     global scratch, no atomics.
//   REDUCE_WORKSPACE  partial tiles go to a global workspace; a per-tile ticket
//                     elects the last CTA, which sums the partials in fixed
//                     order.  Used when the split exceeds the cluster limit.
#pragma once
#include "gemm_kernels.cuh"

namespace flyb200 {

enum : int { REDUCE_NONE = 0, REDUCE_WORKSPACE = 1, REDUCE_CLUSTER = 2 };
// warp 0 producer, warp 1 MMA issuer (even k-blocks), warps 2..5 epilogue, warp 6 MMA issuer (odd k-blocks)
constexpr int DECODE_THREADS = 224;
constexpr int MAX_CLUSTER_SPLIT = 8;

// Shared-memory carve-up for a given ring depth (computed identically on host and device).
struct DecodeLayout {
  int off_w, off_a, off_bar, off_misc, off_sa, off_sf, total;
};
// `sf_atoms`: 512-byte scale atoms that ride along with every stage in the block-scaled
// kinds (weights then tokens): 2 for 8-bit codes, 4 for packed 4-bit codes, else 0.
__host__ __device__ inline DecodeLayout decode_layout(int bn, int stages, int w_rows = BLOCK_ROWS, int sf_atoms = 0) {
  DecodeLayout l;
  l.off_w = 0;
  l.off_a = stages * w_rows * KBLOCK_BYTES;
  l.off_bar = l.off_a + stages * bn * KBLOCK_BYTES;
  l.off_misc = l.off_bar + 8 * (2 * stages + 1);
  l.off_misc = (l.off_misc + 15) & ~15;
  l.off_sa = l.off_misc + 32;
  l.total = l.off_sa + bn * 4;
  l.off_sf = 0;
  if (sf_atoms > 0) {
    l.off_sf = (l.total + 15) & ~15;
    l.total = l.off_sf + stages * sf_atoms * MX_SF_ATOM;
  }
  return l;
}

// Carve-up of the CTA-pair form of the kernel (decode2_kernel.cuh).
struct Decode2Layout {
  int off_w, off_a, off_bar, off_misc, off_sa, total;
};
// bn: tokens of the pair's tile (each CTA stages bn / 2 of them per k-block)
__host__ __device__ inline Decode2Layout decode2_layout(int bn, int stages) {
  Decode2Layout l;
  l.off_w = 0;
  l.off_a = stages * BLOCK_ROWS * KBLOCK_BYTES;
  l.off_bar = l.off_a + stages * (bn / 2) * KBLOCK_BYTES;
  l.off_misc = l.off_bar + 8 * (2 * stages + 1);  // full, empty per stage; tfull
  l.off_misc = (l.off_misc + 15) & ~15;
  l.off_sa = l.off_misc + 32;
  l.total = l.off_sa + bn * 4;
  return l;
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Executed by every thread of every CTA of the cluster.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ uint32_t ld_dsmem(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_dsmem_v4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared::cluster.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr)
               : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_smem_v4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}
// The same two loads, executed only where `on` is set (v keeps its value otherwise): a predicated
// instruction, not a branch, so a run of them stays in flight together.
__device__ __forceinline__ void ld_dsmem_v4_if(uint4& v, uint32_t addr, bool on) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %5, 0;\n\t"
      "@p ld.shared::cluster.v4.u32 {%0, %1, %2, %3}, [%4];\n\t}\n"
      : "+r"(v.x), "+r"(v.y), "+r"(v.z), "+r"(v.w)
      : "r"(addr), "r"(static_cast<uint32_t>(on))
      : "memory");
}
__device__ __forceinline__ void ld_smem_v4_if(uint4& v, uint32_t addr, bool on) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %5, 0;\n\t"
      "@p ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];\n\t}\n"
      : "+r"(v.x), "+r"(v.y), "+r"(v.z), "+r"(v.w)
      : "r"(addr), "r"(static_cast<uint32_t>(on))
      : "memory");
}
// sum of two raw 32-bit accumulators (int32 or fp32 bit patterns)
template <bool IS_INT>
__device__ __forceinline__ uint32_t add_raw(uint32_t a, uint32_t b) {
  if constexpr (IS_INT) {
    return static_cast<uint32_t>(static_cast<int32_t>(a) + static_cast<int32_t>(b));
  } else {
    return __float_as_uint(__uint_as_float(a) + __uint_as_float(b));
  }
}
__device__ __forceinline__ void st_smem(uint32_t addr, uint32_t v) {
  asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}

// Epilogue and store of four consecutive channels of token m (raw sums in `acc`).
template <int KIND, int OUTMODE>
__device__ __forceinline__ void store_reduced(const GemmParams& p, const uint4& acc, int m, int m_base, int n4,
                                              const float* sa_s, const float (&sb4)[4], const float (&bias4)[4],
                                              bool scaled) {
  using KT = KindTraits<KIND>;
  if constexpr (OUTMODE == OUT_RAW32) {
    *reinterpret_cast<uint4*>(reinterpret_cast<uint32_t*>(p.c) + static_cast<size_t>(m_base + m) * p.N + n4) = acc;
  } else {
    const float sa_v = sa_s[m];
    const float v0 = epilogue_value<KT::is_int>(acc.x, sa_v, sb4[0], bias4[0], p.epilogue, scaled);
    const float v1 = epilogue_value<KT::is_int>(acc.y, sa_v, sb4[1], bias4[1], p.epilogue, scaled);
    const float v2 = epilogue_value<KT::is_int>(acc.z, sa_v, sb4[2], bias4[2], p.epilogue, scaled);
    const float v3 = epilogue_value<KT::is_int>(acc.w, sa_v, sb4[3], bias4[3], p.epilogue, scaled);
    *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(p.c) + static_cast<size_t>(m_base + m) * p.N + n4) =
        make_uint2(pack2<OUTMODE>(v0, v1), pack2<OUTMODE>(v2, v3));
  }
}

// Sum, in the fixed order s = 0..S-1, the partial tiles of the S CTAs of the
// cluster for the tokens m_first, m_first + WARPS, ... < m_end (WARPS warps share a slice,
// one token each at a time) and four consecutive channels, apply the epilogue and store.  All S*U peer reads of an iteration
// are issued before the first is used.  The S CTAs are the cluster ranks
// rank_base, rank_base + rank_stride, ...
template <int KIND, int OUTMODE, int SMAX, int U, int WARPS = 4>
__device__ __forceinline__ void cluster_reduce_slice(const GemmParams& p, uint32_t red_mine, uint32_t my_rank, int S,
                                                     int m_first, int m_end, int m_base, int n4, bool col_ok,
                                                     const float* sa_s, const float (&sb4)[4], const float (&bias4)[4],
                                                     bool scaled, uint32_t rank_base = 0, uint32_t rank_stride = 1) {
  using KT = KindTraits<KIND>;
  // The loads below are predicated, not branched around (tokens past the slice and unused peers
  // are skipped), so all SMAX*U of an iteration are in flight together.
  uint32_t peer[SMAX];
#pragma unroll
  for (int s = 0; s < SMAX; ++s)  // split s of this tile lives in cluster rank rank_base + s * rank_stride
    peer[s] = map_to_cta(red_mine, rank_base + rank_stride * static_cast<uint32_t>(s < S ? s : 0));
  const int mine = rank_stride == 0 ? 0 : static_cast<int>((my_rank - rank_base) / rank_stride);  // this CTA's split
#pragma unroll 1
  for (int mb = m_first; mb < m_end; mb += WARPS * U) {
    uint4 v[SMAX][U];
#pragma unroll
    for (int s = 0; s < SMAX; ++s) {
#pragma unroll
      for (int j = 0; j < U; ++j) {
        const int mc = mb + WARPS * j;
        const bool on = mc < m_end && s < S;
        const uint32_t off = static_cast<uint32_t>(mc * BLOCK_ROWS * 4);
        v[s][j] = make_uint4(0u, 0u, 0u, 0u);
        // this CTA's own partial tile is read as plain shared memory, the peers' over the cluster network
        ld_smem_v4_if(v[s][j], red_mine + off, on && s == mine);
        ld_dsmem_v4_if(v[s][j], peer[s] + off, on && s != mine);
      }
    }
#pragma unroll
    for (int j = 0; j < U; ++j) {
      const int m = mb + WARPS * j;
      uint4 acc = v[0][j];
#pragma unroll
      for (int s = 1; s < SMAX; ++s) {
        if (s < S) {
          acc.x = add_raw<KT::is_int>(acc.x, v[s][j].x);
          acc.y = add_raw<KT::is_int>(acc.y, v[s][j].y);
          acc.z = add_raw<KT::is_int>(acc.z, v[s][j].z);
          acc.w = add_raw<KT::is_int>(acc.w, v[s][j].w);
        }
      }
      if (m < m_end && col_ok) store_reduced<KIND, OUTMODE>(p, acc, m, m_base, n4, sa_s, sb4, bias4, scaled);
    }
  }
}

// WROWS: output channels per CTA = UMMA M.  128 is the general form.  64 halves
// the weight tile so that twice as many CTAs stream without any K split (and so
// without a reduction step); its accumulator uses TMEM lanes 0-15 of each
// 32-lane quadrant (row r of the tile sits in lane (r % 16) + 32 * (r / 16)),
// and it supports REDUCE_NONE only.
template <int KIND, int BN, int OUTMODE, int WROWS = BLOCK_ROWS>
__global__ void __launch_bounds__(DECODE_THREADS, 1) gemm_decode_kernel(const __grid_constant__ CUtensorMap tmA,
                                                                  const GemmParams p) {
  static_assert(WROWS == 128 || WROWS == 64, "weight tile of 128 or 64 channels");
  using KT = KindTraits<KIND>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t smem_base = smem_u32(smem_raw);
  const int stages = p.stages;
  // block-scaled kinds: scale atoms ride along with every stage - per operand one atom per 128
  // elements of K, i.e. one for 8-bit codes and two (HALVES) for packed 4-bit codes
  constexpr bool MX = KIND == KIND_MXF8 || KIND == KIND_MXF4;
  constexpr int HALVES = KIND == KIND_MXF4 ? 2 : 1;
  constexpr int SF_ATOMS = MX ? 2 * HALVES : 0;
  static_assert(!MX || (WROWS == BLOCK_ROWS && BN <= 128), "MX kind: 128-channel tiles, at most 128 tokens");
  const DecodeLayout L = decode_layout(BN, stages, WROWS, SF_ATOMS);
  constexpr uint32_t SF_BYTES = SF_ATOMS * MX_SF_ATOM;
  // scale atoms of k-block kb of this CTA -> shared memory at `sf`: [weights h = 0..HALVES-1][tokens h = 0..HALVES-1]
  auto load_scale_atoms = [&](uint32_t sf, int kb, uint32_t bar, uint64_t pol_w_, uint64_t pol_a_, bool weights, bool tokens) {
    if constexpr (MX) {
#pragma unroll
      for (int h = 0; h < HALVES; ++h) {
        const size_t ekb = static_cast<size_t>(kb) * HALVES + h;  // 128-ELEMENT k-block of the scale images
        if (weights)
          bulk_load_1d(sf + h * MX_SF_ATOM, p.sf_w + (ekb * (p.N / BLOCK_ROWS) + blockIdx.x) * MX_SF_ATOM, MX_SF_ATOM, bar,
                       pol_w_);
        if (tokens)
          bulk_load_1d(sf + (HALVES + h) * MX_SF_ATOM, p.sf_a + ekb * p.sf_a_tiles * MX_SF_ATOM, MX_SF_ATOM, bar, pol_a_);
      }
    }
  };
  constexpr int W_STAGE = WROWS * KBLOCK_BYTES;
  constexpr int A_STAGE = BN * KBLOCK_BYTES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_raw + L.off_misc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_raw + L.off_misc + 4);
  volatile int* last_flag = reinterpret_cast<volatile int*>(smem_raw + L.off_misc + 12);
  float* sa_s = reinterpret_cast<float*>(smem_raw + L.off_sa);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t bar_full = smem_base + L.off_bar;
  const uint32_t bar_empty = bar_full + 8 * stages;
  const uint32_t bar_tfull = bar_empty + 8 * stages;

  if ((smem_base & 1023u) != 0) {  // same answer in every CTA of the grid
    if (threadIdx.x == 0) atomicCAS(p.status, 0, ST_SMEM_ALIGN);
    return;
  }
  const int n0 = blockIdx.x * WROWS;
  // grid.z splits the tokens into blocks of BN: each CTA sees only its own block
  const int m_base = blockIdx.z * BN;
  const int M_loc = min(BN, p.M - m_base);  // >= 1 by construction of the grid
  const int tile_id = blockIdx.z * gridDim.x + blockIdx.x;  // (token block, channel tile)
  const int num_kb_total = p.K_bytes / KBLOCK_BYTES;
  const int kb_begin = blockIdx.y * p.kb_per_split;
  const int kb_end = min(num_kb_total, kb_begin + p.kb_per_split);
  const int num_kb = kb_end - kb_begin;  // >= 1 by construction of the grid
  const bool scaled = (p.sa != nullptr) && (p.sb != nullptr);
  const uint32_t w_rows = static_cast<uint32_t>(min(WROWS, p.N - n0));
  const uint32_t w_bytes = w_rows * KBLOCK_BYTES;
  const int pre = min(stages, num_kb);  // k-blocks whose loads are issued before the CTA-wide set-up finishes
  bool ok = true;

  // With programmatic dependent launch (pdl != 0) this kernel may start while
  // the previous kernel on the stream is still running.  Nothing produced by
  // that kernel may be read, and nothing written, before griddepcontrol.wait.
  //   pdl == 1: no global access at all before the wait.
  //   pdl == 2: the weights are model state that no kernel on the stream
  //             writes, so their first loads are issued before the wait.
  if (p.pdl) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#ifdef FLYB200_PROFILE
  const unsigned long long prof_t0 = globaltimer_ns();
  if (threadIdx.x == 0) atomicMin(p.prof + 0, prof_t0);
  // prof[idx]: sum over CTAs of the time since the CTA's own start; prof[8 + idx]: latest absolute time
#define FLYB200_STAMP(idx)                            \
  do {                                                \
    const unsigned long long now_ = globaltimer_ns(); \
    atomicAdd(p.prof + (idx), now_ - prof_t0);        \
    atomicMax(p.prof + 8 + (idx), now_);              \
  } while (0)
#else
#define FLYB200_STAMP(idx)
#endif

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    mbar_init(bar_tfull, num_kb >= 2 ? 2 : 1);  // one commit per MMA issuer that has k-blocks
    abort_flag[0] = 0;
    abort_flag[1] = 0;  // stays zero: lets the drain below wait on time alone
    fence_mbar_init();
    prefetch_tensormap(&tmA);
    // Start the weight stream at once: the ring is empty, so the first `pre`
    // stages need no wait, and the TMEM allocation and the CTA-wide barrier
    // below overlap with these loads.
    const uint64_t pol_w = l2_policy_evict_first();
    const uint64_t pol_a = l2_policy_evict_last();
    // Ask for this CTA's weights (the first p.prefetch k-blocks of its K range)
    // to be brought into L2 right away - also before the previous kernel on the
    // stream has completed: a prefetch reads nothing into the SM, and L2 is where
    // all writes of the GPU meet, so the loads issued after the wait below see
    // current data whatever that kernel still writes.  The DRAM latency is then
    // covered by L2, not by the depth of the shared-memory ring, which can be
    // shallow enough for two CTAs per SM: the next launch's CTAs are resident
    // (and their weights on the way) while this launch finishes.
    const int ahead = min(p.prefetch, num_kb);
    for (int i = 0; i < ahead; ++i)
      bulk_prefetch_l2(p.w + (static_cast<size_t>(kb_begin + i) * p.N + n0) * KBLOCK_BYTES, w_bytes);
    if (p.pdl == 1) asm volatile("griddepcontrol.wait;" ::: "memory");
    for (int i = 0; i < pre; ++i) {
      mbar_expect_tx(bar_full + 8 * i, A_STAGE + w_bytes + SF_BYTES);
      bulk_load_1d(smem_base + L.off_w + i * W_STAGE,
                   p.w + (static_cast<size_t>(kb_begin + i) * p.N + n0) * KBLOCK_BYTES, w_bytes, bar_full + 8 * i, pol_w);
      load_scale_atoms(smem_base + L.off_sf + i * SF_BYTES, kb_begin + i, bar_full + 8 * i, pol_w, pol_a, true, false);
    }
    if (p.pdl == 2) asm volatile("griddepcontrol.wait;" ::: "memory");
    for (int i = 0; i < pre; ++i) {
      tma_load_2d(smem_base + L.off_a + i * A_STAGE, &tmA, bar_full + 8 * i, (kb_begin + i) * KBLOCK_BYTES, m_base, pol_a);
      load_scale_atoms(smem_base + L.off_sf + i * SF_BYTES, kb_begin + i, bar_full + 8 * i, pol_w, pol_a, false, true);
    }
  }
  // Two accumulators (columns [0, BN) and [BN, 2 BN)): even k-blocks are issued by
  // warp 1 into the first, odd k-blocks by warp 6 into the second, so that the
  // ~290 cycles one thread needs to issue a k-block's MMAs are spent by two
  // threads in parallel; the epilogue adds the two.
  // MX kinds: 4 more columns per scale atom and ring stage (at most 8 stages) for the atoms in flight
  constexpr int MX_MAX_STAGES = 8;
  constexpr uint32_t SF_COL0 = 2 * BN;
  constexpr uint32_t SF_COLS = 4 * SF_ATOMS;  // TMEM columns of one stage's scale atoms
  constexpr uint32_t TMEM_NEED = 2 * BN + SF_COLS * MX_MAX_STAGES;
  constexpr uint32_t TMEM_COLS = TMEM_NEED <= 32 ? 32 : TMEM_NEED <= 64 ? 64 : TMEM_NEED <= 128 ? 128 : TMEM_NEED <= 256 ? 256 : 512;
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (p.pdl && threadIdx.x != 0) asm volatile("griddepcontrol.wait;" ::: "memory");
  // Who sums the K splits after the mainloop: from 64 tokens up all seven warps (the producer and
  // the MMA issuers have nothing left to do by then; measured 2-7 % on the whole kernel at 64-256
  // tokens), below that the four epilogue warps (with so few tokens the extra warps only cost).
  constexpr bool ALL_WARPS_REDUCE = BN >= 64;
  constexpr int REDUCE_WARPS = ALL_WARPS_REDUCE ? DECODE_THREADS / 32 : 4;
  const bool reduces = ALL_WARPS_REDUCE || (warp >= 2 && warp <= 5);
  // Per-channel operands of the four consecutive channels a thread owns in that sum, asked for now
  // and met after the mainloop.
  float sb4[4] = {0.f, 0.f, 0.f, 0.f}, bias4[4] = {0.f, 0.f, 0.f, 0.f};
  // An unsplit tile of 64 tokens or more leaves the same way as a reduced one: accumulators -> shared
  // memory as [token][channel], then every warp turns whole token rows into 256-byte stores (four
  // channels per lane).  Storing straight from the accumulator layout (one channel per thread) is
  // kept for smaller tiles: it costs ~45 ns per token (6 us at 128 tokens, 14 us at 256).
  const bool staged_out = p.reduce_mode == REDUCE_NONE && ALL_WARPS_REDUCE && WROWS == BLOCK_ROWS;
  if ((p.reduce_mode != REDUCE_NONE || staged_out) && reduces && n0 + lane * 4 < p.N) {  // (thread 0 has passed its griddepcontrol.wait above)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      if (p.sa != nullptr && p.sb != nullptr) sb4[e] = __ldg(p.sb + n0 + lane * 4 + e);
      if (p.epilogue != EPI_NONE) bias4[e] = load_bias<OUTMODE>(p.bias, n0 + lane * 4 + e);
    }
  }

  if (warp == 0) {
    // ------------------------------ producer ------------------------------
    if (lane == 0) {
      const uint64_t pol_a = l2_policy_evict_last();
      const uint64_t pol_w = l2_policy_evict_first();
      int stage = pre == stages ? 0 : pre;
      uint32_t phase = pre == stages ? 1u : 0u;
      int issued = pre;
      const int ahead = min(p.prefetch, num_kb);
      for (int kb = kb_begin + pre; kb < kb_end; ++kb) {
        if (ahead > 0 && kb - pre + ahead < kb_end)  // the next block not yet asked for
          bulk_prefetch_l2(p.w + (static_cast<size_t>(kb - pre + ahead) * p.N + n0) * KBLOCK_BYTES, w_bytes);
        if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag)) {
          report_failure(p.status, ST_TIMEOUT, abort_flag);
          ok = false;
          break;
        }
        const uint32_t fb = bar_full + 8 * stage;
        mbar_expect_tx(fb, A_STAGE + w_bytes + SF_BYTES);
        bulk_load_1d(smem_base + L.off_w + stage * W_STAGE, p.w + (static_cast<size_t>(kb) * p.N + n0) * KBLOCK_BYTES,
                     w_bytes, fb, pol_w);
        tma_load_2d(smem_base + L.off_a + stage * A_STAGE, &tmA, fb, kb * KBLOCK_BYTES, m_base, pol_a);
        load_scale_atoms(smem_base + L.off_sf + stage * SF_BYTES, kb, fb, pol_w, pol_a, true, true);
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
    const int which = warp == 1 ? 0 : 1;  // issuer 0: k-blocks 0, 2, 4, ...; issuer 1: 1, 3, 5, ...
    if (lane == 0 && which < num_kb) {
      constexpr uint32_t idesc = umma_idesc(KT::dfmt, KT::abfmt, WROWS, BN);
      const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(which * BN);
      for (int kb = which; kb < num_kb; kb += 2) {
        const int stage = kb % stages;
        const uint32_t phase = static_cast<uint32_t>(kb / stages) & 1u;
        if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag)) {
          report_failure(p.status, ST_TIMEOUT, abort_flag);
          ok = false;
          break;
        }
        tc_fence_after();
        if (kb == 0) FLYB200_STAMP(1);  // first stage landed
        const uint64_t wdesc = umma_desc_sw128_kmajor(smem_base + L.off_w + stage * W_STAGE);
        const uint64_t adesc = umma_desc_sw128_kmajor(smem_base + L.off_a + stage * A_STAGE);
        if constexpr (MX) {
          // scale atoms of this stage -> their TMEM columns; the weights are the M-side operand here
          const uint32_t sfw_t = tmem_base + SF_COL0 + static_cast<uint32_t>(stage) * SF_COLS;
          const uint32_t sfa_t = sfw_t + 4 * HALVES;
          const uint32_t sf = smem_base + L.off_sf + stage * SF_BYTES;
#pragma unroll
          for (int h = 0; h < HALVES; ++h) {
            tmem_cp_sf(sfw_t + 4 * h, sf_smem_desc(sf + h * MX_SF_ATOM));
            tmem_cp_sf(sfa_t + 4 * h, sf_smem_desc(sf + (HALVES + h) * MX_SF_ATOM));
          }
          if constexpr (KIND == KIND_MXF4) {
            constexpr uint32_t mx_idesc = umma_idesc_mxf4(WROWS, BN);
#pragma unroll
            for (int k = 0; k < KBLOCK_BYTES / UMMA_K_BYTES; ++k) {
              // 32 bytes = 64 elements = scale blocks 2k, 2k+1: atom k/2, bytes 2(k%2) and 2(k%2)+1 of its columns
              const uint32_t sf_id = static_cast<uint32_t>((k & 1) * 2);
              const uint32_t id = mx_idesc | (sf_id << 4) | (sf_id << 29);
              umma_mxf4(d_tmem, wdesc + static_cast<uint64_t>(k * (UMMA_K_BYTES >> 4)),
                        adesc + static_cast<uint64_t>(k * (UMMA_K_BYTES >> 4)), id, sfw_t + 4 * (k >> 1), sfa_t + 4 * (k >> 1),
                        (kb >= 2 || k != 0) ? 1u : 0u);
            }
          } else {
            constexpr uint32_t mx_idesc = umma_idesc_mxf8(WROWS, BN);
#pragma unroll
            for (int k = 0; k < KBLOCK_BYTES / UMMA_K_BYTES; ++k) {
              const uint32_t id = mx_idesc | (static_cast<uint32_t>(k) << 4) | (static_cast<uint32_t>(k) << 29);
              umma_mxf8(d_tmem, wdesc + static_cast<uint64_t>(k * (UMMA_K_BYTES >> 4)),
                        adesc + static_cast<uint64_t>(k * (UMMA_K_BYTES >> 4)), id, sfw_t, sfa_t, (kb >= 2 || k != 0) ? 1u : 0u);
            }
          }
        } else {
#pragma unroll
          for (int k = 0; k < KBLOCK_BYTES / UMMA_K_BYTES; ++k) {
            umma_ss<KIND>(d_tmem, wdesc + static_cast<uint64_t>(k * (UMMA_K_BYTES >> 4)),
                          adesc + static_cast<uint64_t>(k * (UMMA_K_BYTES >> 4)), idesc, (kb >= 2 || k != 0) ? 1u : 0u);
          }
        }
        umma_commit(bar_empty + 8 * stage);
      }
      if (which == 0) FLYB200_STAMP(2);  // last MMA of this issuer issued
      if (ok) umma_commit(bar_tfull);
    }
    __syncwarp();
  }

  // ------------------------------ epilogue --------------------------------
  // thread <-> output channel (TMEM lane), registers <-> tokens
  const int q = warp & 3;
  // channel of this thread; with 64-channel tiles only lanes 0-15 of a quadrant hold rows
  const int ch_local = WROWS == 128 ? q * 32 + lane : q * 16 + (lane & 15);
  const bool lane_has_row = WROWS == 128 || lane < 16;
  const int n = lane_has_row ? n0 + ch_local : p.N;  // p.N: out of range, never stored
  const uint32_t red_base = smem_base;  // partial tile [BN][128] words, reuses the (by then idle) ring
  float sb_v = 0.0f, bias_v = 0.0f;
  // tokens per TMEM wait: all loads of a chunk (both accumulators) are issued before the one wait
  constexpr int CH = BN >= 64 ? 32 : 16;
  const bool two_acc = num_kb >= 2;
  // accumulator columns [c0, c0 + 16) of this thread's lane: first plus (if used) second accumulator
  auto load_acc = [&](uint32_t t_row, int c0, uint32_t (&r)[CH]) {
#pragma unroll
    for (int i = 0; i < CH / 16; ++i) tmem_ld_x16(t_row + c0 + 16 * i, *reinterpret_cast<uint32_t(*)[16]>(&r[16 * i]));
    if (two_acc) {
      uint32_t r2[CH];
#pragma unroll
      for (int i = 0; i < CH / 16; ++i)
        tmem_ld_x16(t_row + BN + c0 + 16 * i, *reinterpret_cast<uint32_t(*)[16]>(&r2[16 * i]));
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < CH; ++j) r[j] = add_raw<KT::is_int>(r[j], r2[j]);
    } else {
      tmem_ld_wait();
    }
  };


  auto emit = [&](int m, uint32_t raw) {
    if (m < M_loc && n < p.N) {
      if constexpr (OUTMODE == OUT_RAW32) {
        reinterpret_cast<uint32_t*>(p.c)[static_cast<size_t>(m_base + m) * p.N + n] = raw;
      } else {
        const float v = epilogue_value<KT::is_int>(raw, sa_s[m], sb_v, bias_v, p.epilogue, scaled);
        reinterpret_cast<uint16_t*>(p.c)[static_cast<size_t>(m_base + m) * p.N + n] = pack1<OUTMODE>(v);
      }
    }
  };

  if (warp >= 2 && warp <= 5) {
    // epilogue operands, fetched while the weight stream runs
    const int et = threadIdx.x - 64;
    for (int i = et; i < BN; i += 128) sa_s[i] = (scaled && i < M_loc) ? __ldg(p.sa + m_base + i) : 0.0f;
    sb_v = (scaled && n < p.N) ? __ldg(p.sb + n) : 0.0f;
    bias_v = (p.epilogue != EPI_NONE && n < p.N) ? load_bias<OUTMODE>(p.bias, n) : 0.0f;
    named_bar_sync(1, 128);

    ok = mbar_wait(bar_tfull, 0, abort_flag);
    if (!ok && lane == 0) report_failure(p.status, ST_TIMEOUT, abort_flag);
    // uniform verdict over the four epilogue warps: the paths below meet at barriers
    ok = named_bar_and(1, 128, ok);
    if (threadIdx.x == 64) FLYB200_STAMP(3);  // accumulator complete
    if (ok) {
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
      if (p.reduce_mode == REDUCE_NONE && !staged_out) {
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += CH) {
          if (c0 >= M_loc) break;
          uint32_t r[CH];
          load_acc(t_row, c0, r);
#pragma unroll
          for (int j = 0; j < CH; ++j) emit(c0 + j, r[j]);
        }
      } else if (p.reduce_mode == REDUCE_CLUSTER || staged_out) {
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += CH) {
          if (c0 >= M_loc) break;
          uint32_t r[CH];
          load_acc(t_row, c0, r);
#pragma unroll
          for (int j = 0; j < CH; ++j) st_smem(red_base + static_cast<uint32_t>(((c0 + j) * BLOCK_ROWS + ch_local) * 4), r[j]);
        }
      } else {
        // partials: [split][channel tile][token][128 channels], 32-bit
        uint32_t* part = reinterpret_cast<uint32_t*>(p.ws_partials);
        const size_t tile_elems = static_cast<size_t>(BN) * BLOCK_ROWS;
        const size_t split_stride = static_cast<size_t>(gridDim.x) * gridDim.z * tile_elems;
        uint32_t* mine = part + blockIdx.y * split_stride + tile_id * tile_elems + ch_local;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += CH) {
          if (c0 >= M_loc) break;
          uint32_t r[CH];
          load_acc(t_row, c0, r);
#pragma unroll
          for (int j = 0; j < CH; ++j) __stcg(mine + static_cast<size_t>(c0 + j) * BLOCK_ROWS, r[j]);
        }
        __threadfence();
        named_bar_sync(1, 128);
        if (threadIdx.x == 64) {
          const int old = atomicAdd(p.ws_tickets + tile_id, 1);
          const int last = (old == p.split_k - 1) ? 1 : 0;
          if (last) p.ws_tickets[tile_id] = 0;  // leave the ticket ready for the next launch
          *last_flag = last;
        }
        named_bar_sync(1, 128);
        if (*last_flag) {
          __threadfence();
          // Sum the splits in the fixed order k = 0, 1, ... (the result does not depend on which CTA
          // happened to arrive last).  The partial tiles are [token][channel] like the staged tiles of
          // the cluster path, so the same split of work applies: a warp takes one token at a time and
          // each lane four consecutive channels; sixteen 16-byte loads are in flight per thread.
          const int ew4 = warp - 2;  // 0..3
          const int ch4 = lane * 4;
          const int n4 = n0 + ch4;
          const bool col_ok = n4 < p.N;  // N is a multiple of 4
          const uint32_t* src = part + tile_id * tile_elems + ch4;
          const int m_lim = M_loc;
          constexpr int U = 4, KU = 4;  // tokens x splits in flight
#pragma unroll 1
          for (int mb = ew4; mb < m_lim; mb += 4 * U) {
            uint4 acc[U];
#pragma unroll
            for (int j = 0; j < U; ++j) acc[j] = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll 1
            for (int k0 = 0; k0 < p.split_k; k0 += KU) {
              uint4 v[U][KU];
#pragma unroll
              for (int j = 0; j < U; ++j) {
#pragma unroll
                for (int kk = 0; kk < KU; ++kk) {
                  const int m = mb + 4 * j, k = k0 + kk;
                  v[j][kk] = (m < m_lim && k < p.split_k)
                                 ? __ldcg(reinterpret_cast<const uint4*>(src + k * split_stride + static_cast<size_t>(m) * BLOCK_ROWS))
                                 : make_uint4(0u, 0u, 0u, 0u);
                }
              }
#pragma unroll
              for (int j = 0; j < U; ++j) {
#pragma unroll
                for (int kk = 0; kk < KU; ++kk) {
                  if (k0 + kk < p.split_k) {
                    if constexpr (KT::is_int) {
                      acc[j].x = add_raw<true>(acc[j].x, v[j][kk].x);
                      acc[j].y = add_raw<true>(acc[j].y, v[j][kk].y);
                      acc[j].z = add_raw<true>(acc[j].z, v[j][kk].z);
                      acc[j].w = add_raw<true>(acc[j].w, v[j][kk].w);
                    } else if (k0 + kk == 0) {
                      acc[j] = v[j][kk];  // the first partial as it is, as in the cluster path
                    } else {
                      acc[j].x = add_raw<false>(acc[j].x, v[j][kk].x);
                      acc[j].y = add_raw<false>(acc[j].y, v[j][kk].y);
                      acc[j].z = add_raw<false>(acc[j].z, v[j][kk].z);
                      acc[j].w = add_raw<false>(acc[j].w, v[j][kk].w);
                    }
                  }
                }
              }
            }
#pragma unroll
            for (int j = 0; j < U; ++j) {
              const int m = mb + 4 * j;
              if (m < m_lim && col_ok) store_reduced<KIND, OUTMODE>(p, acc[j], m, m_base, n4, sa_s, sb4, bias4, scaled);
            }
          }
        }
      }
    }
  }

  if (p.reduce_mode == REDUCE_CLUSTER) {
    // Every thread of every CTA of the cluster comes here, also after a failed
    // wait (all waits above are bounded), so the cluster barriers always complete.
    tc_fence_before();
    cluster_sync_all();
    if (reduces && abort_flag[0] == 0) {  // abort_flag: the same answer in every thread of the CTA (no role has given up)
      // Reduce-scatter over the cluster: this CTA owns a slice of the tokens.
      // A warp takes one token at a time and each lane four consecutive
      // channels, so every peer read is one 16-byte load and every output row
      // leaves as one 256-byte (bf16) run per warp.
      const uint32_t rank = cluster_ctarank();
      const int S = p.split_k;
      const int m_lim = M_loc;
      const int chunk = (m_lim + S - 1) / S;
      const int m_begin = static_cast<int>(rank) * chunk;
      const int m_end = min(m_lim, m_begin + chunk);
      const int ch4 = lane * 4;
      const int n4 = n0 + ch4;
      const bool col_ok = n4 < p.N;  // N is a multiple of 4: the four channels are in or out together
      const uint32_t red_mine = red_base + static_cast<uint32_t>(ch4 * 4);
      const int m_first = m_begin + (ALL_WARPS_REDUCE ? warp : warp - 2);
      // twenty or more 16-byte loads in flight per thread whatever the split; up to 128 tokens at split 2 (64 at
      // split 4) are done in one or two rounds of loads
      if (S <= 2) {
        cluster_reduce_slice<KIND, OUTMODE, 2, ALL_WARPS_REDUCE ? 10 : 8, REDUCE_WARPS>(p, red_mine, rank, S, m_first, m_end, m_base, n4, col_ok, sa_s, sb4, bias4, scaled);
      } else if (S <= 4) {
        cluster_reduce_slice<KIND, OUTMODE, 4, ALL_WARPS_REDUCE ? 5 : 4, REDUCE_WARPS>(p, red_mine, rank, S, m_first, m_end, m_base, n4, col_ok, sa_s, sb4, bias4, scaled);
      } else {
        cluster_reduce_slice<KIND, OUTMODE, 8, ALL_WARPS_REDUCE ? 3 : 2, REDUCE_WARPS>(p, red_mine, rank, S, m_first, m_end, m_base, n4, col_ok, sa_s, sb4, bias4, scaled);
      }
    }
    if (threadIdx.x == 64) FLYB200_STAMP(4);  // this CTA's slice of the output written
    cluster_sync_all();  // nobody leaves while a peer may still read its shared memory
  } else if (staged_out) {
    __syncthreads();  // the tile is in shared memory (every thread comes here: all waits above are bounded)
    if (abort_flag[0] == 0) {
      const int ch4 = lane * 4;
      const int n4 = n0 + ch4;
      cluster_reduce_slice<KIND, OUTMODE, 1, 16, REDUCE_WARPS>(p, red_base + static_cast<uint32_t>(ch4 * 4), 0u, 1, warp, M_loc,
                                                               m_base, n4, n4 < p.N, sa_s, sb4, bias4, scaled);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
#ifdef FLYB200_PROFILE
  if (threadIdx.x == 0) {
    FLYB200_STAMP(5);
    atomicMax(p.prof + 6, globaltimer_ns());
  }
#endif
#undef FLYB200_STAMP
}

}  // namespace flyb200
