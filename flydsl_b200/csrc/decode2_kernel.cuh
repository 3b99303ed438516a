// Small-M kernel, two-SM form, for 33..256 tokens.  The one-CTA kernel brings
// the whole token tile of a k-block into every SM next to that SM's 16 KiB of
// weights; from 64 tokens up the tokens are as many bytes as the weights and
// the rate at which one SM takes in bytes, not HBM, sets the time.  Here two
// CTAs on neighbouring channel tiles form a pair and drive one
// tcgen05.mma.cta_group::2 (UMMA M = 256 channels, N = BN tokens): the token
// tile is the N-side operand, which the instruction reads half from each CTA,
// so every CTA loads its own 128 channels but only BN / 2 tokens per k-block.
// Nothing is multicast: each CTA fetches its own halves with plain loads.
//
// Cluster = (2, split_k): x is the CTA of the pair, y the K split.  Split-K
// partial tiles are reduced through distributed shared memory exactly as in
// the one-CTA kernel, among the CTAs of the cluster that hold the same channels
// (ranks r, r + 2, r + 4, ...).
//
// Signalling inside a pair (the thread that issues the MMAs does per k-block
// exactly what it does in the one-CTA kernel: one wait, four MMAs, one commit;
// everything that crosses to the other CTA is done by otherwise idle threads):
//   full[s]   one per CTA, completed by that CTA's own loads, so the weight
//             stream starts before the two CTAs have met; the leader's (even
//             cluster rank) takes one more arrival, with which the follower's
//             warp 6 forwards the completion of its own full[s];
//   empty[s]  the leader's is released by the tcgen05.commit of the MMAs that
//             read the stage (in both CTAs); the leader's producer, which waits
//             on it before refilling, passes the release on to the follower's
//             empty[s] with a remote arrive;
//   tfull     one per CTA, one commit per MMA-issuing warp of the leader.
#pragma once
#include "decode_kernel.cuh"
#include "rows2_kernel.cuh"

#ifndef FLYB200_PAIR_ISSUERS
#define FLYB200_PAIR_ISSUERS 2
#endif

namespace flyb200 {

// Arrive on a barrier of the peer CTA without a cluster-scope fence.  What the
// arrival announces was written into THIS CTA's shared memory by its own TMA
// loads and is read by this SM's own tensor core once the leader issues the
// pair's MMA, so nothing has to become visible to the other SM (in the other
// direction, "stage free", the arrival follows a tcgen05.commit that already
// covers the peer SM's reads of its own shared memory); a release at cluster
// scope here costs about half a microsecond per k-block.
__device__ __forceinline__ void mbar_arrive_peer(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

template <int KIND, int BN, int OUTMODE>
__global__ void __launch_bounds__(DECODE_THREADS, 1)
gemm_decode2_kernel(const __grid_constant__ CUtensorMap tmA, const GemmParams p) {
  static_assert(BN >= 32 && BN <= 256 && BN % 32 == 0, "token tile of the pair: 32..256, half of it per CTA");
  constexpr int ISSUERS = FLYB200_PAIR_ISSUERS;  // MMA-issuing warps of the leader (k-blocks dealt round-robin)
  using KT = KindTraits<KIND>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t smem_base = smem_u32(smem_raw);
  const int stages = p.stages;
  const Decode2Layout L = decode2_layout(BN, stages);
  constexpr int W_STAGE = BLOCK_ROWS * KBLOCK_BYTES;
  constexpr int A_HALF = BN / 2;  // tokens this CTA stages
  constexpr int A_STAGE = A_HALF * KBLOCK_BYTES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_raw + L.off_misc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_raw + L.off_misc + 4);
  float* sa_s = reinterpret_cast<float*>(smem_raw + L.off_sa);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t crank = cluster_rank();
  const uint32_t prank = crank & 1u;      // 0 = leader of the pair
  const uint32_t leader = crank & ~1u;    // cluster rank of this pair's leader
  const uint32_t bar_full = smem_base + L.off_bar;
  const uint32_t bar_empty = bar_full + 8 * stages;
  const uint32_t bar_tfull = bar_empty + 8 * stages;

  if ((smem_base & 1023u) != 0) {  // same answer in every CTA of the grid
    if (threadIdx.x == 0) atomicCAS(p.status, 0, ST_SMEM_ALIGN);
    return;
  }
  const int n0 = blockIdx.x * BLOCK_ROWS;
  const int m_base = blockIdx.z * BN;
  const int M_loc = min(BN, p.M - m_base);  // >= 1 by construction of the grid
  const int num_kb_total = p.K_bytes / KBLOCK_BYTES;
  const int kb_begin = blockIdx.y * p.kb_per_split;
  const int kb_end = min(num_kb_total, kb_begin + p.kb_per_split);
  const int num_kb = kb_end - kb_begin;  // >= 1 by construction of the grid
  const bool scaled = (p.sa != nullptr) && (p.sb != nullptr);
  const uint32_t w_bytes = static_cast<uint32_t>(min(BLOCK_ROWS, p.N - n0)) * KBLOCK_BYTES;
  const int m_half = m_base + static_cast<int>(prank) * A_HALF;  // first token this CTA stages
  const int pre = min(stages, num_kb);  // k-blocks whose loads are issued before the pair has met
  bool ok = true;

  // Programmatic dependent launch (pdl != 0): nothing the previous kernel on the
  // stream may still write is read before griddepcontrol.wait (pdl == 2: the
  // weights are static, their first loads go out before it).  An L2 prefetch
  // reads nothing into the SM, so the weights are always requested before it.
  if (p.pdl) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(bar_full + 8 * s, prank == 0 ? 2 : 1);  // leader: its loads and the follower's word
      mbar_init(bar_empty + 8 * s, 1);
    }
    mbar_init(bar_tfull, (ISSUERS == 2 && num_kb >= 2) ? 2 : 1);  // one commit per MMA issuer that has k-blocks
    abort_flag[0] = 0;
    abort_flag[1] = 0;  // stays zero: lets the drain below wait on time alone
    fence_mbar_init();
    prefetch_tensormap(&tmA);
    const uint64_t pol_w = l2_policy_evict_first();
    const uint64_t pol_a = l2_policy_evict_last();
    const int ahead = min(p.prefetch, num_kb);
    for (int i = 0; i < ahead; ++i)
      bulk_prefetch_l2(p.w + (static_cast<size_t>(kb_begin + i) * p.N + n0) * KBLOCK_BYTES, w_bytes);
    // the ring is empty and the full barriers are this CTA's own: start the stream at once
    if (p.pdl == 1) asm volatile("griddepcontrol.wait;" ::: "memory");
    for (int i = 0; i < pre; ++i) {
      mbar_expect_tx(bar_full + 8 * i, A_STAGE + w_bytes);
      bulk_load_1d(smem_base + L.off_w + i * W_STAGE, p.w + (static_cast<size_t>(kb_begin + i) * p.N + n0) * KBLOCK_BYTES,
                   w_bytes, bar_full + 8 * i, pol_w);
    }
    if (p.pdl == 2) asm volatile("griddepcontrol.wait;" ::: "memory");
    for (int i = 0; i < pre; ++i)
      tma_load_2d(smem_base + L.off_a + i * A_STAGE, &tmA, bar_full + 8 * i, (kb_begin + i) * KBLOCK_BYTES, m_half, pol_a);
  }
  // two accumulators of BN columns: even k-blocks -> first, odd -> second (one issuing warp each)
  constexpr uint32_t TMEM_NEED = 2 * BN;
  constexpr uint32_t TMEM_COLS = TMEM_NEED <= 64 ? 64 : TMEM_NEED <= 128 ? 128 : TMEM_NEED <= 256 ? 256 : 512;
  if (warp == 1) {
    tmem_alloc_2sm(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish_2sm();
  }
  tc_fence_before();
  cluster_barrier_all();  // the barriers of both CTAs exist, the pair's TMEM is allocated
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
  // an unsplit tile of 64 tokens or more leaves through shared memory too (whole token rows per warp)
  const bool staged_out = p.reduce_mode == REDUCE_NONE && ALL_WARPS_REDUCE;
  if ((p.reduce_mode == REDUCE_CLUSTER || staged_out) && reduces && n0 + lane * 4 < p.N) {  // (thread 0 has passed its griddepcontrol.wait above)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      if (p.sa != nullptr && p.sb != nullptr) sb4[e] = __ldg(p.sb + n0 + lane * 4 + e);
      if (p.epilogue != EPI_NONE) bias4[e] = load_bias<OUTMODE>(p.bias, n0 + lane * 4 + e);
    }
  }

  if (warp == 0) {
    // ---------------- producer (both CTAs): own 128 channels, own half of the tokens ----------------
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
        if (prank == 0) mbar_arrive_peer(mapa_u32(bar_empty + 8 * stage, leader + 1));  // the follower may refill too
        const uint32_t fb = bar_full + 8 * stage;
        mbar_expect_tx(fb, A_STAGE + w_bytes);
        bulk_load_1d(smem_base + L.off_w + stage * W_STAGE, p.w + (static_cast<size_t>(kb) * p.N + n0) * KBLOCK_BYTES, w_bytes,
                     fb, pol_w);
        tma_load_2d(smem_base + L.off_a + stage * A_STAGE, &tmA, fb, kb * KBLOCK_BYTES, m_half, pol_a);
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
    // ---------------- MMA issue (leader only, two issuing warps) ----------------
    const int which = warp == 1 ? 0 : 1;  // issuer 0: k-blocks 0, 2, 4, ...; issuer 1: 1, 3, 5, ...
    if (lane == 0 && prank == 0 && which < num_kb && which < ISSUERS) {
      constexpr uint32_t idesc = umma_idesc(KT::dfmt, KT::abfmt, 2 * BLOCK_ROWS, BN);
      const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(which * BN);
      for (int kb = which; kb < num_kb; kb += ISSUERS) {
        const int stage = kb % stages;
        const uint32_t phase = static_cast<uint32_t>(kb / stages) & 1u;
        // this CTA's halves have landed and the follower has said the same of its own
        if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag)) {
          report_failure(p.status, ST_TIMEOUT, abort_flag);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint64_t wdesc = umma_desc_sw128_kmajor(smem_base + L.off_w + stage * W_STAGE);
        const uint64_t adesc = umma_desc_sw128_kmajor(smem_base + L.off_a + stage * A_STAGE);
#pragma unroll
        for (int k = 0; k < KBLOCK_BYTES / UMMA_K_BYTES; ++k) {
          umma_ss_2sm<KIND>(d_tmem, wdesc + static_cast<uint64_t>(k * (UMMA_K_BYTES >> 4)),
                            adesc + static_cast<uint64_t>(k * (UMMA_K_BYTES >> 4)), idesc, (kb >= ISSUERS || k != 0) ? 1u : 0u);
        }
        // the stage is free in both CTAs once these MMAs have read it (the producer tells the follower)
        umma_commit_2sm(bar_empty + 8 * stage);
      }
      if (ok) {
        umma_commit_2sm(bar_tfull);
        umma_commit_2sm(mapa_u32(bar_tfull, leader + 1));
      }
    } else if (lane == 0 && prank == 1 && warp == 6) {
      // ---------------- follower: tell the leader when a stage of this CTA has landed ----------------
      for (int kb = 0; kb < num_kb; ++kb) {
        const int stage = kb % stages;
        const uint32_t phase = static_cast<uint32_t>(kb / stages) & 1u;
        if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag)) {
          report_failure(p.status, ST_TIMEOUT, abort_flag);
          break;
        }
        mbar_arrive_peer(mapa_u32(bar_full + 8 * stage, leader));
      }
    }
    __syncwarp();
  }

  // ---------------- epilogue (both CTAs): thread <-> own channel (TMEM lane), registers <-> tokens ----------------
  const int q = warp & 3;
  const int ch_local = q * 32 + lane;
  const int n = n0 + ch_local;
  const uint32_t red_base = smem_base;  // partial tile [BN][128] words, reuses the (by then idle) ring
  float sb_v = 0.0f, bias_v = 0.0f;
  // tokens per TMEM wait: all loads of a chunk (both accumulators) are issued before the one wait
  constexpr int CH = BN >= 64 ? 32 : 16;
  const bool two_acc = ISSUERS == 2 && num_kb >= 2;
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
    const int et = threadIdx.x - 64;
    for (int i = et; i < BN; i += 128) sa_s[i] = (scaled && i < M_loc) ? __ldg(p.sa + m_base + i) : 0.0f;
    sb_v = (scaled && n < p.N) ? __ldg(p.sb + n) : 0.0f;
    bias_v = (p.epilogue != EPI_NONE && n < p.N) ? load_bias<OUTMODE>(p.bias, n) : 0.0f;
    named_bar_sync(1, 128);

    ok = mbar_wait(bar_tfull, 0, abort_flag);
    if (!ok && lane == 0) report_failure(p.status, ST_TIMEOUT, abort_flag);
    ok = named_bar_and(1, 128, ok);  // uniform verdict over the four epilogue warps
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
      } else {
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += CH) {
          if (c0 >= M_loc) break;
          uint32_t r[CH];
          load_acc(t_row, c0, r);
#pragma unroll
          for (int j = 0; j < CH; ++j) st_smem(red_base + static_cast<uint32_t>(((c0 + j) * BLOCK_ROWS + ch_local) * 4), r[j]);
        }
      }
    }
  }

  if (p.reduce_mode == REDUCE_CLUSTER) {
    // Every thread of every CTA of the cluster comes here, also after a failed
    // wait (all waits above are bounded), so the cluster barriers always complete.
    tc_fence_before();
    cluster_barrier_all();
    if (reduces && abort_flag[0] == 0) {  // abort_flag: the same answer in every thread of the CTA (no role has given up)
      // reduce-scatter over the K splits of this CTA's channels (cluster ranks prank, prank + 2, ...)
      const int S = p.split_k;
      const int chunk = (M_loc + S - 1) / S;
      const int m_begin = static_cast<int>(blockIdx.y) * chunk;
      const int m_end = min(M_loc, m_begin + chunk);
      const int ch4 = lane * 4;
      const int n4 = n0 + ch4;
      const bool col_ok = n4 < p.N;  // N is a multiple of 4: the four channels are in or out together
      const uint32_t red_mine = red_base + static_cast<uint32_t>(ch4 * 4);
      const int m_first = m_begin + (ALL_WARPS_REDUCE ? warp : warp - 2);
      if (S <= 2) {
        cluster_reduce_slice<KIND, OUTMODE, 2, ALL_WARPS_REDUCE ? 10 : 8, REDUCE_WARPS>(p, red_mine, crank, S, m_first, m_end, m_base, n4, col_ok, sa_s, sb4, bias4, scaled, prank, 2);
      } else {
        cluster_reduce_slice<KIND, OUTMODE, 4, ALL_WARPS_REDUCE ? 5 : 4, REDUCE_WARPS>(p, red_mine, crank, S, m_first, m_end, m_base, n4, col_ok, sa_s, sb4, bias4, scaled, prank, 2);
      }
    }
  }

  if (staged_out) {
    __syncthreads();  // the tile is in shared memory (every thread comes here: all waits above are bounded)
    if (abort_flag[0] == 0) {
      const int ch4 = lane * 4;
      const int n4 = n0 + ch4;
      cluster_reduce_slice<KIND, OUTMODE, 1, 16, REDUCE_WARPS>(p, red_base + static_cast<uint32_t>(ch4 * 4), crank, 1, warp, M_loc,
                                                               m_base, n4, n4 < p.N, sa_s, sb4, bias4, scaled, crank, 1);
    }
  }

  // Nobody leaves while a peer may still read its shared memory (the leader's
  // MMAs, the split-K reduction) or signal one of its barriers.
  tc_fence_before();
  cluster_barrier_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_2sm(tmem_base, TMEM_COLS);
  }
}

}  // namespace flyb200
