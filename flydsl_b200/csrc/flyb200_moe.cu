// libflyb200: host side of the grouped (mixture-of-experts) entry points of
// include/flyb200.h — argument checks, tensor map, kernel selection, launch.
#include "../../include/flyb200.h"
#include "host_common.h"
#include "moe_kernel.cuh"

#include <atomic>
#include <cstdlib>
#include <cstring>
#include <type_traits>

using namespace flyb200;

namespace {

#define CUDA_TRY(expr)                                                  \
  do {                                                                  \
    cudaError_t _e = (expr);                                            \
    if (_e != cudaSuccess) return host::record_cuda_error(_e, #expr);   \
  } while (0)

constexpr int SMEM_LIMIT = 232448;  // 227 KiB of dynamic shared memory per CTA

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Ring depth.  Up to 128 tokens per block two CTAs share an SM (half of its
// shared memory and of its 512 TMEM columns each), so that one CTA's set-up and
// epilogue overlap the other's mainloop and a grid of up to 296 CTAs runs as one
// wave; 256-token blocks need all TMEM columns and get the whole SM.
inline int moe_stages(int bn) {
  const int stage = 2 * BLOCK_ROWS * KBLOCK_BYTES + bn * KBLOCK_BYTES;
  const int budget = bn <= 128 ? (SMEM_LIMIT + 1024) / 2 - 1024 : SMEM_LIMIT;
  int n = (budget - 1024 - 12 * bn) / stage;
  return n > 8 ? 8 : n;
}

template <int KIND, int BN, int STAGE, int OUTMODE, bool ACCUM>
int launch_moe(const CUtensorMap& tmA, MoeParams p, int blocks, cudaStream_t s) {
  static std::atomic<uint64_t> done{0};
  auto kernel = moe_gemm_kernel<KIND, BN, STAGE, OUTMODE, ACCUM>;
  int dev = 0;
  CUDA_TRY(cudaGetDevice(&dev));
  const uint64_t bit = 1ull << dev;
  if (!(done.load(std::memory_order_acquire) & bit)) {
    CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT));
    done.fetch_or(bit, std::memory_order_release);
  }
  p.stages = moe_stages(BN);
  const MoeLayout L = moe_layout(BN, p.stages);
  if (p.stages < 2 || L.total > SMEM_LIMIT) return FLYB200_E_UNSUPPORTED;
  const int tiles = STAGE == 1 ? (p.n_out + BLOCK_ROWS - 1) / BLOCK_ROWS : (p.n_out + 2 * BLOCK_ROWS - 1) / (2 * BLOCK_ROWS);
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(blocks, tiles, 1);
  cfg.blockDim = dim3(MOE_THREADS, 1, 1);
  cfg.dynamicSmemBytes = L.total;
  cfg.stream = s;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = p.pdl ? 1 : 0;
  CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, tmA, p));
  return FLYB200_OK;
}

int sm_count(int* out) {
  static std::atomic<int> cached[64];
  int dev = 0;
  CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return FLYB200_E_UNSUPPORTED;
  int n = cached[dev].load(std::memory_order_relaxed);
  if (n == 0) {
    CUDA_TRY(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
    cached[dev].store(n, std::memory_order_relaxed);
  }
  *out = n;
  return FLYB200_OK;
}

// Persistent form for routing blocks that are a multiple of 128 rows.
template <int KIND, int STAGE, int OUTMODE, bool ACCUM>
int launch_moe_rows(const CUtensorMap& tmA, const MoeParams& p, int blocks, cudaStream_t s) {
  static std::atomic<uint64_t> done{0};
  auto kernel = moe_rows_kernel<KIND, STAGE, OUTMODE, ACCUM>;
  int dev = 0;
  CUDA_TRY(cudaGetDevice(&dev));
  const uint64_t bit = 1ull << dev;
  if (!(done.load(std::memory_order_acquire) & bit)) {
    CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, MoeRowsSmem::TOTAL));
    done.fetch_or(bit, std::memory_order_release);
  }
  int sms = 0;
  int rc = sm_count(&sms);
  if (rc) return rc;
  const long long row_blocks = (static_cast<long long>(blocks) * p.tile_m + BLOCK_ROWS - 1) / BLOCK_ROWS;
  const int pairs = STAGE == 1 ? (p.n_out + BLOCK_ROWS - 1) / BLOCK_ROWS : (p.n_out + MOE_ROWS_BN - 1) / MOE_ROWS_BN;
  const long long items = row_blocks * pairs;
  const int grid = static_cast<int>(items < sms ? items : sms);
  kernel<<<grid, NUM_THREADS, MoeRowsSmem::TOTAL, s>>>(tmA, p);
  CUDA_TRY(cudaGetLastError());
  return FLYB200_OK;
}

template <int KIND>
int launch_moe_rows_variant(int stage, int out_dtype, bool accumulate, const CUtensorMap& tmA, const MoeParams& p,
                            int blocks, cudaStream_t s) {
  if (stage == 1) {
    if (out_dtype == FLYB200_OUT_BF16) return launch_moe_rows<KIND, 1, MOE_OUT_BF16, false>(tmA, p, blocks, s);
    if (out_dtype == FLYB200_OUT_FP16) return launch_moe_rows<KIND, 1, MOE_OUT_FP16, false>(tmA, p, blocks, s);
    return FLYB200_E_UNSUPPORTED;
  }
  if (accumulate) {
    if (out_dtype == FLYB200_OUT_BF16) return launch_moe_rows<KIND, 2, MOE_OUT_BF16, true>(tmA, p, blocks, s);
    if (out_dtype == FLYB200_OUT_FP16) return launch_moe_rows<KIND, 2, MOE_OUT_FP16, true>(tmA, p, blocks, s);
    if (out_dtype == FLYB200_OUT_F32) return launch_moe_rows<KIND, 2, MOE_OUT_F32, true>(tmA, p, blocks, s);
    return FLYB200_E_UNSUPPORTED;
  }
  if (out_dtype == FLYB200_OUT_BF16) return launch_moe_rows<KIND, 2, MOE_OUT_BF16, false>(tmA, p, blocks, s);
  if (out_dtype == FLYB200_OUT_FP16) return launch_moe_rows<KIND, 2, MOE_OUT_FP16, false>(tmA, p, blocks, s);
  return FLYB200_E_UNSUPPORTED;
}

template <int KIND, int BN>
int launch_moe_variant(int stage, int out_dtype, bool accumulate, const CUtensorMap& tmA, const MoeParams& p, int blocks,
                       cudaStream_t s) {
  if (stage == 1) {
    if (out_dtype == FLYB200_OUT_BF16) return launch_moe<KIND, BN, 1, MOE_OUT_BF16, false>(tmA, p, blocks, s);
    if (out_dtype == FLYB200_OUT_FP16) return launch_moe<KIND, BN, 1, MOE_OUT_FP16, false>(tmA, p, blocks, s);
    return FLYB200_E_UNSUPPORTED;
  }
  if (accumulate) {
    if (out_dtype == FLYB200_OUT_BF16) return launch_moe<KIND, BN, 2, MOE_OUT_BF16, true>(tmA, p, blocks, s);
    if (out_dtype == FLYB200_OUT_FP16) return launch_moe<KIND, BN, 2, MOE_OUT_FP16, true>(tmA, p, blocks, s);
    if (out_dtype == FLYB200_OUT_F32) return launch_moe<KIND, BN, 2, MOE_OUT_F32, true>(tmA, p, blocks, s);
    return FLYB200_E_UNSUPPORTED;
  }
  if (out_dtype == FLYB200_OUT_BF16) return launch_moe<KIND, BN, 2, MOE_OUT_BF16, false>(tmA, p, blocks, s);
  if (out_dtype == FLYB200_OUT_FP16) return launch_moe<KIND, BN, 2, MOE_OUT_FP16, false>(tmA, p, blocks, s);
  return FLYB200_E_UNSUPPORTED;  // per-slot partials are 16-bit only, as in the reference
}

template <int KIND>
int launch_moe_bn(int bn, int stage, int out_dtype, bool accumulate, const CUtensorMap& tmA, const MoeParams& p,
                  int blocks, cudaStream_t s) {
  switch (bn) {
    case 16: return launch_moe_variant<KIND, 16>(stage, out_dtype, accumulate, tmA, p, blocks, s);
    case 32: return launch_moe_variant<KIND, 32>(stage, out_dtype, accumulate, tmA, p, blocks, s);
    case 64: return launch_moe_variant<KIND, 64>(stage, out_dtype, accumulate, tmA, p, blocks, s);
    case 128: return launch_moe_variant<KIND, 128>(stage, out_dtype, accumulate, tmA, p, blocks, s);
    case 256: return launch_moe_variant<KIND, 256>(stage, out_dtype, accumulate, tmA, p, blocks, s);
  }
  return FLYB200_E_UNSUPPORTED;
}

}  // namespace

extern "C" {

int flyb200_moe_gather_rows(void* dst, float* dst_scale, const void* src, const float* src_scale, const int* sorted_ids,
                            const int* num_valid_ids, int tokens, int topk, int by_slot, int row_bytes, int rows,
                            void* stream) {
  if (!dst || !dst_scale || !src || !src_scale || !sorted_ids || !num_valid_ids) return FLYB200_E_BAD_ARG;
  if (tokens < 0 || topk <= 0 || topk > 255 || row_bytes <= 0 || rows < 0 || by_slot < 0 || by_slot > 2)
    return FLYB200_E_BAD_ARG;
  if (row_bytes % 16 != 0) return FLYB200_E_UNSUPPORTED;
  if (!aligned16(dst) || !aligned16(src)) return FLYB200_E_BAD_ALIGN;
  if (rows == 0) return FLYB200_OK;
  const int warps = 8;
  int grid = (rows + warps - 1) / warps;
  if (grid > 148 * 8) grid = 148 * 8;
  moe_gather_rows_kernel<<<grid, warps * 32, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<uint8_t*>(dst), dst_scale, static_cast<const uint8_t*>(src), src_scale, sorted_ids, num_valid_ids,
      tokens, topk, by_slot, row_bytes, rows);
  CUDA_TRY(cudaGetLastError());
  return FLYB200_OK;
}

int flyb200_moe_gemm(int stage, void* out, const void* a_sorted, const void* w_shuf, const float* scale_a_sorted,
                     const float* scale_w, const int* sorted_ids, const int* expert_ids, const float* sorted_weights,
                     const int* num_valid_ids, int tokens, int topk, int experts, int model_dim, int inter_dim,
                     int tile_m, int blocks, int in_dtype, int out_dtype, int doweight, int accumulate, int after_gather,
                     void* stream) {
  if (stage != 1 && stage != 2) return FLYB200_E_BAD_ARG;
  if (!out || !a_sorted || !w_shuf || !scale_a_sorted || !scale_w || !sorted_ids || !expert_ids || !num_valid_ids)
    return FLYB200_E_BAD_ARG;
  if (doweight && !sorted_weights) return FLYB200_E_BAD_ARG;
  if (tokens < 0 || topk <= 0 || topk > 255 || experts <= 0 || model_dim <= 0 || inter_dim <= 0 || blocks < 0)
    return FLYB200_E_BAD_ARG;
  if (tokens >= (1 << 24)) return FLYB200_E_UNSUPPORTED;  // a sorted id keeps the token in 24 bits
  if (in_dtype != FLYB200_DT_FP8 && in_dtype != FLYB200_DT_INT8) return FLYB200_E_UNSUPPORTED;
  if (tile_m < 16 || tile_m > 256 || tile_m % 16 != 0) return FLYB200_E_BAD_ARG;
  if (stage == 1 && accumulate) return FLYB200_E_BAD_ARG;
  const int K = stage == 1 ? model_dim : inter_dim;
  const int n_out = stage == 1 ? inter_dim : model_dim;
  if (K % KBLOCK_BYTES != 0 || n_out % 16 != 0) return FLYB200_E_UNSUPPORTED;
  if (!aligned16(out) || !aligned16(a_sorted) || !aligned16(w_shuf)) return FLYB200_E_BAD_ALIGN;
  if (blocks == 0 || tokens == 0) return FLYB200_OK;

  MoeParams p;
  memset(&p, 0, sizeof(p));
  p.w = static_cast<const uint8_t*>(w_shuf);
  p.sa = scale_a_sorted;
  p.sw = scale_w;
  p.sorted_ids = sorted_ids;
  p.expert_ids = expert_ids;
  p.sorted_w = sorted_weights;
  p.num_valid = num_valid_ids;
  p.out = out;
  p.tokens = tokens;
  p.topk = topk;
  p.experts = experts;
  p.n_expert = stage == 1 ? 2 * inter_dim : model_dim;
  p.n_out = n_out;
  p.K_bytes = K;
  p.tile_m = tile_m;
  p.doweight = doweight ? 1 : 0;
  p.pdl = 0;
  int rc = host::status_word(&p.status);
  if (rc) return rc;

  cudaStream_t s = static_cast<cudaStream_t>(stream);
  CUtensorMap tmA;
  // Routing blocks of 64, 128 or 256 rows: persistent kernel with the tokens on the
  // UMMA M side (FLYB200_MOE_KERNEL=1 in the environment forces the other form, for tests and tuning).
  const char* force = getenv("FLYB200_MOE_KERNEL");
  const bool rows_form = (tile_m % BLOCK_ROWS == 0 || tile_m == 64) && !(force && force[0] == '1');
  if (rows_form) {
    rc = host::byte_matrix_map(&tmA, a_sorted, static_cast<uint64_t>(K), static_cast<uint64_t>(blocks) * tile_m, BLOCK_ROWS);
    if (rc) return rc;
    if (in_dtype == FLYB200_DT_FP8) return launch_moe_rows_variant<KIND_F8>(stage, out_dtype, accumulate != 0, tmA, p, blocks, s);
    return launch_moe_rows_variant<KIND_I8>(stage, out_dtype, accumulate != 0, tmA, p, blocks, s);
  }
  int bn = 16;
  while (bn < tile_m) bn *= 2;
  {
    const char* e = getenv("FLYB200_PDL");
    p.pdl = (after_gather && !(e && e[0] == '0')) ? 1 : 0;
  }
  rc = host::byte_matrix_map(&tmA, a_sorted, static_cast<uint64_t>(K), static_cast<uint64_t>(blocks) * tile_m, bn);
  if (rc) return rc;
  if (in_dtype == FLYB200_DT_FP8) return launch_moe_bn<KIND_F8>(bn, stage, out_dtype, accumulate != 0, tmA, p, blocks, s);
  return launch_moe_bn<KIND_I8>(bn, stage, out_dtype, accumulate != 0, tmA, p, blocks, s);
}

int flyb200_moe_sorting(const int* topk_ids, const float* topk_weights, int tokens, int topk, int experts, int block_size,
                        int* sorted_ids, float* sorted_weights, int* sorted_expert_ids, int* num_tokens_post_pad,
                        int* counts_scratch, void* stream) {
  if (!topk_ids || !topk_weights || !sorted_ids || !sorted_weights || !sorted_expert_ids || !num_tokens_post_pad ||
      !counts_scratch)
    return FLYB200_E_BAD_ARG;
  if (tokens < 0 || topk <= 0 || topk > 255 || experts <= 0 || block_size <= 0) return FLYB200_E_BAD_ARG;
  if (tokens >= (1 << 24)) return FLYB200_E_UNSUPPORTED;
  const long long n_pairs = static_cast<long long>(tokens) * topk;
  const long long max_padded = n_pairs + static_cast<long long>(experts) * block_size - topk;
  if (max_padded > 0x7fffffffLL || max_padded <= 0) return FLYB200_E_UNSUPPORTED;
  const int max_blocks = static_cast<int>((max_padded + block_size - 1) / block_size);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  CUDA_TRY(cudaMemsetAsync(counts_scratch, 0, sizeof(int) * experts, s));
  long long work = max_padded > n_pairs ? max_padded : n_pairs;
  int grid = static_cast<int>((work + 255) / 256);
  if (grid > 148 * 4) grid = 148 * 4;
  moe_sort_count_kernel<<<grid, 256, 0, s>>>(topk_ids, static_cast<int>(n_pairs), experts, counts_scratch, sorted_ids,
                                             sorted_weights, static_cast<int>(max_padded), sorted_expert_ids, max_blocks,
                                             (topk << 24) | tokens);
  CUDA_TRY(cudaGetLastError());
  moe_sort_place_kernel<<<experts, MOE_SORT_THREADS, 0, s>>>(topk_ids, topk_weights, static_cast<int>(n_pairs), topk,
                                                             tokens, experts, block_size, counts_scratch, sorted_ids,
                                                             sorted_weights, sorted_expert_ids, num_tokens_post_pad);
  CUDA_TRY(cudaGetLastError());
  return FLYB200_OK;
}

int flyb200_moe_reduce(void* y, const void* x, int tokens, int topk, int dim, int dtype, const int* expert_mask,
                       const int* topk_ids, int num_experts, void* stream) {
  if (!y || !x || tokens < 0 || topk <= 0 || dim <= 0) return FLYB200_E_BAD_ARG;
  if (expert_mask && (!topk_ids || num_experts <= 0)) return FLYB200_E_BAD_ARG;
  if (dim % 2 != 0) return FLYB200_E_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(y) & 3u) || (reinterpret_cast<uintptr_t>(x) & 3u)) return FLYB200_E_BAD_ALIGN;
  if (tokens == 0) return FLYB200_OK;
  const long long total = static_cast<long long>(tokens) * dim / 2;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == FLYB200_OUT_BF16) {
    moe_reduce_kernel<__nv_bfloat16><<<static_cast<int>(blocks), 256, 0, s>>>(
        static_cast<__nv_bfloat16*>(y), static_cast<const __nv_bfloat16*>(x), tokens, topk, dim, expert_mask, topk_ids,
        num_experts);
  } else if (dtype == FLYB200_OUT_FP16) {
    moe_reduce_kernel<__half><<<static_cast<int>(blocks), 256, 0, s>>>(static_cast<__half*>(y),
                                                                       static_cast<const __half*>(x), tokens, topk, dim,
                                                                       expert_mask, topk_ids, num_experts);
  } else {
    return FLYB200_E_UNSUPPORTED;
  }
  CUDA_TRY(cudaGetLastError());
  return FLYB200_OK;
}

}  // extern "C"
