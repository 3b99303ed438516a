// Kernel launchers of libflyb200, one translation unit per kernel family so
// that the families compile in parallel (not part of the C ABI).
#pragma once
#include "decode_kernel.cuh"
#include "host_common.h"

#include <atomic>

namespace flyb200 {
namespace host {

constexpr int SMEM_LIMIT = 232448;  // 227 KiB of dynamic shared memory per CTA
constexpr int MAX_DEVICES = 64;
constexpr int ROWS_MAX_STAGES = 8;
constexpr int ROWS2_STAGES = 6;

#define FLYB200_CUDA_TRY(expr)                                                          \
  do {                                                                                  \
    cudaError_t _e = (expr);                                                            \
    if (_e != cudaSuccess) return ::flyb200::host::record_cuda_error(_e, #expr);        \
  } while (0)

// One-time (per device) opt-in to large dynamic shared memory for a kernel.
template <typename KernelT>
int ensure_smem(KernelT kernel, int bytes, std::atomic<uint64_t>& done) {
  int dev = 0;
  FLYB200_CUDA_TRY(cudaGetDevice(&dev));
  const uint64_t bit = 1ull << dev;
  if (done.load(std::memory_order_acquire) & bit) return 0;
  FLYB200_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  done.fetch_or(bit, std::memory_order_release);
  return 0;
}

// Deepest ring (at most ROWS_MAX_STAGES) of the large-M kernel that fits shared memory for a tile width.
inline int rows_stages_for(int bn) {
  int s = ROWS_MAX_STAGES;
  while (s > 2 && rows_layout(bn, s).total > SMEM_LIMIT) --s;
  return s;
}

// Large-M kernel (p.bn, p.rows_stages set) in one of three forms: one CTA per 128 x bn tile, CTA pairs
// on 256 x 256 tiles (needs tmW), one CTA per 256 x bn tile (tmA with boxes of 256 rows, three stages).
// `kind` is KIND_*, `outmode` OUT_*.
enum : int { ROWS_FORM_ONE = 0, ROWS_FORM_PAIRS = 1, ROWS_FORM_TALL = 2 };
constexpr int ROWS_TALL_STAGES = 3;
int launch_rows_kind(int kind, int outmode, int form, const CUtensorMap& tmA, const CUtensorMap& tmW,
                     const CUtensorMap& tmC, const GemmParams& p, int sms, cudaStream_t s);
// Large-M kernel storing every tile through p.n_dst output maps.
int launch_rows_scatter_kind(int kind, int outmode, const CUtensorMap& tmA, const OutputMaps& outs, const GemmParams& p,
                             int sms, cudaStream_t s);
// Small-M kernel for a token block of `bn` and weight tiles of `w_rows` channels.
int launch_decode_kind(int kind, int outmode, int bn, int w_rows, const CUtensorMap& tmA, const GemmParams& p,
                       cudaStream_t s);

// Small-M kernel as CTA pairs (256 channels x `bn` tokens per pair, `bn` = 64, 128 or 256); `tmA` has boxes of bn / 2
// tokens.  Needs an even number of channel tiles and an even ring depth.
int launch_decode2_kind(int kind, int outmode, int bn, const CUtensorMap& tmA, const GemmParams& p, cudaStream_t s);

}  // namespace host
}  // namespace flyb200
