// libflyb200: launchers of the large-M kernels (one CTA per 128 x bn tile, one
// CTA per 256 x bn tile, CTA pairs on 256 x 256 tiles, and the form that stores
// every tile to several output buffers).
#include "../../include/flyb200.h"
#include "launch.h"
#include "rows2_kernel.cuh"
#include "rows_tall_kernel.cuh"

#include <cstring>

namespace flyb200 {
namespace host {
namespace {

// One-dimensional launch, optionally with the programmatic-stream-serialisation attribute.
template <typename KernelT, typename... Args>
int launch_plain_or_pdl(KernelT kernel, int grid, int threads, int smem, cudaStream_t s, bool pdl, const Args&... args) {
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(threads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = pdl ? 1 : 0;
  FLYB200_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, args...));
  return FLYB200_OK;
}

template <int KIND, int OUTMODE>
int launch_rows(const CUtensorMap& tmA, const CUtensorMap& tmC, const GemmParams& p, int sms, cudaStream_t s) {
  static std::atomic<uint64_t> done{0};
  auto kernel = gemm_rows_kernel<KIND, OUTMODE>;
  int rc = ensure_smem(kernel, SMEM_LIMIT, done);
  if (rc) return rc;
  const RowsLayout L = rows_layout(p.bn, p.rows_stages);
  if (L.total > SMEM_LIMIT || p.bn < 32 || p.bn > 256 || (p.bn & 31)) return FLYB200_E_UNSUPPORTED;
  const long long tiles = static_cast<long long>((p.M + BLOCK_ROWS - 1) / BLOCK_ROWS) * ((p.N + p.bn - 1) / p.bn);
  const int grid = static_cast<int>(tiles < sms ? tiles : sms);
  return launch_plain_or_pdl(kernel, grid, NUM_THREADS, L.total, s, p.pdl != 0, tmA, tmC, p);
}

// One CTA per 256 x bn tile (tmA: boxes of 256 rows).
template <int KIND, int OUTMODE>
int launch_rows_tall(const CUtensorMap& tmA, const CUtensorMap& tmC, const GemmParams& p, int sms, cudaStream_t s) {
  static std::atomic<uint64_t> done{0};
  auto kernel = gemm_rows_tall_kernel<KIND, OUTMODE>;
  int rc = ensure_smem(kernel, SMEM_LIMIT, done);
  if (rc) return rc;
  const TallLayout L = rows_tall_layout(p.bn, p.rows_stages);
  if (L.total > SMEM_LIMIT || p.rows_stages < 2 || p.bn < 32 || p.bn > 256 || (p.bn & 31)) return FLYB200_E_UNSUPPORTED;
  const long long tiles = static_cast<long long>((p.M + TALL_ROWS - 1) / TALL_ROWS) * ((p.N + p.bn - 1) / p.bn);
  const int grid = static_cast<int>(tiles < sms ? tiles : sms);
  return launch_plain_or_pdl(kernel, grid, TALL_THREADS, L.total, s, p.pdl != 0, tmA, tmC, p);
}

template <int KIND, int OUTMODE>
int launch_rows2(const CUtensorMap& tmA, const CUtensorMap& tmW, const CUtensorMap& tmC, const GemmParams& p, int sms,
                 cudaStream_t s) {
  using L = Rows2Smem<ROWS2_STAGES>;
  static std::atomic<uint64_t> done{0};
  static int max_clusters[MAX_DEVICES] = {0};
  auto kernel = gemm_rows2_kernel<KIND, ROWS2_STAGES, OUTMODE>;
  int rc = ensure_smem(kernel, L::TOTAL, done);
  if (rc) return rc;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.blockDim = dim3(NUM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = L::TOTAL;
  cfg.stream = s;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  int dev = 0;
  FLYB200_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= MAX_DEVICES) return FLYB200_E_UNSUPPORTED;
  if (max_clusters[dev] == 0) {
    cfg.gridDim = dim3(sms & ~1, 1, 1);
    int n = 0;
    FLYB200_CUDA_TRY(cudaOccupancyMaxActiveClusters(&n, kernel, &cfg));
    if (n < 1) return FLYB200_E_UNSUPPORTED;
    max_clusters[dev] = n;
  }
  const int tiles = ((p.M + 255) / 256) * ((p.N + 255) / 256);
  const int clusters = tiles < max_clusters[dev] ? tiles : max_clusters[dev];
  cfg.gridDim = dim3(2 * clusters, 1, 1);
  FLYB200_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, tmA, tmW, tmC, p));
  return FLYB200_OK;
}

template <int KIND, int OUTMODE>
int launch_rows_scatter(const CUtensorMap& tmA, const OutputMaps& outs, const GemmParams& p, int sms, cudaStream_t s) {
  static std::atomic<uint64_t> done{0};
  auto kernel = gemm_rows_scatter_kernel<KIND, OUTMODE>;
  int rc = ensure_smem(kernel, SMEM_LIMIT, done);
  if (rc) return rc;
  const RowsLayout L = rows_layout(p.bn, p.rows_stages);
  // every staged chunk goes out as a 64-column TMA box here: no 32-column remainder
  if (L.total > SMEM_LIMIT || p.bn < 64 || p.bn > 256 || (p.bn & 63)) return FLYB200_E_UNSUPPORTED;
  const long long tiles = static_cast<long long>((p.M + BLOCK_ROWS - 1) / BLOCK_ROWS) * ((p.N + p.bn - 1) / p.bn);
  const int grid = static_cast<int>(tiles < sms ? tiles : sms);
  kernel<<<grid, NUM_THREADS, L.total, s>>>(tmA, outs, p);
  FLYB200_CUDA_TRY(cudaGetLastError());
  return FLYB200_OK;
}

template <int KIND, int OUTMODE>
int rows_any(int form, const CUtensorMap& tmA, const CUtensorMap& tmW, const CUtensorMap& tmC, const GemmParams& p,
             int sms, cudaStream_t s) {
  if (form == ROWS_FORM_PAIRS) return launch_rows2<KIND, OUTMODE>(tmA, tmW, tmC, p, sms, s);
  if (form == ROWS_FORM_TALL) return launch_rows_tall<KIND, OUTMODE>(tmA, tmC, p, sms, s);
  return launch_rows<KIND, OUTMODE>(tmA, tmC, p, sms, s);
}

}  // namespace

int launch_rows_kind(int kind, int outmode, int form, const CUtensorMap& tmA, const CUtensorMap& tmW,
                     const CUtensorMap& tmC, const GemmParams& p, int sms, cudaStream_t s) {
  switch (kind) {
    case KIND_F8:
      if (outmode == OUT_BF16) return rows_any<KIND_F8, OUT_BF16>(form, tmA, tmW, tmC, p, sms, s);
      if (outmode == OUT_FP16) return rows_any<KIND_F8, OUT_FP16>(form, tmA, tmW, tmC, p, sms, s);
      return rows_any<KIND_F8, OUT_RAW32>(form, tmA, tmW, tmC, p, sms, s);
    case KIND_I8:
      if (outmode == OUT_BF16) return rows_any<KIND_I8, OUT_BF16>(form, tmA, tmW, tmC, p, sms, s);
      if (outmode == OUT_FP16) return rows_any<KIND_I8, OUT_FP16>(form, tmA, tmW, tmC, p, sms, s);
      return rows_any<KIND_I8, OUT_RAW32>(form, tmA, tmW, tmC, p, sms, s);
    case KIND_F16:
      if (outmode == OUT_BF16) return rows_any<KIND_F16, OUT_BF16>(form, tmA, tmW, tmC, p, sms, s);
      if (outmode == OUT_FP16) return rows_any<KIND_F16, OUT_FP16>(form, tmA, tmW, tmC, p, sms, s);
      break;
    case KIND_BF16:
      if (outmode == OUT_BF16) return rows_any<KIND_BF16, OUT_BF16>(form, tmA, tmW, tmC, p, sms, s);
      if (outmode == OUT_FP16) return rows_any<KIND_BF16, OUT_FP16>(form, tmA, tmW, tmC, p, sms, s);
      break;
  }
  return FLYB200_E_UNSUPPORTED;
}

int launch_rows_scatter_kind(int kind, int outmode, const CUtensorMap& tmA, const OutputMaps& outs, const GemmParams& p,
                             int sms, cudaStream_t s) {
  const bool f16out = outmode == OUT_FP16;
  switch (kind) {
    case KIND_F8:
      return f16out ? launch_rows_scatter<KIND_F8, OUT_FP16>(tmA, outs, p, sms, s)
                    : launch_rows_scatter<KIND_F8, OUT_BF16>(tmA, outs, p, sms, s);
    case KIND_I8:
      return f16out ? launch_rows_scatter<KIND_I8, OUT_FP16>(tmA, outs, p, sms, s)
                    : launch_rows_scatter<KIND_I8, OUT_BF16>(tmA, outs, p, sms, s);
    case KIND_F16:
      return f16out ? launch_rows_scatter<KIND_F16, OUT_FP16>(tmA, outs, p, sms, s)
                    : launch_rows_scatter<KIND_F16, OUT_BF16>(tmA, outs, p, sms, s);
    case KIND_BF16:
      return f16out ? launch_rows_scatter<KIND_BF16, OUT_FP16>(tmA, outs, p, sms, s)
                    : launch_rows_scatter<KIND_BF16, OUT_BF16>(tmA, outs, p, sms, s);
  }
  return FLYB200_E_UNSUPPORTED;
}

}  // namespace host
}  // namespace flyb200
