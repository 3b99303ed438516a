// libflyb200: launchers of the small-M kernel's CTA-pair form.
#include "../../include/flyb200.h"
#include "launch.h"
#include "decode2_kernel.cuh"

#include <cstring>

namespace flyb200 {
namespace host {
namespace {

// CTA pairs (cluster 2 x split_k): tiles of 256 channels x BN tokens.
template <int KIND, int BN, int OUTMODE>
int launch_decode2(const CUtensorMap& tmA, const GemmParams& p, cudaStream_t s) {
  static std::atomic<uint64_t> done{0};
  auto kernel = gemm_decode2_kernel<KIND, BN, OUTMODE>;
  int rc = ensure_smem(kernel, SMEM_LIMIT, done);
  if (rc) return rc;
  const Decode2Layout L = decode2_layout(BN, p.stages);
  const int tiles = (p.N + BLOCK_ROWS - 1) / BLOCK_ROWS;
  if (L.total > SMEM_LIMIT || BN * BLOCK_ROWS * 4 > L.off_bar || (p.stages & 1) || (tiles & 1)) return FLYB200_E_UNSUPPORTED;
  if (p.reduce_mode == REDUCE_WORKSPACE || 2 * p.split_k > MAX_CLUSTER_SPLIT) return FLYB200_E_UNSUPPORTED;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(tiles, p.split_k, p.token_blocks < 1 ? 1 : p.token_blocks);
  cfg.blockDim = dim3(DECODE_THREADS, 1, 1);
  cfg.dynamicSmemBytes = L.total;
  cfg.stream = s;
  cudaLaunchAttribute attrs[2];
  int na = 0;
  attrs[na].id = cudaLaunchAttributeClusterDimension;
  attrs[na].val.clusterDim.x = 2;
  attrs[na].val.clusterDim.y = p.split_k;
  attrs[na].val.clusterDim.z = 1;
  ++na;
  if (p.pdl) {
    attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = na;
  FLYB200_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, tmA, p));
  return FLYB200_OK;
}

template <int KIND, int OUTMODE>
int launch_decode2_bn(int bn, const CUtensorMap& tmA, const GemmParams& p, cudaStream_t s) {
  switch (bn) {
    case 64: return launch_decode2<KIND, 64, OUTMODE>(tmA, p, s);
    case 128: return launch_decode2<KIND, 128, OUTMODE>(tmA, p, s);
    case 256: return launch_decode2<KIND, 256, OUTMODE>(tmA, p, s);
  }
  return FLYB200_E_UNSUPPORTED;
}

}  // namespace

int launch_decode2_kind(int kind, int outmode, int bn, const CUtensorMap& tmA, const GemmParams& p,
                        cudaStream_t s) {
  switch (kind) {
    case KIND_F8:
      if (outmode == OUT_BF16) return launch_decode2_bn<KIND_F8, OUT_BF16>(bn, tmA, p, s);
      if (outmode == OUT_FP16) return launch_decode2_bn<KIND_F8, OUT_FP16>(bn, tmA, p, s);
      return launch_decode2_bn<KIND_F8, OUT_RAW32>(bn, tmA, p, s);
    case KIND_I8:
      if (outmode == OUT_BF16) return launch_decode2_bn<KIND_I8, OUT_BF16>(bn, tmA, p, s);
      if (outmode == OUT_FP16) return launch_decode2_bn<KIND_I8, OUT_FP16>(bn, tmA, p, s);
      return launch_decode2_bn<KIND_I8, OUT_RAW32>(bn, tmA, p, s);
    case KIND_F16:
      if (outmode == OUT_BF16) return launch_decode2_bn<KIND_F16, OUT_BF16>(bn, tmA, p, s);
      if (outmode == OUT_FP16) return launch_decode2_bn<KIND_F16, OUT_FP16>(bn, tmA, p, s);
      break;
    case KIND_BF16:
      if (outmode == OUT_BF16) return launch_decode2_bn<KIND_BF16, OUT_BF16>(bn, tmA, p, s);
      if (outmode == OUT_FP16) return launch_decode2_bn<KIND_BF16, OUT_FP16>(bn, tmA, p, s);
      break;
  }
  return FLYB200_E_UNSUPPORTED;
}

}  // namespace host
}  // namespace flyb200
