// Launchers of the small-M kernel, shared by the translation units that instantiate it
// (one per group of operand kinds, so that they compile in parallel).
#pragma once
#include "../../include/flyb200.h"
#include "launch.h"

#include <cstring>

namespace flyb200 {
namespace host {
namespace {

template <int KIND, int BN, int OUTMODE, int WROWS = BLOCK_ROWS>
int launch_decode(const CUtensorMap& tmA, const GemmParams& p, cudaStream_t s) {
  static std::atomic<uint64_t> done{0};
  auto kernel = gemm_decode_kernel<KIND, BN, OUTMODE, WROWS>;
  int rc = ensure_smem(kernel, SMEM_LIMIT, done);
  if (rc) return rc;
  constexpr int SF_ATOMS = KIND == KIND_MXF8 ? 2 : KIND == KIND_MXF4 ? 4 : 0;
  const DecodeLayout L = decode_layout(BN, p.stages, WROWS, SF_ATOMS);
  if (L.total > SMEM_LIMIT || BN * BLOCK_ROWS * 4 > L.off_bar) return FLYB200_E_UNSUPPORTED;
  if (SF_ATOMS > 0 && p.stages > 8) return FLYB200_E_UNSUPPORTED;  // scale columns in TMEM for 8 stages
  if (WROWS != BLOCK_ROWS && p.reduce_mode != REDUCE_NONE) return FLYB200_E_UNSUPPORTED;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((p.N + WROWS - 1) / WROWS, p.split_k, p.token_blocks < 1 ? 1 : p.token_blocks);
  cfg.blockDim = dim3(DECODE_THREADS, 1, 1);
  cfg.dynamicSmemBytes = L.total;
  cfg.stream = s;
  cudaLaunchAttribute attrs[2];
  int na = 0;
  if (p.reduce_mode == REDUCE_CLUSTER) {
    attrs[na].id = cudaLaunchAttributeClusterDimension;
    attrs[na].val.clusterDim.x = 1;
    attrs[na].val.clusterDim.y = p.split_k;
    attrs[na].val.clusterDim.z = 1;
    ++na;
  }
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
int launch_decode_bn(int bn, int w_rows, const CUtensorMap& tmA, const GemmParams& p, cudaStream_t s) {
  if constexpr (KIND == KIND_MXF8 || KIND == KIND_MXF4) {  // block-scaled kinds: 128-channel tiles, up to 128 tokens
    if (w_rows != BLOCK_ROWS) return FLYB200_E_UNSUPPORTED;
    switch (bn) {
      case 16: return launch_decode<KIND, 16, OUTMODE>(tmA, p, s);
      case 32: return launch_decode<KIND, 32, OUTMODE>(tmA, p, s);
      case 64: return launch_decode<KIND, 64, OUTMODE>(tmA, p, s);
      case 128: return launch_decode<KIND, 128, OUTMODE>(tmA, p, s);
    }
    return FLYB200_E_UNSUPPORTED;
  } else {
    if (w_rows == 64) {  // half-height weight tiles: built for the token counts where they pay off
      switch (bn) {
        case 16: return launch_decode<KIND, 16, OUTMODE, 64>(tmA, p, s);
        case 32: return launch_decode<KIND, 32, OUTMODE, 64>(tmA, p, s);
        case 64: return launch_decode<KIND, 64, OUTMODE, 64>(tmA, p, s);
      }
      return FLYB200_E_UNSUPPORTED;
    }
    switch (bn) {
      case 16: return launch_decode<KIND, 16, OUTMODE>(tmA, p, s);
      case 32: return launch_decode<KIND, 32, OUTMODE>(tmA, p, s);
      case 64: return launch_decode<KIND, 64, OUTMODE>(tmA, p, s);
      case 128: return launch_decode<KIND, 128, OUTMODE>(tmA, p, s);
      case 256: return launch_decode<KIND, 256, OUTMODE>(tmA, p, s);
    }
    return FLYB200_E_UNSUPPORTED;
  }
}

}  // namespace
}  // namespace host
}  // namespace flyb200
