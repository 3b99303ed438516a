// libflyb200: the small-M (weight-streaming) kernel for 16-bit and block-scaled operands.
#include "decode_launch.h"

namespace flyb200 {
namespace host {

int launch_decode_kind_wide(int kind, int outmode, int bn, int w_rows, const CUtensorMap& tmA, const GemmParams& p,
                            cudaStream_t s) {
  switch (kind) {
    case KIND_F16:
      if (outmode == OUT_BF16) return launch_decode_bn<KIND_F16, OUT_BF16>(bn, w_rows, tmA, p, s);
      if (outmode == OUT_FP16) return launch_decode_bn<KIND_F16, OUT_FP16>(bn, w_rows, tmA, p, s);
      break;
    case KIND_BF16:
      if (outmode == OUT_BF16) return launch_decode_bn<KIND_BF16, OUT_BF16>(bn, w_rows, tmA, p, s);
      if (outmode == OUT_FP16) return launch_decode_bn<KIND_BF16, OUT_FP16>(bn, w_rows, tmA, p, s);
      break;
    case KIND_MXF8:
      if (outmode == OUT_BF16) return launch_decode_bn<KIND_MXF8, OUT_BF16>(bn, w_rows, tmA, p, s);
      if (outmode == OUT_FP16) return launch_decode_bn<KIND_MXF8, OUT_FP16>(bn, w_rows, tmA, p, s);
      break;
    case KIND_MXF4:
      if (outmode == OUT_BF16) return launch_decode_bn<KIND_MXF4, OUT_BF16>(bn, w_rows, tmA, p, s);
      if (outmode == OUT_FP16) return launch_decode_bn<KIND_MXF4, OUT_FP16>(bn, w_rows, tmA, p, s);
      break;
  }
  return FLYB200_E_UNSUPPORTED;
}

}  // namespace host
}  // namespace flyb200
