// libflyb200: the small-M (weight-streaming) kernel for 8-bit operands, and the dispatch over all kinds.
#include "decode_launch.h"

namespace flyb200 {
namespace host {

int launch_decode_kind_wide(int kind, int outmode, int bn, int w_rows, const CUtensorMap& tmA, const GemmParams& p,
                            cudaStream_t s);  // flyb200_decode_wide.cu: 16-bit and block-scaled kinds

int launch_decode_kind(int kind, int outmode, int bn, int w_rows, const CUtensorMap& tmA, const GemmParams& p,
                       cudaStream_t s) {
  switch (kind) {
    case KIND_F8:
      if (outmode == OUT_BF16) return launch_decode_bn<KIND_F8, OUT_BF16>(bn, w_rows, tmA, p, s);
      if (outmode == OUT_FP16) return launch_decode_bn<KIND_F8, OUT_FP16>(bn, w_rows, tmA, p, s);
      return launch_decode_bn<KIND_F8, OUT_RAW32>(bn, w_rows, tmA, p, s);
    case KIND_I8:
      if (outmode == OUT_BF16) return launch_decode_bn<KIND_I8, OUT_BF16>(bn, w_rows, tmA, p, s);
      if (outmode == OUT_FP16) return launch_decode_bn<KIND_I8, OUT_FP16>(bn, w_rows, tmA, p, s);
      return launch_decode_bn<KIND_I8, OUT_RAW32>(bn, w_rows, tmA, p, s);
  }
  return launch_decode_kind_wide(kind, outmode, bn, w_rows, tmA, p, s);
}

}  // namespace host
}  // namespace flyb200
