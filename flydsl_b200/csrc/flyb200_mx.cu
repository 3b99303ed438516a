// libflyb200: host side of the MXFP8 (block-scaled) entry points of
// include/flyb200.h — argument checks, tensor map, launch.
#include "../../include/flyb200.h"
#include "host_common.h"
#include "mx_kernel.cuh"

#include <atomic>
#include <cstdlib>
#include <cstring>

using namespace flyb200;

namespace {

#define CUDA_TRY(expr)                                                  \
  do {                                                                  \
    cudaError_t _e = (expr);                                            \
    if (_e != cudaSuccess) return host::record_cuda_error(_e, #expr);   \
  } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <int OUTMODE, int BN, bool FP4 = false>
int launch_mx(const CUtensorMap& tmA, const MxParams& p, cudaStream_t s) {
  static std::atomic<uint64_t> done{0};
  auto kernel = mx_gemm_kernel<OUTMODE, BN, FP4>;
  using Smem = MxSmem<BN, FP4>;
  int dev = 0;
  CUDA_TRY(cudaGetDevice(&dev));
  const uint64_t bit = 1ull << dev;
  if (!(done.load(std::memory_order_acquire) & bit)) {
    CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::TOTAL));
    done.fetch_or(bit, std::memory_order_release);
  }
  int sms = 0;
  CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const long long tiles = static_cast<long long>((p.M + BLOCK_ROWS - 1) / BLOCK_ROWS) * (p.N / BN);
  const int grid = static_cast<int>(tiles < sms ? tiles : sms);
  kernel<<<grid, NUM_THREADS, Smem::TOTAL, s>>>(tmA, p);
  CUDA_TRY(cudaGetLastError());
  return FLYB200_OK;
}

}  // namespace

extern "C" {

size_t flyb200_mx_scale_image_bytes(int rows, int K) {
  if (rows <= 0 || K <= 0 || K % KBLOCK_BYTES != 0) return 0;
  return static_cast<size_t>(K / KBLOCK_BYTES) * ((rows + 127) / 128) * MX_SF_ATOM;
}

int flyb200_mx_scale_image(void* dst, const void* src, int rows, int K, void* stream) {
  if (!dst || !src || rows <= 0 || K <= 0) return FLYB200_E_BAD_ARG;
  if (K % KBLOCK_BYTES != 0) return FLYB200_E_UNSUPPORTED;
  const int row_tiles = (rows + 127) / 128;
  const long long total = static_cast<long long>(flyb200_mx_scale_image_bytes(rows, K));
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  mx_scale_image_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<uint8_t*>(dst), static_cast<const uint8_t*>(src), rows, K / 32, row_tiles);
  CUDA_TRY(cudaGetLastError());
  return FLYB200_OK;
}

namespace {
// Up to 128 tokens are a weight stream for the small-M kernel in its block-scaled kind - as long as its
// CTAs (one per 128 channels) fit one round: on wider outputs its later rounds run part empty and the
// persistent large-M kernel is 20-45 % faster (MXFP8 128 x 28672 x 8192: 43 against 66 us; MXFP4 128 x
// 57344 x 8192: 51 against 90 us).  FLYB200_MX_SMALL=0 / 1 forces the choice.
bool mx_small_m(int M, int N) {
  if (M > 128) return false;
  if (const char* e = getenv("FLYB200_MX_SMALL")) {
    if (e[0] == '0') return false;
    if (e[0] == '1') return true;
  }
  int sms = 0;
  if (flyb200::host::sm_count(&sms) != FLYB200_OK) return true;
  return (N + 127) / 128 <= sms;
}
// Tile shape of the large-M kernel: 128 x 256 tiles (one accumulator, exposed epilogue) win once a
// tile's mainloop is a few times longer than its epilogue (2.44-2.47 against 1.82-1.88 PFLOP/s at
// K = 8192, M >= 4096) - unless the 128 x 128 tiles cover the output in one round of CTAs: then
// they put twice as many SMs to work (MXFP8 256 x 8192 x 8192: 27.9 against 31.4 us; MXFP4:
// 18.4 against 20.9 us).  `k_bytes`: bytes of codes per row.
bool mx_wide_tiles(int M, int N, int k_bytes) {
  if (N % 256 != 0 || k_bytes < 1024) return false;
  int sms = 0;
  if (flyb200::host::sm_count(&sms) != FLYB200_OK) return true;
  const long long tiles128 = static_cast<long long>((M + 127) / 128) * (N / 128);
  return tiles128 > sms;
}
}  // namespace

int flyb200_gemm_mxfp8(void* c, const void* a, const void* w_shuf, const void* scale_a_image, const void* scale_w_image,
                       int M, int N, int K, int out_dtype, void* stream) {
  if (!c || !a || !w_shuf || !scale_a_image || !scale_w_image || M < 0 || N <= 0 || K <= 0) return FLYB200_E_BAD_ARG;
  if (out_dtype != FLYB200_OUT_BF16 && out_dtype != FLYB200_OUT_FP16) return FLYB200_E_BAD_ARG;
  if (K % KBLOCK_BYTES != 0 || N % 128 != 0) return FLYB200_E_UNSUPPORTED;
  if (!aligned16(c) || !aligned16(a) || !aligned16(w_shuf) || !aligned16(scale_a_image) || !aligned16(scale_w_image))
    return FLYB200_E_BAD_ALIGN;
  if (M == 0) return FLYB200_OK;
  // up to 128 tokens: a weight stream, run by the small-M kernel in its block-scaled kind
  if (mx_small_m(M, N))
    return host::gemm_mx_small(c, a, w_shuf, scale_a_image, scale_w_image, M, N, K, out_dtype == FLYB200_OUT_FP16 ? 1 : 0,
                               false, stream);
  MxParams p;
  memset(&p, 0, sizeof(p));
  p.w = static_cast<const uint8_t*>(w_shuf);
  p.sfa = static_cast<const uint8_t*>(scale_a_image);
  p.sfw = static_cast<const uint8_t*>(scale_w_image);
  p.c = c;
  p.M = M;
  p.N = N;
  p.K_bytes = K;
  p.group_m = 16;
  int rc = host::status_word(&p.status);
  if (rc) return rc;
  CUtensorMap tmA;
  rc = host::byte_matrix_map(&tmA, a, static_cast<uint64_t>(K), static_cast<uint64_t>(M), BLOCK_ROWS);
  if (rc) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // FLYB200_MX_BN forces a tile shape (tuning and tests)
  bool wide = mx_wide_tiles(M, N, K);
  if (const char* e = getenv("FLYB200_MX_BN")) {
    if (e[0] == '1') wide = false;
    if (e[0] == '2' && N % 256 == 0) wide = true;
  }
  if (wide) {
    if (out_dtype == FLYB200_OUT_BF16) return launch_mx<MOE_OUT_BF16, 256>(tmA, p, s);
    return launch_mx<MOE_OUT_FP16, 256>(tmA, p, s);
  }
  if (out_dtype == FLYB200_OUT_BF16) return launch_mx<MOE_OUT_BF16, 128>(tmA, p, s);
  return launch_mx<MOE_OUT_FP16, 128>(tmA, p, s);
}

int flyb200_gemm_mx_mixed(void* c, const void* a, const void* w_shuf, const void* scale_a_image, const void* scale_w_image,
                          int M, int N, int K, int a_format, int w_format, int out_dtype, void* stream) {
  if (!c || !a || !w_shuf || !scale_a_image || !scale_w_image || M < 0 || N <= 0 || K <= 0) return FLYB200_E_BAD_ARG;
  if (out_dtype != FLYB200_OUT_BF16 && out_dtype != FLYB200_OUT_FP16) return FLYB200_E_BAD_ARG;
  auto known = [](int f) { return f == FLYB200_MXFMT_E4M3 || f == FLYB200_MXFMT_E5M2 || f == FLYB200_MXFMT_E2M3 ||
                                  f == FLYB200_MXFMT_E3M2 || f == FLYB200_MXFMT_E2M1; };
  if (!known(a_format) || !known(w_format)) return FLYB200_E_BAD_ARG;
  if (K % KBLOCK_BYTES != 0 || N % 128 != 0) return FLYB200_E_UNSUPPORTED;
  if (!aligned16(c) || !aligned16(a) || !aligned16(w_shuf) || !aligned16(scale_a_image) || !aligned16(scale_w_image))
    return FLYB200_E_BAD_ALIGN;
  if (M == 0) return FLYB200_OK;
  MxParams p;
  memset(&p, 0, sizeof(p));
  p.w = static_cast<const uint8_t*>(w_shuf);
  p.sfa = static_cast<const uint8_t*>(scale_a_image);
  p.sfw = static_cast<const uint8_t*>(scale_w_image);
  p.c = c;
  p.M = M;
  p.N = N;
  p.K_bytes = K;  // one byte per code: sub-byte codes travel in byte containers
  p.group_m = 16;
  p.fmt_bits = (static_cast<uint32_t>(a_format) << 7) | (static_cast<uint32_t>(w_format) << 10);
  int rc = host::status_word(&p.status);
  if (rc) return rc;
  CUtensorMap tmA;
  rc = host::byte_matrix_map(&tmA, a, static_cast<uint64_t>(K), static_cast<uint64_t>(M), BLOCK_ROWS);
  if (rc) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool wide = mx_wide_tiles(M, N, K);  // byte containers: K bytes per row
  if (wide) {
    if (out_dtype == FLYB200_OUT_BF16) return launch_mx<MOE_OUT_BF16, 256>(tmA, p, s);
    return launch_mx<MOE_OUT_FP16, 256>(tmA, p, s);
  }
  if (out_dtype == FLYB200_OUT_BF16) return launch_mx<MOE_OUT_BF16, 128>(tmA, p, s);
  return launch_mx<MOE_OUT_FP16, 128>(tmA, p, s);
}

int flyb200_gemm_mxfp4(void* c, const void* a, const void* w_shuf, const void* scale_a_image, const void* scale_w_image,
                       int M, int N, int K, int out_dtype, void* stream) {
  if (!c || !a || !w_shuf || !scale_a_image || !scale_w_image || M < 0 || N <= 0 || K <= 0) return FLYB200_E_BAD_ARG;
  if (out_dtype != FLYB200_OUT_BF16 && out_dtype != FLYB200_OUT_FP16) return FLYB200_E_BAD_ARG;
  if (K % (2 * KBLOCK_BYTES) != 0 || N % 128 != 0) return FLYB200_E_UNSUPPORTED;  // whole 128-byte k-blocks of packed codes
  if (!aligned16(c) || !aligned16(a) || !aligned16(w_shuf) || !aligned16(scale_a_image) || !aligned16(scale_w_image))
    return FLYB200_E_BAD_ALIGN;
  if (M == 0) return FLYB200_OK;
  // up to 128 tokens: a weight stream (half the bytes of 8-bit codes), run by the small-M kernel
  if (mx_small_m(M, N))
    return host::gemm_mx_small(c, a, w_shuf, scale_a_image, scale_w_image, M, N, K / 2,
                               out_dtype == FLYB200_OUT_FP16 ? 1 : 0, true, stream);
  MxParams p;
  memset(&p, 0, sizeof(p));
  p.w = static_cast<const uint8_t*>(w_shuf);
  p.sfa = static_cast<const uint8_t*>(scale_a_image);
  p.sfw = static_cast<const uint8_t*>(scale_w_image);
  p.c = c;
  p.M = M;
  p.N = N;
  p.K_bytes = K / 2;
  p.group_m = 16;
  int rc = host::status_word(&p.status);
  if (rc) return rc;
  CUtensorMap tmA;
  rc = host::byte_matrix_map(&tmA, a, static_cast<uint64_t>(K / 2), static_cast<uint64_t>(M), BLOCK_ROWS);
  if (rc) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  bool wide = mx_wide_tiles(M, N, K / 2);
  if (const char* e = getenv("FLYB200_MX_BN")) {
    if (e[0] == '1') wide = false;
    if (e[0] == '2' && N % 256 == 0) wide = true;
  }
  if (wide) {
    if (out_dtype == FLYB200_OUT_BF16) return launch_mx<MOE_OUT_BF16, 256, true>(tmA, p, s);
    return launch_mx<MOE_OUT_FP16, 256, true>(tmA, p, s);
  }
  if (out_dtype == FLYB200_OUT_BF16) return launch_mx<MOE_OUT_BF16, 128, true>(tmA, p, s);
  return launch_mx<MOE_OUT_FP16, 128, true>(tmA, p, s);
}

}  // extern "C"
