// Host helpers shared by the translation units of libflyb200 (not part of the C ABI).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace flyb200 {
namespace host {

// Tensor map over a row-major byte matrix [rows, row_bytes]: boxes of
// 128 bytes x box_rows rows, 128-byte swizzle, out-of-bounds rows read as zero.
int byte_matrix_map(CUtensorMap* m, const void* base, uint64_t row_bytes, uint64_t rows, uint32_t box_rows);
// Block-scaled GEMM (MXFP8, or MXFP4 with `fp4`) of up to 128 tokens on the small-M (weight-streaming)
// kernel; K = bytes of codes per row; outmode 0 bf16, 1 fp16.
int gemm_mx_small(void* c, const void* a, const void* w, const void* sf_a, const void* sf_w, int M, int N, int K,
                  int outmode, bool fp4, void* stream);
// Pointer to the current device's status word (first failed bounded wait wins).
int status_word(int** out);
// SM count of the current device.
int sm_count(int* out);
// Remember a CUDA error for flyb200_last_cuda_error(); returns FLYB200_E_CUDA.
int record_cuda_error(cudaError_t e, const char* what);

}  // namespace host
}  // namespace flyb200
