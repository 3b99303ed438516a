// Per-token (per-row) symmetric quantisation fp32/fp16/bf16 -> fp8 e4m3 / int8
// with one fp32 scale per row: the step that feeds the GEMM's A operand.
//
//   h     = x with NaN -> 0, +Inf -> qmax, -Inf -> -qmax
//   scale = max_k |h[k]| * (1 / qmax), 0 -> 1      (qmax = 448 or 127)
//   y[k]  = convert(h[k] / scale)                  fp8: round to nearest even,
//                                                  int8: truncate toward zero
//
// The arithmetic follows what the torch statement of the reference helper
// computes on a GPU, operation by operation, so results are bit-identical to
// it: the division of the row maximum by the Python scalar qmax is executed by
// torch's CUDA backend as a multiplication by the fp32 reciprocal, the
// element-wise division is a true IEEE division.
//
// HBM-bound: one 256-thread block per row, two passes over the row (the second
// one hits L1/L2), 16-byte loads, 4..8-byte stores.
#pragma once
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

namespace flyb200 {

enum : int { QX_F32 = 0, QX_F16 = 1, QX_BF16 = 2 };

template <typename T>
struct QuantIn;
template <>
struct QuantIn<float> {
  static constexpr int VEC = 4;  // elements per 16-byte load
  __device__ static void load(const float* p, float (&v)[4]) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x, v[1] = t.y, v[2] = t.z, v[3] = t.w;
  }
};
template <>
struct QuantIn<__half> {
  static constexpr int VEC = 8;
  __device__ static void load(const __half* p, float (&v)[8]) {
    const uint4 t = *reinterpret_cast<const uint4*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&t);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(h[i]);
      v[2 * i] = f.x, v[2 * i + 1] = f.y;
    }
  }
};
template <>
struct QuantIn<__nv_bfloat16> {
  static constexpr int VEC = 8;
  __device__ static void load(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 t = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&t);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      v[2 * i] = f.x, v[2 * i + 1] = f.y;
    }
  }
};

__device__ __forceinline__ float scrub(float v, float qmax) {
  if (v != v) return 0.0f;
  if (v == INFINITY) return qmax;
  if (v == -INFINITY) return -qmax;
  return v;
}

template <bool FP8>
__device__ __forceinline__ uint8_t quant_one(float v, float s) {
  const float q = __fdiv_rn(v, s);
  if constexpr (FP8) {
    return static_cast<uint8_t>(__nv_cvt_float_to_fp8(q, __NV_SATFINITE, __NV_E4M3));
  } else {
    return static_cast<uint8_t>(static_cast<int8_t>(__float2int_rz(q)));
  }
}

// Single-pass form for rows of at most 256 * VEC * NV elements: every thread
// keeps its NV vectors of the row in registers between the maximum and the
// conversion, so the row is read from memory exactly once and all of a
// thread's loads are in flight together.  One block per row.
template <typename TIn, bool FP8, int NV>
__global__ void __launch_bounds__(256) pertoken_quant_row_kernel(uint8_t* __restrict__ y, float* __restrict__ scale,
                                                                 const TIn* __restrict__ x, int rows, int K) {
  constexpr int VEC = QuantIn<TIn>::VEC;
  constexpr float QMAX = FP8 ? 448.0f : 127.0f;
  __shared__ float warp_max[8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int r = blockIdx.x;
  if (r >= rows) return;
  const TIn* xr = x + static_cast<size_t>(r) * K;
  float v[NV][VEC];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int k = (i * 256 + threadIdx.x) * VEC;
    if (k < K) {
      QuantIn<TIn>::load(xr + k, v[i]);
    } else {
#pragma unroll
      for (int e = 0; e < VEC; ++e) v[i][e] = 0.0f;
    }
  }
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      v[i][e] = scrub(v[i][e], QMAX);
      amax = fmaxf(amax, fabsf(v[i][e]));
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if (lane == 0) warp_max[warp] = amax;
  __syncthreads();
  float m = warp_max[lane & 7];
#pragma unroll
  for (int o = 4; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  float s = __fmul_rn(m, __fdiv_rn(1.0f, QMAX));
  if (s == 0.0f) s = 1.0f;
  if (threadIdx.x == 0) scale[r] = s;
  uint8_t* yr = y + static_cast<size_t>(r) * K;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int k = (i * 256 + threadIdx.x) * VEC;
    if (k < K) {
      uint32_t packed[VEC / 4];
#pragma unroll
      for (int w = 0; w < VEC / 4; ++w) {
        uint32_t b = 0;
#pragma unroll
        for (int e = 0; e < 4; ++e) b |= static_cast<uint32_t>(quant_one<FP8>(v[i][4 * w + e], s)) << (8 * e);
        packed[w] = b;
      }
      if constexpr (VEC == 4) {
        *reinterpret_cast<uint32_t*>(yr + k) = packed[0];
      } else {
        *reinterpret_cast<uint2*>(yr + k) = make_uint2(packed[0], packed[1]);
      }
    }
  }
}

// General form (any row length): two passes over the row, the second one from L1/L2.
template <typename TIn, bool FP8>
__global__ void __launch_bounds__(256) pertoken_quant_kernel(uint8_t* __restrict__ y, float* __restrict__ scale,
                                                             const TIn* __restrict__ x, int rows, int K) {
  constexpr int VEC = QuantIn<TIn>::VEC;
  constexpr float QMAX = FP8 ? 448.0f : 127.0f;
  __shared__ float warp_max[8];
  __shared__ float row_scale;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    const TIn* xr = x + static_cast<size_t>(r) * K;
    float amax = 0.0f;
    for (int k = threadIdx.x * VEC; k < K; k += 256 * VEC) {
      float v[VEC];
      QuantIn<TIn>::load(xr + k, v);
#pragma unroll
      for (int i = 0; i < VEC; ++i) amax = fmaxf(amax, fabsf(scrub(v[i], QMAX)));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (lane == 0) warp_max[warp] = amax;
    __syncthreads();
    if (warp == 0) {
      float m = lane < 8 ? warp_max[lane] : 0.0f;
#pragma unroll
      for (int o = 4; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
      if (lane == 0) {
        float s = __fmul_rn(m, __fdiv_rn(1.0f, QMAX));
        if (s == 0.0f) s = 1.0f;
        row_scale = s;
        scale[r] = s;
      }
    }
    __syncthreads();
    const float s = row_scale;
    uint8_t* yr = y + static_cast<size_t>(r) * K;
    for (int k = threadIdx.x * VEC; k < K; k += 256 * VEC) {
      float v[VEC];
      QuantIn<TIn>::load(xr + k, v);
      uint32_t packed[VEC / 4];
#pragma unroll
      for (int w = 0; w < VEC / 4; ++w) {
        uint32_t b = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) b |= static_cast<uint32_t>(quant_one<FP8>(scrub(v[4 * w + i], QMAX), s)) << (8 * i);
        packed[w] = b;
      }
      if constexpr (VEC == 4) {
        *reinterpret_cast<uint32_t*>(yr + k) = packed[0];
      } else {
        *reinterpret_cast<uint2*>(yr + k) = make_uint2(packed[0], packed[1]);
      }
    }
    __syncthreads();  // row_scale / warp_max are reused by the next row
  }
}

}  // namespace flyb200
