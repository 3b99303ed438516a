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
// One 256-thread block per row, 16-byte loads, 4..8-byte stores.  Rows of up to
// 8192 (fp32) / 16384 (16-bit) elements stay in registers between the maximum
// and the conversion and are read from memory once; longer rows are read twice
// (the second time from L1/L2).
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

// Four finite values -> four packed bytes, bit-identical to four quant_one calls
// but normally without the IEEE divisions.  q' = v * rcp(s) differs from the
// correctly rounded quotient q = v / s by at most 2.5 ulp, so converting q'
// gives the same byte unless a rounding boundary of the target type lies
// within 3 ulp of q': for e4m3 the midpoints between neighbouring values (low
// 20 mantissa bits == 0x80000) and, conservatively, everything below 2^-5
// (subnormal spacing); for int8 (truncation) the integers.  If any of the four
// is that close to a boundary, all four take the exact route.
template <bool FP8>
__device__ __forceinline__ uint32_t quant_four(const float* v, float s, float inv_s) {
  float q[4];
  bool risky = false;
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    q[e] = v[e] * inv_s;
    if constexpr (FP8) {
      const uint32_t b = __float_as_uint(q[e]);
      const uint32_t mag = b & 0x7FFFFFFFu;
      risky |= ((b & 0xFFFFFu) - (0x80000u - 3u)) <= 6u;
      risky |= (mag < 0x3D000000u) && (mag != 0u);
    } else {
      risky |= (fabsf(q[e] - rintf(q[e])) < 6.2e-5f) && (q[e] != 0.0f);
    }
  }
  if (risky) {
    uint32_t b = 0;
#pragma unroll
    for (int e = 0; e < 4; ++e) b |= static_cast<uint32_t>(quant_one<FP8>(v[e], s)) << (8 * e);
    return b;
  }
  if constexpr (FP8) {
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(q[0], q[1]), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(q[2], q[3]), __NV_SATFINITE, __NV_E4M3);
    return lo | (hi << 16);
  } else {
    uint32_t b = 0;
#pragma unroll
    for (int e = 0; e < 4; ++e) b |= (static_cast<uint32_t>(__float2int_rz(q[e])) & 0xFFu) << (8 * e);
    return b;
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
  // Row maximum on the bit patterns: for finite floats the order of |x| is the
  // order of (bits & 0x7fffffff) as unsigned integers, and any Inf / NaN in the
  // row shows up as a maximum >= 0x7f800000, which sends the whole row down the
  // careful path below.  (The kernel is instruction-bound, not memory-bound, for
  // 16-bit inputs: every instruction per element counts.)
  uint32_t bmax = 0u;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
#pragma unroll
    for (int e = 0; e < VEC; ++e) bmax = max(bmax, __float_as_uint(v[i][e]) & 0x7FFFFFFFu);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) bmax = max(bmax, __shfl_xor_sync(0xffffffffu, bmax, o));
  if (lane == 0) warp_max[warp] = __uint_as_float(bmax);
  __syncthreads();
  uint32_t mb = __float_as_uint(warp_max[lane & 7]);
#pragma unroll
  for (int o = 4; o > 0; o >>= 1) mb = max(mb, __shfl_xor_sync(0xffffffffu, mb, o));
  uint8_t* yr = y + static_cast<size_t>(r) * K;

  if (mb >= 0x7F800000u) {
    // ---- careful path: the row holds Inf or NaN (block-uniform branch) ----
    __syncthreads();  // warp_max is reused
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
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int k = (i * 256 + threadIdx.x) * VEC;
      if (k < K) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) yr[k + e] = quant_one<FP8>(v[i][e], s);
      }
    }
    return;
  }

  // ---- fast path: all finite ----
  float s = __fmul_rn(__uint_as_float(mb), __fdiv_rn(1.0f, QMAX));
  if (s == 0.0f) s = 1.0f;
  if (threadIdx.x == 0) scale[r] = s;
  const float inv_s = __frcp_rn(s);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int k = (i * 256 + threadIdx.x) * VEC;
    if (k < K) {
      uint32_t packed[VEC / 4];
#pragma unroll
      for (int w = 0; w < VEC / 4; ++w) packed[w] = quant_four<FP8>(&v[i][4 * w], s, inv_s);
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
