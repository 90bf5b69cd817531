// Shared device/host helpers for the aqt_b200 kernels (sm_100a).
//
// Rounding discipline. The reference computes in eager jax semantics: every
// elementwise op rounds to its result dtype. Here every value of dtype T in
// {f32, bf16} is carried in a float register that holds a T-representable
// number, and each op is written with the non-contracting intrinsics
// (__fmul_rn, __fadd_rn, __fdiv_rn) followed by an explicit rounding to the
// result dtype, so nvcc can never fuse a multiply and an add into an FMA.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/aqt_b200.h"

namespace aqtb200 {

void set_error(const char* fmt, ...);
void count_launch(int n = 1);

#define AQT_CUDA_OK(expr)                                                   \
  do {                                                                      \
    cudaError_t e_ = (expr);                                                \
    if (e_ != cudaSuccess) {                                                \
      ::aqtb200::set_error("%s failed: %s (%s:%d)", #expr,                  \
                           cudaGetErrorString(e_), __FILE__, __LINE__);     \
      return (int)e_;                                                       \
    }                                                                       \
  } while (0)

#define AQT_REQUIRE(cond, code, ...)          \
  do {                                        \
    if (!(cond)) {                            \
      ::aqtb200::set_error(__VA_ARGS__);      \
      return (code);                          \
    }                                         \
  } while (0)

__host__ __device__ inline int dtype_size(int dt) {
  switch (dt) {
    case AQTB200_F32: case AQTB200_S32: return 4;
    case AQTB200_BF16: return 2;
    default: return 1;
  }
}

__device__ __forceinline__ float round_bf16(float v) {
  return __bfloat162float(__float2bfloat16_rn(v));
}
// Rounds v to dtype dt (F32: identity, BF16: RNE to 8 significant bits).
__device__ __forceinline__ float round_to(float v, int dt) {
  return dt == AQTB200_BF16 ? round_bf16(v) : v;
}

__device__ __forceinline__ float fp8_to_float(uint8_t b, int dt) {
  __half_raw h = __nv_cvt_fp8_to_halfraw(
      (__nv_fp8_storage_t)b, dt == AQTB200_E4M3 ? __NV_E4M3 : __NV_E5M2);
  return __half2float(__half(h));
}

// One element of `base` (dtype dt) at element index idx, widened exactly.
__device__ __forceinline__ float load1(const void* base, int dt, int64_t idx) {
  switch (dt) {
    case AQTB200_F32: return __ldg((const float*)base + idx);
    case AQTB200_BF16:
      return __bfloat162float(
          __ushort_as_bfloat16(__ldg((const unsigned short*)base + idx)));
    case AQTB200_S8: return (float)__ldg((const signed char*)base + idx);
    case AQTB200_S32: return (float)__ldg((const int*)base + idx);
    default: return fp8_to_float(__ldg((const uint8_t*)base + idx), dt);
  }
}

__device__ __forceinline__ float bf16lo(uint32_t w) {
  return __uint_as_float(w << 16);
}
__device__ __forceinline__ float bf16hi(uint32_t w) {
  return __uint_as_float(w & 0xffff0000u);
}

// N (4, 8 or 16) consecutive elements starting at idx; idx*size must be
// 16-byte aligned relative to a 16-byte aligned base (N*size >= 16) or
// naturally aligned for the narrower cases.
template <int N>
__device__ __forceinline__ void loadN(const void* base, int dt, int64_t idx,
                                      float* v) {
  if (dt == AQTB200_F32) {
    const float4* p = (const float4*)((const float*)base + idx);
#pragma unroll
    for (int i = 0; i < N / 4; ++i) {
      float4 f = __ldg(p + i);
      v[4 * i] = f.x; v[4 * i + 1] = f.y; v[4 * i + 2] = f.z; v[4 * i + 3] = f.w;
    }
  } else if (dt == AQTB200_BF16) {
    if constexpr (N >= 8) {
      const uint4* p = (const uint4*)((const unsigned short*)base + idx);
#pragma unroll
      for (int i = 0; i < N / 8; ++i) {
        uint4 u = __ldg(p + i);
        v[8 * i] = bf16lo(u.x); v[8 * i + 1] = bf16hi(u.x);
        v[8 * i + 2] = bf16lo(u.y); v[8 * i + 3] = bf16hi(u.y);
        v[8 * i + 4] = bf16lo(u.z); v[8 * i + 5] = bf16hi(u.z);
        v[8 * i + 6] = bf16lo(u.w); v[8 * i + 7] = bf16hi(u.w);
      }
    } else {
      uint2 u = __ldg((const uint2*)((const unsigned short*)base + idx));
      v[0] = bf16lo(u.x); v[1] = bf16hi(u.x);
      v[2] = bf16lo(u.y); v[3] = bf16hi(u.y);
    }
  } else {
    uint8_t b[N];
    if constexpr (N == 16) {
      *(uint4*)b = __ldg((const uint4*)((const uint8_t*)base + idx));
    } else if constexpr (N == 8) {
      *(uint2*)b = __ldg((const uint2*)((const uint8_t*)base + idx));
    } else {
      *(uint32_t*)b = __ldg((const uint32_t*)((const uint8_t*)base + idx));
    }
#pragma unroll
    for (int i = 0; i < N; ++i) {
      v[i] = dt == AQTB200_S8 ? (float)(signed char)b[i] : fp8_to_float(b[i], dt);
    }
  }
}

// Non-negative floats order like their bit patterns, so an unsigned atomicMax
// on the bits is a float max. The cell must start at 0 (= +0.0f).
__device__ __forceinline__ void atomic_max_nonneg(uint32_t* cell, float v) {
  atomicMax(cell, __float_as_uint(v));
}

// Maximum of two NON-NEGATIVE floats through their bit patterns. Unlike fmaxf
// it keeps a NaN (whose pattern, sign cleared, ranks above infinity), which is
// what jnp.max(jnp.abs(x)) does: one NaN in the reduced range gives a NaN
// maximum and so a NaN scale (calibration.py:149).
__device__ __forceinline__ float amax_nn(float a, float b) {
  return __uint_as_float(max(__float_as_uint(a), __float_as_uint(b)));
}

// warp-wide maximum of non-negative floats (NaN-keeping, see amax_nn)
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = amax_nn(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

}  // namespace aqtb200
