// Stochastic-rounding noise generated on the device with the counter layout
// of jax.random (threefry2x32), so that the noise tensor need not be produced
// on the host or by another framework and shipped over.
//
// Replaces: stochastic_rounding.JaxUniform (stochastic_rounding.py:35-46,
// jax.random.uniform(key, shape) - 0.5) and RandomCenteredUniform (:49-78,
// jax.random.bits(key, shape, uint16) placed in an f32 mantissa). jax itself is
// not part of the reference tree; its generator is restated here from the
// published algorithm (Threefry-2x32, 20 rounds, Salmon et al. 2011, and
// jax's two ways of laying counters over an array):
//   original      : counts = iota(n); first half -> x0, second half -> x1 (a
//                   zero pads an odd n); word i of the result is y0[i] for
//                   i < ceil(n/2) and y1[i - ceil(n/2)] after that;
//   partitionable : element i uses the counter pair (hi32(i), lo32(i)) and
//                   the result is y0 ^ y1.
// 16-bit draws take ceil(n/2) 32-bit words and read them as little-endian
// halves (original) or the low half of each element's word (partitionable).
#include <algorithm>

#include "common.cuh"

namespace aqtb200 {

__device__ __forceinline__ uint32_t rotl32(uint32_t x, int r) {
  return __funnelshift_l(x, x, r);
}

__device__ __forceinline__ void threefry2x32(uint32_t k0, uint32_t k1, uint32_t& x0, uint32_t& x1) {
  const uint32_t ks[3] = {k0, k1, k0 ^ k1 ^ 0x1BD11BDAu};
  x0 += ks[0];
  x1 += ks[1];
#pragma unroll
  for (int block = 0; block < 5; ++block) {
    const int r0[4] = {13, 15, 26, 6}, r1[4] = {17, 29, 16, 24};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      x0 += x1;
      x1 = rotl32(x1, (block & 1) ? r1[i] : r0[i]) ^ x0;
    }
    x0 += ks[(block + 1) % 3];
    x1 += ks[(block + 2) % 3] + (uint32_t)(block + 1);
  }
}

// 32 random bits -> uniform [0, 1) as jax.random.uniform does: the top 23 bits
// become the mantissa of a float in [1, 2), minus 1; then the shift.
__device__ __forceinline__ float bits_to_centered(uint32_t bits, float shift) {
  const float u = __fsub_rn(__uint_as_float((bits >> 9) | 0x3f800000u), 1.0f);
  return __fsub_rn(fmaxf(u, 0.f), shift);
}
// 16 random bits -> RandomCenteredUniform's grid inside (-0.5, 0.5)
__device__ __forceinline__ float bits16_to_centered(uint32_t b16) {
  return __fsub_rn(__uint_as_float((b16 << 7) | 0x3f800000u), 1.5f - 1.52587890625e-05f * 0.5f);
}

// mode 0: uniform - shift from 32-bit draws; mode 1: centered grid from 16-bit draws
template <int MODE>
__global__ void __launch_bounds__(256)
jax_noise_kernel(uint32_t k0, uint32_t k1, int64_t n, int partitionable, float shift, float* out) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (partitionable) {
    for (int64_t i = tid; i < n; i += stride) {
      uint32_t x0 = (uint32_t)((uint64_t)i >> 32), x1 = (uint32_t)i;
      threefry2x32(k0, k1, x0, x1);
      const uint32_t w = x0 ^ x1;
      out[i] = MODE == 0 ? bits_to_centered(w, shift) : bits16_to_centered(w & 0xffffu);
    }
    return;
  }
  // words = number of 32-bit draws; one threefry call yields words h and h + half
  const int64_t words = MODE == 0 ? n : (n + 1) / 2;
  const int64_t half = (words + 1) / 2;
  for (int64_t h = tid; h < half; h += stride) {
    uint32_t x0 = (uint32_t)h;
    uint32_t x1 = h + half < words ? (uint32_t)(h + half) : 0u;  // the pad of an odd count
    threefry2x32(k0, k1, x0, x1);
    if (MODE == 0) {
      out[h] = bits_to_centered(x0, shift);
      if (h + half < words) out[h + half] = bits_to_centered(x1, shift);
    } else {
      const int64_t e0 = 2 * h, e1 = 2 * (h + half);
      if (e0 < n) out[e0] = bits16_to_centered(x0 & 0xffffu);
      if (e0 + 1 < n) out[e0 + 1] = bits16_to_centered(x0 >> 16);
      if (h + half < words) {
        if (e1 < n) out[e1] = bits16_to_centered(x1 & 0xffffu);
        if (e1 + 1 < n) out[e1 + 1] = bits16_to_centered(x1 >> 16);
      }
    }
  }
}

int sm_count();

}  // namespace aqtb200

extern "C" int aqtb200_jax_noise(uint32_t key0, uint32_t key1, int64_t n, int32_t kind,
                                 int32_t partitionable, float shift, float* out, void* stream) {
  using namespace aqtb200;
  AQT_REQUIRE(n >= 0 && (n == 0 || out != nullptr), AQTB200_EINVAL, "null output");
  AQT_REQUIRE(kind == 0 || kind == 1, AQTB200_EINVAL, "kind must be 0 (uniform) or 1 (centered 16-bit)");
  AQT_REQUIRE(n < ((int64_t)1 << 32), AQTB200_EUNSUPPORTED,
              "more than 2^32 - 1 elements: jax's counter layout switches to blocks");
  if (n == 0) return 0;
  const int64_t work = partitionable ? n : (n + 1) / 2;
  const int grid = (int)std::max<int64_t>(1, std::min<int64_t>((work + 255) / 256, (int64_t)sm_count() * 16));
  if (kind == 0)
    jax_noise_kernel<0><<<grid, 256, 0, (cudaStream_t)stream>>>(key0, key1, n, partitionable, shift, out);
  else
    jax_noise_kernel<1><<<grid, 256, 0, (cudaStream_t)stream>>>(key0, key1, n, partitionable, shift, out);
  AQT_CUDA_OK(cudaGetLastError());
  count_launch();
  return 0;
}
