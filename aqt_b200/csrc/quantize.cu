// AbsMax calibration and quantization kernels (HBM-bound, CUDA cores).
//
// Three steps per operand, each a grid-stride kernel sized to the SM count:
//   1. absmax_{row,col}_kernel : max |v| per kept row (or per tensor) into a
//      zero-initialised uint32 cell per scale via atomicMax on float bits;
//   2. finalize_scale_kernel   : amax -> scale (reference dtype semantics) and
//      its rounded reciprocal;
//   3. quant_{row,col}_kernel  : v * (1/scale) [+noise] -> clip -> round ->
//      int8 / fp8, written with the contraction index contiguous.
// "row" kernels read inputs whose contraction index is contiguous; "col"
// kernels read inputs whose kept index is contiguous and transpose a 64x128
// tile through shared memory so the output is contraction-contiguous as well.
#include <algorithm>
#include <mutex>

#include "common.cuh"

namespace aqtb200 {

struct DView {
  const void* ptr;
  int dtype;
  int64_t b0, b1, rows, cols;
  int64_t sb0, sb1, sr, sc;
};

struct QParams {
  DView x, pre, noise;  // pre.ptr / noise.ptr null when absent
  int t_dtype, s_dtype, y_dtype;
  int kind, qdtype;
  float clip_bound;
  int per_tensor;
  int pre_vec, noise_vec;  // vector loads allowed on prescale / noise
  int use_lut;    // 1-byte input, one scale and one prescale for the whole call: byte -> byte table
  int fast_bf16;  // bf16 in, bf16 scale, fp8 out, no noise: packed bf16 arithmetic
  int pre_bf16;   // bf16 input, bf16 prescale, bf16 compute dtype: x * pre as packed bf16 multiplies
  int int_bf16;   // bf16 in, bf16 scale and prescale, int8 out (with or without noise): packed bf16 arithmetic
  int s8_bf16;    // int8 in (a stored QTensor counted as bf16), bf16 scale and prescale, int8 out: the same arithmetic
  uint32_t* amax;
  float* sinv;
  uint8_t* q;
  int64_t ldq;
};

static DView to_dview(const aqtb200_view* v) {
  DView d{};
  if (v == nullptr || v->ptr == nullptr) return d;
  d.ptr = v->ptr; d.dtype = v->dtype;
  d.b0 = v->b0; d.b1 = v->b1; d.rows = v->rows; d.cols = v->cols;
  d.sb0 = v->b0_stride; d.sb1 = v->b1_stride;
  d.sr = v->row_stride; d.sc = v->col_stride;
  return d;
}

// v = round_T(x * round_T(pre))
__device__ __forceinline__ float apply_pre(float x, float pre, int t_dtype) {
  return round_to(__fmul_rn(x, round_to(pre, t_dtype)), t_dtype);
}

__device__ __forceinline__ uint8_t quant1(float v, float sinv, float noise,
                                          bool has_noise, const QParams& P) {
  float y = round_to(__fmul_rn(v, sinv), P.y_dtype);
  if (has_noise) y = round_to(__fadd_rn(y, noise), P.y_dtype);
  y = fminf(fmaxf(y, -P.clip_bound), P.clip_bound);
  if (P.kind == AQTB200_NUM_INT) {
    return (uint8_t)(signed char)__float2int_rn(y);  // rn = ties to even
  }
  return (uint8_t)__nv_cvt_float_to_fp8(
      y, __NV_SATFINITE, P.qdtype == AQTB200_E4M3 ? __NV_E4M3 : __NV_E5M2);
}

__device__ __forceinline__ void decode_brow(const DView& x, int64_t brow,
                                            int64_t& i0, int64_t& i1,
                                            int64_t& r) {
  r = brow % x.rows;
  int64_t b = brow / x.rows;
  i1 = b % x.b1;
  i0 = b / x.b1;
}

__device__ __forceinline__ float block_max(float v, float* red) {
  v = warp_max(v);
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  int nw = (blockDim.x * blockDim.y + 31) >> 5;
  v = (threadIdx.x < nw && threadIdx.y == 0) ? red[threadIdx.x] : 0.f;
  if (warp == 0 && threadIdx.y == 0) v = warp_max(v);
  return v;
}

// ---------------------------------------------------------------------------
// absmax, contraction contiguous. One warp per (batch-row, 4096-column chunk).
constexpr int kRowChunk = 4096;

template <bool VEC>
__global__ void __launch_bounds__(256)
absmax_row_kernel(QParams P, int64_t chunks_per_row, int64_t total_units) {
  __shared__ float red[32];
  const int lane = threadIdx.x & 31;
  const int64_t warp_g = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * (blockDim.x >> 5);
  const DView& x = P.x;
  const bool has_pre = P.pre.ptr != nullptr;
  float tmax = 0.f;
  for (int64_t u = warp_g; u < total_units; u += nwarps) {
    int64_t brow = u / chunks_per_row, chunk = u % chunks_per_row;
    int64_t i0, i1, r;
    decode_brow(x, brow, i0, i1, r);
    const int64_t base = i0 * x.sb0 + i1 * x.sb1 + r * x.sr;
    const int64_t pbase = i0 * P.pre.sb0 + i1 * P.pre.sb1;
    const int64_t c0 = chunk * kRowChunk;
    const int64_t c1 = min(x.cols, c0 + (int64_t)kRowChunk);
    float m = 0.f;
    if (VEC) {
      for (int64_t c = c0 + lane * 16; c < c1; c += 32 * 16) {
        float v[16];
        loadN<16>(x.ptr, x.dtype, base + c, v);
        if (has_pre) {
          float p[16];
          if (P.pre_vec) {
            loadN<16>(P.pre.ptr, P.pre.dtype, pbase + c, p);
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              p[j] = load1(P.pre.ptr, P.pre.dtype, pbase + (c + j) * P.pre.sc);
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = apply_pre(v[j], p[j], P.t_dtype);
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) m = amax_nn(m, fabsf(v[j]));
      }
    } else {
      for (int64_t c = c0 + lane; c < c1; c += 32) {
        float v = load1(x.ptr, x.dtype, base + c * x.sc);
        if (has_pre)
          v = apply_pre(v, load1(P.pre.ptr, P.pre.dtype, pbase + c * P.pre.sc),
                        P.t_dtype);
        m = amax_nn(m, fabsf(v));
      }
    }
    if (P.per_tensor) {
      tmax = amax_nn(tmax, m);
    } else {
      m = warp_max(m);
      if (lane == 0 && m != 0.f) atomic_max_nonneg(P.amax + brow, m);
    }
  }
  if (P.per_tensor) {
    tmax = block_max(tmax, red);
    if (threadIdx.x == 0 && tmax != 0.f) atomic_max_nonneg(P.amax, tmax);
  }
}

// ---------------------------------------------------------------------------
// absmax, kept index contiguous. Block (32 x 8): x covers 32*V kept rows, y
// strides over a 256-wide chunk of the contraction index.
constexpr int kColChunk = 256;

template <bool VEC>
__global__ void __launch_bounds__(256)
absmax_col_kernel(QParams P, int64_t row_blocks, int64_t col_chunks,
                  int64_t total_units) {
  constexpr int V = VEC ? 4 : 1;
  __shared__ float red[32];
  const DView& x = P.x;
  const bool has_pre = P.pre.ptr != nullptr;
  const int tx = threadIdx.x, ty = threadIdx.y;
  float tmax = 0.f;
  for (int64_t u = blockIdx.x; u < total_units; u += gridDim.x) {
    int64_t cc = u % col_chunks;
    int64_t t = u / col_chunks;
    int64_t rb = t % row_blocks;
    int64_t b = t / row_blocks;
    int64_t i1 = b % x.b1, i0 = b / x.b1;
    const int64_t r0 = (rb * 32 + tx) * V;
    const int64_t base = i0 * x.sb0 + i1 * x.sb1;
    const int64_t pbase = i0 * P.pre.sb0 + i1 * P.pre.sb1;
    const int64_t cend = min(x.cols, (cc + 1) * (int64_t)kColChunk);
    float m[V];
#pragma unroll
    for (int j = 0; j < V; ++j) m[j] = 0.f;
    if (r0 < x.rows) {
      for (int64_t c = cc * kColChunk + ty; c < cend; c += 8) {
        float v[V];
        if (VEC) {
          loadN<4>(x.ptr, x.dtype, base + c * x.sc + r0, v);
        } else {
          v[0] = load1(x.ptr, x.dtype, base + c * x.sc + r0 * x.sr);
        }
        float p = has_pre ? load1(P.pre.ptr, P.pre.dtype, pbase + c * P.pre.sc) : 0.f;
#pragma unroll
        for (int j = 0; j < V; ++j) {
          float w = has_pre ? apply_pre(v[j], p, P.t_dtype) : v[j];
          m[j] = amax_nn(m[j], fabsf(w));
        }
      }
    }
    if (P.per_tensor) {
#pragma unroll
      for (int j = 0; j < V; ++j) tmax = amax_nn(tmax, m[j]);
    } else if (r0 < x.rows) {
      const int64_t sbase = (i0 * x.b1 + i1) * x.rows;
#pragma unroll
      for (int j = 0; j < V; ++j)
        if (r0 + j < x.rows && m[j] != 0.f)
          atomic_max_nonneg(P.amax + sbase + r0 + j, m[j]);
    }
  }
  if (P.per_tensor) {
    // fold the 8 y-lanes through warp ids: thread linear id = ty*32 + tx
    float v = warp_max(tmax);
    if (tx == 0) red[ty] = v;
    __syncthreads();
    if (ty == 0) {
      v = tx < 8 ? red[tx] : 0.f;
      v = warp_max(v);
      if (tx == 0 && v != 0.f) atomic_max_nonneg(P.amax, v);
    }
  }
}


// ===========================================================================
// Fast paths: 16-byte vector loads, several independent loads in flight per
// thread, branch-free inner loops. EPV = elements per 16-byte vector of the
// INPUT: 4 (f32), 8 (bf16), 16 (int8 / fp8).

__device__ __forceinline__ uint4 ldg16(const void* base, int64_t byte_off) {
  return __ldg((const uint4*)((const char*)base + byte_off));
}

template <int EPV>
__device__ __forceinline__ void unpack(const uint4& raw, int dt, float* v) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  if constexpr (EPV == 4) {
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = __uint_as_float(w[i]);
  } else if constexpr (EPV == 8) {
#pragma unroll
    for (int i = 0; i < 4; ++i) { v[2 * i] = bf16lo(w[i]); v[2 * i + 1] = bf16hi(w[i]); }
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const uint32_t b = (w[i >> 2] >> (8 * (i & 3))) & 0xffu;
      v[i] = dt == AQTB200_S8 ? (float)(signed char)b : fp8_to_float((uint8_t)b, dt);
    }
  }
}

// Running |x| maximum kept in the input's own packed format: magnitudes of
// non-negative floats (any width) order like unsigned integers.
template <int EPV>
__device__ __forceinline__ void packed_absmax(uint4& run, const uint4& raw, int dt) {
  if constexpr (EPV == 4) {
    run.x = max(run.x, raw.x & 0x7fffffffu); run.y = max(run.y, raw.y & 0x7fffffffu);
    run.z = max(run.z, raw.z & 0x7fffffffu); run.w = max(run.w, raw.w & 0x7fffffffu);
  } else if constexpr (EPV == 8) {
    run.x = __vmaxu2(run.x, raw.x & 0x7fff7fffu); run.y = __vmaxu2(run.y, raw.y & 0x7fff7fffu);
    run.z = __vmaxu2(run.z, raw.z & 0x7fff7fffu); run.w = __vmaxu2(run.w, raw.w & 0x7fff7fffu);
  } else if (dt == AQTB200_S8) {
    run.x = __vmaxu4(run.x, __vabsss4(raw.x)); run.y = __vmaxu4(run.y, __vabsss4(raw.y));
    run.z = __vmaxu4(run.z, __vabsss4(raw.z)); run.w = __vmaxu4(run.w, __vabsss4(raw.w));
  } else {
    run.x = __vmaxu4(run.x, raw.x & 0x7f7f7f7fu); run.y = __vmaxu4(run.y, raw.y & 0x7f7f7f7fu);
    run.z = __vmaxu4(run.z, raw.z & 0x7f7f7f7fu); run.w = __vmaxu4(run.w, raw.w & 0x7f7f7f7fu);
  }
}

// The packed running maximum as EPV non-negative floats (one per lane slot).
template <int EPV>
__device__ __forceinline__ void packed_to_floats(const uint4& run, int dt, float* v) {
  if constexpr (EPV == 16) {
    const uint32_t w[4] = {run.x, run.y, run.z, run.w};
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const uint32_t b = (w[i >> 2] >> (8 * (i & 3))) & 0xffu;
      v[i] = dt == AQTB200_S8 ? (float)b : fp8_to_float((uint8_t)b, dt);
    }
  } else {
    unpack<EPV>(run, dt, v);
  }
}

template <int EPV>
__device__ __forceinline__ float packed_hmax(const uint4& run, int dt) {
  float v[EPV];
  packed_to_floats<EPV>(run, dt, v);
  float m = 0.f;
#pragma unroll
  for (int i = 0; i < EPV; ++i) m = amax_nn(m, v[i]);
  return m;
}

// |round_T(x * round_T(p))| for x >= 0 is monotone in x, so a prescale that is
// constant over the reduced range can be applied to the maximum afterwards.
__device__ __forceinline__ float apply_pre_abs(float amax, float pre, int t_dtype) {
  return fabsf(apply_pre(amax, pre, t_dtype));
}

// 4 quantized values -> one little-endian word.
__device__ __forceinline__ uint32_t quant4(const float* v, const float* sinv, const float* nz,
                                           bool has_noise, const QParams& P) {
  float y[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    y[j] = round_to(__fmul_rn(v[j], sinv[j]), P.y_dtype);
    if (has_noise) y[j] = round_to(__fadd_rn(y[j], nz[j]), P.y_dtype);
  }
  if (P.kind == AQTB200_NUM_INT) {
    uint32_t w = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float c = fminf(fmaxf(y[j], -P.clip_bound), P.clip_bound);
      w |= ((uint32_t)__float2int_rn(c) & 0xffu) << (8 * j);
    }
    return w;
  }
  // fp8: the saturating convert clamps to +-max finite, which is the clip bound.
  const __nv_fp8_interpretation_t k = P.qdtype == AQTB200_E4M3 ? __NV_E4M3 : __NV_E5M2;
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(y[0], y[1]), __NV_SATFINITE, k);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(y[2], y[3]), __NV_SATFINITE, k);
  return lo | (hi << 16);
}

// 4 x 4 byte transpose: in[e] holds rows 0..3 of column e, out[j] holds
// columns 0..3 of row j.
__device__ __forceinline__ void transpose4x4(const uint32_t* in, uint32_t* out) {
  const uint32_t t0 = __byte_perm(in[0], in[1], 0x5140);  // a0 b0 a1 b1
  const uint32_t t1 = __byte_perm(in[0], in[1], 0x7362);  // a2 b2 a3 b3
  const uint32_t t2 = __byte_perm(in[2], in[3], 0x5140);  // c0 d0 c1 d1
  const uint32_t t3 = __byte_perm(in[2], in[3], 0x7362);  // c2 d2 c3 d3
  out[0] = __byte_perm(t0, t2, 0x5410);
  out[1] = __byte_perm(t0, t2, 0x7632);
  out[2] = __byte_perm(t1, t3, 0x5410);
  out[3] = __byte_perm(t1, t3, 0x7632);
}

// Requantizing a 1-byte tensor with ONE scale (and at most one prescale) is a
// fixed function of the input byte; each block tabulates it once.
__device__ __forceinline__ void build_lut(uint8_t* lut, const QParams& P, bool has_pre) {
  const int t = threadIdx.y * blockDim.x + threadIdx.x;
  if (t < 256) {
    float v = P.x.dtype == AQTB200_S8 ? (float)(signed char)t : fp8_to_float((uint8_t)t, P.x.dtype);
    if (has_pre) v = apply_pre(v, load1(P.pre.ptr, P.pre.dtype, 0), P.t_dtype);
    lut[t] = quant1(v, P.sinv[0], 0.f, false, P);
  }
  __syncthreads();
}
__device__ __forceinline__ uint32_t lut4(uint32_t w, const uint8_t* lut) {
  return (uint32_t)lut[w & 0xffu] | ((uint32_t)lut[(w >> 8) & 0xffu] << 8) |
         ((uint32_t)lut[(w >> 16) & 0xffu] << 16) | ((uint32_t)lut[w >> 24] << 24);
}

// Two bf16 values (one raw word) -> two fp8 bytes, all arithmetic in packed
// bf16: round_bf16(x * pre) then round_bf16(. * sinv), then the saturating
// RNE convert. A bf16 product is exact in f32, so the packed multiply's single
// rounding equals "multiply in f32, round to bf16".
__device__ __forceinline__ uint32_t bf16x2_to_fp8x2(uint32_t w, uint32_t pre2, bool has_pre,
                                                    uint32_t sinv2, __nv_fp8_interpretation_t k) {
  __nv_bfloat162 v = *(const __nv_bfloat162*)&w;
  if (has_pre) v = __hmul2(v, *(const __nv_bfloat162*)&pre2);
  v = __hmul2(v, *(const __nv_bfloat162*)&sinv2);
  const uint32_t r = *(const uint32_t*)&v;
  return (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(bf16lo(r), bf16hi(r)), __NV_SATFINITE, k);
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
  return *(const uint32_t*)&t;
}

// Four bf16 values (two raw words) -> four int8 bytes, arithmetic in packed
// bf16: round_bf16(x * pre), round_bf16(. * sinv), optionally
// round_bf16(f32(.) + noise), clip, round half to even.
__device__ __forceinline__ uint32_t bf16x4_to_s8x4(uint32_t w0, uint32_t w1, uint32_t p0, uint32_t p1,
                                                   bool has_pre, uint32_t s0, uint32_t s1,
                                                   const float* nz, bool has_noise, float clip) {
  uint32_t out = 0;
  const uint32_t ws[2] = {w0, w1}, ps[2] = {p0, p1}, ss[2] = {s0, s1};
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    __nv_bfloat162 v = *(const __nv_bfloat162*)&ws[h];
    if (has_pre) v = __hmul2(v, *(const __nv_bfloat162*)&ps[h]);
    v = __hmul2(v, *(const __nv_bfloat162*)&ss[h]);
    uint32_t r = *(const uint32_t*)&v;
    float lo = bf16lo(r), hi = bf16hi(r);
    if (has_noise) {
      r = pack_bf16x2(__fadd_rn(lo, nz[2 * h]), __fadd_rn(hi, nz[2 * h + 1]));
      lo = bf16lo(r); hi = bf16hi(r);
    }
    lo = fminf(fmaxf(lo, -clip), clip);
    hi = fminf(fmaxf(hi, -clip), clip);
    out |= (((uint32_t)__float2int_rn(lo) & 0xffu) | (((uint32_t)__float2int_rn(hi) & 0xffu) << 8))
           << (16 * h);
  }
  return out;
}

// four int8 values of one word -> two packed bf16 pairs (exact)
__device__ __forceinline__ void s8x4_to_bf16x2x2(uint32_t w, uint32_t& lo, uint32_t& hi) {
  lo = pack_bf16x2((float)(signed char)(w & 0xffu), (float)(signed char)((w >> 8) & 0xffu));
  hi = pack_bf16x2((float)(signed char)((w >> 16) & 0xffu), (float)(signed char)(w >> 24));
}

constexpr int kFastRowChunk = 8192;  // most elements of one (row, chunk) work unit

// absmax, contraction contiguous, one warp per (batch-row, chunk).
// PRE: 0 none, 1 constant over the row (applied to the maximum), 2 per column.
template <int EPV, int PRE>
__global__ void __launch_bounds__(256, PRE == 2 ? 4 : (EPV == 16 ? 6 : 8))
absmax_row_fast(QParams P, int64_t chunks_per_row, int64_t total_units, int chunk_elems) {
  constexpr int ES = 16 / EPV;
  constexpr int U = 4;
  __shared__ float red[32];
  const int lane = threadIdx.x & 31;
  const int64_t warp_g = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * (blockDim.x >> 5);
  const DView& x = P.x;
  float tmax = 0.f;
  for (int64_t u = warp_g; u < total_units; u += nwarps) {
    const int64_t brow = u / chunks_per_row, chunk = u % chunks_per_row;
    int64_t i0, i1, r;
    decode_brow(x, brow, i0, i1, r);
    const int64_t c0 = chunk * chunk_elems;
    const int64_t nvec = (min(x.cols, c0 + (int64_t)chunk_elems) - c0) / EPV;
    const char* xp = (const char*)x.ptr + (i0 * x.sb0 + i1 * x.sb1 + r * x.sr + c0) * ES;
    const int64_t pbase = i0 * P.pre.sb0 + i1 * P.pre.sb1;
    uint4 run = make_uint4(0u, 0u, 0u, 0u);
    float fm = 0.f;
    for (int64_t i = lane; i < nvec; i += 32 * U) {
      uint4 raw[U];
#pragma unroll
      for (int k = 0; k < U; ++k) {
        const int64_t idx = i + 32 * k;
        raw[k] = idx < nvec ? ldg16(xp, idx * 16) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int k = 0; k < U; ++k) {
        if constexpr (PRE == 2 && EPV == 8) {
          if (P.pre_bf16 && P.pre_vec) {
            // round_bf16(x * p) is the packed bf16 multiply; its magnitude bits
            // order like unsigned integers
            const int64_t idx = i + 32 * k;
            if (idx < nvec) {
              const uint4 pw = ldg16(P.pre.ptr, (pbase + c0 + idx * EPV) * 2);
              const uint32_t xw[4] = {raw[k].x, raw[k].y, raw[k].z, raw[k].w};
              const uint32_t pp[4] = {pw.x, pw.y, pw.z, pw.w};
              uint32_t r[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const __nv_bfloat162 v = __hmul2(*(const __nv_bfloat162*)&xw[j],
                                                 *(const __nv_bfloat162*)&pp[j]);
                r[j] = *(const uint32_t*)&v & 0x7fff7fffu;
              }
              run.x = __vmaxu2(run.x, r[0]); run.y = __vmaxu2(run.y, r[1]);
              run.z = __vmaxu2(run.z, r[2]); run.w = __vmaxu2(run.w, r[3]);
            }
            continue;
          }
        }
        if constexpr (PRE == 2) {
          const int64_t idx = i + 32 * k;
          if (idx < nvec) {
            float v[EPV], p[EPV];
            unpack<EPV>(raw[k], x.dtype, v);
            loadN<EPV>(P.pre.ptr, P.pre.dtype, pbase + c0 + idx * EPV, p);
#pragma unroll
            for (int j = 0; j < EPV; ++j) fm = amax_nn(fm, fabsf(apply_pre(v[j], p[j], P.t_dtype)));
          }
        } else {
          packed_absmax<EPV>(run, raw[k], x.dtype);
        }
      }
    }
    float m = PRE == 2 ? amax_nn(fm, packed_hmax<EPV>(run, x.dtype)) : packed_hmax<EPV>(run, x.dtype);
    if constexpr (PRE == 1)
      m = apply_pre_abs(m, load1(P.pre.ptr, P.pre.dtype, pbase), P.t_dtype);
    if (P.per_tensor) {
      tmax = amax_nn(tmax, m);
    } else {
      m = warp_max(m);
      if (lane == 0 && m != 0.f) atomic_max_nonneg(P.amax + brow, m);
    }
  }
  if (P.per_tensor) {
    tmax = block_max(tmax, red);
    if (threadIdx.x == 0 && tmax != 0.f) atomic_max_nonneg(P.amax, tmax);
  }
}

// absmax, contraction contiguous, rows of at most 32 vectors (a power of two
// of them): one lane per vector, 32 / nvec rows per warp and load, the row
// maximum by a segmented butterfly. absmax_row_fast gives such rows a whole
// warp each and leaves most lanes idle.
template <int EPV, int PRE>
__global__ void __launch_bounds__(256, 5)
absmax_shortrow_fast(QParams P, int64_t nbrow, int nvec) {
  constexpr int ES = 16 / EPV;
  constexpr int U = 4;
  __shared__ float red[32];
  const int lane = threadIdx.x & 31;
  const int rows_per_warp = 32 / nvec;
  const int sub = lane / nvec, vi = lane % nvec;
  const int64_t warp_g = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * (blockDim.x >> 5);
  const DView& x = P.x;
  float tmax = 0.f;
  const int64_t groups = (nbrow + rows_per_warp - 1) / rows_per_warp;
  for (int64_t g0 = warp_g * U; g0 < groups; g0 += nwarps * U) {
    uint4 raw[U];
    int64_t brow[U];
#pragma unroll
    for (int k = 0; k < U; ++k) {
      brow[k] = (g0 + k) * rows_per_warp + sub;
      raw[k] = make_uint4(0u, 0u, 0u, 0u);
      if (g0 + k < groups && brow[k] < nbrow) {
        int64_t i0, i1, r;
        decode_brow(x, brow[k], i0, i1, r);
        raw[k] = ldg16(x.ptr, ((i0 * x.sb0 + i1 * x.sb1 + r * x.sr) * ES) + (int64_t)vi * 16);
      }
    }
#pragma unroll
    for (int k = 0; k < U; ++k) {
      uint4 run = make_uint4(0u, 0u, 0u, 0u);
      packed_absmax<EPV>(run, raw[k], x.dtype);
      float m = packed_hmax<EPV>(run, x.dtype);
      for (int o = nvec >> 1; o > 0; o >>= 1) m = amax_nn(m, __shfl_xor_sync(0xffffffffu, m, o));
      const bool ok = g0 + k < groups && brow[k] < nbrow;
      if constexpr (PRE == 1) {
        if (ok) {
          int64_t i0, i1, r;
          decode_brow(x, brow[k], i0, i1, r);
          m = apply_pre_abs(m, load1(P.pre.ptr, P.pre.dtype, i0 * P.pre.sb0 + i1 * P.pre.sb1),
                            P.t_dtype);
        }
      }
      if (P.per_tensor) {
        if (ok) tmax = amax_nn(tmax, m);
      } else if (ok && vi == 0) {
        P.amax[brow[k]] = __float_as_uint(m);  // the whole row is in this group: no atomic needed
      }
    }
  }
  if (P.per_tensor) {
    tmax = block_max(tmax, red);
    if (threadIdx.x == 0 && tmax != 0.f) atomic_max_nonneg(P.amax, tmax);
  }
}

// absmax, kept index contiguous. Block (32 x 8): thread (tx, ty) owns the EPV
// kept rows of one 16-byte vector and strides over a chunk of the contraction
// index. PRE: 0 none, 1 constant over the contraction index, 2 varying with it.
constexpr int kFastColChunk = 256;

template <int EPV, int PRE>
__global__ void __launch_bounds__(256)
absmax_col_fast(QParams P, int64_t row_blocks, int64_t col_chunks, int64_t total_units,
                int row_lanes) {
  constexpr int ES = 16 / EPV;
  constexpr int U = 4;
  __shared__ float red[32];
  // per kept row of the block: the eight row groups (ty) fold here first, so
  // that one atomic per row and unit reaches global memory instead of eight
  __shared__ uint32_t smax[32 * EPV];
  const DView& x = P.x;
  // A warp's 32 lanes cover row_lanes vectors of kept rows times 32 / row_lanes
  // consecutive contraction indices: with fewer than 32 vectors of rows (the
  // 128-element d of an attention operand) the lanes left over take further
  // contraction indices instead of idling.
  const int tx = threadIdx.x % row_lanes, txc = threadIdx.x / row_lanes, ty = threadIdx.y;
  const int col_lanes = 32 / row_lanes;
  const int tid = ty * 32 + threadIdx.x;
  for (int i = tid; i < 32 * EPV; i += 256) smax[i] = 0u;
  __syncthreads();
  float tmax = 0.f;
  for (int64_t u = blockIdx.x; u < total_units; u += gridDim.x) {
    const int64_t cc = u % col_chunks;
    int64_t t = u / col_chunks;
    const int64_t rb = t % row_blocks;
    const int64_t b = t / row_blocks;
    const int64_t i1 = b % x.b1, i0 = b / x.b1;
    const int64_t r0 = (rb * row_lanes + tx) * EPV;
    const int64_t cbeg = cc * kFastColChunk;
    const int64_t cend = min(x.cols, cbeg + (int64_t)kFastColChunk);
    const char* xp = (const char*)x.ptr + (i0 * x.sb0 + i1 * x.sb1 + r0) * ES;
    const int64_t pbase = i0 * P.pre.sb0 + i1 * P.pre.sb1;
    uint4 run = make_uint4(0u, 0u, 0u, 0u);
    float fm[PRE == 2 ? EPV : 1];
#pragma unroll
    for (int j = 0; j < (PRE == 2 ? EPV : 1); ++j) fm[j] = 0.f;
    if (r0 < x.rows) {
      const int64_t cstep = 8 * col_lanes;
      for (int64_t c = cbeg + ty * col_lanes + txc; c < cend; c += cstep * U) {
        uint4 raw[U];
#pragma unroll
        for (int k = 0; k < U; ++k) {
          const int64_t ck = c + cstep * k;
          raw[k] = ck < cend ? ldg16(xp, ck * x.sc * ES) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int k = 0; k < U; ++k) {
          if constexpr (PRE == 2 && EPV == 8) {
            if (P.pre_bf16) {
              const int64_t ck = c + cstep * k;
              if (ck < cend) {
                const float p = load1(P.pre.ptr, P.pre.dtype, pbase + ck * P.pre.sc);
                const uint32_t p2 = pack_bf16x2(p, p);
                const uint32_t xw[4] = {raw[k].x, raw[k].y, raw[k].z, raw[k].w};
                uint32_t r[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const __nv_bfloat162 v = __hmul2(*(const __nv_bfloat162*)&xw[j],
                                                   *(const __nv_bfloat162*)&p2);
                  r[j] = *(const uint32_t*)&v & 0x7fff7fffu;
                }
                run.x = __vmaxu2(run.x, r[0]); run.y = __vmaxu2(run.y, r[1]);
                run.z = __vmaxu2(run.z, r[2]); run.w = __vmaxu2(run.w, r[3]);
              }
              continue;
            }
          }
          if constexpr (PRE == 2) {
            const int64_t ck = c + cstep * k;
            if (ck < cend) {
              float v[EPV];
              unpack<EPV>(raw[k], x.dtype, v);
              const float p = load1(P.pre.ptr, P.pre.dtype, pbase + ck * P.pre.sc);
#pragma unroll
              for (int j = 0; j < EPV; ++j) fm[j] = amax_nn(fm[j], fabsf(apply_pre(v[j], p, P.t_dtype)));
            }
          } else {
            packed_absmax<EPV>(run, raw[k], x.dtype);
          }
        }
      }
    }
    float m[EPV];
    if constexpr (PRE == 2) {
      float pm[EPV];
      packed_to_floats<EPV>(run, x.dtype, pm);  // the packed-bf16 path's maxima (zero otherwise)
#pragma unroll
      for (int j = 0; j < EPV; ++j) m[j] = amax_nn(fm[j], pm[j]);
    } else {
      packed_to_floats<EPV>(run, x.dtype, m);
      if constexpr (PRE == 1) {
        const float p = load1(P.pre.ptr, P.pre.dtype, pbase);
#pragma unroll
        for (int j = 0; j < EPV; ++j) m[j] = apply_pre_abs(m[j], p, P.t_dtype);
      }
    }
    if (P.per_tensor) {
#pragma unroll
      for (int j = 0; j < EPV; ++j) tmax = amax_nn(tmax, m[j]);
    } else {
      // the maxima are non-negative (or NaN, which as bits is larger than
      // every number): unsigned order is their order
      if (r0 < x.rows) {
#pragma unroll
        for (int j = 0; j < EPV; ++j)
          if (m[j] != 0.f) atomicMax(&smax[tx * EPV + j], __float_as_uint(m[j]));
      }
      __syncthreads();
      const int64_t sbase = (i0 * x.b1 + i1) * x.rows + rb * row_lanes * EPV;
      for (int i = tid; i < row_lanes * EPV; i += 256) {
        const uint32_t v = smax[i];
        if (v != 0u) {
          if (rb * row_lanes * EPV + i < x.rows) atomic_max_nonneg(P.amax + sbase + i, __uint_as_float(v));
          smax[i] = 0u;
        }
      }
      __syncthreads();
    }
  }
  if (P.per_tensor) {
    const int lane = threadIdx.x;
    float v = warp_max(tmax);
    if (lane == 0) red[ty] = v;
    __syncthreads();
    if (ty == 0) {
      v = lane < 8 ? red[lane] : 0.f;
      v = warp_max(v);
      if (lane == 0 && v != 0.f) atomic_max_nonneg(P.amax, v);
    }
  }
}

// quantize, contraction contiguous: one thread per 16 output bytes, two units
// per loop trip so 32-64 bytes of input are in flight per thread. Units are
// walked from the END of the tensor: the calibration pass that just ran read
// it front to back, so its tail is what the L2 still holds.
template <int EPV, int PRE>
__global__ void __launch_bounds__(256)
quant_row_fast(QParams P, int64_t units_per_row, int64_t total_units) {
  constexpr int ES = 16 / EPV;
  constexpr int NV = 16 / EPV;  // input vectors per 16 outputs
  constexpr int UU = 2;
  __shared__ uint8_t lut[256];
  const DView& x = P.x;
  const bool has_noise = P.noise.ptr != nullptr;
  if (EPV == 16 && P.use_lut) build_lut(lut, P, PRE != 0);
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  for (int64_t u0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; u0 < total_units;
       u0 += nthreads * UU) {
    uint4 raw[UU][NV];
    int64_t brow[UU], col[UU];
    bool ok[UU];
#pragma unroll
    for (int k = 0; k < UU; ++k) {
      const int64_t uf = u0 + k * nthreads;
      ok[k] = uf < total_units;
      const int64_t u = total_units - 1 - (ok[k] ? uf : u0);
      brow[k] = u / units_per_row;
      col[k] = (u % units_per_row) * 16;
      int64_t i0, i1, r;
      decode_brow(x, brow[k], i0, i1, r);
      const char* xp = (const char*)x.ptr + (i0 * x.sb0 + i1 * x.sb1 + r * x.sr + col[k]) * ES;
#pragma unroll
      for (int n = 0; n < NV; ++n) raw[k][n] = ldg16(xp, n * 16);
    }
#pragma unroll
    for (int k = 0; k < UU; ++k) {
      if (!ok[k]) continue;
      int64_t i0, i1, r;
      decode_brow(x, brow[k], i0, i1, r);
      const float s = P.sinv[P.per_tensor ? 0 : brow[k]];
      const float sinv4[4] = {s, s, s, s};
      const int64_t pbase = i0 * P.pre.sb0 + i1 * P.pre.sb1;
      const int64_t nbase = i0 * P.noise.sb0 + i1 * P.noise.sb1 + r * P.noise.sr;
      float pconst = 0.f;
      if constexpr (PRE == 1) pconst = load1(P.pre.ptr, P.pre.dtype, pbase);
      uint32_t outw[4];
      if (EPV == 16 && P.use_lut) {
        const uint32_t rw[4] = {raw[k][0].x, raw[k][0].y, raw[k][0].z, raw[k][0].w};
#pragma unroll
        for (int g = 0; g < 4; ++g) outw[g] = lut4(rw[g], lut);
      } else if (EPV == 8 && P.fast_bf16) {
        const __nv_fp8_interpretation_t f8k = P.qdtype == AQTB200_E4M3 ? __NV_E4M3 : __NV_E5M2;
        const uint32_t sinv2 = pack_bf16x2(s, s);
#pragma unroll
        for (int n = 0; n < NV; ++n) {
          const uint32_t rw[4] = {raw[k][n].x, raw[k][n].y, raw[k][n].z, raw[k][n].w};
          uint32_t pw[4] = {0u, 0u, 0u, 0u};
          if constexpr (PRE == 1) {
            pw[0] = pw[1] = pw[2] = pw[3] = pack_bf16x2(pconst, pconst);
          } else if constexpr (PRE == 2) {
            float p[8];
            const int64_t c = col[k] + n * EPV;
            if (P.pre_vec) {
              loadN<8>(P.pre.ptr, P.pre.dtype, pbase + c, p);
            } else {
#pragma unroll
              for (int j = 0; j < 8; ++j) p[j] = load1(P.pre.ptr, P.pre.dtype, pbase + (c + j) * P.pre.sc);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) pw[j] = pack_bf16x2(p[2 * j], p[2 * j + 1]);
          }
#pragma unroll
          for (int g = 0; g < 2; ++g) {
            const uint32_t lo = bf16x2_to_fp8x2(rw[2 * g], pw[2 * g], PRE != 0, sinv2, f8k);
            const uint32_t hi = bf16x2_to_fp8x2(rw[2 * g + 1], pw[2 * g + 1], PRE != 0, sinv2, f8k);
            outw[(n * 2 + g) & 3] = lo | (hi << 16);
          }
        }
      } else if (EPV == 8 && P.int_bf16 && (PRE != 2 || P.pre_vec) && (!has_noise || P.noise_vec)) {
        const uint32_t sinv2 = pack_bf16x2(s, s);
#pragma unroll
        for (int n = 0; n < NV; ++n) {
          const uint32_t rw[4] = {raw[k][n].x, raw[k][n].y, raw[k][n].z, raw[k][n].w};
          const int64_t c = col[k] + n * EPV;
          uint32_t pw[4] = {0u, 0u, 0u, 0u};
          if constexpr (PRE == 1) {
            pw[0] = pw[1] = pw[2] = pw[3] = pack_bf16x2(pconst, pconst);
          } else if constexpr (PRE == 2) {
            const uint4 pv = ldg16(P.pre.ptr, (pbase + c) * 2);
            pw[0] = pv.x; pw[1] = pv.y; pw[2] = pv.z; pw[3] = pv.w;
          }
#pragma unroll
          for (int g = 0; g < 2; ++g) {
            float nz[4] = {0.f, 0.f, 0.f, 0.f};
            if (has_noise) loadN<4>(P.noise.ptr, AQTB200_F32, nbase + c + 4 * g, nz);
            outw[(n * 2 + g) & 3] = bf16x4_to_s8x4(rw[2 * g], rw[2 * g + 1], pw[2 * g], pw[2 * g + 1],
                                                   PRE != 0, sinv2, sinv2, nz, has_noise, P.clip_bound);
          }
        }
      } else {
#pragma unroll
      for (int n = 0; n < NV; ++n) {
        float v[EPV];
        unpack<EPV>(raw[k][n], x.dtype, v);
        const int64_t c = col[k] + n * EPV;
        if constexpr (PRE == 1) {
#pragma unroll
          for (int j = 0; j < EPV; ++j) v[j] = apply_pre(v[j], pconst, P.t_dtype);
        } else if constexpr (PRE == 2) {
          float p[EPV];
          if (P.pre_vec) {
            loadN<EPV>(P.pre.ptr, P.pre.dtype, pbase + c, p);
          } else {
#pragma unroll
            for (int j = 0; j < EPV; ++j) p[j] = load1(P.pre.ptr, P.pre.dtype, pbase + (c + j) * P.pre.sc);
          }
#pragma unroll
          for (int j = 0; j < EPV; ++j) v[j] = apply_pre(v[j], p[j], P.t_dtype);
        }
#pragma unroll
        for (int g = 0; g < EPV / 4; ++g) {
          float nz[4] = {0.f, 0.f, 0.f, 0.f};
          if (has_noise) {
            if (P.noise_vec) {
              loadN<4>(P.noise.ptr, AQTB200_F32, nbase + c + 4 * g, nz);
            } else {
#pragma unroll
              for (int j = 0; j < 4; ++j)
                nz[j] = load1(P.noise.ptr, AQTB200_F32, nbase + (c + 4 * g + j) * P.noise.sc);
            }
          }
          outw[(n * EPV) / 4 + g] = quant4(v + 4 * g, sinv4, nz, has_noise, P);
        }
      }
      }
      *(uint4*)(P.q + brow[k] * P.ldq + col[k]) = make_uint4(outw[0], outw[1], outw[2], outw[3]);
    }
  }
}

// quantize + transpose, kept index contiguous in the input.
// Tile: (16 * EPV) kept rows x 128 contraction indices, 256 threads. Thread
// (tx, ty) = (tid % 16, tid / 16) loads, for i in {0,1} and e in 0..3, the
// 16-byte vector of rows tx*EPV.. at contraction index i*64 + 4*ty + e, packs
// the four e's of each row into one word and parks it in shared memory with a
// per-row-group rotation (kills bank conflicts); the tile then leaves as
// 128-byte row segments.
template <int EPV, int PRE>
__global__ void __launch_bounds__(256)
quant_col_fast(QParams P, int64_t row_tiles, int64_t col_tiles, int64_t total_units) {
  constexpr int ES = 16 / EPV;
  constexpr int TR = 16 * EPV;
  __shared__ __align__(16) uint32_t tile[TR][32];
  __shared__ uint8_t lut[256];
  const DView& x = P.x;
  const bool has_noise = P.noise.ptr != nullptr;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  if (EPV == 16 && P.use_lut) build_lut(lut, P, PRE != 0);
  for (int64_t uf = blockIdx.x; uf < total_units; uf += gridDim.x) {
    const int64_t u = total_units - 1 - uf;  // back to front, see quant_row_fast
    const int64_t ct = u % col_tiles;
    int64_t t = u / col_tiles;
    const int64_t rt = t % row_tiles;
    const int64_t b = t / row_tiles;
    const int64_t i1 = b % x.b1, i0 = b / x.b1;
    const int64_t sbase = (i0 * x.b1 + i1) * x.rows;
    const int64_t r0 = rt * TR + tx * EPV;
    const bool row_ok = r0 < x.rows;  // rows % EPV == 0: a vector is all in or all out
    const char* xp = (const char*)x.ptr + (i0 * x.sb0 + i1 * x.sb1 + (row_ok ? r0 : 0)) * ES;
    const int64_t pbase = i0 * P.pre.sb0 + i1 * P.pre.sb1;
    const int64_t nbase = i0 * P.noise.sb0 + i1 * P.noise.sb1;
    float sinv[EPV];
#pragma unroll
    for (int j = 0; j < EPV; ++j)
      sinv[j] = P.per_tensor ? P.sinv[0] : (row_ok ? P.sinv[sbase + r0 + j] : 1.f);
    float pconst = 0.f;
    if constexpr (PRE == 1) pconst = load1(P.pre.ptr, P.pre.dtype, pbase);
    const __nv_fp8_interpretation_t f8k = P.qdtype == AQTB200_E4M3 ? __NV_E4M3 : __NV_E5M2;
    // One-byte inputs (16 rows per vector) keep the two passes as a loop: the
    // unrolled body of both does not fit the instruction cache, and the eight
    // warps of a block then wait for instructions instead of data.
#pragma unroll(EPV == 16 ? 1 : 2)
    for (int i = 0; i < 2; ++i) {
      uint4 raw[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int64_t c = ct * 128 + i * 64 + ty * 4 + e;
        raw[e] = (row_ok && c < x.cols) ? ldg16(xp, c * x.sc * ES) : make_uint4(0u, 0u, 0u, 0u);
      }
      uint32_t q4[4][EPV / 4];  // [column e][row group g]: bytes of rows 4g..4g+3
      // The noise of the four columns of this pass is requested up front (EPV
      // floats per column, as 16-byte vectors), so that its latency is paid
      // once per pass and not once per group of four rows.
      uint4 nzv[4][EPV / 4];
      const bool nz_pre = has_noise && P.noise_vec;
      if (nz_pre) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int64_t c = ct * 128 + i * 64 + ty * 4 + e;
          const bool in = row_ok && c < x.cols;
#pragma unroll
          for (int g = 0; g < EPV / 4; ++g)
            nzv[e][g] = in ? ldg16(P.noise.ptr, (nbase + c * P.noise.sc + r0 + 4 * g) * 4)
                           : make_uint4(0u, 0u, 0u, 0u);
        }
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int64_t c = ct * 128 + i * 64 + ty * 4 + e;
        const bool in = row_ok && c < x.cols;
        const uint32_t rw[4] = {raw[e].x, raw[e].y, raw[e].z, raw[e].w};
        if (EPV == 16 && P.use_lut) {
#pragma unroll
          for (int g = 0; g < EPV / 4; ++g) q4[e][g] = in ? lut4(rw[g & 3], lut) : 0u;
        } else if (EPV == 8 && P.fast_bf16) {
          float p = pconst;
          if constexpr (PRE == 2) p = in ? load1(P.pre.ptr, P.pre.dtype, pbase + c * P.pre.sc) : 0.f;
          const uint32_t pre2 = pack_bf16x2(p, p);
#pragma unroll
          for (int g = 0; g < EPV / 4; ++g) {
            const uint32_t lo = bf16x2_to_fp8x2(rw[(2 * g) & 3], pre2, PRE != 0,
                                                pack_bf16x2(sinv[(4 * g) % EPV], sinv[(4 * g + 1) % EPV]), f8k);
            const uint32_t hi = bf16x2_to_fp8x2(rw[(2 * g + 1) & 3], pre2, PRE != 0,
                                                pack_bf16x2(sinv[(4 * g + 2) % EPV], sinv[(4 * g + 3) % EPV]), f8k);
            q4[e][g] = in ? (lo | (hi << 16)) : 0u;
          }
        } else if (EPV == 8 && P.int_bf16 && (!has_noise || P.noise_vec)) {
          float p = pconst;
          if constexpr (PRE == 2) p = in ? load1(P.pre.ptr, P.pre.dtype, pbase + c * P.pre.sc) : 0.f;
          const uint32_t pre2 = pack_bf16x2(p, p);
#pragma unroll
          for (int g = 0; g < EPV / 4; ++g) {
            float nz[4] = {0.f, 0.f, 0.f, 0.f};
            if (has_noise && in) {
              nz[0] = __uint_as_float(nzv[e][g].x); nz[1] = __uint_as_float(nzv[e][g].y);
              nz[2] = __uint_as_float(nzv[e][g].z); nz[3] = __uint_as_float(nzv[e][g].w);
            }
            const uint32_t q = bf16x4_to_s8x4(
                rw[(2 * g) & 3], rw[(2 * g + 1) & 3], pre2, pre2, PRE != 0,
                pack_bf16x2(sinv[(4 * g) % EPV], sinv[(4 * g + 1) % EPV]),
                pack_bf16x2(sinv[(4 * g + 2) % EPV], sinv[(4 * g + 3) % EPV]), nz, has_noise,
                P.clip_bound);
            q4[e][g] = in ? q : 0u;
          }
        } else {
          float v[EPV];
          unpack<EPV>(raw[e], x.dtype, v);
          float p = pconst;
          if constexpr (PRE == 2) p = in ? load1(P.pre.ptr, P.pre.dtype, pbase + c * P.pre.sc) : 0.f;
#pragma unroll
          for (int g = 0; g < EPV / 4; ++g) {
            float w4[4], nz[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int j = 0; j < 4; ++j)
              w4[j] = PRE ? apply_pre(v[4 * g + j], p, P.t_dtype) : v[4 * g + j];
            if (has_noise && in) {
              if (P.noise_vec) {
                nz[0] = __uint_as_float(nzv[e][g].x); nz[1] = __uint_as_float(nzv[e][g].y);
                nz[2] = __uint_as_float(nzv[e][g].z); nz[3] = __uint_as_float(nzv[e][g].w);
              } else {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                  nz[j] = load1(P.noise.ptr, AQTB200_F32,
                                nbase + c * P.noise.sc + (r0 + 4 * g + j) * P.noise.sr);
              }
            }
            q4[e][g] = in ? quant4(w4, sinv + 4 * g, nz, has_noise, P) : 0u;
          }
        }
      }
#pragma unroll
      for (int g = 0; g < EPV / 4; ++g) {
        const uint32_t cols4[4] = {q4[0][g], q4[1][g], q4[2][g], q4[3][g]};
        uint32_t rows4[4];
        transpose4x4(cols4, rows4);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          tile[tx * EPV + 4 * g + j][(i * 16 + ty + 4 * tx) & 31] = rows4[j];
      }
    }
    __syncthreads();
#pragma unroll
    for (int s = 0; s < TR / 32; ++s) {
      const int id = tid + 256 * s;
      const int row = id >> 3, seg = id & 7;
      const int64_t gr = rt * TR + row;
      const int64_t gc = ct * 128 + seg * 16;
      if (gr < x.rows && gc < P.ldq) {
        const uint4 o = *(const uint4*)&tile[row][(seg * 4 + 4 * (row / EPV)) & 31];
        *(uint4*)(P.q + (sbase + gr) * P.ldq + gc) = o;
      }
    }
    __syncthreads();
  }
}

// quant_col_fast for one case only: a stored int8 operand re-quantized to int8
// in bf16 arithmetic (the backward pass under use_fwd_quant), with or without a
// vectorisable f32 noise tensor. Same tile and thread layout (256 kept rows x
// 128 contraction indices, thread = 16 rows of 8 columns); compiled without
// the general kernel's other branches it fits two blocks per SM, and the noise
// of two columns at a time (32 registers) is requested ahead of their use.
template <int PRE, bool NOISE>
__global__ void __launch_bounds__(256, 2)
quant_col_s8_kernel(QParams P, int64_t row_tiles, int64_t col_tiles, int64_t total_units) {
  constexpr int EPV = 16, TR = 16 * EPV;
  __shared__ __align__(16) uint32_t tile[TR][32];
  const DView& x = P.x;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  for (int64_t uf = blockIdx.x; uf < total_units; uf += gridDim.x) {
    const int64_t u = total_units - 1 - uf;
    const int64_t ct = u % col_tiles;
    int64_t t = u / col_tiles;
    const int64_t rt = t % row_tiles;
    const int64_t b = t / row_tiles;
    const int64_t i1 = b % x.b1, i0 = b / x.b1;
    const int64_t sbase = (i0 * x.b1 + i1) * x.rows;
    const int64_t r0 = rt * TR + tx * EPV;
    const bool row_ok = r0 < x.rows;
    const char* xp = (const char*)x.ptr + (i0 * x.sb0 + i1 * x.sb1 + (row_ok ? r0 : 0));
    const int64_t pbase = i0 * P.pre.sb0 + i1 * P.pre.sb1;
    const int64_t nbase = i0 * P.noise.sb0 + i1 * P.noise.sb1;
    uint32_t sinv2[EPV / 2];  // reciprocal scales of the thread's rows, as bf16 pairs
#pragma unroll
    for (int j = 0; j < EPV / 2; ++j) {
      const float a = P.per_tensor ? P.sinv[0] : (row_ok ? P.sinv[sbase + r0 + 2 * j] : 1.f);
      const float c = P.per_tensor ? P.sinv[0] : (row_ok ? P.sinv[sbase + r0 + 2 * j + 1] : 1.f);
      sinv2[j] = pack_bf16x2(a, c);
    }
    float pconst = 0.f;
    if constexpr (PRE == 1) pconst = load1(P.pre.ptr, P.pre.dtype, pbase);
#pragma unroll 1
    for (int i = 0; i < 2; ++i) {
      uint4 raw[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int64_t c = ct * 128 + i * 64 + ty * 4 + e;
        raw[e] = (row_ok && c < x.cols) ? ldg16(xp, c * x.sc) : make_uint4(0u, 0u, 0u, 0u);
      }
      uint32_t q4[4][EPV / 4];
#pragma unroll
      for (int eh = 0; eh < 2; ++eh) {
        uint4 nzv[2][EPV / 4];
        if constexpr (NOISE) {
#pragma unroll
          for (int e2 = 0; e2 < 2; ++e2) {
            const int64_t c = ct * 128 + i * 64 + ty * 4 + eh * 2 + e2;
            const bool in = row_ok && c < x.cols;
#pragma unroll
            for (int g = 0; g < EPV / 4; ++g)
              nzv[e2][g] = in ? ldg16(P.noise.ptr, (nbase + c * P.noise.sc + r0 + 4 * g) * 4)
                              : make_uint4(0u, 0u, 0u, 0u);
          }
        }
#pragma unroll
        for (int e2 = 0; e2 < 2; ++e2) {
          const int e = eh * 2 + e2;
          const int64_t c = ct * 128 + i * 64 + ty * 4 + e;
          const bool in = row_ok && c < x.cols;
          const uint32_t rw[4] = {raw[e].x, raw[e].y, raw[e].z, raw[e].w};
          float p = pconst;
          if constexpr (PRE == 2) p = in ? load1(P.pre.ptr, P.pre.dtype, pbase + c * P.pre.sc) : 0.f;
          const uint32_t pre2 = pack_bf16x2(p, p);
#pragma unroll
          for (int g = 0; g < EPV / 4; ++g) {
            float nz[4] = {0.f, 0.f, 0.f, 0.f};
            if constexpr (NOISE) {
              nz[0] = __uint_as_float(nzv[e2][g].x); nz[1] = __uint_as_float(nzv[e2][g].y);
              nz[2] = __uint_as_float(nzv[e2][g].z); nz[3] = __uint_as_float(nzv[e2][g].w);
            }
            uint32_t w0, w1;
            s8x4_to_bf16x2x2(rw[g], w0, w1);
            const uint32_t q = bf16x4_to_s8x4(w0, w1, pre2, pre2, PRE != 0, sinv2[2 * g],
                                              sinv2[2 * g + 1], nz, NOISE, P.clip_bound);
            q4[e][g] = in ? q : 0u;
          }
        }
      }
#pragma unroll
      for (int g = 0; g < EPV / 4; ++g) {
        const uint32_t cols4[4] = {q4[0][g], q4[1][g], q4[2][g], q4[3][g]};
        uint32_t rows4[4];
        transpose4x4(cols4, rows4);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          tile[tx * EPV + 4 * g + j][(i * 16 + ty + 4 * tx) & 31] = rows4[j];
      }
    }
    __syncthreads();
#pragma unroll
    for (int s = 0; s < TR / 32; ++s) {
      const int id = tid + 256 * s;
      const int row = id >> 3, seg = id & 7;
      const int64_t gr = rt * TR + row;
      const int64_t gc = ct * 128 + seg * 16;
      if (gr < x.rows && gc < P.ldq) {
        const uint4 o = *(const uint4*)&tile[row][(seg * 4 + 4 * (row / EPV)) & 31];
        *(uint4*)(P.q + (sbase + gr) * P.ldq + gc) = o;
      }
    }
    __syncthreads();
  }
}

// scale = where(a == 0, 1, a) [* clipping_scale] / quant_bound, in T, stored as S
__device__ __forceinline__ float scale_of_amax(float a, int t_dtype, int s_dtype, float quant_bound,
                                               float clipping_scale, int po2) {
  if (a == 0.f) a = 1.f;
  float bound = clipping_scale != 0.f ? round_to(__fmul_rn(a, clipping_scale), t_dtype) : a;
  float s = round_to(__fdiv_rn(bound, quant_bound), t_dtype);
  if (po2) {
    // 1 / 2**floor(log2(1/s)); the exponent is read off the float directly.
    float r = round_to(__fdiv_rn(1.f, s), t_dtype);
    int e;
    frexpf(r, &e);  // r = m * 2**e, m in [0.5, 1)
    float p = round_to(ldexpf(1.f, e - 1), t_dtype);
    s = round_to(__fdiv_rn(1.f, p), t_dtype);
  }
  return round_to(s, s_dtype);
}
__device__ __forceinline__ float recip_of_scale(float s, int s_dtype) {
  float inv = round_to(__fdiv_rn(1.f, s), s_dtype);
  return isinf(inv) ? 1.f : inv;
}

// ---------------------------------------------------------------------------
// One read, two fp8 quantizations (bf16 input, per-tensor scales): the
// transposed one of quant_col_fast and one in the input's own orientation.
// A training step needs each operand twice -- lhs as [M][K] for the forward
// dot and as [K][M] for drhs, the cotangent as [M][N] for dlhs and [N][M] for
// drhs -- and this way the operand is read from HBM once for both.
// chain 0: both outputs quantize x; 1: the same-orientation output quantizes
// the VALUES of the transposed one (x -> q_t -> q_s, the backward pass's
// re-quantization of a stored forward operand); 2: the other way round.
struct PairParams {
  DView x;                 // rows contiguous (kept index of q_t), cols strided
  void* scale_t;           // one bf16 scale per output (read, or written when amax is given)
  void* scale_s;
  const void* pre_t;       // optional single bf16 / f32 prescale per output
  const void* pre_s;
  int pre_t_dtype, pre_s_dtype;
  int qdtype_t, qdtype_s;   // e4m3 / e5m2 / s8
  float clip_t, clip_s;     // int8 outputs: clip bound
  int chain;
  // amax != null: the scales are computed here from amax[0] and written out
  // (block 0), instead of being read
  const uint32_t* amax;
  // optional: receives max |x| (f32 bits, atomic max; zeroed by the host), for
  // callers whose scales do not come from this step's maximum (delayed scaling)
  uint32_t* amax_out;
  float qb_t, qb_s, cs_t, cs_s;  // quant_bound / clipping_scale per output
  int po2_t, po2_s;
  uint8_t* q_t;            // [b][rows][ld_t]
  uint8_t* q_s;            // [b][cols][ld_s]
  int64_t ld_t, ld_s;
};

__device__ __forceinline__ uint32_t bf16_recip_pair(const void* scale) {
  // round_bf16(1 / s), 1 where that overflows (aqt_tensor.py:151-153), in both halves
  const float s = load1(scale, AQTB200_BF16, 0);
  float inv = round_to(__fdiv_rn(1.f, s), AQTB200_BF16);
  if (isinf(inv)) inv = 1.f;
  return pack_bf16x2(inv, inv);
}
// two fp8 bytes -> their exact values as packed bf16
__device__ __forceinline__ uint32_t fp8x2_to_bf16x2(uint32_t q2, __nv_fp8_interpretation_t k) {
  const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)q2, k);
  const float2 f = __half22float2(*(const __half2*)&h);
  return pack_bf16x2(f.x, f.y);
}

// |value of Q(a)| for a >= 0 already prescaled: the largest magnitude among the
// quantized values of a tensor whose largest magnitude is a.
__device__ __forceinline__ float requant_abs(float a, float s, int t_dtype, int s_dtype, int kind,
                                             int qdtype, float clip_bound) {
  const float inv = recip_of_scale(s, s_dtype);
  const int y_dtype = (t_dtype == AQTB200_F32 || s_dtype == AQTB200_F32) ? AQTB200_F32 : AQTB200_BF16;
  float y = round_to(__fmul_rn(a, inv), y_dtype);
  y = fminf(fmaxf(y, -clip_bound), clip_bound);
  if (kind == AQTB200_NUM_INT) return fabsf((float)__float2int_rn(y));
  const uint8_t q = (uint8_t)__nv_cvt_float_to_fp8(y, __NV_SATFINITE,
                                                   qdtype == AQTB200_E4M3 ? __NV_E4M3 : __NV_E5M2);
  return fabsf(fp8_to_float(q, qdtype));
}

// Two bf16 values -> two quantized bytes (fp8, or int8 with clip and RNE), and back.
__device__ __forceinline__ uint32_t bf16x2_to_q8x2(uint32_t w, uint32_t pre2, bool has_pre,
                                                   uint32_t sinv2, bool is_int, float clip,
                                                   __nv_fp8_interpretation_t k) {
  if (!is_int) return bf16x2_to_fp8x2(w, pre2, has_pre, sinv2, k);
  __nv_bfloat162 v = *(const __nv_bfloat162*)&w;
  if (has_pre) v = __hmul2(v, *(const __nv_bfloat162*)&pre2);
  v = __hmul2(v, *(const __nv_bfloat162*)&sinv2);
  const uint32_t r = *(const uint32_t*)&v;
  const float lo = fminf(fmaxf(bf16lo(r), -clip), clip);
  const float hi = fminf(fmaxf(bf16hi(r), -clip), clip);
  return ((uint32_t)__float2int_rn(lo) & 0xffu) | (((uint32_t)__float2int_rn(hi) & 0xffu) << 8);
}
__device__ __forceinline__ uint32_t q8x2_to_bf16x2(uint32_t q2, bool is_int,
                                                   __nv_fp8_interpretation_t k) {
  if (!is_int) return fp8x2_to_bf16x2(q2, k);
  return pack_bf16x2((float)(signed char)(q2 & 0xffu), (float)(signed char)((q2 >> 8) & 0xffu));
}

// IS_INT: both outputs int8 (else both fp8); CHAIN as PairParams::chain. Compile-
// time, because the kernel is bound by issue slots, not by memory.
template <bool IS_INT, int CHAIN>
__global__ void __launch_bounds__(256, 4)
quant_pair_kernel(PairParams P, int64_t row_tiles, int64_t col_tiles, int64_t total_units) {
  constexpr int EPV = 8, TR = 16 * EPV;
  __shared__ __align__(16) uint32_t tile[TR][32];
  const DView& x = P.x;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const bool has_pre_t = P.pre_t != nullptr, has_pre_s = P.pre_s != nullptr;
  uint32_t pre_t = 0, pre_s = 0;
  float pre_t_f = 1.f, pre_s_f = 1.f;
  if (has_pre_t) { pre_t_f = round_to(load1(P.pre_t, P.pre_t_dtype, 0), AQTB200_BF16); pre_t = pack_bf16x2(pre_t_f, pre_t_f); }
  if (has_pre_s) { pre_s_f = round_to(load1(P.pre_s, P.pre_s_dtype, 0), AQTB200_BF16); pre_s = pack_bf16x2(pre_s_f, pre_s_f); }
  uint32_t sinv_t, sinv_s;
  if (P.amax != nullptr) {
    // Every block derives the two scales from the maximum (a few dozen scalar
    // operations); block 0 also publishes them for the dequantizing epilogue.
    constexpr int B = AQTB200_BF16;
    constexpr int kind = IS_INT ? AQTB200_NUM_INT : AQTB200_NUM_FP8;
    const float a = __uint_as_float(P.amax[0]);
    const float a_t = has_pre_t ? apply_pre_abs(a, pre_t_f, B) : a;
    const float a_s = has_pre_s ? apply_pre_abs(a, pre_s_f, B) : a;
    float s_t, s_s;
    if constexpr (CHAIN == 1) {
      s_t = scale_of_amax(a_t, B, B, P.qb_t, P.cs_t, P.po2_t);
      s_s = scale_of_amax(requant_abs(a_t, s_t, B, B, kind, P.qdtype_t, P.clip_t), B, B, P.qb_s,
                          P.cs_s, P.po2_s);
    } else if constexpr (CHAIN == 2) {
      s_s = scale_of_amax(a_s, B, B, P.qb_s, P.cs_s, P.po2_s);
      s_t = scale_of_amax(requant_abs(a_s, s_s, B, B, kind, P.qdtype_s, P.clip_s), B, B, P.qb_t,
                          P.cs_t, P.po2_t);
    } else {
      s_t = scale_of_amax(a_t, B, B, P.qb_t, P.cs_t, P.po2_t);
      s_s = scale_of_amax(a_s, B, B, P.qb_s, P.cs_s, P.po2_s);
    }
    if (blockIdx.x == 0 && tid == 0) {
      *(__nv_bfloat16*)P.scale_t = __float2bfloat16_rn(s_t);
      *(__nv_bfloat16*)P.scale_s = __float2bfloat16_rn(s_s);
    }
    const float it = recip_of_scale(s_t, B), is = recip_of_scale(s_s, B);
    sinv_t = pack_bf16x2(it, it);
    sinv_s = pack_bf16x2(is, is);
  } else {
    sinv_t = bf16_recip_pair(P.scale_t);
    sinv_s = bf16_recip_pair(P.scale_s);
  }
  const __nv_fp8_interpretation_t kt = P.qdtype_t == AQTB200_E4M3 ? __NV_E4M3 : __NV_E5M2;
  const __nv_fp8_interpretation_t ks = P.qdtype_s == AQTB200_E4M3 ? __NV_E4M3 : __NV_E5M2;
  constexpr bool int_t = IS_INT, int_s = IS_INT;
  uint32_t run_max = 0u;  // packed bf16 magnitudes, when amax_out is wanted
  for (int64_t uf = blockIdx.x; uf < total_units; uf += gridDim.x) {
    const int64_t u = total_units - 1 - uf;  // back to front: the calibration pass's tail is still in L2
    // Neighbouring blocks take neighbouring tiles along the CONTIGUOUS index of
    // the input, so the blocks in flight together stream whole rows of it (and
    // of the same-orientation output) instead of a 256-byte strip of every row.
    const int64_t rt = u % row_tiles;
    int64_t t = u / row_tiles;
    const int64_t ct = t % col_tiles;
    const int64_t b = t / col_tiles;
    const int64_t i1 = b % x.b1, i0 = b / x.b1;
    const int64_t bidx = i0 * x.b1 + i1;
    const int64_t r0 = rt * TR + tx * EPV;
    const bool row_ok = r0 < x.rows;  // rows % 8 == 0: a vector is all in or all out
    const char* xp = (const char*)x.ptr + (i0 * x.sb0 + i1 * x.sb1 + (row_ok ? r0 : 0)) * 2;
    uint8_t* qs_base = P.q_s + (bidx * x.cols + ct * 128 + ty * 4) * P.ld_s + r0;
    uint4 raw[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int64_t c = ct * 128 + i * 64 + ty * 4 + e;
        raw[i][e] = (row_ok && c < x.cols) ? ldg16(xp, c * x.sc * 2) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      uint32_t q4[4][2];  // transposed output: [column e][row group g]
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int64_t c = ct * 128 + i * 64 + ty * 4 + e;
        const bool in = row_ok && c < x.cols;
        const uint32_t rw[4] = {raw[i][e].x, raw[i][e].y, raw[i][e].z, raw[i][e].w};
        if (P.amax_out != nullptr) {  // out-of-range vectors were loaded as zeros
#pragma unroll
          for (int j = 0; j < 4; ++j) run_max = __vmaxu2(run_max, rw[j] & 0x7fff7fffu);
        }
        uint32_t qt[4], qs[4];  // two bytes each (rows 2j, 2j+1)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if constexpr (CHAIN == 1) {
            qt[j] = bf16x2_to_q8x2(rw[j], pre_t, has_pre_t, sinv_t, int_t, P.clip_t, kt);
            qs[j] = bf16x2_to_q8x2(q8x2_to_bf16x2(qt[j], int_t, kt), 0u, false, sinv_s, int_s,
                                   P.clip_s, ks);
          } else if constexpr (CHAIN == 2) {
            qs[j] = bf16x2_to_q8x2(rw[j], pre_s, has_pre_s, sinv_s, int_s, P.clip_s, ks);
            qt[j] = bf16x2_to_q8x2(q8x2_to_bf16x2(qs[j], int_s, ks), 0u, false, sinv_t, int_t,
                                   P.clip_t, kt);
          } else {
            qt[j] = bf16x2_to_q8x2(rw[j], pre_t, has_pre_t, sinv_t, int_t, P.clip_t, kt);
            qs[j] = bf16x2_to_q8x2(rw[j], pre_s, has_pre_s, sinv_s, int_s, P.clip_s, ks);
          }
        }
        q4[e][0] = in ? (qt[0] | (qt[1] << 16)) : 0u;
        q4[e][1] = in ? (qt[2] | (qt[3] << 16)) : 0u;
        if (in) {
          // same orientation: rows r0..r0+7 of column c are 8 contiguous bytes
          *(uint2*)(qs_base + (int64_t)(i * 64 + e) * P.ld_s) =
              make_uint2(qs[0] | (qs[1] << 16), qs[2] | (qs[3] << 16));
        }
      }
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        const uint32_t cols4[4] = {q4[0][g], q4[1][g], q4[2][g], q4[3][g]};
        uint32_t rows4[4];
        transpose4x4(cols4, rows4);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          tile[tx * EPV + 4 * g + j][(i * 16 + ty + 4 * tx) & 31] = rows4[j];
      }
    }
    __syncthreads();
#pragma unroll
    for (int s2 = 0; s2 < TR / 32; ++s2) {
      const int id = tid + 256 * s2;
      const int row = id >> 3, seg = id & 7;
      const int64_t gr = rt * TR + row;
      const int64_t gc = ct * 128 + seg * 16;
      if (gr < x.rows && gc < P.ld_t) {
        const uint4 o = *(const uint4*)&tile[row][(seg * 4 + 4 * (row / EPV)) & 31];
        *(uint4*)(P.q_t + (bidx * x.rows + gr) * P.ld_t + gc) = o;
      }
    }
    __syncthreads();
  }
  if (P.amax_out != nullptr) {
    uint32_t m = max(run_max & 0xffffu, run_max >> 16) << 16;  // f32 bits of the bf16 magnitude
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((tid & 31) == 0 && m != 0u) atomicMax(P.amax_out, m);
  }
}

// |value of Q(amax)|: quantization is monotone and odd, so the largest
// magnitude among the quantized values is the quantized largest magnitude and
// the backward pass can calibrate a stored operand without reading it.
struct RequantAmaxParams {
  const uint32_t* amax;
  const void* scale;
  const void* pre;
  int pre_dtype, t_dtype, s_dtype, kind, qdtype;
  float clip_bound;
  float* out;
  int64_t n;
};
__global__ void requant_amax_kernel(RequantAmaxParams R) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= R.n) return;
  float a = __uint_as_float(R.amax[i]);
  if (R.pre != nullptr) a = apply_pre_abs(a, load1(R.pre, R.pre_dtype, 0), R.t_dtype);
  const float s = load1(R.scale, R.s_dtype, i);
  R.out[i] = requant_abs(a, s, R.t_dtype, R.s_dtype, R.kind, R.qdtype, R.clip_bound);
}

__global__ void prescale_amax_kernel(const uint32_t* amax, int64_t n, const void* pre, int pre_dtype,
                                     int t_dtype, float* out) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = apply_pre_abs(__uint_as_float(amax[i]), load1(pre, pre_dtype, 0), t_dtype);
}

// ---------------------------------------------------------------------------
// amax -> scale and rounded reciprocal (calibration.py:149-157,
// aqt_tensor.py:151-153). All arithmetic in T, stored as S.
struct FinalizeParams {
  const uint32_t* amax;
  const void* scale_in;  // when non-null: skip calibration, use this scale
  void* scale_out;
  float* sinv;
  int64_t n;
  int t_dtype, s_dtype;
  float quant_bound, clipping_scale;
  int po2;
  const void* pre;  // optional single prescale applied to the maximum
  int pre_dtype;
};

__global__ void finalize_scale_kernel(FinalizeParams F) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= F.n) return;
  float s;
  if (F.scale_in != nullptr) {
    s = load1(F.scale_in, F.s_dtype, i);
  } else {
    float a = __uint_as_float(F.amax[i]);
    if (F.pre != nullptr) a = apply_pre_abs(a, load1(F.pre, F.pre_dtype, 0), F.t_dtype);
    s = scale_of_amax(a, F.t_dtype, F.s_dtype, F.quant_bound, F.clipping_scale, F.po2);
  }
  if (F.scale_out != nullptr && F.scale_out != F.scale_in) {
    if (F.s_dtype == AQTB200_BF16)
      ((__nv_bfloat16*)F.scale_out)[i] = __float2bfloat16_rn(s);
    else
      ((float*)F.scale_out)[i] = s;
  }
  if (F.sinv == nullptr) return;
  F.sinv[i] = recip_of_scale(s, F.s_dtype);
}

// ---------------------------------------------------------------------------
// Delayed scaling (flax/delayed_scaling_calibration.py:28-124): the bound comes
// from a history of earlier maxima, not from the tensor being quantized, so
// the quantization of a step does not wait for a reduction over its operand.
//   new_bound = max(history) if that is > 0 and finite, else the previous bound
//   scale     = cast_S(new_bound / quant_bound [-> power of two])       (f32 math)
//   history   = roll(history, -1) with element 0 replaced by max |x|
struct DelayedParams {
  float* history;
  int64_t len;
  float* bound;
  int update_bound;
  float quant_bound;
  int po2, s_dtype;
  void* scale_out;
  const float* amax;
};

// one block; history lengths up to 4096
__global__ void __launch_bounds__(1024) delayed_scale_kernel(DelayedParams D) {
  __shared__ float red[32];
  float m = -INFINITY;
  bool nan = false;
  for (int64_t i = threadIdx.x; i < D.len; i += blockDim.x) {
    const float h = D.history[i];
    nan |= h != h;
    m = fmaxf(m, h);
  }
  // jnp.max propagates NaN
  m = nan ? NAN : m;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, m, o);
    m = (m != m || other != other) ? NAN : fmaxf(m, other);
  }
  if (lane == 0) red[warp] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    float a = red[0];
    const int nw = (blockDim.x + 31) >> 5;
    for (int w = 1; w < nw; ++w) a = (a != a || red[w] != red[w]) ? NAN : fmaxf(a, red[w]);
    const float prev = D.bound[0];
    float nb = a > 0.0f ? a : prev;
    nb = isfinite(a) ? nb : prev;
    if (D.update_bound) D.bound[0] = nb;
    float s = __fdiv_rn(nb, D.quant_bound);
    if (D.po2) {
      // calibration.ceil_to_po2 in f32: 1 / 2**floor(log2(1/s))
      const float r = __fdiv_rn(1.f, s);
      int e;
      frexpf(r, &e);
      s = __fdiv_rn(1.f, ldexpf(1.f, e - 1));
    }
    if (D.s_dtype == AQTB200_BF16) ((__nv_bfloat16*)D.scale_out)[0] = __float2bfloat16_rn(s);
    else ((float*)D.scale_out)[0] = s;
  }
}

__global__ void __launch_bounds__(1024) delayed_push_kernel(DelayedParams D) {
  // every element is read before any is written: one block, values in registers
  float v[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int64_t i = threadIdx.x + 1024 * k;
    v[k] = i < D.len ? D.history[(i + 1) % D.len] : 0.f;
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int64_t i = threadIdx.x + 1024 * k;
    if (i < D.len) D.history[i] = i == 0 ? D.amax[0] : v[k];
  }
}

// ---------------------------------------------------------------------------
// Calibrate and quantize in ONE pass, for per-row scales when a row fits in a
// block's registers (up to 256 threads x 4 vectors): each block takes whole
// rows, keeps the row in registers between the maximum and the quantization,
// so the operand is read once and three launches become one. Same arithmetic
// as absmax_row_fast + finalize_scale_kernel + quant_row_fast (no prescale
// that varies along the row, no noise).
struct OnePassParams {
  QParams q;
  float quant_bound, clipping_scale;
  int po2;
  void* scale_out;
};

template <int EPV, int PRE>
__global__ void __launch_bounds__(256)
quant_row_onepass(OnePassParams O, int64_t nbrow) {
  // A GEMM launched as a programmatic dependent of this kernel may start its
  // prologue and the loads of its other operand now; it waits for this
  // kernel's completion before it touches what is written here.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  constexpr int ES = 16 / EPV;
  constexpr int NV = 16 / EPV;   // input vectors per 16 outputs
  constexpr int UMAX = 4 / NV > 0 ? 4 / NV : 1;  // 16-output units per thread
  __shared__ float red[32];
  const QParams& P = O.q;
  const DView& x = P.x;
  const int64_t units = P.ldq / 16;  // per row; cols % 16 == 0 here
  for (int64_t brow = blockIdx.x; brow < nbrow; brow += gridDim.x) {
    int64_t i0, i1, r;
    decode_brow(x, brow, i0, i1, r);
    const char* xp = (const char*)x.ptr + (i0 * x.sb0 + i1 * x.sb1 + r * x.sr) * ES;
    uint4 raw[UMAX][NV];
    uint4 run = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
    for (int k = 0; k < UMAX; ++k) {
      const int64_t u = threadIdx.x + 256 * k;
#pragma unroll
      for (int n = 0; n < NV; ++n) {
        raw[k][n] = u < units ? ldg16(xp, (u * NV + n) * 16) : make_uint4(0u, 0u, 0u, 0u);
        packed_absmax<EPV>(run, raw[k][n], x.dtype);
      }
    }
    float m = packed_hmax<EPV>(run, x.dtype);
    const int64_t pbase = i0 * P.pre.sb0 + i1 * P.pre.sb1;
    float pconst = 0.f;
    if constexpr (PRE == 1) pconst = load1(P.pre.ptr, P.pre.dtype, pbase);
    m = block_max(m, red);
    if (threadIdx.x == 0) red[0] = m;
    __syncthreads();
    m = red[0];
    __syncthreads();
    if constexpr (PRE == 1) m = apply_pre_abs(m, pconst, P.t_dtype);
    const float s = scale_of_amax(m, P.t_dtype, P.s_dtype, O.quant_bound, O.clipping_scale, O.po2);
    if (threadIdx.x == 0) {
      if (P.s_dtype == AQTB200_BF16) ((__nv_bfloat16*)O.scale_out)[brow] = __float2bfloat16_rn(s);
      else ((float*)O.scale_out)[brow] = s;
    }
    const float sinv = recip_of_scale(s, P.s_dtype);
    const float sinv4[4] = {sinv, sinv, sinv, sinv};
    const float nz[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int k = 0; k < UMAX; ++k) {
      const int64_t u = threadIdx.x + 256 * k;
      if (u >= units) continue;
      uint32_t outw[4];
#pragma unroll
      for (int n = 0; n < NV; ++n) {
        float v[EPV];
        unpack<EPV>(raw[k][n], x.dtype, v);
        if constexpr (PRE == 1) {
#pragma unroll
          for (int j = 0; j < EPV; ++j) v[j] = apply_pre(v[j], pconst, P.t_dtype);
        }
#pragma unroll
        for (int g = 0; g < EPV / 4; ++g)
          outw[(n * EPV) / 4 + g] = quant4(v + 4 * g, sinv4, nz, false, P);
      }
      *(uint4*)(P.q + brow * P.ldq + u * 16) = make_uint4(outw[0], outw[1], outw[2], outw[3]);
    }
  }
}

// Short rows (at most 32 sixteen-byte vectors, e.g. the 128-element rows of an
// attention head): calibrate and quantize in one pass with several rows per
// warp. Each lane holds one vector of its row; the row maximum is a segmented
// butterfly over the row's lanes; the quantized vector goes straight back
// out. One read and one launch where the three-step flow takes two reads and
// three launches. `dense`: the batch strides are those of a dense
// [b0][b1][rows] stack, so a row's offset is its flat index times the row stride.
template <int EPV, int PRE>
__global__ void __launch_bounds__(256)
quant_shortrow_onepass(OnePassParams O, int64_t nbrow, int nvec, int dense) {
  constexpr int ES = 16 / EPV;
  constexpr int U = 4;
  const QParams& P = O.q;
  const DView& x = P.x;
  const int lane = threadIdx.x & 31;
  const int rows_per_warp = 32 / nvec;
  const int sub = lane / nvec, vi = lane % nvec;
  const int64_t warp_g = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * (blockDim.x >> 5);
  const int64_t groups = (nbrow + rows_per_warp - 1) / rows_per_warp;
  const float nz[4] = {0.f, 0.f, 0.f, 0.f};
  for (int64_t g0 = warp_g * U; g0 < groups; g0 += nwarps * U) {
    uint4 raw[U];
    int64_t brow[U];
    float pconst[U];
#pragma unroll
    for (int k = 0; k < U; ++k) {
      brow[k] = (g0 + k) * rows_per_warp + sub;
      raw[k] = make_uint4(0u, 0u, 0u, 0u);
      pconst[k] = 0.f;
      if (g0 + k < groups && brow[k] < nbrow) {
        int64_t off, poff = 0;
        if (dense) {
          off = brow[k] * x.sr;
          if constexpr (PRE == 1) {
            int64_t i0, i1, r;
            decode_brow(x, brow[k], i0, i1, r);
            poff = i0 * P.pre.sb0 + i1 * P.pre.sb1;
          }
        } else {
          int64_t i0, i1, r;
          decode_brow(x, brow[k], i0, i1, r);
          off = i0 * x.sb0 + i1 * x.sb1 + r * x.sr;
          poff = i0 * P.pre.sb0 + i1 * P.pre.sb1;
        }
        raw[k] = ldg16(x.ptr, off * ES + (int64_t)vi * 16);
        if constexpr (PRE == 1) pconst[k] = load1(P.pre.ptr, P.pre.dtype, poff);
      }
    }
    // The maxima of the U x rows_per_warp rows of this pass, then ONE scale
    // computation per row (two divisions, the costly part of this kernel) on
    // as many lanes as there are rows instead of one per row group and pass,
    // then the scales back to the lanes of their rows.
    float mk[U];
#pragma unroll
    for (int k = 0; k < U; ++k) {
      uint4 run = make_uint4(0u, 0u, 0u, 0u);
      packed_absmax<EPV>(run, raw[k], x.dtype);
      float m = packed_hmax<EPV>(run, x.dtype);
      for (int o = nvec >> 1; o > 0; o >>= 1) m = amax_nn(m, __shfl_xor_sync(0xffffffffu, m, o));
      if constexpr (PRE == 1) m = apply_pre_abs(m, pconst[k], P.t_dtype);
      mk[k] = m;
    }
    float sck[U], sinvk[U];
    if (U * rows_per_warp <= 32) {
      // lane L < U * rows_per_warp takes row (k, sub) = (L / rows_per_warp, L % rows_per_warp)
      float mine = 0.f;
#pragma unroll
      for (int k = 0; k < U; ++k) {
        const float t = __shfl_sync(0xffffffffu, mk[k], (lane % rows_per_warp) * nvec);
        if (lane / rows_per_warp == k) mine = t;
      }
      const float sc1 = scale_of_amax(mine, P.t_dtype, P.s_dtype, O.quant_bound, O.clipping_scale, O.po2);
      const float sinv1 = recip_of_scale(sc1, P.s_dtype);
      const int64_t my_row = (g0 + lane / rows_per_warp) * rows_per_warp + lane % rows_per_warp;
      if (lane < U * rows_per_warp && g0 + lane / rows_per_warp < groups && my_row < nbrow) {
        if (P.s_dtype == AQTB200_BF16) ((__nv_bfloat16*)O.scale_out)[my_row] = __float2bfloat16_rn(sc1);
        else ((float*)O.scale_out)[my_row] = sc1;
      }
#pragma unroll
      for (int k = 0; k < U; ++k) {
        sck[k] = __shfl_sync(0xffffffffu, sc1, k * rows_per_warp + sub);
        sinvk[k] = __shfl_sync(0xffffffffu, sinv1, k * rows_per_warp + sub);
      }
    } else {
#pragma unroll
      for (int k = 0; k < U; ++k) {
        sck[k] = scale_of_amax(mk[k], P.t_dtype, P.s_dtype, O.quant_bound, O.clipping_scale, O.po2);
        sinvk[k] = recip_of_scale(sck[k], P.s_dtype);
        if (g0 + k < groups && brow[k] < nbrow && vi == 0) {
          if (P.s_dtype == AQTB200_BF16)
            ((__nv_bfloat16*)O.scale_out)[brow[k]] = __float2bfloat16_rn(sck[k]);
          else
            ((float*)O.scale_out)[brow[k]] = sck[k];
        }
      }
    }
#pragma unroll
    for (int k = 0; k < U; ++k) {
      const bool ok = g0 + k < groups && brow[k] < nbrow;
      const float sinv = sinvk[k];
      const float sinv4[4] = {sinv, sinv, sinv, sinv};
      uint32_t outw[EPV / 4];
      if (EPV == 8 && (P.int_bf16 || P.fast_bf16)) {
        // all-bf16: packed multiplies, one rounding each (see bf16x2_to_fp8x2)
        const uint32_t s2 = pack_bf16x2(sinv, sinv), p2 = pack_bf16x2(pconst[k], pconst[k]);
        const uint32_t w[4] = {raw[k].x, raw[k].y, raw[k].z, raw[k].w};
        if (P.int_bf16) {
#pragma unroll
          for (int g = 0; g < EPV / 4; ++g)
            outw[g] = bf16x4_to_s8x4(w[(2 * g) & 3], w[(2 * g + 1) & 3], p2, p2, PRE == 1, s2, s2,
                                     nz, false, P.clip_bound);
        } else {
          const __nv_fp8_interpretation_t f8k = P.qdtype == AQTB200_E4M3 ? __NV_E4M3 : __NV_E5M2;
#pragma unroll
          for (int g = 0; g < EPV / 4; ++g)
            outw[g] = bf16x2_to_fp8x2(w[(2 * g) & 3], p2, PRE == 1, s2, f8k) |
                      (bf16x2_to_fp8x2(w[(2 * g + 1) & 3], p2, PRE == 1, s2, f8k) << 16);
        }
      } else {
        float v[EPV];
        unpack<EPV>(raw[k], x.dtype, v);
        if constexpr (PRE == 1) {
#pragma unroll
          for (int j = 0; j < EPV; ++j) v[j] = apply_pre(v[j], pconst[k], P.t_dtype);
        }
#pragma unroll
        for (int g = 0; g < EPV / 4; ++g) outw[g] = quant4(v + 4 * g, sinv4, nz, false, P);
      }
      if (ok) {
        uint8_t* qp = P.q + brow[k] * P.ldq + (int64_t)vi * EPV;
        if constexpr (EPV == 8) *(uint2*)qp = make_uint2(outw[0], outw[1]);
        else *(uint32_t*)qp = outw[0];
      }
    }
  }
}

// ---------------------------------------------------------------------------
// quantize, contraction contiguous: one thread per 16 output bytes.
template <bool VEC>
__global__ void __launch_bounds__(256)
quant_row_kernel(QParams P, int64_t units_per_row, int64_t total_units) {
  const DView& x = P.x;
  const bool has_pre = P.pre.ptr != nullptr;
  const bool has_noise = P.noise.ptr != nullptr;
  for (int64_t u = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
       u < total_units; u += (int64_t)gridDim.x * blockDim.x) {
    int64_t brow = u / units_per_row;
    int64_t c = (u % units_per_row) * 16;
    int64_t i0, i1, r;
    decode_brow(x, brow, i0, i1, r);
    const int64_t base = i0 * x.sb0 + i1 * x.sb1 + r * x.sr;
    const int64_t pbase = i0 * P.pre.sb0 + i1 * P.pre.sb1;
    const int64_t nbase = i0 * P.noise.sb0 + i1 * P.noise.sb1 + r * P.noise.sr;
    const float sinv = P.sinv[P.per_tensor ? 0 : brow];
    float v[16], nz[16];
    if (VEC) {
      loadN<16>(x.ptr, x.dtype, base + c, v);
      if (has_pre) {
        float p[16];
        if (P.pre_vec) {
          loadN<16>(P.pre.ptr, P.pre.dtype, pbase + c, p);
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            p[j] = load1(P.pre.ptr, P.pre.dtype, pbase + (c + j) * P.pre.sc);
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = apply_pre(v[j], p[j], P.t_dtype);
      }
      if (has_noise) {
        if (P.noise_vec) {
          loadN<16>(P.noise.ptr, AQTB200_F32, nbase + c, nz);
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            nz[j] = load1(P.noise.ptr, AQTB200_F32, nbase + (c + j) * P.noise.sc);
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        int64_t cj = c + j;
        bool in = cj < x.cols;
        v[j] = in ? load1(x.ptr, x.dtype, base + cj * x.sc) : 0.f;
        if (has_pre && in)
          v[j] = apply_pre(v[j], load1(P.pre.ptr, P.pre.dtype, pbase + cj * P.pre.sc),
                           P.t_dtype);
        nz[j] = (has_noise && in)
                    ? load1(P.noise.ptr, AQTB200_F32, nbase + cj * P.noise.sc)
                    : 0.f;
      }
    }
    uint8_t q[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      q[j] = (c + j < x.cols) ? quant1(v[j], sinv, nz[j], has_noise, P) : 0;
    }
    *(uint4*)(P.q + brow * P.ldq + c) = *(uint4*)q;
  }
}

// ---------------------------------------------------------------------------
// quantize + transpose, kept index contiguous in the input. Tile: 64 kept rows
// x 128 contraction indices; 256 threads, thread (tx,ty) = (tid%16, tid/16)
// owns rows 4*tx..4*tx+3 and contraction indices i*64 + 4*ty + e.
template <bool VEC>
__global__ void __launch_bounds__(256)
quant_col_kernel(QParams P, int64_t row_tiles, int64_t col_tiles,
                 int64_t total_units) {
  __shared__ uint32_t tile[64][33];
  const DView& x = P.x;
  const bool has_pre = P.pre.ptr != nullptr;
  const bool has_noise = P.noise.ptr != nullptr;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  for (int64_t u = blockIdx.x; u < total_units; u += gridDim.x) {
    int64_t ct = u % col_tiles;
    int64_t t = u / col_tiles;
    int64_t rt = t % row_tiles;
    int64_t b = t / row_tiles;
    int64_t i1 = b % x.b1, i0 = b / x.b1;
    const int64_t base = i0 * x.sb0 + i1 * x.sb1;
    const int64_t pbase = i0 * P.pre.sb0 + i1 * P.pre.sb1;
    const int64_t nbase = i0 * P.noise.sb0 + i1 * P.noise.sb1;
    const int64_t sbase = (i0 * x.b1 + i1) * x.rows;
    const int64_t r0 = rt * 64 + tx * 4;
    float sinv[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      sinv[j] = P.per_tensor ? P.sinv[0]
                             : (r0 + j < x.rows ? P.sinv[sbase + r0 + j] : 1.f);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      uint32_t word[4] = {0u, 0u, 0u, 0u};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int64_t c = ct * 128 + i * 64 + ty * 4 + e;
        if (c < x.cols && r0 < x.rows) {
          float v[4], nz[4] = {0.f, 0.f, 0.f, 0.f};
          if (VEC) {
            loadN<4>(x.ptr, x.dtype, base + c * x.sc + r0, v);
            if (has_noise) {
              if (P.noise_vec) {
                loadN<4>(P.noise.ptr, AQTB200_F32, nbase + c * P.noise.sc + r0, nz);
              } else {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                  nz[j] = load1(P.noise.ptr, AQTB200_F32,
                                nbase + c * P.noise.sc + (r0 + j) * P.noise.sr);
              }
            }
          } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              bool in = r0 + j < x.rows;
              v[j] = in ? load1(x.ptr, x.dtype, base + c * x.sc + (r0 + j) * x.sr) : 0.f;
              nz[j] = (in && has_noise)
                          ? load1(P.noise.ptr, AQTB200_F32,
                                  nbase + c * P.noise.sc + (r0 + j) * P.noise.sr)
                          : 0.f;
            }
          }
          float p = has_pre ? load1(P.pre.ptr, P.pre.dtype, pbase + c * P.pre.sc) : 0.f;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float w = has_pre ? apply_pre(v[j], p, P.t_dtype) : v[j];
            uint32_t qb = (r0 + j < x.rows) ? quant1(w, sinv[j], nz[j], has_noise, P) : 0u;
            word[j] |= qb << (8 * e);
          }
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) tile[tx * 4 + j][i * 16 + ty] = word[j];
    }
    __syncthreads();
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      const int id = tid + 256 * s;
      const int row = id >> 3, seg = id & 7;
      const int64_t gr = rt * 64 + row;
      const int64_t gc = ct * 128 + seg * 16;
      if (gr < x.rows && gc < P.ldq) {
        uint4 o;
        o.x = tile[row][seg * 4 + 0]; o.y = tile[row][seg * 4 + 1];
        o.z = tile[row][seg * 4 + 2]; o.w = tile[row][seg * 4 + 3];
        *(uint4*)(P.q + (sbase + gr) * P.ldq + gc) = o;
      }
    }
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------
// dequantize: out = cast_D(q) * scale (aqt_tensor.py:179-198, single scale).
struct DeqParams {
  DView q, s;
  int d_dtype;
  void* out;  // contiguous [b0][b1][rows][cols]
};

__global__ void dequant_kernel(DeqParams D, int64_t total) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    int64_t c = i % D.q.cols;
    int64_t t = i / D.q.cols;
    int64_t r = t % D.q.rows;
    t /= D.q.rows;
    int64_t i1 = t % D.q.b1, i0 = t / D.q.b1;
    float v = load1(D.q.ptr, D.q.dtype, i0 * D.q.sb0 + i1 * D.q.sb1 + r * D.q.sr + c * D.q.sc);
    v = round_to(v, D.d_dtype);  // int32 -> f32 happened in load1 (RNE)
    if (D.s.ptr != nullptr) {
      float s = load1(D.s.ptr, D.s.dtype, i0 * D.s.sb0 + i1 * D.s.sb1 + r * D.s.sr + c * D.s.sc);
      int wide = (D.d_dtype == AQTB200_F32 || D.s.dtype == AQTB200_F32) ? AQTB200_F32 : AQTB200_BF16;
      v = round_to(round_to(__fmul_rn(v, s), wide), D.d_dtype);
    }
    if (D.d_dtype == AQTB200_BF16)
      ((__nv_bfloat16*)D.out)[i] = __float2bfloat16_rn(v);
    else
      ((float*)D.out)[i] = v;
  }
}

// ===========================================================================
// One read of the cotangent for BOTH gradient dots when the scales are per row
// (per token / per channel), the forward scales folded into it vary along
// the contraction and stochastic-rounding noise is added: the batched,
// per-channel counterpart of quant_pair_kernel.
//
// The backward pass quantizes the cotangent g twice (aqt_dot_general.py:
// 1206-1217): for dlhs along its last index, for drhs along the one before.
// With x = g viewed as [b][c][r] (r contiguous):
//   output S [b][c][r]  (x's orientation; contraction index r)
//       v = round(x * pre_s[b][r]);  scale_s[b][c] = max_r |v| / bound
//   output T [b][r][c]  (transposed; contraction index c)
//       v = round(x * pre_t[b][c]);  scale_t[b][r] = max_c |v| / bound
// absmax_dual_kernel takes both families of maxima in one pass over x;
// quant_dual_kernel writes both int8 layouts in one more pass, each with its
// own noise tensor. bf16 input, bf16 arithmetic (packed), int8 outputs.
struct DualParams {
  DView x;                 // bf16, sr == 1; rows % 8 == 0
  const void* pre_t;       // bf16 prescale of output T, indexed [b0][b1][c]; null = none
  int64_t pt_b0, pt_b1, pt_c;
  const void* pre_s;       // bf16 prescale of output S, indexed [b0][b1][r]; null = none
  int64_t ps_b0, ps_b1, ps_r;
  const float* noise_t;    // f32, x's layout [b][c][r]; null = none
  const float* noise_s;
  uint32_t* amax_t;        // [b][rows] f32 bits
  uint32_t* amax_s;        // [b][cols]
  const float* sinv_t;     // [b][rows] reciprocal scales (already rounded to bf16)
  const float* sinv_s;     // [b][cols]
  float clip_t, clip_s;
  uint8_t* q_t;            // [b][rows][ld_t]
  uint8_t* q_s;            // [b][cols][ld_s]
  int64_t ld_t, ld_s;
};

__device__ __forceinline__ uint32_t ld_bf16_pair(const void* base, int64_t i0, int64_t i1) {
  const unsigned short* p = (const unsigned short*)base;
  return (uint32_t)__ldg(p + i0) | ((uint32_t)__ldg(p + i1) << 16);
}
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
  const __nv_bfloat162 r = __hmul2(*(const __nv_bfloat162*)&a, *(const __nv_bfloat162*)&b);
  return *(const uint32_t*)&r;
}

// Block = one strip: 128 rows (r) by ALL columns (c) of one batch element, walked
// 128 columns at a time. Thread (tx, ty): rows r0 + 8 tx .. +7 (one 16-byte
// vector), columns ty*4 + e (+64) of each 128-column tile. The maxima over c
// (amax_t, per row) stay in registers for the whole strip and are written once;
// the maxima over r (amax_s, per column) are folded over the 16 row groups of
// the block with shuffles and merged across strips with one atomic per column.
template <bool PRE_T, bool PRE_S>
__global__ void __launch_bounds__(256)
absmax_dual_kernel(DualParams P, int64_t row_tiles, int64_t col_tiles, int64_t total_strips) {
  __shared__ uint32_t srow[16][128];  // [ty][row in strip]: packed halves folded later
  const DView& x = P.x;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  for (int64_t u = blockIdx.x; u < total_strips; u += gridDim.x) {
    const int64_t rt = u % row_tiles;
    const int64_t b = u / row_tiles;
    const int64_t i1 = b % x.b1, i0 = b / x.b1;
    const int64_t r0 = rt * 128 + tx * 8;
    const bool row_ok = r0 < x.rows;
    const char* xp = (const char*)x.ptr + (i0 * x.sb0 + i1 * x.sb1 + (row_ok ? r0 : 0)) * 2;
    uint32_t ps[4] = {0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u};
    if (PRE_S && row_ok) {
      const int64_t pb = i0 * P.ps_b0 + i1 * P.ps_b1;
#pragma unroll
      for (int j = 0; j < 4; ++j)
        ps[j] = ld_bf16_pair(P.pre_s, pb + (r0 + 2 * j) * P.ps_r, pb + (r0 + 2 * j + 1) * P.ps_r);
    }
    uint32_t run_t[4] = {0u, 0u, 0u, 0u};  // per row pair, max over every column of the strip
    for (int64_t ct = 0; ct < col_tiles; ++ct) {
      uint4 raw[2][4];
      uint32_t ptv[2][4];  // the columns' prescales, requested together with the data
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int64_t c = ct * 128 + i * 64 + ty * 4 + e;
          raw[i][e] = (row_ok && c < x.cols) ? ldg16(xp, c * x.sc * 2) : make_uint4(0u, 0u, 0u, 0u);
          ptv[i][e] = 0x3f80u;
          if (PRE_T && c < x.cols)
            ptv[i][e] = __ldg((const unsigned short*)P.pre_t + i0 * P.pt_b0 + i1 * P.pt_b1 + c * P.pt_c);
        }
#pragma unroll
      for (int i = 0; i < 2; ++i) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int64_t c = ct * 128 + i * 64 + ty * 4 + e;
          const uint32_t w[4] = {raw[i][e].x, raw[i][e].y, raw[i][e].z, raw[i][e].w};
          const uint32_t pt2 = ptv[i][e] | (ptv[i][e] << 16);
          uint32_t m2 = 0u;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t vt = PRE_T ? hmul2_u32(w[j], pt2) : w[j];
            run_t[j] = __vmaxu2(run_t[j], vt & 0x7fff7fffu);
            const uint32_t vs = PRE_S ? hmul2_u32(w[j], ps[j]) : w[j];
            m2 = __vmaxu2(m2, vs & 0x7fff7fffu);
          }
          // this thread's 8 rows of column c -> fold over the 16 row groups
          uint32_t m = max(m2 & 0xffffu, m2 >> 16);
#pragma unroll
          for (int o = 8; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
          if (tx == 0 && m != 0u && c < x.cols)
            atomicMax(P.amax_s + b * x.cols + c, m << 16);
        }
      }
    }
    // rows: fold the 16 column groups (ty) through shared memory
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      srow[ty][tx * 8 + 2 * j] = run_t[j] & 0xffffu;
      srow[ty][tx * 8 + 2 * j + 1] = run_t[j] >> 16;
    }
    __syncthreads();
    if (tid < 128) {
      uint32_t m = 0u;
#pragma unroll
      for (int k = 0; k < 16; ++k) m = max(m, srow[k][tid]);
      const int64_t r = rt * 128 + tid;
      if (r < x.rows) P.amax_t[b * x.rows + r] = m << 16;  // the strip owns these rows
    }
    __syncthreads();
  }
}

// One tile (128 r x 128 c) per step, same thread layout as quant_pair_kernel.
template <bool PRE_T, bool PRE_S, bool NOISE>
__global__ void __launch_bounds__(256, 2)
quant_dual_kernel(DualParams P, int64_t row_tiles, int64_t col_tiles, int64_t total_units) {
  constexpr int EPV = 8, TR = 16 * EPV;
  __shared__ __align__(16) uint32_t tile[TR][32];
  const DView& x = P.x;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  for (int64_t u = blockIdx.x; u < total_units; u += gridDim.x) {
    const int64_t rt = u % row_tiles;
    int64_t t = u / row_tiles;
    const int64_t ct = t % col_tiles;
    const int64_t b = t / col_tiles;
    const int64_t i1 = b % x.b1, i0 = b / x.b1;
    const int64_t r0 = rt * TR + tx * EPV;
    const bool row_ok = r0 < x.rows;  // rows % 8 == 0: a vector is all in or all out
    const int64_t xoff = i0 * x.sb0 + i1 * x.sb1 + (row_ok ? r0 : 0);  // elements
    const char* xp = (const char*)x.ptr + xoff * 2;
    uint8_t* qs_base = P.q_s + (b * x.cols + ct * 128 + ty * 4) * P.ld_s + r0;
    // per-row constants of this thread: prescale of S and reciprocal scale of T
    uint32_t ps[4] = {0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u};
    uint32_t it[4] = {0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u};
    if (row_ok) {
      if (PRE_S) {
        const int64_t pb = i0 * P.ps_b0 + i1 * P.ps_b1;
#pragma unroll
        for (int j = 0; j < 4; ++j)
          ps[j] = ld_bf16_pair(P.pre_s, pb + (r0 + 2 * j) * P.ps_r, pb + (r0 + 2 * j + 1) * P.ps_r);
      }
      const float4 a = __ldg((const float4*)(P.sinv_t + b * x.rows + r0));
      const float4 c4 = __ldg((const float4*)(P.sinv_t + b * x.rows + r0 + 4));
      it[0] = pack_bf16x2(a.x, a.y); it[1] = pack_bf16x2(a.z, a.w);
      it[2] = pack_bf16x2(c4.x, c4.y); it[3] = pack_bf16x2(c4.z, c4.w);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      uint4 raw[4];
      uint4 nt[4][2], ns[4][2];
      uint32_t ptv[4];  // per column: prescale of T (bf16 bits) ...
      float isv[4];     // ... and reciprocal scale of S
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int64_t c = ct * 128 + i * 64 + ty * 4 + e;
        const bool in = row_ok && c < x.cols;
        raw[e] = in ? ldg16(xp, c * x.sc * 2) : make_uint4(0u, 0u, 0u, 0u);
        ptv[e] = 0x3f80u;
        isv[e] = 1.f;
        if (in) {
          if (PRE_T)
            ptv[e] = __ldg((const unsigned short*)P.pre_t + i0 * P.pt_b0 + i1 * P.pt_b1 + c * P.pt_c);
          isv[e] = __ldg(P.sinv_s + b * x.cols + c);
        }
        if (NOISE) {
          const int64_t no = (xoff + c * x.sc) * 4;
          nt[e][0] = in ? ldg16(P.noise_t, no) : make_uint4(0u, 0u, 0u, 0u);
          nt[e][1] = in ? ldg16(P.noise_t, no + 16) : make_uint4(0u, 0u, 0u, 0u);
          ns[e][0] = in ? ldg16(P.noise_s, no) : make_uint4(0u, 0u, 0u, 0u);
          ns[e][1] = in ? ldg16(P.noise_s, no + 16) : make_uint4(0u, 0u, 0u, 0u);
        }
      }
      uint32_t q4[4][2];  // transposed output: [column e][row group g]
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int64_t c = ct * 128 + i * 64 + ty * 4 + e;
        const bool in = row_ok && c < x.cols;
        const uint32_t pt2 = ptv[e] | (ptv[e] << 16);
        const uint32_t is2 = pack_bf16x2(isv[e], isv[e]);
        const uint32_t w[4] = {raw[e].x, raw[e].y, raw[e].z, raw[e].w};
        float fnt[8], fns[8];
        if (NOISE) {
          const uint32_t a[8] = {nt[e][0].x, nt[e][0].y, nt[e][0].z, nt[e][0].w,
                                 nt[e][1].x, nt[e][1].y, nt[e][1].z, nt[e][1].w};
          const uint32_t c8[8] = {ns[e][0].x, ns[e][0].y, ns[e][0].z, ns[e][0].w,
                                  ns[e][1].x, ns[e][1].y, ns[e][1].z, ns[e][1].w};
#pragma unroll
          for (int k = 0; k < 8; ++k) { fnt[k] = __uint_as_float(a[k]); fns[k] = __uint_as_float(c8[k]); }
        }
        // output T: prescale by column, reciprocal scale by row
        const uint32_t qt_lo = bf16x4_to_s8x4(w[0], w[1], pt2, pt2, PRE_T, it[0], it[1], fnt, NOISE, P.clip_t);
        const uint32_t qt_hi = bf16x4_to_s8x4(w[2], w[3], pt2, pt2, PRE_T, it[2], it[3], fnt + 4, NOISE, P.clip_t);
        // output S: prescale by row, reciprocal scale by column
        const uint32_t qs_lo = bf16x4_to_s8x4(w[0], w[1], ps[0], ps[1], PRE_S, is2, is2, fns, NOISE, P.clip_s);
        const uint32_t qs_hi = bf16x4_to_s8x4(w[2], w[3], ps[2], ps[3], PRE_S, is2, is2, fns + 4, NOISE, P.clip_s);
        q4[e][0] = in ? qt_lo : 0u;
        q4[e][1] = in ? qt_hi : 0u;
        if (in) {
          // same orientation: rows r0..r0+7 of column c are 8 contiguous bytes
          *(uint2*)(qs_base + (int64_t)(i * 64 + e) * P.ld_s) = make_uint2(qs_lo, qs_hi);
        }
      }
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        const uint32_t cols4[4] = {q4[0][g], q4[1][g], q4[2][g], q4[3][g]};
        uint32_t rows4[4];
        transpose4x4(cols4, rows4);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          tile[tx * EPV + 4 * g + j][(i * 16 + ty + 4 * tx) & 31] = rows4[j];
      }
    }
    __syncthreads();
#pragma unroll
    for (int s2 = 0; s2 < TR / 32; ++s2) {
      const int id = tid + 256 * s2;
      const int row = id >> 3, seg = id & 7;
      const int64_t gr = rt * TR + row;
      const int64_t gc = ct * 128 + seg * 16;
      if (gr < x.rows && gc < P.ld_t) {
        const uint4 o = *(const uint4*)&tile[row][(seg * 4 + 4 * (row / EPV)) & 31];
        *(uint4*)(P.q_t + (b * x.rows + gr) * P.ld_t + gc) = o;
      }
    }
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------
// host side

// SM count of the CURRENT device (a process may drive several).
static int g_sm_count[64] = {0};
int sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  dev &= 63;
  if (g_sm_count[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0)
      g_sm_count[dev] = n;
    else
      g_sm_count[dev] = 148;
  }
  return g_sm_count[dev];
}

static bool is_float_dt(int dt) { return dt == AQTB200_F32 || dt == AQTB200_BF16; }
static bool is_q_dt(int dt) { return dt == AQTB200_S8 || dt == AQTB200_E4M3 || dt == AQTB200_E5M2; }

static int64_t n_scales(const aqtb200_view* x, const aqtb200_quant_spec* s) {
  return s->per_tensor ? 1 : x->b0 * x->b1 * x->rows;
}

static size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

static int validate(const aqtb200_view* x, const aqtb200_view* pre,
                    const aqtb200_view* noise, const aqtb200_quant_spec* spec,
                    bool need_q) {
  AQT_REQUIRE(x != nullptr && spec != nullptr, AQTB200_EINVAL, "null view or spec");
  AQT_REQUIRE(x->b0 >= 0 && x->b1 >= 0 && x->rows >= 0 && x->cols >= 0,
              AQTB200_EINVAL, "negative extent");
  int64_t total = x->b0 * x->b1 * x->rows * x->cols;
  AQT_REQUIRE(total == 0 || x->ptr != nullptr, AQTB200_EINVAL, "null input pointer");
  AQT_REQUIRE(is_float_dt(x->dtype) || is_q_dt(x->dtype), AQTB200_EINVAL,
              "input dtype %d is not f32/bf16/s8/e4m3/e5m2", x->dtype);
  AQT_REQUIRE(is_float_dt(spec->compute_dtype) && is_float_dt(spec->scale_dtype),
              AQTB200_EINVAL, "compute/scale dtype must be f32 or bf16");
  AQT_REQUIRE(!(x->dtype == AQTB200_F32 && spec->compute_dtype == AQTB200_BF16),
              AQTB200_EINVAL, "f32 input cannot have bf16 compute dtype");
  AQT_REQUIRE(spec->kind == AQTB200_NUM_INT || spec->kind == AQTB200_NUM_FP8,
              AQTB200_EUNSUPPORTED,
              "numerics kind %d: only IntSymmetric and Fp8Numerics are quantized on the device",
              spec->kind);
  if (need_q) {
    if (spec->kind == AQTB200_NUM_INT)
      AQT_REQUIRE(spec->qdtype == AQTB200_S8, AQTB200_EUNSUPPORTED, "int numerics need an int8 container");
    else
      AQT_REQUIRE(spec->qdtype == AQTB200_E4M3 || spec->qdtype == AQTB200_E5M2,
                  AQTB200_EUNSUPPORTED, "fp8 numerics need e4m3 or e5m2");
    AQT_REQUIRE(spec->clip_bound > 0.f, AQTB200_EINVAL, "clip_bound must be positive");
  }
  AQT_REQUIRE(spec->quant_bound > 0.f, AQTB200_EINVAL, "quant_bound must be positive");
  if (pre && pre->ptr)
    AQT_REQUIRE(is_float_dt(pre->dtype), AQTB200_EINVAL, "prescale must be f32 or bf16");
  if (noise && noise->ptr) {
    AQT_REQUIRE(noise->dtype == AQTB200_F32, AQTB200_EINVAL, "noise must be f32");
    AQT_REQUIRE(spec->kind == AQTB200_NUM_INT, AQTB200_EUNSUPPORTED,
                "noise-tensor stochastic rounding applies to int numerics only");
  }
  return 0;
}

static bool aligned(const void* p, size_t a) { return ((uintptr_t)p % a) == 0; }
static bool mult(int64_t v, int64_t m) { return v % m == 0; }

// Can every 16-element group along the contiguous contraction index be loaded
// with 16-byte vector loads?
static bool row_vec_ok(const DView& v, int64_t cols) {
  int es = dtype_size(v.dtype);
  int64_t g = 16 / es > 0 ? 16 / es : 1;  // elements per 16 bytes
  return v.sc == 1 && mult(cols, 16) && aligned(v.ptr, 16) && mult(v.sr, g) &&
         mult(v.sb0, g) && mult(v.sb1, g);
}
// Can 4 consecutive kept rows be loaded as one vector?
static bool col_vec_ok(const DView& v, int64_t rows) {
  int es = dtype_size(v.dtype);
  int64_t g = 4;  // 4 elements: 16/8/4 bytes, natural alignment 4*es
  (void)es;
  return v.sr == 1 && mult(rows, 4) && aligned(v.ptr, 16) && mult(v.sc, g) &&
         mult(v.sb0, g) && mult(v.sb1, g);
}

// 16-byte vectors of `epv` consecutive kept rows at every contraction index?
static bool col_fast_ok(const DView& v, int64_t rows, int epv) {
  return v.sr == 1 && mult(rows, epv) && aligned(v.ptr, 16) && mult(v.sc, epv) &&
         mult(v.sb0, epv) && mult(v.sb1, epv);
}

static int grid_for(int64_t units, int per_sm) {
  int64_t cap = (int64_t)sm_count() * per_sm;
  return (int)std::max<int64_t>(1, std::min<int64_t>(units, cap));
}

static int run(const aqtb200_view* xv, const aqtb200_view* prev,
               const aqtb200_view* noisev, const aqtb200_quant_spec* spec,
               const void* scale_in, void* q_out, void* scale_out,
               void* workspace, size_t workspace_bytes, cudaStream_t st,
               bool want_q, float* amax_only_out = nullptr) {
  int rc = validate(xv, prev, noisev, spec, want_q);
  if (rc) return rc;
  // Kept index contiguous and the inner batch index contiguous right above it
  // (e.g. the d of a [b, t, h, d] operand contracted over t, batched over b and
  // h): the batch index is folded into the kept index. Scales, maxima and the
  // quantized copy are laid out [b0][b1][rows] either way; the column kernels
  // then read 512-byte-wide strips instead of rows of `rows` elements (128
  // bytes for the attention operands, a quarter of every warp).
  aqtb200_view x_merged, n_merged;
  const bool no_pre = prev == nullptr || prev->ptr == nullptr;
  const bool has_noise_view = noisev != nullptr && noisev->ptr != nullptr;
  if (xv->b1 > 1 && xv->row_stride == 1 && xv->col_stride != 1 && xv->b1_stride == xv->rows &&
      no_pre &&
      (!has_noise_view || (noisev->row_stride == 1 && noisev->b1_stride == noisev->rows &&
                           noisev->rows == xv->rows && noisev->b1 == xv->b1))) {
    x_merged = *xv;
    x_merged.rows = xv->rows * xv->b1;
    x_merged.b1 = 1;
    x_merged.b1_stride = 0;
    xv = &x_merged;
    if (has_noise_view) {
      n_merged = *noisev;
      n_merged.rows = noisev->rows * noisev->b1;
      n_merged.b1 = 1;
      n_merged.b1_stride = 0;
      noisev = &n_merged;
    }
  }
  const int64_t ns = n_scales(xv, spec);
  const int64_t nbrow = xv->b0 * xv->b1 * xv->rows;
  const int64_t total = nbrow * xv->cols;
  if (ns == 0) return 0;
  if (amax_only_out != nullptr) {
    workspace = amax_only_out;  // the maxima land in the caller's buffer
  } else {
    size_t need = aqtb200_quantize_workspace_bytes(xv, spec);
    AQT_REQUIRE(workspace != nullptr && workspace_bytes >= need && aligned(workspace, 256),
                AQTB200_EWORKSPACE, "workspace: need %zu bytes, 256-byte aligned (got %zu)",
                need, workspace_bytes);
    AQT_REQUIRE(scale_out != nullptr || scale_in != nullptr, AQTB200_EINVAL,
                "scale_out is null");
  }
  if (want_q) AQT_REQUIRE(q_out != nullptr && aligned(q_out, 16), AQTB200_EINVAL,
                          "q_out null or not 16-byte aligned");

  QParams P{};
  P.x = to_dview(xv);
  P.pre = to_dview(prev);
  P.noise = to_dview(noisev);
  P.t_dtype = spec->compute_dtype;
  P.s_dtype = spec->scale_dtype;
  P.y_dtype = (P.t_dtype == AQTB200_F32 || P.s_dtype == AQTB200_F32) ? AQTB200_F32 : AQTB200_BF16;
  P.kind = spec->kind;
  P.qdtype = spec->qdtype;
  P.clip_bound = spec->clip_bound;
  P.per_tensor = spec->per_tensor;
  P.amax = (uint32_t*)workspace;
  P.sinv = (float*)((char*)workspace + align256((size_t)ns * 4));
  P.q = (uint8_t*)q_out;
  P.ldq = aqtb200_round_up(xv->cols, 16);
  // Row mode reads along the contraction index; its scalar kernel takes any
  // strides, so it also serves degenerate and doubly-strided views.
  const bool row_mode = !(P.x.sr == 1 && P.x.sc != 1);
  P.pre_vec = P.pre.ptr && row_vec_ok({P.pre.ptr, P.pre.dtype, 1, 1, 1, 1,
                                       P.pre.sb0, P.pre.sb1, 16, P.pre.sc}, xv->cols);
  if (P.noise.ptr)
    P.noise_vec = row_mode ? row_vec_ok(P.noise, xv->cols) : col_vec_ok(P.noise, xv->rows);
  const int epv = 16 / dtype_size(P.x.dtype);
  const bool pre_is_scalar = P.pre.ptr == nullptr ||
                             (P.pre.sb0 == 0 && P.pre.sb1 == 0 && (P.pre.sc == 0 || xv->cols <= 1));
  P.use_lut = dtype_size(P.x.dtype) == 1 && P.per_tensor && P.noise.ptr == nullptr && pre_is_scalar;
  P.fast_bf16 = P.x.dtype == AQTB200_BF16 && P.t_dtype == AQTB200_BF16 &&
                P.s_dtype == AQTB200_BF16 && P.kind == AQTB200_NUM_FP8 && P.noise.ptr == nullptr &&
                (P.pre.ptr == nullptr || P.pre.dtype == AQTB200_BF16 || true);
  P.pre_bf16 = P.pre.ptr != nullptr && P.x.dtype == AQTB200_BF16 && P.pre.dtype == AQTB200_BF16 &&
               P.t_dtype == AQTB200_BF16;
  P.int_bf16 = P.x.dtype == AQTB200_BF16 && P.t_dtype == AQTB200_BF16 && P.s_dtype == AQTB200_BF16 &&
               P.kind == AQTB200_NUM_INT && (P.pre.ptr == nullptr || P.pre.dtype == AQTB200_BF16);
  P.s8_bf16 = P.x.dtype == AQTB200_S8 && P.t_dtype == AQTB200_BF16 && P.s_dtype == AQTB200_BF16 &&
              P.kind == AQTB200_NUM_INT && (P.pre.ptr == nullptr || P.pre.dtype == AQTB200_BF16);
  // prescale class: 0 none, 1 constant along the contraction index, 2 varying
  const int pre_kind = P.pre.ptr == nullptr ? 0 : (P.pre.sc == 0 || xv->cols <= 1 ? 1 : 2);
  const bool fast_row = row_mode && row_vec_ok(P.x, xv->cols);
  const bool fast_col = !row_mode && col_fast_ok(P.x, xv->rows, epv);

#define AQT_DISPATCH_EPV_PRE(KERNEL, GRID, BLOCK, ...)                                   \
  do {                                                                                   \
    if (epv == 4) {                                                                      \
      if (pre_kind == 0) KERNEL<4, 0><<<GRID, BLOCK, 0, st>>>(__VA_ARGS__);              \
      else if (pre_kind == 1) KERNEL<4, 1><<<GRID, BLOCK, 0, st>>>(__VA_ARGS__);         \
      else KERNEL<4, 2><<<GRID, BLOCK, 0, st>>>(__VA_ARGS__);                            \
    } else if (epv == 8) {                                                               \
      if (pre_kind == 0) KERNEL<8, 0><<<GRID, BLOCK, 0, st>>>(__VA_ARGS__);              \
      else if (pre_kind == 1) KERNEL<8, 1><<<GRID, BLOCK, 0, st>>>(__VA_ARGS__);         \
      else KERNEL<8, 2><<<GRID, BLOCK, 0, st>>>(__VA_ARGS__);                            \
    } else {                                                                             \
      if (pre_kind == 0) KERNEL<16, 0><<<GRID, BLOCK, 0, st>>>(__VA_ARGS__);             \
      else if (pre_kind == 1) KERNEL<16, 1><<<GRID, BLOCK, 0, st>>>(__VA_ARGS__);        \
      else KERNEL<16, 2><<<GRID, BLOCK, 0, st>>>(__VA_ARGS__);                           \
    }                                                                                    \
  } while (0)

  // Per-row scales over short rows (several rows per warp): one kernel, one read.
  {
    const int64_t row_vecs = xv->cols / epv;
    if (scale_in == nullptr && want_q && amax_only_out == nullptr && fast_row && epv != 16 &&
        !P.per_tensor && P.noise.ptr == nullptr && pre_kind != 2 && xv->cols % 16 == 0 &&
        xv->cols % epv == 0 && row_vecs >= 1 && row_vecs <= 32 && (row_vecs & (row_vecs - 1)) == 0 &&
        nbrow > 0) {
      OnePassParams O{};
      O.q = P;
      O.quant_bound = spec->quant_bound; O.clipping_scale = spec->clipping_scale;
      O.po2 = spec->po2_scale; O.scale_out = scale_out;
      const int dense = (xv->b1 <= 1 || P.x.sb1 == xv->rows * P.x.sr) &&
                        (xv->b0 <= 1 || P.x.sb0 == xv->b1 * xv->rows * P.x.sr);
      const int64_t groups = (nbrow + (32 / row_vecs) - 1) / (32 / row_vecs);
      const int grid = grid_for((groups + 31) / 32, 8);
      if (epv == 4) {
        if (pre_kind == 0) quant_shortrow_onepass<4, 0><<<grid, 256, 0, st>>>(O, nbrow, (int)row_vecs, dense);
        else quant_shortrow_onepass<4, 1><<<grid, 256, 0, st>>>(O, nbrow, (int)row_vecs, dense);
      } else {
        if (pre_kind == 0) quant_shortrow_onepass<8, 0><<<grid, 256, 0, st>>>(O, nbrow, (int)row_vecs, dense);
        else quant_shortrow_onepass<8, 1><<<grid, 256, 0, st>>>(O, nbrow, (int)row_vecs, dense);
      }
      AQT_CUDA_OK(cudaGetLastError()); count_launch();
      return 0;
    }
  }
  // Per-row scales over rows that fit in a block: one kernel, one read.
  {
    const int nv = epv == 16 ? 1 : 16 / epv;     // input vectors per 16 outputs
    const int umax = 4 / nv > 0 ? 4 / nv : 1;    // 16-output units per thread
    if (scale_in == nullptr && want_q && amax_only_out == nullptr && fast_row && epv != 16 &&
        !P.per_tensor && P.noise.ptr == nullptr && pre_kind != 2 && xv->cols >= 1024 &&
        xv->cols % 16 == 0 && xv->cols / 16 <= 256 * (int64_t)umax && nbrow > 0) {
      OnePassParams O{};
      O.q = P;
      O.quant_bound = spec->quant_bound; O.clipping_scale = spec->clipping_scale;
      O.po2 = spec->po2_scale; O.scale_out = scale_out;
      const int grid = grid_for(nbrow, 8);
      if (epv == 4) {
        if (pre_kind == 0) quant_row_onepass<4, 0><<<grid, 256, 0, st>>>(O, nbrow);
        else quant_row_onepass<4, 1><<<grid, 256, 0, st>>>(O, nbrow);
      } else {
        if (pre_kind == 0) quant_row_onepass<8, 0><<<grid, 256, 0, st>>>(O, nbrow);
        else quant_row_onepass<8, 1><<<grid, 256, 0, st>>>(O, nbrow);
      }
      AQT_CUDA_OK(cudaGetLastError()); count_launch();
      return 0;
    }
  }
  if (scale_in == nullptr) {
    AQT_CUDA_OK(cudaMemsetAsync(P.amax, 0, (size_t)ns * 4, st));
    if (total > 0) {
      const int64_t row_vecs = xv->cols / (16 / dtype_size(P.x.dtype));
      if (fast_row && pre_kind != 2 && xv->cols % (16 / dtype_size(P.x.dtype)) == 0 &&
          row_vecs >= 1 && row_vecs <= 16 && (row_vecs & (row_vecs - 1)) == 0) {
        const int64_t groups = (nbrow + (32 / row_vecs) - 1) / (32 / row_vecs);
        const int grid = grid_for((groups + 31) / 32, 8);
        if (epv == 4) {
          if (pre_kind == 0) absmax_shortrow_fast<4, 0><<<grid, 256, 0, st>>>(P, nbrow, (int)row_vecs);
          else absmax_shortrow_fast<4, 1><<<grid, 256, 0, st>>>(P, nbrow, (int)row_vecs);
        } else if (epv == 8) {
          if (pre_kind == 0) absmax_shortrow_fast<8, 0><<<grid, 256, 0, st>>>(P, nbrow, (int)row_vecs);
          else absmax_shortrow_fast<8, 1><<<grid, 256, 0, st>>>(P, nbrow, (int)row_vecs);
        } else {
          if (pre_kind == 0) absmax_shortrow_fast<16, 0><<<grid, 256, 0, st>>>(P, nbrow, (int)row_vecs);
          else absmax_shortrow_fast<16, 1><<<grid, 256, 0, st>>>(P, nbrow, (int)row_vecs);
        }
      } else if (fast_row && (pre_kind != 2 || P.pre_vec)) {
        // a (row, chunk) unit is one warp's work: shorter chunks when the whole
        // tensor would otherwise occupy a handful of warps (decode-time activations)
        int chunk_elems = kFastRowChunk;
        while (chunk_elems > 1024 &&
               nbrow * ((xv->cols + chunk_elems - 1) / chunk_elems) < (int64_t)sm_count() * 8)
          chunk_elems /= 2;
        int64_t chunks = (xv->cols + chunk_elems - 1) / chunk_elems;
        int64_t units = nbrow * chunks;
        int grid = grid_for((units + 7) / 8, 8);
        AQT_DISPATCH_EPV_PRE(absmax_row_fast, grid, 256, P, chunks, units, chunk_elems);
      } else if (row_mode) {
        int64_t chunks = (xv->cols + kRowChunk - 1) / kRowChunk;
        int64_t units = nbrow * chunks;
        int grid = grid_for((units + 7) / 8, 8);
        absmax_row_kernel<false><<<grid, 256, 0, st>>>(P, chunks, units);
      } else if (fast_col) {
        // lanes of a warp along the kept rows: all 32, or the power of two that
        // covers the rows when there are fewer than 32 vectors of them
        int row_lanes = 32;
        while (row_lanes > 1 && (int64_t)(row_lanes / 2) * epv >= xv->rows) row_lanes /= 2;
        int64_t rbs = (xv->rows + row_lanes * epv - 1) / (row_lanes * epv);
        int64_t ccs = (xv->cols + kFastColChunk - 1) / kFastColChunk;
        int64_t units = xv->b0 * xv->b1 * rbs * ccs;
        int grid = grid_for(units, 8);
        dim3 block(32, 8);
        AQT_DISPATCH_EPV_PRE(absmax_col_fast, grid, block, P, rbs, ccs, units, row_lanes);
      } else {
        bool vec = col_vec_ok(P.x, xv->rows);
        int64_t rows_per_block = 32 * (vec ? 4 : 1);
        int64_t rbs = (xv->rows + rows_per_block - 1) / rows_per_block;
        int64_t ccs = (xv->cols + kColChunk - 1) / kColChunk;
        int64_t units = xv->b0 * xv->b1 * rbs * ccs;
        int grid = grid_for(units, 8);
        dim3 block(32, 8);
        if (vec)
          absmax_col_kernel<true><<<grid, block, 0, st>>>(P, rbs, ccs, units);
        else
          absmax_col_kernel<false><<<grid, block, 0, st>>>(P, rbs, ccs, units);
      }
      AQT_CUDA_OK(cudaGetLastError()); count_launch();
    }
  }
  if (amax_only_out != nullptr) return 0;
  FinalizeParams F{};
  F.amax = P.amax; F.scale_in = scale_in; F.scale_out = scale_out; F.sinv = P.sinv;
  F.n = ns; F.t_dtype = P.t_dtype; F.s_dtype = P.s_dtype;
  F.quant_bound = spec->quant_bound; F.clipping_scale = spec->clipping_scale;
  F.po2 = spec->po2_scale;
  finalize_scale_kernel<<<(int)((ns + 255) / 256), 256, 0, st>>>(F);
  AQT_CUDA_OK(cudaGetLastError()); count_launch();
  if (!want_q || nbrow == 0) return 0;

  if (fast_row) {
    int64_t upr = P.ldq / 16;
    int64_t units = nbrow * upr;
    int grid = grid_for((units + 511) / 512, 8);
    AQT_DISPATCH_EPV_PRE(quant_row_fast, grid, 256, P, upr, units);
  } else if (row_mode) {
    int64_t upr = P.ldq / 16;
    int64_t units = nbrow * upr;
    int grid = grid_for((units + 255) / 256, 8);
    quant_row_kernel<false><<<grid, 256, 0, st>>>(P, upr, units);
  } else if (fast_col) {
    int64_t rts = (xv->rows + 16 * epv - 1) / (16 * epv);
    int64_t cts = (P.ldq + 127) / 128;
    int64_t units = xv->b0 * xv->b1 * rts * cts;
    int grid = grid_for(units, 4);
    if (epv == 16 && P.s8_bf16 && !P.use_lut && (P.noise.ptr == nullptr || P.noise_vec)) {
      if (P.noise.ptr != nullptr) {
        if (pre_kind == 0) quant_col_s8_kernel<0, true><<<grid, 256, 0, st>>>(P, rts, cts, units);
        else if (pre_kind == 1) quant_col_s8_kernel<1, true><<<grid, 256, 0, st>>>(P, rts, cts, units);
        else quant_col_s8_kernel<2, true><<<grid, 256, 0, st>>>(P, rts, cts, units);
      } else {
        if (pre_kind == 0) quant_col_s8_kernel<0, false><<<grid, 256, 0, st>>>(P, rts, cts, units);
        else if (pre_kind == 1) quant_col_s8_kernel<1, false><<<grid, 256, 0, st>>>(P, rts, cts, units);
        else quant_col_s8_kernel<2, false><<<grid, 256, 0, st>>>(P, rts, cts, units);
      }
    } else {
      AQT_DISPATCH_EPV_PRE(quant_col_fast, grid, 256, P, rts, cts, units);
    }
  } else {
    int64_t rts = (xv->rows + 63) / 64;
    int64_t cts = (P.ldq + 127) / 128;
    int64_t units = xv->b0 * xv->b1 * rts * cts;
    int grid = grid_for(units, 8);
    if (col_vec_ok(P.x, xv->rows))
      quant_col_kernel<true><<<grid, 256, 0, st>>>(P, rts, cts, units);
    else
      quant_col_kernel<false><<<grid, 256, 0, st>>>(P, rts, cts, units);
  }
#undef AQT_DISPATCH_EPV_PRE
  AQT_CUDA_OK(cudaGetLastError()); count_launch();
  return 0;
}

}  // namespace aqtb200

using namespace aqtb200;

extern "C" {

int64_t aqtb200_round_up(int64_t v, int64_t multiple) {
  return multiple <= 0 ? v : ((v + multiple - 1) / multiple) * multiple;
}

size_t aqtb200_quantize_workspace_bytes(const aqtb200_view* x,
                                        const aqtb200_quant_spec* spec) {
  if (x == nullptr || spec == nullptr) return 0;
  int64_t ns = std::max<int64_t>(1, n_scales(x, spec));
  return 2 * align256((size_t)ns * 4);
}

int aqtb200_quantize(const aqtb200_view* x, const aqtb200_view* prescale,
                     const aqtb200_view* noise, const aqtb200_quant_spec* spec,
                     const void* scale_in, void* q_out, void* scale_out,
                     void* workspace, size_t workspace_bytes, void* stream) {
  return run(x, prescale, noise, spec, scale_in, q_out, scale_out, workspace,
             workspace_bytes, (cudaStream_t)stream, true);
}

// ---------------------------------------------------------------------------
// Allocation-free variant of aqtb200_quantize. Its scratch (the amax cells and
// the reciprocal scales) lives in the library image instead of a caller
// buffer: a file-scope device array, present on every GPU that loads the
// library until the process exits.
static __device__ __align__(256) unsigned char
    g_static_scratch[2 * ((AQTB200_STATIC_MAX_SCALES * 4 + 255) / 256 * 256)];

// In host code the array's name is only a handle for the runtime, not a device
// address; the address is looked up once per device, with that device current.
static void* g_static_scratch_ptr[64] = {nullptr};
static std::mutex g_static_scratch_mu;

static int static_scratch_for_current_device(void** out) {
  int dev = 0;
  AQT_CUDA_OK(cudaGetDevice(&dev));
  AQT_REQUIRE(dev >= 0 && dev < 64, AQTB200_EUNSUPPORTED, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_static_scratch_mu);
  if (g_static_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    AQT_CUDA_OK(cudaGetSymbolAddress(&p, g_static_scratch));
    AQT_REQUIRE(p != nullptr, AQTB200_EDRIVER, "cudaGetSymbolAddress returned a null address");
    g_static_scratch_ptr[dev] = p;
  }
  *out = g_static_scratch_ptr[dev];
  return 0;
}

int aqtb200_quantize_static(const aqtb200_view* x, const aqtb200_view* prescale,
                            const aqtb200_view* noise, const aqtb200_quant_spec* spec,
                            const void* scale_in, void* q_out, void* scale_out, void* stream) {
  AQT_REQUIRE(x != nullptr && spec != nullptr, AQTB200_EINVAL, "null view or spec");
  const int64_t ns = n_scales(x, spec);
  AQT_REQUIRE(ns <= AQTB200_STATIC_MAX_SCALES, AQTB200_EUNSUPPORTED,
              "aqtb200_quantize_static handles at most %d scales (b0*b1*rows, or 1 per tensor); "
              "this call needs %lld -- use aqtb200_quantize with a caller workspace",
              AQTB200_STATIC_MAX_SCALES, (long long)ns);
  void* scratch = nullptr;
  int rc = static_scratch_for_current_device(&scratch);
  if (rc) return rc;
  return run(x, prescale, noise, spec, scale_in, q_out, scale_out, scratch,
             sizeof(g_static_scratch), (cudaStream_t)stream, true);
}

int aqtb200_absmax_raw(const aqtb200_view* x, int32_t per_tensor, float* amax_out, void* stream) {
  AQT_REQUIRE(x != nullptr && amax_out != nullptr, AQTB200_EINVAL, "null argument");
  aqtb200_quant_spec spec{};
  spec.kind = AQTB200_NUM_INT;  // only the reduction runs; numerics are irrelevant
  spec.qdtype = AQTB200_S8;
  spec.quant_bound = spec.clip_bound = 1.f;
  spec.per_tensor = per_tensor;
  spec.compute_dtype = spec.scale_dtype = x->dtype == AQTB200_BF16 ? AQTB200_BF16 : AQTB200_F32;
  return run(x, nullptr, nullptr, &spec, nullptr, nullptr, nullptr, nullptr, 0,
             (cudaStream_t)stream, false, amax_out);
}

int aqtb200_scale_from_amax(const float* amax, int64_t n, const void* prescale,
                            int32_t prescale_dtype, const aqtb200_quant_spec* spec,
                            void* scale_out, void* stream) {
  AQT_REQUIRE(amax != nullptr && spec != nullptr && scale_out != nullptr && n >= 0, AQTB200_EINVAL,
              "null argument");
  AQT_REQUIRE(is_float_dt(spec->compute_dtype) && is_float_dt(spec->scale_dtype), AQTB200_EINVAL,
              "compute/scale dtype must be f32 or bf16");
  AQT_REQUIRE(spec->quant_bound > 0.f, AQTB200_EINVAL, "quant_bound must be positive");
  if (prescale != nullptr)
    AQT_REQUIRE(is_float_dt(prescale_dtype), AQTB200_EINVAL, "prescale must be f32 or bf16");
  if (n == 0) return 0;
  FinalizeParams F{};
  F.amax = (const uint32_t*)amax; F.scale_out = scale_out; F.sinv = nullptr; F.n = n;
  F.t_dtype = spec->compute_dtype; F.s_dtype = spec->scale_dtype;
  F.quant_bound = spec->quant_bound; F.clipping_scale = spec->clipping_scale;
  F.po2 = spec->po2_scale; F.pre = prescale; F.pre_dtype = prescale_dtype;
  finalize_scale_kernel<<<(int)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(F);
  AQT_CUDA_OK(cudaGetLastError()); count_launch();
  return 0;
}

int aqtb200_quantize_pair(const aqtb200_view* x,
                          const aqtb200_quant_spec* spec_t, void* scale_t,
                          const void* prescale_t, int32_t prescale_t_dtype, void* q_t,
                          const aqtb200_quant_spec* spec_s, void* scale_s,
                          const void* prescale_s, int32_t prescale_s_dtype, void* q_s,
                          int32_t chain, const float* amax, float* amax_out, void* stream) {
  AQT_REQUIRE(x != nullptr && spec_t != nullptr && spec_s != nullptr && scale_t != nullptr &&
                  scale_s != nullptr && q_t != nullptr && q_s != nullptr,
              AQTB200_EINVAL, "null argument");
  AQT_REQUIRE(chain >= 0 && chain <= 2, AQTB200_EINVAL, "chain must be 0, 1 or 2");
  for (const aqtb200_quant_spec* sp : {spec_t, spec_s}) {
    const bool fp8 = sp->kind == AQTB200_NUM_FP8 &&
                     (sp->qdtype == AQTB200_E4M3 || sp->qdtype == AQTB200_E5M2);
    const bool i8 = sp->kind == AQTB200_NUM_INT && sp->qdtype == AQTB200_S8;
    AQT_REQUIRE((fp8 || i8) && sp->per_tensor && sp->compute_dtype == AQTB200_BF16 &&
                    sp->scale_dtype == AQTB200_BF16,
                AQTB200_EUNSUPPORTED,
                "aqtb200_quantize_pair: per-tensor fp8 or int8 with bf16 compute and scale dtype only");
  }
  AQT_REQUIRE(x->dtype == AQTB200_BF16, AQTB200_EUNSUPPORTED, "aqtb200_quantize_pair: bf16 input only");
  if (prescale_t != nullptr) AQT_REQUIRE(is_float_dt(prescale_t_dtype), AQTB200_EINVAL, "prescale dtype");
  if (prescale_s != nullptr) AQT_REQUIRE(is_float_dt(prescale_s_dtype), AQTB200_EINVAL, "prescale dtype");
  AQT_REQUIRE(chain == 0 || (chain == 1 ? prescale_s == nullptr : prescale_t == nullptr), AQTB200_EINVAL,
              "the chained output takes no prescale");
  const int64_t nb = x->b0 * x->b1;
  if (nb * x->rows * x->cols == 0) return 0;
  PairParams P{};
  P.x = to_dview(x);
  AQT_REQUIRE(P.x.sr == 1 && x->rows % 16 == 0 && x->cols % 16 == 0 && col_fast_ok(P.x, x->rows, 8),
              AQTB200_EUNSUPPORTED,
              "aqtb200_quantize_pair: rows must be the contiguous index, both extents multiples of "
              "16 and every stride a multiple of 16 bytes");
  AQT_REQUIRE(aligned(q_t, 16) && aligned(q_s, 16), AQTB200_EINVAL, "outputs not 16-byte aligned");
  P.scale_t = scale_t; P.scale_s = scale_s;
  P.pre_t = prescale_t; P.pre_s = prescale_s;
  P.pre_t_dtype = prescale_t_dtype; P.pre_s_dtype = prescale_s_dtype;
  P.qdtype_t = spec_t->qdtype; P.qdtype_s = spec_s->qdtype;
  P.clip_t = spec_t->clip_bound; P.clip_s = spec_s->clip_bound;
  P.amax = (const uint32_t*)amax;
  P.amax_out = (uint32_t*)amax_out;
  P.qb_t = spec_t->quant_bound; P.qb_s = spec_s->quant_bound;
  P.cs_t = spec_t->clipping_scale; P.cs_s = spec_s->clipping_scale;
  P.po2_t = spec_t->po2_scale; P.po2_s = spec_s->po2_scale;
  P.chain = chain;
  P.q_t = (uint8_t*)q_t; P.q_s = (uint8_t*)q_s;
  P.ld_t = x->cols; P.ld_s = x->rows;
  const int64_t rts = (x->rows + 127) / 128, cts = (x->cols + 127) / 128;
  const int64_t units = nb * rts * cts;
  const bool ints = spec_t->kind == AQTB200_NUM_INT;
  AQT_REQUIRE(ints == (spec_s->kind == AQTB200_NUM_INT), AQTB200_EUNSUPPORTED,
              "aqtb200_quantize_pair: both outputs int8 or both fp8");
  const int grid = grid_for(units, 4);
  cudaStream_t st = (cudaStream_t)stream;
  if (amax_out != nullptr) AQT_CUDA_OK(cudaMemsetAsync(amax_out, 0, 4, st));
#define AQT_PAIR(I)                                                                   \
  do {                                                                                \
    if (chain == 0) quant_pair_kernel<I, 0><<<grid, 256, 0, st>>>(P, rts, cts, units);      \
    else if (chain == 1) quant_pair_kernel<I, 1><<<grid, 256, 0, st>>>(P, rts, cts, units); \
    else quant_pair_kernel<I, 2><<<grid, 256, 0, st>>>(P, rts, cts, units);                 \
  } while (0)
  if (ints) AQT_PAIR(true); else AQT_PAIR(false);
#undef AQT_PAIR
  AQT_CUDA_OK(cudaGetLastError()); count_launch();
  return 0;
}

size_t aqtb200_quantize_dual_workspace_bytes(const aqtb200_dual_desc* d) {
  if (d == nullptr) return 0;
  const int64_t nb = d->x.b0 * d->x.b1;
  return 2 * align256((size_t)std::max<int64_t>(1, nb * d->x.rows) * 4) +
         2 * align256((size_t)std::max<int64_t>(1, nb * d->x.cols) * 4);
}

int aqtb200_quantize_dual(const aqtb200_dual_desc* d, void* workspace, size_t workspace_bytes,
                          void* stream) {
  AQT_REQUIRE(d != nullptr, AQTB200_EINVAL, "null descriptor");
  const aqtb200_view& xv = d->x;
  AQT_REQUIRE(xv.b0 >= 0 && xv.b1 >= 0 && xv.rows >= 0 && xv.cols >= 0, AQTB200_EINVAL,
              "negative extent");
  const int64_t nb = xv.b0 * xv.b1;
  if (nb * xv.rows * xv.cols == 0) return 0;
  AQT_REQUIRE(xv.ptr != nullptr && d->q_t != nullptr && d->q_s != nullptr &&
                  d->scale_t != nullptr && d->scale_s != nullptr,
              AQTB200_EINVAL, "null pointer");
  for (const aqtb200_quant_spec* sp : {&d->spec_t, &d->spec_s})
    AQT_REQUIRE(sp->kind == AQTB200_NUM_INT && sp->qdtype == AQTB200_S8 && !sp->per_tensor &&
                    sp->compute_dtype == AQTB200_BF16 && sp->scale_dtype == AQTB200_BF16 &&
                    sp->quant_bound > 0.f && sp->clip_bound > 0.f,
                AQTB200_EUNSUPPORTED,
                "aqtb200_quantize_dual: int8 numerics, per-row scales, bf16 compute and scale dtype");
  DualParams P{};
  P.x = to_dview(&xv);
  AQT_REQUIRE(xv.dtype == AQTB200_BF16 && P.x.sr == 1 && xv.rows % 16 == 0 && xv.cols % 16 == 0 &&
                  col_fast_ok(P.x, xv.rows, 8),
              AQTB200_EUNSUPPORTED,
              "aqtb200_quantize_dual: bf16 input with rows the contiguous index, both extents "
              "multiples of 16, every stride a multiple of 16 bytes");
  AQT_REQUIRE(aligned(d->q_t, 16) && aligned(d->q_s, 16), AQTB200_EINVAL, "outputs not 16-byte aligned");
  if (d->prescale_t.ptr != nullptr) {
    AQT_REQUIRE(d->prescale_t.dtype == AQTB200_BF16, AQTB200_EUNSUPPORTED, "prescales must be bf16");
    P.pre_t = d->prescale_t.ptr; P.pt_b0 = d->prescale_t.b0_stride; P.pt_b1 = d->prescale_t.b1_stride;
    P.pt_c = d->prescale_t.col_stride;
  }
  if (d->prescale_s.ptr != nullptr) {
    AQT_REQUIRE(d->prescale_s.dtype == AQTB200_BF16, AQTB200_EUNSUPPORTED, "prescales must be bf16");
    P.pre_s = d->prescale_s.ptr; P.ps_b0 = d->prescale_s.b0_stride; P.ps_b1 = d->prescale_s.b1_stride;
    P.ps_r = d->prescale_s.row_stride;
  }
  const bool noise = d->noise_t.ptr != nullptr;
  AQT_REQUIRE(noise == (d->noise_s.ptr != nullptr), AQTB200_EUNSUPPORTED,
              "aqtb200_quantize_dual: noise for both outputs or for neither");
  if (noise) {
    for (const aqtb200_view* nv : {&d->noise_t, &d->noise_s})
      AQT_REQUIRE(nv->dtype == AQTB200_F32 && nv->row_stride == 1 && nv->col_stride == xv.col_stride &&
                      nv->b0_stride == xv.b0_stride && nv->b1_stride == xv.b1_stride &&
                      aligned(nv->ptr, 16),
                  AQTB200_EUNSUPPORTED, "aqtb200_quantize_dual: noise must be f32 in x's layout");
    P.noise_t = (const float*)d->noise_t.ptr;
    P.noise_s = (const float*)d->noise_s.ptr;
  }
  const size_t need = aqtb200_quantize_dual_workspace_bytes(d);
  AQT_REQUIRE(workspace != nullptr && workspace_bytes >= need && aligned(workspace, 256),
              AQTB200_EWORKSPACE, "workspace: need %zu bytes, 256-byte aligned (got %zu)", need,
              workspace_bytes);
  const int64_t n_t = nb * xv.rows, n_s = nb * xv.cols;
  char* ws = (char*)workspace;
  P.amax_t = (uint32_t*)ws; ws += align256((size_t)n_t * 4);
  P.amax_s = (uint32_t*)ws; ws += align256((size_t)n_s * 4);
  float* sinv_t = (float*)ws; ws += align256((size_t)n_t * 4);
  float* sinv_s = (float*)ws;
  P.sinv_t = sinv_t; P.sinv_s = sinv_s;
  P.clip_t = d->spec_t.clip_bound; P.clip_s = d->spec_s.clip_bound;
  P.q_t = (uint8_t*)d->q_t; P.q_s = (uint8_t*)d->q_s;
  P.ld_t = xv.cols; P.ld_s = xv.rows;
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t rts = (xv.rows + 127) / 128, cts = (xv.cols + 127) / 128;

  // 1. both families of maxima in one pass
  AQT_CUDA_OK(cudaMemsetAsync(P.amax_s, 0, (size_t)n_s * 4, st));
  {
    const int grid = grid_for(nb * rts, 4);
#define AQT_DUAL_ABSMAX(PT, PS) absmax_dual_kernel<PT, PS><<<grid, 256, 0, st>>>(P, rts, cts, nb * rts)
    if (P.pre_t != nullptr) { if (P.pre_s != nullptr) AQT_DUAL_ABSMAX(true, true); else AQT_DUAL_ABSMAX(true, false); }
    else { if (P.pre_s != nullptr) AQT_DUAL_ABSMAX(false, true); else AQT_DUAL_ABSMAX(false, false); }
#undef AQT_DUAL_ABSMAX
    AQT_CUDA_OK(cudaGetLastError()); count_launch();
  }
  // 2. maxima -> scales and reciprocals
  for (int k = 0; k < 2; ++k) {
    const aqtb200_quant_spec& sp = k == 0 ? d->spec_t : d->spec_s;
    FinalizeParams F{};
    F.amax = k == 0 ? P.amax_t : P.amax_s;
    F.scale_out = k == 0 ? d->scale_t : d->scale_s;
    F.sinv = k == 0 ? sinv_t : sinv_s;
    F.n = k == 0 ? n_t : n_s;
    F.t_dtype = F.s_dtype = AQTB200_BF16;
    F.quant_bound = sp.quant_bound; F.clipping_scale = sp.clipping_scale; F.po2 = sp.po2_scale;
    finalize_scale_kernel<<<(int)((F.n + 255) / 256), 256, 0, st>>>(F);
    AQT_CUDA_OK(cudaGetLastError()); count_launch();
  }
  // 3. both int8 layouts in one pass
  {
    const int64_t units = nb * rts * cts;
    const int grid = grid_for(units, 2);
#define AQT_DUAL_QUANT(PT, PS)                                                                  \
  do {                                                                                          \
    if (noise) quant_dual_kernel<PT, PS, true><<<grid, 256, 0, st>>>(P, rts, cts, units);       \
    else quant_dual_kernel<PT, PS, false><<<grid, 256, 0, st>>>(P, rts, cts, units);            \
  } while (0)
    if (P.pre_t != nullptr) { if (P.pre_s != nullptr) AQT_DUAL_QUANT(true, true); else AQT_DUAL_QUANT(true, false); }
    else { if (P.pre_s != nullptr) AQT_DUAL_QUANT(false, true); else AQT_DUAL_QUANT(false, false); }
#undef AQT_DUAL_QUANT
    AQT_CUDA_OK(cudaGetLastError()); count_launch();
  }
  return 0;
}

int aqtb200_requant_amax(const float* amax, int64_t n, const void* prescale, int32_t prescale_dtype,
                         const aqtb200_quant_spec* spec, const void* scale, float* amax_q_out,
                         void* stream) {
  AQT_REQUIRE(amax != nullptr && spec != nullptr && scale != nullptr && amax_q_out != nullptr && n >= 0,
              AQTB200_EINVAL, "null argument");
  AQT_REQUIRE(is_float_dt(spec->compute_dtype) && is_float_dt(spec->scale_dtype), AQTB200_EINVAL,
              "compute/scale dtype must be f32 or bf16");
  AQT_REQUIRE(spec->kind == AQTB200_NUM_INT || spec->kind == AQTB200_NUM_FP8, AQTB200_EINVAL,
              "numerics kind");
  if (prescale != nullptr)
    AQT_REQUIRE(is_float_dt(prescale_dtype), AQTB200_EINVAL, "prescale must be f32 or bf16");
  if (n == 0) return 0;
  RequantAmaxParams R{};
  R.amax = (const uint32_t*)amax; R.scale = scale; R.pre = prescale; R.pre_dtype = prescale_dtype;
  R.t_dtype = spec->compute_dtype; R.s_dtype = spec->scale_dtype; R.kind = spec->kind;
  R.qdtype = spec->qdtype; R.clip_bound = spec->clip_bound; R.out = amax_q_out; R.n = n;
  requant_amax_kernel<<<(int)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(R);
  AQT_CUDA_OK(cudaGetLastError()); count_launch();
  return 0;
}

int aqtb200_prescale_amax(const float* amax, int64_t n, const void* prescale, int32_t prescale_dtype,
                          int32_t compute_dtype, float* out, void* stream) {
  AQT_REQUIRE(amax != nullptr && prescale != nullptr && out != nullptr && n >= 0, AQTB200_EINVAL,
              "null argument");
  AQT_REQUIRE(is_float_dt(prescale_dtype) && is_float_dt(compute_dtype), AQTB200_EINVAL,
              "prescale / compute dtype must be f32 or bf16");
  if (n == 0) return 0;
  prescale_amax_kernel<<<(int)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (const uint32_t*)amax, n, prescale, prescale_dtype, compute_dtype, out);
  AQT_CUDA_OK(cudaGetLastError()); count_launch();
  return 0;
}

int aqtb200_delayed_scaling_scale(const float* history, int64_t len, float* bound,
                                  int32_t update_bound, const aqtb200_quant_spec* spec,
                                  void* scale_out, void* stream) {
  AQT_REQUIRE(history != nullptr && bound != nullptr && spec != nullptr && scale_out != nullptr,
              AQTB200_EINVAL, "null argument");
  AQT_REQUIRE(len >= 1 && len <= 4096, AQTB200_EUNSUPPORTED,
              "amax history length %lld: 1 ... 4096 elements", (long long)len);
  AQT_REQUIRE(is_float_dt(spec->scale_dtype), AQTB200_EINVAL, "scale dtype must be f32 or bf16");
  AQT_REQUIRE(spec->quant_bound > 0.f, AQTB200_EINVAL, "quant_bound must be positive");
  DelayedParams D{};
  D.history = const_cast<float*>(history); D.len = len; D.bound = bound;
  D.update_bound = update_bound; D.quant_bound = spec->quant_bound; D.po2 = spec->po2_scale;
  D.s_dtype = spec->scale_dtype; D.scale_out = scale_out;
  delayed_scale_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(D);
  AQT_CUDA_OK(cudaGetLastError()); count_launch();
  return 0;
}

int aqtb200_delayed_scaling_push(float* history, int64_t len, const float* amax, void* stream) {
  AQT_REQUIRE(history != nullptr && amax != nullptr, AQTB200_EINVAL, "null argument");
  AQT_REQUIRE(len >= 1 && len <= 4096, AQTB200_EUNSUPPORTED,
              "amax history length %lld: 1 ... 4096 elements", (long long)len);
  DelayedParams D{};
  D.history = history; D.len = len; D.amax = amax;
  delayed_push_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(D);
  AQT_CUDA_OK(cudaGetLastError()); count_launch();
  return 0;
}

int aqtb200_absmax_scale(const aqtb200_view* x, const aqtb200_view* prescale,
                         const aqtb200_quant_spec* spec, void* scale_out,
                         void* workspace, size_t workspace_bytes, void* stream) {
  return run(x, prescale, nullptr, spec, nullptr, nullptr, scale_out, workspace,
             workspace_bytes, (cudaStream_t)stream, false);
}

int aqtb200_dequantize(const aqtb200_view* q, const aqtb200_view* scale,
                       int32_t dequant_dtype, void* out, void* stream) {
  AQT_REQUIRE(q != nullptr && out != nullptr, AQTB200_EINVAL, "null argument");
  AQT_REQUIRE(dequant_dtype == AQTB200_F32 || dequant_dtype == AQTB200_BF16,
              AQTB200_EINVAL, "dequant dtype must be f32 or bf16");
  DeqParams D{};
  D.q = to_dview(q);
  D.s = to_dview(scale);
  D.d_dtype = dequant_dtype;
  D.out = out;
  int64_t total = q->b0 * q->b1 * q->rows * q->cols;
  if (total == 0) return 0;
  AQT_REQUIRE(q->ptr != nullptr, AQTB200_EINVAL, "null q pointer");
  int grid = grid_for((total + 255) / 256, 8);
  dequant_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(D, total);
  AQT_CUDA_OK(cudaGetLastError()); count_launch();
  return 0;
}

}  // extern "C"
