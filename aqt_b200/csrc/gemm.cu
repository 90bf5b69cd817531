// Quantized batched GEMM with fused dequantizing epilogue for sm_100a.
//
//   acc[b,m,n] = sum_k A[b,m,k] * B[b,n,k]      (A, B: int8 or fp8, k contiguous)
//   out        = cast(cast_D(acc) * scale_1 * scale_2)
//
// Persistent kernel, one CTA per SM, 192 threads:
//   warp 0     : TMA producer  (cp.async.bulk.tensor, 128B-swizzled tiles)
//   warp 1     : MMA issuer    (tcgen05.mma kind::i8 / kind::f8f6f4, cta_group::1)
//   warps 2..5 : epilogue      (tcgen05.ld from TMEM -> scale -> global)
// Tile 128 x 256 x 128(bytes of k), 4-stage shared-memory ring (192 KB), two
// 256-column TMEM accumulators so the epilogue of tile i overlaps the
// mainloop of tile i+1. Every mbarrier wait is bounded: when one runs out the
// kernel records a code in `status`, lets in-flight copies land, frees its
// TMEM and returns instead of hanging the device.
#include <cuda.h>
#include <cudaTypedefs.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "common.cuh"

namespace aqtb200 {

int sm_count();

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 128;  // bytes (= elements) of k per stage: one 128B swizzle row
constexpr int STAGES = 4;
constexpr int MAX_STAGES1 = 12;  // single-CTA kernel, narrow B tiles: up to this many stages
constexpr int A_STAGE = BM * BK;
constexpr int B_STAGE = BN * BK;
constexpr int GROUP_M = 32;
constexpr int EPI_WARPS = 8;     // two per TMEM lane quarter, each draining half the columns
constexpr int GEMM_THREADS = 64 + 32 * EPI_WARPS;
constexpr int TMEM_COLS = 512;
constexpr size_t GEMM_SMEM = (size_t)STAGES * (A_STAGE + B_STAGE) + 1024;
constexpr long long WAIT_LIMIT_CYCLES = 4000000000LL;  // ~2 s
constexpr int kStagePitch = 128;  // bytes per staged epilogue row (16-byte pieces XOR-swizzled)

struct GemmParams {
  int64_t b0, b1, m, n, k;
  const void* a_scale;
  int64_t sa_b0, sa_b1, sa_m;
  const void* b_scale;
  int64_t sb_b0, sb_b1, sb_n;
  int a_scale_dtype, b_scale_dtype;
  int b_scale_first, d_dtype, out_dtype, is_int;
  void* out;
  int64_t o_b0, o_b1, o_m, o_n;
  void* acc_out;
  uint32_t* amax_out;  // optional: max |out| as f32 bits (atomic max)
  uint32_t idesc, idesc2;
  int64_t m_tiles, n_tiles, total_tiles, num_kb;
  int64_t m_tiles2, total_tiles2;  // 256-row tiles of the CTA-pair kernel
  int64_t n_tiles3, total_tiles3;  // 512-column tiles of the wide CTA-pair kernel
  int stages1, b_stage;  // single-CTA kernel: ring depth and bytes of one B tile
  // single-CTA kernel launched as a programmatic dependent of the kernel before
  // it on the stream (the one that quantizes the B operand): the A operand was
  // complete earlier, so its first stages are requested before the wait for
  // that kernel
  int pdl;
  // wide kernel, how the epilogue gets each scale: 0 = one value for the whole
  // launch, read once; 1 = contiguous bf16 per row / column, staged in shared
  // memory by the producer warp a tile ahead; 2 = read by the epilogue warps
  int sa_mode, sb_mode;
  // single-CTA kernel, skinny problems: the k-slabs of all tiles form one
  // sequence that is cut into equal shares, one per CTA, so every SM streams
  // the same number of bytes whatever the tile count. A tile whose slabs fall
  // into several shares is computed in parts; the part that finishes last
  // sums the partial accumulators of all of them and dequantizes.
  int stream_k;          // 0: whole tiles, round robin
  int max_parts;         // most parts any tile is cut into (slots per tile in `partials`)
  uint32_t* partials;    // [tile][max_parts][128 rows][n_mma] raw accumulators
  int32_t* tile_counter;  // [tile][4 row quarters], zeroed before the launch
  int n_mma;
  int stage_ok;  // output rows can be written as aligned 16-byte pieces
  int tma_store;  // a tensor map of the bf16 output exists: staged rows leave through the TMA unit
  int32_t* status;
  // SIMT reference kernel only:
  const uint8_t* a; const uint8_t* b;
  int64_t a_b0, a_b1, lda, b_b0, b_b1, ldb;
  int a_dtype, b_dtype;
};

// ---------------------------------------------------------------------------
// PTX wrappers

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait. Returns false when the limit ran out or another role aborted.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity,
                                          volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > WAIT_LIMIT_CYCLES) return false;
  }
}

__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* tm, uint64_t* bar,
                                            int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(smem_u32(dst)),
      "l"(tm), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

// Untiled bulk copy global -> shared memory (16-byte aligned, a multiple of 16
// bytes), completing on an mbarrier; no multicast.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(dst)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

// Shared memory -> global tile store through the TMA unit (bulk async group).
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* tm, const void* src, int c0, int c1,
                                             int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(tm),
      "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// Blocks until the TMA unit has finished READING the shared memory of every
// store this thread has issued (the global writes may still be in flight).
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
template <bool IS_INT>
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                       uint32_t idesc, uint32_t accumulate) {
  if (IS_INT) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// K-major, 128-byte swizzled operand tile: rows of 128 bytes, 8-row groups
// 1024 bytes apart (SBO), descriptor version 1 (sm_100), layout type 2.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;            // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;  // stride byte offset
  d |= (uint64_t)1 << 46;            // descriptor version
  d |= (uint64_t)2 << 61;            // SWIZZLE_128B
  return d;
}

__device__ __forceinline__ void decode_tile(const GemmParams& P, int64_t t, int64_t& i0,
                                            int64_t& i1, int64_t& mt, int64_t& nt) {
  const int64_t per_batch = P.m_tiles * P.n_tiles;
  int64_t b = t / per_batch, r = t % per_batch;
  i1 = b % P.b1;
  i0 = b / P.b1;
  const int64_t group = GROUP_M * P.n_tiles;
  int64_t g = r / group, in = r % group;
  int64_t first = g * GROUP_M;
  int64_t gm = min((int64_t)GROUP_M, P.m_tiles - first);
  mt = first + in % gm;
  nt = in / gm;
}

// One multiply of the dequantization chain: result dtype = promote(cur, sdt).
__device__ __forceinline__ float scale_mul(float r, float s, int& cur, int sdt) {
  if (sdt == AQTB200_F32) cur = AQTB200_F32;
  return round_to(__fmul_rn(r, s), cur);
}

// Running max |v| of an epilogue thread, as f32 bits (non-negative floats order
// like their bit patterns; a NaN pattern ranks above infinity and so survives).
__device__ __forceinline__ void amax_f32(uint32_t& run, float v) {
  run = max(run, __float_as_uint(v) & 0x7fffffffu);
}
// eight packed bf16 pairs
__device__ __forceinline__ void amax_bf16x2(uint32_t& run, const uint32_t* pk, int n) {
  uint32_t m2 = 0;
  for (int j = 0; j < n; ++j) m2 = __vmaxu2(m2, pk[j] & 0x7fff7fffu);
  run = max(run, max(m2 & 0xffffu, m2 >> 16) << 16);
}
// Folds the epilogue threads' maxima of one warp into the caller's cell.
__device__ __forceinline__ void amax_publish(uint32_t* cell, uint32_t run, int lane) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) run = max(run, __shfl_xor_sync(0xffffffffu, run, o));
  if (lane == 0 && run != 0) atomicMax(cell, run);
}

// Drains one 128 x BN accumulator tile: TMEM -> registers -> dequantizing chain
// -> global. `taddr` addresses this warp's 32 lanes and the tile's first column.
// Scales of one output tile, fetched BEFORE the warp waits for the
// accumulator: they do not depend on it, and a load issued per 32-column chunk
// after the wait would put a memory round trip on every chunk's critical path.
struct EpiScales {
  float sa;          // this thread's row scale (1 when absent)
  uint32_t sbw[4];   // EPI == 1: lanes 0..15 hold bf16 pairs (col 2l, 2l+1) of chunk c
  float sbl[4];      // otherwise: lane l holds the scale of column 32c + l
};

template <int EPI>
__device__ __forceinline__ void load_epi_scales(const GemmParams& P, int lane, int64_t i0,
                                                int64_t i1, int64_t row, int64_t ncol0,
                                                EpiScales& sc) {
  const bool has_a = P.a_scale != nullptr, has_b = P.b_scale != nullptr;
  sc.sa = 1.f;
  if (has_a && row < P.m)
    sc.sa = load1(P.a_scale, P.a_scale_dtype, i0 * P.sa_b0 + i1 * P.sa_b1 + row * P.sa_m);
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const int64_t col0 = ncol0 + c * 32;
    if constexpr (EPI == 1) {
      uint32_t w = 0x3f803f80u;  // (1.0, 1.0)
      if (has_b) {
        const unsigned short* sp = (const unsigned short*)P.b_scale + i0 * P.sb_b0 + i1 * P.sb_b1;
        if (P.sb_n == 0) {
          const uint32_t v = __ldg(sp);
          w = v | (v << 16);
        } else if (lane < 16) {
          const int64_t cc = col0 + 2 * lane;
          const uint32_t lo = cc < P.n ? __ldg(sp + cc * P.sb_n) : 0x3f80u;
          const uint32_t hi = cc + 1 < P.n ? __ldg(sp + (cc + 1) * P.sb_n) : 0x3f80u;
          w = lo | (hi << 16);
        }
      }
      sc.sbw[c] = w;
    } else {
      float v = 1.f;
      if (has_b && col0 + lane < P.n)
        v = load1(P.b_scale, P.b_scale_dtype,
                  i0 * P.sb_b0 + i1 * P.sb_b1 + (col0 + lane) * P.sb_n);
      sc.sbl[c] = v;
    }
  }
}

// EPI selects the arithmetic: 0 generic (any mix of f32 / bf16 dtypes),
// 1 dequant, output and scales all bf16, 2 all f32.
template <bool IS_INT, int EPI>
__device__ __forceinline__ void epilogue_tile(const GemmParams& P, uint32_t taddr, int lane,
                                              int64_t i0, int64_t i1, int64_t row, int64_t ncol0,
                                              uint8_t* stage, const EpiScales& sc,
                                              uint32_t& amax) {
  if (P.tma_store && stage != nullptr) {
    // an earlier tile of this warp may have left through the TMA unit
    if (lane == 0) tma_store_wait_read();
    __syncwarp();
  }
  const bool has_a = P.a_scale != nullptr, has_b = P.b_scale != nullptr;
  const int out_es = P.out_dtype == AQTB200_BF16 ? 2 : 4;
  const bool row_ok = row < P.m;
  const float sa = sc.sa;
  const int64_t obase = i0 * P.o_b0 + i1 * P.o_b1 + row * P.o_m;
  const int64_t abase = ((i0 * P.b1 + i1) * P.m + row) * P.n;
#pragma unroll
  for (int chunk = 0; chunk < 4; ++chunk) {
    const int64_t col0 = ncol0 + chunk * 32;
    if (col0 >= P.n) break;  // warp-uniform
    uint32_t acc[32];
    tc_ld32(taddr + (uint32_t)(chunk * 32), acc);
    tc_wait_ld();
    float res[32];
    uint32_t pk[16];  // EPI == 1: the 32 results as packed bf16 pairs
    if constexpr (EPI == 1) {
      // Everything bf16: cast_bf16(acc) then two bf16 multiplies. A bf16 x bf16
      // product is exact in f32, so the hardware's packed bf16 multiply (one
      // rounding) equals "multiply in f32, round to bf16".
      const __nv_bfloat162 sa2 = __float2bfloat162_rn(sa);
      const uint32_t sbw = sc.sbw[chunk];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        uint32_t w = (has_b && P.sb_n != 0) ? __shfl_sync(0xffffffffu, sbw, j) : sbw;
        const __nv_bfloat162 sb2 = *(const __nv_bfloat162*)&w;
        const float f0 = IS_INT ? __int2float_rn((int)acc[2 * j]) : __uint_as_float(acc[2 * j]);
        const float f1 = IS_INT ? __int2float_rn((int)acc[2 * j + 1]) : __uint_as_float(acc[2 * j + 1]);
        __nv_bfloat162 v = __floats2bfloat162_rn(f0, f1);
        if (P.b_scale_first) {
          if (has_b) v = __hmul2(v, sb2);
          if (has_a) v = __hmul2(v, sa2);
        } else {
          if (has_a) v = __hmul2(v, sa2);
          if (has_b) v = __hmul2(v, sb2);
        }
        pk[j] = *(const uint32_t*)&v;
      }
    } else {
      const float sbl = sc.sbl[chunk];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float sb = __shfl_sync(0xffffffffu, sbl, j);
        float r = IS_INT ? __int2float_rn((int)acc[j]) : __uint_as_float(acc[j]);
        if constexpr (EPI == 2) {
          // everything f32: two rounded f32 multiplies
          if (P.b_scale_first) {
            if (has_b) r = __fmul_rn(r, sb);
            if (has_a) r = __fmul_rn(r, sa);
          } else {
            if (has_a) r = __fmul_rn(r, sa);
            if (has_b) r = __fmul_rn(r, sb);
          }
          res[j] = r;
        } else {
          int cur = P.d_dtype;
          r = round_to(r, cur);
          if (P.b_scale_first) {
            if (has_b) r = scale_mul(r, sb, cur, P.b_scale_dtype);
            if (has_a) r = scale_mul(r, sa, cur, P.a_scale_dtype);
          } else {
            if (has_a) r = scale_mul(r, sa, cur, P.a_scale_dtype);
            if (has_b) r = scale_mul(r, sb, cur, P.b_scale_dtype);
          }
          r = round_to(r, P.d_dtype);
          res[j] = round_to(r, P.out_dtype);
        }
      }
    }
    if (row_ok && P.amax_out != nullptr && P.out != nullptr) {
      // rows and columns past the matrix edge hold products of fill zeros
      // with stand-in scales: leave them out
      if constexpr (EPI == 1) {
        if (col0 + 32 <= P.n) {
          amax_bf16x2(amax, pk, 16);
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (col0 + 2 * j < P.n) amax_f32(amax, bf16lo(pk[j]));
            if (col0 + 2 * j + 1 < P.n) amax_f32(amax, bf16hi(pk[j]));
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (col0 + j < P.n) amax_f32(amax, res[j]);
      }
    }
    if (row_ok && P.acc_out != nullptr) {
      uint32_t* ao = (uint32_t*)P.acc_out + abase + col0;
      if (col0 + 32 <= P.n && (((uintptr_t)ao) & 15) == 0) {
#pragma unroll
        for (int v = 0; v < 8; ++v)
          ((uint4*)ao)[v] = make_uint4(acc[4 * v], acc[4 * v + 1], acc[4 * v + 2], acc[4 * v + 3]);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (col0 + j < P.n) ao[j] = acc[j];
      }
    }
    // bf16 fast path: two 32-column chunks are parked in this warp's staging
    // rows and leave together, so that one warp store covers four whole
    // 128-byte lines instead of 32 scattered 16-byte pieces.
    bool staged = false;
    if constexpr (EPI == 1) {
      staged = stage != nullptr && P.stage_ok && P.out != nullptr &&
               ncol0 + (chunk & ~1) * 32 + 64 <= P.n;
      if (staged) {
        uint8_t* srow = stage + lane * kStagePitch;
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          const int piece = ((chunk & 1) * 4 + v) ^ (lane & 7);
          *(uint4*)(srow + piece * 16) =
              make_uint4(pk[4 * v], pk[4 * v + 1], pk[4 * v + 2], pk[4 * v + 3]);
        }
        if (chunk & 1) {
          __syncwarp();
          const int64_t colp = ncol0 + (chunk - 1) * 32;
          const int64_t row0 = row - lane;
          __nv_bfloat16* ob = (__nv_bfloat16*)P.out + i0 * P.o_b0 + i1 * P.o_b1 + colp;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int r = i * 4 + (lane >> 3), seg = lane & 7;
            if (row0 + r < P.m) {
              const uint4 v = *(const uint4*)(stage + r * kStagePitch + ((seg ^ (r & 7)) * 16));
              *(uint4*)(ob + (row0 + r) * P.o_m + seg * 8) = v;
            }
          }
          __syncwarp();
        }
      }
    }
    if (row_ok && P.out != nullptr && !staged) {
      const bool full = col0 + 32 <= P.n;
      const bool vec_ok = full && P.o_n == 1 &&
                          ((((uintptr_t)P.out) + (size_t)(obase + col0) * out_es) & 15) == 0;
      if (vec_ok) {
        if (EPI == 1) {
          uint4* o = (uint4*)((__nv_bfloat16*)P.out + obase + col0);
#pragma unroll
          for (int v = 0; v < 4; ++v)
            o[v] = make_uint4(pk[4 * v], pk[4 * v + 1], pk[4 * v + 2], pk[4 * v + 3]);
        } else if (out_es == 2) {
          uint4* o = (uint4*)((__nv_bfloat16*)P.out + obase + col0);
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            __nv_bfloat162 p0 = __floats2bfloat162_rn(res[8 * v + 0], res[8 * v + 1]);
            __nv_bfloat162 p1 = __floats2bfloat162_rn(res[8 * v + 2], res[8 * v + 3]);
            __nv_bfloat162 p2 = __floats2bfloat162_rn(res[8 * v + 4], res[8 * v + 5]);
            __nv_bfloat162 p3 = __floats2bfloat162_rn(res[8 * v + 6], res[8 * v + 7]);
            uint4 u;
            u.x = *(uint32_t*)&p0; u.y = *(uint32_t*)&p1;
            u.z = *(uint32_t*)&p2; u.w = *(uint32_t*)&p3;
            o[v] = u;
          }
        } else {
          float4* o = (float4*)((float*)P.out + obase + col0);
#pragma unroll
          for (int v = 0; v < 8; ++v)
            o[v] = make_float4(res[4 * v], res[4 * v + 1], res[4 * v + 2], res[4 * v + 3]);
        }
      } else {
        if constexpr (EPI == 1) {
#pragma unroll
          for (int j = 0; j < 16; ++j) { res[2 * j] = bf16lo(pk[j]); res[2 * j + 1] = bf16hi(pk[j]); }
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          if (col0 + j < P.n) {
            const int64_t oi = obase + (col0 + j) * P.o_n;
            if (out_es == 2)
              ((__nv_bfloat16*)P.out)[oi] = __float2bfloat16_rn(res[j]);
            else
              ((float*)P.out)[oi] = res[j];
          }
        }
      }
    }
  }
}

// bf16 epilogue for a full 128-column slice of an accumulator (dequant, output
// and scales all bf16; no raw-accumulator output): TMEM is read 16 columns at a
// time with the next read in flight while the current one is converted, rows
// are staged in the 128-byte swizzle of the output tensor map, and each
// 32 x 64 block leaves with one TMA store (rows past M are clipped by the unit).
// Without an output map the same staged rows are stored by the warp.
template <bool IS_INT>
__device__ __forceinline__ void epilogue_tile_bf16(const GemmParams& P, const CUtensorMap* tmO,
                                                   uint32_t taddr, int lane, int64_t i0,
                                                   int64_t i1, int64_t row, int64_t ncol0,
                                                   uint8_t* stage, const EpiScales& sc,
                                                   uint32_t& amax) {
  const bool has_a = P.a_scale != nullptr, has_b = P.b_scale != nullptr;
  const bool vary_b = has_b && P.sb_n != 0;
  const bool want_amax = P.amax_out != nullptr && row < P.m;
  const __nv_bfloat162 sa2 = __float2bfloat162_rn(sc.sa);
  const int64_t row0 = row - lane;
  uint8_t* srow = stage + lane * kStagePitch;
  uint32_t buf[2][16];
  tc_ld16(taddr, buf[0]);
#pragma unroll 1
  for (int g = 0; g < 2; ++g) {  // 64-column groups
    // the staging rows are free once the store of the previous group has read them
    if (P.tma_store && lane == 0) tma_store_wait_read();
    __syncwarp();
#pragma unroll
    for (int h = 0; h < 4; ++h) {  // 16-column pieces
      tc_wait_ld();
      if (h < 3 || g == 0) tc_ld16(taddr + (uint32_t)((g * 4 + h + 1) * 16), buf[(h + 1) & 1]);
      const uint32_t* acc = buf[h & 1];
      const uint32_t sbw = g ? (h < 2 ? sc.sbw[2] : sc.sbw[3]) : (h < 2 ? sc.sbw[0] : sc.sbw[1]);
      uint32_t pk[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        uint32_t w = vary_b ? __shfl_sync(0xffffffffu, sbw, (h & 1) * 8 + j) : sbw;
        const __nv_bfloat162 sb2 = *(const __nv_bfloat162*)&w;
        const float f0 = IS_INT ? __int2float_rn((int)acc[2 * j]) : __uint_as_float(acc[2 * j]);
        const float f1 = IS_INT ? __int2float_rn((int)acc[2 * j + 1]) : __uint_as_float(acc[2 * j + 1]);
        __nv_bfloat162 v = __floats2bfloat162_rn(f0, f1);
        if (P.b_scale_first) {
          if (has_b) v = __hmul2(v, sb2);
          if (has_a) v = __hmul2(v, sa2);
        } else {
          if (has_a) v = __hmul2(v, sa2);
          if (has_b) v = __hmul2(v, sb2);
        }
        pk[j] = *(const uint32_t*)&v;
      }
      if (want_amax) amax_bf16x2(amax, pk, 8);
#pragma unroll
      for (int v = 0; v < 2; ++v)
        *(uint4*)(srow + (((h * 2 + v) ^ (lane & 7)) * 16)) =
            make_uint4(pk[4 * v], pk[4 * v + 1], pk[4 * v + 2], pk[4 * v + 3]);
    }
    if (P.tma_store) {
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0 && row0 < P.m)
        tma_store_4d(tmO, stage, (int)(ncol0 + g * 64), (int)row0, (int)i1, (int)i0);
    } else {
      __syncwarp();
      __nv_bfloat16* ob = (__nv_bfloat16*)P.out + i0 * P.o_b0 + i1 * P.o_b1 + ncol0 + g * 64;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int r = i * 4 + (lane >> 3), seg = lane & 7;
        if (row0 + r < P.m) {
          const uint4 v = *(const uint4*)(stage + r * kStagePitch + ((seg ^ (r & 7)) * 16));
          *(uint4*)(ob + (row0 + r) * P.o_m + seg * 8) = v;
        }
      }
    }
  }
}

// Picks the epilogue for one 128-column slice (the choice is warp-uniform).
template <bool IS_INT, int EPI>
__device__ __forceinline__ void epilogue_slice(const GemmParams& P, const CUtensorMap* tmO,
                                               uint32_t taddr, int lane, int64_t i0, int64_t i1,
                                               int64_t row, int64_t ncol0, uint8_t* stage,
                                               const EpiScales& sc, uint32_t& amax) {
  if constexpr (EPI == 1) {
    if (P.stage_ok && P.acc_out == nullptr && P.out != nullptr && ncol0 + 128 <= P.n) {
      epilogue_tile_bf16<IS_INT>(P, tmO, taddr, lane, i0, i1, row, ncol0, stage, sc, amax);
      return;
    }
  }
  epilogue_tile<IS_INT, EPI>(P, taddr, lane, i0, i1, row, ncol0, stage, sc, amax);
}

// The work of one CTA of the single-CTA kernel, as a list of segments: k-slabs
// [kb0, kb1) of one tile. Without stream_k: whole tiles, round robin. With it:
// this CTA's share of the sequence of all k-slabs; the tiles it shares with a
// neighbour come first (their fix-up then overlaps with the whole tiles that
// follow), and `part` of `parts` numbers the CTAs of a tile in slab order.
struct Segment {
  int64_t tile, kb0, kb1;
  int part, parts;
};
__device__ __forceinline__ bool cta_segment(const GemmParams& P, int64_t idx, Segment& sg) {
  if (!P.stream_k) {
    sg.tile = blockIdx.x + idx * gridDim.x;
    sg.kb0 = 0;
    sg.kb1 = P.num_kb;
    sg.part = 0;
    sg.parts = 1;
    return sg.tile < P.total_tiles;
  }
  const int64_t G = gridDim.x, total = P.total_tiles * P.num_kb;
  const int64_t beg = ((int64_t)blockIdx.x * total) / G, end = (((int64_t)blockIdx.x + 1) * total) / G;
  if (beg >= end) return false;
  const int64_t t_first = beg / P.num_kb, t_last = (end - 1) / P.num_kb;
  if (idx > t_last - t_first) return false;
  sg.tile = idx == 0 ? t_first : (idx == 1 ? t_last : t_first + idx - 1);
  const int64_t T0 = sg.tile * P.num_kb;
  sg.kb0 = max(beg, T0) - T0;
  sg.kb1 = min(end, T0 + P.num_kb) - T0;
  // the largest g whose share starts at or before slab X is ((X + 1) G - 1) / total
  const int64_t g_first = ((T0 + 1) * G - 1) / total;
  const int64_t g_last = ((T0 + P.num_kb) * G - 1) / total;
  sg.part = (int)((int64_t)blockIdx.x - g_first);
  sg.parts = (int)(g_last - g_first + 1);
  return true;
}

// Epilogue of one (tile, k-part) unit of a split contraction (single-CTA
// kernel, at most 64 columns, so only the warps of the first column half have
// work). Each warp owns 32 rows of the tile. It parks its raw accumulators in
// global scratch and takes a ticket from a counter per (tile, 32-row quarter);
// the warp that draws the last ticket adds up all parts of its quarter -- in
// part order, so the f32 sum does not depend on who came last -- and runs the
// dequantizing chain. Nothing waits on another CTA: whoever is last does the
// work. The counters are zeroed by the host before every launch.
template <bool IS_INT>
__device__ __forceinline__ void epilogue_split(const GemmParams& P, uint32_t taddr, int lane,
                                               int quarter, int64_t tile, int part, int parts,
                                               int64_t i0, int64_t i1, int64_t row, float sa,
                                               uint32_t& amax) {
  const int nm = P.n_mma;  // 16 ... 64, a multiple of 16
  const int row_in_tile = quarter * 32 + lane;
  uint32_t* mine = P.partials + ((tile * P.max_parts + part) * BM + row_in_tile) * nm;
  for (int c = 0; c < nm; c += 16) {
    uint32_t acc[16];
    tc_ld16(taddr + (uint32_t)c, acc);
    tc_wait_ld();
#pragma unroll
    for (int v = 0; v < 4; ++v)
      __stcg((uint4*)(mine + c) + v,
             make_uint4(acc[4 * v], acc[4 * v + 1], acc[4 * v + 2], acc[4 * v + 3]));
  }
  // the lanes' stores happen before the warp barrier, the barrier before lane
  // 0's fence and ticket: whoever draws the last ticket (and fences) sees them
  __syncwarp();
  int prev = 0;
  if (lane == 0) {
    __threadfence();
    prev = atomicAdd(P.tile_counter + tile * 4 + quarter, 1);
  }
  prev = __shfl_sync(0xffffffffu, prev, 0);
  if (prev != parts - 1) return;
  __threadfence();
  // Last to arrive: every part of these 32 rows is in global memory. All loads
  // of a 16-column chunk (up to MAX_SPLIT parts x 4 vectors) and the columns'
  // scales are requested together: the fix-up runs once per tile quarter and
  // would otherwise pay one L2 round trip per vector.
  constexpr int MAX_SPLIT = 6;  // == MAX_PARTS on the host side
  const bool has_a = P.a_scale != nullptr, has_b = P.b_scale != nullptr;
  const bool row_ok = row < P.m;
  const uint32_t* base = P.partials + (tile * P.max_parts * BM + row_in_tile) * nm;
  // lane l holds the scales of columns l and l + 32
  float sb_lane[2] = {1.f, 1.f};
  if (has_b) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int64_t col = lane + 32 * h;
      if (col < P.n && col < nm)
        sb_lane[h] = load1(P.b_scale, P.b_scale_dtype, i0 * P.sb_b0 + i1 * P.sb_b1 + col * P.sb_n);
    }
  }
  for (int c0 = 0; c0 < nm && c0 < P.n; c0 += 16) {
    uint4 v[MAX_SPLIT][4];
#pragma unroll
    for (int p = 0; p < MAX_SPLIT; ++p)
#pragma unroll
      for (int q = 0; q < 4; ++q)
        v[p][q] = p < parts ? __ldcg((const uint4*)(base + (int64_t)p * BM * nm + c0) + q)
                                : make_uint4(0u, 0u, 0u, 0u);
    uint32_t raw[16];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint4 sum = v[0][q];
#pragma unroll
      for (int p = 1; p < MAX_SPLIT; ++p) {
        if (IS_INT) {
          sum.x += v[p][q].x; sum.y += v[p][q].y; sum.z += v[p][q].z; sum.w += v[p][q].w;
        } else if (p < parts) {  // adding +0.0 could turn a -0.0 sum into +0.0
          sum.x = __float_as_uint(__fadd_rn(__uint_as_float(sum.x), __uint_as_float(v[p][q].x)));
          sum.y = __float_as_uint(__fadd_rn(__uint_as_float(sum.y), __uint_as_float(v[p][q].y)));
          sum.z = __float_as_uint(__fadd_rn(__uint_as_float(sum.z), __uint_as_float(v[p][q].z)));
          sum.w = __float_as_uint(__fadd_rn(__uint_as_float(sum.w), __uint_as_float(v[p][q].w)));
        }
      }
      raw[4 * q] = sum.x; raw[4 * q + 1] = sum.y; raw[4 * q + 2] = sum.z; raw[4 * q + 3] = sum.w;
    }
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int64_t col = c0 + j;
      // every lane takes part in the shuffle; the rest is per lane
      const float sb = __shfl_sync(0xffffffffu, (c0 + j) < 32 ? sb_lane[0] : sb_lane[1],
                                   (c0 + j) & 31);
      if (col >= P.n || !row_ok) continue;
      if (P.acc_out != nullptr)
        ((uint32_t*)P.acc_out)[((i0 * P.b1 + i1) * P.m + row) * P.n + col] = raw[j];
      if (P.out == nullptr) continue;
      float r = IS_INT ? __int2float_rn((int)raw[j]) : __uint_as_float(raw[j]);
      int cur = P.d_dtype;
      r = round_to(r, cur);
      if (P.b_scale_first) {
        if (has_b) r = scale_mul(r, sb, cur, P.b_scale_dtype);
        if (has_a) r = scale_mul(r, sa, cur, P.a_scale_dtype);
      } else {
        if (has_a) r = scale_mul(r, sa, cur, P.a_scale_dtype);
        if (has_b) r = scale_mul(r, sb, cur, P.b_scale_dtype);
      }
      r = round_to(round_to(r, P.d_dtype), P.out_dtype);
      if (P.amax_out != nullptr) amax_f32(amax, r);
      const int64_t oi = i0 * P.o_b0 + i1 * P.o_b1 + row * P.o_m + col * P.o_n;
      if (P.out_dtype == AQTB200_BF16) ((__nv_bfloat16*)P.out)[oi] = __float2bfloat16_rn(r);
      else ((float*)P.out)[oi] = r;
    }
  }
}

template <bool IS_INT, int EPI>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA,
                    const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmO, GemmParams P) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* smem_a = smem;
  // The B tile holds as many rows as the MMAs are wide (P.b_stage bytes), and
  // the ring is as deep as shared memory allows (P.stages1): a narrow problem
  // streams its big A operand with far more bytes in flight.
  uint8_t* smem_b = smem + P.stages1 * A_STAGE;
  __shared__ __align__(8) uint64_t full_bar[MAX_STAGES1];
  __shared__ __align__(8) uint64_t empty_bar[MAX_STAGES1];
  __shared__ __align__(8) uint64_t tfull_bar[2];
  __shared__ __align__(8) uint64_t tempty_bar[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ __align__(1024) uint8_t epi_stage[EPI_WARPS][32 * kStagePitch];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < P.stages1; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&tfull_bar[s], 1);
      mbar_init(&tempty_bar[s], EPI_WARPS);
    }
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&tmem_slot)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  volatile int* abortp = &abort_flag;
  int fail = 0;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      Segment sg;
      bool primed = !P.pdl;
      for (int64_t idx = 0; !fail && cta_segment(P, idx, sg); ++idx) {
        int64_t i0, i1, mt, nt;
        decode_tile(P, sg.tile, i0, i1, mt, nt);
        int64_t kb_first = sg.kb0;
        if (!primed) {
          // First segment of a dependent launch: the ring is empty, so the A
          // tiles of its first stages go out at once; the B tiles follow when
          // the kernel that produces B has completed.
          primed = true;
          const int n = (int)min((int64_t)P.stages1, sg.kb1 - sg.kb0);
          for (int j = 0; j < n; ++j) {
            mbar_expect_tx(&full_bar[j], A_STAGE + P.b_stage);
            tma_load_4d(smem_a + j * A_STAGE, &tmA, &full_bar[j], (int)((sg.kb0 + j) * BK),
                        (int)(mt * BM), (int)i1, (int)i0);
          }
          asm volatile("griddepcontrol.wait;" ::: "memory");
          for (int j = 0; j < n; ++j)
            tma_load_4d(smem_b + j * P.b_stage, &tmB, &full_bar[j], (int)((sg.kb0 + j) * BK),
                        (int)(nt * BN), (int)i1, (int)i0);
          kb_first = sg.kb0 + n;
          stage = n;
          if (stage == P.stages1) { stage = 0; phase ^= 1; }
        }
        for (int64_t kb = kb_first; kb < sg.kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abortp)) { fail = 1; break; }
          mbar_expect_tx(&full_bar[stage], A_STAGE + P.b_stage);
          tma_load_4d(smem_a + stage * A_STAGE, &tmA, &full_bar[stage], (int)(kb * BK),
                      (int)(mt * BM), (int)i1, (int)i0);
          tma_load_4d(smem_b + stage * P.b_stage, &tmB, &full_bar[stage], (int)(kb * BK),
                      (int)(nt * BN), (int)i1, (int)i0);
          if (++stage == P.stages1) { stage = 0; phase ^= 1; }
        }
      }
      if (fail) { *abortp = 1; if (P.status) atomicCAS(P.status, 0, 1); }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int buf = 0;
      uint32_t aphase = 0;
      Segment sg;
      for (int64_t idx = 0; !fail && cta_segment(P, idx, sg); ++idx) {
        const int64_t kb0 = sg.kb0, kb1 = sg.kb1;
        if (!mbar_wait(&tempty_bar[buf], aphase ^ 1, abortp)) { fail = 2; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
        for (int64_t kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abortp)) { fail = 2; break; }
          tc_fence_after();
          const uint64_t ad = make_smem_desc(smem_u32(smem_a + stage * A_STAGE));
          const uint64_t bd = make_smem_desc(smem_u32(smem_b + stage * P.b_stage));
#pragma unroll
          for (int k = 0; k < BK / 32; ++k) {
            // advance 32 bytes of k inside the swizzle row: +2 in 16-byte units
            tc_mma<IS_INT>(d_tmem, ad + (uint64_t)(2 * k), bd + (uint64_t)(2 * k), P.idesc,
                           (kb > kb0 || k > 0) ? 1u : 0u);
          }
          tc_commit(&empty_bar[stage]);
          if (++stage == P.stages1) { stage = 0; phase ^= 1; }
        }
        if (fail) break;
        tc_commit(&tfull_bar[buf]);
        buf ^= 1;
        if (buf == 0) aphase ^= 1;
      }
      if (fail) { *abortp = 1; if (P.status) atomicCAS(P.status, 0, 2); }
    }
  } else {
    // ---------------- epilogue ----------------
    // (a dependent launch reads scales the kernel before it wrote)
    if (P.pdl) asm volatile("griddepcontrol.wait;" ::: "memory");
    const int quarter = warp & 3;          // TMEM lanes this warp may read
    const int half = (warp - 2) >> 2;      // which 128 columns of the tile it drains
    int buf = 0;
    uint32_t aphase = 0;
    uint32_t amax = 0;
    Segment sg;
    for (int64_t idx = 0; cta_segment(P, idx, sg); ++idx) {
      const int64_t t = sg.tile;
      int64_t i0, i1, mt, nt;
      decode_tile(P, t, i0, i1, mt, nt);
      const int64_t row = mt * BM + quarter * 32 + lane;
      EpiScales sc;
      load_epi_scales<EPI>(P, lane, i0, i1, row, nt * BN + half * 128, sc);
      int ok = mbar_wait(&tfull_bar[buf], aphase, abortp) ? 1 : 0;
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) { fail = 3; break; }
      tc_fence_after();
      const uint32_t taddr =
          tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN + half * 128);
      if (sg.parts > 1) {
        if (half == 0)
          epilogue_split<IS_INT>(P, taddr, lane, quarter, t, sg.part, sg.parts, i0, i1, row,
                                 sc.sa, amax);
      } else {
        epilogue_slice<IS_INT, EPI>(P, &tmO, taddr, lane, i0, i1, row, nt * BN + half * 128,
                                    epi_stage[warp - 2], sc, amax);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[buf]);
      buf ^= 1;
      if (buf == 0) aphase ^= 1;
    }
    if (P.amax_out != nullptr) amax_publish(P.amax_out, amax, lane);
    if (lane == 0) tma_store_wait_read();  // shared memory outlives its last store
    if (fail && lane == 0) { *abortp = 1; if (P.status) atomicCAS(P.status, 0, 3); }
  }

  __syncwarp();
  if (*abortp) {
    // Give copies that are still in flight time to land before the shared
    // memory they target is released.
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) { }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(TMEM_COLS)
                 : "memory");
  }
}

// ---------------------------------------------------------------------------
// CTA-pair variant: a cluster of two CTAs (one SM pair) computes a 256 x 256
// tile with tcgen05.mma.cta_group::2. CTA r of the pair loads rows
// [r*128, r*128+128) of the A tile and rows [r*128, ...) of the B tile (32 KB
// per stage instead of 48 KB), holds the accumulator rows of its own half in
// its own TMEM, and runs its own epilogue. Only the even CTA issues MMAs; its
// commits are delivered to the barriers of both CTAs. Per flop this pulls one
// third fewer bytes through the L2 -> SM fabric than the 128 x 256 kernel.
constexpr int BM2 = 256;           // tile rows per CTA pair
constexpr int B_HALF = 128 * BK;   // bytes of B one CTA stages per k-block
constexpr int STAGES2 = 6;
constexpr size_t GEMM2_SMEM = (size_t)STAGES2 * (A_STAGE + B_HALF) + 1024;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared variable in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
// Relaxed on purpose: the only thing the waiting MMA thread must observe is
// that this warp's tcgen05.ld reads are done, which tcgen05.wait::ld plus
// tcgen05.fence::before_thread_sync already order. A release at cluster scope
// would also wait for every global store of the tile to drain, and stall the
// accumulator hand-back by microseconds per tile.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
               : "memory");
}
__device__ __forceinline__ void st_cluster_u32(uint32_t cluster_addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tma_load_4d_pair(void* dst, const CUtensorMap* tm,
                                                 uint32_t leader_bar, int c0, int c1, int c2,
                                                 int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(smem_u32(dst)),
      "l"(tm), "r"(leader_bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64"
      " [%0], %1;" ::"r"(smem_u32(bar)),
      "h"((uint16_t)3)
      : "memory");
}
template <bool IS_INT>
__device__ __forceinline__ void tc_mma_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                            uint32_t idesc, uint32_t accumulate) {
  if (IS_INT) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}

__device__ __forceinline__ void decode_tile2(const GemmParams& P, int64_t t, int64_t& i0,
                                             int64_t& i1, int64_t& mt, int64_t& nt) {
  const int64_t per_batch = P.m_tiles2 * P.n_tiles;
  int64_t b = t / per_batch, r = t % per_batch;
  i1 = b % P.b1;
  i0 = b / P.b1;
  constexpr int64_t G = GROUP_M / 2;
  const int64_t group = G * P.n_tiles;
  int64_t g = r / group, in = r % group;
  int64_t first = g * G;
  int64_t gm = min(G, P.m_tiles2 - first);
  mt = first + in % gm;
  nt = in / gm;
}

template <bool IS_INT, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tmA,
                         const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmO, GemmParams P) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + STAGES2 * A_STAGE;
  __shared__ __align__(8) uint64_t full_bar[STAGES2];   // used in the even CTA only
  __shared__ __align__(8) uint64_t empty_bar[STAGES2];  // one per CTA
  __shared__ __align__(8) uint64_t tfull_bar[2];        // one per CTA
  __shared__ __align__(8) uint64_t tempty_bar[2];       // used in the even CTA only
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ __align__(1024) uint8_t epi_stage[EPI_WARPS][32 * kStagePitch];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int64_t cluster_id = blockIdx.x >> 1;
  const int64_t num_clusters = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES2; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&tfull_bar[s], 1);
      mbar_init(&tempty_bar[s], 2 * EPI_WARPS);  // the epilogue warps of both CTAs
    }
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&tmem_slot)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  volatile int* abortp = &abort_flag;
  const uint32_t peer_abort = map_to_cta(smem_u32(&abort_flag), rank ^ 1u);
  int fail = 0;

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int64_t t = cluster_id; t < P.total_tiles2 && !fail; t += num_clusters) {
        int64_t i0, i1, mt, nt;
        decode_tile2(P, t, i0, i1, mt, nt);
        for (int64_t kb = 0; kb < P.num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abortp)) { fail = 1; break; }
          const uint32_t lbar = map_to_cta(smem_u32(&full_bar[stage]), 0);
          if (leader) mbar_expect_tx(&full_bar[stage], 2 * (A_STAGE + B_HALF));
          tma_load_4d_pair(smem_a + stage * A_STAGE, &tmA, lbar, (int)(kb * BK),
                           (int)(mt * BM2 + rank * 128), (int)i1, (int)i0);
          tma_load_4d_pair(smem_b + stage * B_HALF, &tmB, lbar, (int)(kb * BK),
                           (int)(nt * BN + rank * 128), (int)i1, (int)i0);
          if (++stage == STAGES2) { stage = 0; phase ^= 1; }
        }
      }
      if (fail) {
        *abortp = 1;
        st_cluster_u32(peer_abort, 1u);
        if (P.status) atomicCAS(P.status, 0, 1);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (even CTA only) ----------------
    if (lane == 0 && leader) {
      int stage = 0;
      uint32_t phase = 0;
      int buf = 0;
      uint32_t aphase = 0;
      for (int64_t t = cluster_id; t < P.total_tiles2 && !fail; t += num_clusters) {
        if (!mbar_wait(&tempty_bar[buf], aphase ^ 1, abortp)) { fail = 2; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
        for (int64_t kb = 0; kb < P.num_kb; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abortp)) { fail = 2; break; }
          tc_fence_after();
          const uint64_t ad = make_smem_desc(smem_u32(smem_a + stage * A_STAGE));
          const uint64_t bd = make_smem_desc(smem_u32(smem_b + stage * B_HALF));
#pragma unroll
          for (int k = 0; k < BK / 32; ++k) {
            tc_mma_pair<IS_INT>(d_tmem, ad + (uint64_t)(2 * k), bd + (uint64_t)(2 * k), P.idesc2,
                                (kb > 0 || k > 0) ? 1u : 0u);
          }
          tc_commit_pair(&empty_bar[stage]);
          if (++stage == STAGES2) { stage = 0; phase ^= 1; }
        }
        if (fail) break;
        tc_commit_pair(&tfull_bar[buf]);
        buf ^= 1;
        if (buf == 0) aphase ^= 1;
      }
      if (fail) {
        *abortp = 1;
        st_cluster_u32(peer_abort, 1u);
        if (P.status) atomicCAS(P.status, 0, 2);
      }
    }
  } else {
    // ---------------- epilogue (both CTAs, own half of the rows) ----------------
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    int buf = 0;
    uint32_t aphase = 0;
    uint32_t amax = 0;
    // The scales of a tile are requested one tile ahead: with a short
    // contraction the accumulator of the next tile is ready as soon as this
    // one is drained, and a scale fetch issued only then (a round trip to L2,
    // per-column scales being a strided gather) would sit on every tile's
    // critical path.
    int64_t i0 = 0, i1 = 0, mt = 0, nt = 0, row = 0;
    EpiScales sc;
    if (cluster_id < P.total_tiles2) {
      decode_tile2(P, cluster_id, i0, i1, mt, nt);
      row = mt * BM2 + rank * 128 + quarter * 32 + lane;
      load_epi_scales<EPI>(P, lane, i0, i1, row, nt * BN + half * 128, sc);
    }
    for (int64_t t = cluster_id; t < P.total_tiles2; t += num_clusters) {
      int64_t j0 = 0, j1 = 0, mt2 = 0, nt2 = 0, row2 = 0;
      EpiScales sc2;
      if (t + num_clusters < P.total_tiles2) {
        decode_tile2(P, t + num_clusters, j0, j1, mt2, nt2);
        row2 = mt2 * BM2 + rank * 128 + quarter * 32 + lane;
        load_epi_scales<EPI>(P, lane, j0, j1, row2, nt2 * BN + half * 128, sc2);
      }
      int ok = mbar_wait(&tfull_bar[buf], aphase, abortp) ? 1 : 0;
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) { fail = 3; break; }
      tc_fence_after();
      epilogue_slice<IS_INT, EPI>(
          P, &tmO, tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN + half * 128), lane,
          i0, i1, row, nt * BN + half * 128, epi_stage[warp - 2], sc, amax);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tempty_bar[buf]), 0));
      buf ^= 1;
      if (buf == 0) aphase ^= 1;
      i0 = j0; i1 = j1; mt = mt2; nt = nt2; row = row2;
      sc = sc2;
    }
    if (P.amax_out != nullptr) amax_publish(P.amax_out, amax, lane);
    if (lane == 0) tma_store_wait_read();  // shared memory outlives its last store
    if (fail && lane == 0) {
      *abortp = 1;
      st_cluster_u32(peer_abort, 1u);
      if (P.status) atomicCAS(P.status, 0, 3);
    }
  }

  __syncwarp();
  if (*abortp) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) { }
  }
  tc_fence_before();
  __syncthreads();
  // Neither CTA may release its TMEM or leave while the other can still read
  // its shared memory or write its accumulators.
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(TMEM_COLS)
                 : "memory");
  }
}

// ---------------------------------------------------------------------------
// Wide CTA-pair kernel: one 256 x 512 output tile per pair, held as two
// 256-column accumulators that share every A slab. Per 128-byte k-slab each CTA
// loads 128 rows of A and 2 x 128 rows of B (48 KB) for eight MMAs, a quarter
// less operand traffic per flop than the 256 x 256 tile, which is what keeps the
// tensor pipe fed without multicast loads. The price: both accumulators fill
// all 512 TMEM columns, so the epilogue of a tile cannot overlap the mainloop
// of the next one; the producer still runs ahead into the next tile, so only
// the drain itself is exposed. Chosen for long contractions (see gemm_dequant).
constexpr int STAGES3 = 4;
constexpr int W_STAGE = A_STAGE + 2 * B_HALF;  // 48 KB per CTA per stage
constexpr int WIDE_EPI_WARPS = 16;  // four per TMEM lane quarter: the drain is exposed, so it is spread wide
constexpr int kWidePitch = 64;      // bytes per staged row: 32 bf16 columns, 64-byte swizzle
// dynamic shared memory of the wide kernel: the operand ring, the epilogue
// warps' staging rows (2 KB each), the staged scales of one tile (128 row
// scales + 512 column scales, bf16), and the slack of the 1024-byte alignment
constexpr int W_EPI_BYTES = WIDE_EPI_WARPS * 32 * kWidePitch;
constexpr int W_SCALE_BYTES = (128 + 512) * 2;
constexpr size_t GEMM3_SMEM = (size_t)STAGES3 * W_STAGE + W_EPI_BYTES + W_SCALE_BYTES + 1024;
constexpr int BNW = 512;
// Shortest contraction (in 128-byte k-slabs) for which the exposed drain of the
// wide tile costs less than the slower mainloop of the double-buffered one.
constexpr int64_t WIDE_MIN_KB = 16;

__device__ __forceinline__ void decode_tile3(const GemmParams& P, int64_t t, int64_t& i0,
                                             int64_t& i1, int64_t& mt, int64_t& nt) {
  const int64_t per_batch = P.m_tiles2 * P.n_tiles3;
  int64_t b = t / per_batch, r = t % per_batch;
  i1 = b % P.b1;
  i0 = b / P.b1;
  constexpr int64_t G = GROUP_M / 2;
  const int64_t group = G * P.n_tiles3;
  int64_t g = r / group, in = r % group;
  int64_t first = g * G;
  int64_t gm = min(G, P.m_tiles2 - first);
  mt = first + in % gm;
  nt = in / gm;
}

constexpr int WIDE_THREADS = 32 * (2 + WIDE_EPI_WARPS);

// Only the all-bf16 epilogue with a TMA-describable output runs here (the host
// falls back to the 256 x 256 kernel otherwise), which keeps the register need
// of the 18 warps under the 96 the register file allows them.
// RAW: instead of the dequantized bf16 result the epilogue writes the raw
// 32-bit accumulators (tmO then maps the contiguous [b0][b1][m][n] int32 / f32
// accumulator tensor, boxes of 32 rows x 16 columns in the 64-byte swizzle):
// the form a contraction sharded over several GPUs needs, whose partial sums
// are added across ranks before the one dequantization.
template <bool IS_INT, bool RAW>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(WIDE_THREADS, 1)
gemm_tcgen05_wide_kernel(const __grid_constant__ CUtensorMap tmA,
                         const __grid_constant__ CUtensorMap tmB,
                         const __grid_constant__ CUtensorMap tmO, GemmParams P) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[STAGES3];   // used in the even CTA only
  __shared__ __align__(8) uint64_t empty_bar[STAGES3];  // one per CTA
  __shared__ __align__(8) uint64_t tfull_bar[2];        // per accumulator; one per CTA
  __shared__ __align__(8) uint64_t tempty_bar[2];       // per accumulator; even CTA only
  __shared__ __align__(8) uint64_t sfull_bar;            // staged scales of a tile; one per CTA
  __shared__ __align__(8) uint64_t sempty_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  uint8_t* const epi_base = smem + STAGES3 * W_STAGE;   // [WIDE_EPI_WARPS][32 rows][64 bytes]
  uint16_t* const sc_rows = (uint16_t*)(epi_base + W_EPI_BYTES);  // bf16 scales of this CTA's 128 tile rows
  uint16_t* const sc_cols = sc_rows + 128;                         // bf16 scales of the tile's 512 columns

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int64_t cluster_id = blockIdx.x >> 1;
  const int64_t num_clusters = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES3; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&tfull_bar[0], 1);
    mbar_init(&tfull_bar[1], 1);
    mbar_init(&tempty_bar[0], 2 * WIDE_EPI_WARPS);
    mbar_init(&tempty_bar[1], 2 * WIDE_EPI_WARPS);
    mbar_init(&sfull_bar, 1);
    mbar_init(&sempty_bar, WIDE_EPI_WARPS);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&tmem_slot)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  volatile int* abortp = &abort_flag;
  const uint32_t peer_abort = map_to_cta(smem_u32(&abort_flag), rank ^ 1u);
  int fail = 0;

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      const bool stage_scales = !RAW && (P.sa_mode == 1 || P.sb_mode == 1);
      uint32_t sphase = 0;
      for (int64_t t = cluster_id; t < P.total_tiles3 && !fail; t += num_clusters) {
        int64_t i0, i1, mt, nt;
        decode_tile3(P, t, i0, i1, mt, nt);
        const bool two = nt * BNW + 256 < P.n;  // the second accumulator has columns
        if (stage_scales) {
          // The epilogue's scales travel like the operands: bulk copies into
          // shared memory, so the sixteen epilogue warps issue no global load
          // (measured on the K = 128 score einsum: per-tile loads from those
          // warps, even requested a tile ahead, cost 0.2 ms of 0.66 ms). One
          // slot is enough: every warp moves its scales to registers at the top
          // of a tile and hands the slot back, long before the next tile.
          if (!mbar_wait(&sempty_bar, sphase ^ 1, abortp)) { fail = 1; break; }
          const int64_t row0 = mt * BM2 + rank * 128, col0 = nt * BNW;
          const uint32_t bytes_a =
              P.sa_mode == 1 ? (uint32_t)(2 * max((int64_t)0, min((int64_t)128, P.m - row0))) : 0u;
          const uint32_t bytes_b =
              P.sb_mode == 1 ? (uint32_t)(2 * max((int64_t)0, min((int64_t)BNW, P.n - col0))) : 0u;
          mbar_expect_tx(&sfull_bar, bytes_a + bytes_b);
          if (bytes_a)
            bulk_load(sc_rows, (const uint16_t*)P.a_scale + i0 * P.sa_b0 + i1 * P.sa_b1 + row0,
                      bytes_a, &sfull_bar);
          if (bytes_b)
            bulk_load(sc_cols, (const uint16_t*)P.b_scale + i0 * P.sb_b0 + i1 * P.sb_b1 + col0,
                      bytes_b, &sfull_bar);
          sphase ^= 1;
        }
        for (int64_t kb = 0; kb < P.num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abortp)) { fail = 1; break; }
          const uint32_t lbar = map_to_cta(smem_u32(&full_bar[stage]), 0);
          uint8_t* sa = smem + stage * W_STAGE;
          if (leader)
            mbar_expect_tx(&full_bar[stage], 2 * (A_STAGE + (two ? 2 : 1) * B_HALF));
          tma_load_4d_pair(sa, &tmA, lbar, (int)(kb * BK), (int)(mt * BM2 + rank * 128), (int)i1,
                           (int)i0);
          tma_load_4d_pair(sa + A_STAGE, &tmB, lbar, (int)(kb * BK),
                           (int)(nt * BNW + rank * 128), (int)i1, (int)i0);
          if (two)
            tma_load_4d_pair(sa + A_STAGE + B_HALF, &tmB, lbar, (int)(kb * BK),
                             (int)(nt * BNW + 256 + rank * 128), (int)i1, (int)i0);
          if (++stage == STAGES3) { stage = 0; phase ^= 1; }
        }
      }
      if (fail) {
        *abortp = 1;
        st_cluster_u32(peer_abort, 1u);
        if (P.status) atomicCAS(P.status, 0, 1);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (even CTA only) ----------------
    if (lane == 0 && leader) {
      int stage = 0;
      uint32_t phase = 0, aphase = 0;
      for (int64_t t = cluster_id; t < P.total_tiles3 && !fail; t += num_clusters) {
        int64_t i0, i1, mt, nt;
        decode_tile3(P, t, i0, i1, mt, nt);
        const bool two = nt * BNW + 256 < P.n;
        // The two accumulators are staggered at both ends of the tile so the
        // tensor pipe works through most of the drain. The first `head`
        // k-slabs are issued accumulator by accumulator: all into the first
        // one (handed back half way through the previous tile's drain), then
        // all into the second. The last `tail` k-slabs likewise: the first
        // accumulator finishes -- and its drain starts -- while the second is
        // still being fed. The shared-memory stages of such a group are
        // released after its second pass.
        const int head = (int)min((int64_t)STAGES3, P.num_kb);
        const int64_t rest = P.num_kb - head;
        const int tail = (int)min((int64_t)STAGES3, rest);
        const int64_t middle = rest - tail;
        int stage_of[STAGES3];
        // -- one staggered group of `cnt` k-slabs; first == the tile's first slabs
        auto pass_a = [&](int cnt, bool first) {
#pragma unroll
          for (int q = 0; q < STAGES3; ++q) {
            if (q < cnt && !fail) {
              if (!mbar_wait(&full_bar[stage], phase, abortp)) { fail = 2; }
              if (!fail) {
                tc_fence_after();
                const uint8_t* sa = smem + stage * W_STAGE;
                const uint64_t ad = make_smem_desc(smem_u32(sa));
                const uint64_t bd0 = make_smem_desc(smem_u32(sa + A_STAGE));
#pragma unroll
                for (int k = 0; k < BK / 32; ++k)
                  tc_mma_pair<IS_INT>(tmem_base, ad + (uint64_t)(2 * k), bd0 + (uint64_t)(2 * k),
                                      P.idesc2, (!first || q > 0 || k > 0) ? 1u : 0u);
                stage_of[q] = stage;
                if (++stage == STAGES3) { stage = 0; phase ^= 1; }
              }
            }
          }
        };
        auto pass_b = [&](int cnt, bool first) {
#pragma unroll
          for (int q = 0; q < STAGES3; ++q) {
            if (q < cnt) {
              if (two) {
                const uint8_t* sa = smem + stage_of[q] * W_STAGE;
                const uint64_t ad = make_smem_desc(smem_u32(sa));
                const uint64_t bd1 = make_smem_desc(smem_u32(sa + A_STAGE + B_HALF));
#pragma unroll
                for (int k = 0; k < BK / 32; ++k)
                  tc_mma_pair<IS_INT>(tmem_base + 256u, ad + (uint64_t)(2 * k),
                                      bd1 + (uint64_t)(2 * k), P.idesc2,
                                      (!first || q > 0 || k > 0) ? 1u : 0u);
              }
              tc_commit_pair(&empty_bar[stage_of[q]]);
            }
          }
        };
        if (!mbar_wait(&tempty_bar[0], aphase ^ 1, abortp)) { fail = 2; break; }
        tc_fence_after();
        pass_a(head, true);
        if (fail) break;
        if (rest == 0) tc_commit_pair(&tfull_bar[0]);
        if (!mbar_wait(&tempty_bar[1], aphase ^ 1, abortp)) { fail = 2; break; }
        tc_fence_after();
        pass_b(head, true);
        for (int64_t kb = 0; kb < middle; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abortp)) { fail = 2; break; }
          tc_fence_after();
          const uint8_t* sa = smem + stage * W_STAGE;
          const uint64_t ad = make_smem_desc(smem_u32(sa));
          const uint64_t bd0 = make_smem_desc(smem_u32(sa + A_STAGE));
          const uint64_t bd1 = make_smem_desc(smem_u32(sa + A_STAGE + B_HALF));
#pragma unroll
          for (int k = 0; k < BK / 32; ++k) {
            tc_mma_pair<IS_INT>(tmem_base, ad + (uint64_t)(2 * k), bd0 + (uint64_t)(2 * k),
                                P.idesc2, 1u);
            if (two)
              tc_mma_pair<IS_INT>(tmem_base + 256u, ad + (uint64_t)(2 * k),
                                  bd1 + (uint64_t)(2 * k), P.idesc2, 1u);
          }
          tc_commit_pair(&empty_bar[stage]);
          if (++stage == STAGES3) { stage = 0; phase ^= 1; }
        }
        if (fail) break;
        if (tail > 0) {
          pass_a(tail, false);
          if (fail) break;
          tc_commit_pair(&tfull_bar[0]);
          pass_b(tail, false);
        }
        tc_commit_pair(&tfull_bar[1]);
        aphase ^= 1;
      }
      if (fail) {
        *abortp = 1;
        st_cluster_u32(peer_abort, 1u);
        if (P.status) atomicCAS(P.status, 0, 2);
      }
    }
  } else {
    // ---------------- epilogue (both CTAs, own 128 rows) ----------------
    // warp = (TMEM lane quarter, 64-column slice). Each warp drains its slice
    // of the first accumulator, hands that accumulator back, then drains its
    // slice of the second. TMEM is read 16 columns at a time with the next
    // read in flight during the conversion; every 32 columns the staged rows
    // (64-byte swizzle of the output map) leave with one TMA store, which
    // clips rows and columns past the matrix edge.
    const int quarter = warp & 3;
    const int slice = (warp - 2) >> 2;
    const bool has_a = P.a_scale != nullptr, has_b = P.b_scale != nullptr;
    const bool vary_b = has_b && P.sb_n != 0;
    uint8_t* stage_rows = epi_base + (warp - 2) * (32 * kWidePitch);
    uint8_t* srow = stage_rows + lane * kWidePitch;
    const int swz = (lane >> 1) & 3;
    uint32_t aphase = 0;
    uint32_t amax = 0;
    // Scales of a tile: one per row, one pair per two columns. A scale that is
    // one value for the whole launch is read here, once; contiguous bf16
    // scales are taken from the ring the producer warp fills (see there);
    // anything else is read by this warp at the top of the tile.
    float sa_const = 1.f;
    uint32_t sb_const = 0x3f803f80u;  // (1.0, 1.0)
    if constexpr (!RAW) {
      if (has_a && P.sa_mode == 0) sa_const = load1(P.a_scale, P.a_scale_dtype, 0);
      if (has_b && P.sb_mode == 0) {
        const uint32_t v = __ldg((const unsigned short*)P.b_scale);
        sb_const = v | (v << 16);
      }
    }
    const bool staged = !RAW && (P.sa_mode == 1 || P.sb_mode == 1);
    uint32_t sphase = 0;
    for (int64_t t = cluster_id; t < P.total_tiles3; t += num_clusters) {
      int64_t i0, i1, mt, nt;
      decode_tile3(P, t, i0, i1, mt, nt);
      const bool two = nt * BNW + 256 < P.n;
      const int64_t row = mt * BM2 + rank * 128 + quarter * 32 + lane;
      const int64_t row0 = row - lane;
      const int64_t col_s = nt * BNW + slice * 64;  // this warp's first column in accumulator 0
      float sa = sa_const;
      // [accumulator * 2 + 32-column group]: lanes 0..15 hold column pairs
      uint32_t sbw[4] = {sb_const, sb_const, sb_const, sb_const};
      if constexpr (!RAW) {
        if (staged) {
          int oks = mbar_wait(&sfull_bar, sphase, abortp) ? 1 : 0;
          oks = __all_sync(0xffffffffu, oks);
          if (!oks) { fail = 3; break; }
          if (P.sa_mode == 1)
            sa = __bfloat162float(__ushort_as_bfloat16(sc_rows[quarter * 32 + lane]));
          if (P.sb_mode == 1 && lane < 16) {
#pragma unroll
            for (int q = 0; q < 4; ++q)
              sbw[q] = *(const uint32_t*)&sc_cols[slice * 64 + (q >> 1) * 256 + (q & 1) * 32 + 2 * lane];
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(&sempty_bar);
          sphase ^= 1;
        }
        if (has_a && P.sa_mode == 2 && row < P.m)
          sa = load1(P.a_scale, P.a_scale_dtype, i0 * P.sa_b0 + i1 * P.sa_b1 + row * P.sa_m);
        if (has_b && P.sb_mode == 2) {
          const unsigned short* sp = (const unsigned short*)P.b_scale + i0 * P.sb_b0 + i1 * P.sb_b1;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            if (P.sb_n == 0) {
              const uint32_t v = __ldg(sp);
              sbw[q] = v | (v << 16);
            } else if (lane < 16) {
              const int64_t cc = col_s + (q >> 1) * 256 + (q & 1) * 32 + 2 * lane;
              const uint32_t lo = cc < P.n ? __ldg(sp + cc * P.sb_n) : 0x3f80u;
              const uint32_t hi = cc + 1 < P.n ? __ldg(sp + (cc + 1) * P.sb_n) : 0x3f80u;
              sbw[q] = lo | (hi << 16);
            }
          }
        }
      }
      const __nv_bfloat162 sa2 = __float2bfloat162_rn(sa);
      int ok = mbar_wait(&tfull_bar[0], aphase, abortp) ? 1 : 0;
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) { fail = 3; break; }
      tc_fence_after();
      const uint32_t tlane = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(slice * 64);
      const int groups = two ? 4 : 2;  // 32-column groups: two per accumulator
      uint32_t buf[2][16];
      tc_ld16(tlane, buf[0]);
#pragma unroll 1
      for (int g = 0; g < groups; ++g) {
        const int a = g >> 1;
        const int64_t colg = col_s + a * 256 + (g & 1) * 32;
        if constexpr (!RAW) {
          // the staging rows are free once the previous store has read them
          if (lane == 0) tma_store_wait_read();
          __syncwarp();
        }
        uint32_t sb_g = 0;
        if constexpr (!RAW) sb_g = g < 2 ? (g ? sbw[1] : sbw[0]) : (g == 2 ? sbw[2] : sbw[3]);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          tc_wait_ld();
          const int pn = 2 * g + h + 1;  // next 16-column piece
          if (pn < 2 * groups && pn != 4)  // piece 4 opens the second accumulator: see below
            tc_ld16(tlane + (uint32_t)((pn >> 2) * 256 + (pn & 3) * 16), buf[h ^ 1]);
          const uint32_t* acc = buf[h];
          if constexpr (RAW) {
            // one piece = 16 accumulators = the 64 bytes of a staged row
            if (lane == 0) tma_store_wait_read();
            __syncwarp();
#pragma unroll
            for (int v = 0; v < 4; ++v)
              *(uint4*)(srow + ((v ^ swz) * 16)) =
                  make_uint4(acc[4 * v], acc[4 * v + 1], acc[4 * v + 2], acc[4 * v + 3]);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0 && row0 < P.m && colg + h * 16 < P.n)
              tma_store_4d(&tmO, stage_rows, (int)(colg + h * 16), (int)row0, (int)i1, (int)i0);
          } else {
            uint32_t pk[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              uint32_t w = vary_b ? __shfl_sync(0xffffffffu, sb_g, h * 8 + j) : sb_g;
              const __nv_bfloat162 sb2 = *(const __nv_bfloat162*)&w;
              const float f0 = IS_INT ? __int2float_rn((int)acc[2 * j]) : __uint_as_float(acc[2 * j]);
              const float f1 =
                  IS_INT ? __int2float_rn((int)acc[2 * j + 1]) : __uint_as_float(acc[2 * j + 1]);
              __nv_bfloat162 v = __floats2bfloat162_rn(f0, f1);
              if (P.b_scale_first) {
                if (has_b) v = __hmul2(v, sb2);
                if (has_a) v = __hmul2(v, sa2);
              } else {
                if (has_a) v = __hmul2(v, sa2);
                if (has_b) v = __hmul2(v, sb2);
              }
              pk[j] = *(const uint32_t*)&v;
            }
            if (P.amax_out != nullptr && row < P.m) {
              // columns past the matrix edge hold products of fill zeros with
              // stand-in scales: leave them out
              const int64_t cp = colg + h * 16;
              if (cp + 16 <= P.n) {
                amax_bf16x2(amax, pk, 8);
              } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  if (cp + 2 * j < P.n) amax_f32(amax, bf16lo(pk[j]));
                  if (cp + 2 * j + 1 < P.n) amax_f32(amax, bf16hi(pk[j]));
                }
              }
            }
#pragma unroll
            for (int v = 0; v < 2; ++v)
              *(uint4*)(srow + (((h * 2 + v) ^ swz) * 16)) =
                  make_uint4(pk[4 * v], pk[4 * v + 1], pk[4 * v + 2], pk[4 * v + 3]);
          }
        }
        if constexpr (!RAW) {
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0 && row0 < P.m && colg < P.n)
            tma_store_4d(&tmO, stage_rows, (int)colg, (int)row0, (int)i1, (int)i0);
        }
        if (g & 1) {
          // this accumulator's columns have all been read (the read in flight,
          // if any, belongs to the other accumulator)
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tempty_bar[a]), 0));
          if (a == 0 && two) {
            // the second accumulator finishes a little later than the first
            int ok1 = mbar_wait(&tfull_bar[1], aphase, abortp) ? 1 : 0;
            ok1 = __all_sync(0xffffffffu, ok1);
            if (!ok1) { fail = 3; break; }
            tc_fence_after();
            tc_ld16(tlane + 256u, buf[0]);
          }
        }
      }
      if (fail) break;
      if (!two) {
        if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tempty_bar[1]), 0));
      }
      aphase ^= 1;
    }
    if constexpr (!RAW) {
      if (P.amax_out != nullptr) amax_publish(P.amax_out, amax, lane);
    }
    if (lane == 0) tma_store_wait_read();  // shared memory outlives its last store
    if (fail && lane == 0) {
      *abortp = 1;
      st_cluster_u32(peer_abort, 1u);
      if (P.status) atomicCAS(P.status, 0, 3);
    }
  }

  __syncwarp();
  if (*abortp) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) { }
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(TMEM_COLS)
                 : "memory");
  }
}

// ---------------------------------------------------------------------------
// Tensor-pipe ceiling: nothing but tcgen05.mma issue. Each CTA (one per SM)
// fills one 128 x 128-byte A slab and one 256 x 128-byte B slab in shared
// memory with pseudo-random bytes (no global traffic at all), then one thread
// issues 128 x 256 x 32 MMAs into two alternating TMEM accumulators, a commit
// every 16 MMAs, never more than two such batches in flight. No epilogue: the
// accumulators are dropped. What this measures is the rate the tensor pipe
// retires 8-bit MMAs of the shape the GEMM kernels use, on this GPU at the
// clock the power cap allows -- the denominator of their roofline.
constexpr int PEAK_BATCH = 16;

template <bool IS_INT>
__global__ void __launch_bounds__(128, 1)
mma_peak_kernel(int64_t batches, uint32_t idesc, int32_t* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t done_bar[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // int8: any byte is a value. fp8: keep the exponent field away from all-ones
  // (NaN / infinity encodings) by clearing the top exponent bit.
  uint32_t x = 0x9e3779b9u * (threadIdx.x + 1) + 0x85ebca6bu * (blockIdx.x + 1);
  for (int i = threadIdx.x; i < (A_STAGE + B_STAGE) / 4; i += blockDim.x) {
    x ^= x << 13; x ^= x >> 17; x ^= x << 5;
    ((uint32_t*)smem)[i] = IS_INT ? x : (x & 0xbfbfbfbfu);
  }
  if (threadIdx.x == 0) {
    mbar_init(&done_bar[0], 1);
    mbar_init(&done_bar[1], 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&tmem_slot)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  if (warp == 0 && lane == 0) {
    const uint64_t ad = make_smem_desc(smem_u32(smem));
    const uint64_t bd = make_smem_desc(smem_u32(smem + A_STAGE));
    volatile int* abortp = &abort_flag;
    bool ok = true;
    for (int64_t b = 0; b < batches && ok; ++b) {
      const int slot = (int)(b & 1);
      // batch b reuses the barrier of batch b - 2: wait for that one first
      if (b >= 2) ok = mbar_wait(&done_bar[slot], (uint32_t)(((b - 2) >> 1) & 1), abortp);
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int i = 0; i < PEAK_BATCH; ++i)
        tc_mma<IS_INT>(tmem_base + (uint32_t)(slot * BN), ad + (uint64_t)(2 * (i & 3)),
                       bd + (uint64_t)(2 * (i & 3)), idesc, i > 0 ? 1u : 0u);
      tc_commit(&done_bar[slot]);
    }
    // drain: the last two batches
    for (int64_t b = batches > 2 ? batches - 2 : 0; b < batches && ok; ++b)
      ok = mbar_wait(&done_bar[b & 1], (uint32_t)((b >> 1) & 1), abortp);
    if (!ok && status != nullptr) atomicCAS(status, 0, 4);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(TMEM_COLS)
                 : "memory");
  }
}

// ---------------------------------------------------------------------------
// Plain CUDA-core kernel with the same epilogue; selected only through
// aqtb200_set_gemm_impl(1) to cross-check the tensor-core kernel.
__device__ __forceinline__ float qval(const uint8_t* p, int dt, int64_t i) {
  return dt == AQTB200_S8 ? (float)(signed char)p[i] : fp8_to_float(p[i], dt);
}

__global__ void gemm_simt_kernel(GemmParams P) {
  const int64_t total = P.b0 * P.b1 * P.m * P.n;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    int64_t col = i % P.n, t = i / P.n;
    int64_t row = t % P.m;
    t /= P.m;
    int64_t i1 = t % P.b1, i0 = t / P.b1;
    const uint8_t* ar = P.a + i0 * P.a_b0 + i1 * P.a_b1 + row * P.lda;
    const uint8_t* br = P.b + i0 * P.b_b0 + i1 * P.b_b1 + col * P.ldb;
    float r;
    uint32_t raw;
    if (P.is_int) {
      int acc = 0;
      for (int64_t k = 0; k < P.k; ++k) acc += (int)(signed char)ar[k] * (int)(signed char)br[k];
      raw = (uint32_t)acc;
      r = __int2float_rn(acc);
    } else {
      double acc = 0.0;
      for (int64_t k = 0; k < P.k; ++k)
        acc += (double)qval(ar, P.a_dtype, k) * (double)qval(br, P.b_dtype, k);
      r = (float)acc;
      raw = __float_as_uint(r);
    }
    if (P.acc_out) ((uint32_t*)P.acc_out)[i] = raw;
    int cur = P.d_dtype;
    r = round_to(r, cur);
    float sa = P.a_scale ? load1(P.a_scale, P.a_scale_dtype, i0 * P.sa_b0 + i1 * P.sa_b1 + row * P.sa_m) : 1.f;
    float sb = P.b_scale ? load1(P.b_scale, P.b_scale_dtype, i0 * P.sb_b0 + i1 * P.sb_b1 + col * P.sb_n) : 1.f;
    if (P.b_scale_first) {
      if (P.b_scale) r = scale_mul(r, sb, cur, P.b_scale_dtype);
      if (P.a_scale) r = scale_mul(r, sa, cur, P.a_scale_dtype);
    } else {
      if (P.a_scale) r = scale_mul(r, sa, cur, P.a_scale_dtype);
      if (P.b_scale) r = scale_mul(r, sb, cur, P.b_scale_dtype);
    }
    r = round_to(round_to(r, P.d_dtype), P.out_dtype);
    const int64_t oi = i0 * P.o_b0 + i1 * P.o_b1 + row * P.o_m + col * P.o_n;
    if (P.out == nullptr) continue;
    if (P.amax_out != nullptr) atomicMax(P.amax_out, __float_as_uint(r) & 0x7fffffffu);
    if (P.out_dtype == AQTB200_BF16)
      ((__nv_bfloat16*)P.out)[oi] = __float2bfloat16_rn(r);
    else
      ((float*)P.out)[oi] = r;
  }
}

// Dequantizing epilogue alone, on accumulators that already sit in memory
// (contiguous [b0][b1][m][n]); same arithmetic as the GEMM's epilogue.
__device__ __forceinline__ float dequant_one(const GemmParams& P, uint32_t raw, float sa, float sb) {
  float r = P.is_int ? __int2float_rn((int)raw) : __uint_as_float(raw);
  int cur = P.d_dtype;
  r = round_to(r, cur);
  if (P.b_scale_first) {
    if (P.b_scale) r = scale_mul(r, sb, cur, P.b_scale_dtype);
    if (P.a_scale) r = scale_mul(r, sa, cur, P.a_scale_dtype);
  } else {
    if (P.a_scale) r = scale_mul(r, sa, cur, P.a_scale_dtype);
    if (P.b_scale) r = scale_mul(r, sb, cur, P.b_scale_dtype);
  }
  return round_to(round_to(r, P.d_dtype), P.out_dtype);
}

// VEC: n % 4 == 0, acc 16-byte aligned; four consecutive columns per unit and
// two units in flight per thread.
template <bool VEC>
__global__ void __launch_bounds__(256) dequant_acc_kernel(GemmParams P, const uint32_t* acc) {
  constexpr int W = VEC ? 4 : 1;
  constexpr int UU = 2;
  const int64_t total = P.b0 * P.b1 * P.m * P.n / W;
  const int64_t nq = P.n / W;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  const int es = P.out_dtype == AQTB200_BF16 ? 2 : 4;
  uint32_t amax = 0;
  for (int64_t i0u = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i0u < total;
       i0u += nthreads * UU) {
    uint32_t raw[UU][W];
#pragma unroll
    for (int k = 0; k < UU; ++k) {
      const int64_t i = i0u + k * nthreads;
      if (i < total) {
        if (VEC) {
          const uint4 u = __ldg((const uint4*)acc + i);
          raw[k][0] = u.x; raw[k][W > 1 ? 1 : 0] = u.y; raw[k][W > 1 ? 2 : 0] = u.z;
          raw[k][W > 1 ? 3 : 0] = u.w;
        } else {
          raw[k][0] = acc[i];
        }
      }
    }
#pragma unroll
    for (int k = 0; k < UU; ++k) {
      const int64_t i = i0u + k * nthreads;
      if (i >= total) continue;
      const int64_t col = (i % nq) * W;
      int64_t t = i / nq;
      const int64_t row = t % P.m;
      t /= P.m;
      const int64_t i1 = t % P.b1, i0 = t / P.b1;
      const float sa = P.a_scale ? load1(P.a_scale, P.a_scale_dtype,
                                         i0 * P.sa_b0 + i1 * P.sa_b1 + row * P.sa_m)
                                 : 1.f;
      float res[W];
#pragma unroll
      for (int j = 0; j < W; ++j) {
        const float sb = P.b_scale ? load1(P.b_scale, P.b_scale_dtype,
                                           i0 * P.sb_b0 + i1 * P.sb_b1 + (col + j) * P.sb_n)
                                   : 1.f;
        res[j] = dequant_one(P, raw[k][j], sa, sb);
        amax_f32(amax, res[j]);
      }
      const int64_t oi = i0 * P.o_b0 + i1 * P.o_b1 + row * P.o_m + col * P.o_n;
      if (VEC && P.o_n == 1 && ((((uintptr_t)P.out) + (size_t)oi * es) & (4 * es - 1)) == 0) {
        if (es == 2) {
          __nv_bfloat162 p0 = __floats2bfloat162_rn(res[0], res[W > 1 ? 1 : 0]);
          __nv_bfloat162 p1 = __floats2bfloat162_rn(res[W > 1 ? 2 : 0], res[W > 1 ? 3 : 0]);
          *(uint2*)((__nv_bfloat16*)P.out + oi) = make_uint2(*(uint32_t*)&p0, *(uint32_t*)&p1);
        } else {
          *(float4*)((float*)P.out + oi) =
              make_float4(res[0], res[W > 1 ? 1 : 0], res[W > 1 ? 2 : 0], res[W > 1 ? 3 : 0]);
        }
      } else {
#pragma unroll
        for (int j = 0; j < W; ++j) {
          if (es == 2)
            ((__nv_bfloat16*)P.out)[oi + j * P.o_n] = __float2bfloat16_rn(res[j]);
          else
            ((float*)P.out)[oi + j * P.o_n] = res[j];
        }
      }
    }
  }
  // (every thread reaches this point: the loops above have no early exit)
  if (P.amax_out != nullptr) amax_publish(P.amax_out, amax, threadIdx.x & 31);
}


// ---------------------------------------------------------------------------
// Sum of one band of raw accumulators over the ranks of a row-sharded dot,
// dequantized once and written to every rank: the reduce-scatter, the
// dequantizing epilogue and the all-gather of the finished band in ONE kernel
// over peer memory. X.acc[r] is rank r's copy of the band ([m][n] 4-byte
// accumulators; the other ranks' through their peer mappings), X.out[r] rank
// r's copy of the band's place in the output. The copies are added in rank
// order, so the f32 sum does not depend on which rank computes the band. Needs
// n % 4 == 0, an unbatched dot and unit column stride of the output.
struct ExchangeArgs {
  const uint32_t* acc[AQTB200_MAX_RANKS];
  void* out[AQTB200_MAX_RANKS];
  int world;
  // division of an element position (< 2^31) by the column count as a multiply
  // and a shift: q = umulhi(e, div_mul) >> div_shr (div_mul == 0: n == 1)
  uint32_t div_mul, div_shr;
};


// ---------------------------------------------------------------------------
// host side

static int g_gemm_impl = 0;
static int g_sm_budget = 0;
static int gemm_sms() {
  int n = sm_count();
  return (g_sm_budget > 0 && g_sm_budget < n) ? g_sm_budget : n;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &p, 12000, cudaEnableDefault,
                                         &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

// 4-D map over a 1-byte tensor [b0][b1][rows][k] with k contiguous.
static int make_operand_map(CUtensorMap* tm, const void* ptr, int64_t k, int64_t rows, int64_t b1,
                            int64_t b0, int64_t ld, int64_t s_b1, int64_t s_b0, int box_rows) {
  EncodeTiledFn enc = get_encode_fn();
  AQT_REQUIRE(enc != nullptr, AQTB200_EDRIVER, "cuTensorMapEncodeTiled entry point not found");
  AQT_REQUIRE(((uintptr_t)ptr & 15) == 0, AQTB200_EINVAL, "operand not 16-byte aligned");
  if (b1 <= 1 || s_b1 == 0) s_b1 = ld * rows;
  if (b0 <= 1 || s_b0 == 0) s_b0 = s_b1 * std::max<int64_t>(b1, 1);
  AQT_REQUIRE(ld % 16 == 0 && s_b1 % 16 == 0 && s_b0 % 16 == 0, AQTB200_EINVAL,
              "operand strides must be multiples of 16 bytes (ld=%lld)", (long long)ld);
  cuuint64_t dims[4] = {(cuuint64_t)k, (cuuint64_t)rows, (cuuint64_t)std::max<int64_t>(b1, 1),
                        (cuuint64_t)std::max<int64_t>(b0, 1)};
  cuuint64_t strides[3] = {(cuuint64_t)ld, (cuuint64_t)s_b1, (cuuint64_t)s_b0};
  cuuint32_t box[4] = {(cuuint32_t)BK, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(ptr), dims, strides,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  AQT_REQUIRE(r == CUDA_SUCCESS, AQTB200_EDRIVER, "cuTensorMapEncodeTiled failed with %d", (int)r);
  return 0;
}

// 4-D map over a bf16 output [b0][b1][m][n] with n contiguous: boxes of 32 rows
// by 64 columns in the 128-byte swizzle (or 32 columns in the 64-byte swizzle),
// the layouts the epilogues stage their rows in.
static bool make_output_map(CUtensorMap* tm, void* ptr, int64_t n, int64_t m, int64_t b1,
                            int64_t b0, int64_t s_m, int64_t s_b1, int64_t s_b0, int box_cols) {
  EncodeTiledFn enc = get_encode_fn();
  if (enc == nullptr) return false;
  if (b1 <= 1 || s_b1 == 0) s_b1 = s_m * m;
  if (b0 <= 1 || s_b0 == 0) s_b0 = s_b1 * std::max<int64_t>(b1, 1);
  if (((uintptr_t)ptr & 15) || s_m % 8 || s_b1 % 8 || s_b0 % 8 || s_m <= 0 || s_b1 <= 0 || s_b0 <= 0)
    return false;
  cuuint64_t dims[4] = {(cuuint64_t)n, (cuuint64_t)m, (cuuint64_t)std::max<int64_t>(b1, 1),
                        (cuuint64_t)std::max<int64_t>(b0, 1)};
  cuuint64_t strides[3] = {(cuuint64_t)s_m * 2, (cuuint64_t)s_b1 * 2, (cuuint64_t)s_b0 * 2};
  cuuint32_t box[4] = {(cuuint32_t)box_cols, 32, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, ptr, dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE,
                   box_cols == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                   CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// 4-D map over the contiguous 32-bit accumulator tensor [b0][b1][m][n]: boxes
// of 32 rows by 16 columns (64 bytes) in the 64-byte swizzle.
static bool make_acc_map(CUtensorMap* tm, void* ptr, int64_t n, int64_t m, int64_t b1, int64_t b0) {
  EncodeTiledFn enc = get_encode_fn();
  if (enc == nullptr || ((uintptr_t)ptr & 15) || n % 4 != 0) return false;
  b1 = std::max<int64_t>(b1, 1);
  b0 = std::max<int64_t>(b0, 1);
  cuuint64_t dims[4] = {(cuuint64_t)n, (cuuint64_t)m, (cuuint64_t)b1, (cuuint64_t)b0};
  cuuint64_t strides[3] = {(cuuint64_t)n * 4, (cuuint64_t)n * m * 4, (cuuint64_t)n * m * b1 * 4};
  cuuint32_t box[4] = {16, 32, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, ptr, dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
                   CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

static bool is_fp8(int dt) { return dt == AQTB200_E4M3 || dt == AQTB200_E5M2; }

static int fill_params(const aqtb200_gemm_desc* d, int32_t* status, GemmParams& P, bool* empty) {
  AQT_REQUIRE(d != nullptr, AQTB200_EINVAL, "null gemm descriptor");
  AQT_REQUIRE(d->b0 >= 0 && d->b1 >= 0 && d->m >= 0 && d->n >= 0 && d->k >= 0, AQTB200_EINVAL,
              "negative extent");
  const bool ints = d->a_dtype == AQTB200_S8 && d->b_dtype == AQTB200_S8;
  const bool fps = is_fp8(d->a_dtype) && is_fp8(d->b_dtype);
  AQT_REQUIRE(ints || fps, AQTB200_EUNSUPPORTED,
              "operand dtypes %d x %d: need int8 x int8 or fp8 x fp8", d->a_dtype, d->b_dtype);
  AQT_REQUIRE(d->dequant_dtype == AQTB200_F32 || d->dequant_dtype == AQTB200_BF16, AQTB200_EINVAL,
              "dequant dtype must be f32 or bf16");
  AQT_REQUIRE(d->out_dtype == AQTB200_F32 || d->out_dtype == AQTB200_BF16, AQTB200_EINVAL,
              "out dtype must be f32 or bf16");
  *empty = d->b0 * d->b1 * d->m * d->n == 0;
  if (*empty) return 0;
  AQT_REQUIRE(d->out != nullptr || d->acc_out != nullptr, AQTB200_EINVAL, "null output");
  AQT_REQUIRE(d->k == 0 || (d->a != nullptr && d->b != nullptr), AQTB200_EINVAL, "null operand");
  AQT_REQUIRE(d->k < (int64_t)1 << 31 && d->m < (int64_t)1 << 31 && d->n < (int64_t)1 << 31,
              AQTB200_EUNSUPPORTED, "extent too large for a tensor map");

  P = GemmParams{};
  P.b0 = d->b0; P.b1 = d->b1; P.m = d->m; P.n = d->n; P.k = d->k;
  P.a_scale = d->a_scale; P.sa_b0 = d->a_scale_b0_stride; P.sa_b1 = d->a_scale_b1_stride;
  P.sa_m = d->a_scale_m_stride;
  P.b_scale = d->b_scale; P.sb_b0 = d->b_scale_b0_stride; P.sb_b1 = d->b_scale_b1_stride;
  P.sb_n = d->b_scale_n_stride;
  P.a_scale_dtype = d->a_scale_dtype; P.b_scale_dtype = d->b_scale_dtype;
  P.b_scale_first = d->b_scale_first; P.d_dtype = d->dequant_dtype; P.out_dtype = d->out_dtype;
  P.is_int = ints ? 1 : 0;
  P.out = d->out; P.o_b0 = d->out_b0_stride; P.o_b1 = d->out_b1_stride;
  P.o_m = d->out_m_stride; P.o_n = d->out_n_stride;
  P.acc_out = d->acc_out;
  P.amax_out = (uint32_t*)d->amax_out;
  P.stage_ok = d->out != nullptr && d->out_dtype == AQTB200_BF16 && d->out_n_stride == 1 &&
               (((uintptr_t)d->out) & 15) == 0 && d->out_m_stride % 8 == 0 &&
               d->out_b0_stride % 8 == 0 && d->out_b1_stride % 8 == 0;
  P.m_tiles = (d->m + BM - 1) / BM;
  P.n_tiles = (d->n + BN - 1) / BN;
  P.total_tiles = d->b0 * d->b1 * P.m_tiles * P.n_tiles;
  P.num_kb = std::max<int64_t>(1, (d->k + BK - 1) / BK);
  P.status = status;
  P.a = (const uint8_t*)d->a; P.b = (const uint8_t*)d->b;
  P.a_b0 = d->a_b0_stride; P.a_b1 = d->a_b1_stride; P.lda = d->lda;
  P.b_b0 = d->b_b0_stride; P.b_b1 = d->b_b1_stride; P.ldb = d->ldb;
  P.a_dtype = d->a_dtype; P.b_dtype = d->b_dtype;
  const uint32_t cfmt = ints ? 2u : 1u;
  const uint32_t afmt = ints ? 1u : (d->a_dtype == AQTB200_E5M2 ? 1u : 0u);
  const uint32_t bfmt = ints ? 1u : (d->b_dtype == AQTB200_E5M2 ? 1u : 0u);
  // A problem at most one tile wide lets the single-CTA kernel issue MMAs only
  // as wide as the columns that exist (a multiple of 16): the tensor pipe's
  // time scales with N, which is what makes a skinny GEMM -- a few tokens
  // against many weight rows, with the weights on the row side -- stream its
  // big operand at memory speed instead of multiplying zero columns.
  const int64_t n_mma = d->n < BN ? std::max<int64_t>(16, (d->n + 15) / 16 * 16) : BN;
  P.idesc = (cfmt << 4) | (afmt << 7) | (bfmt << 10) | ((uint32_t)(n_mma >> 3) << 17) |
            ((uint32_t)(BM >> 4) << 24);
  P.n_mma = (int)n_mma;
  P.stream_k = 0;
  P.pdl = 0;
  P.max_parts = 1;
  P.b_stage = (int)(n_mma * BK);
  P.stages1 = (int)std::min<int64_t>(MAX_STAGES1, (int64_t)(GEMM_SMEM - 1024) / (A_STAGE + P.b_stage));
  P.idesc2 = (cfmt << 4) | (afmt << 7) | (bfmt << 10) | ((uint32_t)(BN >> 3) << 17) |
             ((uint32_t)(256 >> 4) << 24);
  P.m_tiles2 = (d->m + 255) / 256;
  P.total_tiles2 = d->b0 * d->b1 * P.m_tiles2 * P.n_tiles;
  P.n_tiles3 = (d->n + 511) / 512;
  P.total_tiles3 = d->b0 * d->b1 * P.m_tiles2 * P.n_tiles3;

  return 0;
}

// Skinny problems on the single-CTA kernel with fewer tiles than half the SMs:
// whole tiles would leave most SMs idle while a few stream the long
// contraction. Cutting the sequence of all k-slabs into equal shares, one per
// CTA and up to four CTAs per tile, puts more SMs (and more bytes in flight)
// on the problem; tiles that straddle a share boundary are computed in parts.
// With at least half the SMs busy the stream from DRAM is already the bound
// (measured: equal shares then gain nothing, and the partial tiles cost), so
// whole tiles are kept. Returns the number of CTAs and the most parts a tile
// can have, or parts 1 for whole tiles.
constexpr int MAX_PARTS = 6;  // slots the fix-up can sum (see epilogue_split)
struct StreamPlan {
  int grid, parts;
};
static StreamPlan plan_stream(int64_t tiles, int64_t num_kb, int64_t n_mma, int sms) {
  StreamPlan none = {0, 1};
  if (n_mma > 64 || tiles <= 0 || num_kb < 16 || sms <= 0) return none;
  if (tiles * 2 > sms) return none;
  const int64_t grid = std::min<int64_t>(sms, tiles * 4);
  const int64_t share = tiles * num_kb / grid;  // >= num_kb / 4
  const int64_t parts = (num_kb + share - 1) / share + 1;
  if (parts > MAX_PARTS) return none;
  StreamPlan p = {(int)grid, (int)parts};
  return p;
}

// Whole tiles, round robin over a persistent grid: with w = ceil(tiles / SMs)
// waves no CTA can finish before w tiles' time, so the grid is cut to
// ceil(tiles / w) CTAs, the fewest that still need only w. Measured on the
// serving shape (224 tiles streaming 235 MB of weights): 112 CTAs with two
// tiles each are faster than 148 of which 76 take two -- fewer concurrent
// streams get more out of DRAM while the critical path stays two tiles.
static int balanced_grid(int64_t tiles, int sms) {
  if (tiles <= sms) return (int)std::max<int64_t>(tiles, 1);
  const int64_t waves = (tiles + sms - 1) / sms;
  return (int)((tiles + waves - 1) / waves);
}

static size_t split_workspace_bytes(int64_t tiles, int parts, int64_t n_mma) {
  const size_t counters = ((size_t)tiles * 4 * sizeof(int32_t) + 255) & ~(size_t)255;
  return counters + (size_t)tiles * parts * BM * n_mma * sizeof(uint32_t);
}

static bool single_cta_path(const aqtb200_gemm_desc* d) {
  // mirrors the kernel choice in gemm_dequant for the automatic setting
  return g_gemm_impl == 0 && !(d->m > 128 && d->n >= 128) && d->k > 0;
}

size_t gemm_workspace_bytes(const aqtb200_gemm_desc* d) {
  if (d == nullptr || !single_cta_path(d) || d->b0 * d->b1 * d->m * d->n == 0) return 0;
  const int64_t tiles = d->b0 * d->b1 * ((d->m + BM - 1) / BM) * ((d->n + BN - 1) / BN);
  const int64_t n_mma = d->n < BN ? std::max<int64_t>(16, (d->n + 15) / 16 * 16) : BN;
  const int64_t num_kb = std::max<int64_t>(1, (d->k + BK - 1) / BK);
  // the most any SM count up to the device's can need (fewer CTAs: fewer parts)
  const StreamPlan plan = plan_stream(tiles, num_kb, n_mma, sm_count());
  return plan.parts > 1 ? split_workspace_bytes(tiles, MAX_PARTS, n_mma) : 0;
}

int gemm_dequant(const aqtb200_gemm_desc* d, int32_t* status, cudaStream_t st, bool a_ready) {
  GemmParams P;
  bool empty = false;
  int rc0 = fill_params(d, status, P, &empty);
  if (rc0 || empty) return rc0;
  if (g_gemm_impl == 1 || d->k == 0) {
    int64_t total = d->b0 * d->b1 * d->m * d->n;
    int grid = (int)std::min<int64_t>((total + 255) / 256, (int64_t)sm_count() * 16);
    gemm_simt_kernel<<<grid, 256, 0, st>>>(P);
    AQT_CUDA_OK(cudaGetLastError()); count_launch();
    return 0;
  }

  // CTA pairs pay off once a 256-row tile is mostly full; skinny problems keep
  // the single-CTA 128-row tiles. Long contractions take the 256 x 512 pair
  // tile. g_gemm_impl 2 / 3 / 4 force one kernel.
  // Very short contractions with a large output are bound by the drain of the
  // accumulators alone: the wide kernel's sixteen epilogue warps drain fastest
  // (measured on the attention-score einsum, K = 128: 0.70 ms against 0.96 ms).
  const int64_t wide_tiles = d->b0 * d->b1 * ((d->m + BM2 - 1) / BM2) * ((d->n + BNW - 1) / BNW);
  const bool drain_bound = P.num_kb <= 2 && wide_tiles >= 2 * (int64_t)sm_count();
  bool wide = g_gemm_impl == 4 ? true
              : (g_gemm_impl == 0 && d->m > 128 && d->n > 256 &&
                 (P.num_kb >= WIDE_MIN_KB || drain_bound));
  const bool sa_bf = d->a_scale == nullptr || d->a_scale_dtype == AQTB200_BF16;
  const bool sb_bf = d->b_scale == nullptr || d->b_scale_dtype == AQTB200_BF16;
  const bool sa_f = d->a_scale == nullptr || d->a_scale_dtype == AQTB200_F32;
  const bool sb_f = d->b_scale == nullptr || d->b_scale_dtype == AQTB200_F32;
  int epi = 0;
  if (d->dequant_dtype == AQTB200_BF16 && d->out_dtype == AQTB200_BF16 && sa_bf && sb_bf) epi = 1;
  if (d->dequant_dtype == AQTB200_F32 && d->out_dtype == AQTB200_F32 && sa_f && sb_f) epi = 2;
  // Outputs that qualify for the staged bf16 epilogue leave through the TMA
  // unit when a tensor map can describe them; otherwise the same staged rows
  // are stored by the warps. The 256 x 512 kernel has only that epilogue and
  // one that writes the raw accumulators alone (no dequantized output); for
  // anything else (no map, other dtypes, both outputs wanted) the 256 x 256
  // kernel runs instead, whatever was asked for.
  CUtensorMap tmO;
  memset(&tmO, 0, sizeof(tmO));
  P.tma_store = 0;
  const bool can_map = epi == 1 && P.stage_ok;
  bool wide_raw = false;
  if (wide) {
    if (d->out == nullptr && d->acc_out != nullptr) {
      wide_raw = wide = make_acc_map(&tmO, d->acc_out, d->n, d->m, d->b1, d->b0);
    } else {
      wide = can_map && d->acc_out == nullptr &&
             make_output_map(&tmO, d->out, d->n, d->m, d->b1, d->b0, d->out_m_stride,
                             d->out_b1_stride, d->out_b0_stride, 32);
    }
    P.tma_store = wide ? 1 : 0;
  }
  {
    // how the wide kernel's epilogue gets its scales (see GemmParams)
    auto mode = [&](const void* ptr, int dtype, int64_t s0, int64_t s1, int64_t sx, int64_t extent) {
      if (ptr == nullptr) return 0;
      if (s0 == 0 && s1 == 0 && sx == 0) return 0;
      if (dtype == AQTB200_BF16 && sx == 1 && ((uintptr_t)ptr & 15) == 0 && s0 % 8 == 0 &&
          s1 % 8 == 0 && extent % 8 == 0)
        return 1;
      return 2;
    };
    P.sa_mode = mode(d->a_scale, d->a_scale_dtype, P.sa_b0, P.sa_b1, P.sa_m, d->m);
    P.sb_mode = mode(d->b_scale, d->b_scale_dtype, P.sb_b0, P.sb_b1, P.sb_n, d->n);
  }
  if (!wide && can_map)
    P.tma_store = make_output_map(&tmO, d->out, d->n, d->m, d->b1, d->b0, d->out_m_stride,
                                  d->out_b1_stride, d->out_b0_stride, 64) ? 1 : 0;
  // fewer than 128 columns: the single-CTA kernel with narrow MMAs (see fill_params)
  const bool pair = wide || (g_gemm_impl == 3 ? true
                                              : (g_gemm_impl == 2 ? false : d->m > 128 && d->n >= 128));
  CUtensorMap tmA, tmB;
  int rc = make_operand_map(&tmA, d->a, d->k, d->m, d->b1, d->b0, d->lda, d->a_b1_stride,
                            d->a_b0_stride, BM);
  if (rc) return rc;
  rc = make_operand_map(&tmB, d->b, d->k, d->n, d->b1, d->b0, d->ldb, d->b_b1_stride,
                        d->b_b0_stride, pair ? 128 : P.b_stage / BK);
  if (rc) return rc;
  int stream_grid = 0;
  if (!pair && single_cta_path(d) && d->workspace != nullptr) {
    const StreamPlan plan = plan_stream(P.total_tiles, P.num_kb, P.n_mma, gemm_sms());
    if (plan.parts > 1 &&
        d->workspace_bytes >= split_workspace_bytes(P.total_tiles, plan.parts, P.n_mma) &&
        ((uintptr_t)d->workspace & 255) == 0) {
      P.stream_k = 1;
      P.max_parts = plan.parts;
      stream_grid = plan.grid;
      const size_t counters = ((size_t)P.total_tiles * 4 * sizeof(int32_t) + 255) & ~(size_t)255;
      P.tile_counter = (int32_t*)d->workspace;
      P.partials = (uint32_t*)((char*)d->workspace + counters);
      AQT_CUDA_OK(cudaMemsetAsync(P.tile_counter, 0, counters, st));
    }
  }
  // dependent launch: single-CTA kernel, whole tiles (no memset node between the
  // producing kernel and this one), A complete before that kernel
  P.pdl = (!pair && a_ready && !P.stream_k && g_gemm_impl != 1) ? 1 : 0;
  const int64_t pair_tiles = wide ? P.total_tiles3 : P.total_tiles2;
  const int grid = pair ? 2 * std::max((int)std::min<int64_t>(pair_tiles, gemm_sms() / 2), 1)
                        : (stream_grid ? stream_grid : balanced_grid(P.total_tiles, gemm_sms()));
  const size_t smem = wide ? GEMM3_SMEM : (pair ? GEMM2_SMEM : GEMM_SMEM);
  // the shared-memory opt-in is a per-device attribute of each kernel
  int dev = 0;
  AQT_CUDA_OK(cudaGetDevice(&dev));
  dev = dev & 63;
#define AQT_LAUNCH_GEMM(KERNEL, I, E)                                                         \
  do {                                                                                        \
    static bool attr_done[64] = {false};                                                      \
    if (!attr_done[dev]) {                                                                    \
      AQT_CUDA_OK(cudaFuncSetAttribute(KERNEL<I, E>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                       (int)smem));                                           \
      attr_done[dev] = true;                                                                  \
    }                                                                                         \
    if (P.pdl) {                                                                              \
      cudaLaunchConfig_t cfg = {};                                                            \
      cfg.gridDim = dim3(grid);                                                               \
      cfg.blockDim = dim3(GEMM_THREADS);                                                      \
      cfg.dynamicSmemBytes = smem;                                                            \
      cfg.stream = st;                                                                        \
      cudaLaunchAttribute attr[1];                                                            \
      attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;                        \
      attr[0].val.programmaticStreamSerializationAllowed = 1;                                 \
      cfg.attrs = attr;                                                                       \
      cfg.numAttrs = 1;                                                                       \
      AQT_CUDA_OK(cudaLaunchKernelEx(&cfg, KERNEL<I, E>, tmA, tmB, tmO, P));                  \
    } else {                                                                                  \
      KERNEL<I, E><<<grid, GEMM_THREADS, smem, st>>>(tmA, tmB, tmO, P);                       \
    }                                                                                         \
  } while (0)
#define AQT_LAUNCH_GEMM_E(KERNEL, I)                    \
  do {                                                  \
    if (epi == 1) AQT_LAUNCH_GEMM(KERNEL, I, 1);        \
    else if (epi == 2) AQT_LAUNCH_GEMM(KERNEL, I, 2);   \
    else AQT_LAUNCH_GEMM(KERNEL, I, 0);                 \
  } while (0)
  if (wide) {
#define AQT_LAUNCH_WIDE(I, R)                                                                  \
  do {                                                                                         \
    static bool attr_done[64] = {false};                                                       \
    if (!attr_done[dev]) {                                                                     \
      AQT_CUDA_OK(cudaFuncSetAttribute(gemm_tcgen05_wide_kernel<I, R>,                         \
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
      attr_done[dev] = true;                                                                   \
    }                                                                                          \
    gemm_tcgen05_wide_kernel<I, R><<<grid, WIDE_THREADS, smem, st>>>(tmA, tmB, tmO, P);        \
  } while (0)
    if (P.is_int) { if (wide_raw) AQT_LAUNCH_WIDE(true, true); else AQT_LAUNCH_WIDE(true, false); }
    else { if (wide_raw) AQT_LAUNCH_WIDE(false, true); else AQT_LAUNCH_WIDE(false, false); }
#undef AQT_LAUNCH_WIDE
  } else if (pair) {
    if (P.is_int) AQT_LAUNCH_GEMM_E(gemm_tcgen05_pair_kernel, true);
    else AQT_LAUNCH_GEMM_E(gemm_tcgen05_pair_kernel, false);
  } else {
    if (P.is_int) AQT_LAUNCH_GEMM_E(gemm_tcgen05_kernel, true);
    else AQT_LAUNCH_GEMM_E(gemm_tcgen05_kernel, false);
  }
#undef AQT_LAUNCH_GEMM_E
#undef AQT_LAUNCH_GEMM
  AQT_CUDA_OK(cudaGetLastError()); count_launch();
  return 0;
}

int dequant_acc(const aqtb200_gemm_desc* d, const void* acc, cudaStream_t st) {
  GemmParams P;
  bool empty = false;
  int rc0 = fill_params(d, nullptr, P, &empty);
  if (rc0 || empty) return rc0;
  AQT_REQUIRE(acc != nullptr && d->out != nullptr, AQTB200_EINVAL, "null accumulator or output");
  const int64_t total = d->b0 * d->b1 * d->m * d->n;
  const bool vec = d->n % 4 == 0 && (((uintptr_t)acc) & 15) == 0;
  int grid = (int)std::min<int64_t>((total / (vec ? 4 : 1) + 511) / 512, (int64_t)sm_count() * 8);
  grid = std::max(grid, 1);
  if (vec)
    dequant_acc_kernel<true><<<grid, 256, 0, st>>>(P, (const uint32_t*)acc);
  else
    dequant_acc_kernel<false><<<grid, 256, 0, st>>>(P, (const uint32_t*)acc);
  AQT_CUDA_OK(cudaGetLastError()); count_launch();
  return 0;
}

// The accumulators are pulled through the TMA unit: one
// thread per CTA requests 32 KB stages (one chunk of every rank's band, the
// peers' chunks straight from their memory) with bulk copies into a six-deep
// ring, so 192 KB per SM are in flight whatever the register budget -- what a
// read over NVLink, microseconds away, needs to run at link speed on a few
// SMs (measured at two ranks: 16 SMs do what plain loads from 1024 threads
// per SM needed 32 for). Sixteen warps add the chunks in rank order,
// dequantize and store the result to every rank. Waits are bounded; a wait that runs out sets *status.
constexpr int EX_STAGE_BYTES = 32 * 1024;
constexpr int EX_STAGES = 6;
constexpr int EX_CONSUMERS = 16;
constexpr int EX_THREADS = 32 * (1 + EX_CONSUMERS);
constexpr size_t EX_SMEM = (size_t)EX_STAGES * EX_STAGE_BYTES + 128;

// FAST: the all-bf16 chain (bf16 dequantization, output and scales) in packed
// arithmetic, as in the GEMM's own bf16 epilogue; otherwise the general chain.
// The band has fewer than 2^32 elements (checked by the host), so positions
// are 32-bit.
template <int WORLD, bool FAST>
__global__ void __launch_bounds__(EX_THREADS, 1)
exchange_tma_kernel(GemmParams P, ExchangeArgs X, int32_t* status) {
  constexpr int CHUNK = EX_STAGE_BYTES / WORLD;  // bytes of one rank's share of a stage
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 127) & ~(uintptr_t)127);
  __shared__ __align__(8) uint64_t full_bar[EX_STAGES];
  __shared__ __align__(8) uint64_t empty_bar[EX_STAGES];
  __shared__ int abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t total_bytes = P.m * P.n * 4;
  const int64_t chunks = (total_bytes + CHUNK - 1) / CHUNK;
  if (threadIdx.x == 0) {
    for (int s = 0; s < EX_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], EX_CONSUMERS);
    }
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();
  volatile int* abortp = &abort_flag;
  int stage = 0;
  uint32_t phase = 0;
  if (warp == 0) {
    if (lane == 0) {
      for (int64_t c = blockIdx.x; c < chunks; c += gridDim.x) {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1, abortp)) {
          *abortp = 1;
          if (status) atomicCAS(status, 0, 4);
          break;
        }
        const uint32_t bytes = (uint32_t)min((int64_t)CHUNK, total_bytes - c * CHUNK);
        mbar_expect_tx(&full_bar[stage], WORLD * bytes);
#pragma unroll
        for (int r = 0; r < WORLD; ++r)
          bulk_load(smem + stage * EX_STAGE_BYTES + r * CHUNK, (const char*)X.acc[r] + c * CHUNK,
                    bytes, &full_bar[stage]);
        if (++stage == EX_STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else {
    const int tid = threadIdx.x - 32;
    const int es = P.out_dtype == AQTB200_BF16 ? 2 : 4;
    const uint32_t n32 = (uint32_t)P.n;
    const bool has_a = P.a_scale != nullptr, has_b = P.b_scale != nullptr;
    const bool sa_const = !has_a || P.sa_m == 0, sb_const = !has_b || P.sb_n == 0;
    const float sa0 = has_a ? load1(P.a_scale, P.a_scale_dtype, 0) : 1.f;
    const float sb0 = has_b ? load1(P.b_scale, P.b_scale_dtype, 0) : 1.f;
    for (int64_t c = blockIdx.x; c < chunks; c += gridDim.x) {
      int ok = mbar_wait(&full_bar[stage], phase, abortp) ? 1 : 0;
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) { *abortp = 1; if (status) atomicCAS(status, 0, 5); }
        break;
      }
      const int units = (int)(min((int64_t)CHUNK, total_bytes - c * CHUNK) >> 4);
      const uint8_t* sp = smem + stage * EX_STAGE_BYTES;
      const uint32_t e0 = (uint32_t)c * (uint32_t)(CHUNK >> 2);
#pragma unroll 2
      for (int u = tid; u < units; u += 32 * EX_CONSUMERS) {
        const uint4 v0 = *(const uint4*)(sp + u * 16);
        uint32_t raw[4] = {v0.x, v0.y, v0.z, v0.w};
#pragma unroll
        for (int r = 1; r < WORLD; ++r) {
          const uint4 vr = *(const uint4*)(sp + r * CHUNK + u * 16);
          const uint32_t w[4] = {vr.x, vr.y, vr.z, vr.w};
#pragma unroll
          for (int j = 0; j < 4; ++j)
            raw[j] = P.is_int ? raw[j] + w[j]
                              : __float_as_uint(__fadd_rn(__uint_as_float(raw[j]), __uint_as_float(w[j])));
        }
        const uint32_t e = e0 + (uint32_t)u * 4u;  // first of four elements of one row
        const uint32_t row = X.div_mul ? (__umulhi(e, X.div_mul) >> X.div_shr) : e;
        const uint32_t col = e - row * n32;
        const float sa = sa_const ? sa0 : load1(P.a_scale, P.a_scale_dtype, (int64_t)row * P.sa_m);
        const int64_t oi = (int64_t)row * P.o_m + col;
        if constexpr (FAST) {
          const __nv_bfloat162 sa2 = __float2bfloat162_rn(sa);
          __nv_bfloat162 sb2[2];
          if (sb_const) {
            sb2[0] = sb2[1] = __float2bfloat162_rn(sb0);
          } else if (P.sb_n == 1) {
            const uint2 w2 = __ldg((const uint2*)((const __nv_bfloat16*)P.b_scale + col));
            sb2[0] = *(const __nv_bfloat162*)&w2.x;
            sb2[1] = *(const __nv_bfloat162*)&w2.y;
          } else {
            const __nv_bfloat16* bs = (const __nv_bfloat16*)P.b_scale;
            sb2[0] = __halves2bfloat162(bs[(int64_t)col * P.sb_n], bs[(int64_t)(col + 1) * P.sb_n]);
            sb2[1] = __halves2bfloat162(bs[(int64_t)(col + 2) * P.sb_n], bs[(int64_t)(col + 3) * P.sb_n]);
          }
          uint32_t o[2];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const float f0 = P.is_int ? __int2float_rn((int)raw[2 * h]) : __uint_as_float(raw[2 * h]);
            const float f1 = P.is_int ? __int2float_rn((int)raw[2 * h + 1]) : __uint_as_float(raw[2 * h + 1]);
            __nv_bfloat162 v = __floats2bfloat162_rn(f0, f1);
            if (P.b_scale_first) {
              if (has_b) v = __hmul2(v, sb2[h]);
              if (has_a) v = __hmul2(v, sa2);
            } else {
              if (has_a) v = __hmul2(v, sa2);
              if (has_b) v = __hmul2(v, sb2[h]);
            }
            o[h] = *(const uint32_t*)&v;
          }
#pragma unroll
          for (int r = 0; r < WORLD; ++r)
            *(uint2*)((__nv_bfloat16*)X.out[r] + oi) = make_uint2(o[0], o[1]);
        } else {
          float res[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float sb = sb_const ? sb0
                                      : load1(P.b_scale, P.b_scale_dtype, (int64_t)(col + j) * P.sb_n);
            res[j] = dequant_one(P, raw[j], sa, sb);
          }
          if (es == 2) {
            const __nv_bfloat162 p0 = __floats2bfloat162_rn(res[0], res[1]);
            const __nv_bfloat162 p1 = __floats2bfloat162_rn(res[2], res[3]);
            const uint2 o = make_uint2(*(const uint32_t*)&p0, *(const uint32_t*)&p1);
#pragma unroll
            for (int r = 0; r < WORLD; ++r) *(uint2*)((__nv_bfloat16*)X.out[r] + oi) = o;
          } else {
            const float4 o = make_float4(res[0], res[1], res[2], res[3]);
#pragma unroll
            for (int r = 0; r < WORLD; ++r) *(float4*)((float*)X.out[r] + oi) = o;
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[stage]);
      if (++stage == EX_STAGES) { stage = 0; phase ^= 1; }
    }
  }
  __syncthreads();
  if (*abortp) {
    // copies still in flight must land before the shared memory is released
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) { }
  }
}

int exchange_dequant(const aqtb200_gemm_desc* d, const aqtb200_exchange_desc* x, int32_t* status,
                     cudaStream_t st) {
  GemmParams P;
  bool empty = false;
  int rc0 = fill_params(d, nullptr, P, &empty);
  if (rc0 || empty) return rc0;
  AQT_REQUIRE(x != nullptr, AQTB200_EINVAL, "null exchange descriptor");
  AQT_REQUIRE(x->world == 2 || x->world == 4 || x->world == 8, AQTB200_EUNSUPPORTED,
              "the fused exchange handles 2, 4 or 8 ranks");
  AQT_REQUIRE(x->rank >= 0 && x->rank < x->world, AQTB200_EINVAL, "rank out of range");
  AQT_REQUIRE(d->b0 * d->b1 == 1 && d->n % 4 == 0 && P.o_n == 1, AQTB200_EUNSUPPORTED,
              "the fused exchange needs an unbatched dot, n % 4 == 0 and unit output column stride");
  AQT_REQUIRE(d->amax_out == nullptr, AQTB200_EUNSUPPORTED, "no amax_out in the fused exchange");
  AQT_REQUIRE(d->m * d->n < ((int64_t)1 << 31), AQTB200_EUNSUPPORTED,
              "a band of the fused exchange holds fewer than 2^31 elements");
  const int es = d->out_dtype == AQTB200_BF16 ? 2 : 4;
  AQT_REQUIRE((P.o_m * es) % (4 * es) == 0, AQTB200_EUNSUPPORTED, "output rows must keep 4-element alignment");
  ExchangeArgs X{};
  X.world = x->world;
  // exact for numerators below 2^31: mul = ceil(2^(31 + ceil(log2 n)) / n), shr = ceil(log2 n) - 1
  X.div_mul = 0;
  X.div_shr = 0;
  if (d->n > 1) {
    int lg = 0;
    while (((int64_t)1 << lg) < d->n) ++lg;
    const int p2 = 31 + lg;
    X.div_mul = (uint32_t)((((uint64_t)1 << p2) + (uint64_t)d->n - 1) / (uint64_t)d->n);
    X.div_shr = (uint32_t)(p2 - 32);
  }
  for (int r = 0; r < x->world; ++r) {
    AQT_REQUIRE(x->acc[r] != nullptr && x->out[r] != nullptr, AQTB200_EINVAL, "null band pointer");
    AQT_REQUIRE(((uintptr_t)x->acc[r] & 15) == 0 && ((uintptr_t)x->out[r] & (4 * es - 1)) == 0,
                AQTB200_EINVAL, "band pointers must be 16-byte (accumulators) / 4-element (output) aligned");
    X.acc[r] = (const uint32_t*)x->acc[r];
    X.out[r] = x->out[r];
  }
  const int64_t chunks = (d->m * d->n * 4 + EX_STAGE_BYTES / x->world - 1) / (EX_STAGE_BYTES / x->world);
  const int64_t cap = x->max_sms > 0 ? x->max_sms : sm_count();
  const int grid = (int)std::max<int64_t>(1, std::min(chunks, cap));
  int dev = 0;
  AQT_CUDA_OK(cudaGetDevice(&dev));
  dev &= 63;
#define AQT_LAUNCH_EXCHANGE(W, F)                                                               \
  do {                                                                                          \
    static bool attr_done[64] = {false};                                                        \
    if (!attr_done[dev]) {                                                                      \
      AQT_CUDA_OK(cudaFuncSetAttribute(exchange_tma_kernel<W, F>,                               \
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)EX_SMEM)); \
      attr_done[dev] = true;                                                                    \
    }                                                                                           \
    exchange_tma_kernel<W, F><<<grid, EX_THREADS, EX_SMEM, st>>>(P, X, status);                 \
  } while (0)
  const bool sa_bf = d->a_scale == nullptr || d->a_scale_dtype == AQTB200_BF16;
  const bool sb_bf = d->b_scale == nullptr || d->b_scale_dtype == AQTB200_BF16;
  const bool fast = d->dequant_dtype == AQTB200_BF16 && d->out_dtype == AQTB200_BF16 && sa_bf && sb_bf &&
                    (d->b_scale == nullptr || P.sb_n != 1 || ((uintptr_t)d->b_scale & 7) == 0);
  if (x->world == 2) { if (fast) AQT_LAUNCH_EXCHANGE(2, true); else AQT_LAUNCH_EXCHANGE(2, false); }
  else if (x->world == 4) { if (fast) AQT_LAUNCH_EXCHANGE(4, true); else AQT_LAUNCH_EXCHANGE(4, false); }
  else { if (fast) AQT_LAUNCH_EXCHANGE(8, true); else AQT_LAUNCH_EXCHANGE(8, false); }
#undef AQT_LAUNCH_EXCHANGE
  AQT_CUDA_OK(cudaGetLastError()); count_launch();
  return 0;
}

}  // namespace aqtb200

extern "C" {

int aqtb200_gemm_dequant(const aqtb200_gemm_desc* desc, int32_t* status, void* stream) {
  return aqtb200::gemm_dequant(desc, status, (cudaStream_t)stream, false);
}

size_t aqtb200_gemm_workspace_bytes(const aqtb200_gemm_desc* desc) {
  return aqtb200::gemm_workspace_bytes(desc);
}

int aqtb200_mma_peak(int32_t is_int, int64_t mmas_per_sm, int32_t* status, void* stream) {
  using namespace aqtb200;
  AQT_REQUIRE(mmas_per_sm > 0 && mmas_per_sm < ((int64_t)1 << 40), AQTB200_EINVAL,
              "mmas_per_sm out of range");
  const int64_t batches = (mmas_per_sm + PEAK_BATCH - 1) / PEAK_BATCH;
  const uint32_t cfmt = is_int ? 2u : 1u, abfmt = is_int ? 1u : 0u;  // s8 x s8 -> s32, e4m3 x e4m3 -> f32
  const uint32_t idesc = (cfmt << 4) | (abfmt << 7) | (abfmt << 10) | ((uint32_t)(BN >> 3) << 17) |
                         ((uint32_t)(BM >> 4) << 24);
  const size_t smem = A_STAGE + B_STAGE + 1024;
  if (is_int) {
    AQT_CUDA_OK(cudaFuncSetAttribute(mma_peak_kernel<true>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    mma_peak_kernel<true><<<sm_count(), 128, smem, (cudaStream_t)stream>>>(batches, idesc, status);
  } else {
    AQT_CUDA_OK(cudaFuncSetAttribute(mma_peak_kernel<false>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    mma_peak_kernel<false><<<sm_count(), 128, smem, (cudaStream_t)stream>>>(batches, idesc, status);
  }
  AQT_CUDA_OK(cudaGetLastError());
  count_launch();
  return 0;
}

int aqtb200_set_gemm_sm_budget(int max_sms) {
  if (max_sms < 0) return AQTB200_EINVAL;
  aqtb200::g_sm_budget = max_sms;
  return 0;
}

int aqtb200_set_gemm_impl(int impl) {
  if (impl < 0 || impl > 4) return AQTB200_EINVAL;
  aqtb200::g_gemm_impl = impl;
  return 0;
}

}  // extern "C"
