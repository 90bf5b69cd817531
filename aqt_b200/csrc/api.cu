// C ABI glue: error reporting, device queries and aqtb200_dot_general_raw,
// which strings the quantize kernels and the GEMM into one DotGeneralRaw call.
#include <atomic>
#include <cstdarg>
#include <cstdio>

#include <nvtx3/nvToolsExt.h>

#include "common.cuh"

namespace aqtb200 {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

static std::atomic<long long> g_launches{0};
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

int sm_count();
int gemm_dequant(const aqtb200_gemm_desc* d, int32_t* status, cudaStream_t st, bool a_ready);
size_t gemm_workspace_bytes(const aqtb200_gemm_desc* d);
int dequant_acc(const aqtb200_gemm_desc* d, const void* acc, cudaStream_t st);
int exchange_dequant(const aqtb200_gemm_desc* d, const aqtb200_exchange_desc* x, int32_t* status,
                     cudaStream_t st);

static size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

struct Side {
  const void* q;
  int q_dtype;
  int64_t ld, s_b1, s_b0;
  const void* scale;
  int scale_dtype;
  int64_t sc_b0, sc_b1, sc_row;
};

static int prepare_side(const aqtb200_view& v, const aqtb200_view& pre, const aqtb200_view& noise,
                        const aqtb200_quant_spec& spec, const void* scale_in, int is_quantized,
                        void* q_out, void* scale_out, void* ws, size_t ws_bytes, cudaStream_t st,
                        Side* out) {
  if (is_quantized) {
    AQT_REQUIRE(v.col_stride == 1 || v.cols <= 1, AQTB200_EUNSUPPORTED,
                "a pre-quantized operand must have the contraction index contiguous");
    AQT_REQUIRE(scale_in != nullptr, AQTB200_EINVAL, "pre-quantized operand without scale");
    out->q = v.ptr;
    out->q_dtype = v.dtype;
    out->ld = v.row_stride;
    out->s_b1 = v.b1_stride;
    out->s_b0 = v.b0_stride;
    out->scale = scale_in;
  } else {
    int rc = aqtb200_quantize(&v, pre.ptr ? &pre : nullptr, noise.ptr ? &noise : nullptr, &spec,
                              scale_in, q_out, scale_out, ws, ws_bytes, st);
    if (rc) return rc;
    out->q = q_out;
    out->q_dtype = spec.qdtype;
    out->ld = aqtb200_round_up(v.cols, 16);
    out->s_b1 = v.rows * out->ld;
    out->s_b0 = v.b1 * out->s_b1;
    out->scale = scale_out != nullptr ? scale_out : scale_in;
  }
  out->scale_dtype = spec.scale_dtype;
  if (spec.per_tensor) {
    out->sc_b0 = out->sc_b1 = out->sc_row = 0;
  } else {
    out->sc_row = 1;
    out->sc_b1 = v.rows;
    out->sc_b0 = v.b1 * v.rows;
  }
  return 0;
}

// Scale side of an operand as aqtb200_dot_general_raw left it (no kernels run).
static void side_after_quantize(const aqtb200_view& v, const aqtb200_quant_spec& spec,
                                const void* scale_in, int is_quantized, void* q_out,
                                void* scale_out, Side* out) {
  if (is_quantized) {
    out->q = v.ptr; out->q_dtype = v.dtype; out->ld = v.row_stride;
    out->s_b1 = v.b1_stride; out->s_b0 = v.b0_stride; out->scale = scale_in;
  } else {
    out->q = q_out; out->q_dtype = spec.qdtype; out->ld = aqtb200_round_up(v.cols, 16);
    out->s_b1 = v.rows * out->ld; out->s_b0 = v.b1 * out->s_b1;
    out->scale = scale_out != nullptr ? scale_out : scale_in;
  }
  out->scale_dtype = spec.scale_dtype;
  if (spec.per_tensor) {
    out->sc_b0 = out->sc_b1 = out->sc_row = 0;
  } else {
    out->sc_row = 1; out->sc_b1 = v.rows; out->sc_b0 = v.b1 * v.rows;
  }
}

static void fill_gemm_desc(const aqtb200_dg_raw_desc* d, const Side& L, const Side& R,
                           aqtb200_gemm_desc* gp) {
  aqtb200_gemm_desc& g = *gp;
  g.b0 = d->lhs.b0; g.b1 = d->lhs.b1; g.k = d->lhs.cols;
  const Side& A = d->swap_ab ? R : L;
  const Side& B = d->swap_ab ? L : R;
  g.m = d->swap_ab ? d->rhs.rows : d->lhs.rows;
  g.n = d->swap_ab ? d->lhs.rows : d->rhs.rows;
  g.a = A.q; g.a_b0_stride = A.s_b0; g.a_b1_stride = A.s_b1; g.lda = A.ld; g.a_dtype = A.q_dtype;
  g.b = B.q; g.b_b0_stride = B.s_b0; g.b_b1_stride = B.s_b1; g.ldb = B.ld; g.b_dtype = B.q_dtype;
  g.a_scale = A.scale; g.a_scale_dtype = A.scale_dtype;
  g.a_scale_b0_stride = A.sc_b0; g.a_scale_b1_stride = A.sc_b1; g.a_scale_m_stride = A.sc_row;
  g.b_scale = B.scale; g.b_scale_dtype = B.scale_dtype;
  g.b_scale_b0_stride = B.sc_b0; g.b_scale_b1_stride = B.sc_b1; g.b_scale_n_stride = B.sc_row;
  // The reference multiplies by the lhs scale first (aqt_dot_general.py:939-957).
  g.b_scale_first = d->swap_ab ? 1 : 0;
  g.dequant_dtype = d->dequant_dtype;
  g.out = d->out; g.out_dtype = d->out_dtype;
  g.out_b0_stride = d->out_b0_stride; g.out_b1_stride = d->out_b1_stride;
  g.out_m_stride = d->swap_ab ? d->out_n_stride : d->out_m_stride;
  g.out_n_stride = d->swap_ab ? d->out_m_stride : d->out_n_stride;
  g.acc_out = d->acc_out;
  g.amax_out = d->amax_out;
}

}  // namespace aqtb200

using namespace aqtb200;

extern "C" {

int aqtb200_version(void) { return AQTB200_VERSION; }

const char* aqtb200_last_error(void) { return g_err; }

int64_t aqtb200_kernel_launch_count(void) { return (int64_t)g_launches.load(); }

int aqtb200_device_sm_count(int* out) {
  if (out == nullptr) return AQTB200_EINVAL;
  *out = sm_count();
  return 0;
}

// extents and kernel choice are all gemm_workspace_bytes looks at
static size_t raw_gemm_scratch(const aqtb200_dg_raw_desc* d) {
  aqtb200_gemm_desc g{};
  g.b0 = d->lhs.b0; g.b1 = d->lhs.b1; g.k = d->lhs.cols;
  g.m = d->swap_ab ? d->rhs.rows : d->lhs.rows;
  g.n = d->swap_ab ? d->lhs.rows : d->rhs.rows;
  return gemm_workspace_bytes(&g);
}

size_t aqtb200_dot_general_raw_workspace_bytes(const aqtb200_dg_raw_desc* d) {
  if (d == nullptr) return 0;
  return align256(aqtb200_quantize_workspace_bytes(&d->lhs, &d->lhs_spec)) +
         align256(aqtb200_quantize_workspace_bytes(&d->rhs, &d->rhs_spec)) +
         align256(raw_gemm_scratch(d));
}

int aqtb200_dot_general_raw(const aqtb200_dg_raw_desc* d, void* workspace, size_t workspace_bytes,
                            int32_t* status, void* stream) {
  AQT_REQUIRE(d != nullptr, AQTB200_EINVAL, "null descriptor");
  cudaStream_t st = (cudaStream_t)stream;
  AQT_REQUIRE(d->lhs.b0 == d->rhs.b0 && d->lhs.b1 == d->rhs.b1, AQTB200_EINVAL,
              "batch extents differ: lhs [%lld,%lld] rhs [%lld,%lld]", (long long)d->lhs.b0,
              (long long)d->lhs.b1, (long long)d->rhs.b0, (long long)d->rhs.b1);
  AQT_REQUIRE(d->lhs.cols == d->rhs.cols, AQTB200_EINVAL, "contraction extents differ: %lld vs %lld",
              (long long)d->lhs.cols, (long long)d->rhs.cols);
  size_t need = aqtb200_dot_general_raw_workspace_bytes(d);
  AQT_REQUIRE(workspace != nullptr && workspace_bytes >= need && ((uintptr_t)workspace & 255) == 0,
              AQTB200_EWORKSPACE, "workspace: need %zu bytes, 256-byte aligned (got %zu)", need,
              workspace_bytes);
  size_t lhs_ws = align256(aqtb200_quantize_workspace_bytes(&d->lhs, &d->lhs_spec));
  // NVTX range around the pass (a no-op unless a profiler is attached)
  struct Scope {
    bool on;
    explicit Scope(const char* name) : on(name != nullptr && name[0] != 0) {
      if (on) nvtxRangePushA(name);
    }
    ~Scope() { if (on) nvtxRangePop(); }
  } scope(d->scope_name);
  Side L{}, R{};
  int rc = prepare_side(d->lhs, d->lhs_prescale, d->lhs_noise, d->lhs_spec, d->lhs_scale_in,
                        d->lhs_is_quantized, d->lhs_q, d->lhs_scale, workspace, lhs_ws, st, &L);
  if (rc) return rc;
  rc = prepare_side(d->rhs, d->rhs_prescale, d->rhs_noise, d->rhs_spec, d->rhs_scale_in,
                    d->rhs_is_quantized, d->rhs_q, d->rhs_scale, (char*)workspace + lhs_ws,
                    workspace_bytes - lhs_ws, st, &R);
  if (rc) return rc;

  aqtb200_gemm_desc g{};
  fill_gemm_desc(d, L, R, &g);
  const size_t rhs_ws = align256(aqtb200_quantize_workspace_bytes(&d->rhs, &d->rhs_spec));
  const size_t gemm_ws = raw_gemm_scratch(d);
  if (gemm_ws > 0 && workspace_bytes >= lhs_ws + rhs_ws + gemm_ws) {
    g.workspace = (char*)workspace + lhs_ws + rhs_ws;
    g.workspace_bytes = gemm_ws;
  }
  // the GEMM may start under the kernel that quantizes its B operand when its A
  // operand (the rows side after the swap) came in already quantized
  const bool a_given = d->swap_ab ? d->rhs_is_quantized != 0 : d->lhs_is_quantized != 0;
  const bool b_made_here = d->swap_ab ? d->lhs_is_quantized == 0 : d->rhs_is_quantized == 0;
  return gemm_dequant(&g, status, st, a_given && b_made_here);
}

int aqtb200_dot_general_raw_dequant(const aqtb200_dg_raw_desc* d, void* stream) {
  AQT_REQUIRE(d != nullptr, AQTB200_EINVAL, "null descriptor");
  AQT_REQUIRE(d->acc_out != nullptr && d->out != nullptr, AQTB200_EINVAL,
              "deferred dequantization needs both acc_out and out");
  Side L{}, R{};
  side_after_quantize(d->lhs, d->lhs_spec, d->lhs_scale_in, d->lhs_is_quantized, d->lhs_q,
                      d->lhs_scale, &L);
  side_after_quantize(d->rhs, d->rhs_spec, d->rhs_scale_in, d->rhs_is_quantized, d->rhs_q,
                      d->rhs_scale, &R);
  aqtb200_gemm_desc g{};
  fill_gemm_desc(d, L, R, &g);
  return dequant_acc(&g, d->acc_out, (cudaStream_t)stream);
}

int aqtb200_dot_general_raw_exchange(const aqtb200_dg_raw_desc* d, const aqtb200_exchange_desc* x,
                                     int32_t* status, void* stream) {
  AQT_REQUIRE(d != nullptr && x != nullptr, AQTB200_EINVAL, "null descriptor");
  Side L{}, R{};
  side_after_quantize(d->lhs, d->lhs_spec, d->lhs_scale_in, d->lhs_is_quantized, d->lhs_q,
                      d->lhs_scale, &L);
  side_after_quantize(d->rhs, d->rhs_spec, d->rhs_scale_in, d->rhs_is_quantized, d->rhs_q,
                      d->rhs_scale, &R);
  aqtb200_gemm_desc g{};
  fill_gemm_desc(d, L, R, &g);
  g.out = x->out[x->rank >= 0 && x->rank < AQTB200_MAX_RANKS ? x->rank : 0];
  return exchange_dequant(&g, x, status, (cudaStream_t)stream);
}

}  // extern "C"
