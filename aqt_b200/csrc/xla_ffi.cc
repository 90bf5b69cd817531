// XLA FFI handlers over the C ABI: what lets jax (and so the reference's own
// Python, aqt/jax/v2/aqt_dot_general.py) call the sm_100a path as custom calls.
//
// This translation unit is compiled only where jaxlib's FFI header is on the
// include path (pass -I"$(python -c 'import jax.ffi; print(jax.ffi.include_dir())')");
// everywhere else -- including the image this library is developed on, which
// has no jax -- it is empty, and aqtb200_has_xla_ffi() says so.
//
// One handler per pass-level entry point. Conventions of XLA FFI that the C ABI
// was written to: the handler runs on XLA's host thread and only ENQUEUES on the
// stream it is given; buffers are owned by XLA; scratch arrives as an extra
// result buffer sized by the Python side with aqtb200_*_workspace_bytes; errors
// are returned, never thrown.
#include "../../include/aqt_b200.h"

#if defined(__has_include)
#if __has_include("xla/ffi/api/ffi.h")
#define AQTB200_WITH_XLA_FFI 1
#endif
#endif

#ifdef AQTB200_WITH_XLA_FFI
#include <cuda_runtime.h>

#include "xla/ffi/api/ffi.h"

namespace ffi = xla::ffi;

namespace {

int dtype_code(ffi::DataType dt) {
  switch (dt) {
    case ffi::DataType::F32: return AQTB200_F32;
    case ffi::DataType::BF16: return AQTB200_BF16;
    case ffi::DataType::S8: return AQTB200_S8;
    case ffi::DataType::F8E4M3FN: return AQTB200_E4M3;
    case ffi::DataType::F8E5M2: return AQTB200_E5M2;
    case ffi::DataType::S32: return AQTB200_S32;
    default: return -1;
  }
}

// A rank-4 row-major buffer [b0, b1, rows, cols] as a view; `transposed` reads
// it as [b0, b1, cols, rows] (the kept index contiguous).
aqtb200_view view_of(const ffi::AnyBuffer& b, bool transposed) {
  aqtb200_view v{};
  auto d = b.dimensions();
  v.ptr = b.untyped_data();
  v.dtype = dtype_code(b.element_type());
  v.b0 = d[0]; v.b1 = d[1];
  v.rows = transposed ? d[3] : d[2];
  v.cols = transposed ? d[2] : d[3];
  v.b1_stride = d[2] * d[3];
  v.b0_stride = d[1] * v.b1_stride;
  v.row_stride = transposed ? 1 : d[3];
  v.col_stride = transposed ? d[3] : 1;
  return v;
}

aqtb200_quant_spec spec_of(int64_t kind, int64_t qdtype, float quant_bound, float clip_bound,
                           bool per_tensor, int64_t compute_dtype, int64_t scale_dtype, bool po2,
                           float clipping_scale) {
  aqtb200_quant_spec s{};
  s.kind = (int32_t)kind; s.qdtype = (int32_t)qdtype;
  s.quant_bound = quant_bound; s.clip_bound = clip_bound;
  s.per_tensor = per_tensor ? 1 : 0;
  s.compute_dtype = (int32_t)compute_dtype; s.scale_dtype = (int32_t)scale_dtype;
  s.po2_scale = po2 ? 1 : 0; s.clipping_scale = clipping_scale;
  return s;
}

// DotGeneralRaw.__call__ (aqt_dot_general.py:757-840) for operands the Python
// side has already brought to [b0, b1, rows, K] (or [b0, b1, K, rows] with
// *_transposed). Results: out, q_lhs, s_lhs, q_rhs, s_rhs (the residuals of
// dg_core_vjp_fwd, :1121-1124), workspace, status.
ffi::Error DgRawImpl(cudaStream_t stream, ffi::AnyBuffer lhs, ffi::AnyBuffer rhs,
                     ffi::Result<ffi::AnyBuffer> out, ffi::Result<ffi::AnyBuffer> lhs_q,
                     ffi::Result<ffi::AnyBuffer> lhs_scale, ffi::Result<ffi::AnyBuffer> rhs_q,
                     ffi::Result<ffi::AnyBuffer> rhs_scale, ffi::Result<ffi::AnyBuffer> workspace,
                     ffi::Result<ffi::AnyBuffer> status, bool lhs_transposed, bool rhs_transposed,
                     int64_t kind, int64_t lhs_qdtype, int64_t rhs_qdtype, float lhs_quant_bound,
                     float lhs_clip_bound, float rhs_quant_bound, float rhs_clip_bound,
                     bool lhs_per_tensor, bool rhs_per_tensor, int64_t scale_dtype, bool po2,
                     bool swap_ab, bool out_transposed) {
  if (lhs.dimensions().size() != 4 || rhs.dimensions().size() != 4)
    return ffi::Error::InvalidArgument("aqtb200_dg_raw: operands must be rank 4 [b0, b1, rows, K]");
  aqtb200_dg_raw_desc d{};
  d.lhs = view_of(lhs, lhs_transposed);
  d.rhs = view_of(rhs, rhs_transposed);
  const int64_t t_code = d.lhs.dtype;
  d.lhs_spec = spec_of(kind, lhs_qdtype, lhs_quant_bound, lhs_clip_bound, lhs_per_tensor, t_code,
                       scale_dtype, po2, 0.f);
  d.rhs_spec = spec_of(kind, rhs_qdtype, rhs_quant_bound, rhs_clip_bound, rhs_per_tensor,
                       d.rhs.dtype, scale_dtype, po2, 0.f);
  d.lhs_q = lhs_q->untyped_data(); d.lhs_scale = lhs_scale->untyped_data();
  d.rhs_q = rhs_q->untyped_data(); d.rhs_scale = rhs_scale->untyped_data();
  d.swap_ab = swap_ab ? 1 : 0;
  d.dequant_dtype = (int32_t)t_code;
  d.out = out->untyped_data();
  d.out_dtype = dtype_code(out->element_type());
  const int64_t m = d.lhs.rows, n = d.rhs.rows;
  d.out_b1_stride = m * n; d.out_b0_stride = d.lhs.b1 * m * n;
  d.out_m_stride = out_transposed ? 1 : n;   // out_transposed: result stored [b0, b1, n, m]
  d.out_n_stride = out_transposed ? m : 1;
  d.scope_name = "aqt_dg_raw";
  const int rc = aqtb200_dot_general_raw(&d, workspace->untyped_data(), workspace->size_bytes(),
                                         static_cast<int32_t*>(status->untyped_data()), stream);
  if (rc == 0) return ffi::Error::Success();
  if (rc == AQTB200_EUNSUPPORTED) return ffi::Error(ffi::ErrorCode::kUnimplemented, aqtb200_last_error());
  return ffi::Error::Internal(aqtb200_last_error());
}

}  // namespace

XLA_FFI_DEFINE_HANDLER_SYMBOL(
    AqtB200DgRaw, DgRawImpl,
    ffi::Ffi::Bind()
        .Ctx<ffi::PlatformStream<cudaStream_t>>()
        .Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>()
        .Ret<ffi::AnyBuffer>().Ret<ffi::AnyBuffer>().Ret<ffi::AnyBuffer>()
        .Ret<ffi::AnyBuffer>().Ret<ffi::AnyBuffer>().Ret<ffi::AnyBuffer>().Ret<ffi::AnyBuffer>()
        .Attr<bool>("lhs_transposed").Attr<bool>("rhs_transposed")
        .Attr<int64_t>("kind").Attr<int64_t>("lhs_qdtype").Attr<int64_t>("rhs_qdtype")
        .Attr<float>("lhs_quant_bound").Attr<float>("lhs_clip_bound")
        .Attr<float>("rhs_quant_bound").Attr<float>("rhs_clip_bound")
        .Attr<bool>("lhs_per_tensor").Attr<bool>("rhs_per_tensor")
        .Attr<int64_t>("scale_dtype").Attr<bool>("po2")
        .Attr<bool>("swap_ab").Attr<bool>("out_transposed"));

extern "C" int aqtb200_has_xla_ffi(void) { return 1; }
#else
extern "C" int aqtb200_has_xla_ffi(void) { return 0; }
#endif
