"""ctypes binding of libaqt_b200.so (declarations: include/aqt_b200.h).

There is no fallback: if the shared library is missing or a call fails, the
caller gets an exception.
"""

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, 'libaqt_b200.so')

F32, BF16, S8, E4M3, E5M2, S32 = 0, 1, 2, 3, 4, 5
NUM_NONE, NUM_INT, NUM_FP8 = 0, 1, 2


class View(C.Structure):
  _fields_ = [
      ('ptr', C.c_void_p), ('dtype', C.c_int32), ('reserved', C.c_int32),
      ('b0', C.c_int64), ('b1', C.c_int64), ('rows', C.c_int64),
      ('cols', C.c_int64), ('b0_stride', C.c_int64), ('b1_stride', C.c_int64),
      ('row_stride', C.c_int64), ('col_stride', C.c_int64),
  ]


class QuantSpec(C.Structure):
  _fields_ = [
      ('kind', C.c_int32), ('qdtype', C.c_int32), ('quant_bound', C.c_float),
      ('clip_bound', C.c_float), ('per_tensor', C.c_int32),
      ('compute_dtype', C.c_int32), ('scale_dtype', C.c_int32),
      ('po2_scale', C.c_int32), ('clipping_scale', C.c_float),
      ('reserved', C.c_int32),
  ]


class GemmDesc(C.Structure):
  _fields_ = [
      ('b0', C.c_int64), ('b1', C.c_int64), ('m', C.c_int64), ('n', C.c_int64),
      ('k', C.c_int64),
      ('a', C.c_void_p), ('a_b0_stride', C.c_int64), ('a_b1_stride', C.c_int64),
      ('lda', C.c_int64),
      ('b', C.c_void_p), ('b_b0_stride', C.c_int64), ('b_b1_stride', C.c_int64),
      ('ldb', C.c_int64),
      ('a_dtype', C.c_int32), ('b_dtype', C.c_int32),
      ('a_scale', C.c_void_p), ('a_scale_b0_stride', C.c_int64),
      ('a_scale_b1_stride', C.c_int64), ('a_scale_m_stride', C.c_int64),
      ('b_scale', C.c_void_p), ('b_scale_b0_stride', C.c_int64),
      ('b_scale_b1_stride', C.c_int64), ('b_scale_n_stride', C.c_int64),
      ('a_scale_dtype', C.c_int32), ('b_scale_dtype', C.c_int32),
      ('b_scale_first', C.c_int32), ('dequant_dtype', C.c_int32),
      ('out', C.c_void_p), ('out_dtype', C.c_int32), ('reserved', C.c_int32),
      ('out_b0_stride', C.c_int64), ('out_b1_stride', C.c_int64),
      ('out_m_stride', C.c_int64), ('out_n_stride', C.c_int64),
      ('acc_out', C.c_void_p), ('amax_out', C.c_void_p),
      ('workspace', C.c_void_p), ('workspace_bytes', C.c_size_t),
  ]


class DgRawDesc(C.Structure):
  _fields_ = [
      ('lhs', View), ('rhs', View),
      ('lhs_prescale', View), ('rhs_prescale', View),
      ('lhs_noise', View), ('rhs_noise', View),
      ('lhs_spec', QuantSpec), ('rhs_spec', QuantSpec),
      ('lhs_scale_in', C.c_void_p), ('rhs_scale_in', C.c_void_p),
      ('lhs_is_quantized', C.c_int32), ('rhs_is_quantized', C.c_int32),
      ('lhs_q', C.c_void_p), ('lhs_scale', C.c_void_p),
      ('rhs_q', C.c_void_p), ('rhs_scale', C.c_void_p),
      ('swap_ab', C.c_int32), ('dequant_dtype', C.c_int32),
      ('out', C.c_void_p), ('out_dtype', C.c_int32), ('reserved', C.c_int32),
      ('out_b0_stride', C.c_int64), ('out_b1_stride', C.c_int64),
      ('out_m_stride', C.c_int64), ('out_n_stride', C.c_int64),
      ('acc_out', C.c_void_p), ('amax_out', C.c_void_p),
      ('scope_name', C.c_char_p),
  ]


class DualDesc(C.Structure):
  _fields_ = [
      ('x', View), ('spec_t', QuantSpec), ('spec_s', QuantSpec),
      ('prescale_t', View), ('prescale_s', View),
      ('noise_t', View), ('noise_s', View),
      ('q_t', C.c_void_p), ('scale_t', C.c_void_p),
      ('q_s', C.c_void_p), ('scale_s', C.c_void_p),
  ]


# name -> (restype, argtypes); every symbol include/aqt_b200.h declares.
MAX_RANKS = 8


class ExchangeDesc(C.Structure):
  """aqtb200_exchange_desc."""
  _fields_ = [('world', C.c_int32), ('rank', C.c_int32),
              ('acc', C.c_void_p * MAX_RANKS), ('out', C.c_void_p * MAX_RANKS),
              ('max_sms', C.c_int32)]


SYMBOLS = {
    'aqtb200_quantize': (C.c_int, [
        C.POINTER(View), C.POINTER(View), C.POINTER(View),
        C.POINTER(QuantSpec), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
        C.c_size_t, C.c_void_p]),
    'aqtb200_quantize_static': (C.c_int, [
        C.POINTER(View), C.POINTER(View), C.POINTER(View),
        C.POINTER(QuantSpec), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    'aqtb200_quantize_workspace_bytes': (C.c_size_t, [
        C.POINTER(View), C.POINTER(QuantSpec)]),
    'aqtb200_absmax_scale': (C.c_int, [
        C.POINTER(View), C.POINTER(View), C.POINTER(QuantSpec), C.c_void_p,
        C.c_void_p, C.c_size_t, C.c_void_p]),
    'aqtb200_absmax_raw': (C.c_int, [
        C.POINTER(View), C.c_int32, C.c_void_p, C.c_void_p]),
    'aqtb200_scale_from_amax': (C.c_int, [
        C.c_void_p, C.c_int64, C.c_void_p, C.c_int32, C.POINTER(QuantSpec),
        C.c_void_p, C.c_void_p]),
    'aqtb200_quantize_pair': (C.c_int, [
        C.POINTER(View),
        C.POINTER(QuantSpec), C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p,
        C.POINTER(QuantSpec), C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p,
        C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p]),
    'aqtb200_quantize_dual_workspace_bytes': (C.c_size_t, [
        C.POINTER(DualDesc)]),
    'aqtb200_quantize_dual': (C.c_int, [
        C.POINTER(DualDesc), C.c_void_p, C.c_size_t, C.c_void_p]),
    'aqtb200_requant_amax': (C.c_int, [
        C.c_void_p, C.c_int64, C.c_void_p, C.c_int32, C.POINTER(QuantSpec),
        C.c_void_p, C.c_void_p, C.c_void_p]),
    'aqtb200_round_up': (C.c_int64, [C.c_int64, C.c_int64]),
    'aqtb200_gemm_dequant': (C.c_int, [
        C.POINTER(GemmDesc), C.c_void_p, C.c_void_p]),
    'aqtb200_gemm_workspace_bytes': (C.c_size_t, [C.POINTER(GemmDesc)]),
    'aqtb200_dot_general_raw_workspace_bytes': (C.c_size_t, [
        C.POINTER(DgRawDesc)]),
    'aqtb200_dot_general_raw': (C.c_int, [
        C.POINTER(DgRawDesc), C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p]),
    'aqtb200_dot_general_raw_dequant': (C.c_int, [
        C.POINTER(DgRawDesc), C.c_void_p]),
    'aqtb200_dot_general_raw_exchange': (C.c_int, [
        C.POINTER(DgRawDesc), C.POINTER(ExchangeDesc), C.c_void_p, C.c_void_p]),
    'aqtb200_dequantize': (C.c_int, [
        C.POINTER(View), C.POINTER(View), C.c_int32, C.c_void_p, C.c_void_p]),
    'aqtb200_set_device': (C.c_int, [C.c_int]),
    'aqtb200_dev_alloc': (C.c_int, [C.POINTER(C.c_void_p), C.c_size_t]),
    'aqtb200_dev_free': (C.c_int, [C.c_void_p]),
    'aqtb200_dev_memset': (C.c_int, [C.c_void_p, C.c_int, C.c_size_t,
                                     C.c_void_p]),
    'aqtb200_h2d': (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    'aqtb200_d2h': (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    'aqtb200_sync': (C.c_int, [C.c_void_p]),
    'aqtb200_ipc_export': (C.c_int, [C.c_void_p, C.c_void_p]),
    'aqtb200_ipc_open': (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p)]),
    'aqtb200_ipc_close': (C.c_int, [C.c_void_p]),
    'aqtb200_comm_unique_id': (C.c_int, [C.c_void_p]),
    'aqtb200_comm_init': (C.c_int, [C.c_int, C.c_int, C.c_void_p,
                                    C.POINTER(C.c_void_p)]),
    'aqtb200_comm_destroy': (C.c_int, [C.c_void_p]),
    'aqtb200_allreduce': (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64,
                                    C.c_int32, C.c_int32, C.c_void_p]),
    'aqtb200_reduce_scatter_sum': (C.c_int, [
        C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_void_p]),
    'aqtb200_all_gather': (C.c_int, [
        C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_void_p]),
    'aqtb200_version': (C.c_int, []),
    'aqtb200_has_xla_ffi': (C.c_int, []),
    'aqtb200_last_error': (C.c_char_p, []),
    'aqtb200_device_sm_count': (C.c_int, [C.POINTER(C.c_int)]),
    'aqtb200_kernel_launch_count': (C.c_int64, []),
    'aqtb200_set_gemm_impl': (C.c_int, [C.c_int]),
    'aqtb200_set_gemm_sm_budget': (C.c_int, [C.c_int]),
    'aqtb200_delayed_scaling_scale': (C.c_int, [
        C.c_void_p, C.c_int64, C.c_void_p, C.c_int32, C.POINTER(QuantSpec),
        C.c_void_p, C.c_void_p]),
    'aqtb200_delayed_scaling_push': (C.c_int, [
        C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p]),
    'aqtb200_prescale_amax': (C.c_int, [
        C.c_void_p, C.c_int64, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p,
        C.c_void_p]),
    'aqtb200_jax_noise': (C.c_int, [
        C.c_uint32, C.c_uint32, C.c_int64, C.c_int32, C.c_int32, C.c_float,
        C.c_void_p, C.c_void_p]),
    'aqtb200_mma_peak': (C.c_int, [C.c_int32, C.c_int64, C.c_void_p, C.c_void_p]),
}

_lib = None


class AqtB200Error(RuntimeError):
  pass


def load():
  """Loads the shared library (once) and types its entry points."""
  global _lib
  if _lib is None:
    if not os.path.exists(LIB_PATH):
      raise AqtB200Error(
          f'{LIB_PATH} is missing: build it with `python -m aqt_b200.build` '
          '(needs nvcc). There is no fallback path.')
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SYMBOLS.items():
      fn = getattr(lib, name)
      fn.restype = res
      fn.argtypes = args
    _lib = lib
  return _lib


def check(rc: int, what: str):
  if rc != 0:
    msg = load().aqtb200_last_error().decode(errors='replace')
    kind = {-1: 'EINVAL', -2: 'EUNSUPPORTED', -3: 'EWORKSPACE', -4: 'EDRIVER',
            -5: 'EDEVICE'}.get(rc, f'cudaError {rc}' if rc > 0 else str(rc))
    if rc == -2:
      raise NotImplementedError(f'{what}: {msg}')
    raise AqtB200Error(f'{what} failed ({kind}): {msg}')
