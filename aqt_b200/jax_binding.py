"""The jax side of the XLA FFI binding (csrc/xla_ffi.cc): the layer that lets
the reference's own Python call this library from inside jit.

Importable everywhere; usable only where jax is installed AND the shared
library was built with jaxlib's FFI header on the include path
(`aqtb200_has_xla_ffi() == 1`). Neither is the case on the machine this
library is developed on (no jax, no network), so this module has never run:
it is the written-down form of INTEGRATION.md section 3, kept next to the code
it binds. `available()` says why it cannot be used, instead of failing late.

What it provides once both conditions hold:

  register()          jax.ffi.register_ffi_target('aqtb200_dg_raw', ...)
  dg_raw(...)         one DotGeneralRaw.__call__ (aqt_dot_general.py:757-840)
                      as a jax.ffi.ffi_call: returns (out, q_lhs, s_lhs,
                      q_rhs, s_rhs), the residuals dg_core_vjp_fwd keeps
                      (:1121-1124)

Wiring inside the reference: DotGeneralRaw.__call__ builds its operands'
[b0, b1, rows, K] forms with lax.reshape / no-copy bitcasts, calls dg_raw, and
wraps the results in DotGeneralRes exactly as today; the custom_vjp of
aqt_dot_general.py:993-997 needs no change.
"""

from __future__ import annotations

import ctypes

from aqt_b200 import _lib

TARGET = 'aqtb200_dg_raw'


def available():
  """(True, '') or (False, reason)."""
  try:
    import jax  # pylint: disable=unused-import,import-outside-toplevel
  except ImportError as e:
    return False, f'jax is not installed ({e})'
  lib = ctypes.CDLL(_lib.LIB_PATH)
  if not hasattr(lib, 'aqtb200_has_xla_ffi') or not lib.aqtb200_has_xla_ffi():
    return False, ('libaqt_b200.so was built without xla/ffi/api/ffi.h on the '
                   'include path; rebuild with jax.ffi.include_dir()')
  return True, ''


def register():
  ok, why = available()
  if not ok:
    raise RuntimeError(f'aqt_b200 jax binding unavailable: {why}')
  import jax  # pylint: disable=import-outside-toplevel
  lib = ctypes.CDLL(_lib.LIB_PATH)
  jax.ffi.register_ffi_target(TARGET, jax.ffi.pycapsule(lib.AqtB200DgRaw),
                              platform='CUDA')


def _workspace_bytes(lhs_shape, rhs_shape, lhs_per_tensor, rhs_per_tensor):
  align = lambda v: (v + 255) // 256 * 256
  n_l = 1 if lhs_per_tensor else lhs_shape[0] * lhs_shape[1] * lhs_shape[2]
  n_r = 1 if rhs_per_tensor else rhs_shape[0] * rhs_shape[1] * rhs_shape[2]
  return 2 * align(4 * n_l) + 2 * align(4 * n_r) + (16 << 20)


def dg_raw(lhs, rhs, *, kind, lhs_qdtype, rhs_qdtype, lhs_quant_bound,
           lhs_clip_bound, rhs_quant_bound, rhs_clip_bound, lhs_per_tensor,
           rhs_per_tensor, scale_dtype, po2=False, lhs_transposed=False,
           rhs_transposed=False, swap_ab=False, out_transposed=False):
  """lhs, rhs: rank-4 jax arrays [b0, b1, rows, K] (or [b0, b1, K, rows] with
  *_transposed). Codes are those of include/aqt_b200.h."""
  import jax  # pylint: disable=import-outside-toplevel
  import jax.numpy as jnp  # pylint: disable=import-outside-toplevel
  b0, b1 = lhs.shape[0], lhs.shape[1]
  m = lhs.shape[3] if lhs_transposed else lhs.shape[2]
  k = lhs.shape[2] if lhs_transposed else lhs.shape[3]
  n = rhs.shape[3] if rhs_transposed else rhs.shape[2]
  ldk = (k + 15) // 16 * 16
  q_dt = {_lib.S8: jnp.int8, _lib.E4M3: jnp.float8_e4m3fn,
          _lib.E5M2: jnp.float8_e5m2}
  s_dt = jnp.float32 if scale_dtype == _lib.F32 else jnp.bfloat16
  out_shape = (b0, b1, n, m) if out_transposed else (b0, b1, m, n)
  results = (
      jax.ShapeDtypeStruct(out_shape, lhs.dtype),
      jax.ShapeDtypeStruct((b0, b1, m, ldk), q_dt[lhs_qdtype]),
      jax.ShapeDtypeStruct((1,) if lhs_per_tensor else (b0, b1, m), s_dt),
      jax.ShapeDtypeStruct((b0, b1, n, ldk), q_dt[rhs_qdtype]),
      jax.ShapeDtypeStruct((1,) if rhs_per_tensor else (b0, b1, n), s_dt),
      jax.ShapeDtypeStruct((_workspace_bytes((b0, b1, m), (b0, b1, n),
                                             lhs_per_tensor, rhs_per_tensor),),
                           jnp.uint8),
      jax.ShapeDtypeStruct((4,), jnp.int32),
  )
  out, q_l, s_l, q_r, s_r, _, _ = jax.ffi.ffi_call(TARGET, results)(
      lhs, rhs, lhs_transposed=lhs_transposed, rhs_transposed=rhs_transposed,
      kind=kind, lhs_qdtype=lhs_qdtype, rhs_qdtype=rhs_qdtype,
      lhs_quant_bound=float(lhs_quant_bound),
      lhs_clip_bound=float(lhs_clip_bound),
      rhs_quant_bound=float(rhs_quant_bound),
      rhs_clip_bound=float(rhs_clip_bound), lhs_per_tensor=lhs_per_tensor,
      rhs_per_tensor=rhs_per_tensor, scale_dtype=scale_dtype, po2=po2,
      swap_ab=swap_ab, out_transposed=out_transposed)
  return out, q_l[..., :k], s_l, q_r[..., :k], s_r
