"""CPU oracle: numpy restatement of aqt.jax.v2's quantized dot_general.

TEST INFRASTRUCTURE ONLY. Nothing in the product imports this module; it is
the checker that tests/, the smoke check and the benchmark's CPU-baseline leg
compare the CUDA path against. It restates, op by op, what the reference
computes, citing the reference file:line each function follows (paths are
relative to the reference's aqt/jax/v2/).

Semantics chosen: *eager* jax semantics -- every jnp/lax op produces a value
rounded to its result dtype (bf16 arithmetic = exact f32 op on the widened
inputs, then one rounding to bf16, which is what XLA:CPU and ml_dtypes both do),
true IEEE division, python scalars are weakly typed (adopt the array's dtype).
Under jit XLA may fuse differently; that variant cannot be observed here
because jax is not installed.

Pinning status: the fp8 casts, the int bound table, per-tensor scale and the
local-AQT known answers are pinned against the reference's own test vectors
(tests/test_oracle_pins.py). The contraction itself lives in XLA (jax/jaxlib,
version unpinned by the reference's pyproject.toml): int8->int32 is
mathematically unique; for fp8->f32 accumulation order and for jax.random noise
there is no reference vector -- "parity unpinned" at that boundary, and the
oracle uses exact (f64) accumulation rounded once to f32.

Configuration objects are duck-typed: the functions read the same attribute
names the reference's dataclasses have (DotGeneral.fwd/dlhs/drhs,
DotGeneralRaw.lhs/rhs/dg_quantizer/dg_accumulator_dtype/local_aqt,
Quantizer.numerics/calib_shared_axes/calibration/scale_dtype/context, ...), so
the package's own config builders can drive it.
"""

from __future__ import annotations

import dataclasses
import functools
from typing import Any, Sequence
import weakref

import ml_dtypes
import numpy as np

bfloat16 = np.dtype(ml_dtypes.bfloat16)
float8_e4m3fn = np.dtype(ml_dtypes.float8_e4m3fn)
float8_e5m2 = np.dtype(ml_dtypes.float8_e5m2)
float32 = np.dtype(np.float32)
int8 = np.dtype(np.int8)
int32 = np.dtype(np.int32)

_NP_OF = {
    'float32': float32, 'bfloat16': bfloat16, 'int8': int8, 'int4': int8,
    'float8_e4m3fn': float8_e4m3fn, 'float8_e5m2': float8_e5m2,
    'int32': int32, 'float16': np.dtype(np.float16),
}
_FP8_MAX = {float8_e4m3fn: 448.0, float8_e5m2: 57344.0}


def np_dtype(d) -> None | np.dtype:
  """Maps a dtype token / torch dtype / numpy dtype to a numpy dtype."""
  if d is None:
    return None
  if isinstance(d, np.dtype):
    return d
  name = getattr(d, 'name', None) or str(d)
  name = name.replace('torch.', '').split('.')[-1].replace("'>", '')
  if name in _NP_OF:
    return _NP_OF[name]
  return np.dtype(d)


def promote(a: np.dtype, b: np.dtype) -> np.dtype:
  """jnp.promote_types for the float types on the path."""
  if a == b:
    return a
  if float32 in (a, b):
    return float32
  if {a, b} == {bfloat16, np.dtype(np.float16)}:
    return float32
  raise TypeError(f'promote({a}, {b})')


def _f32(x):
  return np.asarray(x).astype(np.float32)


def _binop(op, a, b):
  """Eager jnp binary op: python scalars are weak, compute in f32, round once."""
  a_is_arr, b_is_arr = isinstance(a, np.ndarray), isinstance(b, np.ndarray)
  if a_is_arr and b_is_arr:
    out = promote(a.dtype, b.dtype)
  elif a_is_arr:
    out = a.dtype
    b = np.asarray(b, dtype=out)  # weak scalar adopts the array dtype
  else:
    out = b.dtype
    a = np.asarray(a, dtype=out)
  with np.errstate(divide='ignore', over='ignore', invalid='ignore'):
    return op(_f32(a), _f32(b)).astype(out)


mul = functools.partial(_binop, np.multiply)
div = functools.partial(_binop, np.divide)
add = functools.partial(_binop, np.add)


def reciprocal(x):
  """lax.reciprocal: 1/x in x's dtype."""
  with np.errstate(divide='ignore'):
    return (np.float32(1.0) / _f32(x)).astype(x.dtype)


def clip(x, lo, hi):
  """jnp.clip with weak python-float bounds (result keeps x's dtype)."""
  return np.clip(_f32(x), np.float32(np.asarray(lo, x.dtype)),
                 np.float32(np.asarray(hi, x.dtype))).astype(x.dtype)


# ---------------------------------------------------------------------------
# numerics


def int_edge_of_last_bucket(n) -> float:
  """numerics/int_numerics.py:51-56."""
  edge = 2.0 ** (n.bits - 1)
  return edge - 0.5 if n.preserve_zero else edge


def int_quant_bound(n) -> float:
  """numerics/int_numerics.py:58-65 (table at :41-49)."""
  edge = int_edge_of_last_bucket(n)
  return edge - 0.5 if n.preserve_max_val else edge


def int_fwd_clip_bound(n) -> float:
  """numerics/int_numerics.py:67-76."""
  edge = int_edge_of_last_bucket(n)
  return edge - 0.5 if n.round else edge


def is_no_numerics(n) -> bool:
  return type(n).__name__ == 'NoNumerics'


def is_fp8(n) -> bool:
  return type(n).__name__ == 'Fp8Numerics'


def is_int(n) -> bool:
  return type(n).__name__ == 'IntSymmetric'


def round_to_nearest_even_fp8(x: np.ndarray, dtype: np.dtype) -> np.ndarray:
  """numerics/fp8_numerics.py:136-145: a plain RNE cast to the fp8 type."""
  return _f32(x).astype(dtype)


def fp8_vjp_fwd(n, x: np.ndarray) -> np.ndarray:
  """numerics/fp8_numerics.py:88-123 without stochastic rounding.

  The clip bound is finfo(dtype).max held as a bf16 *array* (:79-80), so the
  clip runs in promote(x.dtype, bf16).
  """
  dt = np_dtype(n.dtype)
  assert not n.stochastic_rounding, 'fp8 mantissa SR needs jax.random.bits'
  bound = np.asarray(_FP8_MAX[dt], dtype=bfloat16)
  out = promote(x.dtype, bfloat16)
  y = np.clip(_f32(x), -_f32(bound), _f32(bound)).astype(out)
  return round_to_nearest_even_fp8(y, dt)


def int_vjp_fwd(n, x: np.ndarray, noise: None | np.ndarray) -> np.ndarray:
  """numerics/int_numerics.py:81-111: [+noise] -> clip -> round -> cast."""
  input_dtype = x.dtype
  assert n.bits <= 22
  if noise is not None:
    # (x + noise) in the promoted dtype, then back to the input dtype (:93).
    x = add(x, np.asarray(noise, np.float32)).astype(input_dtype)
  if n.clip:
    b = int_fwd_clip_bound(n)
    x = clip(x, -b, b)
  if n.round:
    if not n.preserve_zero:
      x = add(np.floor(_f32(x)).astype(input_dtype), 0.5)
    else:
      x = np.rint(_f32(x)).astype(input_dtype)  # half to even
  dt = np_dtype(n.dtype)
  return x.astype(dt if dt is not None else input_dtype)


def quant_bound_of(n, x_dtype: np.dtype):
  """get_quant_bound(): python float for ints, a bf16 array for fp8."""
  if is_fp8(n):
    return np.asarray(_FP8_MAX[np_dtype(n.dtype)], dtype=bfloat16)
  if is_int(n):
    return int_quant_bound(n)
  return n.get_quant_bound()


# ---------------------------------------------------------------------------
# calibration and quantizer


def ceil_to_po2(scale: np.ndarray) -> np.ndarray:
  """calibration.py:25-30: 1 / 2**floor(log2(1/scale)), in scale's dtype.

  floor(log2(r)) is taken exactly from r's binary exponent; the reference's
  log2 goes through XLA's log, which may differ by one at exact powers of two.
  """
  r = _f32(reciprocal(scale))
  _, e = np.frexp(r)  # r = m * 2**e with m in [0.5, 1)
  p = np.ldexp(np.float32(1.0), e - 1).astype(scale.dtype)
  return reciprocal(p)


def absmax_scale(x: np.ndarray, shared_axes: Sequence[int], numerics_,
                 scale_dtype=None, clipping_scale=None,
                 po2_scale=False) -> np.ndarray:
  """AbsMaxCalibration.get_scale_and_bias_and_sparsity, calibration.py:117-157."""
  dtype = np_dtype(scale_dtype) or x.dtype
  amax = np.max(np.abs(x), axis=tuple(shared_axes), keepdims=True)
  amax = np.where(amax == 0, np.ones_like(amax), amax)
  bound = mul(amax, clipping_scale) if clipping_scale else amax
  scale = div(bound, quant_bound_of(numerics_, x.dtype))
  if po2_scale:
    scale = ceil_to_po2(scale)
  return scale.astype(dtype)


@dataclasses.dataclass
class OQTensor:
  """aqt_tensor.py:54-98 reduced to the fields the path uses."""

  qvalue: Any
  scale: list
  dequant_dtype: Any = None
  bias: list = dataclasses.field(default_factory=list)

  def is_full(self):
    return self.qvalue is not None

  def quant(self, x: np.ndarray) -> np.ndarray:
    """aqt_tensor.py:125-159: multiply by the rounded reciprocal of each scale."""
    q = x
    for s in self.scale:
      s_inv = reciprocal(s)
      s_inv = np.where(np.isinf(_f32(s_inv)), np.ones_like(s_inv), s_inv)
      q = mul(q, s_inv)
    return q

  def dequant(self) -> np.ndarray:
    """aqt_tensor.py:161-200: astype(dequant_dtype), multiply scales, cast."""
    dd = np_dtype(self.dequant_dtype)
    q = np.asarray(self.qvalue)
    if q.dtype == int32 and dd == bfloat16:
      # XLA:CPU converts s32 -> bf16 through f32 (two roundings); ml_dtypes
      # does the same. Written out so the GPU epilogue can match it.
      ret = q.astype(np.float32).astype(dd)
    else:
      ret = q.astype(dd)
    for s in self.scale:
      ret = mul(ret, s)
    return ret.astype(dd)


def _to_numpy(a):
  if a is None or isinstance(a, np.ndarray):
    return a
  if hasattr(a, 'detach'):  # a torch tensor handed over by a shared noise_fn
    import torch
    a = a.detach().cpu()
    if a.dtype == torch.bfloat16:
      return a.view(torch.int16).numpy().view(bfloat16)
    return a.numpy()
  return np.asarray(a)


def _calibration_kwargs(quantizer):
  """Unwraps quantizer.calibration (a class or functools.partial of one)."""
  cal = quantizer.calibration
  kw = {}
  if isinstance(cal, functools.partial):
    kw = dict(cal.keywords)
    cal = cal.func
  assert cal.__name__ in ('AbsMaxCalibration', 'DelayedScalingCalibration'), (
      f'oracle restates AbsMax and delayed-scaling calibration, got {cal}')
  return kw


# Delayed scaling, flax/delayed_scaling_calibration.py:28-124. The oracle keeps
# its OWN copy of every calibrator's state (amax_history f32[L], bound f32[1]),
# keyed by the calibrator's state holder, so that it can be driven with the
# same configuration object as the device path without sharing anything.
_DELAYED_STATE = weakref.WeakKeyDictionary()


def delayed_state(calibrator):
  key = calibrator.stats
  if key not in _DELAYED_STATE:
    _DELAYED_STATE[key] = [
        np.zeros(calibrator.amax_history_length, np.float32),
        np.zeros(1, np.float32)]
  return _DELAYED_STATE[key]


def delayed_scaling_scale(calibrator, x: np.ndarray, numerics_, context,
                          scale_dtype=None) -> np.ndarray:
  """get_bound + get_scale_and_bias_and_sparsity (:57-105), one call."""
  state = delayed_state(calibrator)
  history, prev_bound = state
  quant_mode = context.quant_mode.name if context is not None and getattr(
      context, 'quant_mode', None) is not None else 'SERVE'
  amax = np.max(history, axis=0)  # :82
  # compute_bound (:107-111)
  new_bound = np.where(amax > 0.0, amax, prev_bound)
  new_bound = np.where(np.isfinite(amax), new_bound, prev_bound).astype(
      np.float32)
  # compute_history (:113-118)
  update = np.max(np.abs(_f32(x))).astype(np.float32) if x.size else (
      np.float32(0))
  new_history = np.roll(history, -1)
  new_history[0] = update
  if quant_mode in ('TRAIN', 'CALIBRATE'):  # :93-95
    state[0], state[1] = new_history, new_bound.reshape(1)
  dtype = np_dtype(scale_dtype) or x.dtype
  bound = new_bound.reshape((1,) * x.ndim)
  scale = div(bound, quant_bound_of(numerics_, x.dtype))  # f32 (:103)
  if calibrator.po2_scale:
    scale = ceil_to_po2(scale)
  return scale.astype(dtype)


def quantizer_calibrate(quantizer, x: np.ndarray, calibration_axes) -> OQTensor:
  """Quantizer.calibrate, aqt_quantizer.py:79-157."""
  if is_no_numerics(quantizer.numerics):
    return OQTensor(qvalue=x, scale=[], dequant_dtype=x.dtype)
  if quantizer.calib_shared_axes == 'per_tensor':
    shared = list(range(x.ndim))
  else:
    shared = quantizer.calib_shared_axes or calibration_axes
  assert shared is not None
  kw = _calibration_kwargs(quantizer)
  cal = getattr(quantizer, '_calibrator', None)
  if type(cal).__name__ == 'DelayedScalingCalibration':
    scale = delayed_scaling_scale(cal, x, quantizer.numerics,
                                  quantizer.context,
                                  kw.get('dtype', quantizer.scale_dtype))
    return OQTensor(qvalue=None, scale=[scale], dequant_dtype=x.dtype)
  scale = absmax_scale(
      x, shared, quantizer.numerics,
      scale_dtype=kw.get('dtype', quantizer.scale_dtype),
      clipping_scale=kw.get('clipping_scale'),
      po2_scale=kw.get('po2_scale', False))
  return OQTensor(qvalue=None, scale=[scale], dequant_dtype=x.dtype)


def quantizer_calculate_qvalue(quantizer, x: np.ndarray,
                               qt: OQTensor) -> OQTensor:
  """Quantizer.calculate_qvalue, aqt_quantizer.py:159-176."""
  n = quantizer.numerics
  if is_no_numerics(n):
    return qt
  y = qt.quant(x)
  if is_fp8(n):
    q = fp8_vjp_fwd(n, y)
  else:
    noise = None
    if n.noise_fn:
      assert quantizer.context.key is not None
      noise = _to_numpy(n.noise_fn(tuple(y.shape), quantizer.context.key))
      noise = np.broadcast_to(noise, y.shape)
    q = int_vjp_fwd(n, y, noise)
  return OQTensor(qvalue=q, scale=qt.scale, dequant_dtype=qt.dequant_dtype)


# ---------------------------------------------------------------------------
# scale re-layout (transpose.py)


def remaining_axes(rank, ca, ba):
  """utils.py:138-148."""
  return [i for i in range(rank) if i not in list(ca) + list(ba)]


def _scale_trans(x, ca, ba):
  """transpose.py:98-111."""
  ca, ba = list(ca), list(ba)
  ra = remaining_axes(x.ndim, ca, ba)
  x = np.transpose(x, ba + ra + ca)
  return x.reshape(x.shape[:len(ba) + len(ra)])


def lhs_scale_to_output(s, dims, lhs_shape, rhs_shape):
  """transpose.py:114-132."""
  (lca, rca), (lba, rba) = dims
  t = _scale_trans(s, lca, lba)
  extra = len(rhs_shape) - len(rca) - len(rba)
  return t.reshape(t.shape + (1,) * extra)


def rhs_scale_to_output(s, dims, lhs_shape, rhs_shape):
  """transpose.py:135-148."""
  (lca, rca), (lba, rba) = dims
  t = _scale_trans(s, rca, rba)
  extra = len(lhs_shape) - len(lca) - len(lba)
  nb = len(rba)
  return t.reshape(t.shape[:nb] + (1,) * extra + t.shape[nb:])


def scale_for_other_input(x, my_ca, my_ba, other_ca, other_ba, other_rank):
  """transpose.py:218-263."""
  my_ca, my_ba = list(my_ca), list(my_ba)
  other_ca, other_ba = list(other_ca), list(other_ba)
  if x.ndim < other_rank:
    x = x.reshape(x.shape + (1,) * (other_rank - x.ndim))
  perm = [-1] * x.ndim
  my_ra = remaining_axes(x.ndim, my_ca, my_ba)
  for mine, theirs in zip(my_ca + my_ba, other_ca + other_ba):
    perm[theirs] = mine
  it = iter(my_ra)
  perm = [next(it) if p == -1 else p for p in perm]
  x = np.transpose(x, perm)
  if x.ndim > other_rank:
    x = x.reshape(x.shape[:other_rank])
  return x


# ---------------------------------------------------------------------------
# the contraction


def _group(x, ba, ra, ca):
  """[...]-> [B, R, C] with the given axis groups, plus the group shapes."""
  xt = np.transpose(x, list(ba) + list(ra) + list(ca))
  bs = [x.shape[i] for i in ba]
  rs = [x.shape[i] for i in ra]
  cs = [x.shape[i] for i in ca]
  p = lambda v: int(np.prod(v, dtype=np.int64))
  return xt.reshape(p(bs), p(rs), p(cs)), bs, rs


def _exact_int_matmul(a: np.ndarray, b: np.ndarray) -> np.ndarray:
  """[B,M,K] x [B,N,K] -> int64 [B,M,N], exactly.

  f32 BLAS on K-chunks of <= 1024: every partial sum of <= 1024 products of
  magnitudes <= 127*128 stays below 2**24, so each chunk is exact in f32.
  """
  B, M, K = a.shape
  N = b.shape[1]
  out = np.zeros((B, M, N), np.int64)
  if a.size * N <= 1 << 16:
    return np.einsum('bmk,bnk->bmn', a.astype(np.int64), b.astype(np.int64))
  for k0 in range(0, K, 1024):
    pa = a[:, :, k0:k0 + 1024].astype(np.float32)
    pb = b[:, :, k0:k0 + 1024].astype(np.float32)
    out += np.matmul(pa, np.swapaxes(pb, 1, 2)).astype(np.int64)
  return out


def dot_general(lhs: np.ndarray, rhs: np.ndarray, dims,
                preferred_element_type=None, fast_float=False) -> np.ndarray:
  """lax.dot_general as called at aqt_dot_general.py:921-927.

  int8 x int8 -> exact int32. fp8 x fp8 -> f32: every product is exact in f32;
  the sum is accumulated in f64 and rounded once (f32 BLAS when `fast_float`,
  for full-size property checks). Other floats: f64 accumulate, rounded to the
  promoted input dtype.
  """
  (lca, rca), (lba, rba) = dims
  lra = remaining_axes(lhs.ndim, lca, lba)
  rra = remaining_axes(rhs.ndim, rca, rba)
  a, bs, ms = _group(lhs, lba, lra, lca)
  b, _, ns = _group(rhs, rba, rra, rca)
  pet = np_dtype(preferred_element_type)
  if lhs.dtype == int8 and rhs.dtype == int8:
    acc = _exact_int_matmul(a, b)
    assert np.abs(acc).max(initial=0) < 2**31
    out = acc.astype(pet or int32)
  else:
    wide = np.float32 if fast_float else np.float64
    acc = np.matmul(a.astype(wide), np.swapaxes(b.astype(wide), 1, 2))
    if pet is None:
      fl = [d for d in (lhs.dtype, rhs.dtype) if d.kind == 'f' or d in (
          bfloat16, float8_e4m3fn, float8_e5m2)]
      pet = functools.reduce(promote, fl) if fl else float32
    out = acc.astype(np.float32).astype(pet)
  return out.reshape(bs + ms + ns)


# ---------------------------------------------------------------------------
# DotGeneralRaw / DotGeneral


@dataclasses.dataclass
class OMultiTensor:
  x: np.ndarray
  qx: OQTensor


@dataclasses.dataclass
class ORes:
  lhs: OMultiTensor
  rhs: OMultiTensor


def _calibration_axes(mode, ndim, ca, ba):
  """aqt_dot_general.py:478-492."""
  if mode.name == 'REMAINING_AXIS':
    return remaining_axes(ndim, ca, ba)
  return list(ca)


def _apply_local_aqt(local_aqt, lhs, rhs, dims):
  """aqt_dot_general.py:262-328 (original factor_reshape only)."""
  assert not local_aqt.tile_largest_shape
  factor = local_aqt.contraction_axis_shard_count
  assert factor is not None and local_aqt.contraction_axis_shard_size is None

  def factor_reshape(x, ca, ba):
    ca, ba = list(ca), list(ba)
    if not ca:
      return x, ca, ba
    shape = list(x.shape)
    ax = ca[0]
    assert shape[ax] % factor == 0
    shape[ax:ax + 1] = [factor, shape[ax] // factor]
    new_ca = [c + int(c >= ax) for c in ca]
    new_ba = [ax] + [b + int(b > ax) for b in ba]
    return x.reshape(shape), new_ca, new_ba

  (lca, rca), (lba, rba) = dims
  lhs, lca, lba = factor_reshape(lhs, lca, lba)
  rhs, rca, rba = factor_reshape(rhs, rca, rba)
  return lhs, rhs, ((lca, rca), (lba, rba))


def maybe_use_fwd_quant(lhs: np.ndarray, rhs: OMultiTensor, dims,
                        use_fwd_quant: bool):
  """aqt_dot_general.py:675-729."""
  if not use_fwd_quant:
    return lhs, rhs.x
  assert len(rhs.qx.scale) == 1
  (lca, rca), (lba, rba) = dims
  scale_t = scale_for_other_input(rhs.qx.scale[0], rca, rba, lca, lba, lhs.ndim)
  lhs = mul(lhs, scale_t.astype(lhs.dtype))
  rhs_x = np.asarray(rhs.qx.qvalue).astype(np.float32).astype(
      np_dtype(rhs.qx.dequant_dtype))
  return lhs, rhs_x


def dg_raw(raw, lhs: np.ndarray, rhs, lhs_qt: None | OQTensor,
           rhs_qt: None | OQTensor, dims, fast_float=False,
           return_acc=False):
  """DotGeneralRaw.__call__, aqt_dot_general.py:757-840.

  Returns (out, ORes) or, with return_acc, (out, ORes, raw accumulator).
  """
  if isinstance(rhs, OMultiTensor):
    lhs, rhs = maybe_use_fwd_quant(lhs, rhs, dims, raw.rhs.use_fwd_quant)
  if raw.local_aqt is not None:
    lhs, rhs, dims = _apply_local_aqt(raw.local_aqt, lhs, rhs, dims)
  (lca, rca), (lba, rba) = dims
  q = raw.dg_quantizer
  assert q.lhs_mid_alpha is None and q.rhs_mid_alpha is None

  # quant(): aqt_dot_general.py:598-672
  lhs_inc = quantizer_calibrate(
      q.lhs, lhs, _calibration_axes(raw.lhs.calibration_mode, lhs.ndim, lca,
                                    lba))
  rhs_inc = quantizer_calibrate(
      q.rhs, rhs, _calibration_axes(raw.rhs.calibration_mode, rhs.ndim, rca,
                                    rba))
  if lhs_qt is not None and not lhs_qt.is_full():
    lhs_inc, lhs_qt = lhs_qt, None
  if rhs_qt is not None and not rhs_qt.is_full():
    rhs_inc, rhs_qt = rhs_qt, None
  lhs_calc = quantizer_calculate_qvalue(q.lhs, lhs, lhs_inc)
  rhs_calc = quantizer_calculate_qvalue(q.rhs, rhs, rhs_inc)
  lhs_q = lhs_qt if lhs_qt is not None else lhs_calc
  rhs_q = rhs_qt if rhs_qt is not None else rhs_calc

  # _qtensor_dot_general(): aqt_dot_general.py:843-958
  def maybe_dequant(qt, tcfg):
    if tcfg.dequant_mode.name == 'THIS_INPUT':
      return qt.dequant()
    return np.asarray(qt.qvalue)

  lhs_in = maybe_dequant(lhs_q, raw.lhs)
  rhs_in = maybe_dequant(rhs_q, raw.rhs)
  if raw.lhs.dequant_mode.name == 'OTHER_INPUT':
    for s in lhs_q.scale:
      st = scale_for_other_input(s, lca, lba, rca, rba, rhs_in.ndim)
      rhs_in = mul(rhs_in, st.astype(rhs_in.dtype))
  if raw.rhs.dequant_mode.name == 'OTHER_INPUT':
    for s in rhs_q.scale:
      st = scale_for_other_input(s, rca, rba, lca, lba, lhs_in.ndim)
      lhs_in = mul(lhs_in, st.astype(lhs_in.dtype))
  acc = dot_general(lhs_in, rhs_in, dims,
                    preferred_element_type=raw.dg_accumulator_dtype,
                    fast_float=fast_float)
  out_scales = []
  if raw.lhs.dequant_mode.name == 'OUTPUT':
    out_scales += [lhs_scale_to_output(s, dims, lhs_in.shape, rhs_in.shape)
                   for s in lhs_q.scale]
  if raw.rhs.dequant_mode.name == 'OUTPUT':
    out_scales += [rhs_scale_to_output(s, dims, lhs_in.shape, rhs_in.shape)
                   for s in rhs_q.scale]
  out = OQTensor(qvalue=acc, scale=out_scales,
                 dequant_dtype=promote(lhs.dtype, rhs.dtype)).dequant()
  res = ORes(lhs=OMultiTensor(x=lhs, qx=lhs_q),
             rhs=OMultiTensor(x=rhs, qx=rhs_q))
  if raw.local_aqt is not None:
    if len(lca) > 0:
      out = np.sum(_f32(out), axis=0).astype(out.dtype)
    res = None
  if return_acc:
    return out, res, acc
  return out, res


def dg_fwd(cfg, lhs: np.ndarray, rhs: np.ndarray, dims, lhs_qt=None,
           rhs_qt=None, fast_float=False):
  """dg_core_vjp_fwd, aqt_dot_general.py:1098-1124: (out, residuals)."""
  assert lhs.dtype == rhs.dtype
  out, res = dg_raw(cfg.fwd, lhs, rhs, lhs_qt, rhs_qt, dims,
                    fast_float=fast_float)
  return out.astype(lhs.dtype), res


def bwd_dimension_numbers(fwd_dims, y_is_lhs: bool, gradient_rank: int,
                          y_rank: int):
  """_update_dimension_numbers_for_backward, aqt_dot_general.py:1127-1175."""
  def ranges_like(*xs):
    start = 0
    for x in xs:
      yield tuple(range(start, start + len(x)))
      start += len(x)

  (x_ca, y_ca), (x_ba, y_ba) = fwd_dims
  if y_is_lhs:
    x_ca, y_ca = y_ca, x_ca
    x_ba, y_ba = y_ba, x_ba
  x_rank = gradient_rank - y_rank + len(x_ba) + 2 * len(x_ca)
  x_ra = tuple(remaining_axes(x_rank, x_ca, x_ba))
  y_ra = tuple(remaining_axes(y_rank, y_ca, y_ba))
  if y_is_lhs:
    g_ba, g_ca, _ = ranges_like(x_ba, y_ra, x_ra)
  else:
    g_ba, _, g_ca = ranges_like(x_ba, x_ra, y_ra)
  dims = ((g_ca, y_ra), (g_ba, tuple(y_ba)))
  x_ca_sorted = tuple(np.take(x_ca, np.argsort(y_ca)).tolist())
  perm = tuple(np.argsort(tuple(x_ba) + x_ra + x_ca_sorted).tolist())
  return dims, perm


def dg_bwd(cfg, fwd_dims, res: ORes, g: np.ndarray, fast_float=False):
  """dg_core_vjp_bwd, aqt_dot_general.py:1178-1221: (dlhs, drhs).

  quant_grad (the numerics' vjp_bwd) is the identity for AbsMax-calibrated
  numerics without clip_gradient and is not applied here.
  """
  def grad(y: OMultiTensor, raw, y_is_lhs):
    dims, perm = bwd_dimension_numbers(fwd_dims, y_is_lhs, g.ndim, y.x.ndim)
    out, _ = dg_raw(raw, g, y, None, None, dims, fast_float=fast_float)
    return np.transpose(out, perm)

  dlhs = grad(res.rhs, cfg.dlhs, False)
  drhs = grad(res.lhs, cfg.drhs, True)
  return dlhs, drhs


def dg_fwd_bwd(cfg, lhs, rhs, g, dims, fast_float=False):
  """Forward then backward; returns (out, dlhs, drhs, residuals)."""
  out, res = dg_fwd(cfg, lhs, rhs, dims, fast_float=fast_float)
  dlhs, drhs = dg_bwd(cfg, dims, res, g, fast_float=fast_float)
  return out, dlhs, drhs, res
