"""Quantized dot_general with its two gradient dot_generals.

Mirrors the public surface of the reference's aqt/jax/v2/aqt_dot_general.py:
CalibrationMode/DequantMode (:51-71), Tensor (:74-86), LocalAqt (:89-97),
dot_general_raw_make (:99-156), dot_general_make (:161-203), MultiTensor /
TensorRes / DotGeneralRes (:209-226), einsum (:229-241),
DefaultDotGeneralQuantizer (:426-595), DotGeneralRaw (:732-840), DotGeneral
(:961-1078), dg_core_vjp_fwd (:1098-1124),
_update_dimension_numbers_for_backward (:1127-1175), dg_core_vjp_bwd
(:1178-1221).

The configuration objects are plain Python. The arithmetic of one raw
quantized dot (calibrate -> quantize -> contraction -> dequantize) is executed
by `aqt_b200.engine.dg_raw`, which drives the sm_100a kernels through the C ABI
of libaqt_b200.so; configurations those kernels do not cover raise
NotImplementedError (there is no CPU or eager fallback).

Arrays are torch CUDA tensors (float32 or bfloat16); torch supplies device
memory, streams and autograd bookkeeping only.
"""

from __future__ import annotations

import abc
import enum
from typing import Any, Sequence

import numpy as onp

from aqt_b200.v2 import aqt_quantizer
from aqt_b200.v2 import aqt_tensor
from aqt_b200.v2 import transpose
from aqt_b200.v2 import utils
from aqt_b200.v2.numerics import fp8_numerics

dtypes_allowed_for_int32_accum = [utils.int4, utils.int8]


class CalibrationMode(enum.Enum):
  CONTRACTING_AXIS = 1
  REMAINING_AXIS = 2


class DequantMode(enum.Enum):
  # Multiply the output of the dot by the transposed scale.
  OUTPUT = 1
  # Multiply qvalue by its own scale before the dot ("fake quant").
  THIS_INPUT = 2
  # Multiply the other operand by the transposed scale.
  OTHER_INPUT = 3


@utils.flax_slots_kw_only_dataclass
class Tensor:
  """Per-operand options of one raw dot."""

  use_fwd_quant: bool = utils.static_field(default=False)
  dequant_mode: DequantMode = utils.static_field(default=DequantMode.OUTPUT)
  calibration_mode: CalibrationMode = utils.static_field(
      default=CalibrationMode.CONTRACTING_AXIS)


@utils.flax_slots_kw_only_dataclass
class LocalAqt:
  contraction_axis_shard_count: None | int = utils.static_field(default=None)
  contraction_axis_shard_size: None | int = utils.static_field(default=None)
  tile_largest_shape: bool = utils.static_field(default=False)


def _is_int_bits(b):
  return isinstance(b, int) and not isinstance(b, bool) and 2 <= b <= 8


def dot_general_raw_make(lhs_bits=None, rhs_bits=None, local_aqt=None,
                         jax_scope_name='aqt', initialize_calibration=True,
                         allow_dummy_gradients=False) -> 'DotGeneralRaw':
  """One raw quantized dot; accumulator int32 for 2..8-bit ints, f32 for fp8."""
  if _is_int_bits(lhs_bits) and _is_int_bits(rhs_bits):
    acc = utils.int32
  elif lhs_bits in fp8_numerics.fp8_map and rhs_bits in fp8_numerics.fp8_map:
    acc = utils.float32
  else:
    acc = None
  mk = lambda bits: aqt_quantizer.quantizer_make(
      bits, initialize_calibration=initialize_calibration)
  return DotGeneralRaw(
      lhs=Tensor(),
      rhs=Tensor(),
      dg_quantizer=DefaultDotGeneralQuantizer(
          lhs=mk(lhs_bits), rhs=mk(rhs_bits), lhs_mid=mk(None),
          rhs_mid=mk(None)),
      dg_accumulator_dtype=acc,
      local_aqt=local_aqt,
      jax_scope_name=jax_scope_name,
      allow_dummy_gradient_into_qtensor=allow_dummy_gradients,
  )


def dot_general_make(lhs_bits=None, rhs_bits=None, bwd_bits=None,
                     use_fwd_quant: bool = True, dlhs_local_aqt=None,
                     drhs_local_aqt=None,
                     allow_dummy_gradients: bool = False) -> 'DotGeneral':
  """fwd with (lhs_bits, rhs_bits); both gradient dots with bwd_bits."""
  common = dict(initialize_calibration=False,
                allow_dummy_gradients=allow_dummy_gradients)
  cfg = DotGeneral(
      fwd=dot_general_raw_make(lhs_bits, rhs_bits, jax_scope_name='aqt_fwd',
                               **common),
      dlhs=dot_general_raw_make(bwd_bits, bwd_bits, local_aqt=dlhs_local_aqt,
                                jax_scope_name='aqt_dlhs', **common),
      drhs=dot_general_raw_make(bwd_bits, bwd_bits, local_aqt=drhs_local_aqt,
                                jax_scope_name='aqt_drhs', **common),
  )
  # The forward quantization of lhs is what drhs may reuse, and vice versa.
  if lhs_bits is not None:
    cfg.drhs.rhs.use_fwd_quant = use_fwd_quant
  if rhs_bits is not None:
    cfg.dlhs.rhs.use_fwd_quant = use_fwd_quant
  assert cfg.fwd.local_aqt is None, 'local_aqt is not yet supported in fwd.'
  return cfg


@utils.flax_slots_kw_only_dataclass
class MultiTensor:
  x: Any
  qx: aqt_tensor.QTensor


@utils.flax_slots_kw_only_dataclass
class TensorRes:
  """What the forward pass hands to the backward pass for one operand."""

  mt: MultiTensor
  quant_grad: Any


@utils.flax_slots_kw_only_dataclass
class DotGeneralRes:
  lhs: TensorRes
  rhs: TensorRes


def lax_dot_general(lhs, rhs, dimension_numbers, precision=None,
                    preferred_element_type=None):
  """Unquantized dot_general on torch tensors (library GEMM, not the hot path)."""
  import torch
  del precision, preferred_element_type
  (lca, rca), (lba, rba) = dimension_numbers
  lra = utils.get_remaining_axes(lhs.ndim, lca, lba)
  rra = utils.get_remaining_axes(rhs.ndim, rca, rba)
  a = lhs.permute(*lba, *lra, *lca)
  b = rhs.permute(*rba, *rca, *rra)
  bs = [lhs.shape[i] for i in lba]
  ms = [lhs.shape[i] for i in lra]
  ns = [rhs.shape[i] for i in rra]
  k = int(onp.prod([lhs.shape[i] for i in lca], dtype=onp.int64))
  a = a.reshape(-1, int(onp.prod(ms, dtype=onp.int64)), k)
  b = b.reshape(-1, k, int(onp.prod(ns, dtype=onp.int64)))
  return torch.bmm(a, b).reshape(bs + ms + ns)


def einsum_to_dot_general(eqn: str, lhs_ndim: int, rhs_ndim: int):
  """Lowers a two-operand einsum to (dimension_numbers, output permutation).

  Returns (dims, perm, swap): compute dot_general(lhs, rhs, dims) (operands
  swapped first when `swap`), then transpose the result with `perm` (None when
  it is the identity). The operand order is kept whenever the natural
  dot_general output order (batch, lhs free, rhs free) already matches the
  requested output; otherwise the swapped order is tried before falling back
  to a transpose. Summed-out-alone and repeated indices are not supported.
  """
  eqn = eqn.replace(' ', '')
  assert '->' in eqn and '.' not in eqn, f'unsupported einsum {eqn!r}'
  ins, out = eqn.split('->')
  l, r = ins.split(',')
  assert len(l) == lhs_ndim and len(r) == rhs_ndim, (eqn, lhs_ndim, rhs_ndim)
  assert len(set(l)) == len(l) and len(set(r)) == len(r) and (
      len(set(out)) == len(out)), f'repeated index in {eqn!r}'

  def lower(a, b):
    batch = [c for c in a if c in b and c in out]
    contract = [c for c in a if c in b and c not in out]
    for c in a + b:
      assert (c in a and c in b) or c in out, (
          f'index {c!r} of {eqn!r} is summed over a single operand')
    dims = ((tuple(a.index(c) for c in contract),
             tuple(b.index(c) for c in contract)),
            (tuple(a.index(c) for c in batch),
             tuple(b.index(c) for c in batch)))
    natural = batch + [c for c in a if c not in batch and c not in contract] + [
        c for c in b if c not in batch and c not in contract]
    perm = tuple(natural.index(c) for c in out)
    return dims, perm

  dims, perm = lower(l, r)
  ident = tuple(range(len(out)))
  if perm == ident:
    return dims, None, False
  dims_s, perm_s = lower(r, l)
  if perm_s == ident:
    return dims_s, None, True
  return dims, perm, False


def einsum(eqn: str, lhs, rhs, dg=lax_dot_general):
  """Two-operand einsum through an injectable dot_general (reference :229-241)."""
  dims, perm, swap = einsum_to_dot_general(eqn, lhs.ndim, rhs.ndim)
  a, b = (rhs, lhs) if swap else (lhs, rhs)
  out = dg(a, b, dims, precision=None, preferred_element_type=None)
  return out if perm is None else out.permute(*perm)


def _get_scale_t(qt, transpose_fn, dimension_numbers, lhs_shape, rhs_shape):
  return [transpose_fn(s, dimension_numbers, lhs_shape, rhs_shape)
          for s in qt.scale]


@utils.flax_slots_kw_only_dataclass
class DotGeneralQuantizer(abc.ABC):
  """Quantizes the two operands of a dot_general (reference :331-422)."""

  def __call__(self, lhs, rhs, dimension_numbers, lhs_mode, rhs_mode):
    (lhs, lhs_qt), (rhs, rhs_qt) = self.calibrate(
        lhs, rhs, dimension_numbers, lhs_mode, rhs_mode)
    return self.calculate_qvalue(lhs, lhs_qt, rhs, rhs_qt)

  @abc.abstractmethod
  def init_calibration(self):
    pass

  @abc.abstractmethod
  def calibrate(self, lhs, rhs, dimension_numbers, lhs_mode, rhs_mode):
    pass

  @abc.abstractmethod
  def calculate_qvalue(self, lhs, lhs_qt, rhs, rhs_qt):
    pass

  @abc.abstractmethod
  def swap_lhs_and_rhs(self) -> None:
    pass

  @abc.abstractmethod
  def assert_calib_shared_axes_value(self, lhs_val, rhs_val, msg: str) -> None:
    pass

  @abc.abstractmethod
  def set_context(self, lhs_context, rhs_context) -> None:
    pass


def calibration_axes_for(mode: CalibrationMode, ndim: int, ca, ba):
  if mode == CalibrationMode.REMAINING_AXIS:
    return utils.get_remaining_axes(ndim, ca, ba)
  if mode == CalibrationMode.CONTRACTING_AXIS:
    return list(ca)
  raise ValueError(f'Unknown calibration mode: {mode}')


@utils.flax_slots_kw_only_dataclass
class DefaultDotGeneralQuantizer(DotGeneralQuantizer):
  """One Quantizer per operand (+ optional SmoothQuant-style mid scales)."""

  lhs: aqt_quantizer.Quantizer
  rhs: aqt_quantizer.Quantizer
  lhs_mid: aqt_quantizer.Quantizer
  rhs_mid: aqt_quantizer.Quantizer
  lhs_mid_alpha: None | float = None
  rhs_mid_alpha: None | float = None
  skip_mid_scales: bool = True

  def init_calibration(self):
    self.lhs.init_calibration()
    self.rhs.init_calibration()
    if self.lhs_mid_alpha is not None:
      self.lhs_mid.init_calibration()
    if self.rhs_mid_alpha is not None:
      self.rhs_mid.init_calibration()

  def calibrate(self, lhs, rhs, dimension_numbers, lhs_mode, rhs_mode):
    if self.lhs_mid_alpha is not None or self.rhs_mid_alpha is not None:
      raise NotImplementedError(
          'mid-scale (SmoothQuant-style) quantization is outside the sm_100a '
          'hot path')
    if dimension_numbers is not None:
      (lhs_ca, rhs_ca), (lhs_ba, rhs_ba) = dimension_numbers
      lhs_axes = calibration_axes_for(lhs_mode, lhs.ndim, lhs_ca, lhs_ba)
      rhs_axes = calibration_axes_for(rhs_mode, rhs.ndim, rhs_ca, rhs_ba)
    else:
      lhs_axes = rhs_axes = None
    lhs_qt = self.lhs.calibrate(lhs, calibration_axes=lhs_axes)
    rhs_qt = self.rhs.calibrate(rhs, calibration_axes=rhs_axes)
    return ((lhs, lhs_qt), (rhs, rhs_qt))

  def calculate_qvalue(self, lhs, lhs_qt, rhs, rhs_qt):
    return (self.lhs.calculate_qvalue(lhs, lhs_qt),
            self.rhs.calculate_qvalue(rhs, rhs_qt))

  def swap_lhs_and_rhs(self) -> None:
    self.lhs, self.rhs = self.rhs, self.lhs

  def assert_calib_shared_axes_value(self, lhs_val, rhs_val, msg: str) -> None:
    assert self.lhs.calib_shared_axes == lhs_val, msg
    assert self.rhs.calib_shared_axes == rhs_val, msg

  def set_context(self, lhs_context, rhs_context) -> None:
    self.lhs.context = lhs_context
    self.rhs.context = rhs_context


_POISON = ('Poison. Gradients are not generally expected in serving. '
           'Please set allow_dummy_gradient_into_qtensor to True '
           'if this is the intended behavior.')


def quant(lhs, rhs, lhs_qt, rhs_qt, dg_quantizer, lhs_cfg, rhs_cfg,
          dimension_numbers, allow_dummy_gradient_into_qtensor):
  """Operand quantization, honouring caller-supplied QTensors (reference :598-672).

  A full QTensor (serving) replaces the computed one and poisons the gradient;
  an incomplete one (scale only) replaces just the calibration.
  """
  (lhs, lhs_inc), (rhs, rhs_inc) = dg_quantizer.calibrate(
      lhs, rhs, dimension_numbers, lhs_cfg.calibration_mode,
      rhs_cfg.calibration_mode)
  if lhs_qt is not None and not lhs_qt.is_full():
    lhs_inc, lhs_qt = lhs_qt, None
  if rhs_qt is not None and not rhs_qt.is_full():
    rhs_inc, rhs_qt = rhs_qt, None
  (lhs_calc, lhs_grad), (rhs_calc, rhs_grad) = dg_quantizer.calculate_qvalue(
      lhs, lhs_inc, rhs, rhs_inc)

  def pick(given, calc, grad):
    if given is None:
      return calc, grad
    return given, (grad if allow_dummy_gradient_into_qtensor else _POISON)

  return pick(lhs_qt, lhs_calc, lhs_grad), pick(rhs_qt, rhs_calc, rhs_grad)


@utils.flax_slots_kw_only_dataclass
class DotGeneralRaw:
  """One quantized dot_general without gradient."""

  lhs: Tensor
  rhs: Tensor
  dg_quantizer: DotGeneralQuantizer
  dg_accumulator_dtype: Any = utils.static_field()
  local_aqt: None | LocalAqt = utils.static_field()
  jax_scope_name: str = utils.static_field()
  allow_dummy_gradient_into_qtensor: bool = utils.static_field(default=False)
  # Kept for API parity with the reference's injectable contraction. The
  # sm_100a path fuses the contraction with dequantization, so any value other
  # than the default is rejected by the engine.
  dot_general: utils.DotGeneralT = utils.static_field(default=lax_dot_general)

  @classmethod
  def make(cls, *args, **kwargs) -> 'DotGeneralRaw':
    return dot_general_raw_make(*args, **kwargs)

  def __call__(self, lhs, rhs, lhs_qt, rhs_qt, dimension_numbers):
    """(out, DotGeneralRes). `rhs` may be a MultiTensor in the backward pass."""
    from aqt_b200 import engine
    return engine.dg_raw(self, lhs, rhs, lhs_qt, rhs_qt, dimension_numbers)


@utils.flax_slots_kw_only_dataclass
class DotGeneral:
  """A quantized dot_general and the two dot_generals of its gradient."""

  fwd: DotGeneralRaw
  dlhs: DotGeneralRaw
  drhs: DotGeneralRaw
  apply_custom_vjp_on_jax: bool = utils.static_field(default=True)

  @classmethod
  def make(cls, *args, **kwargs) -> 'DotGeneral':
    return dot_general_make(*args, **kwargs)

  def dg_core(self, lhs, rhs, lhs_qt, rhs_qt, dimension_numbers):
    """dot_general with the expanded API: returns (out, (lhs_qt, rhs_qt))."""
    msg = 'AQT is not yet optimized to accept quantized types directly. '
    msg += f'lhs.dtype: {lhs.dtype}, rhs.dtype: {rhs.dtype}'
    floats = (utils.bfloat16, utils.float32, utils.float16)
    assert utils.as_dtype(lhs.dtype) in floats, msg
    assert utils.as_dtype(rhs.dtype) in floats, msg
    self.assert_config_validity()
    dimension_numbers = _canon_dims(dimension_numbers)
    if self.apply_custom_vjp_on_jax and (
        getattr(lhs, 'requires_grad', False)
        or getattr(rhs, 'requires_grad', False)):
      from aqt_b200 import engine
      return engine.dg_core_autograd(self, lhs, rhs, lhs_qt, rhs_qt,
                                     dimension_numbers)
    return _dg_core(lhs, rhs, lhs_qt, rhs_qt, dimension_numbers, self)

  def __call__(self, lhs, rhs, dimension_numbers, precision=None,
               preferred_element_type=None):
    del preferred_element_type
    assert precision is None, (
        f'Precision {precision} requested together with quantization.')
    out, _ = self.dg_core(lhs=lhs, rhs=rhs, lhs_qt=None, rhs_qt=None,
                          dimension_numbers=dimension_numbers)
    return out

  def vjp(self, lhs, rhs, dimension_numbers, lhs_qt=None, rhs_qt=None):
    """Explicit forward + pullback: returns (out, backprop).

    backprop(g) -> (dlhs, drhs). This is the same pairing jax.vjp builds from
    dg_core_vjp_fwd / dg_core_vjp_bwd, without an autograd tape.
    """
    dimension_numbers = _canon_dims(dimension_numbers)
    (out, _), res = dg_core_vjp_fwd(lhs, rhs, lhs_qt, rhs_qt,
                                    dimension_numbers, self)

    def backprop(g):
      dlhs, drhs, *_ = dg_core_vjp_bwd(dimension_numbers, res, (g, None))
      return dlhs, drhs

    return out, backprop

  def assert_config_validity(self):
    """use_fwd_quant and mode combinations the reference rejects (:1024-1078)."""
    if self.fwd.rhs.calibration_mode == CalibrationMode.REMAINING_AXIS:
      assert self.dlhs.rhs.use_fwd_quant is False, (
          'use_fwd_quant should be set to False when remaining axis are used '
          f'for calibration axis. rhs.calibration_mode: '
          f'{self.fwd.rhs.calibration_mode}, dlhs use_fwd_quant: '
          f'{self.dlhs.rhs.use_fwd_quant}')
    if self.fwd.lhs.calibration_mode == CalibrationMode.REMAINING_AXIS:
      assert self.drhs.rhs.use_fwd_quant is False, (
          'use_fwd_quant should be set to False when remaining axis are used '
          f'for calibration axis. lhs.calibration_mode: '
          f'{self.fwd.lhs.calibration_mode}, drhs use_fwd_quant: '
          f'{self.drhs.rhs.use_fwd_quant}')
    bad = [(DequantMode.OUTPUT, CalibrationMode.REMAINING_AXIS),
           (DequantMode.OTHER_INPUT, CalibrationMode.CONTRACTING_AXIS)]
    for dq, cal in bad:
      for name, t in (('lhs', self.fwd.lhs), ('rhs', self.fwd.rhs)):
        assert not (t.calibration_mode == cal and t.dequant_mode == dq), (
            'Unsupported calibration mode - dequant mode combination  for '
            f'{name}. calibration_mode: {t.calibration_mode}, dequant_mode: '
            f'{t.dequant_mode}')


def _canon_dims(dimension_numbers):
  (lca, rca), (lba, rba) = dimension_numbers
  return ((tuple(int(a) for a in lca), tuple(int(a) for a in rca)),
          (tuple(int(a) for a in lba), tuple(int(a) for a in rba)))


def _dg_core(lhs, rhs, lhs_qt, rhs_qt, dimension_numbers, cfg: DotGeneral):
  out, _ = dg_core_vjp_fwd(lhs, rhs, lhs_qt, rhs_qt, dimension_numbers, cfg)
  return out


def dg_core_vjp_fwd(lhs, rhs, lhs_qt, rhs_qt, dimension_numbers,
                    cfg: DotGeneral):
  """Forward pass: ((out, (q_lhs, q_rhs)), residuals)."""
  assert lhs.dtype == rhs.dtype, (
      f'Unmatched lhs and rhs dtype: {lhs.dtype} vs {rhs.dtype}')
  for raw in (cfg.fwd, cfg.dlhs, cfg.drhs):
    _init_calibration_once(raw.dg_quantizer)
  pre = None
  if lhs_qt is None and rhs_qt is None:
    from aqt_b200 import engine
    # Training reads each operand once for its forward and backward copies
    # when the configuration allows it (per-tensor fp8 matmuls).
    pre = engine.prequantize_for_training(cfg, lhs, rhs, dimension_numbers)
  if pre is not None:
    ret, res = engine.dg_raw(cfg.fwd, lhs, rhs, pre[0], pre[1],
                             dimension_numbers, internal_qt=True)
  else:
    ret, res = cfg.fwd(lhs, rhs, lhs_qt, rhs_qt, dimension_numbers)
  ret = ret.to(lhs.dtype)
  assert res is not None, 'res cannot be None in fwd pass.'
  qret = (res.lhs.mt.qx, res.rhs.mt.qx)
  return ((ret, qret), (res, cfg))


def _init_calibration_once(dg_quantizer):
  # The reference deep-copies the config for every call and initialises the
  # copy; here the same config object may be called repeatedly.
  if isinstance(dg_quantizer, DefaultDotGeneralQuantizer):
    for q in (dg_quantizer.lhs, dg_quantizer.rhs):
      if q._calibrator is None:  # pylint: disable=protected-access
        q.init_calibration()
  else:
    dg_quantizer.init_calibration()


def _update_dimension_numbers_for_backward(fwd_dimension_numbers,
                                           y_is_lhs: bool, gradient_rank: int,
                                           y_rank: int):
  """Dimension numbers of dot_general(g, y) and the transpose that follows.

  With x the operand whose gradient is wanted and y the other one: contract
  g's y-free axes with y's free axes, batch over the batch axes; the raw result
  is ordered (batch, x-free, x-contracting sorted by y's contracting order), so
  `out_transpose_axes` puts it back into x's own axis order.
  """
  def ranges_like(*xs):
    start = 0
    for x in xs:
      yield tuple(range(start, start + len(x)))
      start += len(x)

  (x_ca, y_ca), (x_ba, y_ba) = fwd_dimension_numbers
  if y_is_lhs:
    (y_ca, x_ca) = (x_ca, y_ca)
    (y_ba, x_ba) = (x_ba, y_ba)
  x_rank = gradient_rank - y_rank + len(x_ba) + 2 * len(x_ca)
  x_ra = tuple(utils.get_remaining_axes(x_rank, x_ca, x_ba))
  y_ra = tuple(utils.get_remaining_axes(y_rank, y_ca, y_ba))
  if y_is_lhs:
    g_ba, g_ca, _ = ranges_like(x_ba, y_ra, x_ra)
  else:
    g_ba, _, g_ca = ranges_like(x_ba, x_ra, y_ra)
  dims = ((g_ca, y_ra), (g_ba, tuple(y_ba)))
  x_ca_sorted_by_y = tuple(int(v) for v in onp.take(x_ca, onp.argsort(y_ca)))
  out_transpose_axes = tuple(
      int(v) for v in onp.argsort(tuple(x_ba) + x_ra + x_ca_sorted_by_y))
  return dims, out_transpose_axes


def dg_core_vjp_bwd(fwd_dimension_numbers, res, g):
  """Backward pass: (dlhs, drhs, None, None, None)."""
  dg_res, cfg = res
  assert dg_res is not None, (
      'dg_res can only be None in 2nd derivative. It is not yet supported.')
  g = g[0]  # g[1] would be the gradient w.r.t. the returned QTensors.

  from aqt_b200 import engine
  # One read of the cotangent gives both of its quantized copies when all the
  # scales involved are per-tensor (and the kernel covers the dtypes); failing
  # that, one pass over it can still serve both calibrations; otherwise each
  # raw dot calibrates and quantizes it on its own.
  shared = None
  if cfg.dlhs.local_aqt is None and cfg.drhs.local_aqt is None:
    try:
      shared = engine.cotangent_pair(cfg, dg_res, g)
      if shared is None:
        shared = engine.cotangent_dual(cfg, dg_res, g,
                                       fwd_dimension_numbers)
      if shared is None:
        shared = engine.shared_cotangent_scales(cfg, dg_res, g)
    except NotImplementedError:
      shared = None

  def grad_dot_general(y_res: TensorRes, quant_grad, dg_raw, y_is_lhs):
    dims, out_transpose_axes = _update_dimension_numbers_for_backward(
        fwd_dimension_numbers, y_is_lhs, g.ndim, y_res.mt.x.ndim)
    g_qt = None if shared is None else shared[1 if y_is_lhs else 0]
    # the stored operand's backward copy, when the forward pass made one
    y_qt = engine.bwd_copy(y_res.mt.qx) if dg_raw.rhs.use_fwd_quant else None
    out = engine.dg_raw(dg_raw, g, y_res.mt, g_qt, y_qt, dims,
                        out_transpose_axes=out_transpose_axes,
                        internal_qt=True)[0]
    if isinstance(quant_grad, str):
      raise AssertionError(quant_grad)
    if quant_grad is not None:
      out = quant_grad(out)[0]
    return out

  dlhs = grad_dot_general(dg_res.rhs, dg_res.lhs.quant_grad, cfg.dlhs, False)
  drhs = grad_dot_general(dg_res.lhs, dg_res.rhs.quant_grad, cfg.drhs, True)
  return (dlhs, drhs, None, None, None)
