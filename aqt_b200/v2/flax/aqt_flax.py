"""AqtDotGeneral / AqtEinsum: the objects a model injects in place of
lax.dot_general / jnp.einsum.

Reference: aqt/jax/v2/flax/aqt_flax.py (AqtDotGeneral :278-570, AqtEinsum
:573-732). The reference classes are flax.linen Modules; flax is not a
dependency here, so these are plain callables with the same constructor
arguments and call signatures:

    dg = AqtDotGeneral(cfg, prng_name='params')
    y = dg(lhs, rhs, dimension_numbers)            # like lax.dot_general
    y = AqtEinsum(cfg)('bthd,bshd->bhts', q, k)    # like jnp.einsum

What the Module machinery provided in the reference and how it maps here:
  * make_rng(prng_name) -> `rngs`: a dict name -> key, or a callable
    name -> key, given at construction or per call; each call consumes one
    fresh sub-key (config.set_context splits it per quantizer).
  * Freezer variables (serving): a `variables` dict stands in for the Flax
    variable tree; CONVERT stores the quantized operand under
    variables[quant_collection][var_name] in the reference's layouts, SERVE
    feeds it back into the dot instead of re-quantizing
    (aqt_flax.py:149-232, 440-512; flax/freezer.py:32-100).
"""

from __future__ import annotations

import copy
import enum
from typing import Any

from aqt_b200.v2 import aqt_dot_general
from aqt_b200.v2 import config as aqt_config
from aqt_b200.v2 import stochastic_rounding
from aqt_b200.v2 import transpose
from aqt_b200.v2 import utils
from aqt_b200.v2.flax import freezer as general_freezer

QuantMode = utils.QuantMode


class _Rngs:
  """name -> stream of keys, the stand-in for flax's make_rng."""

  def __init__(self, rngs):
    self._rngs = rngs
    self._counters = {}

  def make_rng(self, name):
    if self._rngs is None:
      return None
    base = self._rngs(name) if callable(self._rngs) else self._rngs.get(name)
    if base is None:
      return None
    n = self._counters.get(name, 0)
    self._counters[name] = n + 1
    return stochastic_rounding.split(base, n + 2)[n + 1] if n else (
        stochastic_rounding.split(base, 2)[1])


class FreezerMode(enum.Enum):
  """What a CONVERT step stores (aqt_flax.py:143-146)."""
  NONE = 1
  CALIBRATION = 2
  CALIBRATION_AND_VALUE = 3


_QUANT_TO_FREEZER_MODE = {
    QuantMode.TRAIN: general_freezer.FreezerMode.NONE,
    QuantMode.CALIBRATE: general_freezer.FreezerMode.NONE,
    QuantMode.CONVERT: general_freezer.FreezerMode.WRITE,
    QuantMode.SERVE: general_freezer.FreezerMode.READ,
}


def _maybe_recover_scale_from_scale_t(qt, dimension_numbers, is_rhs, lhs_shape,
                                      rhs_shape):
  """aqt_flax.py:235-254: a QTensor read from the legacy freezer carries only
  scale_t (output layout); put the scale back into the operand's layout."""
  if qt is None or qt.scale is not None or qt.scale_t is None:
    return qt
  fn = (transpose.rhs_recover_scale_from_scale_t if is_rhs else
        transpose.lhs_recover_scale_from_scale_t)
  return qt.replace(
      scale=[fn(s, dimension_numbers, lhs_shape, rhs_shape)
             for s in qt.scale_t], scale_t=None)


def _populate_scale_t(qt, dimension_numbers, is_rhs, lhs_shape, rhs_shape):
  """aqt_flax.py:257-275."""
  if qt.scale is None:
    return qt
  fn = (transpose.rhs_scale_transpose_to_output if is_rhs else
        transpose.lhs_scale_transpose_to_output)
  return qt.replace(scale_t=[fn(s, dimension_numbers, lhs_shape, rhs_shape)
                             for s in qt.scale])


class AqtDotGeneral:
  """A drop-in dot_general with AQT quantization (aqt_flax.py:278-570).

  Serving conversion follows the reference: with `*_quant_mode=CONVERT` and
  `*_freeze_mode` CALIBRATION_AND_VALUE (or CALIBRATION: scales only) a call
  stores the operand's QTensor in `variables[quant_collection][*_var_name]`,
  in the legacy two-variable layout ('value', 'scale' = scale_t) or, with
  `use_legacy_freezer=False`, as one 'frozen' QTensor; with SERVE it is read
  back from there and fed to the dot instead of quantizing. With
  `*_apply_quant_mode=False` the freezers are bypassed and `*_qtensor` is
  used as given (aqt_flax.py:448-449).
  """

  def __init__(self, cfg: None | aqt_dot_general.DotGeneral = None,
               prng_name: None | str = 'params',
               lhs_quant_mode: QuantMode = QuantMode.TRAIN,
               rhs_quant_mode: QuantMode = QuantMode.TRAIN,
               rngs: Any = None, name: str = 'AqtDotGeneral',
               lhs_apply_quant_mode: bool = True,
               rhs_apply_quant_mode: bool = True,
               lhs_var_name: str = 'qlhs', rhs_var_name: str = 'qrhs',
               lhs_qtensor=None, rhs_qtensor=None,
               lhs_freeze_mode: FreezerMode = FreezerMode.NONE,
               rhs_freeze_mode: FreezerMode = FreezerMode.NONE,
               quant_collection: str = 'aqt',
               use_legacy_freezer: bool = True,
               variables=None):
    self.cfg = cfg
    self.prng_name = prng_name
    self.lhs_quant_mode = lhs_quant_mode
    self.rhs_quant_mode = rhs_quant_mode
    self.name = name
    self._rngs = _Rngs(rngs)
    self.lhs_apply_quant_mode = lhs_apply_quant_mode
    self.rhs_apply_quant_mode = rhs_apply_quant_mode
    self.lhs_var_name, self.rhs_var_name = lhs_var_name, rhs_var_name
    self.lhs_freeze_mode, self.rhs_freeze_mode = lhs_freeze_mode, rhs_freeze_mode
    self.quant_collection = quant_collection
    self.use_legacy_freezer = use_legacy_freezer
    # The variable tree (the 'aqt' collection of the reference's Flax module).
    self.variables = variables if variables is not None else {}
    # Operands handed in directly (used when *_apply_quant_mode is False).
    self.lhs_qtensor = lhs_qtensor
    self.rhs_qtensor = rhs_qtensor

  def _freezer(self, var_name, quant_mode):
    if self.use_legacy_freezer:
      return general_freezer.LegacyFreezer(
          name=var_name, quant_collection=self.quant_collection,
          quant_mode=quant_mode, variables=self.variables)
    return general_freezer.Freezer(
        name=var_name, collection=self.quant_collection,
        mode=_QUANT_TO_FREEZER_MODE[quant_mode], variables=self.variables)

  def make_aqt_dg(self, lhs_shape, rhs_shape, dimension_numbers):
    """Returns the callable for these shapes (reference :326-514)."""
    if self.cfg is None:
      return aqt_dot_general.lax_dot_general
    lhs_shape, rhs_shape = tuple(lhs_shape), tuple(rhs_shape)
    cfg = copy.deepcopy(self.cfg)
    lhs_freezer = self._freezer(self.lhs_var_name, self.lhs_quant_mode)
    rhs_freezer = self._freezer(self.rhs_var_name, self.rhs_quant_mode)
    key = self._rngs.make_rng(self.prng_name) if self.prng_name else None
    cfg = aqt_config.set_context(cfg, key, train_step=None,
                                 lhs_quant_mode=self.lhs_quant_mode,
                                 rhs_quant_mode=self.rhs_quant_mode)

    def ret_dg(lhs, rhs, dimension_numbers=dimension_numbers, precision=None,
               preferred_element_type=None):
      del preferred_element_type
      assert precision is None, (
          f'Precision {precision} requested together with quantization.')
      msg = 'AQT is not yet optimized to accept quantized types directly. '
      msg += f'lhs.dtype: {lhs.dtype}, rhs.dtype: {rhs.dtype}'
      floats = (utils.bfloat16, utils.float32, utils.float16)
      assert utils.as_dtype(lhs.dtype) in floats, msg
      assert utils.as_dtype(rhs.dtype) in floats, msg
      cfg.assert_config_validity()
      dims = aqt_dot_general._canon_dims(dimension_numbers)  # pylint: disable=protected-access

      # Getter
      lhs_qt = (lhs_freezer.get() if self.lhs_apply_quant_mode else
                self.lhs_qtensor)
      rhs_qt = (rhs_freezer.get() if self.rhs_apply_quant_mode else
                self.rhs_qtensor)
      lhs_qt = _maybe_recover_scale_from_scale_t(lhs_qt, dims, False,
                                                 lhs_shape, rhs_shape)
      rhs_qt = _maybe_recover_scale_from_scale_t(rhs_qt, dims, True,
                                                 lhs_shape, rhs_shape)

      out, (out_lhs_qt, out_rhs_qt) = cfg.dg_core(
          lhs=lhs, rhs=rhs, lhs_qt=lhs_qt, rhs_qt=rhs_qt,
          dimension_numbers=dims)

      # What a conversion stores: nothing, the scales, or scales and values.
      def frozen_part(qt, freeze_mode, apply, quant_mode):
        if freeze_mode == FreezerMode.NONE:
          if apply and quant_mode in (QuantMode.CONVERT, QuantMode.SERVE):
            raise ValueError('Freezer is used with Freezer mode NONE.')
          return qt
        if freeze_mode == FreezerMode.CALIBRATION:
          return qt.without_qvalue()
        if freeze_mode == FreezerMode.CALIBRATION_AND_VALUE:
          return qt
        raise ValueError('Unknown freeze mode: %s' % freeze_mode)

      out_lhs_qt = frozen_part(out_lhs_qt, self.lhs_freeze_mode,
                               self.lhs_apply_quant_mode, self.lhs_quant_mode)
      out_rhs_qt = frozen_part(out_rhs_qt, self.rhs_freeze_mode,
                               self.rhs_apply_quant_mode, self.rhs_quant_mode)

      # Setter
      contracting = aqt_dot_general.CalibrationMode.CONTRACTING_AXIS
      if self.use_legacy_freezer:
        if cfg.fwd.lhs.calibration_mode == contracting:
          out_lhs_qt = _populate_scale_t(out_lhs_qt, dims, False, lhs_shape,
                                         rhs_shape)
        if cfg.fwd.rhs.calibration_mode == contracting:
          out_rhs_qt = _populate_scale_t(out_rhs_qt, dims, True, lhs_shape,
                                         rhs_shape)
      if self.lhs_apply_quant_mode:
        lhs_freezer.set(out_lhs_qt)
      elif self.lhs_quant_mode == QuantMode.CONVERT:
        self.lhs_qtensor = out_lhs_qt
      if self.rhs_apply_quant_mode:
        rhs_freezer.set(out_rhs_qt)
      elif self.rhs_quant_mode == QuantMode.CONVERT:
        self.rhs_qtensor = out_rhs_qt
      return out

    return ret_dg

  def frozen(self, side: str):
    """The QTensor a SERVE call would read for 'lhs' / 'rhs' (scale recovered
    needs shapes, so the legacy layout comes back with scale_t only)."""
    mode = QuantMode.SERVE
    name = self.lhs_var_name if side == 'lhs' else self.rhs_var_name
    return self._freezer(name, mode).get()

  def __call__(self, lhs, rhs, dimension_numbers, precision=None,
               preferred_element_type=None):
    aqt_dg = self.make_aqt_dg(lhs.shape, rhs.shape, dimension_numbers)
    return aqt_dg(lhs, rhs, dimension_numbers, precision,
                  preferred_element_type=preferred_element_type)


class AqtEinsum:
  """A drop-in two-operand einsum with AQT quantization (reference :573-732).

  When the einsum lowers to a dot_general whose operand order is swapped
  relative to the arguments, the lhs/rhs roles of the config -- and of every
  lhs_* / rhs_* option, so that "lhs" keeps meaning the FIRST einsum argument
  -- are swapped too (reference :684-704).
  """

  def __init__(self, cfg: None | aqt_dot_general.DotGeneral = None,
               prng_name: None | str = 'params',
               lhs_quant_mode: QuantMode = QuantMode.TRAIN,
               rhs_quant_mode: QuantMode = QuantMode.TRAIN,
               rngs: Any = None, name: str = 'AqtEinsum',
               lhs_apply_quant_mode: bool = True,
               rhs_apply_quant_mode: bool = True,
               lhs_var_name: str = 'qlhs', rhs_var_name: str = 'qrhs',
               lhs_qtensor=None, rhs_qtensor=None,
               lhs_freeze_mode: FreezerMode = FreezerMode.NONE,
               rhs_freeze_mode: FreezerMode = FreezerMode.NONE,
               quant_collection: str = 'aqt',
               use_legacy_freezer: bool = True, variables=None):
    self.cfg = cfg
    self.prng_name = prng_name
    self.rngs = rngs
    self.name = name
    self.quant_collection = quant_collection
    self.use_legacy_freezer = use_legacy_freezer
    self.variables = variables if variables is not None else {}
    self._sides = {
        'lhs': dict(quant_mode=lhs_quant_mode,
                    apply_quant_mode=lhs_apply_quant_mode,
                    var_name=lhs_var_name, qtensor=lhs_qtensor,
                    freeze_mode=lhs_freeze_mode),
        'rhs': dict(quant_mode=rhs_quant_mode,
                    apply_quant_mode=rhs_apply_quant_mode,
                    var_name=rhs_var_name, qtensor=rhs_qtensor,
                    freeze_mode=rhs_freeze_mode),
    }
    # One inner AqtDotGeneral per operand order, built on first use and kept:
    # it owns the position in the rng stream, which must survive from one call
    # to the next. Frozen operands live in `variables`, shared by both.
    self._dgs = {}

  def _inner(self, swap: bool) -> AqtDotGeneral:
    if swap not in self._dgs:
      cfg = copy.deepcopy(self.cfg)
      first, second = ('rhs', 'lhs') if swap else ('lhs', 'rhs')
      if cfg is not None and swap:
        cfg.fwd.dg_quantizer.swap_lhs_and_rhs()
        cfg.fwd.lhs, cfg.fwd.rhs = cfg.fwd.rhs, cfg.fwd.lhs
        cfg.dlhs, cfg.drhs = cfg.drhs, cfg.dlhs
      kw = {}
      for dg_side, my_side in (('lhs', first), ('rhs', second)):
        for opt, val in self._sides[my_side].items():
          kw[f'{dg_side}_{opt}'] = val
      self._dgs[swap] = AqtDotGeneral(
          cfg, prng_name=self.prng_name, rngs=self.rngs, name=self.name,
          quant_collection=self.quant_collection,
          use_legacy_freezer=self.use_legacy_freezer,
          variables=self.variables, **kw)
    return self._dgs[swap]

  def _get_qtensor(self, which: str):
    for swap, dg in self._dgs.items():
      attr = ('rhs' if which == 'lhs' else 'lhs') if swap else which
      qt = getattr(dg, attr + '_qtensor')
      if qt is not None:
        return qt
    return self._sides[which]['qtensor']

  def _set_qtensor(self, which: str, qt):
    self._sides[which]['qtensor'] = qt
    for swap, dg in self._dgs.items():
      attr = ('rhs' if which == 'lhs' else 'lhs') if swap else which
      setattr(dg, attr + '_qtensor', qt)

  # operands handed in directly (used when *_apply_quant_mode is False)
  lhs_qtensor = property(lambda self: self._get_qtensor('lhs'),
                         lambda self, qt: self._set_qtensor('lhs', qt))
  rhs_qtensor = property(lambda self: self._get_qtensor('rhs'),
                         lambda self, qt: self._set_qtensor('rhs', qt))

  def __call__(self, eqn, lhs_g, rhs_g):
    _, _, swap = aqt_dot_general.einsum_to_dot_general(eqn, lhs_g.ndim,
                                                       rhs_g.ndim)
    return aqt_dot_general.einsum(eqn, lhs_g, rhs_g, self._inner(swap))
