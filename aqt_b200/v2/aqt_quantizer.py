"""Quantizer: how ONE tensor is calibrated and quantized.

Reference: aqt/jax/v2/aqt_quantizer.py:37-214.
"""

from typing import Any, Sequence

from aqt_b200.v2 import aqt_tensor
from aqt_b200.v2 import calibration
from aqt_b200.v2 import utils
from aqt_b200.v2.numerics import no_numerics
from aqt_b200.v2.numerics import numerics
from aqt_b200.v2.numerics import utils as numerics_utils

AbstractAqtNumerics = numerics.AqtNumerics
AbstractAqtCalibration = calibration.Calibration


@utils.flax_slots_kw_only_dataclass
class Quantizer:
  """Configuration of quantization of one tensor."""

  numerics: AbstractAqtNumerics = utils.static_field()
  calib_shared_axes: Any = utils.static_field()  # None | axes | "per_tensor"
  scale_stop_grad: bool = utils.static_field()
  scale_dtype: Any = utils.static_field(default=None)
  # A Calibration class or a functools.partial of one; instantiated late by
  # init_calibration() so setters can still wrap it.
  calibration: Any = utils.static_field(default=None)
  _calibrator: Any = utils.static_field(default=None)
  context: utils.Context

  def init_calibration(self):
    assert self._calibrator is None, 'second call to self.init_calibration()'
    if self.calibration is not None:
      self._calibrator = self.calibration(dtype=self.scale_dtype)
      self._calibrator.init_calibration()

  def shared_axes(self, ndim: int, calibration_axes):
    if self.calib_shared_axes == 'per_tensor':
      return list(range(ndim))
    return self.calib_shared_axes or calibration_axes

  def quant(self, x, *, calibration_axes, tiling_state=None):
    qt = self.calibrate(
        x, calibration_axes=calibration_axes, tiling_state=tiling_state)
    return self.calculate_qvalue(x, qt)

  def calibrate(self, x, *, calibration_axes, tiling_state=None):
    """Returns a QTensor holding only the scale (aqt_quantizer.py:79-157)."""
    if tiling_state:
      raise NotImplementedError('tiled (sub-channel) quantization')
    if isinstance(self.numerics, no_numerics.NoNumerics):
      return aqt_tensor.QTensor(
          qvalue=x, scale=[], scale_t=None, bias=[],
          dequant_dtype=utils.as_dtype(x.dtype))
    shared_axes = self.shared_axes(x.ndim, calibration_axes)
    assert self.calibration is not None, (
        f'{self.calibration = } must be set if {self.numerics = } is not'
        ' NoNumerics')
    assert self._calibrator is not None, 'forgot self.init_calibration()?'
    scale, bias, sparsity_mask = (
        self._calibrator.get_scale_and_bias_and_sparsity(
            x, shared_axes, self.numerics, self.context))
    return aqt_tensor.QTensor(
        qvalue=None, sparsity_mask=sparsity_mask, scale=scale, scale_t=None,
        bias=bias, dequant_dtype=utils.as_dtype(x.dtype))

  def calculate_qvalue(self, x, qt: aqt_tensor.QTensor):
    """Fills qt.qvalue from x and qt.scale (aqt_quantizer.py:159-176)."""
    if isinstance(self.numerics, no_numerics.NoNumerics):
      return qt, None
    from aqt_b200 import engine
    import functools
    noise = None
    noise_fn = getattr(self.numerics, 'noise_fn', None)
    if noise_fn:
      assert self.context.key is not None, (
          'noise_fn is set, requestic stochastic rounding, but RNG was not '
          'passed in Context.key')
      noise = noise_fn(tuple(x.shape), self.context.key)
    assert len(qt.scale) == 1 and not qt.bias
    qvalue = engine.quantize_with_scale(x, qt.scale[0], self.numerics, noise)
    qt = qt.replace(qvalue=qvalue)
    quant_grad = functools.partial(self.numerics.vjp_bwd, (x,))
    return qt, quant_grad


def quantizer_make(n_bits, preserve_max_val: bool = False,
                   initialize_calibration: bool = True,
                   scale_stop_grad: bool = True,
                   scale_dtype=None) -> Quantizer:
  quantizer = Quantizer(
      numerics=numerics_utils.get_numerics(n_bits, preserve_max_val),
      calib_shared_axes=None,
      scale_stop_grad=scale_stop_grad,
      scale_dtype=scale_dtype,
      calibration=None if n_bits is None else calibration.AbsMaxCalibration,
      context=utils.Context(key=None, train_step=None),
  )
  if initialize_calibration:
    quantizer.init_calibration()
  return quantizer


def make_fake_quant(quantizer: Quantizer, calibration_axes=None):
  def fake_quant(x):
    x_q, _ = quantizer.quant(x, calibration_axes=calibration_axes)
    return x_q.dequant()
  return fake_quant
