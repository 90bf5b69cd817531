"""Scale calibration (reference: aqt/jax/v2/calibration.py:25-157).

Only the calibrations on the quantized dot_general hot path live here:
AbsMaxCalibration (with clipping_scale and po2_scale) and ConstantCalibration
as configuration objects. The arithmetic runs on the device (engine.absmax_*).
"""

import abc
from typing import Any, Sequence

from aqt_b200.v2 import utils


@utils.flax_slots_kw_only_dataclass
class Calibration(abc.ABC):
  """Produces the scale (list), bias (list) and sparsity mask of one tensor."""

  # dtype of the scale array; None means "the dtype of the input".
  dtype: None | Any = utils.static_field(default=None)
  # Round the scale to a power of two.
  po2_scale: bool = utils.static_field(default=False)

  @abc.abstractmethod
  def get_scale_and_bias_and_sparsity(self, x, shared_axes, numerics_,
                                      context=None):
    pass

  def init_calibration(self):
    pass


@utils.flax_slots_kw_only_dataclass
class AbsMaxCalibration(Calibration):
  """scale = max|x| over shared_axes (0 -> 1) [* clipping_scale] / quant_bound.

  calibration.py:117-157. The division happens in the input dtype, so bf16
  inputs get bf16 scales unless `dtype` says otherwise.
  """

  clipping_scale: None | float = None

  def get_scale_and_bias_and_sparsity(self, x, shared_axes, numerics_,
                                      context=None):
    del context
    from aqt_b200 import engine
    assert shared_axes is not None, (
        'Perhaps you are using DequantMode.THIS_INPUT (fake_quant) and forgot'
        ' to set them.')
    scale = engine.absmax_scale(
        x, list(shared_axes), numerics_, scale_dtype=self.dtype,
        clipping_scale=self.clipping_scale, po2_scale=self.po2_scale)
    return [scale], [], None


@utils.flax_slots_kw_only_dataclass
class ConstantCalibration(Calibration):
  """A fixed bound (calibration.py:67-103). Configuration only on this path."""

  bound: Any
  bias: Any = None

  def get_scale_and_bias_and_sparsity(self, x, shared_axes, numerics_,
                                      context=None):
    raise NotImplementedError(
        'ConstantCalibration is not on the sm_100a hot path; use '
        'AbsMaxCalibration.')
