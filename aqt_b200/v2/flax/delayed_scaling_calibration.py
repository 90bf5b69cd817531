"""Delayed scaling calibration: the scale comes from earlier steps' maxima.

Reference: aqt/jax/v2/flax/delayed_scaling_calibration.py:28-124 (logic from
Transformer Engine). Per-tensor only, as in the reference (:66-75). State, as
the reference's `calibration_stats` collection holds it:

  amax_history : f32[amax_history_length], zeros at first
  bound        : f32[1], zero at first

Every call (get_bound, :57-97):
  new_bound   = max(amax_history) if that is > 0 and finite else bound
  new_history = roll(amax_history, -1), element 0 := max |x|
  TRAIN / CALIBRATE modes write both back; SERVE (and a missing context)
  leaves the state alone. scale = new_bound / quant_bound [-> power of two],
  cast to `dtype` or x's dtype.

On the device the point of the scheme is that the scale does not depend on the
tensor being quantized: aqtb200_delayed_scaling_scale reads 1024 floats, the
quantize kernel starts at once, and max |x| for the history is taken beside
it (or arrives from the kernel that produced x, aqtb200_gemm_desc.amax_out).

The reference keeps the state in Flax variables, which outlive the per-call
deep copy of the configuration (aqt_flax.py:337). Here the calibrator owns a
`CalibrationStats` holder that deep copies share instead of duplicating.
"""

from __future__ import annotations

import ctypes as C
import dataclasses
from typing import Any

from aqt_b200.v2 import calibration
from aqt_b200.v2 import utils

CALIBRATION_STATS = 'calibration_stats'


class CalibrationStats:
  """amax_history and bound of one quantizer, on the device. Deep copies of a
  configuration keep pointing at the same holder."""

  def __init__(self):
    self.amax_history = None
    self.bound = None

  def __deepcopy__(self, memo):
    return self

  def setup(self, length: int, device):
    import torch
    if self.amax_history is None:
      self.amax_history = torch.zeros(length, dtype=torch.float32,
                                      device=device)
      self.bound = torch.zeros(1, dtype=torch.float32, device=device)


@utils.flax_slots_kw_only_dataclass
class DelayedScalingCalibration(calibration.Calibration):
  """Calibration from a history of maxima (see module docstring)."""

  amax_history_length: int = 1024
  stats: Any = dataclasses.field(default_factory=CalibrationStats)

  # -- state -----------------------------------------------------------------
  def setup(self, device) -> None:
    self.stats.setup(self.amax_history_length, device)

  @property
  def amax_history(self):
    return self.stats.amax_history

  @property
  def bound(self):
    return self.stats.bound

  def init_calibration(self):
    # the reference touches its variables here so that they exist (:120-124);
    # the device buffers are made on first use, when the device is known
    self.stats  # pylint: disable=pointless-statement

  # -- the calibration ---------------------------------------------------------
  @staticmethod
  def updates_state(context) -> bool:
    """TRAIN / CALIBRATE write the state back; SERVE, or no context, do not
    (reference :77-79, 93-95)."""
    quant_mode = context.quant_mode if context else utils.QuantMode.SERVE
    return quant_mode in (utils.QuantMode.TRAIN, utils.QuantMode.CALIBRATE)

  def next_scale(self, device, numerics_, compute_dtype, context=None):
    """First half of a step: the one-element scale from the history (dtype
    `dtype` or compute_dtype); updates `bound` in TRAIN / CALIBRATE modes."""
    from aqt_b200 import _lib
    from aqt_b200 import engine
    self.setup(device)
    spec = engine._spec_for(  # pylint: disable=protected-access
        numerics_, engine._code(compute_dtype),  # pylint: disable=protected-access
        self.dtype, True, None, self.po2_scale)
    scale = engine._empty(  # pylint: disable=protected-access
        1, engine._CODE_TORCH[spec.scale_dtype], device)  # pylint: disable=protected-access
    rc = engine._call(  # pylint: disable=protected-access
        _lib.load().aqtb200_delayed_scaling_scale,
        self.amax_history.data_ptr(), self.amax_history_length,
        self.bound.data_ptr(), 1 if self.updates_state(context) else 0,
        C.byref(spec), scale.data_ptr(), engine._stream())  # pylint: disable=protected-access
    _lib.check(rc, 'aqtb200_delayed_scaling_scale')
    return scale

  def push_amax(self, amax):
    """Second half: max |x| (one-element f32 device tensor) enters the history."""
    import torch
    from aqt_b200 import _lib
    from aqt_b200 import engine
    assert amax.dtype == torch.float32 and amax.numel() == 1
    rc = engine._call(  # pylint: disable=protected-access
        _lib.load().aqtb200_delayed_scaling_push, self.amax_history.data_ptr(),
        self.amax_history_length, amax.data_ptr(), engine._stream())  # pylint: disable=protected-access
    _lib.check(rc, 'aqtb200_delayed_scaling_push')

  def device_scale(self, x, numerics_, context=None, amax_fn=None,
                   compute_dtype=None):
    """One step of the scheme for operand x: returns the one-element scale
    and, in TRAIN / CALIBRATE modes, updates bound and amax_history.
    `amax_fn`: optional callable returning a one-element f32 device tensor
    with max |x| (e.g. taken from whoever produced x); otherwise it is reduced
    here. `compute_dtype`: the float dtype x counts as when it is a stored
    int8 / fp8 tensor."""
    from aqt_b200 import engine
    scale = self.next_scale(
        x.device, numerics_,
        compute_dtype if compute_dtype is not None else x.dtype, context)
    if self.updates_state(context):
      self.push_amax(amax_fn() if amax_fn is not None else
                     engine.absmax_raw(x))
    return scale

  def get_bound(self, x, shared_axes, context=None):
    """The bound alone, shape (1,) * x.ndim (reference :57-97)."""
    del x, shared_axes, context
    raise NotImplementedError(
        'get_bound() as a stand-alone call is not part of the device path; '
        'use get_scale_and_bias_and_sparsity()')

  def get_scale_and_bias_and_sparsity(self, x, shared_axes, numerics_,
                                      context=None):
    del shared_axes  # per-tensor whatever the axes (reference :66-75)
    scale = self.device_scale(x, numerics_, context)
    return [scale.view([1] * x.ndim)], [], None
