"""Freezers: where a converted model keeps its quantized operands.

Reference: aqt/jax/v2/flax/freezer.py:24-100 (the general Freezer, one
variable named 'frozen' that holds a whole QTensor) and the legacy Freezer of
aqt/jax/v2/flax/aqt_flax.py:149-232 (two variables, 'value' = the quantized
values and 'scale' = the scale transposed to the dot's OUTPUT layout, i.e.
QTensor.scale_t).

The reference stores these in Flax variable collections. flax is not a
dependency here; a `variables` mapping plays that part:

    variables[collection][freezer name]['frozen']            general freezer
    variables[collection][freezer name]['value' | 'scale']   legacy freezer

It is an ordinary nested dict of tensors / QTensors, so a converted model's
serving checkpoint is `variables['aqt']` saved by whatever means the host
framework has, with the same variable names and layouts as the reference's.
"""

from __future__ import annotations

import enum
from typing import Any, Callable, MutableMapping

from aqt_b200.v2 import aqt_tensor
from aqt_b200.v2 import utils

QuantMode = utils.QuantMode


class FreezerMode(enum.Enum):
  NONE = 1
  WRITE = 2
  READ = 3


_FREEZE_VAR_NAME = 'frozen'


def _scope(variables: MutableMapping, collection: str, name: str, create: bool):
  if not create:
    return variables.get(collection, {}).get(name)
  return variables.setdefault(collection, {}).setdefault(name, {})


class Freezer:
  """General freezer (freezer.py:32-100): get() returns the frozen value in
  READ mode (None when nothing was stored), set() stores it in WRITE mode; in
  READ mode set() only initialises a missing variable, never overwrites."""

  def __init__(self, name: str, collection: str, mode: FreezerMode,
               variables: MutableMapping,
               axis_metadata_wrapper: None | Callable[..., Any] = None):
    self.name, self.collection, self.mode = name, collection, mode
    self.variables = variables
    self.axis_metadata_wrapper = axis_metadata_wrapper

  def _init_value(self, inputs):
    if self.axis_metadata_wrapper is not None:
      return self.axis_metadata_wrapper(inputs)
    return inputs

  def get(self):
    if self.mode in (FreezerMode.NONE, FreezerMode.WRITE):
      return None
    assert self.mode == FreezerMode.READ, 'Unknown quant mode.'
    scope = _scope(self.variables, self.collection, self.name, False)
    if scope is None or _FREEZE_VAR_NAME not in scope:
      return None
    return scope[_FREEZE_VAR_NAME]

  def set(self, inputs) -> None:
    if self.mode == FreezerMode.NONE:
      return None
    scope = _scope(self.variables, self.collection, self.name, True)
    if self.mode == FreezerMode.WRITE:
      scope[_FREEZE_VAR_NAME] = inputs
    elif self.mode == FreezerMode.READ:
      # set() in READ mode works as an initializer for checkpoint reading
      scope.setdefault(_FREEZE_VAR_NAME, self._init_value(inputs))
    else:
      assert False, 'Unknown quant mode.'
    return None


class LegacyFreezer:
  """The two-variable freezer of aqt_flax.py:149-232: 'value' (quantized
  values, the operand's own shape and container dtype) and 'scale' (scale_t:
  the scale in the layout of the dot's output). get() in SERVE mode returns a
  QTensor with scale=None and scale_t set; the caller recovers `scale`
  (aqt_flax.py:235-254)."""

  def __init__(self, name: str, quant_collection: str, quant_mode: QuantMode,
               variables: MutableMapping):
    self.name, self.quant_collection = name, quant_collection
    self.quant_mode = quant_mode
    self.variables = variables

  def get(self):
    if self.quant_mode != QuantMode.SERVE:
      return None
    scope = _scope(self.variables, self.quant_collection, self.name, False)
    assert scope is not None and 'value' in scope and 'scale' in scope, (
        f'SERVE mode without frozen variables {self.quant_collection}/'
        f'{self.name}/(value, scale)')
    return aqt_tensor.QTensor(
        qvalue=scope['value'], scale=None, scale_t=[scope['scale']], bias=[],
        dequant_dtype=utils.as_dtype(scope['scale'].dtype))

  def set(self, inputs: aqt_tensor.QTensor) -> None:
    if inputs.bias:
      raise NotImplementedError(
          'Quantization biases are not supported in AQT Flax Legacy Freezer.')
    if self.quant_mode == QuantMode.CONVERT:
      assert inputs.scale_t is not None and len(inputs.scale_t) == 1
      scope = _scope(self.variables, self.quant_collection, self.name, True)
      scope['value'] = inputs.qvalue
      scope['scale'] = inputs.scale_t[0]
    return None
