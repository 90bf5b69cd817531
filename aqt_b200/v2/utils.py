"""Small shared helpers: dataclass decorators, Context, QuantMode, axis maths.

Mirrors the public names of the reference's aqt/jax/v2/utils.py (Context
:151-155, QuantMode :85-89, infer_dtype_from_bits :120-135,
get_remaining_axes :138-148, static_field/dynamic_field :92-97) without any
jax/flax dependency: the dataclasses here are plain mutable slotted Python
dataclasses, and "dtype" objects are the small DType tokens defined below.
"""

from __future__ import annotations

import dataclasses
import enum
import functools
import pprint
import re
from typing import Any, Sequence

AxisIdx = int
AxisSize = int
ShapeTemplate = Sequence[None | int]
DotGeneralT = Any
AutoScaleSearchConfig = Sequence[float]


class DType:
  """A dtype token. Compares equal to its name and to the same token."""

  __slots__ = ('name', 'itemsize', 'is_float', 'code')

  def __init__(self, name: str, itemsize: int, is_float: bool, code: int):
    self.name = name
    self.itemsize = itemsize
    self.is_float = is_float
    self.code = code  # the aqtb200_dtype value of include/aqt_b200.h

  def __repr__(self):
    return self.name

  def __eq__(self, other):
    if isinstance(other, DType):
      return self.name == other.name
    if isinstance(other, str):
      return self.name == other
    return NotImplemented

  def __hash__(self):
    return hash(self.name)

  def __deepcopy__(self, memo):
    return self

  def __copy__(self):
    return self


float32 = DType('float32', 4, True, 0)
bfloat16 = DType('bfloat16', 2, True, 1)
int8 = DType('int8', 1, False, 2)
float8_e4m3fn = DType('float8_e4m3fn', 1, True, 3)
float8_e5m2 = DType('float8_e5m2', 1, True, 4)
int32 = DType('int32', 4, False, 5)
# int4 values live in an int8 container on the device; the token only records
# what the reference would have called the array's dtype.
int4 = DType('int4', 1, False, 2)
float16 = DType('float16', 2, True, -1)

_ALL_DTYPES = {
    d.name: d
    for d in (float32, bfloat16, int8, float8_e4m3fn, float8_e5m2, int32, int4,
              float16)
}


def as_dtype(x) -> None | DType:
  """Maps torch / numpy / ml_dtypes / string dtypes onto DType tokens."""
  if x is None or isinstance(x, DType):
    return x
  name = getattr(x, 'name', None) or str(x)
  name = name.replace('torch.', '').replace("<class '", '').replace("'>", '')
  name = name.split('.')[-1]
  if name in _ALL_DTYPES:
    return _ALL_DTYPES[name]
  raise TypeError(f'unsupported dtype {x!r}')


def promote_types(a: DType, b: DType) -> DType:
  """jnp.promote_types restricted to the float types of the path."""
  a, b = as_dtype(a), as_dtype(b)
  if a == b:
    return a
  if float32 in (a, b):
    return float32
  if {a.name, b.name} == {'bfloat16', 'float16'}:
    return float32
  raise TypeError(f'no promotion rule for {a} and {b}')


def assert_shape(shape: Sequence[int], shape_template: ShapeTemplate, msg: str):
  shape, shape_template = list(shape), list(shape_template)
  assert len(shape) == len(shape_template), msg
  for got, want in zip(shape, shape_template):
    assert want is None or got == want, (
        f'{msg}: {shape} does not match {shape_template}')


def assert_eq(value: Any, expected: Any, value_name: str):
  assert value == expected, f'{value_name}={value}, {expected=}'


def flax_slots_dataclass(cls=None, **kwargs):
  """Mutable slotted dataclass (the reference uses flax.struct.dataclass)."""
  kwargs.setdefault('slots', True)
  if cls is None:
    return functools.partial(dataclasses.dataclass, **kwargs)
  return dataclasses.dataclass(cls, **kwargs)


flax_slots_kw_only_dataclass = functools.partial(
    flax_slots_dataclass, kw_only=True)


def static_field(**kwargs):
  return dataclasses.field(metadata={'pytree_node': False}, **kwargs)


def dynamic_field(**kwargs):
  return dataclasses.field(metadata={'pytree_node': True}, **kwargs)


class QuantMode(enum.Enum):
  TRAIN = 1
  CALIBRATE = 2
  CONVERT = 3
  SERVE = 4


def test_pprint_eq(input_a: Any, input_b: Any,
                   remove_memory_addresses: bool = False):
  sa = input_a if isinstance(input_a, str) else pprint.pformat(input_a)
  sb = input_b if isinstance(input_b, str) else pprint.pformat(input_b)
  if remove_memory_addresses:
    sa = re.sub(r' at 0x.*>', '>', sa, 0, re.MULTILINE)
    sb = re.sub(r' at 0x.*>', '>', sb, 0, re.MULTILINE)
  assert sa == sb, f'first string (actual):\n{sa}'


test_pprint_eq.__test__ = False  # keep pytest from collecting the helper


def infer_dtype_from_bits(bits: int) -> None | DType:
  """Container dtype for an integer bit width (utils.py:120-135)."""
  if bits == 4:
    return int4
  if 2 <= bits <= 8:
    return int8
  return None


def get_remaining_axes(rank: int, contraction_axes: Sequence[AxisIdx],
                       batch_axes: Sequence[AxisIdx]) -> list[int]:
  used = set(contraction_axes) | set(batch_axes)
  return [i for i in range(rank) if i not in used]


@flax_slots_dataclass
class Context:
  """Per-quantizer dynamic state: the PRNG key and the train step."""

  key: Any = dynamic_field()
  train_step: None | int = dynamic_field()
  quant_mode: QuantMode = static_field(default=QuantMode.TRAIN)
