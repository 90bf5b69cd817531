"""Where a per-channel scale lands after a dot_general.

Reference: aqt/jax/v2/transpose.py:98-285. The reference physically reshapes
and transposes scale arrays; the kernels here read scales through strides, so
these helpers work on *views* (torch tensors or numpy arrays, anything with
reshape/permute semantics through the small adapter below) and never copy.
Axis-name shorthand: ca contraction axes, ba batch axes, ra remaining axes.
Output axis order of a dot_general is: batch..., lhs_ra..., rhs_ra...
"""

from typing import Sequence

from aqt_b200.v2 import utils


def _permute(t, axes):
  axes = list(axes)
  if hasattr(t, 'permute'):
    return t.permute(*axes) if axes else t
  return t.transpose(axes)


def _unsqueeze_many(t, axes):
  shape = list(t.shape)
  for ax in sorted(axes):
    shape.insert(ax, 1)
  return t.reshape(shape)


def _scale_trans(x, ca, ba):
  """[x's axes] -> [ba..., ra...] (contraction axes, all of size 1, dropped)."""
  ca, ba = list(ca), list(ba)
  for i in ca:
    assert x.shape[i] == 1, (tuple(x.shape), ca, ba)
  ra = utils.get_remaining_axes(x.ndim, ca, ba)
  x = _permute(x, ba + ra + ca)
  return x.reshape(list(x.shape[:len(ba) + len(ra)]))


def lhs_scale_transpose_to_output(lhs_scale, dimension_numbers, lhs_shape,
                                  rhs_shape):
  if lhs_scale is None:
    return None
  (lhs_ca, rhs_ca), (lhs_ba, rhs_ba) = dimension_numbers
  s = _scale_trans(lhs_scale, lhs_ca, lhs_ba)
  assert s.ndim == len(lhs_shape) - len(lhs_ca)
  n_rhs_ra = len(rhs_shape) - len(rhs_ca) - len(rhs_ba)
  return _unsqueeze_many(s, range(s.ndim, s.ndim + n_rhs_ra))


def rhs_scale_transpose_to_output(rhs_scale, dimension_numbers, lhs_shape,
                                  rhs_shape):
  if rhs_scale is None:
    return None
  del rhs_shape
  (lhs_ca, rhs_ca), (lhs_ba, rhs_ba) = dimension_numbers
  s = _scale_trans(rhs_scale, rhs_ca, rhs_ba)
  n_lhs_ra = len(lhs_shape) - len(lhs_ca) - len(lhs_ba)
  start = len(rhs_ba)
  return _unsqueeze_many(s, range(start, start + n_lhs_ra))


def _scale_trans_back(scale_t, ca: Sequence[int], ba: Sequence[int]):
  ca, ba = list(ca), list(ba)
  scale = _unsqueeze_many(scale_t, range(scale_t.ndim, scale_t.ndim + len(ca)))
  ra = utils.get_remaining_axes(scale.ndim, ca, ba)
  back = [-1] * scale.ndim
  for orig, moved in enumerate(ba + ra + ca):
    back[moved] = orig
  assert -1 not in back
  return _permute(scale, back)


def lhs_recover_scale_from_scale_t(lhs_scale_t, dimension_numbers, lhs_shape,
                                   rhs_shape):
  (lhs_ca, rhs_ca), (lhs_ba, rhs_ba) = dimension_numbers
  start = len(lhs_shape) - len(lhs_ca)
  shape = list(lhs_scale_t.shape)[:start]
  return _scale_trans_back(lhs_scale_t.reshape(shape), lhs_ca, lhs_ba)


def rhs_recover_scale_from_scale_t(rhs_scale_t, dimension_numbers, lhs_shape,
                                   rhs_shape):
  del rhs_shape
  (lhs_ca, rhs_ca), (lhs_ba, rhs_ba) = dimension_numbers
  start = len(rhs_ba)
  n = len(lhs_shape) - len(lhs_ca) - len(lhs_ba)
  shape = list(rhs_scale_t.shape)
  del shape[start:start + n]
  return _scale_trans_back(rhs_scale_t.reshape(shape), rhs_ca, rhs_ba)


def _scale_trans_for_other_input(x, my_ca, my_ba, other_ca, other_ba,
                                 other_rank: int):
  """Lays a scale of one operand out along the matching axes of the other."""
  my_ca, my_ba = list(my_ca), list(my_ba)
  other_ca, other_ba = list(other_ca), list(other_ba)
  if x.ndim < other_rank:
    x = x.reshape(list(x.shape) + [1] * (other_rank - x.ndim))
  perm = [-1] * x.ndim
  my_ra = utils.get_remaining_axes(x.ndim, my_ca, my_ba)
  for ax in my_ra:
    assert x.shape[ax] == 1
  for mine, theirs in zip(my_ca + my_ba, other_ca + other_ba):
    perm[theirs] = mine
  spare = iter(my_ra)
  perm = [next(spare) if p == -1 else p for p in perm]
  assert next(spare, None) is None
  x = _permute(x, perm)
  if x.ndim > other_rank:
    assert all(n == 1 for n in x.shape[other_rank:])
    x = x.reshape(list(x.shape[:other_rank]))
  return x


def lhs_scale_transpose_for_rhs_input(lhs_scale, dimension_numbers, rhs_shape):
  if lhs_scale is None:
    return None
  (lhs_ca, rhs_ca), (lhs_ba, rhs_ba) = dimension_numbers
  return _scale_trans_for_other_input(lhs_scale, lhs_ca, lhs_ba, rhs_ca,
                                      rhs_ba, len(rhs_shape))


def rhs_scale_transpose_for_lhs_input(rhs_scale, dimension_numbers, lhs_shape):
  if rhs_scale is None:
    return None
  (lhs_ca, rhs_ca), (lhs_ba, rhs_ba) = dimension_numbers
  return _scale_trans_for_other_input(rhs_scale, rhs_ca, rhs_ba, lhs_ca,
                                      lhs_ba, len(lhs_shape))
