"""Symmetric integer numerics (reference: aqt/jax/v2/numerics/int_numerics.py:24-125).

Bound table the methods below implement (8 bit / 2 bit / 1 bit):
  preserve_zero=F preserve_max_val=F : 128.0 2.0 1.0
  preserve_zero=F preserve_max_val=T : 127.5 1.5 0.5
  preserve_zero=T preserve_max_val=F : 127.5 1.5 0.5
  preserve_zero=T preserve_max_val=T : 127.0 1.0 0.0
"""

from typing import Any

from aqt_b200.v2 import utils
from aqt_b200.v2.numerics import numerics


@utils.flax_slots_kw_only_dataclass
class IntSymmetric(numerics.AqtNumerics):
  """sint8 / sint4 / ... symmetric around zero."""

  bits: int
  preserve_zero: bool
  preserve_max_val: bool
  clip: bool
  clip_gradient: bool
  round: bool
  noise_fn: Any
  dtype: None | Any = None

  def get_edge_of_last_int_bucket(self):
    edge = 2.0 ** (self.bits - 1)
    return edge - 0.5 if self.preserve_zero else edge

  def get_center_of_last_int_bucket(self):
    return self.get_edge_of_last_int_bucket() - 0.5

  def get_quant_bound(self):
    if self.preserve_max_val:
      return self.get_center_of_last_int_bucket()
    return self.get_edge_of_last_int_bucket()

  def _get_fwd_clip_bound(self):
    # When rounding follows the clip, pull the bound in by half a bucket so the
    # edge value cannot round into a bucket that does not exist.
    bound = self.get_edge_of_last_int_bucket()
    return bound - 0.5 if self.round else bound

  def get_dtype(self):
    return self.dtype

  def vjp_fwd(self, x, context):
    """noise -> clip -> round -> cast, on the device (int_numerics.py:81-111)."""
    from aqt_b200 import engine  # deferred: config objects need no GPU
    assert self.bits <= 22, 'Too many bits, float32 has less precision.'
    noise = None
    if self.noise_fn:
      assert context.key is not None, (
          'noise_fn is set, requestic stochastic rounding, but RNG was not '
          'passed in Context.key')
      noise = self.noise_fn(tuple(x.shape), context.key)
    return engine.apply_numerics(x, self, noise), (x,)

  def vjp_bwd(self, res, grad):
    ret = grad
    if self.clip_gradient:
      (x,) = res
      b = self._get_fwd_clip_bound()
      ret = ret * ((-b <= x) & (x <= b)).to(ret.dtype)
    return (ret, None)
