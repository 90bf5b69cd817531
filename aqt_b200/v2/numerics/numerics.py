"""Abstract numerics interface (reference: aqt/jax/v2/numerics/numerics.py:20-54)."""

import abc

from aqt_b200.v2 import utils


@utils.flax_slots_kw_only_dataclass
class AqtNumerics(abc.ABC):
  """What a quantizer needs to know about a number format."""

  @abc.abstractmethod
  def get_dtype(self):
    pass

  @abc.abstractmethod
  def get_quant_bound(self):
    pass

  @abc.abstractmethod
  def vjp_fwd(self, x, context):
    pass

  @abc.abstractmethod
  def vjp_bwd(self, res, grad):
    pass
