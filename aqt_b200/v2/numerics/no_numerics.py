"""Pass-through numerics (reference: aqt/jax/v2/numerics/no_numerics.py:22-43)."""

from typing import Any

from aqt_b200.v2 import utils
from aqt_b200.v2.numerics import numerics


@utils.flax_slots_kw_only_dataclass
class NoNumerics(numerics.AqtNumerics):
  """No quantization: the operand stays in its float type."""

  # noise_fn has no effect here; the field exists because config setters
  # assign it uniformly to every numerics object.
  noise_fn: Any = None
  dtype: None | Any = None

  def get_dtype(self):
    return None

  def get_quant_bound(self):
    pass

  def vjp_fwd(self, x, context):
    pass

  def vjp_bwd(self, res, grad):
    pass
