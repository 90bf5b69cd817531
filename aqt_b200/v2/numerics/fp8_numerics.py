"""fp8 numerics (reference: aqt/jax/v2/numerics/fp8_numerics.py:67-145)."""

from typing import Any

from aqt_b200.v2 import utils
from aqt_b200.v2.numerics import numerics

FP8Dtype = str  # 'e4m3' | 'e5m2'
fp8_map = {'e4m3': utils.float8_e4m3fn, 'e5m2': utils.float8_e5m2}
# Largest finite value of each format; both are exactly representable in bf16,
# which is the type the reference holds the bound in (fp8_numerics.py:79-80).
fp8_max = {'float8_e4m3fn': 448.0, 'float8_e5m2': 57344.0}


def _convert_to_fp8dtype(dtype) -> None | FP8Dtype:
  dtype = utils.as_dtype(dtype)
  if dtype == utils.float8_e4m3fn:
    return 'e4m3'
  if dtype == utils.float8_e5m2:
    return 'e5m2'
  return None


@utils.flax_slots_kw_only_dataclass
class Fp8Numerics(numerics.AqtNumerics):
  """e4m3fn / e5m2 storage, round-to-nearest-even, saturating clip."""

  dtype: Any
  exponent_bits: int = 4
  mantissa_bits: int = 3
  stochastic_rounding: bool = utils.static_field(default=False)

  def _get_edge_of_last_fp8_bucket(self):
    return fp8_max[utils.as_dtype(self.dtype).name]

  def get_dtype(self):
    return self.dtype

  def get_quant_bound(self):
    return self._get_edge_of_last_fp8_bucket()

  def check(self):
    dt = utils.as_dtype(self.dtype)
    if dt == utils.float8_e4m3fn:
      assert (self.exponent_bits, self.mantissa_bits) == (4, 3)
    elif dt == utils.float8_e5m2:
      assert (self.exponent_bits, self.mantissa_bits) == (5, 2)
    else:
      assert False, f'Unsupported dtype: {self.dtype}'
    if self.stochastic_rounding:
      raise NotImplementedError(
          'fp8 mantissa-noise stochastic rounding draws raw jax.random bits '
          '(fp8_numerics.py:36-64); it is not part of the sm_100a path.')

  def vjp_fwd(self, x, context):
    from aqt_b200 import engine
    self.check()
    return engine.apply_numerics(x, self, None), (x,)

  def vjp_bwd(self, res, grad):
    del res
    return (grad, None)
