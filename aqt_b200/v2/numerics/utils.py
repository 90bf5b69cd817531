"""bits -> numerics object (reference: aqt/jax/v2/numerics/utils.py:22-48)."""

from aqt_b200.v2 import utils
from aqt_b200.v2.numerics import fp8_numerics
from aqt_b200.v2.numerics import int_numerics
from aqt_b200.v2.numerics import no_numerics


def get_numerics(bits, preserve_max_val=False):
  if bits is None:
    return no_numerics.NoNumerics()
  if bits in fp8_numerics.fp8_map:
    return fp8_numerics.Fp8Numerics(
        exponent_bits=int(bits[1]),
        mantissa_bits=int(bits[3]),
        dtype=fp8_numerics.fp8_map[bits],
    )
  pz = bits != 1
  return int_numerics.IntSymmetric(
      bits=bits,
      preserve_zero=pz,
      preserve_max_val=preserve_max_val,
      clip=True,
      round=True,
      noise_fn=None,
      clip_gradient=False,
      dtype=utils.infer_dtype_from_bits(bits) if pz else None,
  )
