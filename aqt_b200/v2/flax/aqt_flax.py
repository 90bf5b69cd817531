"""AqtDotGeneral / AqtEinsum: the objects a model injects in place of
lax.dot_general / jnp.einsum.

Reference: aqt/jax/v2/flax/aqt_flax.py (AqtDotGeneral :278-570, AqtEinsum
:573-732). The reference classes are flax.linen Modules; flax is not a
dependency here, so these are plain callables with the same constructor
arguments and call signatures:

    dg = AqtDotGeneral(cfg, prng_name='params')
    y = dg(lhs, rhs, dimension_numbers)            # like lax.dot_general
    y = AqtEinsum(cfg)('bthd,bshd->bhts', q, k)    # like jnp.einsum

What the Module machinery provided in the reference and how it maps here:
  * make_rng(prng_name) -> `rngs`: a dict name -> key, or a callable
    name -> key, given at construction or per call; each call consumes one
    fresh sub-key (config.set_context splits it per quantizer).
  * Freezer variables (serving): `rhs_qtensor` / `lhs_qtensor` hold the frozen
    QTensor; CONVERT stores the quantized operand there, SERVE feeds it back
    into the dot instead of re-quantizing (aqt_flax.py:440-512).
"""

from __future__ import annotations

import copy
from typing import Any

from aqt_b200.v2 import aqt_dot_general
from aqt_b200.v2 import config as aqt_config
from aqt_b200.v2 import stochastic_rounding
from aqt_b200.v2 import utils

QuantMode = utils.QuantMode


class _Rngs:
  """name -> stream of keys, the stand-in for flax's make_rng."""

  def __init__(self, rngs):
    self._rngs = rngs
    self._counters = {}

  def make_rng(self, name):
    if self._rngs is None:
      return None
    base = self._rngs(name) if callable(self._rngs) else self._rngs.get(name)
    if base is None:
      return None
    n = self._counters.get(name, 0)
    self._counters[name] = n + 1
    return stochastic_rounding.split(base, n + 2)[n + 1] if n else (
        stochastic_rounding.split(base, 2)[1])


class AqtDotGeneral:
  """A drop-in dot_general with AQT quantization."""

  def __init__(self, cfg: None | aqt_dot_general.DotGeneral = None,
               prng_name: None | str = 'params',
               lhs_quant_mode: QuantMode = QuantMode.TRAIN,
               rhs_quant_mode: QuantMode = QuantMode.TRAIN,
               rngs: Any = None, name: str = 'AqtDotGeneral'):
    self.cfg = cfg
    self.prng_name = prng_name
    self.lhs_quant_mode = lhs_quant_mode
    self.rhs_quant_mode = rhs_quant_mode
    self.name = name
    self._rngs = _Rngs(rngs)
    # Frozen operands (the 'aqt' variable collection of the reference).
    self.lhs_qtensor = None
    self.rhs_qtensor = None

  def make_aqt_dg(self, lhs_shape, rhs_shape, dimension_numbers):
    """Returns the callable for these shapes (reference :326-514)."""
    del lhs_shape, rhs_shape
    if self.cfg is None:
      return aqt_dot_general.lax_dot_general
    cfg = copy.deepcopy(self.cfg)
    key = self._rngs.make_rng(self.prng_name) if self.prng_name else None
    cfg = aqt_config.set_context(cfg, key, train_step=None,
                                 lhs_quant_mode=self.lhs_quant_mode,
                                 rhs_quant_mode=self.rhs_quant_mode)

    def ret_dg(lhs, rhs, dimension_numbers=dimension_numbers, precision=None,
               preferred_element_type=None):
      del preferred_element_type
      assert precision is None, (
          f'Precision {precision} requested together with quantization.')
      msg = 'AQT is not yet optimized to accept quantized types directly. '
      msg += f'lhs.dtype: {lhs.dtype}, rhs.dtype: {rhs.dtype}'
      floats = (utils.bfloat16, utils.float32, utils.float16)
      assert utils.as_dtype(lhs.dtype) in floats, msg
      assert utils.as_dtype(rhs.dtype) in floats, msg
      lhs_qt = self.lhs_qtensor if self.lhs_quant_mode == QuantMode.SERVE else None
      rhs_qt = self.rhs_qtensor if self.rhs_quant_mode == QuantMode.SERVE else None
      if self.lhs_quant_mode == QuantMode.SERVE:
        assert lhs_qt is not None, 'SERVE mode without a frozen lhs QTensor'
      if self.rhs_quant_mode == QuantMode.SERVE:
        assert rhs_qt is not None, 'SERVE mode without a frozen rhs QTensor'
      out, (out_lhs_qt, out_rhs_qt) = cfg.dg_core(
          lhs=lhs, rhs=rhs, lhs_qt=lhs_qt, rhs_qt=rhs_qt,
          dimension_numbers=dimension_numbers)
      if self.lhs_quant_mode == QuantMode.CONVERT:
        self.lhs_qtensor = out_lhs_qt
      if self.rhs_quant_mode == QuantMode.CONVERT:
        self.rhs_qtensor = out_rhs_qt
      return out

    return ret_dg

  def __call__(self, lhs, rhs, dimension_numbers, precision=None,
               preferred_element_type=None):
    aqt_dg = self.make_aqt_dg(lhs.shape, rhs.shape, dimension_numbers)
    return aqt_dg(lhs, rhs, dimension_numbers, precision,
                  preferred_element_type=preferred_element_type)


class AqtEinsum:
  """A drop-in two-operand einsum with AQT quantization (reference :573-732).

  When the einsum lowers to a dot_general whose operand order is swapped
  relative to the arguments, the lhs/rhs roles of the config are swapped too,
  so that "lhs" options keep applying to the first einsum argument.
  """

  def __init__(self, cfg: None | aqt_dot_general.DotGeneral = None,
               prng_name: None | str = 'params',
               lhs_quant_mode: QuantMode = QuantMode.TRAIN,
               rhs_quant_mode: QuantMode = QuantMode.TRAIN,
               rngs: Any = None, name: str = 'AqtEinsum'):
    self.cfg = cfg
    self.prng_name = prng_name
    self.lhs_quant_mode = lhs_quant_mode
    self.rhs_quant_mode = rhs_quant_mode
    self.rngs = rngs
    self.name = name
    # One inner AqtDotGeneral per operand order, built on first use and kept:
    # it owns the frozen QTensors of CONVERT/SERVE and the position in the rng
    # stream, both of which must survive from one call to the next.
    self._dgs = {}

  def _inner(self, swap: bool) -> AqtDotGeneral:
    if swap not in self._dgs:
      cfg = copy.deepcopy(self.cfg)
      lhs_mode, rhs_mode = self.lhs_quant_mode, self.rhs_quant_mode
      if cfg is not None and swap:
        # reference :684-704
        cfg.fwd.dg_quantizer.swap_lhs_and_rhs()
        cfg.fwd.lhs, cfg.fwd.rhs = cfg.fwd.rhs, cfg.fwd.lhs
        cfg.dlhs, cfg.drhs = cfg.drhs, cfg.dlhs
        lhs_mode, rhs_mode = rhs_mode, lhs_mode
      self._dgs[swap] = AqtDotGeneral(cfg, prng_name=self.prng_name,
                                      lhs_quant_mode=lhs_mode,
                                      rhs_quant_mode=rhs_mode, rngs=self.rngs,
                                      name=self.name)
    return self._dgs[swap]

  def _frozen(self, which: str):
    """Frozen QTensor of the FIRST (`lhs`) or SECOND (`rhs`) einsum argument,
    wherever the operand order put it."""
    for swap, dg in self._dgs.items():
      attr = ('rhs' if which == 'lhs' else 'lhs') if swap else which
      qt = getattr(dg, attr + '_qtensor')
      if qt is not None:
        return qt
    return getattr(self, '_pending_' + which, None)

  def _set_frozen(self, which: str, qt):
    setattr(self, '_pending_' + which, qt)
    for swap, dg in self._dgs.items():
      attr = ('rhs' if which == 'lhs' else 'lhs') if swap else which
      setattr(dg, attr + '_qtensor', qt)

  lhs_qtensor = property(lambda self: self._frozen('lhs'),
                         lambda self, qt: self._set_frozen('lhs', qt))
  rhs_qtensor = property(lambda self: self._frozen('rhs'),
                         lambda self, qt: self._set_frozen('rhs', qt))

  def __call__(self, eqn, lhs_g, rhs_g):
    _, _, swap = aqt_dot_general.einsum_to_dot_general(eqn, lhs_g.ndim,
                                                       rhs_g.ndim)
    new = swap not in self._dgs
    dg = self._inner(swap)
    if new:  # frozen tensors assigned before the first call
      for which in ('lhs', 'rhs'):
        qt = getattr(self, '_pending_' + which, None)
        if qt is not None:
          attr = ('rhs' if which == 'lhs' else 'lhs') if swap else which
          setattr(dg, attr + '_qtensor', qt)
    return aqt_dot_general.einsum(eqn, lhs_g, rhs_g, dg)
