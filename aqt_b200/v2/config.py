"""Configuration builders and setters for quantized dot_general.

Same public names and semantics as the reference's aqt/jax/v2/config.py
(set_context :66-90, set_numerics :117-139, set_stochastic_rounding :171-225,
set_use_fwd_quant :268-287, set_bits :463-516, default_unquantized_config
:555-595, fully_quantized :598-658, config_v3 :661-721, config_v4 :724-788,
config_fwd_fp8 :791-809). Everything here is host-side Python that builds and
mutates the dataclasses of aqt_dot_general / aqt_quantizer; no device work.
"""

from __future__ import annotations

import copy
import functools
from typing import Sequence

from aqt_b200.v2 import aqt_dot_general
from aqt_b200.v2 import aqt_quantizer
from aqt_b200.v2 import calibration
from aqt_b200.v2 import stochastic_rounding
from aqt_b200.v2 import utils
from aqt_b200.v2.numerics import fp8_numerics
from aqt_b200.v2.numerics import int_numerics
from aqt_b200.v2.numerics import no_numerics
from aqt_b200.v2.numerics import numerics
from aqt_b200.v2.numerics import utils as numerics_utils

# Re-exported under the reference's names.
CalibrationMode = aqt_dot_general.CalibrationMode
DequantMode = aqt_dot_general.DequantMode
DotGeneral = aqt_dot_general.DotGeneral
DotGeneralRaw = aqt_dot_general.DotGeneralRaw
LocalAqt = aqt_dot_general.LocalAqt
Tensor = aqt_dot_general.Tensor
dot_general_make = aqt_dot_general.dot_general_make
dot_general_raw_make = aqt_dot_general.dot_general_raw_make
dtypes_allowed_for_int32_accum = aqt_dot_general.dtypes_allowed_for_int32_accum
quantizer_make = aqt_quantizer.quantizer_make

# Passing SKIP to a set_xyz argument leaves that option untouched.
SKIP = 'skip'

_DefaultQ = aqt_dot_general.DefaultDotGeneralQuantizer


def _raws(cfg: DotGeneral):
  return (cfg.fwd, cfg.dlhs, cfg.drhs)


def _assert_default_quantizers(cfg: DotGeneral):
  for raw in _raws(cfg):
    assert isinstance(raw.dg_quantizer, _DefaultQ)


def _split_key(key, num_splits: int):
  if key is None:
    return (None,) * num_splits
  return stochastic_rounding.split(key, num_splits)


def set_context(cfg: DotGeneral, key, train_step: None | int,
                lhs_quant_mode: utils.QuantMode = utils.QuantMode.TRAIN,
                rhs_quant_mode: utils.QuantMode = utils.QuantMode.TRAIN):
  """Returns a deep copy of cfg with one sub-key per quantizer.

  key -> (fwd, dlhs, drhs) -> (lhs, rhs) for each, as in the reference.
  """
  ret = copy.deepcopy(cfg)
  for raw, raw_key in zip(_raws(ret), _split_key(key, 3)):
    k_lhs, k_rhs = _split_key(raw_key, 2)
    raw.dg_quantizer.set_context(
        utils.Context(key=k_lhs, train_step=train_step,
                      quant_mode=lhs_quant_mode),
        utils.Context(key=k_rhs, train_step=train_step,
                      quant_mode=rhs_quant_mode))
  return ret


def set_fwd_dequant_mode(cfg: DotGeneral, *, lhs_dequant_mode=None,
                         rhs_dequant_mode=None):
  if lhs_dequant_mode is not None:
    cfg.fwd.lhs.dequant_mode = lhs_dequant_mode
  if rhs_dequant_mode is not None:
    cfg.fwd.rhs.dequant_mode = rhs_dequant_mode


def set_fwd_calibration_mode(cfg: DotGeneral, *, lhs_calibration_mode=SKIP,
                             rhs_calibration_mode=SKIP):
  if lhs_calibration_mode != SKIP:
    cfg.fwd.lhs.calibration_mode = lhs_calibration_mode
  if rhs_calibration_mode != SKIP:
    cfg.fwd.rhs.calibration_mode = rhs_calibration_mode


def set_numerics(cfg: DotGeneralRaw, lhs_numerics: numerics.AqtNumerics,
                 rhs_numerics: numerics.AqtNumerics):
  """Installs numerics on both sides and derives the accumulator dtype."""
  assert isinstance(cfg.dg_quantizer, _DefaultQ)
  cfg.dg_quantizer.lhs.numerics = lhs_numerics
  cfg.dg_quantizer.rhs.numerics = rhs_numerics
  ld, rd = lhs_numerics.get_dtype(), rhs_numerics.get_dtype()
  fp8s = list(fp8_numerics.fp8_map.values())
  if (ld in dtypes_allowed_for_int32_accum
      and rd in dtypes_allowed_for_int32_accum):
    cfg.dg_accumulator_dtype = utils.int32
  elif ld in fp8s or rd in fp8s:
    cfg.dg_accumulator_dtype = utils.float32
  else:
    cfg.dg_accumulator_dtype = None


def set_accumulator_dtype(cfg: DotGeneral, fwd_dtype, dlhs_dtype, drhs_dtype):
  for raw, dt in zip(_raws(cfg), (fwd_dtype, dlhs_dtype, drhs_dtype)):
    if dt != SKIP:
      raw.dg_accumulator_dtype = dt


def set_stochastic_rounding(cfg: DotGeneral, vjp_lhs_stochastic_rounding: bool,
                            vjp_rhs_stochastic_rounding: bool,
                            implementation: str,
                            noise_sharing_axes: Sequence[int] = ()):
  """Chooses the noise source of both gradient dots.

  vjp_lhs_* is the gradient operand of dlhs/drhs, vjp_rhs_* the saved
  activation / weight operand. fp8 numerics flip their own
  `stochastic_rounding` flag instead of receiving a noise_fn.
  """
  impls = {
      'jax.uniform': stochastic_rounding.JaxUniform(),
      'custom-1': stochastic_rounding.RandomCenteredUniform(),
  }
  assert implementation in impls, f'{implementation} not supported.'
  noise_fn = impls[implementation]
  if noise_sharing_axes:
    noise_fn = functools.partial(noise_fn,
                                 noise_sharing_axes=noise_sharing_axes)
  assert isinstance(cfg.dlhs.dg_quantizer, _DefaultQ)
  assert isinstance(cfg.drhs.dg_quantizer, _DefaultQ)
  for raw in (cfg.dlhs, cfg.drhs):
    for quantizer, is_sr in ((raw.dg_quantizer.lhs,
                              vjp_lhs_stochastic_rounding),
                             (raw.dg_quantizer.rhs,
                              vjp_rhs_stochastic_rounding)):
      if isinstance(quantizer.numerics, fp8_numerics.Fp8Numerics):
        quantizer.numerics.stochastic_rounding = is_sr
      else:
        quantizer.numerics.noise_fn = noise_fn if is_sr else None


def _each_quantizer(cfg: DotGeneral):
  for raw in _raws(cfg):
    yield raw.dg_quantizer.lhs
    yield raw.dg_quantizer.rhs


def set_constant_calibration(cfg: DotGeneral, bound: float = 1.0, bias=None):
  """Reference: config.py:142-168. Constant bounds are not among the
  calibrations the sm_100a kernels implement (AbsMax and delayed scaling
  are), so the request is refused here, when the configuration is built,
  rather than at the first dot."""
  del cfg, bound, bias
  raise NotImplementedError(
      'ConstantCalibration (set_constant_calibration, use_dummy_static_bound) '
      'is outside the sm_100a hot path; use AbsMaxCalibration or '
      'DelayedScalingCalibration')


def set_local_aqt(cfg: DotGeneral, fwd_local_aqt, dlhs_local_aqt,
                  drhs_local_aqt):
  for raw, la in zip(_raws(cfg),
                     (fwd_local_aqt, dlhs_local_aqt, drhs_local_aqt)):
    if la != SKIP:
      raw.local_aqt = la


def set_use_fwd_quant(cfg: DotGeneral, dlhs_use_fwd_quant, drhs_use_fwd_quant):
  """Lets the gradient dots reuse the forward pass's quantized operands."""
  msg = 'use_fwd_quant is incompatible with use_mid_quant right now.'
  for raw in _raws(cfg):
    assert raw.dg_quantizer.lhs_mid_alpha is None, msg
    assert raw.dg_quantizer.rhs_mid_alpha is None, msg
  if dlhs_use_fwd_quant != SKIP:
    cfg.dlhs.rhs.use_fwd_quant = dlhs_use_fwd_quant
  if drhs_use_fwd_quant != SKIP:
    cfg.drhs.rhs.use_fwd_quant = drhs_use_fwd_quant


@utils.flax_slots_kw_only_dataclass
class _MidNumerics(numerics.AqtNumerics):
  """Identity numerics with bound 1, used by mid-scale calibration."""

  def get_quant_bound(self):
    return 1.0

  def get_dtype(self):
    assert False, 'Should not request dtype for mid-quantization.'

  def vjp_fwd(self, x, context):
    return x, ()

  def vjp_bwd(self, res, grad):
    assert res == ()
    return grad


def set_use_mid_quant(cfg: DotGeneral, fwd_mid_alpha_both, dlhs_mid_alpha_both,
                      drhs_mid_alpha_both):
  """Configures SmoothQuant/AWQ-style mid scales (configuration only here)."""
  _assert_default_quantizers(cfg)
  # Checked even when every alpha is SKIP, as the reference does (:304-306).
  msg = 'use_fwd_quant is incompatible with use_mid_quant right now.'
  assert not cfg.dlhs.rhs.use_fwd_quant, msg
  assert not cfg.drhs.rhs.use_fwd_quant, msg
  for raw, alpha in zip(_raws(cfg), (fwd_mid_alpha_both, dlhs_mid_alpha_both,
                                     drhs_mid_alpha_both)):
    if alpha == SKIP:
      continue
    q = raw.dg_quantizer
    for mid in (q.lhs_mid, q.rhs_mid):
      mid.numerics = _MidNumerics()
      mid.calibration = calibration.AbsMaxCalibration
    q.lhs_mid_alpha = alpha
    q.rhs_mid_alpha = alpha


def set_int_numerics_preserve_zero(cfg: DotGeneral, preserve_zero: bool):
  _assert_default_quantizers(cfg)
  for quantizer in _each_quantizer(cfg):
    n = quantizer.numerics
    if isinstance(n, int_numerics.IntSymmetric):
      n.preserve_zero = preserve_zero
      n.dtype = utils.infer_dtype_from_bits(n.bits) if preserve_zero else None


def _rewrap_calibration(quantizer, expect_cls=None, **updates):
  """Re-wraps quantizer.calibration as a partial carrying extra keywords."""
  cls = quantizer.calibration
  if cls is None:
    return False
  keywords = {}
  if isinstance(cls, functools.partial):
    keywords = dict(cls.keywords)
    cls = cls.func
  if expect_cls is not None:
    assert cls == expect_cls, (
        f'only available in {expect_cls.__name__}, while '
        f'{quantizer.calibration} is used in current config.')
  keywords.update(updates)
  quantizer.calibration = functools.partial(cls, **keywords)
  return True


def set_absmax_calib_scale(cfg: DotGeneral, scale: float):
  """clipping_scale on every AbsMax quantizer; <1 also turns on clip_gradient."""
  _assert_default_quantizers(cfg)
  for quantizer in _each_quantizer(cfg):
    if not _rewrap_calibration(quantizer, calibration.AbsMaxCalibration,
                               clipping_scale=scale):
      continue
    if scale < 1.0 and isinstance(quantizer.numerics,
                                  int_numerics.IntSymmetric):
      quantizer.numerics.clip_gradient = True


def set_scale_and_bias_dtype(cfg: DotGeneral, dtype):
  _assert_default_quantizers(cfg)
  for quantizer in _each_quantizer(cfg):
    _rewrap_calibration(quantizer, dtype=dtype)


def set_bits(cfg: DotGeneral, fwd_lhs_bit, fwd_rhs_bit, dlhs_lhs_bit,
             dlhs_rhs_bit, drhs_lhs_bit, drhs_rhs_bit) -> DotGeneral:
  """Sets numerics per operand; quantized operands get AbsMaxCalibration."""
  for raw, (lb, rb) in zip(_raws(cfg), ((fwd_lhs_bit, fwd_rhs_bit),
                                        (dlhs_lhs_bit, dlhs_rhs_bit),
                                        (drhs_lhs_bit, drhs_rhs_bit))):
    set_numerics(raw, numerics_utils.get_numerics(lb),
                 numerics_utils.get_numerics(rb))
    if lb is not None:
      raw.dg_quantizer.lhs.calibration = calibration.AbsMaxCalibration
    if rb is not None:
      raw.dg_quantizer.rhs.calibration = calibration.AbsMaxCalibration
  # A quantized forward operand makes use_fwd_quant meaningful; default False.
  set_use_fwd_quant(cfg,
                    False if fwd_rhs_bit is not None else SKIP,
                    False if fwd_lhs_bit is not None else SKIP)
  return cfg


def set_fwd_calibration(cfg: DotGeneral, calibration_factory) -> DotGeneral:
  assert isinstance(cfg.fwd.dg_quantizer, _DefaultQ)
  cfg.fwd.dg_quantizer.lhs.calibration = calibration_factory
  cfg.fwd.dg_quantizer.rhs.calibration = calibration_factory
  return cfg


################################################################################
# Config creators.


def default_unquantized_config() -> DotGeneral:
  """Float dot_general: NoNumerics everywhere, no calibration."""
  def tensor_cfg():
    return Tensor(use_fwd_quant=False, dequant_mode=DequantMode.OUTPUT,
                  calibration_mode=CalibrationMode.CONTRACTING_AXIS)

  def quantizer():
    return aqt_quantizer.Quantizer(
        numerics=no_numerics.NoNumerics(), calib_shared_axes=None,
        scale_stop_grad=True, calibration=None,
        context=utils.Context(key=None, train_step=None))

  def raw(name):
    return DotGeneralRaw(
        lhs=tensor_cfg(), rhs=tensor_cfg(),
        dg_quantizer=_DefaultQ(lhs=quantizer(), rhs=quantizer(),
                               lhs_mid=quantizer(), rhs_mid=quantizer()),
        dg_accumulator_dtype=None, local_aqt=None, jax_scope_name=name)

  return DotGeneral(fwd=raw('aqt_fwd'), dlhs=raw('aqt_dlhs'),
                    drhs=raw('aqt_drhs'))


def fully_quantized(*, fwd_bits=8, bwd_bits=8, use_fwd_quant: bool = True,
                    use_stochastic_rounding: None | bool = True,
                    vjp_lhs_stochastic_rounding: None | bool = None,
                    vjp_rhs_stochastic_rounding: None | bool = None,
                    use_dummy_static_bound: bool = False,
                    dlhs_local_aqt=None, drhs_local_aqt=None) -> DotGeneral:
  """Forward and both gradients quantized.

  Stochastic rounding is configured either old-style (use_stochastic_rounding,
  applied to both operands of both gradient dots) or new-style (the two vjp_*
  flags, which must then both be given and use_stochastic_rounding be None).
  """
  cfg = dot_general_make(lhs_bits=fwd_bits, rhs_bits=fwd_bits,
                         bwd_bits=bwd_bits, use_fwd_quant=use_fwd_quant,
                         dlhs_local_aqt=dlhs_local_aqt,
                         drhs_local_aqt=drhs_local_aqt)
  old_style = use_stochastic_rounding is not None
  new_lhs = vjp_lhs_stochastic_rounding is not None
  new_rhs = vjp_rhs_stochastic_rounding is not None
  assert new_lhs == new_rhs, (
      'if you use new style SR config (vjp_xhs_stochastic_rounding), do pass'
      ' both lhs and rhs explicitely.')
  assert new_lhs != old_style
  assert not (vjp_lhs_stochastic_rounding and vjp_rhs_stochastic_rounding), (
      'This config is buggy when you set both to True. Contact lew@ or use'
      ' config_v3')
  if use_stochastic_rounding is True:
    set_stochastic_rounding(cfg, True, True, 'jax.uniform')
  if vjp_lhs_stochastic_rounding is True:
    set_stochastic_rounding(cfg, True, False, 'jax.uniform')
  if vjp_rhs_stochastic_rounding is True:
    set_stochastic_rounding(cfg, False, True, 'jax.uniform')
  if use_dummy_static_bound:
    set_constant_calibration(cfg, 1.0)
  assert cfg.fwd.local_aqt is None, 'local_aqt is not yet supported in fwd.'
  return cfg


def config_v3(*, fwd_bits=8, dlhs_bits=8, drhs_bits=None,
              use_dummy_static_bound: bool = False,
              rng_type: str = 'jax.uniform', dlhs_local_aqt=None,
              drhs_local_aqt=None, fwd_accumulator_dtype=utils.int32,
              dlhs_accumulator_dtype=utils.int32,
              drhs_accumulator_dtype=None) -> DotGeneral:
  """fwd + dlhs int8, drhs float by default; SR on the gradient operand only."""
  mk = functools.partial(dot_general_raw_make, initialize_calibration=False)
  cfg = DotGeneral(
      fwd=mk(fwd_bits, fwd_bits, jax_scope_name='aqt_fwd'),
      dlhs=mk(dlhs_bits, dlhs_bits, local_aqt=dlhs_local_aqt,
              jax_scope_name='aqt_dlhs'),
      drhs=mk(drhs_bits, drhs_bits, local_aqt=drhs_local_aqt,
              jax_scope_name='aqt_drhs'))
  cfg.dlhs.rhs.use_fwd_quant = False
  cfg.drhs.rhs.use_fwd_quant = False
  set_stochastic_rounding(cfg, vjp_lhs_stochastic_rounding=True,
                          vjp_rhs_stochastic_rounding=False,
                          implementation=rng_type)
  if use_dummy_static_bound:
    set_constant_calibration(cfg, 1.0)
  set_accumulator_dtype(cfg, fwd_dtype=fwd_accumulator_dtype,
                        dlhs_dtype=dlhs_accumulator_dtype,
                        drhs_dtype=drhs_accumulator_dtype)
  assert cfg.fwd.local_aqt is None, 'local_aqt is not yet supported in fwd.'
  return cfg


def config_v4(*, fwd_bits=8, dlhs_bits=8, drhs_bits=None,
              use_dummy_static_bound: bool = False,
              rng_type: str = 'jax.uniform', dlhs_local_aqt=None,
              drhs_local_aqt=None, fwd_accumulator_dtype=SKIP,
              dlhs_accumulator_dtype=SKIP, drhs_accumulator_dtype=SKIP,
              dlhs_use_fwd_quant=SKIP, drhs_use_fwd_quant=SKIP,
              fwd_mid_alpha_both=SKIP, dlhs_mid_alpha_both=SKIP,
              drhs_mid_alpha_both=SKIP) -> DotGeneral:
  """Built by applying setters to default_unquantized_config()."""
  cfg = default_unquantized_config()
  set_bits(cfg, fwd_lhs_bit=fwd_bits, fwd_rhs_bit=fwd_bits,
           dlhs_lhs_bit=dlhs_bits, dlhs_rhs_bit=dlhs_bits,
           drhs_lhs_bit=drhs_bits, drhs_rhs_bit=drhs_bits)
  set_accumulator_dtype(cfg, fwd_dtype=fwd_accumulator_dtype,
                        dlhs_dtype=dlhs_accumulator_dtype,
                        drhs_dtype=drhs_accumulator_dtype)
  set_stochastic_rounding(cfg, vjp_lhs_stochastic_rounding=True,
                          vjp_rhs_stochastic_rounding=False,
                          implementation=rng_type)
  if use_dummy_static_bound:
    set_constant_calibration(cfg, 1.0)
  set_local_aqt(cfg, fwd_local_aqt=SKIP, dlhs_local_aqt=dlhs_local_aqt,
                drhs_local_aqt=drhs_local_aqt)
  set_use_fwd_quant(cfg, dlhs_use_fwd_quant=dlhs_use_fwd_quant,
                    drhs_use_fwd_quant=drhs_use_fwd_quant)
  set_use_mid_quant(cfg, fwd_mid_alpha_both=fwd_mid_alpha_both,
                    dlhs_mid_alpha_both=dlhs_mid_alpha_both,
                    drhs_mid_alpha_both=drhs_mid_alpha_both)
  assert cfg.fwd.local_aqt is None, 'local_aqt is not yet supported in fwd.'
  return cfg


def config_fwd_fp8(fwd_bits: str = 'e4m3') -> DotGeneral:
  """fp8 forward, float gradients, no stochastic rounding."""
  assert fwd_bits in fp8_numerics.fp8_map, (
      'FP8 only supports 4 or 5 exponent bits')
  cfg = config_v4(fwd_bits=8, dlhs_bits=None, drhs_bits=None)
  set_bits(cfg, fwd_lhs_bit=fwd_bits, fwd_rhs_bit=fwd_bits, dlhs_lhs_bit=None,
           dlhs_rhs_bit=None, drhs_lhs_bit=None, drhs_rhs_bit=None)
  set_stochastic_rounding(cfg, False, False, 'jax.uniform')
  assert cfg.fwd.local_aqt is None, 'local_aqt is not yet supported in fwd.'
  return cfg
