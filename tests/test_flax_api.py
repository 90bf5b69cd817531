"""AqtDotGeneral / AqtEinsum wrappers and the autograd bridge (host logic)."""

import numpy as np
import pytest
import torch

from aqt_b200.v2 import aqt_dot_general as aqt
from aqt_b200.v2 import config
from aqt_b200.v2 import utils
from aqt_b200.v2.flax import aqt_flax
from oracle import aqt_oracle as orc
from tests import fake_lib
from tests import util


def test_einsum_lowering():
  dims, perm, swap = aqt.einsum_to_dot_general('bthd,bshd->bhts', 4, 4)
  assert dims == (((3,), (3,)), ((0, 2), (0, 2)))
  assert perm is None and not swap
  dims, perm, swap = aqt.einsum_to_dot_general('ab,bc->ac', 2, 2)
  assert dims == (((1,), (0,)), ((), ())) and perm is None and not swap
  # output wants rhs-free before lhs-free: operands are swapped instead of
  # transposing the result
  dims, perm, swap = aqt.einsum_to_dot_general('ab,bc->ca', 2, 2)
  assert swap and perm is None and dims == (((0,), (1,)), ((), ()))


def test_aqt_einsum_matches_oracle(monkeypatch):
  fake_lib.install(monkeypatch)
  rng = np.random.default_rng(0)
  q = util.rand_normal(rng, (2, 8, 3, 16), 1.0, orc.bfloat16)
  k = util.rand_normal(rng, (2, 6, 3, 16), 1.0, orc.bfloat16)
  cfg = config.fully_quantized(use_stochastic_rounding=False)
  got = aqt_flax.AqtEinsum(cfg)('bthd,bshd->bhts', util.to_torch(q),
                                util.to_torch(k))
  want, _ = orc.dg_fwd(cfg, q, k, (((3,), (3,)), ((0, 2), (0, 2))))
  np.testing.assert_array_equal(util.to_numpy(got).astype(np.float32),
                                want.astype(np.float32))


def test_autograd_bridge(monkeypatch):
  fake_lib.install(monkeypatch)
  rng = np.random.default_rng(1)
  dims = (((1,), (0,)), ((), ()))
  lhs = util.rand_normal(rng, (8, 32), 1.0, np.float32)
  rhs = util.rand_normal(rng, (32, 16), 0.2, np.float32)
  g = util.rand_normal(rng, (8, 16), 1.0, np.float32)
  cfg = config.fully_quantized(use_stochastic_rounding=False)
  tl = util.to_torch(lhs).requires_grad_()
  tr = util.to_torch(rhs).requires_grad_()
  out = aqt_flax.AqtDotGeneral(cfg)(tl, tr, dims)
  out.backward(util.to_torch(g))
  wo, wl, wr, _ = orc.dg_fwd_bwd(cfg, lhs, rhs, g, dims)
  np.testing.assert_array_equal(util.to_numpy(out), wo)
  np.testing.assert_array_equal(util.to_numpy(tl.grad), wl)
  np.testing.assert_array_equal(util.to_numpy(tr.grad), wr)


def test_convert_then_serve_is_bit_identical(monkeypatch):
  # examples/flax_e2e_model_test.py:255-257: logits served from the frozen
  # weights equal the training-mode logits exactly.
  fake_lib.install(monkeypatch)
  rng = np.random.default_rng(2)
  dims = (((1,), (0,)), ((), ()))
  x = util.to_torch(util.rand_normal(rng, (8, 32), 1.0, np.float32))
  w = util.to_torch(util.rand_normal(rng, (32, 16), 0.2, np.float32))
  cfg = config.fully_quantized(use_stochastic_rounding=False)
  train = aqt_flax.AqtDotGeneral(cfg)(x, w, dims)
  both = aqt_flax.FreezerMode.CALIBRATION_AND_VALUE
  with pytest.raises(ValueError, match='Freezer mode NONE'):
    aqt_flax.AqtDotGeneral(cfg, rhs_quant_mode=utils.QuantMode.CONVERT)(
        x, w, dims)
  for legacy in (True, False):
    conv = aqt_flax.AqtDotGeneral(cfg, rhs_quant_mode=utils.QuantMode.CONVERT,
                                  rhs_freeze_mode=both,
                                  use_legacy_freezer=legacy)
    conv(x, w, dims)
    stored = conv.variables['aqt']['qrhs']
    if legacy:  # aqt_flax.py:149-232: 'value' and 'scale' (= scale_t)
      assert set(stored) == {'value', 'scale'}
      assert stored['value'].dtype == torch.int8
      assert tuple(stored['value'].shape) == (32, 16)
      assert tuple(stored['scale'].shape) == (1, 16)  # output layout [M, N]
    else:  # flax/freezer.py: one 'frozen' QTensor
      frozen = stored['frozen']
      assert frozen.qvalue.dtype == torch.int8
      assert tuple(frozen.scale[0].shape) == (1, 16)
    serve = aqt_flax.AqtDotGeneral(cfg, rhs_quant_mode=utils.QuantMode.SERVE,
                                   rhs_freeze_mode=both,
                                   use_legacy_freezer=legacy,
                                   variables=conv.variables)
    got = serve(x, torch.zeros_like(w), dims)  # the float weights are unused
    np.testing.assert_array_equal(util.to_numpy(got), util.to_numpy(train))
  # handing the frozen operand over directly, freezers bypassed
  direct = aqt_flax.AqtDotGeneral(cfg, rhs_quant_mode=utils.QuantMode.SERVE,
                                  rhs_apply_quant_mode=False,
                                  rhs_qtensor=frozen)
  got = direct(x, torch.zeros_like(w), dims)
  np.testing.assert_array_equal(util.to_numpy(got), util.to_numpy(train))


def test_calibration_only_freezing_keeps_static_activation_scales(monkeypatch):
  # FreezerMode.CALIBRATION stores the scale without the values: serving then
  # quantizes new activations with the frozen (static) scale.
  fake_lib.install(monkeypatch)
  rng = np.random.default_rng(8)
  dims = (((1,), (0,)), ((), ()))
  x = util.to_torch(util.rand_normal(rng, (8, 32), 1.0, np.float32))
  w = util.to_torch(util.rand_normal(rng, (32, 16), 0.2, np.float32))
  cfg = config.fully_quantized(use_stochastic_rounding=False)
  cfg.fwd.dg_quantizer.lhs.calib_shared_axes = 'per_tensor'
  conv = aqt_flax.AqtDotGeneral(
      cfg, lhs_quant_mode=utils.QuantMode.CONVERT,
      lhs_freeze_mode=aqt_flax.FreezerMode.CALIBRATION,
      use_legacy_freezer=False)
  conv(x, w, dims)
  frozen = conv.variables['aqt']['qlhs']['frozen']
  assert frozen.qvalue is None and frozen.scale[0].numel() == 1
  serve = aqt_flax.AqtDotGeneral(
      cfg, lhs_quant_mode=utils.QuantMode.SERVE,
      lhs_freeze_mode=aqt_flax.FreezerMode.CALIBRATION,
      use_legacy_freezer=False, variables=conv.variables)
  x2 = x * 0.5  # its own maximum would give another scale
  got = serve(x2, w, dims)
  lhs_qt = orc.OQTensor(qvalue=None, scale=[util.to_numpy(frozen.scale[0])],
                        dequant_dtype=orc.float32)
  want, _ = orc.dg_fwd(cfg, util.to_numpy(x2), util.to_numpy(w), dims,
                       lhs_qt=lhs_qt)
  np.testing.assert_array_equal(util.to_numpy(got), want)


def test_aqt_einsum_convert_then_serve(monkeypatch):
  # the frozen weights live on the AqtEinsum object from one call to the
  # next, also when the einsum swaps its operands ('ab,bc->ca')
  fake_lib.install(monkeypatch)
  rng = np.random.default_rng(3)
  x = util.to_torch(util.rand_normal(rng, (8, 32), 1.0, np.float32))
  w = util.to_torch(util.rand_normal(rng, (32, 16), 0.2, np.float32))
  cfg = config.fully_quantized(use_stochastic_rounding=False)
  for eqn in ('ab,bc->ac', 'ab,bc->ca'):
    train = aqt_flax.AqtEinsum(cfg)(eqn, x, w)
    both = aqt_flax.FreezerMode.CALIBRATION_AND_VALUE
    conv = aqt_flax.AqtEinsum(cfg, rhs_quant_mode=utils.QuantMode.CONVERT,
                              rhs_freeze_mode=both)
    conv(eqn, x, w)
    # "rhs" is the SECOND einsum argument whatever the operand order
    stored = conv.variables['aqt']['qrhs']
    assert stored['value'].dtype == torch.int8
    assert tuple(stored['value'].shape) == (32, 16), eqn
    assert 'qlhs' not in conv.variables['aqt']
    serve = aqt_flax.AqtEinsum(cfg, rhs_quant_mode=utils.QuantMode.SERVE,
                               rhs_freeze_mode=both, variables=conv.variables)
    for _ in range(2):
      got = serve(eqn, x, torch.zeros_like(w))
      np.testing.assert_array_equal(util.to_numpy(got), util.to_numpy(train))


def test_aqt_einsum_draws_fresh_noise_every_call(monkeypatch):
  fake_lib.install(monkeypatch)
  from aqt_b200.v2 import stochastic_rounding as sr
  rng = np.random.default_rng(4)
  x = util.to_torch(util.rand_normal(rng, (8, 32), 1.0, np.float32))
  w = util.to_torch(util.rand_normal(rng, (32, 16), 0.2, np.float32))
  g = util.to_torch(util.rand_normal(rng, (8, 16), 1.0, np.float32))
  keys = []
  cfg = config.fully_quantized(use_stochastic_rounding=True)

  def noise_fn(shape, key):
    keys.append((int(key[0]), int(key[1])))
    return torch.zeros(shape)

  for raw in (cfg.dlhs, cfg.drhs):
    raw.dg_quantizer.lhs.numerics.noise_fn = noise_fn
    raw.dg_quantizer.rhs.numerics.noise_fn = noise_fn
  es = aqt_flax.AqtEinsum(cfg, rngs={'params': sr.PRNGKey(7)})
  for _ in range(2):
    xx, ww = x.clone().requires_grad_(), w.clone().requires_grad_()
    es('ab,bc->ac', xx, ww).backward(g)
  assert len(keys) == 8 and len(set(keys)) == 8, keys
