"""Delayed scaling calibration (flax/delayed_scaling_calibration.py:28-124):
the planner and the state handling against the oracle on the CPU stand-in, the
device kernels against the oracle on a GPU."""

import copy
import functools

import numpy as np
import pytest
import torch

from aqt_b200.v2 import aqt_dot_general as aqt
from aqt_b200.v2 import config
from aqt_b200.v2 import utils
from aqt_b200.v2.flax import delayed_scaling_calibration as dsc
from oracle import aqt_oracle as orc
from tests import util

DIMS = (((1,), (0,)), ((), ()))


def _delayed_cfg(kind, length=16, po2=False):
  if kind == 'int8':
    cfg = config.fully_quantized(fwd_bits=8, bwd_bits=8,
                                 use_stochastic_rounding=False)
  else:
    cfg = config.fully_quantized(fwd_bits='e4m3', bwd_bits='e5m2',
                                 use_stochastic_rounding=False)
  for raw in (cfg.fwd, cfg.dlhs, cfg.drhs):
    for qz in (raw.dg_quantizer.lhs, raw.dg_quantizer.rhs):
      qz.calib_shared_axes = 'per_tensor'
      qz.calibration = functools.partial(
          dsc.DelayedScalingCalibration, amax_history_length=length,
          po2_scale=po2)
  return config.set_context(cfg, key=None, train_step=None)


def _run_steps(cfg, dev, np_dtype, steps, sync=lambda: None):
  rng = np.random.default_rng(0)
  m, k, n = 32, 48, 16
  for step in range(steps):
    # magnitudes that rise and fall, so the history maximum matters
    amp = [1.0, 4.0, 0.5, 2.0, 0.25, 8.0][step % 6]
    lhs = util.rand_normal(rng, (m, k), amp, np_dtype)
    rhs = util.rand_normal(rng, (k, n), 0.2 * amp, np_dtype)
    g = util.rand_normal(rng, (m, n), 1.0 / amp, np_dtype)
    if step == 2:
      lhs[:] = 0  # an all-zero operand pushes a zero into the history
    out, bp = cfg.vjp(util.to_torch(lhs, dev), util.to_torch(rhs, dev), DIMS)
    dl, dr = bp(util.to_torch(g, dev))
    sync()
    wo, wl, wr, _ = orc.dg_fwd_bwd(cfg, lhs, rhs, g, DIMS)
    yield step, (out, dl, dr), (wo, wl, wr)


def _same(got, want, what):
  g = util.to_numpy(got)
  assert g.shape == want.shape and g.dtype == want.dtype, what
  np.testing.assert_array_equal(g.astype(np.float32), want.astype(np.float32),
                                err_msg=what)


def _check_state(cfg):
  for raw in (cfg.fwd, cfg.dlhs, cfg.drhs):
    for qz in (raw.dg_quantizer.lhs, raw.dg_quantizer.rhs):
      cal = qz._calibrator
      hist, bound = orc.delayed_state(cal)
      np.testing.assert_array_equal(cal.amax_history.cpu().numpy(), hist)
      np.testing.assert_array_equal(cal.bound.cpu().numpy(), bound)


@pytest.mark.parametrize('kind', ['int8', 'fp8'])
@pytest.mark.parametrize('np_dtype', [np.float32, orc.bfloat16])
@pytest.mark.parametrize('po2', [False, True])
def test_training_steps_match_oracle_on_the_stand_in(monkeypatch, kind,
                                                     np_dtype, po2):
  from tests import fake_lib
  fake = fake_lib.install(monkeypatch)
  cfg = _delayed_cfg(kind, po2=po2)
  for step, got, want in _run_steps(cfg, 'cpu', np_dtype, 5):
    for a, b, what in zip(got, want, ('out', 'dlhs', 'drhs')):
      if kind == 'int8':
        _same(a, b, f'{what} step {step}')
      else:
        np.testing.assert_allclose(
            util.to_numpy(a).astype(np.float32), b.astype(np.float32),
            rtol=2e-2, atol=1e-3, err_msg=f'{what} step {step}')
    _check_state(cfg)
  # bf16: every operand is read once (paired quantization that also takes the
  # maximum for the histories); f32: one quantization per dot
  paired = any(c[0] == 'quantize_pair' for c in fake.calls)
  assert paired == (np_dtype == orc.bfloat16)


def test_state_survives_deep_copies_and_serve_mode_freezes_it(monkeypatch):
  from tests import fake_lib
  fake_lib.install(monkeypatch)
  cfg = _delayed_cfg('int8', length=4)
  list(_run_steps(cfg, 'cpu', np.float32, 2))
  cal = cfg.fwd.dg_quantizer.lhs._calibrator
  clone = copy.deepcopy(cfg)
  assert clone.fwd.dg_quantizer.lhs._calibrator.stats is cal.stats
  before = cal.amax_history.clone(), cal.bound.clone()
  serve = config.set_context(clone, key=None, train_step=None,
                             lhs_quant_mode=utils.QuantMode.SERVE,
                             rhs_quant_mode=utils.QuantMode.SERVE)
  x = torch.randn(8, 48)
  w = torch.randn(48, 16)
  serve.fwd(x, w, None, None, DIMS)
  assert torch.equal(cal.amax_history, before[0])
  assert torch.equal(cal.bound, before[1])


@pytest.mark.gpu
@pytest.mark.parametrize('kind', ['int8', 'fp8'])
@pytest.mark.parametrize('np_dtype', [np.float32, orc.bfloat16])
def test_training_steps_match_oracle_on_the_device(kind, np_dtype):
  from aqt_b200 import engine

  def sync():
    torch.cuda.synchronize()
    engine.check_status()

  cfg = _delayed_cfg(kind, length=1024)
  for step, got, want in _run_steps(cfg, 'cuda', np_dtype, 8, sync):
    for a, b, what in zip(got, want, ('out', 'dlhs', 'drhs')):
      if kind == 'int8':
        _same(a, b, f'{what} step {step}')
      else:
        g, w = util.to_numpy(a).astype(np.float64), b.astype(np.float64)
        tol = np.maximum(np.abs(w) * 2.0 ** -7, 1e-4 * np.abs(w).max() + 1e-30)
        assert (np.abs(g - w) <= tol).all(), f'{what} step {step}'
    _check_state(cfg)
