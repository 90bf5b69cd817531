"""Host-logic tests: the planner in aqt_b200/engine.py against the oracle.

The shared library is replaced by tests/fake_lib.py (numpy on host memory), so
what is under test is everything ABOVE the C ABI: stride normalisation for
arbitrary dimension_numbers, operand swapping, output-transpose folding,
residual QTensor layouts, use_fwd_quant plumbing, noise plumbing.
"""

import numpy as np
import pytest
import torch

from aqt_b200.v2 import config
from aqt_b200.v2 import aqt_dot_general as aqt
from oracle import aqt_oracle as orc
from tests import fake_lib
from tests import util


def _run_both(cfg, lhs, rhs, g, dims):
  tl, tr, tg = util.to_torch(lhs), util.to_torch(rhs), util.to_torch(g)
  out, backprop = cfg.vjp(tl, tr, dims)
  dl, dr = backprop(tg)
  want = orc.dg_fwd_bwd(cfg, lhs, rhs, g, dims)
  return (out, dl, dr), want


def _assert_same(got, want, what):
  g = util.to_numpy(got)
  assert g.shape == want.shape, (what, g.shape, want.shape)
  assert g.dtype == want.dtype, (what, g.dtype, want.dtype)
  np.testing.assert_array_equal(g.astype(np.float32), want.astype(np.float32),
                                err_msg=what)


CASES = [
    # dims, lhs shape, rhs shape
    ((((1,), (0,)), ((), ())), (12, 40), (40, 24)),
    ((((3,), (3,)), ((0, 2), (0, 2))), (2, 9, 3, 16), (2, 7, 3, 16)),
    ((((2,), (1,)), ((0,), (0,))), (3, 5, 32), (3, 32, 6)),
    ((((1,), (1,)), ((), ())), (8, 20), (10, 20)),
    ((((0,), (0,)), ((), ())), (20, 8), (20, 10)),
    ((((2,), (0,)), ((), ())), (4, 6, 32), (32, 12)),
    # kept axes of lhs on both sides of its contraction axis ('bkh,kd->bhd'):
    # no single strided view exists, the planner regroups with copies
    ((((1,), (0,)), ((), ())), (4, 32, 6), (32, 10)),
    ((((1,), (0,)), ((), ())), (4, 6, 6), (6, 5)),
]


@pytest.mark.parametrize('dims,ls,rs', CASES)
@pytest.mark.parametrize('np_dtype', [np.float32, orc.bfloat16])
@pytest.mark.parametrize('use_fwd_quant', [True, False])
def test_int8_fwd_bwd_matches_oracle(monkeypatch, dims, ls, rs, np_dtype,
                                     use_fwd_quant):
  fake_lib.install(monkeypatch)
  rng = np.random.default_rng(0)
  lhs = util.rand_normal(rng, ls, 1.0, np_dtype)
  rhs = util.rand_normal(rng, rs, 0.2, np_dtype)
  cfg = config.fully_quantized(fwd_bits=8, bwd_bits=8,
                               use_fwd_quant=use_fwd_quant,
                               use_stochastic_rounding=False)
  out_shape = orc.dg_fwd(cfg, lhs, rhs, dims)[0].shape
  g = util.rand_normal(rng, out_shape, 1.0, np_dtype)
  (out, dl, dr), (wo, wl, wr, res) = _run_both(cfg, lhs, rhs, g, dims)
  _assert_same(out, wo, 'out')
  _assert_same(dl, wl, 'dlhs')
  _assert_same(dr, wr, 'drhs')


@pytest.mark.parametrize('fwd,bwd', [('e4m3', 'e5m2'), ('e4m3', 'e4m3')])
@pytest.mark.parametrize('np_dtype', [np.float32, orc.bfloat16])
def test_fp8_per_tensor_matches_oracle(monkeypatch, fwd, bwd, np_dtype):
  fake_lib.install(monkeypatch)
  rng = np.random.default_rng(1)
  dims = (((1,), (0,)), ((), ()))
  lhs = util.rand_normal(rng, (24, 48), 1.0, np_dtype)
  rhs = util.rand_normal(rng, (48, 40), 0.1, np_dtype)
  g = util.rand_normal(rng, (24, 40), 1.0, np_dtype)
  cfg = config.fully_quantized(fwd_bits=fwd, bwd_bits=bwd,
                               use_stochastic_rounding=False)
  for raw in (cfg.fwd, cfg.dlhs, cfg.drhs):
    raw.dg_quantizer.lhs.calib_shared_axes = 'per_tensor'
    raw.dg_quantizer.rhs.calib_shared_axes = 'per_tensor'
  (out, dl, dr), (wo, wl, wr, _) = _run_both(cfg, lhs, rhs, g, dims)
  _assert_same(out, wo, 'out')
  _assert_same(dl, wl, 'dlhs')
  _assert_same(dr, wr, 'drhs')


@pytest.mark.parametrize('fwd,bwd', [('e4m3', 'e5m2'), ('e5m2', 'e5m2'),
                                     (8, 8), (4, 8)])
def test_fp8_per_tensor_paired_quantization_matches_oracle(monkeypatch, fwd,
                                                           bwd):
  """bf16 matmul with extents that are multiples of 16: every operand is read
  once for its two quantized copies (aqtb200_quantize_pair), and the results
  are those of the reference's one-quantization-per-dot flow."""
  fake = fake_lib.install(monkeypatch)
  rng = np.random.default_rng(3)
  dims = (((1,), (0,)), ((), ()))
  lhs = util.rand_normal(rng, (32, 64), 1.0, orc.bfloat16)
  rhs = util.rand_normal(rng, (64, 48), 0.1, orc.bfloat16)
  g = util.rand_normal(rng, (32, 48), 1.0, orc.bfloat16)
  cfg = config.fully_quantized(fwd_bits=fwd, bwd_bits=bwd,
                               use_stochastic_rounding=False)
  for raw in (cfg.fwd, cfg.dlhs, cfg.drhs):
    raw.dg_quantizer.lhs.calib_shared_axes = 'per_tensor'
    raw.dg_quantizer.rhs.calib_shared_axes = 'per_tensor'
  tl, tr, tg = util.to_torch(lhs), util.to_torch(rhs), util.to_torch(g)
  (out, (lq, rq)), vres = aqt.dg_core_vjp_fwd(tl, tr, None, None, dims, cfg)
  dl, dr, *_ = aqt.dg_core_vjp_bwd(dims, vres, (tg, None))
  assert [c for c in fake.calls if c[0] == 'quantize_pair'] == [
      ('quantize_pair', 1), ('quantize_pair', 2), ('quantize_pair', 0)]
  wo, wl, wr, res = orc.dg_fwd_bwd(cfg, lhs, rhs, g, dims)
  _assert_same(lq.qvalue, res.lhs.qx.qvalue, 'q_lhs')
  _assert_same(rq.qvalue, res.rhs.qx.qvalue, 'q_rhs')
  _assert_same(lq.scale[0], res.lhs.qx.scale[0], 's_lhs')
  _assert_same(rq.scale[0], res.rhs.qx.scale[0], 's_rhs')
  _assert_same(out, wo, 'out')
  _assert_same(dl, wl, 'dlhs')
  _assert_same(dr, wr, 'drhs')


def test_residual_qtensors_have_reference_layout(monkeypatch):
  fake_lib.install(monkeypatch)
  rng = np.random.default_rng(2)
  dims = (((3,), (3,)), ((0, 2), (0, 2)))
  lhs = util.rand_normal(rng, (2, 9, 3, 16), 1.0, orc.bfloat16)
  rhs = util.rand_normal(rng, (2, 7, 3, 16), 1.0, orc.bfloat16)
  cfg = config.fully_quantized(use_stochastic_rounding=False)
  (out, (lq, rq)), _ = aqt.dg_core_vjp_fwd(
      util.to_torch(lhs), util.to_torch(rhs), None, None, dims, cfg)
  _, res = orc.dg_fwd(cfg, lhs, rhs, dims)
  for got, want in ((lq, res.lhs.qx), (rq, res.rhs.qx)):
    assert tuple(got.qvalue.shape) == want.qvalue.shape
    np.testing.assert_array_equal(util.to_numpy(got.qvalue), want.qvalue)
    assert tuple(got.scale[0].shape) == want.scale[0].shape
    _assert_same(got.scale[0], want.scale[0], 'scale')


def test_stochastic_rounding_noise_is_plumbed(monkeypatch):
  fake_lib.install(monkeypatch)
  rng = np.random.default_rng(3)
  dims = (((1,), (0,)), ((), ()))
  lhs = util.rand_normal(rng, (16, 32), 1.0, np.float32)
  rhs = util.rand_normal(rng, (32, 48), 0.2, np.float32)
  g = util.rand_normal(rng, (16, 48), 1.0, np.float32)
  cfg = config.fully_quantized(use_stochastic_rounding=True)
  noise_rng = np.random.default_rng(7)
  table = {}

  def noise_fn(shape, key):
    k = (tuple(shape), int(key[0]), int(key[1]))
    if k not in table:
      table[k] = torch.from_numpy(
          (noise_rng.random(shape, np.float32) - 0.5).astype(np.float32))
    return table[k]

  for raw in (cfg.dlhs, cfg.drhs):
    raw.dg_quantizer.lhs.numerics.noise_fn = noise_fn
    raw.dg_quantizer.rhs.numerics.noise_fn = noise_fn
  from aqt_b200.v2 import stochastic_rounding as sr
  cfg = config.set_context(cfg, key=sr.PRNGKey(5), train_step=None)
  (out, dl, dr), (wo, wl, wr, _) = _run_both(cfg, lhs, rhs, g, dims)
  assert len(table) == 4  # four distinct (shape, key) draws
  _assert_same(out, wo, 'out')
  _assert_same(dl, wl, 'dlhs')
  _assert_same(dr, wr, 'drhs')


def test_unsupported_configs_raise(monkeypatch):
  fake_lib.install(monkeypatch)
  x = torch.zeros(4, 16)
  y = torch.zeros(16, 8)
  dims = (((1,), (0,)), ((), ()))
  cfg = config.fully_quantized(use_stochastic_rounding=False)
  cfg.fwd.lhs.dequant_mode = aqt.DequantMode.THIS_INPUT
  with pytest.raises(NotImplementedError):
    cfg(x, y, dims)
  cfg = config.fully_quantized(use_stochastic_rounding=False,
                               drhs_local_aqt=aqt.LocalAqt(
                                   contraction_axis_shard_count=2))
  out, bp = cfg.vjp(x, y, dims)
  with pytest.raises(NotImplementedError):
    bp(torch.zeros(4, 8))
  cfg = config.fully_quantized(use_stochastic_rounding=False)
  with pytest.raises(AssertionError):
    cfg(x, y, dims, precision='highest')
  with pytest.raises(AssertionError):
    cfg(x, y.to(torch.bfloat16), dims)


@pytest.mark.parametrize('kind', ['int8_per_channel', 'fp8_per_tensor'])
def test_traced_step_replays_the_same_calls(monkeypatch, kind):
  """engine.TracedStep: record once, replay; new input VALUES written into the
  traced tensors give the new step's results."""
  from aqt_b200 import engine
  fake_lib.install(monkeypatch)
  rng = np.random.default_rng(5)
  dims = (((1,), (0,)), ((), ()))
  dt = np.float32 if kind == 'int8_per_channel' else orc.bfloat16
  if kind == 'int8_per_channel':
    cfg = config.fully_quantized(fwd_bits=8, bwd_bits=8,
                                 use_stochastic_rounding=False)
  else:
    cfg = config.fully_quantized(fwd_bits='e4m3', bwd_bits='e5m2',
                                 use_stochastic_rounding=False)
    for raw in (cfg.fwd, cfg.dlhs, cfg.drhs):
      raw.dg_quantizer.lhs.calib_shared_axes = 'per_tensor'
      raw.dg_quantizer.rhs.calib_shared_axes = 'per_tensor'
  mk = lambda shape, std: util.rand_normal(rng, shape, std, dt)
  lhs, rhs, g = mk((32, 48), 1.0), mk((48, 16), 0.2), mk((32, 16), 1.0)
  tl, tr, tg = util.to_torch(lhs), util.to_torch(rhs), util.to_torch(g)

  def step(a, b, c):
    out, bp = cfg.vjp(a, b, dims)
    return (out,) + tuple(bp(c))

  traced = engine.TracedStep(step, tl, tr, tg)
  assert traced.n_ops >= 3
  # second step: other values in the same tensors
  lhs2, g2 = mk((32, 48), 2.0), mk((32, 16), 0.5)
  tl.copy_(util.to_torch(lhs2))
  tg.copy_(util.to_torch(g2))
  out, dl, dr = traced(tl, tr, tg)
  wo, wl, wr, _ = orc.dg_fwd_bwd(cfg, lhs2, rhs, g2, dims)
  _assert_same(out, wo, 'out')
  _assert_same(dl, wl, 'dlhs')
  _assert_same(dr, wr, 'drhs')
  with pytest.raises(AssertionError):
    traced(tl.clone(), tr, tg)


@pytest.mark.parametrize('dims,ls,rs', [
    ((((1,), (0,)), ((), ())), (32, 48), (48, 16)),
    ((((3,), (3,)), ((0, 2), (0, 2))), (2, 16, 3, 32), (2, 32, 3, 32)),
    ((((2,), (1,)), ((0,), (0,))), (3, 16, 32), (3, 32, 48)),
])
@pytest.mark.parametrize('use_fwd_quant', [True, False])
@pytest.mark.parametrize('noise', [False, True])
def test_cotangent_read_twice_for_both_gradient_dots(monkeypatch, dims, ls, rs,
                                                     use_fwd_quant, noise):
  """Per-row scales, bf16: aqtb200_quantize_dual calibrates and quantizes the
  cotangent for dlhs and drhs together; same results as one dot at a time."""
  from aqt_b200 import engine
  from aqt_b200.v2 import stochastic_rounding as sr
  fake = fake_lib.install(monkeypatch)
  calls = []
  real = fake.aqtb200_quantize_dual
  fake.aqtb200_quantize_dual = lambda *a: calls.append(1) or real(*a)
  rng = np.random.default_rng(2)
  lhs = util.rand_normal(rng, ls, 1.0, orc.bfloat16)
  rhs = util.rand_normal(rng, rs, 0.3, orc.bfloat16)
  cfg = config.fully_quantized(fwd_bits=8, bwd_bits=8,
                               use_fwd_quant=use_fwd_quant,
                               use_stochastic_rounding=noise)
  if noise:
    table = {}

    def noise_fn(shape, key):
      kk = (tuple(shape), int(key[0]), int(key[1]))
      if kk not in table:
        table[kk] = torch.from_numpy(
            (rng.random(shape, np.float32) - 0.5).astype(np.float32))
      return table[kk]

    for raw in (cfg.dlhs, cfg.drhs):
      raw.dg_quantizer.lhs.numerics.noise_fn = noise_fn
      raw.dg_quantizer.rhs.numerics.noise_fn = noise_fn
    cfg = config.set_context(cfg, key=sr.PRNGKey(1), train_step=None)
  out_shape = orc.dg_fwd(cfg, lhs, rhs, dims)[0].shape
  g = util.rand_normal(rng, out_shape, 1.0, orc.bfloat16)
  (out, dl, dr), (wo, wl, wr, _) = _run_both(cfg, lhs, rhs, g, dims)
  assert calls, 'the two-pass path did not run'
  _assert_same(out, wo, 'out')
  _assert_same(dl, wl, 'dlhs')
  _assert_same(dr, wr, 'drhs')
