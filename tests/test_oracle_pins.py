"""Pins the CPU oracle against the reference's own test vectors.

Each case restates a known-answer test of the reference (path relative to
aqt/jax/v2/) so the oracle is anchored to something other than itself.
"""

import numpy as np
import pytest

from aqt_b200.v2 import aqt_dot_general as aqt
from aqt_b200.v2 import aqt_quantizer
from aqt_b200.v2 import calibration
from aqt_b200.v2 import config
from aqt_b200.v2 import utils
from aqt_b200.v2.numerics import int_numerics
from oracle import aqt_oracle as orc

_FP8_IN = np.array(
    [[0, 1, -1, 0.1234567, 100, 0.5, 0.00000000001, 0.01],
     [-2.9098532, -0.8508397, -0.14903745, -3.572757, 0.63277215, 0.7478278,
      1.3707844, 1.3319879]], np.float32)


def test_fp8_rne_e5m2():
  # numerics/fp8_numerics_test.py:50-79 (test_2bit_mantissa)
  got = orc.round_to_nearest_even_fp8(_FP8_IN, orc.float8_e5m2)
  want = np.array([[0, 1, -1, 0.125, 96, 0.5, 0, 10 / 1024],
                   [-3, -0.875, -0.15625, -3.5, 0.625, 0.75, 1.25, 1.25]],
                  np.float32)
  np.testing.assert_array_equal(got.astype(np.float32), want)


def test_fp8_rne_e4m3():
  # numerics/fp8_numerics_test.py:81-110 (test_3bit_mantissa)
  got = orc.round_to_nearest_even_fp8(_FP8_IN, orc.float8_e4m3fn)
  want = np.array([[0, 1, -1, 0.125, 96, 0.5, 0, 10 / 1024],
                   [-3, -0.875, -0.15625, -3.5, 0.625, 0.75, 1.375, 1.375]],
                  np.float32)
  np.testing.assert_array_equal(got.astype(np.float32), want)


@pytest.mark.parametrize('dt', [orc.float8_e4m3fn, orc.float8_e5m2])
def test_fp8_113_114(dt):
  # numerics/fp8_numerics_test.py:217-242
  got = orc.round_to_nearest_even_fp8(np.array([113.0, 114.0], np.float32), dt)
  np.testing.assert_array_equal(got.astype(np.float32), [112.0, 112.0])


def test_fp8_retains_dtype():
  # numerics/fp8_numerics_test.py:112-121
  a = orc.round_to_nearest_even_fp8(np.array([1], orc.bfloat16),
                                    orc.float8_e5m2)
  b = orc.round_to_nearest_even_fp8(np.array([1], np.float32),
                                    orc.float8_e4m3fn)
  assert a.dtype == orc.float8_e5m2 and b.dtype == orc.float8_e4m3fn


@pytest.mark.parametrize('pz,pmv,want', [
    (False, False, (128.0, 2.0, 1.0)),
    (False, True, (127.5, 1.5, 0.5)),
    (True, False, (127.5, 1.5, 0.5)),
    (True, True, (127.0, 1.0, 0.0)),
])
def test_int_bound_table(pz, pmv, want):
  # numerics/int_numerics.py:41-49
  for bits, w in zip((8, 2, 1), want):
    n = int_numerics.IntSymmetric(
        bits=bits, preserve_zero=pz, preserve_max_val=pmv, clip=True,
        clip_gradient=False, round=True, noise_fn=None)
    assert orc.int_quant_bound(n) == w
    assert n.get_quant_bound() == w


@pytest.mark.parametrize('bits', [2, 3, 4, 8])
@pytest.mark.parametrize('pmv', [False, True])
def test_int_range(bits, pmv):
  # numerics/int_numerics_test.py:58-115: quantized values span the full
  # signed range symmetric around zero and hit both ends.
  n = int_numerics.IntSymmetric(
      bits=bits, preserve_zero=True, preserve_max_val=pmv, clip=True,
      clip_gradient=False, round=True, noise_fn=None, dtype=utils.int8)
  x = np.linspace(-1.0, 1.0, 10001).astype(np.float32)[:, None]
  scale = orc.absmax_scale(x, [0], n)
  q = orc.int_vjp_fwd(n, orc.OQTensor(None, [scale]).quant(x), None)
  top = 2 ** (bits - 1) - 1
  assert q.dtype == np.int8
  assert q.max() == top and q.min() == -top
  assert set(np.unique(q)) == set(range(-top, top + 1))


@pytest.mark.parametrize('shard_count,want', [(2, 1281280.0), (1, 1280000.0)])
def test_local_aqt(shard_count, want):
  # aqt_dot_general_test.py:1079-1113
  dg = config.fully_quantized(
      fwd_bits=8, bwd_bits=8, use_stochastic_rounding=False,
      drhs_local_aqt=aqt.LocalAqt(contraction_axis_shard_count=shard_count))
  for q in (dg.fwd.dg_quantizer, dg.drhs.dg_quantizer):
    q.lhs.numerics.preserve_max_val = True
    q.rhs.numerics.preserve_max_val = True
  dims = (((), ()), ((), ()))
  lhs = np.array([1270.0, 10.0, 1270000.0, 10000.0], np.float32)
  rhs = np.array([1.0], np.float32)
  out, res = orc.dg_fwd(dg, lhs, rhs, dims)
  _, drhs = orc.dg_bwd(dg, dims, res, np.ones_like(out))
  assert drhs.shape == (1,)
  assert float(drhs[0]) == want


def test_per_tensor_scale_is_one():
  # aqt_dot_general_test.py:1115-1144
  bits = 4
  n = int_numerics.IntSymmetric(
      bits=bits, preserve_zero=True, preserve_max_val=False, clip=True,
      clip_gradient=False, round=True, noise_fn=None, dtype=utils.int8)
  quantizer = aqt_quantizer.Quantizer(
      numerics=n, calib_shared_axes='per_tensor', scale_stop_grad=True,
      calibration=calibration.AbsMaxCalibration,
      context=utils.Context(key=None, train_step=None))
  x = np.array([[1, 2, 3, 4], [5, 6, 7, 2 ** (bits - 1) - 0.5],
                [3, 5, 1, -1]], np.float32)
  qt = orc.quantizer_calibrate(quantizer, x, None)
  assert len(qt.scale) == 1
  np.testing.assert_array_equal(qt.scale[0], np.array([[1.0]], np.float32))


def _po2(dg):
  import functools
  for raw in (dg.fwd, dg.dlhs, dg.drhs):
    for q in (raw.dg_quantizer.lhs, raw.dg_quantizer.rhs):
      if q.calibration is not None:
        q.calibration = functools.partial(q.calibration, po2_scale=True)
  return dg


@pytest.mark.parametrize('seed', range(4))
@pytest.mark.parametrize('use_fwd_quant', [False, True])
@pytest.mark.parametrize('bits', [2, 8])
def test_fake_quant_equals_int_path_with_po2_scales(seed, use_fwd_quant, bits):
  # aqt_dot_general_test.py:146-177, 254-264, 615-628: with power-of-two
  # scales the true-integer path and the fake-quant path (dequantize this
  # input before a float dot) agree exactly, gradients included.
  rng = np.random.default_rng(seed)
  lhs = rng.uniform(-1, 1, (10, 20)).astype(np.float32)
  rhs = rng.uniform(-1, 1, (20, 30)).astype(np.float32)
  gra = rng.uniform(-1, 1, (10, 30)).astype(np.float32)
  dims = (((1,), (0,)), ((), ()))

  def make(fq):
    dg = _po2(config.fully_quantized(
        fwd_bits=bits, bwd_bits=bits, use_fwd_quant=use_fwd_quant,
        use_stochastic_rounding=False))
    if fq:
      for raw in (dg.fwd, dg.dlhs, dg.drhs):
        raw.lhs.dequant_mode = aqt.DequantMode.THIS_INPUT
        raw.rhs.dequant_mode = aqt.DequantMode.THIS_INPUT
        raw.dg_quantizer.lhs.numerics.dtype = None
        raw.dg_quantizer.rhs.numerics.dtype = None
        raw.dg_accumulator_dtype = None
    return dg

  a = orc.dg_fwd_bwd(make(False), lhs, rhs, gra, dims)[:3]
  b = orc.dg_fwd_bwd(make(True), lhs, rhs, gra, dims)[:3]
  for x, y in zip(a, b):
    np.testing.assert_array_equal(x, y)


def test_unquantized_equals_plain_dot():
  # aqt_dot_general_test.py:705-715
  rng = np.random.default_rng(0)
  lhs = rng.standard_normal((10, 20)).astype(np.float32)
  rhs = rng.standard_normal((20, 30)).astype(np.float32)
  dims = (((1,), (0,)), ((), ()))
  out, _ = orc.dg_fwd(config.default_unquantized_config(), lhs, rhs, dims)
  want = (lhs.astype(np.float64) @ rhs.astype(np.float64)).astype(np.float32)
  np.testing.assert_array_equal(out, want)


@pytest.mark.parametrize('dims,lhs_shape,rhs_shape', [
    ((((1,), (0,)), ((), ())), (10, 20), (20, 30)),
    ((((3,), (3,)), ((0, 2), (0, 2))), (2, 5, 3, 4), (2, 6, 3, 4)),
    ((((2,), (1,)), ((0,), (0,))), (3, 4, 5), (3, 5, 6)),
    ((((0, 2), (1, 0)), ((), ())), (4, 3, 5), (5, 4, 7)),
])
def test_bwd_dimension_numbers_give_the_true_gradient(dims, lhs_shape,
                                                      rhs_shape):
  # The gradient dot_generals built by aqt_dot_general.py:1127-1175 must
  # reproduce d(sum(out*g)) for an unquantized config.
  rng = np.random.default_rng(1)
  lhs = rng.standard_normal(lhs_shape).astype(np.float32)
  rhs = rng.standard_normal(rhs_shape).astype(np.float32)
  cfg = config.default_unquantized_config()
  out, res = orc.dg_fwd(cfg, lhs, rhs, dims)
  g = rng.standard_normal(out.shape).astype(np.float32)
  dlhs, drhs = orc.dg_bwd(cfg, dims, res, g)
  assert dlhs.shape == lhs.shape and drhs.shape == rhs.shape
  eps = 1e-2
  for arr, grad in ((lhs, dlhs), (rhs, drhs)):
    idx = tuple(rng.integers(0, s) for s in arr.shape)
    bumped = arr.copy()
    bumped[idx] += eps
    o2, _ = orc.dg_fwd(cfg, *((bumped, rhs) if arr is lhs else (lhs, bumped)),
                       dims)
    fd = ((o2.astype(np.float64) - out) * g).sum() / eps
    assert abs(fd - grad[idx]) < 5e-2 * max(1.0, abs(fd))
  # the package's own helper must agree with the oracle's restatement
  for y_is_lhs, y in ((False, rhs), (True, lhs)):
    assert aqt._update_dimension_numbers_for_backward(
        dims, y_is_lhs, g.ndim, y.ndim) == orc.bwd_dimension_numbers(
            dims, y_is_lhs, g.ndim, y.ndim)
