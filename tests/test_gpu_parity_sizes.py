"""Parity against the CPU oracle at the benchmark configurations' own sizes.

Where the whole problem is too big for the numpy oracle to contract in
seconds, everything elementwise (quantized operands, scales) is compared in
full and the contraction is compared on bands of rows: rows of a dot_general
are independent given the scales, so a band of the oracle's result needs only
that band of the operand.

Tolerances: int8 results, every quantized value and every scale are compared
bit for bit. fp8: the tensor core adds the f32 products in another order than
the oracle (exact sum, rounded once), so the f32 accumulators can differ in
their last bits, and the reference's dequantization of a bf16 result rounds
three times (cast of the accumulator, then one rounding per scale multiply,
aqt_tensor.py:161-200): a one-ulp difference in the cast can come out as two
ulps. The fp8 checks are therefore split so that each part is exact:
  (i)   the f32 accumulators against an exact (f64) contraction of the SAME
        quantized operands: |acc - exact| <= 1e-5 * sum_k |a_k b_k|;
  (ii)  the epilogue, bit for bit: the oracle's dequantization applied to the
        device's own accumulators equals the device's output;
  (iii) end to end against the oracle: the device's result lies between the
        oracle's dequantization of (exact - d) and of (exact + d), with
        d = 1e-5 * sum_k |a_k b_k| (dequantization is monotone in the
        accumulator: the scales are positive).
"""

import numpy as np
import pytest
import torch

from aqt_b200 import engine
from aqt_b200.v2 import aqt_dot_general as aqt
from aqt_b200.v2 import config
from aqt_b200.v2 import stochastic_rounding as sr
from aqt_b200.v2 import utils
from aqt_b200.v2.flax import aqt_flax
from oracle import aqt_oracle as orc
from tests import util

pytestmark = pytest.mark.gpu

DEV = 'cuda'
DIMS = (((1,), (0,)), ((), ()))


def _cuda(a):
  return util.to_torch(a, DEV)


def _sync():
  torch.cuda.synchronize()
  engine.check_status()


def _bits(a):
  a = np.ascontiguousarray(a)
  return a.view({1: np.uint8, 2: np.uint16, 4: np.uint32}[a.dtype.itemsize])


def _exact(got, want, what):
  g = util.to_numpy(got) if isinstance(got, torch.Tensor) else np.asarray(got)
  want = np.asarray(want)
  assert g.shape == want.shape, (what, g.shape, want.shape)
  assert g.dtype == want.dtype, (what, g.dtype, want.dtype)
  bad = _bits(g) != _bits(want)
  if bad.any():
    # +0 / -0 differ in bits but not in value
    bad &= g.astype(np.float32) != want.astype(np.float32)
  assert not bad.any(), (
      f'{what}: {int(bad.sum())} of {bad.size} differ; first at '
      f'{np.argwhere(bad)[0].tolist()}')


def _fp8_close(got, want, bound, what, ulps=2.0):
  g = util.to_numpy(got) if isinstance(got, torch.Tensor) else np.asarray(got)
  assert g.shape == want.shape and g.dtype == want.dtype, (
      what, g.shape, want.shape, g.dtype, want.dtype)
  a, b = g.astype(np.float64), want.astype(np.float64)
  tol = 1e-5 * bound
  if want.dtype == orc.bfloat16:
    ulp = 2.0 ** (np.floor(np.log2(np.maximum(np.abs(b), 1e-38))) - 7)
    tol = np.maximum(tol, ulps * ulp)
  bad = np.abs(a - b) > tol
  assert not bad.any(), (
      f'{what}: {int(bad.sum())} of {bad.size} outside tolerance; worst '
      f'{np.max(np.abs(a - b) / tol):.3g}x')


def _per_tensor(cfg):
  for raw in (cfg.fwd, cfg.dlhs, cfg.drhs):
    raw.dg_quantizer.lhs.calib_shared_axes = 'per_tensor'
    raw.dg_quantizer.rhs.calib_shared_axes = 'per_tensor'
  return cfg


def _oracle_quant(quantizer, x, axes):
  return orc.quantizer_calculate_qvalue(
      quantizer, x, orc.quantizer_calibrate(quantizer, x, axes))


def _f64(a):
  return np.asarray(a).astype(np.float32).astype(np.float64)


def _band_dequant(qa, sa, qb, sb, dtype, acc_dev=None):
  """Oracle dequantized rows  qa[band, K] . qb[K, N]  with per-tensor scales
  (lhs scale first), and the tolerance bound sum |a||b| * scales. With
  `acc_dev` (the device's f32 accumulators of the band) also checks them
  against the exact contraction and returns, third, the oracle's
  dequantization of THOSE accumulators."""
  a, b = _f64(qa), _f64(qb)
  exact = a @ b
  mag = np.abs(a) @ np.abs(b)
  scales = [sa.reshape(1, 1), sb.reshape(1, 1)]
  out = orc.OQTensor(qvalue=exact.astype(np.float32), scale=scales,
                     dequant_dtype=dtype).dequant()
  bound = mag * float(_f64(sa).ravel()[0]) * float(_f64(sb).ravel()[0])
  if acc_dev is None:
    return out, bound
  acc_dev = np.asarray(acc_dev, np.float32)
  delta = 1e-5 * mag + 1e-30
  bad = np.abs(acc_dev.astype(np.float64) - exact) > delta
  assert not bad.any(), f'{int(bad.sum())} accumulators off the exact sum'
  deq = lambda a: orc.OQTensor(qvalue=np.asarray(a, np.float32), scale=scales,
                               dequant_dtype=dtype).dequant()
  # f32 neighbours outward, so that rounding (exact -+ delta) to f32 cannot
  # shrink the bracket
  lo = deq(np.nextafter((exact - delta).astype(np.float32), np.float32(-np.inf)))
  hi = deq(np.nextafter((exact + delta).astype(np.float32), np.float32(np.inf)))
  return out, (lo, hi), deq(acc_dev)


def _fp8_training_step_vs_oracle(lhs, rhs, g, bands):
  """The per-tensor fp8 training step (e4m3 forward, e5m2 backward, bf16):
  all six quantized operand copies and their scales bit for bit against the
  oracle over the whole tensors; out / dlhs / drhs on the given row bands."""
  cfg = _per_tensor(config.fully_quantized(
      fwd_bits='e4m3', bwd_bits='e5m2', use_stochastic_rounding=False))
  dt = lhs.dtype
  tl, tr, tg = _cuda(lhs), _cuda(rhs), _cuda(g)
  (out, (lq, rq)), vres = aqt.dg_core_vjp_fwd(tl, tr, None, None, DIMS, cfg)
  res = vres[0]
  pair = engine.cotangent_pair(cfg, res, tg)
  dl, dr, *_ = aqt.dg_core_vjp_bwd(DIMS, vres, (tg, None))
  _sync()

  # -- oracle, operand by operand (aqt_dot_general.py:598-729, 1206-1217)
  o_l = _oracle_quant(cfg.fwd.dg_quantizer.lhs, lhs, [1])
  o_r = _oracle_quant(cfg.fwd.dg_quantizer.rhs, rhs, [0])
  _exact(lq.scale[0], o_l.scale[0], 's_lhs')
  _exact(rq.scale[0], o_r.scale[0], 's_rhs')
  _exact(lq.qvalue, o_l.qvalue, 'q_lhs (e4m3)')
  _exact(rq.qvalue, o_r.qvalue, 'q_rhs (e4m3)')
  ores = orc.ORes(lhs=orc.OMultiTensor(x=lhs, qx=o_l),
                  rhs=orc.OMultiTensor(x=rhs, qx=o_r))
  # dlhs = g[M,N] . rhs[K,N]^T ; drhs = g[M,N]^T . lhs[M,K]
  d_dims, _ = orc.bwd_dimension_numbers(DIMS, False, 2, 2)
  r_dims, _ = orc.bwd_dimension_numbers(DIMS, True, 2, 2)
  g_dl, r_x = orc.maybe_use_fwd_quant(g, ores.rhs, d_dims, True)
  g_dr, l_x = orc.maybe_use_fwd_quant(g, ores.lhs, r_dims, True)
  o_g_dl = _oracle_quant(cfg.dlhs.dg_quantizer.lhs, g_dl, list(d_dims[0][0]))
  o_r_b = _oracle_quant(cfg.dlhs.dg_quantizer.rhs, r_x, list(d_dims[0][1]))
  o_g_dr = _oracle_quant(cfg.drhs.dg_quantizer.lhs, g_dr, list(r_dims[0][0]))
  o_l_b = _oracle_quant(cfg.drhs.dg_quantizer.rhs, l_x, list(r_dims[0][1]))
  got_l_b = engine.bwd_copy(lq)
  got_r_b = engine.bwd_copy(rq)
  assert got_l_b is not None and got_r_b is not None and pair is not None, (
      'the one-read quantization path did not run')
  for got, want, what in (
      (got_l_b, o_l_b, 'lhs re-quantized for drhs (e5m2)'),
      (got_r_b, o_r_b, 'rhs re-quantized for dlhs (e5m2)'),
      (pair[0], o_g_dl, 'cotangent for dlhs (e5m2)'),
      (pair[1], o_g_dr, 'cotangent for drhs (e5m2)')):
    _exact(got.scale[0], want.scale[0], 'scale of ' + what)
    _exact(got.qvalue, want.qvalue, what)

  # -- the device's own f32 accumulators of the three dots: the same kernels
  # run once more on the same quantized operands, writing accumulators only
  d_dims_t, d_perm = aqt._update_dimension_numbers_for_backward(DIMS, False, 2, 2)
  r_dims_t, r_perm = aqt._update_dimension_numbers_for_backward(DIMS, True, 2, 2)
  acc_f = engine.dg_raw(cfg.fwd, tl, tr, lq, rq, DIMS, defer_dequant=True,
                        internal_qt=True)[0].acc_mn[0]          # [M, N]
  acc_dl = engine.dg_raw(cfg.dlhs, tg, res.rhs.mt, pair[0], got_r_b, d_dims_t,
                         out_transpose_axes=d_perm, defer_dequant=True,
                         internal_qt=True)[0].acc_mn[0]         # [M, K]
  acc_dr = engine.dg_raw(cfg.drhs, tg, res.lhs.mt, pair[1], got_l_b, r_dims_t,
                         out_transpose_axes=r_perm, defer_dequant=True,
                         internal_qt=True)[0].acc_mn[0]         # [N, K]
  _sync()

  def band_check(got, want, bracket, from_dev, what):
    # (ii) the epilogue alone, bit for bit; (iii) end to end: inside the
    # oracle's results for accumulators within 1e-5 of the exact sum
    del want
    _exact(got, from_dev.astype(dt), what + ': epilogue on the device\'s own '
           'accumulators')
    g = util.to_numpy(got).astype(np.float64)
    lo, hi = (np.asarray(b).astype(np.float64) for b in bracket)
    bad = (g < np.minimum(lo, hi)) | (g > np.maximum(lo, hi))
    assert not bad.any(), f'{what}: {int(bad.sum())} results outside the bracket'

  # -- dequantized results on bands of rows
  for r0, r1 in bands['out']:
    want, bound, dev = _band_dequant(
        o_l.qvalue[r0:r1], o_l.scale[0], o_r.qvalue, o_r.scale[0], dt,
        util.to_numpy(acc_f[r0:r1]))
    band_check(out[r0:r1], want, bound, dev, f'out[{r0}:{r1}]')
  for r0, r1 in bands['dlhs']:
    want, bound, dev = _band_dequant(
        o_g_dl.qvalue[r0:r1], o_g_dl.scale[0], np.asarray(o_r_b.qvalue).T,
        o_r_b.scale[0], dt, util.to_numpy(acc_dl[r0:r1]))
    band_check(dl[r0:r1], want, bound, dev, f'dlhs[{r0}:{r1}]')
  for r0, r1 in bands['drhs']:
    # raw drhs is [N, K] = g^T . lhs; the result is its transpose [K, N]:
    # a band of drhs ROWS is a band of lhs COLUMNS
    want, bound, dev = _band_dequant(
        np.asarray(o_g_dr.qvalue).T, o_g_dr.scale[0],
        np.asarray(o_l_b.qvalue)[:, r0:r1], o_l_b.scale[0], dt,
        util.to_numpy(acc_dr[:, r0:r1]))
    band_check(dr[r0:r1], want.T, (bound[0].T, bound[1].T), dev.T,
               f'drhs[{r0}:{r1}]')


def test_config2_full_size_against_oracle():
  """BASELINE config 2 at 8192^3: six quantized copies and scales over the
  whole tensors, dequantized results on 256-row bands."""
  n = 8192
  rng = np.random.default_rng(0)
  lhs = util.rand_normal(rng, (n, n), 1.0, orc.bfloat16)
  rhs = util.rand_normal(rng, (n, n), n ** -0.5, orc.bfloat16)
  g = util.rand_normal(rng, (n, n), 1.0, orc.bfloat16)
  bands = {'out': [(0, 256), (7936, 8192)], 'dlhs': [(3840, 4096)],
           'drhs': [(5120, 5376)]}
  _fp8_training_step_vs_oracle(lhs, rhs, g, bands)


@pytest.mark.parametrize('shape', [(2048, 2048, 2048), (384, 4096, 1024)])
def test_fp8_wide_kernel_strict_tolerance(shape):
  """Shapes whose contractions are long enough for the 256 x 512 kernel (2048
  bytes and more), forward and both gradients, every row."""
  m, k, n = shape
  rng = np.random.default_rng(m + n)
  lhs = util.rand_normal(rng, (m, k), 1.0, orc.bfloat16)
  rhs = util.rand_normal(rng, (k, n), k ** -0.5, orc.bfloat16)
  g = util.rand_normal(rng, (m, n), 1.0, orc.bfloat16)
  bands = {'out': [(0, m)], 'dlhs': [(0, m)], 'drhs': [(0, k)]}
  _fp8_training_step_vs_oracle(lhs, rhs, g, bands)


@pytest.mark.parametrize('shape', [(2048, 2048, 2048), (384, 4096, 1024)])
def test_fp8_f32_inputs_strict_tolerance(shape):
  """f32 operands (f32 scales, f32 epilogue), per-tensor fp8, whole result."""
  m, k, n = shape
  rng = np.random.default_rng(m + k)
  lhs = util.rand_normal(rng, (m, k), 1.0, np.float32)
  rhs = util.rand_normal(rng, (k, n), k ** -0.5, np.float32)
  g = util.rand_normal(rng, (m, n), 1.0, np.float32)
  cfg = _per_tensor(config.fully_quantized(
      fwd_bits='e4m3', bwd_bits='e5m2', use_stochastic_rounding=False))
  out, bp = cfg.vjp(_cuda(lhs), _cuda(rhs), DIMS)
  dl, dr = bp(_cuda(g))
  _sync()
  wo, wl, wr, res = orc.dg_fwd_bwd(cfg, lhs, rhs, g, DIMS)
  f = lambda a: np.abs(_f64(a))
  sl, sr_ = f(res.lhs.qx.scale[0]), f(res.rhs.qx.scale[0])
  _fp8_close(out, wo, (f(res.lhs.qx.qvalue) @ f(res.rhs.qx.qvalue)) * sl * sr_,
             'out')
  _fp8_close(dl, wl, 2.0 * ((f(g) * sr_) @ f(rhs / sr_).T) + 1e-30, 'dlhs')
  _fp8_close(dr, wr, 2.0 * (f(lhs / sl).T @ (f(g) * sl)) + 1e-30, 'drhs')


def test_config3_einsum_full_sequence_with_noise():
  """BASELINE config 3 with B*H cut to 1*2: T = S = 2048, D = 128, per-token
  scales, stochastic rounding from four given noise tensors; bit for bit."""
  b, t, h, d = 1, 2048, 2, 128
  rng = np.random.default_rng(3)
  dims = (((3,), (3,)), ((0, 2), (0, 2)))
  q = util.rand_normal(rng, (b, t, h, d), 1.0, orc.bfloat16)
  k = util.rand_normal(rng, (b, t, h, d), 1.0, orc.bfloat16)
  g = util.rand_normal(rng, (b, h, t, t), 1.0, orc.bfloat16)
  cfg = config.fully_quantized(use_stochastic_rounding=True)
  noise_rng = np.random.default_rng(1)
  table = {}

  def noise_fn(shape, key):
    kk = (tuple(shape), int(key[0]), int(key[1]))
    if kk not in table:
      table[kk] = torch.from_numpy(
          (noise_rng.random(shape, np.float32) - 0.5).astype(np.float32)).to(DEV)
    return table[kk]

  for raw in (cfg.dlhs, cfg.drhs):
    raw.dg_quantizer.lhs.numerics.noise_fn = noise_fn
    raw.dg_quantizer.rhs.numerics.noise_fn = noise_fn
  cfg = config.set_context(cfg, key=sr.PRNGKey(1), train_step=None)
  out, bp = cfg.vjp(_cuda(q), _cuda(k), dims)
  dq, dk = bp(_cuda(g))
  _sync()
  wo, wq, wk, _ = orc.dg_fwd_bwd(cfg, q, k, g, dims)
  assert len(table) == 4
  _exact(out, wo, 'scores')
  _exact(dq, wq, 'dq')
  _exact(dk, wk, 'dk')


@pytest.fixture(scope='module')
def serving_weights():
  """Config 4's weights [8192, 28672], frozen once on the device (CONVERT) and
  once by the oracle."""
  kk, n = 8192, 28672
  rng = np.random.default_rng(0)
  w = util.rand_normal(rng, (kk, n), kk ** -0.5, orc.bfloat16)
  cfg = aqt.dot_general_make(lhs_bits=8, rhs_bits=4)
  cfg.fwd.dg_quantizer.rhs.numerics.dtype = utils.int8
  x0 = util.rand_normal(rng, (16, kk), 1.0, orc.bfloat16)
  conv = aqt_flax.AqtDotGeneral(
      cfg, rhs_quant_mode=utils.QuantMode.CONVERT,
      rhs_freeze_mode=aqt_flax.FreezerMode.CALIBRATION_AND_VALUE,
      use_legacy_freezer=False)
  conv(_cuda(x0), _cuda(w), DIMS)
  _sync()
  frozen = conv.variables['aqt']['qrhs']['frozen']
  want = _oracle_quant(cfg.fwd.dg_quantizer.rhs, w, [0])
  return cfg, (frozen, conv.variables), want, (kk, n)


def test_config4_frozen_weights_full_size(serving_weights):
  _, (frozen, _), want, _ = serving_weights
  _exact(frozen.scale[0], want.scale[0], 'weight scales')
  _exact(frozen.qvalue, want.qvalue, 'frozen int4-in-int8 weights')
  assert int(frozen.qvalue.abs().max()) <= 7


@pytest.mark.parametrize('m', [16, 256, 4096])
def test_config4_serving_full_size(serving_weights, m):
  """K = 8192, N = 28672; all of N for M = 16 and 256, a 512-column band of
  the result for M = 4096 (the whole GEMM still runs on the device)."""
  cfg, (_, variables), want_w, (kk, n) = serving_weights
  rng = np.random.default_rng(m)
  x = util.rand_normal(rng, (m, kk), 1.0, orc.bfloat16)
  serve = aqt_flax.AqtDotGeneral(
      cfg, rhs_quant_mode=utils.QuantMode.SERVE,
      rhs_freeze_mode=aqt_flax.FreezerMode.CALIBRATION_AND_VALUE,
      use_legacy_freezer=False, variables=variables)
  dummy_w = torch.empty((kk, n), dtype=torch.bfloat16, device=DEV)
  got = serve(_cuda(x), dummy_w, DIMS)
  _sync()
  cols = slice(0, n) if m <= 256 else slice(14336, 14848)
  o_x = _oracle_quant(cfg.fwd.dg_quantizer.lhs, x, [1])
  acc = orc.dot_general(o_x.qvalue, np.asarray(want_w.qvalue)[:, cols], DIMS,
                        preferred_element_type=orc.int32)
  want = orc.OQTensor(
      qvalue=acc, scale=[o_x.scale[0], want_w.scale[0][:, cols]],
      dequant_dtype=orc.bfloat16).dequant()
  _exact(got[:, cols], want, f'served out M={m}')


# ---------------------------------------------------------------------------
# calibration options of AbsMaxCalibration and the scale dtype


def _with_calibration(cfg, **kw):
  import functools
  from aqt_b200.v2 import calibration
  for raw in (cfg.fwd, cfg.dlhs, cfg.drhs):
    for qz in (raw.dg_quantizer.lhs, raw.dg_quantizer.rhs):
      qz.calibration = functools.partial(calibration.AbsMaxCalibration, **kw)
  return cfg


@pytest.mark.parametrize('np_dtype', [np.float32, orc.bfloat16])
@pytest.mark.parametrize('option', [
    dict(po2_scale=True), dict(clipping_scale=0.3),
    dict(po2_scale=True, clipping_scale=0.1), dict(dtype='float32'),
])
@pytest.mark.parametrize('per_tensor', [False, True])
@pytest.mark.parametrize('shape', [(130, 200, 270), (256, 2048, 512)])
def test_calibration_options_int8_bit_exact(np_dtype, option, per_tensor,
                                            shape):
  """po2_scale, clipping_scale and a scale dtype (f32) different from the
  operands' (bf16), through forward and both gradients."""
  m, k, n = shape
  rng = np.random.default_rng(k)
  lhs = util.rand_normal(rng, (m, k), 1.0, np_dtype)
  rhs = util.rand_normal(rng, (k, n), 0.1, np_dtype)
  g = util.rand_normal(rng, (m, n), 1.0, np_dtype)
  option = dict(option)
  if 'dtype' in option:
    option['dtype'] = utils.float32
  cfg = config.fully_quantized(fwd_bits=8, bwd_bits=8,
                               use_stochastic_rounding=False)
  if per_tensor:
    _per_tensor(cfg)
  _with_calibration(cfg, **option)
  (out, (lq, rq)), vres = aqt.dg_core_vjp_fwd(_cuda(lhs), _cuda(rhs), None,
                                              None, DIMS, cfg)
  dl, dr, *_ = aqt.dg_core_vjp_bwd(DIMS, vres, (_cuda(g), None))
  _sync()
  wo, wl, wr, res = orc.dg_fwd_bwd(cfg, lhs, rhs, g, DIMS)
  _exact(lq.scale[0], res.lhs.qx.scale[0], 's_lhs')
  _exact(rq.scale[0], res.rhs.qx.scale[0], 's_rhs')
  _exact(lq.qvalue, res.lhs.qx.qvalue, 'q_lhs')
  _exact(rq.qvalue, res.rhs.qx.qvalue, 'q_rhs')
  _exact(out, wo, 'out')
  _exact(dl, wl, 'dlhs')
  _exact(dr, wr, 'drhs')


@pytest.mark.parametrize('option', [dict(po2_scale=True),
                                    dict(clipping_scale=0.5),
                                    dict(dtype='float32')])
def test_calibration_options_fp8(option):
  m, k, n = 200, 520, 300
  rng = np.random.default_rng(9)
  lhs = util.rand_normal(rng, (m, k), 1.0, orc.bfloat16)
  rhs = util.rand_normal(rng, (k, n), 0.05, orc.bfloat16)
  option = dict(option)
  if 'dtype' in option:
    option['dtype'] = utils.float32
  cfg = _with_calibration(_per_tensor(config.fully_quantized(
      fwd_bits='e4m3', bwd_bits='e5m2', use_stochastic_rounding=False)),
                          **option)
  (out, (lq, rq)), _ = aqt.dg_core_vjp_fwd(_cuda(lhs), _cuda(rhs), None, None,
                                           DIMS, cfg)
  _sync()
  wo, res = orc.dg_fwd(cfg, lhs, rhs, DIMS)
  _exact(lq.scale[0], res.lhs.qx.scale[0], 's_lhs')
  _exact(rq.scale[0], res.rhs.qx.scale[0], 's_rhs')
  _exact(lq.qvalue, res.lhs.qx.qvalue, 'q_lhs')
  _exact(rq.qvalue, res.rhs.qx.qvalue, 'q_rhs')
  f = lambda a: np.abs(_f64(a))
  _fp8_close(out, wo, (f(res.lhs.qx.qvalue) @ f(res.rhs.qx.qvalue))
             * f(res.lhs.qx.scale[0]) * f(res.rhs.qx.scale[0]), 'out')


def test_f16_operands_are_rejected_with_the_reference_line():
  x = torch.zeros((16, 16), dtype=torch.float16, device=DEV)
  cfg = config.fully_quantized(use_stochastic_rounding=False)
  with pytest.raises(NotImplementedError, match='986-987'):
    cfg(x, x, DIMS)
