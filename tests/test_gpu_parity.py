"""Parity of the sm_100a path against the CPU oracle, through the C ABI.

int8: quantized values, scales, int32 accumulators and dequantized outputs are
compared bit for bit. fp8: quantized values and scales bit for bit; outputs
within max(1 bf16 ulp of the oracle value, 1e-5 * sum_k |a_k b_k| * scales)
for bf16 outputs and 1e-5 * sum_k |a_k b_k| * scales for f32 outputs, because
the tensor core's f32 accumulation order is not the oracle's (exact sum,
rounded once).
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


def _cuda(a):
  return util.to_torch(a, DEV)


def _sync():
  torch.cuda.synchronize()
  engine.check_status()


def _exact(got, want, what):
  g = util.to_numpy(got)
  assert g.shape == want.shape, (what, g.shape, want.shape)
  assert g.dtype == want.dtype, (what, g.dtype, want.dtype)
  a, b = g.astype(np.float32), want.astype(np.float32)
  bad = a != b
  assert not bad.any(), (
      f'{what}: {int(bad.sum())} of {bad.size} differ; first at '
      f'{np.argwhere(bad)[0].tolist()}: got {a[bad][0]!r} want {b[bad][0]!r}')


def _per_tensor(cfg):
  for raw in (cfg.fwd, cfg.dlhs, cfg.drhs):
    raw.dg_quantizer.lhs.calib_shared_axes = 'per_tensor'
    raw.dg_quantizer.rhs.calib_shared_axes = 'per_tensor'
  return cfg


def _fp8_close(got, want, bound, what):
  """|got-want| <= max(1 bf16 ulp of want [bf16 outputs], 1e-5*bound)."""
  g = util.to_numpy(got)
  assert g.shape == want.shape and g.dtype == want.dtype, what
  a, b = g.astype(np.float64), want.astype(np.float64)
  tol = 1e-5 * bound
  if want.dtype == orc.bfloat16:
    ulp = 2.0 ** (np.floor(np.log2(np.maximum(np.abs(b), 1e-38))) - 7)
    tol = np.maximum(tol, ulp)
  bad = np.abs(a - b) > tol
  assert not bad.any(), (
      f'{what}: {int(bad.sum())} of {bad.size} outside tolerance; worst '
      f'{np.max(np.abs(a - b) / tol):.3g}x')


CASES = [
    ((((1,), (0,)), ((), ())), (12, 40), (40, 24)),
    ((((1,), (0,)), ((), ())), (130, 200), (200, 270)),
    ((((1,), (0,)), ((), ())), (256, 512), (512, 384)),
    ((((3,), (3,)), ((0, 2), (0, 2))), (2, 9, 3, 16), (2, 7, 3, 16)),
    ((((3,), (3,)), ((0, 2), (0, 2))), (2, 160, 3, 128), (2, 272, 3, 128)),
    ((((2,), (1,)), ((0,), (0,))), (3, 5, 32), (3, 32, 6)),
    ((((1,), (1,)), ((), ())), (8, 20), (10, 20)),
    ((((0,), (0,)), ((), ())), (20, 8), (20, 10)),
    ((((2,), (0,)), ((), ())), (4, 6, 32), (32, 12)),
    # kept axes of lhs on both sides of its contraction axis ('bkh,kd->bhd'):
    # no single strided view exists, the planner regroups with copies
    ((((1,), (0,)), ((), ())), (4, 32, 6), (32, 10)),
    ((((1,), (0,)), ((), ())), (4, 6, 6), (6, 5)),
    ((((1,), (0,)), ((), ())), (1, 17), (17, 1)),
]


@pytest.mark.parametrize('dims,ls,rs', CASES)
@pytest.mark.parametrize('np_dtype', [np.float32, orc.bfloat16])
@pytest.mark.parametrize('use_fwd_quant', [True, False])
def test_int8_fwd_bwd_bit_exact(dims, ls, rs, np_dtype, use_fwd_quant):
  rng = np.random.default_rng(0)
  lhs = util.rand_normal(rng, ls, 1.0, np_dtype)
  rhs = util.rand_normal(rng, rs, 0.2, np_dtype)
  cfg = config.fully_quantized(fwd_bits=8, bwd_bits=8,
                               use_fwd_quant=use_fwd_quant,
                               use_stochastic_rounding=False)
  wo, res = orc.dg_fwd(cfg, lhs, rhs, dims)
  g = util.rand_normal(rng, wo.shape, 1.0, np_dtype)
  wl, wr = orc.dg_bwd(cfg, dims, res, g)
  (out, (lq, rq)), vres = aqt.dg_core_vjp_fwd(_cuda(lhs), _cuda(rhs), None,
                                              None, dims, cfg)
  dl, dr, *_ = aqt.dg_core_vjp_bwd(dims, vres, (_cuda(g), None))
  _sync()
  _exact(lq.qvalue, res.lhs.qx.qvalue, 'q_lhs')
  _exact(rq.qvalue, res.rhs.qx.qvalue, 'q_rhs')
  _exact(lq.scale[0], res.lhs.qx.scale[0], 's_lhs')
  _exact(rq.scale[0], res.rhs.qx.scale[0], 's_rhs')
  _exact(out, wo, 'out')
  _exact(dl, wl, 'dlhs')
  _exact(dr, wr, 'drhs')


@pytest.mark.parametrize('np_dtype', [np.float32, orc.bfloat16])
@pytest.mark.parametrize('shape', [(256, 512, 384), (130, 200, 270)])
def test_int8_per_tensor_fwd_bwd_bit_exact(np_dtype, shape):
  # per-tensor scales: the stored int8 operands are re-quantized in the
  # backward pass by a byte -> byte table (one scale, one prescale)
  m, k, n = shape
  rng = np.random.default_rng(11)
  dims = (((1,), (0,)), ((), ()))
  lhs = util.rand_normal(rng, (m, k), 1.0, np_dtype)
  rhs = util.rand_normal(rng, (k, n), 0.2, np_dtype)
  g = util.rand_normal(rng, (m, n), 1.0, np_dtype)
  cfg = _per_tensor(config.fully_quantized(fwd_bits=8, bwd_bits=8,
                                           use_stochastic_rounding=False))
  wo, wl, wr, _ = orc.dg_fwd_bwd(cfg, lhs, rhs, g, dims)
  out, bp = cfg.vjp(_cuda(lhs), _cuda(rhs), dims)
  dl, dr = bp(_cuda(g))
  _sync()
  _exact(out, wo, 'out')
  _exact(dl, wl, 'dlhs')
  _exact(dr, wr, 'drhs')


@pytest.mark.parametrize('bits', [2, 4, 8])
@pytest.mark.parametrize('shape', [(64, 256, 96), (130, 200, 270), (5, 33, 7)])
def test_int_accumulators_bit_exact(bits, shape):
  m, k, n = shape
  rng = np.random.default_rng(bits)
  dims = (((1,), (0,)), ((), ()))
  lhs = util.rand_normal(rng, (m, k), 1.0, np.float32)
  rhs = util.rand_normal(rng, (k, n), 1.0, np.float32)
  raw = aqt.dot_general_raw_make(bits, bits)
  raw.dg_quantizer.lhs.numerics.dtype = utils.int8
  raw.dg_quantizer.rhs.numerics.dtype = utils.int8
  wo, _, wacc = orc.dg_raw(raw, lhs, rhs, None, None, dims, return_acc=True)
  out, _, acc = engine.dg_raw(raw, _cuda(lhs), _cuda(rhs), None, None, dims,
                              want_acc=True)
  _sync()
  _exact(acc.reshape(m, n), wacc, 'acc')
  _exact(out, wo, 'out')


def test_tensor_core_kernel_agrees_with_cuda_core_kernel():
  rng = np.random.default_rng(5)
  dims = (((1,), (0,)), ((), ()))
  lhs = _cuda(util.rand_normal(rng, (300, 1000), 1.0, np.float32))
  rhs = _cuda(util.rand_normal(rng, (1000, 520), 1.0, np.float32))
  raw = aqt.dot_general_raw_make(8, 8)
  a = engine.dg_raw(raw, lhs, rhs, None, None, dims, want_acc=True)
  engine.set_gemm_impl('simt')
  try:
    b = engine.dg_raw(raw, lhs, rhs, None, None, dims, want_acc=True)
  finally:
    engine.set_gemm_impl('tcgen05')
  _sync()
  assert torch.equal(a[2], b[2]) and torch.equal(a[0], b[0])


@pytest.mark.parametrize('fwd,bwd', [('e4m3', 'e5m2'), ('e5m2', 'e4m3'),
                                     (8, 8), (4, 8)])
@pytest.mark.parametrize('shape', [(256, 512, 384), (16, 16, 16),
                                   (272, 1040, 48)])
def test_paired_quantization_equals_one_quantization_per_dot(monkeypatch, fwd,
                                                             bwd, shape):
  """aqtb200_quantize_pair / aqtb200_requant_amax (one read per operand) give
  bit for bit what the reference's flow gives: each dot calibrating and
  quantizing its own operands, the stored ones re-read in the backward pass."""
  m, k, n = shape
  rng = np.random.default_rng(m + k)
  dims = (((1,), (0,)), ((), ()))
  lhs = _cuda(util.rand_normal(rng, (m, k), 1.0, orc.bfloat16))
  rhs = _cuda(util.rand_normal(rng, (k, n), 0.05, orc.bfloat16))
  g = _cuda(util.rand_normal(rng, (m, n), 1.0, orc.bfloat16))
  cfg = config.fully_quantized(fwd_bits=fwd, bwd_bits=bwd,
                               use_stochastic_rounding=False)
  _per_tensor(cfg)

  def run():
    (out, (lq, rq)), vres = aqt.dg_core_vjp_fwd(lhs, rhs, None, None, dims, cfg)
    dl, dr, *_ = aqt.dg_core_vjp_bwd(dims, vres, (g, None))
    _sync()
    return out, lq.qvalue, rq.qvalue, lq.scale[0], rq.scale[0], dl, dr

  calls = []
  real = engine._quantize_pair
  monkeypatch.setattr(engine, '_quantize_pair',
                      lambda *a, **kw: calls.append(kw.get('chain')) or real(*a, **kw))
  paired = run()
  assert calls == [1, 2, 0]
  monkeypatch.setattr(engine, 'prequantize_for_training', lambda *a: None)
  monkeypatch.setattr(engine, 'cotangent_pair', lambda *a: None)
  single = run()
  for a, b, what in zip(paired, single, ('out', 'q_lhs', 'q_rhs', 's_lhs',
                                         's_rhs', 'dlhs', 'drhs')):
    assert a.shape == b.shape, what
    assert torch.equal(a.contiguous().view(torch.uint8),
                       b.contiguous().view(torch.uint8)), what


@pytest.mark.parametrize('impl', ['cta1', 'cta2', 'wide'])
@pytest.mark.parametrize('shape', [
    (300, 1000, 520),    # ragged everywhere; second 256-column half partly filled
    (256, 2048, 512),    # exact tiles
    (130, 144, 200),     # one 512-column tile whose second half is empty
    (513, 4096, 1030),   # several tiles per pair, long contraction
    (64, 256, 256),      # fewer rows than a tile
])
@pytest.mark.parametrize('np_dtype', [np.float32, orc.bfloat16])
def test_every_tensor_core_kernel_agrees_with_cuda_core_kernel(impl, shape,
                                                               np_dtype):
  m, k, n = shape
  rng = np.random.default_rng(m + n)
  dims = (((1,), (0,)), ((), ()))
  lhs = _cuda(util.rand_normal(rng, (m, k), 1.0, np_dtype))
  rhs = _cuda(util.rand_normal(rng, (k, n), 1.0, np_dtype))
  raw = aqt.dot_general_raw_make(8, 8)
  try:
    engine.set_gemm_impl(impl)
    a = engine.dg_raw(raw, lhs, rhs, None, None, dims, want_acc=True)
    engine.set_gemm_impl('simt')
    b = engine.dg_raw(raw, lhs, rhs, None, None, dims, want_acc=True)
  finally:
    engine.set_gemm_impl('tcgen05')
  _sync()
  assert torch.equal(a[2], b[2]), 'int32 accumulators'
  assert torch.equal(a[0], b[0]), 'dequantized output'


@pytest.mark.parametrize('shape', [(16, 512, 1024), (1, 256, 4096),
                                   (64, 1040, 520), (40, 144, 2048),
                                   # long contractions: tiles that straddle
                                   # the CTAs' equal shares of the k-slabs are
                                   # computed in 2 to 5 parts, summed by the
                                   # part that finishes last
                                   (16, 4096, 2048), (33, 8192, 1000),
                                   (64, 2048, 4736), (16, 2048, 28672),
                                   (48, 8192, 3584)])
@pytest.mark.parametrize('np_dtype', [np.float32, orc.bfloat16])
def test_skinny_lhs_uses_narrow_mmas_and_agrees(shape, np_dtype):
  """A few rows against many: the planner puts the many on the tile's row side
  and the kernel issues MMAs as wide as the few."""
  m, k, n = shape
  rng = np.random.default_rng(m * n)
  dims = (((1,), (0,)), ((), ()))
  lhs = _cuda(util.rand_normal(rng, (m, k), 1.0, np_dtype))
  rhs = _cuda(util.rand_normal(rng, (k, n), 1.0, np_dtype))
  raw = aqt.dot_general_raw_make(8, 8)
  try:
    a = engine.dg_raw(raw, lhs, rhs, None, None, dims, want_acc=True)
    engine.set_gemm_impl('simt')
    b = engine.dg_raw(raw, lhs, rhs, None, None, dims, want_acc=True)
  finally:
    engine.set_gemm_impl('tcgen05')
  _sync()
  assert torch.equal(a[2], b[2]), 'int32 accumulators'
  assert torch.equal(a[0], b[0]), 'dequantized output'
  want, _ = orc.dg_raw(raw, util.to_numpy(lhs), util.to_numpy(rhs), None, None,
                       dims)
  _exact(a[0], want, 'out vs oracle')


def test_skinny_fp8_with_split_contraction():
  """fp8 through the split contraction: parts are added in part order."""
  m, k, n = 16, 8192, 2048
  rng = np.random.default_rng(21)
  dims = (((1,), (0,)), ((), ()))
  lhs = util.rand_normal(rng, (m, k), 1.0, orc.bfloat16)
  rhs = util.rand_normal(rng, (k, n), 0.02, orc.bfloat16)
  raw = aqt.dot_general_raw_make('e4m3', 'e4m3')
  got, res, acc = engine.dg_raw(raw, _cuda(lhs), _cuda(rhs), None, None, dims,
                                want_acc=True)
  _sync()
  want, wres = orc.dg_raw(raw, lhs, rhs, None, None, dims)
  _exact(res.lhs.mt.qx.qvalue, wres.lhs.qx.qvalue, 'q_lhs')
  f = lambda a: np.abs(np.asarray(a).astype(np.float32).astype(np.float64))
  mag = f(wres.lhs.qx.qvalue) @ f(wres.rhs.qx.qvalue)
  exact = (np.asarray(wres.lhs.qx.qvalue).astype(np.float64) @
           np.asarray(wres.rhs.qx.qvalue).astype(np.float64))
  a = util.to_numpy(acc.reshape(m, n)).astype(np.float64)
  assert (np.abs(a - exact) <= 1e-5 * mag + 1e-30).all()
  _fp8_close(got, want, mag * f(wres.lhs.qx.scale[0]) * f(wres.rhs.qx.scale[0])
             , 'out')


@pytest.mark.parametrize('k', [16, 32, 64, 128])
@pytest.mark.parametrize('np_dtype', [np.float32, orc.bfloat16])
def test_short_contraction_rows(k, np_dtype):
  """Rows of at most 32 sixteen-byte vectors take the several-rows-per-warp
  absmax kernel; batched, as the attention-score einsum uses it."""
  rng = np.random.default_rng(k)
  dims = (((3,), (3,)), ((0, 2), (0, 2)))
  lhs = util.rand_normal(rng, (2, 70, 3, k), 1.0, np_dtype)
  rhs = util.rand_normal(rng, (2, 50, 3, k), 1.0, np_dtype)
  lhs[1, 5, 2, :] = 0  # an all-zero row: scale 1
  raw = aqt.dot_general_raw_make(8, 8)
  got, res = engine.dg_raw(raw, _cuda(lhs), _cuda(rhs), None, None, dims)
  _sync()
  want, wres = orc.dg_raw(raw, lhs, rhs, None, None, dims)
  _exact(res.lhs.mt.qx.scale[0], wres.lhs.qx.scale[0], 's_lhs')
  _exact(res.rhs.mt.qx.scale[0], wres.rhs.qx.scale[0], 's_rhs')
  _exact(res.lhs.mt.qx.qvalue, wres.lhs.qx.qvalue, 'q_lhs')
  _exact(got, want, 'out')


@pytest.mark.parametrize('k', [16, 64, 256])
@pytest.mark.parametrize('bits', [8, 4, 'e4m3', 'e5m2'])
def test_short_rows_quantized_in_one_pass(k, bits):
  """bf16 rows of at most 32 vectors, contraction axis last: calibrated and
  quantized by one kernel in packed bf16 arithmetic; values and scales bit for
  bit for every numerics."""
  rng = np.random.default_rng(k + 7)
  dims = (((3,), (3,)), ((0, 2), (0, 2)))
  lhs = util.rand_normal(rng, (2, 150, 3, k), 1.0, orc.bfloat16)
  rhs = util.rand_normal(rng, (2, 90, 3, k), 3.0, orc.bfloat16)
  lhs[0, 7, 1, :] = 0
  raw = aqt.dot_general_raw_make(bits, bits)
  _, res = engine.dg_raw(raw, _cuda(lhs), _cuda(rhs), None, None, dims)
  _sync()
  _, wres = orc.dg_raw(raw, lhs, rhs, None, None, dims)
  for side in ('lhs', 'rhs'):
    g, w = getattr(res, side).mt.qx, getattr(wres, side).qx
    _exact(g.scale[0], w.scale[0], 's_' + side)
    _exact(g.qvalue, w.qvalue, 'q_' + side)


@pytest.mark.parametrize('world,np_dtype', [(2, orc.bfloat16), (4, orc.bfloat16),
                                            (8, orc.bfloat16), (4, np.float32)])
@pytest.mark.parametrize('bits', [8, 'e4m3'])
@pytest.mark.parametrize('per_tensor', [True, False])
def test_fused_exchange_kernel_on_one_device(world, np_dtype, bits, per_tensor):
  """aqtb200_dot_general_raw_exchange with every "rank's" accumulators and
  result on this one GPU (the kernel does not care whose memory a pointer
  names): the bands are added in rank order, dequantized once and written to
  every result, bit for bit what the band dequantization gives on the sum."""
  rng = np.random.default_rng(world)
  dims = (((1,), (0,)), ((), ()))
  m, k, n = 384, 256, 520
  lhs = _cuda(util.rand_normal(rng, (m, k), 1.0, np_dtype))
  rhs = _cuda(util.rand_normal(rng, (k, n), 0.1, np_dtype))
  raw = aqt.dot_general_raw_make(bits, bits)
  if per_tensor:
    raw.dg_quantizer.lhs.calib_shared_axes = 'per_tensor'
    raw.dg_quantizer.rhs.calib_shared_axes = 'per_tensor'
  # f32 operands take the kernel's general arithmetic (f32 chain and results),
  # bf16 operands the packed bf16 one
  d, _ = engine.dg_raw(raw, lhs, rhs, None, None, dims, defer_dequant=True)
  _sync()
  acc0 = d.acc
  rows = acc0.shape[1]
  if acc0.dtype == torch.int32:
    accs = [(acc0 * (r + 1) - 7 * r).contiguous() for r in range(world)]
    total = accs[0].clone()
    for a in accs[1:]:
      total += a
  else:
    accs = [(acc0 * (0.5 + 0.37 * r)).contiguous() for r in range(world)]
    total = accs[0].clone()
    for a in accs[1:]:  # rank order, one f32 rounding per addition
      total = total + a
  want = d.finish_rows(0, rows, total.reshape(rows, -1)).clone()
  outs = [torch.full_like(want, float('nan')) for _ in range(world)]
  d.exchange_rows(0, rows, world - 1, [a.data_ptr() for a in accs],
                  [o.data_ptr() for o in outs], max_sms=8)
  _sync()
  engine.check_status()
  bits_of = torch.int16 if want.dtype == torch.bfloat16 else torch.int32
  for r, o in enumerate(outs):
    assert torch.equal(o.view(bits_of), want.view(bits_of)), 'copy %d differs' % r
  # a band in the middle, the rest untouched
  outs = [torch.zeros_like(want) for _ in range(world)]
  start, count = 128, 64
  acc_row, out_row = d.band_stride_bytes()
  d.exchange_rows(start, count, 0,
                  [a.data_ptr() + start * acc_row for a in accs],
                  [o.data_ptr() + start * out_row for o in outs])
  _sync()
  full = want if want.shape[0] == rows else want.t()
  for o in outs:
    ob = o if o.shape[0] == rows else o.t()
    assert torch.equal(ob[start:start + count], full[start:start + count])
    assert not ob[:start].any() and not ob[start + count:].any()


def test_wide_kernel_batched_and_transposed_output():
  """The 256 x 512 kernel under batch dims and the drhs output transpose."""
  rng = np.random.default_rng(11)
  dims = (((2,), (2,)), ((0,), (0,)))
  lhs = _cuda(util.rand_normal(rng, (3, 260, 384), 1.0, orc.bfloat16))
  rhs = _cuda(util.rand_normal(rng, (3, 530, 384), 1.0, orc.bfloat16))
  raw = aqt.dot_general_raw_make(8, 8)
  try:
    engine.set_gemm_impl('wide')
    a = engine.dg_raw(raw, lhs, rhs, None, None, dims, want_acc=True,
                      out_transpose_axes=(0, 2, 1))
    engine.set_gemm_impl('simt')
    b = engine.dg_raw(raw, lhs, rhs, None, None, dims, want_acc=True,
                      out_transpose_axes=(0, 2, 1))
  finally:
    engine.set_gemm_impl('tcgen05')
  _sync()
  assert torch.equal(a[2], b[2]) and torch.equal(a[0], b[0])


@pytest.mark.parametrize('impl', ['cta1', 'cta2', 'wide', 'simt'])
@pytest.mark.parametrize('shape', [(300, 2048, 1030), (256, 2048, 512),
                                   (64, 256, 256)])
@pytest.mark.parametrize('np_dtype', [np.float32, orc.bfloat16])
def test_amax_out_is_the_maximum_of_the_output(impl, shape, np_dtype):
  """The optional amax_out of the GEMM epilogues: max |out| over what was
  stored, ragged edges left out."""
  m, k, n = shape
  rng = np.random.default_rng(m + k)
  dims = (((1,), (0,)), ((), ()))
  lhs = _cuda(util.rand_normal(rng, (m, k), 1.0, np_dtype))
  rhs = _cuda(util.rand_normal(rng, (k, n), 1.0, np_dtype))
  raw = aqt.dot_general_raw_make(8, 8)
  amax = torch.zeros(1, dtype=torch.float32, device=DEV)
  try:
    engine.set_gemm_impl(impl)
    out, _ = engine.dg_raw(raw, lhs, rhs, None, None, dims, amax_out=amax)
  finally:
    engine.set_gemm_impl('tcgen05')
  _sync()
  assert amax.item() == out.float().abs().max().item()


@pytest.mark.parametrize('kind', ['int8', 'fp8'])
@pytest.mark.parametrize('shape', [(300, 2048, 1032), (512, 4096, 512)])
def test_wide_kernel_raw_accumulators_and_band_dequantization(kind, shape):
  """The 256 x 512 kernel writing raw accumulators only (the form a sharded
  contraction sums across ranks), then the dequantizing pass over them, whole
  and by bands of rows."""
  m, k, n = shape
  rng = np.random.default_rng(n)
  dims = (((1,), (0,)), ((), ()))
  lhs = _cuda(util.rand_normal(rng, (m, k), 1.0, orc.bfloat16))
  rhs = _cuda(util.rand_normal(rng, (k, n), 1.0, orc.bfloat16))
  raw = aqt.dot_general_raw_make(8, 8) if kind == 'int8' else (
      aqt.dot_general_raw_make('e4m3', 'e4m3'))
  try:
    engine.set_gemm_impl('wide')
    want, _ = engine.dg_raw(raw, lhs, rhs, None, None, dims)
    d, _ = engine.dg_raw(raw, lhs, rhs, None, None, dims, defer_dequant=True)
    engine.set_gemm_impl('simt')
    _, _, acc_simt = engine.dg_raw(raw, lhs, rhs, None, None, dims,
                                   want_acc=True)
  finally:
    engine.set_gemm_impl('tcgen05')
  acc = d.acc.reshape(m, n).clone()
  whole = d.finish().clone()
  _sync()
  if kind == 'int8':
    assert torch.equal(acc, acc_simt.reshape(m, n))
  else:  # the CUDA-core kernel sums in f64; bound: sum |a_k||b_k| of the
    # quantized operands the accumulators are made of
    res = engine.dg_raw(raw, lhs, rhs, None, None, dims)[1]
    bound = (res.lhs.mt.qx.qvalue.float().abs() @
             res.rhs.mt.qx.qvalue.float().abs())
    assert ((acc - acc_simt.reshape(m, n)).abs() <= 1e-5 * bound + 1e-30).all()
  assert torch.equal(whole, want)
  # bands: rows [0, 128) and [128, m) from copies of the accumulator rows
  d._out.zero_()
  d.finish_rows(0, 128, acc[:128].contiguous())
  d.finish_rows(128, m - 128, acc[128:].contiguous())
  _sync()
  assert torch.equal(d._out, want)


def test_mma_peak_kernel_runs():
  from aqt_b200 import _lib
  lib = _lib.load()
  status = torch.zeros(4, dtype=torch.int32, device=DEV)
  for is_int in (1, 0):
    rc = lib.aqtb200_mma_peak(is_int, 4096, status.data_ptr(),
                              torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.aqtb200_last_error()
  torch.cuda.synchronize()
  assert status[0].item() == 0


@pytest.mark.parametrize('fwd,bwd', [('e4m3', 'e5m2'), ('e4m3', 'e4m3'),
                                     ('e5m2', 'e5m2')])
@pytest.mark.parametrize('np_dtype', [np.float32, orc.bfloat16])
@pytest.mark.parametrize('per_tensor', [True, False])
def test_fp8_fwd_bwd(fwd, bwd, np_dtype, per_tensor):
  rng = np.random.default_rng(1)
  dims = (((1,), (0,)), ((), ()))
  m, k, n = 200, 520, 300
  lhs = util.rand_normal(rng, (m, k), 1.0, np_dtype)
  rhs = util.rand_normal(rng, (k, n), 0.05, np_dtype)
  g = util.rand_normal(rng, (m, n), 1.0, np_dtype)
  cfg = config.fully_quantized(fwd_bits=fwd, bwd_bits=bwd,
                               use_stochastic_rounding=False)
  if per_tensor:
    _per_tensor(cfg)
  wo, wl, wr, res = orc.dg_fwd_bwd(cfg, lhs, rhs, g, dims)
  (out, (lq, rq)), vres = aqt.dg_core_vjp_fwd(_cuda(lhs), _cuda(rhs), None,
                                              None, dims, cfg)
  dl, dr, *_ = aqt.dg_core_vjp_bwd(dims, vres, (_cuda(g), None))
  _sync()
  _exact(lq.qvalue, res.lhs.qx.qvalue, 'q_lhs')
  _exact(rq.qvalue, res.rhs.qx.qvalue, 'q_rhs')
  _exact(lq.scale[0], res.lhs.qx.scale[0], 's_lhs')
  _exact(rq.scale[0], res.rhs.qx.scale[0], 's_rhs')
  f = lambda a: np.abs(np.asarray(a).astype(np.float64))
  ql, qr = f(res.lhs.qx.qvalue), f(res.rhs.qx.qvalue)
  sl, sr_ = f(res.lhs.qx.scale[0]), f(res.rhs.qx.scale[0])
  _fp8_close(out, wo, (ql @ qr) * sl * sr_, 'out')
  # gradients: bound from the magnitudes of the operands of each dot
  gl = f(g) * sr_  # |g * s_rhs|
  _fp8_close(dl, wl, 2.0 * (gl @ f(rhs / np.maximum(sr_, 1e-30)).T) + 1e-30,
             'dlhs')
  gr = f(g) * sl
  _fp8_close(dr, wr, 2.0 * (f(lhs / np.maximum(sl, 1e-30)).T @ gr) + 1e-30,
             'drhs')


def test_stochastic_rounding_with_given_noise_bit_exact():
  rng = np.random.default_rng(3)
  dims = (((3,), (3,)), ((0, 2), (0, 2)))
  q = util.rand_normal(rng, (2, 48, 3, 64), 1.0, orc.bfloat16)
  k = util.rand_normal(rng, (2, 40, 3, 64), 1.0, orc.bfloat16)
  g = util.rand_normal(rng, (2, 3, 48, 40), 1.0, orc.bfloat16)
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


def test_einsum_attention_scores():
  rng = np.random.default_rng(4)
  q = util.rand_normal(rng, (2, 256, 4, 128), 1.0, orc.bfloat16)
  k = util.rand_normal(rng, (2, 320, 4, 128), 1.0, orc.bfloat16)
  cfg = config.fully_quantized(use_stochastic_rounding=False)
  got = aqt_flax.AqtEinsum(cfg)('bthd,bshd->bhts', _cuda(q), _cuda(k))
  _sync()
  want, _ = orc.dg_fwd(cfg, q, k, (((3,), (3,)), ((0, 2), (0, 2))))
  _exact(got, want, 'scores')


@pytest.mark.parametrize('m', [16, 64, 256])
def test_serving_int4_weights_in_int8_container(m):
  # activations int8 per token, weights 4-bit values stored as int8 with a
  # per-output-channel scale, fed back as a frozen QTensor.
  rng = np.random.default_rng(6)
  k, n = 1024, 768
  dims = (((1,), (0,)), ((), ()))
  x = util.rand_normal(rng, (m, k), 1.0, orc.bfloat16)
  w = util.rand_normal(rng, (k, n), 1.0 / 32, orc.bfloat16)
  cfg = aqt.dot_general_make(lhs_bits=8, rhs_bits=4)
  cfg.fwd.dg_quantizer.rhs.numerics.dtype = utils.int8
  both = aqt_flax.FreezerMode.CALIBRATION_AND_VALUE
  conv = aqt_flax.AqtDotGeneral(cfg, rhs_quant_mode=utils.QuantMode.CONVERT,
                                rhs_freeze_mode=both, use_legacy_freezer=False)
  train_out = conv(_cuda(x), _cuda(w), dims)
  frozen = conv.variables['aqt']['qrhs']['frozen']
  _sync()
  want, res = orc.dg_fwd(cfg, x, w, dims)
  _exact(frozen.qvalue, res.rhs.qx.qvalue, 'frozen weights')
  assert int(frozen.qvalue.abs().max()) <= 7
  _exact(train_out, want, 'train-mode out')
  serve = aqt_flax.AqtDotGeneral(cfg, rhs_quant_mode=utils.QuantMode.SERVE,
                                 rhs_freeze_mode=both, use_legacy_freezer=False,
                                 variables=conv.variables)
  got = serve(_cuda(x), torch.zeros_like(_cuda(w)), dims)
  _sync()
  _exact(got, want, 'served out')
  # the legacy two-variable layout ('value', 'scale' in the output's layout)
  conv2 = aqt_flax.AqtDotGeneral(cfg, rhs_quant_mode=utils.QuantMode.CONVERT,
                                 rhs_freeze_mode=both)
  conv2(_cuda(x), _cuda(w), dims)
  serve2 = aqt_flax.AqtDotGeneral(cfg, rhs_quant_mode=utils.QuantMode.SERVE,
                                  rhs_freeze_mode=both,
                                  variables=conv2.variables)
  got2 = serve2(_cuda(x), torch.zeros_like(_cuda(w)), dims)
  _sync()
  _exact(got2, want, 'served out (legacy freezer)')


def test_piecewise_quantizer_api():
  rng = np.random.default_rng(7)
  x = util.rand_normal(rng, (96, 200), 3.0, np.float32)
  from aqt_b200.v2 import aqt_quantizer
  for axes in ([1], [0], [0, 1]):
    qz = aqt_quantizer.quantizer_make(8)
    if len(axes) == 2:
      qz.calib_shared_axes = 'per_tensor'
    qt, _ = qz.quant(_cuda(x), calibration_axes=axes)
    _sync()
    oq = orc.quantizer_calculate_qvalue(
        qz, x, orc.quantizer_calibrate(qz, x, axes))
    _exact(qt.scale[0], oq.scale[0], f'scale axes={axes}')
    _exact(qt.qvalue, oq.qvalue, f'qvalue axes={axes}')
    _exact(qt.dequant(), oq.dequant(), f'dequant axes={axes}')


def test_config1_full_size_bit_exact():
  # BASELINE config 1: f32 [1024,4096] x [4096,4096], int8 per-channel, RNE.
  rng = np.random.default_rng(0)
  dims = (((1,), (0,)), ((), ()))
  lhs = util.rand_normal(rng, (1024, 4096), 1.0, np.float32)
  rhs = util.rand_normal(rng, (4096, 4096), 1.0 / 64, np.float32)
  g = util.rand_normal(rng, (1024, 4096), 1.0, np.float32)
  cfg = config.fully_quantized(fwd_bits=8, bwd_bits=8,
                               use_stochastic_rounding=False)
  out, bp = cfg.vjp(_cuda(lhs), _cuda(rhs), dims)
  dl, dr = bp(_cuda(g))
  _sync()
  wo, wl, wr, _ = orc.dg_fwd_bwd(cfg, lhs, rhs, g, dims)
  _exact(out, wo, 'out')
  _exact(dl, wl, 'dlhs')
  _exact(dr, wr, 'drhs')


@pytest.mark.parametrize('kind', ['int8', 'fp8'])
def test_full_size_checksum_8192(kind):
  # Size-independent property at BASELINE config 2's size: the sum of all
  # accumulators equals dot(column sums of A, column sums of B).
  torch.manual_seed(0)
  n = 8192
  dims = (((1,), (0,)), ((), ()))
  lhs = torch.randn(n, n, device=DEV, dtype=torch.bfloat16)
  rhs = torch.randn(n, n, device=DEV, dtype=torch.bfloat16) * (n ** -0.5)
  raw = aqt.dot_general_raw_make(8, 8) if kind == 'int8' else (
      aqt.dot_general_raw_make('e4m3', 'e4m3'))
  raw.dg_quantizer.lhs.calib_shared_axes = 'per_tensor'
  raw.dg_quantizer.rhs.calib_shared_axes = 'per_tensor'
  out, res, acc = engine.dg_raw(raw, lhs, rhs, None, None, dims, want_acc=True)
  _sync()
  qa = res.lhs.mt.qx.qvalue.to(torch.float64)
  qb = res.rhs.mt.qx.qvalue.to(torch.float64)
  want = torch.dot(qa.sum(0), qb.sum(1))
  got = acc.to(torch.float64).sum()
  if kind == 'int8':
    assert got.item() == want.item()
  else:
    ref = torch.dot(qa.abs().sum(0), qb.abs().sum(1)).item()
    assert abs(got.item() - want.item()) <= 1e-6 * ref
  # and a band of rows against an exact product of the same quantized operands
  rows = slice(4000, 4032)
  exact = qa[rows] @ qb
  if kind == 'int8':
    assert torch.equal(acc.reshape(n, n)[rows].to(torch.float64), exact)
  else:
    bound = qa[rows].abs() @ qb.abs()
    assert ((acc.reshape(n, n)[rows].to(torch.float64) - exact).abs()
            <= 1e-5 * bound).all()


@pytest.mark.parametrize('dims,ls,rs', [
    ((((1,), (0,)), ((), ())), (272, 64), (64, 400)),
    ((((3,), (3,)), ((0, 2), (0, 2))), (2, 144, 3, 32), (2, 304, 3, 32)),
    ((((2,), (1,)), ((0,), (0,))), (3, 16, 32), (3, 32, 48)),
])
@pytest.mark.parametrize('use_fwd_quant', [True, False])
@pytest.mark.parametrize('noise', [False, True])
def test_cotangent_two_pass_quantization_bit_exact(monkeypatch, dims, ls, rs,
                                                   use_fwd_quant, noise):
  """aqtb200_quantize_dual (per-row scales, forward scales folded in, optional
  noise; ragged 128 x 128 tiles) against the oracle's one-dot-at-a-time flow."""
  calls = []
  real = engine.cotangent_dual
  monkeypatch.setattr(engine, 'cotangent_dual',
                      lambda *a: calls.append(real(*a)) or calls[-1])
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
            (rng.random(shape, np.float32) - 0.5).astype(np.float32)).to(DEV)
      return table[kk]

    for raw in (cfg.dlhs, cfg.drhs):
      raw.dg_quantizer.lhs.numerics.noise_fn = noise_fn
      raw.dg_quantizer.rhs.numerics.noise_fn = noise_fn
    cfg = config.set_context(cfg, key=sr.PRNGKey(1), train_step=None)
  wo, res = orc.dg_fwd(cfg, lhs, rhs, dims)
  g = util.rand_normal(rng, wo.shape, 1.0, orc.bfloat16)
  out, bp = cfg.vjp(_cuda(lhs), _cuda(rhs), dims)
  dl, dr = bp(_cuda(g))
  _sync()
  assert calls and calls[0] is not None, 'the two-pass path did not run'
  wl, wr = orc.dg_bwd(cfg, dims, res, g)
  _exact(out, wo, 'out')
  _exact(dl, wl, 'dlhs')
  _exact(dr, wr, 'drhs')


@pytest.mark.parametrize('bad', [float('nan'), float('inf')])
@pytest.mark.parametrize('np_dtype', [np.float32, orc.bfloat16])
@pytest.mark.parametrize('per_tensor', [False, True])
def test_nan_and_inf_reach_the_scale_whatever_the_kernel_variant(
    bad, np_dtype, per_tensor):
  """jnp.max(jnp.abs(x)) keeps a NaN; so must every absmax kernel: the
  16-byte-vector ones (aligned view), the scalar ones (a view that starts one
  element in), row-wise and column-wise."""
  from aqt_b200.v2 import aqt_quantizer
  rng = np.random.default_rng(12)
  base = util.rand_normal(rng, (64, 130), 1.0, np_dtype)
  base[5, 17] = bad
  base[40, 3] = bad
  for view in (lambda a: a[:, :128], lambda a: a[:, 1:129],
               lambda a: a[:32, 2:66]):
    for axes in ([1], [0]):
      x = np.ascontiguousarray(view(base))
      t = view(_cuda(base))  # strided, possibly misaligned view of the parent
      qz = aqt_quantizer.quantizer_make(8)
      if per_tensor:
        qz.calib_shared_axes = 'per_tensor'
      got = qz.calibrate(t, calibration_axes=axes)
      _sync()
      want = orc.quantizer_calibrate(qz, x, axes)
      g = util.to_numpy(got.scale[0]).astype(np.float32)
      w = want.scale[0].astype(np.float32)
      assert g.shape == w.shape
      assert np.array_equal(np.isnan(g), np.isnan(w)), (axes, g, w)
      np.testing.assert_array_equal(g[~np.isnan(g)], w[~np.isnan(w)])
