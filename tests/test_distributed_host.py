"""world_size-2 gloo test of the row-sharded path (host logic, CPU only).

Two processes each hold half of the rows of lhs and of the cotangent and run
aqt_b200.distributed.ShardedDotGeneral on the numpy stand-in for the shared
library; the gathered result must equal the oracle on the whole problem, bit
for bit: scales that span the sharded rows are max-all-reduced, and the drhs
accumulators are summed across ranks before one dequantization.
"""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from aqt_b200.v2 import config
from oracle import aqt_oracle as orc
from tests import util

DIMS = (((1,), (0,)), ((), ()))


def _make_cfg(kind, per_tensor, use_fwd_quant):
  if kind == 'int8':
    cfg = config.fully_quantized(fwd_bits=8, bwd_bits=8,
                                 use_fwd_quant=use_fwd_quant,
                                 use_stochastic_rounding=False)
  else:
    cfg = config.fully_quantized(fwd_bits='e4m3', bwd_bits='e5m2',
                                 use_fwd_quant=use_fwd_quant,
                                 use_stochastic_rounding=False)
  if per_tensor:
    for raw in (cfg.fwd, cfg.dlhs, cfg.drhs):
      raw.dg_quantizer.lhs.calib_shared_axes = 'per_tensor'
      raw.dg_quantizer.rhs.calib_shared_axes = 'per_tensor'
  return cfg


def _data(np_dtype=np.float32):
  rng = np.random.default_rng(0)
  # bf16 with extents that are multiples of 16 per shard takes the
  # one-read-per-operand path (aqtb200_quantize_pair)
  n = 48 if np_dtype != np.float32 else 40
  lhs = util.rand_normal(rng, (32, 48), 1.0, np_dtype)
  rhs = util.rand_normal(rng, (48, n), 0.2, np_dtype)
  g = util.rand_normal(rng, (32, n), 1.0, np_dtype)
  # make the two shards' maxima differ clearly
  lhs[20, 3] = 7.0
  g[5, 7] = -9.0
  return lhs, rhs, g


def _worker(rank, world, port, kind, per_tensor, use_fwd_quant, ret,
            np_dtype=np.float32, traced=False):
  os.environ['MASTER_ADDR'] = '127.0.0.1'
  os.environ['MASTER_PORT'] = str(port)
  dist.init_process_group('gloo', rank=rank, world_size=world)
  try:
    import unittest.mock as mock
    from aqt_b200 import _lib, engine
    from aqt_b200 import distributed as aqt_dist
    from tests import fake_lib
    fake = fake_lib.FakeLib()
    with mock.patch.object(_lib, 'load', lambda: fake), \
         mock.patch.object(engine, '_stream', lambda: 0), \
         mock.patch.object(engine, '_on_device', lambda *t: True):
      lhs, rhs, g = _data(np_dtype)
      rows = lhs.shape[0] // world
      sl = slice(rank * rows, (rank + 1) * rows)
      kw = {}
      if np_dtype != np.float32:
        # exercise the sliced drhs: reduce-scatter, band dequantization and
        # all-gather per slice (48 rows of drhs = 2 slices x 2 ranks x 12)
        kw = dict(drhs_slices=2, slice_multiple=4)
      op = aqt_dist.ShardedDotGeneral(_make_cfg(kind, per_tensor,
                                                use_fwd_quant), **kw)
      tl, tr, tg = (util.to_torch(lhs[sl]), util.to_torch(rhs),
                    util.to_torch(g[sl]))
      if traced:
        calls = []
        if kw:
          real = op._drhs_sliced
          op._drhs_sliced = lambda *a: calls.append(1) or real(*a)

        def step(a, b, c):
          out, bp = op.vjp(a, b, DIMS)
          return (out,) + tuple(bp(c))

        replay = engine.TracedStep(step, tl, tr, tg)  # verifies itself
        assert not kw or calls, 'the sliced drhs exchange did not run'
        out, dl, dr = replay(tl, tr, tg)
      else:
        out, bp = op.vjp(tl, tr, DIMS)
        dl, dr = bp(tg)
      ret[rank] = (util.to_numpy(out), util.to_numpy(dl), util.to_numpy(dr))
  finally:
    dist.destroy_process_group()


def _free_port():
  s = socket.socket()
  s.bind(('127.0.0.1', 0))
  port = s.getsockname()[1]
  s.close()
  return port


@pytest.mark.parametrize('kind,per_tensor,use_fwd_quant', [
    ('int8', False, True), ('int8', True, True), ('int8', True, False),
    ('fp8', True, True),
])
def test_two_ranks_equal_one_device(kind, per_tensor, use_fwd_quant):
  world = 2
  mgr = mp.Manager()
  ret = mgr.dict()
  mp.spawn(_worker, args=(world, _free_port(), kind, per_tensor,
                          use_fwd_quant, ret), nprocs=world, join=True)
  lhs, rhs, g = _data()
  cfg = _make_cfg(kind, per_tensor, use_fwd_quant)
  wo, wl, wr, _ = orc.dg_fwd_bwd(cfg, lhs, rhs, g, DIMS)
  out = np.concatenate([ret[r][0] for r in range(world)], axis=0)
  dl = np.concatenate([ret[r][1] for r in range(world)], axis=0)
  np.testing.assert_array_equal(out, wo)
  np.testing.assert_array_equal(dl, wl)
  for r in range(world):
    if kind == 'int8':
      np.testing.assert_array_equal(ret[r][2], wr)
    else:  # f32 partial sums are added in a different order
      np.testing.assert_allclose(ret[r][2], wr, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize('traced', [False, True])
def test_two_ranks_paired_quantization_equal_one_device(traced):
  """bf16 / per-tensor fp8: every rank reads each operand once for both of its
  copies; the raw maxima of lhs and of the cotangent are the only things
  agreed across ranks besides the accumulator sum. drhs goes through the
  sliced reduce-scatter / all-gather exchange. `traced`: the step is recorded
  and replayed (engine.TracedStep), collectives included."""
  world = 2
  mgr = mp.Manager()
  ret = mgr.dict()
  mp.spawn(_worker, args=(world, _free_port(), 'fp8', True, True, ret,
                          orc.bfloat16, traced), nprocs=world, join=True)
  lhs, rhs, g = _data(orc.bfloat16)
  cfg = _make_cfg('fp8', True, True)
  wo, wl, wr, _ = orc.dg_fwd_bwd(cfg, lhs, rhs, g, DIMS)
  f32 = lambda a: np.asarray(a, np.float32)
  out = np.concatenate([f32(ret[r][0]) for r in range(world)], axis=0)
  dl = np.concatenate([f32(ret[r][1]) for r in range(world)], axis=0)
  np.testing.assert_array_equal(out, f32(wo))
  np.testing.assert_array_equal(dl, f32(wl))
  for r in range(world):
    # the f32 partial sums of the two ranks are added in a different order
    # than one device's single sum: at most one bf16 ulp after rounding
    got, want = f32(ret[r][2]), f32(wr)
    assert np.all(np.abs(got - want) <= np.abs(want) * 2.0 ** -7 + 1e-6)
