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


def _data():
  rng = np.random.default_rng(0)
  lhs = util.rand_normal(rng, (32, 48), 1.0, np.float32)
  rhs = util.rand_normal(rng, (48, 40), 0.2, np.float32)
  g = util.rand_normal(rng, (32, 40), 1.0, np.float32)
  # make the two shards' maxima differ clearly
  lhs[20, 3] = 7.0
  g[5, 7] = -9.0
  return lhs, rhs, g


def _worker(rank, world, port, kind, per_tensor, use_fwd_quant, ret):
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
         mock.patch.object(engine, '_HOST_TEST_MODE', True):
      lhs, rhs, g = _data()
      rows = lhs.shape[0] // world
      sl = slice(rank * rows, (rank + 1) * rows)
      op = aqt_dist.ShardedDotGeneral(_make_cfg(kind, per_tensor,
                                                use_fwd_quant))
      out, bp = op.vjp(util.to_torch(lhs[sl]), util.to_torch(rhs), DIMS)
      dl, dr = bp(util.to_torch(g[sl]))
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
