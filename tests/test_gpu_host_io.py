"""HostStepPipeline: results through pinned host buffers equal the direct call."""

import pytest
import torch

from aqt_b200 import engine
from aqt_b200 import host_io
from aqt_b200.v2 import config

pytestmark = pytest.mark.gpu

DIMS = (((1,), (0,)), ((), ()))


def test_pipeline_matches_direct_call_over_changing_inputs():
  dev = torch.device('cuda', 0)
  cfg = config.fully_quantized(fwd_bits=8, bwd_bits=8,
                               use_stochastic_rounding=False)
  gen = torch.Generator().manual_seed(5)
  m, k, n = 256, 512, 384

  def step(a, b, c):
    out, bp = cfg.vjp(a, b, DIMS)
    dl, dr = bp(c)
    return out, dl, dr

  pipe = host_io.HostStepPipeline(step, dev)
  hosts, outs = [], []
  for _ in range(5):  # more steps than buffer sets: slots get reused
    h = [torch.randn(m, k, generator=gen).pin_memory(),
         (torch.randn(k, n, generator=gen) / 16).pin_memory(),
         torch.randn(m, n, generator=gen).pin_memory()]
    o = [torch.empty(m, n).pin_memory(), torch.empty(m, k).pin_memory(),
         torch.empty(k, n).pin_memory()]
    hosts.append(h)
    outs.append(o)
    pipe.submit(h, o)
  pipe.drain()
  torch.cuda.synchronize()
  engine.check_status()
  for h, o in zip(hosts, outs):
    want = step(*[t.to(dev) for t in h])
    for got, w in zip(o, want):
      assert torch.equal(got, w.cpu())


def test_pipeline_rejects_pageable_memory():
  dev = torch.device('cuda', 0)
  pipe = host_io.HostStepPipeline(lambda a: (a,), dev)
  with pytest.raises(ValueError):
    pipe.submit([torch.zeros(4)], [torch.zeros(4).pin_memory()])
