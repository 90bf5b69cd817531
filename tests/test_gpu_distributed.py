"""Row-sharded execution on real GPUs (needs >= 2 devices, else skipped).

Each rank runs ShardedDotGeneral on its half of the rows over NCCL; rank 0
also runs the unsharded op on the whole problem and the two must agree: bit
for bit for int8, to f32 summation order for fp8.
"""

import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

_WORKER = r'''
import os, sys
sys.path.insert(0, %(root)r)
import torch, torch.distributed as dist
from aqt_b200 import engine, distributed as aqt_dist
import bench
rank = int(os.environ['RANK']); world = int(os.environ['WORLD_SIZE'])
torch.cuda.set_device(int(os.environ['LOCAL_RANK']))
dev = torch.device('cuda', int(os.environ['LOCAL_RANK']))
dist.init_process_group('nccl', device_id=dev)
ok = True
for kind in ('int8', 'fp8'):
  for per_tensor in (True, False):
    cfg = bench.make_cfg(kind)
    if not per_tensor:
      for raw in (cfg.fwd, cfg.dlhs, cfg.drhs):
        raw.dg_quantizer.lhs.calib_shared_axes = None
        raw.dg_quantizer.rhs.calib_shared_axes = None
    gen = torch.Generator(device=dev); gen.manual_seed(7)
    m, k, n = 512 * world, 1024, 768
    lhs = torch.randn(m, k, device=dev, generator=gen).to(torch.bfloat16)
    rhs = (torch.randn(k, n, device=dev, generator=gen) * 0.03).to(torch.bfloat16)
    g = torch.randn(m, n, device=dev, generator=gen).to(torch.bfloat16)
    sl = slice(rank * (m // world), (rank + 1) * (m // world))
    out, bp = aqt_dist.ShardedDotGeneral(cfg).vjp(lhs[sl].contiguous(), rhs, bench.DIMS)
    dl, dr = bp(g[sl].contiguous())
    wo, wbp = cfg.vjp(lhs, rhs, bench.DIMS)
    wl, wr = wbp(g)
    torch.cuda.synchronize(); engine.check_status()
    same = torch.equal(out, wo[sl]) and torch.equal(dl, wl[sl])
    if kind == 'int8':
      same = same and torch.equal(dr, wr)
    else:
      same = same and torch.allclose(dr.float(), wr.float(), rtol=2e-2, atol=1e-3)
    print(f'rank {rank} {kind} per_tensor={per_tensor}: {"ok" if same else "MISMATCH"}', flush=True)
    ok = ok and same
dist.destroy_process_group()
sys.exit(0 if ok else 1)
'''


def test_sharded_matches_unsharded(tmp_path):
  if torch.cuda.device_count() < 2:
    pytest.skip('needs at least 2 GPUs')
  script = tmp_path / 'worker.py'
  script.write_text(_WORKER % {'root': ROOT})
  s = socket.socket()
  s.bind(('127.0.0.1', 0))
  port = s.getsockname()[1]
  s.close()
  env = dict(os.environ, NCCL_NVLS_ENABLE='0')
  r = subprocess.run(
      [sys.executable, '-m', 'torch.distributed.run', '--nnodes=1',
       '--nproc-per-node', '2', '--master-addr', '127.0.0.1', '--master-port',
       str(port), str(script)], capture_output=True, text=True, timeout=600,
      env=env)
  assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
