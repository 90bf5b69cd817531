"""Row-sharded execution on real GPUs (needs >= 2 devices, else skipped).

Each rank runs ShardedDotGeneral on its half of the rows over NCCL (the
per-tensor cases recorded and replayed through engine.TracedStep) and the
unsharded op on the whole problem; the two must agree: bit for bit for int8;
for fp8 out and dlhs bit for bit and drhs within max(1 bf16 ulp,
1e-5 * sum |g||lhs|), the ranks' f32 partial sums being added in another order
than one device's.
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
import bench
rank = int(os.environ['RANK']); world = int(os.environ['WORLD_SIZE'])
torch.cuda.set_device(int(os.environ['LOCAL_RANK']))
dev = torch.device('cuda', int(os.environ['LOCAL_RANK']))
dist.init_process_group('nccl', device_id=dev)
# int8: bit for bit. fp8: out and dlhs bit for bit, drhs within
# max(6 bf16 ulps, 1e-5 * sum |g||lhs|) (bench.sharded_parity_check). Once with
# the exchange as one kernel over peer memory, once with the NCCL calls.
result = bench.sharded_parity_check(torch, dist, rank, world, dev)
print(f'rank {rank}: {result}', flush=True)
assert result.pop('exchange') == 'p2p', 'the fused exchange was not used'
nccl = bench.sharded_parity_check(torch, dist, rank, world, dev, exchange='nccl')
print(f'rank {rank}: {nccl}', flush=True)
assert nccl.pop('exchange') == 'nccl'
result.update({k + '/nccl': v for k, v in nccl.items()})

# the library's own collectives (NCCL opened by the library) against torch's
import ctypes as C
from aqt_b200 import _lib
lib = _lib.load()
ident = [bytes(128)]
if rank == 0:
  buf = C.create_string_buffer(128)
  _lib.check(lib.aqtb200_comm_unique_id(buf), 'unique_id')
  ident = [buf.raw]
dist.broadcast_object_list(ident, src=0)
comm = C.c_void_p()
_lib.check(lib.aqtb200_comm_init(world, rank, ident[0], C.byref(comm)), 'comm_init')
st = torch.cuda.current_stream().cuda_stream
x = torch.arange(1024, device=dev, dtype=torch.float32) * (rank + 1)
want = x.clone(); dist.all_reduce(want, op=dist.ReduceOp.MAX)
_lib.check(lib.aqtb200_allreduce(comm, x.data_ptr(), x.numel(), _lib.F32, 1, st), 'allreduce')
acc = (torch.arange(4096 * world, device=dev) %% 97).to(torch.int32) * (rank + 3)
mine = torch.empty(4096, device=dev, dtype=torch.int32)
_lib.check(lib.aqtb200_reduce_scatter_sum(comm, acc.data_ptr(), mine.data_ptr(), 4096, _lib.S32, st), 'rs')
want_rs = acc.clone(); dist.all_reduce(want_rs)
full = torch.zeros(4096 * world, device=dev, dtype=torch.bfloat16)
full[rank * 4096:(rank + 1) * 4096] = rank + 1
_lib.check(lib.aqtb200_all_gather(comm, full[rank * 4096:].data_ptr(), full.data_ptr(), 4096, _lib.BF16, st), 'ag')
torch.cuda.synchronize()
lib_ok = (torch.equal(x, want) and torch.equal(mine, want_rs[rank * 4096:(rank + 1) * 4096])
          and all(bool((full[r * 4096:(r + 1) * 4096] == r + 1).all()) for r in range(world)))
print(f'rank {rank}: library collectives {"ok" if lib_ok else "MISMATCH"}', flush=True)
_lib.check(lib.aqtb200_comm_destroy(comm), 'comm_destroy')
dist.destroy_process_group()
sys.exit(0 if lib_ok and all(v == 'ok' for v in result.values()) else 1)
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
