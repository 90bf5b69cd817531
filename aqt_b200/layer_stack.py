"""The projections of a Llama-3-8B-shaped decoder stack, all through the
quantized dot_general: the caller of the hot path at model scale.

Shape (BASELINE configuration 5): 32 layers, d_model 4096, 32 query heads and
8 key/value heads of 128, SwiGLU FFN of 14336; per layer seven projections

    wq [4096, 4096]  wk [4096, 1024]  wv [4096, 1024]  wo [4096, 4096]
    w_gate [4096, 14336]  w_up [4096, 14336]  w_down [14336, 4096]

= 218.1 M weights per layer, 6.98 G in the stack; sequence 4096, global batch
64 = 262 144 tokens per step; weights ~ N(0, 0.02^2), bf16.

What this is NOT: a transformer. The reference contains no Llama (its caller
is whatever Flax model injects AqtDotGeneral, examples/flax_e2e_model.py:
115-117), and attention, RMSNorm, RoPE, the embedding, the loss and the
optimizer are not part of the quantized dot_general path. They are replaced
by the cheapest elementwise glue that keeps the data flow of a decoder layer
(residual adds, a gated product where SwiGLU sits, key/value heads repeated
over their query groups where attention sits) so that every projection sees
an activation and a cotangent of the right shape and a sane magnitude. The
figure reported is therefore labelled "GEMM-only tokens/s": the time of all
7 x 32 quantized forward / dlhs / drhs dots of a training step plus the
data-parallel gradient exchange, nothing else.

Data parallel (replica mode, what a jax data-parallel job does): every rank
holds all weights and 1/N of the tokens, quantizes with its own scales, and
the dequantized bf16 weight gradients are summed across ranks by NCCL
all-reduces once the step's last micro-batch has been through.
"""

from __future__ import annotations

import json
import os
import time

import torch
import torch.distributed as dist

from aqt_b200.v2 import config

DIMS = (((1,), (0,)), ((), ()))

D_MODEL, N_HEADS, N_KV, HEAD, FFN, LAYERS = 4096, 32, 8, 128, 14336, 32
PROJ = (('wq', D_MODEL, N_HEADS * HEAD), ('wk', D_MODEL, N_KV * HEAD),
        ('wv', D_MODEL, N_KV * HEAD), ('wo', N_HEADS * HEAD, D_MODEL),
        ('w_gate', D_MODEL, FFN), ('w_up', D_MODEL, FFN),
        ('w_down', FFN, D_MODEL))
PARAMS_PER_LAYER = sum(i * o for _, i, o in PROJ)


class ProjectionStack:
  """Weights, gradient buffers and one training step of the stack."""

  def __init__(self, device, layers: int = LAYERS, group=None, seed: int = 0,
               stochastic_rounding: bool = False):
    self.device, self.layers, self.group = device, layers, group
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)  # the same weights on every rank
    self.w = [{n: (torch.randn(i, o, device=device, generator=gen) * 0.02).to(
        torch.bfloat16) for n, i, o in PROJ} for _ in range(layers)]
    self.grad = [{n: torch.zeros(i, o, device=device, dtype=torch.bfloat16)
                  for n, i, o in PROJ} for _ in range(layers)]
    self.cfg = config.fully_quantized(
        fwd_bits=8, bwd_bits=8, use_stochastic_rounding=stochastic_rounding)

  def _dot(self, x, w):
    return self.cfg.vjp(x, w, DIMS)

  def _layer_fwd(self, x, w):
    """Returns (y, tape): the seven projections with stand-in glue between."""
    q, bq = self._dot(x, w['wq'])
    k, bk = self._dot(x, w['wk'])
    v, bv = self._dot(x, w['wv'])
    # where attention sits: every query head takes its group's key + value head
    rep = N_HEADS // N_KV
    kv = (k + v).view(-1, N_KV, 1, HEAD).expand(-1, N_KV, rep, HEAD).reshape(
        -1, N_HEADS * HEAD)
    a = q * 0.5 + kv * 0.5
    o, bo = self._dot(a, w['wo'])
    h = x + o
    gate, bg = self._dot(h, w['w_gate'])
    up, bu = self._dot(h, w['w_up'])
    hid = gate * up  # where SwiGLU sits
    down, bd = self._dot(hid, w['w_down'])
    y = h + down
    return y, (bq, bk, bv, bo, bg, bu, bd, gate, up)

  def _layer_bwd(self, dy, tape, grad):
    bq, bk, bv, bo, bg, bu, bd, gate, up = tape
    dhid, g = bd(dy)
    grad['w_down'] += g
    dh_g, g = bg(dhid * up)
    grad['w_gate'] += g
    dh_u, g = bu(dhid * gate)
    grad['w_up'] += g
    dh = dy + dh_g + dh_u
    da, g = bo(dh)
    grad['wo'] += g
    dq = da * 0.5
    rep = N_HEADS // N_KV
    dkv = (da * 0.5).view(-1, N_KV, rep, HEAD).sum(2).reshape(-1, N_KV * HEAD)
    dx_q, g = bq(dq)
    grad['wq'] += g
    dx_k, g = bk(dkv)
    grad['wk'] += g
    dx_v, g = bv(dkv)
    grad['wv'] += g
    return dh + dx_q + dx_k + dx_v

  def micro_step(self, x):
    """Forward and backward of the whole stack for one micro-batch
    [tokens, 4096]; weight gradients are ADDED to self.grad. Returns the
    micro-batch's stand-in loss (mean square of the stack output, whose
    cotangent is the output itself, scaled)."""
    tapes = []
    for w in self.w:
      x, tape = self._layer_fwd(x, w)
      tapes.append(tape)
    loss = x.float().square().mean()
    dy = (x * (1.0 / x.shape[0])).to(torch.bfloat16)
    for li in reversed(range(self.layers)):
      dy = self._layer_bwd(dy, tapes[li], self.grad[li])
      tapes[li] = None
    return loss

  def zero_grad(self):
    for gl in self.grad:
      for g in gl.values():
        g.zero_()

  def reduce_gradients(self):
    """Data parallel: sum every weight gradient across the ranks."""
    if not dist.is_initialized() or dist.get_world_size(self.group) == 1:
      return
    works = [dist.all_reduce(g, group=self.group, async_op=True)
             for gl in reversed(self.grad) for g in gl.values()]
    for wk in works:
      wk.wait()


def bench_main(args, lines):
  """`bench.py --workload stack`: GEMM-only tokens/s of the projection stack."""
  from aqt_b200 import _lib
  from aqt_b200 import engine
  world = int(os.environ.get('WORLD_SIZE', '1'))
  rank = int(os.environ.get('RANK', '0'))
  local_rank = int(os.environ.get('LOCAL_RANK', '0'))
  torch.cuda.set_device(local_rank)
  dev = torch.device('cuda', local_rank)
  if world > 1:
    dist.init_process_group('nccl', device_id=dev)
  lib = _lib.load()
  layers = int(os.environ.get('AQT_STACK_LAYERS', LAYERS))
  seq, global_batch, micro_seqs = 4096, 64, 2
  tokens_rank = seq * global_batch // world
  micro = seq * micro_seqs
  stack = ProjectionStack(dev, layers=layers)
  gen = torch.Generator(device=dev)
  gen.manual_seed(100 + rank)
  xs = [torch.randn(micro, D_MODEL, device=dev, generator=gen).to(
      torch.bfloat16) for _ in range(tokens_rank // micro)]

  def barrier():
    if world > 1:
      dist.barrier()
    torch.cuda.synchronize()

  steps = max(1, min(args.steps, 3))
  warm = 1
  x_static = xs[0].clone()
  for _ in range(2):
    stack.micro_step(x_static)
  barrier()
  engine.check_status()
  # One micro-batch through the stack is 32 x 7 x 3 quantized dots behind a
  # Python planner; it is captured once as a CUDA graph (kernels of this
  # library and the elementwise glue alike) and replayed per micro-batch. The
  # gradient all-reduce stays outside the graph.
  launch = 'eager'
  micro_step = stack.micro_step
  launches_per_micro = None
  if not args.eager:
    try:
      side = torch.cuda.Stream()
      side.wait_stream(torch.cuda.current_stream())
      with torch.cuda.stream(side):
        stack.micro_step(x_static)
      torch.cuda.current_stream().wait_stream(side)
      barrier()
      graph = torch.cuda.CUDAGraph()
      l0 = lib.aqtb200_kernel_launch_count()
      with torch.cuda.graph(graph):
        stack.micro_step(x_static)
      launches_per_micro = lib.aqtb200_kernel_launch_count() - l0
      micro_step = lambda x: graph.replay()
      launch = 'cuda_graph replay per micro-batch'
    except Exception as e:  # pylint: disable=broad-except
      import sys
      print(f'graph capture failed ({type(e).__name__}: {e}); eager',
            file=sys.stderr)
      torch.cuda.synchronize()

  def step():
    stack.zero_grad()
    for x in xs:
      x_static.copy_(x)
      micro_step(x_static)
    stack.reduce_gradients()

  for _ in range(warm):
    step()
  barrier()
  engine.check_status()
  l0 = lib.aqtb200_kernel_launch_count()
  e0 = torch.cuda.Event(enable_timing=True)
  e1 = torch.cuda.Event(enable_timing=True)
  barrier()
  t0 = time.perf_counter()
  e0.record()
  for _ in range(steps):
    step()
  e1.record()
  barrier()
  host_s = (time.perf_counter() - t0) / steps
  engine.check_status()
  ms = e0.elapsed_time(e1) / steps
  if world > 1:
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
  tokens = seq * global_batch
  ops = 6.0 * PARAMS_PER_LAYER * layers * tokens
  if rank == 0:
    lines.append(json.dumps({
        'metric': 'gemm_only_tokens_per_s', 'value': tokens / (ms * 1e-3),
        'unit': 'tokens/s', 'n_gpus': world, 'steps': steps, 'warmup': warm,
        'ms_per_step': ms, 'higher_is_better': True, 'scaling': 'strong',
        'vs_baseline': None, 'dtype': 's8->s32', 'data': 'synthetic',
        'config': {
            'workload': (
                f'{layers} decoder layers x 7 projections (d_model 4096, 32 q / '
                '8 kv heads of 128, FFN 14336), int8 fwd + dlhs + drhs per '
                'projection, per-channel absmax scales, bf16; seq 4096, global '
                f'batch 64 = {tokens} tokens per step in micro-batches of '
                f'{micro}; GEMM-only: attention, norms, rope, embedding, loss '
                'and optimizer replaced by elementwise glue'),
            'parallelism': f'data parallel over {world} GPU(s), replica-mode '
                           'scales, bf16 gradient all-reduce per layer'},
        'tops': ops / (ms * 1e-3) / 1e12,
        'launch': launch,
        'host_s_per_step': host_s,
        'gpu_launches': int(
            launches_per_micro * len(xs) * steps if launches_per_micro
            is not None else lib.aqtb200_kernel_launch_count() - l0),
    }))
  if world > 1:
    dist.destroy_process_group()
