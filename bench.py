"""Benchmark of the quantized dot_general hot path (forward + dlhs + drhs).

Workload (BASELINE.json configs[1]): fp8 dot_general, 8192 x 8192 x 8192, bf16
inputs lhs ~ N(0,1), rhs ~ N(0,1/8192), cotangent ~ N(0,1); forward operands
e4m3, backward operands e5m2, per-tensor AbsMax scales, f32 accumulation, bf16
outputs. One "step" = forward + both gradient dot_generals, calibration and
quantization kernels included.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                  [--scaling weak|strong] [--size S] [--kind fp8|int8]

Prints ONE JSON line (rank 0). `value` is whole-job TOPS with inputs resident
in HBM; `e2e` is the same metric through the public API with pinned host
buffers, host->device and device->host copies inside the timed region.
`--impl reference` times the CPU restatement of the reference (the reference
itself needs jax, which is not installed here) on a bounded sample.
"""

import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
  sys.path.insert(0, ROOT)

METRIC = 'quantized_dot_general_fwd_bwd_tops'
UNIT = 'TOPS'


def parse_args():
  p = argparse.ArgumentParser()
  p.add_argument('--gpus', type=int, default=1)
  p.add_argument('--steps', type=int, default=20)
  p.add_argument('--warmup', type=int, default=5)
  p.add_argument('--impl', default='ours', choices=['ours', 'reference'])
  p.add_argument('--scaling', default='weak', choices=['weak', 'strong'])
  p.add_argument('--size', type=int, default=8192)
  p.add_argument('--kind', default='fp8', choices=['fp8', 'int8'])
  p.add_argument('--cpu-sample-rows', type=int, default=0,
                 help='rows of lhs/cotangent the CPU arm processes (0 = all: '
                 'the whole workload, which keeps the ratio of contraction to '
                 'quantization work of the real problem)')
  p.add_argument('--no-cpu-baseline', action='store_true')
  p.add_argument('--no-e2e', action='store_true')
  p.add_argument('--workload', default='c2', choices=['c1', 'c2', 'c3', 'c4'],
                 help='BASELINE.json config to time; c2 is the headline '
                 'workload, the others are extra single-GPU measurements')
  p.add_argument('--m', type=int, default=16,
                 help='rows of the activation for --workload c4')
  p.add_argument('--eager', action='store_true',
                 help='main workload at 1 GPU: launch every kernel from Python '
                      'each step instead of replaying the step from a CUDA graph')
  p.add_argument('--graph', action='store_true',
                 help='extra workloads only: replay the step from a CUDA graph '
                 '(removes host launch overhead from small problems)')
  p.add_argument('--gemm', default='tcgen05',
                 choices=['tcgen05', 'cta1', 'cta2', 'wide'],
                 help='tile shape of the tensor-core kernel (default: automatic)')
  return p.parse_args()


def make_cfg(kind):
  from aqt_b200.v2 import config
  if kind == 'fp8':
    cfg = config.fully_quantized(fwd_bits='e4m3', bwd_bits='e5m2',
                                 use_stochastic_rounding=False)
  else:
    cfg = config.fully_quantized(fwd_bits=8, bwd_bits=8,
                                 use_stochastic_rounding=False)
  for raw in (cfg.fwd, cfg.dlhs, cfg.drhs):
    raw.dg_quantizer.lhs.calib_shared_axes = 'per_tensor'
    raw.dg_quantizer.rhs.calib_shared_axes = 'per_tensor'
  return cfg


DIMS = (((1,), (0,)), ((), ()))


def workload_name(args):
  return (f'{args.kind} dot_general {args.size}x{args.size}x{args.size} '
          'fwd+dlhs+drhs, bf16 in/out, per-tensor absmax scales')


# ---------------------------------------------------------------------------
# CPU arm: the oracle on a bounded sample


def cpu_sample(args, rows):
  """Times the numpy restatement on `rows` rows of lhs/cotangent (rhs full)."""
  import numpy as np
  from oracle import aqt_oracle as orc
  n = args.size
  rng = np.random.default_rng(0)
  f = lambda shape, std: (rng.standard_normal(shape, np.float32) * std).astype(
      orc.bfloat16)
  lhs, rhs, g = f((rows, n), 1.0), f((n, n), n ** -0.5), f((rows, n), 1.0)
  cfg = make_cfg(args.kind)
  t0 = time.perf_counter()
  orc.dg_fwd_bwd(cfg, lhs, rhs, g, DIMS, fast_float=True)
  dt = time.perf_counter() - t0
  ops = 3 * 2 * rows * n * n
  return ops / dt / 1e12, dt


def blas_threads():
  try:
    import threadpoolctl
    infos = threadpoolctl.threadpool_info()
    return max([i.get('num_threads', 1) for i in infos] + [1])
  except Exception:  # pylint: disable=broad-except
    return os.cpu_count() or 1


def run_reference_arm(args, lines):
  rank = int(os.environ.get('RANK', '0'))
  if rank != 0:
    return
  rows = args.cpu_sample_rows or args.size
  for _ in range(min(args.warmup, 1)):
    cpu_sample(args, rows)
  steps = max(1, min(args.steps, 3))
  vals, times = [], []
  for _ in range(steps):
    v, dt = cpu_sample(args, rows)
    vals.append(v)
    times.append(dt)
  value = sum(vals) / len(vals)
  sample = (f'{rows} of {args.size} lhs/cotangent rows against the full '
            f'{args.size}x{args.size} rhs, numpy+ml_dtypes restatement '
            '(jax is not installed, so the reference itself cannot run)')
  line = {
      'impl': 'reference', 'metric': METRIC, 'value': value, 'unit': UNIT,
      'n_gpus': args.gpus, 'steps': steps, 'warmup': min(args.warmup, 1),
      'ms_per_step': 1e3 * sum(times) / len(times), 'higher_is_better': True,
      'scaling': args.scaling, 'vs_baseline': None, 'dtype': args.kind,
      'data': 'synthetic',
      'config': {'workload': workload_name(args), 'sample': sample},
      'cpu_baseline': {'value': value, 'unit': UNIT, 'cores': blas_threads(),
                       'kind': 'port', 'sample': sample},
      'e2e': {'value': value, 'unit': UNIT, 'h2d_bytes_per_step': 0,
              'd2h_bytes_per_step': 0},
      'gpu_launches': 0,
  }
  lines.append(json.dumps(line))


# ---------------------------------------------------------------------------
# clocks


class ClockSampler:
  """Samples SM clock and clock event reasons DURING the timed region.

  A separate process polls NVML (read-only queries) every few milliseconds and
  time-stamps each sample; only samples between mark_begin() and mark_end()
  are reported. Polling NVML from a thread of this process stalls kernel
  launches for milliseconds per query and would distort the measurement.
  """

  # NVML bit masks of the clock event reasons the contract asks about
  MASKS = {'sw_power_cap': 0x4, 'hw_slowdown': 0x8, 'sw_thermal_slowdown': 0x20,
           'hw_thermal_slowdown': 0x40}
  POLLER = r"""
import sys, time
import pynvml as N
N.nvmlInit()
h = N.nvmlDeviceGetHandleByIndex(int(sys.argv[1]))
mx = N.nvmlDeviceGetMaxClockInfo(h, N.NVML_CLOCK_SM)
period = float(sys.argv[2])
print('ready', mx, flush=True)
while True:
  t = time.time()
  c = N.nvmlDeviceGetClockInfo(h, N.NVML_CLOCK_SM)
  try:
    r = N.nvmlDeviceGetCurrentClocksEventReasons(h)
  except Exception:
    r = N.nvmlDeviceGetCurrentClocksThrottleReasons(h)
  print(t, c, r, flush=True)
  time.sleep(period)
"""

  def __init__(self, index, period_ms=4):
    self.index, self.period_ms = index, period_ms
    self.proc = None
    self.mx = None
    self.t0 = self.t1 = None

  def start(self):
    """Starts a separate polling process (NVML, every few ms). An in-process
    poller would share the interpreter with the thread that launches kernels."""
    import subprocess
    try:
      self.proc = subprocess.Popen(
          [sys.executable, '-c', self.POLLER, str(self.index),
           str(self.period_ms / 1e3)],
          stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
      first = self.proc.stdout.readline().split()
      if not first or first[0] != 'ready':
        raise RuntimeError('poller did not start')
      self.mx = int(first[1])
    except Exception:  # pylint: disable=broad-except
      self.proc = None

  def mark_begin(self):
    self.t0 = time.time()

  def mark_end(self):
    self.t1 = time.time()

  def stop(self):
    if self.proc is None:
      return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': [], 'samples': 0}
    if self.t1 is None:
      self.t1 = time.time()
    time.sleep(2 * self.period_ms / 1e3)
    self.proc.terminate()
    try:
      rest, _ = self.proc.communicate(timeout=5)
    except Exception:  # pylint: disable=broad-except
      self.proc.kill()
      rest = ''
    clocks, bits = [], 0
    for line in rest.splitlines():
      parts = line.split()
      if len(parts) != 3:
        continue
      try:
        t, c, r = float(parts[0]), int(parts[1]), int(parts[2])
      except ValueError:
        continue
      # only samples taken while the timed region was running count
      if self.t0 is not None and not self.t0 <= t <= self.t1:
        continue
      clocks.append(c)
      bits |= r
    clocks.sort()
    reasons = sorted(k for k, m in self.MASKS.items() if bits & m)
    return {'sm_mhz': clocks[len(clocks) // 2] if clocks else None,
            'sm_min_mhz': clocks[0] if clocks else None,
            'sm_max_mhz': self.mx, 'reasons': reasons,
            'samples': len(clocks)}


# ---------------------------------------------------------------------------
# our arm


def run_ours(args, lines):
  import torch
  import torch.distributed as dist
  from aqt_b200 import _lib
  from aqt_b200 import engine

  world = int(os.environ.get('WORLD_SIZE', '1'))
  rank = int(os.environ.get('RANK', '0'))
  local_rank = int(os.environ.get('LOCAL_RANK', '0'))
  assert world == args.gpus or world == 1 and args.gpus == 1, (
      f'--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun')
  torch.cuda.set_device(local_rank)
  dev = torch.device('cuda', local_rank)
  if world > 1:
    dist.init_process_group('nccl', device_id=dev)
  lib = _lib.load()
  engine.set_gemm_impl(args.gemm)

  n = args.size
  m_local = n if args.scaling == 'weak' else n // world
  m_global = m_local * world
  gen = torch.Generator(device=dev)
  gen.manual_seed(1234 + rank)
  lhs = torch.randn(m_local, n, device=dev, dtype=torch.float32,
                    generator=gen).to(torch.bfloat16)
  g = torch.randn(m_local, n, device=dev, dtype=torch.float32,
                  generator=gen).to(torch.bfloat16)
  gen.manual_seed(99)  # the weights are replicated
  rhs = (torch.randn(n, n, device=dev, dtype=torch.float32, generator=gen)
         * n ** -0.5).to(torch.bfloat16)
  cfg = make_cfg(args.kind)
  op = None
  if world > 1:
    from aqt_b200 import distributed as aqt_dist
    op = aqt_dist.ShardedDotGeneral(cfg)

  def step(a, b, c):
    if op is not None:
      out, bp = op.vjp(a, b, DIMS)
    else:
      out, bp = cfg.vjp(a, b, DIMS)
    dl, dr = bp(c)
    return out, dl, dr

  def barrier():
    if world > 1:
      dist.barrier()
    torch.cuda.synchronize()

  for _ in range(args.warmup):
    step(lhs, rhs, g)
  barrier()
  engine.check_status()

  # One GPU: the step (17 kernels behind a Python planner) is captured once and
  # replayed, as a compiled training step would be; operands keep their
  # addresses, results land in the graph's own buffers. Several GPUs: eager,
  # the collectives stay outside graphs.
  use_graph = world == 1 and not args.eager
  launches_per_step = None
  eager_step = step
  if use_graph:
   try:
    run_step = step
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
      run_step(lhs, rhs, g)
    torch.cuda.current_stream().wait_stream(side)
    barrier()
    graph = torch.cuda.CUDAGraph()
    l0 = lib.aqtb200_kernel_launch_count()
    with torch.cuda.graph(graph):
      graph_outs = run_step(lhs, rhs, g)
    launches_per_step = lib.aqtb200_kernel_launch_count() - l0

    def step(a, b, c):  # pylint: disable=function-redefined
      assert a is lhs and b is rhs and c is g
      graph.replay()
      return graph_outs

    for _ in range(3):
      step(lhs, rhs, g)
    barrier()
    engine.check_status()
   except Exception as e:  # pylint: disable=broad-except
    # capture is an optimisation of the launch path only: run eagerly instead
    print(f'CUDA graph capture failed ({type(e).__name__}: {e}); eager', file=sys.stderr)
    use_graph, launches_per_step, step = False, None, eager_step
    torch.cuda.synchronize()

  sampler = ClockSampler(local_rank)
  launches0 = lib.aqtb200_kernel_launch_count()
  e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  sampler.start()
  barrier()
  sampler.mark_begin()
  e0.record()
  t_host = time.perf_counter()
  for _ in range(args.steps):
    outs = step(lhs, rhs, g)
  host_ms = (time.perf_counter() - t_host) * 1e3 / args.steps
  e1.record()
  barrier()
  sampler.mark_end()
  clocks = sampler.stop()
  launches = lib.aqtb200_kernel_launch_count() - launches0
  if launches_per_step is not None:
    launches = launches_per_step * args.steps  # replayed, not re-issued
  engine.check_status()
  ms = e0.elapsed_time(e1) / args.steps
  if world > 1:
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
  ops_step = 3 * 2 * m_global * n * n
  value = ops_step / (ms * 1e-3) / 1e12

  # ---- end to end through the public API with pinned host buffers
  e2e = None
  if not args.no_e2e:
    h = [t.cpu().pin_memory() for t in (lhs, rhs, g)]
    ho = [torch.empty_like(t, device='cpu').pin_memory() for t in outs]

    # The call a host-memory user makes: a HostStepPipeline around the step.
    # Each step uploads all three operands and downloads all three results;
    # uploads, compute and downloads of neighbouring steps overlap.
    from aqt_b200 import host_io
    pipe = host_io.HostStepPipeline(eager_step, dev)

    for _ in range(3):
      pipe.submit(h, ho)
    pipe.drain()
    barrier()
    k = max(3, min(args.steps, 10))
    e0.record()
    for _ in range(k):
      pipe.submit(h, ho)
    pipe.drain()
    e1.record()
    barrier()
    ems = e0.elapsed_time(e1) / k
    if world > 1:
      t = torch.tensor([ems], device=dev, dtype=torch.float64)
      dist.all_reduce(t, op=dist.ReduceOp.MAX)
      ems = float(t.item())
    e2e = {'value': ops_step / (ems * 1e-3) / 1e12, 'unit': UNIT,
           'h2d_bytes_per_step': sum(t.numel() * t.element_size() for t in h),
           'd2h_bytes_per_step': sum(t.numel() * t.element_size() for t in ho),
           'ms_per_step': ems,
           'path': 'aqt_b200.host_io.HostStepPipeline (pinned host buffers, '
                   'copies of neighbouring steps overlap compute)'}

  # ---- roofline of the dominant kernel: the tcgen05 GEMM, timed alone
  roof = None
  if rank == 0:
    roof = gemm_roofline(args, cfg, lhs, rhs, torch, engine)
    # the whole step (calibration, quantization and the three GEMMs) against
    # the same tensor peak, per GPU
    roof['step_achieved'] = value / world
    roof['step_frac'] = value / world / roof['peak']

  if rank != 0:
    if world > 1:
      dist.destroy_process_group()
    return

  cpu = None
  if not args.no_cpu_baseline and world == 1:
    cpu_rows = args.cpu_sample_rows or n
    v, dt = cpu_sample(args, cpu_rows)
    cpu = {'value': v, 'unit': UNIT, 'cores': blas_threads(), 'kind': 'port',
           'sample': (f'{cpu_rows} of {n} lhs/cotangent rows against '
                      f'the full rhs, one pass, {dt:.1f} s; numpy+ml_dtypes '
                      'restatement (jax not installed)')}
  line = {
      'metric': METRIC, 'value': value, 'unit': UNIT, 'n_gpus': world,
      'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': ms,
      'higher_is_better': True, 'scaling': args.scaling, 'vs_baseline': None,
      'dtype': 'f8e4m3/f8e5m2->f32' if args.kind == 'fp8' else 's8->s32',
      'data': 'synthetic',
      'config': {
          'workload': workload_name(args),
          'rows_per_gpu': m_local, 'global_rows': m_global,
          'parallelism': f'rows sharded over {world} GPU(s)',
          'launch': 'cuda_graph replay of the whole step' if use_graph else 'eager',
          'l2': 'inputs (3 x 134 MB bf16 + quantized copies) exceed the 126 MB L2',
      },
      'clocks': clocks,
      'e2e': e2e,
      'gpu_launches': int(launches),
      'host_issue_ms_per_step': host_ms,
      'roofline': roof,
      'cpu_baseline': cpu,
  }
  lines.append(json.dumps(line))
  if world > 1:
    dist.destroy_process_group()


def gemm_roofline(args, cfg, lhs, rhs, torch, engine):
  """Average duration of the forward GEMM launch alone (CUDA events on the
  launching stream) against the measured tensor peak."""
  import ctypes as C
  from aqt_b200 import _lib
  lib = _lib.load()
  out, res = engine.dg_raw(cfg.fwd, lhs, rhs, None, None, DIMS)
  ql, qr = res.lhs.mt.qx, res.rhs.mt.qx
  m, k = lhs.shape
  n = rhs.shape[1]
  # the quantized buffers are contraction-contiguous: [m, k] and [n, k]
  a = ql.qvalue
  b = qr.qvalue.t()
  assert a.stride(1) == 1 and b.stride(1) == 1
  d = _lib.GemmDesc()
  d.b0 = d.b1 = 1
  d.m, d.n, d.k = m, n, k
  d.a, d.lda, d.a_dtype = a.data_ptr(), a.stride(0), engine._code(a.dtype)
  d.b, d.ldb, d.b_dtype = b.data_ptr(), b.stride(0), engine._code(b.dtype)
  d.a_scale, d.a_scale_dtype = ql.scale[0].data_ptr(), _lib.BF16
  d.b_scale, d.b_scale_dtype = qr.scale[0].data_ptr(), _lib.BF16
  d.dequant_dtype = d.out_dtype = _lib.BF16
  d.out = out.data_ptr()
  d.out_m_stride, d.out_n_stride = n, 1
  stream = torch.cuda.current_stream().cuda_stream
  for _ in range(3):
    _lib.check(lib.aqtb200_gemm_dequant(C.byref(d), None, stream), 'gemm')
  torch.cuda.synchronize()
  reps = 10
  e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  e0.record()
  for _ in range(reps):
    lib.aqtb200_gemm_dequant(C.byref(d), None, stream)
  e1.record()
  torch.cuda.synchronize()
  ms = e0.elapsed_time(e1) / reps
  achieved = 2.0 * m * n * k / (ms * 1e-3) / 1e12
  peaks_path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
  if os.path.exists(peaks_path):
    with open(peaks_path) as f:
      bf16 = json.load(f)['bf16_tflops']
    src = 'of measured: 2 x bf16_tflops (burst) from MEASURED_PEAKS.json'
  else:
    bf16 = 1590.0
    src = 'of fallback: 2 x 1.59 PFLOP/s bf16'
  peak = 2.0 * bf16
  # DRAM bytes (read + write) of one launch of this kernel at this shape, from
  # the ncu capture summarised in profiles/gemm_tcgen05_wide_fp8_8192.md; it
  # is not re-measured here (nothing is timed under a profiler).
  traffic = 446.0e6 if (m, n, k) == (8192, 8192, 8192) else None
  return {'bound': 'tensor',
          'kernel': 'gemm_tcgen05_wide_kernel (forward GEMM, 256x512 CTA-pair tiles)',
          'achieved': achieved, 'peak': peak, 'unit': 'TFLOP/s',
          'frac': achieved / peak, 'traffic': traffic,
          'algorithmic_bytes': float(m * k + n * k + 2 * m * n), 'ms_per_launch': ms,
          'peak_source': src + '; 8-bit operands run at twice the bf16 rate'}


def run_extra_workload(args, lines):
  """Single-GPU timing of BASELINE configs 1, 3 and 4 (device-resident)."""
  import numpy as np
  import torch
  from aqt_b200 import _lib
  from aqt_b200 import engine
  from aqt_b200.v2 import aqt_dot_general as adg
  from aqt_b200.v2 import config
  from aqt_b200.v2 import stochastic_rounding as sr
  from aqt_b200.v2 import utils
  from aqt_b200.v2.flax import aqt_flax
  torch.cuda.set_device(0)
  dev = torch.device('cuda', 0)
  lib = _lib.load()
  engine.set_gemm_impl(args.gemm)
  gen = torch.Generator(device=dev)
  gen.manual_seed(0)
  rn = lambda shape, std, dt: (torch.randn(shape, device=dev, generator=gen)
                               * std).to(dt)
  extra = {}
  if args.workload == 'c1':
    lhs = rn((1024, 4096), 1.0, torch.float32)
    rhs = rn((4096, 4096), 1.0 / 64, torch.float32)
    g = rn((1024, 4096), 1.0, torch.float32)
    cfg = config.fully_quantized(fwd_bits=8, bwd_bits=8,
                                 use_stochastic_rounding=False)
    ops = 3 * 2 * 1024 * 4096 * 4096
    min_bytes = 201e6
    name = ('config 1: int8 [1024,4096]x[4096,4096] f32 in/out, per-channel '
            'absmax, RNE, fwd+dlhs+drhs')

    def step():
      out, bp = cfg.vjp(lhs, rhs, DIMS)
      return out, bp(g)
  elif args.workload == 'c3':
    b, t, h, d = 8, 2048, 32, 128
    q = rn((b, t, h, d), 1.0, torch.bfloat16)
    k = rn((b, t, h, d), 1.0, torch.bfloat16)
    g = rn((b, h, t, t), 1.0, torch.bfloat16)
    cfg = config.fully_quantized(fwd_bits=8, bwd_bits=8,
                                 use_stochastic_rounding=True)
    noise = {}

    def noise_fn(shape, key):
      kk = (tuple(shape), int(key[0]), int(key[1]))
      if kk not in noise:
        noise[kk] = torch.rand(shape, device=dev, generator=gen) - 0.5
      return noise[kk]

    for raw in (cfg.dlhs, cfg.drhs):
      raw.dg_quantizer.lhs.numerics.noise_fn = noise_fn
      raw.dg_quantizer.rhs.numerics.noise_fn = noise_fn
    cfg = config.set_context(cfg, key=sr.PRNGKey(1), train_step=None)
    dims = (((3,), (3,)), ((0, 2), (0, 2)))
    ops = 3 * 2 * b * h * t * t * d
    min_bytes = 5.1e9
    name = ("config 3: int8 einsum 'bthd,bshd->bhts' B8 H32 T=S=2048 D128, "
            'bf16, per-token scales, fwd + both gradients, stochastic '
            'rounding from 4 given f32 noise tensors (2 x 4.29 GB + 2 x 0.27 GB '
            'read on top of the minimum bytes)')

    def step():
      out, bp = cfg.vjp(q, k, dims)
      return out, bp(g)
  else:
    m, kk, n = args.m, 8192, 28672
    x = rn((m, kk), 1.0, torch.bfloat16)
    w = rn((kk, n), kk ** -0.5, torch.bfloat16)
    cfg = adg.dot_general_make(lhs_bits=8, rhs_bits=4)
    cfg.fwd.dg_quantizer.rhs.numerics.dtype = utils.int8
    conv = aqt_flax.AqtDotGeneral(cfg, rhs_quant_mode=utils.QuantMode.CONVERT)
    conv(x, w, DIMS)
    serve = aqt_flax.AqtDotGeneral(cfg, rhs_quant_mode=utils.QuantMode.SERVE)
    serve.rhs_qtensor = conv.rhs_qtensor
    del conv
    wz = torch.empty(0, device=dev)
    dummy_w = w  # the float weights are not read in SERVE mode
    ops = 2 * m * kk * n
    min_bytes = kk * n + m * kk * 2 + m * n * 2 + 2 * n + 2 * m
    name = (f'config 4: serving GEMM M={m} K=8192 N=28672, int8 activations '
            'per token x int4-in-int8 frozen weights per channel, bf16 out')
    del wz

    rhs_qt = serve.rhs_qtensor

    def step():
      # dg_core is what AqtDotGeneral calls after copying its config; calling
      # it directly keeps the per-call deepcopy out of a serving loop.
      return cfg.dg_core(x, dummy_w, None, rhs_qt, DIMS)[0]
  for _ in range(max(args.warmup, 3)):
    step()
  torch.cuda.synchronize()
  engine.check_status()
  if args.graph:
    eager_step = step
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
      keep = eager_step()
    step = graph.replay
    for _ in range(3):
      step()
    torch.cuda.synchronize()
  l0 = lib.aqtb200_kernel_launch_count()
  e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  sampler = ClockSampler(0)
  sampler.start()
  torch.cuda.synchronize()
  sampler.mark_begin()
  e0.record()
  for _ in range(args.steps):
    step()
  e1.record()
  torch.cuda.synchronize()
  sampler.mark_end()
  clocks = sampler.stop()
  engine.check_status()
  ms = e0.elapsed_time(e1) / args.steps
  lines.append(json.dumps({
      'metric': METRIC, 'value': ops / (ms * 1e-3) / 1e12, 'unit': UNIT,
      'n_gpus': 1, 'steps': args.steps, 'warmup': max(args.warmup, 3),
      'ms_per_step': ms, 'higher_is_better': True, 'scaling': 'weak',
      'vs_baseline': None, 'dtype': 's8->s32', 'data': 'synthetic',
      'config': {'workload': name, 'cuda_graph': bool(args.graph)},
      'min_bytes_gbs': min_bytes / (ms * 1e-3) / 1e9,
      'clocks': clocks,
      'gpu_launches': int(lib.aqtb200_kernel_launch_count() - l0),
  }))


def main():
  args = parse_args()
  # Libraries (NCCL's version banner, torchrun notices) write to stdout; the
  # contract is ONE JSON line there, so everything else is sent to stderr.
  real_stdout = os.dup(1)
  os.dup2(2, 1)
  lines = []
  try:
    if args.impl == 'reference':
      run_reference_arm(args, lines)
    elif args.workload != 'c2':
      run_extra_workload(args, lines)
    else:
      run_ours(args, lines)
  finally:
    sys.stdout.flush()
    os.dup2(real_stdout, 1)
    os.close(real_stdout)
  for line in lines:
    print(line, flush=True)


if __name__ == '__main__':
  main()
