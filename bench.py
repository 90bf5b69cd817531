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
buffers, host->device and device->host copies inside the timed region;
`sustained` repeats the device-resident measurement for seconds instead of
milliseconds (the part is power-capped, so a short burst runs at a higher
clock than a long loop); `extras` (1 GPU only) time the other BASELINE.json
configurations. `--impl reference` times the CPU restatement of the reference
(the reference itself needs jax, which is not installed here) on a bounded
sample, with every host core.
"""

import argparse
import json
import math
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
  sys.path.insert(0, ROOT)

METRIC = 'quantized_dot_general_fwd_bwd_tops'
UNIT = 'TOPS'
DIMS = (((1,), (0,)), ((), ()))


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
                 help='rows of lhs/cotangent the CPU leg processes (0 = all '
                 'for the one-pass baseline of the default run; the reference '
                 'arm sizes its sample from --steps/--warmup)')
  p.add_argument('--no-cpu-baseline', action='store_true')
  p.add_argument('--no-e2e', action='store_true')
  p.add_argument('--no-extras', action='store_true',
                 help='skip the other BASELINE.json configurations (1 GPU)')
  p.add_argument('--sustained-seconds', type=float, default=2.0,
                 help='length of the second, long timed region (0 = skip)')
  p.add_argument('--workload', default='c2',
                 choices=['c1', 'c2', 'c3', 'c4', 'int8', 'c2_delayed', 'stack',
                          'exchange'],
                 help='c2 is the headline workload (with the others as '
                 '`extras` in its line); naming another one times that alone')
  p.add_argument('--m', type=int, default=16,
                 help='rows of the activation for --workload c4')
  p.add_argument('--eager', action='store_true',
                 help='launch every kernel from Python each step instead of '
                 'replaying a recorded step (CUDA graph at 1 GPU, call tape '
                 'at several)')
  p.add_argument('--gemm', default='tcgen05',
                 choices=['tcgen05', 'cta1', 'cta2', 'wide'],
                 help='tile shape of the tensor-core kernel (default: automatic)')
  p.add_argument('--drhs-slices', type=int, default=2)
  p.add_argument('--overlap-sms', type=int, default=16)
  p.add_argument('--ranks', type=int, default=2, choices=[2, 4, 8],
                 help='ranks emulated by --workload exchange')
  p.add_argument('--timeline', default='',
                 help='after the measurements, write the device timeline of '
                 'three more steps of rank 0 to this file (torch.profiler)')
  p.add_argument('--exchange', default='auto', choices=['auto', 'nccl'],
                 help='drhs exchange at several GPUs: auto = one kernel over '
                 'peer memory where it can be set up, nccl = reduce-scatter + '
                 'dequantize + all-gather')
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


def workload_name(args):
  return (f'{args.kind} dot_general {args.size}x{args.size}x{args.size} '
          'fwd+dlhs+drhs, bf16 in/out, per-tensor absmax scales')


def config_dict(args, world):
  """The `config` object of the JSON line; both arms print the same one."""
  n = args.size
  m_local = n if args.scaling == 'weak' else n // world
  return {
      'workload': workload_name(args),
      'rows_per_gpu': m_local, 'global_rows': m_local * world,
      'parallelism': f'rows sharded over {world} GPU(s)',
      'l2': 'inputs (3 x 134 MB bf16 + quantized copies) exceed the 126 MB L2',
  }


def measured_peaks():
  path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
  if os.path.exists(path):
    with open(path) as f:
      d = json.load(f)
    return {'hbm_gbs': d['hbm_gbs'], 'bf16': d['bf16_tflops'],
            'bf16_sustained': d.get('bf16_tflops_sustained', d['bf16_tflops']),
            'src': 'of measured (MEASURED_PEAKS.json)'}
  return {'hbm_gbs': 6650.0, 'bf16': 1590.0, 'bf16_sustained': 1400.0,
          'src': 'of fallback (6.65 TB/s, 1.59 PFLOP/s bf16)'}


# ---------------------------------------------------------------------------
# CPU legs: the oracle on a bounded sample


def use_all_host_cores():
  """BLAS threads = host cores (a launcher may have exported OMP_NUM_THREADS=1
  before numpy was loaded). Returns the thread count in effect."""
  n = os.cpu_count() or 1
  try:
    import numpy as np  # the BLAS behind it must be loaded before it is asked
    import threadpoolctl
    np.ones((8, 8), np.float32) @ np.ones((8, 8), np.float32)
    threadpoolctl.threadpool_limits(limits=n)
    infos = threadpoolctl.threadpool_info()
    return max([i.get('num_threads', 1) for i in infos] + [1])
  except Exception:  # pylint: disable=broad-except
    return n


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


def run_reference_arm(args, lines):
  """The reference's CPU path (its numpy restatement) on this box's host
  cores: --warmup + --steps passes, each over a sample of the workload's rows
  sized so that the whole run stays within a few minutes."""
  rank = int(os.environ.get('RANK', '0'))
  if rank != 0:
    return
  cores = use_all_host_cores()
  n = args.size
  if args.cpu_sample_rows:
    rows = args.cpu_sample_rows
  else:
    # cost model t(rows) = fixed (the rhs side) + per_row * rows from two probes
    r1, r2 = min(256, n), min(512, n)
    _, t1 = cpu_sample(args, r1)
    _, t2 = cpu_sample(args, r2)
    per_row = max((t2 - t1) / max(r2 - r1, 1), 1e-6)
    fixed = max(t1 - per_row * r1, 0.0)
    budget = 150.0 / max(args.steps + args.warmup, 1)
    rows = int((budget - fixed) / per_row) if budget > fixed else r1
    rows = max(r1, min(n, rows // 256 * 256))
  for _ in range(args.warmup):
    cpu_sample(args, rows)
  vals, times = [], []
  for _ in range(args.steps):
    v, dt = cpu_sample(args, rows)
    vals.append(v)
    times.append(dt)
  value = sum(vals) / len(vals)
  sample = (f'{rows} of {n} lhs/cotangent rows against the full {n}x{n} rhs '
            f'per step, {args.steps} steps after {args.warmup} warm-up; '
            'numpy+ml_dtypes restatement on all host cores (jax is not '
            'installed, so the reference itself cannot run); TOPS counts the '
            'operations of the sampled rows')
  world = int(os.environ.get('WORLD_SIZE', str(args.gpus)))
  line = {
      'impl': 'reference', 'metric': METRIC, 'value': value, 'unit': UNIT,
      'n_gpus': args.gpus, 'steps': args.steps, 'warmup': args.warmup,
      'ms_per_step': 1e3 * sum(times) / len(times), 'higher_is_better': True,
      'scaling': args.scaling, 'vs_baseline': None,
      'dtype': 'f8e4m3/f8e5m2->f32' if args.kind == 'fp8' else 's8->s32',
      'data': 'synthetic', 'config': config_dict(args, max(world, args.gpus)),
      'cpu_baseline': {'value': value, 'unit': UNIT, 'cores': cores,
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
    return self.summarize(rest.splitlines(), self.t0, self.t1, self.mx)

  @classmethod
  def summarize(cls, lines, t0, t1, mx):
    """Median / minimum SM clock and the clock event reasons of the polls
    ("time clock reasons" per line) that fall between t0 and t1."""
    clocks, bits, every = [], 0, []
    for line in lines:
      parts = line.split()
      if len(parts) != 3:
        continue
      try:
        t, c, r = float(parts[0]), int(parts[1]), int(parts[2])
      except ValueError:
        continue
      every.append((t, c, r))
      # only samples taken while the timed region was running count
      if t0 is not None and not t0 <= t <= t1:
        continue
      clocks.append(c)
      bits |= r
    if not clocks and every and t0 is not None:
      # A region of a few milliseconds can fall between two polls: take the
      # polls on either side of it (the GPU is under the same load there: the
      # warm-up before, the next region after).
      before = [e for e in every if e[0] < t0][-1:]
      after = [e for e in every if e[0] > t1][:1]
      for t, c, r in before + after:
        if min(abs(t - t0), abs(t - t1)) < 0.05:
          clocks.append(c)
          bits |= r
    clocks.sort()
    reasons = sorted(k for k, m in cls.MASKS.items() if bits & m)
    return {'sm_mhz': clocks[len(clocks) // 2] if clocks else None,
            'sm_min_mhz': clocks[0] if clocks else None,
            'sm_max_mhz': mx, 'reasons': reasons,
            'samples': len(clocks)}


def timed_region(torch, step, steps, device_index, barrier=None):
  """`steps` calls of step() between two events on the current stream, with
  the clocks sampled meanwhile. Returns (ms per step, clocks, host ms per step)."""
  barrier = barrier or torch.cuda.synchronize
  sampler = ClockSampler(device_index)
  e0 = torch.cuda.Event(enable_timing=True)
  e1 = torch.cuda.Event(enable_timing=True)
  sampler.start()
  barrier()
  sampler.mark_begin()
  e0.record()
  t_host = time.perf_counter()
  for _ in range(steps):
    step()
  host_ms = (time.perf_counter() - t_host) * 1e3 / steps
  e1.record()
  barrier()
  sampler.mark_end()
  clocks = sampler.stop()
  return e0.elapsed_time(e1) / steps, clocks, host_ms


def write_timeline(torch, step, path, steps=3):
  """Diagnosis, outside every timed region: `steps` more calls of step() under
  torch.profiler (CUPTI activity records, no replay of kernels) and the device
  activities of this rank as text, one line per kernel / copy / collective:
  start [us from the first], duration [us], stream, name."""
  from torch.profiler import ProfilerActivity, profile
  torch.cuda.synchronize()
  with profile(activities=[ProfilerActivity.CUDA]) as prof:
    for _ in range(steps):
      step()
    torch.cuda.synchronize()
  import tempfile
  with tempfile.NamedTemporaryFile(suffix='.json') as f:
    prof.export_chrome_trace(f.name)
    events = json.load(open(f.name)).get('traceEvents', [])
  rows = [(e['ts'], e.get('dur', 0), e.get('args', {}).get('stream', ''),
           e.get('name', '')) for e in events
          if e.get('ph') == 'X' and e.get('cat') in (
              'kernel', 'gpu_memcpy', 'gpu_memset')]
  rows.sort()
  t0 = rows[0][0] if rows else 0
  with open(path, 'w') as f:
    for ts, dur, stream, name in rows:
      f.write('%10.1f %9.1f  s%-3s %s\n' % (ts - t0, dur, stream, name[:120]))


def capture_graph(torch, step, barrier=None):
  """Captures step() in a CUDA graph; returns (replay, outputs of the capture)."""
  barrier = barrier or torch.cuda.synchronize
  side = torch.cuda.Stream()
  side.wait_stream(torch.cuda.current_stream())
  with torch.cuda.stream(side):
    step()
  torch.cuda.current_stream().wait_stream(side)
  barrier()
  graph = torch.cuda.CUDAGraph()
  with torch.cuda.graph(graph):
    outs = step()
  for _ in range(3):
    graph.replay()
  barrier()
  return graph.replay, outs, graph


# ---------------------------------------------------------------------------
# parity of the sharded step against the unsharded one (outside any timing)


def sharded_parity_check(torch, dist, rank, world, dev, m_local=2048, k=1024,
                         n=1024, traced=True, exchange='auto'):
  """Runs a small row-sharded step and, on every rank, the same problem
  unsharded; returns a dict of 'ok' / 'MISMATCH' per case. int8: bit for bit.
  fp8: out and dlhs bit for bit (rows are independent given the agreed
  scales), drhs within max(6 bf16 ulps, 1e-5 * sum |g||lhs|) because the
  ranks' f32 partial sums are added in another order than one device's."""
  from aqt_b200 import distributed as aqt_dist
  from aqt_b200 import engine
  result = {}
  for kind in ('int8', 'fp8'):
    for per_tensor in (True, False):
      cfg = make_cfg(kind)
      if not per_tensor:
        for raw in (cfg.fwd, cfg.dlhs, cfg.drhs):
          raw.dg_quantizer.lhs.calib_shared_axes = None
          raw.dg_quantizer.rhs.calib_shared_axes = None
      gen = torch.Generator(device=dev)
      gen.manual_seed(7)
      m = m_local * world
      lhs = torch.randn(m, k, device=dev, generator=gen).to(torch.bfloat16)
      rhs = (torch.randn(k, n, device=dev, generator=gen) * 0.03).to(
          torch.bfloat16)
      g = torch.randn(m, n, device=dev, generator=gen).to(torch.bfloat16)
      sl = slice(rank * m_local, (rank + 1) * m_local)
      a, c = lhs[sl].contiguous(), g[sl].contiguous()
      op = aqt_dist.ShardedDotGeneral(cfg, exchange=exchange)

      def step(a_, b_, c_, op=op):
        out, bp = op.vjp(a_, b_, DIMS)
        return (out,) + tuple(bp(c_))

      if traced and per_tensor:
        out, dl, dr = engine.TracedStep(step, a, rhs, c)(a, rhs, c)
      else:
        out, dl, dr = step(a, rhs, c)
      wo, wbp = cfg.vjp(lhs, rhs, DIMS)
      wl, wr = wbp(g)
      torch.cuda.synchronize()
      engine.check_status()
      bad = []
      if not torch.equal(out, wo[sl]):
        bad.append('out')
      if not torch.equal(dl, wl[sl]):
        bad.append('dlhs')
      if kind == 'int8':
        if not torch.equal(dr, wr):
          bad.append('drhs')
      else:
        # The f32 accumulators differ by rounding noise; each of the three
        # bf16 roundings of the dequantizing chain (cast, x scale, x scale)
        # can then land one step apart and the steps add up: 2 bf16 ulps
        # per rounding bound the end-to-end difference.
        want = wr.double()
        ulp = 2.0 ** (torch.floor(torch.log2(want.abs().clamp_min(1e-38))) - 7)
        bound = 2.0 * (lhs.float().abs().t() @ g.float().abs()).double()
        tol = torch.maximum(6.0 * ulp, 1e-5 * bound)
        diff = (dr.double() - want).abs()
        if not bool((diff <= tol).all()):
          bad.append('drhs(max %.1f ulp)' % float((diff / ulp).max().item()))
      flag = torch.tensor([0 if bad else 1], device=dev)
      dist.all_reduce(flag, op=dist.ReduceOp.MIN)
      result[f'{kind}_{"per_tensor" if per_tensor else "per_channel"}'] = (
          'ok' if int(flag.item()) else 'MISMATCH' + (
              ': ' + ', '.join(bad) if bad else ' (on another rank)'))
      result.setdefault('exchange', op.exchange_used)
  return result


# ---------------------------------------------------------------------------
# the other BASELINE.json configurations (1 GPU, device-resident)


def build_workload(name, args, torch, dev):
  """Returns (step, ops per step, minimum HBM bytes per step, description,
  bound) for one of: c1, c3, c4 (with args.m), int8 (the 8192^3 step in
  int8), stack (one Llama-3-8B-shaped decoder layer's seven projections)."""
  from aqt_b200.v2 import aqt_dot_general as adg
  from aqt_b200.v2 import config
  from aqt_b200.v2 import stochastic_rounding as sr
  from aqt_b200.v2 import utils
  from aqt_b200.v2.flax import aqt_flax
  gen = torch.Generator(device=dev)
  gen.manual_seed(0)
  rn = lambda shape, std, dt: (torch.randn(shape, device=dev, generator=gen)
                               * std).to(dt)
  if name == 'c1':
    lhs = rn((1024, 4096), 1.0, torch.float32)
    rhs = rn((4096, 4096), 1.0 / 64, torch.float32)
    g = rn((1024, 4096), 1.0, torch.float32)
    cfg = config.fully_quantized(fwd_bits=8, bwd_bits=8,
                                 use_stochastic_rounding=False)

    def step():
      out, bp = cfg.vjp(lhs, rhs, DIMS)
      return out, bp(g)

    return (step, 3 * 2 * 1024 * 4096 * 4096, 201e6,
            'config 1: int8 [1024,4096]x[4096,4096] f32 in/out, per-channel '
            'absmax, RNE, fwd+dlhs+drhs', 'hbm')
  if name in ('int8', 'c2_delayed'):
    n = args.size
    lhs = rn((n, n), 1.0, torch.bfloat16)
    rhs = rn((n, n), n ** -0.5, torch.bfloat16)
    g = rn((n, n), 1.0, torch.bfloat16)
    if name == 'int8':
      cfg = make_cfg('int8')
      what = (f'int8 dot_general {n}^3 fwd+dlhs+drhs, bf16 in/out, per-tensor '
              'absmax scales (config 2 in int8)')
    else:
      import functools
      from aqt_b200.v2.flax import delayed_scaling_calibration as dsc
      cfg = make_cfg('fp8')
      for raw in (cfg.fwd, cfg.dlhs, cfg.drhs):
        for qz in (raw.dg_quantizer.lhs, raw.dg_quantizer.rhs):
          qz.calibration = functools.partial(dsc.DelayedScalingCalibration)
      cfg = config.set_context(cfg, key=None, train_step=None)
      what = (f'fp8 dot_general {n}^3 fwd+dlhs+drhs, bf16 in/out, per-tensor '
              'DELAYED scaling (history of 1024 maxima): config 2 without an '
              'absmax pass on the critical path')

    def step():
      out, bp = cfg.vjp(lhs, rhs, DIMS)
      return out, bp(g)

    return (step, 3 * 2 * n ** 3, 6 * 2 * n * n, what, 'tensor')
  if name == 'c3':
    b, t, h, d = 8, 2048, 32, 128
    if os.environ.get('AQT_C3_BH'):  # a slice of the batch, for profiling
      b, h = (int(v) for v in os.environ['AQT_C3_BH'].split(','))
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

    def step():
      out, bp = cfg.vjp(q, k, dims)
      return out, bp(g)

    return (step, 3 * 2 * b * h * t * t * d, 5.1e9 * (b * h) / 256.0,
            f"config 3: int8 einsum 'bthd,bshd->bhts' B{b} H{h} T=S=2048 D128, "
            'bf16, per-token scales, fwd + both gradients, stochastic '
            'rounding from 4 given f32 noise tensors (2 x 4.29 GB + 2 x 0.27 GB '
            'read on top of the minimum bytes)', 'hbm')
  if name == 'c4':
    m, kk, n = args.m, 8192, 28672
    x = rn((m, kk), 1.0, torch.bfloat16)
    w = rn((kk, n), kk ** -0.5, torch.bfloat16)
    cfg = adg.dot_general_make(lhs_bits=8, rhs_bits=4)
    cfg.fwd.dg_quantizer.rhs.numerics.dtype = utils.int8
    conv = aqt_flax.AqtDotGeneral(
        cfg, rhs_quant_mode=utils.QuantMode.CONVERT,
        rhs_freeze_mode=aqt_flax.FreezerMode.CALIBRATION_AND_VALUE,
        use_legacy_freezer=False)
    conv(x, w, DIMS)
    rhs_qt = conv.variables['aqt']['qrhs']['frozen']
    del conv

    def step():
      # dg_core is what AqtDotGeneral calls after copying its config; calling
      # it directly keeps the per-call deepcopy out of a serving loop. The
      # float weights are not read in SERVE mode.
      return cfg.dg_core(x, w, None, rhs_qt, DIMS)[0]

    return (step, 2 * m * kk * n,
            kk * n + m * kk * 2 + m * n * 2 + 2 * n + 2 * m,
            f'config 4: serving GEMM M={m} K=8192 N=28672, int8 activations '
            'per token x int4-in-int8 frozen weights per channel, bf16 out',
            'hbm' if m <= 256 else 'tensor')
  if name == 'exchange':
    # The fused exchange kernel alone, on ONE device: every "rank's" band of
    # accumulators and its copy of the result are buffers of this GPU (the
    # kernel does not care whose memory a pointer names), so what is timed is
    # the kernel's own rate -- bulk copies, sum, dequantization, stores --
    # against HBM instead of NVLink. Band of the 2-slice 8192^3 step:
    # 4096 / ranks rows x 8192 columns.
    from aqt_b200 import engine
    world = args.ranks
    rows, n = 4096 // world, 8192
    raw = make_cfg(args.kind).drhs
    lhs = rn((rows, 128), 1.0, torch.bfloat16)
    rhs = rn((128, n), 0.1, torch.bfloat16)
    d, _ = engine.dg_raw(raw, lhs, rhs, None, None, DIMS, defer_dequant=True)
    accs = [d.acc.clone() for _ in range(world)]
    outs = [torch.empty((rows, n), device=dev, dtype=torch.bfloat16)
            for _ in range(world)]
    acc_ptrs = [a.data_ptr() for a in accs]
    out_ptrs = [o.data_ptr() for o in outs]

    def step(keep=(accs, outs, lhs, rhs)):
      # (the default argument keeps the buffers alive: the kernel is given
      # their addresses, not the tensors)
      d.exchange_rows(0, rows, 0, acc_ptrs, out_ptrs, max_sms=args.overlap_sms)
      return keep[1]

    moved = world * rows * n * (4 + 2)
    return (step, world * rows * n, moved,
            f'fused exchange kernel on one device: {world} ranks, band of {rows} '
            f'x {n} accumulators ({args.kind}), {args.overlap_sms} SMs '
            '(0 = all), bytes = ranks x band x (4 read + 2 written)', 'hbm')
  raise ValueError(name)


def time_workload(name, args, torch, dev, lib, engine, peaks, steps=None):
  step, ops, min_bytes, desc, bound = build_workload(name, args, torch, dev)
  for _ in range(3):
    step()
  torch.cuda.synchronize()
  engine.check_status()
  l0 = lib.aqtb200_kernel_launch_count()
  replay, keep, graph = capture_graph(torch, step)
  launches = (lib.aqtb200_kernel_launch_count() - l0) // 2  # two passes: dry run, capture
  steps = steps or args.steps
  ms, clocks, _ = timed_region(torch, replay, steps, dev.index or 0)
  engine.check_status()
  tops = ops / (ms * 1e-3) / 1e12
  gbs = min_bytes / (ms * 1e-3) / 1e9
  rec = {'workload': desc, 'ms_per_step': ms, 'tops': tops,
         'min_bytes_gbs': gbs, 'bound': bound, 'launches_per_step': launches,
         'steps': steps, 'launch': 'cuda_graph replay', 'sm_mhz': clocks['sm_mhz'],
         'reasons': clocks['reasons']}
  if bound == 'tensor':
    rec['frac'] = tops / (2.0 * peaks['bf16'])
    rec['frac_of'] = '2 x bf16_tflops, ' + peaks['src']
  else:
    rec['frac'] = gbs / peaks['hbm_gbs']
    rec['frac_of'] = 'minimum bytes / time over hbm_gbs, ' + peaks['src']
  del keep, graph
  return rec


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
  peaks = measured_peaks()

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
    op = aqt_dist.ShardedDotGeneral(cfg, drhs_slices=args.drhs_slices,
                                    overlap_sms=args.overlap_sms,
                                    exchange=args.exchange)

  def eager_step(a, b, c):
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
    eager_step(lhs, rhs, g)
  barrier()
  engine.check_status()

  # The step is recorded once and replayed, as a compiled training step would
  # be. One GPU: a CUDA graph of its kernels. Several GPUs: the call tape of
  # engine.TracedStep (kernels AND collectives re-issued from a flat list, the
  # collectives stay outside graphs); its first replay is compared bit for bit
  # with an eager step.
  launch = 'eager'
  launches_per_step = None
  outs = eager_step(lhs, rhs, g)
  step = lambda: eager_step(lhs, rhs, g)
  if not args.eager:
    try:
      l0 = lib.aqtb200_kernel_launch_count()
      if world == 1:
        step, outs, graph = capture_graph(torch, step, barrier)
        launches_per_step = (lib.aqtb200_kernel_launch_count() - l0) // 2
        launch = 'cuda_graph replay of the whole step'
      else:
        traced = engine.TracedStep(eager_step, lhs, rhs, g)
        outs = traced.outputs
        step = lambda: traced(lhs, rhs, g)
        launch = (f'call tape replay ({traced.n_ops} recorded calls: kernels '
                  'and collectives), first replay verified bit for bit '
                  'against an eager step')
        for _ in range(3):
          step()
      barrier()
      engine.check_status()
    except Exception as e:  # pylint: disable=broad-except
      # recording is an optimisation of the launch path only: run eagerly
      print(f'step recording failed ({type(e).__name__}: {e}); eager',
            file=sys.stderr)
      launch, launches_per_step = 'eager', None
      step = lambda: eager_step(lhs, rhs, g)
      torch.cuda.synchronize()

  launches0 = lib.aqtb200_kernel_launch_count()
  ms, clocks, host_ms = timed_region(torch, step, args.steps, local_rank,
                                     barrier)
  launches = lib.aqtb200_kernel_launch_count() - launches0
  if launches_per_step is not None:
    launches = launches_per_step * args.steps  # replayed, not re-issued
  engine.check_status()

  def max_over_ranks(v):
    if world > 1:
      t = torch.tensor([v], device=dev, dtype=torch.float64)
      dist.all_reduce(t, op=dist.ReduceOp.MAX)
      return float(t.item())
    return v

  ms = max_over_ranks(ms)
  ops_step = 3 * 2 * m_global * n * n
  value = ops_step / (ms * 1e-3) / 1e12

  # ---- the same measurement over seconds instead of milliseconds
  sustained = None
  if args.sustained_seconds > 0:
    k_long = max(args.steps, int(math.ceil(args.sustained_seconds * 1e3 / ms)))
    sms, sclocks, _ = timed_region(torch, step, k_long, local_rank, barrier)
    sms = max_over_ranks(sms)
    sval = ops_step / (sms * 1e-3) / 1e12
    sustained = {
        'value': sval, 'unit': UNIT, 'ms_per_step': sms, 'steps': k_long,
        'seconds': sms * k_long * 1e-3, 'clocks': sclocks,
        'step_frac': sval / world / (2.0 * peaks['bf16_sustained']),
        'step_frac_of': '2 x bf16_tflops_sustained, ' + peaks['src']}
    engine.check_status()

  if args.timeline:
    path = args.timeline if rank == 0 else os.devnull
    write_timeline(torch, step, path)
    barrier()

  # ---- sharded against unsharded results, outside any timed region
  parity = None
  if world > 1:
    try:
      parity = sharded_parity_check(torch, dist, rank, world, dev,
                                    exchange=args.exchange)
    except Exception as e:  # pylint: disable=broad-except
      parity = {'error': f'{type(e).__name__}: {e}'}

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
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(k):
      pipe.submit(h, ho)
    pipe.drain()
    e1.record()
    barrier()
    ems = max_over_ranks(e0.elapsed_time(e1) / k)
    e2e = {'value': ops_step / (ems * 1e-3) / 1e12, 'unit': UNIT,
           'h2d_bytes_per_step': sum(t.numel() * t.element_size() for t in h),
           'd2h_bytes_per_step': sum(t.numel() * t.element_size() for t in ho),
           'ms_per_step': ems,
           'path': 'aqt_b200.host_io.HostStepPipeline (pinned host buffers, '
                   'copies of neighbouring steps overlap compute)'}
    del pipe, h, ho

  # ---- roofline of the dominant kernel: the tcgen05 GEMM, timed alone
  roof = None
  if rank == 0:
    roof = gemm_roofline(args, cfg, lhs, rhs, torch, engine, peaks)
    # the whole step (calibration, quantization and the three GEMMs) against
    # the same tensor peaks, per GPU
    roof['step_achieved'] = value / world
    roof['step_frac'] = value / world / roof['peak']
    roof['step_frac_2x_bf16'] = value / world / roof['peak_2x_bf16']

  if rank != 0:
    if world > 1:
      dist.destroy_process_group()
    return

  extras = None
  if world == 1 and not args.no_extras and args.size == 8192:
    del outs
    extras = {}
    todo = [('int8', None), ('c2_delayed', None), ('c1', None), ('c3', None),
            ('c4', 16), ('c4', 256), ('c4', 4096)]
    if args.kind == 'int8':
      todo = todo[1:]
    for name, m in todo:
      key = name if m is None else f'{name}_m{m}'
      try:
        if m is not None:
          args.m = m
        extras[key] = time_workload(name, args, torch, dev, lib, engine, peaks)
      except Exception as e:  # pylint: disable=broad-except
        extras[key] = {'error': f'{type(e).__name__}: {e}'}
      torch.cuda.empty_cache()

  cpu = None
  if not args.no_cpu_baseline and world == 1:
    cores = use_all_host_cores()
    cpu_rows = args.cpu_sample_rows or n
    v, dt = cpu_sample(args, cpu_rows)
    cpu = {'value': v, 'unit': UNIT, 'cores': cores, 'kind': 'port',
           'sample': (f'{cpu_rows} of {n} lhs/cotangent rows against '
                      f'the full rhs, one pass, {dt:.1f} s; numpy+ml_dtypes '
                      'restatement (jax not installed)')}
  line = {
      'metric': METRIC, 'value': value, 'unit': UNIT, 'n_gpus': world,
      'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': ms,
      'higher_is_better': True, 'scaling': args.scaling, 'vs_baseline': None,
      'dtype': 'f8e4m3/f8e5m2->f32' if args.kind == 'fp8' else 's8->s32',
      'data': 'synthetic',
      'config': config_dict(args, world),
      'launch': launch,
      'clocks': clocks,
      'e2e': e2e,
      'gpu_launches': int(launches),
      'host_issue_ms_per_step': host_ms,
      'sustained': sustained,
      'roofline': roof,
      'cpu_baseline': cpu,
  }
  if parity is not None:
    line['parity_check'] = parity
  if extras is not None:
    line['extras'] = extras
  lines.append(json.dumps(line))
  if world > 1:
    dist.destroy_process_group()


def mma_peak(args, torch, lib, mmas_per_sm=40000, reps=3):
  """8-bit tensor-pipe ceiling of this GPU, measured now: nothing but MMA issue
  from shared memory (aqtb200_mma_peak), a few milliseconds per launch."""
  from aqt_b200 import _lib
  stream = torch.cuda.current_stream().cuda_stream
  status = torch.zeros(4, dtype=torch.int32, device='cuda')
  is_int = 1 if args.kind == 'int8' else 0
  _lib.check(lib.aqtb200_mma_peak(is_int, 2000, status.data_ptr(), stream),
             'mma_peak')
  torch.cuda.synchronize()
  if int(status[0].item()):
    return None
  sampler = ClockSampler(torch.cuda.current_device(), period_ms=2)
  sampler.start()
  e0 = torch.cuda.Event(enable_timing=True)
  e1 = torch.cuda.Event(enable_timing=True)
  torch.cuda.synchronize()
  sampler.mark_begin()
  e0.record()
  for _ in range(reps):
    lib.aqtb200_mma_peak(is_int, mmas_per_sm, status.data_ptr(), stream)
  e1.record()
  torch.cuda.synchronize()
  sampler.mark_end()
  clocks = sampler.stop()
  if int(status[0].item()):
    return None
  ms = e0.elapsed_time(e1) / reps
  sms = ctypes_sm_count(lib)
  launched = (mmas_per_sm + 15) // 16 * 16
  ops = sms * launched * 2.0 * 128 * 256 * 32
  return {'tops': ops / (ms * 1e-3) / 1e12, 'ms_per_launch': ms,
          'sm_mhz': clocks['sm_mhz'], 'reasons': clocks['reasons'],
          'kind': 'kind::i8' if is_int else 'kind::f8f6f4 (e4m3 x e4m3)'}


def ctypes_sm_count(lib):
  import ctypes as C
  n = C.c_int(0)
  lib.aqtb200_device_sm_count(C.byref(n))
  return n.value


def gemm_roofline(args, cfg, lhs, rhs, torch, engine, peaks):
  """Average duration of the forward GEMM launch alone (CUDA events on the
  launching stream) against the 8-bit tensor peak measured in the same run."""
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
  peak2 = 2.0 * peaks['bf16']
  measured = None
  try:
    measured = mma_peak(args, torch, lib)
  except Exception as e:  # pylint: disable=broad-except
    print(f'mma peak measurement failed: {e}', file=sys.stderr)
  if measured is not None:
    peak = measured['tops']
    src = ('measured in this run: tcgen05.mma issue only, operands in shared '
           f"memory, {measured['kind']}, {measured['ms_per_launch']:.2f} ms per "
           f"launch at {measured['sm_mhz']} MHz")
  else:
    peak, src = peak2, '2 x bf16_tflops (burst), ' + peaks['src']
  # DRAM bytes (read + write) of one launch of this kernel at this shape come
  # from an ncu capture of the same kernel (profiles/), not from this run:
  # nothing here is timed under a profiler.
  traffic = 456.5e6 if (m, n, k) == (8192, 8192, 8192) else None
  return {'bound': 'tensor',
          'kernel': 'gemm_tcgen05_wide_kernel (forward GEMM, 256x512 CTA-pair tiles)',
          'achieved': achieved, 'peak': peak, 'unit': 'TFLOP/s',
          'frac': achieved / peak, 'peak_source': src,
          'peak_2x_bf16': peak2, 'frac_2x_bf16': achieved / peak2,
          'peak_2x_bf16_source': '2 x bf16_tflops (burst), ' + peaks['src'],
          'mma_peak': measured,
          'traffic': traffic, 'traffic_source': 'from profile (ncu, same kernel and shape)',
          'algorithmic_bytes': float(m * k + n * k + 2 * m * n), 'ms_per_launch': ms}


def run_single_workload(args, lines):
  """--workload other than c2: that configuration alone, 1 GPU."""
  import torch
  from aqt_b200 import _lib
  from aqt_b200 import engine
  torch.cuda.set_device(0)
  dev = torch.device('cuda', 0)
  lib = _lib.load()
  engine.set_gemm_impl(args.gemm)
  peaks = measured_peaks()
  rec = time_workload(args.workload, args, torch, dev, lib, engine, peaks)
  lines.append(json.dumps({
      'metric': METRIC, 'value': rec['tops'], 'unit': UNIT,
      'n_gpus': 1, 'steps': args.steps, 'warmup': 3,
      'ms_per_step': rec['ms_per_step'], 'higher_is_better': True,
      'scaling': 'weak', 'vs_baseline': None, 'dtype': 's8->s32',
      'data': 'synthetic', 'config': {'workload': rec['workload']},
      'detail': rec,
      'gpu_launches': int(rec['launches_per_step'] * args.steps),
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
    elif args.workload == 'stack':
      from aqt_b200 import layer_stack
      layer_stack.bench_main(args, lines)
    elif args.workload != 'c2':
      run_single_workload(args, lines)
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
