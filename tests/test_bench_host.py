"""The CPU leg of bench.py (no GPU needed): the reference arm prints the line
the measurement contract asks for, with the repo arm's config object."""

import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_line():
  out = subprocess.run(
      [sys.executable, os.path.join(ROOT, 'bench.py'), '--impl', 'reference',
       '--size', '256', '--cpu-sample-rows', '256', '--steps', '2', '--warmup',
       '1'], capture_output=True, text=True, timeout=600, cwd=ROOT)
  assert out.returncode == 0, out.stderr[-2000:]
  line = json.loads(out.stdout.strip().splitlines()[-1])
  assert line['impl'] == 'reference'
  assert line['metric'] == 'quantized_dot_general_fwd_bwd_tops'
  assert line['unit'] == 'TOPS' and line['higher_is_better'] is True
  assert line['steps'] == 2 and line['warmup'] == 1 and line['value'] > 0
  assert line['cpu_baseline']['kind'] == 'port'
  assert line['cpu_baseline']['cores'] >= 1
  assert line['cpu_baseline']['value'] == line['value']
  assert line['e2e'] == {'value': line['value'], 'unit': 'TOPS',
                         'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0}
  sys.path.insert(0, ROOT)
  import bench
  # the config object is the one the repo arm prints for the same flags
  class A:  # the flags above, as bench.parse_args would hold them
    size, scaling, kind = 256, 'weak', 'fp8'
  assert line['config'] == bench.config_dict(A, 1)


def test_other_ranks_of_the_reference_arm_exit_quietly():
  env = dict(os.environ, RANK='1', WORLD_SIZE='2', LOCAL_RANK='1')
  out = subprocess.run(
      [sys.executable, os.path.join(ROOT, 'bench.py'), '--impl', 'reference',
       '--gpus', '2', '--size', '256', '--steps', '1', '--warmup', '0'],
      capture_output=True, text=True, timeout=600, cwd=ROOT, env=env)
  assert out.returncode == 0, out.stderr[-2000:]
  assert out.stdout.strip() == ''


def test_clock_poll_summary():
  sys.path.insert(0, ROOT)
  import bench
  s = bench.ClockSampler.summarize
  # polls inside the region only; reasons are OR-ed (0x4 = sw_power_cap, 0x8 = hw_slowdown)
  r = s(['1.0 1900 0', '1.01 1800 4', '1.02 1700 4', '2.0 1000 8'], 1.005, 1.025,
        1965)
  assert r == {'sm_mhz': 1800, 'sm_min_mhz': 1700, 'sm_max_mhz': 1965,
               'reasons': ['sw_power_cap'], 'samples': 2}
  # a region that falls between two polls takes its neighbours (within 50 ms)
  r = s(['1.0 1900 0', '1.04 1800 8'], 1.01, 1.03, 1965)
  assert r['samples'] == 2 and r['reasons'] == ['hw_slowdown']
  # ... but not polls from another time
  r = s(['0.5 1900 0', '2.0 1800 8'], 1.01, 1.03, 1965)
  assert r['samples'] == 0 and r['sm_mhz'] is None
