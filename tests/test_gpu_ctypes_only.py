"""The C ABI driven from ctypes and numpy alone: no torch in the process.

A host that owns no tensor library binds libaqt_b200.so exactly like this
(device memory through aqtb200_dev_alloc / _h2d / _d2h); the result is checked
against the oracle bit for bit.
"""

import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

_SCRIPT = r'''
import ctypes as C, sys
sys.path.insert(0, %(root)r)
import numpy as np
from aqt_b200 import _lib
from aqt_b200.v2 import aqt_dot_general as aqt
from oracle import aqt_oracle as orc

lib = _lib.load()
chk = lambda rc, what: _lib.check(rc, what)
chk(lib.aqtb200_set_device(0), 'set_device')

def dev(a):
  p = C.c_void_p()
  chk(lib.aqtb200_dev_alloc(C.byref(p), a.nbytes), 'alloc')
  chk(lib.aqtb200_h2d(p, a.ctypes.data, a.nbytes, None), 'h2d')
  return p

def dev_empty(nbytes):
  p = C.c_void_p()
  chk(lib.aqtb200_dev_alloc(C.byref(p), nbytes), 'alloc')
  chk(lib.aqtb200_dev_memset(p, 0, nbytes, None), 'memset')
  return p

m, k, n = 96, 256, 160
rng = np.random.default_rng(0)
lhs = rng.standard_normal((m, k)).astype(np.float32)
rhs = (rng.standard_normal((k, n)) * 0.1).astype(np.float32)
dims = (((1,), (0,)), ((), ()))
raw = aqt.dot_general_raw_make(8, 8)           # int8 x int8, per-channel AbsMax
want, res = orc.dg_raw(raw, lhs, rhs, None, None, dims)

spec = _lib.QuantSpec(kind=_lib.NUM_INT, qdtype=_lib.S8, quant_bound=127.5,
                      clip_bound=127.0, per_tensor=0, compute_dtype=_lib.F32,
                      scale_dtype=_lib.F32)
d = _lib.DgRawDesc()
d_lhs, d_rhs = dev(lhs), dev(rhs)
d.lhs = _lib.View(ptr=d_lhs, dtype=_lib.F32, b0=1, b1=1, rows=m, cols=k,
                  b0_stride=0, b1_stride=0, row_stride=k, col_stride=1)
# rhs [K, N] row-major: rows = N (stride 1), cols = K (stride N)
d.rhs = _lib.View(ptr=d_rhs, dtype=_lib.F32, b0=1, b1=1, rows=n, cols=k,
                  b0_stride=0, b1_stride=0, row_stride=1, col_stride=n)
d.lhs_spec, d.rhs_spec = spec, spec
ldk = (k + 15) // 16 * 16
d.lhs_q, d.rhs_q = dev_empty(m * ldk), dev_empty(n * ldk)
d.lhs_scale, d.rhs_scale = dev_empty(4 * m), dev_empty(4 * n)
d.dequant_dtype = d.out_dtype = _lib.F32
d.out = dev_empty(4 * m * n)
d.out_m_stride, d.out_n_stride = n, 1
d.scope_name = b'aqt_fwd'
ws_bytes = lib.aqtb200_dot_general_raw_workspace_bytes(C.byref(d))
ws = dev_empty(max(ws_bytes, 256))
status = dev_empty(16)
chk(lib.aqtb200_dot_general_raw(C.byref(d), ws, max(ws_bytes, 256), status,
                                None), 'dot_general_raw')
out = np.empty((m, n), np.float32)
q_lhs = np.empty((m, ldk), np.int8)
st = np.empty(4, np.int32)
chk(lib.aqtb200_d2h(out.ctypes.data, d.out, out.nbytes, None), 'd2h')
chk(lib.aqtb200_d2h(q_lhs.ctypes.data, d.lhs_q, q_lhs.nbytes, None), 'd2h')
chk(lib.aqtb200_d2h(st.ctypes.data, status, 16, None), 'd2h')
chk(lib.aqtb200_sync(None), 'sync')
assert st[0] == 0
np.testing.assert_array_equal(q_lhs[:, :k], res.lhs.qx.qvalue)
np.testing.assert_array_equal(out, want)
for p in (d_lhs, d_rhs, d.lhs_q, d.rhs_q, d.lhs_scale, d.rhs_scale, d.out, ws,
          status):
  chk(lib.aqtb200_dev_free(p), 'free')
assert 'torch' not in sys.modules, 'torch was imported'
print('ok: kernels launched', lib.aqtb200_kernel_launch_count())
'''


def test_dot_general_raw_through_ctypes_and_numpy_only(tmp_path):
  script = tmp_path / 'ctypes_only.py'
  script.write_text(_SCRIPT % {'root': ROOT})
  r = subprocess.run([sys.executable, str(script)], capture_output=True,
                     text=True, timeout=300)
  assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
  assert 'ok: kernels launched' in r.stdout
