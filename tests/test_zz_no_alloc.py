"""aqtb200_quantize_static: the quantize entry point that allocates nothing.

Some hosts embed this library where device memory cannot be requested at call
time: the framework owns the allocator and hands a custom call nothing but its
operands and results, or the serving process forbids allocator calls after
start-up. For them the scratch that aqtb200_quantize takes from the caller sits
in a fixed array inside the library instead. This test drives the new entry
point through the C ABI and checks, on two calls in a row (the second one
finds the first one's leftovers in the shared array), that it returns exactly
the bytes the workspace-taking entry point returns, and that a request beyond
the array's capacity is refused with a message instead of being launched.

The file name sorts last on purpose: a run that stops at the first failure has
then already gone through every other test.
"""

import ctypes as C

import numpy as np
import pytest
import torch

from aqt_b200 import _lib

pytestmark = pytest.mark.gpu


def _view(t, rows, cols, row_stride, col_stride, code):
  v = _lib.View()
  v.ptr = t.data_ptr()
  v.dtype = code
  v.b0 = v.b1 = 1
  v.rows, v.cols = rows, cols
  v.b0_stride = v.b1_stride = 0
  v.row_stride, v.col_stride = row_stride, col_stride
  return v


def _spec(kind, qdtype, qb, cb, per_tensor, t_code):
  s = _lib.QuantSpec()
  s.kind, s.qdtype, s.quant_bound, s.clip_bound = kind, qdtype, qb, cb
  s.per_tensor = per_tensor
  s.compute_dtype = s.scale_dtype = t_code
  return s


def _both_ways(lib, x, view, spec, n_scales, rows, cols, q_dtype, s_dtype):
  ldq = (cols + 15) // 16 * 16
  stream = torch.cuda.current_stream().cuda_stream
  outs = []
  for static in (False, True):
    q = torch.full((rows, ldq), 0x55, dtype=torch.uint8, device='cuda')
    s = torch.zeros(n_scales, dtype=s_dtype, device='cuda')
    if static:
      rc = lib.aqtb200_quantize_static(C.byref(view), None, None, C.byref(spec),
                                       None, q.data_ptr(), s.data_ptr(), stream)
    else:
      nbytes = lib.aqtb200_quantize_workspace_bytes(C.byref(view), C.byref(spec))
      ws = torch.empty(nbytes, dtype=torch.uint8, device='cuda')
      rc = lib.aqtb200_quantize(C.byref(view), None, None, C.byref(spec), None,
                                q.data_ptr(), s.data_ptr(), ws.data_ptr(),
                                ws.numel(), stream)
    assert rc == 0, lib.aqtb200_last_error().decode()
    torch.cuda.synchronize()
    outs.append((q.cpu().numpy(), s.view(torch.int16 if s_dtype == torch.bfloat16
                                        else torch.int32).cpu().numpy()))
  (q0, s0), (q1, s1) = outs
  np.testing.assert_array_equal(s1, s0)
  np.testing.assert_array_equal(q1, q0)  # bit-exact, like every int/byte check
  del q_dtype, x


def test_static_entry_point_matches_workspace_entry_point():
  lib = _lib.load()
  torch.manual_seed(0)
  # call 1: bf16 [300, 520], one int8 scale per row (contraction contiguous)
  x1 = (torch.randn(300, 520, device='cuda') * 3).to(torch.bfloat16)
  _both_ways(lib, x1, _view(x1, 300, 520, 520, 1, _lib.BF16),
             _spec(_lib.NUM_INT, _lib.S8, 127.5, 127.0, 0, _lib.BF16),
             300, 300, 520, torch.int8, torch.bfloat16)
  # call 2, straight after: f32 [256, 512] read "transposed" (kept index
  # contiguous), one fp8 scale for the whole tensor; the shared array still
  # holds call 1's per-row maxima when this one starts.
  x2 = torch.randn(512, 256, device='cuda')
  _both_ways(lib, x2, _view(x2, 256, 512, 1, 256, _lib.F32),
             _spec(_lib.NUM_FP8, _lib.E4M3, 448.0, 448.0, 1, _lib.F32),
             1, 256, 512, torch.float8_e4m3fn, torch.float32)
  # and once more with per-row scales over the same memory
  _both_ways(lib, x2, _view(x2, 256, 512, 1, 256, _lib.F32),
             _spec(_lib.NUM_INT, _lib.S8, 127.5, 127.0, 0, _lib.F32),
             256, 256, 512, torch.int8, torch.float32)


def test_static_entry_point_refuses_what_does_not_fit():
  lib = _lib.load()
  rows = 65536 + 16  # one scale per row: more than the built-in array holds
  x = torch.zeros(rows, 16, device='cuda')
  q = torch.zeros(rows, 16, dtype=torch.uint8, device='cuda')
  s = torch.zeros(rows, device='cuda')
  rc = lib.aqtb200_quantize_static(
      C.byref(_view(x, rows, 16, 16, 1, _lib.F32)), None, None,
      C.byref(_spec(_lib.NUM_INT, _lib.S8, 127.5, 127.0, 0, _lib.F32)), None,
      q.data_ptr(), s.data_ptr(), torch.cuda.current_stream().cuda_stream)
  assert rc == -2
  msg = lib.aqtb200_last_error().decode()
  assert '65536' in msg and 'aqtb200_quantize' in msg
  torch.cuda.synchronize()
  assert int(q.sum()) == 0  # nothing was launched
