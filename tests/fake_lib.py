"""A CPU stand-in for libaqt_b200.so, for testing the HOST logic only.

TEST INFRASTRUCTURE. It implements the entry points of include/aqt_b200.h on
host memory with numpy, following the semantics written in that header, so the
planner in aqt_b200/engine.py (stride normalisation, view construction,
operand swapping, residual layouts) can be exercised by the CPU test suite
against the oracle. It is installed by monkeypatching `aqt_b200._lib.load`
inside tests; the product never imports it and never runs on it.
"""

import ctypes as C

import numpy as np

from aqt_b200 import _lib
from oracle import aqt_oracle as orc

_NP = {
    _lib.F32: np.dtype(np.float32), _lib.BF16: orc.bfloat16,
    _lib.S8: np.dtype(np.int8), _lib.E4M3: orc.float8_e4m3fn,
    _lib.E5M2: orc.float8_e5m2, _lib.S32: np.dtype(np.int32),
}


def _strided(ptr, code, extents, strides, writable=False):
  dt = _NP[code]
  extents = [int(e) for e in extents]
  strides = [int(s) for s in strides]
  if any(e == 0 for e in extents):
    return np.zeros(extents, dt)
  span = sum((e - 1) * abs(s) for e, s in zip(extents, strides)) + 1
  raw = (C.c_char * (span * dt.itemsize)).from_address(ptr)
  # as_strided cannot carry ml_dtypes through __array_interface__: stride an
  # unsigned view of the same width, then reinterpret.
  carrier = {1: np.uint8, 2: np.uint16, 4: np.uint32}[dt.itemsize]
  arr = np.frombuffer(raw, dtype=carrier)
  out = np.lib.stride_tricks.as_strided(
      arr, shape=extents, strides=[s * dt.itemsize for s in strides],
      writeable=writable)
  return out.view(dt)


def _view_array(v, rows=None):
  if not v.ptr:
    return None
  return _strided(v.ptr, v.dtype, [v.b0, v.b1, v.rows if rows is None else rows,
                                   v.cols],
                  [v.b0_stride, v.b1_stride, v.row_stride, v.col_stride])


def _deref(p, typ):
  """Unwraps ctypes.byref(struct) (or passes a struct / None through)."""
  del typ
  return getattr(p, '_obj', p)


class FakeLib:
  """Callable attributes named like the C symbols."""

  def __init__(self):
    self.err = b''
    self.calls = []

  # -- misc
  def aqtb200_version(self):
    return 1

  def aqtb200_last_error(self):
    return self.err

  def aqtb200_set_gemm_impl(self, impl):
    return 0

  def aqtb200_set_gemm_sm_budget(self, n):
    return 0

  def aqtb200_round_up(self, v, m):
    return (v + m - 1) // m * m

  def aqtb200_device_sm_count(self, out):
    return 0

  def _fail(self, code, msg):
    self.err = msg.encode()
    return code

  # -- quantize
  def aqtb200_quantize_workspace_bytes(self, x, spec):
    return 512

  def _quantize(self, x, pre, noise, spec, scale_in, q_out, scale_out):
    T = _NP[spec.compute_dtype]
    S = _NP[spec.scale_dtype]
    if not (x.col_stride == 1 or x.row_stride == 1 or x.rows <= 1
            or x.cols <= 1):
      return self._fail(-2, 'view must have a contiguous index')
    xv = _view_array(x)
    v = xv.astype(np.float32).astype(T)
    if pre is not None and pre.ptr:
      pv = _strided(pre.ptr, pre.dtype, [x.b0, x.b1, 1, x.cols],
                    [pre.b0_stride, pre.b1_stride, 0, pre.col_stride])
      v = orc.mul(v, pv.astype(np.float32).astype(T))
    ns = 1 if spec.per_tensor else x.b0 * x.b1 * x.rows
    if scale_in:
      scale = np.array(_strided(scale_in, spec.scale_dtype, [ns], [1]))
    else:
      axes = (0, 1, 2, 3) if spec.per_tensor else (3,)
      amax = np.max(np.abs(v), axis=axes, keepdims=True, initial=0)
      amax = np.where(amax == 0, np.ones_like(amax), amax).astype(T)
      bound = orc.mul(amax, np.asarray(spec.clipping_scale, T)) if (
          spec.clipping_scale) else amax
      scale = orc.div(bound, np.asarray(spec.quant_bound, T))
      if spec.po2_scale:
        scale = orc.ceil_to_po2(scale)
      scale = scale.astype(S).reshape(-1)
    if scale_out and scale_out != scale_in:
      _strided(scale_out, spec.scale_dtype, [ns], [1], True)[...] = scale
    if not q_out:
      return 0
    sc4 = scale.reshape((1, 1, 1, 1) if spec.per_tensor else
                        (x.b0, x.b1, x.rows, 1))
    s_inv = orc.reciprocal(sc4)
    s_inv = np.where(np.isinf(s_inv.astype(np.float32)),
                     np.ones_like(s_inv), s_inv)
    y = orc.mul(v, s_inv)
    if noise is not None and noise.ptr:
      nz = _view_array(noise)
      y = orc.add(y, np.asarray(nz, np.float32)).astype(y.dtype)
    y = orc.clip(y, -spec.clip_bound, spec.clip_bound)
    if spec.kind == _lib.NUM_INT:
      q = np.rint(y.astype(np.float32)).astype(np.int8)
    else:
      q = y.astype(np.float32).astype(_NP[spec.qdtype])
    ldq = (x.cols + 15) // 16 * 16
    out = _strided(q_out, spec.qdtype, [x.b0, x.b1, x.rows, ldq],
                   [x.b1 * x.rows * ldq, x.rows * ldq, ldq, 1], True)
    out[..., :x.cols] = q
    out[..., x.cols:] = np.zeros((), _NP[spec.qdtype])
    return 0

  def aqtb200_quantize(self, x, pre, noise, spec, scale_in, q_out, scale_out,
                       ws, ws_bytes, stream):
    return self._quantize(_deref(x, _lib.View), _deref(pre, _lib.View),
                          _deref(noise, _lib.View),
                          _deref(spec, _lib.QuantSpec), scale_in, q_out,
                          scale_out)

  def aqtb200_quantize_dual_workspace_bytes(self, desc):
    return 1024

  def aqtb200_quantize_dual(self, desc, ws, ws_bytes, stream):
    """Two plain quantizations of the same tensor, one per orientation."""
    d = _deref(desc, _lib.DualDesc)
    x = d.x
    if x.row_stride != 1 or x.rows % 16 or x.cols % 16:
      return self._fail(-2, 'aqtb200_quantize_dual: layout')

    def view(v, transposed):
      if not v.ptr:
        return None
      o = _lib.View()
      o.ptr, o.dtype = v.ptr, v.dtype
      o.b0, o.b1 = x.b0, x.b1
      o.b0_stride, o.b1_stride = v.b0_stride, v.b1_stride
      if transposed:  # rows stay rows, the contraction runs over x's cols
        o.rows, o.cols = x.rows, x.cols
        o.row_stride, o.col_stride = v.row_stride, v.col_stride
      else:           # x's orientation: the contraction runs over x's rows
        o.rows, o.cols = x.cols, x.rows
        o.row_stride, o.col_stride = v.col_stride, v.row_stride
      return o

    rc = self._quantize(view(x, True), view(d.prescale_t, True),
                        view(d.noise_t, True), d.spec_t, None, d.q_t,
                        d.scale_t)
    if rc:
      return rc
    return self._quantize(view(x, False), view(d.prescale_s, False),
                          view(d.noise_s, False), d.spec_s, None, d.q_s,
                          d.scale_s)

  def aqtb200_absmax_scale(self, x, pre, spec, scale_out, ws, ws_bytes,
                           stream):
    return self._quantize(_deref(x, _lib.View), _deref(pre, _lib.View), None,
                          _deref(spec, _lib.QuantSpec), None, None, scale_out)

  def aqtb200_absmax_raw(self, x, per_tensor, amax_out, stream):
    x = _deref(x, _lib.View)
    xv = np.abs(_view_array(x).astype(np.float32))
    n = 1 if per_tensor else x.b0 * x.b1 * x.rows
    a = xv.max(initial=0) if per_tensor else xv.max(axis=3, initial=0).reshape(-1)
    _strided(amax_out, _lib.F32, [n], [1], True)[...] = a
    return 0

  def aqtb200_scale_from_amax(self, amax, n, pre, pre_dtype, spec, scale_out,
                              stream):
    spec = _deref(spec, _lib.QuantSpec)
    T = _NP[spec.compute_dtype]
    S = _NP[spec.scale_dtype]
    a = np.array(_strided(amax, _lib.F32, [n], [1])).astype(T)
    if pre:
      p = np.array(_strided(pre, pre_dtype, [1], [1])).astype(np.float32).astype(T)
      a = np.abs(orc.mul(a, p))
    a = np.where(a == 0, np.ones_like(a), a).astype(T)
    bound = orc.mul(a, np.asarray(spec.clipping_scale, T)) if (
        spec.clipping_scale) else a
    scale = orc.div(bound, np.asarray(spec.quant_bound, T))
    if spec.po2_scale:
      scale = orc.ceil_to_po2(scale)
    _strided(scale_out, spec.scale_dtype, [n], [1], True)[...] = scale.astype(S)
    return 0

  def aqtb200_prescale_amax(self, amax, n, pre, pre_dtype, t_dtype, out,
                            stream):
    T = _NP[t_dtype]
    a = np.array(_strided(amax, _lib.F32, [n], [1])).astype(T)
    p = np.array(_strided(pre, pre_dtype, [1], [1])).astype(np.float32).astype(T)
    _strided(out, _lib.F32, [n], [1], True)[...] = np.abs(
        orc.mul(a, p)).astype(np.float32)
    return 0

  def aqtb200_delayed_scaling_scale(self, history, length, bound, update,
                                    spec, scale_out, stream):
    spec = _deref(spec, _lib.QuantSpec)
    h = _strided(history, _lib.F32, [length], [1])
    b = _strided(bound, _lib.F32, [1], [1], True)
    amax = np.max(np.array(h))
    nb = amax if amax > 0 else b[0]
    nb = np.float32(nb if np.isfinite(amax) else b[0])
    if update:
      b[0] = nb
    with np.errstate(divide='ignore'):
      s = np.asarray(nb, np.float32) / np.float32(spec.quant_bound)
      if spec.po2_scale:
        s = orc.ceil_to_po2(np.asarray(s, np.float32))
    _strided(scale_out, spec.scale_dtype, [1], [1], True)[...] = np.asarray(
        s, np.float32).astype(_NP[spec.scale_dtype])
    return 0

  def aqtb200_delayed_scaling_push(self, history, length, amax, stream):
    h = _strided(history, _lib.F32, [length], [1], True)
    new = np.roll(np.array(h), -1)
    new[0] = _strided(amax, _lib.F32, [1], [1])[0]
    h[...] = new
    return 0

  def aqtb200_requant_amax(self, amax, n, pre, pre_dtype, spec, scale, out,
                           stream):
    spec = _deref(spec, _lib.QuantSpec)
    T = _NP[spec.compute_dtype]
    a = np.array(_strided(amax, _lib.F32, [n], [1])).astype(T)
    if pre:
      p = np.array(_strided(pre, pre_dtype, [1], [1])).astype(np.float32).astype(T)
      a = np.abs(orc.mul(a, p))
    sc = np.array(_strided(scale, spec.scale_dtype, [n], [1]))
    s_inv = orc.reciprocal(sc)
    s_inv = np.where(np.isinf(s_inv.astype(np.float32)), np.ones_like(s_inv),
                     s_inv)
    y = orc.clip(orc.mul(a, s_inv), -spec.clip_bound, spec.clip_bound)
    if spec.kind == _lib.NUM_INT:
      v = np.rint(y.astype(np.float32))
    else:
      v = y.astype(np.float32).astype(_NP[spec.qdtype]).astype(np.float32)
    _strided(out, _lib.F32, [n], [1], True)[...] = np.abs(v)
    return 0

  def aqtb200_quantize_pair(self, x, spec_t, scale_t, pre_t, pre_t_dtype, q_t,
                            spec_s, scale_s, pre_s, pre_s_dtype, q_s, chain,
                            amax, amax_out, stream):
    self.calls.append(('quantize_pair', chain))
    x = _deref(x, _lib.View)
    if amax_out:
      _strided(amax_out, _lib.F32, [1], [1], True)[0] = np.abs(
          _view_array(x).astype(np.float32)).max(initial=0)
    spec_t = _deref(spec_t, _lib.QuantSpec)
    spec_s = _deref(spec_s, _lib.QuantSpec)
    if amax:
      # the scales are outputs: derive them as the separate entry points would
      tmp = (C.c_float * 1)()
      tp = C.addressof(tmp)
      if chain == 1:
        self.aqtb200_scale_from_amax(amax, 1, pre_t, pre_t_dtype, spec_t,
                                     scale_t, None)
        self.aqtb200_requant_amax(amax, 1, pre_t, pre_t_dtype, spec_t, scale_t,
                                  tp, None)
        self.aqtb200_scale_from_amax(tp, 1, None, 0, spec_s, scale_s, None)
      elif chain == 2:
        self.aqtb200_scale_from_amax(amax, 1, pre_s, pre_s_dtype, spec_s,
                                     scale_s, None)
        self.aqtb200_requant_amax(amax, 1, pre_s, pre_s_dtype, spec_s, scale_s,
                                  tp, None)
        self.aqtb200_scale_from_amax(tp, 1, None, 0, spec_t, scale_t, None)
      else:
        self.aqtb200_scale_from_amax(amax, 1, pre_t, pre_t_dtype, spec_t,
                                     scale_t, None)
        self.aqtb200_scale_from_amax(amax, 1, pre_s, pre_s_dtype, spec_s,
                                     scale_s, None)
    if x.dtype != _lib.BF16 or x.row_stride != 1 or x.rows % 16 or x.cols % 16:
      return self._fail(-2, 'quantize_pair: unsupported view')

    def scalar_view(ptr, code):
      if not ptr:
        return None
      v = _lib.View()
      v.ptr, v.dtype = ptr, code
      return v

    def view(ptr, code, rows, cols, rs, cs):
      v = _lib.View()
      v.ptr, v.dtype = ptr, code
      v.b0, v.b1, v.rows, v.cols = x.b0, x.b1, rows, cols
      v.b0_stride = x.b1 * rows * cols
      v.b1_stride = rows * cols
      v.row_stride, v.col_stride = rs, cs
      return v

    # x transposed: rows = x.cols (strided), cols = x.rows (contiguous)
    x_s = _lib.View()
    x_s.ptr, x_s.dtype = x.ptr, x.dtype
    x_s.b0, x_s.b1, x_s.rows, x_s.cols = x.b0, x.b1, x.cols, x.rows
    x_s.b0_stride, x_s.b1_stride = x.b0_stride, x.b1_stride
    x_s.row_stride, x_s.col_stride = x.col_stride, 1
    T = _lib.BF16

    def as_float(spec):
      # the chained quantization sees the first one's values as bf16 numbers
      sp = _lib.QuantSpec()
      for f, _ in _lib.QuantSpec._fields_:
        setattr(sp, f, getattr(spec, f))
      sp.compute_dtype = T
      return sp

    if chain == 1:
      rc = self._quantize(x, scalar_view(pre_t, pre_t_dtype), None, spec_t,
                          scale_t, q_t, None)
      src = view(q_t, spec_t.qdtype, x.cols, x.rows, 1, x.cols)
      return rc or self._quantize(src, None, None, as_float(spec_s), scale_s,
                                  q_s, None)
    if chain == 2:
      rc = self._quantize(x_s, scalar_view(pre_s, pre_s_dtype), None, spec_s,
                          scale_s, q_s, None)
      src = view(q_s, spec_s.qdtype, x.rows, x.cols, 1, x.rows)
      return rc or self._quantize(src, None, None, as_float(spec_t), scale_t,
                                  q_t, None)
    rc = self._quantize(x, scalar_view(pre_t, pre_t_dtype), None, spec_t,
                        scale_t, q_t, None)
    return rc or self._quantize(x_s, scalar_view(pre_s, pre_s_dtype), None,
                                spec_s, scale_s, q_s, None)

  # -- gemm
  def _gemm(self, g, acc_in=None):
    ext = [g.b0, g.b1]
    ints = g.a_dtype == _lib.S8
    if acc_in is not None:
      acc = np.array(_strided(acc_in, _lib.S32 if ints else _lib.F32,
                              ext + [g.m, g.n],
                              [g.b1 * g.m * g.n, g.m * g.n, g.n, 1]))
    else:
      a = _strided(g.a, g.a_dtype, ext + [g.m, g.k],
                   [g.a_b0_stride, g.a_b1_stride, g.lda, 1])
      b = _strided(g.b, g.b_dtype, ext + [g.n, g.k],
                   [g.b_b0_stride, g.b_b1_stride, g.ldb, 1])
      dims = (((3,), (3,)), ((0, 1), (0, 1)))
      acc = orc.dot_general(np.array(a), np.array(b), dims,
                            preferred_element_type=orc.int32 if ints else
                            orc.float32)
    if g.acc_out and acc_in is None:
      _strided(g.acc_out, _lib.S32 if ints else _lib.F32, ext + [g.m, g.n],
               [g.b1 * g.m * g.n, g.m * g.n, g.n, 1], True)[...] = acc
    D = _NP[g.dequant_dtype]
    r = acc.astype(np.float32).astype(D)
    sa = sb = None
    if g.a_scale:
      sa = np.array(_strided(g.a_scale, g.a_scale_dtype, ext + [g.m, 1],
                             [g.a_scale_b0_stride, g.a_scale_b1_stride,
                              g.a_scale_m_stride, 0]))
    if g.b_scale:
      sb = np.array(_strided(g.b_scale, g.b_scale_dtype, ext + [1, g.n],
                             [g.b_scale_b0_stride, g.b_scale_b1_stride, 0,
                              g.b_scale_n_stride]))
    for s in ([sb, sa] if g.b_scale_first else [sa, sb]):
      if s is not None:
        r = orc.mul(r, s)
    r = r.astype(D).astype(_NP[g.out_dtype])
    if not g.out:
      return 0
    if g.amax_out:
      cell = _strided(g.amax_out, _lib.F32, [1], [1], True)
      cell[0] = max(float(cell[0]), float(np.abs(r.astype(np.float32)).max(
          initial=0.0)))
    _strided(g.out, g.out_dtype, ext + [g.m, g.n],
             [g.out_b0_stride, g.out_b1_stride, g.out_m_stride,
              g.out_n_stride], True)[...] = r
    return 0

  def aqtb200_gemm_dequant(self, desc, status, stream):
    return self._gemm(_deref(desc, _lib.GemmDesc))

  # -- the composite, mirroring aqt_b200/csrc/api.cu
  def aqtb200_dot_general_raw_workspace_bytes(self, desc):
    return 1024

  def aqtb200_dot_general_raw_dequant(self, desc, stream):
    return self.aqtb200_dot_general_raw(desc, None, 0, None, stream,
                                        dequant_only=True)

  def aqtb200_dot_general_raw(self, desc, ws, ws_bytes, status, stream,
                              dequant_only=False):
    d = _deref(desc, _lib.DgRawDesc)
    self.calls.append('dg_raw_dequant' if dequant_only else 'dg_raw')
    sides = []
    for (v, pre, noise, spec, sin, isq, qo, so) in (
        (d.lhs, d.lhs_prescale, d.lhs_noise, d.lhs_spec, d.lhs_scale_in,
         d.lhs_is_quantized, d.lhs_q, d.lhs_scale),
        (d.rhs, d.rhs_prescale, d.rhs_noise, d.rhs_spec, d.rhs_scale_in,
         d.rhs_is_quantized, d.rhs_q, d.rhs_scale)):
      if isq:
        if not (v.col_stride == 1 or v.cols <= 1):
          return self._fail(-2, 'pre-quantized operand not k-contiguous')
        side = dict(q=v.ptr, dt=v.dtype, ld=v.row_stride, b1=v.b1_stride,
                    b0=v.b0_stride, scale=sin)
      else:
        rc = 0 if dequant_only else self._quantize(v, pre, noise, spec, sin,
                                                   qo, so)
        if rc:
          return rc
        ld = (v.cols + 15) // 16 * 16
        side = dict(q=qo, dt=spec.qdtype, ld=ld, b1=v.rows * ld,
                    b0=v.b1 * v.rows * ld, scale=so or sin)
      side['sdt'] = spec.scale_dtype
      side['ss'] = (0, 0, 0) if spec.per_tensor else (v.b1 * v.rows, v.rows, 1)
      side['rows'] = v.rows
      sides.append(side)
    L, R = sides
    A, B = (R, L) if d.swap_ab else (L, R)
    g = _lib.GemmDesc()
    g.b0, g.b1, g.k = d.lhs.b0, d.lhs.b1, d.lhs.cols
    g.m, g.n = A['rows'], B['rows']
    g.a, g.a_b0_stride, g.a_b1_stride, g.lda, g.a_dtype = (
        A['q'], A['b0'], A['b1'], A['ld'], A['dt'])
    g.b, g.b_b0_stride, g.b_b1_stride, g.ldb, g.b_dtype = (
        B['q'], B['b0'], B['b1'], B['ld'], B['dt'])
    g.a_scale, g.a_scale_dtype = A['scale'], A['sdt']
    g.a_scale_b0_stride, g.a_scale_b1_stride, g.a_scale_m_stride = A['ss']
    g.b_scale, g.b_scale_dtype = B['scale'], B['sdt']
    g.b_scale_b0_stride, g.b_scale_b1_stride, g.b_scale_n_stride = B['ss']
    g.b_scale_first = 1 if d.swap_ab else 0
    g.dequant_dtype, g.out, g.out_dtype = d.dequant_dtype, d.out, d.out_dtype
    g.out_b0_stride, g.out_b1_stride = d.out_b0_stride, d.out_b1_stride
    g.out_m_stride = d.out_n_stride if d.swap_ab else d.out_m_stride
    g.out_n_stride = d.out_m_stride if d.swap_ab else d.out_n_stride
    g.acc_out = d.acc_out
    g.amax_out = d.amax_out
    return self._gemm(g, acc_in=d.acc_out if dequant_only else None)

  # -- dequantize
  def aqtb200_dequantize(self, q, scale, d_dtype, out, stream):
    q = _deref(q, _lib.View)
    s = _deref(scale, _lib.View)
    D = _NP[d_dtype]
    qv = _view_array(q)
    r = qv.astype(np.float32).astype(D)
    if s is not None and s.ptr:
      r = orc.mul(r, np.array(_view_array(s))).astype(D)
    ext = [q.b0, q.b1, q.rows, q.cols]
    _strided(out, d_dtype, ext, [q.b1 * q.rows * q.cols, q.rows * q.cols,
                                 q.cols, 1], True)[...] = r
    return 0


def install(monkeypatch):
  """Routes aqt_b200._lib.load to a FakeLib and lets the engine take CPU tensors."""
  from aqt_b200 import engine
  fake = FakeLib()
  monkeypatch.setattr(_lib, 'load', lambda: fake)
  monkeypatch.setattr(engine, '_stream', lambda: 0)
  monkeypatch.setattr(engine, '_on_device', lambda *t: True)
  return fake
