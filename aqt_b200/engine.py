"""Host-side planner: turns AQT config objects + torch CUDA tensors into calls
of the C ABI (include/aqt_b200.h).

It owns no arithmetic. Its jobs are (1) to check that a configuration is one
the sm_100a kernels implement and raise NotImplementedError otherwise, (2) to
normalise arbitrary dimension_numbers into the strided [b0][b1][rows][cols]
views the kernels take, without copying whenever the strides allow it, and
(3) to allocate outputs / workspaces from torch's caching allocator and pass
raw pointers and the current stream down.
"""

from __future__ import annotations

import ctypes as C
import functools
from typing import Any, Sequence

import numpy as np
import torch

from aqt_b200 import _lib
from aqt_b200.v2 import utils

_TORCH_CODE = {
    torch.float32: _lib.F32, torch.bfloat16: _lib.BF16, torch.int8: _lib.S8,
    torch.float8_e4m3fn: _lib.E4M3, torch.float8_e5m2: _lib.E5M2,
    torch.int32: _lib.S32,
}
_CODE_TORCH = {v: k for k, v in _TORCH_CODE.items()}
_FLOAT_CODES = (_lib.F32, _lib.BF16)


def _code(dtype) -> int:
  if isinstance(dtype, torch.dtype):
    if dtype == torch.float16:
      raise NotImplementedError(
          'float16 operands: the reference admits them '
          '(aqt_dot_general.py:986-987), the sm_100a kernels compute in '
          'float32 and bfloat16 only; cast the operands')
    if dtype not in _TORCH_CODE:
      raise NotImplementedError(f'dtype {dtype} is not handled on the device')
    return _TORCH_CODE[dtype]
  d = utils.as_dtype(dtype)
  if d.code < 0:
    raise NotImplementedError(f'dtype {d} is not handled on the device')
  return d.code


def _stream() -> int:
  return torch.cuda.current_stream().cuda_stream


def _on_device(*tensors) -> bool:
  """True when every tensor lives in GPU memory (there is no CPU path)."""
  return all(t.is_cuda for t in tensors)


# ---------------------------------------------------------------------------
# Recording a step once and replaying it (see TracedStep below). While a tape
# is open every call into the shared library, and every buffer handed to one,
# is noted on it.


class _Tape:

  def __init__(self):
    # in issue order: (library entry point, its arguments), whose return code
    # is checked on replay, or (host action, None)
    self.ops = []
    self.keep = []   # buffers the recorded calls point into


_tape = None


def _call(fn, *args):
  """Calls one entry point of the shared library; notes it on an open tape."""
  rc = fn(*args)
  if _tape is not None:
    _tape.ops.append((fn, args))
  return rc


def tape_op(op):
  """Runs a host-side action that belongs to the step (a collective, a stream
  wait) and notes it on an open tape, so that a replay repeats it in place."""
  ret = op()
  if _tape is not None:
    _tape.ops.append((op, None))
  return ret


def _empty(shape, dtype, device):
  """Uninitialised device buffer; while a tape is open it is held for the
  tape's lifetime, because the recorded calls carry its address."""
  t = torch.empty(shape, dtype=dtype, device=device)
  if _tape is not None:
    _tape.keep.append(t)
  return t


_status = {}


def _status_buf(device):
  key = str(device)
  if key not in _status:
    _status[key] = torch.zeros(4, dtype=torch.int32, device=device)
  return _status[key]


def check_status():
  """Raises if a kernel reported a bounded wait that ran out (syncs)."""
  for buf in _status.values():
    code = int(buf[0].item())
    if code:
      buf.zero_()
      raise _lib.AqtB200Error(
          f'GEMM kernel gave up waiting on a barrier (role {code})')


_status_host = {}


def poll_status(device):
  """Non-blocking look at the status word: every raw dot starts with one.

  The word travels to pinned host memory by an asynchronous copy; a call
  examines the copy the previous call started (if it has landed) and starts
  the next one. A bounded wait that ran out therefore surfaces as an exception
  one or two dots later, without a synchronisation anywhere -- instead of a
  partially written result going unnoticed until someone calls
  check_status(). Skipped while the stream is being captured into a graph
  (replays are checked by the caller's own check_status())."""
  if device.type != 'cuda' or torch.cuda.is_current_stream_capturing():
    return
  key = str(device)
  slot = _status_host.get(key)
  if slot is None:
    slot = _status_host[key] = {
        'host': torch.zeros(4, dtype=torch.int32).pin_memory(),
        'event': None}
  ev = slot['event']
  if ev is not None:
    if not ev.query():
      return
    code = int(slot['host'][0])
    if code:
      _status_buf(device).zero_()
      slot['host'].zero_()
      slot['event'] = None
      raise _lib.AqtB200Error(
          f'GEMM kernel gave up waiting on a barrier (role {code}); results '
          'since the last check are incomplete')
  slot['host'].copy_(_status_buf(device), non_blocking=True)
  ev = torch.cuda.Event()
  ev.record()
  slot['event'] = ev


def set_gemm_impl(name: str):
  """'tcgen05' (default), 'simt' (cross-check kernel), 'cta1', 'cta2', 'wide'."""
  code = {'tcgen05': 0, 'simt': 1, 'cta1': 2, 'cta2': 3, 'wide': 4}[name]
  _lib.check(_call(_lib.load().aqtb200_set_gemm_impl, code), 'set_gemm_impl')


def set_gemm_sm_budget(max_sms: int):
  """Caps the SMs the persistent GEMM grids take (0 = all)."""
  _lib.check(_call(_lib.load().aqtb200_set_gemm_sm_budget, int(max_sms)),
             'set_gemm_sm_budget')


def sm_count() -> int:
  n = C.c_int(0)
  _lib.check(_lib.load().aqtb200_device_sm_count(C.byref(n)), 'sm_count')
  return n.value


# ---------------------------------------------------------------------------
# stride bookkeeping


def _merge(extents: Sequence[int], strides: Sequence[Sequence[int]],
           max_dims: int):
  """Merges consecutive index positions into at most max_dims strided dims.

  extents[p] is the extent of position p; strides[t][p] its stride in tensor t.
  Two neighbours merge only if they do so in every tensor. Returns a list of
  (extent, [stride per tensor]) or None when more than max_dims dims remain.
  """
  nt = len(strides)
  dims = []
  for p, e in enumerate(extents):
    if e == 1:
      continue
    s = [strides[t][p] for t in range(nt)]
    if dims and all(dims[-1][1][t] == s[t] * e for t in range(nt)):
      dims[-1] = (dims[-1][0] * e, s)
    else:
      dims.append((e, s))
  if len(dims) > max_dims:
    return None
  return dims


class _Unmergeable(Exception):
  pass


_SCOPES = {}


def _scope_bytes(name: str) -> bytes:
  """NUL-terminated name for a descriptor, kept alive for the process."""
  if name not in _SCOPES:
    _SCOPES[name] = name.encode()
  return _SCOPES[name]


def _view(ptr, code, b, rows, cols, bs, rs, cs) -> _lib.View:
  v = _lib.View()
  v.ptr = ptr
  v.dtype = code
  v.b0, v.b1 = b[0], b[1]
  v.rows, v.cols = rows, cols
  v.b0_stride, v.b1_stride = bs[0], bs[1]
  v.row_stride, v.col_stride = rs, cs
  return v


# ---------------------------------------------------------------------------
# config -> spec


def _calibration_kwargs(quantizer):
  cal = quantizer.calibration
  kw = {}
  if isinstance(cal, functools.partial):
    kw = dict(cal.keywords)
    cal = cal.func
  name = None if cal is None else cal.__name__
  if name == 'DelayedScalingCalibration':
    extra = set(kw) - {'dtype', 'po2_scale', 'amax_history_length', 'stats'}
    if extra:
      raise NotImplementedError(
          f'DelayedScalingCalibration options {sorted(extra)}')
    return kw
  if name != 'AbsMaxCalibration':
    raise NotImplementedError(
        f'calibration {cal} is outside the sm_100a hot path '
        '(AbsMaxCalibration and DelayedScalingCalibration)')
  extra = set(kw) - {'dtype', 'clipping_scale', 'po2_scale'}
  if extra:
    raise NotImplementedError(f'AbsMaxCalibration options {sorted(extra)}')
  return kw


def _delayed(quantizer):
  """The quantizer's DelayedScalingCalibration instance, or None."""
  cal = getattr(quantizer, '_calibrator', None)
  if type(cal).__name__ == 'DelayedScalingCalibration':
    return cal
  return None


def _round_to_dtype(value: float, code: int) -> float:
  t = torch.tensor(value, dtype=torch.float64).to(_CODE_TORCH[code])
  return float(t.to(torch.float32))


def _numerics_fields(numerics):
  """(kind, qdtype code, quant_bound, clip_bound) of a numerics object."""
  name = type(numerics).__name__
  if name == 'IntSymmetric':
    if not (numerics.preserve_zero and numerics.clip and numerics.round):
      raise NotImplementedError(
          'IntSymmetric needs preserve_zero, clip and round on the sm_100a '
          'path')
    if not 2 <= numerics.bits <= 8:
      raise NotImplementedError(f'IntSymmetric bits={numerics.bits}')
    dt = numerics.get_dtype()
    if dt is None or utils.as_dtype(dt) not in (utils.int8, utils.int4):
      raise NotImplementedError(
          f'IntSymmetric dtype={dt}: the kernels store int8 containers')
    return (_lib.NUM_INT, _lib.S8, float(numerics.get_quant_bound()),
            float(numerics._get_fwd_clip_bound()))  # pylint: disable=protected-access
  if name == 'Fp8Numerics':
    numerics.check()
    bound = float(numerics.get_quant_bound())
    return (_lib.NUM_FP8, _code(numerics.get_dtype()), bound, bound)
  raise NotImplementedError(f'numerics {name} is outside the sm_100a hot path')


def _make_spec(quantizer, compute_code: int, contraction_axes_ok: bool):
  """aqtb200_quant_spec for one operand, or None for NoNumerics."""
  numerics = quantizer.numerics
  if type(numerics).__name__ == 'NoNumerics':
    return None
  kind, qcode, qb, cb = _numerics_fields(numerics)
  kw = _calibration_kwargs(quantizer)
  csa = quantizer.calib_shared_axes
  if csa not in (None, 'per_tensor') and not contraction_axes_ok:
    raise NotImplementedError(
        f'calib_shared_axes={csa}: only the contraction axes or "per_tensor"')
  scale_dtype = kw.get('dtype', quantizer.scale_dtype)
  spec = _lib.QuantSpec()
  spec.kind = kind
  spec.qdtype = qcode
  spec.quant_bound = qb
  spec.clip_bound = cb
  # delayed scaling keeps one bound per tensor whatever the axes
  # (flax/delayed_scaling_calibration.py:66-75)
  spec.per_tensor = 1 if csa == 'per_tensor' or _delayed(quantizer) else 0
  spec.compute_dtype = compute_code
  spec.scale_dtype = compute_code if scale_dtype is None else _code(scale_dtype)
  if spec.scale_dtype not in _FLOAT_CODES:
    raise NotImplementedError(f'scale dtype {scale_dtype}')
  spec.po2_scale = 1 if kw.get('po2_scale', False) else 0
  cs = kw.get('clipping_scale')
  spec.clipping_scale = _round_to_dtype(cs, compute_code) if cs else 0.0
  return spec


def _noise_for(quantizer, shape, device):
  fn = getattr(quantizer.numerics, 'noise_fn', None)
  if not fn:
    return None
  assert quantizer.context.key is not None, (
      'noise_fn is set, requestic stochastic rounding, but RNG was not '
      'passed in Context.key')
  noise = fn(tuple(shape), quantizer.context.key)
  if not isinstance(noise, torch.Tensor):
    noise = torch.as_tensor(np.asarray(noise))
  noise = noise.to(device=device, dtype=torch.float32)
  return noise.expand(tuple(shape))


# ---------------------------------------------------------------------------
# one raw quantized dot


def _prod(v):
  return int(np.prod(list(v), dtype=np.int64)) if len(v) else 1


def _check_raw_supported(raw):
  from aqt_b200.v2 import aqt_dot_general as adg
  q = raw.dg_quantizer
  if not isinstance(q, adg.DefaultDotGeneralQuantizer):
    raise NotImplementedError(
        f'dg_quantizer {type(q).__name__}: DefaultDotGeneralQuantizer only')
  if q.lhs_mid_alpha is not None or q.rhs_mid_alpha is not None:
    raise NotImplementedError('mid-scale quantization')
  if raw.local_aqt is not None:
    raise NotImplementedError('local AQT (contraction-axis sharding)')
  for side, t in (('lhs', raw.lhs), ('rhs', raw.rhs)):
    if t.dequant_mode != adg.DequantMode.OUTPUT:
      raise NotImplementedError(
          f'{side}.dequant_mode={t.dequant_mode}: the fused epilogue '
          'implements DequantMode.OUTPUT')
    if t.calibration_mode != adg.CalibrationMode.CONTRACTING_AXIS:
      raise NotImplementedError(
          f'{side}.calibration_mode={t.calibration_mode}: CONTRACTING_AXIS '
          'only')
  if raw.dot_general is not adg.lax_dot_general:
    raise NotImplementedError(
        'a custom DotGeneralRaw.dot_general cannot be injected: the '
        'contraction is fused with dequantization')
  return q


class _Operand:
  """One operand of the raw dot with its axis groups."""

  def __init__(self, t, ba, ra, ca):
    self.t = t
    self.ba, self.ra, self.ca = list(ba), list(ra), list(ca)

  def strides_of(self, axes, tensor=None):
    t = self.t if tensor is None else tensor
    return [t.stride(a) for a in axes]

  def extents_of(self, axes):
    return [self.t.shape[a] for a in axes]


def _as_scale_compact(scale, op: _Operand, per_tensor: bool, code: int):
  """A caller-supplied scale (operand rank, shared axes 1) -> compact buffer."""
  want = _CODE_TORCH[code]
  if per_tensor:
    return scale.reshape(1).to(want).contiguous()
  s = scale.permute(*(op.ba + op.ra + op.ca))
  return s.reshape(-1).to(want).contiguous()


def _logical_scale(compact, op: _Operand, per_tensor: bool):
  """Compact [batch..., rows...] scale -> operand-rank tensor, shared axes 1."""
  nd = op.t.ndim
  if per_tensor:
    return compact.view([1] * nd)
  shape = op.extents_of(op.ba) + op.extents_of(op.ra) + [1] * len(op.ca)
  order = op.ba + op.ra + op.ca
  inv = [order.index(i) for i in range(nd)]
  return compact.view(shape).permute(*inv)


def _strided_logical(buf, b_ext, r_ext, k_ext):
  """Views a [B, rows, ld] buffer as a tensor of shape b_ext + r_ext + k_ext.

  The contraction dims subdivide the first prod(k_ext) bytes of each row, the
  kept dims subdivide `rows`, the batch dims subdivide B; no data moves.
  """
  def sub(extents, innermost):
    strides, st = [], innermost
    for e in reversed(list(extents)):
      strides.append(st)
      st *= e
    return list(reversed(strides))

  strides = (sub(b_ext, buf.stride(0)) + sub(r_ext, buf.stride(1))
             + sub(k_ext, 1))
  return buf.as_strided(list(b_ext) + list(r_ext) + list(k_ext), strides,
                        buf.storage_offset())


def _logical_q(buf, op: _Operand, k: int):
  """[B, rows, ldk] byte buffer -> tensor with the operand's logical shape."""
  del k
  order = op.ba + op.ra + op.ca
  inv = [order.index(i) for i in range(op.t.ndim)]
  t = _strided_logical(buf, op.extents_of(op.ba), op.extents_of(op.ra),
                       op.extents_of(op.ca))
  return t.permute(*inv)


def _copy_struct(d):
  return type(d).from_buffer_copy(d)


class DeferredDequant:
  """Accumulators of a raw dot whose dequantization has been postponed.

  `acc` is the raw int32 / f32 accumulator tensor, contiguous
  [batch][tile rows][tile columns] (sum it across ranks when the contraction
  index is sharded); finish() applies the dequantizing epilogue once and
  returns the output. finish_rows() does so for a band of accumulator rows
  that sit in a buffer of their own (one rank's share after a
  reduce-scatter).
  """

  def __init__(self, desc, acc, out, keep):
    self._desc, self.acc, self._out, self._keep = desc, acc, out, keep

  @property
  def acc_mn(self):
    """The accumulators as [batch, lhs rows, rhs rows], whichever operand the
    GEMM put on its tile rows."""
    return self.acc.transpose(1, 2) if self._desc.swap_ab else self.acc

  def finish(self):
    desc = _copy_struct(self._desc)
    desc.out = self._out.data_ptr()
    rc = _call(_lib.load().aqtb200_dot_general_raw_dequant, C.byref(desc),
               _stream())
    _lib.check(rc, 'aqtb200_dot_general_raw_dequant')
    return self._out

  def finish_rows(self, start: int, count: int, acc_band):
    """Dequantizes accumulator rows [start, start + count), read from
    `acc_band` ([count][columns], contiguous), into their place in the output."""
    desc = _copy_struct(self._desc)
    assert desc.lhs.b0 * desc.lhs.b1 == 1, 'finish_rows: unbatched dots only'
    swap = bool(desc.swap_ab)
    side = desc.rhs if swap else desc.lhs
    spec = desc.rhs_spec if swap else desc.lhs_spec
    assert 0 <= start and start + count <= side.rows
    side.rows = count
    stride = desc.out_n_stride if swap else desc.out_m_stride
    desc.out = self._out.data_ptr() + start * stride * self._out.element_size()
    desc.acc_out = acc_band.data_ptr()
    if not spec.per_tensor:
      off = start * (2 if spec.scale_dtype == _lib.BF16 else 4)
      for name in (('rhs_scale', 'rhs_scale_in') if swap else
                   ('lhs_scale', 'lhs_scale_in')):
        ptr = getattr(desc, name)
        if ptr:
          setattr(desc, name, ptr + off)
    rc = _call(_lib.load().aqtb200_dot_general_raw_dequant, C.byref(desc),
               _stream())
    _lib.check(rc, 'aqtb200_dot_general_raw_dequant')
    return self._out


  def exchange_rows(self, start: int, count: int, rank: int, acc_ptrs,
                    out_ptrs, max_sms: int = 0):
    """The fused exchange for accumulator rows [start, start + count): sums
    the band over the ranks (acc_ptrs[r]: address of rank r's band, peer
    mappings for the others), dequantizes once and writes it to every rank
    (out_ptrs[r]: address of the band's place in rank r's output)."""
    desc = _copy_struct(self._desc)
    assert desc.lhs.b0 * desc.lhs.b1 == 1, 'exchange_rows: unbatched dots only'
    swap = bool(desc.swap_ab)
    side = desc.rhs if swap else desc.lhs
    spec = desc.rhs_spec if swap else desc.lhs_spec
    assert 0 <= start and start + count <= side.rows
    side.rows = count
    if not spec.per_tensor:
      off = start * (2 if spec.scale_dtype == _lib.BF16 else 4)
      for name in (('rhs_scale', 'rhs_scale_in') if swap else
                   ('lhs_scale', 'lhs_scale_in')):
        ptr = getattr(desc, name)
        if ptr:
          setattr(desc, name, ptr + off)
    x = _lib.ExchangeDesc()
    x.world, x.rank, x.max_sms = len(acc_ptrs), rank, max_sms
    for r, (a, o) in enumerate(zip(acc_ptrs, out_ptrs)):
      x.acc[r], x.out[r] = a, o
    desc.out = out_ptrs[rank]
    desc.acc_out = acc_ptrs[rank]
    status = _status_buf(self._out.device)
    rc = _call(_lib.load().aqtb200_dot_general_raw_exchange, C.byref(desc),
               C.byref(x), status.data_ptr(), _stream())
    _lib.check(rc, 'aqtb200_dot_general_raw_exchange')

  def band_stride_bytes(self):
    """(accumulator bytes, output bytes) between consecutive accumulator rows."""
    desc = self._desc
    swap = bool(desc.swap_ab)
    n = desc.lhs.rows if swap else desc.rhs.rows
    stride = desc.out_n_stride if swap else desc.out_m_stride
    return 4 * n, stride * self._out.element_size()


def dg_raw(raw, lhs, rhs, lhs_qt, rhs_qt, dimension_numbers,
           out_transpose_axes=None, want_acc=False, defer_dequant=False,
           internal_qt=False, out=None, amax_out=None, _regrouped=False,
           _noise=None, acc_buf=None):
  """DotGeneralRaw.__call__ on the device (aqt_dot_general.py:757-840).

  Returns (out, DotGeneralRes[, acc]). `out` is laid out as
  transpose(out, out_transpose_axes) would be, written by the epilogue.
  internal_qt: the full QTensors passed in were made by this module from the
  same operands (prequantize_for_training / cotangent_pair), so gradients
  still flow to the operands as if they had been quantized here.
  out: optional preallocated result (any strides, e.g. a slice of a larger
  tensor) of the transposed result's shape and the result dtype.
  amax_out: optional one-element f32 device tensor, zeroed by the caller, that
  receives max |out| from the GEMM epilogue (atomic max).
  acc_buf: optional preallocated contiguous int32 / f32 tensor the raw
  accumulators are written to (e.g. memory other ranks can read).
  """
  from aqt_b200.v2 import aqt_dot_general as adg
  from aqt_b200.v2 import aqt_tensor
  q = _check_raw_supported(raw)
  (lca, rca), (lba, rba) = dimension_numbers
  lca, rca, lba, rba = list(lca), list(rca), list(lba), list(rba)

  # _maybe_use_fwd_quant (aqt_dot_general.py:675-729)
  prescale = None  # fwd scale of the other operand, in the rhs operand's rank
  rhs_float = rhs
  rhs_compute_dtype = None
  if isinstance(rhs, adg.MultiTensor):
    if raw.rhs.use_fwd_quant:
      n_scales = len(rhs.qx.scale) if rhs.qx.scale is not None else -1
      assert n_scales == 1, (
          f'Found use_fwd_quant is True in bwd. It is supported only if there '
          f'is exactly one scale in a good shape.\nscale_count={n_scales}')
      if rhs.qx.bias:
        raise NotImplementedError(
            'Quantization biases are not supported in forward quantization.')
      prescale = rhs.qx.scale[0]
      rhs_float = rhs.qx.qvalue
      rhs_compute_dtype = rhs.qx.dequant_dtype
    else:
      rhs_float = rhs.x
  assert isinstance(lhs, torch.Tensor) and isinstance(rhs_float, torch.Tensor)
  if not _on_device(lhs, rhs_float):
    raise _lib.AqtB200Error('operands must be CUDA tensors (no CPU path)')

  lra = utils.get_remaining_axes(lhs.ndim, lca, lba)
  rra = utils.get_remaining_axes(rhs_float.ndim, rca, rba)
  L = _Operand(lhs, lba, lra, lca)
  R = _Operand(rhs_float, rba, rra, rca)
  t_code_l = _code(lhs.dtype)
  t_code_r = _code(rhs_compute_dtype) if rhs_compute_dtype is not None else (
      _code(rhs_float.dtype))
  if t_code_l not in _FLOAT_CODES or t_code_r not in _FLOAT_CODES:
    raise NotImplementedError(
        f'operand dtypes {lhs.dtype}, {rhs_float.dtype}: f32 / bf16 only')
  d_code = _lib.F32 if _lib.F32 in (t_code_l, t_code_r) else _lib.BF16

  lhs_spec = _make_spec(q.lhs, t_code_l,
                        sorted(q.lhs.calib_shared_axes or []) == sorted(lca)
                        if q.lhs.calib_shared_axes not in (None, 'per_tensor')
                        else True)
  rhs_spec = _make_spec(q.rhs, t_code_r,
                        sorted(q.rhs.calib_shared_axes or []) == sorted(rca)
                        if q.rhs.calib_shared_axes not in (None, 'per_tensor')
                        else True)
  if lhs_spec is None and rhs_spec is None:
    return _dg_raw_unquantized(raw, lhs, rhs_float, lhs_qt, rhs_qt,
                               dimension_numbers, out_transpose_axes)
  if lhs_spec is None or rhs_spec is None:
    raise NotImplementedError(
        'one quantized and one unquantized operand: the tensor-core path '
        'needs both operands in int8 or both in fp8')
  ints = (lhs_spec.kind == _lib.NUM_INT, rhs_spec.kind == _lib.NUM_INT)
  if ints[0] != ints[1]:
    raise NotImplementedError('mixing int and fp8 operands in one dot')
  want_accum = utils.int32 if ints[0] else utils.float32
  if raw.dg_accumulator_dtype is not None and (
      utils.as_dtype(raw.dg_accumulator_dtype) != want_accum):
    raise NotImplementedError(
        f'dg_accumulator_dtype={raw.dg_accumulator_dtype}: the tensor cores '
        f'accumulate {want_accum} for these operands')

  # caller-supplied QTensors (aqt_dot_general.py:623-653)
  def split_qt(qt):
    if qt is None:
      return None, None
    if qt.bias or qt.sparsity_mask is not None or qt.tiling_state is not None:
      raise NotImplementedError('bias / sparsity / tiling in a QTensor')
    assert len(qt.scale) == 1, 'exactly one scale per QTensor on this path'
    return (qt.qvalue if qt.is_full() else None), qt.scale[0]

  lhs_qv, lhs_sin = split_qt(lhs_qt)
  rhs_qv, rhs_sin = split_qt(rhs_qt)

  # Delayed scaling: the scale comes from the calibrator's history; max |x|
  # (after the cotangent's prescale, which must then be one value) goes into
  # the history beside the quantization, not before it.
  def delayed_scale(quantizer, x, pre, t_code):
    cal = _delayed(quantizer)
    if cal is None:
      return None

    def amax_fn():
      amax = absmax_raw(x)
      if pre is not None:
        if pre.numel() != 1:
          raise NotImplementedError(
              'delayed scaling of a cotangent that carries a per-channel '
              'forward scale; set use_fwd_quant=False or per-tensor scales')
        amax = prescale_amax(amax, pre, t_code)
      return amax

    return cal.device_scale(x, quantizer.numerics, quantizer.context,
                            amax_fn=amax_fn, compute_dtype=_CODE_TORCH[t_code])

  if lhs_qv is None and lhs_sin is None:
    lhs_sin = delayed_scale(q.lhs, lhs, prescale, t_code_l)
  if rhs_qv is None and rhs_sin is None:
    rhs_sin = delayed_scale(q.rhs, rhs_float, None, t_code_r)

  if _noise is not None:  # drawn by the caller in its own axis order
    noise_l, noise_r = _noise
  else:
    noise_l = None if lhs_qv is not None else _noise_for(q.lhs, lhs.shape,
                                                         lhs.device)
    noise_r = None if rhs_qv is not None else _noise_for(
        q.rhs, rhs_float.shape, lhs.device)
  if noise_l is not None and lhs_spec.kind != _lib.NUM_INT:
    raise NotImplementedError('noise_fn with fp8 numerics')

  if lhs_qv is not None:
    L = _Operand(lhs_qv, lba, lra, lca)
  if rhs_qv is not None:
    R = _Operand(rhs_qv, rba, rra, rca)

  # ---- output tensor, laid out as the transposed result
  nb, nm, nn = len(lba), len(lra), len(rra)
  raw_shape = L.extents_of(lba) + L.extents_of(lra) + R.extents_of(rra)
  perm = list(out_transpose_axes) if out_transpose_axes is not None else list(
      range(len(raw_shape)))
  out_dtype = _CODE_TORCH[d_code]
  out_shape = [raw_shape[p] for p in perm]
  if out is not None:
    assert list(out.shape) == out_shape and out.dtype == out_dtype, (
        f'out must be {out_shape} {out_dtype}, got {list(out.shape)} {out.dtype}')
    out_t = out
  else:
    out_t = _empty(out_shape, out_dtype, lhs.device)
  raw_strides = [0] * len(raw_shape)
  for i, p in enumerate(perm):
    raw_strides[p] = out_t.stride(i)
  out_b = raw_strides[:nb]
  out_m = raw_strides[nb:nb + nm]
  out_n = raw_strides[nb + nm:]

  # prescale strides along the lhs operand's batch and contraction axes
  pre_t = None
  if prescale is not None:
    # scale has the rhs operand's rank; its axes rba/rra map to lhs lba/lca.
    if prescale.ndim < R.t.ndim:
      prescale = prescale.reshape(list(prescale.shape) + [1] * (
          R.t.ndim - prescale.ndim))
    pre_t = prescale
    # In the backward dimension numbers the operand's kept axes are the
    # forward contraction axes, where a forward scale has extent 1; its
    # contraction axes pair, in order, with the cotangent's.
    for ax in rra:
      assert pre_t.shape[ax] == 1, (
          'forward scale varies along an axis the backward dot keeps; set '
          'use_fwd_quant=False')

  def pre_strides(axes):
    return [0 if pre_t.shape[a] == 1 else pre_t.stride(a) for a in axes]

  try:
    # batch group: lhs, rhs, out (+ prescale, noises)
    tensors_b = [L.strides_of(lba), R.strides_of(rba), out_b]
    if pre_t is not None:
      tensors_b.append(pre_strides(rba))
    if noise_l is not None:
      tensors_b.append([noise_l.stride(a) for a in lba])
    if noise_r is not None:
      tensors_b.append([noise_r.stride(a) for a in rba])
    bdims = _merge(L.extents_of(lba), tensors_b, 2)
    tensors_m = [L.strides_of(lra), out_m]
    if noise_l is not None:
      tensors_m.append([noise_l.stride(a) for a in lra])
    mdims = _merge(L.extents_of(lra), tensors_m, 1)
    tensors_n = [R.strides_of(rra), out_n]
    if noise_r is not None:
      tensors_n.append([noise_r.stride(a) for a in rra])
    ndims = _merge(R.extents_of(rra), tensors_n, 1)
    tensors_k = [L.strides_of(lca), R.strides_of(rca)]
    if pre_t is not None:
      tensors_k.append(pre_strides(rca))
    if noise_l is not None:
      tensors_k.append([noise_l.stride(a) for a in lca])
    if noise_r is not None:
      tensors_k.append([noise_r.stride(a) for a in rca])
    kdims = _merge(L.extents_of(lca), tensors_k, 1)
    if None in (bdims, mdims, ndims, kdims):
      raise _Unmergeable()
    if pre_t is not None:
      for a, e in zip(rca, L.extents_of(lca)):
        assert pre_t.shape[a] in (1, e), (
            f'forward scale shape {tuple(pre_t.shape)} does not line up with '
            'the cotangent; set use_fwd_quant=False')
  except _Unmergeable:
    if _regrouped or defer_dequant:
      raise NotImplementedError(
          f'dimension_numbers {dimension_numbers} with these strides cannot '
          'be expressed as one strided batched GEMM')
    return _dg_raw_via_copies(raw, lhs, rhs, lhs_qt, rhs_qt, dimension_numbers,
                              out_transpose_axes, want_acc, out)

  def pad(dims, n, nt):
    dims = list(dims)
    while len(dims) < n:
      dims.insert(0, (1, [0] * nt))
    return dims

  bdims = pad(bdims, 2, len(tensors_b))
  (M, ms), = pad(mdims, 1, len(tensors_m))
  (N, ns), = pad(ndims, 1, len(tensors_n))
  (K, ks), = pad(kdims, 1, len(tensors_k))
  B = [bdims[0][0], bdims[1][0]]
  bs = lambda t: [bdims[0][1][t], bdims[1][1][t]]

  def dense(stride, extent):
    # a dim of extent 1 gets stride 1 so either kernel mode is admissible
    return 1 if extent == 1 else stride

  def row_stride(stride, extent, k_stride):
    # a single row takes the dense stride when the contraction index is
    # contiguous, so that the 16-byte-vector kernels still apply
    if extent == 1:
      return K if dense(k_stride, K) == 1 else 1
    return stride

  desc = _lib.DgRawDesc()
  desc.lhs = _view(L.t.data_ptr(), _code(L.t.dtype), B, M, K, bs(0),
                   row_stride(ms[0], M, ks[0]), dense(ks[0], K))
  desc.rhs = _view(R.t.data_ptr(), _code(R.t.dtype), B, N, K, bs(1),
                   row_stride(ns[0], N, ks[1]), dense(ks[1], K))
  ti_b, ti_m, ti_n, ti_k = 3, 2, 2, 2
  if pre_t is not None:
    desc.lhs_prescale = _view(pre_t.data_ptr(), _code(pre_t.dtype), B, 1, K,
                              bs(ti_b), 0, ks[ti_k])
    ti_b += 1
    ti_k += 1
  keep = [out_t]
  if noise_l is not None:
    desc.lhs_noise = _view(noise_l.data_ptr(), _lib.F32, B, M, K, bs(ti_b),
                           ms[ti_m], ks[ti_k])
    ti_b += 1
    ti_m += 1
    ti_k += 1
    keep.append(noise_l)
  if noise_r is not None:
    desc.rhs_noise = _view(noise_r.data_ptr(), _lib.F32, B, N, K, bs(ti_b),
                           ns[ti_n], ks[ti_k])
    keep.append(noise_r)
  desc.lhs_spec = lhs_spec
  desc.rhs_spec = rhs_spec

  dev = lhs.device
  ldk = (K + 15) // 16 * 16
  nB = B[0] * B[1]

  def side_buffers(spec, rows, qv, sin, op):
    n_sc = 1 if spec.per_tensor else nB * rows
    s_dtype = _CODE_TORCH[spec.scale_dtype]
    if qv is not None:
      # pre-quantized operand: must already be contraction-contiguous
      qbuf = None
    else:
      qbuf = _empty((nB, rows, ldk), _CODE_TORCH[spec.qdtype], dev)
    sbuf = _empty(n_sc, s_dtype, dev)
    sin_c = None
    if sin is not None:
      sin_c = _as_scale_compact(sin, op, bool(spec.per_tensor),
                                spec.scale_dtype)
      sbuf = sin_c
    return qbuf, sbuf, sin_c

  lq, ls, lsin = side_buffers(lhs_spec, M, lhs_qv, lhs_sin, L)
  rq, rs_, rsin = side_buffers(rhs_spec, N, rhs_qv, rhs_sin, R)
  keep += [lq, ls, rq, rs_, lsin, rsin]
  desc.lhs_scale_in = lsin.data_ptr() if lsin is not None else None
  desc.rhs_scale_in = rsin.data_ptr() if rsin is not None else None
  desc.lhs_is_quantized = 1 if lhs_qv is not None else 0
  desc.rhs_is_quantized = 1 if rhs_qv is not None else 0
  if lhs_qv is not None and (desc.lhs.col_stride != 1 and K > 1):
    raise _NeedsKMajor('lhs')
  if rhs_qv is not None and (desc.rhs.col_stride != 1 and K > 1):
    raise _NeedsKMajor('rhs')
  desc.lhs_q = lq.data_ptr() if lq is not None else None
  desc.lhs_scale = ls.data_ptr()
  desc.rhs_q = rq.data_ptr() if rq is not None else None
  desc.rhs_scale = rs_.data_ptr()
  # Put the operand whose kept index is contiguous in the OUTPUT on the
  # column side of the tile so the epilogue stores rows of the result.
  swap = (ns[1] != 1 and ms[1] == 1 and N > 1)
  # A few rows against many (decode-time serving: tokens x weight rows): the
  # many go on the row side of the tile whatever the output layout, so the
  # MMAs are only as wide as the few (see fill_params in csrc/gemm.cu).
  if M <= 64 and N >= 8 * max(M, 16):
    swap = True
  desc.swap_ab = 1 if swap else 0
  desc.dequant_dtype = d_code
  desc.out = out_t.data_ptr()
  desc.out_dtype = _code(out_dtype)
  desc.out_b0_stride, desc.out_b1_stride = bs(2)
  desc.out_m_stride = ms[1]
  desc.out_n_stride = ns[1]
  acc = None
  if defer_dequant:
    want_acc = True
  if want_acc:
    acc_shape = (nB, N, M) if swap else (nB, M, N)
    acc_dtype = torch.int32 if ints[0] else torch.float32
    if acc_buf is not None:
      assert (acc_buf.is_contiguous() and acc_buf.dtype == acc_dtype and
              acc_buf.numel() == nB * M * N), 'acc_buf: wrong size or dtype'
      acc = acc_buf.view(acc_shape)
    else:
      acc = _empty(acc_shape, acc_dtype, dev)
    desc.acc_out = acc.data_ptr()
    acc_storage = acc
    if swap:
      acc = acc.transpose(1, 2)
  if defer_dequant:
    desc.out = None
  if amax_out is not None:
    assert amax_out.dtype == torch.float32 and amax_out.numel() == 1
    desc.amax_out = amax_out.data_ptr()
  if getattr(raw, 'jax_scope_name', None):
    desc.scope_name = _scope_bytes(raw.jax_scope_name)

  lib = _lib.load()
  ws_bytes = lib.aqtb200_dot_general_raw_workspace_bytes(C.byref(desc))
  ws = _empty(max(ws_bytes, 256), torch.uint8, dev)
  if _tape is None:
    poll_status(dev)
  status = _status_buf(dev)
  rc = _call(lib.aqtb200_dot_general_raw, C.byref(desc), ws.data_ptr(),
             ws.numel(), status.data_ptr(), _stream())
  _lib.check(rc, f'aqtb200_dot_general_raw[{raw.jax_scope_name}]')
  del keep  # buffers stay alive until here; frees are stream-ordered

  # residuals: QTensors with the reference's logical shapes
  dd_l = utils.as_dtype(lhs.dtype)
  dd_r = utils.as_dtype(rhs_compute_dtype) if rhs_compute_dtype is not None else (
      utils.as_dtype(rhs_float.dtype))
  if lhs_qv is not None:
    lhs_q_out = lhs_qt
  else:
    lhs_q_out = aqt_tensor.QTensor(
        qvalue=_logical_q(lq.view(nB, M, ldk), L, K),
        scale=[_logical_scale(ls, L, bool(lhs_spec.per_tensor))], scale_t=None,
        bias=[], dequant_dtype=dd_l)
  if rhs_qv is not None:
    rhs_q_out = rhs_qt
  else:
    rhs_q_out = aqt_tensor.QTensor(
        qvalue=_logical_q(rq.view(nB, N, ldk), R, K),
        scale=[_logical_scale(rs_, R, bool(rhs_spec.per_tensor))],
        scale_t=None, bias=[], dequant_dtype=dd_r)

  def grad_fn(quantizer, x, given):
    if given is not None and not raw.allow_dummy_gradient_into_qtensor:
      return adg._POISON  # pylint: disable=protected-access
    n = quantizer.numerics
    if getattr(n, 'clip_gradient', False):
      raise NotImplementedError('clip_gradient on the fused path')
    return functools.partial(n.vjp_bwd, (None,))

  res = adg.DotGeneralRes(
      lhs=adg.TensorRes(mt=adg.MultiTensor(x=lhs, qx=lhs_q_out),
                        quant_grad=grad_fn(q.lhs, lhs,
                                           None if internal_qt else lhs_qv)),
      rhs=adg.TensorRes(mt=adg.MultiTensor(x=rhs_float, qx=rhs_q_out),
                        quant_grad=grad_fn(q.rhs, rhs_float,
                                           None if internal_qt else rhs_qv)))
  if defer_dequant:
    return DeferredDequant(desc, acc_storage, out_t,
                           [lq, ls, rq, rs_, lsin, rsin]), res
  if want_acc:
    return out_t, res, acc
  return out_t, res


class _NeedsKMajor(NotImplementedError):

  def __init__(self, side):
    super().__init__(
        f'the pre-quantized {side} QTensor must store its contraction axis '
        'contiguously; convert it once with engine.to_k_major()')


def to_k_major(qt, contraction_axes: Sequence[int]):
  """Re-lays a QTensor's qvalue so the given contraction axes are innermost.

  A one-off conversion for frozen serving weights (flax/freezer.py keeps them
  in the weight's own layout, contraction axis first for a [K, N] kernel).
  The logical shape is unchanged; only strides differ.
  """
  q = qt.qvalue
  ca = list(contraction_axes)
  rest = [a for a in range(q.ndim) if a not in ca]
  order = rest + ca
  inv = [order.index(i) for i in range(q.ndim)]
  k = _prod([q.shape[a] for a in ca])
  ldk = (k + 15) // 16 * 16
  rows = _prod([q.shape[a] for a in rest])
  buf = torch.zeros((1, rows, ldk), dtype=torch.uint8, device=q.device)
  buf[0, :, :k] = q.permute(*order).reshape(rows, k).contiguous().view(
      torch.uint8)
  buf = buf.view(q.dtype)
  t = _strided_logical(buf, [], [q.shape[a] for a in rest],
                       [q.shape[a] for a in ca])
  return qt.replace(qvalue=t.permute(*inv))


def _dg_raw_unquantized(raw, lhs, rhs, lhs_qt, rhs_qt, dims,
                        out_transpose_axes):
  """Both operands NoNumerics: a plain library GEMM (not the hot path)."""
  from aqt_b200.v2 import aqt_dot_general as adg
  from aqt_b200.v2 import aqt_tensor
  out = adg.lax_dot_general(lhs, rhs, dims)
  if out_transpose_axes is not None:
    out = out.permute(*out_transpose_axes)

  def qt(x):
    return aqt_tensor.QTensor(qvalue=x, scale=[], scale_t=None, bias=[],
                              dequant_dtype=utils.as_dtype(x.dtype))

  res = adg.DotGeneralRes(
      lhs=adg.TensorRes(mt=adg.MultiTensor(x=lhs, qx=qt(lhs)), quant_grad=None),
      rhs=adg.TensorRes(mt=adg.MultiTensor(x=rhs, qx=qt(rhs)), quant_grad=None))
  return out, res


def _dg_raw_via_copies(raw, lhs, rhs, lhs_qt, rhs_qt, dims,
                       out_transpose_axes, want_acc, out=None):
  """Strides the kernels cannot express: regroup axes with copies, then retry.

  Operands (and, in the backward pass, the stored quantized operand with its
  scale) are permuted to (batch, kept, contraction) order and made contiguous,
  the dot runs on the regrouped tensors into a contiguous raw-order result, and
  everything handed back -- the result, the residual operands, the QTensors --
  is a permuted view with the caller's own axis order, so the backward pass
  can keep using the forward dimension numbers.
  """
  from aqt_b200.v2 import aqt_dot_general as adg
  from aqt_b200.v2 import aqt_tensor
  (lca, rca), (lba, rba) = dims
  lca, rca, lba, rba = list(lca), list(rca), list(lba), list(rba)
  is_mt = isinstance(rhs, adg.MultiTensor)
  rhs_x = rhs.x if is_mt else rhs
  lra = utils.get_remaining_axes(lhs.ndim, lca, lba)
  rra = utils.get_remaining_axes(rhs_x.ndim, rca, rba)
  l_order, r_order = lba + lra + lca, rba + rra + rca
  l_inv = [l_order.index(i) for i in range(lhs.ndim)]
  r_inv = [r_order.index(i) for i in range(rhs_x.ndim)]
  regroup_l = lambda t: t.permute(*l_order).contiguous()
  regroup_r = lambda t: t.permute(*r_order).contiguous()

  def regroup_qt(qt, regroup, what):
    """An incomplete (scale-only) caller QTensor follows its operand."""
    if qt is None:
      return None
    if qt.is_full():
      raise NotImplementedError(
          f'a pre-quantized {what} with dimension_numbers that need a '
          'regrouping copy')
    return qt.replace(scale=[regroup(s) if s.numel() > 1 else
                             s.reshape([1] * s.ndim) for s in qt.scale])

  l2 = regroup_l(lhs)
  if is_mt:
    qx = rhs.qx
    if qx is not None and isinstance(qx.qvalue, torch.Tensor):
      qx = qx.replace(
          qvalue=regroup_r(qx.qvalue),
          scale=[regroup_r(s) for s in (qx.scale or [])])
    r2 = adg.MultiTensor(x=regroup_r(rhs_x), qx=qx)
  else:
    r2 = regroup_r(rhs_x)
  nb, nm, nn, nk = len(lba), len(lra), len(rra), len(lca)
  dims2 = ((tuple(range(nb + nm, nb + nm + nk)),
            tuple(range(nb + nn, nb + nn + nk))),
           (tuple(range(nb)), tuple(range(nb))))
  # Stochastic-rounding noise pairs with the operand's elements in the
  # caller's axis order: draw it there, then regroup it like the operand.
  q = raw.dg_quantizer
  noise = (None, None)
  if hasattr(q, 'lhs'):
    nl = _noise_for(q.lhs, lhs.shape, lhs.device) if lhs_qt is None or (
        not lhs_qt.is_full()) else None
    nr = _noise_for(q.rhs, rhs_x.shape, lhs.device) if rhs_qt is None or (
        not rhs_qt.is_full()) else None
    noise = (None if nl is None else regroup_l(nl),
             None if nr is None else regroup_r(nr))
  got = dg_raw(raw, l2, r2, regroup_qt(lhs_qt, regroup_l, 'lhs'),
               regroup_qt(rhs_qt, regroup_r, 'rhs'), dims2, None, want_acc,
               _regrouped=True, _noise=noise)
  res2 = got[1]

  def back(mt, x_orig, inv):
    qx = mt.qx
    if qx is not None and isinstance(qx.qvalue, torch.Tensor):
      qx = qx.replace(qvalue=qx.qvalue.permute(*inv),
                      scale=[s.permute(*inv) for s in (qx.scale or [])])
    return adg.MultiTensor(x=x_orig, qx=qx)

  res = adg.DotGeneralRes(
      lhs=adg.TensorRes(mt=back(res2.lhs.mt, lhs, l_inv),
                        quant_grad=res2.lhs.quant_grad),
      rhs=adg.TensorRes(mt=back(res2.rhs.mt, rhs_x, r_inv),
                        quant_grad=res2.rhs.quant_grad))
  result = got[0]
  if out_transpose_axes is not None:
    result = result.permute(*out_transpose_axes)
  if out is not None:
    out.copy_(result)
    result = out
  return (result, res) + tuple(got[2:])


# ---------------------------------------------------------------------------
# piecewise API (Quantizer.calibrate / calculate_qvalue, QTensor.dequant)


def _single_operand(x, shared_axes):
  nd = x.ndim
  ca = sorted(int(a) % nd for a in shared_axes)
  ra = [a for a in range(nd) if a not in ca]
  op = _Operand(x, [], ra, ca)
  rdims = _merge(op.extents_of(ra), [op.strides_of(ra)], 1)
  kdims = _merge(op.extents_of(ca), [op.strides_of(ca)], 1)
  if rdims is None or kdims is None:
    xc = x.permute(*ra, *ca).contiguous()
    order = ra + ca
    inv = [order.index(i) for i in range(nd)]
    return _single_operand(xc.permute(*inv), shared_axes)
  (rows, rs), = rdims or [(1, [1])]
  (cols, cs), = kdims or [(1, [1])]
  cs = 1 if cols == 1 else cs[0]
  # a single row: give it the dense stride, so the 16-byte-vector kernels
  # (which want row starts aligned) still apply
  rs = (cols * cs if cs == 1 else 1) if rows == 1 else rs[0]
  if rs != 1 and cs != 1:
    xc = x.permute(*ra, *ca).contiguous()
    order = ra + ca
    inv = [order.index(i) for i in range(nd)]
    return _single_operand(xc.permute(*inv), shared_axes)
  view = _view(x.data_ptr(), _code(x.dtype), [1, 1], rows, cols, [0, 0], rs, cs)
  return op, view, rows, cols


def _spec_for(numerics, x_code, scale_dtype, per_tensor, clipping_scale=None,
              po2_scale=False):
  kind, qcode, qb, cb = _numerics_fields(numerics)
  spec = _lib.QuantSpec()
  spec.kind, spec.qdtype, spec.quant_bound, spec.clip_bound = kind, qcode, qb, cb
  spec.per_tensor = 1 if per_tensor else 0
  spec.compute_dtype = x_code
  spec.scale_dtype = x_code if scale_dtype is None else _code(scale_dtype)
  spec.po2_scale = 1 if po2_scale else 0
  spec.clipping_scale = (
      _round_to_dtype(clipping_scale, x_code) if clipping_scale else 0.0)
  return spec


def absmax_scale(x, shared_axes, numerics, scale_dtype=None,
                 clipping_scale=None, po2_scale=False, prescale=None,
                 compute_dtype=None):
  """AbsMaxCalibration on the device: the scale, x's rank, shared axes 1.

  prescale: optional tensor broadcastable against x that is constant along
  the kept (non-shared) axes; x is multiplied by it (rounded to the compute
  dtype) before the maximum is taken, as the backward pass does with the
  other operand's forward scale. compute_dtype: the float dtype x counts as
  when it is a stored int8/fp8 tensor.
  """
  per_tensor = len(shared_axes) == x.ndim
  op, view, rows, cols = _single_operand(x, shared_axes)
  x_code = _code(compute_dtype) if compute_dtype is not None else _code(x.dtype)
  spec = _spec_for(numerics, x_code, scale_dtype, per_tensor,
                   clipping_scale, po2_scale)
  pre_view = None
  if prescale is not None:
    pre = prescale.expand(x.shape) if prescale.ndim == x.ndim else prescale
    pop = _Operand(pre, [], op.ra, op.ca)
    for a in op.ra:
      assert prescale.ndim != x.ndim or prescale.shape[a] == 1 or per_tensor, (
          'prescale must be constant along the kept axes')
    kd = _merge(op.extents_of(op.ca), [pop.strides_of(op.ca)], 1)
    if kd is None or (view.col_stride != 1 and view.row_stride != 1):
      raise NotImplementedError('prescale layout for absmax_scale')
    pcs = kd[0][1][0] if kd else 0
    if per_tensor and any(pre.stride(a) != 0 for a in range(x.ndim)):
      # every axis is reduced: rows/cols came from an arbitrary split, so
      # only a scalar prescale can be expressed
      raise NotImplementedError('non-scalar prescale with a per-tensor scale')
    pre_view = _view(prescale.data_ptr(), _code(prescale.dtype), [1, 1], 1,
                     cols, [0, 0], 0, pcs)
  lib = _lib.load()
  n = 1 if per_tensor else rows
  sbuf = _empty(n, _CODE_TORCH[spec.scale_dtype], x.device)
  ws_bytes = lib.aqtb200_quantize_workspace_bytes(C.byref(view), C.byref(spec))
  ws = _empty(max(ws_bytes, 256), torch.uint8, x.device)
  rc = _call(
      lib.aqtb200_absmax_scale,
      C.byref(view), C.byref(pre_view) if pre_view is not None else None,
      C.byref(spec), sbuf.data_ptr(), ws.data_ptr(), ws.numel(), _stream())
  _lib.check(rc, 'aqtb200_absmax_scale')
  return _logical_scale(sbuf, op, per_tensor)


def absmax_raw(x):
  """max |x| over the whole tensor as a 1-element f32 device tensor."""
  op, view, rows, cols = _single_operand(x, list(range(x.ndim)))
  out = _empty(1, torch.float32, x.device)
  rc = _call(_lib.load().aqtb200_absmax_raw, C.byref(view), 1, out.data_ptr(),
             _stream())
  _lib.check(rc, 'aqtb200_absmax_raw')
  return out


def prescale_amax(amax, prescale, compute_code: int):
  """|round_T(amax * round_T(prescale))|: the maximum of a tensor after one
  prescale value has been folded into it (rounding is monotone)."""
  assert prescale.numel() == 1
  out = _empty(1, torch.float32, amax.device)
  rc = _call(_lib.load().aqtb200_prescale_amax, amax.data_ptr(), 1,
             prescale.data_ptr(), _code(prescale.dtype), compute_code,
             out.data_ptr(), _stream())
  _lib.check(rc, 'aqtb200_prescale_amax')
  return out


def scale_from_amax(amax, numerics, compute_dtype, scale_dtype=None,
                    clipping_scale=None, po2_scale=False, prescale=None,
                    ndim=2):
  """Per-tensor scale from a precomputed maximum (and one prescale value).

  Returns the scale with `ndim` axes of extent 1, like the reference's
  per-tensor scale.
  """
  code = _code(compute_dtype)
  spec = _spec_for(numerics, code, scale_dtype, True, clipping_scale, po2_scale)
  out = _empty(1, _CODE_TORCH[spec.scale_dtype], amax.device)
  pre_ptr, pre_code = None, 0
  if prescale is not None:
    assert prescale.numel() == 1
    pre_ptr, pre_code = prescale.data_ptr(), _code(prescale.dtype)
  rc = _call(
      _lib.load().aqtb200_scale_from_amax,
      amax.data_ptr(), 1, pre_ptr, pre_code, C.byref(spec), out.data_ptr(),
      _stream())
  _lib.check(rc, 'aqtb200_scale_from_amax')
  return out.view([1] * ndim)


def _per_tensor_absmax(quantizer):
  """Calibration keywords if the quantizer is per-tensor AbsMax, else None."""
  if type(quantizer.numerics).__name__ == 'NoNumerics':
    return None
  if quantizer.calib_shared_axes != 'per_tensor' or _delayed(quantizer):
    return None
  kw = _calibration_kwargs(quantizer)
  if getattr(quantizer.numerics, 'noise_fn', None):
    pass  # noise does not change the scale
  return kw


def shared_cotangent_scales(cfg, res, g, reduce_max=None):
  """Scales of the cotangent for dlhs and drhs from ONE pass over it.

  Applies when both gradient dots quantize g with a per-tensor scale and the
  forward scales folded into g (use_fwd_quant) are per-tensor too: then
  max|g * s| = |round(max|g| * s)| and a single raw maximum serves both.
  `reduce_max`, if given, is applied to the raw maximum (cross-rank max).
  Returns (g_qt_dlhs, g_qt_drhs) as incomplete QTensors, or None.
  """
  from aqt_b200.v2 import aqt_tensor
  ql, qr = cfg.dlhs.dg_quantizer.lhs, cfg.drhs.dg_quantizer.lhs
  kwl, kwr = _per_tensor_absmax(ql), _per_tensor_absmax(qr)
  if kwl is None or kwr is None:
    return None
  pres = []
  for raw, mt in ((cfg.dlhs, res.rhs.mt), (cfg.drhs, res.lhs.mt)):
    if raw.rhs.use_fwd_quant:
      if mt.qx.scale is None or len(mt.qx.scale) != 1 or (
          mt.qx.scale[0].numel() != 1):
        return None
      pres.append(mt.qx.scale[0])
    else:
      pres.append(None)
  amax = absmax_raw(g)
  if reduce_max is not None:
    amax = reduce_max(amax)
  out = []
  dd = utils.as_dtype(g.dtype)
  for q, kw, pre in ((ql, kwl, pres[0]), (qr, kwr, pres[1])):
    scale = scale_from_amax(
        amax, q.numerics, g.dtype, kw.get('dtype', q.scale_dtype),
        kw.get('clipping_scale'), kw.get('po2_scale', False), pre, g.ndim)
    out.append(aqt_tensor.QTensor(qvalue=None, scale=[scale], scale_t=None,
                                  bias=[], dequant_dtype=dd))
  return tuple(out)


# ---------------------------------------------------------------------------
# one read of an operand for both layouts a training step needs it in
# (aqtb200_quantize_pair). Applies to 2-D bf16 matmuls whose quantizers are all
# per-tensor fp8 or int8 without noise; everything else keeps the one-quantization-
# per-dot flow of the reference.

_BWD_COPY = '_aqt_b200_bwd_copy'  # attribute of the forward qvalue tensor


def _pair_spec(quantizer):
  """The per-tensor fp8 or int8 / bf16 spec of `quantizer`, or None if it is
  anything else. Delayed scaling counts as per-tensor whatever the axes."""
  if type(quantizer.numerics).__name__ not in ('Fp8Numerics', 'IntSymmetric'):
    return None
  if quantizer.calib_shared_axes != 'per_tensor' and not _delayed(quantizer):
    return None
  if getattr(quantizer.numerics, 'noise_fn', None) or getattr(
      quantizer.numerics, 'stochastic_rounding', False):
    return None
  try:
    spec = _make_spec(quantizer, _lib.BF16, True)
  except NotImplementedError:
    return None
  if spec is None or spec.scale_dtype != _lib.BF16:
    return None
  if spec.kind == _lib.NUM_INT and spec.qdtype != _lib.S8:
    return None
  return spec


def _pair_matrix_ok(x):
  return (isinstance(x, torch.Tensor) and x.ndim == 2 and
          x.dtype == torch.bfloat16 and _on_device(x) and
          x.stride(1) == 1 and x.stride(0) == x.shape[1] and
          x.shape[0] % 16 == 0 and x.shape[1] % 16 == 0 and x.numel() > 0 and
          x.data_ptr() % 16 == 0)


def _scale_of_amax(amax, spec, prescale=None):
  out = _empty(1, _CODE_TORCH[spec.scale_dtype], amax.device)
  pre_ptr, pre_code = None, 0
  if prescale is not None:
    pre_ptr, pre_code = prescale.data_ptr(), _code(prescale.dtype)
  rc = _call(
      _lib.load().aqtb200_scale_from_amax,
      amax.data_ptr(), 1, pre_ptr, pre_code, C.byref(spec), out.data_ptr(),
      _stream())
  _lib.check(rc, 'aqtb200_scale_from_amax')
  return out


def _requant_amax(amax, spec, scale, prescale=None):
  """|value of Q(amax)| under (spec, scale[, prescale]): the maximum of the
  quantized values of a tensor whose maximum is amax (aqtb200_requant_amax)."""
  out = _empty(1, torch.float32, amax.device)
  pre_ptr, pre_code = (None, 0) if prescale is None else (
      prescale.data_ptr(), _code(prescale.dtype))
  rc = _call(_lib.load().aqtb200_requant_amax, amax.data_ptr(), 1, pre_ptr,
             pre_code, C.byref(spec), scale.data_ptr(), out.data_ptr(),
             _stream())
  _lib.check(rc, 'aqtb200_requant_amax')
  return out


def _quantize_pair(x, spec_t, scale_t, pre_t, spec_s, scale_s, pre_s, chain,
                   amax=None, amax_out=None):
  """x: [C, R] row-major bf16. Returns (q_t [R][C], q_s [C][R]) buffers.

  With `amax` (the raw maximum of x) the kernel computes both scales itself
  and writes them into scale_t / scale_s; otherwise it reads them. `amax_out`
  (one f32) receives max |x| from the same read.
  """
  c, r = x.shape
  view = _view(x.data_ptr(), _lib.BF16, [1, 1], r, c, [0, 0], 1, r)
  q_t = _empty((r, c), _CODE_TORCH[spec_t.qdtype], x.device)
  q_s = _empty((c, r), _CODE_TORCH[spec_s.qdtype], x.device)
  ptr = lambda t: (None, 0) if t is None else (t.data_ptr(), _code(t.dtype))
  (pt, ptc), (ps, psc) = ptr(pre_t), ptr(pre_s)
  rc = _call(
      _lib.load().aqtb200_quantize_pair, C.byref(view), C.byref(spec_t),
      scale_t.data_ptr(), pt, ptc,
      q_t.data_ptr(), C.byref(spec_s), scale_s.data_ptr(), ps, psc,
      q_s.data_ptr(), chain, None if amax is None else amax.data_ptr(),
      None if amax_out is None else amax_out.data_ptr(), _stream())
  _lib.check(rc, 'aqtb200_quantize_pair')
  return q_t, q_s


def prequantize_for_training(cfg, lhs, rhs, dimension_numbers,
                             reduce_max_lhs=None):
  """Forward AND backward quantization of both operands of lhs[M,K] @ rhs[K,N].

  The backward pass re-quantizes the stored forward values of each operand
  along the other axis (aqt_dot_general.py:675-729, 1206-1217). Both copies
  are fixed functions of the operand and of its maximum, so they are produced
  together here, in one read. Returns full QTensors (lhs_qt, rhs_qt) for the
  forward dot, each carrying the backward copy, or None when the
  configuration is outside what aqtb200_quantize_pair covers.
  reduce_max_lhs, if given, is applied to lhs's raw maximum (a cross-rank max
  when the rows of lhs are sharded); every scale of lhs follows from it.
  """
  from aqt_b200.v2 import aqt_tensor
  (lca, rca), (lba, rba) = dimension_numbers
  if list(lca) != [1] or list(rca) != [0] or list(lba) or list(rba):
    return None
  if not (_pair_matrix_ok(lhs) and _pair_matrix_ok(rhs)):
    return None
  for raw in (cfg.fwd, cfg.dlhs, cfg.drhs):
    try:
      _check_raw_supported(raw)
    except NotImplementedError:
      return None
  if not (cfg.dlhs.rhs.use_fwd_quant and cfg.drhs.rhs.use_fwd_quant):
    return None
  specs = [_pair_spec(q) for q in (
      cfg.fwd.dg_quantizer.lhs, cfg.fwd.dg_quantizer.rhs,
      cfg.drhs.dg_quantizer.rhs, cfg.dlhs.dg_quantizer.rhs)]
  if any(sp is None for sp in specs):
    return None
  f_lhs, f_rhs, b_lhs, b_rhs = specs
  dd = utils.as_dtype(lhs.dtype)
  quantizers = (cfg.fwd.dg_quantizer.lhs, cfg.fwd.dg_quantizer.rhs,
                cfg.drhs.dg_quantizer.rhs, cfg.dlhs.dg_quantizer.rhs)
  n_delayed = sum(_delayed(q) is not None for q in quantizers)
  if n_delayed not in (0, 4):
    return None  # mixed calibrations: one quantization per dot
  if n_delayed:
    return _prequantize_delayed(quantizers, specs, lhs, rhs, dd,
                                reduce_max_lhs)

  def new_scales(x):
    mk = lambda: _empty(1, torch.bfloat16, x.device)
    return mk(), mk()

  def amax_of(x, reduce_max=None):
    amax = absmax_raw(x)
    return reduce_max(amax) if reduce_max is not None else amax

  def qt(qvalue, scale):
    return aqt_tensor.QTensor(qvalue=qvalue, scale=[scale.view(1, 1)],
                              scale_t=None, bias=[], dequant_dtype=dd)

  # lhs's maximum first: when it has to be agreed across ranks, that exchange
  # (reduce_max_lhs may return (tensor, wait) for one in flight) runs while
  # rhs, which is replicated, is calibrated and quantized.
  lhs_amax = amax_of(lhs, reduce_max_lhs)
  lhs_wait = None
  if isinstance(lhs_amax, tuple):
    lhs_amax, lhs_wait = lhs_amax
  # rhs [K, N]: the transposed copy, [N][K], is the forward one; its own
  # orientation (N contiguous) is what dlhs contracts over.
  s1, s2 = new_scales(rhs)
  q_t, q_s = _quantize_pair(rhs, f_rhs, s1, None, b_rhs, s2, None, chain=1,
                            amax=amax_of(rhs))
  rhs_qt = qt(q_t.t(), s1)
  setattr(rhs_qt.qvalue, _BWD_COPY, qt(q_s, s2))
  # lhs [M, K]: its own orientation is the forward copy (K contiguous); the
  # transposed one, [K][M], is what drhs contracts over M.
  if lhs_wait is not None:
    lhs_wait()
  s1, s2 = new_scales(lhs)
  q_t, q_s = _quantize_pair(lhs, b_lhs, s2, None, f_lhs, s1, None, chain=2,
                            amax=lhs_amax)
  lhs_qt = qt(q_s, s1)
  setattr(lhs_qt.qvalue, _BWD_COPY, qt(q_t.t(), s2))
  return lhs_qt, rhs_qt


def _sync_reduce(reduce_max, t):
  """Applies a cross-rank maximum that may be handed over as (tensor, wait)."""
  if reduce_max is None:
    return t
  r = reduce_max(t)
  if isinstance(r, tuple):
    r[1]()
    return r[0]
  return r


def _prequantize_delayed(quantizers, specs, lhs, rhs, dd, reduce_max_lhs):
  """prequantize_for_training under delayed scaling: every scale comes from
  its quantizer's history, so each operand is read ONCE in all -- the paired
  quantization also takes max |x| for the histories (of the forward quantizer
  directly, of the chained backward quantizer through |Q(max)|)."""
  from aqt_b200.v2 import aqt_tensor
  q_fl, q_fr, q_bl, q_br = quantizers
  f_lhs, f_rhs, b_lhs, b_rhs = specs

  def qt(qvalue, scale):
    return aqt_tensor.QTensor(qvalue=qvalue, scale=[scale.view(1, 1)],
                              scale_t=None, bias=[], dequant_dtype=dd)

  def one(x, q_first, sp_first, q_second, sp_second, chain, reduce_max):
    cal1, cal2 = _delayed(q_first), _delayed(q_second)
    s1 = cal1.next_scale(x.device, q_first.numerics, x.dtype, q_first.context)
    s2 = cal2.next_scale(x.device, q_second.numerics, x.dtype,
                         q_second.context)
    amax = _empty(1, torch.float32, x.device)
    if chain == 1:  # x -> q_t (first) -> q_s (second)
      q_t, q_s = _quantize_pair(x, sp_first, s1, None, sp_second, s2, None,
                                chain=1, amax_out=amax)
    else:           # x -> q_s (first) -> q_t (second)
      q_t, q_s = _quantize_pair(x, sp_second, s2, None, sp_first, s1, None,
                                chain=2, amax_out=amax)
    amax = _sync_reduce(reduce_max, amax)
    if cal1.updates_state(q_first.context):
      cal1.push_amax(amax)
    if cal2.updates_state(q_second.context):
      cal2.push_amax(_requant_amax(amax, sp_first, s1))
    return q_t, q_s, s1, s2

  # rhs [K, N]: the transposed copy, [N][K], is the forward one
  q_t, q_s, s1, s2 = one(rhs, q_fr, f_rhs, q_br, b_rhs, 1, None)
  rhs_qt = qt(q_t.t(), s1)
  setattr(rhs_qt.qvalue, _BWD_COPY, qt(q_s, s2))
  # lhs [M, K]: its own orientation is the forward copy
  q_t, q_s, s1, s2 = one(lhs, q_fl, f_lhs, q_bl, b_lhs, 2, reduce_max_lhs)
  lhs_qt = qt(q_s, s1)
  setattr(lhs_qt.qvalue, _BWD_COPY, qt(q_t.t(), s2))
  return lhs_qt, rhs_qt


def bwd_copy(qt):
  """The backward-pass copy made by prequantize_for_training, if any.

  QTensor is slotted, so the copy rides on the qvalue tensor object, which the
  forward pass hands to the backward pass unchanged inside the residuals.
  """
  if qt is None or not isinstance(qt.qvalue, torch.Tensor):
    return None
  return getattr(qt.qvalue, _BWD_COPY, None)


def cotangent_pair(cfg, res, g, reduce_max=None):
  """Both quantizations of the cotangent g[M,N] in one read (plus one pass for
  its maximum). Returns full QTensors (g for dlhs, g for drhs) or None when
  the configuration is outside what aqtb200_quantize_pair covers.
  `reduce_max`, if given, is applied to the raw maximum (cross-rank max)."""
  from aqt_b200.v2 import aqt_tensor
  if not _pair_matrix_ok(g):
    return None
  sp_dl = _pair_spec(cfg.dlhs.dg_quantizer.lhs)
  sp_dr = _pair_spec(cfg.drhs.dg_quantizer.lhs)
  if sp_dl is None or sp_dr is None or sp_dl.kind != sp_dr.kind:
    return None
  pres = []
  for raw, mt in ((cfg.dlhs, res.rhs.mt), (cfg.drhs, res.lhs.mt)):
    if raw.rhs.use_fwd_quant:
      if mt.qx.scale is None or len(mt.qx.scale) != 1 or (
          mt.qx.scale[0].numel() != 1):
        return None
      pres.append(mt.qx.scale[0])
    else:
      pres.append(None)
  q_dl, q_dr = cfg.dlhs.dg_quantizer.lhs, cfg.drhs.dg_quantizer.lhs
  n_delayed = sum(_delayed(q) is not None for q in (q_dl, q_dr))
  if n_delayed == 1:
    return None
  # g [M, N]: own orientation (N contiguous) feeds dlhs, the transposed copy
  # [N][M] feeds drhs.
  if n_delayed:
    # scales from the histories; max |g| for them from the same read
    s_dl = _delayed(q_dl).next_scale(g.device, q_dl.numerics, g.dtype,
                                     q_dl.context)
    s_dr = _delayed(q_dr).next_scale(g.device, q_dr.numerics, g.dtype,
                                     q_dr.context)
    amax = _empty(1, torch.float32, g.device)
    q_t, q_s = _quantize_pair(g, sp_dr, s_dr, pres[1], sp_dl, s_dl, pres[0],
                              chain=0, amax_out=amax)
    amax = _sync_reduce(reduce_max, amax)
    for q, pre in ((q_dl, pres[0]), (q_dr, pres[1])):
      if _delayed(q).updates_state(q.context):
        _delayed(q).push_amax(amax if pre is None else
                              prescale_amax(amax, pre, _lib.BF16))
  else:
    amax = absmax_raw(g)
    if reduce_max is not None:
      amax = reduce_max(amax)
    mk = lambda: _empty(1, torch.bfloat16, g.device)
    s_dl, s_dr = mk(), mk()
    q_t, q_s = _quantize_pair(g, sp_dr, s_dr, pres[1], sp_dl, s_dl, pres[0],
                              chain=0, amax=amax)
  dd = utils.as_dtype(g.dtype)
  qt = lambda qv, sc: aqt_tensor.QTensor(qvalue=qv, scale=[sc.view(1, 1)],
                                         scale_t=None, bias=[], dequant_dtype=dd)
  return qt(q_s, s_dl), qt(q_t.t(), s_dr)


def cotangent_dual(cfg, res, g, fwd_dimension_numbers):
  """Both quantizations of the cotangent in two passes over it, for per-row
  scales (aqtb200_quantize_dual): the batched / per-channel counterpart of
  cotangent_pair, with the forward scales folded in and stochastic-rounding
  noise. Applies when g is a contiguous bf16 tensor [..., t, s] whose LAST
  axis is what dlhs contracts and whose second-to-last is what drhs
  contracts, the leading axes being batch axes of both gradient dots (a plain
  matmul, or an einsum like 'bthd,bshd->bhts'). Returns full QTensors (g for
  dlhs, g for drhs) or None when the configuration is outside that."""
  from aqt_b200.v2 import aqt_dot_general as adg
  from aqt_b200.v2 import aqt_tensor
  if not (isinstance(g, torch.Tensor) and g.dtype == torch.bfloat16 and
          g.ndim >= 2 and g.is_contiguous() and _on_device(g) and
          g.numel() > 0 and g.data_ptr() % 16 == 0):
    return None
  nd = g.ndim
  t_ext, s_ext = g.shape[-2], g.shape[-1]
  if t_ext % 16 or s_ext % 16:
    return None
  upd = adg._update_dimension_numbers_for_backward  # pylint: disable=protected-access
  d_dims, _ = upd(fwd_dimension_numbers, False, nd, res.rhs.mt.x.ndim)
  r_dims, _ = upd(fwd_dimension_numbers, True, nd, res.lhs.mt.x.ndim)
  batch = list(range(nd - 2))
  for (gca, _), (gba, _), want in ((d_dims[0], d_dims[1], nd - 1),
                                   (r_dims[0], r_dims[1], nd - 2)):
    if list(gca) != [want] or list(gba) != batch:
      return None
  specs, pres, noises = [], [], []
  for raw, mt, dims_b in ((cfg.dlhs, res.rhs.mt, d_dims),
                          (cfg.drhs, res.lhs.mt, r_dims)):
    try:
      q = _check_raw_supported(raw)
    except NotImplementedError:
      return None
    qz = q.lhs
    if type(qz.numerics).__name__ != 'IntSymmetric' or _delayed(qz):
      return None
    (gca, yra), (gba, yba) = dims_b
    if qz.calib_shared_axes not in (None, list(gca), tuple(gca)):
      return None
    try:
      spec = _make_spec(qz, _lib.BF16, True)
    except NotImplementedError:
      return None
    if spec is None or spec.scale_dtype != _lib.BF16 or spec.qdtype != _lib.S8:
      return None
    specs.append(spec)
    pre = None
    if raw.rhs.use_fwd_quant:
      sc = mt.qx.scale
      if sc is None or len(sc) != 1 or sc[0].dtype != torch.bfloat16:
        return None
      pre = sc[0]
      if pre.ndim < mt.x.ndim:
        pre = pre.reshape(list(pre.shape) + [1] * (mt.x.ndim - pre.ndim))
      # a forward scale never varies along the axes the backward dot keeps
      kept = [a for a in range(pre.ndim) if a not in list(yra) + list(yba)]
      if any(pre.shape[a] != 1 for a in kept):
        return None
      st = lambda a: 0 if pre.shape[a] == 1 else pre.stride(a)
      pres.append((pre, [st(a) for a in yba], st(yra[0])))
    else:
      pres.append(None)
    noise = _noise_for(qz, g.shape, g.device)
    if noise is not None and (noise.stride() != g.stride() or
                              noise.data_ptr() % 16):
      return None
    noises.append(noise)
  if (noises[0] is None) != (noises[1] is None):
    return None
  # leading axes -> at most two batch dims on which g and both prescales agree
  strides = [[g.stride(a) for a in batch]]
  strides += [p[1] for p in pres if p is not None]
  bdims = _merge([g.shape[a] for a in batch], strides, 2)
  if bdims is None:
    return None
  while len(bdims) < 2:
    bdims.insert(0, (1, [0] * len(strides)))
  b_ext = [bdims[0][0], bdims[1][0]]
  nb = b_ext[0] * b_ext[1]
  desc = _lib.DualDesc()
  desc.x = _view(g.data_ptr(), _lib.BF16, b_ext, s_ext, t_ext,
                 [bdims[0][1][0], bdims[1][1][0]], 1, s_ext)
  desc.spec_s, desc.spec_t = specs[0], specs[1]
  col = 1
  for which, p in (('prescale_s', pres[0]), ('prescale_t', pres[1])):
    if p is None:
      continue
    bs = [bdims[0][1][col], bdims[1][1][col]]
    col += 1
    # prescale_s varies along x's rows (s), prescale_t along x's cols (t)
    rs, cs = (p[2], 0) if which == 'prescale_s' else (0, p[2])
    setattr(desc, which, _view(p[0].data_ptr(), _lib.BF16, b_ext, s_ext, t_ext,
                               bs, rs, cs))
  if noises[0] is not None:
    for which, nz in (('noise_s', noises[0]), ('noise_t', noises[1])):
      setattr(desc, which, _view(nz.data_ptr(), _lib.F32, b_ext, s_ext, t_ext,
                                 [bdims[0][1][0], bdims[1][1][0]], 1, s_ext))
  dev = g.device
  q_s = _empty((nb, t_ext, s_ext), torch.int8, dev)
  q_t = _empty((nb, s_ext, t_ext), torch.int8, dev)
  sc_s = _empty(nb * t_ext, torch.bfloat16, dev)
  sc_t = _empty(nb * s_ext, torch.bfloat16, dev)
  desc.q_s, desc.q_t = q_s.data_ptr(), q_t.data_ptr()
  desc.scale_s, desc.scale_t = sc_s.data_ptr(), sc_t.data_ptr()
  lib = _lib.load()
  ws_bytes = lib.aqtb200_quantize_dual_workspace_bytes(C.byref(desc))
  ws = _empty(max(ws_bytes, 256), torch.uint8, dev)
  rc = _call(lib.aqtb200_quantize_dual, C.byref(desc), ws.data_ptr(),
             ws.numel(), _stream())
  _lib.check(rc, 'aqtb200_quantize_dual')
  lead = list(g.shape[:-2])
  dd = utils.as_dtype(g.dtype)
  qt = lambda qv, sc: aqt_tensor.QTensor(qvalue=qv, scale=[sc], scale_t=None,
                                         bias=[], dequant_dtype=dd)
  g_dlhs = qt(q_s.view(lead + [t_ext, s_ext]), sc_s.view(lead + [t_ext, 1]))
  g_drhs = qt(q_t.view(lead + [s_ext, t_ext]).transpose(-1, -2),
              sc_t.view(lead + [1, s_ext]))
  return g_dlhs, g_drhs


def quantize_with_scale(x, scale, numerics, noise=None):
  """Quantizer.calculate_qvalue with a given scale: returns qvalue."""
  shared = [a for a in range(x.ndim) if scale.shape[a] == 1 and x.shape[a] != 1]
  per_tensor = scale.numel() == 1
  if per_tensor:
    shared = list(range(x.ndim))
  op, view, rows, cols = _single_operand(x, shared)
  x_code = _code(x.dtype)
  spec = _spec_for(numerics, x_code, utils.as_dtype(scale.dtype), per_tensor)
  sin = _as_scale_compact(scale, op, per_tensor, spec.scale_dtype)
  ldk = (cols + 15) // 16 * 16
  qbuf = _empty((1, rows, ldk), _CODE_TORCH[spec.qdtype], x.device)
  nview = None
  if noise is not None:
    if not isinstance(noise, torch.Tensor):
      noise = torch.as_tensor(np.asarray(noise), device=x.device)
    noise = noise.to(device=x.device, dtype=torch.float32).expand(
        tuple(x.shape)).contiguous()
    nop, nview, _, _ = _single_operand(noise.as_strided(
        x.shape, x.stride()) if noise.stride() == x.stride() else noise, shared)
    if (nview.row_stride, nview.col_stride) != (view.row_stride,
                                                view.col_stride):
      noise = torch.empty_strided(x.shape, x.stride(), dtype=torch.float32,
                                  device=x.device).copy_(noise)
      nop, nview, _, _ = _single_operand(noise, shared)
  lib = _lib.load()
  ws_bytes = lib.aqtb200_quantize_workspace_bytes(C.byref(view), C.byref(spec))
  ws = _empty(max(ws_bytes, 256), torch.uint8, x.device)
  rc = _call(lib.aqtb200_quantize, C.byref(view), None,
             C.byref(nview) if nview is not None else None,
             C.byref(spec), sin.data_ptr(), qbuf.data_ptr(),
             sin.data_ptr(), ws.data_ptr(), ws.numel(), _stream())
  _lib.check(rc, 'aqtb200_quantize')
  return _logical_q(qbuf, op, cols)


def apply_numerics(x, numerics, noise=None):
  """numerics.vjp_fwd on an already scaled tensor (unit scale)."""
  one = torch.ones([1] * x.ndim, dtype=x.dtype, device=x.device)
  return quantize_with_scale(x, one, numerics, noise)


def apply_inv_scales(x, scales):
  raise NotImplementedError(
      'QTensor.quant() as a stand-alone float op is not part of the sm_100a '
      'path; the multiply by 1/scale is fused into the quantize kernel '
      '(use Quantizer.quant / calculate_qvalue)')


def dequant(qvalue, scales, dequant_dtype):
  """QTensor.dequant on the device (zero or one scale)."""
  if len(scales) > 1:
    raise NotImplementedError('dequant with more than one scale')
  d_code = _code(dequant_dtype)
  out = _empty(qvalue.shape, _CODE_TORCH[d_code], qvalue.device)
  if not scales:
    return out.copy_(qvalue)
  scale = scales[0].expand(qvalue.shape)
  nd = qvalue.ndim
  if nd > 4:
    raise NotImplementedError('dequant of tensors with more than 4 axes')
  pad = [1] * (4 - nd)
  ext = pad + list(qvalue.shape)
  qs = [0] * (4 - nd) + list(qvalue.stride())
  ss = [0] * (4 - nd) + list(scale.stride())
  qv = _view(qvalue.data_ptr(), _code(qvalue.dtype), ext[:2], ext[2], ext[3],
             qs[:2], qs[2], qs[3])
  sv = _view(scale.data_ptr(), _code(scale.dtype), ext[:2], ext[2], ext[3],
             ss[:2], ss[2], ss[3])
  rc = _call(_lib.load().aqtb200_dequantize, C.byref(qv), C.byref(sv), d_code,
             out.data_ptr(), _stream())
  _lib.check(rc, 'aqtb200_dequantize')
  return out


# ---------------------------------------------------------------------------
# record once, replay many times


def _flat_tensors(x):
  if isinstance(x, torch.Tensor):
    return [x]
  if isinstance(x, (tuple, list)):
    return [t for e in x for t in _flat_tensors(e)]
  return []


class TracedStep:
  """A step function recorded once and replayed call by call.

  The reference runs under jax.jit: Python builds the computation once and
  every later step only launches it. This is the same idea at the level of
  the C ABI. `fn(*inputs)` is run with a tape open; every call it makes into
  the shared library (with its filled descriptors and buffer addresses) and
  every host action registered through tape_op() -- collectives, stream waits
  -- lands on the tape, and the buffers those calls point into are held.
  Calling the object replays the tape: the same kernels on the same buffers,
  for the cost of one foreign call each instead of the planner's work.

  Like a jitted function with donated buffers it is tied to the tensors it was
  traced with: the inputs must be the same tensors (new values are copied into
  them by the caller), the results are the same tensors every time. Anything
  the step does outside the library and tape_op() is NOT replayed; with
  `verify` (the default) the first replay is compared bit for bit with an
  eager run, so a step that cannot be traced is refused instead of silently
  going wrong.
  """

  def __init__(self, fn, *inputs, verify: bool = True):
    global _tape
    assert _tape is None, 'a step is already being traced'
    self._inputs = inputs
    self._stream = _stream()
    # copies: a step may hand out buffers it owns and overwrites on every run
    want = [t.clone() for t in _flat_tensors(fn(*inputs))] if verify else None
    _tape = tape = _Tape()
    try:
      self.outputs = fn(*inputs)
    finally:
      _tape = None
    self._tape = tape
    if verify:
      self()
      got = _flat_tensors(self.outputs)
      assert len(got) == len(want)
      for i, (a, b) in enumerate(zip(got, want)):
        same = a.shape == b.shape and a.dtype == b.dtype and torch.equal(
            a.contiguous().view(torch.uint8), b.contiguous().view(torch.uint8))
        if not same:
          raise _lib.AqtB200Error(
              f'TracedStep: result {i} of the replay differs from the eager '
              'run; the step does work outside the C ABI and tape_op()')

  @property
  def n_ops(self) -> int:
    return len(self._tape.ops)

  def __call__(self, *inputs):
    for a, b in zip(inputs, self._inputs):
      assert a is b or (isinstance(a, torch.Tensor) and a.data_ptr() ==
                        b.data_ptr() and a.shape == b.shape), (
          'a traced step runs on the tensors it was traced with')
    assert _stream() == self._stream, (
        'a traced step replays on the stream it was traced on')
    for fn, args in self._tape.ops:
      if args is None:
        fn()
      else:
        rc = fn(*args)
        if rc != 0:
          _lib.check(rc, 'replayed call')
    return self.outputs


# ---------------------------------------------------------------------------
# autograd bridge (the custom_vjp of aqt_dot_general.py:993-997)


def dg_core_autograd(cfg, lhs, rhs, lhs_qt, rhs_qt, dimension_numbers):
  from aqt_b200.v2 import aqt_dot_general as adg

  holder = []

  class _Fn(torch.autograd.Function):

    @staticmethod
    def forward(ctx, lhs_, rhs_):
      (out, qret), res = adg.dg_core_vjp_fwd(
          lhs_.detach(), rhs_.detach(), lhs_qt, rhs_qt, dimension_numbers, cfg)
      ctx.res = res
      holder.append(qret)
      return out

    @staticmethod
    def backward(ctx, g):
      dlhs, drhs, *_ = adg.dg_core_vjp_bwd(dimension_numbers, ctx.res,
                                           (g.contiguous(), None))
      return dlhs, drhs

  out = _Fn.apply(lhs, rhs)
  return out, holder[0]
