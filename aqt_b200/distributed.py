"""Row-sharded execution of one quantized dot_general as ONE logical op.

The rows of lhs (and of the cotangent) are split over the ranks of a
torch.distributed group; rhs (the weights) is replicated. The result equals,
rank by rank, the rows a single device would have produced for the
concatenated lhs -- bit for bit for int8, to f32 summation order for fp8:

  * scales that do not span the sharded axis (per-row) stay local;
  * scales that do (per-tensor; every scale of drhs, whose contraction runs
    over the sharded rows) are computed locally, max-all-reduced, and handed
    to the dot through the reference's own "incomplete QTensor" input
    (aqt_dot_general.py:645-653). The scale is a monotone function of the
    absolute maximum, so max(scale_r) == scale(max_r amax);
  * drhs sums raw int32 / f32 accumulators across ranks before the single
    dequantizing epilogue. Where both operands are already quantized (the
    one-read flow) the sum is a reduce-scatter: every rank receives the total
    of its band of drhs rows only, dequantizes that band, and an all-gather
    of the finished (bf16 / f32) bands completes the result -- fewer bytes on
    the links than an all-reduce of the accumulators and 1/N of the
    dequantizing traffic per rank. drhs is produced in row slices so that
    the exchange of one slice runs under the next slice's GEMM and under
    dlhs. Otherwise the accumulators are all-reduced and dequantized whole.

On GPUs of one node the three steps of that exchange are ONE kernel over peer
memory (aqtb200_dot_general_raw_exchange): the accumulators and the result
live in a device allocation whose handle every rank opens; after a small
collective that tells a slice's GEMM has finished everywhere, each rank reads
its band of the slice from every rank's accumulators, adds them in rank
order, dequantizes once and writes the band into every rank's result. The
kernel runs on a second stream beside the next slice's GEMM and beside dlhs.
Where peer mappings cannot be made (host tensors, other world sizes than 2, 4
or 8, no peer access) the NCCL calls above are used instead.

Only a 2-D contraction lhs[M,K] . rhs[K,N] is handled; that is the projection
layer the reference's data-parallel users shard. The reference itself has no
collective on this path (cross-replica statistics raise NotImplementedError,
flax/aqt_flax_calibration.py:161-164).

Every collective and stream dependency is issued through engine.tape_op, so a
sharded step can be recorded and replayed by engine.TracedStep.
"""

from __future__ import annotations

import ctypes as C
import functools

import torch
import torch.distributed as dist

from aqt_b200 import _lib
from aqt_b200 import engine
from aqt_b200.v2 import aqt_dot_general as adg
from aqt_b200.v2 import aqt_tensor
from aqt_b200.v2 import utils

_DIMS_2D = (((1,), (0,)), ((), ()))


def _calib_kwargs(quantizer):
  cal = quantizer.calibration
  kw = dict(cal.keywords) if isinstance(cal, functools.partial) else {}
  return kw


class _StreamCtx:
  """`with` block that makes `stream` current (a no-op for stream None)."""

  def __init__(self, stream):
    self._ctx = torch.cuda.stream(stream) if stream is not None else None

  def __enter__(self):
    if self._ctx is not None:
      self._ctx.__enter__()

  def __exit__(self, *exc):
    if self._ctx is not None:
      self._ctx.__exit__(*exc)


class _DeviceMemory:
  """Zero-copy torch view of a device allocation made outside torch."""

  def __init__(self, ptr, nbytes):
    self.__cuda_array_interface__ = {
        'shape': (nbytes,), 'typestr': '|u1', 'data': (ptr, False),
        'version': 2, 'strides': None}


class PeerBuffers:
  """The accumulators [K][N] (4-byte) and the result [K][N] of a sharded drhs
  in one device allocation per rank that every other rank of the group has
  mapped. acc / out are this rank's torch views; acc_base[r] / out_base[r]
  the addresses of rank r's copies as seen from this rank."""

  def __init__(self, group, device, k, n, acc_dtype, out_dtype):
    lib = _lib.load()
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    acc_bytes = (k * n * 4 + 255) // 256 * 256
    out_bytes = k * n * torch.empty((), dtype=out_dtype).element_size()
    self._own = C.c_void_p()
    self._opened = []
    self._lib = lib
    ok = 1
    handle = C.create_string_buffer(64)
    try:
      _lib.check(lib.aqtb200_dev_alloc(C.byref(self._own), acc_bytes + out_bytes),
                 'dev_alloc')
      _lib.check(lib.aqtb200_ipc_export(self._own, handle), 'ipc_export')
    except Exception:  # pylint: disable=broad-except
      ok = 0
    gathered = [None] * world
    dist.all_gather_object(gathered, (ok, handle.raw), group=group)
    bases = [None] * world
    if all(g[0] for g in gathered):
      try:
        for r, (_, raw) in enumerate(gathered):
          if r == rank:
            bases[r] = self._own.value
            continue
          ptr = C.c_void_p()
          _lib.check(lib.aqtb200_ipc_open(C.create_string_buffer(raw, 64),
                                          C.byref(ptr)), 'ipc_open')
          self._opened.append(ptr)
          bases[r] = ptr.value
      except Exception:  # pylint: disable=broad-except
        ok = 0
    else:
      ok = 0
    if ok:
      try:
        # this rank's views of its own allocation (zero-copy)
        mem = torch.as_tensor(
            _DeviceMemory(self._own.value, acc_bytes + out_bytes), device=device)
        self._mem = mem
        self.acc = mem[:k * n * 4].view(acc_dtype).view(k, n)
        self.out = mem[acc_bytes:acc_bytes + out_bytes].view(out_dtype).view(k, n)
        assert self.acc.data_ptr() == self._own.value
      except Exception:  # pylint: disable=broad-except
        ok = 0
    # every rank takes the same path: all of them made it, or none uses it
    flag = torch.tensor([ok], device=device, dtype=torch.int32)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
    self.ok = bool(int(flag.item()))
    if not self.ok:
      self.close()
      return
    self.acc_base = bases
    self.out_base = [b + acc_bytes for b in bases]

  def close(self):
    for ptr in self._opened:
      self._lib.aqtb200_ipc_close(ptr)
    self._opened = []
    if self._own:
      self._lib.aqtb200_dev_free(self._own)
      self._own = C.c_void_p()


class ShardedDotGeneral:
  """cfg.vjp for row-sharded operands (see module docstring)."""

  def __init__(self, cfg: adg.DotGeneral, group=None, overlap_sms: int = 16,
               drhs_slices: int = 2, slice_multiple: int = 256,
               exchange: str = 'auto'):
    self.cfg = cfg
    self.group = group
    # 'auto': the fused kernel over peer memory where it can be set up, else
    # NCCL reduce-scatter + all-gather; 'nccl': always the latter.
    assert exchange in ('auto', 'nccl')
    self.exchange = exchange
    self._peer = {}
    self.exchange_used = None  # 'p2p' or 'nccl' once a sliced drhs has run
    # SMs left to the exchange while a GEMM runs beside it (measured at two
    # ranks, 8192^3: 12 -> 1.55 ms per step, 16 -> 1.46, 24 -> 1.50, 32 -> 1.50).
    self.overlap_sms = overlap_sms
    # drhs is computed in this many row slices so that the exchange of one
    # slice's accumulators runs under the next slice's GEMM.
    self.drhs_slices = drhs_slices
    # a slice is a whole number of GEMM tile rows
    self.slice_multiple = slice_multiple
    self._side = {}

  # -- plumbing ----------------------------------------------------------------
  def _world(self):
    if not dist.is_initialized():
      return 1
    return dist.get_world_size(self.group)

  def _side_stream(self, device):
    """A second stream per device for the dequantize-and-gather half of the
    drhs exchange (None for host tensors, which have no streams)."""
    if device.type != 'cuda':
      return None
    key = str(device)
    if key not in self._side:
      self._side[key] = torch.cuda.Stream(device=device)
    return self._side[key]

  # -- collectives -----------------------------------------------------------
  def _max(self, t):
    if self._world() > 1:
      engine.tape_op(lambda: dist.all_reduce(t, op=dist.ReduceOp.MAX,
                                             group=self.group))
    return t

  def _max_async(self, t):
    """Starts a max-all-reduce of t in place; returns (t, wait) or t."""
    if self._world() > 1:
      box = {}

      def start():
        box['w'] = dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group,
                                   async_op=True)

      engine.tape_op(start)
      return t, lambda: engine.tape_op(lambda: box['w'].wait())
    return t

  def _sum_async(self, t):
    """Starts a sum-all-reduce of t in place; returns a wait callable or None."""
    if self._world() > 1:
      box = {}

      def start():
        box['w'] = dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group,
                                   async_op=True)

      engine.tape_op(start)
      return lambda: engine.tape_op(lambda: box['w'].wait())
    return None

  # -- scales ------------------------------------------------------------------
  def _global_scale(self, quantizer, x, contraction_axes, sharded_axis,
                    prescale=None, compute_dtype=None):
    """Incomplete QTensor with a cross-rank scale, or None if scales are local."""
    if type(quantizer.numerics).__name__ == 'NoNumerics':
      return None
    per_tensor = quantizer.calib_shared_axes == 'per_tensor'
    shared = list(range(x.ndim)) if per_tensor else list(contraction_axes)
    if sharded_axis not in shared:
      return None
    kw = _calib_kwargs(quantizer)
    scale = engine.absmax_scale(
        x, shared, quantizer.numerics,
        scale_dtype=kw.get('dtype', quantizer.scale_dtype),
        clipping_scale=kw.get('clipping_scale'),
        po2_scale=kw.get('po2_scale', False), prescale=prescale,
        compute_dtype=compute_dtype)
    scale = self._max(scale.contiguous())
    dd = compute_dtype if compute_dtype is not None else utils.as_dtype(x.dtype)
    return aqt_tensor.QTensor(qvalue=None, scale=[scale], scale_t=None,
                              bias=[], dequant_dtype=dd)

  # -- forward / backward ------------------------------------------------------
  def vjp(self, lhs, rhs, dimension_numbers=_DIMS_2D):
    dims = adg._canon_dims(dimension_numbers)  # pylint: disable=protected-access
    if dims != _DIMS_2D or lhs.ndim != 2 or rhs.ndim != 2:
      raise NotImplementedError(
          'ShardedDotGeneral handles lhs[M,K] . rhs[K,N] with M sharded')
    cfg = self.cfg
    cfg.assert_config_validity()
    for raw in (cfg.fwd, cfg.dlhs, cfg.drhs):
      adg._init_calibration_once(raw.dg_quantizer)  # pylint: disable=protected-access
    # Per-tensor fp8 matmuls: each operand is read once for its forward and
    # backward copies; lhs's maximum is agreed across ranks first, which fixes
    # every scale of lhs on every rank without a further collective.
    pre = engine.prequantize_for_training(cfg, lhs, rhs, dims,
                                          reduce_max_lhs=self._max_async)
    if pre is not None:
      out, res = engine.dg_raw(cfg.fwd, lhs, rhs, pre[0], pre[1], dims,
                               internal_qt=True)
    else:
      lhs_qt = self._global_scale(cfg.fwd.dg_quantizer.lhs, lhs, [1], 0)
      out, res = engine.dg_raw(cfg.fwd, lhs, rhs, lhs_qt, None, dims)
    out = out.to(lhs.dtype)

    def backprop(g):
      return self._bwd(dims, res, g)

    return out, backprop

  def _other_operand(self, raw, mt):
    """(tensor the raw dot quantizes, forward scale to fold into g, dtype)."""
    if raw.rhs.use_fwd_quant:
      return mt.qx.qvalue, mt.qx.scale[0], mt.qx.dequant_dtype
    return mt.x, None, None

  def _bwd(self, dims, res, g):
    cfg = self.cfg
    upd = adg._update_dimension_numbers_for_backward  # pylint: disable=protected-access

    # drhs = g[M,N]^T . lhs'[M,K] : contraction over the sharded rows. It runs
    # first so that the exchange of its accumulators overlaps with dlhs.
    r_dims, r_perm = upd(dims, True, g.ndim, res.lhs.mt.x.ndim)
    other, fwd_scale, other_dt = self._other_operand(cfg.drhs, res.lhs.mt)
    pre = None
    if fwd_scale is not None:
      # lhs scale [M,1] (or a scalar) varies along g's contraction axis M
      pre = fwd_scale.reshape(-1, 1) if fwd_scale.numel() > 1 else (
          fwd_scale.reshape(1, 1))
    # Per-tensor scales everywhere: one pass over g and one max-all-reduce give
    # the cotangent's scale for both gradient dots.
    shared, pair = None, None
    try:
      # one read of the cotangent for both of its copies where that applies
      pair = engine.cotangent_pair(cfg, res, g, reduce_max=self._max)
      if pair is None:
        shared = engine.shared_cotangent_scales(cfg, res, g,
                                                reduce_max=self._max)
    except NotImplementedError:
      shared = None
    if pair is not None:
      shared = pair
    d_dims, d_perm = upd(dims, False, g.ndim, res.rhs.mt.x.ndim)
    if shared is not None:
      g_qt_dlhs, g_qt = shared
    else:
      g_qt = self._global_scale(cfg.drhs.dg_quantizer.lhs, g, [0], 0,
                                prescale=pre)
      # Every cross-rank scale is agreed on BEFORE the big exchange starts:
      # a small collective queued behind it on the same communicator would
      # wait for it and serialise the dlhs pass after it.
      _, fwd_scale_r, _ = self._other_operand(cfg.dlhs, res.rhs.mt)
      pre_r = None
      if fwd_scale_r is not None:
        # rhs scale [1,N] laid along g's [M,N]: constant along the kept axis M
        pre_r = fwd_scale_r.reshape(1, -1) if fwd_scale_r.numel() > 1 else (
            fwd_scale_r.reshape(1, 1))
      g_qt_dlhs = self._global_scale(cfg.dlhs.dg_quantizer.lhs, g, [1], 0,
                                     prescale=pre_r)
    # The stored operands' backward copies from the forward pass, when they exist.
    x_qt = engine.bwd_copy(res.lhs.mt.qx) if cfg.drhs.rhs.use_fwd_quant else None
    y_qt = engine.bwd_copy(res.rhs.mt.qx) if cfg.dlhs.rhs.use_fwd_quant else None
    internal = pair is not None or x_qt is not None or y_qt is not None
    if x_qt is None:
      x_qt = self._global_scale(cfg.drhs.dg_quantizer.rhs, other, [0], 0,
                                compute_dtype=other_dt)

    deferred, wait, drhs = None, None, None
    sliced = self._drhs_sliced(g, res, g_qt, x_qt, r_dims, r_perm, internal)
    if sliced is not None:
      pass
    elif g_qt is None and x_qt is None:  # unquantized gradient dot
      drhs = engine.dg_raw(cfg.drhs, g, res.lhs.mt, None, None, r_dims,
                           out_transpose_axes=r_perm)[0].contiguous()
      wait = self._sum_async(drhs)
    else:
      deferred, _ = engine.dg_raw(cfg.drhs, g, res.lhs.mt, g_qt, x_qt, r_dims,
                                  out_transpose_axes=r_perm,
                                  defer_dequant=True, internal_qt=internal)
      wait = self._sum_async(deferred.acc)
    overlapped = sliced is not None or wait is not None

    # dlhs = g[M,N] . rhs'[K,N]^T : rows of g sharded, contraction over N local
    if overlapped and self.overlap_sms:
      engine.set_gemm_sm_budget(max(engine.sm_count() - self.overlap_sms, 2))
    try:
      dlhs = engine.dg_raw(cfg.dlhs, g, res.rhs.mt, g_qt_dlhs, y_qt, d_dims,
                           out_transpose_axes=d_perm, internal_qt=internal)[0]
    finally:
      if overlapped and self.overlap_sms:
        engine.set_gemm_sm_budget(0)

    if sliced is not None:
      drhs, join = sliced
      join()
      return dlhs, drhs
    if wait is not None:
      wait()
    if deferred is not None:
      drhs = deferred.finish()
    return dlhs, drhs

  def _drhs_sliced(self, g, res, g_qt, x_qt, r_dims, r_perm, internal):
    """drhs in row slices; per slice: GEMM into raw accumulators, reduce-scatter
    of the accumulators, dequantization of this rank's band, all-gather of the
    finished bands. The reduce-scatter is issued from the compute stream right
    behind its GEMM; the dequantization and the all-gather run on a second
    stream, so the compute stream goes straight on to the next slice's GEMM.
    Needs both operands already quantized (full QTensors), so that a slice
    costs one GEMM and nothing else. Returns (drhs, join) or None; join()
    makes the compute stream wait for the whole exchange."""
    s = self.drhs_slices
    world = self._world()
    if not (s and s >= 1 and world > 1 and g_qt is not None and
            x_qt is not None and g_qt.is_full() and x_qt.is_full()):
      return None
    k = res.lhs.mt.x.shape[1]
    n = g.shape[1]
    if k % (s * world) != 0 or (k // s) % self.slice_multiple != 0 or n % 4:
      return None
    cfg = self.cfg
    rank = dist.get_rank(self.group)
    rows = k // s
    band = rows // world
    peer = self._peer_buffers(g, k, n, x_qt)
    if peer is not None:
      self.exchange_used = 'p2p'
      return self._drhs_fused(g, res, g_qt, x_qt, r_dims, r_perm, internal,
                              peer, rows, band, rank)
    self.exchange_used = 'nccl'
    drhs = engine._empty((k, n), g.dtype, g.device)  # pylint: disable=protected-access
    side = self._side_stream(g.device)
    mt = res.lhs.mt
    keep, gathers = [], []
    budget = self.overlap_sms
    try:
      for i in range(s):
        sl = slice(i * rows, (i + 1) * rows)
        mt_i = adg.MultiTensor(
            x=mt.x[:, sl], qx=mt.qx.replace(qvalue=mt.qx.qvalue[:, sl]))
        x_i = x_qt.replace(qvalue=x_qt.qvalue[:, sl])
        if i == 1 and budget:
          # from the second slice on a collective is in flight beside the GEMM
          engine.set_gemm_sm_budget(max(engine.sm_count() - budget, 2))
        d, _ = engine.dg_raw(cfg.drhs, g, mt_i, g_qt, x_i, r_dims,
                             out_transpose_axes=r_perm, defer_dequant=True,
                             internal_qt=internal, out=drhs[sl])
        acc = d.acc.reshape(rows, n)
        assert acc.is_contiguous() and acc.data_ptr() == d.acc.data_ptr(), (
            'drhs accumulators are expected as [rows of drhs][columns]')
        mine = engine._empty((band, n), acc.dtype, g.device)  # pylint: disable=protected-access
        keep += [d, acc, mine]
        box = {}

        def scatter(box=box, mine=mine, acc=acc):
          box['rs'] = dist.reduce_scatter_tensor(
              mine, acc, op=dist.ReduceOp.SUM, group=self.group, async_op=True)

        engine.tape_op(scatter)

        def wait_scatter(box=box):
          with _StreamCtx(side):
            box['rs'].wait()

        engine.tape_op(wait_scatter)
        with _StreamCtx(side):
          d.finish_rows(rank * band, band, mine)
        out_i = drhs[sl]

        def gather(box=box, out_i=out_i):
          with _StreamCtx(side):
            box['ag'] = dist.all_gather_into_tensor(
                out_i, out_i[rank * band:(rank + 1) * band], group=self.group,
                async_op=True)

        engine.tape_op(gather)
        gathers.append(box)
    finally:
      if budget:
        engine.set_gemm_sm_budget(0)

    def join():
      for box in gathers:
        engine.tape_op(lambda box=box: box['ag'].wait())
      del keep[:]

    return drhs, join

  # -- the exchange as one kernel over peer memory ---------------------------
  def _peer_buffers(self, g, k, n, x_qt):
    """PeerBuffers for a [k][n] drhs, or None where the NCCL path applies."""
    world = self._world()
    if (self.exchange != 'auto' or g.device.type != 'cuda' or
        world not in (2, 4, 8) or n % 4):
      return None
    ints = x_qt.qvalue.dtype == torch.int8
    key = (k, n, g.dtype, ints, str(g.device))
    if key not in self._peer:
      try:
        pb = PeerBuffers(self.group, g.device, k, n,
                         torch.int32 if ints else torch.float32, g.dtype)
      except Exception:  # pylint: disable=broad-except
        # every rank must take the same path: agree on the failure
        flag = torch.tensor([0], device=g.device, dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
        pb = None
      self._peer[key] = pb if (pb is not None and pb.ok) else None
      self._flag = torch.zeros(1, device=g.device, dtype=torch.int32)
    return self._peer[key]

  def _barrier_on(self, stream):
    """Orders everything queued on `stream` after what every rank had queued
    on its own when it got here (a one-element all-reduce)."""
    flag = self._flag

    def op():
      with _StreamCtx(stream):
        dist.all_reduce(flag, group=self.group)

    engine.tape_op(op)

  def _drhs_fused(self, g, res, g_qt, x_qt, r_dims, r_perm, internal, peer,
                  rows, band, rank):
    """drhs in row slices: GEMM into the shared accumulators on the compute
    stream; on the second stream a barrier and the kernel that sums this
    rank's band of the slice over all ranks, dequantizes it and writes it to
    every rank. Returns (drhs, join); drhs is the shared result buffer, valid
    until this op's next backward pass."""
    cfg = self.cfg
    s = self.drhs_slices
    n = g.shape[1]
    side = self._side_stream(g.device)
    main = torch.cuda.current_stream(g.device)
    mt = res.lhs.mt
    budget = self.overlap_sms
    try:
      for i in range(s):
        sl = slice(i * rows, (i + 1) * rows)
        mt_i = adg.MultiTensor(
            x=mt.x[:, sl], qx=mt.qx.replace(qvalue=mt.qx.qvalue[:, sl]))
        x_i = x_qt.replace(qvalue=x_qt.qvalue[:, sl])
        if i == 1 and budget:
          engine.set_gemm_sm_budget(max(engine.sm_count() - budget, 2))
        d, _ = engine.dg_raw(cfg.drhs, g, mt_i, g_qt, x_i, r_dims,
                             out_transpose_axes=r_perm, defer_dequant=True,
                             internal_qt=internal, out=peer.out[sl],
                             acc_buf=peer.acc[sl])
        assert d.acc.data_ptr() == peer.acc[sl].data_ptr()
        acc_row, out_row = d.band_stride_bytes()
        assert acc_row == 4 * n and out_row == n * peer.out.element_size(), (
            'drhs accumulators are expected as [rows of drhs][columns]')
        first = i * rows + rank * band
        engine.tape_op(lambda: side.wait_stream(main))
        self._barrier_on(side)
        with _StreamCtx(side):
          d.exchange_rows(
              rank * band, band, rank,
              [b + first * acc_row for b in peer.acc_base],
              [b + first * out_row for b in peer.out_base],
              max_sms=budget if budget else 0)
    finally:
      if budget:
        engine.set_gemm_sm_budget(0)

    def join():
      # every rank's bands have landed here once every rank's kernels are done
      self._barrier_on(side)
      engine.tape_op(lambda: main.wait_stream(side))

    return peer.out, join
