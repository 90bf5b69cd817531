"""Pipelined host <-> device staging around a step of the quantized dot_general.

A caller whose operands live in pinned host memory (the situation the ctypes
and FFI bindings of include/aqt_b200.h meet when the framework above them has
not placed the arrays on the GPU) pays two PCIe transfers per step.  Issued on
one stream they serialise: copy in, compute, copy out.  `HostStepPipeline`
keeps three streams busy instead -- the upload of step i+1 and the download of
step i-1 run while step i computes -- with two sets of device input buffers.
Every step still uploads all of its inputs and downloads all of its results;
only the order in which the copy engines and the SMs see the work changes.

The arithmetic is untouched: `step_fn` is called with device tensors and its
results are copied out as they are.
"""

import collections

import torch


class HostStepPipeline:
  """Runs `step_fn(*device_inputs) -> tuple of device tensors` over host data.

  submit(host_inputs, host_outputs): enqueue one step.  `host_inputs` and
    `host_outputs` are sequences of pinned CPU tensors; outputs are filled
    asynchronously.
  drain(): block until every submitted step has landed in host memory.
  """

  def __init__(self, step_fn, device, depth: int = 2):
    assert depth >= 2
    self.step_fn = step_fn
    self.device = device
    self.depth = depth
    self.s_in = torch.cuda.Stream(device=device)
    self.s_out = torch.cuda.Stream(device=device)
    self._bufs = [None] * depth
    self._free = [None] * depth  # event: compute finished reading buffer set
    self._inflight = collections.deque()  # (event, device results kept alive)
    self._n = 0

  def _buffers(self, slot, host_inputs):
    bufs = self._bufs[slot]
    if bufs is None or any(
        b.shape != h.shape or b.dtype != h.dtype
        for b, h in zip(bufs, host_inputs)) or len(bufs) != len(host_inputs):
      with torch.cuda.stream(self.s_in):
        bufs = [torch.empty(h.shape, dtype=h.dtype, device=self.device)
                for h in host_inputs]
      self._bufs[slot] = bufs
    return bufs

  def submit(self, host_inputs, host_outputs):
    for h in list(host_inputs) + list(host_outputs):
      if not h.is_pinned():
        raise ValueError('HostStepPipeline needs pinned host tensors')
    slot = self._n % self.depth
    compute = torch.cuda.current_stream(self.device)
    bufs = self._buffers(slot, host_inputs)
    if self._free[slot] is not None:
      self.s_in.wait_event(self._free[slot])
    with torch.cuda.stream(self.s_in):
      for b, h in zip(bufs, host_inputs):
        b.copy_(h, non_blocking=True)
      uploaded = torch.cuda.Event()
      uploaded.record(self.s_in)
    compute.wait_event(uploaded)
    res = self.step_fn(*bufs)
    if isinstance(res, torch.Tensor):
      res = (res,)
    computed = torch.cuda.Event()
    computed.record(compute)
    self._free[slot] = computed
    if len(res) != len(host_outputs):
      raise ValueError(f'{len(res)} results for {len(host_outputs)} host buffers')
    self.s_out.wait_event(computed)
    with torch.cuda.stream(self.s_out):
      for dst, src in zip(host_outputs, res):
        dst.copy_(src, non_blocking=True)
      landed = torch.cuda.Event()
      landed.record(self.s_out)
    # The results were allocated on the compute stream and are read on s_out:
    # hold them until that copy is done, then let the allocator reuse them.
    self._inflight.append((landed, res))
    while len(self._inflight) > self.depth:
      ev, _ = self._inflight.popleft()
      ev.synchronize()
    self._n += 1

  def drain(self):
    while self._inflight:
      ev, _ = self._inflight.popleft()
      ev.synchronize()
    compute = torch.cuda.current_stream(self.device)
    compute.wait_stream(self.s_out)
    compute.wait_stream(self.s_in)
