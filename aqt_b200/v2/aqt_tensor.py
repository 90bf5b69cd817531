"""QTensor: a quantized value with the scales that undo it.

Reference: aqt/jax/v2/aqt_tensor.py:54-200 (fields, quant :125-159, dequant
:161-200). The KV-cache slicing helpers of the reference (:258-422) are not on
the dot_general path and are not provided.

Device layout. `qvalue` and the entries of `scale` are torch CUDA tensors whose
*logical* shape is the reference's (qvalue like the operand, scale with the
shared axes collapsed to 1) but whose strides are whatever the producing kernel
wrote: the quantize kernel stores qvalues with the contraction index
contiguous (the layout tcgen05 operand tiles want), so for an operand whose
contraction axis is not its last axis `qvalue` is a transposed view of that
buffer. Consumers go through strides; nothing is copied to "fix" a layout.
"""

from typing import Any, Callable

from aqt_b200.v2 import utils

GradientFn = None | Callable[..., Any]

_MSG_NO_QVALUE = (
    'QTensor does not have qvalue, but it is asked to access the qvalue.'
    ' Call QTensor.quant() before using the qvalue.')


@utils.flax_slots_kw_only_dataclass
class QTensor:
  """Quantized tensor plus quantization parameters."""

  # Quantized value (int8 / fp8 container, or the float input for NoNumerics).
  qvalue: Any
  # Scales: dequant(q) = q * prod(scale); each has the operand's rank.
  scale: None | list
  # Legacy transposed scales; kept for API parity, unused on this path.
  scale_t: None | list
  # Biases; only fake-quant mode supports them in the reference, and the
  # device path supports none.
  bias: list = utils.dynamic_field(default_factory=list)
  # dtype dequant() returns.
  dequant_dtype: None | Any = utils.static_field(default=None)
  sparsity_mask: Any = utils.dynamic_field(default=None)
  tiling_state: Any = utils.static_field(default=None)

  @property
  def shape(self):
    assert self.is_full(), _MSG_NO_QVALUE
    return tuple(self.qvalue.shape)

  @property
  def ndim(self) -> int:
    assert self.is_full(), _MSG_NO_QVALUE
    return self.qvalue.ndim

  def is_full(self) -> bool:
    return self.qvalue is not None

  def replace(self, **changes) -> 'QTensor':
    import dataclasses
    return dataclasses.replace(self, **changes)

  def without_qvalue(self) -> 'QTensor':
    return self.replace(qvalue=None)

  def astype(self, dtype) -> 'QTensor':
    return self.replace(dequant_dtype=dtype)

  def quant(self, x) -> 'QTensor':
    """x * (1/scale) per scale, as a float tensor (aqt_tensor.py:125-159)."""
    from aqt_b200 import engine
    assert not self.is_full(), 'Already quantized QTensor.'
    assert self.scale is not None, 'Missing scales to be used for quantization.'
    assert isinstance(self.scale, list), (
        f'QTensor.scale must be a list of arrays, but got {self.scale}')
    assert isinstance(self.bias, list), (
        f'QTensor.bias must be a list of arrays, but got {self.bias}')
    if self.bias or self.sparsity_mask is not None or self.tiling_state:
      raise NotImplementedError(
          'bias / sparsity / tiling are outside the sm_100a hot path')
    return self.replace(qvalue=engine.apply_inv_scales(x, self.scale))

  def dequant(self):
    """qvalue.astype(dequant_dtype) * scales (aqt_tensor.py:161-200)."""
    from aqt_b200 import engine
    assert self.scale is not None, 'Missing scales when dequantizing a QTensor.'
    assert isinstance(self.scale, list)
    assert isinstance(self.bias, list)
    assert self.dequant_dtype is not None, (
        'QTensor is manually created without setting a dequant_dtype. It can'
        ' be used in dot_general, but to dequantize you need to set its dtype.')
    assert self.is_full(), _MSG_NO_QVALUE
    if self.bias or self.sparsity_mask is not None or self.tiling_state:
      raise NotImplementedError(
          'bias / sparsity / tiling are outside the sm_100a hot path')
    return engine.dequant(self.qvalue, self.scale, self.dequant_dtype)

  def qvalue_astype(self, dtype) -> 'QTensor':
    assert self.is_full(), _MSG_NO_QVALUE
    return self.replace(qvalue=self.qvalue.to(dtype))
