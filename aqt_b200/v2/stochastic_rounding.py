"""Noise functions for stochastic rounding.

Reference: aqt/jax/v2/stochastic_rounding.py:22-78. A NoiseFn maps
(shape, key) to an f32 tensor of U[-0.5, 0.5) noise that the int numerics add
before rounding. On this path the noise is an INPUT tensor of the quantize
kernel; these classes only produce it. The reference draws it from jax's
threefry generator, which is not available here, so the values differ from
jax's for the same key; pass a callable returning a prepared tensor when the
exact noise matters (that is what the parity tests do).

Keys are numpy uint32[2] arrays. `split` follows the threefry2x32 counter
construction so that sub-keys are decorrelated; it is not claimed to be
bit-identical to jax.random.split.
"""

from typing import Callable, Sequence

import numpy as np

from aqt_b200.v2 import utils

NoiseFn = Callable[..., object]

_ROT = ((13, 15, 26, 6), (17, 29, 16, 24))


def _rotl(x, r):
  return ((x << np.uint32(r)) | (x >> np.uint32(32 - r))).astype(np.uint32)


def threefry2x32(key, x0, x1):
  """Threefry-2x32, 20 rounds (Salmon et al., SC'11), vectorised over x0/x1."""
  k0, k1 = np.uint32(key[0]), np.uint32(key[1])
  ks = (k0, k1, np.uint32(k0 ^ k1 ^ np.uint32(0x1BD11BDA)))
  x0 = (np.asarray(x0, np.uint32) + ks[0]).astype(np.uint32)
  x1 = (np.asarray(x1, np.uint32) + ks[1]).astype(np.uint32)
  for block in range(5):
    for r in _ROT[block % 2]:
      x0 = (x0 + x1).astype(np.uint32)
      x1 = _rotl(x1, r) ^ x0
    x0 = (x0 + ks[(block + 1) % 3]).astype(np.uint32)
    x1 = (x1 + ks[(block + 2) % 3] + np.uint32(block + 1)).astype(np.uint32)
  return x0, x1


def PRNGKey(seed: int):
  seed = int(seed)
  return np.array([(seed >> 32) & 0xFFFFFFFF, seed & 0xFFFFFFFF], np.uint32)


def split(key, num: int = 2):
  """Derives `num` sub-keys from `key`."""
  with np.errstate(over='ignore'):
    a, b = threefry2x32(key, np.arange(num, dtype=np.uint32),
                        np.arange(num, 2 * num, dtype=np.uint32))
  return [np.array([a[i], b[i]], np.uint32) for i in range(num)]


def _degenerate_noise_shape(shape, noise_sharing_axes: Sequence[int] = ()):
  return tuple(1 if ax in noise_sharing_axes else n
               for ax, n in enumerate(shape))


def _device_uniform(shape, key):
  """U[0,1) f32 on the current CUDA device, seeded from the key."""
  import torch  # device memory plumbing only
  gen = torch.Generator(device='cuda')
  gen.manual_seed((int(key[0]) << 32) | int(key[1]))
  return torch.rand(shape, generator=gen, device='cuda', dtype=torch.float32)


@utils.flax_slots_kw_only_dataclass
class JaxUniform:
  """uniform(key, shape) - 0.5 (stochastic_rounding.py:35-46)."""

  def __call__(self, shape, key, noise_sharing_axes: Sequence[int] = ()):
    return _device_uniform(
        _degenerate_noise_shape(shape, noise_sharing_axes), key) - 0.5


@utils.flax_slots_kw_only_dataclass
class RandomCenteredUniform:
  """16 random bits placed in an f32 mantissa (stochastic_rounding.py:49-78).

  value = bitcast(0x3F800000 | bits16 << 7) - (1.5 - 2**-17), which is a grid
  of 65536 points centred on zero inside (-0.5, 0.5).
  """

  def __call__(self, shape, key, noise_sharing_axes: Sequence[int] = ()):
    import torch
    shape = _degenerate_noise_shape(shape, noise_sharing_axes)
    gen = torch.Generator(device='cuda')
    gen.manual_seed((int(key[0]) << 32) | int(key[1]))
    bits = torch.randint(0, 1 << 16, shape, generator=gen, device='cuda',
                         dtype=torch.int32)
    pattern = (bits << 7) | 0x3F800000
    return pattern.view(torch.float32) - (1.5 - 2.0 ** -17)
