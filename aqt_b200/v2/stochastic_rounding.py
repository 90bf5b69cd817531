"""Noise functions for stochastic rounding.

Reference: aqt/jax/v2/stochastic_rounding.py:22-78. A NoiseFn maps
(shape, key) to an f32 tensor of U[-0.5, 0.5) noise that the int numerics add
before rounding. On this path the noise is an INPUT tensor of the quantize
kernel; these classes produce it on the device (aqtb200_jax_noise), and this
module holds the same generator in numpy as its host-side statement.

The reference draws from jax.random. jax is not part of the reference tree
and is not installed here, so its generator is restated from the published
algorithm: Threefry-2x32 with 20 rounds (Salmon et al., SC'11; checked against
the Random123 known answers in the tests) and jax's layout of counters over
an array, of which there are two:

  original (jax_threefry_partitionable=False, the default before jax 0.5):
    counts = iota(n) is cut into a first and a second half (a zero pads an odd
    n), x0 = first, x1 = second; the result is concat(y0, y1)[:n];
  partitionable (the default from jax 0.5 on):
    element i uses the counter pair (hi32(i), lo32(i)); the result is y0 ^ y1.

`PARTITIONABLE` selects between them for everything below. Equality with an
actual jax installation could not be checked on this machine: parity with
jax.random is unpinned.

Keys are numpy uint32[2] arrays (jax's raw threefry key data).
"""

from typing import Callable, Sequence

import numpy as np

from aqt_b200.v2 import utils

NoiseFn = Callable[..., object]

# jax_threefry_partitionable of the jax version being matched.
PARTITIONABLE = False

_ROT = ((13, 15, 26, 6), (17, 29, 16, 24))


def _rotl(x, r):
  return ((x << np.uint32(r)) | (x >> np.uint32(32 - r))).astype(np.uint32)


def threefry2x32(key, x0, x1):
  """Threefry-2x32, 20 rounds (Salmon et al., SC'11), vectorised over x0/x1."""
  k0, k1 = np.uint32(key[0]), np.uint32(key[1])
  ks = (k0, k1, np.uint32(k0 ^ k1 ^ np.uint32(0x1BD11BDA)))
  with np.errstate(over='ignore'):
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


def _words(key, n: int, partitionable: bool):
  """n 32-bit draws laid out as jax lays them over iota(n)."""
  if n == 0:
    return np.zeros(0, np.uint32)
  if partitionable:
    i = np.arange(n, dtype=np.uint64)
    y0, y1 = threefry2x32(key, (i >> np.uint64(32)).astype(np.uint32),
                          i.astype(np.uint32))
    return y0 ^ y1
  half = (n + 1) // 2
  counts = np.arange(2 * half, dtype=np.uint32)
  counts[n:] = 0  # the pad of an odd count
  y0, y1 = threefry2x32(key, counts[:half], counts[half:])
  return np.concatenate([y0, y1])[:n]


def split(key, num: int = 2, partitionable=None):
  """jax.random.split: `num` sub-keys of `key` (config.py:61-90 uses it to give
  every quantizer of a DotGeneral its own key)."""
  part = PARTITIONABLE if partitionable is None else partitionable
  if part:
    y0, y1 = threefry2x32(key, np.zeros(num, np.uint32),
                          np.arange(num, dtype=np.uint32))
    return [np.array([y0[i], y1[i]], np.uint32) for i in range(num)]
  w = _words(key, 2 * num, False).reshape(num, 2)
  return [np.array(w[i], np.uint32) for i in range(num)]


def random_bits(key, shape, bit_width: int = 32, partitionable=None):
  """jax.random.bits(key, shape, uint32 | uint16) as a numpy array."""
  part = PARTITIONABLE if partitionable is None else partitionable
  n = int(np.prod(shape, dtype=np.int64)) if len(shape) else 1
  if bit_width == 32:
    return _words(key, n, part).reshape(shape)
  assert bit_width == 16
  if part:
    return (_words(key, n, True) & np.uint32(0xFFFF)).astype(np.uint16).reshape(
        shape)
  w = _words(key, (n + 1) // 2, False)
  halves = np.stack([w & np.uint32(0xFFFF), w >> np.uint32(16)], axis=1)
  return halves.reshape(-1)[:n].astype(np.uint16).reshape(shape)


def uniform(key, shape, partitionable=None):
  """jax.random.uniform(key, shape) in [0, 1), float32."""
  bits = random_bits(key, shape, 32, partitionable)
  f = ((bits >> np.uint32(9)) | np.uint32(0x3F800000)).view(np.float32)
  return np.maximum(np.float32(0), f - np.float32(1))


def centered_uniform16(key, shape, partitionable=None):
  """RandomCenteredUniform's values (stochastic_rounding.py:49-78)."""
  bits = random_bits(key, shape, 16, partitionable).astype(np.uint32)
  f = ((bits << np.uint32(7)) | np.uint32(0x3F800000)).view(np.float32)
  return f - np.float32(1.5 - 2.0 ** -17)


def _degenerate_noise_shape(shape, noise_sharing_axes: Sequence[int] = ()):
  return tuple(1 if ax in noise_sharing_axes else n
               for ax, n in enumerate(shape))


def _device_noise(shape, key, kind: int, shift: float):
  """The same draws on the current CUDA device (aqtb200_jax_noise)."""
  import torch  # device memory plumbing only
  from aqt_b200 import _lib
  n = int(np.prod(shape, dtype=np.int64)) if len(shape) else 1
  out = torch.empty(tuple(shape), dtype=torch.float32, device='cuda')
  rc = _lib.load().aqtb200_jax_noise(
      int(key[0]), int(key[1]), n, kind, 1 if PARTITIONABLE else 0,
      float(shift), out.data_ptr(), torch.cuda.current_stream().cuda_stream)
  _lib.check(rc, 'aqtb200_jax_noise')
  return out


@utils.flax_slots_kw_only_dataclass
class JaxUniform:
  """uniform(key, shape) - 0.5 (stochastic_rounding.py:35-46)."""

  def __call__(self, shape, key, noise_sharing_axes: Sequence[int] = ()):
    return _device_noise(_degenerate_noise_shape(shape, noise_sharing_axes),
                         key, 0, 0.5)


@utils.flax_slots_kw_only_dataclass
class RandomCenteredUniform:
  """16 random bits placed in an f32 mantissa (stochastic_rounding.py:49-78).

  value = bitcast(0x3F800000 | bits16 << 7) - (1.5 - 2**-17), which is a grid
  of 65536 points centred on zero inside (-0.5, 0.5).
  """

  def __call__(self, shape, key, noise_sharing_axes: Sequence[int] = ()):
    return _device_noise(_degenerate_noise_shape(shape, noise_sharing_axes),
                         key, 1, 0.0)
