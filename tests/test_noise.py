"""The jax.random restatement behind the stochastic-rounding noise functions.

Threefry-2x32 is pinned to the Random123 known-answer vectors (the generator
jax.random is built on). jax's layout of counters over an array is restated
from its published source and checked here only for the properties that follow
from that description; equality with a jax installation is unpinned (jax is
not installed).
"""

import numpy as np
import pytest

from aqt_b200.v2 import stochastic_rounding as sr


def test_threefry2x32_known_answers():
  # Random123 kat_vectors, threefry2x32 with 20 rounds: counter, key -> output
  cases = [
      ((0x00000000, 0x00000000), (0x00000000, 0x00000000),
       (0x6b200159, 0x99ba4efe)),
      ((0xffffffff, 0xffffffff), (0xffffffff, 0xffffffff),
       (0x1cb996fc, 0xbb002be7)),
      ((0x243f6a88, 0x85a308d3), (0x13198a2e, 0x03707344),
       (0xc4923a9c, 0x483df7a0)),
  ]
  for ctr, key, want in cases:
    y0, y1 = sr.threefry2x32(np.array(key, np.uint32),
                             np.array([ctr[0]], np.uint32),
                             np.array([ctr[1]], np.uint32))
    assert (int(y0[0]), int(y1[0])) == want


@pytest.mark.parametrize('n', [1, 2, 7, 8, 1025])
def test_original_layout_pairs_first_and_second_half(n):
  key = sr.PRNGKey(42)
  w = sr.random_bits(key, (n,), 32, partitionable=False)
  half = (n + 1) // 2
  for i in (0, half - 1):
    x1 = i + half if i + half < n else 0
    y0, y1 = sr.threefry2x32(key, np.array([i], np.uint32),
                             np.array([x1], np.uint32))
    assert w[i] == y0[0]
    if i + half < n:
      assert w[i + half] == y1[0]


def test_partitionable_layout_is_per_element():
  key = sr.PRNGKey(7)
  w = sr.random_bits(key, (3, 5), 32, partitionable=True)
  y0, y1 = sr.threefry2x32(key, np.array([0], np.uint32),
                           np.array([11], np.uint32))
  assert w[2, 1] == (y0[0] ^ y1[0])


@pytest.mark.parametrize('partitionable', [False, True])
def test_uniform_and_centered_ranges(partitionable):
  key = sr.PRNGKey(1)
  u = sr.uniform(key, (4096,), partitionable)
  assert u.dtype == np.float32 and u.min() >= 0.0 and u.max() < 1.0
  assert abs(float(u.mean()) - 0.5) < 0.03
  c = sr.centered_uniform16(key, (4096,), partitionable)
  assert c.min() > -0.5 and c.max() < 0.5 and abs(float(c.mean())) < 0.03
  # 16-bit draws of the original layout are the little-endian halves of the
  # 32-bit draws of half as many words
  if not partitionable:
    b16 = sr.random_bits(key, (10,), 16, False)
    w = sr.random_bits(key, (5,), 32, False)
    assert list(b16[:2]) == [int(w[0]) & 0xFFFF, int(w[0]) >> 16]


def test_split_gives_distinct_keys_in_both_layouts():
  key = sr.PRNGKey(3)
  for part in (False, True):
    ks = sr.split(key, 6, part)
    assert len({(int(k[0]), int(k[1])) for k in ks}) == 6
  # original layout: split(key, n) is random_bits over 2n words, row by row
  w = sr.random_bits(key, (4,), 32, False)
  ks = sr.split(key, 2, False)
  assert [int(ks[0][0]), int(ks[0][1]), int(ks[1][0]), int(ks[1][1])] == [
      int(v) for v in w]


@pytest.mark.gpu
@pytest.mark.parametrize('partitionable', [False, True])
@pytest.mark.parametrize('shape', [(1,), (7,), (64, 33), (3, 5, 1024)])
def test_device_noise_equals_the_host_generator(monkeypatch, partitionable,
                                                shape):
  import torch
  monkeypatch.setattr(sr, 'PARTITIONABLE', partitionable)
  key = sr.PRNGKey(1)
  got = sr.JaxUniform()(shape, key)
  want = sr.uniform(key, shape, partitionable) - np.float32(0.5)
  torch.cuda.synchronize()
  np.testing.assert_array_equal(got.cpu().numpy(), want)
  got = sr.RandomCenteredUniform()(shape, key)
  torch.cuda.synchronize()
  np.testing.assert_array_equal(got.cpu().numpy(),
                                sr.centered_uniform16(key, shape, partitionable))
  # shared axes collapse to extent 1 before the draw
  got = sr.JaxUniform()((4, 6), key, noise_sharing_axes=(0,))
  assert tuple(got.shape) == (1, 6)
