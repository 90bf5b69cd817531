"""Helpers shared by the tests: torch <-> numpy (ml_dtypes) conversion."""

import ml_dtypes
import numpy as np
import torch

_VIEW = {
    torch.bfloat16: (torch.int16, np.dtype(ml_dtypes.bfloat16)),
    torch.float8_e4m3fn: (torch.uint8, np.dtype(ml_dtypes.float8_e4m3fn)),
    torch.float8_e5m2: (torch.uint8, np.dtype(ml_dtypes.float8_e5m2)),
}


def to_numpy(t: torch.Tensor) -> np.ndarray:
  """Bit-exact copy of a (possibly strided, possibly CUDA) tensor to numpy."""
  t = t.detach().contiguous().cpu()
  if t.dtype in _VIEW:
    as_int, np_dt = _VIEW[t.dtype]
    return t.view(as_int).numpy().view(np_dt)
  return t.numpy()


def to_torch(a: np.ndarray, device='cpu') -> torch.Tensor:
  a = np.ascontiguousarray(a)
  for tdt, (as_int, np_dt) in _VIEW.items():
    if a.dtype == np_dt:
      raw = a.view(np.int16 if as_int == torch.int16 else np.uint8)
      return torch.from_numpy(raw.copy()).view(tdt).to(device)
  return torch.from_numpy(a.copy()).to(device)


def rand_normal(rng, shape, std, np_dtype):
  return (rng.standard_normal(shape) * std).astype(np.float32).astype(np_dtype)
