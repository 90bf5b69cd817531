"""Builds libaqt_b200.so (sm_100a) in-tree with nvcc.

Usage: python -m aqt_b200.build [--force]
The shared library lands next to this file so that it travels with the source
tree; nothing is installed into site-packages.
"""

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, 'csrc')
LIB = os.path.join(HERE, 'libaqt_b200.so')
SOURCES = ['quantize.cu', 'gemm.cu', 'noise.cu', 'runtime.cu', 'api.cu',
           'xla_ffi.cc']
HEADERS = [os.path.join(CSRC, 'common.cuh'),
           os.path.join(HERE, '..', 'include', 'aqt_b200.h')]
NVCC_FLAGS = [
    '-gencode', 'arch=compute_100a,code=sm_100a', '-O3', '-lineinfo',
    '-std=c++17', '-Xcompiler', '-fPIC', '--expt-relaxed-constexpr',
]


def _nvcc():
  exe = shutil.which('nvcc') or '/usr/local/cuda/bin/nvcc'
  if not os.path.exists(exe):
    raise RuntimeError('nvcc not found; the sm_100a kernels cannot be built')
  return exe


def _ffi_include():
  """-I for jaxlib's XLA FFI header when jax is installed (csrc/xla_ffi.cc is
  empty without it)."""
  try:
    import jax.ffi  # pylint: disable=import-outside-toplevel
    return ['-I', jax.ffi.include_dir()]
  except Exception:  # pylint: disable=broad-except
    return []


def _stale(target, deps):
  if not os.path.exists(target):
    return True
  t = os.path.getmtime(target)
  return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
  """Compiles every .cu file and links the shared library. Returns its path."""
  nvcc = _nvcc()
  build_dir = os.path.join(HERE, 'build')
  os.makedirs(build_dir, exist_ok=True)
  objs = []
  for src in SOURCES:
    src_path = os.path.join(CSRC, src)
    obj = os.path.join(build_dir, os.path.splitext(src)[0] + '.o')
    objs.append(obj)
    if force or _stale(obj, [src_path] + HEADERS):
      cmd = [nvcc] + NVCC_FLAGS + _ffi_include() + (
          ['-Xptxas', '-v'] if verbose else []) + ['-c', src_path, '-o', obj]
      subprocess.run(cmd, check=True)
  if force or _stale(LIB, objs):
    subprocess.run([nvcc, '-shared', '-o', LIB] + objs + ['-lcudart', '-ldl'],
                   check=True)
  return LIB


if __name__ == '__main__':
  print(build(force='--force' in sys.argv, verbose='-v' in sys.argv))
