"""The C-ABI library loads and exports every symbol include/aqt_b200.h declares."""

import ctypes
import os
import re

import pytest

from aqt_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, 'include', 'aqt_b200.h')


def _declared_symbols():
  text = open(HEADER).read()
  text = re.sub(r'/\*.*?\*/', '', text, flags=re.S)
  return sorted(set(re.findall(r'\b(aqtb200_[a-z0-9_]+)\s*\(', text)))


@pytest.fixture(scope='module')
def lib():
  if not os.path.exists(_lib.LIB_PATH):
    from aqt_b200 import build
    build.build()
  return ctypes.CDLL(_lib.LIB_PATH)


def test_header_and_binding_agree():
  assert _declared_symbols() == sorted(_lib.SYMBOLS)


def test_every_declared_symbol_is_exported(lib):
  for name in _declared_symbols():
    assert hasattr(lib, name), f'{name} missing from libaqt_b200.so'


def test_struct_sizes_match_header_layout():
  # The ctypes mirrors must have the C layout: pointers/int64 8-byte aligned.
  assert ctypes.sizeof(_lib.View) == 8 + 4 + 4 + 8 * 8
  assert ctypes.sizeof(_lib.QuantSpec) == 40
  assert ctypes.sizeof(_lib.GemmDesc) % 8 == 0
  assert ctypes.sizeof(_lib.DgRawDesc) % 8 == 0


def test_calls_that_need_no_device(lib):
  lib.aqtb200_version.restype = ctypes.c_int
  assert lib.aqtb200_version() == 1
  lib.aqtb200_round_up.restype = ctypes.c_int64
  lib.aqtb200_round_up.argtypes = [ctypes.c_int64, ctypes.c_int64]
  assert lib.aqtb200_round_up(20, 16) == 32
  assert lib.aqtb200_round_up(32, 16) == 32
  # argument errors are reported as negative codes, not crashes
  lib.aqtb200_gemm_dequant.restype = ctypes.c_int
  lib.aqtb200_gemm_dequant.argtypes = [ctypes.c_void_p] * 3
  assert lib.aqtb200_gemm_dequant(None, None, None) == -1
  lib.aqtb200_last_error.restype = ctypes.c_char_p
  assert b'null' in lib.aqtb200_last_error()
  assert lib.aqtb200_set_gemm_impl(7) == -1
