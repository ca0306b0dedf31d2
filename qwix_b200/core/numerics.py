"""Host-side description of quantized types: names, storage, value bounds.

Mirrors the query functions of qwix/_src/core/numerics.py:29-136; the conversions
themselves (numerics.py:139-196) run inside the CUDA quantizer kernels.
"""

from __future__ import annotations

import torch

from qwix_b200 import _lib

_QUANTIZABLE = (torch.bfloat16, torch.float16, torch.float32, torch.float64)

# qtype name -> (torch storage dtype, C-ABI code for the logical layout)
_BUILT = {
    'int8': (torch.int8, _lib.S8),
    'int4': (torch.int8, _lib.S4U),  # one sign-extended code per byte
    'float8_e4m3fn': (torch.float8_e4m3fn, _lib.E4M3),
    # e4m3 codes under power-of-two scales per 32 values; the code selects the scale rule in
    # the quantizer and reads as plain e4m3 everywhere else
    'mxfp8': (torch.float8_e4m3fn, _lib.MXFP8),
    # e2m1 codes, one per byte (low nibble), under power-of-two scales per 32 values
    'mxfp4': (torch.uint8, _lib.MXFP4),
    # the same codes under an e4m3-valued scale per 16 values
    'nvfp4': (torch.uint8, _lib.NVFP4),
}
_KNOWN_UNBUILT = ('nf4', 'int2', 'int3', 'int5', 'int6', 'int7', 'int16', 'uint8',
                  'mxfp8_16', 'float8_e5m2',
                  'float4_e2m1fn', 'uint4')


def qtype_name(qtype) -> str:
  """Canonical name of a qtype given as str, torch.dtype, NumPy dtype or scalar type."""
  if isinstance(qtype, str):
    return qtype
  if isinstance(qtype, torch.dtype):
    return str(qtype).replace('torch.', '')
  import numpy as np  # NumPy / ml_dtypes spellings, e.g. jnp.int8-like objects
  return np.dtype(qtype).name


def should_quantize(dtype: torch.dtype) -> bool:
  """numerics.py:29-41."""
  return dtype in _QUANTIZABLE


def can_dequant_on_output(qtype) -> bool:
  """numerics.py:44-61."""
  return qtype_name(qtype) != 'nf4'


def get_symmetric_bound(qtype) -> float:
  """numerics.py:95-136."""
  name = qtype_name(qtype)
  table = {'nf4': 1.0, 'int8': 127.5, 'int4': 7.5, 'uint8': 255.5, 'int16': 32768.0,
           'float8_e4m3fn': 448.0, 'mxfp8': 448.0, 'mxfp8_16': 448.0,
           'float8_e5m2': 57344.0, 'float4_e2m1fn': 6.0, 'mxfp4': 6.0, 'nvfp4': 6.0,
           'uint4': 15.5}
  if name in table:
    return table[name]
  if name in ('int2', 'int3', 'int5', 'int6', 'int7'):
    return 2 ** (int(name[3:]) - 1) - 0.5
  raise ValueError(f'Cannot use {qtype} as qtype.')


def get_asymmetric_bound(qtype) -> tuple[float, float]:
  """numerics.py:64-92."""
  table = {'int8': (-128.0, 127.0), 'int4': (-8.0, 7.0), 'int16': (-32768.0, 32767.0)}
  name = qtype_name(qtype)
  if name not in table:
    raise ValueError(f"{qtype} doesn't support asymmetric quantization.")
  return table[name]


def storage(qtype) -> tuple[torch.dtype, int]:
  """(torch dtype holding the codes, C-ABI dtype code) for a qtype this build runs."""
  name = qtype_name(qtype)
  if name in _BUILT:
    return _BUILT[name]
  if name in _KNOWN_UNBUILT:
    raise NotImplementedError(
        f'qtype {name!r} is valid in qwix but has no sm_100a kernel in this build.')
  raise ValueError(f'Cannot use {qtype} as qtype.')


def code_of_float(dtype: torch.dtype) -> int:
  if dtype not in _lib.FLOAT_CODES:
    raise ValueError(f'Refuse to quantize: {dtype}')
  return _lib.FLOAT_CODES[dtype]
