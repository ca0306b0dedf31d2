"""Oracle numerics: value bounds and the float -> quantized-code conversion.

Test infrastructure only.  Restates qwix/_src/core/numerics.py:64-275 on NumPy.
"""

from __future__ import annotations

import ml_dtypes
import numpy as np

bfloat16 = ml_dtypes.bfloat16
float8_e4m3fn = ml_dtypes.float8_e4m3fn
float4_e2m1fn = ml_dtypes.float4_e2m1fn
int4 = ml_dtypes.int4
uint4 = ml_dtypes.uint4

_FLOAT_INPUTS = (np.dtype(bfloat16), np.dtype(np.float16), np.dtype(np.float32),
                 np.dtype(np.float64))

_SYNTHETIC_INTS = ('int2', 'int3', 'int5', 'int6', 'int7')

# Appendix E of arXiv 2305.14314, as listed in numerics.py:235-252.
NF4_BUCKETS = np.array([
    -1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453,
    -0.28444138169288635, -0.18477343022823334, -0.09105003625154495, 0.0,
    0.07958029955625534, 0.16093020141124725, 0.24611230194568634,
    0.33791524171829224, 0.44070982933044434, 0.5626170039176941,
    0.7229568362236023, 1.0], dtype=np.float32)


def qtype_name(qtype) -> str:
  """Canonical string for a qtype given as a string, NumPy dtype or scalar type."""
  if isinstance(qtype, str):
    return qtype
  return np.dtype(qtype).name


def storage_dtype(qtype) -> np.dtype:
  """NumPy dtype that holds the codes of `qtype`."""
  name = qtype_name(qtype)
  if name == 'nf4':
    return np.dtype(uint4)
  if name in _SYNTHETIC_INTS:
    return np.dtype(int4) if int(name[3:]) <= 4 else np.dtype(np.int8)
  if name in ('mxfp8', 'mxfp8_16'):
    return np.dtype(float8_e4m3fn)
  if name in ('mxfp4', 'nvfp4'):
    return np.dtype(float4_e2m1fn)
  return np.dtype(name)


def should_quantize(dtype) -> bool:
  """numerics.py:29-41 -- only bf16/f16/f32/f64 arrays are quantized."""
  return np.dtype(dtype) in _FLOAT_INPUTS


def can_dequant_on_output(qtype) -> bool:
  """numerics.py:44-61 -- lookup-table types cannot be scaled after the dot."""
  return qtype_name(qtype) != 'nf4'


def _is_float_code(dt: np.dtype) -> bool:
  try:
    ml_dtypes.finfo(dt)
    return True
  except ValueError:
    return False


def get_asymmetric_bound(qtype) -> tuple[float, float]:
  """numerics.py:64-92 -- (qmin, qmax) for int8 / int4 / int16 only."""
  name = qtype_name(qtype)
  table = {'int8': (-128.0, 127.0), 'int4': (-8.0, 7.0),
           'int16': (-32768.0, 32767.0)}
  if name not in table:
    raise ValueError(f"{qtype} doesn't support asymmetric quantization.")
  return table[name]


def get_symmetric_bound(qtype) -> float:
  """numerics.py:95-136 -- magnitude B such that codes cover [-B, B]."""
  name = qtype_name(qtype)
  if name == 'nf4':
    return 1.0
  if name in _SYNTHETIC_INTS:
    return 2 ** (int(name[3:]) - 1) - 0.5
  dt = storage_dtype(name)
  if dt.itemsize > 1 and dt != np.dtype(np.int16):
    raise ValueError(f'Cannot use {qtype} as qtype.')
  if dt == np.dtype(np.int16):
    return 32768.0
  if _is_float_code(dt):
    return float(ml_dtypes.finfo(dt).max)
  return float(ml_dtypes.iinfo(dt).max) + 0.5


def _saturating_int_cast(x: np.ndarray, dt: np.dtype) -> np.ndarray:
  """XLA's float -> int convert: clamp to the range, NaN becomes 0.

  Pinned by tests/_src/core/numerics_test.py:34-56 (129 -> 127, -1300 -> -128,
  +/-inf -> 127 / -128).  NumPy's own cast wraps, hence the explicit clamp.
  """
  info = ml_dtypes.iinfo(dt)
  y = np.asarray(x, dtype=np.float64)
  y = np.where(np.isnan(y), 0.0, y)
  y = np.clip(y, info.min, info.max)
  return y.astype(np.int64).astype(dt)


def convert_to(x: np.ndarray, qtype) -> np.ndarray:
  """numerics.py:139-196 -- scaled floats to codes (no stochastic rounding).

  Integers: round-half-to-even in the array dtype, then a saturating cast.
  Floats (fp8/fp4): clip to the finite range in the array dtype, then cast RN-even.
  """
  name = qtype_name(qtype)
  if name == 'nf4':
    flat = np.asarray(x, dtype=np.float32).ravel()
    idx = np.abs(NF4_BUCKETS[None, :] - flat[:, None]).argmin(axis=1)
    return idx.astype(np.uint8).astype(uint4).reshape(np.shape(x))
  if name in _SYNTHETIC_INTS:
    bits = int(name[3:])
    lo, hi = -(2 ** (bits - 1)), 2 ** (bits - 1) - 1
    r = np.clip(np.rint(np.asarray(x)).astype(np.float64), lo, hi)
    return _saturating_int_cast(r, storage_dtype(name))
  dt = storage_dtype(name)
  x = np.asarray(x)
  if _is_float_code(dt):
    fin = ml_dtypes.finfo(dt)
    lo = np.asarray(float(fin.min), dtype=x.dtype)
    hi = np.asarray(float(fin.max), dtype=x.dtype)
    return np.clip(x, lo, hi).astype(dt)
  return _saturating_int_cast(np.rint(x), dt)


def convert_from(x: np.ndarray, qtype) -> np.ndarray:
  """numerics.py:199-223 -- only nf4 needs un-bucketing."""
  if qtype_name(qtype) == 'nf4':
    return NF4_BUCKETS[np.asarray(x).astype(np.int64)]
  return x
