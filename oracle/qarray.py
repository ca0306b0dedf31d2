"""Oracle QArray: calibrate / scale / quantize / dequantize on NumPy arrays.

Test infrastructure only.  Restates qwix/_src/core/qarray.py (file:line cited
per function).  Arrays are NumPy arrays whose dtype may be an ml_dtypes type;
int4 codes are held one per byte (ml_dtypes.int4), as JAX holds them logically.
"""

from __future__ import annotations

import dataclasses
import math
from typing import Callable, Collection, Mapping, Sequence

import numpy as np

from oracle import numerics

STRICT = 'strict'
FUSED = 'fused'


@dataclasses.dataclass
class QArray:
  """qarray.py:31-100 -- original ~= (qvalue - zero_point) * broadcast(scale)."""

  qvalue: np.ndarray
  scale: np.ndarray
  zero_point: np.ndarray | None = None
  qtype: object = None

  def __post_init__(self):
    if self.qtype is None:
      self.qtype = self.qvalue.dtype.name

  @property
  def shape(self):
    return tuple(self.qvalue.shape)

  @property
  def ndim(self):
    return self.qvalue.ndim

  @property
  def dtype(self):
    return self.scale.dtype

  @property
  def scale_tile_shape(self):
    return tuple(o // s for o, s in zip(self.shape, self.scale.shape))

  def _map(self, fn) -> 'QArray':
    zp = None if self.zero_point is None else fn(self.zero_point)
    return QArray(fn(self.qvalue), fn(self.scale), zp, self.qtype)

  def transpose(self, *axes) -> 'QArray':
    return self._map(lambda a: a.transpose(*axes))

  def swapaxes(self, a: int, b: int) -> 'QArray':
    return self._map(lambda x: x.swapaxes(a, b))

  def astype(self, dtype) -> 'QArray':
    return dataclasses.replace(self, scale=self.scale.astype(dtype))


@dataclasses.dataclass(frozen=True, kw_only=True)
class HowToQuantize:
  """qarray.py:280-325 (noise_fn / mxfp validation omitted: not on this path)."""

  qtype: object
  channelwise_axes: Collection[int] = ()
  tiled_axes: Mapping[int, int | float] = dataclasses.field(default_factory=dict)
  calibration_method: str = 'absmax'


def _tile_of(dim: int, tile) -> int:
  return round(dim * tile) if isinstance(tile, float) else tile


def get_scale_shape(array_shape: Sequence[int], how: HowToQuantize):
  """qarray.py:332-349."""
  if set(how.channelwise_axes) & set(how.tiled_axes):
    raise ValueError('The same axis cannot be both channelwise and tiled.')
  out = []
  for axis, dim in enumerate(array_shape):
    if axis in how.channelwise_axes:
      out.append(dim)
    elif axis in how.tiled_axes:
      t = _tile_of(dim, how.tiled_axes[axis])
      if t <= 0 or dim % t:
        raise ValueError(f'{array_shape} cannot be tiled as {how.tiled_axes}.')
      out.append(dim // t)
    else:
      out.append(1)
  return tuple(out)


def split_axis(array: np.ndarray, tiled_axes: Mapping[int, int | float]):
  """qarray.py:390-406 -- each tiled axis becomes (tile_count, tile_size)."""
  shape = []
  for axis, dim in enumerate(array.shape):
    if axis in tiled_axes:
      t = _tile_of(dim, tiled_axes[axis])
      if dim % t:
        raise ValueError(f'{array.shape} cannot be tiled as {tiled_axes}.')
      shape += [dim // t, t]
    else:
      shape.append(dim)
  return array.reshape(shape)


def get_tiled_axes(array: QArray) -> dict[int, int]:
  """qarray.py:409-422."""
  return {i: q // s for i, (q, s) in
          enumerate(zip(array.qvalue.shape, array.scale.shape))
          if q != s and s != 1}


def transpose_array(array: np.ndarray, order: Sequence[int | None]):
  """qarray.py:352-387 -- transpose allowing dropped size-1 axes and new axes."""
  if any(n > 1 for a, n in enumerate(array.shape) if a not in order):
    raise ValueError(f'Cannot transpose {array.shape} as {order}.')
  kept = [a for a in order if a is not None]
  dropped = [a for a in range(array.ndim) if a not in kept]
  moved = array.transpose(kept + dropped).reshape([array.shape[a] for a in kept])
  return moved.reshape([1 if a is None else array.shape[a] for a in order])


def call_with_generic_broadcast(op: Callable, x: np.ndarray, y: np.ndarray):
  """qarray.py:425-444 -- elementwise op where one extent may divide the other."""
  assert x.ndim == y.ndim
  xs, ys, out = [], [], []
  for a, b in zip(x.shape, y.shape):
    out.append(max(a, b))
    if a == b or a == 1 or b == 1:
      xs.append(a)
      ys.append(b)
    elif a % b == 0:
      xs += [b, a // b]
      ys += [b, 1]
    elif b % a == 0:
      xs += [a, 1]
      ys += [a, b // a]
    else:
      raise ValueError(f'Cannot broadcast between {x.shape} {y.shape}')
  return op(x.reshape(xs), y.reshape(ys)).reshape(out)


def _mean_like_jnp(sq: np.ndarray, axes) -> np.ndarray:
  # jnp.mean sums 16-bit floats in float32, divides, then casts back.
  wide = np.dtype(np.float32) if sq.dtype.itemsize < 4 else sq.dtype
  total = np.sum(sq.astype(wide), axis=axes, keepdims=True, dtype=wide)
  count = math.prod(sq.shape[a] for a in axes)
  return (total / wide.type(count)).astype(sq.dtype)


def calibrate(array: np.ndarray, how: HowToQuantize) -> dict[str, np.ndarray]:
  """qarray.py:470-534 -- statistics shaped like the scale."""
  reduce_axes, shift = [], 0
  for axis in range(array.ndim):
    if axis in how.channelwise_axes:
      continue
    if axis in how.tiled_axes:
      shift += 1
    reduce_axes.append(axis + shift)
  reduce_axes = tuple(reduce_axes)
  shape = get_scale_shape(array.shape, how)
  tiled = split_axis(array, how.tiled_axes)
  dt = array.dtype

  method, *raw = how.calibration_method.lower().split(',')
  args = [float(a) for a in raw]
  as_dt = lambda v: np.asarray(v, dtype=dt)  # weak Python scalar -> array dtype
  if method == 'minmax':
    lo = np.minimum(np.min(tiled, axis=reduce_axes, keepdims=True), as_dt(0))
    hi = np.maximum(np.max(tiled, axis=reduce_axes, keepdims=True), as_dt(0))
    if args:
      lo, hi = lo * as_dt(args[0]), hi * as_dt(args[0])
    return {'min': lo.reshape(shape), 'max': hi.reshape(shape)}
  if method == 'absmax':
    amax = np.max(np.abs(tiled), axis=reduce_axes, keepdims=True)
    if args:
      amax = amax * as_dt(args[0])
    return {'absmax': amax.reshape(shape)}
  if method == 'rms':
    if not args:
      raise ValueError('A scale factor is required for RMS calibration.')
    rms = np.sqrt(_mean_like_jnp(np.square(tiled), reduce_axes))
    return {'absmax': (rms * as_dt(args[0])).reshape(shape)}
  if method == 'fixed':
    if len(args) not in (1, 2):
      raise ValueError('A fixed range is required for fixed calibration.')
    if len(args) == 1:
      args = [-args[0], args[0]]
    if args[0] > 0 or args[1] < 0 or args[0] >= args[1]:
      raise ValueError('The range must contain 0 and be non-empty.')
    shape = tuple(1 for _ in shape)
    if args[0] + args[1] == 0:
      return {'absmax': np.full(shape, args[1], dt)}
    return {'min': np.full(shape, args[0], dt), 'max': np.full(shape, args[1], dt)}
  raise ValueError(f'Unsupported calibration: {how.calibration_method}')


def _tiny_guard(scale: np.ndarray) -> np.ndarray:
  import ml_dtypes
  tiny = ml_dtypes.finfo(scale.dtype).tiny
  thr = np.sqrt(np.asarray(tiny, dtype=scale.dtype))
  return np.where(scale < thr, np.ones_like(scale), scale)


def compute_scale_zero_point(calibration: Mapping[str, np.ndarray], qtype):
  """qarray.py:537-584 -- scale (and zero point) in the calibration dtype."""
  name = numerics.qtype_name(qtype)
  if 'min' in calibration and 'max' in calibration:
    qmin, qmax = numerics.get_asymmetric_bound(qtype)
    dt = calibration['max'].dtype
    scale = (calibration['max'] - calibration['min']) / np.asarray(qmax - qmin, dt)
    scale = _tiny_guard(scale)
    zp = np.asarray(qmin, dt) - calibration['min'] / scale
    zero_point = numerics.convert_to(zp, qtype)
  elif 'absmax' in calibration:
    dt = calibration['absmax'].dtype
    bound = numerics.get_symmetric_bound(qtype)
    scale = _tiny_guard(calibration['absmax'] / np.asarray(bound, dt))
    zero_point = None
  else:
    raise ValueError(f'Unsupported calibration: {calibration}')
  if name in ('mxfp8', 'mxfp8_16', 'mxfp4'):
    # Outlier-aware power-of-two scales (qarray.py:566-581).
    c = 12.0 / 7.0 if name == 'mxfp4' else 60.0 / 31.0
    sb = (scale * np.asarray(c, scale.dtype)).astype(numerics.bfloat16)
    pow2 = (sb.view(np.int16) & np.int16(0x7F80)).view(numerics.bfloat16)
    scale = pow2.astype(scale.dtype)
  elif name == 'nvfp4':
    scale = numerics.convert_to(scale, 'float8_e4m3fn').astype(scale.dtype)
  return scale, zero_point


def quantize_with_scale_zero_point(array: np.ndarray, qtype, scale: np.ndarray,
                                   zero_point: np.ndarray | None,
                                   mode: str = STRICT) -> QArray:
  """qarray.py:594-635 -- true division, optional zero point, convert_to."""
  if not numerics.should_quantize(array.dtype):
    raise ValueError(f'Refuse to quantize: {array.dtype}')
  if zero_point is not None and zero_point.shape != scale.shape:
    raise ValueError(
        f'Expect zero_point shape {scale.shape} but got {zero_point.shape}')
  scale = scale.astype(array.dtype)
  work = array.dtype if mode == STRICT else np.dtype(np.float32)
  if array.dtype.itemsize >= 4:
    work = array.dtype
  q = call_with_generic_broadcast(np.divide, array.astype(work),
                                  scale.astype(work))
  if zero_point is not None:
    q = call_with_generic_broadcast(np.add, q, zero_point.astype(work))
  return QArray(numerics.convert_to(q, qtype), scale, zero_point, qtype)


def quantize(array: np.ndarray, how: HowToQuantize, mode: str = STRICT) -> QArray:
  """qarray.py:638-644."""
  scale, zp = compute_scale_zero_point(calibrate(array, how), how.qtype)
  return quantize_with_scale_zero_point(array, how.qtype, scale, zp, mode)


def quantize_api(array, qtype, *, channelwise_axes=(), tiled_axes=None,
                 calibration_method='absmax', scale_dtype=None,
                 mode: str = STRICT) -> QArray:
  """qarray.py:647-689 -- the public qwix.quantize."""
  how = HowToQuantize(qtype=qtype, channelwise_axes=channelwise_axes,
                      tiled_axes=tiled_axes or {},
                      calibration_method=calibration_method)
  out = quantize(array, how, mode)
  if scale_dtype is not None:
    out = dataclasses.replace(out, scale=out.scale.astype(scale_dtype))
  return out


def validate_qarray(array: QArray):
  """qarray.py:212-247."""
  q, s, z = array.qvalue, array.scale, array.zero_point
  if q.ndim != s.ndim:
    raise ValueError(f'Scale {s.shape} should have the same rank as qvalue {q.shape}.')
  if any(a % b for a, b in zip(q.shape, s.shape)):
    raise ValueError(f'Scale {s.shape} should be broadcastable to qvalue {q.shape}.')
  if q.dtype.itemsize > 1 and q.dtype != np.dtype(np.int16):
    raise ValueError(f'{q.dtype} is not a valid type for qvalue.')
  if not numerics.should_quantize(s.dtype):
    raise ValueError(f'{s.dtype} is not a valid type for scale.')
  if z is not None:
    if z.ndim != q.ndim:
      raise ValueError(f'Zero point {z.shape} should have the same rank as qvalue {q.shape}.')
    if any(a % b for a, b in zip(q.shape, z.shape)):
      raise ValueError(f'Zero point {z.shape} should be broadcastable to qvalue {q.shape}.')
    if z.dtype != q.dtype:
      raise ValueError(f'Zero point {z.dtype} should have the same dtype as qvalue {q.dtype}.')


def dequantize(array: QArray) -> np.ndarray:
  """qarray.py:692-708 -- (qvalue - zero_point) * scale in the scale dtype."""
  validate_qarray(array)
  q = numerics.convert_from(array.qvalue, array.qtype)
  q = np.asarray(q).astype(array.scale.dtype)
  if array.zero_point is not None:
    q = call_with_generic_broadcast(np.subtract, q,
                                    array.zero_point.astype(q.dtype))
  return call_with_generic_broadcast(np.multiply, q, array.scale)


def _is_int_name(dt: np.dtype) -> bool:
  return 'int' in dt.name


def jnp_result_type(*dtypes) -> np.dtype:
  """jnp.result_type restricted to the types that reach this path."""
  dts = [np.dtype(d) for d in dtypes]
  floats = [d for d in dts if not _is_int_name(d)]
  if not floats:
    return np.result_type(*dts)
  if any(d == np.dtype(np.float64) for d in floats):
    return np.dtype(np.float64)
  if any(d == np.dtype(np.float32) for d in floats):
    return np.dtype(np.float32)
  names = {d.name for d in floats}
  if names == {'bfloat16'}:
    return np.dtype(numerics.bfloat16)
  if names == {'float16'}:
    return np.dtype(np.float16)
  return np.dtype(np.float32)  # bf16 with f16 promotes to f32


def get_accumulator_and_result_type(*args, preferred_element_type=None):
  """qarray.py:781-821."""
  qdts, ddts = [], []
  for a in args:
    if isinstance(a, QArray):
      qdts.append(a.qvalue.dtype)
      ddts.append(a.scale.dtype)
    else:
      qdts.append(a.dtype)
      ddts.append(a.dtype)
  result = preferred_element_type
  if result is None:
    widened = []
    for t in ddts:
      if t.itemsize <= 1:
        t = np.dtype(np.int32) if _is_int_name(t) else np.dtype(numerics.bfloat16)
      widened.append(t)
    result = jnp_result_type(*widened)
  result = np.dtype(result)
  acc = np.dtype(np.int32) if all(_is_int_name(t) for t in qdts) else result
  return acc, result
