"""QArray and its quantize / dequantize family on CUDA tensors.

Drop-in for the module the reference injects as `_qarray_module`
(qwix/_src/providers/boxed_param.py:92-107): the same names, arguments and error
behaviour as qwix/_src/core/qarray.py, with the arithmetic done by the sm_100a kernels
behind the C ABI (csrc/quantize.cu).  Shape algebra stays on the host.
"""

from __future__ import annotations

import dataclasses
import math
from typing import Callable, Collection, Mapping, Sequence

import torch

from qwix_b200 import _lib
from qwix_b200.core import numerics

# How intermediates of x / scale (+ zero_point) round: 'strict' = every primitive rounds
# to the array dtype (JAX eager semantics), 'fused' = float32 intermediates (XLA under jit).
ROUNDING = 'strict'


def _rounding_code() -> int:
  if ROUNDING not in ('strict', 'fused'):
    raise ValueError(f'Unknown rounding mode {ROUNDING!r}.')
  return _lib.STRICT if ROUNDING == 'strict' else _lib.FUSED


@dataclasses.dataclass
class QArray:
  """qarray.py:31-100.  original ~= (qvalue - zero_point) * generic_broadcast(scale).

  int4 codes are held one per byte in an int8 tensor with qtype 'int4'.
  """

  qvalue: torch.Tensor
  scale: torch.Tensor
  zero_point: torch.Tensor | None = None
  qtype: object = None

  def __post_init__(self):
    if self.qtype is None:
      self.qtype = numerics.qtype_name(self.qvalue.dtype)
    else:
      self.qtype = numerics.qtype_name(self.qtype)

  shape = property(lambda self: tuple(self.qvalue.shape))
  ndim = property(lambda self: self.qvalue.ndim)
  dtype = property(lambda self: self.scale.dtype)
  device = property(lambda self: self.qvalue.device)
  T = property(lambda self: self.transpose())
  mT = property(lambda self: self._map(lambda x: x.mT))

  @property
  def scale_tile_shape(self) -> tuple[int, ...]:
    return tuple(o // s for o, s in zip(self.shape, self.scale.shape))

  @property
  def zero_point_tile_shape(self) -> tuple[int, ...] | None:
    if self.zero_point is None:
      return None
    return tuple(o // s for o, s in zip(self.shape, self.zero_point.shape))

  def _map(self, fn: Callable[[torch.Tensor], torch.Tensor]) -> 'QArray':
    zp = None if self.zero_point is None else fn(self.zero_point)
    return QArray(fn(self.qvalue), fn(self.scale), zp, self.qtype)

  def reshape(self, *new_shape) -> 'QArray':
    return reshape(self, *new_shape)

  def transpose(self, *axes) -> 'QArray':
    if len(axes) == 1 and not isinstance(axes[0], int):
      axes = tuple(axes[0])
    if not axes:
      axes = tuple(reversed(range(self.ndim)))
    return self._map(lambda x: x.permute(*axes))

  def swapaxes(self, axis1: int, axis2: int) -> 'QArray':
    return self._map(lambda x: x.transpose(axis1, axis2))

  def astype(self, dtype: torch.dtype) -> 'QArray':
    """Casts the dequantized type, i.e. the scale."""
    return dataclasses.replace(self, scale=self.scale.to(dtype))

  def __getitem__(self, idx) -> 'QArray':
    return rewriting_take(self, idx)


def reshape(array: QArray, *new_shape) -> QArray:
  """qarray.py:106-170 -- reshape qvalue and carry scale / zero point along.

  Old and new axes are matched in runs with equal products; inside a run a component
  either has the full extents, is all ones, or carries its extent on the run's first
  axis (a channelwise axis that is being split or merged).
  """
  if len(new_shape) == 1 and not isinstance(new_shape[0], int):
    new_shape = tuple(new_shape[0])
  old_shape = array.shape
  if math.prod(old_shape) != math.prod(new_shape):
    raise ValueError(f'Cannot reshape {old_shape} into {new_shape}.')

  runs, i, j = [], 0, 0
  cur_old, cur_new = [], []
  while i < len(old_shape) or j < len(new_shape):
    po, pn = math.prod(cur_old), math.prod(cur_new)
    take_old = po < pn or (po == pn and i < len(old_shape) and
                           (j >= len(new_shape) or old_shape[i] <= new_shape[j]))
    if po > pn:
      take_old = False
    if take_old:
      cur_old.append(old_shape[i])
      i += 1
    else:
      cur_new.append(new_shape[j])
      j += 1
    if math.prod(cur_old) == math.prod(cur_new):
      runs.append((tuple(cur_old), tuple(cur_new)))
      cur_old, cur_new = [], []
  assert not cur_old and not cur_new

  def apply(x: torch.Tensor) -> torch.Tensor:
    target, at = [], 0
    for old, new in runs:
      have = tuple(x.shape[at:at + len(old)])
      size = math.prod(have)
      if have == old:
        target.extend(new)
      elif size == 1:
        target.extend([1] * len(new))
      elif have and size == have[0] and new and new[0] % have[0] == 0:
        target.extend([have[0]] + [1] * (len(new) - 1))
      else:
        raise ValueError(
            f'Cannot reshape {old_shape} into {new_shape} for {tuple(x.shape)}.')
      at += len(old)
    return x.reshape(target)

  return array._map(apply)


def rewriting_take(array: QArray, idx) -> QArray:
  """qarray.py:173-209 -- array[idx] with the index rewritten for scale / zero point."""
  idx = list(idx) if isinstance(idx, (tuple, list)) else [idx]
  explicit = sum(i is not None and i is not Ellipsis for i in idx)
  fill = [slice(None)] * (array.ndim - explicit)
  if Ellipsis in idx:
    assert idx.count(Ellipsis) == 1
    at = idx.index(Ellipsis)
    idx[at:at + 1] = fill
  else:
    idx += fill

  def take(x: torch.Tensor) -> torch.Tensor:
    out, i = [], 0
    for full, have in zip(array.shape, x.shape):
      while idx[i] is None:
        out.append(None)
        i += 1
      cur = idx[i]
      if full == have or cur == slice(None):
        out.append(cur)
      elif have == 1:
        out.append(0 if isinstance(cur, int) else slice(None))
      elif isinstance(cur, int):
        out.append(cur // (full // have))
      else:
        raise ValueError(f'Unsupported indexing {idx} for {array.shape}.')
      i += 1
    out.extend(idx[i:])
    return x[tuple(out)]

  return array._map(take)


def validate_qarray(array: QArray):
  """qarray.py:212-247."""
  q, s, z = array.qvalue, array.scale, array.zero_point
  if not isinstance(q, torch.Tensor):
    return
  if q.ndim != s.ndim:
    raise ValueError(
        f'Scale {tuple(s.shape)} should have the same rank as qvalue {tuple(q.shape)}.')
  if any(a % b for a, b in zip(q.shape, s.shape)):
    raise ValueError(
        f'Scale {tuple(s.shape)} should be broadcastable to qvalue {tuple(q.shape)}.')
  if q.element_size() > 1 and q.dtype != torch.int16:
    raise ValueError(f'{q.dtype} is not a valid type for qvalue.')
  if not numerics.should_quantize(s.dtype):
    raise ValueError(f'{s.dtype} is not a valid type for scale.')
  if z is not None:
    if z.ndim != q.ndim:
      raise ValueError(f'Zero point {tuple(z.shape)} should have the same rank as'
                       f' qvalue {tuple(q.shape)}.')
    if any(a % b for a, b in zip(q.shape, z.shape)):
      raise ValueError(f'Zero point {tuple(z.shape)} should be broadcastable to'
                       f' qvalue {tuple(q.shape)}.')
    if z.dtype != q.dtype:
      raise ValueError(f'Zero point {z.dtype} should have the same dtype as'
                       f' qvalue {q.dtype}.')


@dataclasses.dataclass(slots=True, frozen=True, kw_only=True)
class HowToQuantize:
  """qarray.py:280-325 (stochastic-rounding noise is a training feature, not built)."""

  qtype: object
  channelwise_axes: Collection[int] = ()
  tiled_axes: Mapping[int, int | float] = dataclasses.field(default_factory=dict)
  calibration_method: str = 'absmax'
  noise_fn: object = None

  def __post_init__(self):
    if isinstance(self.qtype, str) and self.qtype in ('mxfp8', 'mxfp8_16', 'mxfp4', 'nvfp4'):
      want = 32 if self.qtype in ('mxfp8', 'mxfp4') else 16
      if not self.tiled_axes:
        raise ValueError(f'Format {self.qtype} requires `tiled_axes` to be specified.')
      for axis, size in self.tiled_axes.items():
        if size != want:
          raise ValueError(f'Format {self.qtype} requires a tile size of {want}, but'
                           f' axis {axis} got {size}.')


ShapeT = Sequence[int]
MaybeQArray = (torch.Tensor, QArray)


def _tile_size(dim: int, tile) -> int:
  return round(dim * tile) if isinstance(tile, float) else tile


def get_scale_shape(array_shape: ShapeT, how: HowToQuantize) -> tuple[int, ...]:
  """qarray.py:332-349."""
  if set(how.channelwise_axes) & set(how.tiled_axes.keys()):
    raise ValueError('The same axis cannot be both channelwise and tiled.')
  shape = []
  for axis, dim in enumerate(array_shape):
    if axis in how.channelwise_axes:
      shape.append(dim)
    elif axis in how.tiled_axes:
      t = _tile_size(dim, how.tiled_axes[axis])
      if t <= 0 or dim % t != 0:
        raise ValueError(f'{tuple(array_shape)} cannot be tiled as {how.tiled_axes}.')
      shape.append(dim // t)
    else:
      shape.append(1)
  return tuple(shape)


def split_axis(array: torch.Tensor, tiled_axes: Mapping[int, int | float]) -> torch.Tensor:
  """qarray.py:390-406 -- a tiled axis becomes (tile_count, tile_size)."""
  shape = []
  for axis, dim in enumerate(array.shape):
    if axis in tiled_axes:
      t = _tile_size(dim, tiled_axes[axis])
      if dim % t != 0:
        raise ValueError(f'{tuple(array.shape)} cannot be tiled as {tiled_axes}.')
      shape += [dim // t, t]
    else:
      shape.append(dim)
  return array.reshape(shape)


def get_tiled_axes(array: QArray) -> dict[int, int]:
  """qarray.py:409-422."""
  return {i: q // s for i, (q, s) in enumerate(zip(array.qvalue.shape, array.scale.shape))
          if q != s and s != 1}


def transpose_array(array: torch.Tensor, order: Sequence[int | None]) -> torch.Tensor:
  """qarray.py:352-387 -- permute, dropping size-1 axes and inserting new ones."""
  if any(n > 1 for a, n in enumerate(array.shape) if a not in order):
    raise ValueError(f'Cannot transpose {tuple(array.shape)} as {order}.')
  kept = [a for a in order if a is not None]
  rest = [a for a in range(array.ndim) if a not in kept]
  moved = array.permute(kept + rest).reshape([array.shape[a] for a in kept])
  return moved.reshape([1 if a is None else array.shape[a] for a in order])


def call_with_generic_broadcast(op, x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
  """qarray.py:425-444 -- host-side helper for small metadata tensors."""
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
      raise ValueError(f'Cannot broadcast between {tuple(x.shape)} {tuple(y.shape)}')
  return op(x.reshape(xs), y.reshape(ys)).reshape(out)


def broadcast_to(operand, target_shape: tuple[int, ...]):
  """qarray.py:447-467."""
  if tuple(operand.shape) == tuple(target_shape):
    return operand

  def one(x):
    if x.ndim < len(target_shape):
      x = x.reshape((1,) * (len(target_shape) - x.ndim) + tuple(x.shape))
    shape, reps = [], []
    for have, want in zip(x.shape, target_shape):
      if want % have:
        raise ValueError(f'Cannot broadcast between {tuple(x.shape)} {target_shape}')
      shape += [have, 1]
      reps += [have, want // have]
    return x.reshape(shape).expand(reps).reshape(target_shape)

  return operand._map(one) if isinstance(operand, QArray) else one(operand)


# ---- rank collapse: (shape, per-axis tile) -> the [P, R, C] / (tp, tr, tc) kernel view ----


def collapse_view(shape: Sequence[int], tiles: Sequence[int]) -> tuple[int, ...]:
  """Merges adjacent axes whose tiles stay expressible as one tile of the merged axis.

  (a, b) merge when b is reduced whole (tile_b == dim_b) or a is channelwise
  (tile_a == 1).  Raises NotImplementedError if more than three axes remain.
  """
  axes = [(d, t) for d, t in zip(shape, tiles) if d != 1]
  merged = []
  for d, t in axes:
    if merged:
      pd, pt = merged[-1]
      if t == d:
        merged[-1] = (pd * d, pt * d)
        continue
      if pt == 1:
        merged[-1] = (pd * d, t)
        continue
    merged.append((d, t))
  if len(merged) > 3:
    raise NotImplementedError(
        f'shape {tuple(shape)} with tiles {tuple(tiles)} does not collapse to a rank-3'
        ' tiled view; this scale layout has no kernel in this build.')
  merged = [(1, 1)] * (3 - len(merged)) + merged
  (P, tp), (R, tr), (C, tc) = merged
  return P, R, C, tp, tr, tc


def _view_of(shape, scale_shape):
  if len(shape) != len(scale_shape):
    raise ValueError(f'Scale {tuple(scale_shape)} should have the same rank as {tuple(shape)}.')
  if any(s == 0 or a % s for a, s in zip(shape, scale_shape)):
    raise ValueError(f'Cannot broadcast between {tuple(shape)} {tuple(scale_shape)}')
  return collapse_view(shape, [a // s for a, s in zip(shape, scale_shape)])


def _workspace(view, device) -> tuple[torch.Tensor, int]:
  n = _lib.lib().qwx_quantize_workspace_bytes(*view)
  return torch.empty(max(n, 16), dtype=torch.uint8, device=device), n


def _parse_method(method: str):
  name, *raw = method.lower().split(',')
  return name, [float(a) for a in raw]


_METHOD_CODE = {'absmax': _lib.ABSMAX, 'minmax': _lib.MINMAX, 'rms': _lib.RMS}


def _fixed_calibration(args, ndim, dtype, device) -> dict[str, torch.Tensor]:
  """qarray.py:518-532 -- constants, always per-tensor."""
  if len(args) not in (1, 2):
    raise ValueError('A fixed range is required for fixed calibration.')
  if len(args) == 1:
    args = [-args[0], args[0]]
  if args[0] > 0 or args[1] < 0 or args[0] >= args[1]:
    raise ValueError('The range must contain 0 and be non-empty.')
  shape = (1,) * ndim
  if args[0] + args[1] == 0:
    return {'absmax': torch.full(shape, args[1], dtype=dtype, device=device)}
  return {'min': torch.full(shape, args[0], dtype=dtype, device=device),
          'max': torch.full(shape, args[1], dtype=dtype, device=device)}


def calibrate(array: torch.Tensor, how: HowToQuantize) -> dict[str, torch.Tensor]:
  """qarray.py:470-534 -- statistics with the shape of the scale."""
  shape = get_scale_shape(array.shape, how)
  name, args = _parse_method(how.calibration_method)
  if name == 'fixed':
    return _fixed_calibration(args, array.ndim, array.dtype, array.device)
  if name not in _METHOD_CODE:
    raise ValueError(f'Unsupported calibration: {how.calibration_method}')
  if name == 'rms' and not args:
    raise ValueError('A scale factor is required for RMS calibration.')
  _lib.require_cuda(array)
  array = array.contiguous()
  view = _view_of(array.shape, shape)
  ws, ws_bytes = _workspace(view, array.device)
  out_a = torch.empty(shape, dtype=array.dtype, device=array.device)
  out_b = torch.empty_like(out_a) if name == 'minmax' else None
  _lib.check(_lib.lib().qwx_calibrate(
      _lib.ptr(array), numerics.code_of_float(array.dtype), *view, _METHOD_CODE[name],
      int(bool(args)), args[0] if args else 0.0, _lib.ptr(out_a), _lib.ptr(out_b),
      _lib.ptr(ws), ws_bytes, _lib.stream_ptr(array.device)), 'calibrate')
  if name == 'minmax':
    return {'min': out_a, 'max': out_b}
  return {'absmax': out_a}


def compute_scale_zero_point(calibration: Mapping[str, torch.Tensor], qtype):
  """qarray.py:537-584 -- scale (and zero point) from calibrate()'s result."""
  if 'min' in calibration and 'max' in calibration:
    numerics.get_asymmetric_bound(qtype)  # raises for types without asymmetric form
    a, b = calibration['min'], calibration['max']
  elif 'absmax' in calibration:
    a, b = calibration['absmax'], None
  else:
    raise ValueError(f'Unsupported calibration: {calibration}')
  store_dtype, code = numerics.storage(qtype)
  _lib.require_cuda(a, b)
  a = a.contiguous()
  b = None if b is None else b.contiguous()
  scale = torch.empty_like(a)
  zp = None if b is None else torch.empty(a.shape, dtype=store_dtype, device=a.device)
  _lib.check(_lib.lib().qwx_compute_scale_zero_point(
      _lib.ptr(a), _lib.ptr(b), numerics.code_of_float(a.dtype), a.numel(), code,
      _lib.ptr(scale), _lib.ptr(zp), _lib.stream_ptr(a.device)), 'compute_scale_zero_point')
  return scale, zp


# Kept for API parity (qarray.py:591).  The kernels always divide; setting this raises.
USE_RECIPROCAL_FOR_QUANTIZATION = False


def quantize_with_scale_zero_point(array: torch.Tensor, qtype, scale: torch.Tensor,
                                   zero_point: torch.Tensor | None,
                                   noise_fn=None) -> QArray:
  """qarray.py:594-635."""
  if not numerics.should_quantize(array.dtype):
    raise ValueError(f'Refuse to quantize: {array.dtype}')
  if zero_point is not None and zero_point.shape != scale.shape:
    raise ValueError(
        f'Expect zero_point shape {tuple(scale.shape)} but got {tuple(zero_point.shape)}')
  if noise_fn is not None or USE_RECIPROCAL_FOR_QUANTIZATION:
    raise NotImplementedError('stochastic rounding / reciprocal scaling are not built.')
  store_dtype, code = numerics.storage(qtype)
  _lib.require_cuda(array, scale, zero_point)
  array = array.contiguous()
  scale = scale.to(array.dtype).contiguous()
  zp = None if zero_point is None else zero_point.contiguous()
  view = _view_of(array.shape, scale.shape)
  q = torch.empty(array.shape, dtype=store_dtype, device=array.device)
  _lib.check(_lib.lib().qwx_quantize_with_scale(
      _lib.ptr(array), numerics.code_of_float(array.dtype), *view, _lib.ptr(scale),
      _lib.ptr(zp), code, _rounding_code(), _lib.ptr(q), _lib.stream_ptr(array.device)),
      'quantize_with_scale_zero_point')
  return QArray(q, scale, zero_point, numerics.qtype_name(qtype))


def quantize(array: torch.Tensor, how: HowToQuantize) -> QArray:
  """qarray.py:638-644 -- calibrate, scale, quantize; one fused kernel when it can be."""
  if not numerics.should_quantize(array.dtype):
    raise ValueError(f'Refuse to quantize: {array.dtype}')
  name, args = _parse_method(how.calibration_method)
  shape = get_scale_shape(array.shape, how)
  if name == 'fixed' or how.noise_fn is not None:
    scale, zp = compute_scale_zero_point(calibrate(array, how), how.qtype)
    return quantize_with_scale_zero_point(array, how.qtype, scale, zp, how.noise_fn)
  if name not in _METHOD_CODE:
    raise ValueError(f'Unsupported calibration: {how.calibration_method}')
  if name == 'rms' and not args:
    raise ValueError('A scale factor is required for RMS calibration.')
  if name == 'minmax':
    numerics.get_asymmetric_bound(how.qtype)
  store_dtype, code = numerics.storage(how.qtype)
  _lib.require_cuda(array)
  array = array.contiguous()
  view = _view_of(array.shape, shape)
  ws, ws_bytes = _workspace(view, array.device)
  q = torch.empty(array.shape, dtype=store_dtype, device=array.device)
  scale = torch.empty(shape, dtype=array.dtype, device=array.device)
  zp = torch.empty(shape, dtype=store_dtype, device=array.device) if name == 'minmax' else None
  _lib.check(_lib.lib().qwx_quantize(
      _lib.ptr(array), numerics.code_of_float(array.dtype), *view, _METHOD_CODE[name],
      int(bool(args)), args[0] if args else 0.0, code, _rounding_code(), _lib.ptr(q),
      _lib.ptr(scale), _lib.ptr(zp), _lib.ptr(ws), ws_bytes,
      _lib.stream_ptr(array.device)), 'quantize')
  return QArray(q, scale, zp, numerics.qtype_name(how.qtype))


def quantize_api(array: torch.Tensor, qtype, *, channelwise_axes: Collection[int] = (),
                 tiled_axes: Mapping[int, int | float] | None = None,
                 calibration_method: str = 'absmax', scale_dtype=None) -> QArray:
  """qarray.py:647-689 -- the public `quantize`."""
  how = HowToQuantize(qtype=qtype, channelwise_axes=channelwise_axes,
                      tiled_axes=tiled_axes or {}, calibration_method=calibration_method)
  out = quantize(array, how)
  if scale_dtype is not None:
    out = dataclasses.replace(out, scale=out.scale.to(scale_dtype))
  return out


def dequantize(array: QArray) -> torch.Tensor:
  """qarray.py:692-708 -- (qvalue - zero_point) * scale, in the scale dtype."""
  validate_qarray(array)
  _, code = numerics.storage(array.qtype)
  _lib.require_cuda(array.qvalue, array.scale, array.zero_point)
  q = array.qvalue.contiguous()
  scale = array.scale.contiguous()
  zp = None if array.zero_point is None else array.zero_point.contiguous()
  if zp is not None and zp.shape != scale.shape:
    zp = broadcast_to(zp, tuple(scale.shape)).contiguous() if all(
        s % z == 0 for s, z in zip(scale.shape, zp.shape)) else zp
    if zp.shape != scale.shape:
      raise NotImplementedError('zero point tiled differently from the scale.')
  view = _view_of(q.shape, scale.shape)
  out = torch.empty(q.shape, dtype=scale.dtype, device=q.device)
  _lib.check(_lib.lib().qwx_dequantize(
      _lib.ptr(q), code, *view, _lib.ptr(scale), numerics.code_of_float(scale.dtype),
      _lib.ptr(zp), _lib.ptr(out), _lib.stream_ptr(q.device)), 'dequantize')
  return out


def _promote(*dtypes: torch.dtype) -> torch.dtype:
  out = dtypes[0]
  for d in dtypes[1:]:
    out = torch.promote_types(out, d)
  return out


def get_accumulator_and_result_type(*args, preferred_element_type=None):
  """qarray.py:781-821 -- (accumulator dtype, result dtype) of a quantized contraction."""
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
        t = torch.bfloat16 if t.is_floating_point else torch.int32
      widened.append(t)
    result = _promote(*widened)
  is_int = lambda t: not t.is_floating_point and t != torch.bool
  acc = torch.int32 if all(is_int(t) for t in qdts) else result
  return acc, result
