"""Oracle quantized dot_general (fast / slow / loop) on NumPy arrays.

Test infrastructure only.  Restates qwix/_src/core/dot_general.py; the plain
contraction that the reference delegates to jax.lax.dot_general is
`lax_dot_general` below (output axes: batch, lhs free, rhs free).
"""

from __future__ import annotations

import itertools
from typing import Mapping

import numpy as np

from oracle import numerics
from oracle import qarray
from oracle.qarray import QArray

MIN_TILE_SIZE_TO_DEQUANT_ON_OUTPUT = 128  # dot_general.py:404


def lax_dot_general(lhs: np.ndarray, rhs: np.ndarray, dimension_numbers,
                    preferred_element_type=None) -> np.ndarray:
  """jax.lax.dot_general semantics.

  Integer operands accumulate exactly (through float64 BLAS: every partial sum
  of int8 products stays far below 2**53) and wrap to int32 like XLA; floating
  operands accumulate in float32 and round once to the result dtype.
  """
  (lc, rc), (lb, rb) = dimension_numbers
  lc, rc, lb, rb = map(list, (lc, rc, lb, rb))
  lf = [a for a in range(lhs.ndim) if a not in lc and a not in lb]
  rf = [a for a in range(rhs.ndim) if a not in rc and a not in rb]
  lt = lhs.transpose(lb + lf + lc)
  rt = rhs.transpose(rb + rc + rf)
  bshape = [lhs.shape[a] for a in lb]
  lfs = [lhs.shape[a] for a in lf]
  rfs = [rhs.shape[a] for a in rf]
  k = int(np.prod([lhs.shape[a] for a in lc], dtype=np.int64))
  nb = int(np.prod(bshape, dtype=np.int64))
  m = int(np.prod(lfs, dtype=np.int64))
  n = int(np.prod(rfs, dtype=np.int64))
  both_int = 'int' in lhs.dtype.name and 'int' in rhs.dtype.name
  if preferred_element_type is None:
    out_dt = np.dtype(np.int32) if both_int else qarray.jnp_result_type(
        lhs.dtype, rhs.dtype)
  else:
    out_dt = np.dtype(preferred_element_type)
  work = np.float64 if both_int or out_dt == np.dtype(np.float64) else np.float32
  a3 = lt.reshape(nb, m, k).astype(work)
  b3 = rt.reshape(nb, k, n).astype(work)
  out = np.matmul(a3, b3).reshape(bshape + lfs + rfs)
  if 'int' in out_dt.name:
    return out.astype(np.int64).astype(out_dt)
  return out.astype(out_dt)


def get_how_to_quantize(*, dimension_numbers, ndims, for_lhs, tile_size,
                        **kwargs) -> qarray.HowToQuantize:
  """dot_general.py:28-76 -- per-channel on free/batch axes, tile the last
  contracting axis when a tile size is given."""
  side = 0 if for_lhs else 1
  ndim = ndims[side]
  contracting = dimension_numbers[0][side]
  if isinstance(tile_size, Mapping):
    tiled = dict(tile_size)
  else:
    tiled = {contracting[-1]: tile_size} if tile_size else {}
  channelwise = sorted(set(range(ndim)) - set(contracting) - set(tiled))
  return qarray.HowToQuantize(channelwise_axes=channelwise, tiled_axes=tiled,
                              **kwargs)


def _scale_orders(dimension_numbers, ndims):
  """dot_general.py:79-90 -- where each scale axis lands in the output."""
  (lc, rc), (lb, rb) = dimension_numbers
  lf = sorted(set(range(ndims[0])) - set(lc) - set(lb))
  rf = sorted(set(range(ndims[1])) - set(rc) - set(rb))
  return (list(lb) + lf + [None] * len(rf),
          list(rb) + [None] * len(lf) + rf)


def _retile(contracting, batch, tiled):
  """dot_general.py:93-122 -- a tiled contracting axis becomes (count, size);
  the count axis is appended to the batch axes and summed at the end."""
  new_c = [a + sum(t <= a for t in tiled) for a in contracting]
  new_b = [a + sum(t < a for t in tiled) for a in batch]
  new_b += [a + sum(t < a for t in tiled) for a in contracting if a in tiled]
  return tuple(new_c), tuple(new_b), tuple(range(len(batch), len(new_b)))


def _mul(res: np.ndarray, scale: np.ndarray) -> np.ndarray:
  """res * scale with jnp promotion (an int32 result first becomes the float
  type of the scale), broadcasting generically."""
  dt = qarray.jnp_result_type(res.dtype, scale.dtype)
  return qarray.call_with_generic_broadcast(
      np.multiply, res.astype(dt), scale.astype(dt))


def _parts(x):
  if isinstance(x, QArray):
    return x.qvalue, x.scale, x.zero_point, qarray.get_tiled_axes(x)
  return x, None, None, {}


def _storage(v: np.ndarray) -> np.ndarray:
  # int4 codes take part in contractions as small integers.
  return v.astype(np.int8) if v.dtype.name in ('int4', 'uint4') else v


def _common_tiles(lhs_ca, rhs_ca, lt, rt, dimension_numbers):
  ltc, rtc = {}, {}
  for l, r in zip(lhs_ca, rhs_ca):
    a, b = lt.get(l), rt.get(r)
    if a and b and a != b:
      raise ValueError(
          'Contracting axes must be tiled with the same tile size.'
          f' lhs_tiled_axes={lt} rhs_tiled_axes={rt} {dimension_numbers=}')
    if a or b:
      ltc[l] = rtc[r] = a or b
  return ltc, rtc


def fast_dot_general(lhs, rhs, dimension_numbers, preferred_element_type=None):
  """dot_general.py:135-261 -- contract the codes, then apply the scales."""
  lv, ls, lz, lt = _parts(lhs)
  rv, rs, rz, rt = _parts(rhs)
  if lz is not None and rz is not None:
    raise ValueError('Only one operand can be asymmetric.')
  (lca, rca), (lba, rba) = dimension_numbers
  ltc, rtc = _common_tiles(lca, rca, lt, rt, dimension_numbers)

  lv = qarray.split_axis(_storage(lv), ltc)
  rv = qarray.split_axis(_storage(rv), rtc)
  ones = lambda d: {a: 1 for a in d}
  if lz is not None:
    lz = qarray.split_axis(_storage(lz), ones(ltc))
  if rz is not None:
    rz = qarray.split_axis(_storage(rz), ones(rtc))

  lca, lba, sum_axes = _retile(lca, lba, ltc)
  rca, rba, _ = _retile(rca, rba, rtc)
  dn = ((lca, rca), (lba, rba))
  l_order, r_order = _scale_orders(dn, (lv.ndim, rv.ndim))
  if ls is not None:
    ls = qarray.transpose_array(qarray.split_axis(ls, ones(ltc)), l_order)
  if rs is not None:
    rs = qarray.transpose_array(qarray.split_axis(rs, ones(rtc)), r_order)

  acc_t, res_t = qarray.get_accumulator_and_result_type(
      lhs, rhs, preferred_element_type=preferred_element_type)
  res = lax_dot_general(lv, rv, dn, acc_t)

  def spread(zp, like, axes):
    shape = list(zp.shape)
    for a in axes:
      shape[a] = like.shape[a]
    return np.broadcast_to(zp, shape)

  if lz is not None:
    corr = lax_dot_general(spread(lz, lv, lca + lba), rv, dn, acc_t)
    res = qarray.call_with_generic_broadcast(np.subtract, res, corr)
  if rz is not None:
    corr = lax_dot_general(lv, spread(rz, rv, rca + rba), dn, acc_t)
    res = qarray.call_with_generic_broadcast(np.subtract, res, corr)

  if ls is not None:
    res = _mul(res, ls)
  if rs is not None:
    res = _mul(res, rs)
  if sum_axes:
    wide = np.float32 if res.dtype.itemsize < 4 else res.dtype
    res = np.sum(res.astype(wide), axis=sum_axes, dtype=wide).astype(res.dtype)
  return res.astype(res_t)


def slow_dot_general(lhs, rhs, dimension_numbers, preferred_element_type=None):
  """dot_general.py:264-275 -- dequantize, then a floating-point contraction."""
  if isinstance(lhs, QArray):
    lhs = qarray.dequantize(lhs)
  if isinstance(rhs, QArray):
    rhs = qarray.dequantize(rhs)
  return lax_dot_general(lhs, rhs, dimension_numbers, preferred_element_type)


def loop_dot_general(lhs, rhs, dimension_numbers, preferred_element_type=None):
  """dot_general.py:278-399 -- one contraction per K tile, scaled, then added
  in increasing tile order (the in-kernel accumulation loop)."""
  lv, ls, lz, lt = _parts(lhs)
  rv, rs, rz, rt = _parts(rhs)
  assert lz is None and rz is None
  lv, rv = _storage(lv), _storage(rv)
  lca, rca = dimension_numbers[0]
  counts = []
  for l, r in zip(lca, rca):
    a, b = lt.get(l), rt.get(r)
    if a and b and a != b:
      raise ValueError(
          'Contracting axes must be tiled with the same tile size.'
          f' lhs_tiled_axes={lt} rhs_tiled_axes={rt} {dimension_numbers=}')
    t = a or b
    counts.append(lv.shape[l] // t if t else 1)
  acc_t, res_t = qarray.get_accumulator_and_result_type(
      lhs, rhs, preferred_element_type=preferred_element_type)
  l_order, r_order = _scale_orders(dimension_numbers, (lv.ndim, rv.ndim))

  def cut(a, ca, idx):
    sel = []
    for i, s in enumerate(a.shape):
      if i not in ca or s == 1:
        sel.append(slice(None))
        continue
      j = list(ca).index(i)
      size = s // counts[j]
      sel.append(slice(idx[j] * size, (idx[j] + 1) * size))
    return a[tuple(sel)]

  acc = None
  for idx in itertools.product(*map(range, counts)):
    out = lax_dot_general(cut(lv, lca, idx), cut(rv, rca, idx),
                          dimension_numbers, acc_t)
    if ls is not None:
      out = _mul(out, qarray.transpose_array(cut(ls, lca, idx), l_order))
    if rs is not None:
      out = _mul(out, qarray.transpose_array(cut(rs, rca, idx), r_order))
    acc = out if acc is None else acc + out
  return acc.astype(res_t)


def use_fast_path(lhs, rhs, dimension_numbers) -> bool:
  """The path choice of dot_general.py:442-472."""
  for operand, ca in zip((lhs, rhs), dimension_numbers[0]):
    if not isinstance(operand, QArray):
      if numerics.should_quantize(operand.dtype):
        return False
      continue
    qarray.validate_qarray(operand)
    if not numerics.can_dequant_on_output(operand.qtype):
      return False
    for axis in ca:
      if operand.scale.shape[axis] > 1:
        tile = operand.qvalue.shape[axis] // operand.scale.shape[axis]
        if tile < MIN_TILE_SIZE_TO_DEQUANT_ON_OUTPUT:
          return False
  return True


def dot_general(lhs, rhs, dimension_numbers, precision=None,
                preferred_element_type=None):
  """dot_general.py:407-491 without the mxfp probe (not on this path)."""
  del precision
  fn = fast_dot_general if use_fast_path(lhs, rhs, dimension_numbers) \
      else slow_dot_general
  return fn(lhs, rhs, dimension_numbers,
            preferred_element_type=preferred_element_type)
