"""Oracle for the quantized ragged_dot.

Test infrastructure only.  Restates qwix/_src/core/ragged_dot.py:118-353 for the plain form
lhs [M, K] x rhs [G, K, N]: the fast path contracts the codes of every row with the codes of
its group's weight, multiplies by the row's scale and by the group's channel scales (gathered
per row with a ragged dot of ones, :31-57, :196-222) and sums the K tiles (:224-225); the slow
path dequantizes first (:230-243).  Row by row that is `dot_general` of the row with its
group's weight, which is how it is restated here.  `jax.lax.ragged_dot_general` itself is
third-party (jax, unpinned in pyproject.toml:20-27): rows outside every group are zero.
"""

from __future__ import annotations

import numpy as np

from oracle import dot_general as odg
from oracle import numerics
from oracle import qarray
from oracle.qarray import QArray


def use_fast_path(lhs, rhs) -> bool:
  """ragged_dot.py:275-285."""
  for operand in (lhs, rhs):
    if isinstance(operand, QArray):
      if operand.zero_point is not None:
        return False
    elif numerics.should_quantize(operand.dtype):
      return False
  return True


def _take0(aux, full, sel):
  """Index axis 0 of a scale / zero point whose axis 0 is either broadcast (1) or full."""
  if aux is None:
    return None
  if aux.shape[0] == 1:
    return aux if isinstance(sel, slice) else aux[0]
  assert aux.shape[0] == full, 'axis 0 of the scale is tiled: not a form this oracle restates'
  return aux[sel]


def _rows(x, a, b):
  """Rows a..b of the lhs (qarray.py:173-209 for a slice of axis 0)."""
  if isinstance(x, QArray):
    m = x.qvalue.shape[0]
    return QArray(x.qvalue[a:b], _take0(x.scale, m, slice(a, b)), _take0(x.zero_point, m, slice(a, b)),
                  x.qtype)
  return x[a:b]


def _group(x, g):
  """The weight of group g (qarray.py:173-209 for an integer index on axis 0)."""
  if isinstance(x, QArray):
    n = x.qvalue.shape[0]
    return QArray(x.qvalue[g], _take0(x.scale, n, g), _take0(x.zero_point, n, g), x.qtype)
  return x[g]


def ragged_dot(lhs, rhs, group_sizes, preferred_element_type=None) -> np.ndarray:
  lshape = lhs.qvalue.shape if isinstance(lhs, QArray) else lhs.shape
  rshape = rhs.qvalue.shape if isinstance(rhs, QArray) else rhs.shape
  M, N = lshape[0], rshape[2]
  _, result_type = qarray.get_accumulator_and_result_type(
      lhs, rhs, preferred_element_type=preferred_element_type)
  out = np.zeros((M, N), dtype=result_type)
  dn = (((1,), (0,)), ((), ()))
  fn = odg.fast_dot_general if use_fast_path(lhs, rhs) else odg.slow_dot_general
  row = 0
  for g, size in enumerate(group_sizes):
    if size:
      out[row:row + size] = fn(_rows(lhs, row, row + size), _group(rhs, g), dn,
                               preferred_element_type=preferred_element_type)
    row += size
  return out
