"""Oracle for the block-scaled (microscaled) dot_general.

Test infrastructure only: nothing outside tests/, the smoke check and the benchmark's CPU leg
may import this.  Restates qwix/_src/core/mxfp_dot.py:24-163.  The contraction itself lives in
a third-party dependency that is absent here (`jax.nn.scaled_matmul`; jax is listed in the
reference's pyproject.toml:20-27 without a version pin), so its arithmetic is restated from the
reference's own test double for it, `reference_scaled_matmul`
(tests/_src/core/mxfp_dot_test.py:78-103): every 32-wide block of an operand row is multiplied
by its scale, the scaled operands are contracted in float32.  Parity of the contraction is
therefore pinned on that test double and on its tolerance (rtol = atol = 5e-3, :167), not on
outputs of the library call.
"""

from __future__ import annotations

import math

import numpy as np

from oracle import qarray
from oracle.qarray import QArray

MXFP_QTYPES = ('mxfp8', 'mxfp8_16', 'mxfp4', 'nvfp4')


def is_mxfp(operand) -> bool:
  """mxfp_dot.py:82-89."""
  return isinstance(operand, QArray) and operand.qtype in MXFP_QTYPES


def flatten_to_3d(operand: QArray, ca, ba):
  """mxfp_dot.py:106-137 -- codes [B, F, K], scales [B, F, K / block]."""
  val, scale = operand.qvalue, operand.scale
  ndim = val.ndim
  free = [i for i in range(ndim) if i not in ca and i not in ba]
  perm = list(ba) + free + list(ca)
  B = math.prod(val.shape[a] for a in ba)
  F = math.prod(val.shape[a] for a in free)
  K = math.prod(val.shape[a] for a in ca)
  val3 = np.transpose(val, perm).reshape(B, F, K)
  full = [scale.shape[i] if i in ca else val.shape[i] for i in range(ndim)]
  scale = np.broadcast_to(scale, full)
  Ks = math.prod(scale.shape[a] for a in ca)
  return val3, np.transpose(scale, perm).reshape(B, F, Ks)


def inputs_compatible(lv, rv, ls, rs) -> bool:
  """mxfp_dot.py:90-103."""
  return (lv.shape[0] == rv.shape[0] and lv.shape[2] == rv.shape[2]
          and ls.shape[0] == rs.shape[0] and ls.shape[2] == rs.shape[2])


def scaled_matmul(lhs, rhs, lhs_scale, rhs_scale) -> np.ndarray:
  """tests/_src/core/mxfp_dot_test.py:78-103: lhs [B, M, K], rhs [B, N, K], scales
  [B, M | N, K / block]; float32 result [B, M, N]."""
  B, M, K = lhs.shape
  N = rhs.shape[1]
  block = K // lhs_scale.shape[-1]
  lf = (lhs.astype(np.float32).reshape(B, M, -1, block) *
        lhs_scale.astype(np.float32)[..., None]).reshape(B, M, K)
  rf = (rhs.astype(np.float32).reshape(B, N, -1, block) *
        rhs_scale.astype(np.float32)[..., None]).reshape(B, N, K)
  return np.einsum('bmk,bnk->bmn', lf, rf, dtype=np.float32)


def mxfp_dot_general(lhs, rhs, dimension_numbers, preferred_element_type=None):
  """mxfp_dot.py:24-79; None when the reference would fall back."""
  if not (is_mxfp(lhs) and is_mxfp(rhs)):
    return None
  (lca, rca), (lba, rba) = dimension_numbers
  lv, ls = flatten_to_3d(lhs, list(lca), list(lba))
  rv, rs = flatten_to_3d(rhs, list(rca), list(rba))
  if not inputs_compatible(lv, rv, ls, rs):
    return None
  _, result_type = qarray.get_accumulator_and_result_type(
      lhs, rhs, preferred_element_type=preferred_element_type)
  out = scaled_matmul(lv, rv, ls, rs).astype(result_type)
  # mxfp_dot.py:140-163
  bshape = [lhs.qvalue.shape[i] for i in lba]
  lfree = [lhs.qvalue.shape[i] for i in range(lhs.qvalue.ndim) if i not in lca and i not in lba]
  rfree = [rhs.qvalue.shape[i] for i in range(rhs.qvalue.ndim) if i not in rca and i not in rba]
  return out.reshape(bshape + lfree + rfree)
