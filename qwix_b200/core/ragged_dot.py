"""Quantized ragged_dot (qwix/_src/core/ragged_dot.py:24-353): lhs [M, K] whose rows are cut
into consecutive groups, rhs [G, K, N] with one weight per group, out [M, N].

Every group is one contraction of its rows with its weight, so the groups run through
`dot_general` one after the other: the same tensor-core kernels, scales per row and per
(group, channel) applied in the GEMM epilogue (the reference multiplies the integer result by
the row scales and by the group's channel scales gathered per row, ragged_dot.py:196-222 --
row by row the same arithmetic).  Group sizes are read on the host (one synchronisation per
call).  Rows past the last group come out zero, as in jax.lax.ragged_dot.

Only the plain matrix form is built (`ragged_dot`, and `ragged_dot_general` with its dimension
numbers); `group_offset` and batched / transposed forms raise NotImplementedError.
"""

import dataclasses
from typing import Sequence

import torch

from qwix_b200.core import dot_general as dg
from qwix_b200.core import qarray
from qwix_b200.core.qarray import QArray


@dataclasses.dataclass(frozen=True)
class RaggedDotDimensionNumbers:
  """The fields of jax.lax.RaggedDotDimensionNumbers."""
  dot_dimension_numbers: tuple
  lhs_ragged_dimensions: Sequence[int]
  rhs_group_dimensions: Sequence[int]


# ragged_dot.py:24-28
_BASIC_RAGGED_DOT_DIMENSION_NUMBERS = RaggedDotDimensionNumbers(
    dot_dimension_numbers=(((1,), (1,)), ((), ())),
    lhs_ragged_dimensions=[0],
    rhs_group_dimensions=[0],
)


def _is_basic(dn: RaggedDotDimensionNumbers) -> bool:
  (lca, rca), (lba, rba) = dn.dot_dimension_numbers
  return (tuple(lca) == (1,) and tuple(rca) == (1,) and not tuple(lba) and not tuple(rba)
          and list(dn.lhs_ragged_dimensions) == [0] and list(dn.rhs_group_dimensions) == [0])


def _shape(x):
  return tuple(x.qvalue.shape) if isinstance(x, QArray) else tuple(x.shape)


def ragged_dot_general(lhs, rhs, group_sizes, dimension_numbers: RaggedDotDimensionNumbers,
                       precision=None, preferred_element_type=None, group_offset=None) -> torch.Tensor:
  """ragged_dot.py:225-297."""
  del precision
  if group_offset is not None:
    raise NotImplementedError('group_offset is not built.')
  if not _is_basic(dimension_numbers):
    raise NotImplementedError('only the [M, K] x [G, K, N] form of ragged_dot is built.')
  lshape, rshape = _shape(lhs), _shape(rhs)
  if len(lshape) != 2 or len(rshape) != 3 or lshape[1] != rshape[1]:
    raise ValueError(f'ragged_dot expects lhs [M, K] and rhs [G, K, N], got {lshape} and {rshape}.')
  M, (G, _, N) = lshape[0], rshape
  sizes = [int(s) for s in (group_sizes.tolist() if isinstance(group_sizes, torch.Tensor) else group_sizes)]
  if len(sizes) != G or any(s < 0 for s in sizes) or sum(sizes) > M:
    raise ValueError(f'group_sizes {sizes} do not fit {G} groups over {M} rows.')
  _, res_t = qarray.get_accumulator_and_result_type(lhs, rhs, preferred_element_type=preferred_element_type)
  device = (lhs.qvalue if isinstance(lhs, QArray) else lhs).device
  out = torch.zeros((M, N), dtype=res_t, device=device)
  dn = (((1,), (0,)), ((), ()))
  row = 0
  for g, size in enumerate(sizes):
    if size:
      out[row:row + size] = dg.dot_general(lhs[row:row + size], rhs[g], dn,
                                           preferred_element_type=preferred_element_type)
    row += size
  return out


def ragged_dot(lhs, rhs, group_sizes, precision=None, preferred_element_type=None,
               group_offset=None) -> torch.Tensor:
  """ragged_dot.py:320-353."""
  return ragged_dot_general(lhs, rhs, group_sizes, _BASIC_RAGGED_DOT_DIMENSION_NUMBERS,
                            precision=precision, preferred_element_type=preferred_element_type,
                            group_offset=group_offset)
