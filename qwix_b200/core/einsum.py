"""Quantized einsum: drop-in for the `_einsum_fn` hook (qwix/_src/core/einsum.py)."""

from __future__ import annotations

from typing import Any, Callable, Mapping

import torch

from qwix_b200.core import dot_general
from qwix_b200.core import einsum_info
from qwix_b200.core import qarray
from qwix_b200.core.qarray import QArray


def get_how_to_quantize(*, einsum_str: str, ndims: tuple[int, int], for_lhs: bool,
                        tile_size: Mapping[int, int | float] | int | float | None,
                        **kwargs: Any) -> qarray.HowToQuantize:
  """einsum.py:27-81 -- channelwise on non-contracted subscripts, optional sub-channel
  tiles on the last contracted one."""
  info = einsum_info.EinsumInfo.parse(einsum_str, ndims=ndims)
  subs = info.lhs if for_lhs else info.rhs
  channelwise, last_contract = [], None
  for axis, ch in enumerate(subs):
    if ch in info.contract_chars:
      last_contract = axis
    else:
      channelwise.append(axis)
  tiled = {}
  if isinstance(tile_size, Mapping):
    tiled = tile_size
    channelwise = [a for a in channelwise if a not in tiled]
  elif tile_size and last_contract is not None:
    tiled[last_contract] = tile_size
  return qarray.HowToQuantize(channelwise_axes=channelwise, tiled_axes=tiled, **kwargs)


def _binary(lhs, rhs, subs: str, dot_general_fn: Callable, preferred_element_type, **kwargs):
  info = einsum_info.EinsumInfo.parse(subs)
  out = dot_general_fn(lhs, rhs, info.dimension_numbers,
                       preferred_element_type=preferred_element_type, **kwargs)
  perm = info.output_perm
  return out if perm is None else out.permute(perm)


def einsum(*args, _qwix_dot_general=dot_general.dot_general, preferred_element_type=None,
           **kwargs) -> torch.Tensor:
  """einsum.py:106-188 -- einsum('subscripts', a, b) with QArray operands.

  One or two operands are supported (the provider only issues binary einsums); a single
  operand is dequantized and reduced with the library einsum, as in the reference.
  """
  kwargs.pop('out_sharding', None)
  kwargs.pop('precision', None)
  subs, *operands = args
  if not isinstance(subs, str):
    raise NotImplementedError('only the einsum("subscripts", *operands) form is supported.')
  _, preferred_element_type = qarray.get_accumulator_and_result_type(
      *operands, preferred_element_type=preferred_element_type)
  subs = einsum_info.normalize_subscripts(subs, [op.ndim for op in operands])
  ins, out = subs.split('->')
  terms = ins.split(',')
  operands = einsum_info.broadcast_operands(operands, terms)
  if len(operands) == 1:
    op = operands[0]
    op = qarray.dequantize(op) if isinstance(op, QArray) else op
    return torch.einsum(subs, op)
  if len(operands) != 2:
    raise NotImplementedError(
        f'einsum with {len(operands)} operands is not supported; contract pairwise.')
  lhs, rhs = operands
  # Subscripts that appear in one operand only and not in the output are summed first.
  for i, (term, other) in enumerate(((terms[0], terms[1]), (terms[1], terms[0]))):
    lonely = [c for c in term if c not in other and c not in out]
    if lonely:
      op = operands[i]
      op = qarray.dequantize(op) if isinstance(op, QArray) else op
      keep = ''.join(c for c in term if c not in lonely)
      operands[i] = torch.einsum(f'{term}->{keep}', op)
      terms[i] = keep
  lhs, rhs = operands
  return _binary(lhs, rhs, f'{terms[0]},{terms[1]}->{out}', _qwix_dot_general,
                 preferred_element_type, **kwargs)
