"""The ops a model issues: plain when no provider is active, quantized otherwise.

In the reference the model calls jax.lax.dot_general / jnp.einsum / jnp.dot and the
interception layer redirects them (boxed_param.py:402-413).  Modules built on this
backend call these functions instead; the redirection is the same table lookup.
"""

from __future__ import annotations

import torch

from qwix_b200 import _context
from qwix_b200.core import dot_general as _dg


def _unbox(x):
  from qwix_b200.providers import ptq
  return ptq._plain(x)


def dot_general(lhs, rhs, dimension_numbers, precision=None, preferred_element_type=None):
  provider = _context.current_provider()
  if provider is None:
    return _dg._plain_dot_general(_unbox(lhs), _unbox(rhs), dimension_numbers,
                                  preferred_element_type)
  return provider.get_intercept_map()['dot_general'](
      lhs, rhs, dimension_numbers, precision, preferred_element_type)


def einsum(einsum_str: str, *operands, precision=None, preferred_element_type=None):
  provider = _context.current_provider()
  if provider is None:
    return torch.einsum(einsum_str, *[_unbox(o) for o in operands])
  return provider.get_intercept_map()['einsum'](
      einsum_str, *operands, precision=precision,
      preferred_element_type=preferred_element_type)


def dot(a, b, precision=None, preferred_element_type=None):
  provider = _context.current_provider()
  if provider is None:
    return torch.matmul(_unbox(a), _unbox(b))
  return provider.get_intercept_map()['dot'](a, b, precision, preferred_element_type)


def conv_general_dilated(lhs, rhs, window_strides, padding, lhs_dilation=None, rhs_dilation=None,
                         dimension_numbers=None, feature_group_count=1, batch_group_count=1,
                         precision=None, preferred_element_type=None):
  from qwix_b200.core import conv_general as _cg
  provider = _context.current_provider()
  if provider is None:
    return _cg.conv_general_dilated(_unbox(lhs), _unbox(rhs), window_strides, padding, lhs_dilation,
                                    rhs_dilation, dimension_numbers, feature_group_count,
                                    batch_group_count, precision, preferred_element_type)
  return provider.get_intercept_map()['conv_general_dilated'](
      lhs, rhs, window_strides, padding, lhs_dilation, rhs_dilation, dimension_numbers,
      feature_group_count, batch_group_count, precision, preferred_element_type)
