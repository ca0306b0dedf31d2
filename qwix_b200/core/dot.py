"""Quantized jnp.dot equivalent (qwix/_src/core/dot.py:24-71)."""

from __future__ import annotations

from typing import Callable

from qwix_b200.core import dot_general


def dot(a, b, precision=None, preferred_element_type=None, out_sharding=None, *,
        _qwix_dot_general: Callable = dot_general.dot_general):
  """Contracts the last axis of `a` with the second-to-last (or only) axis of `b`."""
  if a.ndim == 0 or b.ndim == 0:
    contract = ((), ())
  elif b.ndim == 1:
    contract = ((a.ndim - 1,), (0,))
  else:
    contract = ((a.ndim - 1,), (b.ndim - 2,))
  return _qwix_dot_general(a, b, dimension_numbers=(contract, ((), ())), precision=precision,
                           preferred_element_type=preferred_element_type,
                           out_sharding=out_sharding)
