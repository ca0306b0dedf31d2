"""Oracle einsum / dot front-ends over the oracle dot_general.

Test infrastructure only.  Restates qwix/_src/core/einsum_info.py:27-174,
einsum.py:27-188 (binary einsums, which is what the provider issues) and
dot.py:58-71.  The reference asks opt_einsum only to expand ellipses and to
order contractions; for two operands there is a single contraction, so the
expansion is done here directly.
"""

from __future__ import annotations

import re
import string
from typing import Mapping

import numpy as np

from oracle import dot_general as dg
from oracle import qarray
from oracle.qarray import QArray


def expand_ellipsis(einsum_str: str, ndims) -> str:
  """Spell out '...' and an implicit output, like np.einsum's parser."""
  s = einsum_str.replace(' ', '')
  ins, _, out = s.partition('->')
  terms = ins.split(',')
  used = set(c for c in s if c.isalpha())
  spare = [c for c in string.ascii_letters[::-1] if c not in used]
  longest = 0
  for t, nd in zip(terms, ndims):
    if '...' in t:
      longest = max(longest, nd - (len(t) - 3))
  ell = ''.join(spare[:longest])[::-1]
  fixed = []
  for t, nd in zip(terms, ndims):
    if '...' in t:
      n = nd - (len(t) - 3)
      t = t.replace('...', ell[len(ell) - n:] if n else '')
    fixed.append(t)
  if '->' not in s:
    joined = ''.join(fixed)
    out = ell + ''.join(sorted(c for c in set(joined)
                               if joined.count(c) == 1 and c not in ell))
  else:
    out = out.replace('...', ell)
  return ','.join(fixed) + '->' + out


class EinsumInfo:
  """einsum_info.py:27-174 -- a binary einsum as dot_general + permutation."""

  def __init__(self, lhs: str, rhs: str, out: str):
    self.lhs, self.rhs, self.out = lhs, rhs, out

  @classmethod
  def parse(cls, einsum_str: str, ndims=None) -> 'EinsumInfo':
    if ndims is not None:
      einsum_str = expand_ellipsis(einsum_str, ndims)
    s = einsum_str.replace(' ', '')
    if not re.match(r'^[a-zA-Z]*,[a-zA-Z]*->[a-zA-Z]*$', s):
      raise NotImplementedError(f'Unsupported einsum string: "{s}".')
    ins, out = s.split('->')
    lhs, rhs = ins.split(',')
    for name, subs in (('lhs', lhs), ('rhs', rhs), ('out', out)):
      if len(set(subs)) != len(subs):
        raise NotImplementedError(
            f'Repeated indices in {name} ("{subs}") are not supported.')
    return cls(lhs, rhs, out)

  @property
  def batch_chars(self):
    return sorted(set(self.lhs) & set(self.rhs) & set(self.out))

  @property
  def contract_chars(self):
    return sorted((set(self.lhs) & set(self.rhs)) - set(self.out))

  @property
  def dimension_numbers(self):
    li = {c: i for i, c in enumerate(self.lhs)}
    ri = {c: i for i, c in enumerate(self.rhs)}
    cc, bc = self.contract_chars, self.batch_chars
    return ((tuple(li[c] for c in cc), tuple(ri[c] for c in cc)),
            (tuple(li[c] for c in bc), tuple(ri[c] for c in bc)))

  @property
  def output_perm(self):
    bc = self.batch_chars
    cur = bc + [c for c in self.lhs if c in self.out and c not in bc] + \
        [c for c in self.rhs if c in self.out and c not in bc]
    pos = {c: i for i, c in enumerate(cur)}
    perm = tuple(pos[c] for c in self.out)
    return None if perm == tuple(range(len(perm))) else perm


def get_how_to_quantize(*, einsum_str, ndims, for_lhs, tile_size, **kwargs):
  """einsum.py:27-81."""
  info = EinsumInfo.parse(einsum_str, ndims=ndims)
  subs = info.lhs if for_lhs else info.rhs
  channelwise, last_contract = [], None
  for axis, ch in enumerate(subs):
    if ch in info.contract_chars:
      last_contract = axis
    else:
      channelwise.append(axis)
  tiled = {}
  if isinstance(tile_size, Mapping):
    tiled = dict(tile_size)
    channelwise = [a for a in channelwise if a not in tiled]
  elif tile_size and last_contract is not None:
    tiled[last_contract] = tile_size
  return qarray.HowToQuantize(channelwise_axes=channelwise, tiled_axes=tiled,
                              **kwargs)


def einsum(einsum_str: str, lhs, rhs, *, _qwix_dot_general=dg.dot_general,
           preferred_element_type=None):
  """einsum.py:106-188 for two operands whose shared extents already agree."""
  _, preferred_element_type = qarray.get_accumulator_and_result_type(
      lhs, rhs, preferred_element_type=preferred_element_type)
  s = expand_ellipsis(einsum_str, (lhs.ndim, rhs.ndim))
  info = EinsumInfo.parse(s)
  out = _qwix_dot_general(lhs, rhs, info.dimension_numbers,
                          preferred_element_type=preferred_element_type)
  perm = info.output_perm
  return out if perm is None else out.transpose(perm)


def dot(a, b, preferred_element_type=None, *, _qwix_dot_general=dg.dot_general):
  """dot.py:58-71."""
  if a.ndim == 0 or b.ndim == 0:
    contract = ((), ())
  elif b.ndim == 1:
    contract = ((a.ndim - 1,), (0,))
  else:
    contract = ((a.ndim - 1,), (b.ndim - 2,))
  return _qwix_dot_general(a, b, (contract, ((), ())),
                           preferred_element_type=preferred_element_type)
