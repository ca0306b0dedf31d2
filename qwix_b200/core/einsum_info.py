"""Binary-einsum bookkeeping: which axes contract, which are batch, output order.

Host logic with the behaviour of qwix/_src/core/einsum_info.py:27-241.  The reference
lets opt_einsum expand ellipses and implicit outputs; that dependency is replaced by the
small parser below (same NumPy einsum conventions).
"""

from __future__ import annotations

import dataclasses
import re
import string
from typing import Any, Sequence

from qwix_b200.core import qarray


def normalize_subscripts(einsum_str: str, ndims: Sequence[int]) -> str:
  """Spells out '...' and a missing '->out' for operands of the given ranks."""
  s = einsum_str.replace(' ', '')
  ins, arrow, out = s.partition('->')
  terms = ins.split(',')
  if len(terms) != len(ndims):
    raise ValueError(f'{einsum_str!r} names {len(terms)} operands, got {len(ndims)}.')
  used = {c for c in s if c.isalpha()}
  spare = [c for c in reversed(string.ascii_letters) if c not in used]
  widest = max([nd - (len(t) - 3) for t, nd in zip(terms, ndims) if '...' in t] or [0])
  ell = ''.join(reversed(spare[:widest]))
  fixed = []
  for t, nd in zip(terms, ndims):
    if '...' in t:
      n = nd - (len(t) - 3)
      if n < 0:
        raise ValueError(f'operand of rank {nd} is too small for {t!r}.')
      t = t.replace('...', ell[len(ell) - n:] if n else '')
    fixed.append(t)
  if arrow:
    out = out.replace('...', ell)
  else:
    joined = ''.join(fixed)
    out = ell + ''.join(sorted(c for c in set(joined) if joined.count(c) == 1 and c not in ell))
  return ','.join(fixed) + '->' + out


@dataclasses.dataclass(slots=True)
class EinsumInfo:
  """einsum_info.py:27-174 -- 'abc,bcd->acd': a free, b contracted, c batch, d free."""

  lhs: str
  rhs: str
  out: str

  @classmethod
  def parse(cls, einsum_str: str, ndims: tuple[int, int] | None = None) -> 'EinsumInfo':
    if ndims is not None:
      einsum_str = normalize_subscripts(einsum_str, ndims)
    s = einsum_str.replace(' ', '')
    if not re.match(r'^[a-zA-Z]*,[a-zA-Z]*->[a-zA-Z]*$', s):
      raise NotImplementedError(
          f'Unsupported einsum string: "{s}". EinsumInfo only supports binary einsums '
          'with explicit output subscripts (e.g., "abc,bcd->acd").')
    ins, out = s.split('->')
    lhs, rhs = ins.split(',')
    for name, subs in (('lhs', lhs), ('rhs', rhs), ('out', out)):
      if len(set(subs)) != len(subs):
        raise NotImplementedError(
            f'Repeated indices in {name} ("{subs}") are not supported. '
            f'Einsum string: "{s}".')
    return cls(lhs, rhs, out)

  @property
  def batch_chars(self) -> list[str]:
    return sorted(set(self.lhs) & set(self.rhs) & set(self.out))

  @property
  def contract_chars(self) -> list[str]:
    return sorted((set(self.lhs) & set(self.rhs)) - set(self.out))

  @property
  def dimension_numbers(self):
    li = {c: i for i, c in enumerate(self.lhs)}
    ri = {c: i for i, c in enumerate(self.rhs)}
    cc, bc = self.contract_chars, self.batch_chars
    return ((tuple(li[c] for c in cc), tuple(ri[c] for c in cc)),
            (tuple(li[c] for c in bc), tuple(ri[c] for c in bc)))

  @property
  def output_perm(self) -> tuple[int, ...] | None:
    """Permutation from dot_general's (batch, lhs free, rhs free) order to `out`."""
    bc = self.batch_chars
    produced = bc + [c for c in self.lhs if c in self.out and c not in bc] + \
        [c for c in self.rhs if c in self.out and c not in bc]
    at = {c: i for i, c in enumerate(produced)}
    perm = tuple(at[c] for c in self.out)
    return None if perm == tuple(range(len(perm))) else perm


def sanitize_shape(shape: Sequence[int | Any]) -> tuple[int, ...]:
  """einsum_info.py:177-194."""
  return tuple(s if isinstance(s, int) else 1 for s in shape)


def broadcast_operands(operands, operand_subs_list: Sequence[str]) -> list:
  """einsum_info.py:197-241 -- grow size-1 (or dividing) extents to the shared size."""
  sizes: dict[str, int] = {}
  for op, subs in zip(operands, operand_subs_list):
    for i, ch in enumerate(subs):
      n = op.shape[i]
      have = sizes.get(ch)
      if have is None or have == 1 or (n > have and n % have == 0):
        sizes[ch] = n
  return [qarray.broadcast_to(op, tuple(sizes[c] for c in subs))
          for op, subs in zip(operands, operand_subs_list)]
