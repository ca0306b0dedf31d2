"""QArray-aware blocked kernel call: the host logic of qwix/_src/core/pallas.py:27-119.

A BlockSpec names, for every grid point, which block of an operand a kernel instance sees.
For a QArray operand the user gives the spec of the full-precision array; the spec of its
scale follows from it (block extent s // (v // bv), index 0 on extents of size 1).  The
TPU-only block-shape transform of the reference (pallas.py:122-207) has no counterpart here.

`pallas_call` runs the kernel body once per grid point on tensor views (what the
reference's tests do with interpret=True off-TPU).  Inside the body, qwix_b200.pallas.
dot_general / dot / einsum are the fused CUDA GEMMs.
"""

from __future__ import annotations

import dataclasses
import itertools
import threading
from typing import Any, Callable, Sequence

import torch

from qwix_b200.core import qarray


@dataclasses.dataclass(frozen=True)
class BlockSpec:
  """block_shape entries are extents, or None for a squeezed axis; index_map maps grid
  indices to block indices (the meaning of jax.experimental.pallas.BlockSpec)."""

  block_shape: tuple | None = None
  index_map: Callable[..., tuple] | None = None


def update_block_specs_for_qarray(block_specs: Any, args: Any) -> Any:
  """pallas.py:90-119 -- replace the spec of each QArray argument by a QArray of specs."""

  def one(spec, arg):
    if not isinstance(arg, qarray.QArray):
      return spec
    assert arg.zero_point is None, 'Zero point is not supported yet.'
    scale_shape = tuple(arg.scale.shape)
    block = []
    for v, bv, s in zip(arg.qvalue.shape, spec.block_shape, scale_shape):
      if bv is None:
        block.append(None)
      elif s == 1:
        block.append(1)
      else:
        assert v % bv == 0 and s % (v // bv) == 0, f'{v=} {bv=} {s=}'
        block.append(s // (v // bv))
    index_map = lambda *a: tuple(i if s > 1 else 0
                                 for i, s in zip(spec.index_map(*a), scale_shape))
    scale_spec = dataclasses.replace(spec, block_shape=tuple(block), index_map=index_map)
    return dataclasses.replace(arg, qvalue=spec, scale=scale_spec)

  if isinstance(block_specs, (list, tuple)):
    return type(block_specs)(one(s, a) for s, a in zip(block_specs, args))
  return one(block_specs, args)


def _take_block(x: torch.Tensor, spec: BlockSpec, grid_idx) -> torch.Tensor:
  if spec is None or spec.block_shape is None:
    return x
  idx = spec.index_map(*grid_idx)
  sel = []
  for i, b in zip(idx, spec.block_shape):
    sel.append(i if b is None else slice(i * b, (i + 1) * b))
  return x[tuple(sel)]


def _block_of(arg, spec, grid_idx):
  if isinstance(arg, qarray.QArray):
    return qarray.QArray(_take_block(arg.qvalue, spec.qvalue, grid_idx),
                         _take_block(arg.scale, spec.scale, grid_idx), None, arg.qtype)
  return _take_block(arg, spec, grid_idx)


_grid_state = threading.local()


def program_id(axis: int) -> int:
  """Index of the running kernel instance along grid axis `axis` (the role of
  jax.experimental.pallas.program_id inside a kernel body)."""
  idx = getattr(_grid_state, 'idx', None)
  if idx is None:
    raise RuntimeError('program_id is only defined inside a pallas_call kernel body.')
  return idx[axis]


def num_programs(axis: int) -> int:
  grid = getattr(_grid_state, 'grid', None)
  if grid is None:
    raise RuntimeError('num_programs is only defined inside a pallas_call kernel body.')
  return grid[axis]


def pallas_call(kernel: Callable[..., None], out_shape: Any, *, grid: Sequence[int] = (),
                in_specs: Sequence[BlockSpec] | None = None,
                out_specs: BlockSpec | Sequence[BlockSpec] | None = None,
                scratch_shapes: Sequence[tuple] = (), **kwargs):
  """pallas.py:27-87 -- returns a function of the operands; `out_shape` is a
  (shape, dtype) pair (or a sequence of them).  The kernel receives input blocks followed
  by output blocks and then one tensor per `scratch_shapes` entry (a (shape, dtype) pair:
  memory that lives across the grid, like the reference's VMEM scratch) and writes the
  outputs in place.  Grid points run in row-major order, the last axis fastest."""
  del kwargs
  single = isinstance(out_shape, tuple) and len(out_shape) == 2 and \
      isinstance(out_shape[1], torch.dtype)
  out_shapes = [out_shape] if single else list(out_shape)
  out_spec_list = [out_specs] if single else list(out_specs or [None] * len(out_shapes))

  def run(*args):
    specs = update_block_specs_for_qarray(list(in_specs or [None] * len(args)), list(args)) \
        if in_specs is not None else [None] * len(args)
    device = next(a.device for a in args if hasattr(a, 'device'))
    outs = [torch.empty(shape, dtype=dtype, device=device) for shape, dtype in out_shapes]
    scratch = [torch.empty(shape, dtype=dtype, device=device) for shape, dtype in scratch_shapes]
    _grid_state.grid = tuple(grid)
    try:
      for grid_idx in itertools.product(*[range(g) for g in grid]):
        _grid_state.idx = grid_idx
        ins = [_block_of(a, s, grid_idx) if s is not None else a for a, s in zip(args, specs)]
        blocks = [_take_block(o, s, grid_idx) for o, s in zip(outs, out_spec_list)]
        kernel(*ins, *blocks, *scratch)
    finally:
      _grid_state.idx = _grid_state.grid = None
    return outs[0] if single else tuple(outs)

  return run
