"""Quantized conv_general_dilated (qwix/_src/core/conv_general.py:26-269) for the layouts flax
uses: lhs [N, spatial..., C] ("NHWC"), rhs [spatial..., C, O] ("HWIO"), out [N, spatial..., O],
one or two spatial axes.

The fast path (both operands QArrays, or non-floating arrays) turns the integer convolution
into the tensor-core GEMM: the codes of the input are gathered into patches
[N * out positions, window * C] (an integer im2col with the padding's zeros), contracted with
the filter codes [window * C, O] in int32, and scaled by the per-image and per-output-channel
scales in the GEMM's epilogue -- the reference multiplies the integer result by the two
scales in the same order (:180-190).  The slow path dequantizes first and calls the library
convolution (:80-100).

Not built: lhs_dilation (transposed convolutions), feature / batch groups, other layouts and an
asymmetric input (its zero-point term is one more integer convolution, :166-178); they raise
NotImplementedError.
"""

import dataclasses
import math
from typing import Sequence

import torch
import torch.nn.functional as F

from qwix_b200.core import dot_general as dg
from qwix_b200.core import numerics
from qwix_b200.core import qarray
from qwix_b200.core.qarray import QArray


@dataclasses.dataclass(frozen=True)
class ConvDimensionNumbers:
  """jax.lax.ConvDimensionNumbers: (batch, feature, spatial...) positions per operand; for the
  kernel (out feature, in feature, spatial...)."""
  lhs_spec: tuple
  rhs_spec: tuple
  out_spec: tuple


def conv_dimension_numbers(lhs_shape, rhs_shape, dimension_numbers=None) -> ConvDimensionNumbers:
  """jax.lax.conv_dimension_numbers for None (the NCHW / OIHW default of lax), a
  ConvDimensionNumbers, or a triple of layout strings such as ('NHWC', 'HWIO', 'NHWC')."""
  nd = len(lhs_shape)
  if isinstance(dimension_numbers, ConvDimensionNumbers):
    return dimension_numbers
  if dimension_numbers is None:
    iota = tuple(range(nd))
    return ConvDimensionNumbers(iota, iota, iota)
  lhs, rhs, out = dimension_numbers
  spatial = [c for c in rhs if c not in 'OI']
  def spec(s, first, second):
    return (s.index(first), s.index(second)) + tuple(s.index(c) for c in spatial)
  return ConvDimensionNumbers(spec(lhs, 'N', 'C'), spec(rhs, 'O', 'I'), spec(out, 'N', 'C'))


def get_how_to_quantize(*, dimension_numbers: ConvDimensionNumbers, for_lhs: bool, **kwargs):
  """conv_general.py:26-52 -- channelwise over the batch axis (lhs) / the out-feature axis (rhs)."""
  axes = [dimension_numbers.lhs_spec[0]] if for_lhs else [dimension_numbers.rhs_spec[0]]
  return qarray.HowToQuantize(channelwise_axes=axes, tiled_axes={}, **kwargs)


def _is_channels_last(dn: ConvDimensionNumbers, nd: int) -> bool:
  sp = tuple(range(1, nd - 1))
  return (dn.lhs_spec == (0, nd - 1) + sp and dn.out_spec == (0, nd - 1) + sp
          and dn.rhs_spec == (nd - 1, nd - 2) + tuple(range(nd - 2)))


def _explicit_padding(padding, in_sizes, windows, strides, dilations):
  if isinstance(padding, str):
    if padding.upper() == 'VALID':
      return [(0, 0)] * len(in_sizes)
    if padding.upper() != 'SAME':
      raise ValueError(f'padding {padding!r}')
    out = []
    for n, k, s, d in zip(in_sizes, windows, strides, dilations):
      eff = (k - 1) * d + 1
      total = max((math.ceil(n / s) - 1) * s + eff - n, 0)
      out.append((total // 2, total - total // 2))
    return out
  return [tuple(p) for p in padding]


def _patches(x: torch.Tensor, windows, strides, pads, dilations) -> torch.Tensor:
  """[N, spatial..., C] -> [N, out positions..., window..., C] by strided views (any dtype)."""
  ns = len(windows)
  flat = []
  for lo, hi in reversed(pads):
    flat += [lo, hi]
  x = F.pad(x, [0, 0] + flat) if any(flat) else x
  for i, (k, s, d) in enumerate(zip(windows, strides, dilations)):
    eff = (k - 1) * d + 1
    x = x.unfold(1 + i, eff, s)                 # window axis appended last
    if d > 1:
      x = x[..., ::d]
  # now [N, out..., C, window...] -> [N, out..., window..., C]
  nd = x.ndim
  perm = list(range(1 + ns)) + list(range(nd - ns, nd)) + [1 + ns]
  return x.permute(perm)


def _check(lhs_dilation, feature_group_count, batch_group_count, dn, nd):
  if lhs_dilation is not None and any(d != 1 for d in lhs_dilation):
    raise NotImplementedError('lhs_dilation is not built.')
  if feature_group_count != 1 or batch_group_count != 1:
    raise NotImplementedError('grouped convolutions are not built.')
  if nd not in (3, 4) or not _is_channels_last(dn, nd):
    raise NotImplementedError('only [N, spatial, C] x [spatial, C, O] layouts are built.')


def _fast(lhs, rhs, window_strides, padding, rhs_dilation, dn, preferred_element_type):
  """conv_general.py:103-192."""
  for x in (lhs, rhs):
    if isinstance(x, QArray) and qarray.get_tiled_axes(x):
      raise ValueError('subchannel is not supported for conv_general_dilated.')
  if isinstance(rhs, QArray) and rhs.zero_point is not None:
    raise ValueError('Asymmetric quantization for rhs is not supported.')
  if isinstance(lhs, QArray) and lhs.zero_point is not None:
    raise NotImplementedError('an asymmetric input is not built for conv_general_dilated.')
  lv = lhs.qvalue if isinstance(lhs, QArray) else lhs
  rv = rhs.qvalue if isinstance(rhs, QArray) else rhs
  nd = lv.ndim
  ns = nd - 2
  windows = list(rv.shape[:ns])
  C, O = rv.shape[ns], rv.shape[ns + 1]
  strides = list(window_strides)
  dil = list(rhs_dilation) if rhs_dilation is not None else [1] * ns
  pads = _explicit_padding(padding, lv.shape[1:1 + ns], windows, strides, dil)
  p = _patches(lv, windows, strides, pads, dil)
  out_sp = list(p.shape[1:1 + ns])
  N = lv.shape[0]
  rows_per_image = math.prod(out_sp)
  a2 = p.reshape(N * rows_per_image, math.prod(windows) * C)
  b2 = rv.reshape(math.prod(windows) * C, O)
  # One GEMM row per output position: the image's scale repeats over its rows.
  def rows(q: QArray, codes2d):
    if q.scale.numel() == N:
      scale = q.scale.reshape(N, 1).expand(N, rows_per_image).reshape(-1, 1)
    else:
      scale = q.scale.reshape(1, 1)
    return QArray(codes2d.contiguous(), scale.contiguous(), None, q.qtype)
  l2 = rows(lhs, a2) if isinstance(lhs, QArray) else a2.contiguous()
  if isinstance(rhs, QArray):
    rs = rhs.scale.reshape(1, O) if rhs.scale.numel() == O else rhs.scale.reshape(1, 1)
    r2 = QArray(b2.contiguous(), rs.contiguous(), None, rhs.qtype)
  else:
    r2 = b2.contiguous()
  out = dg.dot_general(l2, r2, (((1,), (0,)), ((), ())), preferred_element_type=preferred_element_type)
  return out.reshape([N] + out_sp + [O])


def _slow(lhs, rhs, window_strides, padding, rhs_dilation, dn, preferred_element_type):
  """conv_general.py:69-100."""
  lhs = qarray.dequantize(lhs) if isinstance(lhs, QArray) else lhs
  rhs = qarray.dequantize(rhs) if isinstance(rhs, QArray) else rhs
  nd = lhs.ndim
  ns = nd - 2
  windows = list(rhs.shape[:ns])
  dil = list(rhs_dilation) if rhs_dilation is not None else [1] * ns
  pads = _explicit_padding(padding, lhs.shape[1:1 + ns], windows, list(window_strides), dil)
  dt = torch.promote_types(lhs.dtype, rhs.dtype)
  x = lhs.to(dt).movedim(-1, 1)                              # N, C, spatial
  w = rhs.to(dt).permute([ns + 1, ns] + list(range(ns)))     # O, C, window
  flat = []
  for lo, hi in reversed(pads):
    flat += [lo, hi]
  x = F.pad(x, flat) if any(flat) else x
  conv = F.conv1d if ns == 1 else F.conv2d
  out = conv(x, w, stride=tuple(window_strides), dilation=tuple(dil)).movedim(1, -1)
  return out.to(preferred_element_type) if preferred_element_type is not None else out


def conv_general_dilated(lhs, rhs, window_strides: Sequence[int], padding, lhs_dilation=None,
                         rhs_dilation=None, dimension_numbers=None, feature_group_count: int = 1,
                         batch_group_count: int = 1, precision=None, preferred_element_type=None,
                         out_sharding=None) -> torch.Tensor:
  """conv_general.py:195-269 -- drop-in for jax.lax.conv_general_dilated with QArray operands."""
  del precision, out_sharding
  lshape = tuple(lhs.qvalue.shape) if isinstance(lhs, QArray) else tuple(lhs.shape)
  rshape = tuple(rhs.qvalue.shape) if isinstance(rhs, QArray) else tuple(rhs.shape)
  dn = conv_dimension_numbers(lshape, rshape, dimension_numbers)
  _check(lhs_dilation, feature_group_count, batch_group_count, dn, len(lshape))
  fast = True
  for x in (lhs, rhs):
    if not isinstance(x, QArray) and numerics.should_quantize(x.dtype):
      fast = False
  fn = _fast if fast else _slow
  return fn(lhs, rhs, window_strides, padding, rhs_dilation, dn, preferred_element_type)
