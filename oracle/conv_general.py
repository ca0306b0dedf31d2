"""Oracle for the quantized conv_general_dilated, [N, spatial..., C] x [spatial..., C, O].

Test infrastructure only.  Restates qwix/_src/core/conv_general.py:26-269: channelwise scales
over the batch axis of the input and the out-feature axis of the filter (:26-52); the fast path
convolves the codes in the accumulator type, multiplies by the input's scales and then by the
filter's (:146-190) and casts (:192); the slow path dequantizes first (:69-100).  The
convolution itself (jax.lax.conv_general_dilated, third-party, unpinned in
pyproject.toml:20-27) is restated as a sum over window offsets with lax's 'SAME' / 'VALID' /
explicit padding rule: out[n, p, o] = sum_{w, c} x[n, p * stride + w * dilation - pad_lo, c] *
k[w, c, o], integer operands exactly (int32), floating ones in float32.
"""

from __future__ import annotations

import itertools
import math

import numpy as np

from oracle import dot_general as odg
from oracle import numerics
from oracle import qarray
from oracle.qarray import QArray


def get_how_to_quantize(*, for_lhs: bool, ndim: int, **kwargs) -> qarray.HowToQuantize:
  """conv_general.py:26-52 for the channels-last layouts: batch axis 0 of the input, out-feature
  axis (the last) of the filter."""
  return qarray.HowToQuantize(channelwise_axes=[0] if for_lhs else [ndim - 1], tiled_axes={}, **kwargs)


def explicit_padding(padding, in_sizes, windows, strides, dilations):
  if isinstance(padding, str):
    if padding.upper() == 'VALID':
      return [(0, 0)] * len(in_sizes)
    out = []
    for n, k, s, d in zip(in_sizes, windows, strides, dilations):
      eff = (k - 1) * d + 1
      total = max((math.ceil(n / s) - 1) * s + eff - n, 0)
      out.append((total // 2, total - total // 2))
    return out
  return [tuple(p) for p in padding]


def lax_conv(x: np.ndarray, k: np.ndarray, strides, padding, dilations, out_dtype) -> np.ndarray:
  ns = x.ndim - 2
  windows = k.shape[:ns]
  dil = list(dilations) if dilations is not None else [1] * ns
  pads = explicit_padding(padding, x.shape[1:1 + ns], windows, strides, dil)
  both_int = 'int' in x.dtype.name and 'int' in k.dtype.name
  work = np.float64 if both_int else np.float32
  xp = np.pad(x.astype(work), [(0, 0)] + pads + [(0, 0)])
  outs = [(xp.shape[1 + i] - ((windows[i] - 1) * dil[i] + 1)) // strides[i] + 1 for i in range(ns)]
  acc = np.zeros([x.shape[0]] + outs + [k.shape[-1]], dtype=work)
  kw = k.astype(work)
  for w in itertools.product(*[range(n) for n in windows]):
    sl = [slice(None)]
    for i in range(ns):
      start = w[i] * dil[i]
      sl.append(slice(start, start + (outs[i] - 1) * strides[i] + 1, strides[i]))
    acc += xp[tuple(sl)] @ kw[w]
  if 'int' in np.dtype(out_dtype).name:
    return acc.astype(np.int64).astype(out_dtype)
  return acc.astype(out_dtype)


def _parts(x):
  if isinstance(x, QArray):
    return odg._storage(x.qvalue), x.scale, x.zero_point
  return x, None, None


def fast_conv(lhs, rhs, window_strides, padding, rhs_dilation=None, preferred_element_type=None):
  """conv_general.py:103-192 (symmetric operands)."""
  lv, ls, lz = _parts(lhs)
  rv, rs, rz = _parts(rhs)
  for x in (lhs, rhs):
    if isinstance(x, QArray) and qarray.get_tiled_axes(x):
      raise ValueError('subchannel is not supported for conv_general_dilated.')
  if rz is not None:
    raise ValueError('Asymmetric quantization for rhs is not supported.')
  assert lz is None, 'the zero-point term (:166-178) is not restated'
  acc_t, res_t = qarray.get_accumulator_and_result_type(
      lhs, rhs, preferred_element_type=preferred_element_type)
  res = lax_conv(lv, rv, list(window_strides), padding, rhs_dilation, acc_t)
  nd = res.ndim
  if ls is not None:     # [N, 1, .., 1] against [N, spatial, O]
    res = odg._mul(res, ls.reshape([ls.shape[0]] + [1] * (nd - 1)))
  if rs is not None:     # [1, .., 1, O]
    res = odg._mul(res, rs.reshape([1] * (nd - 1) + [rs.shape[-1]]))
  return res.astype(res_t)


def slow_conv(lhs, rhs, window_strides, padding, rhs_dilation=None, preferred_element_type=None):
  """conv_general.py:69-100."""
  lhs = qarray.dequantize(lhs) if isinstance(lhs, QArray) else lhs
  rhs = qarray.dequantize(rhs) if isinstance(rhs, QArray) else rhs
  out_t = preferred_element_type or qarray.jnp_result_type(lhs.dtype, rhs.dtype)
  return lax_conv(lhs, rhs, list(window_strides), padding, rhs_dilation, out_t)


def conv_general_dilated(lhs, rhs, window_strides, padding, rhs_dilation=None,
                         preferred_element_type=None):
  """conv_general.py:195-269."""
  fast = True
  for x in (lhs, rhs):
    if not isinstance(x, QArray) and numerics.should_quantize(x.dtype):
      fast = False
  fn = fast_conv if fast else slow_conv
  return fn(lhs, rhs, window_strides, padding, rhs_dilation, preferred_element_type)
