"""Small module library whose contractions go through qwix_b200.ops.

Stands in for the Flax layers the reference quantizes (flax.linen.Dense issues
jax.lax.dot_general on a [in, out] `kernel`; DenseGeneral / Einsum issue einsums).
Weights keep Flax's layout and names so that param trees line up with the reference's.
"""

from __future__ import annotations

import math
from typing import Sequence

import torch

from qwix_b200 import ops


def lecun_normal_(t: torch.Tensor, fan_in: int, generator=None) -> torch.Tensor:
  """flax's default kernel init: truncated normal (+/-2 sigma), variance 1 / fan_in."""
  std = math.sqrt(1.0 / fan_in) / 0.87962566103423978
  with torch.no_grad():
    torch.nn.init.trunc_normal_(t, mean=0.0, std=std, a=-2 * std, b=2 * std,
                                generator=generator)
  return t


class Dense(torch.nn.Module):
  """y = x @ kernel (+ bias); kernel is [in_features, features] like flax.linen.Dense."""

  def __init__(self, in_features: int, features: int, use_bias: bool = True,
               dtype=torch.float32, device=None, generator=None):
    super().__init__()
    self.kernel = torch.nn.Parameter(
        lecun_normal_(torch.empty(in_features, features, dtype=dtype, device=device),
                      in_features, generator), requires_grad=False)
    self.bias = torch.nn.Parameter(torch.zeros(features, dtype=dtype, device=device),
                                   requires_grad=False) if use_bias else None

  def forward(self, x):
    y = ops.dot_general(x, self.kernel, (((x.ndim - 1,), (0,)), ((), ())))
    return y if self.bias is None else y + self.bias


class Einsum(torch.nn.Module):
  """y = einsum(subscripts, x, kernel) with a weight of the given shape."""

  def __init__(self, subscripts: str, shape: Sequence[int], fan_in: int | None = None,
               dtype=torch.float32, device=None, generator=None):
    super().__init__()
    self.subscripts = subscripts
    self.kernel = torch.nn.Parameter(
        lecun_normal_(torch.empty(*shape, dtype=dtype, device=device),
                      fan_in or shape[0], generator), requires_grad=False)

  def forward(self, x):
    return ops.einsum(self.subscripts, x, self.kernel)


class Conv(torch.nn.Module):
  """Channels-last convolution, y = conv(x [N, spatial..., C], kernel [window..., C, features])
  (+ bias): the layout and defaults of flax.linen.Conv ('SAME' padding, unit strides)."""

  def __init__(self, in_features: int, features: int, kernel_size: Sequence[int],
               strides: Sequence[int] | None = None, padding='SAME', use_bias: bool = True,
               dtype=torch.float32, device=None, generator=None):
    super().__init__()
    self.kernel_size = tuple(kernel_size)
    self.strides = tuple(strides) if strides is not None else (1,) * len(self.kernel_size)
    self.padding = padding
    fan_in = in_features
    for k in self.kernel_size:
      fan_in *= k
    self.kernel = torch.nn.Parameter(
        lecun_normal_(torch.empty(*self.kernel_size, in_features, features, dtype=dtype, device=device),
                      fan_in, generator), requires_grad=False)
    self.bias = torch.nn.Parameter(torch.zeros(features, dtype=dtype, device=device),
                                   requires_grad=False) if use_bias else None

  def forward(self, x):
    ns = len(self.kernel_size)
    layouts = ('NHWC', 'HWIO', 'NHWC') if ns == 2 else ('NWC', 'WIO', 'NWC')
    y = ops.conv_general_dilated(x, self.kernel, self.strides, self.padding,
                                 dimension_numbers=layouts)
    return y if self.bias is None else y + self.bias.to(y.dtype)
