"""Quantized ragged_dot against the oracle (after tests/_src/core/ragged_dot_test.py:44-131:
lhs [128, 256], rhs [4, 256, 64], group sizes (64, 32, 16, 16), plus empty groups, rows outside
every group and a weight-only int4 form)."""

import dataclasses

import ml_dtypes
import numpy as np
import pytest
import torch

from oracle import qarray as oq
from oracle import ragged_dot as orr
from qwix_b200.core import qarray as bq
from qwix_b200.core import ragged_dot as brr
from tests import helpers as h

pytestmark = pytest.mark.gpu
bf16 = ml_dtypes.bfloat16


def _close(got, want):
  g, r = h.to_numpy(got).astype(np.float32), np.asarray(want).astype(np.float32)
  assert g.shape == r.shape
  bad = np.abs(g - r) > 1e-2 + 2e-2 * np.abs(r)
  assert not bad.any(), f'{bad.sum()} of {bad.size} outside 1e-2 / 2e-2, worst {np.abs(g - r).max()}'


CASES = [
    # name, lhs how, rhs how, group sizes
    ('int8 per tensor', dict(qtype='int8'), dict(qtype='int8'), (64, 32, 16, 16)),
    ('int8 per token, per group and channel', dict(qtype='int8', channelwise_axes=[0]),
     dict(qtype='int8', channelwise_axes=[0, 2]), (64, 32, 16, 16)),
    ('empty group and leftover rows', dict(qtype='int8', channelwise_axes=[0]),
     dict(qtype='int8', channelwise_axes=[0, 2]), (5, 0, 100, 7)),
    ('e4m3', dict(qtype='float8_e4m3fn', channelwise_axes=[0]),
     dict(qtype='float8_e4m3fn', channelwise_axes=[0, 2]), (40, 40, 40, 8)),
    ('sub-channel', dict(qtype='int8', channelwise_axes=[0], tiled_axes={1: 128}),
     dict(qtype='int8', channelwise_axes=[0, 2], tiled_axes={1: 128}), (64, 32, 16, 16)),
]


@pytest.mark.parametrize('case', CASES, ids=[c[0] for c in CASES])
@pytest.mark.parametrize('dtype', ['float32', 'bfloat16'])
def test_ragged_dot_matches_oracle(case, dtype):
  _, lhow, rhow, sizes = case
  rng = np.random.default_rng(len(sizes) + sum(sizes))
  x = rng.standard_normal((128, 256)).astype(np.float32).astype(h.np_dtype(dtype))
  w = (0.1 * rng.standard_normal((4, 256, 64))).astype(np.float32).astype(h.np_dtype(dtype))
  lo, ro = oq.quantize(x, oq.HowToQuantize(**lhow)), oq.quantize(w, oq.HowToQuantize(**rhow))
  lb = bq.quantize(h.to_torch(x), bq.HowToQuantize(**lhow))
  rb = bq.quantize(h.to_torch(w), bq.HowToQuantize(**rhow))
  assert h.codes_equal(lb.qvalue, lo.qvalue) and h.codes_equal(rb.qvalue, ro.qvalue)
  want = orr.ragged_dot(lo, ro, sizes)
  got = brr.ragged_dot(lb, rb, torch.tensor(sizes, device='cuda'))
  assert h.to_numpy(got).dtype == want.dtype
  if dtype == 'bfloat16' and 'tiled_axes' in lhow:
    # The reference rounds every K tile's product to bfloat16 three times before the tile sum,
    # so its own result carries a few bfloat16 ulps of the largest tile term; the float32
    # epilogue is held to the same contraction with float32 scales (as in test_gpu_gemm.py).
    wide = lambda q: dataclasses.replace(q, scale=q.scale.astype(np.float32))
    _close(got, orr.ragged_dot(wide(lo), wide(ro), sizes))
  else:
    _close(got, want)
  used = sum(sizes)
  assert not h.to_numpy(got)[used:].astype(np.float32).any()      # rows outside every group
  # quantization error against the float product, as the reference's test measures it
  ref = np.zeros((128, 64), np.float32)
  row = 0
  for g, s in enumerate(sizes):
    ref[row:row + s] = x[row:row + s].astype(np.float32) @ w[g].astype(np.float32)
    row += s
  g32 = h.to_numpy(got).astype(np.float32)
  assert np.abs(g32 - ref).mean() / np.abs(ref).mean() < 0.06


def test_weight_only_int4_groups():
  """bf16 rows against int4 group weights: the reference dequantizes first (ragged_dot.py:230-243)."""
  sizes = (3, 40, 0, 21)
  rng = np.random.default_rng(2)
  x = rng.standard_normal((64, 256)).astype(np.float32).astype(bf16)
  w = (0.05 * rng.standard_normal((4, 256, 128))).astype(np.float32).astype(bf16)
  how = dict(qtype='int4', channelwise_axes=[0, 2], tiled_axes={1: 128})
  ro = oq.quantize(w, oq.HowToQuantize(**how))
  rb = bq.quantize(h.to_torch(w), bq.HowToQuantize(**how))
  assert h.codes_equal(rb.qvalue, ro.qvalue)
  want = orr.ragged_dot(x, ro, sizes)
  got = brr.ragged_dot(h.to_torch(x), rb, list(sizes))
  _close(got, want)


def test_refusals():
  x = torch.zeros((8, 16), device='cuda')
  w = torch.zeros((2, 16, 4), device='cuda')
  with pytest.raises(NotImplementedError):
    brr.ragged_dot(x, w, [4, 4], group_offset=torch.zeros(1))
  with pytest.raises(ValueError):
    brr.ragged_dot(x, w, [4, 5])
  with pytest.raises(NotImplementedError):
    brr.ragged_dot_general(x, w, [4, 4], brr.RaggedDotDimensionNumbers((((1,), (2,)), ((), ())), [0], [0]))
  out = brr.ragged_dot(x, w, [4, 4])
  assert out.shape == (8, 4)
