"""GPU parity at the sizes the benchmark times.

The small-shape tests elsewhere give every CTA one tile; the timed workloads give a persistent
CTA (or CTA pair) several, so the tile loop, the accumulator ping-pong, the phase flips of the
shared-memory ring across tiles and the scheduler's tail run only at full size.  Here the CUDA
path runs the whole problem and the oracle recomputes a sample of its rows (or columns), which
keeps the CPU side to seconds: per-token activation scales make rows independent, per-channel
weight scales make columns independent, and an integer contraction of a row sample against
the device's own codes is an exact float64 BLAS product (all |sums| < 2^53).
"""

import ml_dtypes
import numpy as np
import pytest
import torch

from oracle import dot_general as odg
from oracle import hadamard as ohd
from oracle import qarray as oq
from qwix_b200 import _lib
from qwix_b200.contrib import hadamard as bhd
from qwix_b200.core import dot_general as bdg
from qwix_b200.core import qarray as bq
from tests import helpers as h

pytestmark = pytest.mark.gpu
bf16 = ml_dtypes.bfloat16
DN = (((1,), (0,)), ((), ()))


def _within(got, want):
  g, w = got.astype(np.float32), want.astype(np.float32)
  bad = np.abs(g - w) > 1e-2 + 2e-2 * np.abs(w)     # max-abs 1e-2 or rel 2e-2
  return not bad.any(), f'{bad.sum()} of {bad.size} outside 1e-2 / 2e-2, max {np.abs(g - w).max()}'


def _exact_int_product(a_codes: np.ndarray, b_codes_kn: np.ndarray) -> np.ndarray:
  return (a_codes.astype(np.float64) @ b_codes_kn.astype(np.float64)).astype(np.int64)


def test_w8a8_prefill_full_size():
  """A [4096, 8192] with 1 % outlier columns x W [8192, 8192]: 512 CTA-pair tiles on 74 pairs,
  about seven tiles per pair."""
  M, K, N = 4096, 8192, 8192
  rng = np.random.default_rng(0)
  a = rng.standard_normal((M, K), dtype=np.float32)
  a[:, np.random.default_rng(1).choice(K, K // 100, replace=False)] *= 20.0
  a = a.astype(bf16)
  w = (0.02 * np.random.default_rng(2).standard_normal((K, N), dtype=np.float32)).astype(bf16)
  kw = dict(dimension_numbers=DN, ndims=(2, 2), tile_size=None, qtype='int8')
  aq = bq.quantize(h.to_torch(a), bdg.get_how_to_quantize(for_lhs=True, **kw))
  wq = bq.quantize(h.to_torch(w), bdg.get_how_to_quantize(for_lhs=False, **kw))

  # 4 rows of every 256-row pair tile, one per 64-row band so that both CTAs of a pair and
  # several epilogue warps are looked at: 64 rows over the 16 row tiles
  rows = np.array([t * 256 + b * 64 + (7 * t + 13 * b) % 64 for t in range(16) for b in range(4)])
  cols = np.random.default_rng(3).choice(N, 512, replace=False)

  a_o = oq.quantize(a[rows], odg.get_how_to_quantize(for_lhs=True, **kw))
  assert h.codes_equal(aq.qvalue[torch.as_tensor(rows, device='cuda')], a_o.qvalue)
  assert np.array_equal(h.to_numpy(aq.scale)[rows].view(np.uint8), a_o.scale.view(np.uint8))
  w_o = oq.quantize(w[:, cols], odg.get_how_to_quantize(for_lhs=False, **kw))
  assert h.codes_equal(wq.qvalue[:, torch.as_tensor(cols, device='cuda')], w_o.qvalue)
  assert np.array_equal(h.to_numpy(wq.scale)[:, cols].view(np.uint8), w_o.scale.view(np.uint8))

  w_codes = h.to_numpy(wq.qvalue)
  want_acc = _exact_int_product(a_o.qvalue, w_codes)
  acc = bdg.dot_general(aq.qvalue, wq.qvalue, DN)           # raw codes -> int32 accumulator
  assert acc.dtype == torch.int32
  assert np.array_equal(acc[torch.as_tensor(rows, device='cuda')].cpu().numpy().astype(np.int64), want_acc)

  out = bdg.dot_general(aq, wq, DN)
  _lib.raise_on_device_error()
  got = h.to_numpy(out[torch.as_tensor(rows, device='cuda')])
  w_full = oq.QArray(w_codes, h.to_numpy(wq.scale), None, 'int8')
  ok, msg = _within(got, odg.dot_general(a_o, w_full, DN))
  assert ok, msg
  # the step-by-step rounding of dot_general.py:255-261, bit for bit
  old = bdg.EPILOGUE
  try:
    bdg.EPILOGUE = 'reference'
    strict = bdg.dot_general(aq, wq, DN)
  finally:
    bdg.EPILOGUE = old
  want = odg.dot_general(a_o, w_full, DN)
  assert np.array_equal(h.to_numpy(strict[torch.as_tensor(rows, device='cuda')]).view(np.uint16),
                        want.view(np.uint16))


@pytest.mark.parametrize('layout', ['nk', 'kn'])
def test_lm_head_shape_many_tiles_per_cta(layout):
  """32 x 128256 x 4096: 501 output tiles of the single-CTA kernel on 148 persistent CTAs."""
  M, N, K = 32, 128256, 4096
  rng = np.random.default_rng(4)
  a = rng.integers(-128, 128, (M, K), dtype=np.int8)
  b = rng.integers(-128, 128, (K, N), dtype=np.int8)
  want = _exact_int_product(a, b)
  bt = h.to_torch(b)
  if layout == 'nk':
    bt = bt.t().contiguous().t()          # [K, N] view of [N, K] storage
  got = bdg.dot_general(h.to_torch(a), bt, DN)
  _lib.raise_on_device_error()
  assert got.dtype == torch.int32
  assert np.array_equal(got.cpu().numpy().astype(np.int64), want)


def test_k_tiled_more_tiles_than_ctas():
  """Sub-channel scales on both sides, 8 x 11 = 88 tiles of 256 x 256 on 74 CTA pairs."""
  M, K, N, tile = 2048, 1024, 2816, 256
  rng = np.random.default_rng(5)
  a = rng.standard_normal((M, K), dtype=np.float32).astype(bf16)
  w = (0.02 * rng.standard_normal((K, N), dtype=np.float32)).astype(bf16)
  kw = dict(dimension_numbers=DN, ndims=(2, 2), tile_size=tile, qtype='int8')
  a_o = oq.quantize(a, odg.get_how_to_quantize(for_lhs=True, **kw))
  w_o = oq.quantize(w, odg.get_how_to_quantize(for_lhs=False, **kw))
  aq = bq.quantize(h.to_torch(a), bdg.get_how_to_quantize(for_lhs=True, **kw))
  wq = bq.quantize(h.to_torch(w), bdg.get_how_to_quantize(for_lhs=False, **kw))
  assert h.codes_equal(aq.qvalue, a_o.qvalue) and h.codes_equal(wq.qvalue, w_o.qvalue)
  got = h.to_numpy(bdg.dot_general(aq, wq, DN))
  _lib.raise_on_device_error()
  # The reference rounds every tile's product to bf16 three times before the tile sum, so its
  # own result carries a few bf16 ulps of the largest tile term.  The float32 epilogue is held
  # to the stated tolerance against the same contraction with float32 scales; the
  # reference-order epilogue is held to the oracle itself (freedom left: the order of the
  # tile sum, one bf16 ulp).
  import dataclasses
  wide = lambda q: dataclasses.replace(q, scale=q.scale.astype(np.float32))
  ok, msg = _within(got, odg.dot_general(wide(a_o), wide(w_o), DN))
  assert ok, msg
  old = bdg.EPILOGUE
  try:
    bdg.EPILOGUE = 'reference'
    strict = h.to_numpy(bdg.dot_general(aq, wq, DN)).astype(np.float32)
  finally:
    bdg.EPILOGUE = old
  want = odg.dot_general(a_o, w_o, DN).astype(np.float32)
  assert np.all(np.abs(strict - want) <= 2.0 ** -7 * np.maximum(np.abs(want), 2.0 ** -6))
  assert np.mean(strict == want) > 0.98


@pytest.mark.parametrize('tokens', [1, 16, 128])
def test_int4_weight_only_full_size(tokens):
  """W [8192, 28672] int4 with 128-wide scale tiles along K (float32 scales [64, 28672])."""
  K, N = 8192, 28672
  w = torch.randn(K, N, generator=torch.Generator().manual_seed(3)).mul_(0.02).to(torch.bfloat16)
  a = torch.randn(tokens, K, generator=torch.Generator().manual_seed(4)).to(torch.bfloat16)
  wq = bq.quantize_api(w.cuda(), 'int4', channelwise_axes=[1], tiled_axes={0: 128},
                       scale_dtype=torch.float32)
  got = bdg.dot_general(a.cuda(), wq, DN, preferred_element_type=torch.bfloat16)
  assert got.shape == (tokens, N)
  # columns are independent: two from each of 128 spread-out 16-channel groups, and the edges
  cols = np.unique(np.concatenate([np.arange(0, N, 224), np.arange(0, N, 224) + 9, [N - 1]]))
  w_np, a_np = h.to_numpy(w[:, cols]), h.to_numpy(a)
  w_o = oq.quantize_api(w_np, 'int4', channelwise_axes=[1], tiled_axes={0: 128},
                        scale_dtype=np.float32)
  ci = torch.as_tensor(cols, device='cuda')
  assert h.codes_equal(wq.qvalue[:, ci], w_o.qvalue)
  assert np.array_equal(h.to_numpy(wq.scale[:, ci]).view(np.uint8), w_o.scale.view(np.uint8))
  want = odg.dot_general(a_np, w_o, DN, preferred_element_type=bf16)
  ok, msg = _within(h.to_numpy(got[:, ci]), want)
  assert ok, msg


def test_mxfp8_block_scaled_full_size():
  """A [4096, 8192] x W [8192, 8192] under an mxfp8 rule: 32 x 37 tiles of 128 x 224, eight per
  CTA; the oracle recomputes a sample of rows against the device's weight codes."""
  from oracle import mxfp_dot as omx
  M, K, N = 4096, 8192, 8192
  a = np.random.default_rng(8).standard_normal((M, K), dtype=np.float32)
  a[:, np.random.default_rng(9).choice(K, K // 100, replace=False)] *= 20.0
  a = a.astype(bf16)
  w = (0.02 * np.random.default_rng(10).standard_normal((K, N), dtype=np.float32)).astype(bf16)
  kw = dict(dimension_numbers=DN, ndims=(2, 2), tile_size=32, qtype='mxfp8')
  aq = bq.quantize(h.to_torch(a), bdg.get_how_to_quantize(for_lhs=True, **kw))
  wq = bq.quantize(h.to_torch(w), bdg.get_how_to_quantize(for_lhs=False, **kw))
  out = bdg.dot_general(aq, wq, DN)
  _lib.raise_on_device_error()
  rows = np.array([t * 128 + (37 * t + 11) % 128 for t in range(32)])
  a_o = oq.quantize(a[rows], odg.get_how_to_quantize(for_lhs=True, **kw))
  ri = torch.as_tensor(rows, device='cuda')
  assert h.codes_equal(aq.qvalue[ri], a_o.qvalue)
  assert np.array_equal(h.to_numpy(aq.scale[ri]).view(np.uint8), a_o.scale.view(np.uint8))
  cols = np.random.default_rng(11).choice(N, 256, replace=False)
  w_o = oq.quantize(w[:, cols], odg.get_how_to_quantize(for_lhs=False, **kw))
  ci = torch.as_tensor(cols, device='cuda')
  assert h.codes_equal(wq.qvalue[:, ci], w_o.qvalue)
  assert np.array_equal(h.to_numpy(wq.scale[:, ci]).view(np.uint8),
                        np.ascontiguousarray(w_o.scale).view(np.uint8))
  w_full = oq.QArray(h.to_numpy(wq.qvalue), h.to_numpy(wq.scale), None, 'mxfp8')
  want = omx.mxfp_dot_general(a_o, w_full, DN).astype(np.float32)
  got = h.to_numpy(out[ri]).astype(np.float32)
  # float32 accumulation of exact block products, one rounding to bf16
  assert np.all(np.abs(got - want) <= 2.0 ** -7 * np.maximum(np.abs(want), 2.0 ** -6))
  assert np.mean(got == want) > 0.98


def test_hadamard_fp8_full_size():
  """A [8192, 4096] Student-t x W [4096, 14336]: 128-point blocks, e4m3 per row / per column."""
  M, K, N = 8192, 4096, 14336
  a = (0.5 * np.random.default_rng(5).standard_t(3, (M, K))).astype(np.float32).astype(bf16)
  w = (0.02 * np.random.default_rng(6).standard_normal((K, N), dtype=np.float32)).astype(bf16)
  wq = bhd.quantize_rotated_weight(h.to_torch(w))
  out = bhd.hadamard_quantize_multiply(h.to_torch(a), wq)
  _lib.raise_on_device_error()
  rows = np.array([t * 256 + b * 64 + (5 * t + 11 * b) % 64 for t in range(32) for b in range(4)])
  cols = np.random.default_rng(7).choice(N, 768, replace=False)
  want, _, _ = ohd.hadamard_quantized_matmul(a[rows], w[:, cols])
  got = h.to_numpy(out[torch.as_tensor(rows, device='cuda')][:, torch.as_tensor(cols, device='cuda')])
  g, r = got.astype(np.float32), want.astype(np.float32)
  assert np.linalg.norm(g - r) <= 1e-2 * np.linalg.norm(r)      # rel-L2 <= 1e-2
  exact = a[rows].astype(np.float32) @ w[:, cols].astype(np.float32)
  assert np.linalg.norm(g - exact) <= 6e-2 * np.linalg.norm(exact)
