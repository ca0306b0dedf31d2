"""GPU parity: fused int4 weight-only GEMM (through the C ABI) vs the CPU oracle's
dequantize-then-dot path."""

import ml_dtypes
import numpy as np
import pytest
import torch

from oracle import dot_general as odg
from oracle import qarray as oq
from qwix_b200.core import dot_general as bdg
from qwix_b200.core import qarray as bq
from qwix_b200.core import weight_only
from tests import helpers as h

pytestmark = pytest.mark.gpu
DN = (((1,), (0,)), ((), ()))

CASES = [
    # M, K, N, tile, scale dtype
    (1, 512, 256, 128, 'float32'),
    (16, 512, 256, 128, 'float32'),
    (16, 1024, 384, 256, 'bfloat16'),
    (7, 4096, 1024, 128, 'float32'),      # more units than SMs: whole and split tiles mixed
    (128, 1024, 512, 128, 'float32'),
    (48, 512, 256, 512, 'bfloat16'),      # one scale per channel
    (200, 512, 256, 128, 'float32'),      # more than 128 tokens: two launches
    (16, 8192, 2048, 128, 'float32'),
    (16, 8192, 4096, 128, 'float32'),     # ~14 units per CTA: rings and operand slots wrap
    (128, 2048, 2048, 128, 'bfloat16'),   # 128 tokens, several units per CTA
    (3, 1024, 8192, 256, 'float32'),      # short tiles: a CTA crosses several tile segments
    (33, 512, 4096, 128, 'float32'),      # two launches: 32 tokens + 1 token
    (5, 14336, 512, 128, 'float32'),      # K / 128 = 112: slices must divide it
    (32, 8192, 1024 + 16, 128, 'bfloat16'),  # four K slices; N a multiple of 16 only
]


@pytest.mark.parametrize('case', CASES, ids=lambda c: 'x'.join(map(str, c)))
def test_a16w4_matches_oracle(case):
  M, K, N, tile, sdt = case
  rng = np.random.default_rng(M + K + N)
  w = (0.02 * rng.standard_normal((K, N))).astype(np.float32).astype(ml_dtypes.bfloat16)
  a = rng.standard_normal((M, K)).astype(np.float32).astype(ml_dtypes.bfloat16)
  sd = np.float32 if sdt == 'float32' else ml_dtypes.bfloat16
  wo = oq.quantize_api(w, 'int4', channelwise_axes=[1], tiled_axes={0: tile}, scale_dtype=sd)
  want = odg.dot_general(a, wo, DN, preferred_element_type=ml_dtypes.bfloat16)
  assert not odg.use_fast_path(a, wo, DN)  # the reference takes the dequantize-first path

  wq = bq.quantize_api(h.to_torch(w), 'int4', channelwise_axes=[1], tiled_axes={0: tile},
                       scale_dtype=torch.float32 if sdt == 'float32' else torch.bfloat16)
  assert h.codes_equal(wq.qvalue, wo.qvalue)
  assert np.array_equal(h.to_numpy(wq.scale).view(np.uint8), wo.scale.view(np.uint8))
  at = h.to_torch(a)
  assert weight_only.eligible(at, wq, DN)
  got = bdg.dot_general(at, wq, DN, preferred_element_type=torch.bfloat16)
  again = bdg.dot_general(at, wq, DN, preferred_element_type=torch.bfloat16)
  torch.cuda.synchronize()
  g = h.to_numpy(got).astype(np.float32)
  r = want.astype(np.float32)
  assert g.shape == r.shape
  bad = np.abs(g - r) > 1e-2 + 2e-2 * np.abs(r)
  assert not bad.any(), f'{bad.sum()} of {bad.size} out of tolerance, max {np.abs(g - r).max()}'
  # the scratch buffer is left zero: a second call agrees (split tiles are summed with float
  # atomics, so the last bit may depend on arrival order)
  assert torch.allclose(got.float(), again.float(), rtol=2 ** -7, atol=1e-3)
  # and the unfused path (dequantize kernel + library GEMM) agrees as well
  old = bdg.FUSE_WEIGHT_ONLY
  try:
    bdg.FUSE_WEIGHT_ONLY = False
    slow = bdg.dot_general(at, wq, DN, preferred_element_type=torch.bfloat16)
  finally:
    bdg.FUSE_WEIGHT_ONLY = old
  s = h.to_numpy(slow).astype(np.float32)
  assert np.all(np.abs(s - r) <= 1e-2 + 2e-2 * np.abs(r))


@pytest.mark.parametrize('sdt', ['float32', 'bfloat16'])
def test_a16w4_float32_output_is_tight(sdt):
  M, K, N = 16, 2048, 512
  rng = np.random.default_rng(5)
  w = (0.02 * rng.standard_normal((K, N))).astype(np.float32).astype(ml_dtypes.bfloat16)
  a = rng.standard_normal((M, K)).astype(np.float32).astype(ml_dtypes.bfloat16)
  sd = np.float32 if sdt == 'float32' else ml_dtypes.bfloat16
  wo = oq.quantize_api(w, 'int4', channelwise_axes=[1], tiled_axes={0: 128}, scale_dtype=sd)
  # The kernel multiplies exact code products by the scale in float32: W~ = q * s without an
  # intermediate rounding (what the reference computes when the scale is float32); float64
  # accumulation is the yardstick.
  wt = wo.qvalue.astype(np.float64) * np.repeat(wo.scale.astype(np.float64), 128, axis=0)
  want = a.astype(np.float64) @ wt
  wq = bq.quantize_api(h.to_torch(w), 'int4', channelwise_axes=[1], tiled_axes={0: 128},
                       scale_dtype=torch.float32 if sdt == 'float32' else torch.bfloat16)
  got = bdg.dot_general(h.to_torch(a), wq, DN, preferred_element_type=torch.float32)
  assert np.abs(got.cpu().numpy() - want).max() <= 2e-5 * np.abs(want).max()


@pytest.mark.parametrize('M', [33, 64, 100, 128])
def test_tensor_core_path_with_bf16_scales_is_the_reference_arithmetic(M):
  """From 33 tokens on the weight is dequantized to bfloat16 in shared memory and contracted on
  the tcgen05 tensor cores with one float32 accumulation: with bfloat16 scales exactly what the
  reference does (qarray.py:692-708, dot_general.py:264-275), so only the order of the float32
  sum and the final rounding can differ."""
  K, N = 2048, 1152           # nine channel tiles on 148 CTAs: every tile is shared (split K)
  rng = np.random.default_rng(M)
  w = (0.02 * rng.standard_normal((K, N))).astype(np.float32).astype(ml_dtypes.bfloat16)
  a = rng.standard_normal((M, K)).astype(np.float32).astype(ml_dtypes.bfloat16)
  wo = oq.quantize_api(w, 'int4', channelwise_axes=[1], tiled_axes={0: 128},
                       scale_dtype=ml_dtypes.bfloat16)
  wq = bq.quantize_api(h.to_torch(w), 'int4', channelwise_axes=[1], tiled_axes={0: 128},
                       scale_dtype=torch.bfloat16)
  assert M >= weight_only.TENSOR_CORE_MIN_ROWS
  got = bdg.dot_general(h.to_torch(a), wq, DN, preferred_element_type=torch.float32)
  from qwix_b200 import _lib
  _lib.raise_on_device_error()
  wt = oq.dequantize(wo)                                  # bf16( q * s ), the reference's weight
  assert wt.dtype == np.dtype(ml_dtypes.bfloat16)
  want = a.astype(np.float64) @ wt.astype(np.float64)
  assert np.abs(got.cpu().numpy() - want).max() <= 2e-5 * np.abs(want).max()


def test_tensor_core_entry_point_takes_few_tokens_too():
  """qwx_gemm_a16w4_mma called directly with 5 and 32 tokens (32 tensor-memory columns)."""
  from qwix_b200 import _lib
  L = _lib.lib()
  K, N = 1024, 400            # N is no multiple of 128: the last channel tile is ragged
  rng = np.random.default_rng(3)
  w = (0.02 * rng.standard_normal((K, N))).astype(np.float32).astype(ml_dtypes.bfloat16)
  wo = oq.quantize_api(w, 'int4', channelwise_axes=[1], tiled_axes={0: 256}, scale_dtype=np.float32)
  wq = bq.quantize_api(h.to_torch(w), 'int4', channelwise_axes=[1], tiled_axes={0: 256},
                       scale_dtype=torch.float32)
  tiles = weight_only.prepare_tiles(wq)
  for M in (5, 32):
    a = rng.standard_normal((M, K)).astype(np.float32).astype(ml_dtypes.bfloat16)
    at = h.to_torch(a)
    out = torch.empty((M, N), dtype=torch.float32, device='cuda')
    nws = L.qwx_gemm_a16w4_mma_workspace_bytes(M, N)
    ws = torch.zeros(nws, dtype=torch.uint8, device='cuda')
    err = _lib.error_flag(out.device)
    _lib.check(L.qwx_gemm_a16w4_mma(_lib.ptr(at), _lib.ptr(tiles), _lib.ptr(wq._w4_scale), _lib.F32, M, N, K,
                                    256, _lib.ptr(out), _lib.F32, _lib.ptr(ws), nws, 1, _lib.ptr(err),
                                    _lib.stream_ptr()), 'gemm_a16w4_mma')
    _lib.raise_on_device_error()
    wt = (wo.qvalue.astype(np.float32) * np.repeat(wo.scale, 256, axis=0)).astype(ml_dtypes.bfloat16)
    want = a.astype(np.float64) @ wt.astype(np.float64)
    assert np.abs(out.cpu().numpy() - want).max() <= 2e-5 * np.abs(want).max()
    assert int(ws.view(torch.int32).abs().max().item()) == 0      # the scratch is left zero
