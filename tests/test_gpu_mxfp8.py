"""MXFP8: e4m3 codes under one power-of-two scale per 32 contracted elements.

Quantization (qwix/_src/core/qarray.py:306-325 tile rule, :566-579 outlier-aware power-of-two
scales) is held bit-exact to the oracle; the block-scaled contraction
(qwix/_src/core/mxfp_dot.py:24-79) to the oracle's restatement of the reference's test double
within the reference's own tolerance (tests/_src/core/mxfp_dot_test.py:167, rtol = atol = 5e-3)
and, since the tensor cores accumulate the exact block products in float32, to a much tighter
bound as well.
"""

import ml_dtypes
import numpy as np
import pytest
import torch

from oracle import dot_general as odg
from oracle import mxfp_dot as omx
from oracle import qarray as oq
from qwix_b200 import _lib
from qwix_b200.core import dot_general as bdg
from qwix_b200.core import mxfp_dot as bmx
from qwix_b200.core import qarray as bq
from tests import helpers as h

pytestmark = pytest.mark.gpu
bf16 = ml_dtypes.bfloat16
DN = (((1,), (0,)), ((), ()))


def _pair(x, w, dn=DN):
  """Quantizes lhs and rhs as a `qtype='mxfp8', tile_size=32` rule does, on both sides."""
  kw = dict(dimension_numbers=dn, ndims=(x.ndim, w.ndim), tile_size=32, qtype='mxfp8')
  lo = oq.quantize(x, odg.get_how_to_quantize(for_lhs=True, **kw))
  ro = oq.quantize(w, odg.get_how_to_quantize(for_lhs=False, **kw))
  lb = bq.quantize(h.to_torch(x), bdg.get_how_to_quantize(for_lhs=True, **kw))
  rb = bq.quantize(h.to_torch(w), bdg.get_how_to_quantize(for_lhs=False, **kw))
  return lo, ro, lb, rb


@pytest.mark.parametrize('dtype', ['bfloat16', 'float32'])
def test_quantize_codes_and_scales_bit_exact(dtype):
  rng = np.random.default_rng(0)
  x = rng.standard_normal((96, 256)).astype(np.float32)
  x[:, ::37] *= 40.0                      # outliers inside some blocks
  x[3] = 0.0                              # an all-zero row: scale falls back to 1 -> 2^0
  x[5, :32] = 1e-30                       # a tiny block
  w = (0.02 * rng.standard_normal((256, 80))).astype(np.float32)
  x, w = x.astype(h.np_dtype(dtype)), w.astype(h.np_dtype(dtype))
  lo, ro, lb, rb = _pair(x, w)
  for o, b in ((lo, lb), (ro, rb)):
    assert b.qtype == 'mxfp8' and b.qvalue.dtype == torch.float8_e4m3fn
    assert tuple(b.scale.shape) == o.scale.shape
    assert np.array_equal(h.to_numpy(b.scale).view(np.uint8), o.scale.view(np.uint8))
    assert h.codes_equal(b.qvalue, o.qvalue)
    s = h.to_numpy(b.scale).astype(np.float32)
    assert np.all(np.frexp(s)[0] == 0.5)  # powers of two
    # and the round trip through the dequantize kernel is the oracle's
    assert np.array_equal(h.to_numpy(bq.dequantize(b)).view(np.uint8), oq.dequantize(o).view(np.uint8))


def test_tile_size_is_checked():
  with pytest.raises(ValueError, match='requires a tile size of 32'):
    bq.HowToQuantize(qtype='mxfp8', channelwise_axes=[0], tiled_axes={1: 64})
  with pytest.raises(ValueError, match='requires `tiled_axes`'):
    bq.HowToQuantize(qtype='mxfp8', channelwise_axes=[0])


CASES = [
    # (M, K, N, input dtype, preferred result dtype)
    (32, 128, 32, 'float32', None),
    (200, 256, 272, 'bfloat16', None),
    (130, 384, 1000, 'bfloat16', 'float32'),     # N % 16 != 0: the weight is repacked [N, K]
    (640, 1024, 672, 'float32', None),           # five row tiles, three 224-column tiles
    (300, 768, 450, 'bfloat16', None),           # CTA pairs, three stages, ragged rows and columns
    (257, 256, 225, 'float32', None),            # CTA pairs, one stage, one row and one column over a tile
    (300, 384, 450, 'bfloat16', None),           # K not whole 256-byte stages: single CTAs
]


@pytest.mark.parametrize('case', CASES, ids=[str(c) for c in CASES])
def test_block_scaled_dot_matches_oracle(case):
  M, K, N, dtype, pref = case
  rng = np.random.default_rng(M + N)
  x = rng.standard_normal((M, K)).astype(np.float32)
  x[:, rng.choice(K, 6, replace=False)] *= 25.0
  w = (0.05 * rng.standard_normal((K, N))).astype(np.float32)
  x, w = x.astype(h.np_dtype(dtype)), w.astype(h.np_dtype(dtype))
  lo, ro, lb, rb = _pair(x, w)
  pt = None if pref is None else getattr(torch, pref)
  pn = None if pref is None else h.np_dtype(pref)
  got = bmx.mxfp_dot_general(lb, rb, DN, pt)
  assert got is not None, 'the block-scaled kernel refused operands it is built for'
  _lib.raise_on_device_error()
  want = omx.mxfp_dot_general(lo, ro, DN, pn)
  assert want is not None
  g, r = h.to_numpy(got).astype(np.float32), np.asarray(want).astype(np.float32)
  assert g.shape == r.shape
  assert h.to_numpy(got).dtype == np.asarray(want).dtype
  np.testing.assert_allclose(g, r, rtol=5e-3, atol=5e-3)          # the reference's own bound
  # exact block products, float32 accumulation: only the summation order and the last
  # rounding to the result dtype can differ
  lv, ls = omx.flatten_to_3d(lo, [1], [])
  rv, rs = omx.flatten_to_3d(ro, [0], [])
  lf = (lv.astype(np.float64).reshape(1, M, -1, 32) * ls.astype(np.float64)[..., None]).reshape(M, K)
  rf = (rv.astype(np.float64).reshape(1, N, -1, 32) * rs.astype(np.float64)[..., None]).reshape(N, K)
  exact = lf @ rf.T
  ulp = 2.0 ** -8 if np.asarray(want).dtype == np.dtype(bf16) else 2.0 ** -22
  mag = np.abs(exact).max()
  assert np.all(np.abs(g - exact) <= ulp * np.maximum(np.abs(exact), 1e-3 * mag) + 1e-6 * mag)
  # the public entry point takes the same route
  assert torch.equal(bdg.dot_general(lb, rb, DN, preferred_element_type=pt), got)


def test_weight_stored_n_by_k_and_batched():
  """einsum-shaped operands: lhs [B, M, K], rhs [B, N, K], both contracted over the last axis."""
  B, M, K, N = 3, 70, 256, 48
  dn = (((2,), (2,)), ((0,), (0,)))
  rng = np.random.default_rng(9)
  x = rng.standard_normal((B, M, K)).astype(np.float32).astype(bf16)
  w = rng.standard_normal((B, N, K)).astype(np.float32).astype(bf16)
  lo, ro, lb, rb = _pair(x, w, dn)
  got = bdg.dot_general(lb, rb, dn)
  _lib.raise_on_device_error()
  want = omx.mxfp_dot_general(lo, ro, dn)
  assert tuple(got.shape) == want.shape == (B, M, N)
  np.testing.assert_allclose(h.to_numpy(got).astype(np.float32), want.astype(np.float32),
                             rtol=2.0 ** -7, atol=1e-3)


def test_falls_back_when_the_kernel_does_not_apply():
  """K = 96 is not whole 128-wide stages, and a float rhs is not microscaled: both take the
  dequantize-then-contract path, like the reference's fallback (mxfp_dot.py:51-57)."""
  rng = np.random.default_rng(4)
  x = rng.standard_normal((40, 96)).astype(np.float32)
  w = (0.1 * rng.standard_normal((96, 32))).astype(np.float32)
  lo, ro, lb, rb = _pair(x, w)
  assert bmx.mxfp_dot_general(lb, rb, DN) is None
  got = bdg.dot_general(lb, rb, DN)
  want = odg.dot_general(lo, ro, DN)
  np.testing.assert_allclose(h.to_numpy(got), want, rtol=1e-5, atol=1e-5)
  assert bmx.mxfp_dot_general(lb, h.to_torch(w), DN) is None


def test_c_abi_refusals():
  L = _lib.lib()
  assert L.qwx_mx_scales_packed_bytes(0, 128, 96) == 0
  assert L.qwx_mx_scales_packed_bytes(0, 130, 256) == 2 * 2 * 512
  assert L.qwx_mx_scales_packed_bytes(1, 225, 256) == 2 * 2 * 1024
  a = torch.zeros((128, 256), dtype=torch.uint8, device='cuda')
  s = torch.zeros(4096, dtype=torch.uint8, device='cuda')
  out = torch.empty((128, 128), dtype=torch.float32, device='cuda')
  err = _lib.error_flag(out.device)
  args = lambda k: (_lib.ptr(a), _lib.ptr(a), _lib.B_NK, 128, 128, k, _lib.ptr(s), _lib.ptr(s),
                    _lib.ptr(out), _lib.F32, _lib.ptr(err), _lib.stream_ptr())
  assert L.qwx_gemm_mx8(*args(96)) == 5       # QWX_ERR_UNSUPPORTED
  assert L.qwx_gemm_mx8(None, *args(256)[1:]) == 1   # QWX_ERR_NULL
  assert L.qwx_gemm_mx8(*args(256)) == 0
  torch.cuda.synchronize()
  _lib.raise_on_device_error()
