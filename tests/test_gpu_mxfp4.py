"""MXFP4 (e2m1 codes, power-of-two scale per 32 contracted elements): the block-scaled GEMM
through the C-ABI and, further down, the quantizer and dot_general.  GPU only."""
import numpy as np
import pytest
import torch

from tests import helpers as h

pytestmark = pytest.mark.gpu

E2M1 = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6], np.float64)


def _gemm_mx4(codes_a, scale_a, codes_b_kn, scale_b_kn, out_dtype=torch.float32):
  """codes_a [M, K] uint8, scale_a [M, K/32] f32; codes_b_kn [K, N], scale_b_kn [K/32, N]."""
  from qwix_b200 import _lib
  L = _lib.lib()
  dev = torch.device('cuda')
  M, K = codes_a.shape
  N = codes_b_kn.shape[1]
  a = torch.from_numpy(codes_a).to(dev)
  b = torch.from_numpy(codes_b_kn).to(dev)
  sa = torch.from_numpy(scale_a).to(dev)
  sb = torch.from_numpy(scale_b_kn).to(dev)
  st = _lib.stream_ptr(dev)
  ap = torch.empty((M, K // 2), dtype=torch.uint8, device=dev)
  bp = torch.empty((N, K // 2), dtype=torch.uint8, device=dev)
  _lib.check(L.qwx_mx4_pack_codes(_lib.ptr(a), M, K, 0, _lib.ptr(ap), st), 'pack a')
  _lib.check(L.qwx_mx4_pack_codes(_lib.ptr(b), N, K, 1, _lib.ptr(bp), st), 'pack b')
  sfa = torch.empty(L.qwx_mx4_scales_packed_bytes(0, M, K), dtype=torch.uint8, device=dev)
  sfb = torch.empty(L.qwx_mx4_scales_packed_bytes(1, N, K), dtype=torch.uint8, device=dev)
  _lib.check(L.qwx_mx4_pack_scales(0, _lib.ptr(sa), _lib.F32, M, K, 0, _lib.ptr(sfa), sfa.numel(), st), 'sfa')
  _lib.check(L.qwx_mx4_pack_scales(1, _lib.ptr(sb), _lib.F32, N, K, 1, _lib.ptr(sfb), sfb.numel(), st), 'sfb')
  out = torch.empty((M, N), dtype=out_dtype, device=dev)
  err = _lib.error_flag(dev)
  oc = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16}[out_dtype]
  _lib.check(L.qwx_gemm_mx4(_lib.ptr(ap), _lib.ptr(bp), M, N, K, _lib.ptr(sfa), _lib.ptr(sfb),
                            _lib.ptr(out), oc, _lib.ptr(err), st), 'gemm_mx4')
  torch.cuda.synchronize()
  _lib.raise_on_device_error()
  return out, ap, bp


def _reference(codes_a, scale_a, codes_b_kn, scale_b_kn):
  af = E2M1[codes_a] * np.repeat(scale_a.astype(np.float64), 32, axis=1)
  bf = E2M1[codes_b_kn] * np.repeat(scale_b_kn.astype(np.float64), 32, axis=0)
  return af @ bf


# up to 128 rows: single CTAs; more rows and whole 256-byte K: CTA pairs (one, two, three stages)
@pytest.mark.parametrize('M,N,K', [(128, 224, 256), (100, 200, 512), (300, 500, 512), (300, 500, 1024),
                                   (256, 448, 2048), (513, 225, 1536), (200, 300, 768)])
def test_block_scaled_gemm_of_e2m1_codes(M, N, K):
  rng = np.random.default_rng(M + N + K)
  ca = rng.integers(0, 16, (M, K), dtype=np.uint8)
  cb = rng.integers(0, 16, (K, N), dtype=np.uint8)
  sa = np.exp2(rng.integers(-3, 4, (M, K // 32))).astype(np.float32)
  sb = np.exp2(rng.integers(-3, 4, (K // 32, N))).astype(np.float32)
  got, ap, bp = _gemm_mx4(ca, sa, cb, sb)
  # the packed operands: even K index in the low nibble
  assert np.array_equal(ap.cpu().numpy(), ca[:, 0::2] | (ca[:, 1::2] << 4))
  assert np.array_equal(bp.cpu().numpy(), (cb[0::2, :] | (cb[1::2, :] << 4)).T)
  want = _reference(ca, sa, cb, sb)
  # every product is exact in float32; only the order of the float32 sums differs
  assert np.abs(got.cpu().numpy() - want).max() <= 2e-6 * np.abs(want).max() * np.sqrt(K / 256)


def test_each_scale_block_reaches_its_own_elements():
  """One non-unit scale at a time: a wrong byte order of the scales in tensor memory shows as a
  wrong block being scaled."""
  M, N, K = 128, 224, 512
  ca = np.full((M, K), 2, np.uint8)   # 1.0 everywhere
  cb = np.full((K, N), 2, np.uint8)
  for blk in range(K // 32):
    sa = np.ones((M, K // 32), np.float32)
    sb = np.ones((K // 32, N), np.float32)
    sa[:, blk] = 4.0
    sb[(blk * 5 + 3) % (K // 32), :] = 8.0
    got, _, _ = _gemm_mx4(ca, sa, cb, sb)
    want = _reference(ca, sa, cb, sb)
    assert np.array_equal(got.cpu().numpy(), want.astype(np.float32)), blk


def test_k_not_a_multiple_of_256_is_refused():
  from qwix_b200 import _lib
  L = _lib.lib()
  assert L.qwx_mx4_scales_packed_bytes(0, 128, 384) == 0


# ---- the quantizer and dot_general ------------------------------------------------------------

import ml_dtypes  # noqa: E402

from oracle import dot_general as odg  # noqa: E402
from oracle import mxfp_dot as omx  # noqa: E402
from oracle import qarray as oq  # noqa: E402
from qwix_b200 import _lib  # noqa: E402
from qwix_b200.core import dot_general as bdg  # noqa: E402
from qwix_b200.core import mxfp_dot as bmx  # noqa: E402
from qwix_b200.core import qarray as bq  # noqa: E402

bf16 = ml_dtypes.bfloat16
DN = (((1,), (0,)), ((), ()))


def _pair(x, w, dn=DN):
  """Quantizes lhs and rhs as a `qtype='mxfp4', tile_size=32` rule does, on both sides."""
  kw = dict(dimension_numbers=dn, ndims=(x.ndim, w.ndim), tile_size=32, qtype='mxfp4')
  lo = oq.quantize(x, odg.get_how_to_quantize(for_lhs=True, **kw))
  ro = oq.quantize(w, odg.get_how_to_quantize(for_lhs=False, **kw))
  lb = bq.quantize(h.to_torch(x), bdg.get_how_to_quantize(for_lhs=True, **kw))
  rb = bq.quantize(h.to_torch(w), bdg.get_how_to_quantize(for_lhs=False, **kw))
  return lo, ro, lb, rb


@pytest.mark.parametrize('dtype', ['bfloat16', 'float32'])
def test_quantize_codes_and_scales_bit_exact(dtype):
  """qarray.py:566-579 with the e2m1 bias 12/7; numerics.py:186-187 clip to +/-6, round to
  nearest even."""
  rng = np.random.default_rng(0)
  x = rng.standard_normal((96, 256)).astype(np.float32)
  x[:, ::37] *= 40.0                      # outliers inside some blocks
  x[3] = 0.0                              # an all-zero row: scale falls back to 1 -> 2^0
  x[5, :32] = 1e-30                       # a tiny block
  x[7, :8] = [0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 7.0]   # ties of the e2m1 grid (before scaling)
  w = (0.02 * rng.standard_normal((256, 80))).astype(np.float32)
  x, w = x.astype(h.np_dtype(dtype)), w.astype(h.np_dtype(dtype))
  lo, ro, lb, rb = _pair(x, w)
  for o, b in ((lo, lb), (ro, rb)):
    assert b.qtype == 'mxfp4' and b.qvalue.dtype == torch.uint8
    assert tuple(b.scale.shape) == o.scale.shape
    assert np.array_equal(h.to_numpy(b.scale).view(np.uint8), o.scale.view(np.uint8))
    assert np.array_equal(h.to_numpy(b.qvalue), o.qvalue.view(np.uint8))
    s = h.to_numpy(b.scale).astype(np.float32)
    assert np.all(np.frexp(s)[0] == 0.5)  # powers of two
    # and the round trip through the dequantize kernel is the oracle's
    assert np.array_equal(h.to_numpy(bq.dequantize(b)).view(np.uint8), oq.dequantize(o).view(np.uint8))


def test_every_code_is_reached_and_read_back():
  """All sixteen e2m1 codes through quantize (scale 1 blocks) and dequantize."""
  vals = np.array([0, .5, 1, 1.5, 2, 3, 4, 6], np.float32)
  row = np.concatenate([vals, -vals, np.full(16, 3.5, np.float32)])   # absmax 6 -> 6/6 * 12/7 -> 2^0
  x = np.tile(row, (8, 4)).astype(np.float32)
  how = bq.HowToQuantize(qtype='mxfp4', channelwise_axes=[0], tiled_axes={1: 32})
  b = bq.quantize(h.to_torch(x), how)
  o = oq.quantize(x, oq.HowToQuantize(qtype='mxfp4', channelwise_axes=[0], tiled_axes={1: 32}))
  assert np.array_equal(h.to_numpy(b.scale), o.scale) and float(o.scale.max()) == 1.0
  codes = h.to_numpy(b.qvalue)
  assert np.array_equal(codes, o.qvalue.view(np.uint8))
  assert set(codes[0, :16].tolist()) == set(range(16))
  assert np.array_equal(h.to_numpy(bq.dequantize(b)), oq.dequantize(o))


CASES = [
    # (M, K, N, input dtype, preferred result dtype)
    (32, 256, 32, 'float32', None),
    (200, 512, 272, 'bfloat16', None),
    (130, 768, 1000, 'bfloat16', 'float32'),
    (640, 1024, 672, 'float32', None),           # five row tiles, three 224-column tiles
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
  np.testing.assert_allclose(g, r, rtol=5e-3, atol=5e-3)          # the reference's own bound (mxfp_dot_test.py:167)
  lv, ls = omx.flatten_to_3d(lo, [1], [])
  rv, rs = omx.flatten_to_3d(ro, [0], [])
  lf = (lv.astype(np.float64).reshape(1, M, -1, 32) * ls.astype(np.float64)[..., None]).reshape(M, K)
  rf = (rv.astype(np.float64).reshape(1, N, -1, 32) * rs.astype(np.float64)[..., None]).reshape(N, K)
  exact = lf @ rf.T
  ulp = 2.0 ** -8 if np.asarray(want).dtype == np.dtype(bf16) else 2.0 ** -22
  mag = np.abs(exact).max()
  assert np.all(np.abs(g - exact) <= ulp * np.maximum(np.abs(exact), 1e-3 * mag) + 1e-6 * mag)
  # the public entry point takes the same route, and the weight's packed form is reused
  assert torch.equal(bdg.dot_general(lb, rb, DN, preferred_element_type=pt), got)
  assert getattr(rb, '_mx4_packed', None) is not None


def test_weight_stored_n_by_k_and_batched():
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
  """K = 128 is not whole 256-element stages, a mixed mxfp8 x mxfp4 pair has no kernel: both
  take the dequantize-then-contract path, like the reference's fallback (mxfp_dot.py:51-57)."""
  rng = np.random.default_rng(4)
  x = rng.standard_normal((40, 128)).astype(np.float32)
  w = (0.1 * rng.standard_normal((128, 32))).astype(np.float32)
  lo, ro, lb, rb = _pair(x, w)
  assert bmx.mxfp_dot_general(lb, rb, DN) is None
  got = bdg.dot_general(lb, rb, DN)
  want = odg.dot_general(lo, ro, DN)
  np.testing.assert_allclose(h.to_numpy(got), want, rtol=1e-5, atol=1e-5)
  kw = dict(dimension_numbers=DN, ndims=(2, 2), tile_size=32, qtype='mxfp8')
  l8 = bq.quantize(h.to_torch(x), bdg.get_how_to_quantize(for_lhs=True, **kw))
  assert bmx.mxfp_dot_general(l8, rb, DN) is None
