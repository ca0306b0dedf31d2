"""NVFP4 (e2m1 codes, an e4m3-valued scale per 16 contracted elements): the block-scaled GEMM
through the C-ABI and, further down, the quantizer and dot_general.  GPU only."""
import ml_dtypes
import numpy as np
import pytest
import torch

from tests import helpers as h

pytestmark = pytest.mark.gpu

E2M1 = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6], np.float64)


def _gemm_nvfp4(codes_a, scale_a, codes_b_kn, scale_b_kn, out_dtype=torch.float32):
  """codes_a [M, K] uint8, scale_a [M, K/16] f32; codes_b_kn [K, N], scale_b_kn [K/16, N]."""
  from qwix_b200 import _lib
  L = _lib.lib()
  dev = torch.device('cuda')
  M, K = codes_a.shape
  N = codes_b_kn.shape[1]
  a, b = torch.from_numpy(codes_a).to(dev), torch.from_numpy(codes_b_kn).to(dev)
  sa, sb = torch.from_numpy(scale_a).to(dev), torch.from_numpy(scale_b_kn).to(dev)
  st = _lib.stream_ptr(dev)
  ap = torch.empty((M, K // 2), dtype=torch.uint8, device=dev)
  bp = torch.empty((N, K // 2), dtype=torch.uint8, device=dev)
  _lib.check(L.qwx_mx4_pack_codes(_lib.ptr(a), M, K, 0, _lib.ptr(ap), st), 'pack a')
  _lib.check(L.qwx_mx4_pack_codes(_lib.ptr(b), N, K, 1, _lib.ptr(bp), st), 'pack b')
  sfa = torch.empty(L.qwx_nvfp4_scales_packed_bytes(0, M, K), dtype=torch.uint8, device=dev)
  sfb = torch.empty(L.qwx_nvfp4_scales_packed_bytes(1, N, K), dtype=torch.uint8, device=dev)
  _lib.check(L.qwx_nvfp4_pack_scales(0, _lib.ptr(sa), _lib.F32, M, K, 0, _lib.ptr(sfa), sfa.numel(), st), 'sfa')
  _lib.check(L.qwx_nvfp4_pack_scales(1, _lib.ptr(sb), _lib.F32, N, K, 1, _lib.ptr(sfb), sfb.numel(), st), 'sfb')
  out = torch.empty((M, N), dtype=out_dtype, device=dev)
  err = _lib.error_flag(dev)
  oc = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16}[out_dtype]
  _lib.check(L.qwx_gemm_nvfp4(_lib.ptr(ap), _lib.ptr(bp), M, N, K, _lib.ptr(sfa), _lib.ptr(sfb),
                              _lib.ptr(out), oc, _lib.ptr(err), st), 'gemm_nvfp4')
  torch.cuda.synchronize()
  _lib.raise_on_device_error()
  return out


def _reference(codes_a, scale_a, codes_b_kn, scale_b_kn):
  af = E2M1[codes_a] * np.repeat(scale_a.astype(np.float64), 16, axis=1)
  bf = E2M1[codes_b_kn] * np.repeat(scale_b_kn.astype(np.float64), 16, axis=0)
  return af @ bf


def _e4m3_scales(rng, shape):
  """Positive e4m3 numbers with every significand."""
  v = rng.uniform(0.05, 30.0, shape).astype(np.float32)
  return v.astype(ml_dtypes.float8_e4m3fn).astype(np.float32)


@pytest.mark.parametrize('M,N,K', [(128, 224, 256), (100, 200, 512), (300, 500, 512), (300, 500, 1024),
                                   (513, 225, 1536), (200, 300, 768)])
def test_block_scaled_gemm_of_e2m1_codes(M, N, K):
  rng = np.random.default_rng(M + N + K)
  ca = rng.integers(0, 16, (M, K), dtype=np.uint8)
  cb = rng.integers(0, 16, (K, N), dtype=np.uint8)
  sa, sb = _e4m3_scales(rng, (M, K // 16)), _e4m3_scales(rng, (K // 16, N))
  got = _gemm_nvfp4(ca, sa, cb, sb)
  want = _reference(ca, sa, cb, sb)
  assert np.abs(got.cpu().numpy() - want).max() <= 2e-6 * np.abs(want).max() * np.sqrt(K / 256)


def test_each_scale_block_reaches_its_own_elements():
  M, N, K = 128, 224, 512
  ca = np.full((M, K), 2, np.uint8)   # 1.0 everywhere
  cb = np.full((K, N), 2, np.uint8)
  for blk in range(K // 16):
    sa = np.ones((M, K // 16), np.float32)
    sb = np.ones((K // 16, N), np.float32)
    sa[:, blk] = 3.0
    sb[(blk * 5 + 3) % (K // 16), :] = 10.0
    got = _gemm_nvfp4(ca, sa, cb, sb)
    want = _reference(ca, sa, cb, sb)
    assert np.array_equal(got.cpu().numpy(), want.astype(np.float32)), blk


# ---- the quantizer and dot_general ------------------------------------------------------------

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
  """Quantizes lhs and rhs as a `qtype='nvfp4', tile_size=16` rule does, on both sides."""
  kw = dict(dimension_numbers=dn, ndims=(x.ndim, w.ndim), tile_size=16, qtype='nvfp4')
  lo = oq.quantize(x, odg.get_how_to_quantize(for_lhs=True, **kw))
  ro = oq.quantize(w, odg.get_how_to_quantize(for_lhs=False, **kw))
  lb = bq.quantize(h.to_torch(x), bdg.get_how_to_quantize(for_lhs=True, **kw))
  rb = bq.quantize(h.to_torch(w), bdg.get_how_to_quantize(for_lhs=False, **kw))
  return lo, ro, lb, rb


@pytest.mark.parametrize('dtype', ['bfloat16', 'float32'])
def test_quantize_codes_and_scales_bit_exact(dtype):
  """qarray.py:580-581: the scale absmax / 6 is rounded to an e4m3 number; numerics.py:186-187
  for the codes."""
  rng = np.random.default_rng(0)
  x = rng.standard_normal((96, 256)).astype(np.float32)
  x[:, ::37] *= 40.0                      # outliers inside some blocks
  x[3] = 0.0                              # an all-zero row: scale falls back to 1
  x[9, :16] *= 1e4                        # absmax / 6 beyond 448: the scale saturates
  w = (0.5 * rng.standard_normal((256, 80))).astype(np.float32)
  x, w = x.astype(h.np_dtype(dtype)), w.astype(h.np_dtype(dtype))
  lo, ro, lb, rb = _pair(x, w)
  for o, b in ((lo, lb), (ro, rb)):
    assert b.qtype == 'nvfp4' and b.qvalue.dtype == torch.uint8
    assert tuple(b.scale.shape) == o.scale.shape
    assert np.array_equal(h.to_numpy(b.scale).view(np.uint8), o.scale.view(np.uint8))
    assert np.array_equal(h.to_numpy(b.qvalue), o.qvalue.view(np.uint8))
    s = h.to_numpy(b.scale).astype(np.float32)
    assert np.array_equal(s.astype(ml_dtypes.float8_e4m3fn).astype(np.float32), s)   # e4m3 numbers
    assert np.array_equal(h.to_numpy(bq.dequantize(b)).view(np.uint8), oq.dequantize(o).view(np.uint8))


def test_tile_size_is_checked():
  with pytest.raises(ValueError, match='requires a tile size of 16'):
    bq.HowToQuantize(qtype='nvfp4', channelwise_axes=[0], tiled_axes={1: 32})


CASES = [
    (32, 256, 32, 'float32', None),
    (200, 512, 272, 'bfloat16', None),
    (130, 768, 1000, 'bfloat16', 'float32'),
    (640, 1024, 672, 'float32', None),
]


@pytest.mark.parametrize('case', CASES, ids=[str(c) for c in CASES])
def test_block_scaled_dot_matches_oracle(case):
  M, K, N, dtype, pref = case
  rng = np.random.default_rng(M + N)
  x = rng.standard_normal((M, K)).astype(np.float32)
  x[:, rng.choice(K, 6, replace=False)] *= 25.0
  w = (0.5 * rng.standard_normal((K, N))).astype(np.float32)
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
  assert g.shape == r.shape and h.to_numpy(got).dtype == np.asarray(want).dtype
  np.testing.assert_allclose(g, r, rtol=5e-3, atol=5e-3 * max(1.0, float(np.abs(r).max()) / 50))
  lv, ls = omx.flatten_to_3d(lo, [1], [])
  rv, rs = omx.flatten_to_3d(ro, [0], [])
  lf = (lv.astype(np.float64).reshape(1, M, -1, 16) * ls.astype(np.float64)[..., None]).reshape(M, K)
  rf = (rv.astype(np.float64).reshape(1, N, -1, 16) * rs.astype(np.float64)[..., None]).reshape(N, K)
  exact = lf @ rf.T
  ulp = 2.0 ** -8 if np.asarray(want).dtype == np.dtype(bf16) else 2.0 ** -22
  mag = np.abs(exact).max()
  assert np.all(np.abs(g - exact) <= ulp * np.maximum(np.abs(exact), 1e-3 * mag) + 1e-6 * mag)
  assert torch.equal(bdg.dot_general(lb, rb, DN, preferred_element_type=pt), got)


def test_falls_back_when_the_kernel_does_not_apply():
  rng = np.random.default_rng(4)
  x = rng.standard_normal((40, 128)).astype(np.float32)
  w = (0.5 * rng.standard_normal((128, 32))).astype(np.float32)
  lo, ro, lb, rb = _pair(x, w)
  assert bmx.mxfp_dot_general(lb, rb, DN) is None          # K = 128: not whole 256-element stages
  got = bdg.dot_general(lb, rb, DN)
  want = odg.dot_general(lo, ro, DN)
  np.testing.assert_allclose(h.to_numpy(got), want, rtol=1e-5, atol=1e-5)
