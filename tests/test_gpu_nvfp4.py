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


@pytest.mark.parametrize('M,N,K', [(128, 224, 256), (100, 200, 512), (300, 500, 1024)])
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
