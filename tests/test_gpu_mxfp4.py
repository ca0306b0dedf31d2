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


@pytest.mark.parametrize('M,N,K', [(128, 224, 256), (100, 200, 512), (300, 500, 1024), (256, 448, 2048)])
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
