"""GPU parity: tcgen05 quantized GEMM (through the C ABI) vs the CPU oracle."""

import dataclasses

import numpy as np
import pytest
import torch

from oracle import dot_general as odg
from oracle import qarray as oq
from qwix_b200 import _lib
from qwix_b200.core import dot_general as bdg
from qwix_b200.core import qarray as bq
from tests import helpers as h

pytestmark = pytest.mark.gpu

DN = (((1,), (0,)), ((), ()))


def _raw_gemm(a: torch.Tensor, b: torch.Tensor, layout: int, code=_lib.S8, out_dtype=torch.int32):
  M, K = a.shape
  N = b.shape[1] if layout == _lib.B_KN else b.shape[0]
  out = torch.empty((M, N), dtype=out_dtype, device='cuda')
  err = torch.zeros(1, dtype=torch.int32, device='cuda')
  oc = {torch.int32: _lib.S32, torch.float32: _lib.F32}[out_dtype]
  _lib.check(_lib.lib().qwx_gemm_q8(_lib.ptr(a), _lib.ptr(b), code, layout, M, N, K, 0, None, 0,
                                    None, 0, _lib.F32, _lib.ptr(out), oc, 0, _lib.ptr(err),
                                    _lib.stream_ptr()), 'gemm')
  torch.cuda.synchronize()
  assert int(err.item()) == 0
  return out


def _splitk_gemm(a, b, layout, code=_lib.S8, out_dtype=torch.int32, sa=None, sb=None, ws=None):
  """The workspace form; returns (out, workspace) so a test can reuse the buffer."""
  M, K = a.shape
  N = b.shape[1] if layout == _lib.B_KN else b.shape[0]
  L = _lib.lib()
  need = L.qwx_gemm_q8_workspace_bytes(M, N, K)
  if ws is None:
    ws = torch.zeros(max(need, 16), dtype=torch.uint8, device='cuda')
  out = torch.empty((M, N), dtype=out_dtype, device='cuda')
  err = torch.zeros(1, dtype=torch.int32, device='cuda')
  oc = {torch.int32: _lib.S32, torch.float32: _lib.F32, torch.bfloat16: _lib.BF16}[out_dtype]
  _lib.check(L.qwx_gemm_q8_ws(_lib.ptr(a), _lib.ptr(b), code, layout, M, N, K, 0, _lib.ptr(sa), 0,
                              _lib.ptr(sb), 0, _lib.F32, _lib.ptr(out), oc, 0, _lib.ptr(ws), need,
                              1, _lib.ptr(err), _lib.stream_ptr()), 'gemm_ws')
  torch.cuda.synchronize()
  assert int(err.item()) == 0
  return out, ws, need


DECODE_SHAPES = [(32, 4096, 4096), (1, 1024, 14336), (8, 6144, 4096), (33, 512 + 32, 2048 + 128),
                 (128, 2048, 8192), (160, 256, 16384)]


@pytest.mark.parametrize('layout', [_lib.B_NK, _lib.B_KN], ids=['b_nk', 'b_kn'])
@pytest.mark.parametrize('mnk', DECODE_SHAPES, ids=[f'{m}x{n}x{k}' for m, n, k in DECODE_SHAPES])
def test_split_k_int8_bit_exact_and_workspace_reusable(mnk, layout):
  M, N, K = mnk
  rng = np.random.default_rng(M + N + K)
  a = rng.integers(-128, 128, (M, K), dtype=np.int8)
  b = rng.integers(-128, 128, (K, N), dtype=np.int8)
  want = a.astype(np.int32) @ b.astype(np.int32)
  bt = h.to_torch(b if layout == _lib.B_KN else np.ascontiguousarray(b.T))
  at = h.to_torch(a)
  got, ws, need = _splitk_gemm(at, bt, layout)
  assert need > 0, 'shape was expected to be cut along K'
  assert np.array_equal(got.cpu().numpy(), want)
  # second call on the same, uncleared workspace; scaled bf16 output equals the unsplit kernel
  sa = torch.rand(M, device='cuda') + 0.5
  sb = torch.rand(N, device='cuda') * 1e-3
  got2, ws, _ = _splitk_gemm(at, bt, layout, out_dtype=torch.bfloat16, sa=sa, sb=sb, ws=ws)
  ref = torch.empty_like(got2)
  err = torch.zeros(1, dtype=torch.int32, device='cuda')
  _lib.check(_lib.lib().qwx_gemm_q8(_lib.ptr(at), _lib.ptr(bt), _lib.S8, layout, M, N, K, 0,
                                    _lib.ptr(sa), 0, _lib.ptr(sb), 0, _lib.F32, _lib.ptr(ref),
                                    _lib.BF16, 0, _lib.ptr(err), _lib.stream_ptr()), 'gemm')
  torch.cuda.synchronize()
  assert torch.equal(got2.view(torch.int16), ref.view(torch.int16))
  tiles = -(-M // 128) * -(-N // 256)
  assert int(ws[:tiles * 8].count_nonzero().item()) == 0   # tile counters are left zero


def test_split_k_workspace_shared_between_shapes():
  """One zeroed buffer serves calls with different tile counts: the counters of one call never
  lie where another call left partial sums."""
  L = _lib.lib()
  shapes = [(32, 3072, 4096), (32, 14336, 4096), (32, 4096, 2048), (32, 14336, 4096), (32, 3072, 4096)]
  need = max(L.qwx_gemm_q8_workspace_bytes(*s) for s in shapes)
  ws = torch.zeros(need, dtype=torch.uint8, device='cuda')
  for i, (M, N, K) in enumerate(shapes):
    rng = np.random.default_rng(i)
    a = rng.integers(-128, 128, (M, K), dtype=np.int8)
    b = rng.integers(-128, 128, (N, K), dtype=np.int8)
    want = a.astype(np.int32) @ b.astype(np.int32).T
    got, _, n = _splitk_gemm(h.to_torch(a), h.to_torch(b), _lib.B_NK, ws=ws)
    assert n > 0
    assert np.array_equal(got.cpu().numpy(), want), f'call {i} {M}x{N}x{K}'


def test_split_k_fp8():
  M, N, K = 16, 1024, 4096
  rng = np.random.default_rng(5)
  import ml_dtypes
  a = rng.standard_normal((M, K)).astype(np.float32).astype(ml_dtypes.float8_e4m3fn)
  b = rng.standard_normal((N, K)).astype(np.float32).astype(ml_dtypes.float8_e4m3fn)
  want = a.astype(np.float32) @ b.astype(np.float32).T
  got, ws, need = _splitk_gemm(h.to_torch(a), h.to_torch(b), _lib.B_NK, code=_lib.E4M3,
                               out_dtype=torch.float32)
  assert need > 0
  assert np.abs(got.cpu().numpy() - want).max() <= 1e-3 * np.abs(want).max()
  again, _, _ = _splitk_gemm(h.to_torch(a), h.to_torch(b), _lib.B_NK, code=_lib.E4M3,
                             out_dtype=torch.float32, ws=ws)
  assert torch.equal(got, again)   # partial sums are added in a fixed order


def test_split_k_workspace_query_and_errors():
  L = _lib.lib()
  assert L.qwx_gemm_q8_workspace_bytes(4096, 8192, 8192) == 0      # enough tiles already
  assert L.qwx_gemm_q8_workspace_bytes(32, 4096, 256) == 0         # K too short to cut
  need = L.qwx_gemm_q8_workspace_bytes(32, 4096, 4096)
  assert need == 1024 + 8 * 16 * 128 * 256 * 4, need   # counters + 16 tiles x 8 ranges of slabs
  a = torch.zeros((32, 4096), dtype=torch.int8, device='cuda')
  b = torch.zeros((4096, 4096), dtype=torch.int8, device='cuda')
  out = torch.empty((32, 4096), dtype=torch.int32, device='cuda')
  ws = torch.zeros(need, dtype=torch.uint8, device='cuda')
  rc = L.qwx_gemm_q8_ws(_lib.ptr(a), _lib.ptr(b), _lib.S8, _lib.B_NK, 32, 4096, 4096, 0, None, 0,
                        None, 0, _lib.F32, _lib.ptr(out), _lib.S32, 0, _lib.ptr(ws), need - 4, 1,
                        None, _lib.stream_ptr())
  assert rc == 6  # QWX_ERR_WORKSPACE


SKINNY_SHAPES = [(1, 4096, 4096), (8, 512, 1024), (17, 48, 14336), (32, 6144, 4096), (32, 1024, 14336),
                 (5, 16, 256), (32, 128256 // 8, 512)]


@pytest.mark.parametrize('mnk', SKINNY_SHAPES, ids=[f'{m}x{n}x{k}' for m, n, k in SKINNY_SHAPES])
def test_skinny_int8_bit_exact(mnk):
  """The warp-level decode kernel ([N, K] weight, at most 32 rows): raw accumulators against
  NumPy, scaled bf16 output against the tcgen05 kernel, workspace reusable."""
  M, N, K = mnk
  rng = np.random.default_rng(M + N + K)
  a = rng.integers(-128, 128, (M, K), dtype=np.int8)
  w = rng.integers(-128, 128, (N, K), dtype=np.int8)
  want = a.astype(np.int32) @ w.astype(np.int32).T
  at, wt = h.to_torch(a), h.to_torch(w)
  L = _lib.lib()
  need = L.qwx_gemm_q8_skinny_workspace_bytes(M, N)
  ws = torch.zeros(need, dtype=torch.uint8, device='cuda')
  out = torch.empty((M, N), dtype=torch.int32, device='cuda')
  _lib.check(L.qwx_gemm_q8_skinny(_lib.ptr(at), _lib.ptr(wt), M, N, K, None, None, _lib.F32,
                                  _lib.ptr(out), _lib.S32, 0, _lib.ptr(ws), need, 1,
                                  _lib.stream_ptr()), 'skinny')
  torch.cuda.synchronize()
  assert np.array_equal(out.cpu().numpy(), want)
  assert int(ws.count_nonzero().item()) == 0
  sa = (torch.rand(M, device='cuda') + 0.5).to(torch.bfloat16)
  sb = (torch.rand(N, device='cuda') * 1e-3).to(torch.bfloat16)
  got = torch.empty((M, N), dtype=torch.bfloat16, device='cuda')
  _lib.check(L.qwx_gemm_q8_skinny(_lib.ptr(at), _lib.ptr(wt), M, N, K, _lib.ptr(sa), _lib.ptr(sb),
                                  _lib.BF16, _lib.ptr(got), _lib.BF16, 0, _lib.ptr(ws), need, 1,
                                  _lib.stream_ptr()), 'skinny')
  ref = torch.empty_like(got)
  err = torch.zeros(1, dtype=torch.int32, device='cuda')
  _lib.check(L.qwx_gemm_q8(_lib.ptr(at), _lib.ptr(wt), _lib.S8, _lib.B_NK, M, N, K, 0, _lib.ptr(sa), 0,
                           _lib.ptr(sb), 0, _lib.BF16, _lib.ptr(ref), _lib.BF16, 0, _lib.ptr(err),
                           _lib.stream_ptr()), 'gemm')
  torch.cuda.synchronize()
  assert torch.equal(got.view(torch.int16), ref.view(torch.int16))
  assert int(ws.count_nonzero().item()) == 0


def test_dot_general_takes_the_skinny_kernel_for_nk_weights():
  M, K, N = 8, 1024, 512
  rng = np.random.default_rng(2)
  x = rng.standard_normal((M, K)).astype(np.float32)
  w = (0.02 * rng.standard_normal((K, N))).astype(np.float32)
  kw = dict(dimension_numbers=DN, ndims=(2, 2), tile_size=None, qtype='int8')
  xo = oq.quantize(x, odg.get_how_to_quantize(for_lhs=True, **kw))
  wo = oq.quantize(w, odg.get_how_to_quantize(for_lhs=False, **kw))
  want = odg.dot_general(xo, wo, DN)
  xq = bq.quantize(h.to_torch(x), bdg.get_how_to_quantize(for_lhs=True, **kw))
  wq = bq.quantize(h.to_torch(w), bdg.get_how_to_quantize(for_lhs=False, **kw))
  # the same codes stored [N, K]: the logical [K, N] qvalue is a transposed view
  wq_nk = bq.QArray(qvalue=wq.qvalue.t().contiguous().t(), scale=wq.scale, zero_point=None,
                    qtype=wq.qtype)
  got_kn = bdg.dot_general(xq, wq, DN)
  got_nk = bdg.dot_general(xq, wq_nk, DN)
  assert torch.equal(got_kn, got_nk)
  _close(got_nk, want)


SHAPES = [(128, 256, 128), (128, 256, 512), (256, 512, 1024), (384, 768, 4096),
          (100, 200 + 8, 256 + 16), (1, 16, 128), (130, 272, 144), (512, 1024, 8192)]


@pytest.mark.parametrize('layout', [_lib.B_NK, _lib.B_KN], ids=['b_nk', 'b_kn'])
@pytest.mark.parametrize('mnk', SHAPES, ids=[f'{m}x{n}x{k}' for m, n, k in SHAPES])
def test_int8_accumulator_bit_exact(mnk, layout):
  M, N, K = mnk
  rng = np.random.default_rng(M + N + K)
  a = rng.integers(-128, 128, (M, K), dtype=np.int8)
  b = rng.integers(-128, 128, (K, N), dtype=np.int8)
  want = (a.astype(np.float64) @ b.astype(np.float64)).astype(np.int64)
  bt = h.to_torch(b if layout == _lib.B_KN else np.ascontiguousarray(b.T))
  got = _raw_gemm(h.to_torch(a), bt, layout).cpu().numpy().astype(np.int64)
  bad = np.argwhere(got != want)
  assert bad.size == 0, f'{len(bad)} mismatches, first {bad[:5].tolist()}'


@pytest.mark.parametrize('layout', [_lib.B_NK, _lib.B_KN], ids=['b_nk', 'b_kn'])
def test_fp8_accumulator(layout):
  M, N, K = 256, 512, 1024
  rng = np.random.default_rng(0)
  import ml_dtypes
  a = rng.standard_normal((M, K)).astype(np.float32).astype(ml_dtypes.float8_e4m3fn)
  b = rng.standard_normal((K, N)).astype(np.float32).astype(ml_dtypes.float8_e4m3fn)
  want = a.astype(np.float32) @ b.astype(np.float32)
  bt = h.to_torch(b if layout == _lib.B_KN else np.ascontiguousarray(b.T))
  got = _raw_gemm(h.to_torch(a), bt, layout, code=_lib.E4M3, out_dtype=torch.float32).cpu().numpy()
  assert np.abs(got - want).max() <= 1e-3 * np.abs(want).max()


@pytest.mark.parametrize('dtype', ['float32', 'bfloat16'])
@pytest.mark.parametrize('qtype', ['int8', 'float8_e4m3fn'])
def test_w8a8_dot_general_matches_oracle(qtype, dtype):
  M, K, N = 192, 1024, 512
  rng = np.random.default_rng(1)
  x = rng.standard_normal((M, K)).astype(np.float32)
  x[:, rng.choice(K, 10, replace=False)] *= 20
  w = (0.02 * rng.standard_normal((K, N))).astype(np.float32)
  x, w = x.astype(h.np_dtype(dtype)), w.astype(h.np_dtype(dtype))
  kw = dict(dimension_numbers=DN, ndims=(2, 2), tile_size=None, qtype=qtype)
  xo = oq.quantize(x, odg.get_how_to_quantize(for_lhs=True, **kw))
  wo = oq.quantize(w, odg.get_how_to_quantize(for_lhs=False, **kw))
  want = odg.dot_general(xo, wo, DN)
  xq = bq.quantize(h.to_torch(x), bdg.get_how_to_quantize(for_lhs=True, **kw))
  wq = bq.quantize(h.to_torch(w), bdg.get_how_to_quantize(for_lhs=False, **kw))
  assert h.codes_equal(xq.qvalue, xo.qvalue) and h.codes_equal(wq.qvalue, wo.qvalue)
  got = bdg.dot_general(xq, wq, DN)
  assert got.dtype == h.to_torch(want[:1]).dtype
  g = h.to_numpy(got).astype(np.float32)
  r = want.astype(np.float32)
  # Stated tolerance for dequantized outputs: max-abs 1e-2 or rel 2e-2.
  assert np.all(np.abs(g - r) <= 1e-2 + 2e-2 * np.abs(r))
  if qtype == 'int8':
    # Reference-order epilogue: bit-exact with the strict oracle.
    old = bdg.EPILOGUE
    try:
      bdg.EPILOGUE = 'reference'
      exact = bdg.dot_general(xq, wq, DN)
    finally:
      bdg.EPILOGUE = old
    assert np.array_equal(h.to_numpy(exact).view(np.uint8), want.view(np.uint8))


# ---------------------------------------------------------------------------------------------
# Scales that change along K (sub-channel tiles) and asymmetric operands: the general form of
# the reference's dequantize-on-output contraction (dot_general.py:187-259).

def _quantize_pair(x, w, dn, l_kw, r_kw):
  ndims = (x.ndim, w.ndim)
  lo = oq.quantize(x, odg.get_how_to_quantize(dimension_numbers=dn, ndims=ndims, for_lhs=True, **l_kw))
  ro = oq.quantize(w, odg.get_how_to_quantize(dimension_numbers=dn, ndims=ndims, for_lhs=False, **r_kw))
  lb = bq.quantize(h.to_torch(x), bdg.get_how_to_quantize(dimension_numbers=dn, ndims=ndims, for_lhs=True, **l_kw))
  rb = bq.quantize(h.to_torch(w), bdg.get_how_to_quantize(dimension_numbers=dn, ndims=ndims, for_lhs=False, **r_kw))
  assert h.codes_equal(lb.qvalue, lo.qvalue) and h.codes_equal(rb.qvalue, ro.qvalue)
  return lo, ro, lb, rb


def _close(got, want):
  g = h.to_numpy(got).astype(np.float32)
  r = np.asarray(want).astype(np.float32)
  assert g.shape == r.shape
  # tolerance stated for dequantized outputs: max-abs 1e-2 or relative 2e-2
  bad = np.abs(g - r) > 1e-2 + 2e-2 * np.abs(r)
  assert not bad.any(), f'{bad.sum()} of {bad.size} outside tolerance; worst {np.abs(g - r).max()}'


TILED_CASES = [
    # (M, K, N, lhs tile, rhs tile, qtype, dtype)
    (192, 1024, 384, 128, 128, 'int8', 'float32'),
    (192, 1024, 384, 256, 256, 'int8', 'bfloat16'),
    (200, 1024, 264, None, 128, 'int8', 'float32'),      # per-row activations, sub-channel weight
    (64, 2048, 512, 512, None, 'int8', 'bfloat16'),
    (130, 1024, 256, 128, 128, 'float8_e4m3fn', 'float32'),
    # several 256 x 256 tiles of the CTA-pair form, ragged in M and N
    (520, 1024, 784, 128, 128, 'int8', 'bfloat16'),
    (300, 1536, 528, 512, 512, 'int8', 'float32'),
    (260, 512, 272, 256, 256, 'float8_e4m3fn', 'bfloat16'),
    # an odd count of 128-wide K blocks: the last two-block stage of the pair form is half zeros
    (300, 384, 272, 128, 128, 'int8', 'float32'),
    (260, 640, 528, 128, 128, 'int8', 'bfloat16'),
]


@pytest.mark.parametrize('case', TILED_CASES, ids=[str(c) for c in TILED_CASES])
def test_tiled_scales_match_oracle(case):
  M, K, N, lt, rt, qtype, dtype = case
  rng = np.random.default_rng(M + K + N)
  x = rng.standard_normal((M, K)).astype(np.float32)
  x[:, rng.choice(K, 8, replace=False)] *= 12
  w = (0.05 * rng.standard_normal((K, N))).astype(np.float32)
  x, w = x.astype(h.np_dtype(dtype)), w.astype(h.np_dtype(dtype))
  lo, ro, lb, rb = _quantize_pair(x, w, DN, dict(tile_size=lt, qtype=qtype),
                                  dict(tile_size=rt, qtype=qtype))
  assert bdg.use_fast_path(lb, rb, DN)
  want = odg.dot_general(lo, ro, DN)
  got = bdg.dot_general(lb, rb, DN)
  assert got.dtype == h.to_torch(np.asarray(want)[:1]).dtype
  if dtype == 'float32':
    _close(got, want)
  else:
    # The reference rounds every tile's product to bfloat16 three times before the tile sum,
    # so its own result carries a few bfloat16 ulps of the largest tile term.  The float32
    # epilogue is held to the stated tolerance against the same contraction with float32
    # scales; the reference-order epilogue is held to the oracle itself.
    wide = lambda q: dataclasses.replace(q, scale=q.scale.astype(np.float32))
    _close(got, odg.dot_general(wide(lo), wide(ro), DN))
    old = bdg.EPILOGUE
    try:
      bdg.EPILOGUE = 'reference'
      strict = h.to_numpy(bdg.dot_general(lb, rb, DN)).astype(np.float32)
    finally:
      bdg.EPILOGUE = old
    w32 = np.asarray(want).astype(np.float32)
    # the only freedom left is the order of the float32 tile sum: at most one bfloat16 ulp
    assert np.all(np.abs(strict - w32) <= 2.0 ** -7 * np.maximum(np.abs(w32), 2.0 ** -6))
    assert np.mean(strict == w32) > 0.98
  # the loop form (one contraction per K tile, added in order) is the same kernel here
  if lt == rt and dtype == 'float32':
    _close(bdg.loop_dot_general(lb, rb, DN), odg.loop_dot_general(lo, ro, DN))


@pytest.mark.parametrize('scale_dtype', [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize('corr', [False, True])
@pytest.mark.parametrize('shape', [(300, 250, 384, 128), (129, 1000, 512, 256), (640, 72, 1024, 512)],
                         ids=['300x250x384', '129x1000x512', '640x72x1024'])
def test_tiled_c_abi_weight_stored_n_by_k(shape, corr, scale_dtype):
  """qwx_gemm_q8_tiled with the weight as [N, K], N a multiple of neither 4 nor 32 in two of the
  shapes (single scale loads, ragged stores), every scale dtype, with and without the integer
  zero-point term, against the formula in float64."""
  M, N, K, tile = shape
  T = K // tile
  rng = np.random.default_rng(M * 7 + N + int(corr))
  a = rng.integers(-128, 128, (M, K), dtype=np.int8)
  b = rng.integers(-128, 128, (N, K), dtype=np.int8)
  sa = torch.as_tensor(rng.random((M, T), dtype=np.float32) + 0.5).to(scale_dtype)
  sb = torch.as_tensor(rng.random((T, N), dtype=np.float32) + 0.5).to(scale_dtype)
  cr = rng.integers(-128, 128, (M, T), dtype=np.int32)
  cc = rng.integers(-2000, 2000, (T, N), dtype=np.int32)
  want = np.zeros((M, N), dtype=np.float64)
  for t in range(T):
    acc = a[:, t * tile:(t + 1) * tile].astype(np.float64) @ b[:, t * tile:(t + 1) * tile].astype(np.float64).T
    if corr:
      acc -= cr[:, t:t + 1].astype(np.float64) * cc[t:t + 1].astype(np.float64)
    want += acc * sa[:, t:t + 1].double().numpy() * sb[t:t + 1].double().numpy()
  L = _lib.lib()
  dev = [h.to_torch(x) for x in (a, b, cr, cc)]
  sa_d, sb_d = sa.cuda(), sb.cuda()
  out = torch.empty((M, N), dtype=torch.float32, device='cuda')
  err = _lib.error_flag(out.device)
  _lib.check(L.qwx_gemm_q8_tiled(_lib.ptr(dev[0]), _lib.ptr(dev[1]), _lib.S8, _lib.B_NK, M, N, K, tile,
                                 _lib.ptr(sa_d), 1, _lib.ptr(sb_d), 1, _lib.FLOAT_CODES[scale_dtype],
                                 _lib.ptr(dev[2]) if corr else None, _lib.ptr(dev[3]) if corr else None,
                                 _lib.ptr(out), _lib.F32, 0, _lib.ptr(err), _lib.stream_ptr()), 'tiled')
  _lib.raise_on_device_error()
  got = out.cpu().numpy().astype(np.float64)
  # float32 running sums of T terms: a few float32 ulps of the largest partial sum
  assert np.all(np.abs(got - want) <= 1e-5 * np.abs(want) + 1e-5 * np.abs(want).max())


@pytest.mark.parametrize('side', ['lhs', 'rhs'])
@pytest.mark.parametrize('tile', [None, 128])
def test_asymmetric_operand_matches_oracle(side, tile):
  M, K, N = 160, 512, 272
  rng = np.random.default_rng(7)
  x = (rng.random((M, K)) * 3 + 1).astype(np.float32)           # far from symmetric
  w = (0.05 * rng.standard_normal((K, N)) + 0.02).astype(np.float32)
  sym = dict(tile_size=tile, qtype='int8')
  asym = dict(tile_size=tile, qtype='int8', calibration_method='minmax')
  lo, ro, lb, rb = _quantize_pair(x, w, DN, asym if side == 'lhs' else sym,
                                  asym if side == 'rhs' else sym)
  assert (lb.zero_point is not None) == (side == 'lhs')
  assert (rb.zero_point is not None) == (side == 'rhs')
  want = odg.dot_general(lo, ro, DN)
  got = bdg.dot_general(lb, rb, DN)
  _close(got, want)
  # and the result approximates the float product much better than a symmetric int8 lhs would
  ref = x @ w
  assert np.abs(h.to_numpy(got) - ref).mean() / np.abs(ref).mean() < 2e-2


def test_mismatched_tiles_raise():
  x = np.random.default_rng(0).random((32, 768)).astype(np.float32)
  w = np.random.default_rng(1).random((768, 32)).astype(np.float32)
  _, _, lb, rb = _quantize_pair(x, w, DN, dict(tile_size=128, qtype='int8'),
                                dict(tile_size=384, qtype='int8'))
  with pytest.raises(ValueError, match='same tile size'):
    bdg.dot_general(lb, rb, DN)


def test_both_asymmetric_raises():
  x = np.random.default_rng(0).random((32, 128)).astype(np.float32)
  w = np.random.default_rng(1).random((128, 32)).astype(np.float32)
  kw = dict(tile_size=None, qtype='int8', calibration_method='minmax')
  _, _, lb, rb = _quantize_pair(x, w, DN, kw, kw)
  with pytest.raises(ValueError, match='Only one operand can be asymmetric'):
    bdg.dot_general(lb, rb, DN)


def test_w4a8_sub_channel_matches_oracle():
  """int4 weight codes with 128-wide tiles against int8 per-token activations."""
  M, K, N = 48, 1024, 512
  rng = np.random.default_rng(11)
  x = rng.standard_normal((M, K)).astype(np.float32)
  w = (0.02 * rng.standard_normal((K, N))).astype(np.float32)
  lo, ro, lb, rb = _quantize_pair(x, w, DN, dict(tile_size=None, qtype='int8'),
                                  dict(tile_size=128, qtype='int4'))
  _close(bdg.dot_general(lb, rb, DN), odg.dot_general(lo, ro, DN))


def test_tiled_batched_einsum_shape():
  """Batch axis plus two contracting axes, the last one tiled: K runs are numbered by
  (first contracting axis, tile)."""
  Bn, M, C1, C2, N = 2, 40, 2, 256, 64
  rng = np.random.default_rng(3)
  x = rng.standard_normal((Bn, M, C1, C2)).astype(np.float32)
  w = (0.05 * rng.standard_normal((Bn, C1, C2, N))).astype(np.float32)
  dn = (((2, 3), (1, 2)), ((0,), (0,)))
  lo, ro, lb, rb = _quantize_pair(x, w, dn, dict(tile_size=128, qtype='int8'),
                                  dict(tile_size=128, qtype='int8'))
  _close(bdg.dot_general(lb, rb, dn), odg.dot_general(lo, ro, dn))


@pytest.mark.parametrize('k_axis', [0, 1])
@pytest.mark.parametrize('t_major', [0, 1])
def test_code_sums(k_axis, t_major):
  rng = np.random.default_rng(k_axis * 2 + t_major)
  other, K, tile = 70, 512 + 128, 128
  codes = rng.integers(-128, 128, (other, K) if k_axis == 1 else (K, other), dtype=np.int8)
  T = K // tile
  src = codes if k_axis == 1 else codes.T
  want = src.astype(np.int32).reshape(other, T, tile).sum(-1)       # [other, T]
  if t_major:
    want = want.T
  out = torch.empty(want.shape, dtype=torch.int32, device='cuda')
  ct = h.to_torch(codes)
  _lib.check(_lib.lib().qwx_code_sums(_lib.ptr(ct), codes.shape[0], codes.shape[1], k_axis, tile,
                                      t_major, _lib.ptr(out), _lib.stream_ptr()), 'code_sums')
  torch.cuda.synchronize()
  assert np.array_equal(out.cpu().numpy(), want)


# ---------------------------------------------------------------------------------------------
# Activation quantization + GEMM as one call (qwx_quant_gemm_q8).

QUANT_GEMM_CASES = [('int8', 192, 1024, 512, False), ('int8', 640, 2048, 768, True),
                    ('int8', 5, 512, 264, False), ('float8_e4m3fn', 320, 1024, 512, False),
                    ('float8_e4m3fn', 48, 768, 256, True)]


@pytest.mark.parametrize('case', QUANT_GEMM_CASES,
                         ids=[f'{q}-{m}x{k}x{n}-{"nk" if t else "kn"}'
                              for q, m, k, n, t in QUANT_GEMM_CASES])
def test_quantized_matmul_one_call_matches_oracle_and_two_calls(case):
  from qwix_b200 import fused
  qtype, M, K, N, nk = case
  rng = np.random.default_rng(11)
  x = rng.standard_normal((M, K)).astype(np.float32)
  x[:, rng.choice(K, 8, replace=False)] *= 20
  x[M // 2] = 0                       # an all-zero token: scale 1, codes 0
  w = (0.02 * rng.standard_normal((K, N))).astype(np.float32)
  x, w = x.astype(h.np_dtype('bfloat16')), w.astype(h.np_dtype('bfloat16'))
  kw = dict(dimension_numbers=DN, ndims=(2, 2), tile_size=None, qtype=qtype)
  xo = oq.quantize(x, odg.get_how_to_quantize(for_lhs=True, **kw))
  wo = oq.quantize(w, odg.get_how_to_quantize(for_lhs=False, **kw))
  want = odg.dot_general(xo, wo, DN).astype(np.float32)

  xt = h.to_torch(x)
  wq = bq.quantize(h.to_torch(w), bdg.get_how_to_quantize(for_lhs=False, **kw))
  if nk:    # codes held [N, K], seen as [K, N]
    wq = dataclasses.replace(wq, qvalue=wq.qvalue.t().contiguous().t())
  out, act = fused.quantized_matmul(xt, wq, return_act=True)
  assert h.codes_equal(act.qvalue, xo.qvalue)
  assert np.array_equal(h.to_numpy(act.scale).view(np.uint16), xo.scale.view(np.uint16))
  g = h.to_numpy(out).astype(np.float32)
  assert np.all(np.abs(g - want) <= 1e-2 + 2e-2 * np.abs(want))
  two = bdg.dot_general(bq.quantize(xt, bdg.get_how_to_quantize(for_lhs=True, **kw)), wq, DN)
  if qtype == 'int8':   # exact int32 sums: any split of K gives the same bits
    assert torch.equal(out.view(torch.int16), two.view(torch.int16))
  else:                 # float32 sums may be added in another order when K is split
    assert torch.allclose(out.float(), two.float(), rtol=2 ** -7, atol=1e-3)
  _lib.raise_on_device_error()


def test_quantized_matmul_rejects_bad_arguments():
  from qwix_b200 import fused
  x = torch.zeros((4, 256), dtype=torch.bfloat16, device='cuda')
  w = bq.quantize(torch.ones((256, 32), dtype=torch.bfloat16, device='cuda'),
                  bq.HowToQuantize(qtype='int8', channelwise_axes=[1]))
  with pytest.raises(ValueError):
    fused.quantized_matmul(x.float(), w)
  with pytest.raises(ValueError):
    fused.quantized_matmul(x[:, :128], w)
  L = _lib.lib()
  out = torch.empty((4, 32), dtype=torch.bfloat16, device='cuda')
  ws = torch.empty(L.qwx_quant_gemm_q8_workspace_bytes(4, 256), dtype=torch.uint8, device='cuda')
  args = lambda nbytes: (_lib.ptr(x), 4, 256, _lib.ptr(w.qvalue), _lib.ptr(w.scale), 32, _lib.S8,
                         _lib.B_KN, 0, _lib.ptr(out), _lib.BF16, 0, _lib.ptr(ws), nbytes, None,
                         _lib.stream_ptr())
  assert L.qwx_quant_gemm_q8(*args(ws.numel() - 1)) == 6      # QWX_ERR_WORKSPACE
  assert L.qwx_quant_gemm_q8(*args(ws.numel())) == 0
  torch.cuda.synchronize()


# ---- the swapped-operand decode kernel (tokens are the MMA's N) ---------------------------------

def _decode_gemm(a, w, out_dtype=torch.int32, sa=None, sb=None, ws=None, epilogue=0):
  M, K = a.shape
  N = w.shape[0]
  L = _lib.lib()
  need = L.qwx_gemm_q8_decode_workspace_bytes(M, N)
  if ws is None:
    ws = torch.zeros(need, dtype=torch.uint8, device='cuda')
  out = torch.empty((M, N), dtype=out_dtype, device='cuda')
  err = torch.zeros(1, dtype=torch.int32, device='cuda')
  oc = {torch.int32: _lib.S32, torch.float32: _lib.F32, torch.bfloat16: _lib.BF16}[out_dtype]
  _lib.check(L.qwx_gemm_q8_decode(_lib.ptr(a), _lib.ptr(w), M, N, K, _lib.ptr(sa), _lib.ptr(sb),
                                  _lib.F32, _lib.ptr(out), oc, epilogue, _lib.ptr(ws), ws.numel(), 1,
                                  _lib.ptr(err), _lib.stream_ptr()), 'gemm_q8_decode')
  torch.cuda.synchronize()
  assert int(err.item()) == 0
  return out, ws


DECODE_KERNEL_SHAPES = [
    (32, 4096, 4096),     # 32 tiles x 16 stages on 148 CTAs: every tile shared by 4-5 CTAs
    (32, 6144, 4096), (32, 28672, 4096), (32, 4096, 14336),
    (32, 128256, 4096),   # 1002 tiles: most owned whole, one shared at every CTA boundary
    (32, 768, 4096), (32, 4096, 512), (32, 3584, 4096), (32, 4096, 1792),   # 1/8 shards: units < SMs
    (1, 1024, 14336), (7, 1000, 272), (33, 2048 + 48, 512 + 32), (64, 4096, 4096),
    (100, 1536, 2048), (128, 8192, 2048), (5, 128, 256), (32, 128, 128),
]


@pytest.mark.parametrize('mnk', DECODE_KERNEL_SHAPES, ids=[f'{m}x{n}x{k}' for m, n, k in DECODE_KERNEL_SHAPES])
def test_decode_kernel_bit_exact(mnk):
  M, N, K = mnk
  rng = np.random.default_rng(M + N + K)
  a = rng.integers(-128, 128, (M, K), dtype=np.int8)
  w = rng.integers(-128, 128, (N, K), dtype=np.int8)
  want = (a.astype(np.float64) @ w.astype(np.float64).T).astype(np.int64)   # exact: |sums| < 2^53
  at, wt = h.to_torch(a), h.to_torch(w)
  got, ws = _decode_gemm(at, wt)
  assert np.array_equal(got.cpu().numpy().astype(np.int64), want)
  assert int(ws.count_nonzero().item()) == 0          # scratch slots and counters are left zero
  # second call on the same scratch; scaled outputs equal the ordinary kernel's bit for bit
  sa = torch.rand(M, device='cuda') + 0.5
  sb = torch.rand(N, device='cuda') * 1e-3
  for epi in (0, 1):
    got2, ws = _decode_gemm(at, wt, out_dtype=torch.bfloat16, sa=sa, sb=sb, ws=ws, epilogue=epi)
    ref = torch.empty_like(got2)
    err = torch.zeros(1, dtype=torch.int32, device='cuda')
    _lib.check(_lib.lib().qwx_gemm_q8(_lib.ptr(at), _lib.ptr(wt), _lib.S8, _lib.B_NK, M, N, K, 0,
                                      _lib.ptr(sa), 0, _lib.ptr(sb), 0, _lib.F32, _lib.ptr(ref),
                                      _lib.BF16, epi, _lib.ptr(err), _lib.stream_ptr()), 'gemm')
    torch.cuda.synchronize()
    assert torch.equal(got2.view(torch.int16), ref.view(torch.int16))
  assert int(ws.count_nonzero().item()) == 0


def test_decode_kernel_through_dot_general_and_errors():
  L = _lib.lib()
  rng = np.random.default_rng(1)
  a = rng.integers(-128, 128, (32, 1024), dtype=np.int8)
  w = rng.integers(-128, 128, (1024, 512), dtype=np.int8)       # logical [K, N]
  wt = h.to_torch(w).t().contiguous().t()                       # stored [N, K]
  old = bdg.DECODE_MAX_ROWS
  try:
    bdg.DECODE_MAX_ROWS = 128            # route this contraction through the decode kernel
    got = bdg.dot_general(h.to_torch(a), wt, DN)
  finally:
    bdg.DECODE_MAX_ROWS = old
  assert np.array_equal(got.cpu().numpy(), a.astype(np.int32) @ w.astype(np.int32))
  # with programmatic dependent launch switched on the results are the same
  L.qwx_set_programmatic_launch(1)
  try:
    bdg.DECODE_MAX_ROWS = 128
    again = bdg.dot_general(h.to_torch(a), wt, DN)
    q = bq.quantize(torch.randn(64, 4096, device='cuda').to(torch.bfloat16),
                    bq.HowToQuantize(qtype='int8', channelwise_axes=[0]))
  finally:
    bdg.DECODE_MAX_ROWS = old
    L.qwx_set_programmatic_launch(0)
  assert L.qwx_get_programmatic_launch() == 0
  assert torch.equal(again, got) and q.qvalue.shape == (64, 4096)
  assert L.qwx_gemm_q8_decode_workspace_bytes(129, 512) == 0
  x = torch.zeros(16, dtype=torch.uint8, device='cuda')
  args = (_lib.ptr(x), _lib.ptr(x), 200, 512, 1024, None, None, _lib.F32, _lib.ptr(x), _lib.S32, 0,
          _lib.ptr(x), 16, 1, None, _lib.stream_ptr())
  assert L.qwx_gemm_q8_decode(*args) == 5                        # more than 128 rows: unsupported
  args = (_lib.ptr(x), _lib.ptr(x), 32, 512, 1024, None, None, _lib.F32, _lib.ptr(x), _lib.S32, 0,
          _lib.ptr(x), 16, 1, None, _lib.stream_ptr())
  assert L.qwx_gemm_q8_decode(*args) == 6                        # workspace too small


# ---- decode-shaped calls on narrow column tiles (no K cut) -------------------------------------

NARROW_SHAPES = [(32, 4096, 4096), (1, 4736, 512), (7, 6144, 1024), (100, 3000, 384), (128, 28672, 256),
                 (33, 2400, 4096 + 128), (32, 14336, 5120)]


@pytest.mark.parametrize('mnk', NARROW_SHAPES, ids=[f'{m}x{n}x{k}' for m, n, k in NARROW_SHAPES])
def test_narrow_tiles_int8_bit_exact(mnk):
  """Up to 128 rows against an [N, K] weight whose narrow column tiles fill at least half of the
  SMs: raw int32 accumulator bit-exact, the float32 and the reference-order epilogue equal to
  the wide kernel's arithmetic (restated here in NumPy)."""
  M, N, K = mnk
  rng = np.random.default_rng(M + N + K)
  a = rng.integers(-128, 128, (M, K), dtype=np.int8)
  b = rng.integers(-128, 128, (N, K), dtype=np.int8)
  want = a.astype(np.int32) @ b.astype(np.int32).T
  at, bt = h.to_torch(a), h.to_torch(b)
  L = _lib.lib()
  err = torch.zeros(1, dtype=torch.int32, device='cuda')
  out = torch.empty((M, N), dtype=torch.int32, device='cuda')
  _lib.check(L.qwx_gemm_q8(_lib.ptr(at), _lib.ptr(bt), _lib.S8, _lib.B_NK, M, N, K, 0, None, 0, None, 0,
                           _lib.F32, _lib.ptr(out), _lib.S32, 0, _lib.ptr(err), _lib.stream_ptr()), 'gemm')
  torch.cuda.synchronize()
  assert int(err.item()) == 0
  assert np.array_equal(out.cpu().numpy(), want)
  sa = (rng.random(M) + 0.5).astype(np.float32)
  sb = (rng.random(N) * 1e-3).astype(np.float32)
  sa_t, sb_t = h.to_torch(sa), h.to_torch(sb)
  for epi, odt in ((0, torch.float32), (0, torch.bfloat16), (1, torch.bfloat16)):
    o = torch.empty((M, N), dtype=odt, device='cuda')
    oc = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16}[odt]
    _lib.check(L.qwx_gemm_q8(_lib.ptr(at), _lib.ptr(bt), _lib.S8, _lib.B_NK, M, N, K, 0,
                             _lib.ptr(sa_t), 0, _lib.ptr(sb_t), 0, _lib.F32, _lib.ptr(o), oc,
                             epi, _lib.ptr(err), _lib.stream_ptr()), 'gemm')
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    f = want.astype(np.float32)
    if epi == 0:
      ref = (f * sa[:, None]) * sb[None, :]
      ref_t = torch.from_numpy(ref).to(odt)
    else:
      import ml_dtypes
      bf = ml_dtypes.bfloat16
      r = f.astype(bf).astype(np.float32)
      r = (r * sa[:, None]).astype(bf).astype(np.float32)
      r = (r * sb[None, :]).astype(bf)
      ref_t = torch.from_numpy(r.astype(np.float32)).to(odt)
    assert torch.equal(o.cpu(), ref_t), (epi, odt)


def test_narrow_tiles_fp8():
  import ml_dtypes
  M, N, K = 16, 4096, 2048
  rng = np.random.default_rng(5)
  a = rng.standard_normal((M, K)).astype(np.float32).astype(ml_dtypes.float8_e4m3fn)
  b = rng.standard_normal((N, K)).astype(np.float32).astype(ml_dtypes.float8_e4m3fn)
  want = a.astype(np.float32) @ b.astype(np.float32).T
  got = _raw_gemm(h.to_torch(a), h.to_torch(b), _lib.B_NK, code=_lib.E4M3, out_dtype=torch.float32)
  assert np.abs(got.cpu().numpy() - want).max() <= 1e-3 * np.abs(want).max()
