"""CPU checks of the oracles for the microscaled dot, ragged_dot and conv: properties the
restated arithmetic must have, and an independent library (PyTorch on the CPU) for the
convolution's index arithmetic.  The reference's own contraction for these paths lives in jax,
which is absent, so these pins are properties, not outputs of the reference."""

import ml_dtypes
import numpy as np
import pytest
import torch

from oracle import conv_general as oc
from oracle import dot_general as odg
from oracle import mxfp_dot as omx
from oracle import qarray as oq
from oracle import ragged_dot as orr

bf16 = ml_dtypes.bfloat16
DN = (((1,), (0,)), ((), ()))


def test_scaled_matmul_with_unit_scales_is_matmul():
  # tests/_src/core/mxfp_dot_test.py:154-167 (test_matmul_f32_baseline)
  rng = np.random.default_rng(123)
  lhs = rng.uniform(-1, 1, (1, 32, 64)).astype(np.float32)
  rhs = rng.uniform(-1, 1, (1, 32, 64)).astype(np.float32)
  one = np.ones((1, 32, 2), np.float32)
  np.testing.assert_allclose(omx.scaled_matmul(lhs, rhs, one, one),
                             np.einsum('bmk,bnk->bmn', lhs, rhs), rtol=5e-3, atol=5e-3)


def test_scaled_matmul_scales_act_per_block():
  rng = np.random.default_rng(0)
  lhs = rng.standard_normal((1, 4, 64)).astype(np.float32)
  rhs = rng.standard_normal((1, 3, 64)).astype(np.float32)
  sa, sb = np.ones((1, 4, 2), np.float32), np.ones((1, 3, 2), np.float32)
  base = omx.scaled_matmul(lhs, rhs, sa, sb)
  sa2 = sa.copy(); sa2[0, 1, 1] = 4.0                      # row 1, second block of 32
  want = base.copy()
  want[0, 1] += 3.0 * (lhs[0, 1, 32:] @ rhs[0, :, 32:].T)
  np.testing.assert_allclose(omx.scaled_matmul(lhs, rhs, sa2, sb), want, rtol=1e-5, atol=1e-5)


def test_mxfp8_quantize_then_dot_is_close_to_the_float_product():
  rng = np.random.default_rng(1)
  x = rng.standard_normal((16, 128)).astype(np.float32)
  w = (0.1 * rng.standard_normal((128, 24))).astype(np.float32)
  kw = dict(dimension_numbers=DN, ndims=(2, 2), tile_size=32, qtype='mxfp8')
  a = oq.quantize(x, odg.get_how_to_quantize(for_lhs=True, **kw))
  b = oq.quantize(w, odg.get_how_to_quantize(for_lhs=False, **kw))
  assert a.scale.shape == (16, 4) and b.scale.shape == (4, 24)
  assert np.all(np.frexp(a.scale)[0] == 0.5) and np.all(np.frexp(b.scale)[0] == 0.5)
  out = omx.mxfp_dot_general(a, b, DN)
  ref = x @ w
  assert np.abs(out - ref).mean() / np.abs(ref).mean() < 0.05
  # the microscaled dispatcher declines anything that is not microscaled on both sides (mxfp_dot.py:51-52)
  assert omx.mxfp_dot_general(a, w, DN) is None
  # and agrees with dequantize-then-contract, which is what the fallback computes
  np.testing.assert_allclose(out, odg.slow_dot_general(a, b, DN), rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize('qtype,tile,bound', [('mxfp4', 32, 0.25), ('nvfp4', 16, 0.2)])
def test_four_bit_quantize_then_dot(qtype, tile, bound):
  """e2m1 codes (qarray.py:566-581, numerics.py:186-187): the scales are powers of two (mxfp4)
  or e4m3 numbers (nvfp4), the codes lie on the e2m1 grid, and the microscaled dot agrees with
  dequantize-then-contract."""
  import ml_dtypes
  rng = np.random.default_rng(3)
  x = rng.standard_normal((16, 128)).astype(np.float32)
  w = (0.1 * rng.standard_normal((128, 24))).astype(np.float32)
  kw = dict(dimension_numbers=DN, ndims=(2, 2), tile_size=tile, qtype=qtype)
  a = oq.quantize(x, odg.get_how_to_quantize(for_lhs=True, **kw))
  b = oq.quantize(w, odg.get_how_to_quantize(for_lhs=False, **kw))
  assert a.scale.shape == (16, 128 // tile) and b.scale.shape == (128 // tile, 24)
  if qtype == 'mxfp4':
    assert np.all(np.frexp(a.scale)[0] == 0.5) and np.all(np.frexp(b.scale)[0] == 0.5)
  else:
    for s in (a.scale, b.scale):
      assert np.array_equal(s.astype(ml_dtypes.float8_e4m3fn).astype(np.float32), s.astype(np.float32))
  grid = {0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0}
  assert set(np.abs(a.qvalue.astype(np.float32)).ravel().tolist()) <= grid
  # absmax of every block maps to a code of magnitude at least 4 (the scale keeps the range in use)
  assert np.all(np.abs(a.qvalue.astype(np.float32)).reshape(16, -1, tile).max(axis=2) >= 3.0)
  out = omx.mxfp_dot_general(a, b, DN)
  ref = x @ w
  assert np.abs(out - ref).mean() / np.abs(ref).mean() < bound
  np.testing.assert_allclose(out, odg.slow_dot_general(a, b, DN), rtol=1e-5, atol=1e-5)


def test_ragged_dot_groups_and_leftover_rows():
  rng = np.random.default_rng(2)
  x = rng.standard_normal((20, 32)).astype(np.float32)
  w = rng.standard_normal((3, 32, 8)).astype(np.float32)
  a = oq.quantize(x, oq.HowToQuantize(qtype='int8', channelwise_axes=[0]))
  b = oq.quantize(w, oq.HowToQuantize(qtype='int8', channelwise_axes=[0, 2]))
  out = orr.ragged_dot(a, b, [6, 0, 9])
  ref = np.zeros((20, 8), np.float32)
  ref[:6], ref[6:15] = x[:6] @ w[0], x[6:15] @ w[2]
  assert not out[15:].any()
  assert np.abs(out - ref).mean() / np.abs(ref[:15]).mean() < 0.03
  # a float operand sends the call down the dequantize-first path (ragged_dot.py:275-285)
  assert not orr.use_fast_path(x, b) and orr.use_fast_path(a, b)
  np.testing.assert_allclose(orr.ragged_dot(x, w, [6, 0, 9])[:15], ref[:15], rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize('padding', ['SAME', 'VALID', [(1, 2), (0, 1)]])
@pytest.mark.parametrize('strides', [(1, 1), (2, 2), (1, 3)])
@pytest.mark.parametrize('dilation', [(1, 1), (2, 1)])
def test_conv_index_arithmetic_against_an_independent_library(padding, strides, dilation):
  rng = np.random.default_rng(3)
  x = rng.standard_normal((2, 9, 11, 3)).astype(np.float32)
  k = rng.standard_normal((3, 2, 3, 5)).astype(np.float32)
  got = oc.lax_conv(x, k, list(strides), padding, list(dilation), np.float32)
  pads = oc.explicit_padding(padding, x.shape[1:3], k.shape[:2], strides, dilation)
  xt = torch.from_numpy(x).permute(0, 3, 1, 2)
  xt = torch.nn.functional.pad(xt, [pads[1][0], pads[1][1], pads[0][0], pads[0][1]])
  want = torch.nn.functional.conv2d(xt, torch.from_numpy(k).permute(3, 2, 0, 1), stride=strides,
                                    dilation=dilation).permute(0, 2, 3, 1).numpy()
  assert got.shape == want.shape
  np.testing.assert_allclose(got, want, rtol=1e-4, atol=1e-4)
  if padding == 'SAME':      # lax: ceil(in / stride) output positions
    assert got.shape[1:3] == (-(-9 // strides[0]), -(-11 // strides[1]))


def test_integer_conv_is_exact_and_scales_factor_out():
  rng = np.random.default_rng(4)
  x = rng.standard_normal((2, 6, 6, 8)).astype(np.float32)
  k = rng.standard_normal((3, 3, 8, 4)).astype(np.float32)
  a = oq.quantize(x, oc.get_how_to_quantize(for_lhs=True, ndim=4, qtype='int8'))
  b = oq.quantize(k, oc.get_how_to_quantize(for_lhs=False, ndim=4, qtype='int8'))
  assert a.scale.shape == (2, 1, 1, 1) and b.scale.shape == (1, 1, 1, 4)
  acc = oc.lax_conv(a.qvalue, b.qvalue, [1, 1], 'SAME', None, np.int32)
  assert acc.dtype == np.int32
  out = oc.conv_general_dilated(a, b, (1, 1), 'SAME')
  np.testing.assert_array_equal(out, (acc.astype(np.float32) * a.scale) * b.scale)
  ref = oc.lax_conv(x, k, [1, 1], 'SAME', None, np.float32)
  assert np.abs(out - ref).mean() / np.abs(ref).mean() < 0.03


def test_host_side_conv_helpers():
  from qwix_b200.core import conv_general as bc
  dn = bc.conv_dimension_numbers((2, 8, 8, 3), (3, 3, 3, 4), ('NHWC', 'HWIO', 'NHWC'))
  assert dn.lhs_spec == (0, 3, 1, 2) and dn.rhs_spec == (3, 2, 0, 1) and dn.out_spec == (0, 3, 1, 2)
  assert bc.get_how_to_quantize(dimension_numbers=dn, for_lhs=True, qtype='int8').channelwise_axes == [0]
  assert bc.get_how_to_quantize(dimension_numbers=dn, for_lhs=False, qtype='int8').channelwise_axes == [3]
  same = bc._explicit_padding('SAME', (9, 11), (3, 2), (2, 2), (1, 1))
  assert same == oc.explicit_padding('SAME', (9, 11), (3, 2), (2, 2), (1, 1))
  x = torch.arange(2 * 5 * 6 * 3, dtype=torch.int8).reshape(2, 5, 6, 3)
  p = bc._patches(x, [3, 2], [1, 2], [(1, 1), (0, 1)], [1, 1])
  assert tuple(p.shape) == (2, 5, 3, 3, 2, 3)
  assert int(p[0, 0, 0, 0, 0, 0]) == 0                     # the padding row above the image
  assert torch.equal(p[1, 2, 1, 1, 0], x[1, 2, 2])         # centre tap of a window


def test_how_to_quantize_validates_microscaling_tiles():
  from qwix_b200.core import qarray as bq
  with pytest.raises(ValueError):
    bq.HowToQuantize(qtype='mxfp8', channelwise_axes=[0], tiled_axes={1: 16})
  bq.HowToQuantize(qtype='mxfp8', channelwise_axes=[0], tiled_axes={1: 32})
