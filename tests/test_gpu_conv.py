"""Quantized conv_general_dilated against the oracle (after tests/_src/core/conv_general_test.py:
int8 / e4m3 operands quantized per image and per output channel, strides, paddings, filter
dilation; one- and two-dimensional windows)."""

import ml_dtypes
import numpy as np
import pytest
import torch

from oracle import conv_general as oc
from oracle import qarray as oq
from qwix_b200.core import conv_general as bc
from qwix_b200.core import qarray as bq
from tests import helpers as h

pytestmark = pytest.mark.gpu
bf16 = ml_dtypes.bfloat16
DN = ('NHWC', 'HWIO', 'NHWC')


def _close(got, want):
  g, r = h.to_numpy(got).astype(np.float32), np.asarray(want).astype(np.float32)
  assert g.shape == r.shape
  bad = np.abs(g - r) > 1e-2 + 2e-2 * np.abs(r)
  assert not bad.any(), f'{bad.sum()} of {bad.size} outside 1e-2 / 2e-2, worst {np.abs(g - r).max()}'


CASES = [
    # x shape, filter shape, strides, padding, filter dilation, qtype
    ((3, 16, 16, 32), (3, 3, 32, 48), (1, 1), 'SAME', None, 'int8'),
    ((2, 17, 15, 16), (3, 3, 16, 32), (2, 2), 'SAME', None, 'int8'),
    ((2, 12, 12, 16), (5, 3, 16, 16), (1, 2), 'VALID', (2, 1), 'int8'),
    ((2, 9, 10, 32), (1, 1, 32, 64), (1, 1), [(0, 0), (0, 0)], None, 'float8_e4m3fn'),
    ((2, 11, 9, 16), (3, 3, 16, 24), (1, 1), [(1, 2), (0, 1)], None, 'int8'),
    ((4, 64, 16), (5, 16, 32), (2,), 'SAME', None, 'int8'),                  # one spatial axis
]


@pytest.mark.parametrize('case', CASES, ids=[str(c[:2]) + str(c[3]) for c in CASES])
@pytest.mark.parametrize('dtype', ['float32', 'bfloat16'])
def test_conv_matches_oracle(case, dtype):
  xs, ks, strides, padding, dil, qtype = case
  rng = np.random.default_rng(sum(xs))
  x = rng.standard_normal(xs).astype(np.float32).astype(h.np_dtype(dtype))
  k = (0.2 * rng.standard_normal(ks)).astype(np.float32).astype(h.np_dtype(dtype))
  nd = len(xs)
  dn = bc.conv_dimension_numbers(xs, ks, DN if nd == 4 else ('NWC', 'WIO', 'NWC'))
  lo = oq.quantize(x, oc.get_how_to_quantize(for_lhs=True, ndim=nd, qtype=qtype))
  ro = oq.quantize(k, oc.get_how_to_quantize(for_lhs=False, ndim=nd, qtype=qtype))
  lb = bq.quantize(h.to_torch(x), bc.get_how_to_quantize(dimension_numbers=dn, for_lhs=True, qtype=qtype))
  rb = bq.quantize(h.to_torch(k), bc.get_how_to_quantize(dimension_numbers=dn, for_lhs=False, qtype=qtype))
  assert h.codes_equal(lb.qvalue, lo.qvalue) and h.codes_equal(rb.qvalue, ro.qvalue)
  assert tuple(lb.scale.shape) == lo.scale.shape and tuple(rb.scale.shape) == ro.scale.shape
  want = oc.conv_general_dilated(lo, ro, strides, padding, dil)
  got = bc.conv_general_dilated(lb, rb, strides, padding, rhs_dilation=dil, dimension_numbers=dn)
  assert h.to_numpy(got).dtype == want.dtype
  _close(got, want)
  # and the quantized result approximates the float convolution
  ref = oc.lax_conv(x.astype(np.float32), k.astype(np.float32), list(strides), padding, dil, np.float32)
  g = h.to_numpy(got).astype(np.float32)
  assert np.abs(g - ref).mean() / np.abs(ref).mean() < (0.08 if qtype != 'int8' else 0.04)


def test_float_filter_takes_the_dequantize_path_and_refusals():
  rng = np.random.default_rng(1)
  x = rng.standard_normal((2, 8, 8, 16)).astype(np.float32)
  k = rng.standard_normal((3, 3, 16, 8)).astype(np.float32)
  dn = bc.conv_dimension_numbers(x.shape, k.shape, DN)
  lo = oq.quantize(x, oc.get_how_to_quantize(for_lhs=True, ndim=4, qtype='int8'))
  lb = bq.quantize(h.to_torch(x), bc.get_how_to_quantize(dimension_numbers=dn, for_lhs=True, qtype='int8'))
  want = oc.conv_general_dilated(lo, k, (1, 1), 'SAME')                      # conv_general.py:252-256
  got = bc.conv_general_dilated(lb, h.to_torch(k), (1, 1), 'SAME', dimension_numbers=dn)
  # the library convolution may run float32 operands on TF32 tensor cores: the stated output tolerance
  np.testing.assert_allclose(h.to_numpy(got), want, rtol=2e-2, atol=1e-2)
  with pytest.raises(NotImplementedError):
    bc.conv_general_dilated(lb, h.to_torch(k), (1, 1), 'SAME', dimension_numbers=dn, feature_group_count=2)
  with pytest.raises(NotImplementedError):
    bc.conv_general_dilated(lb, h.to_torch(k), (1, 1), 'SAME', lhs_dilation=(2, 2), dimension_numbers=dn)
  with pytest.raises(NotImplementedError):
    bc.conv_general_dilated(lb, h.to_torch(k), (1, 1), 'SAME')               # lax's NCHW / OIHW default
  tiled = bq.quantize(h.to_torch(x), bq.HowToQuantize(qtype='int8', channelwise_axes=[0], tiled_axes={3: 8}))
  rq = bq.quantize(h.to_torch(k), bc.get_how_to_quantize(dimension_numbers=dn, for_lhs=False, qtype='int8'))
  with pytest.raises(ValueError, match='subchannel'):
    bc.conv_general_dilated(tiled, rq, (1, 1), 'SAME', dimension_numbers=dn)


def test_conv_module_under_the_ptq_provider():
  """A small convolutional stack (Conv 3x3 -> ReLU -> Conv 3x3 stride 2) under a `.*` int8 rule:
  the provider quantizes each filter per output channel at first use and each input per image
  (boxed_param.py:238-314), against the oracle on the same weights."""
  import qwix_b200 as qwix
  from qwix_b200 import nn

  class Net(torch.nn.Module):
    def __init__(self):
      super().__init__()
      g = torch.Generator().manual_seed(3)
      self.Conv_0 = nn.Conv(16, 32, (3, 3), use_bias=False, generator=g)
      self.Conv_1 = nn.Conv(32, 16, (3, 3), strides=(2, 2), use_bias=False, generator=g)

    def forward(self, x):
      return self.Conv_1(torch.relu(self.Conv_0(x)))

  model = Net().cuda()
  x = torch.randn(2, 12, 12, 16, generator=torch.Generator().manual_seed(4)).cuda()
  k0, k1 = h.to_numpy(model.Conv_0.kernel.data), h.to_numpy(model.Conv_1.kernel.data)
  float_out = h.to_numpy(model(x))
  rules = [qwix.QuantizationRule(module_path='.*', weight_qtype='int8', act_qtype='int8')]
  ptq_model = qwix.quantize_model(model, qwix.PtqProvider(rules))
  got = ptq_model(x)

  how = lambda for_lhs: oc.get_how_to_quantize(for_lhs=for_lhs, ndim=4, qtype='int8')
  k0q, k1q = oq.quantize(k0, how(False)), oq.quantize(k1, how(False))
  hid = oc.conv_general_dilated(oq.quantize(h.to_numpy(x), how(True)), k0q, (1, 1), 'SAME')
  hid = np.maximum(hid, np.zeros((), hid.dtype))
  want = oc.conv_general_dilated(oq.quantize(hid, how(True)), k1q, (2, 2), 'SAME')
  box = ptq_model.params()['Conv_0']['kernel']
  assert isinstance(box, qwix.WithAux) and h.codes_equal(box.array.qvalue, k0q.qvalue)
  assert tuple(box.array.scale.shape) == k0q.scale.shape == (1, 1, 1, 32)
  _close(got, want)
  g = h.to_numpy(got)
  assert np.abs(g - float_out).mean() / np.abs(float_out).mean() < 0.05
