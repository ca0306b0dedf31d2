"""GPU: the README MLP (Dense 16->64, ReLU, Dense 64->16) under PtqProvider (w8a8), end to end through the
provider / model wrapper / quantize_params, against the CPU oracle on the same weights."""

import ml_dtypes
import numpy as np
import pytest
import torch

import qwix_b200 as qwix
from oracle import dot_general as odg
from oracle import qarray as oq
from qwix_b200 import nn
from tests import helpers as h

pytestmark = pytest.mark.gpu
DN = (((1,), (0,)), ((), ()))


class MLP(torch.nn.Module):
  """Dense 16 -> 64 (no bias), ReLU, Dense 64 -> 16 (no bias), lecun_normal init."""

  def __init__(self, dtype=torch.float32, seed=1):
    super().__init__()
    g = torch.Generator().manual_seed(seed)
    self.Dense_0 = nn.Dense(16, 64, use_bias=False, dtype=dtype, generator=g)
    self.Dense_1 = nn.Dense(64, 16, use_bias=False, dtype=dtype, generator=g)

  def forward(self, x):
    return self.Dense_1(torch.relu(self.Dense_0(x)))


def _oracle_forward(x, w0, w1):
  kw = dict(dimension_numbers=DN, ndims=(2, 2), tile_size=None, qtype='int8')
  how_l = odg.get_how_to_quantize(for_lhs=True, **kw)
  how_r = odg.get_how_to_quantize(for_lhs=False, **kw)
  w0q, w1q = oq.quantize(w0, how_r), oq.quantize(w1, how_r)
  hid = odg.dot_general(oq.quantize(x, how_l), w0q, DN)
  hid = np.maximum(hid, np.zeros((), hid.dtype))
  return odg.dot_general(oq.quantize(hid, how_l), w1q, DN), w0q, w1q, hid


@pytest.mark.parametrize('dtype', ['float32', 'bfloat16'])
def test_readme_mlp_w8a8(dtype):
  tdt = {'float32': torch.float32, 'bfloat16': torch.bfloat16}[dtype]
  model = MLP(dtype=tdt).cuda()
  x = torch.rand(8, 16, generator=torch.Generator().manual_seed(0)).to(tdt).cuda()
  w0, w1 = h.to_numpy(model.Dense_0.kernel.data), h.to_numpy(model.Dense_1.kernel.data)
  fp_params = qwix.model.get_params(model)
  fp_out = model(x)

  rules = [qwix.QuantizationRule(module_path='.*', weight_qtype='int8', act_qtype='int8')]
  provider = qwix.PtqProvider(rules)
  ptq_model = qwix.quantize_model(model, provider)
  got = ptq_model(x)                      # first call quantizes the weights in place
  want, w0q, w1q, _ = _oracle_forward(h.to_numpy(x), w0, w1)

  tree = ptq_model.params()
  for name, wq in (('Dense_0', w0q), ('Dense_1', w1q)):
    box = tree[name]['kernel']
    assert isinstance(box, qwix.WithAux) and isinstance(box.array, qwix.QArray)
    assert box.array.qvalue.dtype == torch.int8 and box.array.scale.dtype == tdt
    assert tuple(box.array.scale.shape) == (1, wq.qvalue.shape[1])
    assert h.codes_equal(box.array.qvalue, wq.qvalue)
    assert np.array_equal(h.to_numpy(box.array.scale).view(np.uint8), wq.scale.view(np.uint8))
    assert list(box.how.channelwise_axes) == [1] and box.how.qtype == 'int8'

  g, r = h.to_numpy(got).astype(np.float32), want.astype(np.float32)
  if dtype == 'float32':
    # float32: the epilogue keeps the reference's order (float(acc) * sa) * sw -> same bits
    assert np.array_equal(g, r)
  else:
    assert np.all(np.abs(g - r) <= 1e-2 + 2e-2 * np.abs(r))
  rel = np.abs(g - h.to_numpy(fp_out).astype(np.float32)).mean() / np.abs(h.to_numpy(fp_out).astype(np.float32)).mean()
  assert rel < 0.03                       # einsum_test.py:40-127: w8a8 stays within ~2 %
  assert provider.get_unused_rules() == []
  again = ptq_model(x)                    # weights are now WithAux: no re-quantization
  assert torch.equal(again, got)

  # quantize_params offline == what the first call produced (ptq_test.py:36-86)
  offline = qwix.quantize_params(fp_params, tree)
  for name in ('Dense_0', 'Dense_1'):
    a, b = offline[name]['kernel'].array, tree[name]['kernel'].array
    assert torch.equal(a.qvalue, b.qvalue) and torch.equal(a.scale, b.scale)
  fresh = MLP(dtype=tdt, seed=99).cuda()
  qwix.model.set_params(fresh, offline)
  assert torch.equal(qwix.quantize_model(fresh, qwix.PtqProvider(rules))(x), got)


def test_weight_only_and_subchannel_rules():
  # Dense 12 -> 5 with tile_size 4 on weights only (ptq_test.py:36-86 structure).
  lin = nn.Dense(12, 5, use_bias=False, dtype=torch.float32).cuda()
  w = h.to_numpy(lin.kernel.data)
  x = torch.rand(3, 12).cuda()

  class Wrap(torch.nn.Module):
    def __init__(self):
      super().__init__()
      self.Dense_0 = lin
    def forward(self, v):
      return self.Dense_0(v)

  rules = [qwix.QuantizationRule(module_path='Dense_0', weight_qtype='int8', tile_size=4)]
  m = qwix.quantize_model(Wrap(), qwix.PtqProvider(rules))
  got = m(x)
  box = m.params()['Dense_0']['kernel']
  assert tuple(box.array.scale.shape) == (3, 5) and dict(box.how.tiled_axes) == {0: 4}
  wq = oq.quantize(w, oq.HowToQuantize(qtype='int8', channelwise_axes=[1], tiled_axes={0: 4}))
  assert h.codes_equal(box.array.qvalue, wq.qvalue)
  want = odg.dot_general(h.to_numpy(x), wq, DN)     # weight-only: dequantize-first path
  assert np.allclose(h.to_numpy(got), want, rtol=1e-5, atol=1e-6)
