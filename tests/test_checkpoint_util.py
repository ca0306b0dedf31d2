"""Pre-quantized checkpoints (qwix/_src/utils/checkpoint_util.py:383-587): rule
reconstruction, the disk format and the validation errors on CPU; loading into a PTQ model
(the three checkpoint x template cases) on the GPU."""

import numpy as np
import pytest
import torch

import qwix_b200 as qwix
from qwix_b200 import nn
from qwix_b200.utils import checkpoint_util as cu


def _tree():
  g = torch.Generator().manual_seed(0)
  q4 = torch.randint(-8, 8, (6, 10), generator=g, dtype=torch.int8)
  q8 = torch.randint(-128, 128, (6, 10), generator=g, dtype=torch.int8)
  return {'layers': {'0': {'attn': {'kernel': {'qvalue': q4, 'scale': torch.rand(1, 10), 'qtype': 'int4'}},
                           'norm': {'scale': torch.ones(6)}},
                     '1': {'mlp': {'kernel': {'array': {'qvalue': q8, 'scale': torch.rand(1, 10),
                                                        'zero_point': torch.zeros(1, 10, dtype=torch.int8)}}}}}}


def test_restore_quantization_rules():
  rules = cu.restore_quantization_rules(_tree(), tile_size=128)
  got = {r.module_path: r for r in rules}
  assert set(got) == {'layers/[^/]+/attn', 'layers/[^/]+/mlp'}       # indices became wildcards
  a, m = got['layers/[^/]+/attn'], got['layers/[^/]+/mlp']
  assert (a.weight_qtype, a.act_qtype, a.weight_calibration_method, a.tile_size) == ('int4', 'int4', 'absmax', 128)
  assert (m.weight_qtype, m.weight_calibration_method) == ('int8', 'minmax')   # zero point -> minmax
  wo = cu.restore_quantization_rules(_tree(), tile_size=None, act_qtype=None)
  assert all(r.act_qtype is None for r in wo)                         # weight-only on request
  assert cu.restore_quantization_rules({'a': {'w': torch.ones(3)}}, tile_size=None) == []


def test_disk_round_trip_packs_int4(tmp_path):
  tree = _tree()
  f = str(tmp_path / 'w.safetensors')
  cu.save_prequantized(tree, f)
  back = cu.load_prequantized(f)
  k0 = back['layers']['0']['attn']['kernel']
  assert k0['qtype'] == 'int4' and torch.equal(k0['qvalue'], tree['layers']['0']['attn']['kernel']['qvalue'])
  k1 = back['layers']['1']['mlp']['kernel']['array']
  assert torch.equal(k1['qvalue'], tree['layers']['1']['mlp']['kernel']['array']['qvalue'])
  assert torch.equal(k1['zero_point'], tree['layers']['1']['mlp']['kernel']['array']['zero_point'])
  assert torch.equal(back['layers']['0']['norm']['scale'], torch.ones(6))
  # two codes per byte on disk, low nibble = even index
  from safetensors import safe_open
  with safe_open(f, framework='pt') as h:
    raw = h.get_tensor('layers/0/attn/kernel.qvalue')
  q = tree['layers']['0']['attn']['kernel']['qvalue']
  assert raw.shape == (6, 5) and raw.dtype == torch.uint8
  assert int(raw[0, 0]) == ((int(q[0, 0]) & 0xf) | ((int(q[0, 1]) & 0xf) << 4))
  with pytest.raises(ValueError, match='even'):
    cu._pack_int4(torch.zeros((2, 3), dtype=torch.int8))


class _Two(torch.nn.Module):
  def __init__(self):
    super().__init__()
    g = torch.Generator().manual_seed(1)
    self.Dense_0 = nn.Dense(256, 128, use_bias=False, dtype=torch.bfloat16, generator=g)
    self.Dense_1 = nn.Dense(128, 64, use_bias=False, dtype=torch.bfloat16, generator=g)

  def forward(self, x):
    return self.Dense_1(torch.relu(self.Dense_0(x)))


@pytest.mark.gpu
def test_load_prequantized_into_ptq_model(tmp_path):
  rules = [qwix.QuantizationRule(module_path='Dense_0', weight_qtype='int8', act_qtype='int8')]
  x = torch.randn(8, 256, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16).cuda()
  src = qwix.quantize_model(_Two().cuda(), qwix.PtqProvider(rules))
  want = src(x)                                    # Dense_0 is quantized in place, Dense_1 stays bf16
  f = str(tmp_path / 'model.safetensors')
  cu.save_prequantized(src.params(), f)
  ckpt = cu.load_prequantized(f, device='cuda')
  assert set(ckpt['Dense_0']['kernel']) == {'qvalue', 'scale', 'qtype'} and torch.is_tensor(ckpt['Dense_1']['kernel'])
  assert [r.module_path for r in cu.restore_quantization_rules(ckpt, tile_size=None)] == ['Dense_0']

  # case 1 (quantized -> quantized) and case 3 (float -> float): same outputs as the source model
  dst = qwix.quantize_model(_Two().cuda(), qwix.PtqProvider(rules))
  dst(x)                                           # creates the quantized template
  dst.model.Dense_1.kernel.data.zero_()
  tree = cu.process_prequantized_params(ckpt, dst)
  assert isinstance(tree['Dense_0']['kernel'], qwix.WithAux)
  qwix.model.set_params(dst.model, tree)
  assert torch.equal(dst(x), want)

  # case 2 (quantized checkpoint, floating-point template): the leaf is dequantized on the device
  fp = _Two().cuda()
  tree = cu.process_prequantized_params(ckpt, fp)
  k = tree['Dense_0']['kernel']
  assert torch.is_tensor(k) and k.dtype == torch.bfloat16
  assert torch.equal(k, qwix.dequantize(src.params()['Dense_0']['kernel'].array))

  # errors of the reference: extra params, float leaf for a quantized template, shape mismatch
  with pytest.raises(ValueError, match='extra parameters'):
    cu.process_prequantized_params({'Nope': {'kernel': torch.ones(2)}}, dst)
  assert cu.process_prequantized_params({'Nope': {'kernel': torch.ones(2)}}, dst, allow_extra_params=True) == {}
  with pytest.raises(ValueError, match='invalid parameter combination'):
    cu.process_prequantized_params({'Dense_0': {'kernel': torch.ones(256, 128)}}, dst)
  bad = {'Dense_0': {'kernel': {'qvalue': torch.zeros((4, 4), dtype=torch.int8), 'scale': torch.ones(1, 4)}}}
  with pytest.raises(ValueError, match='template expects'):
    cu.process_prequantized_params(bad, dst)
  with pytest.raises(ValueError, match='unexpected "zero_point"'):
    leaf = dict(ckpt['Dense_0']['kernel'], zero_point=torch.zeros(1, 128, dtype=torch.int8))
    cu.process_prequantized_params({'Dense_0': {'kernel': leaf}}, dst)
