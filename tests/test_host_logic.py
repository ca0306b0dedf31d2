"""CPU: shape algebra, rule matching, einsum parsing, path choice, ABI exports -- the host
logic around the kernels, checked against the reference's own shape-only tests."""

import json
import pathlib
import re

import pytest
import torch

import qwix_b200 as qwix
from qwix_b200 import _context
from qwix_b200 import _lib
from qwix_b200 import nn
from qwix_b200 import pallas as qpl
from qwix_b200.core import dot_general as bdg
from qwix_b200.core import einsum as bes
from qwix_b200.core import einsum_info
from qwix_b200.core import numerics
from qwix_b200.core import pallas as bpl
from qwix_b200.core import qarray as bq

ROOT = pathlib.Path(__file__).resolve().parents[1]
GOLD = json.loads((ROOT / 'tests' / 'golden' / 'reference_known_answers.json').read_text())


def _fake_qarray(shape, scale_shape, qdtype=torch.int8, sdtype=torch.float32, qtype=None):
  return bq.QArray(torch.ones(shape, dtype=qdtype), torch.ones(scale_shape, dtype=sdtype),
                   qtype=qtype)


def test_abi_exports_every_declared_symbol():
  header = (ROOT / 'include' / 'qwix_b200.h').read_text()
  declared = set(re.findall(r'\b(qwx_[a-z0-9_]+)\s*\(', header))
  assert declared, 'no declarations found in the header'
  handle = _lib.lib()
  for name in declared:
    assert hasattr(handle, name), f'{name} is declared but not exported'
  assert set(_lib.exported_symbols()) == declared
  assert handle.qwx_version() >= 100
  assert handle.qwx_status_string(0) == b'ok'
  assert b'aligned' in handle.qwx_status_string(3)


def test_no_cpu_fallback():
  x = torch.randn(4, 16)
  with pytest.raises(RuntimeError, match='no CPU fallback'):
    bq.quantize(x, bq.HowToQuantize(qtype='int8', channelwise_axes=(0,)))
  q = _fake_qarray((4, 16), (4, 1))
  with pytest.raises(RuntimeError, match='no CPU fallback'):
    bq.dequantize(q)


def test_scale_shape_rules():
  how = bq.HowToQuantize(qtype='int8', channelwise_axes=[0], tiled_axes={2: 2})
  assert bq.get_scale_shape((2, 2, 6), how) == (2, 1, 3)
  assert bq.get_scale_shape((8, 12), bq.HowToQuantize(qtype='int8', tiled_axes={1: 1 / 3})) == (1, 3)
  with pytest.raises(ValueError, match='both channelwise and tiled'):
    bq.get_scale_shape((4, 4), bq.HowToQuantize(qtype='int8', channelwise_axes=[0],
                                                tiled_axes={0: 2}))
  with pytest.raises(ValueError, match='cannot be tiled'):
    bq.get_scale_shape((4, 6), bq.HowToQuantize(qtype='int8', tiled_axes={1: 4}))
  c = GOLD['ptq_dense_tile']
  how = bdg.get_how_to_quantize(dimension_numbers=(((1,), (0,)), ((), ())), ndims=(2, 2),
                                for_lhs=False, tile_size=c['tile_size'], qtype='int8')
  assert list(bq.get_scale_shape(c['kernel_shape'], how)) == c['scale_shape']


def test_array_methods_match_reference_shapes():
  c = GOLD['array_methods']
  q = _fake_qarray(c['shape'], c['scale_shape'])
  assert list(q.scale_tile_shape) == c['scale_tile_shape']
  assert q.zero_point_tile_shape is None
  for new, scale in c['reshape']:
    r = q.reshape(*new)
    assert list(r.shape) == new and list(r.scale.shape) == scale
  chain = c['reshape_chain']
  assert list(q.reshape(chain['first']).reshape(chain['then']).scale.shape) == chain['scale_shape']
  for axes, shape, scale in c['transpose']:
    t = q.transpose(*axes)
    assert list(t.shape) == shape and list(t.scale.shape) == scale
  assert [list(q.T.shape), list(q.T.scale.shape)] == c['T']
  assert [list(q.mT.shape), list(q.mT.scale.shape)] == c['mT']
  s = q.swapaxes(1, 2)
  assert [list(s.shape), list(s.scale.shape)] == c['swapaxes_1_2']
  # qarray_test.py:270-284: slicing
  assert q[..., 1].shape == (2, 2) and tuple(q[..., 1].scale.shape) == (2, 1)
  assert tuple(q[0:1, 1:2, 4].scale.shape) == (1, 1)
  assert tuple(q[0].scale.shape) == (1, 3)
  assert tuple(q[..., None].scale.shape) == (2, 1, 3, 1)
  assert tuple(q[None].scale.shape) == (1, 2, 1, 3)
  assert q.astype(torch.bfloat16).scale.dtype == torch.bfloat16
  with pytest.raises(ValueError):
    q.reshape(4, 7)
  with pytest.raises(ValueError):
    bq.validate_qarray(_fake_qarray((10, 10), (10, 3)))


def test_get_tiled_axes():
  c = GOLD['get_tiled_axes']
  q = _fake_qarray(c['qvalue_shape'], c['scale_shape'])
  assert bq.get_tiled_axes(q) == {int(k): v for k, v in c['want'].items()}


def test_collapse_view():
  cv = bq.collapse_view
  assert cv((4096, 8192), (1, 8192)) == (1, 1, 4096 * 8192, 1, 1, 8192)          # per token
  assert cv((8192, 8192), (8192, 1)) == (1, 8192, 8192, 1, 8192, 1)              # per channel
  assert cv((8192, 28672), (128, 1)) == (1, 8192, 28672, 1, 128, 1)              # sub-channel
  assert cv((32, 2048, 4096), (1, 1, 4096)) == (1, 1, 32 * 2048 * 4096, 1, 1, 4096)
  assert cv((4096, 32, 128), (4096, 1, 1)) == (1, 4096, 4096, 1, 4096, 1)        # [d, n, h] weight
  assert cv((128, 256), (128, 256)) == (1, 1, 128 * 256, 1, 1, 128 * 256)        # per tensor
  assert cv((4, 48, 64), (1, 48, 1)) == (1, 4 * 48, 64, 1, 48, 1)
  assert cv((6, 40, 24), (1, 40, 1)) == (1, 240, 24, 1, 40, 1)
  assert cv((6, 40, 24), (6, 1, 24)) == (1, 6, 960, 1, 6, 24)
  assert cv((8, 6, 10), (8, 3, 1)) == (8, 6, 10, 8, 3, 1)                        # needs all three axes
  with pytest.raises(NotImplementedError):
    cv((4, 6, 8, 10), (2, 3, 2, 5))


def test_symmetric_bounds_and_storage():
  for case in GOLD['symmetric_bound']:
    assert numerics.get_symmetric_bound(case['qtype']) == case['want']
  assert numerics.get_asymmetric_bound('int4') == (-8.0, 7.0)
  with pytest.raises(ValueError, match="doesn't support asymmetric quantization"):
    numerics.get_asymmetric_bound('nf4')
  with pytest.raises(ValueError, match='Cannot use'):
    numerics.get_symmetric_bound(torch.bfloat16)
  with pytest.raises(NotImplementedError):
    numerics.storage('nf4')
  assert numerics.qtype_name(torch.float8_e4m3fn) == 'float8_e4m3fn'
  assert numerics.can_dequant_on_output('int8') and not numerics.can_dequant_on_output('nf4')


DN = (((1,), (0,)), ((), ()))


def test_how_to_quantize_for_dot_general_and_einsum():
  how = bdg.get_how_to_quantize(dimension_numbers=DN, ndims=(2, 2), for_lhs=True,
                                tile_size=None, qtype='int8')
  assert list(how.channelwise_axes) == [0] and dict(how.tiled_axes) == {}
  dn = (((2, 3), (0, 1)), ((), ()))
  assert bdg.get_how_to_quantize(dimension_numbers=dn, ndims=(4, 3), for_lhs=True,
                                 qtype='int8', tile_size=32).tiled_axes == {3: 32}
  assert bdg.get_how_to_quantize(dimension_numbers=dn, ndims=(4, 3), for_lhs=False,
                                 qtype='int8', tile_size=32).tiled_axes == {1: 32}
  how = bes.get_how_to_quantize(einsum_str='btd,dnh->btnh', ndims=(3, 3), for_lhs=False,
                                qtype='int8', tile_size=None)
  assert list(how.channelwise_axes) == [1, 2]
  how = bes.get_how_to_quantize(einsum_str='...d,df->...f', ndims=(3, 2), for_lhs=True,
                                qtype='int8', tile_size=128)
  assert list(how.channelwise_axes) == [0, 1] and dict(how.tiled_axes) == {2: 128}


def test_einsum_info():
  info = einsum_info.EinsumInfo.parse('abc,bcd->acd')
  assert info.batch_chars == ['c'] and info.contract_chars == ['b']
  assert info.dimension_numbers == (((1,), (0,)), ((2,), (1,)))
  assert info.output_perm == (1, 0, 2)
  assert einsum_info.EinsumInfo.parse('ab,bc->ac').output_perm is None
  assert einsum_info.normalize_subscripts('...d,df', (3, 2)).endswith('->' + 'f') is False
  assert einsum_info.normalize_subscripts('ab,bc', (2, 2)) == 'ab,bc->ac'
  with pytest.raises(NotImplementedError):
    einsum_info.EinsumInfo.parse('aab,bc->ac')
  with pytest.raises(NotImplementedError):
    einsum_info.EinsumInfo.parse('ab,bc')
  a = torch.ones(1, 4)
  q = _fake_qarray((2, 4), (2, 1))
  out = einsum_info.broadcast_operands([a, q], ['ab', 'ab'])
  assert tuple(out[0].shape) == (2, 4) and tuple(out[1].scale.shape) == (2, 1)


def test_path_choice_follows_reference():
  f32 = torch.ones(10, 10)
  w8 = _fake_qarray((10, 10), (1, 10))
  a8 = _fake_qarray((10, 10), (10, 1))
  assert bdg.use_fast_path(a8, w8, DN)
  assert not bdg.use_fast_path(f32, w8, DN)                       # weight-only -> slow path
  small_tile = _fake_qarray((256, 10), (4, 10))                  # tile 64 < 128 on K
  big_tile = _fake_qarray((256, 10), (2, 10))                    # tile 128
  a = _fake_qarray((10, 256), (10, 1))
  assert not bdg.use_fast_path(a, small_tile, DN)
  assert bdg.use_fast_path(a, big_tile, DN)
  nf4 = _fake_qarray((10, 10), (1, 10), qdtype=torch.uint8, qtype='nf4')
  assert not bdg.use_fast_path(a8, nf4, DN)
  raw_fp8 = torch.ones(10, 10).to(torch.float8_e4m3fn)
  assert bdg.use_fast_path(raw_fp8, w8, DN)


@pytest.mark.parametrize('lhs,rhs,want', [
    (torch.bfloat16, torch.float32, torch.float32),
    (torch.bfloat16, (torch.int8, torch.bfloat16), torch.bfloat16),
    (torch.bfloat16, (torch.int8, torch.float32), torch.float32),
    ((torch.int8, torch.bfloat16), (torch.int8, torch.float32), torch.float32),
    ((torch.float8_e4m3fn, torch.bfloat16), (torch.float8_e4m3fn, torch.float32), torch.float32),
])
def test_result_dtype_matrix(lhs, rhs, want):
  make = lambda s: _fake_qarray((10, 10), (1, 1), s[0], s[1]) if isinstance(s, tuple) \
      else torch.ones(10, 10, dtype=s)
  l, r = make(lhs), make(rhs)
  for pref in (None, torch.bfloat16, torch.float32):
    acc, res = bq.get_accumulator_and_result_type(l, r, preferred_element_type=pref)
    assert res == (pref or want)
    both_int = all(isinstance(s, tuple) and s[0] == torch.int8 for s in (lhs, rhs))
    assert acc == (torch.int32 if both_int else res)


def test_rule_defaults_and_matching():
  with pytest.raises(ValueError, match='act_static_scale'):
    qwix.PtqProvider([qwix.QuantizationRule(act_static_scale=True)])
  rules = [
      qwix.QuantizationRule(module_path='layers/0/.*', weight_qtype='int4', tile_size=128),
      qwix.QuantizationRule(module_path='.*', op_names=('einsum',), weight_qtype='float8_e4m3fn'),
      qwix.QuantizationRule(module_path='.*', weight_qtype='int8', act_qtype='int8'),
      qwix.QuantizationRule(module_path='never', weight_qtype='int8'),
  ]
  p = qwix.PtqProvider(rules)
  assert p._rules[2].act_static_scale is False and p._rules[2].act_calibration_method == 'absmax'
  mod_a, mod_b = torch.nn.Identity(), torch.nn.Identity()
  with _context.provider_scope(p):
    _context.push_module(mod_a, ('layers', '0', 'mlp'))
    r, op = p._get_current_rule_and_op_id('dot_general')
    assert r.weight_qtype == 'int4' and op == 'dot_general0'
    assert p._get_current_rule_and_op_id('dot_general')[1] == 'dot_general1'
    assert p._get_current_rule_and_op_id('dot_general', repeated_call=True)[1] == 'dot_general1'
    assert qwix.get_current_rule('einsum').weight_qtype == 'int4'
    _context.pop_module()
    _context.push_module(mod_b, ('layers', '1', 'mlp'))
    assert p._get_current_rule_and_op_id('einsum')[0].weight_qtype == 'float8_e4m3fn'
    r, op = p._get_current_rule_and_op_id('dot_general')
    assert r.act_qtype == 'int8' and op == 'dot_general0'
    _context.pop_module()
  assert qwix.get_current_rule('dot_general') is None
  with pytest.raises(ValueError, match='not completed'):
    p.get_unused_rules()
  p.process_model_output('__call__', None)
  assert [r.module_path for r in p.get_unused_rules()] == ['never']


def test_model_wrapper_tracks_module_paths_and_param_tree():
  class MLP(torch.nn.Module):
    def __init__(self):
      super().__init__()
      self.Dense_0 = nn.Dense(16, 64, use_bias=False)
      self.Dense_1 = nn.Dense(64, 16, use_bias=False)

    def forward(self, x):
      return self.Dense_1(torch.relu(self.Dense_0(x)))

  seen = []

  class Spy(qwix.QuantizationProvider):
    def get_intercept_map(self):
      def dg(lhs, rhs, dn, *a, **k):
        seen.append(('/'.join(_context.current_module_path()),
                     self._get_current_rule_and_op_id('dot_general')[1]))
        return bdg._plain_dot_general(lhs, rhs, dn)
      return {'dot_general': dg}

  model = MLP()
  x = torch.rand(8, 16)
  want = model(x)
  q = qwix.quantize_model(model, Spy([qwix.QuantizationRule()]))
  assert torch.equal(q(x), want)
  assert seen == [('Dense_0', 'dot_general0'), ('Dense_1', 'dot_general0')]
  q(x)
  assert seen[2:] == seen[:2]  # op ids restart with every model call
  tree = q.params()
  assert set(tree) == {'Dense_0', 'Dense_1'} and tuple(tree['Dense_0']['kernel'].shape) == (16, 64)


def test_quantize_params_errors():
  how = bq.HowToQuantize(qtype='int8', channelwise_axes=[1])
  template = {'Dense_0': {'kernel': qwix.WithAux(_fake_qarray((16, 64), (1, 64)), how)}}
  with pytest.raises(ValueError, match='not found'):
    qwix.quantize_params({'other': {'kernel': torch.ones(2, 2)}}, template)
  assert qwix.quantize_params({'other': {'kernel': torch.ones(2, 2)}}, template,
                              allow_extra_params=True) == {}
  with pytest.raises(TypeError):
    qwix.quantize_params({'Dense_0': {'kernel': 3}}, template)
  w = qwix.WithAux(_fake_qarray((16, 64), (1, 64)), how)
  assert w.reshape(16, 64) is w
  with pytest.raises(ValueError, match='target shape'):
    w.reshape(64, 16)


@pytest.mark.parametrize('case', GOLD['pallas_block_specs'], ids=lambda c: c['src'])
def test_pallas_scale_block_specs(case):
  spec = bpl.BlockSpec(tuple(case['block_shape']), lambda *a: tuple(a))
  arr = _fake_qarray(case['qvalue_shape'], case['scale_shape'], qtype='int8')
  new = bpl.update_block_specs_for_qarray(spec, arr)
  assert isinstance(new, bq.QArray) and new.qvalue is spec
  assert list(new.scale.block_shape) == case['scale_block_shape']
  assert list(new.scale.index_map(*case['index'])) == case['scale_index']
  assert qpl.dot_general is bdg.loop_dot_general and qpl.QArray is bq.QArray


def test_scales_along_k_layout():
  """How a scale (or zero point) with tiled contracting axes is laid out for the GEMM kernels:
  [batch, free, K tiles], with the tile length along the flattened K."""
  from qwix_b200.core import dot_general as dg
  from qwix_b200.core.qarray import QArray
  # one contracting axis, 128-wide tiles
  x = QArray(qvalue=torch.zeros(6, 512, dtype=torch.int8),
             scale=torch.arange(6 * 4, dtype=torch.float32).reshape(6, 4), zero_point=None, qtype='int8')
  t, k_tile = dg._along_k(x.scale, x, [1], [], [0])
  assert t.shape == (1, 6, 4) and k_tile == 128
  assert torch.equal(t[0], x.scale)
  # untiled: one run of K
  y = QArray(qvalue=torch.zeros(6, 512, dtype=torch.int8), scale=torch.ones(6, 1), zero_point=None, qtype='int8')
  t, k_tile = dg._along_k(y.scale, y, [1], [], [0])
  assert t.shape == (1, 6, 1) and k_tile == 512
  # two contracting axes (4, 256), the last tiled by 128: runs are numbered (first axis, tile)
  z = QArray(qvalue=torch.zeros(6, 4, 256, dtype=torch.int8),
             scale=torch.arange(6 * 2, dtype=torch.float32).reshape(6, 1, 2), zero_point=None, qtype='int8')
  t, k_tile = dg._along_k(z.scale, z, [1, 2], [], [0])
  assert t.shape == (1, 6, 8) and k_tile == 128
  assert torch.equal(t[0, 1], torch.tensor([2., 3.] * 4))
  # the same axes contracted in the other order: the tiled axis is outermost, runs are longer
  t, k_tile = dg._along_k(z.scale, z, [2, 1], [], [0])
  assert t.shape == (1, 6, 2) and k_tile == 128 * 4
  # a weight [K, N] with sub-channel tiles: free axis second, batch absent
  w = QArray(qvalue=torch.zeros(512, 5, dtype=torch.int8),
             scale=torch.arange(4 * 5, dtype=torch.float32).reshape(4, 5), zero_point=None, qtype='int8')
  t, k_tile = dg._along_k(w.scale, w, [0], [], [1])
  assert t.shape == (1, 5, 4) and k_tile == 128
  assert torch.equal(t[0], w.scale.t())
  # refining per-tile values to a finer common tiling
  assert torch.equal(dg._refine(torch.tensor([[[1., 2.]]]), 256, 128), torch.tensor([[[1., 1., 2., 2.]]]))


def test_lazy_activation_protocol_is_host_only_until_consumed():
  """fused.LazyAct: shape / ndim / which quantization recipes the producing kernel can emit."""
  from qwix_b200 import fused
  from qwix_b200.core import qarray as q

  class Fake(fused.LazyAct):
    def __init__(self):
      self.shape, self.device = (2, 3, 64), torch.device('cpu')
  f = Fake()
  assert f.ndim == 3 and f.dtype == torch.bfloat16
  assert f._fusable(q.HowToQuantize(qtype='int8', channelwise_axes=[0, 1]))
  assert not f._fusable(q.HowToQuantize(qtype='int8', channelwise_axes=[0]))            # per-row of axis 0 only
  assert not f._fusable(q.HowToQuantize(qtype='int4', channelwise_axes=[0, 1]))
  assert not f._fusable(q.HowToQuantize(qtype='int8', channelwise_axes=[0, 1], tiled_axes={2: 32}))
  assert not f._fusable(q.HowToQuantize(qtype='int8', channelwise_axes=[0, 1], calibration_method='minmax'))
  with pytest.raises(RuntimeError):      # CPU tensors never reach a kernel
    fused.AddRmsNorm(torch.zeros(2, 8, dtype=torch.bfloat16), None, torch.ones(8, dtype=torch.bfloat16), 1e-5)


def test_microscaled_dispatcher_declines_what_has_no_kernel():
  """mxfp_dot.py:51-57: the dispatcher returns None (the caller dequantizes) for operands it
  cannot take.  Here: one side not microscaled, mixed formats, a contracted length that is not
  whole 128-byte stages; decided on the host, before any device call."""
  from qwix_b200.core import mxfp_dot as bmx
  DN = (((1,), (0,)), ((), ()))

  def qa(rows, K, qtype, block, k_major=False):
    dt = torch.float8_e4m3fn if qtype == 'mxfp8' else torch.uint8
    if k_major:
      return bq.QArray(torch.zeros((K, rows), dtype=dt), torch.ones((K // block, rows)), None, qtype)
    return bq.QArray(torch.zeros((rows, K), dtype=dt), torch.ones((rows, K // block)), None, qtype)

  assert bmx.mxfp_dot_general(qa(8, 256, 'mxfp4', 32), torch.zeros(256, 16), DN) is None
  assert bmx.mxfp_dot_general(qa(8, 256, 'mxfp4', 32), qa(16, 256, 'nvfp4', 16, True), DN) is None
  assert bmx.mxfp_dot_general(qa(8, 256, 'mxfp8', 32), qa(16, 256, 'mxfp4', 32, True), DN) is None
  assert bmx.mxfp_dot_general(qa(8, 128, 'mxfp4', 32), qa(16, 128, 'mxfp4', 32, True), DN) is None   # K % 256
  assert bmx.mxfp_dot_general(qa(8, 128, 'nvfp4', 16), qa(16, 128, 'nvfp4', 16, True), DN) is None
  assert bmx.mxfp_dot_general(qa(8, 64, 'mxfp8', 32), qa(16, 64, 'mxfp8', 32, True), DN) is None      # K % 128
  # operands it is built for go on to the device library, which refuses host tensors loudly
  with pytest.raises(RuntimeError, match='CUDA device only'):
    bmx.mxfp_dot_general(qa(8, 256, 'mxfp4', 32), qa(16, 256, 'mxfp4', 32, True), DN)


def test_four_bit_qtypes_are_built():
  assert numerics.storage('mxfp4') == (torch.uint8, _lib.MXFP4)
  assert numerics.storage('nvfp4') == (torch.uint8, _lib.NVFP4)
  assert numerics.get_symmetric_bound('mxfp4') == numerics.get_symmetric_bound('nvfp4') == 6.0
  with pytest.raises(NotImplementedError):
    numerics.storage('mxfp8_16')
  with pytest.raises(ValueError, match='requires a tile size of 16'):
    bq.HowToQuantize(qtype='nvfp4', channelwise_axes=[0], tiled_axes={1: 32})
  with pytest.raises(ValueError, match='requires a tile size of 32'):
    bq.HowToQuantize(qtype='mxfp4', channelwise_axes=[0], tiled_axes={1: 16})
