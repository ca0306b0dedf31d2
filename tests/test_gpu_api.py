"""GPU parity of the front-ends that sit on dot_general: einsum, dot, the qwix.pallas entry
points (pallas_call with QArray operands and the in-kernel dot_general), static-range
activation scales and the `fixed` calibration, each against the CPU oracle."""

import functools

import ml_dtypes
import numpy as np
import pytest
import torch

import qwix_b200 as qwix
from oracle import dot_general as odg
from oracle import einsum as oes
from oracle import qarray as oq
from qwix_b200 import nn
from qwix_b200 import pallas as qpl
from qwix_b200.core import einsum as bes
from qwix_b200.core import qarray as bq
from tests import helpers as h

pytestmark = pytest.mark.gpu
bf16 = ml_dtypes.bfloat16


def _within(got, want):
  g, w = got.astype(np.float32), want.astype(np.float32)
  return np.all(np.abs(g - w) <= 1e-2 + 2e-2 * np.abs(w))   # max-abs 1e-2 or rel 2e-2


def _pair(einsum_str, lhs_shape, rhs_shape, seed, rhs_std=0.02):
  rng = np.random.default_rng(seed)
  lhs = rng.standard_normal(lhs_shape, dtype=np.float32).astype(bf16)
  rhs = (rhs_std * rng.standard_normal(rhs_shape, dtype=np.float32)).astype(bf16)
  nd = (len(lhs_shape), len(rhs_shape))
  hows = {}
  for mod, name in ((oes, 'oracle'), (bes, 'device')):
    hows[name] = [mod.get_how_to_quantize(einsum_str=einsum_str, ndims=nd, for_lhs=side,
                                          tile_size=None, qtype='int8') for side in (True, False)]
  return lhs, rhs, hows


EINSUMS = [
    ('btd,dnh->btnh', (2, 48, 256), (256, 4, 64)),       # a projection onto heads
    ('btnh,nhd->btd', (2, 48, 4, 64), (4, 64, 256)),     # two contracted axes
    ('...d,df->...f', (3, 5, 16, 256), (256, 384)),      # ellipsis
    ('bqd,bkd->bqk', (4, 160, 128), (4, 96, 128)),       # activation x activation, batched
    ('nk,mk->mn', (200, 256), (72, 256)),                # output transposed
]


@pytest.mark.parametrize('case', EINSUMS, ids=[c[0] for c in EINSUMS])
def test_einsum_matches_oracle(case):
  einsum_str, ls, rs = case
  lhs, rhs, hows = _pair(einsum_str, ls, rs, seed=len(einsum_str), rhs_std=1.0 if 'bkd' in einsum_str else 0.02)
  lo, ro = oq.quantize(lhs, hows['oracle'][0]), oq.quantize(rhs, hows['oracle'][1])
  want = oes.einsum(einsum_str, lo, ro)
  lq = bq.quantize(h.to_torch(lhs), hows['device'][0])
  rq = bq.quantize(h.to_torch(rhs), hows['device'][1])
  assert h.codes_equal(lq.qvalue, lo.qvalue) and h.codes_equal(rq.qvalue, ro.qvalue)
  got = qwix.einsum(einsum_str, lq, rq)
  assert tuple(got.shape) == want.shape and got.dtype == torch.bfloat16
  assert _within(h.to_numpy(got), want)
  # weight-only: the left operand stays floating point -> the dequantize-first path
  got_wo = qwix.einsum(einsum_str, h.to_torch(lhs), rq)
  assert _within(h.to_numpy(got_wo), oes.einsum(einsum_str, lhs, ro))


def test_dot_matches_oracle():
  rng = np.random.default_rng(3)
  a = rng.standard_normal((4, 8, 256), dtype=np.float32).astype(bf16)
  b = (0.02 * rng.standard_normal((256, 128), dtype=np.float32)).astype(bf16)
  ha = oq.HowToQuantize(qtype='int8', channelwise_axes=[0, 1])
  hb = oq.HowToQuantize(qtype='int8', channelwise_axes=[1])
  want = oes.dot(oq.quantize(a, ha), oq.quantize(b, hb))
  got = qwix.dot(bq.quantize(h.to_torch(a), bq.HowToQuantize(qtype='int8', channelwise_axes=[0, 1])),
                 bq.quantize(h.to_torch(b), bq.HowToQuantize(qtype='int8', channelwise_axes=[1])))
  assert tuple(got.shape) == (4, 8, 128)
  assert _within(h.to_numpy(got), want)


# ---- qwix.pallas (tests/_src/core/pallas_test.py:150-292) -------------------------------------

@pytest.mark.parametrize('shape,tiled,bs', [
    ((256, 256), {}, (128, 128)), ((256, 256), {0: 1}, (128, 128)), ((256, 256), {1: 1}, (128, 128)),
    ((256, 256), {0: 128}, (128, 128)), ((256, 256), {0: 128, 1: 128}, (128, 128)),
    ((256, 256), {0: 128, 1: 1}, (128, 128)), ((4, 256, 256), {1: 1, 2: 128}, (128, 128)),
    ((128, 2048), {0: 1, 1: 128}, (128, 1024)),
], ids=['tensorwise', 'channelwise0', 'channelwise1', 'blockwise0', 'blockwise2',
        'blockwise_and_channelwise', '3d', 'wide'])
def test_pallas_dequantize(shape, tiled, bs):
  """Each grid point sees a block of the codes and the matching block of the scale."""
  def kernel(q_ref, out_ref):
    out_ref[...] = qpl.dequantize(q_ref)

  x = torch.rand(shape, generator=torch.Generator().manual_seed(0)).cuda()
  qx = bq.quantize(x, bq.HowToQuantize(qtype='int8', tiled_axes=tiled))
  block = (1,) * (len(shape) - 2) + bs
  out = qpl.pallas_call(
      kernel, out_shape=(shape, qx.scale.dtype), grid=tuple(s // b for s, b in zip(shape, block)),
      in_specs=[qpl.BlockSpec(block, lambda *a: a)], out_specs=qpl.BlockSpec(block, lambda *a: a))(qx)
  assert torch.equal(out, qwix.dequantize(qx))
  want = oq.dequantize(oq.QArray(h.to_numpy(qx.qvalue), h.to_numpy(qx.scale), None, 'int8'))
  assert np.array_equal(h.to_numpy(out), want)


def test_pallas_batch_matmul():
  """The blocked batch matmul of pallas_test.py:222-292: sub-channel scales (tile 128 along
  K) on both operands, the in-kernel dot_general accumulated over the K grid axis."""
  def kernel(x_ref, y_ref, z_ref, acc_ref, *, nsteps):
    if qpl.program_id(3) == 0:
      acc_ref.zero_()
    acc_ref += qpl.dot_general(x_ref, y_ref, (((1,), (0,)), ((), ())),
                               preferred_element_type=torch.float32)
    if qpl.program_id(3) == nsteps - 1:
      z_ref[...] = acc_ref

  b, m, k, n, bm, bk, bn = 4, 256, 256, 256, 128, 128, 128
  g = torch.Generator().manual_seed(0)
  x = torch.rand((b, m, k), generator=g).cuda()
  y = torch.rand((b, k, n), generator=g).cuda()
  qx = bq.quantize(x, bq.HowToQuantize(qtype='int8', channelwise_axes=[0, 1], tiled_axes={2: 128}))
  qy = bq.quantize(y, bq.HowToQuantize(qtype='int8', channelwise_axes=[2], tiled_axes={1: 128}))
  out = qpl.pallas_call(
      functools.partial(kernel, nsteps=k // bk), out_shape=((b, m, n), torch.float32),
      grid=(b, m // bm, n // bn, k // bk),
      in_specs=[qpl.BlockSpec((None, bm, bk), lambda b, i, j, k: (b, i, k)),
                qpl.BlockSpec((None, bk, bn), lambda b, i, j, k: (b, k, j))],
      out_specs=qpl.BlockSpec((None, bm, bn), lambda b, i, j, k: (b, i, j)),
      scratch_shapes=[((bm, bn), torch.float32)])(qx, qy)
  dn = (((2,), (1,)), ((0,), (0,)))
  whole = qwix.dot_general(qx, qy, dn)
  assert torch.allclose(out, whole, rtol=1e-5, atol=1e-4)
  xo = oq.QArray(h.to_numpy(qx.qvalue), h.to_numpy(qx.scale), None, 'int8')
  yo = oq.QArray(h.to_numpy(qy.qvalue), h.to_numpy(qy.scale), None, 'int8')
  want = odg.dot_general(xo, yo, dn)
  assert np.allclose(out.cpu().numpy(), want, rtol=1e-5, atol=1e-4)
  assert np.allclose(out.cpu().numpy(), odg.loop_dot_general(xo, yo, dn), rtol=1e-5, atol=1e-4)


# ---- static-range activations and fixed calibration ---------------------------------------------

class _OneDense(torch.nn.Module):
  def __init__(self, dtype):
    super().__init__()
    self.Dense_0 = nn.Dense(256, 128, use_bias=False, dtype=dtype,
                            generator=torch.Generator().manual_seed(1))

  def forward(self, x):
    return self.Dense_0(x)


@pytest.mark.parametrize('method', ['absmax', 'minmax'])
def test_static_scale_activation(method):
  """boxed_param.py:416-455 with act_static_scale: the first call calibrates (mean over the
  batch axis), later calls reuse the stored scale whatever the input's range."""
  dtype = torch.float32
  model = _OneDense(dtype).cuda()
  w = h.to_numpy(model.Dense_0.kernel.data)
  rule = qwix.QuantizationRule(module_path='.*', weight_qtype='int8', act_qtype='int8',
                               act_static_scale=True, act_calibration_method=method)
  ptq = qwix.quantize_model(model, qwix.PtqProvider([rule]))
  g = torch.Generator().manual_seed(2)
  x0 = (torch.rand(16, 256, generator=g) * 2 - 0.5).cuda()
  x1 = (torch.rand(16, 256, generator=g) * 6 - 3).cuda()    # wider than the calibrated range
  y0, y1 = ptq(x0), ptq(x1)

  dn = (((1,), (0,)), ((), ()))
  # per-token statistics of the first batch, averaged over the batch axis (act_batch_axes)
  how_a = oq.HowToQuantize(qtype='int8', channelwise_axes=[0], calibration_method=method)
  cal = {k: v.astype(np.float32).mean(axis=0, keepdims=True).astype(v.dtype)
         for k, v in oq.calibrate(h.to_numpy(x0), how_a).items()}
  scale, zp = oq.compute_scale_zero_point(cal, 'int8')
  wq = oq.quantize(w, oq.HowToQuantize(qtype='int8', channelwise_axes=[1]))
  for x, y in ((x0, y0), (x1, y1)):
    xq = oq.quantize_with_scale_zero_point(h.to_numpy(x), 'int8', scale, zp)
    want = odg.dot_general(xq, wq, dn)
    assert np.allclose(h.to_numpy(y), want, rtol=1e-5, atol=1e-5)
  box = ptq.params()['Dense_0']['dot_general0_lhs_scale']
  assert isinstance(box, qwix.WithAux) and box.how.qtype == 'int8'
  assert np.array_equal(h.to_numpy(box.array), scale)


def test_static_scale_from_quant_stats():
  """ptq.py:106-129: quantize_params turns averaged statistics into the static scale."""
  dtype = torch.float32
  rule = qwix.QuantizationRule(module_path='.*', weight_qtype='int8', act_qtype='int8',
                               act_static_scale=True)
  model = _OneDense(dtype).cuda()
  fp_params = qwix.model.get_params(model)
  ptq = qwix.quantize_model(model, qwix.PtqProvider([rule]))
  x = torch.rand(8, 256, generator=torch.Generator().manual_seed(3)).cuda()
  ptq(x)                                                         # creates the abstract tree
  stats = {'Dense_0': {'dot_general0_lhs': {
      'count': torch.tensor(4, dtype=torch.int32, device='cuda'),
      'sum_of_absmax': torch.full((1, 1), 10.0, device='cuda')}}}
  tree = qwix.quantize_params(fp_params, ptq.params(), stats)
  box = tree['Dense_0']['dot_general0_lhs_scale']
  assert isinstance(box, qwix.WithAux)
  assert torch.allclose(box.array.cpu(), torch.full((1, 1), 2.5 / 127.5))
  fresh = _OneDense(dtype).cuda()
  qwix.model.set_params(fresh, tree)
  y = qwix.quantize_model(fresh, qwix.PtqProvider([rule]))(x)
  wq = oq.quantize(h.to_numpy(fp_params['Dense_0']['kernel']),
                   oq.HowToQuantize(qtype='int8', channelwise_axes=[1]))
  xq = oq.quantize_with_scale_zero_point(h.to_numpy(x), 'int8',
                                         np.full((1, 1), 2.5, np.float32) / np.float32(127.5), None)
  want = odg.dot_general(xq, wq, (((1,), (0,)), ((), ())))
  assert np.allclose(h.to_numpy(y), want, rtol=1e-5, atol=1e-5)
  with pytest.raises(ValueError, match='not initialized'):
    stats['Dense_0']['dot_general0_lhs']['count'] = torch.tensor(0)
    qwix.quantize_params(fp_params, ptq.params(), stats)


@pytest.mark.parametrize('method,qtype', [('fixed,-3,3', 'int8'), ('fixed,0,6', 'int8'),
                                          ('fixed,2', 'int4')])
@pytest.mark.parametrize('dtype', ['float32', 'bfloat16'])
def test_fixed_calibration(method, qtype, dtype):
  """qarray.py:518-532: constants instead of statistics, always per tensor."""
  rng = np.random.default_rng(9)
  x = (2.0 * rng.standard_normal((64, 96), dtype=np.float32)).astype(h.np_dtype(dtype))
  want = oq.quantize(x, oq.HowToQuantize(qtype=qtype, channelwise_axes=[0], calibration_method=method))
  got = bq.quantize(h.to_torch(x), bq.HowToQuantize(qtype=qtype, channelwise_axes=[0],
                                                    calibration_method=method))
  assert tuple(got.scale.shape) == (1, 1)
  assert h.codes_equal(got.qvalue, want.qvalue)
  assert np.array_equal(h.to_numpy(got.scale).view(np.uint8), want.scale.view(np.uint8))
  assert (got.zero_point is None) == (want.zero_point is None)
  if want.zero_point is not None:
    assert h.codes_equal(got.zero_point, want.zero_point)
  assert np.array_equal(h.to_numpy(bq.dequantize(got)).view(np.uint8), oq.dequantize(want).view(np.uint8))
