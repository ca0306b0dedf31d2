"""GPU parity: CUDA quantize / dequantize (through the C ABI) vs the CPU oracle, bit-exact."""

import numpy as np
import pytest
import torch

from oracle import qarray as oq
from qwix_b200.core import qarray as bq
from tests import helpers as h

pytestmark = pytest.mark.gpu


def _data(shape, dtype, seed, dist='normal'):
  rng = np.random.default_rng(seed)
  x = rng.standard_normal(shape) if dist == 'normal' else rng.uniform(0, 1, shape)
  x = x.astype(np.float32)
  # outliers, exact zeros and one all-zero group to exercise the tiny-scale guard
  flat = x.reshape(-1)
  flat[:: 97] *= 20.0
  flat[5:: 131] = 0.0
  x.reshape(-1, shape[-1])[0, :] = 0.0
  return x.astype(h.np_dtype(dtype))


CASES = [
    # shape, channelwise, tiled, what it exercises
    ((64, 1024), (0,), {}, 'per-token rows (warp per row)'),
    ((16, 8192), (0,), {}, 'per-token rows (CTA per row)'),
    ((8, 16384), (0,), {}, 'rows longer than the register cache'),
    ((700, 14336), (0,), {}, 'rows of 14336: several rows per persistent CTA'),
    ((9, 8200), (0,), {}, 'rows just past 8192'),
    ((3, 16392), (0,), {}, 'rows just past 16384: general kernel'),
    ((256, 512), (1,), {}, 'per-output-channel columns'),
    ((512, 384), (1,), {0: 128}, 'sub-channel tiles along K'),
    ((32, 1024), (0,), {1: 128}, 'sub-channel tiles along the row'),
    ((128, 256), (), {}, 'per-tensor'),
    ((256, 256), (), {0: 64, 1: 32}, '2-D tiles'),
    ((4, 48, 64), (0, 2), {}, '3-D, reduce the middle axis'),
    ((6, 40, 24), (1,), {}, '3-D, channelwise middle axis'),
    ((37, 24), (0,), {}, 'odd row count'),
    ((33, 20), (1,), {}, 'columns not a multiple of 8'),
]


@pytest.mark.parametrize('dtype', ['float32', 'bfloat16'])
@pytest.mark.parametrize('qtype', ['int8', 'int4', 'float8_e4m3fn'])
@pytest.mark.parametrize('case', CASES, ids=[c[3] for c in CASES])
def test_quantize_absmax_matches_oracle(case, qtype, dtype):
  shape, cw, tiled, _ = case
  x = _data(shape, dtype, seed=hash((shape, qtype)) % 1000)
  want = oq.quantize(x, oq.HowToQuantize(qtype=qtype, channelwise_axes=cw, tiled_axes=tiled))
  got = bq.quantize(h.to_torch(x), bq.HowToQuantize(qtype=qtype, channelwise_axes=cw,
                                                    tiled_axes=tiled))
  assert tuple(got.scale.shape) == want.scale.shape
  assert np.array_equal(h.to_numpy(got.scale).view(np.uint8), want.scale.view(np.uint8))
  assert h.codes_equal(got.qvalue, want.qvalue)
  # dequantize round trip, bit-exact as well
  deq = bq.dequantize(got)
  assert np.array_equal(h.to_numpy(deq).view(np.uint8), oq.dequantize(want).view(np.uint8))


@pytest.mark.parametrize('dtype', ['float32', 'bfloat16'])
@pytest.mark.parametrize('method', ['minmax', 'minmax,0.9', 'absmax,0.8'])
@pytest.mark.parametrize('case', CASES[:3] + CASES[6:11], ids=[c[3] for c in CASES[:3] + CASES[6:11]])
def test_quantize_other_calibrations(case, method, dtype):
  shape, cw, tiled, _ = case
  x = _data(shape, dtype, seed=7)
  for qtype in ('int8', 'int4'):
    how = dict(qtype=qtype, channelwise_axes=cw, tiled_axes=tiled, calibration_method=method)
    want = oq.quantize(x, oq.HowToQuantize(**how))
    got = bq.quantize(h.to_torch(x), bq.HowToQuantize(**how))
    assert np.array_equal(h.to_numpy(got.scale).view(np.uint8), want.scale.view(np.uint8))
    if want.zero_point is not None:
      assert h.codes_equal(got.zero_point, want.zero_point)
    assert h.codes_equal(got.qvalue, want.qvalue)
    deq = bq.dequantize(got)
    assert np.array_equal(h.to_numpy(deq).view(np.uint8), oq.dequantize(want).view(np.uint8))


@pytest.mark.parametrize('dtype', ['float32', 'bfloat16'])
def test_rms_calibration_close(dtype):
  # The sum of squares is accumulated in another order than NumPy's: scales may differ by
  # one unit in the last place of the array dtype, codes by one step.
  x = _data((64, 1024), dtype, seed=3)
  how = dict(qtype='int8', channelwise_axes=(0,), calibration_method='rms,7')
  want = oq.quantize(x, oq.HowToQuantize(**how))
  got = bq.quantize(h.to_torch(x), bq.HowToQuantize(**how))
  ws = want.scale.astype(np.float32)
  gs = h.to_numpy(got.scale).astype(np.float32)
  tol = 2.0 ** -7 if dtype == 'bfloat16' else 1e-6
  assert np.all(np.abs(gs - ws) <= tol * np.abs(ws))
  same = gs == ws
  diff = np.abs(h.to_numpy(got.qvalue).astype(np.int32) - want.qvalue.astype(np.int32))
  assert diff[np.broadcast_to(same, diff.shape)].max() == 0
  assert diff.max() <= 2


def test_fused_rounding_mode_matches_oracle_fused():
  x = _data((64, 1024), 'bfloat16', seed=11)
  how = dict(qtype='int8', channelwise_axes=(0,))
  old = bq.ROUNDING
  try:
    bq.ROUNDING = 'fused'
    got = bq.quantize(h.to_torch(x), bq.HowToQuantize(**how))
  finally:
    bq.ROUNDING = old
  want = oq.quantize(x, oq.HowToQuantize(**how), mode=oq.FUSED)
  strict = oq.quantize(x, oq.HowToQuantize(**how), mode=oq.STRICT)
  assert h.codes_equal(got.qvalue, want.qvalue)
  assert not np.array_equal(want.qvalue, strict.qvalue)  # the two modes do differ


def test_reference_known_answers_on_device():
  # tests/_src/core/qarray_test.py:191-219 (without_error): 0..255/255 with minmax int8.
  a = (np.arange(256) / 255.0).astype(np.float32)
  got = bq.quantize(h.to_torch(a), bq.HowToQuantize(qtype='int8', calibration_method='minmax'))
  assert h.to_numpy(got.zero_point).tolist() == [-128]
  assert np.array_equal(h.to_numpy(got.qvalue), np.arange(-128, 128, dtype=np.int8))
  assert np.allclose(h.to_numpy(bq.dequantize(got)), a)
  # tests/_src/core/numerics_test.py:34-56 through quantize_with_scale (scale 1).
  one = torch.ones(1, device='cuda')
  v = torch.tensor([1.2, 3.5, -127.5, 129, -1300, float('inf'), float('-inf')], device='cuda')
  q = bq.quantize_with_scale_zero_point(v, 'int8', one, None)
  assert h.to_numpy(q.qvalue).tolist() == [1, 4, -128, 127, -128, 127, -128]
  v4 = torch.tensor([1.2, 3.5, 8, -1300], device='cuda')
  q4 = bq.quantize_with_scale_zero_point(v4, 'int4', one, None)
  assert h.to_numpy(q4.qvalue).tolist() == [1, 4, 7, -8]
  vf = torch.tensor([10.0, 500.0, -1000.0], device='cuda')
  qf = bq.quantize_with_scale_zero_point(vf, 'float8_e4m3fn', one, None)
  assert h.to_numpy(qf.qvalue).astype(np.float32).tolist() == [10.0, 448.0, -448.0]


def test_split_api_equals_fused_api():
  x = _data((96, 640), 'bfloat16', seed=5)
  xt = h.to_torch(x)
  how = bq.HowToQuantize(qtype='int8', channelwise_axes=(1,), tiled_axes={0: 32},
                         calibration_method='minmax')
  whole = bq.quantize(xt, how)
  cal = bq.calibrate(xt, how)
  scale, zp = bq.compute_scale_zero_point(cal, 'int8')
  parts = bq.quantize_with_scale_zero_point(xt, 'int8', scale, zp)
  assert torch.equal(whole.qvalue, parts.qvalue)
  assert torch.equal(whole.scale, parts.scale)
  assert torch.equal(whole.zero_point, parts.zero_point)
  want = oq.calibrate(x, oq.HowToQuantize(qtype='int8', channelwise_axes=(1,),
                                          tiled_axes={0: 32}, calibration_method='minmax'))
  assert np.array_equal(h.to_numpy(cal['min']).view(np.uint8), want['min'].view(np.uint8))
  assert np.array_equal(h.to_numpy(cal['max']).view(np.uint8), want['max'].view(np.uint8))
