"""CPU: the oracle replays every known-answer vector of the reference's own tests that is
reproducible without JAX (tests/golden/reference_known_answers.json), plus the
invariants those tests state for seeded inputs."""

import json
import pathlib

import ml_dtypes
import numpy as np
import pytest

from oracle import dot_general as odg
from oracle import einsum as oes
from oracle import hadamard as ohd
from oracle import numerics as onu
from oracle import qarray as oq

GOLD = json.loads((pathlib.Path(__file__).parent / 'golden' /
                   'reference_known_answers.json').read_text())


def _floats(xs):
  return np.array([float(x) for x in xs], dtype=np.float32)


@pytest.mark.parametrize('case', GOLD['convert_to'], ids=lambda c: f"{c['qtype']}@{c['src']}")
def test_convert_to(case):
  got = onu.convert_to(_floats(case['x']), case['qtype'])
  assert got.astype(np.float32).tolist() == [float(v) for v in case['want']]


@pytest.mark.parametrize('case', GOLD['symmetric_bound'], ids=lambda c: c['qtype'])
def test_symmetric_bound(case):
  assert onu.get_symmetric_bound(case['qtype']) == case['want']


def test_asymmetric_bound_rejects_nf4():
  with pytest.raises(ValueError, match="doesn't support asymmetric quantization"):
    onu.get_asymmetric_bound('nf4')


def test_nf4_convert_from():
  c = GOLD['nf4_convert_from']
  got = onu.convert_from(np.array(c['codes'], dtype=np.uint8), 'nf4')
  assert got.tolist() == c['want']


def test_exact_minmax_round_trip():
  c = GOLD['exact_minmax_round_trip']
  a = (np.arange(c['count']) / (c['count'] - 1.0)).astype(np.float32)
  q = oq.quantize(a, oq.HowToQuantize(qtype='int8', calibration_method='minmax'))
  assert q.zero_point.tolist() == [c['zero_point']]
  assert np.array_equal(q.qvalue, np.arange(c['first_code'], c['last_code'] + 1, dtype=np.int8))
  assert np.allclose(oq.dequantize(q), a)


def test_get_tiled_axes():
  c = GOLD['get_tiled_axes']
  arr = oq.QArray(np.ones(c['qvalue_shape'], np.int8), np.ones(c['scale_shape'], np.float32))
  assert oq.get_tiled_axes(arr) == {int(k): v for k, v in c['want'].items()}


@pytest.mark.parametrize('case', GOLD['mxfp_scales'], ids=lambda c: c['qtype'])
def test_outlier_aware_scales(case):
  scale, _ = oq.compute_scale_zero_point({'absmax': _floats(case['absmax'])}, case['qtype'])
  assert scale.tolist() == case['want']


def test_hadamard_orthogonality():
  for power in GOLD['hadamard_orthogonality']['powers']:
    h = ohd.sylvester(power)
    d = 2 ** power
    assert np.array_equal(h @ h.T, d * np.eye(d, dtype=np.float32))


def test_hadamard_rotation_leaves_product_unchanged():
  # tests/contrib/hadamard_rot_test.py:91-111: (x H)(H w / d) == x w.
  rng = np.random.default_rng(0)
  x = rng.standard_normal((8, 256)).astype(np.float32)
  w = rng.standard_normal((256, 16)).astype(np.float32)
  got = ohd.rotate_lhs(x, 128) @ ohd.rotate_rhs(w, 128)
  assert np.allclose(got, x @ w, atol=1e-3)


def test_hadamard_identity_round_trip():
  # tests/contrib/kernels/fused_hadamard_quantized_matmul_test.py:64-103 with seeded signs:
  # I . H' . H'^T / d . I ~= I after int8 quantization of both sides, atol 1e-2.
  size, block = 256, 128
  rng = np.random.default_rng(0)
  s_in = rng.choice([-1.0, 1.0], size)
  s_out = rng.choice([-1.0, 1.0], size)
  eye = np.eye(size, dtype=np.float32).astype(ml_dtypes.bfloat16)
  w = ohd.rotate_rhs(eye, block, signs_in=s_in, signs_out=s_out)
  x = ohd.rotate_lhs(eye, block, signs_in=s_in, signs_out=s_out)
  xq, sx = ohd.quantize_a_tile(x.astype(np.float32), axis=1)
  wq = oq.quantize(w.astype(np.float32), oq.HowToQuantize(qtype='int8', channelwise_axes=[1]))
  out = (xq.astype(np.float32) @ wq.qvalue.astype(np.float32)) * sx * wq.scale
  assert np.allclose(out, np.eye(size), rtol=1e-2, atol=1e-2)


DN = (((1,), (0,)), ((), ()))


@pytest.mark.parametrize('tile', [None, 128, 256])
def test_fast_slow_loop_agree(tile):
  # tests/_src/core/two_dim_scales_test.py:56-93 and dot_general_tpu_test.py:215-219.
  rng = np.random.default_rng(1)
  x = rng.standard_normal((16, 512)).astype(np.float32)
  w = rng.standard_normal((512, 24)).astype(np.float32)
  kw = dict(dimension_numbers=DN, ndims=(2, 2), tile_size=tile, qtype='int8')
  xq = oq.quantize(x, odg.get_how_to_quantize(for_lhs=True, **kw))
  wq = oq.quantize(w, odg.get_how_to_quantize(for_lhs=False, **kw))
  f = odg.fast_dot_general(xq, wq, DN)
  s = odg.slow_dot_general(xq, wq, DN)
  l = odg.loop_dot_general(xq, wq, DN)
  assert np.allclose(f, s, atol=1e-4 * np.abs(s).max())
  assert np.allclose(f, l, atol=1e-4 * np.abs(s).max())
  rel_mae = np.abs(f - x @ w).mean() / np.abs(x @ w).mean()
  assert rel_mae < 0.02  # einsum_test.py:40-127: w8a8 bound


def test_asymmetric_lhs_fast_equals_slow():
  rng = np.random.default_rng(2)
  x = rng.uniform(0, 1, (8, 256)).astype(np.float32)
  w = rng.standard_normal((256, 8)).astype(np.float32)
  xq = oq.quantize(x, oq.HowToQuantize(qtype='int8', channelwise_axes=[0],
                                       calibration_method='minmax'))
  wq = oq.quantize(w, oq.HowToQuantize(qtype='int8', channelwise_axes=[1]))
  f = odg.fast_dot_general(xq, wq, DN)
  s = odg.slow_dot_general(xq, wq, DN)
  assert np.allclose(f, s, atol=1e-4)
  with pytest.raises(ValueError, match='Only one operand can be asymmetric'):
    odg.fast_dot_general(xq, oq.quantize(w, oq.HowToQuantize(
        qtype='int8', channelwise_axes=[1], calibration_method='minmax')), DN)


@pytest.mark.parametrize('lhs,rhs,want', [
    ('bfloat16', 'float32', 'float32'),
    ('bfloat16', ('int8', 'bfloat16'), 'bfloat16'),
    ('bfloat16', ('int8', 'float32'), 'float32'),
    (('int4', 'bfloat16'), ('int8', 'float32'), 'float32'),
    (('float8_e4m3fn', 'bfloat16'), ('float8_e4m3fn', 'float32'), 'float32'),
])
def test_result_dtype_matrix(lhs, rhs, want):
  # tests/_src/core/dot_general_test.py:28-146 (the entries without mxfp / bool operands).
  def make(spec):
    if isinstance(spec, tuple):
      return oq.QArray(np.ones((10, 10), np.dtype(getattr(ml_dtypes, spec[0], spec[0]))),
                       np.ones((1, 1), np.dtype(getattr(ml_dtypes, spec[1], spec[1]))))
    return np.ones((10, 10), np.dtype(getattr(ml_dtypes, spec, spec)))
  l, r = make(lhs), make(rhs)
  for pref in (None, ml_dtypes.bfloat16, np.float32):
    expect = np.dtype(pref) if pref is not None else np.dtype(getattr(ml_dtypes, want, want))
    for fn in (odg.slow_dot_general, odg.fast_dot_general, odg.loop_dot_general, odg.dot_general):
      assert fn(l, r, DN, preferred_element_type=pref).dtype == expect
    assert oes.einsum('ab,bc->ac', l, r, preferred_element_type=pref).dtype == expect


def test_innermost_tiling_heuristic():
  # dot_general_test.py:175-197 and einsum_test.py:450-473.
  dn = (((2, 3), (0, 1)), ((), ()))
  assert odg.get_how_to_quantize(dimension_numbers=dn, ndims=(4, 3), for_lhs=True,
                                 qtype='int8', tile_size=32).tiled_axes == {3: 32}
  assert odg.get_how_to_quantize(dimension_numbers=dn, ndims=(4, 3), for_lhs=False,
                                 qtype='int8', tile_size=32).tiled_axes == {1: 32}
  how = oes.get_how_to_quantize(einsum_str='abcd,cde->abe', ndims=(4, 3), for_lhs=True,
                                qtype='int8', tile_size=32)
  assert how.tiled_axes == {3: 32} and list(how.channelwise_axes) == [0, 1]


def test_strict_and_fused_rounding_differ_only_for_16_bit_inputs():
  rng = np.random.default_rng(3)
  x32 = rng.standard_normal((32, 256)).astype(np.float32)
  how = oq.HowToQuantize(qtype='int8', channelwise_axes=[0])
  assert np.array_equal(oq.quantize(x32, how, oq.STRICT).qvalue,
                        oq.quantize(x32, how, oq.FUSED).qvalue)
  x16 = x32.astype(ml_dtypes.bfloat16)
  a, b = oq.quantize(x16, how, oq.STRICT), oq.quantize(x16, how, oq.FUSED)
  assert np.array_equal(a.scale.view(np.uint16), b.scale.view(np.uint16))
  assert np.abs(a.qvalue.astype(np.int32) - b.qvalue.astype(np.int32)).max() == 1
