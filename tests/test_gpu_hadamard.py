"""GPU parity: Hadamard rotation / rotate+quantize / Hadamard-quantized matmul vs the oracle."""

import ml_dtypes
import numpy as np
import pytest
import torch

from oracle import hadamard as ohd
from oracle import qarray as oq
from qwix_b200.contrib import hadamard as bhd
from tests import helpers as h

pytestmark = pytest.mark.gpu
bf16 = ml_dtypes.bfloat16


def _student_t(shape, seed, scale=0.5):
  rng = np.random.default_rng(seed)
  return (scale * rng.standard_t(3, shape)).astype(np.float32).astype(bf16)


def _close_bf16(got, want, ulps=1):
  g, w = got.astype(np.float32), want.astype(np.float32)
  return np.all(np.abs(g - w) <= ulps * 2.0 ** -7 * np.maximum(np.abs(w), 1e-30) + 1e-30)


@pytest.mark.parametrize('signed', [False, True])
def test_rotations_match_oracle(signed):
  rng = np.random.default_rng(0)
  x = _student_t((48, 512), 1)
  w = (0.02 * rng.standard_normal((512, 200))).astype(np.float32).astype(bf16)
  si = rng.choice([-1, 1], 512).astype(np.int8) if signed else None
  so = rng.choice([-1, 1], 512).astype(np.int8) if signed else None
  got_x = h.to_numpy(bhd.rotate_lhs(h.to_torch(x), si, so))
  got_w = h.to_numpy(bhd.hadamard_transform_rhs(h.to_torch(w), si, so))
  # float32 butterflies add in another order than the oracle's matmul: at most one bf16 ulp
  assert _close_bf16(got_x, ohd.rotate_lhs(x, 128, si, so))
  assert _close_bf16(got_w, ohd.rotate_rhs(w, 128, si, so))
  # (x H)(H w / d) == x w  (tests/contrib/hadamard_rot_test.py:91-111)
  prod = got_x.astype(np.float32) @ got_w.astype(np.float32)
  ref = x.astype(np.float32) @ w.astype(np.float32)
  assert np.abs(prod - ref).max() <= 2e-2 * np.abs(ref).max()


# Rows of 1..32 blocks (a power of two) take the thread-per-block kernel, partial last
# groups included; 3 and 40 blocks per row take the shuffle kernel.
@pytest.mark.parametrize('shape', [(96, 4096), (3, 1024), (1000, 128), (70, 2048), (33, 256),
                                   (50, 384), (20, 5120)],
                         ids=lambda s: f'{s[0]}x{s[1]}')
@pytest.mark.parametrize('qtype', ['float8_e4m3fn', 'int8'])
def test_rotate_quantize_matches_oracle(qtype, shape):
  x = _student_t(shape, 2)
  x[min(5, shape[0] - 1)] = 0          # an all-zero row: scale 1, codes 0
  x[0, :7] *= 1e-30                    # values far below the row maximum
  got = bhd.hadamard_quantize(h.to_torch(x), qtype)
  rot = h.to_numpy(bhd.rotate_lhs(h.to_torch(x)))
  # Given the device's rotated array, scales and codes follow the absmax recipe bit for bit.
  want = oq.quantize(rot, oq.HowToQuantize(qtype=qtype, channelwise_axes=[0]))
  assert np.array_equal(h.to_numpy(got.scale).view(np.uint8), want.scale.view(np.uint8))
  assert h.codes_equal(got.qvalue, want.qvalue)
  # And against the oracle's own rotation the dequantized arrays agree closely.
  full = oq.quantize(ohd.rotate_lhs(x, 128), oq.HowToQuantize(qtype=qtype, channelwise_axes=[0]))
  a = oq.dequantize(full).astype(np.float32)
  b = oq.dequantize(oq.QArray(h.to_numpy(got.qvalue), h.to_numpy(got.scale), None, qtype)).astype(np.float32)
  assert np.linalg.norm(a - b) <= 1e-2 * np.linalg.norm(a)


@pytest.mark.parametrize('mkn', [(256, 1024, 512), (300, 4096, 768)])
def test_hadamard_quantized_matmul(mkn):
  # The benchmarked Hadamard workload at reduced size: Student-t activations, N(0, 0.02) weights, fp8 e4m3,
  # absmax per row / per column, float32 accumulation, bf16 out; rel-L2 <= 1e-2.
  M, K, N = mkn
  a = _student_t((M, K), 5)
  w = (0.02 * np.random.default_rng(6).standard_normal((K, N))).astype(np.float32).astype(bf16)
  want, aq, wq = ohd.hadamard_quantized_matmul(a, w)
  wq_dev = bhd.quantize_rotated_weight(h.to_torch(w))
  got = h.to_numpy(bhd.hadamard_quantize_multiply(h.to_torch(a), wq_dev)).astype(np.float32)
  ref = want.astype(np.float32)
  assert np.linalg.norm(got - ref) <= 1e-2 * np.linalg.norm(ref)
  exact = a.astype(np.float32) @ w.astype(np.float32)
  assert np.linalg.norm(got - exact) <= 6e-2 * np.linalg.norm(exact)  # fp8 quantization noise


def test_identity_round_trip():
  # tests/contrib/kernels/fused_hadamard_quantized_matmul_test.py:64-103 with seeded signs and
  # int8 codes: I . H' . H'^T / d . I ~= I within 1e-2.
  size = 512
  rng = np.random.default_rng(0)
  si = rng.choice([-1, 1], size).astype(np.int8)
  so = rng.choice([-1, 1], size).astype(np.int8)
  eye = torch.eye(size, dtype=torch.bfloat16, device='cuda')
  wq = bhd.quantize_rotated_weight(eye, 'int8', si, so)
  out = bhd.hadamard_quantize_multiply(eye, wq, si, so)
  assert torch.allclose(out.float().cpu(), torch.eye(size), rtol=1e-2, atol=1e-2)
