"""Oracle Hadamard rotation and the fused Hadamard-quantized matmul.

Test infrastructure only.  Restates qwix/contrib/hadamard_rot.py:35-117 and
qwix/contrib/kernels/fused_hadamard_quantized_matmul.py:50-56, 150-170, 443-478.
The reference draws its optional +/-1 sign flips from the TPU hardware PRNG,
which exists nowhere else; here the flips are explicit +/-1 vectors (or None).
"""

from __future__ import annotations

import numpy as np

from oracle import numerics
from oracle import qarray


def sylvester(power: int, dtype=np.float32) -> np.ndarray:
  """hadamard_rot.py:35-42 -- H_{2n} = [[H, H], [H, -H]], entries +/-1."""
  if power < 0:
    raise ValueError('Power must be non-negative.')
  h = np.ones((1, 1), dtype=np.float32)
  for _ in range(power):
    h = np.block([[h, h], [h, -h]])
  return h.astype(dtype)


def rotate_lhs(x: np.ndarray, block: int, signs_in=None, signs_out=None):
  """Per `block` columns: x_blk . (diag(signs_in) H diag(signs_out)), computed
  in float32 and rounded to x.dtype (hadamard_rot.py:99-106 for one block;
  fused_hadamard_quantized_matmul.py:150-160 per K block)."""
  m, k = x.shape
  assert k % block == 0
  h = sylvester(int(np.log2(block)))
  xb = x.astype(np.float32).reshape(m, k // block, block)
  if signs_in is not None:
    xb = xb * np.asarray(signs_in, np.float32).reshape(1, k // block, block)
  y = xb @ h
  if signs_out is not None:
    y = y * np.asarray(signs_out, np.float32).reshape(1, k // block, block)
  return y.reshape(m, k).astype(x.dtype)


def rotate_rhs(w: np.ndarray, block: int, signs_in=None, signs_out=None):
  """Per `block` rows: (diag(signs_out) H diag(signs_in)) . w_blk / block
  (hadamard_rot.py:109-117; fused_hadamard_quantized_matmul.py:443-478)."""
  k, n = w.shape
  assert k % block == 0
  h = sylvester(int(np.log2(block)))
  wb = w.astype(np.float32).reshape(k // block, block, n)
  if signs_in is not None:
    wb = wb * np.asarray(signs_in, np.float32).reshape(k // block, block, 1)
  y = np.einsum('ij,bjn->bin', h, wb)
  if signs_out is not None:
    y = y * np.asarray(signs_out, np.float32).reshape(k // block, block, 1)
  return (y / np.float32(block)).reshape(k, n).astype(w.dtype)


def quantize_a_tile(x: np.ndarray, axis: int, qtype='int8'):
  """fused_hadamard_quantized_matmul.py:50-56 -- s = max|x| / (qmax + 0.5),
  q = rint(x / s); the absmax recipe without the tiny-scale guard."""
  bound = numerics.get_symmetric_bound(qtype)
  s = np.max(np.abs(x), axis=axis, keepdims=True) / np.asarray(bound, x.dtype)
  return numerics.convert_to(x / s, qtype), s


def hadamard_quantized_matmul(a: np.ndarray, w: np.ndarray, *, block=128,
                              qtype='float8_e4m3fn', out_dtype=None,
                              mode=qarray.STRICT):
  """The benchmarked configuration: rotate both operands per K block (A.H and H.W/block),
  quantize A per row and W per column with absmax, contract the codes with
  float32 accumulation, scale, round to the output dtype.

  Returns (out, a_q, w_q) so tests can also compare the codes.
  """
  ar = rotate_lhs(a, block)
  wr = rotate_rhs(w, block)
  how_a = qarray.HowToQuantize(qtype=qtype, channelwise_axes=[0])
  how_w = qarray.HowToQuantize(qtype=qtype, channelwise_axes=[1])
  aq = qarray.quantize(ar, how_a, mode)
  wq = qarray.quantize(wr, how_w, mode)
  acc = aq.qvalue.astype(np.float32) @ wq.qvalue.astype(np.float32)
  out = acc * aq.scale.astype(np.float32) * wq.scale.astype(np.float32)
  return out.astype(out_dtype or a.dtype), aq, wq
