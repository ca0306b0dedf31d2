"""Hadamard rotation and the Hadamard-quantized matmul on CUDA tensors.

Same operations as qwix/contrib/hadamard_rot.py (rotate both operands of a contraction so that
the product is unchanged but outliers are spread) and
qwix/contrib/kernels/fused_hadamard_quantized_matmul.py (rotate + quantize the activation,
contract with a pre-rotated, pre-quantized weight).  Blocks are 128 wide (hadamard_power 7).
The reference draws its optional sign flips from the TPU hardware PRNG; here they are explicit
+/-1 int8 vectors over the contraction axis (or None).
"""

from __future__ import annotations

import torch

from qwix_b200 import _lib
from qwix_b200.core import numerics
from qwix_b200.core import qarray
from qwix_b200.core.qarray import QArray

BLOCK = 128


def _signs(v, k, device):
  if v is None:
    return None
  t = torch.as_tensor(v, device=device).to(torch.int8).contiguous()
  if t.numel() != k or not bool(((t == 1) | (t == -1)).all()):
    raise ValueError(f'sign vectors must hold {k} entries of +/-1.')
  return t


def _rotate(x: torch.Tensor, axis: int, signs_in, signs_out) -> torch.Tensor:
  if x.ndim != 2 or x.dtype != torch.bfloat16:
    raise ValueError('Hadamard rotation expects a 2-D bfloat16 array.')
  if x.shape[axis] % BLOCK:
    raise ValueError(f'the rotated axis ({x.shape[axis]}) must be a multiple of {BLOCK}.')
  _lib.require_cuda(x)
  x = x.contiguous()
  k = x.shape[axis]
  si, so = _signs(signs_in, k, x.device), _signs(signs_out, k, x.device)
  out = torch.empty_like(x)
  _lib.check(_lib.lib().qwx_hadamard_rotate(
      _lib.ptr(x), _lib.BF16, x.shape[0], x.shape[1], axis, BLOCK, _lib.ptr(si), _lib.ptr(so),
      _lib.ptr(out), _lib.stream_ptr(x.device)), 'hadamard_rotate')
  return out


def rotate_lhs(x: torch.Tensor, signs_in=None, signs_out=None) -> torch.Tensor:
  """x . H per 128 columns (hadamard_rot.py:99-106)."""
  return _rotate(x, 1, signs_in, signs_out)


def hadamard_transform_rhs(w: torch.Tensor, signs_in=None, signs_out=None) -> torch.Tensor:
  """H . w / 128 per 128 rows (hadamard_rot.py:109-117;
  fused_hadamard_quantized_matmul.py:443-478)."""
  return _rotate(w, 0, signs_in, signs_out)


def hadamard_quantize(x: torch.Tensor, qtype='float8_e4m3fn', signs_in=None,
                      signs_out=None) -> QArray:
  """Rotate per 128 columns and quantize per row in one pass
  (fused_hadamard_quantize.py:43-119 with whole-row tiles)."""
  if x.ndim != 2 or x.dtype != torch.bfloat16:
    raise ValueError('hadamard_quantize expects a 2-D bfloat16 array.')
  store, code = numerics.storage(qtype)
  if code not in (_lib.S8, _lib.E4M3):
    raise NotImplementedError(f'hadamard_quantize to {qtype} is not built.')
  _lib.require_cuda(x)
  x = x.contiguous()
  m, k = x.shape
  si, so = _signs(signs_in, k, x.device), _signs(signs_out, k, x.device)
  q = torch.empty((m, k), dtype=store, device=x.device)
  scale = torch.empty((m, 1), dtype=torch.bfloat16, device=x.device)
  _lib.check(_lib.lib().qwx_hadamard_quantize(
      _lib.ptr(x), _lib.BF16, m, k, BLOCK, _lib.ptr(si), _lib.ptr(so), code,
      qarray._rounding_code(), _lib.ptr(q), _lib.ptr(scale), _lib.stream_ptr(x.device)),
      'hadamard_quantize')
  return QArray(q, scale, None, numerics.qtype_name(qtype))


def quantize_rotated_weight(w: torch.Tensor, qtype='float8_e4m3fn', signs_in=None,
                            signs_out=None) -> QArray:
  """Offline half: rotate a [K, N] weight and quantize it per output channel."""
  rot = hadamard_transform_rhs(w, signs_in, signs_out)
  return qarray.quantize(rot, qarray.HowToQuantize(qtype=qtype, channelwise_axes=[1]))


def hadamard_quantize_multiply(x: torch.Tensor, wq: QArray, signs_in=None, signs_out=None,
                               out_dtype=torch.bfloat16) -> torch.Tensor:
  """fused_hadamard_quantized_matmul.py:349-414: rotate + quantize x per row, contract with
  the rotated, quantized weight, scales in the epilogue."""
  if x.ndim != 2 or x.dtype != torch.bfloat16:
    raise ValueError('hadamard_quantize_multiply expects a 2-D bfloat16 activation.')
  _, code = numerics.storage(wq.qtype)
  k, n = wq.shape
  if tuple(wq.scale.shape) != (1, n) or wq.zero_point is not None:
    raise NotImplementedError('the weight must be quantized per output channel, symmetric.')
  _lib.require_cuda(x, wq.qvalue)
  x = x.contiguous()
  m = x.shape[0]
  si, so = _signs(signs_in, k, x.device), _signs(signs_out, k, x.device)
  L = _lib.lib()
  ws = torch.empty(L.qwx_hadamard_gemm_workspace_bytes(m, k), dtype=torch.uint8, device=x.device)
  out = torch.empty((m, n), dtype=out_dtype, device=x.device)
  err = _lib.error_flag(x.device)
  oc = {torch.bfloat16: _lib.BF16, torch.float32: _lib.F32}[out_dtype]
  _lib.check(L.qwx_hadamard_gemm(
      _lib.ptr(x), m, k, _lib.ptr(si), _lib.ptr(so), _lib.ptr(wq.qvalue.contiguous()),
      _lib.ptr(wq.scale.to(torch.bfloat16).contiguous()), n, code, _lib.B_KN,
      qarray._rounding_code(), _lib.ptr(out), oc, _lib.EPI_F32, _lib.ptr(ws), ws.numel(),
      _lib.ptr(err), _lib.stream_ptr(x.device)), 'hadamard_quantize_multiply')
  return out
