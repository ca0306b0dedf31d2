"""Block-scaled dot_general for microscaled operands (qwix/_src/core/mxfp_dot.py:24-79).

When both operands are MXFP8 QArrays (e4m3 codes, one power-of-two scale per 32 contracted
elements) the contraction runs as one block-scaled tensor-core GEMM: `qwx_gemm_mx8` applies
the scales inside `tcgen05.mma.kind::mxf8f6f4.block_scale` and accumulates in float32, which
is what `jax.nn.scaled_matmul` computes for the reference.  Two MXFP4 QArrays (e2m1 codes) take
`qwx_gemm_mx4` (`kind::mxf4.block_scale`) after their codes are packed two per byte along the
contracted axis; two NVFP4 QArrays (the same codes, an e4m3-valued scale per 16 elements) take
`qwx_gemm_nvfp4` (`kind::mxf4nvf4.block_scale`).  Anything else returns None and the caller falls back to the ordinary paths,
as in the reference.
"""

import math
from typing import Sequence

import torch

from qwix_b200 import _lib
from qwix_b200.core import numerics
from qwix_b200.core import qarray
from qwix_b200.core.qarray import QArray

_MX_BLOCK = 32


def _is_mxfp(operand) -> bool:
  """mxfp_dot.py:82-89."""
  return isinstance(operand, QArray) and operand.qtype in ('mxfp8', 'mxfp8_16', 'mxfp4', 'nvfp4')


def _flatten_to_3d(operand: QArray, ca: Sequence[int], ba: Sequence[int], free_last: bool = False):
  """mxfp_dot.py:106-137 -- codes [B, F, K] and scales [B, F, K / block] (scale broadcast over
  the batch and free axes).  `free_last`: also give the [B, K, F] views."""
  ndim = operand.qvalue.ndim
  free = [i for i in range(ndim) if i not in ca and i not in ba]
  perm = list(ba) + free + list(ca)
  val = operand.qvalue.permute(perm)
  B = math.prod(operand.qvalue.shape[a] for a in ba)
  F = math.prod(operand.qvalue.shape[a] for a in free)
  K = math.prod(operand.qvalue.shape[a] for a in ca)
  scale = operand.scale
  full = [scale.shape[i] if i in ca else operand.qvalue.shape[i] for i in range(ndim)]
  scale = scale.expand(full).permute(perm)
  Ks = math.prod(operand.scale.shape[a] for a in ca)
  return val, scale, (B, F, K, Ks)


def _inputs_compatible(ldims, rdims) -> bool:
  """mxfp_dot.py:90-103."""
  return ldims[0] == rdims[0] and ldims[2] == rdims[2] and ldims[3] == rdims[3]


def mxfp_dot_general(lhs, rhs, dimension_numbers, preferred_element_type=None):
  """mxfp_dot.py:24-79.  Returns None when the operands are not both microscaled, their
  scale layouts do not match, or the pair has no kernel here (mxfp8_16, mixed formats)."""
  if not (_is_mxfp(lhs) and _is_mxfp(rhs)):
    return None
  if lhs.qtype != rhs.qtype or lhs.qtype not in ('mxfp8', 'mxfp4', 'nvfp4'):
    return None          # mxfp8 with 16-wide blocks, mixed formats: not built; the caller dequantizes
  four_bit = lhs.qtype in ('mxfp4', 'nvfp4')
  block = 16 if lhs.qtype == 'nvfp4' else _MX_BLOCK
  (lca, rca), (lba, rba) = dimension_numbers
  lca, rca, lba, rba = map(list, (lca, rca, lba, rba))
  lval, lscale, ldims = _flatten_to_3d(lhs, lca, lba)
  rval, rscale, rdims = _flatten_to_3d(rhs, rca, rba)
  if not _inputs_compatible(ldims, rdims):
    return None
  B, M, K, Ks = ldims
  N = rdims[1]
  if Ks * block != K or K % (256 if four_bit else 128):
    return None          # blocks of flattened K must be the format's blocks; whole 128-byte stages
  _, res_t = qarray.get_accumulator_and_result_type(
      lhs, rhs, preferred_element_type=preferred_element_type)
  if res_t not in _lib.FLOAT_CODES:
    return None
  _lib.require_cuda(lhs.qvalue, rhs.qvalue, lhs.scale, rhs.scale)

  a3 = lval.reshape(B, M, K).contiguous()
  sa3 = lscale.reshape(B, M, Ks).contiguous()
  # The weight where it lies: [.., K, N] needs no repack (MN-major operand of the MMA).
  rndim = rhs.qvalue.ndim
  rfree = [i for i in range(rndim) if i not in rca and i not in rba]
  kn = rhs.qvalue.permute(rba + rca + rfree)
  # More than 128 rows take the CTA-pair kernel, which wants both operands K-major: a [K, N]
  # weight is transposed once and kept beside the QArray (the 4-bit forms repack anyway).
  pair_form = M > 128 and K % 256 == 0 and not four_bit
  if pair_form and B == 1 and kn.is_contiguous() and not rval.is_contiguous():
    cached = getattr(rhs, '_mx_nk', None)
    if cached is None or cached[0] != rhs.qvalue.data_ptr():
      cached = (rhs.qvalue.data_ptr(), rval.reshape(N, K).contiguous())
      try:
        object.__setattr__(rhs, '_mx_nk', cached)
      except Exception:  # noqa: BLE001 -- a QArray that cannot carry the cache transposes per call
        pass
    b3, layout = cached[1].reshape(1, N, K), _lib.B_NK
    sb3 = None       # made below only if the packed scale bytes are not beside the QArray yet
    k_major = 0
  elif kn.is_contiguous() and not rval.is_contiguous() and N % 16 == 0:
    b3, layout = kn.reshape(B, K, N), _lib.B_KN
    full = [rhs.scale.shape[i] if i in rca else rhs.qvalue.shape[i] for i in range(rndim)]
    sb3 = rhs.scale.expand(full).permute(rba + rca + rfree).reshape(B, Ks, N).contiguous()
    k_major = 1
  else:
    b3, layout = rval.reshape(B, N, K).contiguous(), _lib.B_NK
    sb3 = rscale.reshape(B, N, Ks).contiguous()
    k_major = 0

  L = _lib.lib()
  dev = a3.device
  stream = _lib.stream_ptr(dev)
  out = torch.empty((B, M, N), dtype=res_t, device=dev)
  err = _lib.error_flag(dev)
  if four_bit:
    _fp4_batches(L, lhs.qtype, rhs, a3, sa3, b3, sb3, k_major, layout, B, M, N, K, out, res_t, err, stream)
    bshape = [lhs.qvalue.shape[i] for i in lba]
    lfree = [lhs.qvalue.shape[i] for i in range(lhs.qvalue.ndim) if i not in lca and i not in lba]
    return out.reshape(bshape + lfree + [rhs.qvalue.shape[i] for i in rfree])
  na = L.qwx_mx_scales_packed_bytes(0, M, K)
  nb = L.qwx_mx_scales_packed_bytes(1, N, K)
  for b in range(B):
    pa = torch.empty(na, dtype=torch.uint8, device=dev)
    _lib.check(L.qwx_mx_pack_scales(0, _lib.ptr(sa3[b]), numerics.code_of_float(sa3.dtype), M, K, 0,
                                    _lib.ptr(pa), na, stream), 'mx_pack_scales')
    cached = getattr(rhs, '_mx_packed', None) if B == 1 else None
    if cached is not None and cached[0] == (layout, N, K, rhs.scale.data_ptr()):
      pb = cached[1]
    else:
      if sb3 is None:
        sb3 = rscale.reshape(B, N, Ks).contiguous()
      pb = torch.empty(nb, dtype=torch.uint8, device=dev)
      _lib.check(L.qwx_mx_pack_scales(1, _lib.ptr(sb3[b]), numerics.code_of_float(sb3.dtype), N, K, k_major,
                                      _lib.ptr(pb), nb, stream), 'mx_pack_scales')
      if B == 1:
        try:
          object.__setattr__(rhs, '_mx_packed', ((layout, N, K, rhs.scale.data_ptr()), pb))
        except Exception:  # noqa: BLE001 -- a QArray that cannot carry the cache just repacks
          pass
    _lib.check(L.qwx_gemm_mx8(_lib.ptr(a3[b]), _lib.ptr(b3[b]), layout, M, N, K, _lib.ptr(pa), _lib.ptr(pb),
                              _lib.ptr(out[b]), _lib.FLOAT_CODES[res_t], _lib.ptr(err), stream), 'gemm_mx8')
  # mxfp_dot.py:140-163
  bshape = [lhs.qvalue.shape[i] for i in lba]
  lfree = [lhs.qvalue.shape[i] for i in range(lhs.qvalue.ndim) if i not in lca and i not in lba]
  rfree_shape = [rhs.qvalue.shape[i] for i in rfree]
  return out.reshape(bshape + lfree + rfree_shape)


def _fp4_batches(L, qtype, rhs, a3, sa3, b3, sb3, k_major, layout, B, M, N, K, out, res_t, err, stream):
  """The 4-bit leg: codes packed two per byte along K (the weight's packed codes and scale bytes
  are kept beside the QArray), then one block-scaled GEMM per batch element."""
  dev = a3.device
  if qtype == 'nvfp4':
    packed_bytes, pack_scales, gemm = L.qwx_nvfp4_scales_packed_bytes, L.qwx_nvfp4_pack_scales, L.qwx_gemm_nvfp4
  else:
    packed_bytes, pack_scales, gemm = L.qwx_mx4_scales_packed_bytes, L.qwx_mx4_pack_scales, L.qwx_gemm_mx4
  na = packed_bytes(0, M, K)
  nb = packed_bytes(1, N, K)
  for b in range(B):
    ap = torch.empty((M, K // 2), dtype=torch.uint8, device=dev)
    _lib.check(L.qwx_mx4_pack_codes(_lib.ptr(a3[b]), M, K, 0, _lib.ptr(ap), stream), 'mx4_pack_codes')
    pa = torch.empty(na, dtype=torch.uint8, device=dev)
    _lib.check(pack_scales(0, _lib.ptr(sa3[b]), numerics.code_of_float(sa3.dtype), M, K, 0,
                           _lib.ptr(pa), na, stream), 'pack_scales')
    key = (qtype, layout, N, K, rhs.qvalue.data_ptr(), rhs.scale.data_ptr())
    cached = getattr(rhs, '_mx4_packed', None) if B == 1 else None
    if cached is not None and cached[0] == key:
      bp, pb = cached[1], cached[2]
    else:
      bp = torch.empty((N, K // 2), dtype=torch.uint8, device=dev)
      _lib.check(L.qwx_mx4_pack_codes(_lib.ptr(b3[b]), N, K, k_major, _lib.ptr(bp), stream), 'mx4_pack_codes')
      pb = torch.empty(nb, dtype=torch.uint8, device=dev)
      _lib.check(pack_scales(1, _lib.ptr(sb3[b]), numerics.code_of_float(sb3.dtype), N, K, k_major,
                             _lib.ptr(pb), nb, stream), 'pack_scales')
      if B == 1:
        try:
          object.__setattr__(rhs, '_mx4_packed', (key, bp, pb))
        except Exception:  # noqa: BLE001 -- a QArray that cannot carry the cache just repacks
          pass
    _lib.check(gemm(_lib.ptr(ap), _lib.ptr(bp), M, N, K, _lib.ptr(pa), _lib.ptr(pb),
                    _lib.ptr(out[b]), _lib.FLOAT_CODES[res_t], _lib.ptr(err), stream), 'gemm_fp4')
