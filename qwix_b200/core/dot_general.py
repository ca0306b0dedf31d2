"""Quantized dot_general on CUDA tensors: drop-in for the `_dot_general_fn` hook.

Same signature, path choice and error behaviour as qwix/_src/core/dot_general.py.  The
fast path (codes x codes, dequantize on output) is one tcgen05 GEMM with the scales fused
into its epilogue (csrc/gemm_q8.cu); the slow path dequantizes with the CUDA kernel and
hands the floating-point contraction to a plain library GEMM, as the reference hands it
to XLA.
"""

from __future__ import annotations

import contextlib
import math
import threading
from typing import Any, Mapping, Sequence

import torch

from qwix_b200 import _lib
from qwix_b200.core import numerics
from qwix_b200.core import qarray
from qwix_b200.core.qarray import QArray

# Tiles smaller than this on a contracting axis force the dequantize-first path
# (dot_general.py:402-404).
MIN_TILE_SIZE_TO_DEQUANT_ON_OUTPUT = 128
# Rows up to which an [N, K] int8 weight takes the warp-level kernel: measured against the
# split-K tcgen05 kernel it wins up to 8 rows (9-17 us against 15-23 us on 16-58 MB weights,
# 6.0 against 5.0 TB/s on 525 MB) and loses from 32 rows on, where its MMAs crowd the loads.
SKINNY_MAX_ROWS = 8
# Rows up to which an [N, K] int8 weight takes the swapped-operand tensor-core kernel
# (qwx_gemm_q8_decode: tokens are the MMA's N).  0 = never: measured against the split-K kernel
# on the decoder's shapes at 32 tokens it is level on 16-25 MB weights (14.7 against 13.6 us,
# 16.5 against 15.4 us) and behind on the large ones (31 against 25.5 us at 117 MB), because
# what bounds a launch of this size is not the MMA shape but launch gap, first-byte latency
# and the reduction of shared tiles (the breakdown is in gemm_q8_decode.cu); a whole decode
# step of the 32-layer model takes 5.2 ms with it and 4.7 ms without.
DECODE_MAX_ROWS = 0

# 'f32': float(acc) * sa * sb in float32, rounded once (default).  'reference': every step
# rounds to the result dtype in the reference's order (dot_general.py:255-261).
EPILOGUE = 'f32'

# Weight-only int4 contractions stream the packed weight through one fused kernel instead of
# materialising the dequantized weight (same W~ = bf16(q * s) operand, float32 accumulation).
FUSE_WEIGHT_ONLY = True


def get_how_to_quantize(*, dimension_numbers, ndims: tuple[int, int], for_lhs: bool,
                        tile_size: Mapping[int, int | float] | int | float | None,
                        **kwargs: Any) -> qarray.HowToQuantize:
  """dot_general.py:28-76 -- channelwise on every non-contracting axis; sub-channel tiles
  on the last contracting axis when a tile size is given."""
  side = 0 if for_lhs else 1
  ndim = ndims[side]
  contracting = dimension_numbers[0][side]
  if isinstance(tile_size, Mapping):
    tiled = tile_size
  else:
    tiled = {contracting[-1]: tile_size} if tile_size else {}
  channelwise = sorted(set(range(ndim)) - set(contracting) - set(tiled.keys()))
  return qarray.HowToQuantize(channelwise_axes=channelwise, tiled_axes=tiled, **kwargs)


def _free_axes(ndim, contracting, batch):
  return [a for a in range(ndim) if a not in contracting and a not in batch]


def _is_low_precision(t: torch.Tensor) -> bool:
  return not numerics.should_quantize(t.dtype)


def use_fast_path(lhs, rhs, dimension_numbers) -> bool:
  """The path choice of dot_general.py:442-472."""
  for operand, ca in zip((lhs, rhs), dimension_numbers[0]):
    if not isinstance(operand, QArray):
      if numerics.should_quantize(operand.dtype):
        return False
      continue
    qarray.validate_qarray(operand)
    if not numerics.can_dequant_on_output(operand.qtype):
      return False
    for axis in ca:
      if operand.scale.shape[axis] > 1:
        tile = operand.qvalue.shape[axis] // operand.scale.shape[axis]
        if tile < MIN_TILE_SIZE_TO_DEQUANT_ON_OUTPUT:
          return False
  return True


def _out_code(dtype: torch.dtype) -> int:
  table = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16, torch.float16: _lib.F16,
           torch.int32: _lib.S32}
  if dtype not in table:
    raise ValueError(f'unsupported result dtype {dtype} for the quantized GEMM')
  return table[dtype]


def _along_k(aux: torch.Tensor, x: QArray, contracting, batch, free):
  """Lays a scale (or zero point) of `x` out as [B, F, T]: batch axes, free axes (expanded to
  the operand's extents) and the contracting axes flattened into T tiles of the flattened K.

  K is the contracting axes flattened in the given order.  With j the last contracting axis
  along which the scale varies, one run of K that shares a scale is the tile of axis j times
  the extents of the later axes, and the runs are numbered by (earlier axes, tile of j).
  Returns (tensor [B, F, T], k_tile) with k_tile == K when T == 1.
  """
  dims = [x.qvalue.shape[a] for a in contracting]
  sdims = [aux.shape[a] for a in contracting]
  K = math.prod(dims)
  full = [x.qvalue.shape[a] for a in list(batch) + list(free)]
  t = aux.permute(list(batch) + list(free) + list(contracting))
  t = t.expand(full + sdims)
  varying = [i for i, n in enumerate(sdims) if n > 1]
  if not varying:
    return t.reshape(math.prod(full[:len(batch)]), math.prod(full[len(batch):]), 1), K
  j = varying[-1]
  for i in range(j):          # earlier axes: one run per index
    if sdims[i] != dims[i]:
      t = t.repeat_interleave(dims[i] // sdims[i], dim=len(full) + i)
  t = t.reshape(full + [-1])  # later axes have extent 1
  k_tile = (dims[j] // sdims[j]) * math.prod(dims[j + 1:])
  return t.reshape(math.prod(full[:len(batch)]), math.prod(full[len(batch):]), K // k_tile), k_tile


def _operand(x, contracting, batch, free):
  """Returns (codes, qtype name, scale [B, F, T] | None, zero point [B, F, T] | None, k_tile)."""
  if isinstance(x, QArray):
    scale, k_tile = _along_k(x.scale, x, contracting, batch, free)
    zp = None
    if x.zero_point is not None:
      zp, zk = _along_k(x.zero_point, x, contracting, batch, free)
      if zk != k_tile:   # zero point and scale share one shape in a valid QArray
        raise ValueError('zero_point and scale must have the same shape.')
    return x.qvalue, x.qtype, scale, zp, k_tile
  K = math.prod(x.shape[a] for a in contracting)
  return x, numerics.qtype_name(x.dtype), None, None, K


def _refine(t: torch.Tensor | None, k_from: int, k_to: int) -> torch.Tensor | None:
  """Repeats per-tile values [B, F, T] for a finer tiling of K."""
  if t is None or k_from == k_to or t.shape[-1] == 1:
    return t
  return t.repeat_interleave(k_from // k_to, dim=-1)


_INT_CODES = ('int8', 'int4')


_placement = threading.local()


@contextlib.contextmanager
def output_into(buffer: torch.Tensor):
  """While active, the next tensor-core contraction of this thread whose result has the
  dtype and element count of `buffer` (contiguous) is written straight into it instead of
  into a fresh allocation -- for callers whose consumer reads a fixed buffer (a partial sum
  that peers read over NVLink).  The caller checks `result.data_ptr()` to see whether the
  offer was taken."""
  _placement.buffer = buffer
  try:
    yield
  finally:
    _placement.buffer = None


def _result_buffer(shape, dtype, device) -> torch.Tensor:
  buf = getattr(_placement, 'buffer', None)
  if (buf is not None and buf.dtype == dtype and buf.device == device and buf.is_contiguous()
      and buf.numel() == math.prod(shape)):
    _placement.buffer = None
    return buf.view(shape)
  return torch.empty(shape, dtype=dtype, device=device)


def _fast_dot_general(lhs, rhs, dimension_numbers, preferred_element_type=None,
                      **kwargs) -> torch.Tensor:
  """dot_general.py:135-261 on the tensor cores."""
  del kwargs
  (lca, rca), (lba, rba) = dimension_numbers
  lca, rca, lba, rba = map(list, (lca, rca, lba, rba))
  if isinstance(lhs, QArray) and isinstance(rhs, QArray) and \
      lhs.zero_point is not None and rhs.zero_point is not None:
    raise ValueError('Only one operand can be asymmetric.')
  if isinstance(lhs, QArray) and isinstance(rhs, QArray):
    lt, rt = qarray.get_tiled_axes(lhs), qarray.get_tiled_axes(rhs)
    for l, r in zip(lca, rca):
      if lt.get(l) and rt.get(r) and lt[l] != rt[r]:
        raise ValueError('Contracting axes must be tiled with the same tile size.'
                         f' lhs_tiled_axes={lt} rhs_tiled_axes={rt} {dimension_numbers=}')
  lfa = _free_axes(lhs.ndim, lca, lba)
  rfa = _free_axes(rhs.ndim, rca, rba)
  acc_t, res_t = qarray.get_accumulator_and_result_type(
      lhs, rhs, preferred_element_type=preferred_element_type)

  lq, lname, ls, lz, lk = _operand(lhs, lca, lba, lfa)
  rq, rname, rs, rz, rk = _operand(rhs, rca, rba, rfa)
  if lname in _INT_CODES and rname in _INT_CODES and lq.dtype == rq.dtype == torch.int8:
    code = _lib.S8     # int4 codes are small int8 values to the tensor cores
  elif lname == rname == 'float8_e4m3fn':
    code = _lib.E4M3
  else:
    raise NotImplementedError(
        f'tensor-core path needs int8/int4 x int8/int4 or e4m3 x e4m3 codes, got {lname} x {rname}.')
  _lib.require_cuda(lq, rq)

  bshape = [lq.shape[a] for a in lba]
  mshape = [lq.shape[a] for a in lfa]
  nshape = [rq.shape[a] for a in rfa]
  B, M, N = math.prod(bshape), math.prod(mshape), math.prod(nshape)
  K = math.prod(lq.shape[a] for a in lca)
  k_tile = min(lk, rk)
  if max(lk, rk) % k_tile:
    raise ValueError(f'K tiles of {lk} and {rk} do not nest.')
  if k_tile != K and k_tile % 128:
    raise NotImplementedError(
        f'the tensor-core path takes scale tiles that are multiples of 128 along K, got {k_tile}.')
  ls, lz = _refine(ls, lk, k_tile), _refine(lz, lk, k_tile)
  rs, rz = _refine(rs, rk, k_tile), _refine(rz, rk, k_tile)
  T = K // k_tile

  a3 = lq.permute(lba + lfa + lca).reshape(B, M, K).contiguous()
  # Use the weight where it lies: [.., K, N] order needs no repack (MN-major operand).
  kn = rq.permute(rba + rca + rfa)
  nk = rq.permute(rba + rfa + rca)
  if nk.is_contiguous() and not kn.is_contiguous():
    b3, layout = nk.reshape(B, N, K), _lib.B_NK
  else:
    b3, layout = kn.reshape(B, K, N).contiguous(), _lib.B_KN
  if layout == _lib.B_KN and N % 16:
    b3, layout = nk.reshape(B, N, K).contiguous(), _lib.B_NK

  scale_dt = None
  for sc in (ls, rs):
    if sc is not None:
      scale_dt = sc.dtype if scale_dt is None else torch.promote_types(scale_dt, sc.dtype)
  # Kernel layouts: a-side values [B, M, T], b-side values [B, T, N].
  ls = None if ls is None else ls.to(scale_dt).contiguous()
  rs = None if rs is None else rs.to(scale_dt).transpose(1, 2).contiguous()
  scale_code = numerics.code_of_float(scale_dt) if scale_dt is not None else _lib.F32
  raw = ls is None and rs is None and code == _lib.S8
  out_t = torch.int32 if raw else res_t
  out = _result_buffer((B, M, N), out_t, lq.device)
  err = _lib.error_flag(lq.device)
  epi = _lib.EPI_REFERENCE if EPILOGUE == 'reference' else _lib.EPI_F32
  L = _lib.lib()
  stream = _lib.stream_ptr(lq.device)

  if T > 1 or lz is not None or rz is not None:
    if raw:
      raise NotImplementedError('raw accumulators of a tiled contraction are not offered.')
    corr_row = corr_col = None
    if lz is not None:      # dot_general.py:228-240
      corr_row = lz.to(torch.int32).expand(B, M, T).contiguous()
      corr_col = torch.empty((B, T, N), dtype=torch.int32, device=lq.device)
    elif rz is not None:    # dot_general.py:241-253
      corr_col = rz.to(torch.int32).expand(B, N, T).transpose(1, 2).contiguous()
      corr_row = torch.empty((B, M, T), dtype=torch.int32, device=lq.device)
    for b in range(B):
      if lz is not None:
        rows, cols, k_axis = (N, K, 1) if layout == _lib.B_NK else (K, N, 0)
        _lib.check(L.qwx_code_sums(_lib.ptr(b3[b]), rows, cols, k_axis, k_tile, 1,
                                   _lib.ptr(corr_col[b]), stream), 'code_sums')
      elif rz is not None:
        _lib.check(L.qwx_code_sums(_lib.ptr(a3[b]), M, K, 1, k_tile, 0,
                                   _lib.ptr(corr_row[b]), stream), 'code_sums')
      _lib.check(L.qwx_gemm_q8_tiled(
          _lib.ptr(a3[b]), _lib.ptr(b3[b]), code, layout, M, N, K, k_tile,
          _lib.ptr(None if ls is None else ls[b]), int(ls is not None and ls.shape[-1] > 1),
          _lib.ptr(None if rs is None else rs[b]), int(rs is not None and rs.shape[1] > 1),
          scale_code, _lib.ptr(None if corr_row is None else corr_row[b]),
          _lib.ptr(None if corr_col is None else corr_col[b]), _lib.ptr(out[b]),
          _out_code(out_t), epi, _lib.ptr(err), stream), 'dot_general')
  elif (code == _lib.S8 and layout == _lib.B_NK and M <= SKINNY_MAX_ROWS and K % 256 == 0
        and N % 16 == 0):
    # decode-shaped: the warp-level kernel streams the [N, K] weight once
    ws_bytes = L.qwx_gemm_q8_skinny_workspace_bytes(M, N)
    ws = _splitk_workspace(lq.device, ws_bytes, 'skinny')
    for b in range(B):
      _lib.check(L.qwx_gemm_q8_skinny(
          _lib.ptr(a3[b]), _lib.ptr(b3[b]), M, N, K,
          _lib.ptr(None if ls is None else ls[b]), _lib.ptr(None if rs is None else rs[b]),
          scale_code, _lib.ptr(out[b]), _out_code(out_t), epi, _lib.ptr(ws), ws.numel(), 1,
          stream), 'dot_general')
  elif (code == _lib.S8 and layout == _lib.B_NK and M <= DECODE_MAX_ROWS and K % 16 == 0):
    # a few token rows against an [N, K] weight: operands swapped on the tensor cores, the
    # weight dealt to the SMs in equal shares
    ws_bytes = L.qwx_gemm_q8_decode_workspace_bytes(M, N)
    ws = _splitk_workspace(lq.device, ws_bytes, 'decode')
    for b in range(B):
      _lib.check(L.qwx_gemm_q8_decode(
          _lib.ptr(a3[b]), _lib.ptr(b3[b]), M, N, K,
          _lib.ptr(None if ls is None else ls[b]), _lib.ptr(None if rs is None else rs[b]),
          scale_code, _lib.ptr(out[b]), _out_code(out_t), epi, _lib.ptr(ws), ws.numel(), 1,
          _lib.ptr(err), stream), 'dot_general')
  else:
    ws_bytes = L.qwx_gemm_q8_workspace_bytes(M, N, K)
    ws = _splitk_workspace(lq.device, ws_bytes) if ws_bytes else None
    for b in range(B):
      _lib.check(L.qwx_gemm_q8_ws(
          _lib.ptr(a3[b]), _lib.ptr(b3[b]), code, layout, M, N, K, 0,
          _lib.ptr(None if ls is None else ls[b]), 0, _lib.ptr(None if rs is None else rs[b]), 0,
          scale_code, _lib.ptr(out[b]), _out_code(out_t), epi, _lib.ptr(ws), ws_bytes, 1,
          _lib.ptr(err), stream), 'dot_general')
  out = out.reshape(bshape + mshape + nshape)
  return out if out.dtype == res_t else out.to(res_t)


_ws_lock = threading.Lock()
_ws_cache: dict = {}


def _drop_workspaces():
  with _ws_lock:
    _ws_cache.clear()


# a kernel that gave up on a wait skips the reset of its tile counters: start from new buffers
_lib.on_device_error(_drop_workspaces)


def _splitk_workspace(device, nbytes: int, kind: str = 'split') -> torch.Tensor:
  """Zero-filled scratch for the split-K and the decode-shaped form of the GEMM, one per
  (device, stream, kind).  The kernels leave what they need zero and calls on one stream run
  in order, so it is cleared only when it is created or grown."""
  key = (device, torch.cuda.current_stream(device).cuda_stream, kind)
  with _ws_lock:
    ws = _ws_cache.get(key)
    if ws is None or ws.numel() < nbytes:
      ws = torch.zeros(max(nbytes, 1 << 22), dtype=torch.uint8, device=device)
      _ws_cache[key] = ws
  return ws


def _plain_dot_general(lhs: torch.Tensor, rhs: torch.Tensor, dimension_numbers,
                       preferred_element_type=None) -> torch.Tensor:
  """jax.lax.dot_general on floating tensors (library GEMM): output axes are
  batch, lhs free, rhs free."""
  (lca, rca), (lba, rba) = dimension_numbers
  lca, rca, lba, rba = map(list, (lca, rca, lba, rba))
  lfa = _free_axes(lhs.ndim, lca, lba)
  rfa = _free_axes(rhs.ndim, rca, rba)
  compute = torch.promote_types(lhs.dtype, rhs.dtype)
  bshape = [lhs.shape[a] for a in lba]
  mshape = [lhs.shape[a] for a in lfa]
  nshape = [rhs.shape[a] for a in rfa]
  K = math.prod(lhs.shape[a] for a in lca)
  a3 = lhs.permute(lba + lfa + lca).reshape(math.prod(bshape), math.prod(mshape), K)
  b3 = rhs.permute(rba + rca + rfa).reshape(math.prod(bshape), K, math.prod(nshape))
  out = torch.bmm(a3.to(compute), b3.to(compute)).reshape(bshape + mshape + nshape)
  want = preferred_element_type or compute
  return out if out.dtype == want else out.to(want)


def _slow_dot_general(lhs, rhs, dimension_numbers, preferred_element_type=None,
                      **kwargs) -> torch.Tensor:
  """dot_general.py:264-275 -- dequantize the operands, then a floating-point dot."""
  del kwargs
  from qwix_b200.core import weight_only
  if FUSE_WEIGHT_ONLY and weight_only.eligible(lhs, rhs, dimension_numbers):
    want = preferred_element_type or torch.promote_types(lhs.dtype, rhs.scale.dtype)
    if want in (torch.bfloat16, torch.float32):
      return weight_only.matmul(lhs, rhs, want)
  if isinstance(lhs, QArray):
    lhs = qarray.dequantize(lhs)
  if isinstance(rhs, QArray):
    rhs = qarray.dequantize(rhs)
  return _plain_dot_general(lhs, rhs, dimension_numbers, preferred_element_type)


def loop_dot_general(lhs, rhs, dimension_numbers, preferred_element_type=None,
                     **kwargs) -> torch.Tensor:
  """dot_general.py:278-399 -- the in-kernel accumulation loop of the reference's Pallas
  entry point.  On this backend the loop over K tiles lives inside the GEMM kernel, so the
  entry point resolves to the same fused kernel as the fast path."""
  for x in (lhs, rhs):
    if isinstance(x, QArray):
      assert x.zero_point is None
  return _fast_dot_general(lhs, rhs, dimension_numbers, preferred_element_type, **kwargs)


def dot_general(lhs, rhs, dimension_numbers, precision=None, preferred_element_type=None,
                **kwargs) -> torch.Tensor:
  """dot_general.py:407-491 -- drop-in for jax.lax.dot_general with QArray operands.

  `out_sharding` and `precision` are accepted and ignored (one device per process).
  """
  del precision
  kwargs.pop('out_sharding', None)
  # dot_general.py:432-437: microscaled operands go to the block-scaled tensor-core GEMM first
  from qwix_b200.core import mxfp_dot
  mx = mxfp_dot.mxfp_dot_general(lhs, rhs, dimension_numbers, preferred_element_type)
  if mx is not None:
    return mx
  if use_fast_path(lhs, rhs, dimension_numbers):
    return _fast_dot_general(lhs, rhs, dimension_numbers,
                             preferred_element_type=preferred_element_type, **kwargs)
  return _slow_dot_general(lhs, rhs, dimension_numbers,
                           preferred_element_type=preferred_element_type, **kwargs)
