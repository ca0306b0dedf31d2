"""Fused weight-only int4 contraction: the kernel-side form of the reference's
dequantize-then-dot path (qwix/_src/core/dot_general.py:264-275, 444-452) for a bf16
activation and an int4 weight whose scales tile the contraction axis.

The logical QArray keeps its [K, N] codes; the streaming layout the kernel reads is built
once per weight (weights are static under PTQ) and cached on the QArray object.
"""

from __future__ import annotations

import threading

import torch

from qwix_b200 import _lib
from qwix_b200.core import numerics
from qwix_b200.core.qarray import QArray

_MAX_ROWS_PER_CALL = 128
# The fused kernel streams the weight once per 32 tokens (45-80 us per pass at 8192 x 28672);
# the unfused path (generic dequantize kernel + library GEMM) measured 1.8 ms at 128 tokens, so
# the fused kernel stays the better fit far beyond its 32-token pass.
_MAX_FUSED_ROWS = 1024

_ws_lock = threading.Lock()
_ws_cache: dict = {}


def _drop_workspaces():
  with _ws_lock:
    _ws_cache.clear()


_lib.on_device_error(_drop_workspaces)


def eligible(lhs, rhs, dimension_numbers) -> bool:
  """True when (lhs, rhs) is [.., K] bf16 x int4 [K, N] with K-tiled symmetric scales that
  the fused kernel supports."""
  if isinstance(lhs, QArray) or not isinstance(rhs, QArray):
    return False
  (lca, rca), (lba, rba) = dimension_numbers
  if lhs.dtype != torch.bfloat16 or rhs.qtype != 'int4' or rhs.zero_point is not None:
    return False
  if rhs.ndim != 2 or tuple(rca) != (0,) or tuple(lca) != (lhs.ndim - 1,) or lba or rba:
    return False
  if rhs.scale.dtype not in (torch.float32, torch.bfloat16):
    return False
  K, N = rhs.shape
  sk, sn = rhs.scale.shape
  if sn != N or K % 128 or N % 16 or K % sk or (K // sk) % 128:
    return False
  rows = lhs.numel() // K
  return 0 < rows <= _MAX_FUSED_ROWS and lhs.is_cuda


def prepare(rhs: QArray) -> torch.Tensor:
  """Packs the weight into the kernel's unit layout (once; cached on the QArray)."""
  cached = getattr(rhs, '_w4_packed', None)
  if cached is not None:
    return cached
  K, N = rhs.shape
  L = _lib.lib()
  q = rhs.qvalue.contiguous()
  packed = torch.empty(L.qwx_w4_packed_bytes(K, N), dtype=torch.uint8, device=q.device)
  _lib.check(L.qwx_pack_w4(_lib.ptr(q), K, N, _lib.ptr(packed), _lib.stream_ptr(q.device)),
             'pack_w4')
  rhs._w4_packed = packed
  rhs._w4_scale = rhs.scale.contiguous()
  return packed


# From this many token rows on the contraction runs on the tcgen05 tensor cores
# (csrc/gemm_w4_mma.cu: int4 -> scaled bf16 in shared memory, one float32 accumulation over all
# of K); below it the warp-level kernel keeps float32 scales in float32.
TENSOR_CORE_MIN_ROWS = 33


def prepare_tiles(rhs: QArray) -> torch.Tensor:
  """Packs the weight into the tensor-core kernel's tile layout (once; cached on the QArray)."""
  cached = getattr(rhs, '_w4_tiles', None)
  if cached is not None:
    return cached
  K, N = rhs.shape
  L = _lib.lib()
  q = rhs.qvalue.contiguous()
  packed = torch.empty(L.qwx_w4_tiles_packed_bytes(K, N), dtype=torch.uint8, device=q.device)
  _lib.check(L.qwx_pack_w4_tiles(_lib.ptr(q), K, N, _lib.ptr(packed), _lib.stream_ptr(q.device)),
             'pack_w4_tiles')
  rhs._w4_tiles = packed
  rhs._w4_scale = rhs.scale.contiguous()
  return packed


def _workspace_mma(device, M: int, N: int) -> torch.Tensor:
  key = (device, torch.cuda.current_stream(device).cuda_stream, 'mma', 32 if M <= 32 else (64 if M <= 64 else 128))
  with _ws_lock:
    ws = _ws_cache.get(key)
    if ws is None:
      ws = torch.zeros(_lib.lib().qwx_gemm_a16w4_mma_workspace_bytes(M, N), dtype=torch.uint8, device=device)
      _ws_cache[key] = ws
  return ws


def _workspace(device, M: int, N: int) -> torch.Tensor:
  """A zero-filled scratch buffer per (device, stream, shape).  The kernel leaves it zero, so
  it is cleared only once."""
  key = (device, torch.cuda.current_stream(device).cuda_stream, M, N)
  with _ws_lock:
    ws = _ws_cache.get(key)
    if ws is None:
      n = _lib.lib().qwx_gemm_a16w4_workspace_bytes(M, N)
      ws = torch.zeros(n, dtype=torch.uint8, device=device)
      _ws_cache[key] = ws
  return ws


def matmul(lhs: torch.Tensor, rhs: QArray, out_dtype: torch.dtype) -> torch.Tensor:
  """lhs [.., K] @ dequantize(rhs) [K, N] -> [.., N]."""
  K, N = rhs.shape
  x = lhs.reshape(-1, K).contiguous()
  rows = x.shape[0]
  out = torch.empty((rows, N), dtype=out_dtype, device=x.device)
  err = _lib.error_flag(x.device)
  L = _lib.lib()
  tile = K // rhs.scale.shape[0]
  oc = _lib.BF16 if out_dtype == torch.bfloat16 else _lib.F32
  if rows >= TENSOR_CORE_MIN_ROWS:
    tiles = prepare_tiles(rhs)
    scale = rhs._w4_scale
    for r0 in range(0, rows, _MAX_ROWS_PER_CALL):
      m = min(_MAX_ROWS_PER_CALL, rows - r0)
      ws = _workspace_mma(x.device, m, N)
      _lib.check(L.qwx_gemm_a16w4_mma(
          _lib.ptr(x[r0:r0 + m]), _lib.ptr(tiles), _lib.ptr(scale),
          numerics.code_of_float(scale.dtype), m, N, K, tile, _lib.ptr(out[r0:r0 + m]), oc,
          _lib.ptr(ws), ws.numel(), 1, _lib.ptr(err), _lib.stream_ptr(x.device)), 'gemm_a16w4_mma')
    return out.reshape(*lhs.shape[:-1], N)
  packed = prepare(rhs)
  scale = rhs._w4_scale
  for r0 in range(0, rows, _MAX_ROWS_PER_CALL):
    m = min(_MAX_ROWS_PER_CALL, rows - r0)
    ws = _workspace(x.device, m, N)
    _lib.check(L.qwx_gemm_a16w4(
        _lib.ptr(x[r0:r0 + m]), _lib.ptr(packed), _lib.ptr(scale),
        numerics.code_of_float(scale.dtype), m, N, K, tile, _lib.ptr(out[r0:r0 + m]), oc,
        _lib.ptr(ws), ws.numel(), 1, _lib.ptr(err), _lib.stream_ptr(x.device)), 'gemm_a16w4')
  return out.reshape(*lhs.shape[:-1], N)
