"""ctypes binding of libqwix_b200.so.  There is no fallback: a missing library or a
nonzero status raises."""

from __future__ import annotations

import ctypes
import pathlib
import threading

import torch

_LIB_PATH = pathlib.Path(__file__).resolve().parent / 'libqwix_b200.so'
_lock = threading.Lock()
_lib = None

# enum qwx_dtype
F32, BF16, F16, S8, S4, E4M3, S32, S4U, MXFP8, MXFP4, NVFP4 = range(11)
# enum qwx_calibration
ABSMAX, MINMAX, RMS = range(3)
# enum qwx_rounding
STRICT, FUSED = 0, 1
# enum qwx_b_layout
B_KN, B_NK = 0, 1
# enum qwx_epilogue
EPI_F32, EPI_REFERENCE = 0, 1

_VALUE_ERRORS = {2, 3, 4}  # shape / align / dtype -> ValueError like the reference

FLOAT_CODES = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}

_i64, _int, _vp, _sz, _dbl = (ctypes.c_int64, ctypes.c_int, ctypes.c_void_p,
                              ctypes.c_size_t, ctypes.c_double)

_SIGNATURES = {
    'qwx_version': (_int, []),
    'qwx_status_string': (ctypes.c_char_p, [_int]),
    'qwx_set_programmatic_launch': (None, [_int]),
    'qwx_get_programmatic_launch': (_int, []),
    'qwx_quantize_workspace_bytes': (_sz, [_i64] * 6),
    'qwx_calibrate': (_int, [_vp, _int] + [_i64] * 6 + [_int, _int, _dbl, _vp, _vp, _vp, _sz, _vp]),
    'qwx_compute_scale_zero_point': (_int, [_vp, _vp, _int, _i64, _int, _vp, _vp, _vp]),
    'qwx_quantize_with_scale': (_int, [_vp, _int] + [_i64] * 6 + [_vp, _vp, _int, _int, _vp, _vp]),
    'qwx_quantize': (_int, [_vp, _int] + [_i64] * 6 + [_int, _int, _dbl, _int, _int, _vp, _vp, _vp, _vp, _sz, _vp]),
    'qwx_quantize_builtin_scratch_bytes': (_sz, []),
    'qwx_quantize_noalloc': (_int, [_vp, _int] + [_i64] * 6 + [_int, _int, _dbl, _int, _int, _vp, _vp, _vp, _vp]),
    'qwx_dequantize': (_int, [_vp, _int] + [_i64] * 6 + [_vp, _int, _vp, _vp, _vp]),
    'qwx_transpose_codes': (_int, [_vp, _i64, _i64, _vp, _vp]),
    'qwx_w4_packed_bytes': (_sz, [_i64, _i64]),
    'qwx_pack_w4': (_int, [_vp, _i64, _i64, _vp, _vp]),
    'qwx_gemm_a16w4_workspace_bytes': (_sz, [_i64, _i64]),
    'qwx_w4_tiles_packed_bytes': (_sz, [_i64, _i64]),
    'qwx_pack_w4_tiles': (_int, [_vp, _i64, _i64, _vp, _vp]),
    'qwx_gemm_a16w4_mma_workspace_bytes': (_sz, [_i64, _i64]),
    'qwx_gemm_a16w4_mma': (_int, [_vp, _vp, _vp, _int, _i64, _i64, _i64, _i64, _vp, _int, _vp, _sz, _int,
                                  _vp, _vp]),
    'qwx_gemm_a16w4': (_int, [_vp, _vp, _vp, _int, _i64, _i64, _i64, _i64, _vp, _int, _vp, _sz, _int,
                              _vp, _vp]),
    'qwx_hadamard_rotate': (_int, [_vp, _int, _i64, _i64, _int, _int, _vp, _vp, _vp, _vp]),
    'qwx_hadamard_quantize': (_int, [_vp, _int, _i64, _i64, _int, _vp, _vp, _int, _int, _vp, _vp, _vp]),
    'qwx_hadamard_gemm_workspace_bytes': (_sz, [_i64, _i64]),
    'qwx_hadamard_gemm': (_int, [_vp, _i64, _i64, _vp, _vp, _vp, _vp, _i64, _int, _int, _int, _vp, _int,
                                 _int, _vp, _sz, _vp, _vp]),
    'qwx_quant_gemm_q8_workspace_bytes': (_sz, [_i64, _i64]),
    'qwx_quant_gemm_q8': (_int, [_vp, _i64, _i64, _vp, _vp, _i64, _int, _int, _int, _vp, _int, _int,
                                 _vp, _sz, _vp, _vp]),
    'qwx_gemm_q8': (_int, [_vp, _vp, _int, _int, _i64, _i64, _i64, _i64, _vp, _int, _vp, _int,
                           _int, _vp, _int, _int, _vp, _vp]),
    'qwx_gemm_q8_tiled': (_int, [_vp, _vp, _int, _int, _i64, _i64, _i64, _i64, _vp, _int, _vp, _int,
                                 _int, _vp, _vp, _vp, _int, _int, _vp, _vp]),
    'qwx_code_sums': (_int, [_vp, _i64, _i64, _int, _i64, _int, _vp, _vp]),
    'qwx_mx_scales_packed_bytes': (_sz, [_int, _i64, _i64]),
    'qwx_mx_pack_scales': (_int, [_int, _vp, _int, _i64, _i64, _int, _vp, _sz, _vp]),
    'qwx_gemm_mx8': (_int, [_vp, _vp, _int, _i64, _i64, _i64, _vp, _vp, _vp, _int, _vp, _vp]),
    'qwx_mx4_scales_packed_bytes': (_sz, [_int, _i64, _i64]),
    'qwx_mx4_pack_scales': (_int, [_int, _vp, _int, _i64, _i64, _int, _vp, _sz, _vp]),
    'qwx_mx4_pack_codes': (_int, [_vp, _i64, _i64, _int, _vp, _vp]),
    'qwx_gemm_mx4': (_int, [_vp, _vp, _i64, _i64, _i64, _vp, _vp, _vp, _int, _vp, _vp]),
    'qwx_nvfp4_scales_packed_bytes': (_sz, [_int, _i64, _i64]),
    'qwx_nvfp4_pack_scales': (_int, [_int, _vp, _int, _i64, _i64, _int, _vp, _sz, _vp]),
    'qwx_gemm_nvfp4': (_int, [_vp, _vp, _i64, _i64, _i64, _vp, _vp, _vp, _int, _vp, _vp]),
    'qwx_add_rmsnorm_quantize': (_int, [_vp, _vp, _vp, _dbl, _i64, _i64, _vp, _vp, _vp, _vp, _vp]),
    'qwx_add_rmsnorm_quantize_peer': (_int, [_vp, _vp, _vp, _int, _int, _vp, _int, _vp, _dbl, _i64, _i64,
                                             _vp, _vp, _vp, _vp, _vp, _i64, _vp]),
    'qwx_peer_allreduce': (_int, [_vp, _vp, _int, _int, _vp, _int, _i64, _i64, _vp, _i64, _vp]),
    'qwx_silu_mul_quantize': (_int, [_vp, _i64, _i64, _vp, _vp, _vp, _vp]),
    'qwx_argmax_rows_workspace_bytes': (_sz, [_i64, _i64]),
    'qwx_argmax_rows': (_int, [_vp, _int, _i64, _i64, _i64, _vp, _vp, _vp, _sz, _vp]),
    'qwx_rope_cache': (_int, [_vp, _i64, _i64, _int, _int, _int, _vp, _vp, _i64, _vp, _vp, _vp, _vp,
                              _i64, _i64, _vp]),
    'qwx_gemm_q8_skinny_workspace_bytes': (_sz, [_i64, _i64]),
    'qwx_gemm_q8_skinny': (_int, [_vp, _vp, _i64, _i64, _i64, _vp, _vp, _int, _vp, _int, _int, _vp, _sz,
                                  _int, _vp]),
    'qwx_gemm_q8_decode_workspace_bytes': (_sz, [_i64, _i64]),
    'qwx_gemm_q8_decode': (_int, [_vp, _vp, _i64, _i64, _i64, _vp, _vp, _int, _vp, _int, _int, _vp, _sz,
                                  _int, _vp, _vp]),
    'qwx_gemm_q8_workspace_bytes': (_sz, [_i64, _i64, _i64]),
    'qwx_gemm_q8_ws': (_int, [_vp, _vp, _int, _int, _i64, _i64, _i64, _i64, _vp, _int, _vp, _int,
                              _int, _vp, _int, _int, _vp, _sz, _int, _vp, _vp]),
}


def exported_symbols():
  """Names that include/qwix_b200.h declares and the library must export."""
  return tuple(_SIGNATURES)


def lib() -> ctypes.CDLL:
  global _lib
  if _lib is None:
    with _lock:
      if _lib is None:
        if not _LIB_PATH.exists():
          raise RuntimeError(
              f'{_LIB_PATH} is missing: build it with `python -m qwix_b200.build` '
              '(there is no CPU or PyTorch fallback for the quantized kernels).')
        handle = ctypes.CDLL(str(_LIB_PATH))
        for name, (res, args) in _SIGNATURES.items():
          fn = getattr(handle, name)
          fn.restype, fn.argtypes = res, args
        _lib = handle
  return _lib


def check(status: int, what: str):
  if status == 0:
    return
  msg = lib().qwx_status_string(status).decode()
  exc = ValueError if status in _VALUE_ERRORS else (
      NotImplementedError if status == 5 else RuntimeError)
  raise exc(f'{what}: {msg} (status {status})')


def ptr(t: torch.Tensor | None):
  return None if t is None else ctypes.c_void_p(t.data_ptr())


def stream_ptr(device=None):
  return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


_error_flags: dict = {}


def error_flag(device) -> torch.Tensor:
  """The device int32 that kernels with bounded waits write when a wait runs out, one per
  device for the life of the process (allocating and clearing one per call would be a kernel
  launch per GEMM).  It is never cleared: `raise_on_device_error` reports a failure once it
  happened."""
  device = torch.device(device)
  key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
  flag = _error_flags.get(key)
  if flag is None:
    flag = _error_flags[key] = torch.zeros(1, dtype=torch.int32, device=device)
  return flag


_error_hooks: list = []


def on_device_error(hook):
  """Registers a callable that runs when a device-side failure is reported or cleared: the
  owners of scratch buffers that kernels are supposed to leave zeroed drop them, because a
  kernel that gave up on a wait leaves its counters as they were."""
  _error_hooks.append(hook)


def raise_on_device_error(device=None):
  """Synchronises and raises if any kernel of this process reported a wait that ran out."""
  for key, flag in list(_error_flags.items()):
    if device is not None and torch.device(device).index not in (None, key[1]):
      continue
    code = int(flag.item())
    if code:
      for hook in _error_hooks:
        hook()
      raise RuntimeError(f'a device-side wait ran out on cuda:{key[1]} (status {code}: '
                         f'{lib().qwx_status_string(code).decode()})')


def clear_device_error(device=None):
  """Forgets a reported failure (after the caller has dealt with it) and drops the cached
  scratch buffers, so that the next call starts from zeroed counters."""
  for key, flag in list(_error_flags.items()):
    if device is None or torch.device(device).index in (None, key[1]):
      flag.zero_()
  for hook in _error_hooks:
    hook()


def require_cuda(*tensors):
  for t in tensors:
    if t is not None and not t.is_cuda:
      raise RuntimeError(
          'qwix_b200 kernels run on a CUDA device only; got a tensor on '
          f'{t.device}.  There is no CPU fallback.')
