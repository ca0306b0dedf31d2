"""Conversions between the oracle's NumPy arrays and the package's CUDA tensors."""

import ml_dtypes
import numpy as np
import torch


def to_numpy(t: torch.Tensor) -> np.ndarray:
  t = t.detach().cpu().contiguous()
  if t.dtype == torch.bfloat16:
    return t.view(torch.int16).numpy().view(ml_dtypes.bfloat16)
  if t.dtype == torch.float8_e4m3fn:
    return t.view(torch.uint8).numpy().view(ml_dtypes.float8_e4m3fn)
  return t.numpy()


def to_torch(a: np.ndarray, device='cuda') -> torch.Tensor:
  a = np.ascontiguousarray(a)
  if a.dtype == np.dtype(ml_dtypes.bfloat16):
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16).to(device)
  if a.dtype == np.dtype(ml_dtypes.float8_e4m3fn):
    return torch.from_numpy(a.view(np.uint8).copy()).view(torch.float8_e4m3fn).to(device)
  if a.dtype == np.dtype(ml_dtypes.int4):
    return torch.from_numpy(a.astype(np.int8)).to(device)
  return torch.from_numpy(a.copy()).to(device)


def codes_equal(t: torch.Tensor, a: np.ndarray) -> bool:
  """Bit-exact comparison of quantized codes (int8 / int4-in-int8 / e4m3 bytes)."""
  got = to_numpy(t)
  if a.dtype == np.dtype(ml_dtypes.int4):
    a = a.astype(np.int8)
  return got.shape == a.shape and np.array_equal(
      got.view(np.uint8), np.ascontiguousarray(a).view(np.uint8))


def np_dtype(name: str):
  return {'float32': np.float32, 'bfloat16': ml_dtypes.bfloat16,
          'float16': np.float16}[name]
