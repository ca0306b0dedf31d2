"""Builds libqwix_b200.so (hand-written sm_100a CUDA + the C ABI) with nvcc, in tree."""

from __future__ import annotations

import os
import pathlib
import subprocess

ROOT = pathlib.Path(__file__).resolve().parent
CSRC = ROOT / 'csrc'
LIB = ROOT / 'libqwix_b200.so'
SOURCES = ('capi.cu', 'quantize.cu', 'gemm_q8.cu', 'gemm_q8_pair.cu', 'gemm_q8_tiled.cu', 'gemm_q8_skinny.cu', 'gemm_w4.cu', 'hadamard.cu', 'decoder_ops.cu')
FLAGS = ('-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo', '-O3',
         '-std=c++17', '-shared', '-Xcompiler', '-fPIC')


def _newest_source_mtime() -> float:
  files = list(CSRC.glob('*.cu')) + list(CSRC.glob('*.cuh'))
  files.append(ROOT.parent / 'include' / 'qwix_b200.h')
  return max(f.stat().st_mtime for f in files)


def build(force: bool = False, verbose: bool = False) -> pathlib.Path:
  """Compiles every kernel for sm_100a; returns the path of the shared library."""
  if not force and LIB.exists() and LIB.stat().st_mtime >= _newest_source_mtime():
    return LIB
  nvcc = os.environ.get('NVCC', 'nvcc')
  cmd = [nvcc, *FLAGS, '-o', str(LIB), *[str(CSRC / s) for s in SOURCES]]
  if verbose:
    cmd.insert(1, '-Xptxas')
    cmd.insert(2, '-v')
  subprocess.run(cmd, check=True, cwd=str(CSRC))
  return LIB


if __name__ == '__main__':
  print(build(force=True, verbose=True))
