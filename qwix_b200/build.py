"""Builds libqwix_b200.so (hand-written sm_100a CUDA + the C ABI) with nvcc, in tree."""

from __future__ import annotations

import os
import pathlib
import subprocess

ROOT = pathlib.Path(__file__).resolve().parent
CSRC = ROOT / 'csrc'
LIB = ROOT / 'libqwix_b200.so'
SOURCES = ('capi.cu', 'quantize.cu', 'gemm_q8.cu', 'gemm_q8_pair.cu', 'gemm_q8_narrow.cu', 'gemm_q8_tiled.cu', 'gemm_q8_tiled_pair.cu', 'gemm_q8_skinny.cu', 'gemm_q8_decode.cu', 'gemm_mx8.cu', 'gemm_mx_pair.cu', 'gemm_w4.cu', 'gemm_w4_mma.cu', 'hadamard.cu', 'decoder_ops.cu',
           'xla_ffi_shim.cc')   # compiles to nothing where the XLA FFI headers are absent
FLAGS = ('-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo', '-O3',
         '-std=c++17', '-shared', '-Xcompiler', '-fPIC')


def _newest_source_mtime() -> float:
  files = list(CSRC.glob('*.cu')) + list(CSRC.glob('*.cuh')) + list(CSRC.glob('*.cc'))
  files.append(ROOT.parent / 'include' / 'qwix_b200.h')
  return max(f.stat().st_mtime for f in files)


def build(force: bool = False, verbose: bool = False) -> pathlib.Path:
  """Compiles every kernel for sm_100a; returns the path of the shared library.  Translation
  units are compiled side by side (objects under csrc/build/, which is not tracked) and linked
  into one library."""
  if not force and LIB.exists() and LIB.stat().st_mtime >= _newest_source_mtime():
    return LIB
  from concurrent.futures import ThreadPoolExecutor
  nvcc = os.environ.get('NVCC', 'nvcc')
  objdir = CSRC / 'build'
  objdir.mkdir(exist_ok=True)
  compile_flags = [f for f in FLAGS if f != '-shared']

  def compile_one(src: str) -> str:
    obj = objdir / (src.rsplit('.', 1)[0] + '.o')
    cmd = [nvcc, *compile_flags, '-c', '-o', str(obj), str(CSRC / src)]
    if verbose:
      cmd[1:1] = ['-Xptxas', '-v']
    subprocess.run(cmd, check=True, cwd=str(CSRC))
    return str(obj)

  with ThreadPoolExecutor(max_workers=min(len(SOURCES), os.cpu_count() or 1)) as pool:
    objects = list(pool.map(compile_one, SOURCES))
  subprocess.run([nvcc, '-gencode', 'arch=compute_100a,code=sm_100a', '-shared', '-o', str(LIB), *objects], check=True, cwd=str(CSRC))
  return LIB


if __name__ == '__main__':
  print(build(force=True, verbose=True))
