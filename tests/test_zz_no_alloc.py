"""GPU: the allocation-free quantize entry point against the ordinary one.

qwx_quantize_noalloc serves callers that cannot hand the library a workspace and cannot
allocate one either (a handler running inside a framework with a fixed buffer plan, a warm
serving loop that must stay away from cudaMalloc).  Its scratch is an array inside the library,
shared by every call, so this test calls it twice in a row with different inputs and with a
different tiling: the second call must not be disturbed by what the first one left behind.
Both results must equal qwx_quantize's bit for bit (codes, scales and zero points are
integer / exactly rounded quantities; the suite's tolerance for them is zero).

The file name sorts last so that, in a run that stops at the first failure, every other test
has already been executed.
"""

import pytest
import torch

from qwix_b200 import _lib

pytestmark = pytest.mark.gpu


def _quantize(entry, x, tiles, method, qtype_code, workspace=None):
  """Calls qwx_quantize (workspace given) or qwx_quantize_noalloc through the C ABI."""
  R, C = x.shape
  tr, tc = tiles
  groups = (R // tr) * (C // tc)
  q = torch.empty((R, C), dtype=torch.int8, device=x.device)
  scale = torch.empty(groups, dtype=x.dtype, device=x.device)
  zp = torch.empty(groups, dtype=torch.int8, device=x.device) if method == _lib.MINMAX else None
  L = _lib.lib()
  head = (_lib.ptr(x), _lib.BF16, 1, R, C, 1, tr, tc, method, 0, 0.0, qtype_code, _lib.STRICT,
          _lib.ptr(q), _lib.ptr(scale), _lib.ptr(zp))
  if entry == 'noalloc':
    rc = L.qwx_quantize_noalloc(*head, _lib.stream_ptr(x.device))
  else:
    rc = L.qwx_quantize(*head, _lib.ptr(workspace), workspace.numel(), _lib.stream_ptr(x.device))
  _lib.check(rc, entry)
  torch.cuda.synchronize()
  return q, scale, zp


def test_noalloc_entry_matches_workspace_entry_twice_in_a_row():
  L = _lib.lib()
  assert L.qwx_quantize_builtin_scratch_bytes() == 1 << 20
  g = torch.Generator(device='cpu').manual_seed(7)
  calls = [
      # per-output-channel columns of a [K, N] weight: statistics go through the scratch
      (torch.randn(384, 512, generator=g) * 0.02, (384, 1), _lib.ABSMAX, _lib.S8),
      # then sub-channel tiles with zero points, larger values, other tile count
      (torch.randn(256, 768, generator=g) * 3.0 + 1.0, (64, 1), _lib.MINMAX, _lib.S4U),
  ]
  for x_cpu, tiles, method, qcode in calls:
    x = x_cpu.to(torch.bfloat16).cuda()
    R, C = x.shape
    need = L.qwx_quantize_workspace_bytes(1, R, C, 1, tiles[0], tiles[1])
    assert 0 < need <= L.qwx_quantize_builtin_scratch_bytes()
    ws = torch.empty(need, dtype=torch.uint8, device='cuda')
    want = _quantize('workspace', x, tiles, method, qcode, workspace=ws)
    got = _quantize('noalloc', x, tiles, method, qcode)
    for a, b in zip(got, want):
      assert (a is None) == (b is None)
      if a is not None:
        assert torch.equal(a.view(torch.uint8) if a.dtype != torch.int8 else a,
                           b.view(torch.uint8) if b.dtype != torch.int8 else b)


def test_noalloc_entry_refuses_views_beyond_its_scratch():
  L = _lib.lib()
  R, C = 1024, 4096                      # one tile per 16 elements: 262,144 tiles > 65,520
  x = torch.zeros((R, C), dtype=torch.bfloat16, device='cuda')
  q = torch.empty((R, C), dtype=torch.int8, device='cuda')
  scale = torch.empty(R * C // 16, dtype=torch.bfloat16, device='cuda')
  assert L.qwx_quantize_workspace_bytes(1, R, C, 1, 16, 1) > L.qwx_quantize_builtin_scratch_bytes()
  rc = L.qwx_quantize_noalloc(_lib.ptr(x), _lib.BF16, 1, R, C, 1, 16, 1, _lib.ABSMAX, 0, 0.0,
                              _lib.S8, _lib.STRICT, _lib.ptr(q), _lib.ptr(scale), None,
                              _lib.stream_ptr(x.device))
  assert rc == 6  # QWX_ERR_WORKSPACE
  with pytest.raises(RuntimeError, match='workspace'):
    _lib.check(rc, 'quantize_noalloc')


def test_noalloc_entry_never_refuses_row_segment_views():
  """Per-token scales of 70,000 rows: 70,000 tiles would not fit the built-in array, but tiles
  that are row segments are quantized in one pass without scratch, so the call must go through
  and equal qwx_quantize bit for bit (the shape of a long prefill in a warm serving loop)."""
  L = _lib.lib()
  R, C = 70000, 64
  g = torch.Generator(device='cpu').manual_seed(11)
  x = torch.randn(R, C, generator=g).to(torch.bfloat16).cuda()
  assert L.qwx_quantize_workspace_bytes(1, R, C, 1, 1, C) > L.qwx_quantize_builtin_scratch_bytes()
  ws = torch.empty(1, dtype=torch.uint8, device='cuda')   # the one-pass path ignores it
  want = _quantize('workspace', x, (1, C), _lib.ABSMAX, _lib.S8, workspace=ws)
  got = _quantize('noalloc', x, (1, C), _lib.ABSMAX, _lib.S8)
  assert torch.equal(got[0], want[0])
  assert torch.equal(got[1].view(torch.int16), want[1].view(torch.int16))
