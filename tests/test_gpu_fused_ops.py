"""GPU parity of the fused decoder stages against their unfused PyTorch composition and
against the quantizer applied to their own floating-point output."""

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from qwix_b200 import fused
from qwix_b200.core import qarray as bq

pytestmark = pytest.mark.gpu

HOW = lambda nd: bq.HowToQuantize(qtype='int8', channelwise_axes=list(range(nd - 1)))


def _rmsnorm(x, w, eps):
  v = x.float()
  v = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)
  return (v * w.float()).to(x.dtype)


@pytest.mark.parametrize('shape', [(32, 1, 4096), (3, 50, 1024), (2, 7, 8192), (5, 136)])
@pytest.mark.parametrize('with_delta', [False, True])
def test_add_rmsnorm_matches_unfused(shape, with_delta):
  g = torch.Generator(device='cuda').manual_seed(sum(shape))
  x = torch.randn(shape, device='cuda', generator=g).to(torch.bfloat16)
  x[..., :3] *= 30
  x[0].reshape(-1, shape[-1])[0] = 0       # a zero row: y = 0, scale 1, codes 0
  delta = (0.5 * torch.randn(shape, device='cuda', generator=g)).to(torch.bfloat16) if with_delta else None
  w = (1 + 0.1 * torch.randn(shape[-1], device='cuda', generator=g)).to(torch.bfloat16)
  eps = 1e-5
  xs = x + delta if with_delta else x
  want = _rmsnorm(xs, w, eps)

  a = fused.AddRmsNorm(x, delta, w, eps)
  y = a.materialize()
  assert torch.equal(a.residual, xs)
  # only the order of the float32 sum of squares differs: at most one bf16 ulp, almost never
  diff = (y.float() - want.float()).abs()
  assert torch.all(diff <= 2.0 ** -7 * want.float().abs().clamp_min(2.0 ** -20))
  assert (y == want).float().mean() > 0.995

  b = fused.AddRmsNorm(x, delta, w, eps)
  qa = b.quantized(HOW(len(shape)))
  ref = bq.quantize(y, HOW(len(shape)))        # the quantizer on the kernel's own output
  assert torch.equal(qa.qvalue, ref.qvalue)
  assert torch.equal(qa.scale.view(torch.int16), ref.scale.view(torch.int16))
  assert qa.scale.shape == ref.scale.shape
  assert torch.equal(b.residual, xs)


@pytest.mark.parametrize('shape', [(32, 1, 2 * 14336), (4, 33, 2 * 1024), (6, 2 * 72)])
def test_silu_mul_matches_unfused(shape):
  g = torch.Generator(device='cuda').manual_seed(sum(shape))
  gu = (2 * torch.randn(shape, device='cuda', generator=g)).to(torch.bfloat16)
  f = shape[-1] // 2
  want = F.silu(gu[..., :f]) * gu[..., f:]
  y = fused.SiluMul(gu).materialize()
  mism = (y != want)
  # expf / division are the same float32 operations: identical up to rare last-bit cases
  assert mism.float().mean() < 1e-3
  assert torch.all((y.float() - want.float()).abs() <= 2.0 ** -7 * want.float().abs().clamp_min(2.0 ** -30))
  qa = fused.SiluMul(gu).quantized(HOW(len(shape)))
  ref = bq.quantize(y, HOW(len(shape)))
  assert torch.equal(qa.qvalue, ref.qvalue)
  assert torch.equal(qa.scale.view(torch.int16), ref.scale.view(torch.int16))


def test_lazy_act_other_rules_fall_back():
  gu = torch.randn((4, 2 * 256), device='cuda').to(torch.bfloat16)
  how = bq.HowToQuantize(qtype='int8', channelwise_axes=[0], tiled_axes={1: 128})
  qa = fused.SiluMul(gu).quantized(how)
  ref = bq.quantize(fused.SiluMul(gu).materialize(), how)
  assert torch.equal(qa.qvalue, ref.qvalue) and qa.scale.shape == ref.scale.shape


@pytest.mark.parametrize('tensor_pos', [False, True])
def test_rope_cache_matches_unfused(tensor_pos):
  B, T, hq, hkv, hd, S = 3, (1 if tensor_pos else 5), 4, 2, 128, 40
  g = torch.Generator(device='cuda').manual_seed(1)
  qkv = torch.randn((B, T, (hq + 2 * hkv) * hd), device='cuda', generator=g).to(torch.bfloat16)
  pos = 7
  ang = torch.arange(S, device='cuda', dtype=torch.float32)[:, None] * (
      1.0 / (10000.0 ** (torch.arange(0, hd, 2, device='cuda', dtype=torch.float32) / hd)))[None, :]
  cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
  cache = torch.zeros((2, B + 2, hkv, S, hd), dtype=torch.bfloat16, device='cuda')
  ck, cv = cache[0, 1:1 + B], cache[1, 1:1 + B]          # views with a batch offset
  p = torch.tensor([pos], device='cuda') if tensor_pos else pos
  q = fused.rope_cache(qkv, hq, hkv, hd, cos, sin, p, ck, cv)

  def rope(x, c, s):
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half].float(), x[..., half:].float()
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)
  qq, kk, vv = qkv.split([hq * hd, hkv * hd, hkv * hd], dim=-1)
  qq = qq.view(B, T, hq, hd).transpose(1, 2)
  kk = kk.view(B, T, hkv, hd).transpose(1, 2)
  vv = vv.view(B, T, hkv, hd).transpose(1, 2)
  c, s = cos[pos:pos + T], sin[pos:pos + T]
  assert torch.equal(q, rope(qq, c, s))
  assert torch.equal(ck[:, :, pos:pos + T], rope(kk, c, s))
  assert torch.equal(cv[:, :, pos:pos + T], vv)
  # nothing else in the cache was touched
  assert int(cache.count_nonzero()) == int(ck[:, :, pos:pos + T].count_nonzero() + cv[:, :, pos:pos + T].count_nonzero())


# ---- the all-reduce folded into add + norm + quantize, on ONE GPU ------------------------------
#
# Both "ranks'" partial buffers and flag arrays live on this device.  Only rank 0's kernel is
# launched; the flags its peer would have raised are written from the host beforehand, so no
# kernel ever waits for another one.

def _peer_setup(rows, d, world=2, max_ctas=148 * 8, seed=0):
  import ctypes
  g = torch.Generator(device='cuda').manual_seed(seed)
  x = torch.randn((rows, d), device='cuda', generator=g).to(torch.bfloat16)
  parts = [(0.5 * torch.randn((rows, d), device='cuda', generator=g)).to(torch.bfloat16)
           for _ in range(world)]
  w = (1 + 0.1 * torch.randn(d, device='cuda', generator=g)).to(torch.bfloat16)
  flags = [torch.zeros(max_ctas * world, dtype=torch.int32, device='cuda') for _ in range(world)]
  launches = torch.zeros(max_ctas, dtype=torch.int32, device='cuda')
  arr = ctypes.c_void_p * world
  return dict(x=x, parts=parts, w=w, flags=flags, launches=launches, max_ctas=max_ctas, world=world,
              part_ptrs=arr(*[p.data_ptr() for p in parts]), flag_ptrs=arr(*[f.data_ptr() for f in flags]))


def _peer_call(s, err, wait_cycles=0, quantize=True):
  from qwix_b200 import _lib
  rows, d = s['x'].shape
  out = dict(x_out=torch.full_like(s['x'], 7.0),
             q=torch.full((rows, d), 7, dtype=torch.int8, device='cuda') if quantize else None,
             scale=torch.full((rows,), 7.0, dtype=torch.bfloat16, device='cuda') if quantize else None,
             y=None if quantize else torch.full_like(s['x'], 7.0))
  _lib.check(_lib.lib().qwx_add_rmsnorm_quantize_peer(
      _lib.ptr(s['x']), s['part_ptrs'], s['flag_ptrs'], s['world'], 0, _lib.ptr(s['launches']),
      s['max_ctas'], _lib.ptr(s['w']), 1e-5, rows, d, _lib.ptr(out['x_out']), _lib.ptr(out['y']),
      _lib.ptr(out['q']), _lib.ptr(out['scale']), _lib.ptr(err), wait_cycles, _lib.stream_ptr()),
      'add_rmsnorm_quantize_peer')
  torch.cuda.synchronize()
  return out


@pytest.mark.parametrize('rows,d,world', [(32, 4096, 2), (3000, 1024, 2), (70, 4096, 4), (8192, 512, 8)])
def test_peer_add_rmsnorm_equals_local_on_summed_partials(rows, d, world):
  from qwix_b200 import _lib
  s = _peer_setup(rows, d, world)
  err = torch.zeros(1, dtype=torch.int32, device='cuda')
  # what an all-reduce would deliver: the float32 sum in rank order, rounded once to bf16
  total = s['parts'][0].float()
  for p in s['parts'][1:]:
    total = total + p.float()
  delta = total.to(torch.bfloat16)
  want = dict(x_out=torch.empty_like(s['x']), q=torch.empty((rows, d), dtype=torch.int8, device='cuda'),
              scale=torch.empty((rows,), dtype=torch.bfloat16, device='cuda'))
  _lib.check(_lib.lib().qwx_add_rmsnorm_quantize(
      _lib.ptr(s['x']), _lib.ptr(delta), _lib.ptr(s['w']), 1e-5, rows, d, _lib.ptr(want['x_out']),
      None, _lib.ptr(want['q']), _lib.ptr(want['scale']), _lib.stream_ptr()), 'add_rmsnorm_quantize')
  for call in (1, 2):                       # the second call waits for launch count 2
    s['flags'][0].fill_(call)               # "every peer has finished its GEMM `call` times"
    got = _peer_call(s, err)
    assert int(err.item()) == 0
    assert torch.equal(got['x_out'], want['x_out'])
    assert torch.equal(got['q'], want['q'])
    assert torch.equal(got['scale'].view(torch.int16), want['scale'].view(torch.int16))
    # rank 0 told every peer, in that peer's flag array, that its own partial is complete
    ctas = int((s['launches'] == call).sum().item())
    assert 0 < ctas <= min(rows, s['max_ctas'])
    for r in range(1, world):
      mine = s['flags'][r].view(-1, world)[:, 0]
      assert int((mine == call).sum().item()) == ctas


def test_peer_wait_runs_out_and_reports():
  """The peer never raises its flags: the bounded hand-shake gives up after its budget, the
  call reports QWX_ERR_DEVICE_WAIT, writes nothing, and the context stays usable."""
  from qwix_b200 import _lib
  s = _peer_setup(64, 2048)
  err = _lib.error_flag(torch.device('cuda'))
  assert int(err.item()) == 0
  got = _peer_call(s, err, wait_cycles=2_000_000)        # about a millisecond
  assert int(err.item()) == 8                             # QWX_ERR_DEVICE_WAIT
  assert bool((got['x_out'] == 7.0).all()) and bool((got['q'] == 7).all())
  assert bool((got['scale'] == 7.0).all())
  with pytest.raises(RuntimeError, match='wait ran out'):
    _lib.raise_on_device_error()
  _lib.clear_device_error()
  _lib.raise_on_device_error()                            # cleared: no longer raises
  # a healthy call afterwards (launch counts went on to 1, so the peer's flags say 2 next)
  s['flags'][0].fill_(2)
  got = _peer_call(s, err)
  assert int(err.item()) == 0
  assert not bool((got['q'] == 7).all())


@pytest.mark.parametrize('shape', [(32, 128256), (4, 16032), (1, 1000), (7, 50), (64, 4096), (3, 8 * 2048 + 5)])
def test_argmax_rows_matches_library(shape):
  g = torch.Generator(device='cuda').manual_seed(sum(shape))
  x = torch.randn(shape, device='cuda', generator=g).to(torch.bfloat16)
  x[0, shape[1] // 3] = x.max() + 1                     # a clear winner
  if shape[0] > 1:
    top = x[1].max()
    x[1, min(5, shape[1] - 1)] = top                    # ties: the lowest index wins
    x[1, shape[1] - 1] = top
  for _ in range(2):                                    # second call: counters were left zero
    idx, val = fused.argmax_rows(x, index_offset=1000, want_values=True)
    want_val, _ = x.float().max(dim=-1)
    assert torch.equal(val, want_val)
    # lowest index among the maxima (the library's own argmax documents the first maximum)
    first = (x.float() == want_val[:, None]).float().argmax(dim=-1)
    assert torch.equal(idx, first + 1000)
  assert torch.equal(fused.argmax_rows(x), first)


@pytest.mark.parametrize('rows,d,world', [(8192, 512, 2), (1030, 1024, 4), (4099, 256, 8), (3, 4096, 2)])
def test_peer_allreduce_in_place_one_gpu(rows, d, world):
  """Every "rank" runs on this GPU, one after the other, with the marks its peers would have
  raised written beforehand: rank r sums its share of the rows and writes the sums into all
  buffers; after the last rank every buffer holds the all-reduced tensor."""
  import ctypes
  from qwix_b200 import _lib
  max_ctas = 148 * 8
  g = torch.Generator(device='cuda').manual_seed(rows + d)
  parts = [torch.randn((rows, d), device='cuda', generator=g).to(torch.bfloat16) for _ in range(world)]
  total = parts[0].float()
  for p in parts[1:]:
    total = total + p.float()                 # rank order, float32
  want = total.to(torch.bfloat16)
  flags = [torch.zeros((max_ctas + 1) * world, dtype=torch.int32, device='cuda') for _ in range(world)]
  launches = [torch.zeros(max_ctas + 2, dtype=torch.int32, device='cuda') for _ in range(world)]
  arr = ctypes.c_void_p * world
  part_ptrs = arr(*[p.data_ptr() for p in parts])
  flag_ptrs = arr(*[f.data_ptr() for f in flags])
  err = torch.zeros(1, dtype=torch.int32, device='cuda')
  for call in (1, 2):
    if call == 2:                             # a second exchange through the same marks
      for p in parts:
        p.copy_(torch.randn((rows, d), device='cuda', generator=g).to(torch.bfloat16))
      total = parts[0].float()
      for p in parts[1:]:
        total = total + p.float()
      want = total.to(torch.bfloat16)
    for r in range(world):
      flags[r].fill_(call)                    # "all peers are ready and done" for this call
      _lib.check(_lib.lib().qwx_peer_allreduce(
          part_ptrs, flag_ptrs, world, r, _lib.ptr(launches[r]), max_ctas, rows, d, _lib.ptr(err), 0,
          _lib.stream_ptr()), 'peer_allreduce')
      torch.cuda.synchronize()
      assert int(err.item()) == 0
      lo, hi = rows * r // world, rows * (r + 1) // world
      for p in parts:                         # rank r's rows are reduced everywhere
        assert torch.equal(p[lo:hi], want[lo:hi])
    for p in parts:
      assert torch.equal(p, want)
    assert all(int(l[max_ctas + 1].item()) == call and int(l[max_ctas].item()) == 0 for l in launches)


def test_peer_allreduce_done_wait_runs_out():
  import ctypes
  from qwix_b200 import _lib
  max_ctas, world, rows, d = 148 * 8, 2, 64, 512
  parts = [torch.ones((rows, d), dtype=torch.bfloat16, device='cuda') for _ in range(world)]
  flags = [torch.zeros((max_ctas + 1) * world, dtype=torch.int32, device='cuda') for _ in range(world)]
  flags[0][:max_ctas * world].fill_(1)        # the peer is ready, but never says "done"
  launches = torch.zeros(max_ctas + 2, dtype=torch.int32, device='cuda')
  arr = ctypes.c_void_p * world
  err = torch.zeros(1, dtype=torch.int32, device='cuda')
  _lib.check(_lib.lib().qwx_peer_allreduce(
      arr(*[p.data_ptr() for p in parts]), arr(*[f.data_ptr() for f in flags]), world, 0,
      _lib.ptr(launches), max_ctas, rows, d, _lib.ptr(err), 2_000_000, _lib.stream_ptr()), 'peer_allreduce')
  torch.cuda.synchronize()
  assert int(err.item()) == 8                 # QWX_ERR_DEVICE_WAIT: reported, the context lives on
  assert bool((parts[0][:32] == 2).all()) and bool((parts[1][:32] == 2).all())
