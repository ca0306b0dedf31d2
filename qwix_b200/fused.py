"""Fused element-wise stages of a decoder layer: the activation of a quantized projection is
produced and quantized in one kernel.

A `LazyAct` stands for "the bf16 tensor this stage would produce".  Model code hands it to a
projection (`qwix_b200.nn.Dense`, or anything that ends in `ops.dot_general`) like a tensor.
The provider decides what is needed: under a rule that quantizes activations to int8 with
per-token absmax scales (`boxed_param.py:416-455` calling `qarray.quantize`, qarray.py:638-644)
the kernel emits the QArray directly; otherwise the bf16 tensor is materialised.  Either way
the arithmetic is that of the unfused composition.
"""

from __future__ import annotations

import torch

from qwix_b200 import _lib
from qwix_b200.core import qarray
from qwix_b200.core.qarray import QArray


class LazyAct:
  """An activation [.., features] that has not been computed yet."""

  shape: tuple
  dtype = torch.bfloat16

  @property
  def ndim(self) -> int:
    return len(self.shape)

  def _fusable(self, how: qarray.HowToQuantize) -> bool:
    method = (how.calibration_method or 'absmax').lower()
    return (how.qtype == 'int8' and method == 'absmax' and not how.tiled_axes
            and sorted(how.channelwise_axes) == list(range(self.ndim - 1)))

  def quantized(self, how: qarray.HowToQuantize, _qarray_module=qarray) -> QArray:
    if not self._fusable(how):
      return _qarray_module.quantize(self.materialize(), how)
    rows = 1
    for n in self.shape[:-1]:
      rows *= n
    dev = self.device
    q = torch.empty(self.shape, dtype=torch.int8, device=dev)
    scale = torch.empty(tuple(self.shape[:-1]) + (1,), dtype=torch.bfloat16, device=dev)
    self._run(None, q, scale)
    return QArray(qvalue=q, scale=scale, zero_point=None, qtype='int8')

  def materialize(self) -> torch.Tensor:
    y = torch.empty(self.shape, dtype=torch.bfloat16, device=self.device)
    self._run(y, None, None)
    return y

  def _run(self, y, q, scale):
    raise NotImplementedError


class PeerExchange:
  """Buffers through which the ranks of a tensor-parallel group read each other's partial
  sums with peer loads (symmetric memory over NVLink): two alternating partial buffers, a flag
  array per rank and this rank's launch counts.  Built by `open`, which is collective."""

  MAX_CTAS = 148 * 8

  def __init__(self, group, rank: int, world: int, capacity: int, device):
    import ctypes
    import torch.distributed as dist
    import torch.distributed._symmetric_memory as symm
    self.rank, self.world, self.capacity, self.device = rank, world, capacity, device
    self.partials = [symm.empty((capacity,), dtype=torch.bfloat16, device=device) for _ in range(2)]
    self.flags = symm.empty((self.MAX_CTAS * world,), dtype=torch.int32, device=device)
    self.flags.zero_()
    handles = [symm.rendezvous(t, group) for t in self.partials]
    fh = symm.rendezvous(self.flags, group)
    self._keep = handles + [fh]
    arr = ctypes.c_void_p * world
    self.partial_ptrs = [arr(*[int(p) for p in h.buffer_ptrs]) for h in handles]
    self.flag_ptrs = arr(*[int(p) for p in fh.buffer_ptrs])
    self.launches = torch.zeros(self.MAX_CTAS, dtype=torch.int32, device=device)
    # the in-place all-reduce of many rows has its own marks: ready per CTA, done per rank
    self.reduce_flags = symm.empty(((self.MAX_CTAS + 1) * world,), dtype=torch.int32, device=device)
    self.reduce_flags.zero_()
    rh = symm.rendezvous(self.reduce_flags, group)
    self._keep.append(rh)
    self.reduce_flag_ptrs = arr(*[int(p) for p in rh.buffer_ptrs])
    self.reduce_launches = torch.zeros(self.MAX_CTAS + 2, dtype=torch.int32, device=device)
    self.turn = 0
    self.wait_cycles = 0           # 0: the library's default budget for the hand-shake
    torch.cuda.synchronize(device)
    dist.barrier(group=group)      # every rank's flags are zero before anyone raises one

  @classmethod
  def open(cls, group, rank, world, capacity, device):
    """Returns the exchange, or None where symmetric memory cannot be set up (the caller then
    keeps the NCCL all-reduce)."""
    import torch.distributed as dist
    import warnings
    ex, why = None, None
    try:
      ex = cls(group, rank, world, capacity, device)
    except Exception as e:   # noqa: BLE001 -- any failure here means: no peer path
      why = repr(e)
    # The ranks must agree on the path: one rank on NCCL while the others spin in the peer
    # hand-shake would stall all of them.  Every rank reaches this reduction.
    ok = torch.tensor([1 if ex is not None else 0], dtype=torch.int32, device=device)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
    if int(ok.item()) == 0:
      if ex is not None:
        why = 'another rank could not set it up'
      warnings.warn(f'peer-memory exchange unavailable, using NCCL all-reduce: {why}')
      return None
    return ex

  def reserve(self, shape) -> tuple[int, torch.Tensor]:
    """The buffer whose turn it is, viewed as `shape`: the place where this rank's next
    partial output belongs (a projection writes it there directly, or `publish` copies)."""
    n = 1
    for d in shape:
      n *= d
    if n > self.capacity:
      raise ValueError('partial does not fit the exchange buffers')
    which = self.turn
    self.turn ^= 1
    return which, self.partials[which][:n].view(tuple(shape))

  def publish(self, y: torch.Tensor) -> 'PeerPartial':
    """Copies this rank's partial output into the buffer whose turn it is."""
    if y.dtype != torch.bfloat16:
      raise ValueError('partial does not fit the exchange buffers')
    which, view = self.reserve(y.shape)
    view.copy_(y)
    return PeerPartial(self, which, view)


class PeerPartial:
  """This rank's partial output of a row-parallel projection, published for its peers; the
  sum over ranks is formed by whoever consumes it (AddRmsNorm, or `all_reduce`)."""

  def __init__(self, exchange: PeerExchange, which: int, local: torch.Tensor):
    self.exchange, self.which, self.local = exchange, which, local
    self.shape = tuple(local.shape)

  def all_reduce(self, comm) -> torch.Tensor:
    """The plain tensor, through the group's NCCL all-reduce (a collective all ranks make)."""
    return comm.all_reduce_sum(self.local.clone())

  def reduce_in_place(self) -> torch.Tensor:
    """All ranks' partials summed into every rank's buffer by the ranks themselves (each sums
    a share of the rows and writes the sums to all peers): the reduced tensor, a view of the
    exchange buffer.  A collective: every rank calls it for the same partial."""
    ex = self.exchange
    d = self.shape[-1]
    rows = self.local.numel() // d
    _lib.check(_lib.lib().qwx_peer_allreduce(
        ex.partial_ptrs[self.which], ex.reduce_flag_ptrs, ex.world, ex.rank,
        _lib.ptr(ex.reduce_launches), ex.MAX_CTAS, rows, d, _lib.ptr(_lib.error_flag(ex.device)),
        ex.wait_cycles, _lib.stream_ptr(ex.device)), 'peer_allreduce')
    return self.local


class AddRmsNorm(LazyAct):
  """RMSNorm(x + delta) * weight; after it has been consumed, `.residual` is bf16(x + delta)
  (x itself when delta is None)."""

  # From this many rows on, peer partials are all-reduced in place before the local kernel
  # (every rank moves (world - 1) / world of the tensor each way); below it the kernel reads
  # all ranks' partials itself (one launch, (world - 1) x the tensor inbound: a decode step).
  REDUCE_ROWS = 1024
  # With two ranks both forms move the same bytes over the links and the second launch and the
  # extra pass over local memory only cost (measured: 2 x 2048-token chunks, 295 against 315 ms
  # for the prefill of the 8B decoder): the separate all-reduce is used from three ranks on.
  REDUCE_WORLD = 3

  def __init__(self, x: torch.Tensor, delta, weight: torch.Tensor, eps: float):
    if (isinstance(delta, PeerPartial) and delta.exchange.world >= self.REDUCE_WORLD
        and delta.local.numel() // delta.shape[-1] >= self.REDUCE_ROWS):
      # many rows: the ranks reduce the partials among themselves first (each a share of the
      # rows), then this is the ordinary local kernel on the reduced tensor
      delta = delta.reduce_in_place()
    self.peer = delta if isinstance(delta, PeerPartial) else None
    if self.peer is not None:
      if tuple(delta.shape) != tuple(x.shape):
        raise ValueError('partial and residual shapes differ')
      delta = delta.local
    _lib.require_cuda(x, delta, weight)
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
      raise ValueError('AddRmsNorm takes bfloat16 tensors.')
    self.x = x.contiguous()
    self.delta = None if delta is None else delta.contiguous()
    self.weight, self.eps = weight.contiguous(), float(eps)
    self.shape, self.device = tuple(x.shape), x.device
    self.residual = self.x if delta is None else None

  def _run(self, y, q, scale):
    d = self.shape[-1]
    rows = self.x.numel() // d
    x_out = None
    if self.delta is not None:
      x_out = torch.empty_like(self.x) if self.residual is None else self.residual
    if self.peer is not None:
      if self.residual is not None:
        raise RuntimeError('a peer partial is consumed once: every rank makes the same calls')
      ex = self.peer.exchange
      _lib.check(_lib.lib().qwx_add_rmsnorm_quantize_peer(
          _lib.ptr(self.x), ex.partial_ptrs[self.peer.which], ex.flag_ptrs, ex.world, ex.rank,
          _lib.ptr(ex.launches), ex.MAX_CTAS, _lib.ptr(self.weight), self.eps, rows, d,
          _lib.ptr(x_out), _lib.ptr(y), _lib.ptr(q), _lib.ptr(scale),
          _lib.ptr(_lib.error_flag(self.device)), ex.wait_cycles, _lib.stream_ptr(self.device)),
          'add_rmsnorm_quantize_peer')
      self.residual = x_out
      return
    _lib.check(_lib.lib().qwx_add_rmsnorm_quantize(
        _lib.ptr(self.x), _lib.ptr(self.delta), _lib.ptr(self.weight), self.eps, rows, d,
        _lib.ptr(x_out), _lib.ptr(y), _lib.ptr(q), _lib.ptr(scale),
        _lib.stream_ptr(self.device)), 'add_rmsnorm_quantize')
    if self.delta is not None:
      self.residual = x_out


class SiluMul(LazyAct):
  """silu(gate) * up for gu = [.., 2 f] holding [gate | up]."""

  def __init__(self, gu: torch.Tensor):
    _lib.require_cuda(gu)
    if gu.dtype != torch.bfloat16 or gu.shape[-1] % 16:
      raise ValueError('SiluMul takes a bfloat16 tensor whose last extent is 2 f, f % 8 == 0.')
    self.gu = gu.contiguous()
    self.f = gu.shape[-1] // 2
    self.shape, self.device = tuple(gu.shape[:-1]) + (self.f,), gu.device

  def _run(self, y, q, scale):
    rows = self.gu.numel() // (2 * self.f)
    _lib.check(_lib.lib().qwx_silu_mul_quantize(
        _lib.ptr(self.gu), rows, self.f, _lib.ptr(y), _lib.ptr(q), _lib.ptr(scale),
        _lib.stream_ptr(self.device)), 'silu_mul_quantize')


def rope_cache(qkv: torch.Tensor, hq: int, hkv: int, hd: int, cos: torch.Tensor,
               sin: torch.Tensor, pos, cache_k: torch.Tensor, cache_v: torch.Tensor) -> torch.Tensor:
  """Rotates the q and k heads of qkv [B, T, (hq + 2 hkv) * hd] with the float32 tables
  cos/sin [positions, hd / 2], writes k and v into the cache views [B, hkv, S, hd] at
  positions pos .. pos + T - 1 and returns q as a [B, hq, T, hd] view of token-major storage
  [B, T, hq, hd] (so that an attention kernel that keeps the query's layout hands back
  [B, T, hq * hd] without a transposing copy).  `pos` is an int or a one-element int64 device
  tensor."""
  _lib.require_cuda(qkv, cos, sin, cache_k, cache_v)
  B, T, _ = qkv.shape
  if (cache_k.stride(3) != 1 or cache_k.stride(2) != hd or cache_v.stride() != cache_k.stride()
      or cos.dtype != torch.float32 or not cos.is_contiguous() or not sin.is_contiguous()):
    raise ValueError('rope_cache: unexpected cache or table layout.')
  qkv = qkv.contiguous()
  q = torch.empty((B, T, hq, hd), dtype=qkv.dtype, device=qkv.device)
  pos_dev = pos if isinstance(pos, torch.Tensor) else None
  _lib.check(_lib.lib().qwx_rope_cache(
      _lib.ptr(qkv), B, T, hq, hkv, hd, _lib.ptr(cos), _lib.ptr(sin),
      0 if pos_dev is not None else int(pos), _lib.ptr(pos_dev), _lib.ptr(q), _lib.ptr(cache_k),
      _lib.ptr(cache_v), cache_k.stride(0), cache_k.stride(1), _lib.stream_ptr(qkv.device)),
      'rope_cache')
  return q.transpose(1, 2)


_argmax_ws: dict = {}


def argmax_rows(x: torch.Tensor, index_offset: int = 0, want_values: bool = False):
  """For every row of the bf16 matrix x [rows, cols]: index_offset + the lowest index of its
  largest value (int64 [rows]), and with `want_values` that value (float32 [rows])."""
  _lib.require_cuda(x)
  if x.ndim != 2 or x.dtype != torch.bfloat16:
    raise ValueError('argmax_rows takes a 2-D bfloat16 tensor.')
  x = x.contiguous()
  rows, cols = x.shape
  L = _lib.lib()
  need = L.qwx_argmax_rows_workspace_bytes(rows, cols)
  key = (x.device, torch.cuda.current_stream(x.device).cuda_stream)
  ws = _argmax_ws.get(key)
  if ws is None or ws.numel() < need:
    ws = _argmax_ws[key] = torch.zeros(max(need, 1 << 16), dtype=torch.uint8, device=x.device)
  idx = torch.empty((rows,), dtype=torch.int64, device=x.device)
  val = torch.empty((rows,), dtype=torch.float32, device=x.device) if want_values else None
  _lib.check(L.qwx_argmax_rows(_lib.ptr(x), _lib.BF16, rows, cols, int(index_offset), _lib.ptr(val),
                               _lib.ptr(idx), _lib.ptr(ws), ws.numel(), _lib.stream_ptr(x.device)),
             'argmax_rows')
  return (idx, val) if want_values else idx


def quantized_matmul(x: torch.Tensor, w: QArray, out_dtype=torch.bfloat16,
                     return_act: bool = False):
  """x [M, K] bf16 times a quantized weight [K, N]: the activation is quantized per token
  (absmax, the weight's qtype; boxed_param.py:416-455) and contracted on the tensor cores with
  the scales in the epilogue (dot_general.py:135-261), as one library call.  Bit-identical to
  `dot_general(quantize(x, per token), w)`.  With `return_act` the QArray of x is returned
  too (views of the call's workspace)."""
  from qwix_b200.core import dot_general as _dg
  from qwix_b200.core import numerics
  if x.ndim != 2 or x.dtype != torch.bfloat16:
    raise ValueError('quantized_matmul expects a 2-D bfloat16 activation.')
  store, code = numerics.storage(w.qtype)
  if code not in (_lib.S8, _lib.E4M3):
    raise NotImplementedError(f'quantized_matmul takes int8 or float8_e4m3fn weights, got {w.qtype}.')
  k, n = w.shape
  if x.shape[1] != k:
    raise ValueError(f'contracting sizes differ: {x.shape[1]} and {k}.')
  if tuple(w.scale.shape) != (1, n) or w.zero_point is not None:
    raise NotImplementedError('the weight must be quantized per output channel, symmetric.')
  _lib.require_cuda(x, w.qvalue)
  x = x.contiguous()
  m = x.shape[0]
  wq = w.qvalue
  if wq.t().is_contiguous() and not wq.is_contiguous():
    codes, layout = wq.t(), _lib.B_NK
  else:
    codes, layout = wq.contiguous(), _lib.B_KN
  if layout == _lib.B_KN and n % 16:
    codes, layout = wq.t().contiguous(), _lib.B_NK
  L = _lib.lib()
  ws = torch.empty(L.qwx_quant_gemm_q8_workspace_bytes(m, k), dtype=torch.uint8, device=x.device)
  out = torch.empty((m, n), dtype=out_dtype, device=x.device)
  err = _lib.error_flag(x.device)
  oc = {torch.bfloat16: _lib.BF16, torch.float32: _lib.F32}[out_dtype]
  epi = _lib.EPI_REFERENCE if _dg.EPILOGUE == 'reference' else _lib.EPI_F32
  _lib.check(L.qwx_quant_gemm_q8(
      _lib.ptr(x), m, k, _lib.ptr(codes), _lib.ptr(w.scale.to(torch.bfloat16).contiguous()), n,
      code, layout, qarray._rounding_code(), _lib.ptr(out), oc, epi, _lib.ptr(ws), ws.numel(),
      _lib.ptr(err), _lib.stream_ptr(x.device)), 'quantized_matmul')
  if not return_act:
    return out
  off = (m * 2 + 255) // 256 * 256
  act = QArray(qvalue=ws[off:off + m * k].view(store).view(m, k),
               scale=ws[:m * 2].view(torch.bfloat16).view(m, 1), zero_point=None,
               qtype=numerics.qtype_name(w.qtype))
  return out, act
