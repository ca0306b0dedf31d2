"""Llama-shaped decoder whose projections run through the quantized path, tensor-parallel.

This is the decoder workload of the benchmark (Llama-3-8B shape): every Dense of the decoder is issued through
qwix_b200.ops, so under `quantize_model(model, PtqProvider(w8a8 rule))` each projection is a
per-token int8 activation quantization plus one int8 tcgen05 GEMM with the scales fused in its
epilogue.  Everything that is not a contraction with a weight (RMSNorm, RoPE, the attention
core, sampling) is ordinary tensor code; the attention core is the library's fused
scaled-dot-product kernel, which -- like a fused attention primitive under the reference's
interception -- is not a quantized op.

Tensor parallelism (one process per GPU): q/k/v and gate/up are column-parallel (heads and
FFN columns split across ranks), o_proj and down_proj are row-parallel and followed by one
all-reduce (NCCL over NVLink through torch.distributed).  Weights are quantized per output
channel from the full matrix and then sliced, so a rank's codes and scales are exactly the
slices of the single-GPU model's (what sharding propagation gives the reference under GSPMD,
utils/flax_util.py:320-426).
"""

from __future__ import annotations

import dataclasses
import math

import torch
import torch.nn.functional as F

import qwix_b200 as qwix
from qwix_b200 import _lib
from qwix_b200 import fused
from qwix_b200 import nn
from qwix_b200 import ops
from qwix_b200.core import qarray
from qwix_b200.providers import ptq


@dataclasses.dataclass(frozen=True)
class DecoderConfig:
  layers: int = 32
  d_model: int = 4096
  q_heads: int = 32
  kv_heads: int = 8
  head_dim: int = 128
  ffn: int = 14336
  vocab: int = 128256
  rope_theta: float = 500000.0
  norm_eps: float = 1e-5
  dtype: torch.dtype = torch.bfloat16
  # 'sdpa': the library's fused attention on bf16 q / k / v.  'einsum': scores and the weighted
  # sum as two einsums issued through qwix_b200.ops, so that a rule which matches them
  # quantizes the attention core too -- both operands are activations, as in the reference
  # (boxed_param.py:149-157, 216-224).  Eager steps only: generate() does not graph this form.
  attention_core: str = 'sdpa'

  @staticmethod
  def llama3_8b() -> 'DecoderConfig':
    return DecoderConfig()

  @staticmethod
  def tiny() -> 'DecoderConfig':
    """Two layers, same structure: the cut-down used for oracle parity."""
    return DecoderConfig(layers=2, d_model=512, q_heads=8, kv_heads=2, head_dim=64, ffn=1024,
                         vocab=1024)


class _Comm:
  """The tensor-parallel group: rank, size and the two collectives the path needs."""

  def __init__(self, group=None):
    import torch.distributed as dist
    self.dist = dist if (dist.is_available() and dist.is_initialized()) else None
    self.group = group
    self.size = self.dist.get_world_size(group) if self.dist else 1
    self.rank = self.dist.get_rank(group) if self.dist else 0
    self.exchange = None      # fused.PeerExchange once opened
    self.peer_active = False  # set while the fused layer loop runs

  def open_exchange(self, capacity: int, device):
    """Collective: maps every rank's partial-sum buffers into every other rank (symmetric
    memory over NVLink), so that the consumer of a row-parallel projection can add the ranks'
    partials itself.  Leaves `exchange` None where that is not possible."""
    if self.size > 1 and self.exchange is None and torch.device(device).type == 'cuda':
      group = self.group if self.group is not None else self.dist.group.WORLD
      self.exchange = fused.PeerExchange.open(group, self.rank, self.size, capacity, device)
    elif self.exchange is not None and self.exchange.capacity < capacity:
      raise ValueError('exchange buffers are smaller than this call needs')

  def all_reduce_sum(self, x: torch.Tensor) -> torch.Tensor:
    if self.size > 1:
      self.dist.all_reduce(x, op=self.dist.ReduceOp.SUM, group=self.group)
    return x

  def all_reduce_max(self, x: torch.Tensor) -> torch.Tensor:
    if self.size > 1:
      self.dist.all_reduce(x, op=self.dist.ReduceOp.MAX, group=self.group)
    return x

  def all_gather_last(self, x: torch.Tensor) -> torch.Tensor:
    if self.size == 1:
      return x
    parts = [torch.empty_like(x) for _ in range(self.size)]
    self.dist.all_gather(parts, x.contiguous(), group=self.group)
    return torch.cat(parts, dim=-1)


def _normal(shape, seed: int, device, dtype, std=0.02) -> torch.Tensor:
  g = torch.Generator(device=device).manual_seed(seed)
  return (torch.randn(shape, generator=g, device=device, dtype=torch.float32) * std).to(dtype)


class RMSNorm(torch.nn.Module):

  def __init__(self, d: int, eps: float, dtype, device):
    super().__init__()
    self.scale = torch.nn.Parameter(torch.ones(d, dtype=dtype, device=device), requires_grad=False)
    self.eps = eps

  def forward(self, x):
    v = x.float()
    v = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + self.eps)
    return (v * self.scale.float()).to(x.dtype)


class RowParallelDense(nn.Dense):
  """Dense whose input features are sharded: y = all_reduce(x_shard @ kernel_shard).

  exact_act_scale: quantize the activation with the absmax of the whole (unsharded) row, which
  takes one extra max all-reduce of a [tokens] vector -- the collective that dynamic
  calibration over a sharded contraction axis needs in the reference
  (docs/source/basics.md:83-86).  Otherwise every shard scales its own slice, which is
  sub-channel quantization with tile K / ranks."""

  def __init__(self, *a, comm: _Comm, exact_act_scale: bool, **k):
    super().__init__(*a, **k)
    self.comm = comm
    self.exact_act_scale = exact_act_scale

  def forward(self, x):
    dn = (((x.ndim - 1,), (0,)), ((), ()))
    rule = qwix.get_current_rule('dot_general')
    kernel = self.kernel
    if (self.exact_act_scale and self.comm.size > 1 and rule is not None
        and rule.act_qtype is not None and isinstance(kernel, ptq.WithAux)):
      if isinstance(x, fused.LazyAct):
        x = x.materialize()
      how = qarray.HowToQuantize(qtype=rule.act_qtype, channelwise_axes=list(range(x.ndim - 1)),
                                 calibration_method=rule.act_calibration_method or 'absmax')
      cal = qarray.calibrate(x, how)
      cal = {k: self.comm.all_reduce_max(v) for k, v in cal.items()}
      scale, zp = qarray.compute_scale_zero_point(cal, how.qtype)
      xq = qarray.quantize_with_scale_zero_point(x, how.qtype, scale, zp)
      from qwix_b200.core import dot_general as dg
      # float32 partial products, summed across ranks before the one rounding to the model
      # dtype: the nearest a sharded contraction gets to the unsharded result
      y = dg.dot_general(xq, kernel.array, dn, preferred_element_type=torch.float32)
      return self.comm.all_reduce_sum(y).to(x.dtype)
    ex = self.comm.exchange
    out_shape = tuple(x.shape[:-1]) + (kernel.shape[-1],)
    numel = math.prod(out_shape)
    if (self.comm.peer_active and ex is not None and x.dtype == torch.bfloat16
        and numel <= ex.capacity):
      # Leave the partial where the peers can read it (the next add + norm kernel sums the
      # ranks): the GEMM is offered the exchange buffer as its output, so nothing is copied.
      from qwix_b200.core import dot_general as dg
      which, view = ex.reserve(out_shape)
      with dg.output_into(view):
        y = ops.dot_general(x, kernel, dn)
      if y.data_ptr() != view.data_ptr():      # the contraction took another path: copy
        view.copy_(y)
      return fused.PeerPartial(ex, which, view)
    y = ops.dot_general(x, kernel, dn)
    return self.comm.all_reduce_sum(y)


class Attention(torch.nn.Module):

  def __init__(self, cfg: DecoderConfig, comm: _Comm, layer: int, device, exact: bool):
    super().__init__()
    t = comm.size
    assert cfg.q_heads % t == 0 and cfg.kv_heads % t == 0
    self.cfg, self.comm = cfg, comm
    self.hq, self.hkv = cfg.q_heads // t, cfg.kv_heads // t
    d, hd = cfg.d_model, cfg.head_dim
    # One fused column-parallel projection [d, (hq + 2 hkv) * hd] per rank.
    self.qkv = nn.Dense(d, (self.hq + 2 * self.hkv) * hd, use_bias=False, dtype=cfg.dtype,
                        device=device)
    self.o = RowParallelDense(self.hq * hd, d, use_bias=False, dtype=cfg.dtype, device=device,
                              comm=comm, exact_act_scale=exact)
    self.layer = layer

  def forward(self, x, cos, sin, cache_k, cache_v, pos, mask=None):
    B, T, _ = x.shape
    hd = self.cfg.head_dim
    qkv = self.qkv(x)
    if isinstance(x, fused.LazyAct):
      # cos / sin are the whole tables here: the kernel indexes them by position, rotates q
      # and k and writes k and v straight into the cache
      q = fused.rope_cache(qkv, self.hq, self.hkv, hd, cos, sin, pos, cache_k, cache_v)
      if self.cfg.attention_core == 'einsum':
        if isinstance(pos, torch.Tensor):
          m = mask if mask is not None else _key_mask(cache_k.shape[2], pos, q.dtype)
          out = _einsum_attention(q, cache_k, cache_v, m)
        else:
          out = _einsum_attention(q, cache_k[:, :, :pos + T], cache_v[:, :, :pos + T],
                                  _causal_mask(T, pos + T, q.device))
      elif isinstance(pos, torch.Tensor):
        if mask is None:
          mask = _key_mask(cache_k.shape[2], pos, q.dtype)
        out = F.scaled_dot_product_attention(q, cache_k, cache_v, attn_mask=mask, enable_gqa=True)
      else:
        out = F.scaled_dot_product_attention(q, cache_k[:, :, :pos + T], cache_v[:, :, :pos + T],
                                             is_causal=pos == 0, enable_gqa=True)
      return self.o(out.transpose(1, 2).reshape(B, T, self.hq * hd))
    q, k, v = qkv.split([self.hq * hd, self.hkv * hd, self.hkv * hd], dim=-1)
    q = q.view(B, T, self.hq, hd).transpose(1, 2)
    k = k.view(B, T, self.hkv, hd).transpose(1, 2)
    v = v.view(B, T, self.hkv, hd).transpose(1, 2)
    q, k = _rope(q, cos, sin), _rope(k, cos, sin)
    if isinstance(pos, torch.Tensor):
      # One new token at a position held on the device (the form a CUDA graph can replay):
      # write it into the cache by index and mask the keys that lie beyond it.
      cache_k.index_copy_(2, pos, k)
      cache_v.index_copy_(2, pos, v)
      if mask is None:
        mask = _key_mask(cache_k.shape[2], pos, q.dtype)
      if self.cfg.attention_core == 'einsum':
        out = _einsum_attention(q, cache_k, cache_v, mask)
      else:
        out = F.scaled_dot_product_attention(q, cache_k, cache_v, attn_mask=mask, enable_gqa=True)
      out = out.transpose(1, 2).reshape(B, T, self.hq * hd)
      return self.o(out)
    cache_k[:, :, pos:pos + T] = k
    cache_v[:, :, pos:pos + T] = v
    if self.cfg.attention_core == 'einsum':
      out = _einsum_attention(q, cache_k[:, :, :pos + T], cache_v[:, :, :pos + T],
                              _causal_mask(T, pos + T, q.device))
    elif pos == 0:
      out = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
    else:
      out = F.scaled_dot_product_attention(q, cache_k[:, :, :pos + T], cache_v[:, :, :pos + T],
                                           is_causal=False, enable_gqa=True)
    out = out.transpose(1, 2).reshape(B, T, self.hq * hd)
    return self.o(out)


def _einsum_attention(q, k, v, mask):
  """softmax(q k^T / sqrt(hd) + mask) v with the two contractions as interceptable einsums.
  q [B, hq, T, hd]; k, v [B, hkv, S, hd]; mask additive, broadcastable to [B, hq, T, S]."""
  from qwix_b200 import ops
  rep = q.shape[1] // k.shape[1]
  if rep > 1:
    k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
  pad = (-k.shape[2]) % 16
  if pad:
    # the tensor-core contraction over the keys wants a multiple of 16: zero keys behind a
    # -inf mask change neither the probabilities nor any scale
    if mask is None:
      mask = torch.zeros((1, 1, 1, k.shape[2]), device=q.device)
    k, v = F.pad(k, (0, 0, 0, pad)), F.pad(v, (0, 0, 0, pad))
    mask = F.pad(mask.float(), (0, pad), value=float('-inf'))
  s = ops.einsum('bnth,bnsh->bnts', q.contiguous(), k.contiguous()).float() * (q.shape[-1] ** -0.5)
  if mask is not None:
    s = s + mask.float()
  p = torch.softmax(s, dim=-1).to(q.dtype)
  return ops.einsum('bnts,bnsh->bnth', p, v.contiguous())


def _causal_mask(T: int, S: int, device) -> torch.Tensor:
  """Additive mask of a block of T queries that ends at key S - 1."""
  i = torch.arange(T, device=device).view(T, 1) + (S - T)
  j = torch.arange(S, device=device).view(1, S)
  return torch.zeros((T, S), device=device).masked_fill_(j > i, float('-inf'))


def _key_mask(length: int, pos: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
  """Keys a single-token step at device-held position `pos` may attend to, [1, 1, 1, length],
  as the additive mask (0 / -inf, in the dtype of the queries) that the attention call would
  otherwise derive from a boolean one at every layer."""
  beyond = (torch.arange(length, device=pos.device) > pos).view(1, 1, 1, -1)
  return torch.zeros(beyond.shape, dtype=dtype, device=pos.device).masked_fill_(
      beyond, float('-inf'))


def _rope(x, cos, sin):
  half = x.shape[-1] // 2
  x1, x2 = x[..., :half].float(), x[..., half:].float()
  return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).to(x.dtype)


class FeedForward(torch.nn.Module):

  def __init__(self, cfg: DecoderConfig, comm: _Comm, device, exact: bool):
    super().__init__()
    assert cfg.ffn % comm.size == 0
    self.local = cfg.ffn // comm.size
    self.gate_up = nn.Dense(cfg.d_model, 2 * self.local, use_bias=False, dtype=cfg.dtype,
                            device=device)
    self.down = RowParallelDense(self.local, cfg.d_model, use_bias=False, dtype=cfg.dtype,
                                 device=device, comm=comm, exact_act_scale=exact)

  def forward(self, x):
    gu = self.gate_up(x)
    if isinstance(x, fused.LazyAct):
      return self.down(fused.SiluMul(gu))
    g, u = gu.split(self.local, dim=-1)
    return self.down(F.silu(g) * u)


class Block(torch.nn.Module):

  def __init__(self, cfg, comm, layer, device, exact):
    super().__init__()
    self.attn_norm = RMSNorm(cfg.d_model, cfg.norm_eps, cfg.dtype, device)
    self.attn = Attention(cfg, comm, layer, device, exact)
    self.ffn_norm = RMSNorm(cfg.d_model, cfg.norm_eps, cfg.dtype, device)
    self.ffn = FeedForward(cfg, comm, device, exact)

  def forward(self, x, cos, sin, ck, cv, pos, mask=None):
    x = x + self.attn(self.attn_norm(x), cos, sin, ck, cv, pos, mask)
    return x + self.ffn(self.ffn_norm(x))

  def forward_fused(self, x, delta, cos, sin, ck, cv, pos, mask=None):
    """The same layer with the residual add, the norm and the activation quantization of the
    next projection in one kernel each.  Takes the residual stream x and the not yet added
    output `delta` of the previous layer's MLP; returns the new pair."""
    a = fused.AddRmsNorm(x, delta, self.attn_norm.scale, self.attn_norm.eps)
    attn_out = self.attn(a, cos, sin, ck, cv, pos, mask)
    f = fused.AddRmsNorm(a.residual, attn_out, self.ffn_norm.scale, self.ffn_norm.eps)
    ffn_out = self.ffn(f)
    return f.residual, ffn_out


class Decoder(torch.nn.Module):
  """Random-init decoder of the given shape, sharded for this rank of the TP group.

  Weights come from per-tensor seeds and are generated as the full matrix then sliced, so all
  TP degrees hold slices of the same model."""

  def __init__(self, cfg: DecoderConfig, device='cuda', group=None, exact_act_scale: bool = False,
               seed: int = 0):
    super().__init__()
    self.cfg = cfg
    self.comm = _Comm(group)
    self.device = torch.device(device)
    t, r = self.comm.size, self.comm.rank
    assert cfg.vocab % t == 0
    self.embed = torch.nn.Parameter(_normal((cfg.vocab, cfg.d_model), seed + 1, self.device,
                                            cfg.dtype), requires_grad=False)
    self.layers = torch.nn.ModuleList(
        [Block(cfg, self.comm, i, self.device, exact_act_scale) for i in range(cfg.layers)])
    self.final_norm = RMSNorm(cfg.d_model, cfg.norm_eps, cfg.dtype, self.device)
    self.lm_head = nn.Dense(cfg.d_model, cfg.vocab // t, use_bias=False, dtype=cfg.dtype,
                            device=self.device)
    self._init_weights(seed, t, r)
    self.cache = None
    self.fuse = True   # fused element-wise kernels on CUDA bf16 tensors (same arithmetic)
    # Under tensor parallelism, fold the all-reduce of the row-parallel projections into the
    # add + norm kernel that consumes them (peer loads over NVLink) instead of calling NCCL.
    self.peer_exchange = not exact_act_scale
    self.prefill_rows = 4 * 2048   # tokens per prefill chunk the exchange buffers are sized for

  # -- weights ---------------------------------------------------------------------------

  def _full(self, shape, seed):
    return _normal(shape, seed, self.device, self.cfg.dtype)

  def _init_weights(self, seed, t, r):
    cfg, hd = self.cfg, self.cfg.head_dim
    hq, hkv, fl = cfg.q_heads // t, cfg.kv_heads // t, cfg.ffn // t
    for i, blk in enumerate(self.layers):
      s = seed + 100 * (i + 1)
      wq = self._full((cfg.d_model, cfg.q_heads * hd), s + 1)[:, r * hq * hd:(r + 1) * hq * hd]
      wk = self._full((cfg.d_model, cfg.kv_heads * hd), s + 2)[:, r * hkv * hd:(r + 1) * hkv * hd]
      wv = self._full((cfg.d_model, cfg.kv_heads * hd), s + 3)[:, r * hkv * hd:(r + 1) * hkv * hd]
      blk.attn.qkv.kernel.data = torch.cat([wq, wk, wv], dim=1).contiguous()
      blk.attn.o.kernel.data = self._full((cfg.q_heads * hd, cfg.d_model), s + 4)[
          r * hq * hd:(r + 1) * hq * hd].contiguous()
      wg = self._full((cfg.d_model, cfg.ffn), s + 5)[:, r * fl:(r + 1) * fl]
      wu = self._full((cfg.d_model, cfg.ffn), s + 6)[:, r * fl:(r + 1) * fl]
      blk.ffn.gate_up.kernel.data = torch.cat([wg, wu], dim=1).contiguous()
      blk.ffn.down.kernel.data = self._full((cfg.ffn, cfg.d_model), s + 7)[
          r * fl:(r + 1) * fl].contiguous()
    vl = cfg.vocab // t
    self.lm_head.kernel.data = self._full((cfg.d_model, cfg.vocab), seed + 2)[
        :, r * vl:(r + 1) * vl].contiguous()

  def quantize_weights(self, qtype='int8'):
    """Offline PTQ of every projection (the role of quantize_params): per output channel,
    computed on the full matrix so that row-parallel shards share the unsharded scales."""
    t, r = self.comm.size, self.comm.rank
    how = qarray.HowToQuantize(qtype=qtype, channelwise_axes=[1])

    def box(mod, full_rows=None):
      w = mod.kernel.data
      if full_rows is None or t == 1:
        qa = qarray.quantize(w, how)
      else:
        # row-parallel: scale from the absmax over all ranks' rows of each column
        cal = qarray.calibrate(w, how)
        cal = {k: self.comm.all_reduce_max(v) for k, v in cal.items()}
        scale, _ = qarray.compute_scale_zero_point(cal, qtype)
        qa = qarray.quantize_with_scale_zero_point(w, qtype, scale, None)
      # Store the codes [N, K] (K contiguous): the layout the decode-step kernel streams; the
      # logical [K, N] qvalue is its transposed view and the prefill kernels take either order.
      qa = qarray.QArray(qvalue=qa.qvalue.t().contiguous().t(), scale=qa.scale,
                         zero_point=qa.zero_point, qtype=qa.qtype)
      del mod._parameters['kernel']
      mod.kernel = ptq.WithAux(qa, how)

    for blk in self.layers:
      box(blk.attn.qkv)
      box(blk.attn.o, full_rows=True)
      box(blk.ffn.gate_up)
      box(blk.ffn.down, full_rows=True)
    box(self.lm_head)
    torch.cuda.empty_cache()

  # -- inference -------------------------------------------------------------------------

  def alloc_cache(self, batch: int, max_len: int):
    cfg = self.cfg
    hkv = cfg.kv_heads // self.comm.size
    shape = (cfg.layers, 2, batch, hkv, max_len, cfg.head_dim)
    self.cache = torch.zeros(shape, dtype=cfg.dtype, device=self.device)
    pos = torch.arange(max_len, device=self.device, dtype=torch.float32)
    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.head_dim, 2, device=self.device,
                                                 dtype=torch.float32) / cfg.head_dim))
    ang = pos[:, None] * inv[None, :]
    self.cos, self.sin = ang.cos(), ang.sin()
    if self.peer_exchange and self.comm.size > 1:
      # room for the partial sums of one prefill chunk (prefill_rows tokens) or one decode step
      self.comm.open_exchange(max(self.prefill_rows, batch) * cfg.d_model, self.device)

  def forward(self, tokens: torch.Tensor, pos=0, batch_offset: int = 0,
              last_only: bool = True, local_logits: bool = False) -> torch.Tensor:
    """tokens [B, T] at positions pos..pos+T-1 of sequences batch_offset..batch_offset+B-1.
    `pos` is an int, or for single-token steps a one-element int64 device tensor.
    Returns full-vocabulary logits [B, 1 or T, vocab] (float32), or with `local_logits` this
    rank's vocabulary shard [B, 1 or T, vocab / ranks] in the model dtype."""
    B, T = tokens.shape
    x = self.embed[tokens]
    mask = None
    if isinstance(pos, torch.Tensor):
      assert T == 1
      cos, sin = self.cos.index_select(0, pos), self.sin.index_select(0, pos)
      mask = _key_mask(self.cache.shape[4], pos, x.dtype)   # one per step, shared by the layers
    else:
      cos, sin = self.cos[pos:pos + T], self.sin[pos:pos + T]
    if self.fuse and x.is_cuda and x.dtype == torch.bfloat16:
      delta = None
      self.comm.peer_active = self.comm.exchange is not None
      try:
        for i, blk in enumerate(self.layers):
          ck = self.cache[i, 0, batch_offset:batch_offset + B]
          cv = self.cache[i, 1, batch_offset:batch_offset + B]
          x, delta = blk.forward_fused(x, delta, self.cos, self.sin, ck, cv, pos, mask)
      finally:
        self.comm.peer_active = False
      if isinstance(delta, fused.PeerPartial):   # the last layer's MLP output
        rows = delta.local.numel() // delta.shape[-1]
        delta = (delta.reduce_in_place()
                 if (rows >= fused.AddRmsNorm.REDUCE_ROWS
                     and self.comm.size >= fused.AddRmsNorm.REDUCE_WORLD)
                 else delta.all_reduce(self.comm))
      if last_only:
        x, delta = x[:, -1:], delta[:, -1:]
      x = fused.AddRmsNorm(x, delta, self.final_norm.scale, self.final_norm.eps)
    else:
      for i, blk in enumerate(self.layers):
        ck = self.cache[i, 0, batch_offset:batch_offset + B]
        cv = self.cache[i, 1, batch_offset:batch_offset + B]
        x = blk(x, cos, sin, ck, cv, pos, mask)
      x = self.final_norm(x[:, -1:] if last_only else x)
    logits = self.lm_head(x)
    if local_logits:
      return logits
    return self.comm.all_gather_last(logits).float()

  def greedy_ids(self, tokens: torch.Tensor, pos=0, batch_offset: int = 0) -> torch.Tensor:
    """The argmax token of the last position, [B]: every rank takes the argmax of its own
    vocabulary shard and the ranks exchange one (value, index) pair per sequence, instead of
    gathering and widening [B, vocab] logits.  Ties go to the lowest index, as a global argmax
    would have it."""
    local = self.forward(tokens, pos, batch_offset, local_logits=True)[:, -1]     # [B, vocab / t]
    if local.is_cuda and local.dtype == torch.bfloat16:
      if self.comm.size == 1:
        return fused.argmax_rows(local)
      idx, val = fused.argmax_rows(local, self.comm.rank * local.shape[-1], want_values=True)
      pair = torch.stack([val, idx.float()], dim=-1)
    else:
      val, idx = local.max(dim=-1)
      if self.comm.size == 1:
        return idx
      pair = torch.stack([val.float(), (idx + self.comm.rank * local.shape[-1]).float()], dim=-1)
    parts = torch.empty((self.comm.size,) + tuple(pair.shape), dtype=pair.dtype, device=pair.device)
    self.comm.dist.all_gather_into_tensor(parts, pair.contiguous(), group=self.comm.group)
    best = parts[..., 0].argmax(dim=0)                # first maximum: the lowest rank, lowest ids
    return parts[..., 1].gather(0, best[None])[0].long()


def w8a8_rules():
  return [qwix.QuantizationRule(module_path='.*', weight_qtype='int8', act_qtype='int8')]


class _StepGraph:
  """The single-token decode step with its static buffers, captured once per batch size."""

  def __init__(self, model, batch: int, device):
    self.tok = torch.zeros((batch, 1), dtype=torch.long, device=device)
    self.pos = torch.zeros((1,), dtype=torch.long, device=device)
    self.model = model
    self.graph = None

  def step(self):
    self.tok.copy_(_greedy(self.model, self.tok, self.pos, 0).view(-1, 1))
    self.pos.add_(1)

  def capture(self):
    torch.cuda.synchronize()
    self.graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(self.graph):   # records the step; it runs only when replayed
      self.step()


def _greedy(model, tokens, pos, batch_offset):
  """Greedy next ids through the (possibly quantized) model: the wrapper's call activates the
  provider, the decoder's `greedy_ids` does the rest."""
  if isinstance(model, qwix.model.QuantizedModel):
    return model(tokens, pos, batch_offset, _method='greedy_ids')
  return model.greedy_ids(tokens, pos, batch_offset)


@torch.no_grad()
def generate(model, tokens: torch.Tensor, steps: int, prefill_batch: int = 4,
             use_graph: bool = True, timings: dict | None = None):
  """Greedy decoding: chunked prefill of [B, T] prompts, then `steps` tokens per sequence.
  `model` is a Decoder or its quantized wrapper.  The single-token step is launch-bound
  (hundreds of small kernels), so it is captured in a CUDA graph (once per batch size, after
  one eager step that warms every kernel up) and replayed.  Returns the ids [B, steps];
  `timings`, if given, receives the device time of the two phases in ms."""
  dec = model.model if isinstance(model, qwix.model.QuantizedModel) else model
  if dec.cfg.attention_core == 'einsum':
    use_graph = False      # the einsum core allocates per (batch, head) call: eager steps
  B, T = tokens.shape
  if dec.cache is None or dec.cache.shape[2] < B or dec.cache.shape[4] < T + steps:
    dec.alloc_cache(B, T + steps)
    dec._step_graphs = {}
  ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
  ev[0].record()
  nxt = torch.empty((B,), dtype=torch.long, device=tokens.device)
  for b0 in range(0, B, prefill_batch):
    nxt[b0:b0 + prefill_batch] = _greedy(model, tokens[b0:b0 + prefill_batch], 0, b0)
  ev[1].record()
  out = torch.empty((B, steps), dtype=torch.long, device=tokens.device)
  out[:, 0] = nxt
  graphs = dec.__dict__.setdefault('_step_graphs', {})
  runner = graphs.get(B)
  if runner is None:
    runner = graphs[B] = _StepGraph(model, B, tokens.device)
  runner.tok.copy_(nxt.view(B, 1))
  runner.pos.fill_(T)
  for s in range(1, steps):
    if not use_graph:
      runner.step()
    elif runner.graph is None:
      runner.step()            # eager once, then record for all later steps and calls
      out[:, s] = runner.tok[:, 0]
      runner.capture()
      continue
    else:
      runner.graph.replay()
    out[:, s] = runner.tok[:, 0]
  ev[2].record()
  if timings is not None:
    torch.cuda.synchronize()
    timings['prefill_ms'] = ev[0].elapsed_time(ev[1])
    timings['decode_ms'] = ev[1].elapsed_time(ev[2])
  # A bounded wait inside a kernel (tensor-core pipeline, peer hand-shake) that ran out leaves
  # its outputs unwritten: the ids would be garbage, so fail loudly instead.
  _lib.raise_on_device_error(tokens.device)
  return out
