"""Oracle decoder: a NumPy restatement of a Llama-shaped decoder under a w8a8 PTQ rule.

Test infrastructure only (parity tests and the timed CPU baseline).  Every projection goes
through the oracle's per-token quantize + dot_general, i.e. what BoxedParamProvider.dot_general
does for a rule with act_qtype set (qwix/_src/providers/boxed_param.py:109-171, 416-455;
qwix/_src/core/dot_general.py:135-261); everything else (RMSNorm, RoPE, attention, SwiGLU) is
model code outside qwix, computed in float32 and rounded to bf16 where the model holds bf16
tensors."""

import ml_dtypes
import numpy as np

from oracle import dot_general as odg
from oracle import einsum as oe
from oracle import qarray as oq

bf16 = ml_dtypes.bfloat16
DN2 = lambda nd: (((nd - 1,), (0,)), ((), ()))


def _dense(x, wq):
  dn = DN2(x.ndim)
  how = odg.get_how_to_quantize(dimension_numbers=dn, ndims=(x.ndim, 2), for_lhs=True,
                                tile_size=None, qtype='int8')
  return odg.dot_general(oq.quantize(x, how), wq, dn)


def _rms(x, eps):
  v = x.astype(np.float32)
  v = v / np.sqrt((v * v).mean(-1, keepdims=True) + eps)
  return v.astype(bf16)


def _rope(x, cos, sin):
  half = x.shape[-1] // 2
  x1, x2 = x[..., :half].astype(np.float32), x[..., half:].astype(np.float32)
  return np.concatenate([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1).astype(bf16)


def _act_einsum(einsum_str, a, b):
  """An einsum of two activations under a rule with act_qtype set: both operands are quantized
  per call (qwix/_src/providers/boxed_param.py:204-235)."""
  how = lambda for_lhs: oe.get_how_to_quantize(einsum_str=einsum_str, ndims=(a.ndim, b.ndim),
                                               for_lhs=for_lhs, tile_size=None, qtype='int8')
  return oe.einsum(einsum_str, oq.quantize(a, how(True)), oq.quantize(b, how(False)))


def quantize_weight(w):
  return oq.quantize(w, oq.HowToQuantize(qtype='int8', channelwise_axes=[1]))


def forward(cfg, weights, tokens, quantized_attention: bool = False):
  """weights: dict of bf16 NumPy arrays named like the torch model's full (unsharded) matrices.
  tokens [B, T].  Returns float32 logits [B, T, vocab] of a causal prefill.
  `quantized_attention`: the attention core as two intercepted einsums (scores and weighted
  sum), both operands quantized per token, instead of float32 arithmetic."""
  B, T = tokens.shape
  hd, hq, hkv = cfg.head_dim, cfg.q_heads, cfg.kv_heads
  x = weights['embed'][tokens]
  pos = np.arange(T, dtype=np.float32)
  inv = 1.0 / (cfg.rope_theta ** (np.arange(0, hd, 2, dtype=np.float32) / hd))
  ang = pos[:, None] * inv[None, :]
  cos, sin = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
  mask = np.triu(np.full((T, T), -np.inf, np.float32), 1)
  for i in range(cfg.layers):
    w = weights['layers'][i]
    h = _rms(x, cfg.norm_eps)
    qkv = _dense(h, w['qkv'])
    q, k, v = np.split(qkv, [hq * hd, (hq + hkv) * hd], axis=-1)
    q = _rope(q.reshape(B, T, hq, hd).transpose(0, 2, 1, 3), cos, sin)
    k = _rope(k.reshape(B, T, hkv, hd).transpose(0, 2, 1, 3), cos, sin)
    v = v.reshape(B, T, hkv, hd).transpose(0, 2, 1, 3)
    rep = hq // hkv
    if quantized_attention:
      kr, vr = np.repeat(k, rep, axis=1), np.repeat(v, rep, axis=1)
      s = _act_einsum('bnth,bnsh->bnts', q, kr).astype(np.float32) * np.float32(hd ** -0.5) + mask
      p = np.exp(s - s.max(-1, keepdims=True))
      p = (p / p.sum(-1, keepdims=True)).astype(bf16)
      att = _act_einsum('bnts,bnsh->bnth', p, vr).astype(bf16)
      att = att.transpose(0, 2, 1, 3).reshape(B, T, hq * hd)
    else:
      kf = np.repeat(k.astype(np.float32), rep, axis=1)
      vf = np.repeat(v.astype(np.float32), rep, axis=1)
      s = q.astype(np.float32) @ kf.transpose(0, 1, 3, 2) / np.sqrt(hd) + mask
      p = np.exp(s - s.max(-1, keepdims=True))
      p = p / p.sum(-1, keepdims=True)
      att = (p @ vf).astype(bf16).transpose(0, 2, 1, 3).reshape(B, T, hq * hd)
    x = (x.astype(np.float32) + _dense(att, w['o']).astype(np.float32)).astype(bf16)
    h = _rms(x, cfg.norm_eps)
    gu = _dense(h, w['gate_up']).astype(np.float32)
    g, u = np.split(gu, 2, axis=-1)
    g, u = g.astype(bf16).astype(np.float32), u.astype(bf16).astype(np.float32)
    act = ((g / (1.0 + np.exp(-g))).astype(bf16).astype(np.float32) * u).astype(bf16)
    x = (x.astype(np.float32) + _dense(act, w['down']).astype(np.float32)).astype(bf16)
  h = _rms(x, cfg.norm_eps)
  return _dense(h, weights['lm_head']).astype(np.float32)
