"""GPU: the w8a8 decoder (Llama-3-8B architecture, cut down to two layers) against a
NumPy oracle decoder, decode steps against prefill, and tensor-parallel against single-GPU."""

import os
import socket
import subprocess
import sys

import numpy as np
import pytest
import torch

import qwix_b200 as qwix
from qwix_b200 import decoder as D
from oracle import decoder as DO
from tests import helpers as h

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _full_weights(model: D.Decoder):
  """Unsharded bf16 weights of a TP=1 model as NumPy, quantized for the oracle."""
  out = {'embed': h.to_numpy(model.embed.data), 'layers': []}
  for blk in model.layers:
    out['layers'].append({
        'qkv': DO.quantize_weight(h.to_numpy(blk.attn.qkv.kernel.data)),
        'o': DO.quantize_weight(h.to_numpy(blk.attn.o.kernel.data)),
        'gate_up': DO.quantize_weight(h.to_numpy(blk.ffn.gate_up.kernel.data)),
        'down': DO.quantize_weight(h.to_numpy(blk.ffn.down.kernel.data)),
    })
  out['lm_head'] = DO.quantize_weight(h.to_numpy(model.lm_head.kernel.data))
  return out


def test_tiny_decoder_matches_oracle_and_decode_matches_prefill():
  cfg = D.DecoderConfig.tiny()
  model = D.Decoder(cfg, device='cuda')
  weights = _full_weights(model)
  model.quantize_weights()
  for i, blk in enumerate(model.layers):   # offline PTQ gives the oracle's codes bit for bit
    assert h.codes_equal(blk.attn.qkv.kernel.array.qvalue, weights['layers'][i]['qkv'].qvalue)
    assert h.codes_equal(blk.ffn.down.kernel.array.qvalue, weights['layers'][i]['down'].qvalue)
  ptq_model = qwix.quantize_model(model, qwix.PtqProvider(D.w8a8_rules()))
  B, T = 2, 32
  tokens = torch.randint(0, cfg.vocab, (B, T), generator=torch.Generator().manual_seed(0)).cuda()
  model.alloc_cache(B, T + 8)
  with torch.no_grad():
    got = ptq_model(tokens, 0, 0, last_only=False).cpu().numpy()
  want = DO.forward(cfg, weights, tokens.cpu().numpy())
  rel = np.linalg.norm(got - want) / np.linalg.norm(want)
  assert rel < 3e-2, rel
  assert (got.argmax(-1) == want.argmax(-1)).mean() > 0.9

  # Decode: feeding token t at position t against the cache reproduces the prefill logits.
  with torch.no_grad():
    ptq_model(tokens[:, :T - 1], 0, 0)
    step = ptq_model(tokens[:, T - 1:], T - 1, 0).cpu().numpy()
  rel = np.linalg.norm(step[:, 0] - got[:, -1]) / np.linalg.norm(got[:, -1])
  assert rel < 3e-2, rel

  ids = D.generate(ptq_model, tokens, steps=6, prefill_batch=1, use_graph=False)
  assert ids.shape == (B, 6) and int(ids.max()) < cfg.vocab
  # the first generated token is the argmax of the prefill's last position
  assert torch.equal(ids[:, 0].cpu(), torch.from_numpy(got[:, -1].argmax(-1)))
  # replaying the captured single-token step gives the same ids as running it eagerly
  replay = D.generate(ptq_model, tokens, steps=6, prefill_batch=1, use_graph=True)
  assert torch.equal(ids, replay)


def test_attention_core_as_quantized_einsums():
  """`attention_core='einsum'`: scores and weighted sum are einsums a rule can match, so under
  the `.*` w8a8 rule q, k, the probabilities and v are quantized per token
  (boxed_param.py:149-157, 216-224).  Without a provider the same code is float attention."""
  import dataclasses
  cfg = dataclasses.replace(D.DecoderConfig.tiny(), attention_core='einsum')
  model = D.Decoder(cfg, device='cuda')
  weights = _full_weights(model)
  B, T = 2, 32
  tokens = torch.randint(0, cfg.vocab, (B, T), generator=torch.Generator().manual_seed(1)).cuda()
  model.alloc_cache(B, T + 8)
  # float: the einsum core agrees with the library's fused attention
  sdpa = D.Decoder(dataclasses.replace(cfg, attention_core='sdpa'), device='cuda')
  sdpa.load_state_dict(model.state_dict())
  sdpa.alloc_cache(B, T + 8)
  with torch.no_grad():
    a = model(tokens, 0, 0, last_only=False).float()
    b = sdpa(tokens, 0, 0, last_only=False).float()
  assert (a - b).norm() / b.norm() < 2e-2
  # quantized: against the oracle decoder with the same switch
  model.quantize_weights()
  ptq_model = qwix.quantize_model(model, qwix.PtqProvider(D.w8a8_rules()))
  with torch.no_grad():
    got = ptq_model(tokens, 0, 0, last_only=False).cpu().numpy()
  want = DO.forward(cfg, weights, tokens.cpu().numpy(), quantized_attention=True)
  rel = np.linalg.norm(got - want) / np.linalg.norm(want)
  assert rel < 3e-2, rel
  assert (got.argmax(-1) == want.argmax(-1)).mean() > 0.9
  plain = DO.forward(cfg, weights, tokens.cpu().numpy())
  assert np.linalg.norm(want - plain) / np.linalg.norm(plain) > 1e-4     # the switch does change the arithmetic
  # decode steps run eagerly with this core and stay consistent with the prefill
  with torch.no_grad():
    ptq_model(tokens[:, :T - 1], 0, 0)
    step = ptq_model(tokens[:, T - 1:], T - 1, 0).cpu().numpy()
  assert np.linalg.norm(step[:, 0] - got[:, -1]) / np.linalg.norm(got[:, -1]) < 5e-2
  ids = D.generate(ptq_model, tokens, steps=4, prefill_batch=1)
  assert ids.shape == (B, 4)
  assert torch.equal(ids[:, 0].cpu(), torch.from_numpy(got[:, -1].argmax(-1)))


TP_WORKER = '''
import os, sys, json
sys.path.insert(0, os.environ["REPO_ROOT"])
import torch, torch.distributed as dist
rank = int(os.environ["LOCAL_RANK"])
torch.cuda.set_device(rank)
os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
import qwix_b200 as qwix
from qwix_b200 import decoder as D
cfg = D.DecoderConfig.tiny()
tokens = torch.randint(0, cfg.vocab, (2, 24), generator=torch.Generator().manual_seed(0)).cuda()
from qwix_b200 import _lib
def run(group, exact):
  m = D.Decoder(cfg, device="cuda", group=group, exact_act_scale=exact)
  m.quantize_weights()
  m.alloc_cache(2, 32)
  if group is None and not exact:
    # the default mode must really take the peer-memory path, not the NCCL fall-back
    assert m.comm.exchange is not None, "peer exchange was not set up"
  q = qwix.quantize_model(m, qwix.PtqProvider(D.w8a8_rules()))
  with torch.no_grad():
    out = q(tokens, 0, 0, last_only=False)
  _lib.raise_on_device_error()     # no hand-shake between the ranks ran out
  return out
solo = dist.new_group([rank]) if False else None
# TP=1 reference on every rank: a one-rank group
groups = [dist.new_group([r]) for r in range(dist.get_world_size())]
ref = run(groups[rank], False)
res = {}
for exact in (True, False):
  out = run(None, exact)
  res["exact" if exact else "local"] = float((out - ref).norm() / ref.norm())
  res["max_" + ("exact" if exact else "local")] = float((out - ref).abs().max())
if rank == 0:
  print(json.dumps(res))
dist.barrier()
dist.destroy_process_group()
'''


def _free_port():
  with socket.socket() as s:
    s.bind(('127.0.0.1', 0))
    return s.getsockname()[1]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason='needs two GPUs')
def test_tensor_parallel_matches_single_gpu(tmp_path):
  script = tmp_path / 'tp_worker.py'
  script.write_text(TP_WORKER)
  env = dict(os.environ, REPO_ROOT=ROOT)
  cmd = [sys.executable, '-m', 'torch.distributed.run', '--nnodes=1', '--nproc-per-node=2',
         '--master-addr', '127.0.0.1', '--master-port', str(_free_port()), str(script)]
  out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
  assert out.returncode == 0, out.stderr[-3000:]
  import json
  res = json.loads([l for l in out.stdout.splitlines() if l.startswith('{')][-1])
  # global activation scales + float32 partial sums reproduce the single-GPU model up to
  # float32 summation order; per-shard scales are a (finer) different quantization
  assert res['exact'] < 1e-2 and res['local'] < 4e-2, res
