"""CPU: the multi-rank plumbing of the benchmark (token sharding, barrier, max-over-ranks
timing, whole-job throughput) with two gloo ranks."""

import os
import socket
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent('''
    import os, sys, json
    sys.path.insert(0, os.environ['REPO_ROOT'])
    import torch, torch.distributed as dist
    import bench
    dist.init_process_group('gloo')
    rank, world = dist.get_rank(), dist.get_world_size()
    # every rank owns its own token shard: seeds differ per rank, shapes agree
    shard = bench.token_shard(rank, world, tokens_per_rank=4)
    gathered = [None] * world
    dist.all_gather_object(gathered, shard)
    assert sorted(sum(gathered, [])) == list(range(4 * world)), gathered
    # timing: the job time is the slowest rank's time
    ms = bench.max_over_ranks(10.0 + 5.0 * rank, dist, device='cpu')
    value = bench.whole_job_tops(ms_per_step=ms, world=world)
    if rank == 0:
      print(json.dumps({'ms': ms, 'value': value, 'world': world}))
    dist.destroy_process_group()
''')


def _free_port():
  with socket.socket() as s:
    s.bind(('127.0.0.1', 0))
    return s.getsockname()[1]


def test_two_gloo_ranks(tmp_path):
  script = tmp_path / 'worker.py'
  script.write_text(WORKER)
  env = dict(os.environ, REPO_ROOT=ROOT)
  cmd = [sys.executable, '-m', 'torch.distributed.run', '--nnodes=1', '--nproc-per-node=2',
         '--master-addr', '127.0.0.1', '--master-port', str(_free_port()), str(script)]
  out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=240)
  assert out.returncode == 0, out.stderr[-2000:]
  import json
  line = [l for l in out.stdout.splitlines() if l.startswith('{')][-1]
  res = json.loads(line)
  assert res['world'] == 2 and res['ms'] == 15.0
  import bench
  assert abs(res['value'] - 2 * bench.OPS_PER_STEP / 15e-3 / 1e12) < 1e-6


# ---- the decoder's tensor-parallel partitioning, two gloo ranks on CPU ---------------------------

TP_WORKER = textwrap.dedent('''
    import os, sys, json, dataclasses
    sys.path.insert(0, os.environ['REPO_ROOT'])
    import torch, torch.distributed as dist
    dist.init_process_group('gloo')
    rank, world = dist.get_rank(), dist.get_world_size()
    from qwix_b200 import decoder as D
    cfg = dataclasses.replace(D.DecoderConfig.tiny(), dtype=torch.float32)
    solo = [dist.new_group([r]) for r in range(world)][rank]     # a one-rank group: TP = 1
    full = D.Decoder(cfg, device='cpu', group=solo)
    part = D.Decoder(cfg, device='cpu')                          # sharded over the two ranks
    assert part.comm.size == world and full.comm.size == 1
    hd, t = cfg.head_dim, world
    hq, hkv, fl, vl = cfg.q_heads // t, cfg.kv_heads // t, cfg.ffn // t, cfg.vocab // t
    checks = 0
    for fb, pb in zip(full.layers, part.layers):
      # column-parallel: this rank's output columns of q, k, v / gate, up
      fq, fk, fv = fb.attn.qkv.kernel.split([cfg.q_heads * hd, cfg.kv_heads * hd, cfg.kv_heads * hd], dim=1)
      want = torch.cat([fq[:, rank * hq * hd:(rank + 1) * hq * hd],
                        fk[:, rank * hkv * hd:(rank + 1) * hkv * hd],
                        fv[:, rank * hkv * hd:(rank + 1) * hkv * hd]], dim=1)
      assert torch.equal(pb.attn.qkv.kernel, want)
      fg, fu = fb.ffn.gate_up.kernel.split(cfg.ffn, dim=1)
      assert torch.equal(pb.ffn.gate_up.kernel,
                         torch.cat([fg[:, rank * fl:(rank + 1) * fl], fu[:, rank * fl:(rank + 1) * fl]], dim=1))
      # row-parallel: this rank's input rows of o_proj / down_proj
      assert torch.equal(pb.attn.o.kernel, fb.attn.o.kernel[rank * hq * hd:(rank + 1) * hq * hd])
      assert torch.equal(pb.ffn.down.kernel, fb.ffn.down.kernel[rank * fl:(rank + 1) * fl])
      # the ranks' row slices put together are the whole matrix, each row once
      rows = [None] * world
      dist.all_gather_object(rows, pb.ffn.down.kernel)
      assert torch.equal(torch.cat(rows, dim=0), fb.ffn.down.kernel)
      # partial products summed over the ranks equal the unsharded product
      x = torch.randn(5, cfg.ffn, generator=torch.Generator().manual_seed(7))
      partial = x[:, rank * fl:(rank + 1) * fl] @ pb.ffn.down.kernel
      dist.all_reduce(partial)
      assert torch.allclose(partial, x @ fb.ffn.down.kernel, rtol=1e-4, atol=1e-5)
      checks += 1
    assert torch.equal(part.lm_head.kernel, full.lm_head.kernel[:, rank * vl:(rank + 1) * vl])
    # the whole forward pass (unquantized): the sharded model computes the same logits
    tokens = torch.randint(0, cfg.vocab, (2, 12), generator=torch.Generator().manual_seed(0))
    full.alloc_cache(2, 16); part.alloc_cache(2, 16)
    with torch.no_grad():
      a = full(tokens, 0, 0, last_only=False)
      b = part(tokens, 0, 0, last_only=False)
    err = float((a - b).abs().max() / a.abs().max())
    assert a.shape == (2, 12, cfg.vocab) and err < 1e-4, err
    # the KV cache is sharded by heads
    assert part.cache.shape[3] == cfg.kv_heads // world
    if rank == 0:
      print(json.dumps({'layers_checked': checks, 'logit_err': err}))
    dist.destroy_process_group()
''')


def _run_two_ranks(tmp_path, source, timeout=300):
  script = tmp_path / 'worker.py'
  script.write_text(source)
  env = dict(os.environ, REPO_ROOT=ROOT)
  cmd = [sys.executable, '-m', 'torch.distributed.run', '--nnodes=1', '--nproc-per-node=2',
         '--master-addr', '127.0.0.1', '--master-port', str(_free_port()), str(script)]
  out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)
  assert out.returncode == 0, out.stderr[-3000:]
  import json
  return json.loads([l for l in out.stdout.splitlines() if l.startswith('{')][-1])


def test_decoder_partitioning_two_gloo_ranks(tmp_path):
  res = _run_two_ranks(tmp_path, TP_WORKER)
  assert res['layers_checked'] == 2 and res['logit_err'] < 1e-4


# ---- failure detection on the host: a rank that never joins a collective -------------------------

ABSENT_WORKER = textwrap.dedent('''
    import os, sys, json, time, datetime, dataclasses
    sys.path.insert(0, os.environ['REPO_ROOT'])
    import torch, torch.distributed as dist
    dist.init_process_group('gloo', timeout=datetime.timedelta(seconds=3))
    rank = dist.get_rank()
    from qwix_b200 import decoder as D
    cfg = dataclasses.replace(D.DecoderConfig.tiny(), dtype=torch.float32, layers=1)
    model = D.Decoder(cfg, device='cpu')
    model.alloc_cache(1, 8)
    tokens = torch.zeros((1, 4), dtype=torch.long)
    with torch.no_grad():
      model(tokens, 0, 0)                      # a healthy step on both ranks
    dist.barrier()
    verdict = None
    if rank == 0:
      t0 = time.time()
      try:
        with torch.no_grad():
          model(tokens, 0, 0)                  # rank 1 skips this step
        verdict = 'no error'
      except Exception as e:                   # the group's timeout ends the all-reduce
        verdict = 'reported'
      print(json.dumps({'verdict': verdict, 'seconds': time.time() - t0}), flush=True)
    else:
      time.sleep(8)                            # alive, but absent from the step
    os._exit(0)                                # the group is broken: no orderly teardown
''')


def test_absent_rank_is_reported_by_the_group_timeout(tmp_path):
  res = _run_two_ranks(tmp_path, ABSENT_WORKER)
  assert res['verdict'] == 'reported' and res['seconds'] < 8
