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
