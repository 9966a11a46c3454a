"""Tensor parallelism: the sharding arithmetic on CPU ranks (gloo, world size 2) and, where two GPUs
are present, the real thing over NCCL."""
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

_GLOO_WORKER = r'''
import os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
import oracle
from ter_b200 import synth
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
K, N = 256, 192
t = synth.trits(K, N, 7)
packed = synth.pack_v11(t)                       # [N/4][K]
x, xs = synth.activation(K, 3)
ws = synth.weight_scale(7)
# this rank's column range is one contiguous run of byte-columns of the v11 bytes
n0, n1 = N * rank // world, N * (rank + 1) // world
mine = packed[n0 // 4:n1 // 4]
assert np.array_equal(mine, synth.pack_v11(t[:, n0:n1]))
acc = oracle.gemv_packed_acc(x, mine, K, n1 - n0)
out = torch.from_numpy(oracle.gemv_epilogue(acc, xs, ws))
full = torch.empty(N)
dist.all_gather_into_tensor(full, out)
want = oracle.gemv_epilogue(oracle.gemv_packed_acc(x, packed, K, N), xs, ws)
ok = np.array_equal(full.numpy().view(np.uint32), want.view(np.uint32))
# a rank that holds only its slice of a residual stream reproduces the single-process update
hidden = torch.from_numpy(np.random.default_rng(1).standard_normal(N).astype(np.float32))
upd = hidden.clone()
upd[n0:n1] = hidden[n0:n1] + out
g = torch.empty(N)
dist.all_gather_into_tensor(g, upd[n0:n1].contiguous())
ok = ok and np.array_equal(g.numpy(), hidden.numpy() + want)
flag = torch.tensor([1 if ok else 0]); dist.all_reduce(flag, op=dist.ReduceOp.MIN)
if rank == 0: print("GLOO_OK" if int(flag) == 1 else "GLOO_FAIL")
dist.destroy_process_group()
'''


def test_sharding_arithmetic_on_two_cpu_ranks(tmp_path):
    w = tmp_path / "w.py"
    w.write_text(_GLOO_WORKER)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29617", str(w), ROOT],
                       capture_output=True, text=True, timeout=300)
    assert "GLOO_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


@pytest.mark.gpu
@pytest.mark.parametrize("p2p,shard", [(1, 3), (0, 3), (1, 0), (1, 2)])
def test_tensor_parallel_decode_matches_checker(p2p, shard):
    """p2p=1: slices exchanged by the peer-memory kernel; p2p=0: NCCL all-gathers.  shard: which blocks are
    column-sharded (bit 0 attention, bit 1 FFN; the lm_head always is)."""
    import torch
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs two GPUs")
    world = 2
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", TER_TP_P2P=str(p2p), TER_TP_SHARD=str(shard))
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
                        "--master-addr", "127.0.0.1", "--master-port", str(29618 + p2p + 2 * shard),
                        os.path.join(ROOT, "tests", "tp_worker.py")], capture_output=True, text=True, timeout=900, env=env)
    assert "TP_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
