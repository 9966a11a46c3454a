"""Worker of the tensor-parallel test: run with torch.distributed.run, one rank per GPU.
Every rank builds the same synthetic model (the library keeps its own column slice), generates
greedy tokens with the output slices exchanged inside the captured step (peer-memory kernel, or NCCL
all-gathers with TER_TP_P2P=0), and rank 0
checks tokens and final logits against the CPU checker (which knows nothing about sharding)."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import modelutil  # noqa: E402
from ter_b200 import TerB200  # noqa: E402


def main():
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    rank, world = dist.get_rank(), dist.get_world_size()
    tb = TerB200(local)
    tb.comm_init_from_torch()
    tb.set_option("tp_shard", int(os.environ.get("TER_TP_SHARD", "3")))   # bit 0: attention block sharded, bit 1: FFN block
    tb.set_option("tp_p2p", int(os.environ.get("TER_TP_P2P", "1")))   # 1: peer-memory exchange kernel, 0: NCCL all-gathers
    ok = True
    cases = [
        (dict(arch=0, H=256, F=512, L=3, V=4096, Nh=4, Nkv=2, Hd=64, Smax=320, eps=1e-5, rope_theta=500000.0), 11, 260, 12),
        (dict(arch=1, H=512, F=768, L=2, V=4096, Nh=4, Nkv=2, Hd=128, Smax=64, eps=1e-5, rope_theta=500000.0), 12, 5, 20),
        (dict(arch=0, H=256, F=512, L=2, V=4096, Nh=4, Nkv=2, Hd=64, Smax=64, eps=1e-5, rope_theta=500000.0,
              lm_head_packed=1), 13, 4, 16),
    ]
    for cfg, seed, n_prompt, n_gen in cases:
        modelutil.build_gpu(tb, cfg, seed)
        prompt = np.random.default_rng(seed).integers(0, cfg["V"], size=n_prompt).astype(np.int32)
        out = tb.generate(prompt, n_gen)
        lg = tb.model_logits()[0]
        if rank == 0:
            om = modelutil.build_oracle(cfg, seed)
            want, wl = modelutil.oracle_generate(om, prompt, n_gen, want_logits=True)
            ok = ok and out[0].tolist() == want.tolist() and np.array_equal(lg.view(np.uint32), wl[-1].view(np.uint32))
        # every rank must hold the same tokens
        t = torch.from_numpy(out[0].astype(np.int64)).cuda()
        ref = t.clone()
        dist.broadcast(ref, 0)
        ok = ok and bool(torch.equal(t, ref))
        ok = ok and tb.device_status() == 0
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("TP_OK" if int(flag.item()) == 1 else "TP_FAIL", "world", world, "p2p", os.environ.get("TER_TP_P2P", "1"), "shard", os.environ.get("TER_TP_SHARD", "3"),
              flush=True)
    tb.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
