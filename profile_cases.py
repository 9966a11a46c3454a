"""Small, self-contained workloads for profiling one kernel at a time:

    python profile_cases.py gemv_stream      # 2048 x 513024 GEMV (263 MB of trits), 4 launches
    python profile_cases.py sweep            # Llama-1B fabric (113 matrices, 309 MB) as one sweep-plan launch, 8 launches
    python profile_cases.py gemm             # BitNet gate 2560 x 6912 GEMM at M = 16, 256, 1024
    python profile_cases.py decode llama     # three decode steps at position ~300 (or: bitnet, position ~2100)
    python profile_cases.py decode bitnet 64 # the same for a batch of 64 sequences
    python profile_cases.py glue             # the glue kernels alone: RMSNorm + int8 quantiser (64 rows x 2560), batched
                                             # attention (24 sequences x 5 KV heads x 2048 positions, 126 MB of K/V),
                                             # bf16 lm_head for 1 row (CUDA cores) and 64 rows (tensor cores), 657 MB table
    python profile_cases.py attn 64          # attention of 64 sequences at context 2048 (335 MB of K/V): tensor-core and
                                             # fixed-order kernels, 4 launches each, CUDA-event times printed

    python profile_cases.py trace_gemm       # with a library built by `TER_B200_NVCC_EXTRA=-DTERB_TRACE python -m
    python profile_cases.py trace_decode bitnet 2100   # ter_b200.build --force`: phase timestamps (globaltimer) of the
                                             # GEMM's CTAs / of one layer inside the persistent decode kernel

Each holds at most a few GB on the device and finishes in seconds, so an `ncu` capture of it ends by itself.
"""
from __future__ import annotations

import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def build_random_model(tb, cfg, dev, max_batch=1, seed=1):
    """Random-init ternarised model generated on the device (weights never visit the host)."""
    import torch
    from ter_b200 import FMT_V11, synth
    tb.model_create(cfg, max_batch=max_batch)
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    emb = (torch.randn((cfg["V"], cfg["H"]), generator=g, device=dev) * 0.02).to(torch.bfloat16)
    tb.model_set_embd(emb.view(torch.int16))
    tb.model_set_vector(-1, 0, np.ones(cfg["H"], np.float32))
    shapes = synth.model_shapes(cfg)
    for L in range(cfg["L"]):
        for wi, nm in enumerate(synth.MAT_ORDER):
            K, N = shapes[nm]
            tb.model_set_matrix(L, wi, synth.packed_v11_cuda(K, N, seed * 1000 + L * 7 + wi, dev), FMT_V11, 0.02)
        for vi in range(4 if cfg["arch"] == 1 else 2):
            n = cfg["F"] if vi == 3 else cfg["H"]
            tb.model_set_vector(L, vi, np.ones(n, np.float32))


def gemv_stream():
    import torch
    from ter_b200 import FMT_V11, TerB200, synth
    tb = TerB200(0)
    dev = torch.device("cuda:0")
    K, N = 2048, 128256 * 4
    tb.install("big", synth.packed_v11_cuda(K, N, 1, dev), FMT_V11, K, N, 0.03)
    x, xs = synth.activation(K, 4)
    xd = torch.from_numpy(x).cuda()
    sd = torch.tensor([xs], device=dev)
    out = torch.empty(N, device=dev)
    for _ in range(3):
        tb.gemv("big", xd, sd, out)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    tb.gemv("big", xd, sd, out)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    print(f"gemv {K}x{N}: {ms * 1e3:.1f} us  {K * N // 4 / ms / 1e6:.0f} GB/s  status {tb.device_status()}")


def sweep():
    import torch
    from ter_b200 import FMT_V11, TerB200, synth
    tb = TerB200(0)
    dev = torch.device("cuda:0")
    names, xs, ss, outs, nbytes = [], [], [], [], 0
    acts = {}
    for K in (2048, 8192):
        x, sc = synth.activation(K, K)
        acts[K] = (torch.from_numpy(x).cuda(), torch.tensor([sc], device=dev))
    mats = [(f"L{L}.{nm}", *synth.LLAMA_1B_SHAPES[nm]) for L in range(16) for nm in synth.MAT_ORDER]
    mats.append(("lm_head", *synth.LLAMA_1B_SHAPES["lm_head"]))
    for i, (nm, K, N) in enumerate(mats):
        tb.install(nm, synth.packed_v11_cuda(K, N, i + 1, dev), FMT_V11, K, N, 0.03)
        names.append(nm)
        xs.append(acts[K][0])
        ss.append(acts[K][1])
        outs.append(torch.empty(N, device=dev))
        nbytes += K * N // 4
    plan = tb.gemv_plan(names, xs, ss, outs)
    cur = torch.cuda.current_stream()
    for _ in range(3):
        tb.gemv_plan_launch(plan, stream=cur)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(4):
        tb.gemv_plan_launch(plan, stream=cur)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / 4
    print(f"sweep of {len(mats)} matrices, {nbytes / 1e6:.1f} MB: {ms * 1e3:.1f} us  {nbytes / ms / 1e6:.0f} GB/s  "
          f"status {tb.device_status()}")


def gemm():
    import torch
    from ter_b200 import FMT_V11, TerB200, synth
    tb = TerB200(0)
    dev = torch.device("cuda:0")
    K, N = synth.BITNET_2B_SHAPES["gate"]
    tb.install("gate", synth.packed_v11_cuda(K, N, 3, dev), FMT_V11, K, N, 0.02)
    for M in (16, 256, 1024):
        X = torch.randint(-127, 128, (M, K), dtype=torch.int8, device=dev)
        xs = torch.rand(M, device=dev) * 0.05
        out = torch.empty((M, N), device=dev)
        for _ in range(2):
            tb.gemm("gate", X, xs, out)
        torch.cuda.synchronize()
    print("gemm ok, status", tb.device_status())


def decode(which="llama", batch="1"):
    import torch
    from ter_b200 import TerB200, synth
    batch = int(batch)
    base, smax, pos0 = (synth.LLAMA_1B_CFG, 512, 300) if which == "llama" else (synth.BITNET_2B_CFG, 2304, 2100)
    tb = TerB200(0)
    dev = torch.device("cuda:0")
    cfg = dict(base, Smax=smax)
    build_random_model(tb, cfg, dev, max_batch=batch)
    tb.model_reset(batch)
    tok = [5 + b for b in range(batch)]
    for i in range(3):
        tok = [int(t) for t in tb.decode_step(tok, [pos0 + i] * batch)]
    torch.cuda.synchronize()
    print("decode ok", which, "batch", batch, tok[0], tb.device_status())


def glue():
    import torch
    from ter_b200 import TerB200
    tb = TerB200(0)
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev)
    g.manual_seed(3)
    # RMSNorm + absmax int8 quantiser, 64 rows of the BitNet hidden size
    x = torch.randn((64, 2560), generator=g, device=dev)
    gamma = torch.ones(2560, device=dev)
    for _ in range(3):
        tb.rmsnorm_quant(x, gamma, 1e-5)
    # batched attention: 24 sequences, 20 query / 5 KV heads of 128, context 2048 (the batch-64 decode kernel)
    B, Nh, Nkv, Hd, Smax = 24, 20, 5, 128, 2048
    q = torch.randn((B, Nh * Hd), generator=g, device=dev)
    kc = torch.randn((B, Nkv, Smax, Hd), generator=g, device=dev).to(torch.bfloat16)
    vc = torch.randn((B, Nkv, Smax, Hd), generator=g, device=dev).to(torch.bfloat16)
    pos = torch.full((B,), Smax - 1, dtype=torch.int32, device=dev)
    for _ in range(3):
        tb.attention(q, kc, vc, pos, Nh, Nkv, Hd, Smax)
    del kc, vc
    # bf16 lm_head: one row on the CUDA cores, 64 rows on the tensor cores
    table = (torch.randn((128256, 2560), generator=g, device=dev) * 0.02).to(torch.bfloat16).view(torch.int16)
    x1 = torch.randn((1, 2560), generator=g, device=dev)
    x64 = torch.randn((64, 2560), generator=g, device=dev)
    for _ in range(3):
        tb.lm_head_bf16(table, x1)
    for _ in range(3):
        tb.lm_head_bf16_tc(table, x64)
    torch.cuda.synchronize()
    print("glue ok, status", tb.device_status())


def attn(batch="64"):
    """Attention of a token batch alone: `batch` sequences, 20 query / 5 KV heads of 128, context 2048, on the
    tensor cores and in the fixed-order form; CUDA-event times of both are printed."""
    import torch
    from ter_b200 import TerB200
    tb = TerB200(0)
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev)
    g.manual_seed(5)
    B, Nh, Nkv, Hd, Smax = int(batch), 20, 5, 128, 2048
    q = torch.randn((B, Nh * Hd), generator=g, device=dev)
    kc = torch.randn((B, Nkv, Smax, Hd), generator=g, device=dev).to(torch.bfloat16)
    vc = torch.randn((B, Nkv, Smax, Hd), generator=g, device=dev).to(torch.bfloat16)
    pos = torch.full((B,), Smax - 1, dtype=torch.int32, device=dev)
    for mode, name in ((1, "tensor cores"), (0, "fixed order")):
        tb.set_option("attn_mma_min", mode)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        for i in range(4):
            if i == 1:
                ev[0].record()
            tb.attention(q, kc, vc, pos, Nh, Nkv, Hd, Smax)
        ev[1].record()
        torch.cuda.synchronize()
        us = ev[0].elapsed_time(ev[1]) / 3 * 1e3
        tb.set_option("attn_mma_min", 0)
        print(f"attention {name}: {us:.1f} us per call, {2 * kc.numel() * 2 / us / 1e6:.2f} TB/s of K/V")
    print("attn ok, status", tb.device_status())


def trace_gemm():
    """Phase timestamps of the GEMM's CTAs (library built with -DTERB_TRACE): microseconds from the first CTA's
    entry to: tensor memory allocated, griddepcontrol.wait passed, first stage full, last MMA issued, accumulators
    complete, epilogue done, exit (minimum / median / maximum over the CTAs of the last launch)."""
    import ctypes
    import torch
    from ter_b200 import FMT_V11, TerB200, synth
    tb = TerB200(0)
    if not hasattr(tb.L, "ter_b200_debug_gemm_trace"):
        raise SystemExit("build the library with TER_B200_NVCC_EXTRA=-DTERB_TRACE first")
    dev = torch.device("cuda:0")
    names = ["entry", "tmem", "pdl", "first_full", "mma_issued", "done", "epi_end", "end"]
    for nm, M in (("q", 1024), ("gate", 1024), ("gate", 64)):
        K, N = synth.BITNET_2B_SHAPES[nm]
        tb.install("g", synth.packed_v11_cuda(K, N, 5, dev), FMT_V11, K, N, 0.02)
        X = torch.randint(-127, 128, (M, K), dtype=torch.int8, device=dev)
        xs = torch.rand(M, device=dev) * 0.05 + 0.001
        out = torch.empty((M, N), device=dev)
        for _ in range(3):
            tb.gemm("g", X, xs, out)
        torch.cuda.synchronize()
        buf = np.zeros((512, 8), np.uint64)
        tb.L.ter_b200_debug_gemm_trace(buf.ctypes.data_as(ctypes.c_void_p))
        t = buf.astype(np.int64)
        t = t[t[:, 0] > 0]
        rel = (t - t[:, 0].min()) / 1e3
        print(nm, "M", M, "CTAs", len(t))
        for k in range(8):
            print(f"  {names[k]:10s} min {rel[:, k].min():7.2f} med {np.median(rel[:, k]):7.2f} max {rel[:, k].max():7.2f}")
        tb.remove("g")
    tb.close()


def trace_decode(which="llama", n_prompt="300"):
    """Timestamps of layer 1 inside the persistent decode kernel (library built with -DTERB_TRACE): per CTA the
    stage boundaries (microseconds from the first CTA's entry into the layer) and, for CTAs with an attention item,
    its phases (start, q staged, K landed, scores, softmax, output, merged)."""
    import ctypes
    import torch
    from ter_b200 import TerB200, synth
    tb = TerB200(0)
    if not hasattr(tb.L, "ter_b200_debug_trace"):
        raise SystemExit("build the library with TER_B200_NVCC_EXTRA=-DTERB_TRACE first")
    dev = torch.device("cuda:0")
    n_prompt = int(n_prompt)
    base = synth.LLAMA_1B_CFG if which == "llama" else synth.BITNET_2B_CFG
    cfg = dict(base, Smax=n_prompt + 40)
    build_random_model(tb, cfg, dev)
    prompt = np.random.default_rng(1).integers(0, cfg["V"], size=n_prompt).astype(np.int32)
    tb.generate(prompt, 16)
    tb.generate(prompt, 16)
    print(which, "ms per step", (tb.last_generate_ms() - tb.last_prompt_ms()) / 15)
    buf = np.zeros((148, 32), np.uint64)
    tb.L.ter_b200_debug_trace(buf.ctypes.data_as(ctypes.c_void_p))
    t = buf.astype(np.int64)
    rel = np.where(t > 0, (t - t[:, 0].min()) / 1000.0, -1)
    np.set_printoptions(linewidth=250, precision=2, suppress=True)
    for c in (0, 50, 100, 127, 140, 147):
        print(c, "stages", rel[c, :20])
        print(c, "  attention", rel[c, 20:28])
    tb.close()


if __name__ == "__main__":
    case = sys.argv[1] if len(sys.argv) > 1 else "gemv_stream"
    {"gemv_stream": gemv_stream, "sweep": sweep, "gemm": gemm, "decode": lambda: decode(*sys.argv[2:4]), "glue": glue,
     "attn": lambda: attn(*sys.argv[2:3]), "trace_gemm": trace_gemm,
     "trace_decode": lambda: trace_decode(*sys.argv[2:4])}[case]()
