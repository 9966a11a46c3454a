#!/usr/bin/env python3
"""Benchmark of the packed-trit GEMV fabric (the reference's headline kernel metric:
packed-trit GEMV GB/s, weights-only bytes K*N/4, cuda/ter_cuda_forward_packed_v12.cu:457).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one M=1 pass over every projection of the Llama-3.2-1B architecture: 16 layers x
{q,k,v,o,gate,up,down} + the packed lm_head (K=2048, N=128256): 113 distinct seeded matrices,
309 MB of packed trits (2.4x the 126 MB L2, streamed in the same order each step, so every
weight byte comes from HBM).  At N>1 every rank owns such a shard of an N-times wider fabric
(weak scaling, no data-path collective: output columns are independent).

Prints ONE JSON line (rank 0).  `value` = packed bytes of all ranks / max-over-ranks device
time; `e2e` = the same pass through the host-buffer C-ABI entry point (pinned host x in, fp32
outputs back to pinned host memory, copies inside the timed region).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "packed-trit GEMV HBM GB/s (M=1, Llama-3.2-1B fabric sweep)"
UNIT = "GB/s"
# DRAM bytes of one sweep launch over the full fabric (ncu: 308,983,296 read + 5,458,688 written)
NCU_TRAFFIC_BYTES = 314441984
LAYER_MATS = ["q", "k", "v", "o", "gate", "up", "down"]


def fabric_spec(n_layers=16):
    from ter_b200 import synth
    mats = []
    for L in range(n_layers):
        for nm in LAYER_MATS:
            K, N = synth.LLAMA_1B_SHAPES[nm]
            mats.append((f"L{L}.{nm}", K, N, L, nm))
    K, N = synth.LLAMA_1B_SHAPES["lm_head"]
    mats.append(("lm_head", K, N, -1, "lm_head"))
    return mats


def packed_bytes(mats):
    return sum(K * N // 4 for _, K, N, _, _ in mats)


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:  # noqa: BLE001
            pass
    return 6650.0, "fallback"


class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.p = None
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                       "-lms", "20", "-i", str(gpu_index)], stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:  # noqa: BLE001
            self.p = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.p is None:
            return out
        for _ in range(30):                      # a very short timed region: wait for the first samples
            self.f.flush()
            if os.path.getsize(self.f.name) > 0:
                break
            time.sleep(0.02)
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except Exception:  # noqa: BLE001
            self.p.kill()
        self.f.flush()
        rows = [r.split(",") for r in open(self.f.name).read().strip().splitlines() if r.strip()]
        os.unlink(self.f.name)
        sm, mx, reasons = [], [], set()
        for r in rows:
            try:
                r = [c.strip() for c in r]
                sm.append(float(r[1])); mx.append(float(r[2]))
                for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7),
                                  ("sw_power_cap", 8)):
                    if r[col].lower().startswith("active"):
                        reasons.add(name)
            except Exception:  # noqa: BLE001
                continue
        if sm:
            hot = [s for s in sm if s >= 0.5 * max(sm)]
            out.update(sm_mhz=statistics.median(hot), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return out


def per_shape_bench(tb, dev, peak, reps=20):
    """Packed-trit GEMV GB/s per projection shape (Llama-3.2-1B and BitNet-2B).  A single small matrix
    would sit in the 126 MB L2, so every shape is measured over R distinct device copies (at least
    256 MB in total, at most 512 copies) touched once each per pass, as a decode step touches a layer's
    weights once per token: `sweep` = the R copies as ONE sweep-plan launch, `per_launch` = R separate
    launches in stream order (CUDA-graph replay)."""
    import torch
    from ter_b200 import FMT_V11, synth
    shapes = [("llama-1b", nm, *synth.LLAMA_1B_SHAPES[nm]) for nm in ("q", "k", "gate", "down", "lm_head")]
    shapes += [("bitnet-2b", nm, *synth.BITNET_2B_SHAPES[nm]) for nm in ("q", "k", "gate", "down")]
    rows = []
    cur = torch.cuda.current_stream()
    for model, nm, K, N in shapes:
        nbytes = K * N // 4
        R = max(2, min(512, -(-(256 << 20) // nbytes)))
        seed = synth.seed_for("shape", K, N)
        w = synth.packed_v11_cuda(K, N, seed, dev)
        names = [f"ps{i}" for i in range(R)]
        for n_ in names:
            tb.install(n_, w, FMT_V11, K, N, float(synth.weight_scale(seed)))
        del w
        x, sc = synth.activation(K, synth.seed_for("x", K))
        xd, sd = torch.from_numpy(x).to(dev), torch.tensor([sc], dtype=torch.float32, device=dev)
        outs = [torch.empty(N, dtype=torch.float32, device=dev) for _ in range(R)]
        plan = tb.gemv_plan(names, [xd] * R, [sd] * R, outs)

        def run_single():
            for n_, o in zip(names, outs):
                tb.gemv(n_, xd, sd, o)
        graph = tb.capture(run_single)

        def t(fn):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / reps
        ms_sweep = t(lambda: tb.gemv_plan_launch(plan, stream=cur))
        ms_single = t(lambda: tb.graph_launch(graph, stream=cur))
        sweep_gbs = R * nbytes / (ms_sweep * 1e-3) / 1e9
        rows.append({"model": model, "proj": nm, "K": K, "N": N, "copies": R,
                     "sweep_gbs": round(sweep_gbs, 1), "sweep_frac": round(sweep_gbs / peak, 3),
                     "sweep_frac_of_8tbs_nominal": round(sweep_gbs / 8000.0, 3),
                     "per_launch_gbs": round(R * nbytes / (ms_single * 1e-3) / 1e9, 1),
                     "per_launch_us": round(ms_single * 1e3 / R, 2)})
        tb.gemv_plan_destroy(plan)
        tb.graph_destroy(graph)
        for n_ in names:
            tb.remove(n_)
        del outs
    return rows


def reference_gpu_bench(tb, dev, n_gen=48):
    """The UNMODIFIED reference CUDA decode programs (cuda/ter_cuda_forward_packed.cu and
    cuda/ter_cuda_forward_bitnet.cu, built for sm_100a into oracle/_ref/ by oracle/Makefile) in their
    random-weight bench mode on this GPU: packed-trit lm_head, context limit 64, 4 warm-up positions, then
    n_gen graph-replayed decode steps; and this library on the same terms (same architecture, packed-trit
    lm_head, Smax 64, generation steps at positions 4 .. 4 + n_gen)."""
    import re
    out = []
    for which, exe in (("llama", "ref_forward_packed"), ("bitnet", "ref_forward_bitnet")):
        row = {"arch": "llama-3.2-1b" if which == "llama" else "bitnet-b1.58-2b", "n_gen": n_gen}
        path = os.path.join(ROOT, "oracle", "_ref", exe)
        if os.path.exists(path):
            try:
                r = subprocess.run([path, str(n_gen)], capture_output=True, text=True, timeout=300)
                m = re.search(r"tokens/s\s*:\s*([0-9.]+)", r.stdout)
                row["reference_tokens_per_s"] = float(m.group(1)) if m else None
                if not m:
                    row["reference_error"] = (r.stdout[-200:] + r.stderr[-200:]).strip()
            except Exception as e:  # noqa: BLE001
                row["reference_tokens_per_s"], row["reference_error"] = None, str(e)
        else:
            row["reference_tokens_per_s"], row["reference_error"] = None, "oracle/_ref/" + exe + " not built"
        d = decode_bench(tb, dev, 0, which, n_prompt=4, n_gen=n_gen, smax=64, lm_head_packed=True)
        row["ours_tokens_per_s"] = d["tokens_per_s"]
        if row.get("reference_tokens_per_s"):
            row["ratio"] = d["tokens_per_s"] / row["reference_tokens_per_s"]
        out.append(row)
    return out


def reference_gpu_gemv():
    """The reference's own packed-trit GEMV benchmark (cuda/ter_cuda_forward_packed_v12.cu, unmodified, built
    for sm_100a into oracle/_ref/): kernels v11 and v12 on the five Llama-1B shapes, median of 200 launches on
    one weight buffer per shape (its method: the small shapes stay in L2), GB/s on packed bytes K*N/4."""
    path = os.path.join(ROOT, "oracle", "_ref", "ref_gemv_bench")
    if not os.path.exists(path):
        return {"error": "oracle/_ref/ref_gemv_bench not built"}
    try:
        r = subprocess.run([path], capture_output=True, text=True, timeout=300)
    except Exception as e:  # noqa: BLE001
        return {"error": str(e)}
    rows = []
    for line in r.stdout.splitlines():
        f = line.strip().split(",")
        if len(f) == 5 and f[0] in ("v11", "v12"):
            rows.append({"kernel": f[0], "shape": f[1], "ms": float(f[2]), "gbs": float(f[3])})
    return {"rows": rows} if rows else {"error": (r.stdout[-200:] + r.stderr[-200:]).strip()}


def gemm_bench(tb, dev):
    """Batched ternary GEMM (tcgen05 kind::i8) on the BitNet-2B projection shapes at M = 16, 64, 256, 1024 tokens:
    microseconds per call (CUDA events around graph replays; every launch of a call included) and int8 TOPS =
    2*M*K*N / time.  At M <= 64 the call is bound by the weight bytes, so it is measured over R distinct copies of
    the matrix (at least 256 MB in total, twice the L2) touched once each per pass, and the weight GB/s is
    reported; at M >= 256 one matrix (1-4 MB, L2-resident: the tensor-pipe regime) is called 20 times."""
    import torch
    from ter_b200 import FMT_V11, synth
    rows = []
    cur = torch.cuda.current_stream()
    for nm in ("q", "k", "gate", "down"):
        K, N = synth.BITNET_2B_SHAPES[nm]
        nbytes = K * N // 4
        R = max(2, min(256, -(-(256 << 20) // nbytes)))
        w = synth.packed_v11_cuda(K, N, synth.seed_for("gemm", K, N), dev)
        names = [f"gm{i}" for i in range(R)]
        for n_ in names:
            tb.install(n_, w, FMT_V11, K, N, 0.02)
        del w
        for M in (16, 64, 256, 1024):
            g = torch.Generator(device=dev)
            g.manual_seed(M)
            X = torch.randint(-127, 128, (M, K), dtype=torch.int8, device=dev, generator=g)
            xs = torch.rand(M, device=dev, generator=g) * 0.05 + 0.001
            out = torch.empty((M, N), device=dev)
            use = names if M <= 64 else names[:1] * 20
            for _ in range(3):
                tb.gemm(use[0], X, xs, out)
            torch.cuda.synchronize()
            gid = tb.capture(lambda: [tb.gemm(n_, X, xs, out) for n_ in use])
            tb.graph_launch(gid, stream=cur)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(3):
                tb.graph_launch(gid, stream=cur)
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) / (3 * len(use)) * 1e3
            tb.graph_destroy(gid)
            row = {"proj": nm, "K": K, "N": N, "M": M, "us": round(us, 2), "tops": round(2 * M * K * N / us / 1e6, 1),
                   "weights": f"{len(use)} distinct copies" if M <= 64 else "one matrix, L2-resident"}
            if M <= 64:
                row["weight_gbs"] = round(nbytes / us / 1e3, 1)
            rows.append(row)
        for n_ in names:
            tb.remove(n_)
    return rows


def cpu_reference_run(steps: int, warmup: int, threads: int):
    """Times the reference's CPU GEMV (mm_row, src/tx/forward.cpp:299-352) on the host cores over the SAME
    workload as the GPU arm: one step = one M=1 pass over all 113 matrices of the Llama-3.2-1B fabric (int32
    payloads, as ter::TritTensor holds them).  The reference is single-threaded; the matrices of a pass are
    dealt to `threads` threads (largest first, the lm_head cut into per-thread column blocks), every thread
    calling the unmodified mm_row (oracle/_ref) or, where that was not built, the C restatement."""
    import threading
    import oracle
    from ter_b200 import synth
    kind = "reference" if oracle.Ref.available() else "port"
    units = []                                   # (K, N) pieces of one pass
    for _, K, N, _, nm in fabric_spec(16):
        if nm == "lm_head":
            step = -(-N // threads)
            units += [(K, min(step, N - c0)) for c0 in range(0, N, step)]
        else:
            units.append((K, N))
    units.sort(key=lambda kn: -kn[0] * kn[1])
    load = [0] * threads
    mine = [[] for _ in range(threads)]
    for K, N in units:
        t = load.index(min(load))
        mine[t].append((K, N))
        load[t] += K * N
    ctxs = []
    rng = np.random.default_rng(7)
    for t in range(threads):
        ref = oracle.Ref() if kind == "reference" else None
        items = []
        for (K, N) in mine[t]:
            W = (rng.integers(0, 10, size=(K, N), dtype=np.int8))
            W = ((W >= 7).astype(np.int32) - (W < 3).astype(np.int32))      # P(-1)=0.3, P(0)=0.4, P(+1)=0.3
            x, xs = synth.activation(K, 5)
            if ref:
                items.append((ref.tensor(x.astype(np.int32), float(xs), 1, K), ref.tensor(W, 0.03, K, N), K, N))
            else:
                items.append((x.astype(np.int32), W, K, N))
            del W
        ctxs.append((ref, items))
    bytes_step = sum(K * N // 4 for K, N in units)

    def one_pass(ctx):
        ref, items = ctx
        for a, b, K, N in items:
            if ref:
                ref.mm_row_repeat(a, b, K, N, 1)
            else:
                oracle.mm_row(a, 0.01, b, 0.03)

    def step():
        th = [threading.Thread(target=one_pass, args=(c,)) for c in ctxs]
        for t in th:
            t.start()
        for t in th:
            t.join()

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = time.perf_counter() - t0
    return {"value": bytes_step * steps / dt / 1e9, "unit": UNIT, "cores": threads, "kind": kind,
            "sample": f"the whole fabric pass (113 matrices, {bytes_step / 1e6:.1f} MB packed; int32 payload mm_row) dealt to "
                      f"{threads} threads, {steps} steps, {dt:.1f} s; GB/s counted on packed bytes K*N/4",
            "ms_per_step": dt / steps * 1e3}


def cpu_forward_baseline(n_tokens=3):
    """The reference's CPU decode forward (ter::tx::forward_token, src/tx/transformer.cpp:116-223, unmodified, from
    oracle/_ref) on a synthetic model of the Llama-3.2-1B architecture (BASELINE configs[3]): seconds per token on
    ONE core (the reference is single-threaded), a few tokens at positions >= 27."""
    import oracle
    from ter_b200 import synth
    if not oracle.Ref.available():
        return {"error": "oracle/_ref/libter_ref.so not built"}
    try:
        ref = oracle.Ref()
        t0 = time.perf_counter()
        s_tok, toks = ref.forward_token_seconds(dict(synth.LLAMA_1B_CFG, Smax=64), n_tokens=n_tokens, first_pos=27)
        return {"s_per_token": s_tok, "tokens_per_s": 1.0 / s_tok, "tokens": n_tokens, "cores": 1,
                "host_cores": os.cpu_count(), "kind": "reference",
                "workload": "llama-3.2-1b architecture (16 layers, H 2048, FFN 8192, vocab 128256), random ternary int32 "
                            "payloads, 9-trit tied embedding, batch 1, positions 27.." + str(27 + n_tokens - 1),
                "wall_s_with_model_fill": time.perf_counter() - t0}
    except Exception as e:  # noqa: BLE001
        return {"error": str(e)}


def oracle_tokens(cfg, host_items, prompt, n_tokens):
    """Greedy tokens of the CPU checker (oracle.Model, all host threads) for one sequence: the prompt is fed one
    position at a time, then n_tokens are generated.  host_items: the model's tensors as numpy arrays."""
    import oracle
    om = oracle.Model(cfg)
    for item in host_items:
        if item[0] == "embd":
            om.set_embd(item[1])
        elif item[0] == "vector":
            om.set_vector(item[1], item[2], item[3])
        else:
            om.set_matrix(item[1], item[2], item[3], float(item[4]))
    st = om.new_state(1)
    tok, toks = int(prompt[0]), []
    for pos in range(len(prompt) + n_tokens - 1):
        nxt, _, _ = om.forward(st, 0, tok, pos, want_logits=False)
        if pos + 1 < len(prompt):
            tok = int(prompt[pos + 1])
        else:
            tok = nxt
            toks.append(int(nxt))
    om.close()
    return toks


HOST_BARRIER = None     # set when the job has several ranks: a barrier that waits on the host (gloo)


def decode_bench(tb, dev, rank, which="llama", n_prompt=128, n_gen=256, batch=1, smax=512, warm=True,
                 lm_head_packed=False, check=None):
    """Random-init ternarised decode of one of the two benchmark architectures (tied bf16 lm_head, bf16 KV
    cache): Llama-3.2-1B (16 layers, H 2048, 32/8 heads x 64, FFN 8192 SiLU) or BitNet-b1.58-2B (30 layers,
    H 2560, 20/5 heads x 128, FFN 6912 squared-ReLU with sub-norms), vocab 128256.  n_prompt random prompt
    ids are fed one position at a time (the reference's only method), then n_gen greedy tokens; every step
    is one replay of the captured decode graph."""
    import torch
    from ter_b200 import FMT_V11, synth
    base = synth.LLAMA_1B_CFG if which == "llama" else synth.BITNET_2B_CFG
    cfg = dict(base, Smax=smax, lm_head_packed=1 if lm_head_packed else 0)
    tb.model_create(cfg, max_batch=batch)
    # the CPU checker runs in ONE process of the job (the others would only fight it for the host cores)
    checker = check is not None and int(os.environ.get("RANK", "0")) == 0
    host = [] if checker else None        # the same tensors for the CPU checker (check = (prompt length, tokens))
    if lm_head_packed:   # the reference's bench mode: random packed-trit lm_head instead of the tied table
        seed = synth.seed_for(rank, "dec", which, "lm_head")
        tb.model_set_matrix(-1, 0, synth.packed_v11_cuda(cfg["H"], cfg["V"], seed, dev), FMT_V11, float(synth.weight_scale(seed)))
    g = torch.Generator(device=dev)
    g.manual_seed(synth.seed_for(rank, "embd") & 0x7FFFFFFF)
    emb = (torch.randn((cfg["V"], cfg["H"]), generator=g, device=dev) * 0.02).to(torch.bfloat16)
    tb.model_set_embd(emb.view(torch.int16))
    if host is not None:
        host.append(("embd", emb.view(torch.int16).cpu().numpy().view(np.uint16)))
    del emb
    rng = np.random.default_rng(synth.seed_for(rank, "vec"))
    v = rng.normal(1.0, 0.02, cfg["H"]).astype(np.float32)
    tb.model_set_vector(-1, 0, v)
    if host is not None:
        host.append(("vector", -1, 0, v))
    shapes = synth.model_shapes(cfg)
    for L in range(cfg["L"]):
        for wi, nm in enumerate(synth.MAT_ORDER):
            K, N = shapes[nm]
            seed = synth.seed_for(rank, "dec", which, L, nm)
            w = synth.packed_v11_cuda(K, N, seed, dev)
            tb.model_set_matrix(L, wi, w, FMT_V11, float(synth.weight_scale(seed)))
            if host is not None:
                host.append(("matrix", L, wi, w.cpu().numpy(), float(synth.weight_scale(seed))))
            del w
        for vi in range(4 if cfg["arch"] == 1 else 2):
            n = cfg["F"] if vi == 3 else (cfg["Nh"] * cfg["Hd"] if vi == 2 else cfg["H"])
            v = rng.normal(1.0, 0.02, n).astype(np.float32)
            tb.model_set_vector(L, vi, v)
            if host is not None:
                host.append(("vector", L, vi, v))
    prompt = np.random.default_rng(synth.seed_for(rank, "prompt", which)).integers(
        0, cfg["V"], size=(batch, n_prompt)).astype(np.int32)
    if batch == 1:
        prompt = prompt[0]
    if warm:
        tb.generate(prompt, n_gen)             # captures the graph, warms up
    l0 = tb.launch_count()
    t0 = time.perf_counter()
    out = tb.generate(prompt, n_gen)           # host tokens in, host tokens out
    wall = time.perf_counter() - t0
    launches = tb.launch_count() - l0
    ms = tb.last_generate_ms()
    prompt_ms = tb.last_prompt_ms()
    batched_prompt = tb.last_prefill_ms() > 0.0
    # generation phase: the steps after the prompt has been consumed (the first generated token belongs to
    # the prompt phase when the prompt ran as token batches)
    gen_steps = n_gen - 1 if batched_prompt else n_gen
    gen_ms = ms - prompt_ms
    shapes_bytes = sum(K * N // 4 for K, N in shapes.values()) * cfg["L"]
    # per generation step: packed layer weights + bf16 lm_head + the KV cache read at the mean context
    kv_bytes = batch * (n_prompt + n_gen / 2) * cfg["L"] * 2 * cfg["Nkv"] * cfg["Hd"] * 2
    step_bytes = shapes_bytes + (cfg["V"] * cfg["H"] // 4 if lm_head_packed else 2 * cfg["V"] * cfg["H"]) + kv_bytes
    peak, _ = peaks()
    name = "llama-3.2-1b" if which == "llama" else "bitnet-b1.58-2b"
    parity = None
    if check:
        # outside every timed region: greedy tokens against the CPU checker on the same weights (rank 0 computes)
        cp, cn = check
        t0 = time.perf_counter()
        pr = prompt if batch == 1 else prompt[0]
        got = [int(t) for t in (out[0][:cn] if cp == n_prompt else tb.generate(pr[:cp], cn)[0])]
        want = oracle_tokens(cfg, host, pr[:cp], cn) if checker else None
        if HOST_BARRIER is not None:
            HOST_BARRIER()                  # the other ranks sleep in a socket wait, not in a spinning collective
        parity = {"prompt": cp, "tokens": cn, "got": got, "want": want, "seconds": round(time.perf_counter() - t0, 1),
                  "checker": "oracle.Model (CPU restatement, all host threads), prompt fed one position at a time",
                  "ok": (got == want) if want is not None else None}
    res = {"workload": f"{name} architecture decode, batch {batch}, prompt {n_prompt} + {n_gen} greedy tokens, random-init"
                        + (", packed-trit lm_head" if lm_head_packed else ""),
            "tokens_per_s": batch * gen_steps / gen_ms * 1e3, "ms_per_step": gen_ms / gen_steps,
            "ms_per_token": gen_ms / gen_steps / batch, "steps": gen_steps, "batch": batch,
            "prompt_ms": prompt_ms, "prompt_tokens_per_s": batch * n_prompt / prompt_ms * 1e3,
            "prompt_mode": "token batches of up to 1024 positions through the tensor-core GEMM" if batched_prompt
                           else "one position per step (the reference's method)",
            "e2e_tokens_per_s": batch * n_gen / wall, "first_tokens": [int(t) for t in out[0][:4]],
            "roofline_frac_hbm": (step_bytes / (gen_ms / gen_steps * 1e-3) / 1e9) / peak,
            "bytes_per_step": int(step_bytes),
            "note": "tokens_per_s = generated tokens per second of device time (CUDA events) over the generation steps, "
                    "at contexts n_prompt .. n_prompt + n_gen; e2e = generated tokens / wall clock of the whole generate() "
                    "call (prompt included)" + ("" if warm else "; single call, includes the graph's first replays")}
    if parity is not None:
        res["parity"] = parity
    res["launches_in_call"] = int(launches)
    return res


def workload_config(layers=16):
    """The `config` of both arms (this library and --impl reference): the same workload, named the same way."""
    nbytes = packed_bytes(fabric_spec(layers))
    return {"workload": f"llama-3.2-1b GEMV fabric sweep: {layers} layers x 7 projections + packed lm_head, M=1, "
                        f"{nbytes / 1e6:.1f} MB packed trits per GPU per step",
            "l2": "inputs larger than L2 (309 MB vs 126 MB), same order every step"}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    r = cpu_reference_run(args.steps, args.warmup, threads)
    line = {"impl": "reference", "metric": METRIC, "value": r["value"], "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms_per_step"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int32 x int32 -> int64",
            "data": "synthetic", "config": workload_config(),
            "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": r["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-decode", action="store_true")
    ap.add_argument("--no-per-shape", action="store_true")
    ap.add_argument("--no-gemm", action="store_true")
    ap.add_argument("--no-bitnet", action="store_true", help="skip the BitNet-2B decode runs")
    ap.add_argument("--no-reference-gpu", action="store_true", help="skip the reference's CUDA programs on this GPU")
    ap.add_argument("--no-batch64", action="store_true", help="skip the batch-64 BitNet decode run (about 30 s)")
    ap.add_argument("--no-parity", action="store_true", help="skip the decode token checks against the CPU checker")
    ap.add_argument("--no-mma-attention", action="store_true",
                    help="skip the extra batch-64 run with the opt-in tensor-core attention (about 20 s)")
    ap.add_argument("--cold-batch64", action="store_true", help="time the batch-64 run without a warm-up call")
    ap.add_argument("--layers", type=int, default=16, help="layers of the fabric (profiling captures use fewer)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    if args.impl == "reference":
        run_reference_arm(args)
        return

    import torch
    import torch.distributed as dist
    from ter_b200 import FMT_V11, TerB200, synth

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
        global HOST_BARRIER
        host_group = dist.new_group(backend="gloo")
        HOST_BARRIER = lambda: dist.barrier(group=host_group)
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")

    tb = TerB200(local)
    mats = fabric_spec(args.layers)
    for name, K, N, L, nm in mats:
        seed = synth.seed_for(rank, K, N, L, nm)
        w = synth.packed_v11_cuda(K, N, seed, dev)
        tb.install(name, w, FMT_V11, K, N, float(synth.weight_scale(seed)))
        del w
    torch.cuda.synchronize()
    step_bytes = packed_bytes(mats)

    # device-resident activations: one int8 vector + scale per distinct K
    xs_dev, host_x, host_s = {}, {}, {}
    for K in sorted({K for _, K, _, _, _ in mats}):
        x, s = synth.activation(K, synth.seed_for("x", K))
        xs_dev[K] = (torch.from_numpy(x).to(dev), torch.tensor([s], dtype=torch.float32, device=dev))
        host_x[K] = torch.from_numpy(x).pin_memory()
        host_s[K] = float(s)
    outs = {name: torch.empty(N, dtype=torch.float32, device=dev) for name, _, N, _, _ in mats}
    # host results: one pinned buffer, the outputs back to back in call order
    host_out_all = torch.empty(sum(N for _, _, N, _, _ in mats), dtype=torch.float32).pin_memory()
    host_out, off = {}, 0
    for name, _, N, _, _ in mats:
        host_out[name] = host_out_all[off:off + N]
        off += N

    side = [torch.cuda.Stream(device=dev) for _ in range(8)]

    def step_device(streams=None):
        """One fabric pass.  streams=None: every launch on the current stream, a dependent chain
        as in a decode step.  streams=[...]: the 65 launches are independent (x is fixed), so
        they are spread round-robin over side streams and may overlap."""
        cur = torch.cuda.current_stream()
        n = [0]

        def nxt():
            if not streams:
                return None
            st = streams[n[0] % len(streams)]
            n[0] += 1
            return st
        if streams:
            for st in streams:
                st.wait_stream(cur)
        for L in range(args.layers):
            x, s = xs_dev[2048]
            tb.gemv_group([f"L{L}.q", f"L{L}.k", f"L{L}.v"], x, s,
                          [outs[f"L{L}.q"], outs[f"L{L}.k"], outs[f"L{L}.v"]], stream=nxt())
            tb.gemv(f"L{L}.o", x, s, outs[f"L{L}.o"], stream=nxt())
            tb.gemv_group([f"L{L}.gate", f"L{L}.up"], x, s, [outs[f"L{L}.gate"], outs[f"L{L}.up"]], stream=nxt())
            x8, s8 = xs_dev[8192]
            tb.gemv(f"L{L}.down", x8, s8, outs[f"L{L}.down"], stream=nxt())
        x, s = xs_dev[2048]
        tb.gemv("lm_head", x, s, outs["lm_head"], stream=nxt())
        if streams:
            for st in streams:
                cur.wait_stream(st)

    host_plan = tb.gemv_host_batch_plan([m_[0] for m_ in mats], [host_x[m_[1]] for m_ in mats],
                                        [host_s[m_[1]] for m_ in mats], [host_out[m_[0]] for m_ in mats])

    def step_host():
        # every projection through the host-buffer C-ABI call: pinned int8 x in, fp32 outputs back
        tb.gemv_host_batch(host_plan)
        tb.sync()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0 = tb.launch_count()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, tb.launch_count() - l0

    step_device()
    torch.cuda.synchronize()
    if tb.device_status() != 0:
        raise RuntimeError("device reported a timed-out wait")

    # The timed step replays a CUDA graph of the pass (as the reference's decode loop replays its
    # captured forward): graph_par = independent launches over 8 streams, graph_chain = one stream.
    graph_par = tb.capture(lambda: step_device(side))
    # the whole pass as ONE launch: a sweep plan (descriptor table in device memory)
    sweep = tb.gemv_plan([m_[0] for m_ in mats], [xs_dev[m_[1]][0] for m_ in mats], [xs_dev[m_[1]][1] for m_ in mats],
                         [outs[m_[0]] for m_ in mats])
    check = {m_[0]: outs[m_[0]].clone() for m_ in mats}
    for o in outs.values():
        o.zero_()
    tb.gemv_plan_launch(sweep, stream=torch.cuda.current_stream())
    torch.cuda.synchronize()
    for name, o in outs.items():
        if not torch.equal(o, check[name]):
            raise RuntimeError(f"sweep plan and per-matrix launches disagree on {name}")
    del check
    cur_stream = torch.cuda.current_stream()
    graph_chain = tb.capture(lambda: step_device(None))

    sampler = ClockSampler(local) if rank == 0 else None
    ms, launches = timed(lambda: tb.gemv_plan_launch(sweep, stream=cur_stream), args.steps, args.warmup)
    ms_par, launches_par = timed(lambda: tb.graph_launch(graph_par), args.steps, args.warmup)
    ms_chain, _ = timed(lambda: tb.graph_launch(graph_chain), args.steps, args.warmup)
    e2e_steps = max(3, args.steps // 5)
    ms_e2e, _ = timed(step_host, e2e_steps, 3)
    clocks = {}

    total_bytes = step_bytes * world
    value = total_bytes * args.steps / (ms * 1e-3) / 1e9
    e2e_value = total_bytes * e2e_steps / (ms_e2e * 1e-3) / 1e9
    peak, peak_src = peaks()
    per_gpu = step_bytes * args.steps / (ms * 1e-3) / 1e9

    per_shape = None
    if not args.no_per_shape and rank == 0:
        per_shape = per_shape_bench(tb, dev, peak)
    gemm = None
    if not args.no_gemm and rank == 0:
        gemm = gemm_bench(tb, dev)
    if sampler:
        clocks = sampler.stop()

    # ---- decode tokens/s (Llama-3.2-1B architecture, batch 1, prompt 128 + 256 greedy tokens)
    decode = None
    decode_bitnet = None
    if not args.no_decode:
        tb.close()
        torch.cuda.empty_cache()
        tb = TerB200(local)
        if world > 1:
            tb.comm_init_from_torch()      # tensor parallel: output-dimension sharding, slices exchanged over peer memory
            tb.set_option("tp_p2p", int(os.environ.get("TER_TP_P2P", "1")))   # 0: NCCL all-gathers, for comparison
            if "TER_TP_SHARD" in os.environ:                                  # else the library's default policy
                tb.set_option("tp_shard", int(os.environ["TER_TP_SHARD"]))
        failures = []

        def tp_fix(d):
            # parity first: every rank must hold rank 0's tokens, and rank 0's must be the CPU checker's
            if d.get("parity") is not None:
                par = d["parity"]
                if world > 1:
                    mine = torch.tensor(par["got"], dtype=torch.int64, device=dev)
                    ref = mine.clone()
                    dist.broadcast(ref, 0)
                    same = torch.tensor([1 if torch.equal(mine, ref) else 0], device=dev)
                    dist.all_reduce(same, op=dist.ReduceOp.MIN)
                    par["all_ranks_equal"] = bool(int(same.item()))
                    flag = torch.tensor([1 if (par["ok"] in (True, None)) else 0], device=dev)
                    dist.broadcast(flag, 0)
                    par["ok"] = bool(int(flag.item())) and par["all_ranks_equal"]
                if not par["ok"]:
                    failures.append(d["workload"])
            if world > 1:
                t = torch.tensor([d["ms_per_step"]], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                d["ms_per_step"] = float(t.item())
                d["ms_per_token"] = d["ms_per_step"] / d["batch"]
                d["tokens_per_s"] = 1e3 / d["ms_per_token"]
                d["note"] += f"; tensor parallel over {world} GPUs (strong scaling, max over ranks)"
                d["parallelism"] = f"tp{world}"
                d["sharded_blocks"] = os.environ.get("TER_TP_SHARD", "library default")
                d["exchange"] = "peer-memory kernel" if os.environ.get("TER_TP_P2P", "1") != "0" else "nccl all-gather"
            return d
        # the same model on every rank; the library keeps its slice.  Checked: the first 16 greedy tokens of the
        # full-depth run against the CPU checker (whole 128-token prompt)
        decode = tp_fix(decode_bench(tb, dev, 0, check=None if args.no_parity else (128, 16)))
        if not args.no_bitnet:
            # BitNet-2B architecture, context 2048 + 128 greedy tokens; batch 1 (tensor
            # parallel at N > 1) and, on one GPU, batch 64 (token batch through the tensor-core GEMM)
            # checked against the CPU checker at a SHORTENED prompt (48 positions + 8 tokens, all 30 layers): the
            # checker needs about half a second per position, the 2048-position prompt would take a quarter hour
            decode_bitnet = [tp_fix(decode_bench(tb, dev, 0, "bitnet", n_prompt=2048, n_gen=128, smax=2176,
                                                 check=None if args.no_parity else (48, 8)))]
            if not args.no_batch64 and 64 % world == 0:
                # 64 sequences: on one GPU a token batch through the tensor-core GEMM; on N GPUs every rank
                # owns 64/N whole sequences and their KV cache with a full copy of the weights (no collective:
                # sequences are independent), through a second handle that has no communicator
                per_rank = 64 // world
                tb2 = tb if world == 1 else TerB200(local)
                d = decode_bench(tb2, dev, rank, "bitnet", n_prompt=2048, n_gen=128, batch=per_rank, smax=2176,
                                 warm=not args.cold_batch64)
                if world > 1:
                    t = torch.tensor([d["ms_per_step"], d["prompt_ms"]], device=dev)
                    dist.all_reduce(t, op=dist.ReduceOp.MAX)
                    d["ms_per_step"], d["prompt_ms"] = float(t[0].item()), float(t[1].item())
                    d["batch"] = 64
                    d["ms_per_token"] = d["ms_per_step"] / 64
                    d["tokens_per_s"] = 64e3 / d["ms_per_step"]
                    d["prompt_tokens_per_s"] = 64 * 2048 / d["prompt_ms"] * 1e3
                    d["parallelism"] = f"{world} ranks x {per_rank} sequences, weights replicated, no collective"
                    d["workload"] = d["workload"].replace(f"batch {per_rank}", f"batch 64 ({per_rank} per GPU)")
                    d.pop("e2e_tokens_per_s", None)
                    tb2.close()
                decode_bitnet.append(d)
                if world == 1 and not args.no_mma_attention:
                    # the same batch with option "attn_mma_min" = 8: attention of token batches sums its two
                    # contractions on the tensor cores.  Opt-in, because the result is no longer bit-equal to the
                    # CPU checker: sums differ in the last places, the int8 quantisers downstream turn some of
                    # that into different roundings, and greedy tokens drift apart after some steps.
                    tb.set_option("attn_mma_min", 8)
                    try:
                        m = decode_bench(tb, dev, rank, "bitnet", n_prompt=2048, n_gen=128, batch=64, smax=2176)
                    finally:
                        tb.set_option("attn_mma_min", 0)
                    m["workload"] += ", opt-in tensor-core attention"
                    m["option"] = "attn_mma_min=8 (default: off)"
                    m["first_tokens_equal_to_default_path"] = m["first_tokens"] == d["first_tokens"]
                    decode_bitnet.append(m)

    reference_gpu = None
    if rank == 0 and world == 1 and not args.no_decode and not args.no_reference_gpu:
        reference_gpu = {"decode": reference_gpu_bench(tb, dev), "gemv": reference_gpu_gemv()}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        try:
            r = cpu_reference_run(steps=6, warmup=1, threads=os.cpu_count() or 1)
            cpu = {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")}
            cpu["forward_token"] = cpu_forward_baseline()
        except Exception as e:  # noqa: BLE001
            cpu = {"value": None, "unit": UNIT, "cores": 0, "kind": "port", "sample": f"failed: {e}"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int8 x trit -> int32", "data": "synthetic",
            "config": workload_config(args.layers),
            "timed": {"launches_per_step": launches // args.steps,
                      "how": "one sweep-plan launch per step (ter_b200_gemv_plan_launch): the 113 independent GEMVs are "
                             "rows of a device descriptor table and one persistent grid streams all of them"},
            "per_matrix_launches": {"value": total_bytes * args.steps / (ms_par * 1e-3) / 1e9, "unit": UNIT,
                                    "ms_per_step": ms_par / args.steps, "launches_per_step": launches_par // args.steps,
                                    "note": "same pass as 65 launches (q+k+v and gate+up grouped) replayed from a CUDA "
                                            "graph over 8 streams"},
            "dependent_chain": {"value": total_bytes * args.steps / (ms_chain * 1e-3) / 1e9, "unit": UNIT,
                                "ms_per_step": ms_chain / args.steps,
                                "note": "same pass as one stream-ordered chain with programmatic dependent launch "
                                        "(each GEMV waits for the previous one, as in a decode step)"},
            "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": peak, "unit": "GB/s", "frac": per_gpu / peak,
                         "traffic": NCU_TRAFFIC_BYTES if args.layers == 16 else None, "peak_source": peak_src,
                         "algorithmic_bytes": step_bytes,
                         "traffic_note": "dram__bytes_read.sum + dram__bytes_write.sum of one launch of this workload, from "
                                         "the ncu capture summarised in profiles/gemv_trit_kernel_table_sweep_llama1b_fabric.md",
                         "note": "achieved = packed weight bytes of the launch / its CUDA-event time (one launch per step)"},
            "per_shape": per_shape,
            "gemm": gemm,
            "cpu_baseline": cpu,
            "e2e": {"value": e2e_value, "unit": UNIT, "steps": e2e_steps,
                    # what the call copies up: each distinct activation vector once, a 32-byte descriptor per
                    # matrix and the scales (one 256-byte block)
                    "h2d_bytes_per_step": (sum(sorted({K for _, K, _, _, _ in mats})) + 32 * len(mats) + 256) * world,
                    "note": "ter_b200_gemv_host_batch: pinned host x in, one launch, fp32 outputs back to one pinned "
                            "host buffer; synchronous call",
                    "d2h_bytes_per_step": sum(4 * N for _, _, N, _, _ in mats) * world},
            "decode_scaling": None if decode is None else {
                "n_gpus": world,
                "llama_1b_batch1_tokens_per_s": decode["tokens_per_s"],
                "bitnet_2b_batch1_tokens_per_s": decode_bitnet[0]["tokens_per_s"] if decode_bitnet else None,
                "bitnet_2b_batch64_tokens_per_s": decode_bitnet[1]["tokens_per_s"] if decode_bitnet and len(decode_bitnet) > 1 else None,
                "tokens_checked": None if args.no_parity else "first tokens equal on every rank and equal to the CPU checker's",
                "note": "strong scaling of one model over the GPUs of this run (batch 1: tensor parallel; batch 64: whole "
                        "sequences per GPU); compare the same keys across the N = 1, 2, 4, 8 runs"},
            "decode": decode,
            "decode_bitnet": decode_bitnet,
            "reference_gpu": reference_gpu,
            "gpu_launches": launches,
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    tb.close()
    if world > 1:
        dist.destroy_process_group()
    if not args.no_decode and failures:
        sys.stderr.write("decode tokens differ from the CPU checker: " + "; ".join(failures) + "\n")
        sys.exit(3)


if __name__ == "__main__":
    main()
