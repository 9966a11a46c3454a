#!/usr/bin/env python3
"""Regenerates tests/golden/*.npz by running the UNMODIFIED reference CPU code
(oracle/_ref/libter_ref.so, built from the reference checkout by oracle/Makefile).

Run from the repository root in a container that has the reference checkout:
    make -C oracle all && python tests/golden/make_golden.py

Fixtures (all small):
  mm_row_small.npz      reference mm_row outputs (float bits) on seeded small shapes, and the
                        reference quantize() payloads/scales on seeded vectors.
  mm_row_recipes.npz    the reference's own known-answer recipes evaluated by reference mm_row:
                        - the deterministic K=64,N=16 pattern of
                          cuda/ter_cuda_forward_packed_v13_int4tc.cu:511-541
                          (code (7k+13n)%3, x (11k+3)%15-7, scales 1)
                        - the four shapes of tests/cuda_forward_correctness.cu:77-123
                          (X ~ U[-127,127], codes ~ U{0,1,2}, scale_x 0.0312, w_scale 0.05),
                          inputs drawn from numpy's seeded generator, outputs stored as a
                          SHA-256 over the float32 bytes plus the first 16 values.
"""
import hashlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))

CORRECTNESS_SHAPES = [("tiny", 128, 64), ("medium", 2048, 512), ("big", 2048, 8192), ("huge", 8192, 2048)]


def correctness_inputs(name, K, N):
    rng = np.random.default_rng([42, K, N])
    x = rng.integers(-127, 128, size=K).astype(np.int8)
    codes = rng.integers(0, 3, size=(K, N)).astype(np.int8)
    trits = np.where(codes == 1, 1, np.where(codes == 2, -1, 0)).astype(np.int8)
    return x, trits


def int4tc_pattern():
    K, N = 64, 16
    k = np.arange(K)[:, None]
    n = np.arange(N)[None, :]
    code = (k * 7 + n * 13) % 3
    trits = np.where(code == 1, 1, np.where(code == 2, -1, 0)).astype(np.int8)
    x = ((np.arange(K) * 11 + 3) % 15 - 7).astype(np.int8)
    return x, trits


def main():
    ref = oracle.Ref()
    small = {}
    rng = np.random.default_rng(20261125)
    for i, (K, N) in enumerate([(16, 4), (27, 8), (64, 16), (128, 64), (256, 96), (432, 80)]):
        W = rng.choice([-1, 0, 1], size=(K, N), p=[0.3, 0.4, 0.3]).astype(np.int32)
        X = rng.integers(-128, 128, size=(3, K)).astype(np.int32)
        X[1, ::3] = 0                      # exercise the zero-skip
        xs, ws = np.float32(rng.uniform(0.001, 0.1)), np.float32(rng.uniform(0.01, 0.05))
        outs = np.stack([ref.mm_row(X, float(xs), W, float(ws), row=r) for r in range(3)])
        small[f"W{i}"] = W.astype(np.int8)
        small[f"X{i}"] = X
        small[f"s{i}"] = np.array([xs, ws], dtype=np.float32)
        small[f"out{i}"] = outs
    # 9-trit weights too (general int32 payload, as the CPU forward uses them)
    W = rng.integers(-9841, 9842, size=(81, 40)).astype(np.int32)
    X = rng.integers(-9841, 9842, size=(2, 81)).astype(np.int32)
    small["W9"] = W
    small["X9"] = X
    small["s9"] = np.array([0.00123, 0.00045], dtype=np.float32)
    small["out9"] = np.stack([ref.mm_row(X, 0.00123, W, 0.00045, row=r) for r in range(2)])
    # reference quantize()
    for i, n in enumerate([7, 64, 1000]):
        v = (rng.standard_normal(n) * rng.uniform(0.1, 30)).astype(np.float32)
        for nt in (2, 9):
            q, s = ref.quantize(v, nt)
            small[f"qv{i}"] = v
            small[f"qq{i}_{nt}"] = q
            small[f"qs{i}_{nt}"] = np.array([s], dtype=np.float32)
    np.savez_compressed(os.path.join(HERE, "mm_row_small.npz"), **small)

    rec = {}
    x, t = int4tc_pattern()
    ref.reset_counters()
    rec["int4tc_out"] = ref.mm_row(x.astype(np.int32), 1.0, t.astype(np.int32), 1.0)
    rec["int4tc_tvmac"] = np.array([ref.tvmac()], dtype=np.uint64)
    for name, K, N in CORRECTNESS_SHAPES:
        x, t = correctness_inputs(name, K, N)
        out = ref.mm_row(x.astype(np.int32), 0.0312, t.astype(np.int32), 0.05)
        rec[f"{name}_sha256"] = np.frombuffer(hashlib.sha256(out.tobytes()).digest(), dtype=np.uint8)
        rec[f"{name}_head"] = out[:16].copy()
        rec[f"{name}_x_sha256"] = np.frombuffer(hashlib.sha256(x.tobytes() + t.tobytes()).digest(), dtype=np.uint8)
    np.savez_compressed(os.path.join(HERE, "mm_row_recipes.npz"), **rec)

    # microsoft/BitNet i2_s blocks decoded by the reference's own nt::dequant_i2_s
    # (vendor/ntransformer/core/dequant.cpp:114-145): 8 x 384 elements = 24 blocks, every byte value present
    irng = np.random.default_rng(20261125)
    N, K = 8, 384
    raw = np.concatenate([irng.integers(0, 256, size=N * K // 4, dtype=np.uint8), np.zeros(32, np.uint8)])
    raw[N * K // 4:N * K // 4 + 4] = np.array([0.0371], np.float32).view(np.uint8)
    raw[:256] = np.arange(256, dtype=np.uint8)
    np.savez(os.path.join(HERE, "i2s_blocks.npz"), raw=raw, N=np.array([N]), K=np.array([K]),
             dequant=ref.dequant_i2s(raw, N * K))
    print("wrote", sorted(os.listdir(HERE)))


if __name__ == "__main__":
    main()
