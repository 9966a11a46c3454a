"""Seeded synthetic workloads with the shapes and value distributions of the
reference's benchmarks: ternary weights iid {-1: 0.3, 0: 0.4, +1: 0.3} packed 4 per byte,
one fp32 scale per tensor ~ U(0.01, 0.05), int8 activations from absmax-quantising N(0,1).

Host side is numpy (reproducible everywhere); ``packed_v11_cuda`` draws the same
distribution on the GPU for tensors too large to be worth generating on the host.
"""
from __future__ import annotations

import zlib

import numpy as np

BASE_SEED = 20261125

# (K, N) of every Llama-3.2-1B projection (H=2048, F=8192, 8 KV heads x 64, V=128256)
LLAMA_1B_SHAPES = {
    "q": (2048, 2048), "k": (2048, 512), "v": (2048, 512), "o": (2048, 2048),
    "gate": (2048, 8192), "up": (2048, 8192), "down": (8192, 2048), "lm_head": (2048, 128256),
}
# BitNet-b1.58-2B (H=2560, F=6912, 5 KV heads x 128)
BITNET_2B_SHAPES = {
    "q": (2560, 2560), "k": (2560, 640), "v": (2560, 640), "o": (2560, 2560),
    "gate": (2560, 6912), "up": (2560, 6912), "down": (6912, 2560),
}
LLAMA_1B_CFG = dict(arch=0, H=2048, F=8192, L=16, V=128256, Nh=32, Nkv=8, Hd=64, eps=1e-5, rope_theta=500000.0)
BITNET_2B_CFG = dict(arch=1, H=2560, F=6912, L=30, V=128256, Nh=20, Nkv=5, Hd=128, eps=1e-5, rope_theta=500000.0)


def seed_for(*key) -> int:
    """Stable 63-bit seed from the base seed and a key such as (K, N, layer, 'q')."""
    h = zlib.crc32(repr(key).encode())
    return (BASE_SEED * 1000003 + h) & 0x7FFFFFFFFFFFFFFF


def trits(K: int, N: int, seed: int) -> np.ndarray:
    """int8 [K][N] with P(-1)=0.3, P(0)=0.4, P(+1)=0.3."""
    rng = np.random.default_rng(seed)
    u = rng.random((K, N), dtype=np.float32)
    return (u >= 0.7).astype(np.int8) - (u < 0.3).astype(np.int8)


def _codes(t: np.ndarray) -> np.ndarray:
    # trit -> boundary 2-bit code: 0 -> 0, +1 -> 1, -1 -> 2
    return np.where(t > 0, 1, np.where(t < 0, 2, 0)).astype(np.uint8)


def pack_v11(t: np.ndarray) -> np.ndarray:
    """[K][N] trits -> bytes [N/4][K] (byte (j/4)*K + k, column j in bits 2*(j%4))."""
    K, N = t.shape
    c = _codes(t).reshape(K, N // 4, 4)
    b = c[:, :, 0] | (c[:, :, 1] << 2) | (c[:, :, 2] << 4) | (c[:, :, 3] << 6)
    return np.ascontiguousarray(b.T)


def pack_rowmajor(t: np.ndarray) -> np.ndarray:
    """[K][N] trits -> bytes [K][N/4]."""
    K, N = t.shape
    c = _codes(t).reshape(K, N // 4, 4)
    return np.ascontiguousarray(c[:, :, 0] | (c[:, :, 1] << 2) | (c[:, :, 2] << 4) | (c[:, :, 3] << 6))


def unpack_v11(p: np.ndarray, K: int, N: int) -> np.ndarray:
    """bytes [N/4][K] -> int8 trits [K][N]; code 3 decodes to 0."""
    p = np.asarray(p, dtype=np.uint8).reshape(N // 4, K)
    out = np.empty((K, N), dtype=np.int8)
    for f in range(4):
        c = (p >> (2 * f)) & 3
        out[:, f::4] = ((c == 1).astype(np.int8) - (c == 2).astype(np.int8)).T
    return out


def weight_scale(seed: int) -> np.float32:
    return np.float32(np.random.default_rng(seed ^ 0x5CA1E).uniform(0.01, 0.05))


def quant_int8(x: np.ndarray):
    """Per-token absmax int8 as the reference's quantiser kernels do
    (cuda/ter_cuda_forward_packed.cu:40-62): scale = 127/(amax+1e-9), round to nearest even,
    clamp; the stored scale is 1/scale.  All in fp32."""
    x = np.asarray(x, dtype=np.float32)
    amax = np.float32(np.abs(x).max()) + np.float32(1e-9)
    scale = np.float32(127.0) / amax
    q = np.clip(np.rint(x * scale), -128, 127).astype(np.int8)
    return q, np.float32(1.0) / scale


def activation(K: int, seed: int):
    """int8[K] and fp32 scale from N(0,1)."""
    rng = np.random.default_rng(seed ^ 0xAC7)
    return quant_int8(rng.standard_normal(K).astype(np.float32))


def packed_v11_cuda(K: int, N: int, seed: int, device="cuda"):
    """uint8 [N/4][K] on the GPU with the same per-trit distribution (torch RNG, seeded)."""
    import torch
    g = torch.Generator(device=device)
    g.manual_seed(seed & 0x7FFFFFFFFFFFFFFF)
    out = torch.zeros((N // 4, K), dtype=torch.uint8, device=device)
    for f in range(4):
        u = torch.rand((N // 4, K), generator=g, device=device)
        code = (u >= 0.7).to(torch.uint8) + 2 * (u < 0.3).to(torch.uint8)   # +1 -> 1, -1 -> 2
        out |= code << (2 * f)
    return out


MAT_ORDER = ["q", "k", "v", "o", "gate", "up", "down"]


def model_shapes(cfg: dict) -> dict:
    Hq, Hkv = cfg["Nh"] * cfg["Hd"], cfg["Nkv"] * cfg["Hd"]
    return {"q": (cfg["H"], Hq), "k": (cfg["H"], Hkv), "v": (cfg["H"], Hkv), "o": (Hq, cfg["H"]),
            "gate": (cfg["H"], cfg["F"]), "up": (cfg["H"], cfg["F"]), "down": (cfg["F"], cfg["H"])}


def f32_to_bf16(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16 bit patterns (uint16)."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    r = u + (np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1)))     # finite inputs: no wrap-around
    return (r >> np.uint32(16)).astype(np.uint16)


def model_weights(cfg: dict, seed: int = BASE_SEED):
    """Random-init ternarised model of the given architecture, host side (numpy):
    yields ("matrix", layer, which, packed_v11 bytes, scale), ("vector", layer, which, fp32),
    ("embd", bf16 table [V][H]).  Embeddings ~ N(0, 0.02) in bf16; norm gains ~ N(1, 0.02)."""
    shapes = model_shapes(cfg)
    rng = np.random.default_rng(seed_for(seed, "vec"))
    emb = np.random.default_rng(seed_for(seed, "embd")).standard_normal((cfg["V"], cfg["H"]), dtype=np.float32)
    # N(0, 0.02), snapped to multiples of 2^-14 so that the bf16 values are also exact in fp16 (the
    # reference's packed-model files store the table in fp16); in place to keep memory flat
    emb *= np.float32(0.02 * 16384.0)
    np.rint(emb, out=emb)
    emb *= np.float32(1.0 / 16384.0)
    yield ("embd", f32_to_bf16(emb))
    del emb
    yield ("vector", -1, 0, rng.normal(1.0, 0.02, cfg["H"]).astype(np.float32))
    if cfg.get("lm_head_packed"):
        s = seed_for(seed, "lm_head")
        yield ("matrix", -1, 0, pack_v11(trits(cfg["H"], cfg["V"], s)), weight_scale(s))
    for L in range(cfg["L"]):
        for wi, nm in enumerate(MAT_ORDER):
            K, N = shapes[nm]
            s = seed_for(seed, L, nm)
            yield ("matrix", L, wi, pack_v11(trits(K, N, s)), weight_scale(s))
        n_vec = 4 if cfg["arch"] == 1 else 2
        for vi in range(n_vec):
            n = cfg["F"] if vi == 3 else (cfg["Nh"] * cfg["Hd"] if vi == 2 else cfg["H"])
            yield ("vector", L, vi, rng.normal(1.0, 0.02, n).astype(np.float32))
