"""Writer / header reader for the reference's packed-model files, 'LLRT' (Llama architecture,
tools/convert_llama_to_packed.py:13-43) and 'TERT' (BitNet architecture,
tools/convert_bitnet_to_packed.py:4-31).  The library's own reader is ter_b200_model_load_file
(csrc/loader.cpp); this writer exists so that synthetic models can be put on disk in the format the
reference's programs and scripts read.
"""
from __future__ import annotations

import struct

import numpy as np

MAGIC_LLAMA = 0x4C4C5254   # 'LLRT'
MAGIC_BITNET = 0x54455254  # 'TERT'


def bf16_to_f32(a: np.ndarray) -> np.ndarray:
    return (a.astype(np.uint32) << 16).view(np.float32)


def write_packed_model(path: str, cfg: dict, items) -> None:
    """cfg: arch, H, F, L, V, Nh, Nkv, Hd, Smax, eps, rope_theta.  items: what
    synth.model_weights yields: ("embd", bf16 bits [V][H]), ("vector", layer, which, f32[n]),
    ("matrix", layer, which, v11 packed bytes, scale).  The embeddings must be exact in fp16."""
    mats, vecs, embd = {}, {}, None
    for item in items:
        if item[0] == "embd":
            embd = item[1]
        elif item[0] == "vector":
            vecs[(item[1], item[2])] = item[3]
        else:
            mats[(item[1], item[2])] = (item[3], item[4])
    e32 = bf16_to_f32(embd)
    e16 = e32.astype(np.float16)
    if not np.array_equal(e16.astype(np.float32), e32):
        raise ValueError("bf16 embeddings must be exact in fp16 to be stored in this format")
    magic = MAGIC_BITNET if cfg["arch"] == 1 else MAGIC_LLAMA
    with open(path, "wb") as f:
        hdr = struct.pack("<II8Iff", magic, 1, cfg["H"], cfg["F"], cfg["L"], cfg["V"], cfg["Nh"], cfg["Nkv"],
                          cfg["Hd"], cfg["Smax"], cfg["rope_theta"], cfg["eps"])
        f.write(hdr + b"\0" * (64 - len(hdr)))
        f.write(e16.tobytes())
        f.write(vecs[(-1, 0)].astype(np.float32).tobytes())
        for L in range(cfg["L"]):
            for vi in range(4 if cfg["arch"] == 1 else 2):
                f.write(vecs[(L, vi)].astype(np.float32).tobytes())
            for wi in range(7):
                packed, scale = mats[(L, wi)]
                f.write(np.ascontiguousarray(packed).tobytes())
                f.write(struct.pack("<f", float(scale)))


def read_header(path: str) -> dict:
    with open(path, "rb") as f:
        raw = f.read(64)
    magic, version, H, F, L, V, Nh, Nkv, Hd, Smax, theta, eps = struct.unpack("<II8Iff", raw[:48])
    if magic not in (MAGIC_LLAMA, MAGIC_BITNET) or version != 1:
        raise ValueError(f"not a packed-model file: magic 0x{magic:08x} version {version}")
    return dict(arch=1 if magic == MAGIC_BITNET else 0, H=H, F=F, L=L, V=V, Nh=Nh, Nkv=Nkv, Hd=Hd, Smax=Smax,
                rope_theta=theta, eps=eps)
