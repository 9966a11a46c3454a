#!/usr/bin/env python3
"""Regenerates tests/golden/pyfwd_tokens.npz by running the reference's own NumPy statements of
the GPU forward, UNMODIFIED, on synthetic packed-model files:

    tools/llama_pyfwd.py   reads /tmp/llama_3_2_1b_packed.bin  ('LLRT'), 16 greedy tokens from BOS
    tools/bitnet_pyfwd.py  reads /tmp/bitnet_2b_4t_packed.bin  ('TERT'),  8 greedy tokens from BOS

The files are written here in the reference's on-disk format
(tools/convert_llama_to_packed.py:13-43, tools/convert_bitnet_to_packed.py:4-31) from
ter_b200.synth.model_weights(cfg, seed), so the tests can rebuild the same model without the
reference.  Run from the repository root in a container that has the reference checkout:
    python tests/golden/make_pyfwd_golden.py
"""
import ast
import os
import re
import struct
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from ter_b200 import synth  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.environ.get("TER_REFERENCE", "/root/reference")

TINY = dict(H=128, F=256, L=2, V=128256, Nh=2, Nkv=1, Hd=64, Smax=32, eps=1e-5, rope_theta=500000.0)
CASES = {
    "llama": dict(TINY, arch=0, seed=101, script="tools/llama_pyfwd.py", bin="/tmp/llama_3_2_1b_packed.bin",
                  magic=0x4C4C5254),
    "bitnet": dict(TINY, arch=1, seed=202, script="tools/bitnet_pyfwd.py", bin="/tmp/bitnet_2b_4t_packed.bin",
                   magic=0x54455254),
}


def bf16_to_f32(a):
    return (a.astype(np.uint32) << 16).view(np.float32)


def write_bin(case):
    c = case
    mats, vecs, embd = {}, {}, None
    for item in synth.model_weights(c, c["seed"]):
        if item[0] == "embd":
            embd = item[1]
        elif item[0] == "vector":
            vecs[(item[1], item[2])] = item[3]
        else:
            mats[(item[1], item[2])] = (item[3], item[4])
    e32 = bf16_to_f32(embd)
    e16 = e32.astype(np.float16)
    assert np.array_equal(e16.astype(np.float32), e32), "bf16 embeddings must be exact in fp16"
    with open(c["bin"], "wb") as f:
        hdr = struct.pack("<II8Iff", c["magic"], 1, c["H"], c["F"], c["L"], c["V"], c["Nh"], c["Nkv"], c["Hd"],
                          c["Smax"], c["rope_theta"], c["eps"])
        f.write(hdr + b"\0" * (64 - len(hdr)))
        f.write(e16.tobytes())
        f.write(vecs[(-1, 0)].astype(np.float32).tobytes())
        for L in range(c["L"]):
            for vi in range(4 if c["arch"] == 1 else 2):
                f.write(vecs[(L, vi)].astype(np.float32).tobytes())
            for wi in range(7):
                packed, scale = mats[(L, wi)]
                f.write(np.ascontiguousarray(packed).tobytes())
                f.write(struct.pack("<f", float(scale)))


def main():
    out = {}
    for name, case in CASES.items():
        write_bin(case)
        r = subprocess.run([sys.executable, os.path.join(REF, case["script"])], capture_output=True, text=True,
                           check=True)
        lists = re.findall(r"\[[0-9, ]+\]", r.stdout)
        toks = ast.literal_eval(lists[0])
        if name == "bitnet":
            toks = toks[1:]           # the script prints BOS first
        out[f"{name}_tokens"] = np.array(toks, dtype=np.int32)
        out[f"{name}_seed"] = np.array([case["seed"]])
        print(name, toks)
        os.unlink(case["bin"])
    np.savez(os.path.join(HERE, "pyfwd_tokens.npz"), **out)


if __name__ == "__main__":
    main()
