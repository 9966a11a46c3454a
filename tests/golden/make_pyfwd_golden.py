#!/usr/bin/env python3
"""Regenerates tests/golden/pyfwd_tokens.npz by running the reference's own NumPy statements of
the GPU forward, UNMODIFIED, on synthetic packed-model files:

    tools/llama_pyfwd.py   reads /tmp/llama_3_2_1b_packed.bin  ('LLRT'), 16 greedy tokens from BOS
    tools/bitnet_pyfwd.py  reads /tmp/bitnet_2b_4t_packed.bin  ('TERT'),  8 greedy tokens from BOS

The files are written here in the reference's on-disk format
(tools/convert_llama_to_packed.py:13-43, tools/convert_bitnet_to_packed.py:4-31) from
ter_b200.synth.model_weights(cfg, seed), so the tests can rebuild the same model without the
reference.  Run from the repository root in a container that has the reference checkout:
    TER_REFERENCE=<reference checkout> python tests/golden/make_pyfwd_golden.py
"""
import ast
import os
import re
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from ter_b200 import modelfile, synth  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.environ.get("TER_REFERENCE", "")   # path of the reference checkout

TINY = dict(H=256, F=256, L=2, V=128256, Nh=4, Nkv=2, Hd=64, Smax=32, eps=1e-5, rope_theta=500000.0)
CASES = {
    "llama": dict(TINY, arch=0, seed=101, script="tools/llama_pyfwd.py", bin="/tmp/llama_3_2_1b_packed.bin",
                  magic=0x4C4C5254),
    "bitnet": dict(TINY, arch=1, seed=202, script="tools/bitnet_pyfwd.py", bin="/tmp/bitnet_2b_4t_packed.bin",
                   magic=0x54455254),
}


def write_bin(case):
    modelfile.write_packed_model(case["bin"], case, synth.model_weights(case, case["seed"]))


def main():
    if not REF:
        sys.exit("set TER_REFERENCE to the reference checkout")
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
