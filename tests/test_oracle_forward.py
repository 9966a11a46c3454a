"""Pins the CPU checker's decode forward (stage order, GQA mapping, rotary conventions, tied
lm_head) against greedy tokens produced by the reference's own NumPy forwards
(tools/llama_pyfwd.py, tools/bitnet_pyfwd.py) run unmodified on the same synthetic model
(tests/golden/make_pyfwd_golden.py)."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
sys.path.insert(0, os.path.dirname(__file__))
import make_pyfwd_golden as mk  # noqa: E402
import modelutil  # noqa: E402

BOS = 128000


@pytest.mark.parametrize("name", ["llama", "bitnet"])
def test_forward_matches_reference_numpy_tokens(golden_dir, name):
    g = np.load(os.path.join(golden_dir, "pyfwd_tokens.npz"))
    want = g[f"{name}_tokens"]
    case = mk.CASES[name]
    cfg = {k: case[k] for k in ("arch", "H", "F", "L", "V", "Nh", "Nkv", "Hd", "Smax", "eps", "rope_theta")}
    # the reference scripts keep the KV cache in fp32 and quantise with np.round(x / (amax/127))
    m = modelutil.build_oracle(cfg, case["seed"], kv_f32=1, np_quant=1)
    got, _ = modelutil.oracle_generate(m, [BOS], len(want))
    assert got.tolist() == want.tolist()
    # the shipped semantics (bf16 cache, reciprocal-scale quantiser) agree on this model too
    m2 = modelutil.build_oracle(cfg, case["seed"])
    got2, _ = modelutil.oracle_generate(m2, [BOS], len(want))
    assert got2.tolist() == want.tolist()
