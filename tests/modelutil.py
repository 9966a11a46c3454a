"""Builds the same synthetic model on both sides: the CPU checker and the CUDA library."""
import numpy as np

import oracle
from ter_b200 import FMT_V11, synth


_cache = {}


def weights(cfg, seed):
    """The model's tensors, generated once per (cfg, seed) and shared by both sides."""
    key = (tuple(sorted((k, v) for k, v in cfg.items() if k in
                        ("arch", "H", "F", "L", "V", "Nh", "Nkv", "Hd", "lm_head_packed"))), seed)
    if key not in _cache:
        _cache.clear()
        _cache[key] = list(synth.model_weights(cfg, seed))
    return _cache[key]


def build_oracle(cfg, seed, **modes):
    m = oracle.Model(dict(cfg, **modes))
    for item in weights(cfg, seed):
        if item[0] == "embd":
            m.set_embd(item[1])
        elif item[0] == "vector":
            m.set_vector(item[1], item[2], item[3])
        else:
            m.set_matrix(item[1], item[2], item[3], float(item[4]))
    return m


def build_gpu(tb, cfg, seed, max_batch=1):
    tb.model_create(cfg, max_batch=max_batch)
    for item in weights(cfg, seed):
        if item[0] == "embd":
            tb.model_set_embd(item[1])
        elif item[0] == "vector":
            tb.model_set_vector(item[1], item[2], item[3])
        else:
            tb.model_set_matrix(item[1], item[2], item[3], FMT_V11, float(item[4]))


def oracle_generate(m, prompt, n_gen, want_logits=False):
    """Greedy tokens (and per-step logits) of one sequence, prompt fed one position at a time."""
    st = m.new_state(1)
    toks, logits = [], []
    tok = int(prompt[0])
    steps = len(prompt) + n_gen - 1
    for pos in range(steps):
        nxt, lg, _ = m.forward(st, 0, tok, pos, want_logits=want_logits)
        if pos + 1 < len(prompt):
            tok = int(prompt[pos + 1])
        else:
            tok = nxt
            toks.append(nxt)
        if want_logits:
            logits.append(lg)
    return np.array(toks, dtype=np.int32), logits
