"""End-to-end parity of the CUDA decode forward with the CPU checker: logits within 1e-3 relative
(asserted, and in fact bit-for-bit), greedy tokens identical."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(__file__))
sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
import modelutil  # noqa: E402
from ter_b200 import api, synth  # noqa: E402

pytestmark = pytest.mark.gpu

SMALL_LLAMA = dict(arch=0, H=256, F=512, L=3, V=4096, Nh=4, Nkv=2, Hd=64, Smax=320, eps=1e-5, rope_theta=500000.0)
SMALL_BITNET = dict(arch=1, H=512, F=768, L=2, V=3000, Nh=4, Nkv=1, Hd=128, Smax=300, eps=1e-5, rope_theta=500000.0)
SMALL_PACKED_HEAD = dict(SMALL_LLAMA, lm_head_packed=1, L=2, Smax=64)


def rel_err(a, b):
    return np.max(np.abs(a - b) / (np.abs(b) + 1e-3 * np.max(np.abs(b))))


@pytest.mark.parametrize("cfg,seed,n_prompt,n_gen", [
    (SMALL_LLAMA, 11, 250, 40), (SMALL_BITNET, 12, 270, 20), (SMALL_PACKED_HEAD, 13, 5, 30)])
def test_step_by_step_logits_and_tokens(tb, cfg, seed, n_prompt, n_gen):
    modelutil.build_gpu(tb, cfg, seed)
    om = modelutil.build_oracle(cfg, seed)
    prompt = np.random.default_rng(seed).integers(0, cfg["V"], size=n_prompt).astype(np.int32)
    want, want_logits = modelutil.oracle_generate(om, prompt, n_gen, want_logits=True)
    tb.model_reset(1)
    tok, got = int(prompt[0]), []
    for pos in range(n_prompt + n_gen - 1):
        nxt = int(tb.decode_step([tok], [pos])[0])
        if pos in (0, 1, n_prompt - 1, n_prompt + n_gen - 2) or pos % 37 == 0:
            lg = tb.model_logits()[0]
            assert rel_err(lg, want_logits[pos]) < 1e-3, pos
            assert np.array_equal(lg.view(np.uint32), want_logits[pos].view(np.uint32)), pos
        if pos + 1 < n_prompt:
            tok = int(prompt[pos + 1])
        else:
            tok = nxt
            got.append(nxt)
    assert got == want.tolist()
    # the graph-replayed generate() gives the same tokens
    out = tb.generate(prompt, n_gen)
    assert out[0].tolist() == want.tolist()
    assert tb.last_generate_ms() > 0
    assert tb.device_status() == 0


@pytest.mark.parametrize("cfg,seed,n_prompt", [(SMALL_LLAMA, 51, 300), (SMALL_BITNET, 52, 280)])
def test_persistent_kernel_and_launch_chain_agree(tb, cfg, seed, n_prompt):
    """One sequence runs embedding + all layers of a step in ONE persistent kernel (option
    "decode_persistent", default 1); the chain of per-stage launches must give the same bits, and the
    persistent step must be the shorter launch sequence."""
    modelutil.build_gpu(tb, cfg, seed)
    prompt = np.random.default_rng(seed).integers(0, cfg["V"], size=n_prompt).astype(np.int32)
    res = []
    try:
        for persistent in (1, 0):
            tb.set_option("decode_persistent", persistent)
            l0 = tb.launch_count()
            out = tb.generate(prompt, 12)
            res.append((out[0].copy(), tb.model_logits()[0].copy(), tb.launch_count() - l0))
    finally:
        tb.set_option("decode_persistent", 1)
    assert res[0][0].tolist() == res[1][0].tolist()
    assert np.array_equal(res[0][1].view(np.uint32), res[1][1].view(np.uint32))
    assert res[0][2] < res[1][2]
    assert tb.device_status() == 0


def test_bounded_wait_runs_out_and_the_context_survives(tb):
    """Inside the persistent kernel a CTA waits for values that other CTAs publish.  With the test hook
    "decode_fault_cta" one CTA keeps its q/k/v columns of layer 0 to itself, so its consumers' waits run out
    after "wait_ms": the kernel must return by itself, the call must report TER_B200_E_TIMEOUT, and the next
    call on the same handle must work and give the right tokens.  Nothing faults or hangs."""
    from ter_b200 import TerB200Error
    cfg, seed = SMALL_LLAMA, 61
    modelutil.build_gpu(tb, cfg, seed)
    om = modelutil.build_oracle(cfg, seed)
    prompt = np.random.default_rng(seed).integers(0, cfg["V"], size=5).astype(np.int32)
    want, _ = modelutil.oracle_generate(om, prompt, 6)
    assert tb.generate(prompt, 6)[0].tolist() == want.tolist()
    try:
        tb.set_option("wait_ms", 20)
        tb.set_option("decode_fault_cta", 147)       # owns the last strip of v in this model
        with pytest.raises(TerB200Error) as e:
            tb.generate(prompt, 6)
        assert e.value.code == api.E_TIMEOUT
    finally:
        tb.set_option("decode_fault_cta", -1)
        tb.set_option("wait_ms", 2000)
    assert tb.device_status() == 0                   # the status word was cleared by the failed call
    assert tb.generate(prompt, 6)[0].tolist() == want.tolist()
    assert tb.device_status() == 0


def test_batch_sequences_are_independent(tb):
    cfg, seed = SMALL_LLAMA, 21
    modelutil.build_gpu(tb, cfg, seed, max_batch=3)
    om = modelutil.build_oracle(cfg, seed)
    rng = np.random.default_rng(5)
    prompts = rng.integers(0, cfg["V"], size=(3, 12)).astype(np.int32)
    out = tb.generate(prompts, 10)
    for b in range(3):
        want, _ = modelutil.oracle_generate(om, prompts[b], 10)
        assert out[b].tolist() == want.tolist(), b
    # a smaller batch on the same handle, and position bounds
    out1 = tb.generate(prompts[1], 10)
    assert out1[0].tolist() == out[1].tolist()
    from ter_b200 import TerB200Error, api
    with pytest.raises(TerB200Error) as e:
        tb.generate(prompts[0], cfg["Smax"])          # would run past Smax
    assert e.value.code == api.E_SHAPE


@pytest.mark.parametrize("cfg,seed", [(SMALL_LLAMA, 41), (SMALL_BITNET, 42), (SMALL_PACKED_HEAD, 43)])
def test_token_batch_through_tensor_core_gemm(tb, cfg, seed):
    """Batches of at least 4 sequences take the tcgen05 GEMM for every projection; each sequence
    must still reproduce its own single-sequence tokens and logits exactly."""
    B = 9
    modelutil.build_gpu(tb, cfg, seed, max_batch=B)
    om = modelutil.build_oracle(cfg, seed)
    rng = np.random.default_rng(seed)
    prompts = rng.integers(0, cfg["V"], size=(B, 7)).astype(np.int32)
    out = tb.generate(prompts, 6)
    lg = tb.model_logits()
    for b in range(B):
        want, wl = modelutil.oracle_generate(om, prompts[b], 6, want_logits=True)
        assert out[b].tolist() == want.tolist(), b
        assert np.array_equal(lg[b].view(np.uint32), wl[-1].view(np.uint32)), b
    assert tb.device_status() == 0


def test_batch_of_sixteen_prompts_as_token_batches_and_tensor_core_lm_head(tb):
    """Sixteen sequences: the prompts run one sequence after the other as token batches, the decode steps take
    the tensor-core GEMM (bit-exact integer sums), and the lm_head runs on the tensor cores (rounding-level
    differences in the logits).
    Every sequence must reproduce its own single-sequence tokens; logits within 1e-4 of the largest."""
    cfg, seed, B = dict(SMALL_BITNET, H=512, V=3000), 71, 16
    modelutil.build_gpu(tb, cfg, seed, max_batch=B)
    om = modelutil.build_oracle(cfg, seed)
    prompts = np.random.default_rng(seed).integers(0, cfg["V"], size=(B, 21)).astype(np.int32)
    out = tb.generate(prompts, 5)
    lg = tb.model_logits()
    try:
        tb.set_option("lm_head_tc_min", 0)          # the exact CUDA-core lm_head for every batch size
        out_exact = tb.generate(prompts, 5)
        lg_exact = tb.model_logits()
    finally:
        tb.set_option("lm_head_tc_min", 16)
    for b in range(B):
        want, wl = modelutil.oracle_generate(om, prompts[b], 5, want_logits=True)
        assert out_exact[b].tolist() == want.tolist(), b
        assert np.array_equal(lg_exact[b].view(np.uint32), wl[-1].view(np.uint32)), b
        assert out[b].tolist() == want.tolist(), b
        assert np.max(np.abs(lg[b] - wl[-1])) <= 1e-4 * np.max(np.abs(wl[-1])), b
    assert tb.device_status() == 0


@pytest.mark.parametrize("cfg,seed", [(SMALL_LLAMA, 81), (SMALL_BITNET, 82)])
def test_opt_in_tensor_core_attention_stays_close(tb, cfg, seed):
    """Option "attn_mma_min" (off by default) sums the two contractions of attention on the tensor cores for
    token batches and prompt tiles.  Its output differs from the checker's in the last places, and the int8
    quantisers after it turn some of those differences into different roundings, so this path is NOT held to
    token equality: the logits at the end of a 40-position prompt must stay within 5 % of the largest logit, nothing may
    be NaN, and with the option off again the forward is the checker's bit for bit."""
    B = 8
    modelutil.build_gpu(tb, cfg, seed, max_batch=B)
    om = modelutil.build_oracle(cfg, seed)
    prompts = np.random.default_rng(seed).integers(0, cfg["V"], size=(B, 40)).astype(np.int32)
    tb.set_option("lm_head_tc_min", 0)
    try:
        tb.set_option("attn_mma_min", 2)
        tb.generate(prompts, 1)
        lg_mma = tb.model_logits().copy()
        tb.set_option("attn_mma_min", 0)
        out = tb.generate(prompts, 1)
        lg = tb.model_logits().copy()
    finally:
        tb.set_option("attn_mma_min", 0)
        tb.set_option("lm_head_tc_min", 16)
    assert not np.isnan(lg_mma).any()
    for b in range(B):
        want, wl = modelutil.oracle_generate(om, prompts[b], 1, want_logits=True)
        assert out[b].tolist() == want.tolist(), b
        assert np.array_equal(lg[b].view(np.uint32), wl[-1].view(np.uint32)), b
    # both runs fed the same 40 prompt tokens: the logits of the last prompt position
    assert np.max(np.abs(lg_mma - lg)) <= 5e-2 * np.max(np.abs(lg)), float(np.max(np.abs(lg_mma - lg)) / np.max(np.abs(lg)))
    assert tb.device_status() == 0


def test_reference_numpy_forward_tokens_on_gpu(tb, golden_dir):
    """Greedy tokens printed by the reference's own tools/llama_pyfwd.py / bitnet_pyfwd.py."""
    import make_pyfwd_golden as mk
    g = np.load(os.path.join(golden_dir, "pyfwd_tokens.npz"))
    for name in ("llama", "bitnet"):
        case = mk.CASES[name]
        cfg = {k: case[k] for k in ("arch", "H", "F", "L", "V", "Nh", "Nkv", "Hd", "Smax", "eps", "rope_theta")}
        modelutil.build_gpu(tb, cfg, case["seed"])
        want = g[f"{name}_tokens"]
        out = tb.generate(np.array([128000], np.int32), len(want))
        assert out[0].tolist() == want.tolist(), name


@pytest.mark.parametrize("cfg,seed", [(SMALL_LLAMA, 41), (SMALL_BITNET, 42), (SMALL_PACKED_HEAD, 43)])
def test_prompt_as_token_batches_equals_one_position_at_a_time(tb, cfg, seed):
    """Prompt processing through the tensor-core GEMM (passes of `prefill_tile` positions, causal attention
    over the shared cache) leaves tokens and logits bit-identical to feeding the prompt position by position."""
    rng = np.random.default_rng(seed)
    lengths = [2, 17, 40] if cfg["Smax"] < 300 else [2, 17, 255, 256, 290]
    try:
        tb.set_option("prefill_tile", 64)     # several passes per prompt, ragged last pass
        for n_prompt in lengths:
            n_gen = min(6, cfg["Smax"] - n_prompt + 1)
            prompt = rng.integers(0, cfg["V"], size=n_prompt).astype(np.int32)
            res = []
            for prefill in (0, 1):
                tb.set_option("prefill", prefill)
                modelutil.build_gpu(tb, cfg, seed)
                out = tb.generate(prompt, n_gen)
                res.append((out[0].copy(), tb.model_logits()[0].copy(), tb.last_prefill_ms()))
            assert res[0][2] == 0.0 and res[1][2] > 0.0
            assert res[0][0].tolist() == res[1][0].tolist(), n_prompt
            assert np.array_equal(res[0][1].view(np.uint32), res[1][1].view(np.uint32)), n_prompt
            assert tb.device_status() == 0
    finally:
        tb.set_option("prefill", 1)
        tb.set_option("prefill_tile", 1024)


def test_packed_model_files_load_and_reproduce_reference_tokens(tb, golden_dir, tmp_path):
    """'LLRT' and 'TERT' files byte-identical to the ones the reference's scripts were run on, read by
    the library's loader: the greedy tokens are the ones those scripts printed."""
    import make_pyfwd_golden as mk
    from ter_b200 import TerB200Error, modelfile
    g = np.load(os.path.join(golden_dir, "pyfwd_tokens.npz"))
    for name in ("llama", "bitnet"):
        case = mk.CASES[name]
        path = str(tmp_path / f"{name}.bin")
        modelfile.write_packed_model(path, case, synth.model_weights(case, case["seed"]))
        cfg = tb.model_load_file(path)
        assert (cfg["arch"], cfg["H"], cfg["L"], cfg["Smax"]) == (case["arch"], case["H"], case["L"], case["Smax"])
        want = g[f"{name}_tokens"]
        out = tb.generate(np.array([128000], np.int32), len(want))
        assert out[0].tolist() == want.tolist(), name
        # a longer context than the file's, and a truncated file
        cfg2 = tb.model_load_file(path, smax=96)
        assert cfg2["Smax"] == 96
        assert tb.generate(np.array([128000], np.int32), len(want))[0].tolist() == want.tolist()
        cut = str(tmp_path / f"{name}_cut.bin")
        with open(path, "rb") as f, open(cut, "wb") as o:
            o.write(f.read(os.path.getsize(path) - 1000))
        with pytest.raises(TerB200Error) as ei:
            tb.model_load_file(cut)
        assert ei.value.code == api.E_IO


@pytest.mark.parametrize("base,L", [(synth.LLAMA_1B_CFG, 3), (synth.BITNET_2B_CFG, 2)])
def test_full_size_shapes_few_layers(tb, base, L):
    """The real layer shapes and vocabulary of the two benchmark architectures, a few layers deep."""
    cfg = dict(base, L=L, Smax=64)
    modelutil.build_gpu(tb, cfg, 31)
    om = modelutil.build_oracle(cfg, 31)
    prompt = np.random.default_rng(1).integers(0, cfg["V"], size=6).astype(np.int32)
    want, want_logits = modelutil.oracle_generate(om, prompt, 4, want_logits=True)
    out = tb.generate(prompt, 4)
    assert out[0].tolist() == want.tolist()
    lg = tb.model_logits()[0]
    assert rel_err(lg, want_logits[-1]) < 1e-3
    assert np.array_equal(lg.view(np.uint32), want_logits[-1].view(np.uint32))


def test_long_prompt_at_full_width_through_the_token_batch_path(tb):
    """One BitNet-2B layer at full width and the benchmark's cache length, a 520-position prompt: the prompt runs
    as token batches (three token tiles, so the gate+up group takes the two-tiles-per-CTA form of the GEMM and the
    rows' attention the three-CTA form); the decode steps after it run in the persistent kernel with three context
    chunks and, at this cache length, two attention items per KV head.  The checker is fed one position at a time.
    Same tokens; logits of the last step bit for bit."""
    cfg = dict(synth.BITNET_2B_CFG, L=1, Smax=2176)
    n_gen = 4
    modelutil.build_gpu(tb, cfg, 33)
    om = modelutil.build_oracle(cfg, 33)
    prompt = np.random.default_rng(2).integers(0, cfg["V"], size=520).astype(np.int32)
    st = om.new_state(1)
    for pos in range(len(prompt) - 1):
        om.forward(st, 0, int(prompt[pos]), pos, want_logits=False)
    tok, want, want_lg = int(prompt[-1]), [], None
    for i in range(n_gen):
        tok, want_lg, _ = om.forward(st, 0, tok, len(prompt) - 1 + i, want_logits=True)
        want.append(int(tok))
    out = tb.generate(prompt, n_gen)
    assert tb.last_prefill_ms() > 0.0                   # the prompt did run as token batches
    lg = tb.model_logits()[0]
    assert out[0].tolist() == want
    assert np.array_equal(lg.view(np.uint32), want_lg.view(np.uint32))
    assert tb.device_status() == 0


def test_command_line_front_end_prints_the_reference_tokens(golden_dir, tmp_path):
    """ter_b200_generate (the counterpart of the reference programs' main(): n_gen, model file) on a packed-model
    file: greedy tokens from BOS equal to the ones the reference's NumPy forward printed, with the device
    sampler and with the host argmax sampler; the op-count report comes in the reference's format."""
    import re
    import subprocess
    import make_pyfwd_golden as mk
    from ter_b200 import build, modelfile
    g = np.load(os.path.join(golden_dir, "pyfwd_tokens.npz"))
    for name in ("llama", "bitnet"):
        case = mk.CASES[name]
        path = str(tmp_path / f"{name}.bin")
        modelfile.write_packed_model(path, case, synth.model_weights(case, case["seed"]))
        want = g[f"{name}_tokens"].tolist()
        for extra in ([], ["--host-sampler"], ["--op-stats"]):
            r = subprocess.run([build.CLI, str(len(want)), path] + extra, capture_output=True, text=True, timeout=600)
            assert r.returncode == 0, r.stdout[-500:] + r.stderr[-500:]
            line = r.stdout.split("Greedy tokens")[1].splitlines()[1]
            assert [int(t) for t in line.split()] == want, (name, extra)
            if extra == ["--op-stats"]:
                assert "=== op-stats:" in r.stderr and "TVMAC" in r.stderr
                tv = int(re.search(r"TVMAC\s*:\s*(\d+)", r.stderr).group(1))
                assert tv > 0


def test_dispatch_rule_names_the_kernel(tb):
    """ter_b200_pick_kernel is the one rule every launch goes through."""
    assert tb.pick_kernel(1, 2048, 512) == "gemv_trit_split_kernel"
    assert tb.pick_kernel(1, 2048, 128256) == "gemv_trit_kernel"
    assert tb.pick_kernel(8, 2560, 6912) == "gemv_trit_rows_kernel"
    assert tb.pick_kernel(9, 2560, 6912) == "gemm_trit_kernel"
    assert tb.pick_kernel(64, 2560, 6912) == "gemm_trit_kernel"
    try:
        tb.set_option("gemm_min_m", 4)
        assert tb.pick_kernel(8, 2560, 6912) == "gemm_trit_kernel"
        tb.set_option("gemm_min_m", 17)
        assert tb.pick_kernel(16, 2560, 6912) == "gemv_trit_rows_kernel"
    finally:
        tb.set_option("gemm_min_m", 9)


def test_model_state_errors(tb):
    from ter_b200 import TerB200, TerB200Error, api
    h = TerB200(0)
    try:
        assert h.L.ter_b200_decode_step(h.h, None, None, None, None) == api.E_STATE      # no model yet
        with pytest.raises(TerB200Error):
            h.model_create(dict(SMALL_LLAMA, Hd=48))                                     # unsupported head_dim
        h.model_create(SMALL_LLAMA)
        assert h.L.ter_b200_decode_step(h.h, None, None, None, None) == api.E_STATE      # weights missing
    finally:
        h.close()
