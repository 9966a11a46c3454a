"""Pins the CPU checker (oracle/) before anything trusts it:
against committed outputs of the unmodified reference (tests/golden, made by
tests/golden/make_golden.py), against the reference library itself where it is present
(oracle/_ref), and against the reference's own known-answer recipes."""
import hashlib
import os
import sys

import numpy as np
import pytest

import oracle
from ter_b200 import synth

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
import make_golden  # noqa: E402

have_ref = pytest.mark.skipif(not oracle.Ref.available(), reason="reference library not built here")


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def test_mm_row_matches_golden(golden_dir):
    g = np.load(os.path.join(golden_dir, "mm_row_small.npz"))
    for i in range(6):
        W, X, s, out = g[f"W{i}"].astype(np.int32), g[f"X{i}"], g[f"s{i}"], g[f"out{i}"]
        for r in range(X.shape[0]):
            got = oracle.mm_row(X[r], s[0], W, s[1])
            assert np.array_equal(bits(got), bits(out[r])), (i, r)
    got = np.stack([oracle.mm_row(g["X9"][r], g["s9"][0], g["W9"], g["s9"][1]) for r in range(2)])
    assert np.array_equal(bits(got), bits(g["out9"]))


def test_quantize_matches_golden(golden_dir):
    g = np.load(os.path.join(golden_dir, "mm_row_small.npz"))
    for i in range(3):
        for nt in (2, 9):
            q, s = oracle.quantize_trit(g[f"qv{i}"], nt)
            assert np.array_equal(q, g[f"qq{i}_{nt}"])
            assert np.float32(s) == g[f"qs{i}_{nt}"][0]


def test_int4tc_recipe_bit_exact(golden_dir):
    """K=64,N=16 deterministic pattern (cuda/ter_cuda_forward_packed_v13_int4tc.cu:511-541):
    with both scales 1 the output IS the integer accumulator."""
    g = np.load(os.path.join(golden_dir, "mm_row_recipes.npz"))
    x, t = make_golden.int4tc_pattern()
    acc = oracle.mm_row_acc(x.astype(np.int32), t.astype(np.int32))
    assert np.array_equal(acc.astype(np.float32), g["int4tc_out"])
    assert np.array_equal(oracle.gemv_packed_acc(x, oracle.pack_v11(t), 64, 16).astype(np.int64), acc)
    # TVMAC counter formula, pinned by tests/test_kernel_matmul_b_32.cpp:88-89
    assert oracle.tvmac(64, 16) == int(g["int4tc_tvmac"][0]) == ((64 + 26) // 27) * 16


@pytest.mark.parametrize("name,K,N", make_golden.CORRECTNESS_SHAPES)
def test_correctness_recipe_shapes(golden_dir, name, K, N):
    """The four shapes of tests/cuda_forward_correctness.cu:77-123 (scale_x 0.0312, w_scale 0.05)."""
    g = np.load(os.path.join(golden_dir, "mm_row_recipes.npz"))
    x, t = make_golden.correctness_inputs(name, K, N)
    assert hashlib.sha256(x.tobytes() + t.tobytes()).digest() == g[f"{name}_x_sha256"].tobytes()
    acc = oracle.gemv_acc_fast(x, t)
    out = oracle.gemv_epilogue(acc, 0.0312, 0.05)
    assert np.array_equal(bits(out[:16]), bits(g[f"{name}_head"]))
    assert hashlib.sha256(out.tobytes()).digest() == g[f"{name}_sha256"].tobytes()
    if K * N <= 2048 * 512:   # the scalar packed loop as well, on the smaller shapes
        acc2 = oracle.gemv_packed_acc(x, oracle.pack_v11(t), K, N)
        assert np.array_equal(acc2, acc)


def test_numpy_64x64_exact():
    """tools/matmul_reference.py:8-22 + tests/test_matmul_reference.cpp:33-62: exact int64."""
    rng = np.random.default_rng(0xC0FFEE)
    A = rng.integers(-9841, 9842, size=(64, 64), dtype=np.int32)
    B = rng.integers(-9841, 9842, size=(64, 64), dtype=np.int32)
    Cref = A.astype(np.int64) @ B.astype(np.int64)
    for i in range(64):
        assert np.array_equal(oracle.mm_row_acc(A[i], B), Cref[i])


@have_ref
def test_mm_row_against_reference_library():
    ref = oracle.Ref()
    rng = np.random.default_rng(7)
    for K, N in [(8, 4), (100, 36), (512, 256), (2048, 512)]:
        W = rng.choice([-1, 0, 1], size=(K, N), p=[0.3, 0.4, 0.3]).astype(np.int32)
        X = rng.integers(-128, 128, size=K).astype(np.int32)
        xs, ws = float(np.float32(rng.uniform(1e-3, 1e-1))), float(np.float32(rng.uniform(0.01, 0.05)))
        ref.reset_counters()
        a = ref.mm_row(X, xs, W, ws)
        assert ref.tvmac() == oracle.tvmac(K, N)
        assert np.array_equal(bits(a), bits(oracle.mm_row(X, xs, W, ws)))
        # the packed GPU-path semantics give the same floats for int8 activations
        acc = oracle.gemv_packed_acc(X.astype(np.int8), oracle.pack_v11(W.astype(np.int8)), K, N) \
            if K * N <= 512 * 256 else oracle.gemv_acc_fast(X.astype(np.int8), W.astype(np.int8))
        assert np.array_equal(bits(oracle.gemv_epilogue(acc, xs, ws)), bits(a))


@have_ref
def test_quantize_against_reference_library():
    ref = oracle.Ref()
    rng = np.random.default_rng(11)
    for n in (1, 5, 333, 4096):
        v = (rng.standard_normal(n) * 3).astype(np.float32)
        for nt in (1, 2, 5, 9):
            q, s = ref.quantize(v, nt)
            q2, s2 = oracle.quantize_trit(v, nt)
            assert np.array_equal(q, q2) and np.float32(s) == np.float32(s2)
    q, s = oracle.quantize_trit(np.zeros(8, np.float32), 9)
    assert s == 0.0 and not q.any()          # all-zero input -> scale 0 (quantize.cpp:22-25)


def test_pack_layouts_roundtrip_and_code3():
    t = synth.trits(64, 32, 3)
    v11, rm = oracle.pack_v11(t), oracle.pack_rowmajor(t)
    assert np.array_equal(v11, synth.pack_v11(t)) and np.array_equal(rm, synth.pack_rowmajor(t))
    assert np.array_equal(rm.T, v11)                      # one is the byte-transpose of the other
    assert np.array_equal(oracle.unpack_v11(v11, 64, 32), t)
    assert np.array_equal(oracle.unpack_rowmajor(rm, 64, 32), t)
    assert np.array_equal(synth.unpack_v11(v11, 64, 32), t)
    # code 3 decodes to 0 (cuda/ter_cuda_forward_packed.cu:371-372)
    allc = np.arange(256, dtype=np.uint8).reshape(1, 256)
    dec = oracle.unpack_v11(allc, 256, 4)
    for b in range(256):
        for f in range(4):
            c = (b >> (2 * f)) & 3
            assert dec[b, f] == (1 if c == 1 else -1 if c == 2 else 0)


def test_quantiser_properties():
    """Bounds from tests/test_numfmt_quantize.cpp:9-53 restated for the int8 quantiser:
    |q| <= 127, the absmax element maps to +-127, dequantised error <= scale/2."""
    rng = np.random.default_rng(5)
    for n in (16, 2048, 8192):
        x = rng.standard_normal(n).astype(np.float32)
        q, s = oracle.quant_int8(x)
        q2, s2 = synth.quant_int8(x)
        assert np.array_equal(q, q2) and s == s2
        assert np.abs(q.astype(int)).max() == 127
        assert np.all(np.abs(q.astype(np.float32) * s - x) <= s * 0.5001)
        qq, ss, normed = oracle.rmsnorm_quant(x, np.ones(n, np.float32), 1e-5)
        ref = x / np.sqrt(np.mean(x.astype(np.float64) ** 2) + 1e-5)
        assert np.allclose(normed, ref, rtol=2e-6, atol=1e-7)


def test_expf_and_bf16():
    xs = np.linspace(-86, 86, 4001).astype(np.float32)
    got = np.array([oracle.expf(float(v)) for v in xs])
    assert np.max(np.abs(got - np.exp(xs.astype(np.float64))) / np.exp(xs.astype(np.float64))) < 2e-7
    assert oracle.expf(-100.0) == 0.0
    import torch
    v = np.random.default_rng(1).standard_normal(4096).astype(np.float32)
    want = torch.from_numpy(v).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(oracle.f32_to_bf16(v), want)
    assert np.array_equal(np.array([oracle.lib().orc_f32_to_bf16(oracle.C.c_float(float(a))) for a in v[:64]],
                                   dtype=np.uint16), want[:64])


def test_attention_chunked_vs_twopass():
    rng = np.random.default_rng(9)
    for (Nh, Nkv, Hd, T) in [(4, 2, 64, 1), (4, 2, 64, 77), (8, 2, 128, 300), (4, 1, 64, 700)]:
        smax = 768
        q = rng.standard_normal(Nh * Hd).astype(np.float32)
        kc = oracle.f32_to_bf16(rng.standard_normal((Nkv, smax, Hd)).astype(np.float32))
        vc = oracle.f32_to_bf16(rng.standard_normal((Nkv, smax, Hd)).astype(np.float32))
        a = oracle.attention(q, kc, vc, Nh, Nkv, Hd, smax, T)
        b = oracle.attention(q, kc, vc, Nh, Nkv, Hd, smax, T, twopass=True)
        assert np.allclose(a, b, rtol=2e-5, atol=2e-6)


def test_rope_conventions():
    """Interleaved pairs (2k,2k+1) for Llama, half-split (k,k+Hd/2) for BitNet
    (cuda/ter_cuda_forward_packed.cu:64-76, cuda/ter_cuda_forward_bitnet.cu:185-201)."""
    Hd, pos, theta = 64, 37, 500000.0
    tab = oracle.rope_table(64, Hd, theta)
    v = np.random.default_rng(2).standard_normal(2 * Hd).astype(np.float32)
    k = np.arange(Hd // 2)
    ang = pos / theta ** (2.0 * k / Hd)
    c, s = np.cos(ang), np.sin(ang)
    a = oracle.rope(v, 2, Hd, tab[pos], neox=0).reshape(2, Hd)
    b = oracle.rope(v, 2, Hd, tab[pos], neox=1).reshape(2, Hd)
    vv = v.reshape(2, Hd).astype(np.float64)
    assert np.allclose(a[:, 0::2], vv[:, 0::2] * c - vv[:, 1::2] * s, atol=1e-6)
    assert np.allclose(a[:, 1::2], vv[:, 0::2] * s + vv[:, 1::2] * c, atol=1e-6)
    assert np.allclose(b[:, :32], vv[:, :32] * c - vv[:, 32:] * s, atol=1e-6)
    assert np.allclose(b[:, 32:], vv[:, :32] * s + vv[:, 32:] * c, atol=1e-6)


def test_i2s_decode_and_converter_against_the_reference_decoder(golden_dir):
    """microsoft/BitNet i2_s tensors: the checker's decode and the library's host-side converter
    (ter_b200_convert_i2s, no GPU needed) against values decoded by the reference's own nt::dequant_i2_s
    (committed fixture; live when oracle/_ref is present), and the reference test's own known-answer block
    (tests/test_nt_dequant.cpp:37-60: all code bytes 0x1B, scale 2)."""
    from ter_b200 import api, synth
    g = np.load(os.path.join(golden_dir, "i2s_blocks.npz"))
    raw, N, K = g["raw"], int(g["N"][0]), int(g["K"][0])
    trits, scale = oracle.i2s_decode(raw, N * K)
    assert np.array_equal(trits.astype(np.float32) * np.float32(scale), g["dequant"])
    if oracle.Ref.available():
        assert np.array_equal(oracle.Ref().dequant_i2s(raw, N * K), g["dequant"])
    v11, sc = api.convert_i2s(raw, N, K)
    assert sc == np.float32(0.0371)
    # the tensor is N output rows x K inputs; the library's matrices are [K][N]
    want = synth.pack_v11(np.ascontiguousarray(trits.reshape(N, K).T))
    assert np.array_equal(v11, want)
    # the reference test's block: positions 0..31 -> -1, 32..63 -> 0, 64..95 -> +1, 96..127 -> 0
    blk = np.concatenate([np.full(32, 0x1B, np.uint8), np.array([2.0], np.float32).view(np.uint8), np.zeros(28, np.uint8)])
    t1, s1 = oracle.i2s_decode(blk, 128)
    assert s1 == 2.0 and np.all(t1[:32] == -1) and np.all(t1[32:64] == 0) and np.all(t1[64:96] == 1) and np.all(t1[96:] == 0)
    v1, _ = api.convert_i2s(blk, 4, 32)
    assert np.array_equal(v1, synth.pack_v11(np.ascontiguousarray(t1.reshape(4, 32).T)))
    # errors are return codes
    with pytest.raises(api.TerB200Error) as e:
        api.convert_i2s(raw[:100], N, K)
    assert e.value.code == api.E_IO
