"""Parity of the CUDA GEMV with the CPU checker, through the C ABI.
Integer accumulators: bit-exact.  Scaled fp32 outputs: bit-exact too (one fp32 multiply),
asserted at the 1e-3 relative tolerance the specification states and at equality."""
import numpy as np
import pytest
import torch

import oracle
from ter_b200 import FMT_I32, FMT_ROWMAJOR, FMT_V11, TerB200Error, api, synth

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def exact_acc(x, t):
    # float64 BLAS is exact here: every partial sum is an integer far below 2^53
    return (x.astype(np.float64) @ t.astype(np.float64)).astype(np.int64)


def run_case(tb, K, N, seed, fmt=FMT_V11, name="w"):
    t = synth.trits(K, N, seed)
    ws = synth.weight_scale(seed)
    x, xs = synth.activation(K, seed)
    if fmt == FMT_V11:
        data = synth.pack_v11(t)
    elif fmt == FMT_ROWMAJOR:
        data = synth.pack_rowmajor(t)
    else:
        data = t.astype(np.int32)
    tb.install(name, data, fmt, K, N, float(ws))
    xd, sd = dev(x), dev(np.array([xs], np.float32))
    acc = tb.gemv_acc(name, xd).cpu().numpy()
    out = tb.gemv(name, xd, sd).cpu().numpy()
    want = exact_acc(x, t)
    assert np.array_equal(acc.astype(np.int64), want), f"int32 mismatch K={K} N={N}"
    want_f = oracle.gemv_epilogue(want.astype(np.int32), xs, ws)
    assert np.allclose(out, want_f, rtol=1e-3, atol=0)
    assert np.array_equal(out.view(np.uint32), want_f.view(np.uint32))
    return t, x, xs, ws


@pytest.mark.parametrize("K,N", [(16, 4), (64, 16), (128, 64), (432, 80), (2048, 512), (2560, 640)])
def test_small_shapes_vs_scalar_oracle(tb, K, N):
    t, x, xs, ws = run_case(tb, K, N, seed=K * 7 + N)
    # the scalar packed-loop checker and the reference-form mm_row agree as well
    acc = tb.gemv_acc("w", dev(x)).cpu().numpy()
    assert np.array_equal(acc, oracle.gemv_packed_acc(x, synth.pack_v11(t), K, N))
    mm = oracle.mm_row(x.astype(np.int32), xs, t.astype(np.int32), ws)
    assert np.array_equal(tb.gemv("w", dev(x), dev(np.array([xs], np.float32))).cpu().numpy().view(np.uint32),
                          mm.view(np.uint32))


@pytest.mark.parametrize("name,shape", list(synth.LLAMA_1B_SHAPES.items()) + list(synth.BITNET_2B_SHAPES.items()))
def test_model_shapes_bit_exact(tb, name, shape):
    K, N = shape
    run_case(tb, K, N, seed=synth.seed_for(K, N, name))


@pytest.mark.parametrize("fmt", [FMT_ROWMAJOR, FMT_I32])
def test_other_boundary_formats(tb, fmt):
    run_case(tb, 256, 96, seed=5, fmt=fmt)
    run_case(tb, 2048, 2048, seed=6, fmt=fmt)


def test_i32_format_non_multiple_of_4_columns(tb):
    K, N = 64, 10
    t = synth.trits(K, N, 1)
    tb.install("odd", t.astype(np.int32), FMT_I32, K, N, 1.0)
    x, _ = synth.activation(K, 2)
    assert np.array_equal(tb.gemv_acc("odd", dev(x)).cpu().numpy().astype(np.int64), exact_acc(x, t))


def test_code3_is_zero_and_extreme_values(tb):
    K, N = 256, 64
    rng = np.random.default_rng(3)
    raw = rng.integers(0, 256, size=(N // 4, K), dtype=np.uint8)      # all byte values, code 3 included
    t = synth.unpack_v11(raw, K, N)
    tb.install("raw", raw, FMT_V11, K, N, 0.05)
    for x in (np.full(K, -128, np.int8), np.full(K, 127, np.int8), np.zeros(K, np.int8),
              rng.integers(-128, 128, size=K).astype(np.int8)):
        assert np.array_equal(tb.gemv_acc("raw", dev(x)).cpu().numpy().astype(np.int64), exact_acc(x, t))
    # all +1 / all -1 weights at the largest K: the extreme accumulator magnitudes
    K, N = 8192, 16
    for sign in (1, -1):
        t = np.full((K, N), sign, np.int8)
        tb.install("ext", synth.pack_v11(t), FMT_V11, K, N, 1.0)
        for xv in (-128, 127):
            x = np.full(K, xv, np.int8)
            assert np.array_equal(tb.gemv_acc("ext", dev(x)).cpu().numpy().astype(np.int64), exact_acc(x, t))


def test_known_answer_recipes(tb, golden_dir):
    """The reference's own recipes, checked against outputs of the unmodified reference mm_row."""
    import hashlib
    import os
    import sys
    sys.path.insert(0, golden_dir)
    import make_golden
    g = np.load(os.path.join(golden_dir, "mm_row_recipes.npz"))
    x, t = make_golden.int4tc_pattern()
    tb.install("kat", synth.pack_v11(t), FMT_V11, 64, 16, 1.0)
    out = tb.gemv("kat", dev(x), dev(np.ones(1, np.float32))).cpu().numpy()
    assert np.array_equal(out, g["int4tc_out"])
    for name, K, N in make_golden.CORRECTNESS_SHAPES:
        x, t = make_golden.correctness_inputs(name, K, N)
        tb.install("kat", synth.pack_v11(t), FMT_V11, K, N, 0.05)
        out = tb.gemv("kat", dev(x), dev(np.array([0.0312], np.float32))).cpu().numpy()
        assert hashlib.sha256(out.tobytes()).digest() == g[f"{name}_sha256"].tobytes(), name


def test_group_launch_matches_single(tb):
    K = 2048
    names, xs_all = [], []
    for nm, N in (("gq", 2048), ("gk", 512), ("gv", 512)):
        t = synth.trits(K, N, synth.seed_for(nm))
        tb.install(nm, synth.pack_v11(t), FMT_V11, K, N, float(synth.weight_scale(N)))
        names.append(nm)
    x, xs = synth.activation(K, 77)
    xd, sd = dev(x), dev(np.array([xs], np.float32))
    outs = tb.gemv_group(names, xd, sd)
    for nm, o in zip(names, outs):
        assert torch.equal(o, tb.gemv(nm, xd, sd))


def test_multi_launch_matches_single(tb):
    """Independent GEMVs with different K and different activations in one launch."""
    specs = [("mq", 2048, 2048), ("mk", 2048, 512), ("md", 8192, 2048), ("mo", 2048, 2048), ("mg", 2560, 640)]
    xs, scs, names = {}, {}, []
    for nm, K, N in specs:
        tb.install(nm, synth.pack_v11(synth.trits(K, N, synth.seed_for(nm))), FMT_V11, K, N, float(synth.weight_scale(N + K)))
        names.append(nm)
    for K in (2048, 8192, 2560):
        x, s = synth.activation(K, K)
        xs[K], scs[K] = dev(x), dev(np.array([s], np.float32))
    x2, s2 = synth.activation(2048, 5)
    xin = [xs[2048], xs[2048], xs[8192], dev(x2), xs[2560]]
    sin = [scs[2048], scs[2048], scs[8192], dev(np.array([s2], np.float32)), scs[2560]]
    outs = tb.gemv_multi(names, xin, sin)
    for nm, x, s, o in zip(names, xin, sin, outs):
        assert torch.equal(o, tb.gemv(nm, x, s)), nm
    assert tb.device_status() == 0


def test_linearity_and_tuning_invariance(tb):
    """Size-independent properties at a full-size shape: acc(x1)+acc(x2) == acc(x1+x2) (no clamp),
    and the result does not depend on grid/stage choices."""
    K, N = 8192, 2048
    t = synth.trits(K, N, 99)
    tb.install("lin", synth.pack_v11(t), FMT_V11, K, N, 0.02)
    rng = np.random.default_rng(4)
    x1 = rng.integers(-60, 60, size=K).astype(np.int8)
    x2 = rng.integers(-60, 60, size=K).astype(np.int8)
    a1, a2 = tb.gemv_acc("lin", dev(x1)), tb.gemv_acc("lin", dev(x2))
    a12 = tb.gemv_acc("lin", dev((x1 + x2).astype(np.int8)))
    assert torch.equal(a1 + a2, a12)
    base = a12.clone()
    for ctas, stages, pdl in [(1, 2, 0), (2, 3, 1), (8, 1, 1), (3, 8, 0)]:
        tb.set_option("gemv_ctas_per_sm", ctas)
        tb.set_option("gemv_stages", stages)
        tb.set_option("pdl", pdl)
        assert torch.equal(tb.gemv_acc("lin", dev((x1 + x2).astype(np.int8))), base)
    tb.set_option("gemv_ctas_per_sm", 4)
    tb.set_option("gemv_stages", 0)
    tb.set_option("pdl", 1)


def test_counters_follow_mm_row_formula(tb):
    tb.install("cnt", synth.pack_v11(synth.trits(128, 64, 1)), FMT_V11, 128, 64, 1.0)
    tb.reset_counters()
    x, _ = synth.activation(128, 1)
    tb.gemv_acc("cnt", dev(x))
    tb.gemv_acc("cnt", dev(x))
    c = tb.op_counts()
    assert c["tvmac"] == 2 * oracle.tvmac(128, 64) == c["total_ops"]
    assert tb.launch_count() == 2
    tb.reset_counters()
    assert tb.op_counts()["tvmac"] == 0


def test_error_paths(tb):
    x = torch.zeros(128, dtype=torch.int8, device="cuda")
    s = torch.ones(1, device="cuda")
    with pytest.raises(TerB200Error) as e:
        tb.install("bad", np.zeros((3, 30), np.uint8), FMT_V11, 30, 12, 1.0)     # K not a multiple of 16
    assert e.value.code == api.E_SHAPE
    with pytest.raises(TerB200Error) as e:
        tb.install("bad", np.full((16, 8), 2, np.int32), FMT_I32, 16, 8, 1.0)    # value outside {-1,0,1}
    assert e.value.code == api.E_VALUE
    with pytest.raises(TerB200Error) as e:
        tb.install("n" * 32, np.zeros((1, 16), np.uint8), FMT_V11, 16, 4, 1.0)
    assert e.value.code == api.E_NAME
    assert tb.L.ter_b200_gemv(tb.h, b"nonexistent", x.data_ptr(), s.data_ptr(), x.data_ptr(), None) == api.E_UNKNOWN
    assert tb.call("nonexistent_kernel", []) == api.E_UNKNOWN          # tests/test_ter_k4.cpp:21-23
    assert tb.call("tk_matmul_b_9t", [0] * 8) == api.E_NARGS
    tb.install("al", synth.pack_v11(synth.trits(128, 16, 1)), FMT_V11, 128, 16, 1.0)
    xm = torch.zeros(256, dtype=torch.int8, device="cuda")[1:129]                 # misaligned x
    assert tb.L.ter_b200_gemv_acc(tb.h, b"al", xm.data_ptr(), x.data_ptr(), None) == api.E_SHAPE


def test_slot_table_limits(tb):
    from ter_b200 import TerB200
    h = TerB200(0)
    try:
        w = synth.pack_v11(synth.trits(16, 4, 1))
        for i in range(1024):
            h.install(f"s{i}", w, FMT_V11, 16, 4, 1.0)
        with pytest.raises(TerB200Error) as e:
            h.install("one_too_many", w, FMT_V11, 16, 4, 1.0)
        assert e.value.code == api.E_FULL
        h.install("s3", w, FMT_V11, 16, 4, 2.0)            # re-install replaces
        assert h.weight_info("s3") == (16, 4, 2.0)
        h.remove("s5")
        h.install("again", w, FMT_V11, 16, 4, 1.0)
        h.close()
        h.close()                                          # double destroy is harmless
    finally:
        h.close()


def test_call_and_blob_verbs(tb):
    import ctypes as C
    K, N = 256, 64
    t = synth.trits(K, N, 8)
    tb.install_blob("blob", synth.pack_v11(t), FMT_V11, K, N, 0.03)
    x, xs = synth.activation(K, 8)
    xd, sd = dev(x), dev(np.array([xs], np.float32))
    out = torch.empty(N, dtype=torch.float32, device="cuda")
    name = C.c_char_p(b"blob")
    st = torch.cuda.current_stream().cuda_stream
    rc = tb.call("tk_matmul_b_9t", [C.cast(name, C.c_void_p).value, xd.data_ptr(), sd.data_ptr(), out.data_ptr(), 1, st])
    assert rc == 0
    assert torch.equal(out, tb.gemv("blob", xd, sd))


def test_host_buffer_entry_point(tb):
    K, N = 2048, 2048
    t = synth.trits(K, N, 21)
    ws = synth.weight_scale(21)
    tb.install("hb", synth.pack_v11(t), FMT_V11, K, N, float(ws))
    x, xs = synth.activation(K, 21)
    xh = torch.from_numpy(x).pin_memory()
    oh = torch.empty(N, dtype=torch.float32).pin_memory()
    tb.gemv_host("hb", xh, float(xs), oh)
    tb.sync()
    want = oracle.gemv_epilogue(exact_acc(x, t).astype(np.int32), xs, ws)
    assert np.array_equal(oh.numpy().view(np.uint32), want.view(np.uint32))


def test_host_batch_entry_point(tb):
    specs = [("hb1", 256, 64), ("hb2", 2048, 512), ("hb3", 128, 96)]
    xs_h, outs_h, scales, wants = [], [], [], []
    for nm, K, N in specs:
        t = synth.trits(K, N, K + N)
        ws = synth.weight_scale(K)
        tb.install(nm, synth.pack_v11(t), FMT_V11, K, N, float(ws))
        x, xs = synth.activation(K, N)
        xs_h.append(torch.from_numpy(x).pin_memory())
        outs_h.append(torch.empty(N, dtype=torch.float32).pin_memory())
        scales.append(float(xs))
        wants.append(oracle.gemv_epilogue(exact_acc(x, t).astype(np.int32), xs, ws))
    plan = tb.gemv_host_batch_plan([s[0] for s in specs], xs_h, scales, outs_h)
    try:
        for direct in (1, 0):     # results written by the kernel into the pinned buffers / staged and copied
            tb.set_option("host_batch_direct", direct)
            for o in outs_h:
                o.fill_(float("nan"))
            tb.gemv_host_batch(plan)
            for o, w in zip(outs_h, wants):
                assert np.array_equal(o.numpy().view(np.uint32), w.view(np.uint32)), direct
        # pageable outputs always take the staged path
        pag = [np.full(N, np.nan, np.float32) for _, _, N in specs]
        tb.set_option("host_batch_direct", 1)
        tb.gemv_host_batch(tb.gemv_host_batch_plan([s[0] for s in specs], xs_h, scales, pag))
        for o, w in zip(pag, wants):
            assert np.array_equal(o.view(np.uint32), w.view(np.uint32))
    finally:
        tb.set_option("host_batch_direct", 1)


def test_host_batch_shared_vectors_contiguous_outputs_and_chunking(tb):
    """Shared x (one copy), outputs back to back (one copy down), and more distinct vectors than one
    launch stages (forces several launches)."""
    specs = [(f"hc{i}", 256 if i % 3 else 384, 64 + 16 * (i % 4)) for i in range(40)]
    shared = {K: synth.activation(K, K + 1) for K in (256, 384)}
    total = sum(N for _, _, N in specs)
    out_all = torch.full((total,), float("nan"), dtype=torch.float32).pin_memory()
    xs_h, outs_h, scales, wants, off = [], [], [], [], 0
    for i, (nm, K, N) in enumerate(specs):
        t = synth.trits(K, N, 7 * i + 1)
        ws = synth.weight_scale(i + 3)
        tb.install(nm, synth.pack_v11(t), FMT_V11, K, N, float(ws))
        if i < 12:
            x, xsc = shared[K]                      # same pointer for every user of this K
            key = ("s", K)
        else:
            x, xsc = synth.activation(K, 100 + i)   # its own vector: 28 distinct ones
            key = ("o", i)
        xs_h.append((key, x, xsc))
        outs_h.append(out_all[off:off + N])
        off += N
        scales.append(float(xsc))
        wants.append(oracle.gemv_epilogue(exact_acc(x, t).astype(np.int32), xsc, ws))
    pinned = {}
    for key, x, _ in xs_h:
        if key not in pinned:
            pinned[key] = torch.from_numpy(x).pin_memory()
    plan = tb.gemv_host_batch_plan([s[0] for s in specs], [pinned[k] for k, _, _ in xs_h], scales, outs_h)
    l0 = tb.launch_count()
    tb.gemv_host_batch(plan)
    assert tb.launch_count() - l0 == 2          # 2 shared + 28 own vectors: 16 per launch
    for o, w in zip(outs_h, wants):
        assert np.array_equal(o.numpy().view(np.uint32), w.view(np.uint32))
    assert tb.device_status() == 0
    for nm, _, _ in specs:
        tb.remove(nm)


def test_sweep_plan_matches_single_launches(tb):
    specs = [(f"sp{i}", (2048, 8192, 2560, 128)[i % 4], (512, 2048, 640, 96, 4096)[i % 5]) for i in range(23)]
    xs = {}
    for K in (2048, 8192, 2560, 128):
        x, s = synth.activation(K, K + 9)
        xs[K] = (dev(x), dev(np.array([s], np.float32)))
    names, xin, sin, outs = [], [], [], []
    for i, (nm, K, N) in enumerate(specs):
        tb.install(nm, synth.pack_v11(synth.trits(K, N, 11 * i + 2)), FMT_V11, K, N, float(synth.weight_scale(i)))
        names.append(nm)
        xin.append(xs[K][0])
        sin.append(xs[K][1])
        outs.append(torch.full((N,), float("nan"), dtype=torch.float32, device="cuda"))
    pid = tb.gemv_plan(names, xin, sin, outs)
    l0 = tb.launch_count()
    tb.gemv_plan_launch(pid)
    tb.sync()
    assert tb.launch_count() - l0 == 1
    for nm, x, s, o in zip(names, xin, sin, outs):
        assert torch.equal(o, tb.gemv(nm, x, s)), nm
    # the plan reads x where it lies: new activations, same plan
    x2, s2 = synth.activation(2048, 77)
    xs[2048][0].copy_(torch.from_numpy(x2))
    xs[2048][1].fill_(float(s2))
    tb.gemv_plan_launch(pid)
    tb.sync()
    for nm, x, s, o in zip(names, xin, sin, outs):
        assert torch.equal(o, tb.gemv(nm, x, s)), nm
    # any change of the weight slots makes the plan stale
    tb.remove(names[-1])
    with pytest.raises(RuntimeError):
        tb.gemv_plan_launch(pid)
    tb.gemv_plan_destroy(pid)
    assert tb.device_status() == 0
    for nm in names[:-1]:
        tb.remove(nm)


def test_gemm_rows_match_gemv(tb):
    K, N, M = 2560, 640, 5
    t = synth.trits(K, N, 31)
    tb.install("gm", synth.pack_v11(t), FMT_V11, K, N, 0.04)
    rng = np.random.default_rng(1)
    X = rng.integers(-128, 128, size=(M, K)).astype(np.int8)
    xs = rng.uniform(0.001, 0.1, size=M).astype(np.float32)
    acc = tb.gemm_acc("gm", dev(X)).cpu().numpy()
    assert np.array_equal(acc.astype(np.int64), (X.astype(np.float64) @ t.astype(np.float64)).astype(np.int64))
    out = tb.gemm("gm", dev(X), dev(xs)).cpu().numpy()
    oacc, oout = oracle.gemm_packed(X[:2], xs[:2], synth.pack_v11(t), 0.04, K, N)
    assert np.array_equal(out[:2].view(np.uint32), oout.view(np.uint32))
