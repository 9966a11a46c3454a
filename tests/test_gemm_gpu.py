"""Parity of the tensor-core (tcgen05 kind::i8) ternary GEMM with the CPU checker through the C ABI:
int32 accumulators bit-exact row by row against exact integer arithmetic and the scalar checker,
fp32 outputs bit-exact (one fp32 multiply per element), with and without split-K."""
import numpy as np
import pytest
import torch

import oracle
from ter_b200 import FMT_V11, synth

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def make(K, N, M, seed):
    t = synth.trits(K, N, seed)
    ws = synth.weight_scale(seed)
    rng = np.random.default_rng(seed + 1)
    xf = rng.standard_normal((M, K)).astype(np.float32)
    qs = [synth.quant_int8(xf[m]) for m in range(M)]
    X = np.stack([q for q, _ in qs])
    xs = np.array([s for _, s in qs], np.float32)
    return t, ws, X, xs


def check(tb, K, N, M, seed, name="gm"):
    t, ws, X, xs = make(K, N, M, seed)
    tb.install(name, synth.pack_v11(t), FMT_V11, K, N, float(ws))
    want = (X.astype(np.float64) @ t.astype(np.float64)).astype(np.int64)
    acc = tb.gemm_acc(name, dev(X)).cpu().numpy()
    assert np.array_equal(acc.astype(np.int64), want), f"int32 mismatch K={K} N={N} M={M}"
    out = tb.gemm(name, dev(X), dev(xs)).cpu().numpy()
    want_f = np.stack([oracle.gemv_epilogue(want[m].astype(np.int32), xs[m], ws) for m in range(M)])
    assert np.allclose(out, want_f, rtol=1e-3, atol=0)
    assert np.array_equal(out.view(np.uint32), want_f.view(np.uint32))
    assert tb.device_status() == 0
    return t, ws, X, xs


@pytest.mark.parametrize("K,N,M", [(128, 128, 16), (256, 64, 5), (512, 144, 33), (1024, 256, 16), (432, 80, 64),
                                   (2560, 640, 16)])
def test_small_shapes(tb, K, N, M):
    t, ws, X, xs = check(tb, K, N, M, seed=K + N + M)
    # the scalar checker as well, on a couple of rows
    oacc, oout = oracle.gemm_packed(X[:2], xs[:2], synth.pack_v11(t), ws, K, N)
    got = tb.gemm("gm", dev(X), dev(xs)).cpu().numpy()
    assert np.array_equal(got[:2].view(np.uint32), oout.view(np.uint32))


@pytest.mark.parametrize("name", ["q", "k", "gate", "down"])
@pytest.mark.parametrize("M", [16, 64, 256, 1024])
def test_bitnet_shapes(tb, name, M):
    K, N = synth.BITNET_2B_SHAPES[name]
    check(tb, K, N, M, seed=synth.seed_for(K, N, M) & 0xFFFF)


@pytest.mark.parametrize("K,N", [(2560, 640), (6912, 2560), (432, 80)])
def test_few_rows_one_launch_and_tensor_core_gemm_agree(tb, K, N):
    """Few token rows take the multi-row GEMV (one launch for up to 16 rows; the default rule uses it up to 8); from
    option "gemm_min_m" rows on the tcgen05 GEMM.  Both must give the checker's bits at the same M."""
    for M in (2, 3, 8, 13, 16):
        t, ws, X, xs = make(K, N, M, K + M)
        tb.install("fr", synth.pack_v11(t), FMT_V11, K, N, float(ws))
        want = (X.astype(np.int64) @ t.astype(np.int64))
        want_f = np.stack([oracle.gemv_epilogue(want[m].astype(np.int32), xs[m], ws) for m in range(M)])
        try:
            tb.set_option("gemm_min_m", 17)
            l0 = tb.launch_count()
            out_rows = tb.gemm("fr", dev(X), dev(xs)).cpu().numpy()
            assert tb.launch_count() - l0 == 1                       # one launch for all rows
            assert np.array_equal(tb.gemm_acc("fr", dev(X)).cpu().numpy().astype(np.int64), want)
            tb.set_option("gemm_min_m", 2)
            out_tc = tb.gemm("fr", dev(X), dev(xs)).cpu().numpy()
        finally:
            tb.set_option("gemm_min_m", 9)
        assert np.array_equal(out_rows.view(np.uint32), want_f.view(np.uint32)), (K, N, M)
        assert np.array_equal(out_tc.view(np.uint32), want_f.view(np.uint32)), (K, N, M)
    assert tb.device_status() == 0


def test_split_k_and_row_path_agree(tb):
    K, N, M = 2560, 2560, 24
    t, ws, X, xs = make(K, N, M, 9)
    tb.install("sk", synth.pack_v11(t), FMT_V11, K, N, float(ws))
    Xd, sd = dev(X), dev(xs)
    base = tb.gemm("sk", Xd, sd)
    tb.set_option("gemm_split_k", 0)
    assert torch.equal(tb.gemm("sk", Xd, sd), base)
    tb.set_option("gemm_split_k", 1)
    tb.set_option("gemm_min_m", 1000)              # row-at-a-time through the GEMV kernel
    assert torch.equal(tb.gemm("sk", Xd, sd), base)
    tb.set_option("gemm_min_m", 9)


def test_extreme_values(tb):
    K, N, M = 1024, 128, 16
    for sign in (1, -1):
        t = np.full((K, N), sign, np.int8)
        tb.install("ex", synth.pack_v11(t), FMT_V11, K, N, 1.0)
        for xv in (-128, 127):
            X = np.full((M, K), xv, np.int8)
            acc = tb.gemm_acc("ex", dev(X)).cpu().numpy()
            assert np.all(acc == sign * xv * K)


def test_captured_graph_survives_scratch_growth(tb):
    """A captured GEMM keeps the scratch addresses it was recorded with.  A later eager call that needs a
    larger scratch must not free them: the replay after it gives the same bits as before."""
    from ter_b200 import TerB200
    h = TerB200(0)            # a fresh handle: its scratch starts empty, so the second call has to grow it
    try:
        K, N = 512, 256
        t, ws, X, xs = make(K, N, 24, 77)
        h.install("sg", synth.pack_v11(t), FMT_V11, K, N, float(ws))
        Xd, sd = dev(X), dev(xs)
        out = torch.zeros((24, N), device="cuda")
        base = h.gemm("sg", Xd, sd).clone()                        # split-K path (M <= 256): uses the partial buffer
        gid = h.capture(lambda: h.gemm("sg", Xd, sd, out))
        h.graph_launch(gid)
        h.sync()
        assert torch.equal(out, base)
        t2, ws2, X2, xs2 = make(K, N, 200, 78)                     # 200 x 256 partials: outgrows the scratch
        h.install("sg2", synth.pack_v11(t2), FMT_V11, K, N, float(ws2))
        h.gemm("sg2", dev(X2), dev(xs2))
        junk = [torch.full((1 << 20,), 7, dtype=torch.int32, device="cuda") for _ in range(4)]   # reuse freed memory, if any
        out.zero_()
        h.graph_launch(gid)
        h.sync()
        del junk
        assert torch.equal(out, base)
        assert h.device_status() == 0
    finally:
        h.close()
