"""Parity of the decode glue kernels with the CPU checker, through the C ABI.
int8 outputs and indices: bit-exact.  fp32 outputs: asserted within 1e-3 relative (the stated
tolerance) and, because both sides use the same fixed reduction order, also bit-for-bit."""
import numpy as np
import pytest
import torch

import oracle
from ter_b200 import synth

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def close(a, b, rtol=1e-3, atol=1e-6):
    return np.allclose(a, b, rtol=rtol, atol=atol)


@pytest.mark.parametrize("n", [8, 100, 2048, 2560, 6912, 8192])
def test_rmsnorm_quant(tb, n):
    rng = np.random.default_rng(n)
    x = (rng.standard_normal((3, n)) * rng.uniform(0.1, 20)).astype(np.float32)
    g = rng.normal(1.0, 0.02, size=n).astype(np.float32)
    q, sc, normed = tb.rmsnorm_quant(dev(x), dev(g), 1e-5, want_normed=True)
    q, sc, normed = q.cpu().numpy(), sc.cpu().numpy(), normed.cpu().numpy()
    for r in range(3):
        oq, os_, on = oracle.rmsnorm_quant(x[r], g, 1e-5)
        assert close(normed[r], on) and np.array_equal(bits(normed[r]), bits(on))
        assert np.array_equal(q[r], oq)
        assert bits(sc[r]) == bits(os_)
    # RMSNorm only
    _, _, only = tb.rmsnorm_quant(dev(x), dev(g), 1e-5, quant=False)
    assert np.array_equal(bits(only.cpu().numpy()[1]), bits(oracle.rmsnorm(x[1], g, 1e-5)))
    # absmax quantiser only (quant_int8_k)
    q2, s2, _ = tb.rmsnorm_quant(dev(x), None, 0.0)
    oq, os_ = oracle.quant_int8(x[2])
    assert np.array_equal(q2.cpu().numpy()[2], oq) and bits(s2.cpu().numpy()[2]) == bits(os_)


def test_quantiser_edge_cases(tb):
    z = np.zeros((1, 64), np.float32)
    q, s, _ = tb.rmsnorm_quant(dev(z), None, 0.0)
    oq, os_ = oracle.quant_int8(z[0])
    assert not q.cpu().numpy().any() and bits(s.cpu().numpy()[0]) == bits(os_)
    one = np.zeros((1, 64), np.float32); one[0, 7] = -3.0
    q, s, _ = tb.rmsnorm_quant(dev(one), None, 0.0)
    assert q.cpu().numpy()[0, 7] == -127 and np.count_nonzero(q.cpu().numpy()) == 1


@pytest.mark.parametrize("n", [64, 8192, 6912])
def test_act_quant(tb, n):
    rng = np.random.default_rng(n + 1)
    g = (rng.standard_normal((2, n)) * 4).astype(np.float32)
    u = (rng.standard_normal((2, n)) * 3).astype(np.float32)
    gam = rng.normal(1.0, 0.02, size=n).astype(np.float32)
    q, s = tb.act_quant(1, dev(g), dev(u), None, 0.0)
    for r in range(2):
        oq, os_ = oracle.silu_mul_quant(g[r], u[r])
        assert np.array_equal(q.cpu().numpy()[r], oq) and bits(s.cpu().numpy()[r]) == bits(os_)
    q, s = tb.act_quant(2, dev(g), dev(u), dev(gam), 1e-5)
    for r in range(2):
        oq, os_ = oracle.relu2_mul_rmsnorm_quant(g[r], u[r], gam, 1e-5)
        assert np.array_equal(q.cpu().numpy()[r], oq) and bits(s.cpu().numpy()[r]) == bits(os_)


def make_cache(rng, B, Nkv, Smax, Hd):
    k = oracle.f32_to_bf16(rng.standard_normal((B, Nkv, Smax, Hd)).astype(np.float32))
    v = oracle.f32_to_bf16(rng.standard_normal((B, Nkv, Smax, Hd)).astype(np.float32))
    return k, v


@pytest.mark.parametrize("Nh,Nkv,Hd,neox", [(32, 8, 64, 0), (20, 5, 128, 1), (4, 2, 64, 1)])
def test_rope_and_kv_append(tb, Nh, Nkv, Hd, neox):
    rng = np.random.default_rng(Nh)
    B, Smax, theta = 3, 300, 500000.0
    pos = np.array([0, 37, 299], np.int32)
    q = rng.standard_normal((B, Nh * Hd)).astype(np.float32)
    k = rng.standard_normal((B, Nkv * Hd)).astype(np.float32)
    v = rng.standard_normal((B, Nkv * Hd)).astype(np.float32)
    kc0, vc0 = make_cache(rng, B, Nkv, Smax, Hd)
    qd, kd, vd, kcd, vcd = dev(q), dev(k), dev(v), dev(kc0.view(np.int16)), dev(vc0.view(np.int16))
    tb.rope_kv(qd, kd, vd, dev(pos), Nh, Nkv, Hd, Smax, theta, neox, kcd, vcd)
    tab = oracle.rope_table(Smax, Hd, theta)
    kc, vc = kcd.cpu().numpy().view(np.uint16), vcd.cpu().numpy().view(np.uint16)
    for b in range(B):
        oq = oracle.rope(q[b], Nh, Hd, tab[pos[b]], neox)
        ok = oracle.rope(k[b], Nkv, Hd, tab[pos[b]], neox)
        assert np.array_equal(bits(qd.cpu().numpy()[b]), bits(oq))
        assert np.array_equal(bits(kd.cpu().numpy()[b]), bits(ok))
        want_k, want_v = kc0[b].copy(), vc0[b].copy()
        want_k[:, pos[b], :] = oracle.f32_to_bf16(ok).reshape(Nkv, Hd)
        want_v[:, pos[b], :] = oracle.f32_to_bf16(v[b]).reshape(Nkv, Hd)
        assert np.array_equal(kc[b], want_k) and np.array_equal(vc[b], want_v)   # only row pos[b] changed


@pytest.mark.parametrize("Nh,Nkv,Hd,Smax,lens", [
    (32, 8, 64, 512, [1, 2, 255, 256, 257, 512]),
    (20, 5, 128, 2176, [1, 300, 2048, 2176]),
    (4, 1, 64, 700, [77, 700]),
    (8, 1, 128, 64, [64]),
])
def test_attention(tb, Nh, Nkv, Hd, Smax, lens):
    rng = np.random.default_rng(Smax)
    B = len(lens)
    q = rng.standard_normal((B, Nh * Hd)).astype(np.float32)
    kc, vc = make_cache(rng, B, Nkv, Smax, Hd)
    pos = np.array([n - 1 for n in lens], np.int32)
    out = tb.attention(dev(q), dev(kc.view(np.int16)), dev(vc.view(np.int16)), dev(pos), Nh, Nkv, Hd, Smax)
    out = out.cpu().numpy()
    for b, n in enumerate(lens):
        want = oracle.attention(q[b], kc[b], vc[b], Nh, Nkv, Hd, Smax, n)
        spec = oracle.attention(q[b], kc[b], vc[b], Nh, Nkv, Hd, Smax, n, twopass=True)
        assert close(out[b], spec, rtol=1e-3, atol=1e-5), (b, n)      # the reference's two-pass form
        assert np.array_equal(bits(out[b]), bits(want)), (b, n)        # the chunked form, bit for bit


@pytest.mark.parametrize("Nh,Nkv,Hd,Smax,lens", [
    (32, 8, 64, 512, [1, 2, 15, 16, 17, 255, 256, 257, 400, 512]),
    (20, 5, 128, 2176, [1, 300, 2048, 2176, 33, 1000, 513, 2047]),
    (4, 1, 64, 700, [77, 700, 1, 256]),
    (8, 1, 128, 300, [64, 300]),
    (8, 4, 128, 600, [600, 31, 272]),
    (3, 3, 64, 300, [300, 8, 129]),
])
def test_attention_on_tensor_cores(tb, Nh, Nkv, Hd, Smax, lens):
    """Token batches sum the two contractions of attention on the tensor cores (bf16 mma, q and the
    probabilities split into three bf16 parts, so every product is exact).  Only the order of the fp32 sums
    differs from the checker's (and the tensor core truncates where the checker rounds), hence a tolerance:
    1e-5 of the largest output of the head per element (measured: 2.5e-6)."""
    rng = np.random.default_rng(Smax + Hd)
    B = len(lens)
    q = rng.standard_normal((B, Nh * Hd)).astype(np.float32)
    kc, vc = make_cache(rng, B, Nkv, Smax, Hd)
    pos = np.array([n - 1 for n in lens], np.int32)
    args = (dev(q), dev(kc.view(np.int16)), dev(vc.view(np.int16)), dev(pos), Nh, Nkv, Hd, Smax)
    tb.set_option("attn_mma_min", 1)
    try:
        got = tb.attention(*args).cpu().numpy()
    finally:
        tb.set_option("attn_mma_min", 0)
    exact = tb.attention(*args).cpu().numpy()
    for b, n in enumerate(lens):
        want = oracle.attention(q[b], kc[b], vc[b], Nh, Nkv, Hd, Smax, n)
        assert np.array_equal(bits(exact[b]), bits(want)), (b, n)
    g3, e3 = got.reshape(B, Nh, Hd), exact.reshape(B, Nh, Hd)
    tol = 1e-5 * np.max(np.abs(e3), axis=2, keepdims=True)
    assert not np.isnan(got).any()
    assert np.all(np.abs(g3 - e3) <= tol), float(np.max(np.abs(g3 - e3) / tol))
    assert tb.device_status() == 0


@pytest.mark.parametrize("V,H,B", [(1000, 256, 1), (4099, 2048, 2), (128256, 2048, 1), (3000, 2560, 3)])
def test_lm_head_and_argmax(tb, V, H, B):
    rng = np.random.default_rng(V)
    table = oracle.f32_to_bf16((rng.standard_normal((V, H)) * 0.02).astype(np.float32))
    x = rng.standard_normal((B, H)).astype(np.float32)
    logits = tb.lm_head_bf16(dev(table.view(np.int16)), dev(x))
    lg = logits.cpu().numpy()
    for b in range(B):
        if V <= 5000:
            want = oracle.lm_head_bf16(table, x[b])
            assert np.array_equal(bits(lg[b]), bits(want))
        ref = oracle.bf16_to_f32(table).astype(np.float64) @ x[b].astype(np.float64)
        assert np.allclose(lg[b], ref, rtol=1e-3, atol=1e-4)
    am = tb.argmax(logits).cpu().numpy()
    for b in range(B):
        assert am[b] == oracle.argmax(lg[b])
    # ties resolve to the lowest index
    t = torch.zeros((2, 70000), device="cuda")
    t[0, 69999] = 5.0; t[0, 1234] = 5.0; t[0, 40000] = 5.0
    t[1, :] = -3.0
    am = tb.argmax(t).cpu().numpy()
    assert am[0] == 1234 and am[1] == 0


def test_fused_quantiser_gemv_matches_two_step(tb):
    """ter_b200_norm_gemv_group == rmsnorm_quant / act_quant followed by the GEMV, bit for bit."""
    from ter_b200 import FMT_V11
    rng = np.random.default_rng(77)
    K = 2560
    names = []
    for nm, N in (("fz_a", 640), ("fz_b", 2560)):
        tb.install(nm, synth.pack_v11(synth.trits(K, N, N)), FMT_V11, K, N, float(synth.weight_scale(N)))
        names.append(nm)
    x = (rng.standard_normal(K) * 3).astype(np.float32)
    u = rng.standard_normal(K).astype(np.float32)
    g = rng.normal(1.0, 0.02, size=K).astype(np.float32)
    xd, ud, gd = dev(x), dev(u), dev(g)
    for act, gamma in ((0, gd), (0, None), (1, None), (2, gd)):
        if act == 0:
            q, sc, _ = tb.rmsnorm_quant(xd, gamma, 1e-5)
        else:
            q, sc = tb.act_quant(act, xd, ud, gamma, 1e-5)
        want = tb.gemv_group(names, q[0], sc)
        got = tb.norm_gemv_group(names, xd, gamma, 1e-5, act=act, up=ud if act else None)
        for a, b in zip(got, want):
            assert torch.equal(a, b), (act, gamma is None)
        # residual accumulate
        base = torch.full_like(want[1], 0.25)
        acc = tb.norm_gemv_group(names[1:], xd, gamma, 1e-5, act=act, up=ud if act else None,
                                 outs=[base.clone()], accumulate=True)[0]
        assert torch.equal(acc, base + want[1])
    # and against the CPU checker for one case
    oq, os_, _ = oracle.rmsnorm_quant(x, g, 1e-5)
    t = synth.trits(K, 640, 640)
    want = oracle.gemv_epilogue(oracle.gemv_acc_fast(oq, t), os_, synth.weight_scale(640))
    got = tb.norm_gemv_group(names[:1], xd, gd, 1e-5)[0].cpu().numpy()
    assert np.array_equal(bits(got), bits(want))


def test_named_operator_calls_equal_typed_entry_points(tb):
    """The reference's five operator slot names (src/tx/forward.cpp:376-380) through the K4-style call verb."""
    import struct
    from ter_b200 import api
    dev = torch.device("cuda")
    g = torch.Generator(device=dev)
    g.manual_seed(5)
    stream = torch.cuda.current_stream()
    n, rows = 512, 3
    x = torch.randn((rows, n), device=dev, generator=g)
    gamma = torch.rand(n, device=dev, generator=g) + 0.5
    eps = 1e-5
    q_t, s_t, _ = tb.rmsnorm_quant(x, gamma, eps)
    tb.sync()
    q_c = torch.empty_like(q_t)
    s_c = torch.empty_like(s_t)
    eps_bits = struct.unpack("<I", struct.pack("<f", eps))[0]
    assert tb.call("tk_rmsnorm", [x.data_ptr(), gamma.data_ptr(), n, rows, eps_bits, q_c.data_ptr(), s_c.data_ptr()]) == 0
    tb.sync()
    torch.cuda.synchronize()
    assert torch.equal(q_c, q_t) and torch.equal(s_c, s_t)

    gate = torch.randn((rows, n), device=dev, generator=g)
    up = torch.randn((rows, n), device=dev, generator=g)
    q_t, s_t = tb.act_quant(api.ACT_SILU, gate, up, None, 0.0)
    tb.sync()
    q_c = torch.empty_like(q_t)
    s_c = torch.empty_like(s_t)
    assert tb.call("tk_silu", [gate.data_ptr(), up.data_ptr(), n, rows, q_c.data_ptr(), s_c.data_ptr()]) == 0
    tb.sync()
    torch.cuda.synchronize()
    assert torch.equal(q_c, q_t) and torch.equal(s_c, s_t)

    B, Nh, Nkv, Hd, Smax, theta = 2, 4, 2, 64, 300, 500000.0
    pos = torch.tensor([7, 270], dtype=torch.int32, device=dev)
    qv = torch.randn((B, Nh * Hd), device=dev, generator=g)
    kv = torch.randn((B, Nkv * Hd), device=dev, generator=g)
    vv = torch.randn((B, Nkv * Hd), device=dev, generator=g)
    kc = torch.zeros((B, Nkv, Smax, Hd), dtype=torch.int16, device=dev)
    vc = torch.zeros_like(kc)
    q1, k1 = qv.clone(), kv.clone()
    tb.rope_kv(q1, k1, vv, pos, Nh, Nkv, Hd, Smax, theta, 0, kc, vc)
    tb.sync()
    q2, k2 = qv.clone(), kv.clone()
    dims = B | (Nh << 16) | (Nkv << 32) | (Hd << 48)
    theta_bits = struct.unpack("<q", struct.pack("<d", theta))[0]
    assert tb.call("tk_rope", [q2.data_ptr(), k2.data_ptr(), pos.data_ptr(), dims, Smax, theta_bits, 0]) == 0
    tb.sync()
    torch.cuda.synchronize()
    assert torch.equal(q1, q2) and torch.equal(k1, k2)

    kc.copy_(torch.randn(kc.shape, device=dev, generator=g).to(torch.bfloat16).view(torch.int16))
    vc.copy_(torch.randn(vc.shape, device=dev, generator=g).to(torch.bfloat16).view(torch.int16))
    want = tb.attention(q1, kc, vc, pos, Nh, Nkv, Hd, Smax)
    tb.sync()
    out = torch.empty_like(want)
    assert tb.call("tk_softmax", [q1.data_ptr(), kc.data_ptr(), vc.data_ptr(), pos.data_ptr(), dims, Smax, out.data_ptr()]) == 0
    tb.sync()
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.int32), want.view(torch.int32)) and not torch.isnan(out).any()

    assert tb.call("tk_rmsnorm", [1, 2, 3]) == api.E_SHAPE
    assert tb.call("tk_nothing", [0]) == api.E_UNKNOWN
    assert tb.call("tk_rope", [0] * 8) == api.E_NARGS
    assert tb.device_status() == 0


@pytest.mark.parametrize("V,H,B", [(4099, 2048, 16), (128256, 2560, 64), (3000, 256, 37), (1000, 2560, 300)])
def test_lm_head_on_tensor_cores(tb, V, H, B):
    """Token batches run the bf16 lm_head on tcgen05 (x split into two bf16 parts, fp32 accumulators).  The
    summation order is the tensor core's, not the checker's, so the comparison is a tolerance: 1e-4 of the
    largest logit of the row per element (measured: about 1e-6), and the greedy token must be the checker's
    unless its two best logits are closer than that tolerance."""
    rng = np.random.default_rng(V + B)
    table = oracle.f32_to_bf16((rng.standard_normal((V, H)) * 0.02).astype(np.float32))
    x = rng.standard_normal((B, H)).astype(np.float32)
    td = dev(table.view(np.int16))
    got = tb.lm_head_bf16_tc(td, dev(x)).cpu().numpy()
    exact = tb.lm_head_bf16(td, dev(x)).cpu().numpy()          # bit-equal to the checker (test_lm_head_and_argmax)
    for b in range(0, B, max(1, B // 4)):
        want = oracle.lm_head_bf16(table, x[b])
        assert np.array_equal(exact[b].view(np.uint32), want.view(np.uint32))
    tol = 1e-4 * np.max(np.abs(exact), axis=1, keepdims=True)
    assert np.all(np.abs(got - exact) <= tol), float(np.max(np.abs(got - exact) / tol))
    for b in range(B):
        i, j = int(np.argmax(got[b])), int(np.argmax(exact[b]))
        if i != j:
            assert abs(exact[b][i] - exact[b][j]) <= tol[b, 0], (b, i, j)
    assert tb.device_status() == 0


def test_exchange_wait_runs_out_without_a_peer(tb):
    """The tensor-parallel exchange polls for words that a peer stores.  On one GPU, against a stand-in
    peer that never sends, the wait must run out after "wait_ms": the kernel returns by itself, the status
    word reports the timeout once, and the handle keeps working."""
    from ter_b200 import api
    try:
        tb.set_option("wait_ms", 10)
        tb.selftest_exchange_timeout()
    finally:
        tb.set_option("wait_ms", 2000)
    assert tb.device_status() == api.E_TIMEOUT      # reported once ...
    assert tb.device_status() == 0                   # ... and cleared
    x = np.linspace(-1.0, 1.0, 256, dtype=np.float32).reshape(1, 256)
    tb.rmsnorm_quant(dev(x), None, 1e-5)              # a following normal call works
    assert tb.device_status() == 0
