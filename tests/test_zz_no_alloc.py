"""Attention through the entry point that allocates nothing.

`ter_b200_attention_noalloc` serves callers that cannot call cudaMalloc where they need attention
(inside a stream capture, in a loop that handed all memory out at start-up, under a foreign
allocator): its scratch is a fixed array in the library's device image.  The test calls it through
the C ABI twice in a row on different inputs -- the array is shared and keeps the previous call's
contents -- and requires the same bits as the regular entry point given a caller's scratch buffer,
and as the CPU checker's chunked attention (so the comparison is not CUDA against itself only).
It builds its own handle so that it passes alone in a fresh process as well as after the rest of
the suite.  (The file name sorts last: a run that stops at the first failure has then already run
every other test.)"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(rng, B, Nh, Nkv, Hd, Smax, lens):
    q = torch.from_numpy(rng.standard_normal((B, Nh * Hd)).astype(np.float32)).cuda()
    kc = torch.from_numpy(rng.standard_normal((B, Nkv, Smax, Hd)).astype(np.float32)).cuda().to(torch.bfloat16)
    vc = torch.from_numpy(rng.standard_normal((B, Nkv, Smax, Hd)).astype(np.float32)).cuda().to(torch.bfloat16)
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device="cuda")
    return q, kc, vc, pos


def test_noalloc_attention_matches_regular_entry_point():
    from ter_b200 import TerB200, TerB200Error, api
    h = TerB200(0)
    try:
        rng = np.random.default_rng(2026)
        cap = h.L.ter_b200_attention_noalloc_max_floats()
        assert cap == 1 << 20
        # two calls in a row: a long multi-chunk case, then a shorter one that reuses the array
        for (B, Nh, Nkv, Hd, Smax, lens) in [(3, 20, 5, 128, 1100, [1100, 257, 1]), (2, 32, 8, 64, 512, [300, 512])]:
            assert h.L.ter_b200_attention_scratch_floats(B, Nh, Hd, Smax) <= cap
            q, kc, vc, pos = _case(rng, B, Nh, Nkv, Hd, Smax, lens)
            want = h.attention(q, kc, vc, pos, Nh, Nkv, Hd, Smax)
            out = torch.empty_like(want)
            got = h.attention_noalloc(q, kc, vc, pos, Nh, Nkv, Hd, Smax, out=out)
            torch.cuda.synchronize()
            assert torch.equal(got, want)                                  # same bits as the regular entry point
            # ... and as the CPU checker, sequence by sequence
            import oracle
            qh, gh = q.cpu().numpy(), got.cpu().numpy()
            kh = kc.view(torch.int16).cpu().numpy().view(np.uint16)
            vh = vc.view(torch.int16).cpu().numpy().view(np.uint16)
            for b, n in enumerate(lens):
                ref = oracle.attention(qh[b], kh[b], vh[b], Nh, Nkv, Hd, Smax, n)
                assert np.array_equal(gh[b].view(np.uint32), ref.view(np.uint32)), (b, n)
        # a problem whose records do not fit the fixed array is refused with a clear error
        B, Nh, Nkv, Hd, Smax = 64, 32, 8, 128, 2176
        assert h.L.ter_b200_attention_scratch_floats(B, Nh, Hd, Smax) > cap
        q = torch.zeros((B, Nh * Hd), device="cuda")
        pos = torch.zeros(B, dtype=torch.int32, device="cuda")
        tiny = torch.zeros(8, dtype=torch.bfloat16, device="cuda")   # never read: the call is rejected first
        with pytest.raises(TerB200Error) as e:
            h.attention_noalloc(q, tiny, tiny, pos, Nh, Nkv, Hd, Smax)
        assert e.value.code == api.E_SHAPE
        assert h.device_status() == 0
    finally:
        h.close()
