// Persistent decode kernel for sm_100a: embedding and all layers of one decode step of one sequence in
// ONE launch.
//
// A decode step at batch 1 is a chain of dependent stages (q/k/v -> attention -> o -> gate/up -> down,
// per layer; the reference's forward_token_dev, cuda/ter_cuda_forward_packed.cu:505-563, BitNet:
// cuda/ter_cuda_forward_bitnet.cu:850-913) whose useful work is a few hundred nanoseconds each: as
// separate launches the step is bound by launch-to-launch latency, not by the 15 MB of weights a layer
// streams.  Here one CTA per SM stays resident for the whole step:
//   * Stages are not separated by kernel boundaries or device-wide barriers but by DATAFLOW: every
//     activation vector travels as flag-in-data words {v0, seq, v1, seq} (tagged.cuh).  A producer stores
//     its columns once; a consumer polls the words it needs until they carry the generation it expects.
//     One store and one load per hand-over: no fence, no atomic, no barrier.  A buffer is rewritten only
//     by a stage that transitively depends on every reader of its previous generation, so no reader can
//     lose a value.
//   * Weights never wait for the chain.  Every WARP streams its share of the step's weight blocks
//     (4 KB = 16 output columns x 1024 k, kernels.h) through its own ring of shared-memory stages with
//     1-D TMA bulk copies and mbarriers; the cursor that issues the copies runs `stages` blocks ahead of
//     the warp and crosses stage and layer boundaries, because weights are immutable.  HBM therefore
//     streams continuously while values are handed over.
//   * A stage's input vector is normalised and quantised to int8 by EVERY CTA for itself into shared
//     memory (the arithmetic of norm_quant_kernel, normq.cuh).
//   * A work unit is one (strip, 1024-k block); a CTA owns a contiguous range of strips of the stage, its
//     8 warps share the units, partial integer sums meet in shared-memory atomics (integer addition is
//     associative: the result is bit-exact whatever the split).  The epilogue is the GEMV's:
//     (float)acc * (x_scale * w_scale), with the gated activation fused for gate/up and the residual add
//     done on the CTA's own columns of the residual stream, which live in shared memory for the step.
//   * Attention: (chunk, KV head) items over the CTAs (attn.cuh: the arithmetic of attn_partial_kernel);
//     the copies of an item's cached K/V rows start a stage early, while q/k/v are still being computed;
//     the CTA of chunk 0 merges the chunks in order, polling the other chunks' tagged records.
// Every wait is bounded; a wait that runs out publishes an abort mark for the step and records a code in
// the status word; every CTA then drains its own copies and returns.
#include "attn.cuh"
#include "decode.h"
#include "kernels.h"

namespace terb {
namespace {

constexpr int kDecWarps = kT / 32;
constexpr int kDecMaxStages = 8;
constexpr int kRoundStrips = 8;          // accumulator rows per round
constexpr int kBlockBytes = 4 * kGemvKC; // one weight block

// fixed shared-memory header
constexpr int kOffRingBars = 0;                 // u64[8][8]
constexpr int kOffAcc = 512;                    // int[8][16]
constexpr int kOffRed16 = 1024;                 // float[16]
constexpr int kOffRedg = 1088;                  // float[64]
constexpr int kOffMisc = 1344;                  // int[8]: [1] xsum, [2] abort
constexpr int kOffMl = 1376;                    // float[16]: (m, l) of the attention chunk
constexpr int kOffRope = 1440;                  // float[<=128]: rotary row of the position
constexpr int kHdr = 2304;                     // + StageGeo[4] at 2048

// Geometry of the four GEMV stages of a layer.
struct StageGeo {
    int K, Kpad, nb, last_kc;   // blocks per strip, k of the last block
    int slots;                  // strips (pairs of strips for gate/up)
    int pair;
    int s1, s2;                 // stage 0: first slot of k and of v
    int lo, n_slots;            // this CTA's slot range
    int inv_nb;                 // ceil(65536 / nb): u / nb == (u * inv_nb) >> 16 for the small u used here
};
__device__ __forceinline__ StageGeo stage_geo(const DecodeParams& p, int ph, int cta, int grid) {
    StageGeo g;
    const int Hq = p.Nh * p.Hd, Hkv = p.Nkv * p.Hd;
    g.pair = 0; g.s1 = g.s2 = 0;
    if (ph == 0) { g.K = p.H; g.slots = (Hq + 2 * Hkv) >> 4; g.s1 = Hq >> 4; g.s2 = (Hq + Hkv) >> 4; }
    else if (ph == 1) { g.K = Hq; g.slots = p.H >> 4; }
    else if (ph == 2) { g.K = p.H; g.slots = p.F >> 4; g.pair = 1; }
    else { g.K = p.F; g.slots = p.H >> 4; }
    g.Kpad = (g.K + 127) & ~127;
    g.nb = (g.Kpad + kGemvKC - 1) / kGemvKC;
    g.last_kc = g.Kpad - (g.nb - 1) * kGemvKC;
    g.lo = (int)((long long)cta * g.slots / grid);
    g.n_slots = (int)((long long)(cta + 1) * g.slots / grid) - g.lo;
    g.inv_nb = (65536 + g.nb - 1) / g.nb;
    return g;
}
__device__ __forceinline__ int stage_first_mat(int ph) { return ph == 0 ? 0 : (ph == 1 ? 3 : (ph == 2 ? 4 : 6)); }

// Matrix (relative to the stage's first) and strip within it of slot `s` (non-pair stages).
__device__ __forceinline__ void slot_to_mat(const StageGeo& g, int ph, int s, int& mat, int& ls) {
    mat = 0; ls = s;
    if (ph == 0) {
        if (s >= g.s2) { mat = 2; ls = s - g.s2; }
        else if (s >= g.s1) { mat = 1; ls = s - g.s1; }
    }
}
__device__ __forceinline__ int slot_lo(int cta, int slots, int grid) { return (int)((long long)cta * slots / grid); }
// The four stages' geometry is the same in every layer: computed once per CTA into shared memory.
constexpr int kOffStages = 2048;
static_assert(4 * sizeof(StageGeo) <= 256, "stage table");

// Cursor over one warp's weight blocks of the whole step, in the order the warp consumes them:
// layer -> stage -> round -> unit (u = warp, warp + 8, ...).
struct Cursor {
    int layer, ph, round, u;
    int lo, n_slots;      // the CTA's slot range in this stage
    int ns, units;        // slots and units of this round
    StageGeo g;
    const uint8_t *W0, *W1, *W2;
    bool done;
};

__device__ __forceinline__ void cursor_round(Cursor& c, int warp) {
    const int rs = c.g.pair ? kRoundStrips / 2 : kRoundStrips;
    const int left = c.n_slots - c.round * rs;
    c.ns = left < rs ? left : rs;
    c.units = c.ns > 0 ? c.ns * (c.g.pair ? 2 : 1) * c.g.nb : 0;
    c.u = warp;
}
__device__ __forceinline__ void cursor_stage(Cursor& c, const StageGeo* stab, const DecodeLayerDev* tab, int L, int warp) {
    c.g = stab[c.ph];                              // shared memory
    c.lo = c.g.lo;
    c.n_slots = c.g.n_slots;
    const DecodeLayerDev* ld = tab + c.layer;      // shared memory
    const int m0 = stage_first_mat(c.ph);
    c.W0 = ld->W[m0];
    c.W1 = (c.ph == 0 || c.ph == 2) ? ld->W[m0 + 1] : nullptr;
    c.W2 = c.ph == 0 ? ld->W[m0 + 2] : nullptr;
    c.round = 0;
    cursor_round(c, warp);
}
// Moves to the next valid unit (or sets done).
__device__ __forceinline__ void cursor_settle(Cursor& c, const StageGeo* stab, const DecodeLayerDev* tab, int L, int warp) {
    while (!c.done) {
        if (c.u < c.units) return;
        const int rs = c.g.pair ? kRoundStrips / 2 : kRoundStrips;
        if ((c.round + 1) * rs < c.n_slots) { ++c.round; cursor_round(c, warp); continue; }
        if (++c.ph == 4) {
            c.ph = 0;
            if (++c.layer >= L) { c.done = true; return; }
        }
        cursor_stage(c, stab, tab, L, warp);
    }
}
// Source address and k count of the cursor's unit.
__device__ __forceinline__ const uint8_t* unit_src(const Cursor& c, int& kc) {
    const int row = (c.u * c.g.inv_nb) >> 16;
    const int q = c.u - row * c.g.nb;
    kc = (q == c.g.nb - 1) ? c.g.last_kc : kGemvKC;
    int mat, ls;
    if (c.g.pair) {
        mat = row >= c.ns ? 1 : 0;
        ls = c.lo + c.round * (kRoundStrips / 2) + (row - mat * c.ns);
    } else {
        slot_to_mat(c.g, c.ph, c.lo + c.round * kRoundStrips + row, mat, ls);
    }
    const uint8_t* W = mat == 0 ? c.W0 : (mat == 1 ? c.W1 : c.W2);
    return W + (size_t)ls * 4u * (size_t)c.g.Kpad + (size_t)q * kBlockBytes;
}

// Query heads per attention item: with four or more query heads per KV head the heads of a KV head are dealt to
// two items.  A lone sequence has far fewer (chunk, KV head) pairs than there are CTAs, and an item with half the
// heads is the shorter link in the layer's chain.  Both items of a KV head stage the same K/V chunk.
__host__ __device__ constexpr int attn_item_heads(int G) { return G >= 4 ? G / 2 : G; }

// GA: query heads per attention item (attn_item_heads(G), or 1 where even one item per query head and chunk of the
// longest context leaves CTAs to spare).
template <int HD, int G, int GA>
__global__ void __launch_bounds__(kT, 1) decode_layers_kernel(const __grid_constant__ DecodeParams p) {
    extern __shared__ __align__(128) uint8_t sm[];
    constexpr int KVD = G / GA;
    using AL = AttnSmem<HD, GA, false>;
    constexpr int kAttnBytes = (AL::kBytes + 127) & ~127;
    uint64_t* ring_bars = reinterpret_cast<uint64_t*>(sm + kOffRingBars);
    int* acc_s = reinterpret_cast<int*>(sm + kOffAcc);
    float* red16 = reinterpret_cast<float*>(sm + kOffRed16);
    float* redg = reinterpret_cast<float*>(sm + kOffRedg);
    int* misc = reinterpret_cast<int*>(sm + kOffMisc);
    float* ml_s = reinterpret_cast<float*>(sm + kOffMl);
    float* rope_s = reinterpret_cast<float*>(sm + kOffRope);
    StageGeo* stab = reinterpret_cast<StageGeo*>(sm + kOffStages);
    DecodeLayerDev* tab = reinterpret_cast<DecodeLayerDev*>(sm + kHdr);
    float* own = reinterpret_cast<float*>(sm + kHdr + p.tab_bytes);
    int8_t* xq = reinterpret_cast<int8_t*>(sm + kHdr + p.tab_bytes + p.own_bytes);
    uint8_t* asmem = sm + kHdr + p.tab_bytes + p.own_bytes + p.x_bytes;
    uint64_t* abars = reinterpret_cast<uint64_t*>(asmem + AL::kBarOff);
    uint8_t* ring = asmem + kAttnBytes;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int cta = blockIdx.x, grid = gridDim.x;
    const int S = p.stages;
    uint64_t* mybars = ring_bars + warp * kDecMaxStages;
    uint8_t* mybuf = ring + (size_t)warp * S * kBlockBytes;

    if (lane == 0) {
        for (int i = 0; i < S; ++i) mbar_init(&mybars[i], 1);
        if (warp == 0) { mbar_init(&abars[0], 1); mbar_init(&abars[1], 1); }
        mbar_fence_init();
    }
    if (tid < 8) misc[tid] = 0;
    if (tid < kRoundStrips * 16) acc_s[tid] = 0;
    if (tid >= 32 && tid < 36) stab[tid - 32] = stage_geo(p, tid - 32, cta, grid);
    {   // per-layer constants into shared memory: the weight cursor and the epilogues read them all the time
        const int n = p.L * (int)(sizeof(DecodeLayerDev) / 4);
        const int* src = reinterpret_cast<const int*>(p.layers);
        int* dst = reinterpret_cast<int*>(tab);
        for (int i = tid; i < n; i += kT) dst[i] = src[i];
    }
    const int pos = p.pos[0];
    int tok = p.tokens[0];
    if (tok < 0 || tok >= p.V) tok = 0;
    const bool ok = pos >= 0 && pos < p.Smax;    // uniform over the grid
    if (ok && tid < HD) rope_s[tid] = p.rope[(size_t)pos * HD + tid];
    __syncthreads();
    if (!ok) return;       // nothing was issued

    // ---- the weight stream: producer cursor `stages` units ahead of the consumer
    Cursor pc;
    pc.layer = 0; pc.ph = 0; pc.done = false;
    cursor_stage(pc, stab, tab, p.L, warp);
    cursor_settle(pc, stab, tab, p.L, warp);
    int p_stage = 0, inflight = 0;
    auto issue = [&]() {
        if (pc.done) return;
        int kc;
        const uint8_t* src = unit_src(pc, kc);
        if (lane == 0) {
            mbar_arrive_expect_tx(&mybars[p_stage], 4u * (uint32_t)kc);
            bulk_g2s(mybuf + (size_t)p_stage * kBlockBytes, src, 4u * (uint32_t)kc, &mybars[p_stage]);
        }
        ++inflight;
        if (++p_stage == S) p_stage = 0;
        pc.u += kDecWarps;
        cursor_settle(pc, stab, tab, p.L, warp);
    };
    for (int i = 0; i < S; ++i) issue();
    int c_stage = 0;
    uint32_t c_parity = 0;
    uint32_t kv_parity = 0;
    bool kv_pending = false;

    // waits (bounded) for this CTA's copies in flight; called on every early exit
    auto drain = [&]() {
        for (; inflight > 0; --inflight) {
            mbar_wait_bounded(&mybars[c_stage], c_parity, p.status);
            if (++c_stage == S) { c_stage = 0; c_parity ^= 1u; }
        }
        if (kv_pending && tid == 0) {
            mbar_wait_bounded(&abars[0], kv_parity, p.status);
            mbar_wait_bounded(&abars[1], kv_parity, p.status);
        }
        __syncthreads();
    };

    // generations of this step
    const uint32_t step = ld_volatile32(p.ctl);
    const PollCtx ctx{p.wait_ns, &misc[2], p.ctl + 1, step + 1u, p.status, (unsigned)p.poll_sleep_ns};
    auto seq_layer = [&](int l) -> uint32_t { return step * (uint32_t)p.L + (uint32_t)l + 1u; };
    auto seq_hid = [&](int i) -> uint32_t { return step * (uint32_t)(2 * p.L + 1) + (uint32_t)i + 1u; };

    // this CTA's columns of the residual stream (the slots of the o / down stages): embedding gather
    const int h_slots = p.H >> 4;
    const int lo_h = slot_lo(cta, h_slots, grid);
    const int n_h = slot_lo(cta + 1, h_slots, grid) - lo_h;
    for (int i = tid; i < n_h * 16; i += kT) own[i] = bf16_bits_to_f32(p.embd[(size_t)tok * p.H + lo_h * 16 + i]);
    __syncthreads();
    for (int i = tid; i < n_h * 8; i += kT)
        st_volatile16(p.hid_t + (lo_h * 16 + 2 * i) / 2, tag2(own[2 * i], own[2 * i + 1], seq_hid(0)));

    const int nc = pos / kAttnChunk + 1;                 // chunks of the context
    const int nkv_v = p.Nkv * KVD;
    const int n_items = nc * nkv_v;
    const int act = p.bitnet ? PRE_RELU2_MUL : PRE_SILU_MUL;
    // attention items of this CTA: i = my_first, my_first - grid, ... (descending: the merging items of
    // chunk 0 have the lowest numbers and come last, so a merger never waits on work queued behind it)
    const int my_slot = grid - 1 - cta;
    const int my_first = my_slot < n_items ? my_slot + ((n_items - 1 - my_slot) / grid) * grid : -1;

#ifdef TERB_TRACE
    int tr_n = 0;
#define TR() do { if (tid == 0 && layer == 1 && p.trace && tr_n < 32) p.trace[(size_t)cta * 32 + tr_n++] = globaltimer_ns(); } while (0)
#else
#define TR() do {} while (0)
#endif

    for (int layer = 0; layer < p.L; ++layer) {
        const DecodeLayerDev* ld = tab + layer;
        const uint32_t sl = seq_layer(layer);
        AttnParams ap{nullptr, ld->kcache, ld->vcache, p.pos, nullptr, nullptr, 1, p.Nh, nkv_v, p.Hd, p.Smax,
                      (p.Smax + kAttnChunk - 1) / kAttnChunk, p.rope, nullptr, nullptr, ld->kcache, ld->vcache,
                      p.bitnet ? 1 : 0, p.status, nullptr, 0, KVD};
        // the cached K/V rows of this CTA's first attention item start moving now
        if (my_first >= 0) {
            const AttnItem it = attn_item<HD>(ap, my_first / nkv_v, my_first % nkv_v, 0, pos);
            if (tid == 0 && it.active && it.n_copy > 0) {
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                attn_issue_kv<HD, GA, false>(ap, it, asmem);
            }
            kv_pending = it.active && it.n_copy > 0;
        }

        for (int ph = 0; ph < 4; ++ph) {
            const StageGeo g = stab[ph];
            const int lo = g.lo, n_slots = g.n_slots;
            const int m0 = stage_first_mat(ph);
            TR();
            if (n_slots > 0) {
                // ---- prologue: this stage's input vector, polled, normalised and quantised by this CTA for itself
                NormQuantParams nq;
                nq.x = nullptr; nq.u = nullptr; nq.q = nullptr; nq.scale_out = nullptr; nq.normed = nullptr; nq.rows = 1;
                nq.eps = p.eps; nq.rowsum_out = nullptr; nq.pre = PRE_NONE; nq.n = g.K;
                TaggedSrc ts;
                ts.ctx = ctx;
                if (ph == 0) { ts.words = p.hid_t; ts.seq = seq_hid(2 * layer); nq.gamma = ld->gamma[0]; }
                else if (ph == 1) { ts.words = p.att_t; ts.seq = sl; nq.gamma = p.bitnet ? ld->gamma[2] : nullptr; }
                else if (ph == 2) { ts.words = p.hid_t; ts.seq = seq_hid(2 * layer + 1); nq.gamma = ld->gamma[1]; }
                else { ts.words = p.gate_t; ts.seq = sl; nq.gamma = p.bitnet ? ld->gamma[3] : nullptr; }
                const float xscale = block_norm_quant_fast(nq, 0, red16, xq, nullptr, &ts);
                if (tid < g.Kpad - g.K) xq[g.K + tid] = 0;
                __syncthreads();
                if (misc[2]) { drain(); return; }        // a wait ran out (here or elsewhere): give up the step
                TR();
                {
                    int local = 0;
                    for (int i = tid * 16; i < g.Kpad; i += kT * 16) {
                        const int4 v = *reinterpret_cast<const int4*>(xq + i);
                        local = __dp4a(v.x, 0x01010101, local);
                        local = __dp4a(v.y, 0x01010101, local);
                        local = __dp4a(v.z, 0x01010101, local);
                        local = __dp4a(v.w, 0x01010101, local);
                    }
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
                    if (lane == 0 && local != 0) atomicAdd(&misc[1], local);
                }
                // ---- rounds of up to 8 strips
                const int rs = g.pair ? kRoundStrips / 2 : kRoundStrips;
                const int c = lane >> 3, sgm = lane & 7;
                for (int r0 = 0; r0 < n_slots; r0 += rs) {
                    const int ns = min(rs, n_slots - r0);
                    const int units = ns * (g.pair ? 2 : 1) * g.nb;
                    for (int u = warp; u < units; u += kDecWarps) {
                        const int row = (u * g.inv_nb) >> 16, q = u - row * g.nb;
                        const int kc = (q == g.nb - 1) ? g.last_kc : kGemvKC;
                        mbar_wait_bounded(&mybars[c_stage], c_parity, p.status);
                        const uint8_t* wt = mybuf + (size_t)c_stage * kBlockBytes + c * kc + sgm * 16;
                        const int8_t* xp = xq + q * kGemvKC + sgm * 16;
                        int a0 = 0, a1 = 0, a2 = 0, a3 = 0;
                        if (kc == kGemvKC) {
#pragma unroll
                            for (int j = 0; j < kGemvKC / 128; ++j)
                                mac64(*reinterpret_cast<const uint4*>(wt + j * 128),
                                      *reinterpret_cast<const int4*>(xp + j * 128), a0, a1, a2, a3);
                        } else {
                            for (int j = 0; j < (kc >> 7); ++j)
                                mac64(*reinterpret_cast<const uint4*>(wt + j * 128),
                                      *reinterpret_cast<const int4*>(xp + j * 128), a0, a1, a2, a3);
                        }
#pragma unroll
                        for (int o = 1; o < 8; o <<= 1) {
                            a0 += __shfl_xor_sync(0xffffffffu, a0, o);
                            a1 += __shfl_xor_sync(0xffffffffu, a1, o);
                            a2 += __shfl_xor_sync(0xffffffffu, a2, o);
                            a3 += __shfl_xor_sync(0xffffffffu, a3, o);
                        }
                        if (sgm == 0) {
                            int* a = acc_s + row * 16 + c * 4;
                            atomicAdd(a + 0, a0 - a1 - a2 - a3);
                            atomicAdd(a + 1, a1);
                            atomicAdd(a + 2, a2);
                            atomicAdd(a + 3, a3);
                        }
                        __syncwarp();          // every lane has finished reading this stage
                        --inflight;
                        if (++c_stage == S) { c_stage = 0; c_parity ^= 1u; }
                        if (u + kDecWarps < units) issue();      // more to consume in this round: keep the ring fed
                    }
                    __syncthreads();
                    TR();
                    // ---- epilogue of the round: one thread per pair of adjacent columns
                    const int xsum = misc[1];
                    if (tid < ns * 8) {
                        const int row = tid >> 3, lc0 = 2 * (tid & 7), lc1 = lc0 + 1;
                        auto val = [&](int r, int lc) -> int { return (acc_s[r * 16 + lc] >> (2 * (lc & 3))) - xsum; };
                        if (g.pair) {
                            const int col0 = (lo + r0 + row) * 16 + lc0;
                            const float sg = xscale * ld->ws[m0], su = xscale * ld->ws[m0 + 1];
                            const float a = pre_op(act, (float)val(row, lc0) * sg, (float)val(row + ns, lc0) * su);
                            const float b = pre_op(act, (float)val(row, lc1) * sg, (float)val(row + ns, lc1) * su);
                            st_volatile16(p.gate_t + col0 / 2, tag2(a, b, sl));
                        } else {
                            int mat, ls;
                            slot_to_mat(g, ph, lo + r0 + row, mat, ls);
                            const int col0 = ls * 16 + lc0;
                            const float sc = xscale * ld->ws[m0 + mat];
                            const float f0 = (float)val(row, lc0) * sc, f1 = (float)val(row, lc1) * sc;
                            if (ph == 0) {
                                uint4* dst = mat == 0 ? p.q_t : (mat == 1 ? p.k_t : p.v_t);
                                if (!(layer == 0 && cta == p.fault_cta)) st_volatile16(dst + col0 / 2, tag2(f0, f1, sl));
                            } else {
                                // residual add on the CTA's own columns
                                float* o = own + (r0 + row) * 16 + lc0;
                                const float h0 = o[0] + f0, h1 = o[1] + f1;
                                o[0] = h0; o[1] = h1;
                                st_volatile16(p.hid_t + col0 / 2, tag2(h0, h1, seq_hid(2 * layer + (ph == 1 ? 1 : 2))));
                                if (layer == p.L - 1 && ph == 3) *reinterpret_cast<float2*>(p.hidden + col0) = make_float2(h0, h1);
                            }
                        }
                    }
                    // the weight stream moves on: the stage freed by the warp's last unit is refilled now, off
                    // the path from the last multiply to the store above
                    if (warp < units) issue();
                    __syncthreads();
                    if (tid < kRoundStrips * 16) acc_s[tid] = 0;
                    if (r0 + rs < n_slots) __syncthreads();      // zeroed before the next round adds
                }
                if (tid == 0) misc[1] = 0;
                TR();
            }

            if (ph == 0 && my_first >= 0) {
                // ---- attention: this CTA's (chunk, KV head) items
                TR();
                AttnTagged tg;
                tg.q.words = p.q_t; tg.q.seq = sl; tg.q.ctx = ctx;
                tg.k.words = p.k_t; tg.k.seq = sl; tg.k.ctx = ctx;
                tg.v.words = p.v_t; tg.v.seq = sl; tg.v.ctx = ctx;
                tg.rope_row = rope_s; tg.rec_t = p.rec_t; tg.att_t = p.att_t; tg.seq = sl; tg.ml_s = ml_s;
#ifdef TERB_TRACE
                tg.trace = (layer == 1 && p.trace) ? p.trace + (size_t)cta * 32 + 20 : nullptr;
#endif
                for (int i = my_first; i >= 0; i -= grid) {
                    const AttnItem it = attn_item<HD>(ap, i / nkv_v, i % nkv_v, 0, pos);
                    if (i != my_first) {
                        __syncthreads();
                        if (tid == 0 && it.active && it.n_copy > 0) {
                            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                            attn_issue_kv<HD, GA, false>(ap, it, asmem);
                        }
                    }
                    kv_pending = false;
                    attn_compute<HD, GA, false, 2>(ap, it, asmem, redg, &misc[0], kv_parity, &tg);
                    if (it.active && it.n_copy > 0) kv_parity ^= 1u;
                }
                __syncthreads();
                if (misc[2]) { drain(); return; }
                TR();
            }
        }
    }
#undef TR
}

}  // namespace

DecodeStateLayout decode_state_layout(int H, int F, int Nh, int Nkv, int Hd, int Smax) {
    DecodeStateLayout l;
    const size_t Hq = (size_t)Nh * Hd, Hkv = (size_t)Nkv * Hd;
    const size_t mc = (size_t)(Smax + kAttnChunk - 1) / kAttnChunk;
    size_t o = 0;
    l.hid = o; o += (size_t)H / 2;
    l.q = o; o += Hq / 2;
    l.k = o; o += Hkv / 2;
    l.v = o; o += Hkv / 2;
    l.att = o; o += Hq / 2;
    l.gate = o; o += (size_t)F / 2;
    l.rec = o; o += (size_t)Nh * mc * ((size_t)Hd / 2 + 1);
    l.total = o;
    return l;
}

bool decode_layers_supported(int H, int F, int Nh, int Nkv, int Hd, int L) {
    const int Hq = Nh * Hd;
    if (Hd != 64 && Hd != 128) return false;
    if (Nkv < 1 || Nh % Nkv != 0) return false;
    const int G = Nh / Nkv;
    if (G != 1 && G != 2 && G != 4 && G != 8) return false;
    if (H > kNqFastMax || F > kNqFastMax || Hq > kNqFastMax) return false;
    if (H % 16 || F % 16 || Hq % 16 || (Nkv * Hd) % 16) return false;
    if (L < 1 || L > 128) return false;      // the per-layer constants are staged in shared memory
    return true;
}

namespace {
template <int HD, int G, int GA>
cudaError_t launch_variant_ga(DecodeParams& p, int sm_count, cudaStream_t st, int dev) {
    constexpr int kMaxSmem = 227 * 1024;
    constexpr int kAttnBytes = (AttnSmem<HD, GA, false>::kBytes + 127) & ~127;
    const size_t fixed = (size_t)kHdr + (size_t)p.tab_bytes + (size_t)p.own_bytes + (size_t)p.x_bytes + kAttnBytes;
    if (fixed + (size_t)kDecWarps * kBlockBytes > (size_t)kMaxSmem) return cudaErrorInvalidValue;
    int stages = (int)((kMaxSmem - fixed) / ((size_t)kDecWarps * kBlockBytes));
    if (stages > kDecMaxStages) stages = kDecMaxStages;
    p.stages = stages;
    const size_t smem = fixed + (size_t)kDecWarps * stages * kBlockBytes;
    static bool attr_set[64] = {};
    auto kern = decode_layers_kernel<HD, G, GA>;
    if (!attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3((unsigned)sm_count);
    lc.blockDim = dim3(kT);
    lc.dynamicSmemBytes = smem;
    lc.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;     // all CTAs resident: they wait on each other's values
    attr[0].val.cooperative = 1;
    lc.attrs = attr;
    lc.numAttrs = 1;
    return cudaLaunchKernelEx(&lc, kern, p);
}
template <int HD, int G>
cudaError_t launch_variant(DecodeParams& p, int sm_count, cudaStream_t st, int dev) {
    // one item per query head when the items of the longest context still fit the CTAs
    const long per_head_items = (long)((p.Smax + kAttnChunk - 1) / kAttnChunk) * p.Nh;
    if (G >= 2 && per_head_items <= sm_count) return launch_variant_ga<HD, G, 1>(p, sm_count, st, dev);
    return launch_variant_ga<HD, G, attn_item_heads(G)>(p, sm_count, st, dev);
}
template <int HD>
cudaError_t launch_hd(DecodeParams& p, int sm_count, cudaStream_t st, int dev) {
    switch (p.Nh / p.Nkv) {
        case 1: return launch_variant<HD, 1>(p, sm_count, st, dev);
        case 2: return launch_variant<HD, 2>(p, sm_count, st, dev);
        case 4: return launch_variant<HD, 4>(p, sm_count, st, dev);
        case 8: return launch_variant<HD, 8>(p, sm_count, st, dev);
        default: return cudaErrorInvalidValue;
    }
}
}  // namespace

cudaError_t launch_decode_layers(const DecodeParams& p_in, int sm_count, cudaStream_t st) {
    if (!decode_layers_supported(p_in.H, p_in.F, p_in.Nh, p_in.Nkv, p_in.Hd, p_in.L)) return cudaErrorInvalidValue;
    DecodeParams p = p_in;
    int kmax = p.H > p.F ? p.H : p.F;
    if (p.Nh * p.Hd > kmax) kmax = p.Nh * p.Hd;
    p.x_bytes = (kmax + 127) & ~127;
    p.tab_bytes = (p.L * (int)sizeof(DecodeLayerDev) + 127) & ~127;
    const int own_slots = ((p.H >> 4) + sm_count - 1) / sm_count;
    p.own_bytes = (own_slots * 16 * 4 + 127) & ~127;
    if (p.wait_ns == 0) p.wait_ns = 2000000000ull;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    return p.Hd == 64 ? launch_hd<64>(p, sm_count, st, dev) : launch_hd<128>(p, sm_count, st, dev);
}

}  // namespace terb
