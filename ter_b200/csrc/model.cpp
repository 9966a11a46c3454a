// Decode forward: model weights, per-sequence state and the per-token launch sequence, in host
// C++ over the kernel launchers.  Stage order follows the reference's forward_token_dev
// (cuda/ter_cuda_forward_packed.cu:505-563; BitNet: cuda/ter_cuda_forward_bitnet.cu:850-913) and
// its NumPy statement (tools/llama_pyfwd.py:103-161, tools/bitnet_pyfwd.py:94-152).
#include <new>
#include <stdlib.h>

#include "decode.h"
#include "glue.h"
#include "handle.h"

using namespace terb;
#ifdef TERB_TRACE
unsigned long long* g_terb_trace = nullptr;
#endif

struct TerbModel {
    ter_b200_model_cfg_t c;
    DevWeight* mats;     // [L][7]
    float** vecs;        // [L][4] device vectors
    DevWeight lm_head;   // packed lm_head (optional)
    uint16_t* embd;      // bf16 [V][H]
    bool embd_owned;
    float* out_norm;
    const float* rope;   // owned by the handle's table cache
    // state
    int batch;
    float *hidden, *q, *k, *v, *att, *gate, *up, *xnorm, *logits, *attn_scratch, *argmax_scratch, *xs;
    int8_t* xq;
    uint16_t *kcache, *vcache;   // [L][B][Nkv][Smax][Hd]
    int *tokens, *pos, *greedy, *forced, *log, *ctl, *attn_counters;
    int forced_cap, log_cap;     // ints per sequence
    cudaGraphExec_t graph;
    int graph_batch;
    bool graph_forced;
    uint64_t graph_launches;
    uint64_t graph_tvmac;        // op-counter increment of one replay of the captured step
    cudaEvent_t ev0, ev1;
    float last_ms;
    // tensor parallelism over peer memory: the exchanged buffers (hidden, q, k, v, gate, up, logits) and
    // the flag words of the exchange points live in one arena that the peers have mapped
    PeerArena arena;
    size_t xrecv_off, xrecv_bytes;   // receive blocks of the exchange points, handed out in forward() order
    int* xseq;                       // int[kMaxExchangePoints][kMaxExchangeCtas], inside the arena
    bool shard_attn, shard_ffn;      // which blocks are column-sharded over the ranks (the lm_head always is)
    // prompt processing (prefill): the activation buffers hold `rows_cap` rows; a tile of prompt positions
    // goes through the layers as a token batch (tensor-core GEMM), all rows sharing sequence 0's cache
    int rows_cap;
    int *tok_rows, *pos_rows;        // [rows_cap] token ids and positions of the tile
    int32_t* xrs;                    // [rows_cap] row sums of the quantised activations (for the GEMM)
    cudaEvent_t ev_mid;
    float last_prefill_ms, last_prompt_ms;
    // persistent decode kernel (decode_sm100.cu): per-layer constants in device memory, its barrier word
    uint16_t* xsplit;        // bf16 hi / lo parts of the normalised rows (tensor-core lm_head, batches of 16 or more)
    DecodeLayerDev* dec_layers;
    uint4* dec_state;        // tagged activation vectors + attention records (decode_state_layout), then 4 control words
    bool dec_dirty;
};

constexpr int kPrefillTile = 1024;   // prompt positions per pass (four 256-token tiles of the GEMM)

namespace {

void mat_dims(const ter_b200_model_cfg_t& c, int which, int* K, int* N) {
    const int Hq = c.Nh * c.Hd, Hkv = c.Nkv * c.Hd;
    switch (which) {
        case TER_B200_WQ: *K = c.H; *N = Hq; break;
        case TER_B200_WK: case TER_B200_WV: *K = c.H; *N = Hkv; break;
        case TER_B200_WO: *K = Hq; *N = c.H; break;
        case TER_B200_WGATE: case TER_B200_WUP: *K = c.H; *N = c.F; break;
        default: *K = c.F; *N = c.H; break;
    }
}
int vec_len(const ter_b200_model_cfg_t& c, int which) {
    return which == TER_B200_FFN_SUB_NORM ? c.F : (which == TER_B200_ATTN_SUB_NORM ? c.Nh * c.Hd : c.H);
}
size_t cache_elems(const ter_b200_model_cfg_t& c) {
    return (size_t)c.L * c.max_batch * c.Nkv * (size_t)c.Smax * c.Hd;
}
void drop_graph(TerbModel* m) {
    if (m->graph) cudaGraphExecDestroy(m->graph);
    m->graph = nullptr;
}
template <typename T>
cudaError_t dalloc(T** p, size_t n) { return cudaMalloc((void**)p, n * sizeof(T)); }

// GEMV for every sequence of the batch (rows of X against the same weights).  With `nq` the
// quantiser runs inside the GEMV launch (fp32 rows in, no int8 round trip through memory).
int mm(ter_b200_handle_t* h, const DevWeight* const* ws, int n, const int8_t* xq, int K, const float* xs,
       float* const* outs, bool accumulate, int B, cudaStream_t st, const NormQuantParams* nq = nullptr,
       const int32_t* xrs = nullptr) {
    if (!nq && B >= 2)     // token batch: one launch over all rows and all the matrices (multi-row GEMV for a few
                           // rows, the tensor-core GEMM from gemm_min_m rows on)
        return run_gemm_group(h, ws, n, xq, xs, B, outs, nullptr, st, accumulate, B >= h->gemm_min_m ? xrs : nullptr);
    for (int b = 0; b < B; ++b) {
        float* o[kGemvMaxGroup];
        for (int i = 0; i < n; ++i) o[i] = outs[i] + (size_t)b * ws[i]->N;
        int rc = nq ? run_gemv(h, ws, n, nullptr, nullptr, 1.0f, o, nullptr, accumulate, st, nq, b)
                    : run_gemv(h, ws, n, xq + (size_t)b * K, xs + b, 1.0f, o, nullptr, accumulate, st);
        if (rc) return rc;
    }
    return TER_B200_OK;
}

bool can_fuse(const ter_b200_handle_t* h, const DevWeight* const* ws, int n, int B) {
    if (B >= 2) return false;   // batches go through the multi-row GEMV / the GEMM, which take quantised rows
    int tiles = 0;
    for (int i = 0; i < n; ++i) tiles += ws[i]->tiles();
    return h->gemv_cfg.fuse_quant && h->gemv_cfg.split_max_strips > 0 && tiles <= h->gemv_cfg.split_max_strips;
}

#define CK(call)                                              \
    do {                                                      \
        cudaError_t e__ = (call);                             \
        if (e__ != cudaSuccess) return cuda_fail(h, e__);     \
        h->launches += 1;                                     \
    } while (0)

// The launch sequence of one decode step for `B` sequences.
// prefill_rows > 0: the rows are `prefill_rows` consecutive positions of ONE prompt (tokens m->tok_rows,
// positions m->pos_rows, all in sequence 0's cache): rotary + append for all rows first, then causal
// attention per row; only the last row goes through the lm_head, and the step bookkeeping is left out.
// pre_seq: the sequence whose prompt the rows belong to (its cache, its logits row, its greedy token).
int forward(ter_b200_handle_t* h, TerbModel* m, bool use_forced, cudaStream_t st, int prefill_rows = 0, int pre_seq = 0) {
    const ter_b200_model_cfg_t& c = m->c;
    const bool pre = prefill_rows > 0;
    const int B = pre ? prefill_rows : m->batch, H = c.H, F = c.F, Hq = c.Nh * c.Hd;
    const bool gemm_rows = B >= h->gemm_min_m;   // token batch: projections on the tensor-core GEMM
    const int* posv = pre ? m->pos_rows : m->pos;
    const int* tokv = pre ? m->tok_rows : m->tokens;
    const bool pdl = h->gemv_cfg.pdl != 0;
    const bool bitnet = c.arch == TER_B200_ARCH_BITNET;
    const size_t layer_cache = (size_t)c.max_batch * c.Nkv * (size_t)c.Smax * c.Hd;
    // Tensor parallelism (batch 1): this rank computes columns [N*R/G, N*(R+1)/G) of every projection into
    // its slice of the full-size buffer; an in-place all-gather then gives every rank the whole vector.
    const int G = comm_size(h), R = comm_rank(h);
    const int Hkv = c.Nkv * c.Hd;
    // Per block: sharded over the G ranks, or replicated (every rank computes all columns, no exchange).
    // A batch-1 step is bound by kernel-to-kernel latency, not by weight bandwidth, so a replicated
    // block costs the same time and saves its two exchanges; the lm_head (the one large matrix) is
    // always split over the vocabulary.
    const bool sa = G > 1 && m->shard_attn, sf = G > 1 && m->shard_ffn;
    auto off = [&](int full_n) { return (size_t)(full_n / G) * (size_t)R; };
    auto offa = [&](int full_n) { return sa ? off(full_n) : (size_t)0; };
    auto offf = [&](int full_n) { return sf ? off(full_n) : (size_t)0; };
    auto ag = [&](float* buf, int full_n) -> int {
        return G > 1 ? comm_all_gather_bytes(h, buf, (size_t)(full_n / G) * sizeof(float), st) : TER_B200_OK;
    };
    // One exchange point: every rank's slices of up to three buffers reach every rank.  Peer memory path:
    // one kernel of peer stores + flags; otherwise NCCL all-gathers in one group.
    int point = 0;
    size_t recv_cursor = 0;
    auto exchange = [&](float* const* bufs, const int* full_n, int nb, bool sharded) -> int {
        if (G == 1 || !sharded) return TER_B200_OK;
        if (!m->arena.open) {
            int rc = nb > 1 ? comm_group_start(h) : TER_B200_OK;
            for (int i = 0; i < nb && !rc; ++i) rc = ag(bufs[i], full_n[i]);
            if (!rc && nb > 1) rc = comm_group_end(h);
            return rc;
        }
        if (point >= kMaxExchangePoints) return TER_B200_E_SHAPE;
        ExchangeParams xp;
        memset(&xp, 0, sizeof xp);
        for (int r = 0; r < G; ++r) xp.base[r] = m->arena.peer[r];
        for (int i = 0; i < nb; ++i) {
            xp.seg_buf_off[i] = (size_t)((uint8_t*)bufs[i] - m->arena.base);
            xp.seg_floats[i] = full_n[i] / G;
            xp.words_total += full_n[i] / G / 2;
        }
        xp.n_seg = nb;
        xp.rank = R;
        xp.size = G;
        // this point's two receive blocks (used in turn): one 16-byte word per pair of floats and per source rank
        const size_t block = 2u * (size_t)xp.words_total * 16u * (size_t)G;
        if (recv_cursor + block > m->xrecv_bytes) return TER_B200_E_SHAPE;
        xp.recv_off = m->xrecv_off + recv_cursor;
        recv_cursor += block;
        xp.seq = m->xseq + (size_t)point * kMaxExchangeCtas;
        xp.status = h->status_dev;
        xp.point = point;
        xp.wait_ns = (unsigned long long)h->wait_ms * 1000000ull;
        ++point;
        cudaError_t e = launch_peer_exchange(xp, pdl, st);
        if (e != cudaSuccess) return cuda_fail(h, e);
        h->launches += 1;
        return TER_B200_OK;
    };
#define XCHG1(buf, n, sharded) do { float* b__[1] = {(buf)}; int n__[1] = {(n)}; int rc__ = exchange(b__, n__, 1, (sharded)); if (rc__) return rc__; } while (0)

    // One sequence on one GPU: embedding and all layers in ONE cooperative launch (decode_sm100.cu).
    // (under tensor parallelism when the layers are replicated: every rank runs them whole)
    const bool persist = !pre && B == 1 && (G == 1 || (!sa && !sf)) && h->decode_persistent && m->dec_layers && !m->dec_dirty &&
                         decode_layers_supported(c.H, c.F, c.Nh, c.Nkv, c.Hd, c.L);
    if (persist) {
        DecodeParams dp;
        memset(&dp, 0, sizeof dp);
        const DecodeStateLayout sl = decode_state_layout(c.H, c.F, c.Nh, c.Nkv, c.Hd, c.Smax);
        dp.layers = m->dec_layers; dp.embd = m->embd; dp.tokens = m->tokens; dp.pos = m->pos;
        dp.hidden = m->hidden;
        dp.hid_t = m->dec_state + sl.hid; dp.q_t = m->dec_state + sl.q; dp.k_t = m->dec_state + sl.k;
        dp.v_t = m->dec_state + sl.v; dp.att_t = m->dec_state + sl.att; dp.gate_t = m->dec_state + sl.gate;
        dp.rec_t = m->dec_state + sl.rec;
        dp.ctl = reinterpret_cast<unsigned*>(m->dec_state + sl.total);
        dp.rope = m->rope; dp.status = h->status_dev;
        dp.L = c.L; dp.H = H; dp.F = F; dp.Nh = c.Nh; dp.Nkv = c.Nkv; dp.Hd = c.Hd; dp.Smax = c.Smax; dp.V = c.V;
        dp.bitnet = bitnet ? 1 : 0; dp.eps = c.eps;
        dp.wait_ns = (unsigned long long)h->wait_ms * 1000000ull;
        dp.fault_cta = h->decode_fault_cta;
        dp.poll_sleep_ns = h->decode_poll_ns;
#ifdef TERB_TRACE
        dp.trace = g_terb_trace;
#endif
        CK(launch_decode_layers(dp, h->sm_count, st));
        for (int L = 0; L < c.L; ++L)
            for (int w = 0; w < 7; ++w) count_gemv(h, m->mats[(size_t)L * 7 + w].K, m->mats[(size_t)L * 7 + w].N, 1);
    } else {
    CK(launch_embed(m->embd, tokv, m->hidden, H, B, c.V, pdl, st));
    }
    for (int L = 0; L < c.L && !persist; ++L) {
        const DevWeight* W = m->mats + (size_t)L * 7;
        float** vec = m->vecs + (size_t)L * 4;
        // ---- attention block
        {
            const DevWeight* ws[3] = {&W[TER_B200_WQ], &W[TER_B200_WK], &W[TER_B200_WV]};
            float* outs[3] = {m->q + offa(Hq), m->k + offa(Hkv), m->v + offa(Hkv)};
            NormQuantParams nq{m->hidden, nullptr, vec[TER_B200_ATTN_NORM], m->xq, m->xs, nullptr, H, B, PRE_NONE, c.eps};
            const bool fz = can_fuse(h, ws, 3, B);
            if (gemm_rows) nq.rowsum_out = m->xrs;
            if (!fz) CK(launch_norm_quant(nq, pdl, st));
            int rc = mm(h, ws, 3, m->xq, H, m->xs, outs, false, B, st, fz ? &nq : nullptr, gemm_rows ? m->xrs : nullptr);
            if (rc) return rc;
            float* xb[3] = {m->q, m->k, m->v};
            const int xn[3] = {Hq, Hkv, Hkv};
            if ((rc = exchange(xb, xn, 3, sa))) return rc;
        }
        // rotary, KV append and attention in one launch (+ the ordered merge of the chunks)
        uint16_t* kc = m->kcache + L * layer_cache;
        uint16_t* vc = m->vcache + L * layer_cache;
        if (pre) {
            RopeKvParams rp{m->q, m->k, m->v, m->rope, posv, kc, vc, B, c.Nh, c.Nkv, c.Hd, c.Smax, bitnet ? 1 : 0, pre_seq + 1};
            CK(launch_rope_kv(rp, pdl, st));
            AttnParams ap{m->q, kc, vc, posv, m->attn_scratch, m->att, B, c.Nh, c.Nkv, c.Hd, c.Smax,
                          (c.Smax + kAttnChunk - 1) / kAttnChunk, nullptr, nullptr, nullptr, nullptr, nullptr, 0,
                          h->status_dev, h->attn_inline_merge ? m->attn_counters : nullptr, pre_seq + 1};
            ap.mma = B >= h->attn_mma_min;
            CK(launch_attention(ap, pdl, st));
        } else {
            AttnParams ap{m->q, kc, vc, m->pos, m->attn_scratch, m->att, B, c.Nh, c.Nkv, c.Hd, c.Smax,
                          (c.Smax + kAttnChunk - 1) / kAttnChunk, m->rope, m->k, m->v, kc, vc, bitnet ? 1 : 0,
                          h->status_dev, h->attn_inline_merge ? m->attn_counters : nullptr, 0};
            ap.mma = B >= h->attn_mma_min;
            CK(launch_attention(ap, pdl, st));
        }
        if (!h->attn_inline_merge) h->launches += 1;
        {
            const DevWeight* ws[1] = {&W[TER_B200_WO]};
            float* outs[1] = {m->hidden + offa(H)};
            NormQuantParams aq{m->att, nullptr, bitnet ? vec[TER_B200_ATTN_SUB_NORM] : nullptr, m->xq, m->xs, nullptr,
                               Hq, B, PRE_NONE, c.eps};
            const bool fz = can_fuse(h, ws, 1, B);
            if (gemm_rows) aq.rowsum_out = m->xrs;
            if (!fz) CK(launch_norm_quant(aq, pdl, st));
            int rc = mm(h, ws, 1, m->xq, Hq, m->xs, outs, true, B, st, fz ? &aq : nullptr, gemm_rows ? m->xrs : nullptr);   // hidden += Wo(attn)
            if (rc) return rc;
            XCHG1(m->hidden, H, sa);
        }
        // ---- FFN block: gate and up in one launch whose epilogue applies the gated activation, then
        // the down projection whose prologue normalises (BitNet sub-norm) and quantises it.
        {
            const DevWeight* ws[2] = {&W[TER_B200_WGATE], &W[TER_B200_WUP]};
            float* outs[2] = {m->gate + offf(F), m->up + offf(F)};
            NormQuantParams fq{m->hidden, nullptr, vec[TER_B200_FFN_NORM], m->xq, m->xs, nullptr, H, B, PRE_NONE, c.eps};
            const bool fz = can_fuse(h, ws, 2, B);
            const DevWeight* wd[1] = {&W[TER_B200_WDOWN]};
            const bool pair = fz && can_fuse(h, wd, 1, B) && (((ws[0]->Kpad >> 7) + 7) / 8) <= 4;
            const int act = bitnet ? PRE_RELU2_MUL : PRE_SILU_MUL;
            if (gemm_rows) fq.rowsum_out = m->xrs;
            if (!fz) CK(launch_norm_quant(fq, pdl, st));
            if (pair) {
                for (int b = 0; b < B; ++b) {
                    int rc = run_gemv(h, ws, 2, nullptr, nullptr, 1.0f, outs, nullptr, false, st, &fq, b, act,
                                      m->gate + (size_t)b * F + offf(F));
                    if (rc) return rc;
                }
            } else {
                int rc = mm(h, ws, 2, m->xq, H, m->xs, outs, false, B, st, fz ? &fq : nullptr, gemm_rows ? m->xrs : nullptr);
                if (rc) return rc;
            }
            if (pair) {
                XCHG1(m->gate, F, sf);
            } else {
                float* xb[2] = {m->gate, m->up};
                const int xn[2] = {F, F};
                int rc = exchange(xb, xn, 2, sf);
                if (rc) return rc;
            }
            float* outd[1] = {m->hidden + offf(H)};
            NormQuantParams gq{m->gate, pair ? nullptr : m->up, bitnet ? vec[TER_B200_FFN_SUB_NORM] : nullptr, m->xq,
                               m->xs, nullptr, F, B, pair ? PRE_NONE : act, c.eps};
            const bool fd = can_fuse(h, wd, 1, B);
            if (gemm_rows) gq.rowsum_out = m->xrs;
            if (!fd) CK(launch_norm_quant(gq, pdl, st));
            int rc = mm(h, wd, 1, m->xq, F, m->xs, outd, true, B, st, fd ? &gq : nullptr, gemm_rows ? m->xrs : nullptr);    // hidden += Wdown(ffn)
            if (rc) return rc;
            XCHG1(m->hidden, H, sf);
        }
    }
    // lm_head: every sequence of a decode step; of a prompt tile only its last position
    const int Bh = pre ? 1 : B;
    const float* hid = pre ? m->hidden + (size_t)(B - 1) * H : m->hidden;
    float* logits = m->logits + (pre ? (size_t)pre_seq * c.V : 0);      // a prompt's last row fills its sequence's row
    if (c.lm_head_packed) {
        // bench-mode packed lm_head: cuda/ter_cuda_forward_packed.cu:541-545
        NormQuantParams oq{hid, nullptr, m->out_norm, m->xq, m->xs, nullptr, H, Bh, PRE_NONE, c.eps};
        CK(launch_norm_quant(oq, pdl, st));
        const DevWeight* ws[1] = {&m->lm_head};
        float* outs[1] = {logits + off(c.V)};
        int rc = mm(h, ws, 1, m->xq, H, m->xs, outs, false, Bh, st);
        if (rc) return rc;
        XCHG1(logits, c.V, true);
    } else {
        NormQuantParams on{hid, nullptr, m->out_norm, nullptr, nullptr, m->xnorm, H, Bh, PRE_NONE, c.eps};
        CK(launch_norm_quant(on, pdl, st));
        if (m->xsplit && Bh >= h->lm_head_tc_min && H % 64 == 0) {
            // a token batch: the table goes through the tensor cores once for all rows (rounding-level differences
            // from the exact kernel; option "lm_head_tc_min" moves or disables the switch)
            CK(launch_lm_head_tc(m->embd + off(c.V) * H, m->xnorm, logits + off(c.V), c.V / G, H, Bh, m->xsplit,
                                 h->status_dev, pdl, st));
            h->launches += 1;
        } else {
            CK(launch_lm_head_bf16(m->embd + off(c.V) * H, m->xnorm, logits + off(c.V), c.V / G, H, Bh, h->sm_count, pdl, st));
        }
        XCHG1(logits, c.V, true);
        const uint64_t n = (uint64_t)((H + 26) / 27) * (uint64_t)c.V * (uint64_t)Bh;
        h->counts.tvmac += n;
        h->counts.total_ops += n;
    }
    CK(launch_argmax(logits, c.V, Bh, m->argmax_scratch, m->greedy + (pre ? pre_seq : 0), pdl, st));
    h->launches += 1;
    if (pre) return TER_B200_OK;
    SelectParams sp{m->greedy, use_forced ? m->forced : nullptr, m->tokens, m->pos, use_forced ? m->log : nullptr,
                    m->ctl, B, m->forced_cap, m->log_cap,
                    persist ? reinterpret_cast<unsigned*>(m->dec_state + decode_state_layout(c.H, c.F, c.Nh, c.Nkv, c.Hd, c.Smax).total)
                            : nullptr};
    CK(launch_select(sp, pdl, st));
    return TER_B200_OK;
}

bool model_complete(const TerbModel* m) {
    if (!m->embd || !m->out_norm) return false;
    const bool bitnet = m->c.arch == TER_B200_ARCH_BITNET;
    for (int L = 0; L < m->c.L; ++L) {
        for (int w = 0; w < 7; ++w)
            if (!m->mats[(size_t)L * 7 + w].data) return false;
        if (!m->vecs[(size_t)L * 4 + TER_B200_ATTN_NORM] || !m->vecs[(size_t)L * 4 + TER_B200_FFN_NORM]) return false;
        if (bitnet && (!m->vecs[(size_t)L * 4 + TER_B200_ATTN_SUB_NORM] || !m->vecs[(size_t)L * 4 + TER_B200_FFN_SUB_NORM]))
            return false;
    }
    if (m->c.lm_head_packed && !m->lm_head.data) return false;
    return true;
}

// Writes the per-layer constants of the persistent decode kernel to device memory (synchronous: not for
// use while a stream is capturing) and clears its barrier word.
int prepare_decode(ter_b200_handle_t* h, TerbModel* m) {
#ifdef TERB_TRACE
    if (!g_terb_trace) { cudaMalloc((void**)&g_terb_trace, 148 * 32 * 8); cudaMemset(g_terb_trace, 0, 148 * 32 * 8); }
#endif
    if (!m->dec_dirty && m->dec_layers) return TER_B200_OK;
    const ter_b200_model_cfg_t& c = m->c;
    if (!m->dec_layers) TERB_CUDA(h, dalloc(&m->dec_layers, (size_t)c.L));
    const size_t state_words = decode_state_layout(c.H, c.F, c.Nh, c.Nkv, c.Hd, c.Smax).total + 1;
    if (!m->dec_state) {
        TERB_CUDA(h, dalloc(&m->dec_state, state_words));
        TERB_CUDA(h, cudaMemset(m->dec_state, 0, state_words * sizeof(uint4)));
    }
    DecodeLayerDev* host = new (std::nothrow) DecodeLayerDev[(size_t)c.L];
    if (!host) return TER_B200_E_ALLOC;
    const size_t layer_cache = (size_t)c.max_batch * c.Nkv * (size_t)c.Smax * c.Hd;
    for (int L = 0; L < c.L; ++L) {
        memset(&host[L], 0, sizeof host[L]);
        for (int w = 0; w < 7; ++w) {
            host[L].W[w] = m->mats[(size_t)L * 7 + w].data;
            host[L].ws[w] = m->mats[(size_t)L * 7 + w].scale;
        }
        for (int v = 0; v < 4; ++v) host[L].gamma[v] = m->vecs[(size_t)L * 4 + v];
        host[L].kcache = m->kcache + L * layer_cache;
        host[L].vcache = m->vcache + L * layer_cache;
    }
    TERB_CUDA(h, cudaDeviceSynchronize());
    cudaError_t e = cudaMemcpy(m->dec_layers, host, (size_t)c.L * sizeof(DecodeLayerDev), cudaMemcpyHostToDevice);
    delete[] host;
    if (e != cudaSuccess) return cuda_fail(h, e);
    m->dec_dirty = false;
    return TER_B200_OK;
}

}  // namespace

#ifdef TERB_TRACE
extern "C" int ter_b200_debug_trace(unsigned long long* host) {
    if (!g_terb_trace) return -1;
    cudaDeviceSynchronize();
    return (int)cudaMemcpy(host, g_terb_trace, 148 * 32 * 8, cudaMemcpyDeviceToHost);
}
#endif
namespace terb {
// A tuning knob changed: the captured decode step no longer matches the settings.
void model_invalidate_graph(ter_b200_handle_t* h) {
    if (h && h->model) drop_graph(h->model);
}
}  // namespace terb

extern "C" {

void ter_b200_model_free(ter_b200_handle_t* h) {
    if (!h || !h->model) return;
    TerbModel* m = h->model;
    cudaSetDevice(h->device);
    cudaDeviceSynchronize();
    drop_graph(m);
    if (m->mats) {
        for (int i = 0; i < m->c.L * 7; ++i) free_weight(&m->mats[i]);
        delete[] m->mats;
    }
    if (m->vecs) {
        for (int i = 0; i < m->c.L * 4; ++i)
            if (m->vecs[i]) cudaFree(m->vecs[i]);
        delete[] m->vecs;
    }
    free_weight(&m->lm_head);
    if (m->arena.base) {   // the exchanged buffers are part of the arena (collective: every rank frees together)
        m->hidden = m->q = m->k = m->v = m->gate = m->up = m->logits = nullptr;
        comm_arena_destroy(h, &m->arena, h->stream);
    }
    if (m->embd && m->embd_owned) cudaFree(m->embd);
    void* bufs[] = {m->out_norm, m->hidden, m->q, m->k, m->v, m->att, m->gate, m->up, m->xnorm, m->logits,
                    m->attn_scratch, m->argmax_scratch, m->xs, m->xq, m->kcache, m->vcache, m->tokens, m->pos,
                    m->greedy, m->forced, m->log, m->ctl, m->attn_counters, m->tok_rows, m->pos_rows, m->xrs,
                    m->dec_layers, m->dec_state, m->xsplit};
    for (void* b : bufs)
        if (b) cudaFree(b);
    if (m->ev0) cudaEventDestroy(m->ev0);
    if (m->ev1) cudaEventDestroy(m->ev1);
    if (m->ev_mid) cudaEventDestroy(m->ev_mid);
    delete m;
    h->model = nullptr;
}

int ter_b200_model_create(ter_b200_handle_t* h, const ter_b200_model_cfg_t* cfg) {
    if (!h || !cfg) return TER_B200_E_NULL;
    const ter_b200_model_cfg_t& c = *cfg;
    if (c.H < 16 || c.F < 16 || c.L < 1 || c.V < 1 || c.Nh < 1 || c.Nkv < 1 || c.Smax < 1 || c.max_batch < 1 ||
        c.max_batch > 1024)
        return TER_B200_E_SHAPE;
    if ((c.Hd != 64 && c.Hd != 128) || c.Nh % c.Nkv != 0) return TER_B200_E_SHAPE;
    { const int gq = c.Nh / c.Nkv; if (gq != 1 && gq != 2 && gq != 4 && gq != 8) return TER_B200_E_SHAPE; }
    if (c.H % 16 || c.F % 16 || (c.Nh * c.Hd) % 16 || c.H % 8) return TER_B200_E_SHAPE;
    if (c.arch != TER_B200_ARCH_LLAMA && c.arch != TER_B200_ARCH_BITNET) return TER_B200_E_SHAPE;
    {
        const int G = comm_size(h);
        if (G > 1) {   // every sharded width must split into whole 16-column strips per rank
            const bool sa = (h->tp_shard & 1) != 0, sf = (h->tp_shard & 2) != 0;
            const int widths[5] = {(sa || sf) ? c.H : 0, sf ? c.F : 0, sa ? c.Nh * c.Hd : 0, sa ? c.Nkv * c.Hd : 0, c.V};
            for (int w : widths)
                if (w % (16 * G) != 0) return TER_B200_E_SHAPE;
            if (c.max_batch != 1) return TER_B200_E_SHAPE;   // tensor parallelism serves one sequence; batches are sharded by sequence
        }
    }
    TERB_CUDA(h, cudaSetDevice(h->device));
    ter_b200_model_free(h);
    TerbModel* m = new (std::nothrow) TerbModel();
    if (!m) return TER_B200_E_ALLOC;
    m->c = c;
    m->batch = 1;
    m->dec_dirty = true;
    m->shard_attn = (h->tp_shard & 1) != 0;
    m->shard_ffn = (h->tp_shard & 2) != 0;
    h->model = m;
    m->mats = new (std::nothrow) DevWeight[(size_t)c.L * 7];
    m->vecs = new (std::nothrow) float*[(size_t)c.L * 4]();
    if (!m->mats || !m->vecs) { ter_b200_model_free(h); return TER_B200_E_ALLOC; }
    const int Hq = c.Nh * c.Hd, Hkv = c.Nkv * c.Hd;
    // rows of the activation buffers: the decode batch, or a tile of prompt positions (prefill)
    const int R = (h->prefill && c.max_batch < kPrefillTile) ? kPrefillTile : c.max_batch;
    m->rows_cap = R;
    const int B = c.max_batch;
    const int wide = c.F > Hq ? (c.F > c.H ? c.F : c.H) : (Hq > c.H ? Hq : c.H);
    cudaError_t e = cudaSuccess;
    auto A = [&](cudaError_t r) { if (e == cudaSuccess) e = r; };
    // Buffers that ranks exchange.  With a communicator of more than one rank they are carved out of one
    // arena that the peers map, followed by the words of the exchange points.
    {
        float** xb[7] = {&m->hidden, &m->q, &m->k, &m->v, &m->gate, &m->up, &m->logits};
        const size_t xn[7] = {(size_t)R * c.H, (size_t)R * Hq, (size_t)R * Hkv, (size_t)R * Hkv, (size_t)R * c.F,
                              (size_t)R * c.F, (size_t)B * c.V};
        bool carved = false;
        if (comm_size(h) > 1 && h->tp_p2p) {
            size_t total = 0, offs[7];
            for (int i = 0; i < 7; ++i) { offs[i] = total; total += (xn[i] * sizeof(float) + 255) & ~(size_t)255; }
            // receive blocks: 16 bytes per pair of floats of every exchanged vector of a step (see forward())
            const size_t recv_off = total;
            const size_t recv_bytes = ((size_t)c.L * ((size_t)Hq + 2 * Hkv + 2 * (size_t)c.H + 2 * (size_t)c.F) + c.V) * 16u;
            total += (recv_bytes + 255) & ~(size_t)255;
            const size_t seq_off = total;
            total += (size_t)kMaxExchangePoints * kMaxExchangeCtas * sizeof(int);
            const int rc = comm_arena_create(h, total, &m->arena, h->stream);
            if (rc == TER_B200_OK) {
                for (int i = 0; i < 7; ++i) *xb[i] = (float*)(m->arena.base + offs[i]);
                m->xrecv_off = recv_off;
                m->xrecv_bytes = recv_bytes;
                m->xseq = (int*)(m->arena.base + seq_off);
                carved = true;
            } else if (rc != TER_B200_E_STATE) {    // E_STATE: no peer access anywhere, stay on NCCL
                ter_b200_model_free(h);
                return rc;
            }
        }
        if (!carved)
            for (int i = 0; i < 7; ++i) A(dalloc(xb[i], xn[i]));
    }
    A(dalloc(&m->att, (size_t)R * Hq));
    A(dalloc(&m->xnorm, (size_t)B * c.H));
    if (B >= 16 && !c.lm_head_packed) A(dalloc(&m->xsplit, (size_t)2 * B * c.H));
    A(dalloc(&m->attn_scratch, attention_scratch_floats(R, c.Nh, c.Hd, c.Smax)));
    A(dalloc(&m->argmax_scratch, (size_t)B * kArgmaxParts * 2));
    A(dalloc(&m->xs, (size_t)R));
    A(dalloc(&m->xq, (size_t)R * wide));
    A(dalloc(&m->tok_rows, (size_t)R));
    A(dalloc(&m->pos_rows, (size_t)R));
    A(dalloc(&m->xrs, (size_t)R));
    A(dalloc(&m->kcache, cache_elems(c)));
    A(dalloc(&m->vcache, cache_elems(c)));
    A(dalloc(&m->tokens, (size_t)B));
    A(dalloc(&m->pos, (size_t)B));
    A(dalloc(&m->greedy, (size_t)B));
    A(dalloc(&m->ctl, 2));
    A(dalloc(&m->attn_counters, (size_t)R * c.Nkv));
    if (e == cudaSuccess) e = cudaMemset(m->kcache, 0, cache_elems(c) * 2);
    if (e == cudaSuccess) e = cudaMemset(m->vcache, 0, cache_elems(c) * 2);
    if (e == cudaSuccess) e = cudaMemset(m->tokens, 0, B * sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(m->pos, 0, B * sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(m->ctl, 0, 2 * sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(m->attn_counters, 0, (size_t)R * c.Nkv * sizeof(int));
    if (e == cudaSuccess) e = cudaEventCreate(&m->ev0);
    if (e == cudaSuccess) e = cudaEventCreate(&m->ev1);
    if (e == cudaSuccess) e = cudaEventCreate(&m->ev_mid);
    if (e != cudaSuccess) { ter_b200_model_free(h); return cuda_fail(h, e); }
    int rc = get_rope_table(h, c.Smax, c.Hd, c.rope_theta, &m->rope);
    if (rc) { ter_b200_model_free(h); return rc; }
    return TER_B200_OK;
}

static int set_matrix_common(ter_b200_handle_t* h, int layer, int which, const void* data, bool on_device,
                             int format, float scale) {
    if (!h || !data) return TER_B200_E_NULL;
    TerbModel* m = h->model;
    if (!m) return TER_B200_E_STATE;
    int K, N;
    DevWeight* dst;
    if (layer < 0) {
        K = m->c.H; N = m->c.V; dst = &m->lm_head;
    } else {
        if (layer >= m->c.L || which < 0 || which > TER_B200_WDOWN) return TER_B200_E_SHAPE;
        mat_dims(m->c, which, &K, &N);
        dst = &m->mats[(size_t)layer * 7 + which];
    }
    if (format < 0 || format > TER_B200_FMT_I32) return TER_B200_E_SHAPE;
    if (format != TER_B200_FMT_I32 && N % 4 != 0) return TER_B200_E_SHAPE;
    {
        // tensor parallelism: keep this rank's column range.  In the v11 layout byte-column jb is a run of
        // K bytes, so columns [N*R/G, N*(R+1)/G) are one contiguous byte range of the caller's matrix.
        const int G = comm_size(h), R = comm_rank(h);
        const bool sharded = layer < 0 || (which <= TER_B200_WO ? m->shard_attn : m->shard_ffn);
        if (G > 1 && sharded) {
            if (format != TER_B200_FMT_V11 || N % (16 * G) != 0) return TER_B200_E_SHAPE;
            data = (const uint8_t*)data + (size_t)(N / G) * R / 4 * (size_t)K;
            N = N / G;
        }
    }
    TERB_CUDA(h, cudaSetDevice(h->device));
    drop_graph(m);
    void* tmp = nullptr;
    const void* src = data;
    if (!on_device) {
        const size_t bytes = format == TER_B200_FMT_I32 ? (size_t)K * N * 4u : (size_t)K * (size_t)(N / 4);
        TERB_CUDA(h, cudaMalloc(&tmp, bytes));
        cudaError_t e = cudaMemcpyAsync(tmp, data, bytes, cudaMemcpyHostToDevice, h->stream);
        if (e != cudaSuccess) { cudaFree(tmp); return cuda_fail(h, e); }
        src = tmp;
    } else {
        TERB_CUDA(h, cudaDeviceSynchronize());   // the caller's producer stream is unknown
    }
    DevWeight w;
    int rc = build_weight_from_dev(h, src, format, K, N, scale, h->stream, &w);
    if (tmp) cudaFree(tmp);
    if (rc) return rc;
    free_weight(dst);
    *dst = w;
    m->dec_dirty = true;
    return TER_B200_OK;
}

int ter_b200_model_set_matrix(ter_b200_handle_t* h, int layer, int which, const void* data, int format, float scale) {
    return set_matrix_common(h, layer, which, data, false, format, scale);
}
int ter_b200_model_set_matrix_dev(ter_b200_handle_t* h, int layer, int which, const void* data_dev, int format,
                                  float scale) {
    return set_matrix_common(h, layer, which, data_dev, true, format, scale);
}

int ter_b200_model_set_vector(ter_b200_handle_t* h, int layer, int which, const float* v) {
    if (!h || !v) return TER_B200_E_NULL;
    TerbModel* m = h->model;
    if (!m) return TER_B200_E_STATE;
    TERB_CUDA(h, cudaSetDevice(h->device));
    float** slot;
    int n;
    if (layer < 0) {
        slot = &m->out_norm; n = m->c.H;
    } else {
        if (layer >= m->c.L || which < 0 || which > TER_B200_FFN_SUB_NORM) return TER_B200_E_SHAPE;
        slot = &m->vecs[(size_t)layer * 4 + which];
        n = vec_len(m->c, which);
    }
    drop_graph(m);
    m->dec_dirty = true;
    if (!*slot) TERB_CUDA(h, dalloc(slot, (size_t)n));
    TERB_CUDA(h, cudaMemcpy(*slot, v, (size_t)n * sizeof(float), cudaMemcpyHostToDevice));
    return TER_B200_OK;
}

int ter_b200_model_set_embd(ter_b200_handle_t* h, const uint16_t* table) {
    if (!h || !table) return TER_B200_E_NULL;
    TerbModel* m = h->model;
    if (!m) return TER_B200_E_STATE;
    TERB_CUDA(h, cudaSetDevice(h->device));
    drop_graph(m);
    const size_t n = (size_t)m->c.V * m->c.H;
    if (m->embd && !m->embd_owned) m->embd = nullptr;
    if (!m->embd) TERB_CUDA(h, dalloc(&m->embd, n));
    m->embd_owned = true;
    TERB_CUDA(h, cudaMemcpy(m->embd, table, n * 2, cudaMemcpyHostToDevice));
    return TER_B200_OK;
}
int ter_b200_model_set_embd_dev(ter_b200_handle_t* h, const uint16_t* table_dev) {
    if (!h || !table_dev) return TER_B200_E_NULL;
    TerbModel* m = h->model;
    if (!m) return TER_B200_E_STATE;
    TERB_CUDA(h, cudaSetDevice(h->device));
    TERB_CUDA(h, cudaDeviceSynchronize());
    drop_graph(m);
    const size_t n = (size_t)m->c.V * m->c.H;
    if (m->embd && !m->embd_owned) m->embd = nullptr;
    if (!m->embd) TERB_CUDA(h, dalloc(&m->embd, n));
    m->embd_owned = true;
    TERB_CUDA(h, cudaMemcpy(m->embd, table_dev, n * 2, cudaMemcpyDeviceToDevice));
    return TER_B200_OK;
}

int ter_b200_model_reset(ter_b200_handle_t* h, int batch) {
    if (!h) return TER_B200_E_NULL;
    TerbModel* m = h->model;
    if (!m) return TER_B200_E_STATE;
    if (batch < 1 || batch > m->c.max_batch) return TER_B200_E_SHAPE;
    TERB_CUDA(h, cudaSetDevice(h->device));
    TERB_CUDA(h, cudaDeviceSynchronize());
    if (batch != m->batch) drop_graph(m);
    m->batch = batch;
    TERB_CUDA(h, cudaMemset(m->pos, 0, batch * sizeof(int)));
    TERB_CUDA(h, cudaMemset(m->tokens, 0, batch * sizeof(int)));
    return TER_B200_OK;
}

int ter_b200_decode_step(ter_b200_handle_t* h, const int32_t* tokens_host, const int32_t* pos_host,
                         int32_t* next_host, void* stream) {
    if (!h) return TER_B200_E_NULL;
    TerbModel* m = h->model;
    if (!m || !model_complete(m)) return TER_B200_E_STATE;
    TERB_CUDA(h, cudaSetDevice(h->device));
    cudaStream_t st = pick_stream(h, stream);
    const int B = m->batch;
    { int rc0 = prepare_decode(h, m); if (rc0) return rc0; }
    if (pos_host)
        for (int b = 0; b < B; ++b)
            if (pos_host[b] < 0 || pos_host[b] >= m->c.Smax) return TER_B200_E_SHAPE;
    if (tokens_host) TERB_CUDA(h, cudaMemcpyAsync(m->tokens, tokens_host, B * sizeof(int), cudaMemcpyHostToDevice, st));
    if (pos_host) TERB_CUDA(h, cudaMemcpyAsync(m->pos, pos_host, B * sizeof(int), cudaMemcpyHostToDevice, st));
    int rc = forward(h, m, false, st);
    if (rc) return rc;
    if (next_host) {
        TERB_CUDA(h, cudaMemcpyAsync(next_host, m->tokens, B * sizeof(int), cudaMemcpyDeviceToHost, st));
        TERB_CUDA(h, cudaStreamSynchronize(st));
    }
    return TER_B200_OK;
}

int ter_b200_model_logits(ter_b200_handle_t* h, float* logits_host) {
    if (!h || !logits_host) return TER_B200_E_NULL;
    TerbModel* m = h->model;
    if (!m) return TER_B200_E_STATE;
    TERB_CUDA(h, cudaSetDevice(h->device));
    TERB_CUDA(h, cudaDeviceSynchronize());
    TERB_CUDA(h, cudaMemcpy(logits_host, m->logits, (size_t)m->batch * m->c.V * sizeof(float), cudaMemcpyDeviceToHost));
    return TER_B200_OK;
}
int ter_b200_model_hidden(ter_b200_handle_t* h, float* hidden_host) {
    if (!h || !hidden_host) return TER_B200_E_NULL;
    TerbModel* m = h->model;
    if (!m) return TER_B200_E_STATE;
    TERB_CUDA(h, cudaSetDevice(h->device));
    TERB_CUDA(h, cudaDeviceSynchronize());
    TERB_CUDA(h, cudaMemcpy(hidden_host, m->hidden, (size_t)m->batch * m->c.H * sizeof(float), cudaMemcpyDeviceToHost));
    return TER_B200_OK;
}

int ter_b200_generate(ter_b200_handle_t* h, const int32_t* prompts, int batch, int n_prompt, int n_gen,
                      int32_t* out_tokens, void* stream) {
    if (!h || !prompts || !out_tokens) return TER_B200_E_NULL;
    TerbModel* m = h->model;
    if (!m || !model_complete(m)) return TER_B200_E_STATE;
    if (batch < 1 || batch > m->c.max_batch || n_prompt < 1 || n_gen < 1 || n_prompt + n_gen - 1 > m->c.Smax)
        return TER_B200_E_SHAPE;
    TERB_CUDA(h, cudaSetDevice(h->device));
    // The steps are captured into a graph; the legacy default stream cannot be captured, so such a
    // request runs on the handle's own stream (the call is synchronous either way).
    cudaStream_t st = pick_stream(h, stream);
    if (st == cudaStreamLegacy || st == cudaStreamPerThread) st = h->stream;
    const int steps = n_prompt + n_gen - 1;
    int rc = ter_b200_model_reset(h, batch);
    if (rc) return rc;
    if ((rc = prepare_decode(h, m))) return rc;
    if (m->forced_cap < n_prompt || m->log_cap < steps) {
        drop_graph(m);
        if (m->forced) cudaFree(m->forced);
        if (m->log) cudaFree(m->log);
        m->forced = m->log = nullptr;
        m->forced_cap = m->log_cap = 0;
        TERB_CUDA(h, dalloc(&m->forced, (size_t)m->c.max_batch * n_prompt));
        m->forced_cap = n_prompt;
        TERB_CUDA(h, dalloc(&m->log, (size_t)m->c.max_batch * steps));
        m->log_cap = steps;
    }
    int* first = (int*)malloc(sizeof(int) * (size_t)batch);
    if (!first) return TER_B200_E_ALLOC;
    for (int b = 0; b < batch; ++b) {
        first[b] = prompts[(size_t)b * n_prompt];
        cudaError_t e = cudaMemcpy(m->forced + (size_t)b * m->forced_cap, prompts + (size_t)b * n_prompt,
                                   n_prompt * sizeof(int), cudaMemcpyHostToDevice);
        if (e != cudaSuccess) { free(first); return cuda_fail(h, e); }
    }
    cudaError_t e = cudaMemcpy(m->tokens, first, batch * sizeof(int), cudaMemcpyHostToDevice);
    free(first);
    if (e != cudaSuccess) return cuda_fail(h, e);
    const int ctl[2] = {n_prompt, steps};
    TERB_CUDA(h, cudaMemcpy(m->ctl, ctl, sizeof ctl, cudaMemcpyHostToDevice));

    if (batch >= h->gemm_min_m) {   // the GEMM scratch cannot grow while the step is being captured
        int widest = m->c.F > m->c.H ? m->c.F : m->c.H;
        if (m->c.Nh * m->c.Hd > widest) widest = m->c.Nh * m->c.Hd;
        if (m->c.lm_head_packed && m->c.V > widest) widest = m->c.V;
        rc = ensure_gemm_scratch(h, batch, widest);
        if (rc) return rc;
    }
    if (!m->graph || m->graph_batch != batch || !m->graph_forced) {
        drop_graph(m);
        const uint64_t mark = h->launches;
        const ter_b200_op_counts_t cmark = h->counts;
        TERB_CUDA(h, cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
        rc = forward(h, m, true, st);
        cudaGraph_t g = nullptr;
        cudaError_t ce = cudaStreamEndCapture(st, &g);
        if (rc) { if (g) cudaGraphDestroy(g); return rc; }
        if (ce != cudaSuccess) return cuda_fail(h, ce);
        ce = cudaGraphInstantiate(&m->graph, g, 0);
        cudaGraphDestroy(g);
        if (ce != cudaSuccess) { m->graph = nullptr; return cuda_fail(h, ce); }
        m->graph_launches = h->launches - mark;
        h->launches = mark;
        m->graph_tvmac = h->counts.tvmac - cmark.tvmac;      // recording is not executing: counted per replay below
        h->counts = cmark;
        m->graph_batch = batch;
        m->graph_forced = true;
    }
    if (m->arena.open) {   // ranks enter the replay loop together: the peer exchanges wait with a time limit
        rc = comm_barrier(h, st);
        if (rc) return rc;
    }
    // Prompt processing.  Prompts of at least two tokens go through the layers in passes of up to 1024
    // positions as a token batch (tensor-core GEMM, causal attention per row over the sequence's cache),
    // one sequence after the other, which leaves the caches, the positions and the first generated tokens
    // exactly as feeding the prompts one position at a time does.  Under tensor parallelism only with
    // replicated layers (the default policy).  Otherwise: one graph replay per prompt position.
    const bool use_prefill = h->prefill && n_prompt >= 2 && m->rows_cap >= 2 &&
                             (comm_size(h) == 1 || (!m->shard_attn && !m->shard_ffn));
    TERB_CUDA(h, cudaEventRecord(m->ev0, st));
    int replays = steps;
    if (use_prefill) {
        const int T = m->rows_cap < h->prefill_tile ? m->rows_cap : h->prefill_tile;
        int widest = m->c.F > m->c.H ? m->c.F : m->c.H;
        if (m->c.Nh * m->c.Hd > widest) widest = m->c.Nh * m->c.Hd;
        rc = ensure_gemm_scratch(h, T, widest);
        if (rc) return rc;
        int* iota = (int*)malloc(sizeof(int) * (size_t)T);
        if (!iota) return TER_B200_E_ALLOC;
        for (int b = 0; b < batch && !rc; ++b)
            for (int p0 = 0; p0 < n_prompt && !rc; p0 += T) {
                const int rows = n_prompt - p0 < T ? n_prompt - p0 : T;
                for (int r = 0; r < rows; ++r) iota[r] = p0 + r;
                cudaError_t ce = cudaMemcpyAsync(m->tok_rows, prompts + (size_t)b * n_prompt + p0, rows * sizeof(int),
                                                 cudaMemcpyHostToDevice, st);
                if (ce == cudaSuccess) ce = cudaMemcpyAsync(m->pos_rows, iota, rows * sizeof(int), cudaMemcpyHostToDevice, st);
                if (ce != cudaSuccess) { rc = cuda_fail(h, ce); break; }
                rc = forward(h, m, false, st, rows, b);
            }
        if (rc) { free(iota); return rc; }
        // bookkeeping of the last prompt position of every sequence: log the first generated token, pos = n_prompt
        for (int b = 0; b < batch; ++b) iota[b % T] = n_prompt - 1;
        cudaError_t cp = cudaSuccess;
        for (int b0 = 0; b0 < batch && cp == cudaSuccess; b0 += T)
            cp = cudaMemcpyAsync(m->pos + b0, iota, (size_t)(batch - b0 < T ? batch - b0 : T) * sizeof(int), cudaMemcpyHostToDevice, st);
        free(iota);
        if (cp != cudaSuccess) return cuda_fail(h, cp);
        SelectParams sp{m->greedy, m->forced, m->tokens, m->pos, m->log, m->ctl, batch, m->forced_cap, m->log_cap, nullptr};
        cudaError_t ce = launch_select(sp, h->gemv_cfg.pdl != 0, st);
        if (ce != cudaSuccess) return cuda_fail(h, ce);
        h->launches += 1;
        replays = n_gen - 1;
    }
    if (use_prefill) TERB_CUDA(h, cudaEventRecord(m->ev_mid, st));
    for (int i = 0; i < replays; ++i) {
        // without prefill the first n_prompt - 1 replays feed the prompt; the mark splits prompt from generation
        if (!use_prefill && i == n_prompt - 1) TERB_CUDA(h, cudaEventRecord(m->ev_mid, st));
        TERB_CUDA(h, cudaGraphLaunch(m->graph, st));
        h->launches += m->graph_launches;
        h->counts.tvmac += m->graph_tvmac;
        h->counts.total_ops += m->graph_tvmac;
    }
    TERB_CUDA(h, cudaEventRecord(m->ev1, st));
    TERB_CUDA(h, cudaStreamSynchronize(st));
    TERB_CUDA(h, cudaEventElapsedTime(&m->last_ms, m->ev0, m->ev1));
    TERB_CUDA(h, cudaEventElapsedTime(&m->last_prompt_ms, m->ev0, m->ev_mid));
    m->last_prefill_ms = use_prefill ? m->last_prompt_ms : 0.0f;
    for (int b = 0; b < batch; ++b)
        TERB_CUDA(h, cudaMemcpy(out_tokens + (size_t)b * n_gen, m->log + (size_t)b * m->log_cap + (n_prompt - 1),
                                n_gen * sizeof(int), cudaMemcpyDeviceToHost));
    int dst = 0;
    TERB_CUDA(h, cudaMemcpy(&dst, h->status_dev, sizeof(int), cudaMemcpyDeviceToHost));
    if (dst != 0) {
        cudaMemset(h->status_dev, 0, sizeof(int));
        cudaMemset(m->attn_counters, 0, (size_t)m->rows_cap * m->c.Nkv * sizeof(int));
        return TER_B200_E_TIMEOUT;
    }
    return TER_B200_OK;
}

float ter_b200_last_generate_ms(const ter_b200_handle_t* h) { return (h && h->model) ? h->model->last_ms : 0.0f; }
float ter_b200_last_prefill_ms(const ter_b200_handle_t* h) { return (h && h->model) ? h->model->last_prefill_ms : 0.0f; }
float ter_b200_last_prompt_ms(const ter_b200_handle_t* h) { return (h && h->model) ? h->model->last_prompt_ms : 0.0f; }

}  // extern "C"
