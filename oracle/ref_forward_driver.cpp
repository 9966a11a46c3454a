// TEST INFRASTRUCTURE, NOT PRODUCT CODE.
//
// C-ABI driver around the UNMODIFIED reference CPU decode forward, ter::tx::forward_token
// (src/tx/transformer.cpp:116-223), for the timed CPU baseline of bench.py.  It is linked with the
// reference's own translation units where they lie (oracle/Makefile); nothing is copied.
//
// The reference loads its models from GGUF files that are not available here, so the driver fills a
// synthetic ter::tx::BrandonTransformer (include/ter/tx/transformer.hpp:17-52) of a given architecture in
// place: ternary projection weights iid {-1: 0.3, 0: 0.4, +1: 0.3} as int32 payloads with one fp32 scale
// per tensor (the layout ter::TritTensor holds, include/ter/numfmt.hpp:17-36), a 9-trit token embedding
// table (tied lm_head), unit norm gains.  Positions below 27 route the softmax through the ternary
// simulator's bytecode kernels (src/tx/forward.cpp:469-470), which need kernel blobs and tables from disk;
// the timed tokens therefore sit at positions >= 27 (the cache below is zero: same arithmetic, same cost).
//
// Exports: ref_tx_create / ref_tx_destroy / ref_tx_forward_tokens, and ref_dequant_i2s = nt::dequant_i2_s
// (vendor/ntransformer/core/dequant.cpp:114-145), the reference's decode of microsoft/BitNet "i2_s" tensors.
#include <ter/kernels.hpp>
#include <ter/numfmt.hpp>
#include <ter/sim.hpp>
#include <ter/tx/forward.hpp>
#include <ter/tx/transformer.hpp>

#include <core/dequant.hpp>

#include <chrono>
#include <cstdint>
#include <new>
#include <vector>

namespace {

struct Rng {
    uint64_t s;
    explicit Rng(uint64_t seed) : s(seed * 0x9E3779B97F4A7C15ull + 0x1234567ull) {}
    uint32_t next() {
        s = s * 6364136223846793005ull + 1442695040888963407ull;
        return static_cast<uint32_t>(s >> 33);
    }
};

void fill_trits(ter::TritTensor& t, int rows, int cols, Rng& r, float scale) {
    t.shape = {rows, cols};
    t.scale = scale;
    t.n_trits_per_elem = 1;
    t.payload.resize(static_cast<size_t>(rows) * static_cast<size_t>(cols));
    for (auto& v : t.payload) {
        const uint32_t u = r.next() % 10u;
        v = u < 3 ? -1 : (u < 7 ? 0 : 1);
    }
}

struct RefTx {
    ter::Sim sim;
    ter::KernelTable kt;
    ter::tx::BrandonTransformer tx;
    RefTx() : sim(4096) {}
};

}  // namespace

extern "C" {

void* ref_tx_create(int bitnet, int H, int F, int L, int V, int Nh, int Nkv, int Hd, int Smax, float eps,
                    double rope_theta, uint64_t seed) {
    auto* c = new (std::nothrow) RefTx();
    if (!c) return nullptr;
    try {
        Rng r(seed);
        auto& tx = c->tx;
        tx.vocab_size = V; tx.hidden_size = H; tx.head_dim = Hd; tx.n_heads = Nh; tx.n_kv_heads = Nkv;
        tx.intermediate_size = F; tx.n_layers = L; tx.weight_tying = true;
        tx.rmsnorm_eps = eps; tx.rope_theta = static_cast<float>(rope_theta); tx.ffn_relu2 = bitnet != 0;
        tx.blocks.resize(static_cast<size_t>(L));
        tx.layer_map.resize(static_cast<size_t>(L));
        const int Hq = Nh * Hd, Hkv = Nkv * Hd;
        for (int l = 0; l < L; ++l) {
            auto& b = tx.blocks[static_cast<size_t>(l)];
            tx.layer_map[static_cast<size_t>(l)] = l;
            fill_trits(b.Wq, H, Hq, r, 0.02f);
            fill_trits(b.Wk, H, Hkv, r, 0.02f);
            fill_trits(b.Wv, H, Hkv, r, 0.02f);
            fill_trits(b.Wo, Hq, H, r, 0.02f);
            fill_trits(b.Wgate, H, F, r, 0.02f);
            fill_trits(b.Wup, H, F, r, 0.02f);
            fill_trits(b.Wdown, F, H, r, 0.02f);
            b.attn_norm_w.assign(static_cast<size_t>(H), 1.0f);
            b.ffn_norm_w.assign(static_cast<size_t>(H), 1.0f);
            if (bitnet) {
                b.attn_sub_norm_w.assign(static_cast<size_t>(Hq), 1.0f);
                b.ffn_sub_norm_w.assign(static_cast<size_t>(F), 1.0f);
            }
        }
        tx.kv_caches.resize(static_cast<size_t>(L));
        for (auto& kc : tx.kv_caches) kc.resize(Smax, Nkv, Hd);
        // 9-trit embedding table: integers in [-9841, 9841], scale so that values are ~U(-0.035, 0.035)
        tx.token_embd.shape = {V, H};
        tx.token_embd.n_trits_per_elem = 9;
        tx.token_embd.scale = 0.035f / 9841.0f;
        tx.token_embd.payload.resize(static_cast<size_t>(V) * static_cast<size_t>(H));
        for (auto& v : tx.token_embd.payload) v = static_cast<int32_t>(r.next() % 19683u) - 9841;
        tx.output_norm_w.assign(static_cast<size_t>(H), 1.0f);
    } catch (...) {
        delete c;
        return nullptr;
    }
    return c;
}

void ref_tx_destroy(void* c) { delete static_cast<RefTx*>(c); }

// Runs forward_token for n_tokens consecutive positions starting at first_pos (greedy: each token is the
// argmax of the previous logits), returns the seconds spent inside forward_token, or a negative value on
// an exception.  tokens_out receives the n_tokens greedy tokens.
double ref_tx_forward_tokens(void* c, int first_token, int first_pos, int n_tokens, int* tokens_out) {
    auto* ctx = static_cast<RefTx*>(c);
    if (!ctx || first_pos < 27) return -1.0;
    const ter::tx::LutAddrs luts{0, 0, 0, 0};
    double total = 0.0;
    int tok = first_token;
    try {
        for (int i = 0; i < n_tokens; ++i) {
            const auto t0 = std::chrono::steady_clock::now();
            const std::vector<float> logits =
                ter::tx::forward_token(ctx->sim, ctx->kt, ctx->tx, tok, first_pos + i, luts, nullptr, nullptr);
            total += std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
            int best = 0;
            for (int v = 1; v < static_cast<int>(logits.size()); ++v)
                if (logits[static_cast<size_t>(v)] > logits[static_cast<size_t>(best)]) best = v;
            tok = best;
            if (tokens_out) tokens_out[i] = best;
        }
    } catch (...) {
        return -2.0;
    }
    return total;
}

// src: n_elems/4 code bytes followed by the 32-byte trailer whose first fp32 is the scale.
void ref_dequant_i2s(const void* src, size_t n_elems, float* out) { nt::dequant_i2_s(src, n_elems, out); }

}  // extern "C"
