// ter_b200_generate: the command-line front end of the decode forward, over the C ABI only.
// Mirrors the main() of the reference's CUDA forwards (cuda/ter_cuda_forward_packed.cu:680-748,
// cuda/ter_cuda_forward_bitnet.cu): first argument n_gen, second argument the packed-model file.
//   ter_b200_generate [n_gen] [model.bin] [--prompt id,id,...] [--arch llama|bitnet] [--layers L]
//                     [--host-sampler] [--op-stats]
//   * with a model file ('LLRT' / 'TERT'): prints n_gen greedy tokens from BOS = 128000 (or from --prompt),
//     the reference's real-weight mode;
//   * without: a random-init model of the architecture (the reference's bench mode, random weights), 4 warm-up
//     positions, then n_gen graph-replayed steps, and prints ms/token and tokens/s in the reference's format.
// Sampling is greedy, as in the reference: on the device (argmax kernels) or, with --host-sampler, by the
// argmax sampler on the host over the logits (first maximum wins: vendor/ntransformer/inference/sampler.cpp:19-29).
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <string>
#include <vector>

#include "ter_b200.h"

namespace {

struct Lcg {
    uint64_t s;
    explicit Lcg(uint64_t seed) : s(seed * 0x9E3779B97F4A7C15ull + 77) {}
    uint32_t next() { s = s * 6364136223846793005ull + 1442695040888963407ull; return (uint32_t)(s >> 33); }
};

uint16_t f32_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

int argmax_sampler(const float* logits, int vocab) {   // first maximum wins
    int best = 0;
    float bv = logits[0];
    for (int i = 1; i < vocab; ++i)
        if (logits[i] > bv) { bv = logits[i]; best = i; }
    return best;
}

int fail(const char* what, int rc) {
    fprintf(stderr, "%s: %s (%d)\n", what, ter_b200_strerror(rc), rc);
    return 1;
}

// Random-init model: trits iid {-1: 0.3, 0: 0.4, +1: 0.3} as v11 bytes, scales 0.02, bf16 embeddings ~U(-0.035, 0.035).
int fill_random(ter_b200_handle_t* h, const ter_b200_model_cfg_t& c) {
    Lcg r(42);
    const int Hq = c.Nh * c.Hd, Hkv = c.Nkv * c.Hd;
    const int K[7] = {c.H, c.H, c.H, Hq, c.H, c.H, c.F};
    const int N[7] = {Hq, Hkv, Hkv, c.H, c.F, c.F, c.H};
    std::vector<uint8_t> buf;
    std::vector<float> ones((size_t)(c.F > c.H ? c.F : c.H), 1.0f);
    for (int L = 0; L < c.L; ++L) {
        for (int w = 0; w < 7; ++w) {
            buf.resize((size_t)K[w] * (size_t)(N[w] / 4));
            for (auto& b : buf) {
                uint8_t v = 0;
                for (int i = 0; i < 4; ++i) {
                    const uint32_t u = r.next() % 10u;
                    v |= (uint8_t)((u < 3 ? 2u : (u < 7 ? 0u : 1u)) << (2 * i));
                }
                b = v;
            }
            int rc = ter_b200_model_set_matrix(h, L, w, buf.data(), TER_B200_FMT_V11, 0.02f);
            if (rc) return rc;
        }
        for (int v = 0; v < (c.arch == TER_B200_ARCH_BITNET ? 4 : 2); ++v) {
            int rc = ter_b200_model_set_vector(h, L, v, ones.data());
            if (rc) return rc;
        }
    }
    int rc = ter_b200_model_set_vector(h, -1, 0, ones.data());
    if (rc) return rc;
    std::vector<uint16_t> emb((size_t)c.V * (size_t)c.H);
    for (auto& e : emb) e = f32_to_bf16(((float)(r.next() % 20001u) - 10000.0f) * 3.5e-6f);
    return ter_b200_model_set_embd(h, emb.data());
}

}  // namespace

int main(int argc, char** argv) {
    int n_gen = 32, layers = 0;
    const char* bin_path = nullptr;
    const char* arch = "llama";
    bool host_sampler = false, op_stats = false;
    std::vector<int32_t> prompt;
    int positional = 0;
    for (int i = 1; i < argc; ++i) {
        const std::string a = argv[i];
        if (a == "--prompt" && i + 1 < argc) {
            char* s = argv[++i];
            for (char* tok = strtok(s, ","); tok; tok = strtok(nullptr, ",")) prompt.push_back(atoi(tok));
        } else if (a == "--arch" && i + 1 < argc) {
            arch = argv[++i];
        } else if (a == "--layers" && i + 1 < argc) {
            layers = atoi(argv[++i]);
        } else if (a == "--host-sampler") {
            host_sampler = true;
        } else if (a == "--op-stats") {
            op_stats = true;
        } else if (a == "--help" || a == "-h") {
            printf("usage: %s [n_gen] [model.bin] [--prompt id,id,...] [--arch llama|bitnet] [--layers L] "
                   "[--host-sampler] [--op-stats]\n", argv[0]);
            return 0;
        } else if (positional == 0) {
            n_gen = atoi(argv[i]); ++positional;
        } else if (positional == 1) {
            bin_path = argv[i]; ++positional;
        }
    }
    if (n_gen < 1) n_gen = 1;

    ter_b200_handle_t* h = ter_b200_create(0);
    if (!h) { fprintf(stderr, "no CUDA device (this program has no CPU path)\n"); return 1; }
    ter_b200_model_cfg_t c;
    memset(&c, 0, sizeof c);
    int rc;
    if (bin_path) {
        printf("Loading weights from %s...\n", bin_path);
        if (prompt.empty()) prompt.push_back(128000);      // Llama 3 BOS, as the reference
        rc = ter_b200_model_load_file(h, bin_path, (int)prompt.size() + n_gen + 8, 1, &c);
        if (rc) return fail("load", rc);
        printf("Weights loaded: %s H=%d F=%d L=%d Nh=%d Nkv=%d Hd=%d V=%d\n", c.arch ? "bitnet" : "llama", c.H, c.F, c.L,
               c.Nh, c.Nkv, c.Hd, c.V);
    } else {
        const bool bitnet = strcmp(arch, "bitnet") == 0;
        c.arch = bitnet ? TER_B200_ARCH_BITNET : TER_B200_ARCH_LLAMA;
        c.H = bitnet ? 2560 : 2048; c.F = bitnet ? 6912 : 8192; c.L = layers > 0 ? layers : (bitnet ? 30 : 16);
        c.V = 128256; c.Nh = bitnet ? 20 : 32; c.Nkv = bitnet ? 5 : 8; c.Hd = bitnet ? 128 : 64;
        c.eps = 1e-5f; c.rope_theta = 500000.0; c.lm_head_packed = 0; c.max_batch = 1;
        if (prompt.empty()) prompt.assign(4, 1);            // the reference warms up on 4 positions of token 1
        c.Smax = (int)prompt.size() + n_gen + 8;
        printf("%s: H=%d F=%d L=%d Nh=%d Nkv=%d Hd=%d V=%d Smax=%d (random weights)\n", bitnet ? "BitNet 2B" : "Llama 1B",
               c.H, c.F, c.L, c.Nh, c.Nkv, c.Hd, c.V, c.Smax);
        printf("Weights: 1.58 bits/elem packed (4 trits/byte)\n");
        rc = ter_b200_model_create(h, &c);
        if (rc) return fail("model_create", rc);
        rc = fill_random(h, c);
        if (rc) return fail("fill", rc);
    }

    std::vector<int32_t> out((size_t)n_gen);
    if (host_sampler) {
        // one step at a time: logits to the host, the argmax sampler picks
        rc = ter_b200_model_reset(h, 1);
        if (rc) return fail("reset", rc);
        std::vector<float> logits((size_t)c.V);
        int32_t tok = prompt[0];
        const int steps = (int)prompt.size() + n_gen - 1;
        for (int pos = 0; pos < steps; ++pos) {
            int32_t nxt;
            rc = ter_b200_decode_step(h, &tok, &pos, &nxt, nullptr);
            if (rc) return fail("decode_step", rc);
            rc = ter_b200_model_logits(h, logits.data());
            if (rc) return fail("logits", rc);
            const int pick = argmax_sampler(logits.data(), c.V);
            if (pos + 1 < (int)prompt.size()) tok = prompt[(size_t)pos + 1];
            else { tok = pick; out[(size_t)(pos + 1 - (int)prompt.size())] = pick; }
        }
    } else {
        rc = ter_b200_generate(h, prompt.data(), 1, (int)prompt.size(), n_gen, out.data(), nullptr);
        if (rc) return fail("generate", rc);
        if (!bin_path) {                                    // timed run after the warm-up call
            rc = ter_b200_generate(h, prompt.data(), 1, (int)prompt.size(), n_gen, out.data(), nullptr);
            if (rc) return fail("generate", rc);
        }
    }
    if (bin_path || host_sampler) {
        printf("\nGreedy tokens from %s (n_gen=%d):\n", prompt.size() == 1 && prompt[0] == 128000 ? "BOS=128000" : "the prompt", n_gen);
        for (int i = 0; i < n_gen; ++i) printf(" %d", out[(size_t)i]);
        printf("\n");
    } else {
        const double ms = (double)ter_b200_last_generate_ms(h) - (double)ter_b200_last_prompt_ms(h);
        const int steps = ter_b200_last_prefill_ms(h) > 0.0f ? n_gen - 1 : n_gen;
        const double per_tok = steps > 0 ? ms / steps : 0.0;
        printf("\n=== ter_b200 packed-trit forward (1.58b weights, end-to-end) ===\n");
        printf("n_gen tokens : %d\n", n_gen);
        printf("total ms     : %.3f\n", ms);
        printf("ms / token   : %.4f\n", per_tok);
        printf("tokens/s     : %.1f\n", per_tok > 0 ? 1000.0 / per_tok : 0.0);
        printf("first tokens :");
        for (int i = 0; i < n_gen && i < 8; ++i) printf(" %d", out[(size_t)i]);
        printf("\n");
    }
    if (op_stats) {
        char buf[2048];
        ter_b200_dump_op_stats(h, bin_path ? bin_path : arch, c.H, c.F, c.Nh, c.Nkv, c.Hd, c.L, c.V,
                               (int)prompt.size() + n_gen - 1, buf, sizeof buf);
        fputs(buf, stderr);
    }
    const int st = ter_b200_device_status(h);
    ter_b200_destroy(h);
    return st == 0 ? 0 : 1;
}
