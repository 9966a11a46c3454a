// Reader for the reference's packed-model files: 'LLRT' (Llama architecture,
// tools/convert_llama_to_packed.py:13-43, loader cuda/ter_cuda_forward_packed.cu:589-667) and
// 'TERT' (BitNet architecture, tools/convert_bitnet_to_packed.py:4-31, loader
// cuda/ter_cuda_forward_bitnet.cu:698-784).  Layout, little-endian:
//   64-byte header: magic u32, version u32 (= 1), H F L V Nh Nkv Hd Smax u32, rope_theta f32, eps f32
//   token_embd fp16 [V][H] (tied lm_head), output_norm f32 [H]
//   per layer: attn_norm f32[H], ffn_norm f32[H], (TERT only: attn_sub_norm f32[H], ffn_sub_norm f32[F]),
//              then Wq Wk Wv Wo Wgate Wup Wdown, each K*N/4 bytes in the v11 byte order + one f32 scale.
// The file's fp16 embeddings are rounded to bf16 (nearest even), the storage type of this library's table.
// Unlike the reference's loaders nothing here exits the process: every failure is a return code.
#include <stdio.h>
#include <stdlib.h>

#include "handle.h"

namespace {

constexpr uint32_t kMagicLlama = 0x4C4C5254u;    // 'LLRT'
constexpr uint32_t kMagicBitnet = 0x54455254u;   // 'TERT'

float half_to_float(uint16_t hbits) {
    const uint32_t sign = (uint32_t)(hbits & 0x8000u) << 16;
    uint32_t exp = (hbits >> 10) & 0x1Fu, man = hbits & 0x3FFu, out;
    if (exp == 0) {
        if (man == 0) {
            out = sign;
        } else {   // subnormal half: normalise
            int e = -1;
            do { man <<= 1; ++e; } while (!(man & 0x400u));
            out = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FFu) << 13);
        }
    } else if (exp == 31) {
        out = sign | 0x7F800000u | (man << 13);
    } else {
        out = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &out, 4);
    return f;
}

uint16_t float_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7F800000u) == 0x7F800000u && (u & 0x007FFFFFu)) return (uint16_t)((u >> 16) | 0x40u);   // NaN stays NaN
    u += 0x7FFFu + ((u >> 16) & 1u);   // round to nearest even
    return (uint16_t)(u >> 16);
}

struct FileHdr {
    uint32_t magic, version, H, F, L, V, Nh, Nkv, Hd, Smax;
    float rope_theta, eps;
};

int read_header(FILE* fp, FileHdr* hd) {
    uint8_t raw[64];
    if (fread(raw, 1, 64, fp) != 64) return TER_B200_E_IO;
    memcpy(hd, raw, sizeof(FileHdr));
    if ((hd->magic != kMagicLlama && hd->magic != kMagicBitnet) || hd->version != 1) return TER_B200_E_IO;
    if (!hd->H || !hd->F || !hd->L || !hd->V || !hd->Nh || !hd->Nkv || !hd->Hd) return TER_B200_E_SHAPE;
    if (hd->H > (1u << 20) || hd->F > (1u << 20) || hd->L > 4096 || hd->V > (1u << 24)) return TER_B200_E_SHAPE;
    return TER_B200_OK;
}

void fill_cfg(const FileHdr& hd, int smax, int max_batch, ter_b200_model_cfg_t* c) {
    memset(c, 0, sizeof *c);
    c->arch = hd.magic == kMagicBitnet ? TER_B200_ARCH_BITNET : TER_B200_ARCH_LLAMA;
    c->H = (int)hd.H; c->F = (int)hd.F; c->L = (int)hd.L; c->V = (int)hd.V;
    c->Nh = (int)hd.Nh; c->Nkv = (int)hd.Nkv; c->Hd = (int)hd.Hd;
    c->Smax = smax > 0 ? smax : (int)hd.Smax;
    c->eps = hd.eps;
    c->rope_theta = (double)hd.rope_theta;
    c->lm_head_packed = 0;
    c->max_batch = max_batch > 0 ? max_batch : 1;
}

}  // namespace

extern "C" {

int ter_b200_model_file_info(const char* path, ter_b200_model_cfg_t* cfg_out) {
    if (!path || !cfg_out) return TER_B200_E_NULL;
    FILE* fp = fopen(path, "rb");
    if (!fp) return TER_B200_E_IO;
    FileHdr hd;
    const int rc = read_header(fp, &hd);
    fclose(fp);
    if (rc) return rc;
    fill_cfg(hd, 0, 1, cfg_out);
    return TER_B200_OK;
}

int ter_b200_model_load_file(ter_b200_handle_t* h, const char* path, int smax, int max_batch,
                             ter_b200_model_cfg_t* cfg_out) {
    if (!h || !path) return TER_B200_E_NULL;
    FILE* fp = fopen(path, "rb");
    if (!fp) return TER_B200_E_IO;
    FileHdr hd;
    int rc = read_header(fp, &hd);
    if (rc) { fclose(fp); return rc; }
    ter_b200_model_cfg_t cfg;
    fill_cfg(hd, smax, max_batch, &cfg);
    rc = ter_b200_model_create(h, &cfg);
    if (rc) { fclose(fp); return rc; }

    const size_t H = hd.H, F = hd.F, V = hd.V, Hkv = (size_t)hd.Nkv * hd.Hd, Hq = (size_t)hd.Nh * hd.Hd;
    size_t big = V * H * sizeof(uint16_t);
    size_t dmax = H > F ? H : F;
    if (Hq > dmax) dmax = Hq;
    const size_t mat_max = dmax * (dmax / 4 + 1);
    if (mat_max > big) big = mat_max;
    uint8_t* buf = (uint8_t*)malloc(big);
    float* vec = (float*)malloc(sizeof(float) * (F > H ? F : H));
    if (!buf || !vec) { free(buf); free(vec); fclose(fp); return TER_B200_E_ALLOC; }
    auto fail = [&](int code) { free(buf); free(vec); fclose(fp); return code; };

    // embeddings: fp16 in the file, bf16 in the library
    if (fread(buf, sizeof(uint16_t), V * H, fp) != V * H) return fail(TER_B200_E_IO);
    uint16_t* e = (uint16_t*)buf;
    for (size_t i = 0; i < V * H; ++i) e[i] = float_to_bf16(half_to_float(e[i]));
    rc = ter_b200_model_set_embd(h, e);
    if (rc) return fail(rc);
    if (fread(vec, sizeof(float), H, fp) != H) return fail(TER_B200_E_IO);
    rc = ter_b200_model_set_vector(h, -1, 0, vec);
    if (rc) return fail(rc);

    const int n_vec = cfg.arch == TER_B200_ARCH_BITNET ? 4 : 2;
    const size_t vec_len[4] = {H, H, H, F};   // attn_norm, ffn_norm, attn_sub_norm, ffn_sub_norm
    const size_t mK[7] = {H, H, H, Hq, H, H, F};
    const size_t mN[7] = {Hq, Hkv, Hkv, H, F, F, H};
    for (int L = 0; L < cfg.L; ++L) {
        for (int v = 0; v < n_vec; ++v) {
            if (fread(vec, sizeof(float), vec_len[v], fp) != vec_len[v]) return fail(TER_B200_E_IO);
            rc = ter_b200_model_set_vector(h, L, v, vec);
            if (rc) return fail(rc);
        }
        for (int w = 0; w < 7; ++w) {
            const size_t bytes = mK[w] * (mN[w] / 4);
            float scale;
            if (fread(buf, 1, bytes, fp) != bytes || fread(&scale, sizeof(float), 1, fp) != 1) return fail(TER_B200_E_IO);
            rc = ter_b200_model_set_matrix(h, L, w, buf, TER_B200_FMT_V11, scale);
            if (rc) return fail(rc);
        }
    }
    free(buf);
    free(vec);
    fclose(fp);
    if (cfg_out) *cfg_out = cfg;
    return TER_B200_OK;
}


// microsoft/BitNet "i2_s" tensor -> the v11 packed-trit bytes this library (and the reference's CUDA
// forward) takes.  What the reference's converter does in NumPy (tools/convert_bitnet_to_packed.py:85-152:
// read_i2s_scale, i2s_to_col_packed) and its CPU loader in C++ (vendor/ntransformer/core/dequant.cpp:114-145):
//   * the tensor is N rows (output features) of K inputs, flat row-major, in blocks of 128 elements;
//     a block is 32 bytes; byte p holds the codes of block positions p, p+32, p+64, p+96, position p
//     (group 0) in the HIGH two bits; codes 0 -> -1, 1 -> 0, 2 -> +1, 3 -> 0;
//   * 32 bytes follow the codes, the first four an fp32: the per-tensor scale.
// Output: bytes [N/4][K]; byte (n/4)*K + k holds output column n at bits 2*(n%4), codes 0 -> 0, +1 -> 1,
// -1 -> 2 (cuda/ter_cuda_forward_packed.cu:354-372).  Host memory only; needs no handle and no GPU.
int ter_b200_convert_i2s(const void* i2s, size_t i2s_bytes, int N, int K, uint8_t* v11_out, float* scale_out) {
    if (!i2s || !v11_out) return TER_B200_E_NULL;
    if (N < 4 || K < 1 || (N & 3) != 0) return TER_B200_E_SHAPE;
    const size_t total = (size_t)N * (size_t)K;
    if (total % 128 != 0) return TER_B200_E_SHAPE;
    if (i2s_bytes < total / 4 + (scale_out ? 4 : 0)) return TER_B200_E_IO;
    const uint8_t* src = static_cast<const uint8_t*>(i2s);
    if (scale_out) memcpy(scale_out, src + total / 4, sizeof(float));
    static const uint8_t kCode[4] = {2, 0, 1, 0};            // i2_s code -> v11 code (-1 -> 2, 0 -> 0, +1 -> 1)
    memset(v11_out, 0, total / 4);
    for (size_t blk = 0; blk < total / 128; ++blk) {
        const uint8_t* bb = src + blk * 32;
        for (int g = 0; g < 4; ++g) {
            const int shift = 6 - 2 * g;
            for (int p = 0; p < 32; ++p) {
                const size_t e = blk * 128 + (size_t)g * 32 + (size_t)p;   // flat element: row n, input k
                const size_t n = e / (size_t)K, k = e % (size_t)K;
                const uint8_t code = kCode[(bb[p] >> shift) & 3];
                v11_out[(n >> 2) * (size_t)K + k] |= (uint8_t)(code << (2 * (n & 3)));
            }
        }
    }
    return TER_B200_OK;
}

}  // extern "C"
