/* TEST INFRASTRUCTURE, NOT PRODUCT CODE.  See ter_oracle.h.
 *
 * Build: -O3 -ffp-contract=off (no implicit fused multiply-add): every fmaf()
 * below is a deliberate fused operation and every `a*b+c` is two roundings.
 * The CUDA kernels are written with the same explicit operations, so the two
 * sides agree bit-for-bit wherever the arithmetic is IEEE (+,-,*,/,sqrt,fma,
 * rint); exp() is a polynomial defined here (orc_expf) for the same reason.
 *
 * Floating-point reductions use ONE fixed order that depends on the problem
 * only ("block order"): 256 lane partials over elements 1024*r + 4*t + e
 * (t = lane, e = 0..3), an xor butterfly (16,8,4,2,1) inside each group of
 * 32 lanes, then the 8 group sums added left to right.
 */
#include "ter_oracle.h"
#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------ utils */
static inline float f32_from_bits(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t bits_from_f32(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

uint16_t orc_f32_to_bf16(float f) {            /* round to nearest even */
    uint32_t u = bits_from_f32(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40u); /* NaN */
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
float orc_bf16_to_f32(uint16_t h) { return f32_from_bits((uint32_t)h << 16); }

/* exp(x) in fp32: n = rint(x*log2e); r = x - n*ln2 (two-step); degree-5
 * polynomial in r times r^2, plus r, plus 1; scaled by 2^n.  Arguments are
 * clamped to [-87, 88]; below -87 the result is 0. */
float orc_expf(float x) {
    if (!(x >= -87.0f)) return 0.0f;
    if (x > 88.0f) x = 88.0f;
    float n = rintf(x * 1.44269504088896341f);
    float r = fmaf(n, -0.693145751953125f, x);
    r = fmaf(n, -1.42860682030941723212e-6f, r);
    float p = 1.9875691500e-4f;
    p = fmaf(p, r, 1.3981999507e-3f);
    p = fmaf(p, r, 8.3334519073e-3f);
    p = fmaf(p, r, 4.1665795894e-2f);
    p = fmaf(p, r, 1.6666665459e-1f);
    p = fmaf(p, r, 5.0000001201e-1f);
    float r2 = r * r;
    float y = fmaf(p, r2, r);
    y = y + 1.0f;
    int ni = (int)n;
    return y * f32_from_bits((uint32_t)(ni + 127) << 23);
}

static float block_reduce_sum(const float* p /*256*/) {
    float total = 0.0f;
    for (int w = 0; w < 8; ++w) {
        float v[32], nv[32];
        memcpy(v, p + 32 * w, sizeof v);
        for (int o = 16; o > 0; o >>= 1) {
            for (int l = 0; l < 32; ++l) nv[l] = v[l] + v[l ^ o];
            memcpy(v, nv, sizeof v);
        }
        total = (w == 0) ? v[0] : total + v[0];
    }
    return total;
}

static float block_sum_sq(const float* x, int n) {
    float p[256];
    for (int t = 0; t < 256; ++t) {
        float a = 0.0f;
        for (int base = 4 * t; base < n; base += 1024)
            for (int e = 0; e < 4; ++e) {
                int i = base + e;
                if (i < n) a = fmaf(x[i], x[i], a);
            }
        p[t] = a;
    }
    return block_reduce_sum(p);
}

/* ------------------------------------------------------------ pack/unpack */
static inline int code_of_trit(int t) { return t > 0 ? 1 : (t < 0 ? 2 : 0); }
static inline int trit_of_code(int c) { return (c == 1) - (c == 2); }

void orc_pack_v11(const int8_t* trits, int K, int N, uint8_t* out) {
    memset(out, 0, (size_t)K * (size_t)(N / 4));
    for (int k = 0; k < K; ++k)
        for (int j = 0; j < N; ++j)
            out[(size_t)(j >> 2) * K + k] |=
                (uint8_t)(code_of_trit(trits[(size_t)k * N + j]) << (2 * (j & 3)));
}
void orc_pack_rowmajor(const int8_t* trits, int K, int N, uint8_t* out) {
    memset(out, 0, (size_t)K * (size_t)(N / 4));
    for (int k = 0; k < K; ++k)
        for (int j = 0; j < N; ++j)
            out[(size_t)k * (N / 4) + (j >> 2)] |=
                (uint8_t)(code_of_trit(trits[(size_t)k * N + j]) << (2 * (j & 3)));
}
void orc_unpack_v11(const uint8_t* in, int K, int N, int8_t* trits) {
    for (int k = 0; k < K; ++k)
        for (int j = 0; j < N; ++j)
            trits[(size_t)k * N + j] =
                (int8_t)trit_of_code((in[(size_t)(j >> 2) * K + k] >> (2 * (j & 3))) & 3);
}
void orc_unpack_rowmajor(const uint8_t* in, int K, int N, int8_t* trits) {
    for (int k = 0; k < K; ++k)
        for (int j = 0; j < N; ++j)
            trits[(size_t)k * N + j] =
                (int8_t)trit_of_code((in[(size_t)k * (N / 4) + (j >> 2)] >> (2 * (j & 3))) & 3);
}

/* ------------------------------------------------------------------ mm_row */
void orc_mm_row_acc(const int32_t* X, const int32_t* W, int K, int N, int64_t* acc) {
    for (int j = 0; j < N; ++j) acc[j] = 0;
    for (int k = 0; k < K; ++k) {
        int64_t xv = X[k];
        if (xv == 0) continue;                     /* zero-skip, forward.cpp:335 */
        const int32_t* w = W + (size_t)k * N;
        for (int j = 0; j < N; ++j) acc[j] += xv * (int64_t)w[j];
    }
}
void orc_mm_row(const int32_t* X, float x_scale, const int32_t* W, float w_scale,
                int K, int N, float* out) {
    int64_t* acc = (int64_t*)malloc(sizeof(int64_t) * (size_t)N);
    orc_mm_row_acc(X, W, K, N, acc);
    float s = x_scale * w_scale;                   /* forward.cpp:342 */
    for (int j = 0; j < N; ++j) out[j] = (float)acc[j] * s;
    free(acc);
}
uint64_t orc_tvmac(int K, int N) { return (uint64_t)((K + 26) / 27) * (uint64_t)N; }

/* ------------------------------------------------------- packed GEMV (GPU) */
void orc_gemv_packed_v11_acc(const int8_t* x, const uint8_t* Wcol, int K, int N, int32_t* acc) {
    for (int jb = 0; jb < N / 4; ++jb) {
        const uint8_t* w = Wcol + (size_t)jb * K;
        int32_t a0 = 0, a1 = 0, a2 = 0, a3 = 0;
        for (int k = 0; k < K; ++k) {
            int b = w[k], xv = x[k];
            a0 += xv * trit_of_code(b & 3);
            a1 += xv * trit_of_code((b >> 2) & 3);
            a2 += xv * trit_of_code((b >> 4) & 3);
            a3 += xv * trit_of_code((b >> 6) & 3);
        }
        acc[4 * jb] = a0; acc[4 * jb + 1] = a1; acc[4 * jb + 2] = a2; acc[4 * jb + 3] = a3;
    }
}
void orc_gemv_epilogue(const int32_t* acc, int N, float x_scale, float w_scale, float* out) {
    float s = x_scale * w_scale;                   /* forward_packed.cu:358 */
    for (int j = 0; j < N; ++j) out[j] = (float)acc[j] * s;
}
void orc_gemm_packed_v11(const int8_t* X, const float* x_scales, int M,
                         const uint8_t* Wcol, float w_scale, int K, int N,
                         int32_t* acc, float* out) {
    int32_t* tmp = (int32_t*)malloc(sizeof(int32_t) * (size_t)N);
    for (int m = 0; m < M; ++m) {
        int32_t* a = acc ? acc + (size_t)m * N : tmp;
        orc_gemv_packed_v11_acc(X + (size_t)m * K, Wcol, K, N, a);
        if (out) orc_gemv_epilogue(a, N, x_scales[m], w_scale, out + (size_t)m * N);
    }
    free(tmp);
}

/* -------------------------------------------------------------- quantisers */
float orc_quantize_trit(const float* x, int n, int n_trits, int32_t* payload) {
    int64_t mti = 1;
    for (int i = 0; i < n_trits; ++i) mti *= 3;
    mti = (mti - 1) / 2;
    float amax = 0.0f;
    for (int i = 0; i < n; ++i) { float a = fabsf(x[i]); if (a > amax) amax = a; }
    if (amax == 0.0f) { for (int i = 0; i < n; ++i) payload[i] = 0; return 0.0f; }
    float scale = amax / (float)mti;
    for (int i = 0; i < n; ++i) {
        int64_t r = (int64_t)lroundf(x[i] / scale);
        if (r > mti) r = mti;
        if (r < -mti) r = -mti;
        payload[i] = (int32_t)r;
    }
    return scale;
}

static void quant_from_amax(const float* v, int n, float amax_raw, int8_t* q, float* scale_out) {
    float amax = amax_raw + 1e-9f;
    float scale = 127.0f / amax;
    *scale_out = 1.0f / scale;
    for (int i = 0; i < n; ++i) {
        int qi = (int)rintf(v[i] * scale);
        if (qi > 127) qi = 127;
        if (qi < -128) qi = -128;
        q[i] = (int8_t)qi;
    }
}
static float absmax(const float* v, int n) {
    float a = 0.0f;
    for (int i = 0; i < n; ++i) { float t = fabsf(v[i]); if (t > a) a = t; }
    return a;
}
/* tools/llama_pyfwd.py:82-86 form, for the pyfwd-compatible mode only. */
static void quant_np(const float* v, int n, int8_t* q, float* scale_out) {
    double amax = (double)absmax(v, n);
    if (amax < 1e-9) amax = 1e-9;
    double scale = amax / 127.0;
    float s32 = (float)scale;
    for (int i = 0; i < n; ++i) {
        float r = rintf(v[i] / s32);
        if (r > 127.0f) r = 127.0f;
        if (r < -128.0f) r = -128.0f;
        q[i] = (int8_t)r;
    }
    *scale_out = (float)scale;
}

void orc_quant_int8(const float* x, int n, int8_t* q, float* scale_out) {
    quant_from_amax(x, n, absmax(x, n), q, scale_out);
}

static float rms_inv_of(const float* x, int n, float eps) {
    float ss = block_sum_sq(x, n);
    float mean = ss / (float)n;
    return 1.0f / sqrtf(mean + eps);
}

void orc_rmsnorm(const float* x, const float* gamma, int n, float eps, float* y) {
    float ri = rms_inv_of(x, n, eps);
    for (int i = 0; i < n; ++i) y[i] = (x[i] * ri) * gamma[i];
}

void orc_rmsnorm_quant(const float* x, const float* gamma, int n, float eps,
                       int8_t* q, float* scale_out, float* normed) {
    float* v = (float*)malloc(sizeof(float) * (size_t)n);
    orc_rmsnorm(x, gamma, n, eps, v);
    quant_from_amax(v, n, absmax(v, n), q, scale_out);
    if (normed) memcpy(normed, v, sizeof(float) * (size_t)n);
    free(v);
}

static inline float silu_mul(float g, float u) {
    float e = orc_expf(-g);
    float sg = g / (1.0f + e);
    return sg * u;
}
void orc_silu_mul_quant(const float* g, const float* u, int n, int8_t* q, float* scale_out) {
    float* v = (float*)malloc(sizeof(float) * (size_t)n);
    for (int i = 0; i < n; ++i) v[i] = silu_mul(g[i], u[i]);
    quant_from_amax(v, n, absmax(v, n), q, scale_out);
    free(v);
}
static inline float relu2_mul(float g, float u) {
    float r = g > 0.0f ? g * g : 0.0f;
    return r * u;
}
void orc_relu2_mul_rmsnorm_quant(const float* g, const float* u, const float* gamma, int n,
                                 float eps, int8_t* q, float* scale_out) {
    float* v = (float*)malloc(sizeof(float) * (size_t)n);
    for (int i = 0; i < n; ++i) v[i] = relu2_mul(g[i], u[i]);
    float ri = rms_inv_of(v, n, eps);
    for (int i = 0; i < n; ++i) v[i] = (v[i] * ri) * gamma[i];
    quant_from_amax(v, n, absmax(v, n), q, scale_out);
    free(v);
}

/* ------------------------------------------------------------------- rope */
void orc_rope_table(int n_pos, int head_dim, double theta, float* table) {
    int half = head_dim / 2;
    for (int p = 0; p < n_pos; ++p)
        for (int k = 0; k < half; ++k) {
            double freq = 1.0 / pow(theta, (2.0 * k) / (double)head_dim);
            double a = (double)p * freq;
            table[((size_t)p * half + k) * 2 + 0] = (float)cos(a);
            table[((size_t)p * half + k) * 2 + 1] = (float)sin(a);
        }
}
void orc_rope(float* v, int n_heads, int head_dim, const float* row, int neox) {
    int half = head_dim / 2;
    for (int h = 0; h < n_heads; ++h)
        for (int k = 0; k < half; ++k) {
            float c = row[2 * k], s = row[2 * k + 1];
            int i0 = neox ? h * head_dim + k : h * head_dim + 2 * k;
            int i1 = neox ? i0 + half : i0 + 1;
            float v0 = v[i0], v1 = v[i1];
            float a = v0 * c, b = v1 * s;
            float d = v0 * s, e = v1 * c;
            v[i0] = a - b;
            v[i1] = d + e;
        }
}

/* -------------------------------------------------------------- attention */
#define ORC_CHUNK 256
/* score of one (head, position): 8 lanes each take 8 consecutive dims out of
 * every 64, fused multiply-adds in ascending dim order, xor butterfly 4,2,1. */
static float score_dot(const float* q, const uint16_t* krow, int head_dim) {
    float lane[8], nl[8];
    for (int j = 0; j < 8; ++j) {
        float a = 0.0f;
        for (int d0 = 8 * j; d0 < head_dim; d0 += 64)
            for (int e = 0; e < 8; ++e)
                a = fmaf(q[d0 + e], orc_bf16_to_f32(krow[d0 + e]), a);
        lane[j] = a;
    }
    for (int o = 4; o > 0; o >>= 1) {
        for (int j = 0; j < 8; ++j) nl[j] = lane[j] + lane[j ^ o];
        memcpy(lane, nl, sizeof lane);
    }
    return lane[0];
}

void orc_attention(const float* q, const uint16_t* kc, const uint16_t* vc,
                   int n_heads, int n_kv, int head_dim, int smax, int seq_len, float* out) {
    float inv_sqrt = 1.0f / sqrtf((float)head_dim);
    float* O = (float*)malloc(sizeof(float) * (size_t)head_dim);
    float* oc = (float*)malloc(sizeof(float) * (size_t)head_dim);
    int n_chunks = (seq_len + ORC_CHUNK - 1) / ORC_CHUNK;
    for (int h = 0; h < n_heads; ++h) {
        int kvh = (int)((long)h * n_kv / n_heads);      /* forward_packed.cu:124 */
        const uint16_t* K = kc + (size_t)kvh * smax * head_dim;
        const uint16_t* V = vc + (size_t)kvh * smax * head_dim;
        const float* qh = q + (size_t)h * head_dim;
        float M = 0.0f, L = 0.0f;
        for (int c = 0; c < n_chunks; ++c) {
            int s0 = c * ORC_CHUNK;
            int cnt = seq_len - s0 < ORC_CHUNK ? seq_len - s0 : ORC_CHUNK;
            float sc[ORC_CHUNK], p[ORC_CHUNK];
            float mc = -INFINITY;
            for (int t = 0; t < cnt; ++t) {
                sc[t] = score_dot(qh, K + (size_t)(s0 + t) * head_dim, head_dim) * inv_sqrt;
                if (sc[t] > mc) mc = sc[t];
            }
            for (int t = 0; t < ORC_CHUNK; ++t) p[t] = t < cnt ? orc_expf(sc[t] - mc) : 0.0f;
            float lc = block_reduce_sum(p);
            for (int d = 0; d < head_dim; ++d) {
                float a = 0.0f;
                for (int t = 0; t < cnt; ++t)
                    a = fmaf(p[t], orc_bf16_to_f32(V[(size_t)(s0 + t) * head_dim + d]), a);
                oc[d] = a;
            }
            if (c == 0) {
                M = mc; L = lc;
                memcpy(O, oc, sizeof(float) * (size_t)head_dim);
            } else {
                float Mn = M > mc ? M : mc;
                float a = orc_expf(M - Mn), b = orc_expf(mc - Mn);
                L = fmaf(lc, b, L * a);
                for (int d = 0; d < head_dim; ++d) O[d] = fmaf(oc[d], b, O[d] * a);
                M = Mn;
            }
        }
        for (int d = 0; d < head_dim; ++d) out[(size_t)h * head_dim + d] = O[d] / L;
    }
    free(O); free(oc);
}

void orc_attention_twopass(const float* q, const uint16_t* kc, const uint16_t* vc,
                           int n_heads, int n_kv, int head_dim, int smax, int seq_len, float* out) {
    double* sc = (double*)malloc(sizeof(double) * (size_t)seq_len);
    double inv_sqrt = 1.0 / sqrt((double)head_dim);
    for (int h = 0; h < n_heads; ++h) {
        int kvh = (int)((long)h * n_kv / n_heads);
        const uint16_t* K = kc + (size_t)kvh * smax * head_dim;
        const uint16_t* V = vc + (size_t)kvh * smax * head_dim;
        double mx = -INFINITY;
        for (int s = 0; s < seq_len; ++s) {
            double d = 0.0;
            for (int i = 0; i < head_dim; ++i)
                d += (double)q[(size_t)h * head_dim + i] *
                     (double)orc_bf16_to_f32(K[(size_t)s * head_dim + i]);
            sc[s] = d * inv_sqrt;
            if (sc[s] > mx) mx = sc[s];
        }
        double sum = 0.0;
        for (int s = 0; s < seq_len; ++s) { sc[s] = exp(sc[s] - mx); sum += sc[s]; }
        for (int i = 0; i < head_dim; ++i) {
            double a = 0.0;
            for (int s = 0; s < seq_len; ++s)
                a += sc[s] * (double)orc_bf16_to_f32(V[(size_t)s * head_dim + i]);
            out[(size_t)h * head_dim + i] = (float)(a / sum);
        }
    }
    free(sc);
}

/* ------------------------------------------------------- lm_head / argmax */
static float lm_row_dot(const uint16_t* row, const float* x, int H) {
    float lane[32], nl[32];
    for (int l = 0; l < 32; ++l) {
        float a = 0.0f;
        for (int base = 8 * l; base < H; base += 256)
            for (int e = 0; e < 8; ++e)
                if (base + e < H) a = fmaf(orc_bf16_to_f32(row[base + e]), x[base + e], a);
        lane[l] = a;
    }
    for (int o = 16; o > 0; o >>= 1) {
        for (int l = 0; l < 32; ++l) nl[l] = lane[l] + lane[l ^ o];
        memcpy(lane, nl, sizeof lane);
    }
    return lane[0];
}
void orc_lm_head_bf16(const uint16_t* embd, const float* x, int V, int H, float* logits) {
    for (int v = 0; v < V; ++v) logits[v] = lm_row_dot(embd + (size_t)v * H, x, H);
}
int orc_argmax(const float* v, int n) {
    int bi = 0; float best = v[0];
    for (int i = 1; i < n; ++i) if (v[i] > best) { best = v[i]; bi = i; }
    return bi;
}

/* ------------------------------------------------------------------ model */
typedef struct { int8_t* t; /* [N][K] trits */ float scale; int K, N; } orc_mat_t;
struct orc_model {
    orc_cfg_t c;
    int n_threads;
    uint16_t* embd;
    float* out_norm;
    orc_mat_t* mats;      /* [L][ORC_NMAT] */
    float** vecs;         /* [L][ORC_NVEC] */
    orc_mat_t lm_head;
    float* rope;          /* [Smax][Hd/2][2] */
};
struct orc_state {
    const orc_model_t* m;
    int batch;
    void* kc; void* vc;   /* [batch][L][Nkv][Smax][Hd] bf16 or f32 */
    float* layer_hidden;  /* [L][H] of the latest call */
};

static void mat_dims(const orc_cfg_t* c, int which, int* K, int* N) {
    int Hkv = c->Nkv * c->Hd, Hq = c->Nh * c->Hd;
    switch (which) {
        case ORC_WQ: *K = c->H; *N = Hq; break;
        case ORC_WK: case ORC_WV: *K = c->H; *N = Hkv; break;
        case ORC_WO: *K = Hq; *N = c->H; break;
        case ORC_WGATE: case ORC_WUP: *K = c->H; *N = c->F; break;
        default: *K = c->F; *N = c->H; break;
    }
}
static int vec_len(const orc_cfg_t* c, int which) {
    return which == ORC_FFN_SUB_NORM ? c->F : (which == ORC_ATTN_SUB_NORM ? c->Nh * c->Hd : c->H);
}

orc_model_t* orc_model_create(const orc_cfg_t* cfg) {
    orc_model_t* m = (orc_model_t*)calloc(1, sizeof *m);
    if (!m) return NULL;
    m->c = *cfg;
    m->n_threads = 1;
    m->mats = (orc_mat_t*)calloc((size_t)cfg->L * ORC_NMAT, sizeof(orc_mat_t));
    m->vecs = (float**)calloc((size_t)cfg->L * ORC_NVEC, sizeof(float*));
    m->rope = (float*)malloc(sizeof(float) * (size_t)cfg->Smax * (size_t)cfg->Hd);
    orc_rope_table(cfg->Smax, cfg->Hd, cfg->rope_theta, m->rope);
    return m;
}
void orc_model_destroy(orc_model_t* m) {
    if (!m) return;
    for (int i = 0; i < m->c.L * ORC_NMAT; ++i) free(m->mats[i].t);
    for (int i = 0; i < m->c.L * ORC_NVEC; ++i) free(m->vecs[i]);
    free(m->mats); free(m->vecs); free(m->lm_head.t); free(m->embd); free(m->out_norm); free(m->rope);
    free(m);
}
void orc_model_set_threads(orc_model_t* m, int n) { m->n_threads = n < 1 ? 1 : (n > 64 ? 64 : n); }

static int set_mat(orc_mat_t* dst, const uint8_t* packed, float scale, int K, int N) {
    free(dst->t);
    dst->t = (int8_t*)malloc((size_t)K * (size_t)N);
    if (!dst->t) return -3;
    dst->K = K; dst->N = N; dst->scale = scale;
    for (int j = 0; j < N; ++j) {                  /* transpose-unpack to [N][K] */
        const uint8_t* w = packed + (size_t)(j >> 2) * K;
        int sh = 2 * (j & 3);
        int8_t* o = dst->t + (size_t)j * K;
        for (int k = 0; k < K; ++k) o[k] = (int8_t)trit_of_code((w[k] >> sh) & 3);
    }
    return 0;
}
int orc_model_set_matrix(orc_model_t* m, int layer, int which, const uint8_t* packed, float scale) {
    if (!m || !packed) return -1;
    if (layer < 0) return set_mat(&m->lm_head, packed, scale, m->c.H, m->c.V);
    if (layer >= m->c.L || which < 0 || which >= ORC_NMAT) return -2;
    int K, N; mat_dims(&m->c, which, &K, &N);
    return set_mat(&m->mats[layer * ORC_NMAT + which], packed, scale, K, N);
}
int orc_model_set_vector(orc_model_t* m, int layer, int which, const float* v) {
    if (!m || !v) return -1;
    if (layer < 0) {
        free(m->out_norm);
        m->out_norm = (float*)malloc(sizeof(float) * (size_t)m->c.H);
        memcpy(m->out_norm, v, sizeof(float) * (size_t)m->c.H);
        return 0;
    }
    if (layer >= m->c.L || which < 0 || which >= ORC_NVEC) return -2;
    int n = vec_len(&m->c, which);
    float** slot = &m->vecs[layer * ORC_NVEC + which];
    free(*slot);
    *slot = (float*)malloc(sizeof(float) * (size_t)n);
    memcpy(*slot, v, sizeof(float) * (size_t)n);
    return 0;
}
int orc_model_set_embd(orc_model_t* m, const uint16_t* t) {
    if (!m || !t) return -1;
    size_t n = (size_t)m->c.V * (size_t)m->c.H;
    free(m->embd);
    m->embd = (uint16_t*)malloc(n * 2);
    if (!m->embd) return -3;
    memcpy(m->embd, t, n * 2);
    return 0;
}

orc_state_t* orc_state_create(const orc_model_t* m, int batch) {
    orc_state_t* s = (orc_state_t*)calloc(1, sizeof *s);
    if (!s) return NULL;
    s->m = m; s->batch = batch;
    size_t n = (size_t)batch * m->c.L * m->c.Nkv * m->c.Smax * m->c.Hd;
    size_t es = m->c.kv_f32 ? 4 : 2;
    s->kc = calloc(n, es); s->vc = calloc(n, es);
    s->layer_hidden = (float*)calloc((size_t)m->c.L * m->c.H, sizeof(float));
    return s;
}
void orc_state_destroy(orc_state_t* s) {
    if (!s) return;
    free(s->kc); free(s->vc); free(s->layer_hidden); free(s);
}
int orc_state_layer_hidden(const orc_state_t* s, int layer, float* out) {
    if (!s || layer < 0 || layer >= s->m->c.L) return -1;
    memcpy(out, s->layer_hidden + (size_t)layer * s->m->c.H, sizeof(float) * (size_t)s->m->c.H);
    return 0;
}

/* ---- threaded int8 x trit GEMV over the unpacked [N][K] form ---- */
typedef struct { const orc_mat_t* w; const int8_t* x; float s; float* out; int j0, j1; } gemv_job_t;
static void* gemv_worker(void* arg) {
    gemv_job_t* jb = (gemv_job_t*)arg;
    int K = jb->w->K;
    for (int j = jb->j0; j < jb->j1; ++j) {
        const int8_t* w = jb->w->t + (size_t)j * K;
        int32_t acc = 0;
        for (int k = 0; k < K; ++k) acc += (int32_t)jb->x[k] * (int32_t)w[k];
        jb->out[j] = (float)acc * jb->s;
    }
    return NULL;
}
static void gemv(const orc_model_t* m, const orc_mat_t* w, const int8_t* x, float xs, float* out) {
    float s = xs * w->scale;
    int nt = m->n_threads;
    if (nt <= 1 || w->N < 4 * nt) {
        gemv_job_t jb = { w, x, s, out, 0, w->N };
        gemv_worker(&jb);
        return;
    }
    pthread_t th[64]; gemv_job_t jobs[64];
    for (int t = 0; t < nt; ++t) {
        jobs[t] = (gemv_job_t){ w, x, s, out, (int)((long)w->N * t / nt), (int)((long)w->N * (t + 1) / nt) };
        pthread_create(&th[t], NULL, gemv_worker, &jobs[t]);
    }
    for (int t = 0; t < nt; ++t) pthread_join(th[t], NULL);
}
typedef struct { const uint16_t* e; const float* x; float* out; int H, v0, v1; } lm_job_t;
static void* lm_worker(void* arg) {
    lm_job_t* j = (lm_job_t*)arg;
    for (int v = j->v0; v < j->v1; ++v) j->out[v] = lm_row_dot(j->e + (size_t)v * j->H, j->x, j->H);
    return NULL;
}
static void lm_head_mt(const orc_model_t* m, const float* x, float* logits) {
    int nt = m->n_threads, V = m->c.V;
    if (nt <= 1) { orc_lm_head_bf16(m->embd, x, V, m->c.H, logits); return; }
    pthread_t th[64]; lm_job_t jobs[64];
    for (int t = 0; t < nt; ++t) {
        jobs[t] = (lm_job_t){ m->embd, x, logits, m->c.H, (int)((long)V * t / nt), (int)((long)V * (t + 1) / nt) };
        pthread_create(&th[t], NULL, lm_worker, &jobs[t]);
    }
    for (int t = 0; t < nt; ++t) pthread_join(th[t], NULL);
}

static void attention_f32(const float* q, const float* kc, const float* vc, int n_heads, int n_kv,
                          int head_dim, int smax, int seq_len, float* out) {
    /* tools/llama_pyfwd.py:116-123 with an fp32 cache (pyfwd-compatible mode). */
    double* sc = (double*)malloc(sizeof(double) * (size_t)seq_len);
    for (int h = 0; h < n_heads; ++h) {
        int kvh = (int)((long)h * n_kv / n_heads);
        const float* K = kc + (size_t)kvh * smax * head_dim;
        const float* V = vc + (size_t)kvh * smax * head_dim;
        double mx = -INFINITY, inv = 1.0 / sqrt((double)head_dim);
        for (int s = 0; s < seq_len; ++s) {
            double d = 0.0;
            for (int i = 0; i < head_dim; ++i) d += (double)q[(size_t)h * head_dim + i] * (double)K[(size_t)s * head_dim + i];
            sc[s] = d * inv; if (sc[s] > mx) mx = sc[s];
        }
        double sum = 0.0;
        for (int s = 0; s < seq_len; ++s) { sc[s] = exp(sc[s] - mx); sum += sc[s]; }
        for (int i = 0; i < head_dim; ++i) {
            double a = 0.0;
            for (int s = 0; s < seq_len; ++s) a += sc[s] * (double)V[(size_t)s * head_dim + i];
            out[(size_t)h * head_dim + i] = (float)(a / sum);
        }
    }
    free(sc);
}

int orc_forward_token(const orc_model_t* m, orc_state_t* st, int seq, int token, int pos,
                      float* logits, float* hidden_out) {
    const orc_cfg_t* c = &m->c;
    int H = c->H, F = c->F, Hd = c->Hd, Hq = c->Nh * Hd, Hkv = c->Nkv * Hd;
    int neox = c->arch == ORC_ARCH_BITNET;
    float* hidden = (float*)malloc(sizeof(float) * (size_t)H);
    float* q = (float*)malloc(sizeof(float) * (size_t)Hq);
    float* k = (float*)malloc(sizeof(float) * (size_t)Hkv);
    float* v = (float*)malloc(sizeof(float) * (size_t)Hkv);
    float* att = (float*)malloc(sizeof(float) * (size_t)Hq);
    float* proj = (float*)malloc(sizeof(float) * (size_t)H);
    float* gate = (float*)malloc(sizeof(float) * (size_t)F);
    float* up = (float*)malloc(sizeof(float) * (size_t)F);
    float* tmpf = (float*)malloc(sizeof(float) * (size_t)(F > Hq ? (F > H ? F : H) : (Hq > H ? Hq : H)));
    int8_t* xq = (int8_t*)malloc((size_t)(F > Hq ? (F > H ? F : H) : (Hq > H ? Hq : H)));
    float xs;
    const float* rope_row = m->rope + (size_t)pos * Hd;

    for (int i = 0; i < H; ++i) hidden[i] = orc_bf16_to_f32(m->embd[(size_t)token * H + i]);

    for (int L = 0; L < c->L; ++L) {
        const orc_mat_t* W = m->mats + (size_t)L * ORC_NMAT;
        float** vec = m->vecs + (size_t)L * ORC_NVEC;
        size_t coff = ((size_t)seq * c->L + L) * (size_t)c->Nkv * c->Smax * Hd;

        /* attention block */
        if (c->np_quant) { orc_rmsnorm(hidden, vec[ORC_ATTN_NORM], H, c->eps, tmpf); quant_np(tmpf, H, xq, &xs); }
        else orc_rmsnorm_quant(hidden, vec[ORC_ATTN_NORM], H, c->eps, xq, &xs, NULL);
        gemv(m, &W[ORC_WQ], xq, xs, q);
        gemv(m, &W[ORC_WK], xq, xs, k);
        gemv(m, &W[ORC_WV], xq, xs, v);
        orc_rope(q, c->Nh, Hd, rope_row, neox);
        orc_rope(k, c->Nkv, Hd, rope_row, neox);
        if (c->kv_f32) {
            float* kc = (float*)st->kc + coff; float* vc = (float*)st->vc + coff;
            for (int g = 0; g < c->Nkv; ++g)
                for (int d = 0; d < Hd; ++d) {
                    kc[((size_t)g * c->Smax + pos) * Hd + d] = k[g * Hd + d];
                    vc[((size_t)g * c->Smax + pos) * Hd + d] = v[g * Hd + d];
                }
            attention_f32(q, kc, vc, c->Nh, c->Nkv, Hd, c->Smax, pos + 1, att);
        } else {
            uint16_t* kc = (uint16_t*)st->kc + coff; uint16_t* vc = (uint16_t*)st->vc + coff;
            for (int g = 0; g < c->Nkv; ++g)
                for (int d = 0; d < Hd; ++d) {
                    kc[((size_t)g * c->Smax + pos) * Hd + d] = orc_f32_to_bf16(k[g * Hd + d]);
                    vc[((size_t)g * c->Smax + pos) * Hd + d] = orc_f32_to_bf16(v[g * Hd + d]);
                }
            orc_attention(q, kc, vc, c->Nh, c->Nkv, Hd, c->Smax, pos + 1, att);
        }
        if (c->arch == ORC_ARCH_BITNET) {
            if (c->np_quant) { orc_rmsnorm(att, vec[ORC_ATTN_SUB_NORM], Hq, c->eps, tmpf); quant_np(tmpf, Hq, xq, &xs); }
            else orc_rmsnorm_quant(att, vec[ORC_ATTN_SUB_NORM], Hq, c->eps, xq, &xs, NULL);
        } else {
            if (c->np_quant) quant_np(att, Hq, xq, &xs); else orc_quant_int8(att, Hq, xq, &xs);
        }
        gemv(m, &W[ORC_WO], xq, xs, proj);
        for (int i = 0; i < H; ++i) hidden[i] = hidden[i] + proj[i];

        /* FFN block */
        if (c->np_quant) { orc_rmsnorm(hidden, vec[ORC_FFN_NORM], H, c->eps, tmpf); quant_np(tmpf, H, xq, &xs); }
        else orc_rmsnorm_quant(hidden, vec[ORC_FFN_NORM], H, c->eps, xq, &xs, NULL);
        gemv(m, &W[ORC_WGATE], xq, xs, gate);
        gemv(m, &W[ORC_WUP], xq, xs, up);
        if (c->arch == ORC_ARCH_BITNET) {
            if (c->np_quant) {
                for (int i = 0; i < F; ++i) tmpf[i] = relu2_mul(gate[i], up[i]);
                orc_rmsnorm(tmpf, vec[ORC_FFN_SUB_NORM], F, c->eps, gate);
                quant_np(gate, F, xq, &xs);
            } else orc_relu2_mul_rmsnorm_quant(gate, up, vec[ORC_FFN_SUB_NORM], F, c->eps, xq, &xs);
        } else {
            if (c->np_quant) {
                for (int i = 0; i < F; ++i) tmpf[i] = (float)((double)gate[i] / (1.0 + exp(-(double)gate[i]))) * up[i];
                quant_np(tmpf, F, xq, &xs);
            } else orc_silu_mul_quant(gate, up, F, xq, &xs);
        }
        gemv(m, &W[ORC_WDOWN], xq, xs, proj);
        for (int i = 0; i < H; ++i) hidden[i] = hidden[i] + proj[i];
        memcpy(st->layer_hidden + (size_t)L * H, hidden, sizeof(float) * (size_t)H);
    }
    if (hidden_out) memcpy(hidden_out, hidden, sizeof(float) * (size_t)H);

    float* lg = logits ? logits : (float*)malloc(sizeof(float) * (size_t)c->V);
    if (c->lm_head_packed) {
        /* bench-mode packed lm_head: forward_packed.cu:541-545 */
        orc_rmsnorm_quant(hidden, m->out_norm, H, c->eps, xq, &xs, NULL);
        gemv(m, &m->lm_head, xq, xs, lg);
    } else {
        orc_rmsnorm(hidden, m->out_norm, H, c->eps, tmpf);
        lm_head_mt(m, tmpf, lg);
    }
    int tok = orc_argmax(lg, c->V);
    if (!logits) free(lg);
    free(hidden); free(q); free(k); free(v); free(att); free(proj); free(gate); free(up); free(tmpf); free(xq);
    return tok;
}
