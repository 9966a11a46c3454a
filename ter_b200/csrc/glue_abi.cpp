// extern "C" entry points of the decode glue operators (include/ter_b200.h).
#include <math.h>
#include <new>

#include "glue.h"
#include "handle.h"

using namespace terb;

namespace terb {

// cos/sin table [n_pos][head_dim/2][2], freq = theta^(-2k/head_dim), evaluated in double on
// the host as the reference's CPU rotary does (src/tx/forward.cpp:78-88), rounded to fp32.
int get_rope_table(ter_b200_handle_t* h, int n_pos, int head_dim, double theta, const float** out) {
    for (int i = 0; i < 4; ++i) {
        RopeTable& t = h->rope[i];
        if (t.data && t.n_pos == n_pos && t.head_dim == head_dim && t.theta == theta) {
            *out = t.data;
            return TER_B200_OK;
        }
    }
    int slot = -1;
    for (int i = 0; i < 4; ++i)
        if (!h->rope[i].data) { slot = i; break; }
    if (slot < 0) {
        slot = 0;
        cudaStreamSynchronize(h->stream);
        cudaFree(h->rope[0].data);
        h->rope[0] = RopeTable();
    }
    const int half = head_dim / 2;
    const size_t n = (size_t)n_pos * half * 2;
    float* host = new (std::nothrow) float[n];
    if (!host) return TER_B200_E_ALLOC;
    for (int p = 0; p < n_pos; ++p)
        for (int k = 0; k < half; ++k) {
            const double freq = 1.0 / pow(theta, (2.0 * k) / (double)head_dim);
            const double a = (double)p * freq;
            host[((size_t)p * half + k) * 2 + 0] = (float)cos(a);
            host[((size_t)p * half + k) * 2 + 1] = (float)sin(a);
        }
    float* dev = nullptr;
    cudaError_t e = cudaMalloc((void**)&dev, n * sizeof(float));
    if (e == cudaSuccess) e = cudaMemcpy(dev, host, n * sizeof(float), cudaMemcpyHostToDevice);
    delete[] host;
    if (e != cudaSuccess) {
        if (dev) cudaFree(dev);
        return cuda_fail(h, e);
    }
    h->rope[slot].data = dev;
    h->rope[slot].n_pos = n_pos;
    h->rope[slot].head_dim = head_dim;
    h->rope[slot].theta = theta;
    *out = dev;
    return TER_B200_OK;
}

}  // namespace terb

extern "C" {

int ter_b200_rmsnorm_quant(ter_b200_handle_t* h, const float* x_dev, const float* gamma_dev, int n, int rows,
                           float eps, int8_t* q_dev, float* scale_dev, float* normed_dev, void* stream) {
    if (!h || !x_dev) return TER_B200_E_NULL;
    if ((q_dev && !scale_dev) || (!q_dev && !normed_dev)) return TER_B200_E_NULL;
    if (n < 1 || rows < 1) return TER_B200_E_SHAPE;
    TERB_CUDA(h, cudaSetDevice(h->device));
    NormQuantParams p{x_dev, nullptr, gamma_dev, q_dev, scale_dev, normed_dev, n, rows, PRE_NONE, eps};
    TERB_CUDA(h, launch_norm_quant(p, h->gemv_cfg.pdl != 0, pick_stream(h, stream)));
    h->launches += 1;
    return TER_B200_OK;
}

int ter_b200_act_quant(ter_b200_handle_t* h, int act, const float* gate_dev, const float* up_dev,
                       const float* gamma_dev, int n, int rows, float eps, int8_t* q_dev, float* scale_dev,
                       void* stream) {
    if (!h || !gate_dev || !up_dev || !q_dev || !scale_dev) return TER_B200_E_NULL;
    if (n < 1 || rows < 1 || (act != TER_B200_ACT_SILU && act != TER_B200_ACT_RELU2)) return TER_B200_E_SHAPE;
    TERB_CUDA(h, cudaSetDevice(h->device));
    NormQuantParams p{gate_dev, up_dev, gamma_dev, q_dev, scale_dev, nullptr, n, rows,
                      act == TER_B200_ACT_SILU ? PRE_SILU_MUL : PRE_RELU2_MUL, eps};
    TERB_CUDA(h, launch_norm_quant(p, h->gemv_cfg.pdl != 0, pick_stream(h, stream)));
    h->launches += 1;
    return TER_B200_OK;
}

int ter_b200_rope_kv(ter_b200_handle_t* h, float* q_dev, float* k_dev, const float* v_dev, const int* pos_dev,
                     int B, int Nh, int Nkv, int Hd, int Smax, double theta, int neox, uint16_t* kcache_dev,
                     uint16_t* vcache_dev, void* stream) {
    if (!h || !q_dev || !k_dev || !pos_dev) return TER_B200_E_NULL;
    // all three of v / kcache / vcache, or none of them (rotation only, nothing appended)
    if ((v_dev || kcache_dev || vcache_dev) && !(v_dev && kcache_dev && vcache_dev)) return TER_B200_E_NULL;
    if (B < 1 || Nh < 1 || Nkv < 1 || Hd < 2 || (Hd & 1) || Smax < 1) return TER_B200_E_SHAPE;
    TERB_CUDA(h, cudaSetDevice(h->device));
    const float* table = nullptr;
    int rc = get_rope_table(h, Smax, Hd, theta, &table);
    if (rc) return rc;
    RopeKvParams p{q_dev, k_dev, v_dev, table, pos_dev, kcache_dev, vcache_dev, B, Nh, Nkv, Hd, Smax, neox};
    TERB_CUDA(h, launch_rope_kv(p, h->gemv_cfg.pdl != 0, pick_stream(h, stream)));
    h->launches += 1;
    return TER_B200_OK;
}

size_t ter_b200_attention_scratch_floats(int B, int Nh, int Hd, int Smax) {
    if (B < 1 || Nh < 1 || Hd < 1 || Smax < 1) return 0;
    return attention_scratch_floats(B, Nh, Hd, Smax);
}

int ter_b200_attention(ter_b200_handle_t* h, const float* q_dev, const uint16_t* kcache_dev,
                       const uint16_t* vcache_dev, const int* pos_dev, int B, int Nh, int Nkv, int Hd, int Smax,
                       float* scratch_dev, size_t scratch_floats, float* out_dev, void* stream) {
    if (!h || !q_dev || !kcache_dev || !vcache_dev || !pos_dev || !scratch_dev || !out_dev) return TER_B200_E_NULL;
    if (B < 1 || Nkv < 1 || Nh % Nkv != 0 || (Nh / Nkv != 1 && Nh / Nkv != 2 && Nh / Nkv != 4 && Nh / Nkv != 8) || (Hd != 64 && Hd != 128) || Smax < 1)
        return TER_B200_E_SHAPE;
    if (scratch_floats < attention_scratch_floats(B, Nh, Hd, Smax)) return TER_B200_E_SHAPE;
    TERB_CUDA(h, cudaSetDevice(h->device));
    AttnParams p{q_dev, kcache_dev, vcache_dev, pos_dev, scratch_dev, out_dev, B, Nh, Nkv, Hd, Smax,
                 (Smax + kAttnChunk - 1) / kAttnChunk, nullptr, nullptr, nullptr, nullptr, nullptr, 0,
                 h->status_dev};
    p.mma = B >= h->attn_mma_min;
    TERB_CUDA(h, launch_attention(p, h->gemv_cfg.pdl != 0, pick_stream(h, stream)));
    h->launches += 2;
    return TER_B200_OK;
}

int ter_b200_lm_head_bf16(ter_b200_handle_t* h, const uint16_t* table_dev, const float* x_dev, float* logits_dev,
                          int V, int H, int B, void* stream) {
    if (!h || !table_dev || !x_dev || !logits_dev) return TER_B200_E_NULL;
    if (V < 1 || B < 1 || H < 8 || H % 8 != 0) return TER_B200_E_SHAPE;
    TERB_CUDA(h, cudaSetDevice(h->device));
    TERB_CUDA(h, launch_lm_head_bf16(table_dev, x_dev, logits_dev, V, H, B, h->sm_count, h->gemv_cfg.pdl != 0,
                                     pick_stream(h, stream)));
    h->launches += 1;
    const uint64_t n = (uint64_t)((H + 26) / 27) * (uint64_t)V * (uint64_t)B;   // src/tx/transformer.cpp:208-211
    h->counts.tvmac += n;
    h->counts.total_ops += n;
    return TER_B200_OK;
}

int ter_b200_argmax(ter_b200_handle_t* h, const float* logits_dev, int V, int B, float* scratch_dev, int* out_dev,
                    void* stream) {
    if (!h || !logits_dev || !scratch_dev || !out_dev) return TER_B200_E_NULL;
    if (V < 1 || B < 1) return TER_B200_E_SHAPE;
    TERB_CUDA(h, cudaSetDevice(h->device));
    TERB_CUDA(h, launch_argmax(logits_dev, V, B, scratch_dev, out_dev, h->gemv_cfg.pdl != 0, pick_stream(h, stream)));
    h->launches += 2;
    return TER_B200_OK;
}


int ter_b200_lm_head_bf16_tc(ter_b200_handle_t* h, const uint16_t* table_dev, const float* x_dev, float* logits_dev,
                             int V, int H, int B, void* scratch_dev, size_t scratch_bytes, void* stream) {
    if (!h || !table_dev || !x_dev || !logits_dev || !scratch_dev) return TER_B200_E_NULL;
    if (V < 1 || B < 1 || H < 64 || H % 64 != 0 || scratch_bytes < lm_head_tc_scratch_bytes(B, H)) return TER_B200_E_SHAPE;
    TERB_CUDA(h, cudaSetDevice(h->device));
    TERB_CUDA(h, launch_lm_head_tc(table_dev, x_dev, logits_dev, V, H, B, scratch_dev, h->status_dev,
                                   h->gemv_cfg.pdl != 0, pick_stream(h, stream)));
    h->launches += 2;
    return TER_B200_OK;
}
size_t ter_b200_lm_head_tc_scratch_bytes(int B, int H) { return lm_head_tc_scratch_bytes(B, H); }

// Self-test of the bounded wait of the tensor-parallel exchange on ONE GPU: the exchange kernel runs as
// rank 0 of 2 against a second local buffer that stands for a peer which never sends.  Its wait runs out
// after "wait_ms", the kernel returns by itself and the status word reads as TER_B200_E_TIMEOUT through
// ter_b200_device_status.  Nothing faults and nothing hangs; the handle stays usable.
int ter_b200_selftest_exchange_timeout(ter_b200_handle_t* h) {
    if (!h) return TER_B200_E_NULL;
    TERB_CUDA(h, cudaSetDevice(h->device));
    const int n_floats = 256;                       // per-rank slice
    const size_t buf_bytes = 2 * n_floats * sizeof(float);
    const size_t recv_bytes = 2u * (n_floats / 2) * 16u * 2u;
    const size_t total = buf_bytes + recv_bytes + kMaxExchangeCtas * sizeof(int);
    uint8_t* arena[2] = {nullptr, nullptr};
    for (int i = 0; i < 2; ++i) {
        cudaError_t e = cudaMalloc((void**)&arena[i], total);
        if (e == cudaSuccess) e = cudaMemset(arena[i], 0, total);
        if (e != cudaSuccess) {
            for (int k = 0; k < 2; ++k) if (arena[k]) cudaFree(arena[k]);
            return cuda_fail(h, e);
        }
    }
    ExchangeParams xp;
    memset(&xp, 0, sizeof xp);
    xp.base[0] = arena[0];
    xp.base[1] = arena[1];                          // the "peer": receives this rank's words, sends nothing
    xp.seg_buf_off[0] = 0;
    xp.seg_floats[0] = n_floats;
    xp.n_seg = 1;
    xp.words_total = n_floats / 2;
    xp.rank = 0;
    xp.size = 2;
    xp.recv_off = buf_bytes;
    xp.seq = reinterpret_cast<int*>(arena[0] + buf_bytes + recv_bytes);
    xp.status = h->status_dev;
    xp.point = 0;
    xp.wait_ns = (unsigned long long)h->wait_ms * 1000000ull;
    cudaError_t e = launch_peer_exchange(xp, false, h->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(h->stream);
    h->launches += 1;
    cudaFree(arena[0]);
    cudaFree(arena[1]);
    if (e != cudaSuccess) return cuda_fail(h, e);
    return TER_B200_OK;
}

}  // extern "C"
