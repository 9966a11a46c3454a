// ter_b200_call: the named-operator entry point (ter_k4_call, src/k4/ter_k4.cpp:47-59),
// plus the batched GEMM entry points.
#include <stdio.h>

#include "handle.h"

using namespace terb;

namespace terb {

// Grows the handle's GEMM scratch (row sums + split-K partials) for M tokens x N columns.  Not for use
// while a stream is capturing.
// Row-sum scratch for M tokens and, when split-K may be used (M <= 256), a zeroed partial buffer of M*N ints.
int ensure_gemm_scratch(ter_b200_handle_t* h, int M, int N) {
    const size_t need_part = (h->gemm_split_k && M <= 256) ? (size_t)M * (size_t)N : 0;
    if (h->gemm_scratch_cap >= (size_t)M && h->gemm_part_cap >= need_part) return TER_B200_OK;
    TERB_CUDA(h, cudaDeviceSynchronize());
    // An outgrown buffer is parked, not freed: a captured graph may still launch kernels on it.
    auto retire = [&](void* p) -> bool {
        if (!p) return true;
        if (h->n_retired >= (int)(sizeof h->retired / sizeof h->retired[0])) return false;
        h->retired[h->n_retired++] = p;
        return true;
    };
    if (h->gemm_scratch_cap < (size_t)M) {
        if (!retire(h->gemm_scratch)) return TER_B200_E_ALLOC;
        h->gemm_scratch = nullptr;
        h->gemm_scratch_cap = 0;
        // grow at least geometrically, so the parked list stays short
        const size_t cap = (size_t)M > 2 * h->gemm_scratch_cap_prev ? (size_t)M : 2 * h->gemm_scratch_cap_prev;
        TERB_CUDA(h, cudaMalloc((void**)&h->gemm_scratch, cap * sizeof(int)));
        h->gemm_scratch_cap = h->gemm_scratch_cap_prev = cap;
    }
    if (h->gemm_part_cap < need_part) {
        if (!retire(h->gemm_part)) return TER_B200_E_ALLOC;
        h->gemm_part = nullptr;
        h->gemm_part_cap = 0;
        const size_t cap = need_part > 2 * h->gemm_part_cap_prev ? need_part : 2 * h->gemm_part_cap_prev;
        // the partials stay zero between calls (whoever reads them clears them)
        TERB_CUDA(h, cudaMalloc((void**)&h->gemm_part, cap * sizeof(int)));
        TERB_CUDA(h, cudaMemset(h->gemm_part, 0, cap * sizeof(int)));
        h->gemm_part_cap = h->gemm_part_cap_prev = cap;
    }
    return TER_B200_OK;
}

// Up to kGemmMaxGroup weights with the same K against the same X in one tensor-core launch (M >= gemm_min_m),
// else one GEMV launch per row and matrix.
int run_gemm_group(ter_b200_handle_t* h, const DevWeight* const* ws, int n, const int8_t* X, const float* x_scales,
                   int M, float* const* outs, int32_t* acc, cudaStream_t st, bool accumulate, const int32_t* x_rowsum) {
    if (n < 1 || n > kGemmMaxGroup || (n > 1 && acc)) return TER_B200_E_SHAPE;
    if (((uintptr_t)X & 15u) != 0) return TER_B200_E_SHAPE;
    for (int i = 1; i < n; ++i)
        if (ws[i]->K != ws[0]->K) return TER_B200_E_SHAPE;
    int group_strips = 0;
    for (int i = 0; i < n; ++i) group_strips += ws[i]->tiles();
    const int kernel = pick_kernel(h, M, ws[0]->K, group_strips);
    if (kernel != TER_B200_KERNEL_GEMM_TCGEN05) {
        if (kernel == TER_B200_KERNEL_GEMV_ROWS && n <= kGemvMaxGroup) {
            // a small token batch: ONE launch, the weights stream once for all rows (gemv_trit_rows_kernel)
            if (!x_scales && outs && outs[0]) return TER_B200_E_NULL;
            GemvParams gp;
            memset(&gp, 0, sizeof gp);
            gp.K = ws[0]->K;
            gp.Kpad = ws[0]->Kpad;
            int tiles = 0;
            for (int i = 0; i < n; ++i) {
                gp.W[i] = ws[i]->data;
                gp.out[i] = outs ? outs[i] : nullptr;
                gp.acc_out[i] = (acc && i == 0) ? acc : nullptr;
                gp.w_scale[i] = ws[i]->scale;
                gp.N[i] = ws[i]->N;
                gp.tile_begin[i] = tiles;
                tiles += ws[i]->tiles();
            }
            for (int i = n; i <= kGemvMaxGroup; ++i) gp.tile_begin[i] = tiles;
            gp.x = X;
            gp.x_scale = x_scales;
            gp.n_mats = n;
            gp.n_tiles = tiles;
            gp.rows = M;
            gp.status = h->status_dev;
            gp.accumulate = accumulate ? 1 : 0;
            GemvLaunchCfg cfg = h->gemv_cfg;
            cfg.sm_count = h->sm_count;
            TERB_CUDA(h, launch_gemv(gp, cfg, st));
            h->launches += 1;
            for (int i = 0; i < n; ++i) count_gemv(h, ws[i]->K, ws[i]->N, M);
            return TER_B200_OK;
        }
        // otherwise one GEMV launch per row (exact; the weights are re-read M times)
        for (int i = 0; i < n; ++i) {
            const DevWeight* w = ws[i];
            float* out = outs ? outs[i] : nullptr;
            for (int m = 0; m < M; ++m) {
                const DevWeight* w1[1] = {w};
                float* o[1] = {out ? out + (size_t)m * w->N : nullptr};
                int32_t* a[1] = {acc ? acc + (size_t)m * w->N : nullptr};
                int rc = run_gemv(h, w1, 1, X + (size_t)m * w->K, x_scales ? x_scales + m : nullptr, 1.0f,
                                  out ? o : nullptr, acc ? a : nullptr, accumulate, st);
                if (rc) return rc;
            }
        }
        return TER_B200_OK;
    }
    if (!x_scales && outs && outs[0]) return TER_B200_E_NULL;
    GemmParams p;
    memset(&p, 0, sizeof p);
    p.X = X;
    p.x_scales = x_scales;
    p.acc_out = acc;
    p.M = M; p.K = ws[0]->K; p.Kpad = ws[0]->Kpad;
    p.n_w = n;
    size_t n_sum = 0;
    for (int i = 0; i < n; ++i) {
        p.Wg[i] = ws[i]->data;
        p.outg[i] = outs ? outs[i] : nullptr;
        p.wsg[i] = ws[i]->scale;
        p.Ng[i] = ws[i]->N;
        p.stripsg[i] = ws[i]->tiles();
        n_sum += (size_t)ws[i]->N;
    }
    p.W = p.Wg[0]; p.out = p.outg[0]; p.w_scale = p.wsg[0]; p.N = p.Ng[0]; p.n_strips = p.stripsg[0];
    p.status = h->status_dev;
    p.accumulate = accumulate ? 1 : 0;
    p.x_rowsum = x_rowsum;
    {
        const size_t need_part = (h->gemm_split_k && M <= 256) ? (size_t)M * n_sum : 0;
        if (h->gemm_scratch_cap < (size_t)M || h->gemm_part_cap < need_part) {
            cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
            cudaStreamIsCapturing(st, &cs);
            if (cs != cudaStreamCaptureStatusNone && h->gemm_scratch_cap < (size_t)M && !x_rowsum) return TER_B200_E_STATE;
            if (cs == cudaStreamCaptureStatusNone) {
                int rc = ensure_gemm_scratch(h, M, (int)n_sum);
                if (rc) return rc;
            }
        }
        p.scratch = h->gemm_scratch;
        p.part_buf = (need_part && h->gemm_part_cap >= need_part) ? h->gemm_part : nullptr;
    }
    TERB_CUDA(h, launch_gemm(p, h->sm_count, h->gemv_cfg.pdl != 0, st));
    h->launches += 2;
    for (int i = 0; i < n; ++i) count_gemv(h, ws[i]->K, ws[i]->N, M);
    return TER_B200_OK;
}

int run_gemm(ter_b200_handle_t* h, const DevWeight* w, const int8_t* X, const float* x_scales, int M, float* out,
             int32_t* acc, cudaStream_t st, bool accumulate, const int32_t* x_rowsum) {
    const DevWeight* ws[1] = {w};
    float* outs[1] = {out};
    return run_gemm_group(h, ws, 1, X, x_scales, M, out ? outs : nullptr, acc, st, accumulate, x_rowsum);
}

}  // namespace terb

extern "C" {

int ter_b200_gemm(ter_b200_handle_t* h, const char* slot, const int8_t* X_dev, const float* x_scales_dev, int M,
                  float* out_dev, void* stream) {
    if (!h || !slot || !X_dev || !x_scales_dev || !out_dev) return TER_B200_E_NULL;
    if (M < 1) return TER_B200_E_SHAPE;
    TerbSlot* s = find_slot(h, slot);
    if (!s) return TER_B200_E_UNKNOWN;
    TERB_CUDA(h, cudaSetDevice(h->device));
    return run_gemm(h, &s->w, X_dev, x_scales_dev, M, out_dev, nullptr, pick_stream(h, stream));
}

int ter_b200_gemm_acc(ter_b200_handle_t* h, const char* slot, const int8_t* X_dev, int M, int32_t* acc_dev,
                      void* stream) {
    if (!h || !slot || !X_dev || !acc_dev) return TER_B200_E_NULL;
    if (M < 1) return TER_B200_E_SHAPE;
    TerbSlot* s = find_slot(h, slot);
    if (!s) return TER_B200_E_UNKNOWN;
    TERB_CUDA(h, cudaSetDevice(h->device));
    return run_gemm(h, &s->w, X_dev, nullptr, M, nullptr, acc_dev, pick_stream(h, stream));
}

int ter_b200_call(ter_b200_handle_t* h, const char* name, const int64_t* args, size_t n_args) {
    if (!h || !name) return TER_B200_E_NULL;
    if (n_args > 7) return TER_B200_E_NARGS;
    if (strcmp(name, "tk_matmul_b_9t") == 0) {
        if (!args || n_args < 5) return TER_B200_E_SHAPE;
        const char* slot = (const char*)(intptr_t)args[0];
        const int8_t* x = (const int8_t*)(intptr_t)args[1];
        const float* xs = (const float*)(intptr_t)args[2];
        float* out = (float*)(intptr_t)args[3];
        const int M = (int)args[4];
        void* stream = n_args > 5 ? (void*)(intptr_t)args[5] : nullptr;
        if (M == 1) return ter_b200_gemv(h, slot, x, xs, out, stream);
        return ter_b200_gemm(h, slot, x, xs, M, out, stream);
    }
    // The other four operator names the reference's forward looks up (src/tx/forward.cpp:376-380), mapped
    // onto the typed entry points; several small integers share one argument where seven would not do.
    auto f32 = [](int64_t a) { uint32_t b = (uint32_t)a; float f; memcpy(&f, &b, 4); return f; };
    auto f64 = [](int64_t a) { double d; memcpy(&d, &a, 8); return d; };
    auto ptr = [](int64_t a) { return (void*)(intptr_t)a; };
    if (strcmp(name, "tk_rmsnorm") == 0) {   // x, gamma, n, rows, eps (float bits), q, scale
        if (!args || n_args < 7) return TER_B200_E_SHAPE;
        return ter_b200_rmsnorm_quant(h, (const float*)ptr(args[0]), (const float*)ptr(args[1]), (int)args[2], (int)args[3],
                                      f32(args[4]), (int8_t*)ptr(args[5]), (float*)ptr(args[6]), nullptr, nullptr);
    }
    if (strcmp(name, "tk_silu") == 0) {      // gate, up, n, rows, q, scale[, stream]
        if (!args || n_args < 6) return TER_B200_E_SHAPE;
        return ter_b200_act_quant(h, TER_B200_ACT_SILU, (const float*)ptr(args[0]), (const float*)ptr(args[1]), nullptr,
                                  (int)args[2], (int)args[3], 0.0f, (int8_t*)ptr(args[4]), (float*)ptr(args[5]),
                                  n_args > 6 ? ptr(args[6]) : nullptr);
    }
    if (strcmp(name, "tk_rope") == 0) {      // q, k, pos, dims = B | Nh<<16 | Nkv<<32 | Hd<<48, Smax, theta (double bits), neox
        if (!args || n_args < 7) return TER_B200_E_SHAPE;
        const uint64_t d = (uint64_t)args[3];
        return ter_b200_rope_kv(h, (float*)ptr(args[0]), (float*)ptr(args[1]), nullptr, (const int*)ptr(args[2]),
                                (int)(d & 0xffff), (int)((d >> 16) & 0xffff), (int)((d >> 32) & 0xffff), (int)(d >> 48),
                                (int)args[4], f64(args[5]), (int)args[6], nullptr, nullptr, nullptr);
    }
    if (strcmp(name, "tk_softmax") == 0) {   // the softmax of the path lives inside attention: q, kcache, vcache, pos, dims, Smax, out
        if (!args || n_args < 7) return TER_B200_E_SHAPE;
        const uint64_t d = (uint64_t)args[4];
        return ter_b200_attention_noalloc(h, (const float*)ptr(args[0]), (const uint16_t*)ptr(args[1]),
                                          (const uint16_t*)ptr(args[2]), (const int*)ptr(args[3]), (int)(d & 0xffff),
                                          (int)((d >> 16) & 0xffff), (int)((d >> 32) & 0xffff), (int)(d >> 48),
                                          (int)args[5], (float*)ptr(args[6]), nullptr);
    }
    return TER_B200_E_UNKNOWN;
}

}  // extern "C"
