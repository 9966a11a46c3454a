// ter_b200_call: the named-operator entry point (ter_k4_call, src/k4/ter_k4.cpp:47-59),
// plus the batched GEMM entry points.
#include "handle.h"

using namespace terb;

extern "C" {

int ter_b200_gemm(ter_b200_handle_t* h, const char* slot, const int8_t* X_dev, const float* x_scales_dev, int M,
                  float* out_dev, void* stream) {
    if (!h || !slot || !X_dev || !x_scales_dev || !out_dev) return TER_B200_E_NULL;
    if (M < 1) return TER_B200_E_SHAPE;
    TerbSlot* s = find_slot(h, slot);
    if (!s) return TER_B200_E_UNKNOWN;
    // Row-at-a-time through the GEMV kernel (exact; the tensor-core path replaces this for M >= 16).
    for (int m = 0; m < M; ++m) {
        int rc = ter_b200_gemv(h, slot, X_dev + (size_t)m * s->w.K, x_scales_dev + m,
                               out_dev + (size_t)m * s->w.N, stream);
        if (rc) return rc;
    }
    return TER_B200_OK;
}

int ter_b200_gemm_acc(ter_b200_handle_t* h, const char* slot, const int8_t* X_dev, int M, int32_t* acc_dev,
                      void* stream) {
    if (!h || !slot || !X_dev || !acc_dev) return TER_B200_E_NULL;
    if (M < 1) return TER_B200_E_SHAPE;
    TerbSlot* s = find_slot(h, slot);
    if (!s) return TER_B200_E_UNKNOWN;
    for (int m = 0; m < M; ++m) {
        int rc = ter_b200_gemv_acc(h, slot, X_dev + (size_t)m * s->w.K, acc_dev + (size_t)m * s->w.N, stream);
        if (rc) return rc;
    }
    return TER_B200_OK;
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
    return TER_B200_E_UNKNOWN;
}

}  // extern "C"
