// TEST INFRASTRUCTURE, NOT PRODUCT CODE.
//
// Thin C-ABI driver around the UNMODIFIED reference CPU implementation of the
// ternary matmul fabric.  It is compiled against the reference sources where
// they lie (see oracle/Makefile, variable REF) and never copies them: the
// translation unit textually includes the reference's src/tx/forward.cpp so
// that the file-local GEMV `mm_row` (src/tx/forward.cpp:299-352, inside an
// anonymous namespace) can be called, exactly as the reference's own
// forward_layer calls it (src/tx/forward.cpp:401-403).
//
// Exports:
//   ref_tensor_*      build a ter::TritTensor (include/ter/numfmt.hpp:17-36)
//   ref_mm_row        ter::tx::mm_row on row `row` of X against W [K][N]
//   ref_quantize      ter::quantize (src/numfmt/quantize.cpp:7-41)
//   ref_tvmac         the analytic TVMAC counter mm_row bumps
//                     (src/tx/forward.cpp:349-350)
//
// Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may
// load the library built from this file.
#include "src/tx/forward.cpp"   // resolved through -I$(REF)

#include <ter/numfmt.hpp>
#include <ter/sim.hpp>
#include <ter/kernels.hpp>
#include <cstdint>
#include <cstring>
#include <new>
#include <vector>

namespace {
struct RefCtx {
    ter::Sim sim;
    ter::KernelTable kt;
    RefCtx() : sim(4096) {}
};
}  // namespace

extern "C" {

void* ref_ctx_create() { return new (std::nothrow) RefCtx(); }
void ref_ctx_destroy(void* c) { delete static_cast<RefCtx*>(c); }

// Analytic TVMAC count accumulated by mm_row calls on this context.
uint64_t ref_tvmac(void* c) {
    return static_cast<RefCtx*>(c)->sim.counters().get(ter::Opcode::TVMAC);
}
void ref_reset_counters(void* c) { static_cast<RefCtx*>(c)->sim.counters().reset(); }

// A TritTensor holding `n` int32 payload values and one per-tensor scale.
void* ref_tensor_create(const int32_t* payload, size_t n, float scale, int rows, int cols) {
    auto* t = new (std::nothrow) ter::TritTensor();
    if (!t) return nullptr;
    t->scale = scale;
    t->shape = {rows, cols};
    t->payload.assign(payload, payload + n);
    return t;
}
void ref_tensor_set_scale(void* t, float scale) { static_cast<ter::TritTensor*>(t)->scale = scale; }
// Overwrite the payload in place (same element count) — lets a caller reuse
// one activation tensor across calls without reallocating.
void ref_tensor_set_payload(void* t, const int32_t* payload, size_t n) {
    auto* tt = static_cast<ter::TritTensor*>(t);
    if (tt->payload.size() != n) tt->payload.resize(n);
    std::memcpy(tt->payload.data(), payload, n * sizeof(int32_t));
}
void ref_tensor_destroy(void* t) { delete static_cast<ter::TritTensor*>(t); }

// out[j] = float(sum_k X[row*K+k] * W[k*N+j]) * (X.scale * W.scale), j < N.
int ref_mm_row(void* c, const void* Xt, int row, const void* Wt, int K, int N, float* out) {
    if (!c || !Xt || !Wt || !out) return -1;
    auto* ctx = static_cast<RefCtx*>(c);
    std::vector<float> o;
    ter::tx::mm_row(ctx->sim, ctx->kt, ter::KernelId{},
                    *static_cast<const ter::TritTensor*>(Xt), row,
                    *static_cast<const ter::TritTensor*>(Wt), K, N, o);
    std::memcpy(out, o.data(), static_cast<size_t>(N) * sizeof(float));
    return 0;
}

// Same call, `iters` times back to back (CPU-baseline timing loop; the output
// of the last call is returned).
int ref_mm_row_repeat(void* c, const void* Xt, const void* Wt, int K, int N, float* out, int iters) {
    if (!c || !Xt || !Wt || !out) return -1;
    auto* ctx = static_cast<RefCtx*>(c);
    std::vector<float> o;
    for (int i = 0; i < iters; ++i)
        ter::tx::mm_row(ctx->sim, ctx->kt, ter::KernelId{},
                        *static_cast<const ter::TritTensor*>(Xt), 0,
                        *static_cast<const ter::TritTensor*>(Wt), K, N, o);
    std::memcpy(out, o.data(), static_cast<size_t>(N) * sizeof(float));
    return 0;
}

// ter::quantize: absmax / ((3^n-1)/2), lround, clamp.  Returns the scale.
float ref_quantize(const float* data, int n, int n_trits, int32_t* payload_out) {
    ter::TritTensor t = ter::quantize(data, {1, n}, n_trits);
    if (t.payload.size() == static_cast<size_t>(n))
        std::memcpy(payload_out, t.payload.data(), static_cast<size_t>(n) * sizeof(int32_t));
    return t.scale;
}

}  // extern "C"
