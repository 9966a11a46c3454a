// Sweeps: many independent packed-trit GEMVs in ONE launch of the streaming kernel.
//
// The reference times its packed GEMV one launch per matrix (cuda/ter_cuda_forward_packed_v12.cu:414-464)
// and its forwards call mm_packed_dispatch once per projection (cuda/ter_cuda_forward_packed.cu:505-563).
// A B200 drains a 1 MB projection in well under a microsecond, so per-launch cost dominates such a
// sequence; here every matrix of a sweep is a row of a descriptor table in device memory and one
// persistent grid streams all of them.
//
//   * plans  (ter_b200_gemv_plan_*): device-resident inputs and outputs, table built once.
//   * ter_b200_gemv_multi: at most 8 matrices, descriptors passed by value (no table).
//   * ter_b200_gemv_host_batch: host buffers; the table, the scales and the activation vectors travel in
//     ONE host-to-device copy from pinned staging, the results come back in as few copies as the caller's
//     output layout allows.
#include <stdlib.h>

#include <algorithm>

#include "handle.h"

#include <cuda.h>

namespace terb {
int ensure_host_staging(ter_b200_handle_t* h, size_t x_bytes, size_t out_floats);   // abi.cpp
}
using namespace terb;

namespace {

// Collects the distinct activation vectors of a sweep and the per-matrix descriptors.
struct SweepBuilder {
    GemvParams p;
    GemvDesc descs[kGemvMaxTable];
    const void* key_a[kGemvMaxX];
    const void* key_b[kGemvMaxX];
    int n = 0, tiles = 0;

    SweepBuilder() {
        memset(&p, 0, sizeof p);
        p.multi = 1;
    }
    // Which vector (key_a, key_b, K) is; -1 when it is new.
    int find_x(const void* a, const void* b, int K) const {
        for (int u = 0; u < p.n_x; ++u)
            if (key_a[u] == a && key_b[u] == b && p.uK[u] == K) return u;
        return -1;
    }
    bool fits(const DevWeight& w, const void* a, const void* b) const {
        if (n >= kGemvMaxTable) return false;
        if (find_x(a, b, w.K) >= 0) return true;
        return p.n_x < kGemvMaxX && p.x_bytes + w.Kpad <= kGemvMaxXBytes;
    }
    // Returns the vector index the matrix uses.
    int add(const DevWeight& w, const void* a, const void* b, float* out) {
        int u = find_x(a, b, w.K);
        if (u < 0) {
            u = p.n_x++;
            key_a[u] = a;
            key_b[u] = b;
            p.uK[u] = w.K;
            p.uKpad[u] = w.Kpad;
            p.uoff[u] = p.x_bytes;
            p.x_bytes += w.Kpad;
        }
        GemvDesc& d = descs[n];
        d.W = w.data;
        d.out = out;
        d.w_scale = w.scale;
        d.N = w.N;
        d.tile_begin = tiles;
        d.xid = u;
        tiles += w.tiles();
        ++n;
        return u;
    }
    // Table launches: longest strips first.  Strips go to warps round-robin, so equal strips in a row are
    // spread evenly, and the long ones (large K) end up one per warp instead of clustering.
    void sort_by_work() {
        std::stable_sort(descs, descs + n, [&](const GemvDesc& a, const GemvDesc& b) {
            return p.uKpad[a.xid] > p.uKpad[b.xid];
        });
        int t = 0;
        for (int i = 0; i < n; ++i) {
            descs[i].tile_begin = t;
            t += (descs[i].N + 15) / 16;
        }
    }
    void finish(int* status) {
        p.n_mats = n;
        p.n_tiles = tiles;
        p.K = p.uK[0];
        p.Kpad = p.uKpad[0];
        p.status = status;
    }
    // By-value form for at most kGemvMaxGroup matrices.
    void to_arrays() {
        for (int i = 0; i < n; ++i) {
            p.W[i] = descs[i].W;
            p.out[i] = descs[i].out;
            p.w_scale[i] = descs[i].w_scale;
            p.N[i] = descs[i].N;
            p.tile_begin[i] = descs[i].tile_begin;
            p.xid[i] = (uint8_t)descs[i].xid;
        }
        for (int i = n; i <= kGemvMaxGroup; ++i) p.tile_begin[i] = tiles;
        p.table = nullptr;
    }
};

int launch_sweep(ter_b200_handle_t* h, const GemvParams& p, cudaStream_t st) {
    GemvLaunchCfg cfg = h->gemv_cfg;
    cfg.sm_count = h->sm_count;
    TERB_CUDA(h, launch_gemv(p, cfg, st));
    h->launches += 1;
    return TER_B200_OK;
}

size_t round256(size_t v) { return (v + 255) & ~(size_t)255; }

}  // namespace

extern "C" {

int ter_b200_gemv_multi(ter_b200_handle_t* h, int n, const char* const* slots, const int8_t* const* x_devs,
                        const float* const* x_scale_devs, float* const* outs_dev, void* stream) {
    if (!h || !slots || !x_devs || !x_scale_devs || !outs_dev) return TER_B200_E_NULL;
    if (n < 1 || n > kGemvMaxGroup) return TER_B200_E_SHAPE;
    SweepBuilder* b = new SweepBuilder();
    int rc = TER_B200_OK;
    for (int i = 0; i < n && !rc; ++i) {
        if (!slots[i] || !x_devs[i] || !x_scale_devs[i] || !outs_dev[i]) { rc = TER_B200_E_NULL; break; }
        if (((uintptr_t)x_devs[i] & 15u) != 0) { rc = TER_B200_E_SHAPE; break; }
        TerbSlot* s = find_slot(h, slots[i]);
        if (!s) { rc = TER_B200_E_UNKNOWN; break; }
        if (!b->fits(s->w, x_devs[i], x_scale_devs[i])) { rc = TER_B200_E_SHAPE; break; }
        const int u = b->add(s->w, x_devs[i], x_scale_devs[i], outs_dev[i]);
        b->p.ux[u] = x_devs[i];
        b->p.uxs[u] = x_scale_devs[i];
        count_gemv(h, s->w.K, s->w.N, 1);
    }
    if (!rc) {
        b->finish(h->status_dev);
        b->to_arrays();
        cudaError_t e = cudaSetDevice(h->device);
        rc = e == cudaSuccess ? launch_sweep(h, b->p, pick_stream(h, stream)) : cuda_fail(h, e);
    }
    delete b;
    return rc;
}

int ter_b200_gemv_plan_create(ter_b200_handle_t* h, int n, const char* const* slots, const int8_t* const* x_devs,
                              const float* const* x_scale_devs, float* const* outs_dev, int* plan_id) {
    if (!h || !slots || !x_devs || !x_scale_devs || !outs_dev || !plan_id) return TER_B200_E_NULL;
    if (n < 1 || n > kGemvMaxTable) return TER_B200_E_SHAPE;
    int id = -1;
    for (int i = 0; i < TER_B200_MAX_PLANS; ++i)
        if (!h->plans[i].used) { id = i; break; }
    if (id < 0) return TER_B200_E_FULL;
    SweepBuilder* b = new SweepBuilder();
    int rc = TER_B200_OK;
    uint64_t tvmac = 0;
    for (int i = 0; i < n; ++i) {
        if (!slots[i] || !x_devs[i] || !x_scale_devs[i] || !outs_dev[i]) { rc = TER_B200_E_NULL; break; }
        if (((uintptr_t)x_devs[i] & 15u) != 0) { rc = TER_B200_E_SHAPE; break; }
        TerbSlot* s = find_slot(h, slots[i]);
        if (!s) { rc = TER_B200_E_UNKNOWN; break; }
        if (!b->fits(s->w, x_devs[i], x_scale_devs[i])) { rc = TER_B200_E_SHAPE; break; }
        const int u = b->add(s->w, x_devs[i], x_scale_devs[i], outs_dev[i]);
        b->p.ux[u] = x_devs[i];
        b->p.uxs[u] = x_scale_devs[i];
        tvmac += (uint64_t)((s->w.K + 26) / 27) * (uint64_t)s->w.N;
    }
    GemvDesc* tab = nullptr;
    if (!rc) {
        cudaError_t e = cudaSetDevice(h->device);
        const size_t tab_bytes = round256((size_t)n * sizeof(GemvDesc));
        b->sort_by_work();
        if (e == cudaSuccess) e = cudaMalloc((void**)&tab, tab_bytes);
        if (e == cudaSuccess) e = cudaMemcpy(tab, b->descs, (size_t)n * sizeof(GemvDesc), cudaMemcpyHostToDevice);
        if (e != cudaSuccess) {
            if (tab) cudaFree(tab);
            rc = cuda_fail(h, e);
        }
    }
    if (!rc) {
        b->finish(h->status_dev);
        b->p.table = tab;
        TerbPlan& pl = h->plans[id];
        pl.used = true;
        pl.epoch = h->weights_epoch;
        pl.p = b->p;
        pl.table_dev = tab;
        pl.tvmac = tvmac;
        *plan_id = id;
    }
    delete b;
    return rc;
}

int ter_b200_gemv_plan_launch(ter_b200_handle_t* h, int plan_id, void* stream) {
    if (!h) return TER_B200_E_NULL;
    if (plan_id < 0 || plan_id >= TER_B200_MAX_PLANS || !h->plans[plan_id].used) return TER_B200_E_UNKNOWN;
    TerbPlan& pl = h->plans[plan_id];
    if (pl.epoch != h->weights_epoch) return TER_B200_E_STATE;   // a weight slot changed since the plan was made
    TERB_CUDA(h, cudaSetDevice(h->device));
    h->counts.tvmac += pl.tvmac;
    h->counts.total_ops += pl.tvmac;
    return launch_sweep(h, pl.p, pick_stream(h, stream));
}

int ter_b200_gemv_plan_destroy(ter_b200_handle_t* h, int plan_id) {
    if (!h) return TER_B200_E_NULL;
    if (plan_id < 0 || plan_id >= TER_B200_MAX_PLANS || !h->plans[plan_id].used) return TER_B200_E_UNKNOWN;
    cudaSetDevice(h->device);
    cudaStreamSynchronize(h->stream);
    if (h->plans[plan_id].table_dev) cudaFree(h->plans[plan_id].table_dev);
    h->plans[plan_id] = TerbPlan{};
    return TER_B200_OK;
}


// True when [dev_ptr, dev_ptr + bytes) lies inside a single allocation (or host registration) known to the driver.
static bool run_in_one_allocation(void* dev_ptr, size_t bytes) {
    typedef CUresult (*RangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);
    static RangeFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (RangeFn)ptr;
    }
    if (!fn) return false;
    CUdeviceptr base = 0;
    size_t size = 0;
    if (fn(&base, &size, (CUdeviceptr)(uintptr_t)dev_ptr) != CUDA_SUCCESS) return false;
    const uintptr_t p0 = (uintptr_t)dev_ptr;
    return p0 >= (uintptr_t)base && p0 + bytes <= (uintptr_t)base + size;
}

int ter_b200_gemv_host_batch(ter_b200_handle_t* h, int n, const char* const* slots, const int8_t* const* x_hosts,
                             const float* x_scales, float* const* out_hosts, void* stream) {
    if (!h || !slots || !x_hosts || !x_scales || !out_hosts) return TER_B200_E_NULL;
    if (n < 1) return TER_B200_E_SHAPE;
    TERB_CUDA(h, cudaSetDevice(h->device));
    cudaStream_t st = pick_stream(h, stream);

    // Pass 1: resolve the slots; cut chunks where a launch's limits (matrices, distinct vectors, bytes of
    // x) would be exceeded.  Every chunk has its own [table][scales][x] region in the staging buffer.
    // A host vector is identified by (pointer, scale bits, K).
    struct Chunk { int i0, i1; size_t off; GemvParams p; };
    TerbSlot** sl = (TerbSlot**)malloc(sizeof(TerbSlot*) * (size_t)n);
    Chunk* chunks = (Chunk*)malloc(sizeof(Chunk) * (size_t)n);
    SweepBuilder* b = new SweepBuilder();
    auto cleanup = [&]() { free(sl); free(chunks); delete b; };
    if (!sl || !chunks) { cleanup(); return TER_B200_E_ALLOC; }
    size_t o_total = 0;
    for (int i = 0; i < n; ++i) {
        if (!slots[i] || !x_hosts[i] || !out_hosts[i]) { cleanup(); return TER_B200_E_NULL; }
        // a loop that calls with the same list finds every slot where the previous call found it
        TerbSlot* m = i < h->hb_memo_n ? h->hb_memo[i] : nullptr;
        if (m && m->used && strncmp(m->name, slots[i], TER_B200_MAX_NAME + 1) == 0) sl[i] = m;
        else sl[i] = find_slot(h, slots[i]);
        if (!sl[i]) { cleanup(); return TER_B200_E_UNKNOWN; }
        o_total += (size_t)sl[i]->w.Npad;
    }
    auto scale_key = [&](int i) {
        uint32_t bits;
        memcpy(&bits, &x_scales[i], sizeof bits);
        return (const void*)(uintptr_t)bits;
    };
    int n_chunks = 0;
    size_t stage_bytes = 0;
    for (int i = 0; i < n;) {
        *b = SweepBuilder();
        const int i0 = i;
        while (i < n && b->fits(sl[i]->w, x_hosts[i], scale_key(i))) {
            b->add(sl[i]->w, x_hosts[i], scale_key(i), nullptr);
            ++i;
        }
        if (i == i0) { cleanup(); return TER_B200_E_SHAPE; }   // one matrix alone exceeds the limits
        chunks[n_chunks].i0 = i0;
        chunks[n_chunks].i1 = i;
        chunks[n_chunks].off = stage_bytes;
        stage_bytes += round256(sizeof(GemvDesc) * (size_t)(i - i0)) + 256 + round256((size_t)b->p.x_bytes);
        ++n_chunks;
    }
    int rc = ensure_host_staging(h, stage_bytes, o_total);
    if (!rc && h->hpin_cap < stage_bytes) {
        if (h->hpin) cudaFreeHost(h->hpin);
        h->hpin = nullptr;
        h->hpin_cap = 0;
        cudaError_t e = cudaMallocHost((void**)&h->hpin, stage_bytes);
        if (e != cudaSuccess) rc = cuda_fail(h, e); else h->hpin_cap = stage_bytes;
    }
    if (rc) { cleanup(); return rc; }

    // Outputs that lie back to back in host memory form a run.  A run in PINNED host memory that the
    // device can address is written by the kernel itself (its 2 MB of results leave over PCIe while the
    // weights are still streaming), the others are staged on the device and copied afterwards.
    float** direct = (float**)calloc((size_t)n, sizeof(float*));   // device-visible address of out_hosts[i], or null
    if (!direct) { cleanup(); return TER_B200_E_ALLOC; }
    if (h->host_batch_direct) {
        for (int i = 0; i < n;) {
            size_t len = (size_t)sl[i]->w.N;
            int j = i + 1;
            while (j < n && sl[j - 1]->w.N == sl[j - 1]->w.Npad && out_hosts[j] == out_hosts[i] + len) {
                len += (size_t)sl[j]->w.N;
                ++j;
            }
            // The whole run must lie inside ONE pinned allocation or registration: with unified addressing the two
            // ends alone prove nothing (pageable memory may lie between two pinned regions).
            cudaPointerAttributes a0;
            if (cudaPointerGetAttributes(&a0, out_hosts[i]) == cudaSuccess && a0.type == cudaMemoryTypeHost &&
                a0.devicePointer && run_in_one_allocation(a0.devicePointer, len * sizeof(float))) {
                for (int k = i; k < j; ++k) direct[k] = (float*)a0.devicePointer + (out_hosts[k] - out_hosts[i]);
            } else {
                (void)cudaGetLastError();
            }
            i = j;
        }
    }

    // Pass 3: fill the pinned image of the staging buffer and the launch parameters.
    size_t oo = 0;
    for (int c = 0; c < n_chunks; ++c) {
        Chunk& ch = chunks[c];
        *b = SweepBuilder();
        const int cn = ch.i1 - ch.i0;
        const size_t tab_off = ch.off, sc_off = tab_off + round256(sizeof(GemvDesc) * (size_t)cn), x_off = sc_off + 256;
        float* sc_host = (float*)(h->hpin + sc_off);
        for (int i = ch.i0; i < ch.i1; ++i) {
            TerbSlot* s = sl[i];
            const int before = b->p.n_x;
            const int u = b->add(s->w, x_hosts[i], scale_key(i), direct[i] ? direct[i] : h->hout_dev + oo);
            if (u == before) {   // a new vector: copy it into the image
                memcpy(h->hpin + x_off + b->p.uoff[u], x_hosts[i], (size_t)s->w.K);
                sc_host[u] = x_scales[i];
                b->p.ux[u] = h->hx_dev + x_off + b->p.uoff[u];
                b->p.uxs[u] = (const float*)(h->hx_dev + sc_off) + u;
            }
            oo += (size_t)s->w.Npad;
            count_gemv(h, s->w.K, s->w.N, 1);
        }
        b->sort_by_work();
        memcpy(h->hpin + tab_off, b->descs, sizeof(GemvDesc) * (size_t)cn);
        b->finish(h->status_dev);
        b->p.table = (const GemvDesc*)(h->hx_dev + tab_off);
        ch.p = b->p;
    }
    cudaError_t e = cudaMemcpyAsync(h->hx_dev, h->hpin, stage_bytes, cudaMemcpyHostToDevice, st);
    for (int c = 0; c < n_chunks && e == cudaSuccess && !rc; ++c) rc = launch_sweep(h, chunks[c].p, st);
    if (e != cudaSuccess) rc = cuda_fail(h, e);

    // Results: one copy per run of outputs that is contiguous on both sides.
    oo = 0;
    for (int i = 0; i < n && !rc;) {
        float* dst = out_hosts[i];
        const size_t src_off = oo;
        size_t len = (size_t)sl[i]->w.N;
        oo += (size_t)sl[i]->w.Npad;
        int j = i + 1;
        while (j < n && sl[j - 1]->w.N == sl[j - 1]->w.Npad && out_hosts[j] == dst + len) {
            len += (size_t)sl[j]->w.N;
            oo += (size_t)sl[j]->w.Npad;
            ++j;
        }
        if (!direct[i]) {
            e = cudaMemcpyAsync(dst, h->hout_dev + src_off, len * sizeof(float), cudaMemcpyDeviceToHost, st);
            if (e != cudaSuccess) rc = cuda_fail(h, e);
        }
        i = j;
    }
    free(direct);
    if (!rc) {      // keep the resolved slots for the next call
        free(h->hb_memo);
        h->hb_memo = sl;
        h->hb_memo_n = n;
        sl = nullptr;
    }
    cleanup();
    if (rc) return rc;
    TERB_CUDA(h, cudaStreamSynchronize(st));   // the pinned image is reused by the next call
    return TER_B200_OK;
}

}  // extern "C"
