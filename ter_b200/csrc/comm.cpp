// NCCL plumbing for tensor-parallel decode: one process per GPU, one communicator per handle.
// The reference has no multi-GPU code; this is new.  NCCL is resolved at run time with dlopen (the
// copy already loaded by the host process, e.g. the one bundled with torch, or the system library),
// so the library itself links against nothing but the CUDA runtime.
#include <dlfcn.h>
#include <new>
#include <stdlib.h>

#include "handle.h"

namespace terb {

struct NcclId { char bytes[128]; };
typedef int (*fn_get_unique_id)(NcclId*);
typedef int (*fn_comm_init_rank)(void**, int, NcclId, int);
typedef int (*fn_comm_destroy)(void*);
typedef int (*fn_all_gather)(const void*, void*, size_t, int, void*, cudaStream_t);
typedef int (*fn_group)(void);
typedef const char* (*fn_err)(int);

struct Comm {
    void* lib = nullptr;
    fn_get_unique_id get_unique_id = nullptr;
    fn_comm_init_rank comm_init_rank = nullptr;
    fn_comm_destroy comm_destroy = nullptr;
    fn_all_gather all_gather = nullptr;
    fn_group group_start = nullptr, group_end = nullptr;
    void* comm = nullptr;
    int rank = 0, size = 1;
    uint8_t* scratch = nullptr;   // device, kMaxRanks * 64 bytes: handle exchange and barriers
};

static void* open_nccl() {
    const char* env = getenv("TER_B200_NCCL_LIB");
    const char* names[] = {env, "libnccl.so.2", "libnccl.so"};
    for (const char* n : names) {
        if (!n || !*n) continue;
        void* l = dlopen(n, RTLD_NOW | RTLD_NOLOAD);     // a copy the process already holds wins
        if (!l) l = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (l) return l;
    }
    return nullptr;
}

static int load_syms(Comm* c) {
    c->lib = open_nccl();
    if (!c->lib) return TER_B200_E_NCCL;
    c->get_unique_id = (fn_get_unique_id)dlsym(c->lib, "ncclGetUniqueId");
    c->comm_init_rank = (fn_comm_init_rank)dlsym(c->lib, "ncclCommInitRank");
    c->comm_destroy = (fn_comm_destroy)dlsym(c->lib, "ncclCommDestroy");
    c->all_gather = (fn_all_gather)dlsym(c->lib, "ncclAllGather");
    c->group_start = (fn_group)dlsym(c->lib, "ncclGroupStart");
    c->group_end = (fn_group)dlsym(c->lib, "ncclGroupEnd");
    if (!c->get_unique_id || !c->comm_init_rank || !c->comm_destroy || !c->all_gather || !c->group_start || !c->group_end)
        return TER_B200_E_NCCL;
    return TER_B200_OK;
}

int comm_rank(const ter_b200_handle_t* h) { return h->comm ? h->comm->rank : 0; }
int comm_size(const ter_b200_handle_t* h) { return h->comm ? h->comm->size : 1; }

// In-place all-gather of `n` equal byte slices: rank r's slice already sits at buf + r*bytes.
int comm_all_gather_bytes(ter_b200_handle_t* h, void* buf, size_t bytes, cudaStream_t st) {
    Comm* c = h->comm;
    if (!c || c->size == 1) return TER_B200_OK;
    const int rc = c->all_gather((const char*)buf + (size_t)c->rank * bytes, buf, bytes, /*ncclInt8*/ 0, c->comm, st);
    return rc == 0 ? TER_B200_OK : TER_B200_E_NCCL;
}
// Host-level barrier over the communicator (a tiny all-gather followed by a stream synchronise).
int comm_barrier(ter_b200_handle_t* h, cudaStream_t st) {
    Comm* c = h->comm;
    if (!c || c->size == 1) return TER_B200_OK;
    int rc = comm_all_gather_bytes(h, c->scratch, 64, st);
    if (rc) return rc;
    TERB_CUDA(h, cudaStreamSynchronize(st));
    return TER_B200_OK;
}

// Gathers one 64-byte record per rank (blocking).
static int gather64(ter_b200_handle_t* h, const void* mine, void* all, cudaStream_t st) {
    Comm* c = h->comm;
    TERB_CUDA(h, cudaMemcpyAsync(c->scratch + (size_t)c->rank * 64, mine, 64, cudaMemcpyHostToDevice, st));
    int rc = comm_all_gather_bytes(h, c->scratch, 64, st);
    if (rc) return rc;
    TERB_CUDA(h, cudaMemcpyAsync(all, c->scratch, (size_t)c->size * 64, cudaMemcpyDeviceToHost, st));
    TERB_CUDA(h, cudaStreamSynchronize(st));
    return TER_B200_OK;
}

// Allocates `bytes` of zeroed device memory that every peer maps (CUDA IPC, one process per GPU).
// All ranks call this together.  Returns TER_B200_E_STATE on EVERY rank when any rank could not map
// a peer (no peer access between the GPUs): the caller then stays on NCCL collectives.
int comm_arena_create(ter_b200_handle_t* h, size_t bytes, PeerArena* a, cudaStream_t st) {
    Comm* c = h->comm;
    if (!c || c->size < 2 || c->size > kMaxRanks) return TER_B200_E_STATE;
    memset(a, 0, sizeof *a);
    TERB_CUDA(h, cudaMalloc((void**)&a->base, bytes));
    a->bytes = bytes;
    cudaError_t e = cudaMemset(a->base, 0, bytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    union { cudaIpcMemHandle_t hd; char raw[64]; } mine, all[kMaxRanks];
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    memset(&mine, 0, sizeof mine);
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&mine.hd, a->base);
    int ok = e == cudaSuccess ? 1 : 0;
    int rc = gather64(h, &mine, all, st);       // everybody's memset is done once this returns
    if (rc) { cudaFree(a->base); a->base = nullptr; return rc; }
    for (int r = 0; r < c->size && ok; ++r) {
        if (r == c->rank) { a->peer[r] = a->base; continue; }
        void* ptr = nullptr;
        if (cudaIpcOpenMemHandle(&ptr, all[r].hd, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
            (void)cudaGetLastError();
            ok = 0;
        } else {
            a->peer[r] = (uint8_t*)ptr;
        }
    }
    // consensus: one rank without peer access turns the arena off everywhere
    char vote[64] = {}, votes[kMaxRanks][64];
    vote[0] = (char)ok;
    rc = gather64(h, vote, votes, st);
    int all_ok = rc == 0;
    for (int r = 0; r < c->size && all_ok; ++r) all_ok = votes[r][0] != 0;
    if (!all_ok) {
        for (int r = 0; r < c->size; ++r)
            if (r != c->rank && a->peer[r]) cudaIpcCloseMemHandle(a->peer[r]);
        comm_barrier(h, st);                    // nobody frees while a peer may still be mapping
        cudaFree(a->base);
        memset(a, 0, sizeof *a);
        return rc ? rc : TER_B200_E_STATE;
    }
    a->open = true;
    return TER_B200_OK;
}

// All ranks call this together, between steps: waits until every rank has stopped using the arenas.
void comm_arena_destroy(ter_b200_handle_t* h, PeerArena* a, cudaStream_t st) {
    if (!a->base) return;
    Comm* c = h->comm;
    cudaDeviceSynchronize();
    if (c && a->open) {
        comm_barrier(h, st);
        for (int r = 0; r < c->size; ++r)
            if (r != c->rank && a->peer[r]) cudaIpcCloseMemHandle(a->peer[r]);
        comm_barrier(h, st);
    }
    cudaFree(a->base);
    memset(a, 0, sizeof *a);
}

int comm_group_start(ter_b200_handle_t* h) {
    return (h->comm && h->comm->size > 1 && h->comm->group_start() != 0) ? TER_B200_E_NCCL : TER_B200_OK;
}
int comm_group_end(ter_b200_handle_t* h) {
    return (h->comm && h->comm->size > 1 && h->comm->group_end() != 0) ? TER_B200_E_NCCL : TER_B200_OK;
}

}  // namespace terb

using namespace terb;

extern "C" {

int ter_b200_comm_unique_id(uint8_t* id128) {
    if (!id128) return TER_B200_E_NULL;
    Comm tmp;
    int rc = load_syms(&tmp);
    if (rc) return rc;
    NcclId id;
    if (tmp.get_unique_id(&id) != 0) return TER_B200_E_NCCL;
    memcpy(id128, id.bytes, 128);
    return TER_B200_OK;
}

int ter_b200_comm_init(ter_b200_handle_t* h, const uint8_t* id128, int rank, int size) {
    if (!h || !id128) return TER_B200_E_NULL;
    if (size < 1 || rank < 0 || rank >= size) return TER_B200_E_SHAPE;
    if (h->comm) return TER_B200_E_STATE;
    TERB_CUDA(h, cudaSetDevice(h->device));
    Comm* c = new (std::nothrow) Comm();
    if (!c) return TER_B200_E_ALLOC;
    c->rank = rank;
    c->size = size;
    if (size > 1) {
        int rc = load_syms(c);
        if (rc) { delete c; return rc; }
        NcclId id;
        memcpy(id.bytes, id128, 128);
        if (c->comm_init_rank(&c->comm, size, id, rank) != 0) { delete c; return TER_B200_E_NCCL; }
        if (cudaMalloc((void**)&c->scratch, (size_t)kMaxRanks * 64) != cudaSuccess ||
            cudaMemset(c->scratch, 0, (size_t)kMaxRanks * 64) != cudaSuccess) {
            (void)cudaGetLastError();
            c->comm_destroy(c->comm);
            if (c->scratch) cudaFree(c->scratch);
            delete c;
            return TER_B200_E_ALLOC;
        }
    }
    h->comm = c;
    return TER_B200_OK;
}

void ter_b200_model_free(ter_b200_handle_t* h);   // model.cpp: a model may hold a peer arena of this communicator

void ter_b200_comm_destroy(ter_b200_handle_t* h) {
    if (!h || !h->comm) return;
    cudaSetDevice(h->device);
    if (h->comm->size > 1) ter_b200_model_free(h);
    cudaDeviceSynchronize();
    if (h->comm->scratch) cudaFree(h->comm->scratch);
    if (h->comm->comm) h->comm->comm_destroy(h->comm->comm);
    delete h->comm;
    h->comm = nullptr;
}

int ter_b200_comm_rank(const ter_b200_handle_t* h) { return h ? comm_rank(h) : 0; }
int ter_b200_comm_size(const ter_b200_handle_t* h) { return h ? comm_size(h) : 1; }

}  // extern "C"
