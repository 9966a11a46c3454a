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
    }
    h->comm = c;
    return TER_B200_OK;
}

void ter_b200_comm_destroy(ter_b200_handle_t* h) {
    if (!h || !h->comm) return;
    cudaSetDevice(h->device);
    cudaDeviceSynchronize();
    if (h->comm->comm) h->comm->comm_destroy(h->comm->comm);
    delete h->comm;
    h->comm = nullptr;
}

int ter_b200_comm_rank(const ter_b200_handle_t* h) { return h ? comm_rank(h) : 0; }
int ter_b200_comm_size(const ter_b200_handle_t* h) { return h ? comm_size(h) : 1; }

}  // extern "C"
