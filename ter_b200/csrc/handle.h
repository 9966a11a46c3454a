// Internal definition of the opaque handle behind include/ter_b200.h.
// Plain arrays and explicit error codes only: no exceptions cross the C boundary
// (the reference builds its wrapper the same way, CMakeLists.txt:52-57).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "../../include/ter_b200.h"
#include "kernels.h"

struct TerbSlot {
    char name[TER_B200_MAX_NAME + 1];
    bool used;
    uint32_t hash;   // name_hash(name): lookups compare this before the string
    terb::DevWeight w;
};

// A sweep plan: launch parameters + the device descriptor table of ter_b200_gemv_plan_create.
struct TerbPlan {
    bool used = false;
    uint64_t epoch = 0;    // weights_epoch when the plan was made
    uint64_t tvmac = 0;    // op-counter increment of one launch
    terb::GemvParams p;
    terb::GemvDesc* table_dev = nullptr;
};

// Device memory that every rank of the communicator has mapped (comm.cpp).
struct PeerArena {
    uint8_t* base;                  // local allocation
    size_t bytes;
    uint8_t* peer[terb::kMaxRanks]; // peer[r] = rank r's arena in this process's address space; peer[rank] = base
    bool open;
};

struct TerbModel;   // decode-forward state (model.cpp)
namespace terb { struct Comm; }

struct RopeTable {
    float* data = nullptr;   // device [n_pos][head_dim/2][2]
    int n_pos = 0, head_dim = 0;
    double theta = 0.0;
};

struct ter_b200_handle_t {
    int device;
    int sm_count;
    cudaStream_t stream;
    TerbSlot slots[TER_B200_MAX_SLOTS];
    ter_b200_op_counts_t counts;
    int* status_dev;          // device status word written by bounded waits
    int last_cuda;
    uint64_t launches;
    terb::GemvLaunchCfg gemv_cfg;
    // staging for the host-buffer entry points
    int8_t* hx_dev;   // also holds the descriptor tables of the host batch entry point
    size_t hx_cap;
    float* hout_dev;
    size_t hout_cap;
    float* hscale_dev;
    uint8_t* hpin;            // pinned host image of the staging buffer (host batch entry point)
    size_t hpin_cap;
    TerbSlot** hb_memo;       // slots resolved by the previous host-batch call, by position (tried first)
    int hb_memo_n;
    TerbPlan plans[TER_B200_MAX_PLANS];
    uint64_t weights_epoch;   // advances whenever a weight slot is replaced or removed
    TerbModel* model;
    RopeTable rope[4];
    terb::Comm* comm;           // tensor-parallel communicator (comm.cpp), or null
    int32_t* gemm_scratch;      // row sums of the activations of the tensor-core GEMM (one int per token)
    size_t gemm_scratch_cap;    // ints
    int32_t* gemm_part;         // split-K partials
    size_t gemm_part_cap;       // ints
    // Scratch buffers that were outgrown.  Captured graphs (the model's decode step, user graphs) keep
    // the addresses they were recorded with, so an outgrown buffer stays allocated until the handle goes.
    void* retired[64];
    int n_retired;
    size_t gemm_scratch_cap_prev, gemm_part_cap_prev;   // sizes of the latest allocations (growth is geometric)
    int gemm_min_m;             // batches below this take the multi-row GEMV (or, past its limits, one GEMV per row)
    int gemm_split_k;           // 0 = never split K
    int host_batch_direct;      // 1: ter_b200_gemv_host_batch lets the kernel write results into pinned host buffers
    int prefill_tile;           // prompt positions per pass (at most 1024)
    int prefill;                // 1: ter_b200_generate runs the prompt of a single sequence as token batches
    int tp_shard;               // bit 0: attention block column-sharded, bit 1: FFN block; the lm_head always is
    int tp_p2p;                 // 1: tensor-parallel exchanges over peer memory (exchange_sm100.cu); 0: NCCL all-gathers
    int attn_mma_min;           // attention over at least this many rows (sequences of a batch, positions of a prompt tile)
                                // sums its two contractions on the tensor cores (default: never)
    int lm_head_tc_min;         // batches of at least this many sequences run the bf16 lm_head on the tensor cores (0: never)
    int decode_persistent;      // 1: a lone sequence on one GPU runs embedding + all layers of a step in one persistent kernel
    int decode_poll_ns;         // persistent decode kernel: pause between polls of a value that has not arrived
    int decode_fault_cta;       // test hook (-1: off): see DecodeParams::fault_cta
    int wait_ms;                // limit of a device-side wait on another CTA or rank (milliseconds)
    int attn_inline_merge;      // 1: the last attention CTA of a KV head merges the chunks (no second kernel)
    cudaGraphExec_t graphs[16];
    uint64_t graph_launches[16];   // kernels recorded in each graph
    uint64_t capture_mark;
    bool capturing;
};

namespace terb {

inline int cuda_fail(ter_b200_handle_t* h, cudaError_t e) {
    if (e == cudaSuccess) return TER_B200_OK;
    if (h) h->last_cuda = (int)e;
    (void)cudaGetLastError();   // clear the sticky-free error state
    return e == cudaErrorMemoryAllocation ? TER_B200_E_ALLOC : TER_B200_E_CUDA;
}

#define TERB_CUDA(h, call)                                   \
    do {                                                     \
        cudaError_t e__ = (call);                            \
        if (e__ != cudaSuccess) return terb::cuda_fail((h), e__); \
    } while (0)

inline cudaStream_t pick_stream(ter_b200_handle_t* h, void* stream) {
    return stream ? (cudaStream_t)stream : h->stream;
}

inline uint32_t name_hash(const char* name) {
    uint32_t v = 2166136261u;
    for (int i = 0; i < TER_B200_MAX_NAME && name[i]; ++i) v = (v ^ (uint8_t)name[i]) * 16777619u;
    return v;
}

inline TerbSlot* find_slot(ter_b200_handle_t* h, const char* name) {
    const uint32_t hv = name_hash(name);
    for (int i = 0; i < TER_B200_MAX_SLOTS; ++i)
        if (h->slots[i].used && h->slots[i].hash == hv && strncmp(h->slots[i].name, name, TER_B200_MAX_NAME + 1) == 0) return &h->slots[i];
    return nullptr;
}
inline const TerbSlot* find_slot(const ter_b200_handle_t* h, const char* name) {
    return find_slot(const_cast<ter_b200_handle_t*>(h), name);
}

// The one dispatch rule: which kernel multiplies M activation rows by a K x N weight (n_strips = total strips
// of the launch group).  Everything that launches a GEMV or GEMM asks here.
inline int pick_kernel(const ter_b200_handle_t* h, int M, int K, int n_strips) {
    if (M <= 1)
        return (h->gemv_cfg.split_max_strips > 0 && n_strips <= h->gemv_cfg.split_max_strips) ? TER_B200_KERNEL_GEMV_SPLIT
                                                                                              : TER_B200_KERNEL_GEMV_STREAM;
    if (M >= h->gemm_min_m) return TER_B200_KERNEL_GEMM_TCGEN05;
    if (M <= kGemvMaxRows && (K & 15) == 0) return TER_B200_KERNEL_GEMV_ROWS;
    return TER_B200_KERNEL_GEMV_PER_ROW;
}

inline void count_gemv(ter_b200_handle_t* h, int K, int N, int rows) {
    const uint64_t n = (uint64_t)((K + 26) / 27) * (uint64_t)N * (uint64_t)rows;
    h->counts.tvmac += n;
    h->counts.total_ops += n;
}

// Allocates and fills a DevWeight from a DEVICE pointer in one of the boundary formats.
int build_weight_from_dev(ter_b200_handle_t* h, const void* data_dev, int format, int K, int N, float scale,
                          cudaStream_t st, DevWeight* out);
void free_weight(DevWeight* w);
int comm_rank(const ter_b200_handle_t* h);
int comm_size(const ter_b200_handle_t* h);
int comm_all_gather_bytes(ter_b200_handle_t* h, void* buf, size_t bytes_per_rank, cudaStream_t st);
int comm_barrier(ter_b200_handle_t* h, cudaStream_t st);
int comm_arena_create(ter_b200_handle_t* h, size_t bytes, PeerArena* a, cudaStream_t st);
void comm_arena_destroy(ter_b200_handle_t* h, PeerArena* a, cudaStream_t st);
int comm_group_start(ter_b200_handle_t* h);
int comm_group_end(ter_b200_handle_t* h);
void model_invalidate_graph(ter_b200_handle_t* h);
int ensure_gemm_scratch(ter_b200_handle_t* h, int M, int N);
// Batched GEMM over one weight (tensor cores for M >= gemm_min_m, else GEMV per row).
// x_rowsum: sum_k X[m][k] per token when the caller has it (the quantiser kernel can produce it), else null
int run_gemm(ter_b200_handle_t* h, const DevWeight* w, const int8_t* X, const float* x_scales, int M, float* out,
             int32_t* acc, cudaStream_t st, bool accumulate = false, const int32_t* x_rowsum = nullptr);
int run_gemm_group(ter_b200_handle_t* h, const DevWeight* const* ws, int n, const int8_t* X, const float* x_scales,
                   int M, float* const* outs, int32_t* acc, cudaStream_t st, bool accumulate = false,
                   const int32_t* x_rowsum = nullptr);
// One launch over up to kGemvMaxGroup weights sharing x (abi.cpp).
int run_gemv(ter_b200_handle_t* h, const DevWeight* const* ws, int n, const int8_t* x_dev, const float* x_scale_dev,
             float x_scale_imm, float* const* outs, int32_t* const* accs, bool accumulate, cudaStream_t st,
             const NormQuantParams* fuse = nullptr, int fuse_row = 0, int act_pair = 0, float* act_out = nullptr);
int get_rope_table(ter_b200_handle_t* h, int n_pos, int head_dim, double theta, const float** out);

}  // namespace terb
