// Peer exchange: the all-gather of tensor-parallel decode as ONE small kernel over NVLink peer memory.
//
// Every rank holds the exchanged activation buffers (q, k, v, residual stream, FFN intermediate,
// logits) and a receive area at the same offsets of an "arena" that its peers have mapped (CUDA IPC).
// The messages are 1-64 KB and their cost is pure latency, so the kernel uses flag-in-data words: a
// sender packs two floats with the sequence number of the exchange into one 16-byte word
// {v0, seq, v1, seq} and stores it straight into every peer's receive area; a receiver polls each
// word until both halves carry the expected number and copies the floats into its full-size buffer.
// Each 8-byte half validates itself, so no fence, no separate flag and no second round trip is
// needed: one NVLink crossing per exchange.  A point owns TWO receive blocks, used in turn by sequence
// parity: a rank that has everything it needs may run ahead and start execution n+1 of the point while a
// peer still reads the words of execution n, so n+1 must not land on them.  It cannot reach n+2 (the
// block of n again) before that peer has sent its own n+1 slice, which the peer does only after it has
// finished reading n.  Sequence numbers only grow (one per execution of an
// exchange point, kept per CTA in device memory), every point has its own receive block, nothing
// is ever reset, and a replayed CUDA graph needs no new arguments.  The reference has no multi-GPU
// code; this stands where ncclAllGather calls would.
//
// Bounded wait: a peer that never arrives makes the kernel record a status code and return after
// the limit it is given (handle option "wait_ms"); the context stays usable and the host reads TER_B200_E_TIMEOUT from the status word.
#include "common.cuh"
#include "glue.h"
#include "tagged.cuh"

namespace terb {

namespace {

constexpr int kXThreads = 256;

__global__ void __launch_bounds__(kXThreads) peer_exchange_kernel(const __grid_constant__ ExchangeParams p) {
    const int tid = threadIdx.x;
    int* my_seq = p.seq + blockIdx.x;
    pdl_launch_dependents();
    pdl_wait();   // this rank's slices are complete, and so is the previous execution of this point
    const uint32_t seq = (uint32_t)(*my_seq) + 1u;   // written by this CTA of the previous execution only

    const int words_total = p.words_total;           // 16-byte words per rank for this point
    uint8_t* my_base = p.base[p.rank];
    // this execution's receive block (two per point, by sequence parity)
    const size_t recv_off = p.recv_off + (size_t)(seq & 1u) * (size_t)words_total * 16u * (size_t)p.size;
    bool timed_out = false;
    for (int w = blockIdx.x * kXThreads + tid; w < words_total; w += gridDim.x * kXThreads) {
        // which segment, which pair of floats
        int s = 0, idx = w;
        while (s + 1 < p.n_seg && idx >= p.seg_floats[s] / 2) { idx -= p.seg_floats[s] / 2; ++s; }
        const int slice = p.seg_floats[s];
        float* full = reinterpret_cast<float*>(my_base + p.seg_buf_off[s]);
        const float2 v = *reinterpret_cast<const float2*>(full + (size_t)p.rank * slice + 2 * idx);
        const uint4 word = make_uint4(__float_as_uint(v.x), seq, __float_as_uint(v.y), seq);
        for (int r = 0; r < p.size; ++r)
            if (r != p.rank)
                st_volatile16(reinterpret_cast<uint4*>(p.base[r] + recv_off) + (size_t)p.rank * words_total + w, word);
    }
    for (int w = blockIdx.x * kXThreads + tid; w < words_total; w += gridDim.x * kXThreads) {
        int s = 0, idx = w;
        while (s + 1 < p.n_seg && idx >= p.seg_floats[s] / 2) { idx -= p.seg_floats[s] / 2; ++s; }
        const int slice = p.seg_floats[s];
        float* full = reinterpret_cast<float*>(my_base + p.seg_buf_off[s]);
        for (int r = 0; r < p.size; ++r) {
            if (r == p.rank) continue;
            const uint4* src = reinterpret_cast<const uint4*>(my_base + recv_off) + (size_t)r * words_total + w;
            uint4 got = ld_volatile16(src);
            if (got.y != seq || got.w != seq) {
                const unsigned long long t0 = globaltimer_ns();
                unsigned spins = 0;
                while (!timed_out) {
                    got = ld_volatile16(src);
                    if (got.y == seq && got.w == seq) break;
                    if ((++spins & 255u) == 0 && globaltimer_ns() - t0 > p.wait_ns) {
                        atomicExch(p.status, 0x7e000000 | (p.point << 8) | r);   // which point, which peer
                        timed_out = true;
                    }
                }
            }
            *reinterpret_cast<float2*>(full + (size_t)r * slice + 2 * idx) =
                make_float2(__uint_as_float(got.x), __uint_as_float(got.z));
        }
    }
    __syncthreads();
    if (tid == 0) *my_seq = (int)seq;
}

}  // namespace

int peer_exchange_grid(int words_total) {
    int grid = (words_total + kXThreads - 1) / kXThreads;
    if (grid < 1) grid = 1;
    if (grid > kMaxExchangeCtas) grid = kMaxExchangeCtas;
    return grid;
}

cudaError_t launch_peer_exchange(const ExchangeParams& p, bool pdl, cudaStream_t st) {
    if (p.size < 2 || p.size > kMaxRanks || p.n_seg < 1 || p.n_seg > kMaxExchangeSegs) return cudaErrorInvalidValue;
    int words = 0;
    for (int s = 0; s < p.n_seg; ++s) {
        if (p.seg_floats[s] < 2 || (p.seg_floats[s] & 1) || (p.seg_buf_off[s] & 7u)) return cudaErrorInvalidValue;
        words += p.seg_floats[s] / 2;
    }
    if (words != p.words_total || (p.recv_off & 15u)) return cudaErrorInvalidValue;
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3((unsigned)peer_exchange_grid(words));
    lc.blockDim = dim3(kXThreads);
    lc.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = attr;
    lc.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&lc, peer_exchange_kernel, p);
}

}  // namespace terb
