// Host-side declarations of the decode glue launchers (glue_sm100.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace terb {

enum PreOp : int { PRE_NONE = 0, PRE_SILU_MUL = 1, PRE_RELU2_MUL = 2 };

// v = pre(x, u) ; optional RMSNorm(gamma, eps) ; optional absmax int8 quantisation.
// Row r of a batch of `rows` uses x + r*n (and u, q, normed likewise), scale_out[r].
struct NormQuantParams {
    const float* x;        // [rows][n]  (gate for the SILU/RELU2 pre-ops)
    const float* u;        // [rows][n]  up-projection, or null
    const float* gamma;    // [n] or null (no normalisation)
    int8_t* q;             // [rows][n] or null (no quantisation)
    float* scale_out;      // [rows]
    float* normed;         // [rows][n] or null: the fp32 values before quantisation
    int n, rows, pre;
    float eps;
    int32_t* rowsum_out;   // [rows] or null: sum of the int8 values of each row (what the tensor-core GEMM
                           // subtracts; stand-alone kernel only, n a multiple of 16)
};
cudaError_t launch_norm_quant(const NormQuantParams& p, bool pdl, cudaStream_t st);

// Rotary embedding of q [B][Nh*Hd] and k [B][Nkv*Hd] in place at position pos[b], then
// append of k, v (rounded to bf16) to the cache of one layer, laid out
// [B][Nkv][Smax][Hd].  table: [Smax][Hd/2][2] (cos, sin).
struct RopeKvParams {
    float* q;
    float* k;
    const float* v;
    const float* table;
    const int* pos;        // [B] device
    uint16_t* kcache;
    uint16_t* vcache;
    int B, Nh, Nkv, Hd, Smax, neox;
    int shared_seq;        // 0: row b belongs to sequence b; s > 0: every row belongs to sequence s - 1 (prompt rows)
};
cudaError_t launch_rope_kv(const RopeKvParams& p, bool pdl, cudaStream_t st);

constexpr int kAttnChunk = 256;
// Partial record per (b, head, chunk): m, l, o[Hd]  -> Hd + 2 floats.
struct AttnParams {
    const float* q;          // [B][Nh*Hd] (after rotary)
    const uint16_t* kcache;  // [B][Nkv][Smax][Hd] bf16
    const uint16_t* vcache;
    const int* pos;          // [B]: seq_len = pos[b] + 1
    float* scratch;          // [B][Nh][max_chunks][Hd+2]
    float* out;              // [B][Nh*Hd]
    int B, Nh, Nkv, Hd, Smax, max_chunks;
    // Fused rotary + KV append (all null/0 when q is already rotated and the cache already appended):
    const float* rope_table; // [Smax][Hd/2][2]
    const float* k_new;      // [B][Nkv*Hd] un-rotated k of the new position
    const float* v_new;      // [B][Nkv*Hd]
    uint16_t* kcache_w;      // same buffers as kcache / vcache, writable
    uint16_t* vcache_w;
    int neox;
    int* status;             // device status word for bounded waits (may be null)
    int* counters;           // [B][Nkv] arrival counters, zero between steps: the last CTA of a KV head merges
                             // the chunks itself (no second kernel); null = merge in attn_combine_kernel
    int shared_seq;          // 0: row b reads the cache of sequence b; s > 0: every row reads sequence s - 1
                             // (the rows are positions of one prompt, each with its own pos[b])
    int kv_div;              // 0 / 1: Nkv counts the KV heads.  d > 1: the query heads of a KV head are dealt to d items
                             // (Nkv = d x the KV heads, Nh / Nkv query heads per item; item g reads KV head g / d): more,
                             // shorter items for a lone sequence whose items do not fill the SMs
    int mma;                 // 1: the two contractions on the tensor cores (attn_mma.cuh): equal to the fixed-order
                             // kernel up to the rounding of fp32 sums, not bit for bit; for token batches
};
cudaError_t launch_attention(const AttnParams& p, bool pdl, cudaStream_t st);
size_t attention_scratch_floats(int B, int Nh, int Hd, int Smax);

// logits[b][v] = sum_h bf16(table[v][h]) * x[b][h], fp32 accumulate.
cudaError_t launch_lm_head_bf16(const uint16_t* table, const float* x, float* logits, int V, int H, int B,
                                int sm_count, bool pdl, cudaStream_t st);
// The same product on the tensor cores (tcgen05 kind::f16) for B >= 16 rows: x is split into two bf16 parts, the
// accumulators are fp32; equal to the exact kernel up to rounding (about 1e-6 relative), not bit for bit.
// scratch: lm_head_tc_scratch_bytes(B, H) bytes of device memory, 16-byte aligned; H a multiple of 64.
size_t lm_head_tc_scratch_bytes(int B, int H);
cudaError_t launch_lm_head_tc(const uint16_t* table, const float* x, float* logits, int V, int H, int B, void* scratch,
                              int* status, bool pdl, cudaStream_t st);
// out[b] = lowest index among the maxima of logits[b][0..V).  scratch: [B][kArgmaxParts][2] floats.
constexpr int kArgmaxParts = 128;
cudaError_t launch_argmax(const float* logits, int V, int B, float* scratch, int* out, bool pdl, cudaStream_t st);
// hidden[b][:] = float(table[token[b]][:])
cudaError_t launch_embed(const uint16_t* table, const int* tokens, float* hidden, int H, int B, int V, bool pdl,
                         cudaStream_t st);
// x[i] += y[i]
cudaError_t launch_add(float* x, const float* y, size_t n, bool pdl, cudaStream_t st);
// pos[b] += 1
cudaError_t launch_inc(int* pos, int B, bool pdl, cudaStream_t st);
// End of a decode step: next token = forced[b][pos+1] while pos+1 < ctl[0] (prompt feeding), else the
// greedy token; logged to log[b][pos] when pos < ctl[1]; pos += 1.  ctl = {n_forced, log_len} on device.
struct SelectParams {
    const int* greedy;   // [B]
    const int* forced;   // [B][forced_stride] or null
    int* tokens;         // [B]
    int* pos;            // [B]
    int* log;            // [B][log_stride] or null
    const int* ctl;
    int B, forced_stride, log_stride;
    unsigned* step_word;  // or null: the step number of the persistent decode kernel, advanced by this last kernel of the step
};
cudaError_t launch_select(const SelectParams& p, bool pdl, cudaStream_t st);

// Tensor-parallel exchange of output slices over peer memory (exchange_sm100.cu).  base[r] = rank r's
// arena as mapped in THIS process (base[rank] = the local one).  A segment is one exchanged buffer:
// seg_buf_off = byte offset of the FULL buffer in the arena, seg_floats = floats per rank slice (rank
// r's slice starts at float r*seg_floats).  recv_off: byte offset of this point's TWO receive blocks,
// uint4[2][size][words_total] (used in turn by sequence parity); seq: this point's int[kMaxExchangeCtas]
// sequence words (local).  wait_ns: limit of a wait for a peer's word.
constexpr int kMaxRanks = 8;
constexpr int kMaxExchangeSegs = 3;
constexpr int kMaxExchangePoints = 512;
constexpr int kMaxExchangeCtas = 64;
struct ExchangeParams {
    uint8_t* base[kMaxRanks];
    size_t seg_buf_off[kMaxExchangeSegs];
    int seg_floats[kMaxExchangeSegs];
    int n_seg, words_total;
    int rank, size;
    size_t recv_off;
    int* seq;
    int* status;
    int point;
    unsigned long long wait_ns;
};
cudaError_t launch_peer_exchange(const ExchangeParams& p, bool pdl, cudaStream_t st);

}  // namespace terb
