/* ter_b200 — C ABI of the B200 (sm_100a) ternary matmul fabric and decode forward.
 *
 * The library keeps the conventions of the reference's K4 C interface
 * (include/ter_k4/ter_k4.h:27-55, src/k4/ter_k4.cpp:14-75): an opaque handle,
 * named slots in a fixed-size table with names of at most 31 characters
 * (include/ter/kernels.hpp:21-38), integer return codes (0 ok, -1 null
 * argument, -2 unknown name, -3 allocation failure, -4 more than 7 call
 * arguments), void functions that ignore NULL, and no exception or exit()
 * across the boundary.
 *
 * All `*_dev` pointers are CUDA device pointers on the handle's device;
 * `stream` is a cudaStream_t passed as void* (NULL = the handle's own stream).
 * A handle serves one GPU and is not thread-safe; use one handle per GPU/rank.
 * There is no CPU fallback: every compute entry point runs CUDA kernels or
 * returns an error code.
 */
#ifndef TER_B200_H
#define TER_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct ter_b200_handle_t ter_b200_handle_t;

/* ---- return codes (first four: src/k4/ter_k4.cpp:33,40,52-54) ---- */
#define TER_B200_OK            0
#define TER_B200_E_NULL       (-1)   /* null handle / name / pointer            */
#define TER_B200_E_UNKNOWN    (-2)   /* no slot or operator of that name         */
#define TER_B200_E_ALLOC      (-3)   /* host or device allocation failed         */
#define TER_B200_E_NARGS      (-4)   /* ter_b200_call with more than 7 arguments */
#define TER_B200_E_SHAPE      (-5)   /* unsupported K/N/M, misaligned pointer    */
#define TER_B200_E_FULL       (-6)   /* every slot of the table is in use        */
#define TER_B200_E_NAME       (-7)   /* name longer than 31 characters           */
#define TER_B200_E_CUDA       (-8)   /* a CUDA runtime call failed               */
#define TER_B200_E_NCCL       (-9)   /* an NCCL call failed                      */
#define TER_B200_E_STATE      (-10)  /* call made in the wrong state             */
#define TER_B200_E_TIMEOUT    (-11)  /* a bounded device-side wait ran out       */
#define TER_B200_E_VALUE      (-12)  /* payload value outside {-1,0,+1}          */
#define TER_B200_E_IO         (-13)  /* file missing, short, or not a model file */

/* The reference's KernelTable has 32 slots of 32-character names
 * (include/ter/kernels.hpp:21-38) because it holds five bytecode kernels.  Here a slot holds a
 * weight tensor and one model has 7 per layer, so the fixed table is larger; the name limit and
 * the behaviour on overflow (an error code, never an exception) are the reference's. */
#define TER_B200_MAX_SLOTS     1024
#define TER_B200_MAX_PLANS     16     /* sweep plans per handle */
#define TER_B200_MAX_PLAN_MATS 512    /* matrices in one sweep plan */
#define TER_B200_MAX_NAME      31

const char* ter_b200_strerror(int code);

/* ---- lifecycle: replaces ter_k4_create / ter_k4_destroy
 *      (include/ter_k4/ter_k4.h:29-30).  `device` is the CUDA ordinal. */
ter_b200_handle_t* ter_b200_create(int device);
void               ter_b200_destroy(ter_b200_handle_t* h);

/* ---- weight formats accepted at the boundary ------------------------------
 * V11      bytes [N/4][K], byte (j/4)*K + k, column j in bits 2*(j%4)
 *          (cuda/ter_cuda_forward_packed.cu:354-355,370-372;
 *           tools/convert_llama_to_packed.py:128-140)
 * ROWMAJOR bytes [K][N/4], byte k*(N/4) + j/4 (cuda/ter_cuda_packed.cu:32-34,47-53)
 * I32      TritTensor payload, int32 [K][N] with values in {-1,0,+1}
 *          (include/ter/numfmt.hpp:17-36; W[k*N+j] as mm_row reads it,
 *           src/tx/forward.cpp:338)
 * 2-bit code in both packed forms: 0 -> 0, 1 -> +1, 2 -> -1, 3 -> 0. */
#define TER_B200_FMT_V11       0
#define TER_B200_FMT_ROWMAJOR  1
#define TER_B200_FMT_I32       2

/* Blob header for ter_b200_install_kernel: the payload follows the header. */
typedef struct {
    uint32_t magic;      /* 'TB2W' = 0x54423257 */
    uint32_t format;     /* TER_B200_FMT_* */
    uint32_t K, N;
    float    scale;      /* per-tensor weight scale */
    uint32_t reserved[3];
} ter_b200_blob_hdr_t;
#define TER_B200_BLOB_MAGIC 0x54423257u

/* Same verb and argument list as ter_k4_install_kernel
 * (include/ter_k4/ter_k4.h:33-36): registers a weight tensor under `name`,
 * copying (and re-packing) it to the device once.  blob_n_words counts 32-bit
 * words including the header.  Re-installing an existing name replaces it. */
int ter_b200_install_kernel(ter_b200_handle_t* h, const char* name,
                            const void* blob_bytes, size_t blob_n_words);

/* Typed form of the same operation.  `data` is a HOST pointer. */
int ter_b200_install_weight(ter_b200_handle_t* h, const char* name, const void* data,
                            int format, int K, int N, float scale);
/* `data_dev` is a DEVICE pointer (the weights never visit the host). */
int ter_b200_install_weight_dev(ter_b200_handle_t* h, const char* name, const void* data_dev,
                                int format, int K, int N, float scale, void* stream);
int ter_b200_remove_weight(ter_b200_handle_t* h, const char* name);
int ter_b200_weight_info(const ter_b200_handle_t* h, const char* name, int* K, int* N, float* scale);

/* ---- ter_k4_call (include/ter_k4/ter_k4.h:40-43): run a named operator with
 * at most 7 int64 arguments.  Operator names are the reference's slot names
 * (src/tx/forward.cpp:376-380):
 *   "tk_matmul_b_9t"  args = { (int64)(const char*)weight_slot_name, x_dev, x_scale_dev,
 *                              out_dev, M, stream }            M = 1 -> GEMV, M > 1 -> GEMM
 *   "tk_rmsnorm"      args = { x_dev, gamma_dev, n, rows, eps (float bits), q_dev, scale_dev }
 *                              = ter_b200_rmsnorm_quant on the handle's stream
 *   "tk_silu"         args = { gate_dev, up_dev, n, rows, q_dev, scale_dev [, stream] }
 *                              = ter_b200_act_quant with the SiLU gate
 *   "tk_rope"         args = { q_dev, k_dev, pos_dev, dims, Smax, theta (double bits), neox }
 *                              = ter_b200_rope_kv without the cache append (rotation in place)
 *   "tk_softmax"      args = { q_dev, kcache_dev, vcache_dev, pos_dev, dims, Smax, out_dev }
 *                              = ter_b200_attention_noalloc (on this path the softmax lives inside
 *                                the attention kernel; there is no stand-alone softmax)
 *   dims = B | Nh << 16 | Nkv << 32 | Hd << 48.  Unknown names return TER_B200_E_UNKNOWN, more than
 *   7 arguments TER_B200_E_NARGS, too few TER_B200_E_SHAPE.
 */
int ter_b200_call(ter_b200_handle_t* h, const char* name, const int64_t* args, size_t n_args);

/* ---- op counters (include/ter_k4/ter_k4.h:46-55).  tvmac advances by
 * ceil(K/27)*N per GEMV row, as mm_row accounts it (src/tx/forward.cpp:349-350). */
typedef struct {
    uint64_t total_ops;
    uint64_t tvmac;
    uint64_t tvadd;
    uint64_t tvsub;
    uint64_t tvmul;
} ter_b200_op_counts_t;
void ter_b200_op_counts(const ter_b200_handle_t* h, ter_b200_op_counts_t* out);
void ter_b200_reset_counters(ter_b200_handle_t* h);
/* The report of dump_op_stats (include/ter/tx/op_stats.hpp:86-127) for this handle's counters, written into
 * `buf` (at most buf_len bytes, always terminated): total kernel ops, TVMAC and lane-MACs (TVMAC*27), the
 * analytical fp16 MACs of `n_forwards` forwards of the architecture (Q+K+V+O+gate+up+down per layer + lm_head)
 * and their ratio.  Counters this path never bumps print as 0.  Returns the length the full report needs. */
int ter_b200_dump_op_stats(const ter_b200_handle_t* h, const char* label, int hidden_size, int intermediate_size,
                           int n_heads, int n_kv_heads, int head_dim, int n_layers, int vocab_size, int n_forwards,
                           char* buf, size_t buf_len);
/* Which kernel serves a product of M activation rows with a K x N weight on this handle: the ONE dispatch rule
 * of the library (the reference's pick_kernel(K, N), cuda/ter_cuda_hybrid_dispatch_v13.cu:120-126, extended by
 * the row count).  Returns one of TER_B200_KERNEL_*; ter_b200_kernel_name gives its name. */
#define TER_B200_KERNEL_GEMV_SPLIT   0   /* M = 1, few strips: register-prefetch split-K GEMV (decode projections) */
#define TER_B200_KERNEL_GEMV_STREAM  1   /* M = 1, many strips: persistent TMA-ring GEMV (lm_head, sweeps) */
#define TER_B200_KERNEL_GEMV_ROWS    2   /* 2 <= M < "gemm_min_m" (at most 16): multi-row GEMV, the weights stream once */
#define TER_B200_KERNEL_GEMM_TCGEN05 3   /* M >= "gemm_min_m": tcgen05 kind::i8 GEMM, TMEM accumulators */
#define TER_B200_KERNEL_GEMV_PER_ROW 4   /* otherwise: one GEMV launch per row */
int ter_b200_pick_kernel(const ter_b200_handle_t* h, int M, int K, int N);
const char* ter_b200_kernel_name(int kernel);

/* ---- packed-trit GEMV, M = 1 ------------------------------------------------
 * Replaces mm_packed_dispatch / mm_packed_v4 (cuda/ter_cuda_forward_packed.cu:346-397,
 * 493-500) and mm_bitnet_addonly_dev (cuda/ter_cuda_forward_bitnet.cu:497-559), and
 * computes what mm_row computes (src/tx/forward.cpp:299-352) for int8 X:
 *   out[j] = (float)(sum_k x[k] * trit(k,j)) * (x_scale_dev[0] * w_scale),  exact int32 sum.
 * x_dev: int8[K], 16-byte aligned.  out_dev: float[N]. */
int ter_b200_gemv(ter_b200_handle_t* h, const char* slot, const int8_t* x_dev,
                  const float* x_scale_dev, float* out_dev, void* stream);
/* Raw int32 accumulators (no scale): the bit-exact check against mm_row. */
int ter_b200_gemv_acc(ter_b200_handle_t* h, const char* slot, const int8_t* x_dev,
                      int32_t* acc_dev, void* stream);
/* Up to 4 weight slots with the same K sharing one activation vector in ONE launch
 * (q/k/v: cuda/ter_cuda_forward_packed.cu:516-518; gate/up: :533-534). */
int ter_b200_gemv_group(ter_b200_handle_t* h, const char* const* slots, int n_slots,
                        const int8_t* x_dev, const float* x_scale_dev,
                        float* const* outs_dev, void* stream);
#define TER_B200_ACT_SILU  1
#define TER_B200_ACT_RELU2 2
/* `n` (at most 8) INDEPENDENT GEMVs in one launch: slot i with its own activation vector x_devs[i]
 * (int8[K_i]) and scale x_scale_devs[i]; the K_i may differ.  Same results as n calls of
 * ter_b200_gemv; one grid streams all the weights (the reference's benches time such sweeps one
 * kernel at a time, cuda/ter_cuda_forward_packed_v12.cu:414-464). */
int ter_b200_gemv_multi(ter_b200_handle_t* h, int n, const char* const* slots, const int8_t* const* x_devs,
                        const float* const* x_scale_devs, float* const* outs_dev, void* stream);
/* Sweep plan: up to TER_B200_MAX_PLAN_MATS independent GEMVs (at most 16 distinct (x, scale, K)
 * vectors, 64 KB of x in total) whose descriptors are written to device memory ONCE; every
 * ter_b200_gemv_plan_launch then streams all the matrices in a single launch and reads x / scales /
 * writes outs at the addresses given here.  Installing, replacing or removing ANY weight slot makes
 * existing plans stale: launch returns TER_B200_E_STATE, destroy and re-create them.  The reference
 * issues such sequences one kernel per matrix (cuda/ter_cuda_forward_packed.cu:505-563). */
int ter_b200_gemv_plan_create(ter_b200_handle_t* h, int n, const char* const* slots, const int8_t* const* x_devs,
                              const float* const* x_scale_devs, float* const* outs_dev, int* plan_id);
int ter_b200_gemv_plan_launch(ter_b200_handle_t* h, int plan_id, void* stream);
int ter_b200_gemv_plan_destroy(ter_b200_handle_t* h, int plan_id);
/* Quantiser fused into the GEMV: y = W^T q(x) where q() is exactly ter_b200_rmsnorm_quant (act = 0:
 * RMSNorm with gamma_dev, or plain absmax quantisation when gamma_dev is NULL) or ter_b200_act_quant
 * (act = TER_B200_ACT_SILU / _RELU2 with up_dev, optional sub-norm gamma_dev) applied to the fp32 vector
 * x_dev[K].  One launch replaces the reference's rmsnorm_quant / silu_mul_quant kernel plus the
 * GEMVs that consume its output (cuda/ter_cuda_forward_packed.cu:514-518,531-536); every CTA derives
 * the int8 vector itself, in the same fixed reduction order, so results are bit-identical to the
 * two-step form.  accumulate != 0 adds into outs (the residual add, add_k, :529,:538).  Only for
 * slot groups of at most 1184 strips (N total <= 18944), i.e. every projection but the lm_head. */
int ter_b200_norm_gemv_group(ter_b200_handle_t* h, const char* const* slots, int n_slots, int act,
                             const float* x_dev, const float* up_dev, const float* gamma_dev, float eps,
                             float* const* outs_dev, int accumulate, void* stream);
/* Host-buffer form: copies x (K bytes) and the scale in, the N floats out, on `stream`,
 * asynchronously; ter_b200_sync() completes it.  Buffers must stay valid until then
 * (pinned host memory makes the copies truly asynchronous). */
int ter_b200_gemv_host(ter_b200_handle_t* h, const char* slot, const int8_t* x_host,
                       float x_scale, float* out_host, void* stream);
/* The same for `n` GEMVs in one call (e.g. every projection of a model): slots[i], x_hosts[i]
 * (int8[K_i]), x_scales[i], out_hosts[i] (float[N_i]).  SYNCHRONOUS: the results are in out_hosts when
 * it returns.  Vectors given with the same pointer, scale and K travel once; all inputs go up in one
 * copy; the GEMVs run as one launch (more only past 512 matrices, 16 distinct vectors or 64 KB of x);
 * outputs that lie back to back in host memory, in call order, form a run: a run in pinned host memory
 * is written by the kernel itself while it streams the weights (option "host_batch_direct", default
 * 1), any other run comes down in one copy. */
int ter_b200_gemv_host_batch(ter_b200_handle_t* h, int n, const char* const* slots, const int8_t* const* x_hosts,
                             const float* x_scales, float* const* out_hosts, void* stream);
int ter_b200_sync(ter_b200_handle_t* h, void* stream);

/* ---- batched ternary GEMM, M > 1 -------------------------------------------
 * Replaces mm_bitnet_addonly_batched_k (cuda/ter_cuda_addonly_batched.cu:32-123) and
 * mm_int4_tc* (cuda/ter_cuda_int4_tc.cu:36-82): X int8 [M][K] row-major, one scale per
 * row, out float [M][N]; out[m][j] = (float)acc * (x_scales[m] * w_scale). */
int ter_b200_gemm(ter_b200_handle_t* h, const char* slot, const int8_t* X_dev,
                  const float* x_scales_dev, int M, float* out_dev, void* stream);
int ter_b200_gemm_acc(ter_b200_handle_t* h, const char* slot, const int8_t* X_dev, int M,
                      int32_t* acc_dev, void* stream);

/* ---- decode glue operators -------------------------------------------------
 * All activations are fp32 device arrays; `rows`/`B` is the number of sequences.
 *
 * RMSNorm + absmax int8 quantisation: replaces rmsnorm_quant_fp16_in_k / rmsnorm_quant_f32_in_k
 * (cuda/ter_cuda_forward_packed.cu:269-309, cuda/ter_cuda_forward_bitnet.cu:64-146):
 *   n_i = (x_i * (1/sqrt(mean(x^2)+eps))) * gamma_i ; amax = max|n| + 1e-9 ; s = 127/amax ;
 *   q_i = clamp(rint(n_i*s), -128, 127) ; scale[row] = 1/s.
 * gamma_dev NULL: no normalisation = quant_int8_k (cuda/ter_cuda_forward_packed.cu:40-62).
 * q_dev NULL with normed_dev set: RMSNorm only = rmsnorm_f32_in_k (cuda/ter_cuda_forward_bitnet.cu:149-159).
 * normed_dev (optional) receives the fp32 values that were quantised. */
int ter_b200_rmsnorm_quant(ter_b200_handle_t* h, const float* x_dev, const float* gamma_dev, int n, int rows,
                           float eps, int8_t* q_dev, float* scale_dev, float* normed_dev, void* stream);
/* Gated activation + quantisation.  act = SILU: silu_mul_quant_k
 * (cuda/ter_cuda_forward_packed.cu:312-344), v = gate/(1+exp(-gate))*up.  act = RELU2:
 * relu2_mul_rmsnorm_quant_k (cuda/ter_cuda_forward_bitnet.cu:258-309), v = max(gate,0)^2*up followed by
 * RMSNorm with gamma_dev (the ffn sub-norm) when gamma_dev is not NULL. */
int ter_b200_act_quant(ter_b200_handle_t* h, int act, const float* gate_dev, const float* up_dev,
                       const float* gamma_dev, int n, int rows, float eps, int8_t* q_dev, float* scale_dev,
                       void* stream);
/* Rotary embedding in place on q [B][Nh*Hd] and k [B][Nkv*Hd] at position pos_dev[b], then append of
 * k and v, rounded to bf16, to one layer's cache laid out [B][Nkv][Smax][Hd]: rope_k + kv_copy_k
 * (cuda/ter_cuda_forward_packed.cu:64-90).  neox = 0: pairs (2k,2k+1); neox = 1: pairs (k,k+Hd/2)
 * (cuda/ter_cuda_forward_bitnet.cu:185-201).  Angles pos*theta^(-2k/Hd) come from a table evaluated
 * in double on the host (src/tx/forward.cpp:78-88). */
/* v_dev, kcache_dev and vcache_dev may all be NULL: rotation only, nothing appended. */
int ter_b200_rope_kv(ter_b200_handle_t* h, float* q_dev, float* k_dev, const float* v_dev, const int* pos_dev,
                     int B, int Nh, int Nkv, int Hd, int Smax, double theta, int neox, uint16_t* kcache_dev,
                     uint16_t* vcache_dev, void* stream);
/* Causal GQA attention of one new token per sequence over the bf16 cache, seq_len = pos_dev[b]+1:
 * attention_k (cuda/ter_cuda_forward_packed.cu:118-157), kv head = h*Nkv/Nh, scores/sqrt(Hd),
 * max-subtracted softmax, sum p*V; evaluated as a split-KV online softmax over chunks of 256
 * positions.  scratch_dev: ter_b200_attention_scratch_floats() floats of device memory that the
 * call may overwrite.  Hd in {64,128}; Nh/Nkv <= 8. */
size_t ter_b200_attention_scratch_floats(int B, int Nh, int Hd, int Smax);
int ter_b200_attention(ter_b200_handle_t* h, const float* q_dev, const uint16_t* kcache_dev,
                       const uint16_t* vcache_dev, const int* pos_dev, int B, int Nh, int Nkv, int Hd, int Smax,
                       float* scratch_dev, size_t scratch_floats, float* out_dev, void* stream);
/* The same attention for callers that cannot allocate device memory where they need it: code
 * between cudaStreamBeginCapture and cudaStreamEndCapture, a decode loop that gave all of its
 * memory out at start-up, a host whose allocator belongs to another runtime.  (No counterpart in
 * the reference, which allocates its scratch once in alloc_scratch.)  The partial records go to
 * a fixed 4 MiB array inside the library's device image instead of a caller buffer; every GPU
 * that loads the library holds that array until the process exits.  Calls whose records do not
 * fit -- ter_b200_attention_scratch_floats(B, Nh, Hd, Smax) > ter_b200_attention_noalloc_max_floats()
 * -- return TER_B200_E_SHAPE.  The call itself makes no cudaMalloc / cudaFree.  The first call on
 * a device looks the array's address up (cudaGetSymbolAddress); make that call before any stream
 * capture.  All calls on a device share the one array and it keeps whatever the last call left:
 * nothing in it needs clearing (every record that is read is written first by the same call), but
 * two calls that overlap on the GPU (different streams) race on it -- serialise them. */
size_t ter_b200_attention_noalloc_max_floats(void);
int ter_b200_attention_noalloc(ter_b200_handle_t* h, const float* q_dev, const uint16_t* kcache_dev,
                               const uint16_t* vcache_dev, const int* pos_dev, int B, int Nh, int Nkv, int Hd,
                               int Smax, float* out_dev, void* stream);
/* logits[b][v] = sum_h bf16(table[v][h]) * x[b][h]: mm_fp16_lm_head_k
 * (cuda/ter_cuda_forward_packed.cu:165-206) with a bf16 table and fp32 activations. */
int ter_b200_lm_head_bf16(ter_b200_handle_t* h, const uint16_t* table_dev, const float* x_dev, float* logits_dev,
                          int V, int H, int B, void* stream);
/* The same product for token batches (B >= 16 is where it pays) on the tensor cores: tcgen05 kind::f16 with the
 * fp32 activations split into two bf16 parts and fp32 accumulators in tensor memory.  Equal to
 * ter_b200_lm_head_bf16 up to rounding (about 1e-6 relative; the summation order differs), not bit for bit.
 * H a multiple of 64; scratch_dev: ter_b200_lm_head_tc_scratch_bytes(B, H) bytes, 16-byte aligned. */
int ter_b200_lm_head_bf16_tc(ter_b200_handle_t* h, const uint16_t* table_dev, const float* x_dev, float* logits_dev,
                             int V, int H, int B, void* scratch_dev, size_t scratch_bytes, void* stream);
size_t ter_b200_lm_head_tc_scratch_bytes(int B, int H);
/* out[b] = lowest index among the maxima of logits[b][0..V): argmax_local_k + argmax_final_k
 * (cuda/ter_cuda_forward_packed.cu:209-241).  scratch_dev: B*256 floats. */
int ter_b200_argmax(ter_b200_handle_t* h, const float* logits_dev, int V, int B, float* scratch_dev, int* out_dev,
                    void* stream);

/* ---- decode forward -----------------------------------------------------------
 * One model per handle.  Replaces the Model/Scratch structs and forward_token_dev of the reference's
 * CUDA forwards (cuda/ter_cuda_forward_packed.cu:399-421,505-563; cuda/ter_cuda_forward_bitnet.cu:850-913)
 * and, on the CPU side, forward_token (src/tx/transformer.cpp:116-223).  arch 0 = Llama (interleaved
 * rotary, SiLU gate, plain absmax quantisation before Wo); arch 1 = BitNet (NEOX rotary, ReLU^2 gate,
 * attn_sub_norm / ffn_sub_norm).  Residual stream fp32, KV cache bf16, embeddings bf16. */
typedef struct {
    int32_t arch;
    int32_t H, F, L, V, Nh, Nkv, Hd, Smax;
    float   eps;
    double  rope_theta;
    int32_t lm_head_packed;   /* 1: packed-trit lm_head (K=H, N=V); 0: bf16 table tied to the embeddings */
    int32_t max_batch;        /* sequences decoded together (KV cache is allocated for this many) */
} ter_b200_model_cfg_t;
#define TER_B200_ARCH_LLAMA  0
#define TER_B200_ARCH_BITNET 1
/* matrices of a layer, in the order of the packed-model files (tools/convert_llama_to_packed.py:13-43) */
enum { TER_B200_WQ = 0, TER_B200_WK, TER_B200_WV, TER_B200_WO, TER_B200_WGATE, TER_B200_WUP, TER_B200_WDOWN };
enum { TER_B200_ATTN_NORM = 0, TER_B200_FFN_NORM, TER_B200_ATTN_SUB_NORM, TER_B200_FFN_SUB_NORM };

int ter_b200_model_create(ter_b200_handle_t* h, const ter_b200_model_cfg_t* cfg);
/* data: HOST pointer in a TER_B200_FMT_* format; layer = -1 installs the packed lm_head. */
int ter_b200_model_set_matrix(ter_b200_handle_t* h, int layer, int which, const void* data, int format, float scale);
int ter_b200_model_set_matrix_dev(ter_b200_handle_t* h, int layer, int which, const void* data_dev, int format,
                                  float scale);
/* v: HOST fp32 vector; layer = -1 installs output_norm. */
int ter_b200_model_set_vector(ter_b200_handle_t* h, int layer, int which, const float* v);
/* bf16 [V][H] embedding table (also the lm_head when lm_head_packed = 0): host / device pointer. */
int ter_b200_model_set_embd(ter_b200_handle_t* h, const uint16_t* table);
int ter_b200_model_set_embd_dev(ter_b200_handle_t* h, const uint16_t* table_dev);
/* Start `batch` sequences at position 0 (the KV cache content is simply overwritten as they grow). */
/* Creates the model from one of the reference's packed-model files and fills it: 'LLRT'
 * (tools/convert_llama_to_packed.py:13-43; the reference reads it in load_model_from_bin,
 * cuda/ter_cuda_forward_packed.cu:589-667) or 'TERT' (tools/convert_bitnet_to_packed.py:4-31,
 * cuda/ter_cuda_forward_bitnet.cu:698-784).  smax > 0 overrides the file's context length (the
 * reference's files say 64), max_batch as in the cfg.  The fp16 embeddings of the file are rounded
 * to bf16.  cfg_out (may be NULL) receives the configuration.  Errors are return codes
 * (TER_B200_E_IO for a missing / short / foreign file); nothing exits the process.
 * ter_b200_model_file_info only reads the header and needs no handle and no GPU. */
int ter_b200_model_load_file(ter_b200_handle_t* h, const char* path, int smax, int max_batch,
                             ter_b200_model_cfg_t* cfg_out);
int ter_b200_model_file_info(const char* path, ter_b200_model_cfg_t* cfg_out);
/* microsoft/BitNet GGUF "i2_s" tensor (N output rows x K inputs, 128-element blocks of 32 bytes, the scale in
 * the 32 bytes after the codes) -> TER_B200_FMT_V11 bytes [N/4][K] and the per-tensor scale: the conversion of
 * tools/convert_bitnet_to_packed.py:85-152 (read_i2s_scale, i2s_to_col_packed; decode as in
 * vendor/ntransformer/core/dequant.cpp:114-145).  i2s_bytes: bytes available at `i2s` (codes + trailer).
 * Host memory only: needs no handle and no GPU.  scale_out may be NULL. */
int ter_b200_convert_i2s(const void* i2s, size_t i2s_bytes, int N, int K, uint8_t* v11_out, float* scale_out);
int ter_b200_model_reset(ter_b200_handle_t* h, int batch);
/* One decode step for every sequence: forward_token (cuda/ter_cuda_forward_packed.cu:671-678).
 * tokens_host / pos_host ([batch], may be NULL: continue from the device-resident state, i.e. the
 * greedy token and position left by the previous step).  next_host ([batch], may be NULL) receives
 * the greedy next tokens after a stream synchronisation. */
int ter_b200_decode_step(ter_b200_handle_t* h, const int32_t* tokens_host, const int32_t* pos_host,
                         int32_t* next_host, void* stream);
/* Copies of the state of the latest step: logits [batch][V], residual stream [batch][H]. */
int ter_b200_model_logits(ter_b200_handle_t* h, float* logits_host);
int ter_b200_model_hidden(ter_b200_handle_t* h, float* hidden_host);
/* Greedy generation: feeds `n_prompt` prompt tokens per sequence one position at a time (the
 * reference's only prefill method, cuda/ter_cuda_forward_packed.cu:706-712) and then `n_gen` greedy
 * tokens, replaying ONE captured CUDA graph per step with no host round trip in between.
 * prompts [batch][n_prompt], out [batch][n_gen]. */
int ter_b200_generate(ter_b200_handle_t* h, const int32_t* prompts, int batch, int n_prompt, int n_gen,
                      int32_t* out_tokens, void* stream);
/* Milliseconds the device spent in the latest ter_b200_generate call (CUDA events), and the part of
 * it spent on the prompt when the prompt was run as token batches (0 otherwise).  With option
 * "prefill" 1 (default) a single sequence's prompt of 2 or more tokens goes through the layers in
 * passes of up to 1024 positions (option "prefill_tile") on the tensor-core GEMM with causal attention
 * over the shared cache;
 * cache, position and tokens come out exactly as from feeding it one position at a time, which is
 * what the reference does (cuda/ter_cuda_forward_packed.cu:729-747) and what option 0 does. */
float ter_b200_last_generate_ms(const ter_b200_handle_t* h);
float ter_b200_last_prefill_ms(const ter_b200_handle_t* h);
/* Device milliseconds of the latest ter_b200_generate call up to (not including) the first step that
 * produces a generated token beyond the first, i.e. the prompt phase, whichever way it ran. */
float ter_b200_last_prompt_ms(const ter_b200_handle_t* h);

/* ---- tensor parallelism (no counterpart in the reference, which is single-GPU) -------------
 * One process per GPU, one handle per process.  Rank 0 creates a 128-byte id and hands it to the
 * other ranks by any host channel; every rank then calls ter_b200_comm_init BEFORE
 * ter_b200_model_create.  With a communicator of size G the model keeps columns
 * [N*r/G, N*(r+1)/G) of every SHARDED projection (output-dimension sharding: each output column is
 * an independent exact dot product; option "tp_shard" says which blocks), the vocabulary rows
 * [V*r/G, V*(r+1)/G) of the lm_head, and
 * exchanges the fp32 output slices inside the captured step, so every rank holds the same bits as a
 * single GPU would and greedy tokens are identical at every G.  The exchange is a kernel of peer
 * stores over NVLink into buffers that every rank has mapped (CUDA IPC; NCCL only carries the
 * set-up), or NCCL all-gathers when the GPUs have no peer access or option "tp_p2p" is 0.
 * ter_b200_model_create, the destruction of a model and ter_b200_generate are then COLLECTIVE: every
 * rank makes the same calls in the same order.  A rank that stops arriving makes the others' waits
 * run out after 2 s (TER_B200_E_TIMEOUT), not hang.  Requirements: at most 8 ranks, N/G a multiple
 * of 16 for every projection, matrices given in TER_B200_FMT_V11. */
int ter_b200_comm_unique_id(uint8_t* id128);
int ter_b200_comm_init(ter_b200_handle_t* h, const uint8_t* id128, int rank, int size);
void ter_b200_comm_destroy(ter_b200_handle_t* h);
int ter_b200_comm_rank(const ter_b200_handle_t* h);
int ter_b200_comm_size(const ter_b200_handle_t* h);

/* ---- CUDA graphs ------------------------------------------------------------
 * Record every launch made through this handle on `stream` between begin and end into a
 * CUDA graph and replay it with one call, as the reference's decode loop does
 * (cuda/ter_cuda_forward_packed.cu:729-747).  Up to 16 graphs per handle. */
int ter_b200_capture_begin(ter_b200_handle_t* h, void* stream);
int ter_b200_capture_end(ter_b200_handle_t* h, void* stream, int* graph_id);
int ter_b200_graph_launch(ter_b200_handle_t* h, int graph_id, void* stream);
int ter_b200_graph_destroy(ter_b200_handle_t* h, int graph_id);

/* ---- device status ---------------------------------------------------------
 * Kernels never spin without a bound; a wait that ran out records a code that this call
 * returns (TER_B200_E_TIMEOUT) after synchronising the handle's streams. */
int ter_b200_device_status(ter_b200_handle_t* h);
/* Self-test of the bounded waits (no counterpart in the reference): runs the tensor-parallel exchange kernel
 * on this one GPU against a stand-in peer that never sends.  The wait runs out after option "wait_ms", the
 * kernel returns, and the next ter_b200_device_status reports TER_B200_E_TIMEOUT once.  Returns 0 when the
 * kernel came back by itself. */
int ter_b200_selftest_exchange_timeout(ter_b200_handle_t* h);
/* Last CUDA error code seen by the handle (cudaError_t as int), 0 if none. */
int ter_b200_last_cuda_error(const ter_b200_handle_t* h);
/* Tuning knobs (integers): "gemv_ctas_per_sm", "gemv_stages", "gemv_split_max_strips", "pdl",
 * "fuse_quant", "gemm_min_m" (rows from which the tcgen05 GEMM runs, default 9; 2..8 rows take the multi-row GEMV),
 * "gemm_split_k", "attn_inline_merge", "prefill", "prefill_tile", "host_batch_direct",
 * "decode_persistent" (1, default: one sequence runs the embedding and all layers of a step in one persistent kernel),
 * "decode_poll_ns" (pause between polls inside that kernel, default 0), "decode_fault_cta" (test hook, -1 = off: that
 * CTA keeps its q/k/v columns of layer 0 to itself so that its consumers' waits run out), "wait_ms" (limit of a
 * device-side wait on another CTA or GPU, default 2000), "lm_head_tc_min" (batch size from which the bf16 lm_head runs
 * on the tensor cores, default 16, 0 = never), "attn_mma_min" (rows, i.e. sequences of a batch or positions of a
 * prompt tile, from which attention sums its two contractions on the tensor cores; default 0 = never, because the
 * result then differs from the fixed-order kernel in the last places and, after the int8 quantisers of the following
 * layers, in some greedy tokens of a long generation; about 1.4x on a 64-sequence step at context 2048), "tp_p2p" (1, default: tensor-
 * parallel output slices travel by peer stores over NVLink inside one small kernel per exchange;
 * 0: NCCL all-gathers) and "tp_shard" (which blocks of a layer are column-sharded over the ranks:
 * bit 0 the attention block q/k/v/o, bit 1 the FFN block gate/up/down; the lm_head always is.
 * Default 0: at batch 1 a layer is bound by kernel-to-kernel latency, so sharding it only adds two
 * exchanges per block; 3 shards everything).  Both are read by the next ter_b200_model_create.
 * Returns -2 if unknown. */
int ter_b200_set_option(ter_b200_handle_t* h, const char* key, int value);
/* Number of kernels this handle has launched since creation (or the last reset). */
uint64_t ter_b200_launch_count(const ter_b200_handle_t* h);

#ifdef __cplusplus
}
#endif
#endif /* TER_B200_H */
