/* TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * CPU restatement (plain C) of the reference's ternary matmul fabric and of
 * the single-token decode forward built on it.  Only tests/,
 * __graft_entry__.smoke() and bench.py's CPU-baseline legs may load the
 * library built from this file; the shipped CUDA path never does.
 *
 * Pinning: orc_mm_row / orc_quantize_trit are checked bit-for-bit against the
 * unmodified reference (oracle/_ref/libter_ref.so, built from the reference
 * sources) and against committed fixtures that library produced
 * (tests/golden/); the packed-GEMV and glue restatements are checked against
 * the reference's own known-answer recipes (see tests/test_oracle_pins.py).
 *
 * Every function cites the reference file:line it restates.
 */
#ifndef TER_ORACLE_H
#define TER_ORACLE_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- packed-trit formats (cuda/ter_cuda_packed.cu:32-34, ---------------
 *      cuda/ter_cuda_packed_v3.cu:95-111, tools/convert_llama_to_packed.py:128-140)
 * 2-bit code: 0 -> 0, 1 -> +1, 2 -> -1, 3 -> 0.  trits is [K][N] row-major. */
void orc_pack_v11(const int8_t* trits, int K, int N, uint8_t* out);      /* out [N/4][K] */
void orc_pack_rowmajor(const int8_t* trits, int K, int N, uint8_t* out); /* out [K][N/4] */
void orc_unpack_v11(const uint8_t* in, int K, int N, int8_t* trits);
void orc_unpack_rowmajor(const uint8_t* in, int K, int N, int8_t* trits);

/* ---- CPU GEMV: mm_row (src/tx/forward.cpp:299-352, per-tensor branch) --- */
void orc_mm_row_acc(const int32_t* X, const int32_t* W, int K, int N, int64_t* acc);
void orc_mm_row(const int32_t* X, float x_scale, const int32_t* W, float w_scale,
                int K, int N, float* out);
uint64_t orc_tvmac(int K, int N);   /* src/tx/forward.cpp:349-350 */

/* ---- GPU-path GEMV semantics: mm_packed_v4 (cuda/ter_cuda_forward_packed.cu:346-397)
 * int8 x times v11-packed trits, exact int32 accumulate; fp32 epilogue
 * out = (float)acc * (x_scale * w_scale) (kept in fp32, not rounded to fp16). */
void orc_gemv_packed_v11_acc(const int8_t* x, const uint8_t* Wcol, int K, int N, int32_t* acc);
void orc_gemv_epilogue(const int32_t* acc, int N, float x_scale, float w_scale, float* out);
/* Batched form (cuda/ter_cuda_addonly_batched.cu:32-123): X [M][K], per-row scale. */
void orc_gemm_packed_v11(const int8_t* X, const float* x_scales, int M,
                         const uint8_t* Wcol, float w_scale, int K, int N,
                         int32_t* acc /*[M][N] or NULL*/, float* out /*[M][N]*/);

/* ---- quantisers -------------------------------------------------------- */
/* ter::quantize (src/numfmt/quantize.cpp:7-41): returns scale. */
float orc_quantize_trit(const float* x, int n, int n_trits, int32_t* payload);
/* quant_int8_k (cuda/ter_cuda_forward_packed.cu:40-62). */
void orc_quant_int8(const float* x, int n, int8_t* q, float* scale_out);
/* rmsnorm_quant_*_in_k (cuda/ter_cuda_forward_packed.cu:269-309,
 * cuda/ter_cuda_forward_bitnet.cu:64-146).  normed may be NULL. */
void orc_rmsnorm_quant(const float* x, const float* gamma, int n, float eps,
                       int8_t* q, float* scale_out, float* normed);
/* rmsnorm_f32_in_k (cuda/ter_cuda_forward_bitnet.cu:149-159): no quantisation. */
void orc_rmsnorm(const float* x, const float* gamma, int n, float eps, float* y);
/* silu_mul_quant_k (cuda/ter_cuda_forward_packed.cu:312-344). */
void orc_silu_mul_quant(const float* g, const float* u, int n, int8_t* q, float* scale_out);
/* relu2_mul_rmsnorm_quant_k (cuda/ter_cuda_forward_bitnet.cu:258-309). */
void orc_relu2_mul_rmsnorm_quant(const float* g, const float* u, const float* gamma, int n,
                                 float eps, int8_t* q, float* scale_out);

/* ---- rotary, attention, lm_head, argmax -------------------------------- */
/* cos/sin table [n_pos][head_dim/2][2] with freq = theta^(-2k/head_dim),
 * evaluated in double as the CPU reference does (src/tx/forward.cpp:78-88). */
void orc_rope_table(int n_pos, int head_dim, double theta, float* table);
/* rope_k: neox=0 interleaved pairs (cuda/ter_cuda_forward_packed.cu:64-76),
 * neox=1 half-split pairs (cuda/ter_cuda_forward_bitnet.cu:185-201). */
void orc_rope(float* v, int n_heads, int head_dim, const float* table_row, int neox);
/* attention_k (cuda/ter_cuda_forward_packed.cu:118-157) over a bf16 cache laid
 * out [n_kv][smax][head_dim]; seq_len = pos+1 rows valid.  Softmax evaluated
 * as a 256-position chunked online softmax in a fixed order (see ter_oracle.c). */
void orc_attention(const float* q, const uint16_t* kc, const uint16_t* vc,
                   int n_heads, int n_kv, int head_dim, int smax, int seq_len, float* out);
/* Same result in the reference's two-pass form with double accumulation —
 * used to bound the chunked form (tools/llama_pyfwd.py:116-123). */
void orc_attention_twopass(const float* q, const uint16_t* kc, const uint16_t* vc,
                           int n_heads, int n_kv, int head_dim, int smax, int seq_len, float* out);
/* mm_fp16_lm_head_k (cuda/ter_cuda_forward_packed.cu:165-206) with a bf16 table. */
void orc_lm_head_bf16(const uint16_t* embd, const float* x, int V, int H, float* logits);
/* argmax: lowest index among maxima. */
int orc_argmax(const float* v, int n);

float orc_expf(float x);
uint16_t orc_f32_to_bf16(float f);
float orc_bf16_to_f32(uint16_t h);

/* ---- decode forward (cuda/ter_cuda_forward_packed.cu:505-563,
 *      cuda/ter_cuda_forward_bitnet.cu:850-913; tools/llama_pyfwd.py:103-161,
 *      tools/bitnet_pyfwd.py:94-152) ------------------------------------ */
enum { ORC_ARCH_LLAMA = 0, ORC_ARCH_BITNET = 1 };
enum { ORC_WQ = 0, ORC_WK, ORC_WV, ORC_WO, ORC_WGATE, ORC_WUP, ORC_WDOWN, ORC_NMAT };
enum { ORC_ATTN_NORM = 0, ORC_FFN_NORM, ORC_ATTN_SUB_NORM, ORC_FFN_SUB_NORM, ORC_NVEC };

typedef struct {
    int arch;
    int H, F, L, V, Nh, Nkv, Hd, Smax;
    float eps;
    double rope_theta;
    int lm_head_packed;   /* 1: packed-trit lm_head K=H,N=V; 0: tied bf16 table */
    int kv_f32;           /* 1: keep the KV cache in fp32 (pyfwd-compatible mode) */
    int np_quant;         /* 1: quantise as tools/llama_pyfwd.py:82-86 does
                                (scale = amax/127, q = rint(x/scale)) */
} orc_cfg_t;

typedef struct orc_model orc_model_t;
typedef struct orc_state orc_state_t;

orc_model_t* orc_model_create(const orc_cfg_t* cfg);
void orc_model_destroy(orc_model_t* m);
/* Copies. packed is the v11 layout [N/4][K]. layer = -1 with which = 0 is the packed lm_head. */
int orc_model_set_matrix(orc_model_t* m, int layer, int which, const uint8_t* packed_v11, float scale);
int orc_model_set_vector(orc_model_t* m, int layer, int which, const float* v); /* layer -1: output_norm */
int orc_model_set_embd(orc_model_t* m, const uint16_t* bf16_table);            /* [V][H] */
void orc_model_set_threads(orc_model_t* m, int n_threads);

orc_state_t* orc_state_create(const orc_model_t* m, int batch);
void orc_state_destroy(orc_state_t* s);
/* One decode step for sequence `seq` at position `pos`; writes V logits (may be
 * NULL) and returns the greedy token.  hidden_out (may be NULL) receives the
 * final residual stream. */
int orc_forward_token(const orc_model_t* m, orc_state_t* s, int seq, int token, int pos,
                      float* logits, float* hidden_out);
/* Per-stage taps of the most recent orc_forward_token call on this state:
 * copies the H-vector residual stream after layer `layer`. */
int orc_state_layer_hidden(const orc_state_t* s, int layer, float* out);

#ifdef __cplusplus
}
#endif
#endif
