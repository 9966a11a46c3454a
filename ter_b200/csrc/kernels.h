// Host-side declarations of the kernel launchers (implemented in the .cu files).
// Every launcher returns a cudaError_t and launches on the given stream.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "glue.h"

namespace terb {

// ---- internal weight layout -------------------------------------------------
// A "strip" is 16 output columns = 4 byte-columns of the reference's v11 arrangement
// (byte-column jb holds columns 4*jb..4*jb+3, cuda/ter_cuda_forward_packed.cu:354-355)
// over all of K.  A strip is stored as consecutive "blocks": block q covers
// k in [q*kGemvKC, min((q+1)*kGemvKC, Kpad)) and is the contiguous byte array
// [4 byte-columns][kc], so one 1-D TMA bulk copy fetches one block.  Also:
//   * the 2-bit field is re-coded to u = trit + 1 (0 -> -1, 1 -> 0, 2 -> +1), so that a
//     masked word is directly an unsigned dp4a operand,
//   * K is padded to a multiple of 128 with u = 1 (trit 0), N to a multiple of 16.
// Bytes per strip: 4*Kpad; strips: Npad/16; algorithmic bytes stay K*N/4.
constexpr int kGemvKC = 1024;

struct DevWeight {
    uint8_t* data = nullptr;
    int K = 0, N = 0, Kpad = 0, Npad = 0;
    float scale = 0.f;
    size_t bytes() const { return (size_t)(Npad / 4) * (size_t)Kpad; }
    int tiles() const { return Npad / 16; }   // strips
};

// Byte offset of (byte-column jb, k) in the internal layout.
__host__ __device__ inline size_t weight_offset(int jb, int k, int Kpad) {
    const int strip = jb >> 2, c = jb & 3;
    const int q = k / kGemvKC;
    const int kc = (Kpad - q * kGemvKC) < kGemvKC ? (Kpad - q * kGemvKC) : kGemvKC;
    return (size_t)strip * 4u * (size_t)Kpad + (size_t)q * 4u * kGemvKC + (size_t)c * kc + (size_t)(k - q * kGemvKC);
}

constexpr int kGemvMaxGroup = 8;
constexpr int kGemvMaxRows = 16;       // token rows one multi-row GEMV launch takes
constexpr int kGemvMaxK = 32768;
constexpr int kGemvMaxX = 16;          // distinct activation vectors one streaming launch can stage
constexpr int kGemvMaxTable = 512;     // matrices in one table-mode launch
constexpr int kGemvMaxXBytes = 64 * 1024;

// Per-matrix descriptor of a table-mode launch (device memory, 32 bytes).
struct GemvDesc {
    const uint8_t* W;
    float* out;
    float w_scale;
    int N;
    int tile_begin;   // first strip of this matrix in the launch's strip numbering
    int xid;          // which activation vector
};

struct GemvParams {
    const uint8_t* W[kGemvMaxGroup];
    float* out[kGemvMaxGroup];
    int32_t* acc_out[kGemvMaxGroup];
    float w_scale[kGemvMaxGroup];
    int N[kGemvMaxGroup];
    int tile_begin[kGemvMaxGroup + 1];
    const int8_t* x;
    const float* x_scale;   // device scalar; when null, x_scale_imm is used
    // Streaming kernel: the launch reads n_x activation vectors (vector u: int8[uK[u]] at ux[u], scale at
    // uxs[u], staged at byte uoff[u] of the shared-memory activation area of x_bytes bytes); matrix m
    // multiplies vector xid[m].  multi == 0: the launcher fills these from x / x_scale / K (one vector).
    int multi;
    int n_x;
    const int8_t* ux[kGemvMaxX];
    const float* uxs[kGemvMaxX];
    int uK[kGemvMaxX], uKpad[kGemvMaxX], uoff[kGemvMaxX];
    int x_bytes;
    uint8_t xid[kGemvMaxGroup];
    // Table mode (n_mats may exceed kGemvMaxGroup): the per-matrix fields come from this device array
    // instead of W/out/w_scale/N/tile_begin/xid above; acc_out is not available.
    const GemvDesc* table;
    float x_scale_imm;
    int K, Kpad;
    int n_mats, n_tiles, stages;
    int accumulate;         // out[j] = out[j] + value (residual add fused in the epilogue)
    // Multi-row form (rows >= 2, at most kGemvMaxRows): x is [rows][K] int8, x_scale [rows], out[m] / acc_out[m]
    // are [rows][N[m]]; K a multiple of 16.  No fused prologue, no paired epilogue, no table.
    int rows;
    // Fused prologue (latency path only): when fuse.x is set, every CTA derives the int8 activation
    // vector and its scale itself from fp32 inputs (pre-op -> RMSNorm -> absmax int8, row fuse_row)
    // instead of reading x / x_scale.
    NormQuantParams fuse;
    int fuse_row;
    // Paired activation epilogue (latency path, two matrices gate and up of equal N): instead of the
    // two projections, write act(gate, up) (PRE_SILU_MUL / PRE_RELU2_MUL) for every column to act_out.
    int act_pair;
    float* act_out;
    int* status;
};

struct GemvLaunchCfg {
    int ctas_per_sm = 2;
    int stages = 0;      // per-warp ring depth; 0 = default
    int pdl = 1;
    // matrices (or groups) with at most this many strips take the register-prefetch split-K path
    int split_max_strips = 148 * 8;
    int fuse_quant = 1;   // decode forward: run the quantisers inside the GEMV launches
    int sm_count = 148;
};

cudaError_t launch_gemv(const GemvParams& p, const GemvLaunchCfg& cfg, cudaStream_t st);

// ---- batched GEMM (tcgen05) ---------------------------------------------------
constexpr int kGemmMaxGroup = 3;

struct GemmParams {
    // TMA descriptor of X as a 2-D byte tensor {K, M}, box {128 k, token tile}, 128-byte swizzle: one copy
    // lands a whole activation stage in the layout the tensor core reads.  Set by the launcher.
    alignas(64) CUtensorMap xmap;
    const uint8_t* W;         // internal layout (strips)
    const int8_t* X;          // [M][K] row-major
    const float* x_scales;    // [M]
    float* out;               // [M][N] or null
    int32_t* acc_out;         // [M][N] or null (raw int32 dot products)
    const int32_t* x_rowsum;  // [M] sum_k X[m][k], or null: computed into the scratch by a pre-kernel
    int32_t* scratch;         // M ints: row sums computed by the pre-kernel when x_rowsum is null
    int32_t* part_buf;        // M*N ints or null: split-K partials, ZERO between calls (the finalize kernel clears them)
    int accumulate;           // out[m][n] = out[m][n] + value (residual add)
    int32_t* part;            // set by the launcher
    int32_t* x_rowsum_w;      // set by the launcher
    float w_scale;
    int M, N, K, Kpad, n_strips;
    int tokens, tmem_cols, ksplits, stages;   // set by the launcher
    // Group of up to kGemmMaxGroup weight matrices with the same K multiplied by the same X in ONE launch
    // (q/k/v, gate/up).  n_w == 0: the single matrix described by W / out / w_scale / N / n_strips; the
    // launcher then fills entry 0 from them.  tile_begin: first 128-column tile of each matrix in the grid's
    // tile numbering; part_off: offset (ints) of each matrix's split-K partials in part_buf.
    int n_w;
    const uint8_t* Wg[kGemmMaxGroup];
    float* outg[kGemmMaxGroup];
    float wsg[kGemmMaxGroup];
    int Ng[kGemmMaxGroup], stripsg[kGemmMaxGroup], tile_begin[kGemmMaxGroup + 1];
    size_t part_off[kGemmMaxGroup];
    int* status;
};
cudaError_t launch_gemm(const GemmParams& p, int sm_count, bool pdl, cudaStream_t st);

// ---- install-time re-pack (device side) --------------------------------------
cudaError_t launch_recode_v11(const uint8_t* src, uint8_t* dst, int K, int N, int Kpad, int Npad, cudaStream_t st);
cudaError_t launch_recode_rowmajor(const uint8_t* src, uint8_t* dst, int K, int N, int Kpad, int Npad, cudaStream_t st);
// bad_count receives the number of payload values outside {-1,0,+1}.
cudaError_t launch_pack_i32(const int32_t* src, uint8_t* dst, int K, int N, int Kpad, int Npad, int* bad_count,
                            cudaStream_t st);

}  // namespace terb
