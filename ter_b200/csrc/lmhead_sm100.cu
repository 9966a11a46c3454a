// bf16 lm_head for token batches on the sm_100a tensor cores (tcgen05 kind::f16, TMEM accumulators).
//
//     logits[b][v] = sum_h bf16(table[v][h]) * x[b][h]
// is the reference's mm_fp16_lm_head_k (cuda/ter_cuda_forward_packed.cu:165-206) for a batch of rows: with 16
// or more rows it is a real contraction ([B x H] . [H x V]) and the CUDA-core kernel of glue_sm100.cu turns
// compute-bound (1.9 ms at 64 rows for a table that streams in 0.1 ms).  Here:
//   * the fp32 activations are split once into two bf16 parts, x = hi + lo (hi = bf16(x), lo = bf16(x - hi)),
//     so that the tensor core sees x to 16 mantissa bits; products of bf16 values are exact in fp32 and the
//     accumulators are fp32 in tensor memory.  The result differs from the fixed-order fp32 sum of the exact
//     kernel by rounding only (about 1e-6 relative); callers that need bit-identical logits use the exact
//     kernel (batches below 16 rows always do).
//   * swap-AB as in the ternary GEMM: 128 vocabulary rows are the M side of the MMA, the token rows (16..256)
//     the N side.  One CTA per 128-row tile of the table; per 64-wide k step one TMA tensor copy brings the
//     table slice (128 x 64 bf16, 128-byte swizzle: the layout the tensor core reads) and two bring the hi
//     and lo slices of the activations; 2 x 4 tcgen05.mma (K = 16 each) accumulate into TMEM.
//   * roles: warp 4 lane 0 = TMA loader, warp 5 lane 0 = MMA issuer (warp 5 allocates / frees TMEM),
//     warps 0-3 = epilogue (tcgen05.ld, one vocabulary row per thread, stores coalesced over the vocabulary).
//   * two CTAs per SM (three stages each), so one CTA's epilogue overlaps the other's main loop.
// The TMA loads are plain per-CTA loads.  Every wait is bounded; TMEM is freed on every path.
#include <cuda_bf16.h>
#include <string.h>

#include "common.cuh"
#include "glue.h"
#include "umma.cuh"

namespace terb {
namespace {

constexpr int kLmThreads = 192;          // 4 epilogue warps + loader warp + MMA warp
constexpr int kLmTileV = 128;            // vocabulary rows per CTA = MMA M
constexpr int kLmKStep = 64;             // bf16 elements per k step = one 128-byte swizzle row
constexpr int kLmAStage = kLmTileV * kLmKStep * 2;   // 16 KB

struct LmTcParams {
    alignas(64) CUtensorMap tmap;        // table [V][H] bf16, box {64, 128}
    alignas(64) CUtensorMap hmap;        // x hi [B][H] bf16, box {64, tokens}
    alignas(64) CUtensorMap lmap;        // x lo
    float* logits;                       // [B][V]
    int V, H, B, tokens, tmem_cols, stages;
    int* status;
};

// Instruction descriptor, kind::f16: D = f32, A = B = bf16, both K-major, M = 128, N = tokens.
__device__ __forceinline__ uint32_t umma_idesc_bf16(int n_tokens) {
    uint32_t d = 0;
    d |= 1u << 4;                       // accumulator format: f32
    d |= 1u << 7;                       // A: bf16
    d |= 1u << 10;                      // B: bf16
    d |= (uint32_t)(n_tokens >> 3) << 17;
    d |= (uint32_t)(kLmTileV >> 4) << 24;
    return d;
}

__global__ void __launch_bounds__(kLmThreads, 2) lm_head_tc_kernel(const __grid_constant__ LmTcParams p) {
    extern __shared__ uint8_t lsm_raw[];
    uint8_t* lsm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(lsm_raw) + 1023) & ~(uintptr_t)1023);
    const int S = p.stages;
    const int b_bytes = p.tokens * kLmKStep * 2;                 // one activation part of one stage
    const int stage_bytes = kLmAStage + 2 * b_bytes;
    uint64_t* full = reinterpret_cast<uint64_t*>(lsm + (size_t)S * stage_bytes);
    uint64_t* empty = full + 8;
    uint64_t* done = full + 16;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int v0 = blockIdx.x * kLmTileV;
    const int m0 = blockIdx.y * p.tokens;
    const int n_steps = p.H / kLmKStep;

    if (tid == 0) {
        for (int i = 0; i < S; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
        mbar_init(done, 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 5) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"((uint32_t)p.tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    pdl_launch_dependents();
    pdl_wait();

    if (warp == 4) {
        if (lane == 0) {
            // ---------------------------------------------------------------- loader: three tensor copies per stage
            const uint32_t bytes = (uint32_t)stage_bytes;
            bool ok = true;
            for (int j = 0; j < n_steps && ok; ++j) {
                const int s = j % S;
                if (j >= S) ok = mbar_wait_abortable(&empty[s], ((uint32_t)(j / S) & 1u) ^ 1u, abort_flag, p.status);
                if (!ok) break;
                uint8_t* st = lsm + (size_t)s * stage_bytes;
                mbar_arrive_expect_tx(&full[s], bytes);
                asm volatile(
                    "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                    ::"r"(smem_u32(st)), "l"(reinterpret_cast<uint64_t>(&p.tmap)), "r"(j * kLmKStep), "r"(v0),
                      "r"(smem_u32(&full[s]))
                    : "memory");
                asm volatile(
                    "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                    ::"r"(smem_u32(st + kLmAStage)), "l"(reinterpret_cast<uint64_t>(&p.hmap)), "r"(j * kLmKStep), "r"(m0),
                      "r"(smem_u32(&full[s]))
                    : "memory");
                asm volatile(
                    "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                    ::"r"(smem_u32(st + kLmAStage + b_bytes)), "l"(reinterpret_cast<uint64_t>(&p.lmap)), "r"(j * kLmKStep),
                      "r"(m0), "r"(smem_u32(&full[s]))
                    : "memory");
            }
        }
    } else if (warp == 5) {
        if (lane == 0) {
            // ---------------------------------------------------------------- MMA issuer
            const uint32_t idesc = umma_idesc_bf16(p.tokens);
            bool ok = true;
            for (int it = 0; it < n_steps && ok; ++it) {
                const int s = it % S;
                ok = mbar_wait_abortable(&full[s], (uint32_t)(it / S) & 1u, abort_flag, p.status);
                if (!ok) break;
                tc_fence_after();
                uint8_t* st = lsm + (size_t)s * stage_bytes;
                const uint64_t adesc = umma_desc_sw128(smem_u32(st));
                const uint64_t hdesc = umma_desc_sw128(smem_u32(st + kLmAStage));
                const uint64_t ldesc = umma_desc_sw128(smem_u32(st + kLmAStage + b_bytes));
#pragma unroll
                for (int part = 0; part < 2; ++part) {
                    const uint64_t bdesc = part == 0 ? hdesc : ldesc;
#pragma unroll
                    for (int kk = 0; kk < kLmKStep / 16; ++kk) {
                        const uint32_t accum = (it > 0 || part > 0 || kk > 0) ? 1u : 0u;
                        asm volatile(
                            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                            ::"r"(tmem_base), "l"(adesc + (uint64_t)(kk * 2)), "l"(bdesc + (uint64_t)(kk * 2)), "r"(idesc),
                              "r"(accum)
                            : "memory");
                    }
                }
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                                 smem_u32(&empty[s]))
                             : "memory");
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(done))
                         : "memory");
        }
    } else {
        // -------------------------------------------------------------------- epilogue (warps 0-3)
        const bool ok = n_steps > 0 && mbar_wait_abortable(done, 0, abort_flag, p.status);
        tc_fence_after();
        const int v = v0 + warp * 32 + lane;            // TMEM lane = vocabulary row of the tile
        if (ok) {
            for (int c0 = 0; c0 < p.tokens; c0 += 32) {
                uint32_t d[32];
                const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0;
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                    "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                    "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                    : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]), "=r"(d[4]), "=r"(d[5]), "=r"(d[6]), "=r"(d[7]),
                      "=r"(d[8]), "=r"(d[9]), "=r"(d[10]), "=r"(d[11]), "=r"(d[12]), "=r"(d[13]), "=r"(d[14]), "=r"(d[15]),
                      "=r"(d[16]), "=r"(d[17]), "=r"(d[18]), "=r"(d[19]), "=r"(d[20]), "=r"(d[21]), "=r"(d[22]), "=r"(d[23]),
                      "=r"(d[24]), "=r"(d[25]), "=r"(d[26]), "=r"(d[27]), "=r"(d[28]), "=r"(d[29]), "=r"(d[30]), "=r"(d[31])
                    : "r"(taddr));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (v < p.V) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int m = m0 + c0 + j;
                        if (c0 + j < p.tokens && m < p.B) p.logits[(size_t)m * p.V + v] = __uint_as_float(d[j]);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 5) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)p.tmem_cols)
                     : "memory");
    }
}

// x (fp32) -> hi = bf16(x), lo = bf16(x - hi)
struct SplitParams { const float* x; uint16_t* hi; uint16_t* lo; size_t n; };
__global__ void __launch_bounds__(256) split_bf16_kernel(const SplitParams p) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < p.n; i += (size_t)gridDim.x * 256) {
        const float x = p.x[i];
        const __nv_bfloat16 h = __float2bfloat16_rn(x);
        const float r = x - __bfloat162float(h);
        p.hi[i] = __bfloat16_as_ushort(h);
        p.lo[i] = __bfloat16_as_ushort(__float2bfloat16_rn(r));
    }
}

}  // namespace

size_t lm_head_tc_scratch_bytes(int B, int H) { return 2u * (size_t)B * (size_t)H * sizeof(uint16_t); }

cudaError_t launch_lm_head_tc(const uint16_t* table, const float* x, float* logits, int V, int H, int B, void* scratch,
                              int* status, bool pdl, cudaStream_t st) {
    if (B < 1 || V < 1 || H < kLmKStep || H % kLmKStep != 0 || !scratch) return cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(table) & 15u) || (reinterpret_cast<uintptr_t>(scratch) & 15u)) return cudaErrorInvalidValue;
    uint16_t* hi = static_cast<uint16_t*>(scratch);
    uint16_t* lo = hi + (size_t)B * H;
    LmTcParams p;
    memset(&p, 0, sizeof p);
    int tokens = (B + 15) / 16 * 16;
    if (tokens > 256) tokens = 256;
    p.tokens = tokens;
    int cols = 32;
    while (cols < tokens) cols *= 2;
    p.tmem_cols = cols;
    p.logits = logits; p.V = V; p.H = H; p.B = B; p.status = status;
    const int m_tiles = (B + tokens - 1) / tokens;
    const int stage_bytes = kLmAStage + 2 * tokens * kLmKStep * 2;
    // two CTAs per SM when the stages allow it (their TMEM shares fit: at most 256 columns each)
    int stages = (110 * 1024 - 2048) / stage_bytes;
    if (stages > 4) stages = 4;
    if (stages < 2) stages = (220 * 1024 - 2048) / stage_bytes;
    if (stages > 8) stages = 8;
    if (stages < 2) return cudaErrorInvalidValue;
    p.stages = stages;
    EncodeTiledFn enc = encode_tiled();
    if (!enc) return cudaErrorNotSupported;
    const cuuint32_t estr[2] = {1, 1};
    {
        const cuuint64_t dims[2] = {(cuuint64_t)H, (cuuint64_t)V};
        const cuuint64_t strides[1] = {(cuuint64_t)H * 2};
        const cuuint32_t box[2] = {(cuuint32_t)kLmKStep, (cuuint32_t)kLmTileV};
        if (enc(&p.tmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<uint16_t*>(table), dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    for (int part = 0; part < 2; ++part) {
        const cuuint64_t dims[2] = {(cuuint64_t)H, (cuuint64_t)B};
        const cuuint64_t strides[1] = {(cuuint64_t)H * 2};
        const cuuint32_t box[2] = {(cuuint32_t)kLmKStep, (cuuint32_t)tokens};
        if (enc(part == 0 ? &p.hmap : &p.lmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, part == 0 ? hi : lo, dims, strides, box,
                estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    {
        SplitParams sp{x, hi, lo, (size_t)B * H};
        cudaLaunchConfig_t lc = {};
        size_t g = (sp.n + 255) / 256;
        lc.gridDim = dim3((unsigned)(g > 2048 ? 2048 : g));
        lc.blockDim = dim3(256);
        lc.stream = st;
        lc.attrs = attr;
        lc.numAttrs = pdl ? 1 : 0;
        cudaError_t e = cudaLaunchKernelEx(&lc, split_bf16_kernel, sp);
        if (e != cudaSuccess) return e;
    }
    const size_t smem = (size_t)stages * stage_bytes + 17 * 8 + 16 + 1024;
    static bool attr_set[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (!attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(lm_head_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3((unsigned)((V + kLmTileV - 1) / kLmTileV), (unsigned)m_tiles);
    lc.blockDim = dim3(kLmThreads);
    lc.dynamicSmemBytes = smem;
    lc.stream = st;
    lc.attrs = attr;
    lc.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&lc, lm_head_tc_kernel, p);
}

}  // namespace terb
