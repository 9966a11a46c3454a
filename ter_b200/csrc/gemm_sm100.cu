// Batched ternary GEMM, M >= 2 tokens, on the sm_100a tensor cores (tcgen05, kind::i8, TMEM).
//
// Replaces mm_bitnet_addonly_batched_k (cuda/ter_cuda_addonly_batched.cu:32-123) and mm_int4_tc*
// (cuda/ter_cuda_int4_tc.cu:36-82, cuda/ter_cuda_int4_tc_tiled.cu:28-104):
//     out[m][j] = (float)(sum_k X[m][k] * trit(k, j)) * (x_scale[m] * w_scale),  exact int32 sum.
//
// This is the one dense contraction of the path.  "Swap AB": the 128-row side of the MMA is a tile
// of 128 OUTPUT COLUMNS (weights), the N side of the MMA is the token batch (16..256), so a small
// batch does not waste the 128-lane datapath.  Per CTA: one tile of 128 columns x a K range x one
// token tile.
//   * loader (warp 9, one lane): one TMA tensor copy (cp.async.bulk.tensor.2d, 128-byte swizzle) per
//     stage brings the 128-k slice of the int8 activations of the token tile into the B stage, in the
//     layout the tensor core reads; it runs as far ahead as there are free stages.
//   * producers (warps 0-7): fetch the packed trits (2 bits) of the tile with 16-byte cp.async copies
//     into a thread-private ring (6 steps deep, 4 in flight), expand them in registers to unsigned
//     bytes and store them into the A stage in the same 128-byte-swizzled layout.  The expansion needs no
//     shift and no sign decode: row r of A holds column 4*b + f, whose bytes are (w & (3 << 2f)),
//     i.e. 4^f * (trit + 1); the accumulator of row r is divided by 4^f in the epilogue (exact) and
//     the "+1" is removed by subtracting sum_k X[m][k].
//   * MMA warp (warp 8, one lane): tcgen05.mma kind::i8 (A unsigned, B signed), M=128, N=token
//     tile, K=32 per instruction, int32 accumulators in tensor memory; tcgen05.commit releases a
//     stage back to the producers through an mbarrier.
//   * epilogue (warps 0-7): tcgen05.ld the accumulators (TMEM lane = output column), scale, store
//     out[m][n] coalesced over n.  With split-K the int32 partials are added into a scratch array
//     with red.global.add.s32 (integer adds are exact and order-free) and a second, wide kernel scales the
//     sums, stores the outputs and clears the partials again, so the scratch is zero between calls and needs
//     no kernel to prepare it.  (Letting the last CTA of a tile to arrive do that work was measured slower:
//     one CTA then reads a whole tile's partials back, 14 against 10 microseconds at 64 tokens.)
// Every wait is bounded; on expiry a status code is recorded and all roles run to the end, so
// tensor memory is always freed.
#include "common.cuh"
#include "kernels.h"
#include "umma.cuh"

namespace terb {

namespace {

constexpr int kProducerWarps = 8;
constexpr int kGemmThreads = 32 * (kProducerWarps + 2);   // 8 producer/epilogue warps + MMA warp + loader warp
constexpr int kTileN = 128;                  // output columns per CTA = MMA M
constexpr int kKStep = 128;                  // k per pipeline stage = one 128-byte swizzle row
constexpr int kAStageBytes = kTileN * kKStep;   // 16 KB
constexpr int kRawStageBytes = 4096;            // the packed trits of one step (128 columns x 128 k, 2 bits each)
// The packed trits travel through a thread-private ring of RING steps (template parameter of the kernel), RING - 2 of
// them in flight as cp.async copies (a step is 4 KB per CTA).

#ifdef TERB_TRACE
// diagnostic build only: timestamps of the phases of each CTA of the last launch
__device__ unsigned long long g_gemm_trace[512][8];
__device__ __forceinline__ void gtr(int k) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    const int cta = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
    if (cta < 512) g_gemm_trace[cta][k] = t;
}
#define GTR(k) gtr(k)
// per-step timestamps of CTA 0: [step][0] MMA warp saw the stage full, [1] producer warp 0 has its packed bytes,
// [2] ... has the free stage, [3] ... has arrived, [4] loader issued the copy
__device__ unsigned long long g_gemm_steps[64][8];
__device__ __forceinline__ void gts(int step, int k) {
    if (blockIdx.x + blockIdx.y + blockIdx.z == 0 && step < 64) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        g_gemm_steps[step][k] = t;
    }
}
#define GTS(s, k) gts(s, k)
#else
#define GTR(k) do {} while (0)
#define GTS(s, k) do {} while (0)
#endif

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Instruction descriptor, kind::i8: D = s32, A = u8, B = s8, both K-major, M = 128, N = n_tokens.
__device__ __forceinline__ uint32_t umma_idesc_i8(int n_tokens) {
    uint32_t d = 0;
    d |= 2u << 4;                       // accumulator format: s32
    d |= 0u << 7;                       // A: unsigned 8-bit
    d |= 1u << 10;                      // B: signed 8-bit
    d |= (uint32_t)(n_tokens >> 3) << 17;
    d |= (uint32_t)(kTileN >> 4) << 24;
    return d;
}

struct GemmSmemLayout {
    int stages, tokens, ring;   // tokens = padded token tile (multiple of 16); ring = packed-trit steps buffered
    int tiles;                  // 128-column tiles per CTA (1 or 2)
    __host__ __device__ int a_stage_bytes() const { return tiles * kAStageBytes; }
    __host__ __device__ int raw_stage_bytes() const { return tiles * kRawStageBytes; }
    __host__ __device__ int b_stage_bytes() const { return tokens * kKStep; }
    __host__ __device__ int a_off(int s) const { return s * a_stage_bytes(); }
    __host__ __device__ int b_off(int s) const { return stages * a_stage_bytes() + s * b_stage_bytes(); }
    __host__ __device__ int raw_off(int s) const { return stages * (a_stage_bytes() + b_stage_bytes()) + s * raw_stage_bytes(); }
    __host__ __device__ int tail_off() const { return stages * (a_stage_bytes() + b_stage_bytes()) + ring * raw_stage_bytes(); }
    // tail: full[8], empty[8], done, pad (u64 each) | tmem base, abort (16 B) | scale[256] (float) | rowsum[256] (int)
    __host__ __device__ int bytes() const { return tail_off() + 18 * 8 + 16 + 2 * 256 * 4 + 1024; }
};

// TILES: 128-column tiles per CTA.  With two, both tiles are multiplied by the same activation stage (two
// accumulators in tensor memory), which halves the activation bytes a CTA pulls from L2 per multiply-add: for
// batches whose one-tile grid would not fit the SMs in one wave.
// PG: producer groups.  The eight producer warps form PG groups and group g expands steps g, g + PG, ...: what
// paces a producer is the chain wait -> expand -> proxy fence -> arrive of one step, so several steps are expanded
// side by side (a thread then owns PG times as many bytes of its steps).
template <int kRawRing, int TILES, int PG>
__global__ void __launch_bounds__(kGemmThreads) gemm_trit_kernel(const __grid_constant__ GemmParams p) {
    constexpr int kRawAhead = (kRawRing - 2) / PG;      // own steps in flight per thread
    constexpr int kGroupThreads = 32 * kProducerWarps / PG;
    extern __shared__ uint8_t gsm_raw[];
    // 1024-byte alignment: the swizzle pattern is a function of the shared-memory address bits
    uint8_t* gsm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(gsm_raw) + 1023) & ~(uintptr_t)1023);
    GemmSmemLayout L{p.stages, p.tokens, kRawRing, TILES};
    uint64_t* full = reinterpret_cast<uint64_t*>(gsm + L.tail_off());
    uint64_t* empty = full + 8;
    uint64_t* done = full + 16;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done + 2);   // keeps the arrays behind it 16-byte aligned
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* tok_scale = reinterpret_cast<float*>(tmem_slot + 4);     // [256] x_scales[m] * w_scale
    int* tok_sum = reinterpret_cast<int*>(tok_scale + 256);         // [256] sum_k X[m][k]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) GTR(0);
    // 128-column tile of which matrix of the group
    int mi = 0;
    while (mi + 1 < p.n_w && (int)blockIdx.x >= p.tile_begin[mi + 1]) ++mi;
    const int tile = (int)blockIdx.x - p.tile_begin[mi];
    const uint8_t* Wm = p.Wg[mi];
    const int Nm = p.Ng[mi], strips_m = p.stripsg[mi];
    float* outm = p.outg[mi];
    const float wsm = p.wsg[mi];
    int32_t* partm = p.part ? p.part + p.part_off[mi] : nullptr;
    const int ksplit = blockIdx.y;                     // K range
    const int m0 = blockIdx.z * p.tokens;              // first token of this token tile
    const int steps_total = p.Kpad / kKStep;
    const int step_begin = (int)((long)steps_total * ksplit / p.ksplits);
    const int step_end = (int)((long)steps_total * (ksplit + 1) / p.ksplits);
    const int n_steps = step_end - step_begin;
    const int S = p.stages;

    if (tid == 0) {
        for (int i = 0; i < S; ++i) { mbar_init(&full[i], kProducerWarps / PG + 1 /* the warps of one producer group + the loader */); mbar_init(&empty[i], 1); }
        mbar_init(done, 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == kProducerWarps) {   // tensor memory for the accumulators: tmem_cols 32-bit columns x 128 lanes
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"((uint32_t)p.tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (tid == 0) GTR(1);

    pdl_launch_dependents();
    pdl_wait();
    if (tid == 0) GTR(2);

    if (warp < kProducerWarps) {
        // ------------------------------------------------------------------ producers (256 threads)
        // A thread owns 16-byte pieces of the packed bytes of its group's steps (segment = (strip, byte-column) of
        // 128 bytes, part = 16 of them): it copies them with cp.async into its private slots of a ring (kRawAhead
        // of its steps in flight, no barrier needed: the same thread reads them back), then expands each piece
        // into 4 rows of the A stage.  A group waits on the stage barriers of its own steps only; a barrier cannot
        // run two phases ahead of such a wait, because the later phase needs this group's step to be multiplied.
        const int nb = (p.Kpad + kGemvKC - 1) / kGemvKC;
        const int last_kc = p.Kpad - (nb - 1) * kGemvKC;
        // a 128-column tile of a step is 32 segments x 8 parts of 16 bytes; a thread of a group owns PG of those pairs
        const int grp = tid / kGroupThreads, gtid = tid % kGroupThreads;
        // per-token epilogue constants
        if (tid < p.tokens) {
            const int m = m0 + tid;
            tok_scale[tid] = (m < p.M && p.x_scales) ? p.x_scales[m] * wsm : 0.0f;
            tok_sum[tid] = (m < p.M) ? p.x_rowsum[m] : 0;
        }
        bool ok = true;
        auto issue = [&](int j) {      // the packed bytes this thread owns of step j
            const int ks = step_begin + j;
            const int q = ks >> 3;
            const int kc = (q == nb - 1) ? last_kc : kGemvKC;
#pragma unroll
            for (int t = 0; t < TILES; ++t)
#pragma unroll
                for (int i = 0; i < PG; ++i) {
                    const int pr = gtid + i * kGroupThreads, seg = pr >> 3, part = pr & 7;
                    const int strip = (tile * TILES + t) * 8 + (seg >> 2), bc = seg & 3;
                    uint8_t* raw = gsm + L.raw_off(j % kRawRing) + t * kRawStageBytes + seg * 128 + part * 16;
                    if (strip < strips_m) {
                        cp_async16(raw, Wm + (size_t)strip * 4u * (size_t)p.Kpad + (size_t)q * (4 * kGemvKC) + (size_t)bc * kc +
                                            (ks & 7) * 128 + part * 16);
                    } else {
                        *reinterpret_cast<uint4*>(raw) = make_uint4(0x55555555u, 0x55555555u, 0x55555555u, 0x55555555u);
                    }
                }
            cp_async_commit();
        };
        for (int j = 0; j < kRawAhead; ++j)
            if (grp + j * PG < n_steps) issue(grp + j * PG); else cp_async_commit();
        for (int it = grp; it < n_steps; it += PG) {
            const int s = it % S;
            if (it + kRawAhead * PG < n_steps) issue(it + kRawAhead * PG); else cp_async_commit();
            cp_async_wait<kRawAhead>();      // this thread's packed bytes of step `it` have landed
            if (gtid == 0) GTS(it, 1);
            // the A stage is free once the MMAs of step it - S have completed
            if (it >= S) ok = ok && mbar_wait_abortable(&empty[s], ((uint32_t)(it / S) & 1u) ^ 1u, abort_flag, p.status);
            if (!ok) break;
            if (gtid == 0) GTS(it, 2);
#pragma unroll
            for (int t = 0; t < TILES; ++t)
#pragma unroll
                for (int i = 0; i < PG; ++i) {
                    const int pr = gtid + i * kGroupThreads, seg = pr >> 3, part = pr & 7;
                    uint8_t* A = gsm + L.a_off(s) + t * kAStageBytes;
                    const uint4 w = *reinterpret_cast<const uint4*>(gsm + L.raw_off(it % kRawRing) + t * kRawStageBytes + seg * 128 + part * 16);
#pragma unroll
                    for (int f = 0; f < 4; ++f) {
                        const uint32_t mk = 0x03030303u << (2 * f);
                        const int r = (seg >> 2) * 16 + (seg & 3) * 4 + f;           // A row = local output column
                        *reinterpret_cast<uint4*>(A + (r >> 3) * 1024 + (r & 7) * 128 + ((part ^ (r & 7)) * 16)) =
                            make_uint4(w.x & mk, w.y & mk, w.z & mk, w.w & mk);
                    }
                }
            fence_async_smem();          // make the generic-proxy writes visible to the tensor core
            __syncwarp();
            if (lane == 0) mbar_arrive(&full[s]);
            if (gtid == 0) GTS(it, 3);
        }
        cp_async_wait<0>();
    } else if (warp == kProducerWarps + 1) {
        // ------------------------------------------------------------------ activation loader (TMA)
        if (lane == 0) {
            const uint32_t bytes = (uint32_t)p.tokens * kKStep;
            bool ok = true;
            for (int j = 0; j < n_steps && ok; ++j) {
                const int s = j % S;
                if (j >= S) ok = mbar_wait_abortable(&empty[s], ((uint32_t)(j / S) & 1u) ^ 1u, abort_flag, p.status);
                if (!ok) break;
                mbar_arrive_expect_tx(&full[s], bytes);
                GTS(j, 4);
                asm volatile(
                    "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                    ::"r"(smem_u32(gsm + L.b_off(s))), "l"(reinterpret_cast<uint64_t>(&p.xmap)),
                      "r"((step_begin + j) * kKStep), "r"(m0), "r"(smem_u32(&full[s]))
                    : "memory");
            }
        }
    } else if (lane == 0) {
        // ------------------------------------------------------------------ MMA issuer
        const uint32_t idesc = umma_idesc_i8(p.tokens);
        bool ok = true;
        for (int it = 0; it < n_steps && ok; ++it) {
            const int s = it % S;
            const uint32_t ph = (uint32_t)(it / S) & 1u;
            ok = mbar_wait_abortable(&full[s], ph, abort_flag, p.status);
            if (!ok) break;
            if (it == 0) GTR(3);
            GTS(it, 0);
            tc_fence_after();
            const uint64_t bdesc = umma_desc_sw128(smem_u32(gsm + L.b_off(s)));
#pragma unroll
            for (int t = 0; t < TILES; ++t) {
                const uint64_t adesc = umma_desc_sw128(smem_u32(gsm + L.a_off(s) + t * kAStageBytes));
#pragma unroll
                for (int kk = 0; kk < kKStep / 32; ++kk) {
                    const uint32_t accum = (it > 0 || kk > 0) ? 1u : 0u;
                    asm volatile(
                        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
                        ::"r"(tmem_base + (uint32_t)(t * p.tokens)), "l"(adesc + (uint64_t)(kk * 2)),
                          "l"(bdesc + (uint64_t)(kk * 2)), "r"(idesc), "r"(accum)
                        : "memory");
                }
            }
            // release the stage when the MMAs that read it have completed
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                             smem_u32(&empty[s]))
                         : "memory");
        }
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(done))
                     : "memory");
        GTR(4);
    }
    __syncwarp();

    if (warp < kProducerWarps) {
        // ------------------------------------------------------------------ epilogue (8 warps)
        asm volatile("bar.sync 1, 256;" ::: "memory");     // tok_scale / tok_sum visible to all producer warps
        const bool ok = n_steps > 0 && mbar_wait_abortable(done, 0, abort_flag, p.status);
        if (tid == 0) GTR(5);
        tc_fence_after();
        const int quarter = warp & 3;                      // the TMEM lanes this warp may read
        const int nl = quarter * 32 + lane;                // TMEM lane = local output column
        const int shift = 2 * (nl & 3);
        // warps 0-3 take the even 32-token groups, warps 4-7 the odd ones
        if (ok) {
#pragma unroll
            for (int t = 0; t < TILES; ++t) {
                const int n = (tile * TILES + t) * kTileN + nl;
                for (int c0 = (warp >> 2) * 32; c0 < p.tokens; c0 += 64) {
                    uint32_t d[32];
                    const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(t * p.tokens + c0);
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
                    if (n < Nm) {
                        // tokens of this group that exist; the common case (a full group, plain fp32 output) runs
                        // without a test per element: the epilogue is instruction-bound (8 warps, 128 values a thread)
                        const int rows = min(32, min(p.tokens - c0, p.M - (m0 + c0)));
                        if (p.ksplits > 1) {
                            int32_t* po = partm + (size_t)(m0 + c0) * Nm + n;
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (j < rows) atomicAdd(po + (size_t)j * Nm, (int)d[j]);
                        } else if (rows == 32 && !p.acc_out && outm && !p.accumulate) {
                            float* po = outm + (size_t)(m0 + c0) * Nm + n;
#pragma unroll
                            for (int j4 = 0; j4 < 8; ++j4) {
                                const int4 ts = *reinterpret_cast<const int4*>(&tok_sum[c0 + 4 * j4]);
                                const float4 sc = *reinterpret_cast<const float4*>(&tok_scale[c0 + 4 * j4]);
                                po[(size_t)(4 * j4 + 0) * Nm] = (float)(((int)d[4 * j4 + 0] >> shift) - ts.x) * sc.x;
                                po[(size_t)(4 * j4 + 1) * Nm] = (float)(((int)d[4 * j4 + 1] >> shift) - ts.y) * sc.y;
                                po[(size_t)(4 * j4 + 2) * Nm] = (float)(((int)d[4 * j4 + 2] >> shift) - ts.z) * sc.z;
                                po[(size_t)(4 * j4 + 3) * Nm] = (float)(((int)d[4 * j4 + 3] >> shift) - ts.w) * sc.w;
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                if (j < rows) {
                                    const size_t o = (size_t)(m0 + c0 + j) * Nm + n;
                                    const int v = ((int)d[j] >> shift) - tok_sum[c0 + j];
                                    if (p.acc_out) p.acc_out[o] = v;
                                    if (outm) {
                                        const float f = (float)v * tok_scale[c0 + j];
                                        outm[o] = p.accumulate ? outm[o] + f : f;
                                    }
                                }
                            }
                        }
                    }
                }
            }
        }
    }
    if (tid == 0) GTR(6);
    tc_fence_before();
    __syncthreads();
    if (tid == 0) GTR(7);
    if (warp == kProducerWarps) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)p.tmem_cols)
                     : "memory");
    }
}

// Row sums of the activations: rowsum[m] = sum_k X[m][k] (one warp per row).  They remove the "+1" of
// the unsigned weight bytes: sum_k x*(t+1) - sum_k x = sum_k x*t.
__global__ void __launch_bounds__(256) gemm_prep_kernel(const GemmParams p) {
    pdl_launch_dependents();
    pdl_wait();
    if (!p.x_rowsum_w) return;
    const int lane = threadIdx.x & 31;
    for (int m = blockIdx.x * 8 + (threadIdx.x >> 5); m < p.M; m += gridDim.x * 8) {
        const int8_t* row = p.X + (size_t)m * p.K;
        int acc = 0;
        for (int k = lane * 16; k < p.K; k += 512) {
            const int4 v = *reinterpret_cast<const int4*>(row + k);
            acc = __dp4a(v.x, 0x01010101, acc);
            acc = __dp4a(v.y, 0x01010101, acc);
            acc = __dp4a(v.z, 0x01010101, acc);
            acc = __dp4a(v.w, 0x01010101, acc);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0) p.x_rowsum_w[m] = acc;
    }
}

// Split-K second pass: out[m][n] = float((part[m][n] >> 2*(n%4)) - rowsum[m]) * (x_scales[m] * w_scale); the partials
// are cleared on the way, ready for the next call.  Grid: (column groups of 1024, token rows, matrices); a thread
// takes four adjacent columns (N is a multiple of 16), so there is no index arithmetic beyond a multiply-add.
__global__ void __launch_bounds__(256) gemm_finalize_kernel(const GemmParams p) {
    pdl_launch_dependents();
    pdl_wait();
    const int w = blockIdx.z, m = blockIdx.y;
    const int N = p.Ng[w];
    const int n = (blockIdx.x * 256 + threadIdx.x) * 4;
    if (n >= N) return;
    const size_t i = (size_t)m * N + n;
    int32_t* part = p.part + p.part_off[w] + i;
    const int4 raw = *reinterpret_cast<const int4*>(part);
    *reinterpret_cast<int4*>(part) = make_int4(0, 0, 0, 0);
    const int rs = p.x_rowsum[m];
    const int v0 = raw.x - rs, v1 = (raw.y >> 2) - rs, v2 = (raw.z >> 4) - rs, v3 = (raw.w >> 6) - rs;   // n % 4 == 0
    if (p.acc_out) *reinterpret_cast<int4*>(p.acc_out + i) = make_int4(v0, v1, v2, v3);
    if (float* out = p.outg[w]) {
        const float sc = p.x_scales[m] * p.wsg[w];
        float4 f = make_float4((float)v0 * sc, (float)v1 * sc, (float)v2 * sc, (float)v3 * sc);
        if (p.accumulate) {
            const float4 o = *reinterpret_cast<const float4*>(out + i);
            f.x = o.x + f.x; f.y = o.y + f.y; f.z = o.z + f.z; f.w = o.w + f.w;
        }
        *reinterpret_cast<float4*>(out + i) = f;
    }
}

}  // namespace

#ifndef TERB_GEMM_PG
#define TERB_GEMM_PG 1     // 2 and 4 measured the same: the MMA-issuing thread paces the loop, not the producers
#endif
constexpr int kPG = TERB_GEMM_PG;

cudaError_t launch_gemm(const GemmParams& p_in, int sm_count, bool pdl, cudaStream_t st) {
    GemmParams p = p_in;
    if (p.M < 1 || p.K % 16 != 0 || p.Kpad % kKStep != 0) return cudaErrorInvalidValue;
    // token tile: multiple of 16, at most 256 (the N extent of one MMA)
    int tokens = (p.M + 15) / 16 * 16;
    if (tokens > 256) tokens = 256;
    p.tokens = tokens;
    const int m_tiles = (p.M + tokens - 1) / tokens;
    if (p.n_w == 0) {   // the single matrix given by the scalar fields
        p.n_w = 1;
        p.Wg[0] = p.W; p.outg[0] = p.out; p.wsg[0] = p.w_scale; p.Ng[0] = p.N; p.stripsg[0] = p.n_strips;
    }
    if (p.n_w < 1 || p.n_w > kGemmMaxGroup || (p.n_w > 1 && p.acc_out)) return cudaErrorInvalidValue;
    // Two 128-column tiles per CTA when the one-tile grid would need more than one wave of the SMs (several token
    // tiles): the CTA then reads each activation stage once for 256 columns.
    int tiles = 1;
    {
        int t1 = 0;
        for (int w = 0; w < p.n_w; ++w) t1 += (p.stripsg[w] + 7) / 8;
        if (m_tiles >= 2 && (long)t1 * m_tiles > sm_count && tokens == 256) tiles = 2;
    }
    int cols = 32;
    while (cols < tiles * tokens) cols *= 2;
    p.tmem_cols = cols;
    int n_tiles = 0;
    size_t part_ints = 0;
    for (int w = 0; w < p.n_w; ++w) {
        p.tile_begin[w] = n_tiles;
        n_tiles += (p.stripsg[w] + 8 * tiles - 1) / (8 * tiles);
        p.part_off[w] = part_ints;
        part_ints += (size_t)p.M * (size_t)p.Ng[w];
    }
    p.tile_begin[p.n_w] = n_tiles;
    const int steps = p.Kpad / kKStep;
    // Split K so that the grid covers the SMs, when that pays: a CTA's main loop costs about 0.48 us per 128-k step
    // whatever the token tile (the MMA-issuing thread paces it), and splitting saves (1 - 1/ksplits) of it; against
    // that stand the integer atomics of the partial sums and the second kernel, about 1.5 us + 1 us per 100 k
    // outputs (measured on the BitNet-2B shapes, 17 to 256 rows).
    int ksplits = 1;
    if (p.part_buf && p.M <= 256) {
        int ks = sm_count / (n_tiles * m_tiles);
        if (ks > steps / 4) ks = steps / 4;
        if (ks > 1) {
            size_t outputs = 0;
            for (int w = 0; w < p.n_w; ++w) outputs += (size_t)p.M * (size_t)p.Ng[w];
            const double gain = 0.48 * steps * (1.0 - 1.0 / ks), cost = 1.5 + (double)outputs / 1.0e5;
            if (gain > cost) ksplits = ks;
        }
    }
    for (int w = 0; w < p.n_w; ++w)     // the second pass moves four columns at a time
        if ((p.Ng[w] & 3) || (reinterpret_cast<uintptr_t>(p.outg[w]) & 15u)) ksplits = 1;
    if (reinterpret_cast<uintptr_t>(p.acc_out) & 15u) ksplits = 1;
    p.ksplits = ksplits;
    const int ring = 8;     // a 24-step ring for small token tiles measured no faster: the producers' work per step paces the loop
    GemmSmemLayout L{8, tokens, ring, tiles};                   // as many stages as fit, at most 8
    while (L.stages > 2 && L.bytes() > 220 * 1024) --L.stages;
    if (L.bytes() > 220 * 1024) return cudaErrorInvalidValue;
    p.stages = L.stages;
    {
        // X as a 2-D byte tensor: dim 0 = k (K bytes per row), dim 1 = token; one box = 128 k x the token tile
        if ((reinterpret_cast<uintptr_t>(p.X) & 15u) != 0) return cudaErrorInvalidValue;
        EncodeTiledFn enc = encode_tiled();
        if (!enc) return cudaErrorNotSupported;
        const cuuint64_t dims[2] = {(cuuint64_t)p.K, (cuuint64_t)p.M};
        const cuuint64_t strides[1] = {(cuuint64_t)p.K};
        const cuuint32_t box[2] = {(cuuint32_t)kKStep, (cuuint32_t)tokens};
        const cuuint32_t estr[2] = {1, 1};
        if (enc(&p.xmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t*>(p.X), dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    const size_t smem = (size_t)L.bytes();
    static bool attr_set[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (!attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_trit_kernel<8, 1, kPG>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
        if (e != cudaSuccess) return e;
        e = cudaFuncSetAttribute(gemm_trit_kernel<8, 2, kPG>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    cudaError_t e;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    p.part = nullptr;
    p.x_rowsum_w = nullptr;
    if (ksplits > 1) p.part = p.part_buf;
    if (!p.x_rowsum) {   // the caller did not supply the row sums: compute them into the scratch
        if (!p.scratch) return cudaErrorInvalidValue;
        p.x_rowsum_w = p.scratch;
        p.x_rowsum = p.scratch;
    }
    if (p.x_rowsum_w) {
        cudaLaunchConfig_t lr = {};
        size_t g = (size_t)(p.M + 7) / 8;
        if (g > (size_t)sm_count * 8) g = (size_t)sm_count * 8;
        lr.gridDim = dim3((unsigned)g);
        lr.blockDim = dim3(256);
        lr.stream = st;
        lr.attrs = attr;
        lr.numAttrs = pdl ? 1 : 0;
        e = cudaLaunchKernelEx(&lr, gemm_prep_kernel, p);
        if (e != cudaSuccess) return e;
    }
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3((unsigned)n_tiles, (unsigned)ksplits, (unsigned)m_tiles);
    lc.blockDim = dim3(kGemmThreads);
    lc.dynamicSmemBytes = smem;
    lc.stream = st;
    lc.attrs = attr;
    lc.numAttrs = pdl ? 1 : 0;   // after a memset node keep plain stream order
    e = tiles == 2 ? cudaLaunchKernelEx(&lc, gemm_trit_kernel<8, 2, kPG>, p) : cudaLaunchKernelEx(&lc, gemm_trit_kernel<8, 1, kPG>, p);
    if (e != cudaSuccess || ksplits == 1) return e;
    cudaLaunchConfig_t lf = {};
    int max_n = 0;
    for (int w = 0; w < p.n_w; ++w) max_n = p.Ng[w] > max_n ? p.Ng[w] : max_n;
    lf.gridDim = dim3((unsigned)((max_n + 1023) / 1024), (unsigned)p.M, (unsigned)p.n_w);
    lf.blockDim = dim3(256);
    lf.stream = st;
    lf.attrs = attr;
    lf.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&lf, gemm_finalize_kernel, p);
}

#ifdef TERB_TRACE
extern "C" int ter_b200_debug_gemm_steps(unsigned long long* host) {
    cudaDeviceSynchronize();
    return (int)cudaMemcpyFromSymbol(host, g_gemm_steps, sizeof(unsigned long long) * 64 * 8);
}
extern "C" int ter_b200_debug_gemm_trace(unsigned long long* host) {
    cudaDeviceSynchronize();
    cudaError_t e = cudaMemcpyFromSymbol(host, g_gemm_trace, sizeof(unsigned long long) * 512 * 8);
    void* ptr = nullptr;     // cleared for the next launch (a smaller grid would leave old rows behind)
    if (e == cudaSuccess && cudaGetSymbolAddress(&ptr, g_gemm_trace) == cudaSuccess)
        e = cudaMemset(ptr, 0, sizeof(unsigned long long) * 512 * 8);
    return (int)e;
}
#endif

}  // namespace terb
