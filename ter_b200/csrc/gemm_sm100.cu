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
//   * producers (warps 0-3): read the packed trits (2 bits) of the tile straight from global with
//     16-byte read-only loads, expand them in registers to unsigned bytes and store them into the
//     A stage in the 128-byte-swizzled K-major layout the tensor core reads; copy the matching
//     128-k slice of the int8 activations into the B stage (same layout).  The expansion needs no
//     shift and no sign decode: row r of A holds column 4*b + f, whose bytes are (w & (3 << 2f)),
//     i.e. 4^f * (trit + 1); the accumulator of row r is divided by 4^f in the epilogue (exact) and
//     the "+1" is removed by subtracting sum_k X[m][k].
//   * MMA warp (warp 4, one lane): tcgen05.mma kind::i8 (A unsigned, B signed), M=128, N=token
//     tile, K=32 per instruction, int32 accumulators in tensor memory; tcgen05.commit releases a
//     stage back to the producers through an mbarrier.
//   * epilogue (warps 0-3): tcgen05.ld the accumulators (TMEM lane = output column), scale, store
//     out[m][n] coalesced over n.  With split-K the int32 partials are added into a scratch array
//     with red.global.add.s32 (integer adds are exact and order-free) and a second kernel scales.
// Every wait is bounded; on expiry a status code is recorded and all roles run to the end, so
// tensor memory is always freed.
#include "common.cuh"
#include "kernels.h"

namespace terb {

namespace {

constexpr int kGemmThreads = 160;            // 4 producer/epilogue warps + 1 MMA warp
constexpr int kTileN = 128;                  // output columns per CTA = MMA M
constexpr int kKStep = 128;                  // k per pipeline stage = one 128-byte swizzle row
constexpr int kAStageBytes = kTileN * kKStep;   // 16 KB

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Bounded wait that also gives up as soon as another role has flagged an abort.
__device__ __forceinline__ bool mbar_wait_abortable(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                                    int* status) {
    for (uint32_t i = 0; i < (1u << 21); ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 255u && *abort_flag) return false;
    }
    *abort_flag = 1;
    if (status) atomicExch(status, DEV_TIMEOUT_MBAR);
    return false;
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows of 128 bytes, 8-row groups
// 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);          // start address
    d |= (uint64_t)1 << 16;                                // leading byte offset (unused for this layout)
    d |= (uint64_t)(1024 >> 4) << 32;                      // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                                // descriptor version (sm_100)
    d |= (uint64_t)2 << 61;                                // 128-byte swizzle
    return d;
}
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
    int stages, tokens;   // tokens = padded token tile (multiple of 16)
    __host__ __device__ int b_stage_bytes() const { return tokens * kKStep; }
    __host__ __device__ int a_off(int s) const { return s * kAStageBytes; }
    __host__ __device__ int b_off(int s) const { return stages * kAStageBytes + s * b_stage_bytes(); }
    __host__ __device__ int tail_off() const { return stages * (kAStageBytes + b_stage_bytes()); }
    // tail: full[8], empty[8], done (u64 each) | tmem base (u32) | abort (int) | xsum[256] (int)
    __host__ __device__ int bytes() const { return tail_off() + 17 * 8 + 16 + 256 * 4 + 1024; }
};

__global__ void __launch_bounds__(kGemmThreads) gemm_trit_kernel(const __grid_constant__ GemmParams p) {
    extern __shared__ uint8_t gsm_raw[];
    // 1024-byte alignment: the swizzle pattern is a function of the shared-memory address bits
    uint8_t* gsm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(gsm_raw) + 1023) & ~(uintptr_t)1023);
    GemmSmemLayout L{p.stages, p.tokens};
    uint64_t* full = reinterpret_cast<uint64_t*>(gsm + L.tail_off());
    uint64_t* empty = full + 8;
    uint64_t* done = full + 16;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    int* xsum_s = reinterpret_cast<int*>(tmem_slot + 4);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tile = blockIdx.x;                       // 128-column tile
    const int ksplit = blockIdx.y;                     // K range
    const int m0 = blockIdx.z * p.tokens;              // first token of this token tile
    const int steps_total = p.Kpad / kKStep;
    const int step_begin = (int)((long)steps_total * ksplit / p.ksplits);
    const int step_end = (int)((long)steps_total * (ksplit + 1) / p.ksplits);
    const int n_steps = step_end - step_begin;
    const int S = p.stages;

    if (tid == 0) {
        for (int i = 0; i < S; ++i) { mbar_init(&full[i], 4); mbar_init(&empty[i], 1); }
        mbar_init(done, 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    for (int i = tid; i < 256; i += kGemmThreads) xsum_s[i] = 0;
    if (warp == 4) {   // tensor memory for the accumulators: tmem_cols 32-bit columns x 128 lanes
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

    if (warp < 4) {
        // ------------------------------------------------------------------ producers
        const int nb = (p.Kpad + kGemvKC - 1) / kGemvKC;
        const int last_kc = p.Kpad - (nb - 1) * kGemvKC;
        const int seg = tid >> 2, part = tid & 3;          // 32 segments (strip, byte-column) x 4 x 32 bytes
        const int strip_l = seg >> 2, bc = seg & 3;
        const int strip = tile * 8 + strip_l;
        const bool strip_ok = strip < p.n_strips;
        const uint8_t* sbase = p.W + (size_t)strip * 4u * (size_t)p.Kpad;
        const int xr = tid >> 3, xci = tid & 7;            // activation copy: row xr + 16*i, 16-byte chunk xci
        const int nt16 = p.tokens / 16;
        int psum[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) psum[i] = 0;
        bool ok = true;
        for (int it = 0; it < n_steps && ok; ++it) {
            const int s = it % S;
            const uint32_t ph = (uint32_t)(it / S) & 1u;
            if (it >= S) ok = mbar_wait_abortable(&empty[s], ph ^ 1u, abort_flag, p.status);
            if (!ok) break;
            const int ks = step_begin + it;
            // ---- A: expand 32 packed bytes (32 k x 4 columns) of this thread's segment
            uint8_t* A = gsm + L.a_off(s);
            {
                const int q = ks >> 3;
                const int kc = (q == nb - 1) ? last_kc : kGemvKC;
                const uint8_t* src = sbase + (size_t)q * (4 * kGemvKC) + (size_t)bc * kc + (ks & 7) * 128 + part * 32;
                uint4 w0 = make_uint4(0x55555555u, 0x55555555u, 0x55555555u, 0x55555555u), w1 = w0;
                if (strip_ok) {
                    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                                 : "=r"(w0.x), "=r"(w0.y), "=r"(w0.z), "=r"(w0.w) : "l"(src));
                    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                                 : "=r"(w1.x), "=r"(w1.y), "=r"(w1.z), "=r"(w1.w) : "l"(src + 16));
                }
#pragma unroll
                for (int f = 0; f < 4; ++f) {
                    const uint32_t mk = 0x03030303u << (2 * f);
                    const int r = strip_l * 16 + bc * 4 + f;                     // A row = local output column
                    uint8_t* rowp = A + (r >> 3) * 1024 + (r & 7) * 128;
                    const int c0 = (part * 2) ^ (r & 7), c1 = (part * 2 + 1) ^ (r & 7);
                    *reinterpret_cast<uint4*>(rowp + c0 * 16) = make_uint4(w0.x & mk, w0.y & mk, w0.z & mk, w0.w & mk);
                    *reinterpret_cast<uint4*>(rowp + c1 * 16) = make_uint4(w1.x & mk, w1.y & mk, w1.z & mk, w1.w & mk);
                }
            }
            // ---- B: the 128-k slice of the activations of this token tile
            uint8_t* Bm = gsm + L.b_off(s);
            const int kbyte = ks * kKStep + xci * 16;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                if (i >= nt16) break;
                const int ml = xr + 16 * i;
                int4 v = make_int4(0, 0, 0, 0);
                if (m0 + ml < p.M && kbyte < p.K)
                    v = *reinterpret_cast<const int4*>(p.X + (size_t)(m0 + ml) * p.K + kbyte);
                *reinterpret_cast<int4*>(Bm + (ml >> 3) * 1024 + (ml & 7) * 128 + ((xci ^ (ml & 7)) * 16)) = v;
                int sacc = psum[i];
                sacc = __dp4a(v.x, 0x01010101, sacc);
                sacc = __dp4a(v.y, 0x01010101, sacc);
                sacc = __dp4a(v.z, 0x01010101, sacc);
                sacc = __dp4a(v.w, 0x01010101, sacc);
                psum[i] = sacc;
            }
            fence_async_smem();          // make the generic-proxy stores visible to the tensor core
            __syncwarp();
            if (lane == 0) mbar_arrive(&full[s]);
        }
        // row sums of X over this CTA's K range (8 lanes share a row)
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            int v = psum[i];
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            v += __shfl_xor_sync(0xffffffffu, v, 2);
            v += __shfl_xor_sync(0xffffffffu, v, 4);
            if (xci == 0 && i < p.tokens / 16) xsum_s[xr + 16 * i] = v;
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
            tc_fence_after();
            const uint64_t adesc = umma_desc_sw128(smem_u32(gsm + L.a_off(s)));
            const uint64_t bdesc = umma_desc_sw128(smem_u32(gsm + L.b_off(s)));
#pragma unroll
            for (int kk = 0; kk < kKStep / 32; ++kk) {
                const uint32_t accum = (it > 0 || kk > 0) ? 1u : 0u;
                asm volatile(
                    "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                    "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
                    ::"r"(tmem_base), "l"(adesc + (uint64_t)(kk * 2)), "l"(bdesc + (uint64_t)(kk * 2)), "r"(idesc),
                      "r"(accum)
                    : "memory");
            }
            // release the stage when the MMAs that read it have completed
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                             smem_u32(&empty[s]))
                         : "memory");
        }
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(done))
                     : "memory");
    }
    __syncwarp();

    if (warp < 4) {
        // ------------------------------------------------------------------ epilogue
        asm volatile("bar.sync 1, 128;" ::: "memory");     // xsum_s complete (producer warps only)
        const bool ok = n_steps > 0 && mbar_wait_abortable(done, 0, abort_flag, p.status);
        tc_fence_after();
        const int nl = warp * 32 + lane;                   // TMEM lane = local output column
        const int n = tile * kTileN + nl;
        const int shift = 2 * (nl & 3);
        if (ok) {
            for (int c0 = 0; c0 < p.tokens; c0 += 16) {
                uint32_t d[16];
                const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0;
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                    : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]), "=r"(d[4]), "=r"(d[5]), "=r"(d[6]), "=r"(d[7]),
                      "=r"(d[8]), "=r"(d[9]), "=r"(d[10]), "=r"(d[11]), "=r"(d[12]), "=r"(d[13]), "=r"(d[14]), "=r"(d[15])
                    : "r"(taddr));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (n < p.N) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int m = m0 + c0 + j;
                        if (m >= p.M) break;
                        const size_t o = (size_t)m * p.N + n;
                        if (p.ksplits > 1) {
                            atomicAdd(&p.part[o], (int)d[j]);
                        } else {
                            const int v = ((int)d[j] >> shift) - xsum_s[c0 + j];
                            if (p.acc_out) p.acc_out[o] = v;
                            if (p.out) p.out[o] = (float)v * (p.x_scales[m] * p.w_scale);
                        }
                    }
                }
            }
            if (p.ksplits > 1 && tile == 0) {
                // each K range contributes its part of the row sums once (tile 0 only)
                for (int i = tid; i < p.tokens; i += 128)
                    if (m0 + i < p.M) atomicAdd(&p.part_xsum[m0 + i], xsum_s[i]);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 4) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)p.tmem_cols)
                     : "memory");
    }
}

// Split-K second pass: out[m][n] = float((part[m][n] >> 2*(n%4)) - xsum[m]) * (x_scales[m] * w_scale).
__global__ void __launch_bounds__(256) gemm_finalize_kernel(const GemmParams p) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t total = (size_t)p.M * p.N;
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (size_t)gridDim.x * 256) {
        const int m = (int)(i / p.N), n = (int)(i % p.N);
        const int v = (p.part[i] >> (2 * (n & 3))) - p.part_xsum[m];
        if (p.acc_out) p.acc_out[i] = v;
        if (p.out) p.out[i] = (float)v * (p.x_scales[m] * p.w_scale);
    }
}

}  // namespace

size_t gemm_scratch_ints(int M, int N) { return (size_t)M * (size_t)N + (size_t)M; }

cudaError_t launch_gemm(const GemmParams& p_in, int sm_count, bool pdl, cudaStream_t st) {
    GemmParams p = p_in;
    if (p.M < 1 || p.K % 16 != 0 || p.Kpad % kKStep != 0) return cudaErrorInvalidValue;
    // token tile: multiple of 16, at most 256 (the N extent of one MMA)
    int tokens = (p.M + 15) / 16 * 16;
    if (tokens > 256) tokens = 256;
    p.tokens = tokens;
    int cols = 32;
    while (cols < tokens) cols *= 2;
    p.tmem_cols = cols;
    const int m_tiles = (p.M + tokens - 1) / tokens;
    const int n_tiles = (p.n_strips + 7) / 8;
    const int steps = p.Kpad / kKStep;
    // split K so that the grid covers the SMs (the weights are the traffic; every CTA streams its share)
    int ksplits = 1;
    if (p.part) {
        ksplits = sm_count / (n_tiles * m_tiles);
        if (ksplits > steps / 4) ksplits = steps / 4;
        if (ksplits < 1) ksplits = 1;
    }
    p.ksplits = ksplits;
    GemmSmemLayout L{4, tokens};
    while (L.stages > 2 && L.bytes() > 200 * 1024) --L.stages;
    p.stages = L.stages;
    const size_t smem = (size_t)L.bytes();
    static bool attr_set[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (!attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_trit_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    cudaError_t e;
    if (ksplits > 1) {
        e = cudaMemsetAsync(p.part, 0, gemm_scratch_ints(p.M, p.N) * sizeof(int), st);
        if (e != cudaSuccess) return e;
        p.part_xsum = p.part + (size_t)p.M * p.N;
    }
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3((unsigned)n_tiles, (unsigned)ksplits, (unsigned)m_tiles);
    lc.blockDim = dim3(kGemmThreads);
    lc.dynamicSmemBytes = smem;
    lc.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = attr;
    lc.numAttrs = (pdl && ksplits == 1) ? 1 : 0;   // after a memset node keep plain stream order
    e = cudaLaunchKernelEx(&lc, gemm_trit_kernel, p);
    if (e != cudaSuccess || ksplits == 1) return e;
    cudaLaunchConfig_t lf = {};
    size_t g = ((size_t)p.M * p.N + 255) / 256;
    lf.gridDim = dim3((unsigned)(g > (size_t)sm_count * 8 ? (size_t)sm_count * 8 : g));
    lf.blockDim = dim3(256);
    lf.stream = st;
    lf.attrs = attr;
    lf.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&lf, gemm_finalize_kernel, p);
}

}  // namespace terb
