// Packed-trit GEMV, M = 1, for sm_100a.
//
// Computes what the reference's mm_packed_v4 computes
// (cuda/ter_cuda_forward_packed.cu:346-397) and what the CPU mm_row computes for int8
// activations (src/tx/forward.cpp:299-352):
//     out[j] = (float)(sum_k x[k] * trit(k, j)) * (x_scale[0] * w_scale)
// with the integer sum exact.
//
// Design (bandwidth kernel; the weights are read exactly once):
//   * a tile = 16 output columns x all of K = 4*Kpad contiguous bytes of the internal
//     layout (kernels.h).  One thread issues ONE 1-D TMA bulk copy per tile into a
//     ring of shared-memory stages; an mbarrier per stage counts the bytes in.
//   * CTAs are persistent over tiles (tile = blockIdx.x + i*gridDim.x); the copies
//     for the first `stages` tiles are issued BEFORE griddepcontrol.wait, so under
//     programmatic dependent launch the weight stream of this GEMV overlaps the
//     kernel that is still producing x.
//   * 8 warps split K in 128-byte chunks; lane = (byte-column 0..3, 16-byte segment
//     0..7): one LDS.128 of weights + one LDS.128 of x feed 16 AND + 16 dp4a.
//     Field i of every byte is column i, so  dp4a(x4, w & (0x03030303 << 2i))  adds
//     4^i * sum x*u  for column i: no shifts, no sign decode.  u = trit + 1, so the
//     true dot product is (acc >> 2i) - sum_k x[k].
//   * int32 partials are reduced by shuffles over the 8 segment lanes and through
//     shared memory over the 8 warps; integer addition is associative, so the result
//     is bit-exact whatever the grid.
#include "common.cuh"
#include "kernels.h"

namespace terb {

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kMaxStages = 8;
// Fixed shared-memory header: barriers, reduction scratch, sum of x.
constexpr int kBarOff = 0;                       // 8 x u64
constexpr int kRedOff = 64;                      // int[2][8][16]
constexpr int kXsumOff = kRedOff + 2 * kWarps * 16 * 4;   // 1088
constexpr int kHdrBytes = 1152;                  // multiple of 128

__device__ __forceinline__ void mac16(uint32_t w, int x, int& a0, int& a1, int& a2, int& a3) {
    a0 = dp4a_su(x, w & 0x03030303u, a0);
    a1 = dp4a_su(x, w & 0x0C0C0C0Cu, a1);
    a2 = dp4a_su(x, w & 0x30303030u, a2);
    a3 = dp4a_su(x, w & 0xC0C0C0C0u, a3);
}

__device__ __forceinline__ const uint8_t* tile_src(const GemvParams& p, int tile, int& m, int& lt) {
    m = 0;
#pragma unroll
    for (int i = 1; i < kGemvMaxGroup; ++i)
        if (i < p.n_mats && tile >= p.tile_begin[i]) m = i;
    lt = tile - p.tile_begin[m];
    return p.W[m] + (size_t)lt * (size_t)(4 * p.Kpad);
}

__global__ void __launch_bounds__(kThreads) gemv_trit_kernel(const __grid_constant__ GemvParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kBarOff);
    int* red = reinterpret_cast<int*>(smem + kRedOff);
    int* xsum_s = reinterpret_cast<int*>(smem + kXsumOff);
    int8_t* xs = reinterpret_cast<int8_t*>(smem + kHdrBytes);
    uint8_t* wbuf = smem + kHdrBytes + p.Kpad;

    const int tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    const int S = p.stages;
    const uint32_t tile_bytes = 4u * (uint32_t)p.Kpad;

    if (tid == 0) {
        for (int i = 0; i < S; ++i) mbar_init(&bars[i], 1);
        *xsum_s = 0;
        mbar_fence_init();
    }
    __syncthreads();

    // Weights are immutable: start streaming them before waiting on the producer of x.
    if (tid == 0) {
        for (int i = 0; i < S; ++i) {
            int tile = blockIdx.x + i * gridDim.x;
            if (tile < p.n_tiles) {
                int m, lt;
                const uint8_t* src = tile_src(p, tile, m, lt);
                mbar_arrive_expect_tx(&bars[i], tile_bytes);
                bulk_g2s(wbuf + (size_t)i * tile_bytes, src, tile_bytes, &bars[i]);
            }
        }
    }
    pdl_launch_dependents();
    pdl_wait();

    // Stage x (int8[K], zero-padded to Kpad) and sum it.
    {
        int local = 0;
        for (int i = tid * 16; i < p.Kpad; i += kThreads * 16) {
            int4 v = make_int4(0, 0, 0, 0);
            if (i < p.K) v = *reinterpret_cast<const int4*>(p.x + i);
            *reinterpret_cast<int4*>(xs + i) = v;
            local = __dp4a(v.x, 0x01010101, local);
            local = __dp4a(v.y, 0x01010101, local);
            local = __dp4a(v.z, 0x01010101, local);
            local = __dp4a(v.w, 0x01010101, local);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
        if (lane == 0 && local != 0) atomicAdd(xsum_s, local);
    }
    __syncthreads();
    const int xsum = *xsum_s;
    const float xscale = p.x_scale ? p.x_scale[0] : p.x_scale_imm;

    const int c = lane >> 3, sgm = lane & 7;
    const int n_chunks = p.Kpad >> 7;
    const int8_t* xp = xs + sgm * 16;

    int it = 0;
    for (int tile = blockIdx.x; tile < p.n_tiles; tile += gridDim.x, ++it) {
        const int stage = it % S;
        const uint32_t parity = (uint32_t)(it / S) & 1u;
        mbar_wait_bounded(&bars[stage], parity, p.status);

        const uint8_t* wt = wbuf + (size_t)stage * tile_bytes + (size_t)c * p.Kpad + sgm * 16;
        int a0 = 0, a1 = 0, a2 = 0, a3 = 0;
#pragma unroll 2
        for (int ch = warp; ch < n_chunks; ch += kWarps) {
            const uint4 w = *reinterpret_cast<const uint4*>(wt + ch * 128);
            const int4 xv = *reinterpret_cast<const int4*>(xp + ch * 128);
            mac16(w.x, xv.x, a0, a1, a2, a3);
            mac16(w.y, xv.y, a0, a1, a2, a3);
            mac16(w.z, xv.z, a0, a1, a2, a3);
            mac16(w.w, xv.w, a0, a1, a2, a3);
        }
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) {
            a0 += __shfl_xor_sync(0xffffffffu, a0, o);
            a1 += __shfl_xor_sync(0xffffffffu, a1, o);
            a2 += __shfl_xor_sync(0xffffffffu, a2, o);
            a3 += __shfl_xor_sync(0xffffffffu, a3, o);
        }
        int* rbuf = red + (it & 1) * (kWarps * 16);
        if (sgm == 0) {
            int* r = rbuf + warp * 16 + c * 4;
            r[0] = a0; r[1] = a1; r[2] = a2; r[3] = a3;
        }
        __syncthreads();   // every read of this stage is done; partials are visible

        if (tid == 0) {    // refill the stage with the tile `S` rounds ahead
            int nt = tile + S * gridDim.x;
            if (nt < p.n_tiles) {
                int m, lt;
                const uint8_t* src = tile_src(p, nt, m, lt);
                mbar_arrive_expect_tx(&bars[stage], tile_bytes);
                bulk_g2s(wbuf + (size_t)stage * tile_bytes, src, tile_bytes, &bars[stage]);
            }
        }
        if (tid < 16) {
            int sum = 0;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) sum += rbuf[w * 16 + tid];
            const int v = (sum >> (2 * (tid & 3))) - xsum;
            int m, lt;
            (void)tile_src(p, tile, m, lt);
            const int col = lt * 16 + tid;
            if (col < p.N[m]) {
                if (p.acc_out[m]) p.acc_out[m][col] = v;
                if (p.out[m]) p.out[m][col] = (float)v * (xscale * p.w_scale[m]);
            }
        }
    }
}

}  // namespace

static size_t gemv_smem_bytes(int Kpad, int stages) {
    return (size_t)kHdrBytes + (size_t)Kpad + (size_t)stages * 4u * (size_t)Kpad;
}

cudaError_t launch_gemv(const GemvParams& p_in, const GemvLaunchCfg& cfg, cudaStream_t st) {
    static bool attr_set[64] = {};   // the attribute is per device
    constexpr int kMaxSmem = 227 * 1024;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (!attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemv_trit_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    GemvParams p = p_in;
    const size_t tile_bytes = 4u * (size_t)p.Kpad;
    int stages = cfg.stages;
    if (stages <= 0) {
        // About 32 KB of weights in flight per CTA, at least a double buffer.
        stages = (int)((32 * 1024) / tile_bytes);
    }
    if (stages < 2) stages = 2;
    if (stages > kMaxStages) stages = kMaxStages;
    while (stages > 1 && gemv_smem_bytes(p.Kpad, stages) > (size_t)kMaxSmem) --stages;
    if (gemv_smem_bytes(p.Kpad, stages) > (size_t)kMaxSmem) return cudaErrorInvalidValue;
    p.stages = stages;
    const size_t smem = gemv_smem_bytes(p.Kpad, stages);

    int occ = 0;
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, gemv_trit_kernel, kThreads, smem);
    if (e != cudaSuccess) return e;
    if (occ < 1) return cudaErrorInvalidValue;
    int per_sm = cfg.ctas_per_sm < occ ? cfg.ctas_per_sm : occ;
    if (per_sm < 1) per_sm = 1;
    int grid = cfg.sm_count * per_sm;
    if (grid > p.n_tiles) grid = p.n_tiles;
    if (grid < 1) return cudaErrorInvalidValue;

    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3((unsigned)grid);
    lc.blockDim = dim3(kThreads);
    lc.dynamicSmemBytes = smem;
    lc.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = attr;
    lc.numAttrs = cfg.pdl ? 1 : 0;
    return cudaLaunchKernelEx(&lc, gemv_trit_kernel, p);
}

}  // namespace terb
