// Packed-trit GEMV, M = 1, for sm_100a.
//
// Computes what the reference's mm_packed_v4 computes
// (cuda/ter_cuda_forward_packed.cu:346-397) and what the CPU mm_row computes for int8
// activations (src/tx/forward.cpp:299-352):
//     out[j] = (float)(sum_k x[k] * trit(k, j)) * (x_scale[0] * w_scale)
// with the integer sum exact.
//
// Design (bandwidth kernel; every weight byte is read exactly once):
//   * Work unit: a strip = 16 output columns x all of K, stored as contiguous blocks of
//     [4 byte-columns][<=1024 k] (kernels.h).  Each WARP owns whole strips and streams
//     their blocks through its own ring of shared-memory stages: lane 0 issues one 1-D
//     TMA bulk copy per block, an mbarrier per stage counts the bytes in.  Warps never
//     synchronise with each other after the prologue, so there is no per-strip
//     __syncthreads and no cross-warp reduction.
//   * The copies for the first `stages` blocks are issued BEFORE griddepcontrol.wait:
//     under programmatic dependent launch the weight stream of this GEMV starts while
//     the kernel that produces x is still running.  x (int8[K]) is then staged once per
//     CTA in shared memory and shared by the 8 warps.
//   * lane = (byte-column c = lane/8, 16-byte segment s = lane%8); per 128 k a lane does
//     one LDS.128 of weights + one LDS.128 of x feeding 16 AND + 16 dp4a.  Field i of
//     every weight byte is column i, so dp4a(x4, w & (0x03030303 << 2i)) accumulates
//     4^i * sum x*u for column i: no shifts, no sign decode.  u = trit + 1, so the true
//     dot product is (acc >> 2i) - sum_k x[k].
//   * The 8 segment lanes of a byte-column are reduced with 3 xor-shuffles per strip.
//     Integer addition is associative: the result is bit-exact whatever the grid.
#include "common.cuh"
#include "kernels.h"
#include "normq.cuh"

namespace terb {

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kMaxStages = 8;
constexpr int kStageBytes = 4 * kGemvKC;
// Fixed shared-memory header.
constexpr int kBarOff = 0;                          // u64[kWarps][kMaxStages] = 512 B
constexpr int kXsumOff = kWarps * kMaxStages * 8;   // 512
constexpr int kHdrBytes = 640;                      // multiple of 128

// Matrix and local strip of global strip number `strip` (by-value parameter arrays).
__device__ __forceinline__ void locate(const GemvParams& p, int strip, int& m, int& ls) {
    m = 0;
#pragma unroll
    for (int i = 1; i < kGemvMaxGroup; ++i)
        if (i < p.n_mats && strip >= p.tile_begin[i]) m = i;
    ls = strip - p.tile_begin[m];
}

// Shared-memory bytes of a table-mode launch: the descriptors plus a coarse index (for every 64th strip the
// matrix that holds it), which replaces a binary search per strip by a short scan.
constexpr int kCoarseShift = 6;     // one coarse entry per 64 strips
__host__ __device__ inline int gemv_table_bytes(int n_mats, int n_tiles) {
    const int desc = (n_mats * (int)sizeof(GemvDesc) + 15) & ~15;
    const int coarse = ((n_tiles >> kCoarseShift) + 1) * 2;
    return (desc + coarse + 127) & ~127;
}

// Per-matrix fields of strip `strip`: from the by-value parameter arrays, or (TABLE) from the
// descriptor table that the CTA copied into shared memory.
struct MatRef {
    const uint8_t* W;
    float* out;
    int32_t* acc;
    float w_scale;
    int N, xid, ls;
};

template <bool TABLE>
__device__ __forceinline__ MatRef locate(const GemvParams& p, const GemvDesc* tab, int strip) {
    MatRef r;
    if constexpr (TABLE) {
        // last matrix whose first strip is <= strip: start from the coarse index, scan forward
        const uint16_t* coarse = reinterpret_cast<const uint16_t*>(reinterpret_cast<const uint8_t*>(tab) +
                                                                   ((p.n_mats * (int)sizeof(GemvDesc) + 15) & ~15));
        int lo = coarse[strip >> kCoarseShift];
        while (lo + 1 < p.n_mats && tab[lo + 1].tile_begin <= strip) ++lo;
        const GemvDesc d = tab[lo];
        r.W = d.W; r.out = d.out; r.acc = nullptr; r.w_scale = d.w_scale; r.N = d.N; r.xid = d.xid;
        r.ls = strip - d.tile_begin;
    } else {
        int m = 0;
#pragma unroll
        for (int i = 1; i < kGemvMaxGroup; ++i)
            if (i < p.n_mats && strip >= p.tile_begin[i]) m = i;
        r.W = p.W[m]; r.out = p.out[m]; r.acc = p.acc_out[m]; r.w_scale = p.w_scale[m]; r.N = p.N[m];
        r.xid = p.xid[m];
        r.ls = strip - p.tile_begin[m];
    }
    return r;
}

template <bool TABLE>
__global__ void __launch_bounds__(kThreads) gemv_trit_kernel(const __grid_constant__ GemvParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kBarOff);
    int* xsum_s = reinterpret_cast<int*>(smem + kXsumOff);           // one per activation vector
    const int tab_bytes = TABLE ? gemv_table_bytes(p.n_mats, p.n_tiles) : 0;
    GemvDesc* tab = reinterpret_cast<GemvDesc*>(smem + kHdrBytes);
    int8_t* xs = reinterpret_cast<int8_t*>(smem + kHdrBytes + tab_bytes);
    uint8_t* wbuf = smem + kHdrBytes + tab_bytes + p.x_bytes;

    const int tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    const int S = p.stages;
    uint64_t* mybars = bars + warp * kMaxStages;
    uint8_t* mybuf = wbuf + (size_t)warp * S * kStageBytes;
    // strip t is handled by CTA t % gridDim, warp (t / gridDim) % 8: strips spread over SMs first
    const int first = blockIdx.x + gridDim.x * warp;
    const int stride = gridDim.x * kWarps;

    if (lane == 0) {
        for (int i = 0; i < S; ++i) mbar_init(&mybars[i], 1);
        mbar_fence_init();
    }
    if (tid < kGemvMaxX) xsum_s[tid] = 0;
    if constexpr (TABLE) {
        // the table is written once when the plan is made, long before this launch
        const int4* src = reinterpret_cast<const int4*>(p.table);
        int4* dst = reinterpret_cast<int4*>(tab);
        for (int i = tid; i < p.n_mats * (int)(sizeof(GemvDesc) / 16); i += kThreads) dst[i] = src[i];
        __syncthreads();
        // coarse index: one binary search per kCoarse strips, once per CTA
        uint16_t* coarse = reinterpret_cast<uint16_t*>(reinterpret_cast<uint8_t*>(tab) + ((p.n_mats * (int)sizeof(GemvDesc) + 15) & ~15));
        for (int c = tid; c <= (p.n_tiles >> kCoarseShift); c += kThreads) {
            const int strip = c << kCoarseShift;
            int lo = 0, hi = p.n_mats - 1;
            while (lo < hi) {
                const int mid = (lo + hi + 1) >> 1;
                if (tab[mid].tile_begin <= strip) lo = mid; else hi = mid - 1;
            }
            coarse[c] = (uint16_t)lo;
        }
        __syncthreads();
    } else {
        __syncwarp();
    }

    // Producer cursor over this warp's (strip, block) items; uniform across the warp.
    int p_strip = first, p_q = 0, p_stage = 0, p_nb = 1, p_last = kGemvKC;
    const uint8_t* p_src = nullptr;
    auto cursor_load = [&]() {
        if (p_strip < p.n_tiles) {
            const MatRef r = locate<TABLE>(p, tab, p_strip);
            const int kp = p.uKpad[r.xid];
            p_nb = (kp + kGemvKC - 1) / kGemvKC;
            p_last = kp - (p_nb - 1) * kGemvKC;
            p_src = r.W + (size_t)r.ls * 4u * (size_t)kp;
        }
    };
    cursor_load();
    auto issue = [&]() {
        if (p_strip < p.n_tiles) {
            if (lane == 0) {
                const int kc = (p_q == p_nb - 1) ? p_last : kGemvKC;
                mbar_arrive_expect_tx(&mybars[p_stage], 4u * (uint32_t)kc);
                bulk_g2s(mybuf + (size_t)p_stage * kStageBytes, p_src + (size_t)p_q * kStageBytes, 4u * (uint32_t)kc,
                         &mybars[p_stage]);
            }
            if (++p_q == p_nb) { p_q = 0; p_strip += stride; cursor_load(); }
            if (++p_stage == S) p_stage = 0;
        }
    };
    // Weights are immutable: start streaming them before waiting on the producer of x.
    for (int i = 0; i < S; ++i) issue();

    pdl_launch_dependents();
    pdl_wait();

    // Stage every activation vector (int8[K_u], zero-padded to Kpad_u) once per CTA and sum it.
    for (int u = 0; u < p.n_x; ++u) {
        int local = 0;
        int8_t* dst = xs + p.uoff[u];
        const int8_t* srcx = p.ux[u];
        const int K = p.uK[u], Kpad = p.uKpad[u];
        for (int i = tid * 16; i < Kpad; i += kThreads * 16) {
            int4 v = make_int4(0, 0, 0, 0);
            if (i < K) v = *reinterpret_cast<const int4*>(srcx + i);
            *reinterpret_cast<int4*>(dst + i) = v;
            local = __dp4a(v.x, 0x01010101, local);
            local = __dp4a(v.y, 0x01010101, local);
            local = __dp4a(v.z, 0x01010101, local);
            local = __dp4a(v.w, 0x01010101, local);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
        if (lane == 0 && local != 0) atomicAdd(&xsum_s[u], local);
    }
    __syncthreads();

    const int c = lane >> 3, sgm = lane & 7;
    int stage = 0;
    uint32_t parity = 0;
    for (int strip = first; strip < p.n_tiles; strip += stride) {
        const MatRef r = locate<TABLE>(p, tab, strip);
        const int kp = p.uKpad[r.xid];
        const int nb = (kp + kGemvKC - 1) / kGemvKC;
        const int last_kc = kp - (nb - 1) * kGemvKC;
        const int8_t* xm = xs + p.uoff[r.xid] + sgm * 16;
        int a0 = 0, a1 = 0, a2 = 0, a3 = 0;
        for (int q = 0; q < nb; ++q) {
            const int kc = (q == nb - 1) ? last_kc : kGemvKC;
            mbar_wait_sleepy(&mybars[stage], parity, p.status);
            const uint8_t* wt = mybuf + (size_t)stage * kStageBytes + c * kc + sgm * 16;
            const int8_t* xp = xm + q * kGemvKC;
            if (kc == kGemvKC) {
#pragma unroll
                for (int j = 0; j < kGemvKC / 128; ++j)
                    mac64(*reinterpret_cast<const uint4*>(wt + j * 128), *reinterpret_cast<const int4*>(xp + j * 128),
                          a0, a1, a2, a3);
            } else {
                for (int j = 0; j < (kc >> 7); ++j)
                    mac64(*reinterpret_cast<const uint4*>(wt + j * 128), *reinterpret_cast<const int4*>(xp + j * 128),
                          a0, a1, a2, a3);
            }
            __syncwarp();          // every lane has finished reading this stage
            issue();               // refill it with the block `S` items ahead
            if (++stage == S) { stage = 0; parity ^= 1u; }
        }
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) {
            a0 += __shfl_xor_sync(0xffffffffu, a0, o);
            a1 += __shfl_xor_sync(0xffffffffu, a1, o);
            a2 += __shfl_xor_sync(0xffffffffu, a2, o);
            a3 += __shfl_xor_sync(0xffffffffu, a3, o);
        }
        if (sgm == 0) {
            const int xsum = xsum_s[r.xid];
            const float xscale = p.uxs[r.xid] ? p.uxs[r.xid][0] : p.x_scale_imm;
            const int col = r.ls * 16 + c * 4;
            const int v0 = (a0 - a1 - a2 - a3) - xsum, v1 = (a1 >> 2) - xsum, v2 = (a2 >> 4) - xsum, v3 = (a3 >> 6) - xsum;
            const int N = r.N;
            if (int32_t* ao = r.acc) {
                if (col + 3 < N && ((reinterpret_cast<uintptr_t>(ao) & 15u) == 0)) {
                    *reinterpret_cast<int4*>(ao + col) = make_int4(v0, v1, v2, v3);
                } else {
                    if (col < N) ao[col] = v0;
                    if (col + 1 < N) ao[col + 1] = v1;
                    if (col + 2 < N) ao[col + 2] = v2;
                    if (col + 3 < N) ao[col + 3] = v3;
                }
            }
            if (float* fo = r.out) {
                const float sc = xscale * r.w_scale;
                float f0 = (float)v0 * sc, f1 = (float)v1 * sc, f2 = (float)v2 * sc, f3 = (float)v3 * sc;
                if (p.accumulate) {
                    if (col < N) f0 = fo[col] + f0;
                    if (col + 1 < N) f1 = fo[col + 1] + f1;
                    if (col + 2 < N) f2 = fo[col + 2] + f2;
                    if (col + 3 < N) f3 = fo[col + 3] + f3;
                }
                if (col + 3 < N && ((reinterpret_cast<uintptr_t>(fo) & 15u) == 0)) {
                    *reinterpret_cast<float4*>(fo + col) = make_float4(f0, f1, f2, f3);
                } else {
                    if (col < N) fo[col] = f0;
                    if (col + 1 < N) fo[col + 1] = f1;
                    if (col + 2 < N) fo[col + 2] = f2;
                    if (col + 3 < N) fo[col + 3] = f3;
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------
// Latency path for matrices with few strips (every projection except the lm_head).
// One CTA per strip; the 8 warps split K in 128-byte chunks (chunk j -> warp j % 8).
// Each lane fetches its weights with 16-byte read-only global loads straight into
// registers BEFORE griddepcontrol.wait, so when the producer of x finishes the only
// work left on the critical path is: load x (L2), 16 AND + 16 dp4a per chunk, a
// shuffle + shared-memory reduction, one store.  No TMA ring, no staging of x.
// ---------------------------------------------------------------------------------
constexpr int kSplitBatch = 8;   // chunks per warp held in registers at once (covers K <= 8192)

__device__ __forceinline__ uint4 ldg_stream(const uint8_t* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// SPC = strips handled by one CTA at once (1, 2 or 4); a strip then has at most 8/SPC chunks per
// warp in registers (SPC = 1 loops over further batches for long K).  Fatter CTAs keep the grid
// within one wave, so the per-CTA prologue (fused quantiser) is paid once per SM slot.
// p.act_pair (needs SPC >= 2, exactly two matrices gate and up): the CTA takes the SAME strip
// range of both matrices and writes act(gate, up) = silu(g)*u or relu(g)^2*u for its columns to
// p.act_out instead of the two raw projections.
template <int SPC>
__global__ void __launch_bounds__(kThreads) gemv_trit_split_kernel(const __grid_constant__ GemvParams p) {
    constexpr int CPW = kSplitBatch / SPC;            // register slots (chunks per warp) per strip
    extern __shared__ __align__(16) uint8_t fsm[];    // fused prologue only: float vals[K] | int8 xq[Kpad]
    __shared__ int red[kWarps][SPC * 16 + 4];
    __shared__ float red_f[2 * kWarps];
    const int tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    const int c = lane >> 3, sgm = lane & 7;
    const int n_chunks = p.Kpad >> 7;
    const int nb = (p.Kpad + kGemvKC - 1) / kGemvKC;
    const int last_kc = p.Kpad - (nb - 1) * kGemvKC;

    // strips of this CTA
    int sm[SPC], sls[SPC];
    const uint8_t* sbase[SPC];
#pragma unroll
    for (int i = 0; i < SPC; ++i) {
        int m, ls;
        if (p.act_pair) {
            constexpr int HALF = SPC >= 2 ? SPC / 2 : 1;
            m = i / HALF;
            ls = blockIdx.x * HALF + (i % HALF);
            if (ls >= p.tile_begin[1]) ls = -1;               // both matrices have tile_begin[1] strips
        } else {
            const int strip = blockIdx.x * SPC + i;
            if (strip < p.n_tiles) locate(p, strip, m, ls); else { m = 0; ls = -1; }
        }
        sm[i] = m; sls[i] = ls;
        sbase[i] = ls >= 0 ? p.W[m] + (size_t)ls * 4u * (size_t)p.Kpad : nullptr;
    }
    auto waddr = [&](const uint8_t* base, int j) -> const uint8_t* {
        const int q = j >> 3;                                   // 8 chunks per 1024-k block
        const int kc = (q == nb - 1) ? last_kc : kGemvKC;
        return base + (size_t)q * kStageBytes + c * kc + (j & 7) * 128 + sgm * 16;
    };

    uint4 w[kSplitBatch];
#pragma unroll
    for (int i = 0; i < kSplitBatch; ++i) {
        const int si = i / CPW, j = warp + kWarps * (i % CPW);
        w[i] = (sbase[si] && j < n_chunks) ? ldg_stream(waddr(sbase[si], j)) : make_uint4(0, 0, 0, 0);
    }
    if (p.fuse.x) norm_quant_prefetch_gamma(p.fuse);
    pdl_launch_dependents();
    pdl_wait();

    const int8_t* xsrc = p.x;
    float xscale_f = 0.0f;
    if (p.fuse.x) {
        float* vals = reinterpret_cast<float*>(fsm);
        int8_t* xq = reinterpret_cast<int8_t*>(fsm + 4 * (size_t)((p.K + 3) & ~3));
        xscale_f = norm_quant_fast_ok(p.fuse, p.fuse_row, xq, nullptr)
                       ? block_norm_quant_fast(p.fuse, p.fuse_row, red_f, xq, nullptr)
                       : block_norm_quant(p.fuse, p.fuse_row, vals, red_f, xq, nullptr);
        __syncthreads();
        xsrc = xq;
    }

    int acc[SPC][4];
#pragma unroll
    for (int i = 0; i < SPC; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0;
    int xl = 0;
    const int n_batches = SPC == 1 ? (n_chunks + kSplitBatch * kWarps - 1) / (kSplitBatch * kWarps) : 1;
    for (int b = 0; b < n_batches; ++b) {
        if (b > 0) {
#pragma unroll
            for (int i = 0; i < kSplitBatch; ++i) {
                const int j = warp + kWarps * (i + b * kSplitBatch);
                w[i] = (sbase[0] && j < n_chunks) ? ldg_stream(waddr(sbase[0], j)) : make_uint4(0, 0, 0, 0);
            }
        }
#pragma unroll
        for (int i = 0; i < kSplitBatch; ++i) {
            const int si = i / CPW;
            const int j = warp + kWarps * ((i % CPW) + b * kSplitBatch);
            const int k0 = j * 128 + sgm * 16;
            int4 xv = make_int4(0, 0, 0, 0);
            if (j < n_chunks && k0 < p.K) xv = *reinterpret_cast<const int4*>(xsrc + k0);
            mac64(w[i], xv, acc[si][0], acc[si][1], acc[si][2], acc[si][3]);
            if (si == 0) {
                xl = __dp4a(xv.x, 0x01010101, xl);
                xl = __dp4a(xv.y, 0x01010101, xl);
                xl = __dp4a(xv.z, 0x01010101, xl);
                xl = __dp4a(xv.w, 0x01010101, xl);
            }
        }
    }
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) {
#pragma unroll
        for (int i = 0; i < SPC; ++i) {
            acc[i][0] += __shfl_xor_sync(0xffffffffu, acc[i][0], o);
            acc[i][1] += __shfl_xor_sync(0xffffffffu, acc[i][1], o);
            acc[i][2] += __shfl_xor_sync(0xffffffffu, acc[i][2], o);
            acc[i][3] += __shfl_xor_sync(0xffffffffu, acc[i][3], o);
        }
        xl += __shfl_xor_sync(0xffffffffu, xl, o);
    }
    if (sgm == 0) {
#pragma unroll
        for (int i = 0; i < SPC; ++i) {
            int* r = &red[warp][i * 16 + c * 4];
            r[0] = acc[i][0] - acc[i][1] - acc[i][2] - acc[i][3];
            r[1] = acc[i][1]; r[2] = acc[i][2]; r[3] = acc[i][3];
        }
        if (c == 0) red[warp][SPC * 16] = xl;
    }
    __syncthreads();
    const float xscale = p.fuse.x ? xscale_f : (p.x_scale ? p.x_scale[0] : p.x_scale_imm);
    auto column_value = [&](int si, int lc) -> int {
        int sum = 0, xsum = 0;
#pragma unroll
        for (int wi = 0; wi < kWarps; ++wi) { sum += red[wi][si * 16 + lc]; xsum += red[wi][SPC * 16]; }
        return (sum >> (2 * (lc & 3))) - xsum;
    };
    if (p.act_pair) {
        constexpr int HALF = SPC >= 2 ? SPC / 2 : 1;
        if (tid < HALF * 16) {
            const int si = tid >> 4, lc = tid & 15;
            if (sls[si] >= 0) {
                const int col = sls[si] * 16 + lc;
                if (col < p.N[0]) {
                    const float g = (float)column_value(si, lc) * (xscale * p.w_scale[0]);
                    const float u = (float)column_value(si + HALF, lc) * (xscale * p.w_scale[1]);
                    p.act_out[col] = pre_op(p.act_pair, g, u);
                }
            }
        }
    } else if (tid < SPC * 16) {
        const int si = tid >> 4, lc = tid & 15;
        if (sls[si] >= 0) {
            const int m = sm[si];
            const int col = sls[si] * 16 + lc;
            if (col < p.N[m]) {
                const int v = column_value(si, lc);
                if (p.acc_out[m]) p.acc_out[m][col] = v;
                if (p.out[m]) {
                    const float f = (float)v * (xscale * p.w_scale[m]);
                    p.out[m][col] = p.accumulate ? p.out[m][col] + f : f;
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------
// Small token batches (2 <= M <= 16 rows of X against the same weights), one launch for up to
// kGemvMaxGroup matrices: the weights stream ONCE (16-byte read-only loads into registers, one CTA per
// strip, the 8 warps split K as in the latency path) and every unpacked word feeds the multiply-adds of
// all rows.  Below the token count where the tensor-core GEMM pays, this replaces one GEMV launch per
// row (the reference's batched decode does the same per-row work, cuda/ter_cuda_addonly_batched.cu:32-123).
// Rows are processed RB at a time (accumulators in registers); a second pass re-reads the strip from L2.
// ---------------------------------------------------------------------------------
template <int RB>
__global__ void __launch_bounds__(kThreads, 2) gemv_trit_rows_kernel(const __grid_constant__ GemvParams p) {
    extern __shared__ __align__(16) uint8_t xrows[];   // [RB][Kpad] int8: the rows of this pass, zero-padded
    __shared__ int red[kWarps][RB][16];
    __shared__ int xsum_s[RB];                // sum of each staged row
    const int tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    const int c = lane >> 3, sgm = lane & 7;
    const int n_chunks = p.Kpad >> 7;
    const int nb = (p.Kpad + kGemvKC - 1) / kGemvKC;
    const int last_kc = p.Kpad - (nb - 1) * kGemvKC;
    constexpr int CB = 4;                    // chunks per warp held in registers at once
    const int n_batches = (n_chunks + CB * kWarps - 1) / (CB * kWarps);
    // chunk j of strip `strip` for this lane (chunk j -> warp j % kWarps)
    auto load_batch = [&](int strip, int bt, uint4 (&w)[CB]) {
        int m, ls;
        locate(p, strip, m, ls);
        const uint8_t* sbase = p.W[m] + (size_t)ls * 4u * (size_t)p.Kpad;
#pragma unroll
        for (int i = 0; i < CB; ++i) {
            const int j = warp + kWarps * (i + bt * CB);
            if (j < n_chunks) {
                const int q = j >> 3;
                const int kc = (q == nb - 1) ? last_kc : kGemvKC;
                w[i] = ldg_stream(sbase + (size_t)q * kStageBytes + c * kc + (j & 7) * 128 + sgm * 16);
            }
        }
    };
    uint4 w[CB];
    int strip = (int)blockIdx.x;
    load_batch(strip, 0, w);                 // weights are immutable: fetched before the producer of x is waited for
    bool preloaded = true;                   // w holds batch 0 of the strip about to be processed
    pdl_launch_dependents();
    pdl_wait();
    for (int r0 = 0; r0 < p.rows; r0 += RB) {
        // stage the rows of this pass in shared memory with one batch of coalesced 16-byte loads, then sum each
        {
            const int per_row = p.Kpad >> 4;
            for (int i = tid; i < RB * per_row; i += kThreads) {
                const int rr = i / per_row, k0 = (i - rr * per_row) << 4;
                int4 v = make_int4(0, 0, 0, 0);
                if (r0 + rr < p.rows && k0 < p.K) v = *reinterpret_cast<const int4*>(p.x + (size_t)(r0 + rr) * p.K + k0);
                *reinterpret_cast<int4*>(xrows + (size_t)rr * p.Kpad + k0) = v;
            }
            __syncthreads();
            if (warp < RB) {
                int local = 0;
                for (int i = lane; i < per_row; i += 32) {
                    const int4 v = *reinterpret_cast<const int4*>(xrows + (size_t)warp * p.Kpad + (i << 4));
                    local = __dp4a(v.x, 0x01010101, local);
                    local = __dp4a(v.y, 0x01010101, local);
                    local = __dp4a(v.z, 0x01010101, local);
                    local = __dp4a(v.w, 0x01010101, local);
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
                if (lane == 0) xsum_s[warp] = local;
            }
        }
        // this CTA's strips: blockIdx, blockIdx + grid, ...
        for (strip = (int)blockIdx.x; strip < p.n_tiles; strip += (int)gridDim.x) {
            int m, ls;
            locate(p, strip, m, ls);
            int acc[RB][4];
#pragma unroll
            for (int rr = 0; rr < RB; ++rr) acc[rr][0] = acc[rr][1] = acc[rr][2] = acc[rr][3] = 0;
            for (int bt = 0; bt < n_batches; ++bt) {
                if (bt > 0 || !preloaded) load_batch(strip, bt, w);
                preloaded = false;
#pragma unroll
                for (int i = 0; i < CB; ++i) {
                    const int j = warp + kWarps * (i + bt * CB);
                    if (j < n_chunks) {                     // uniform over the warp
                        const int k0 = j * 128 + sgm * 16;
#pragma unroll
                        for (int rr = 0; rr < RB; ++rr)
                            mac64(w[i], *reinterpret_cast<const int4*>(xrows + (size_t)rr * p.Kpad + k0), acc[rr][0],
                                  acc[rr][1], acc[rr][2], acc[rr][3]);
                    }
                }
            }
            // the 8 segment lanes of a byte-column: halve the values a lane carries at every step of the butterfly
            // (lanes whose bit is set keep the upper half), so 4 + 2 + 1 row-quads cross lanes instead of 3 x 8
            int v[RB * 4];
#pragma unroll
            for (int rr = 0; rr < RB; ++rr)
#pragma unroll
                for (int e = 0; e < 4; ++e) v[rr * 4 + e] = acc[rr][e];
            int n = RB * 4;
#pragma unroll
            for (int o = 4; o >= 1; o >>= 1) {
                const bool up = (sgm & o) != 0;
                n >>= 1;
#pragma unroll
                for (int i = 0; i < RB * 2; ++i) {
                    if (i < n) {
                        const int send = up ? v[i] : v[i + n];
                        const int keep = up ? v[i + n] : v[i];
                        v[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
                    }
                }
            }
            // lane sgm now holds values [sgm' * n, sgm' * n + n) of the RB*4, n = RB/2, with sgm' the bit-reversal
            // implied by the three steps: the index of value i is  ((sgm&4) ? RB*2 : 0) + ((sgm&2) ? RB : 0) + ((sgm&1) ? RB/2 : 0) + i
            {
                const int base = ((sgm & 4) ? RB * 2 : 0) + ((sgm & 2) ? RB : 0) + ((sgm & 1) ? RB / 2 : 0);
#pragma unroll
                for (int i = 0; i < RB / 2; ++i) {
                    const int idx = base + i, rr = idx >> 2, e = idx & 3;
                    red[warp][rr][c * 4 + e] = v[i];
                }
            }
            __syncthreads();
            // the next strip's first weights travel while this one is reduced and stored
            const int next = strip + (int)gridDim.x;
            if (next < p.n_tiles) { load_batch(next, 0, w); preloaded = true; }
            else if (r0 + RB < p.rows) { load_batch((int)blockIdx.x, 0, w); preloaded = true; }
            if (tid < RB * 16) {
                const int rr = tid >> 4, lc = tid & 15;
                const int row = r0 + rr, col = ls * 16 + lc;
                if (row < p.rows && col < p.N[m]) {
                    int sum = 0;
#pragma unroll
                    for (int wi = 0; wi < kWarps; ++wi) sum += red[wi][rr][lc];
                    // fields 1..3 of a byte-column carry 4^i times their sum; field 0 is what is left of the
                    // unmasked product after the other three are taken off
                    const int f = lc & 3;
                    int val;
                    if (f == 0) {
                        int s1 = 0, s2 = 0, s3 = 0;
#pragma unroll
                        for (int wi = 0; wi < kWarps; ++wi) { s1 += red[wi][rr][lc + 1]; s2 += red[wi][rr][lc + 2]; s3 += red[wi][rr][lc + 3]; }
                        val = sum - s1 - s2 - s3;
                    } else {
                        val = sum >> (2 * f);
                    }
                    const int vv = val - xsum_s[rr];
                    const size_t o = (size_t)row * (size_t)p.N[m] + col;
                    if (p.acc_out[m]) p.acc_out[m][o] = vv;
                    if (p.out[m]) {
                        const float fl = (float)vv * (p.x_scale[row] * p.w_scale[m]);
                        p.out[m][o] = p.accumulate ? p.out[m][o] + fl : fl;
                    }
                }
            }
            __syncthreads();
        }
    }
}

}  // namespace

static size_t gemv_smem_bytes(int tab_bytes, int x_bytes, int stages) {
    return (size_t)kHdrBytes + (size_t)tab_bytes + (size_t)x_bytes + (size_t)kWarps * (size_t)stages * kStageBytes;
}

cudaError_t launch_gemv(const GemvParams& p_in, const GemvLaunchCfg& cfg, cudaStream_t st) {
    static bool attr_set[64] = {};   // the attribute is per device
    constexpr int kMaxSmem = 227 * 1024;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (!attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemv_trit_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem);
        if (e != cudaSuccess) return e;
        e = cudaFuncSetAttribute(gemv_trit_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    if (p_in.rows >= 2) {   // a small token batch: all rows in one launch
        if (p_in.multi || p_in.fuse.x || p_in.act_pair || p_in.table || !p_in.x || (p_in.K & 15) ||
            (p_in.out[0] && !p_in.x_scale) || p_in.n_mats < 1 || p_in.n_mats > kGemvMaxGroup || p_in.rows > kGemvMaxRows)
            return cudaErrorInvalidValue;
        cudaLaunchConfig_t lc = {};
        const int rb = p_in.rows <= 4 ? 4 : 8;
        const size_t xsm = (size_t)rb * (size_t)p_in.Kpad;
        if (xsm > 200 * 1024) return cudaErrorInvalidValue;
        static bool rows_attr[64][2] = {};
        if (xsm > 40 * 1024 && !rows_attr[dev][rb == 8]) {
            cudaError_t e = rb == 8 ? cudaFuncSetAttribute(gemv_trit_rows_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)
                                    : cudaFuncSetAttribute(gemv_trit_rows_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            if (e != cudaSuccess) return e;
            rows_attr[dev][rb == 8] = true;
        }
        // two CTAs per SM, every CTA resident; a CTA takes strips blockIdx, blockIdx + grid, ... and stages x once
        const int wave = 2 * (cfg.sm_count > 0 ? cfg.sm_count : 148);
        lc.gridDim = dim3((unsigned)(p_in.n_tiles < wave ? p_in.n_tiles : wave));
        lc.blockDim = dim3(kThreads);
        lc.dynamicSmemBytes = xsm;
        lc.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        lc.attrs = attr;
        lc.numAttrs = cfg.pdl ? 1 : 0;
        return rb == 4 ? cudaLaunchKernelEx(&lc, gemv_trit_rows_kernel<4>, p_in)
                       : cudaLaunchKernelEx(&lc, gemv_trit_rows_kernel<8>, p_in);
    }
    GemvParams p = p_in;
    if (!p.multi) {   // one shared activation vector, in the form the streaming kernel reads
        p.n_x = 1;
        p.ux[0] = p.x; p.uxs[0] = p.x_scale; p.uK[0] = p.K; p.uKpad[0] = p.Kpad; p.uoff[0] = 0;
        for (int i = 0; i < kGemvMaxGroup; ++i) p.xid[i] = 0;
        p.x_bytes = p.Kpad;
        p.table = nullptr;
    }
    if (!p.multi && cfg.split_max_strips > 0 && p.n_tiles <= cfg.split_max_strips) {
        size_t fsmem = 0;
        if (p.fuse.x) {
            fsmem = 4 * (size_t)((p.K + 3) & ~3) + (size_t)p.Kpad;
            if (fsmem > (size_t)kMaxSmem - 4096) return cudaErrorInvalidValue;
        }
        // Strips per CTA: as few as keep the grid within one resident wave (about 3 CTAs per SM with the
        // fused prologue), limited by the 8 register slots per warp.
        const int cpw = ((p.Kpad >> 7) + kWarps - 1) / kWarps;
        const int max_spc = cpw <= 2 ? 4 : (cpw <= 4 ? 2 : 1);
        const int wave = cfg.sm_count * 2;   // 128 registers x 256 threads: two CTAs per SM
        int spc = 1;
        while (spc < max_spc && (p.n_tiles + spc - 1) / spc > wave) spc *= 2;
        if (p.act_pair) {
            if (p.n_mats != 2 || p.tile_begin[1] * 2 != p.n_tiles || max_spc < 2 || p.N[0] != p.N[1] || !p.act_out)
                return cudaErrorInvalidValue;
            if (spc < 2) spc = 2;
        }
        const int grid = p.act_pair ? (p.tile_begin[1] + spc / 2 - 1) / (spc / 2) : (p.n_tiles + spc - 1) / spc;
        void (*kern)(GemvParams) = spc == 4 ? gemv_trit_split_kernel<4>
                                  : (spc == 2 ? gemv_trit_split_kernel<2> : gemv_trit_split_kernel<1>);
        static bool split_attr[64][3] = {};
        const int ai = spc == 4 ? 2 : (spc == 2 ? 1 : 0);
        if (fsmem > 48 * 1024 && !split_attr[dev][ai]) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem - 4096);
            if (e != cudaSuccess) return e;
            split_attr[dev][ai] = true;
        }
        cudaLaunchConfig_t lc = {};
        lc.gridDim = dim3((unsigned)grid);
        lc.blockDim = dim3(kThreads);
        lc.dynamicSmemBytes = fsmem;
        lc.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        lc.attrs = attr;
        lc.numAttrs = cfg.pdl ? 1 : 0;
        return cudaLaunchKernelEx(&lc, kern, p);
    }
    if (p.fuse.x) return cudaErrorNotSupported;   // the streaming kernel takes a quantised x only
    if (p.table ? (p.n_mats < 1 || p.n_mats > kGemvMaxTable) : (p.n_mats < 1 || p.n_mats > kGemvMaxGroup))
        return cudaErrorInvalidValue;
    if (p.n_x < 1 || p.n_x > kGemvMaxX || p.x_bytes > kGemvMaxXBytes) return cudaErrorInvalidValue;
    const int tab_bytes = p.table ? gemv_table_bytes(p.n_mats, p.n_tiles) : 0;
    int per_sm = cfg.ctas_per_sm < 1 ? 1 : cfg.ctas_per_sm;
    int stages = cfg.stages > 0 ? cfg.stages : 3;
    if (stages > kMaxStages) stages = kMaxStages;
    // keep `per_sm` CTAs resident: shrink the ring first, then the residency
    while (stages > 2 && gemv_smem_bytes(tab_bytes, p.x_bytes, stages) * per_sm > (size_t)kMaxSmem) --stages;
    while (per_sm > 1 && gemv_smem_bytes(tab_bytes, p.x_bytes, stages) * per_sm > (size_t)kMaxSmem) --per_sm;
    while (stages > 1 && gemv_smem_bytes(tab_bytes, p.x_bytes, stages) > (size_t)kMaxSmem) --stages;
    if (gemv_smem_bytes(tab_bytes, p.x_bytes, stages) > (size_t)kMaxSmem) return cudaErrorInvalidValue;
    p.stages = stages;
    const size_t smem = gemv_smem_bytes(tab_bytes, p.x_bytes, stages);

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
    return p.table ? cudaLaunchKernelEx(&lc, gemv_trit_kernel<true>, p) : cudaLaunchKernelEx(&lc, gemv_trit_kernel<false>, p);
}

}  // namespace terb
