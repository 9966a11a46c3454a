// Decode glue kernels for sm_100a: fused RMSNorm / activation + absmax int8 quantisation,
// rotary embedding + KV-cache append, split-KV GQA attention over a bf16 cache, bf16
// lm_head, argmax, embedding gather, residual add.  Each is a single-pass bandwidth kernel.
//
// Numerics: this file is compiled with -fmad=false; every fused multiply-add below is an
// explicit fmaf().  Floating-point reductions use one fixed order that depends on the
// problem only ("block order"): 256 lane partials over elements 1024*r + 4*t + e, an xor
// butterfly (16,8,4,2,1) inside each warp, then the 8 warp sums added left to right.  The
// result therefore does not depend on the grid, the batch size or the number of GPUs, and
// the CPU checker reproduces it bit for bit.
//
// Reference kernels restated here (formulas, not code): rmsnorm_quant_*_in_k,
// quant_int8_k, silu_mul_quant_k (cuda/ter_cuda_forward_packed.cu:40-62,269-344),
// relu2_mul_rmsnorm_quant_k (cuda/ter_cuda_forward_bitnet.cu:258-309), rope_k / kv_copy_k /
// attention_k (cuda/ter_cuda_forward_packed.cu:64-90,118-157; NEOX variant
// cuda/ter_cuda_forward_bitnet.cu:185-201), mm_fp16_lm_head_k and argmax_*_k
// (cuda/ter_cuda_forward_packed.cu:165-259).
#include "attn_mma.cuh"

namespace terb {

// ============================================================ norm / activation / quantise
namespace {

__global__ void __launch_bounds__(kT) norm_quant_kernel(const NormQuantParams p) {
    extern __shared__ float vals[];   // n floats: the row after pre-op / normalisation
    __shared__ float red[kT / 32];
    pdl_launch_dependents();
    pdl_wait();
    const size_t off = (size_t)blockIdx.x * (size_t)p.n;
    int8_t* qo = p.q ? p.q + off : nullptr;
    float* no = p.normed ? p.normed + off : nullptr;
    __shared__ float red16[16];
    const bool fast = norm_quant_fast_ok(p, (int)blockIdx.x, qo, no);
    int mine = 0;      // fast path: the sum of the int8 values this thread wrote
    const float stored = fast ? block_norm_quant_fast(p, (int)blockIdx.x, red16, qo, no, nullptr, &mine)
                              : block_norm_quant(p, (int)blockIdx.x, vals, red, qo, no);
    if (p.q && threadIdx.x == 0) p.scale_out[blockIdx.x] = stored;
    if (p.rowsum_out && qo && fast) {
        // exact integer sum of the row from the values still in registers: no second pass over the stores
        __shared__ int rsf;
        if (threadIdx.x == 0) rsf = 0;
        __syncthreads();
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, o);
        if ((threadIdx.x & 31) == 0 && mine != 0) atomicAdd(&rsf, mine);
        __syncthreads();
        if (threadIdx.x == 0) p.rowsum_out[blockIdx.x] = rsf;
    } else if (p.rowsum_out && qo) {
        // exact integer sum of the row just written (this CTA's own stores, visible after the barrier)
        __shared__ int rs;
        if (threadIdx.x == 0) rs = 0;
        __syncthreads();
        int local = 0;
        for (int i = threadIdx.x * 16; i < p.n; i += kT * 16) {
            const int4 v = *reinterpret_cast<const int4*>(qo + i);
            local = __dp4a(v.x, 0x01010101, local);
            local = __dp4a(v.y, 0x01010101, local);
            local = __dp4a(v.z, 0x01010101, local);
            local = __dp4a(v.w, 0x01010101, local);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
        if ((threadIdx.x & 31) == 0 && local != 0) atomicAdd(&rs, local);
        __syncthreads();
        if (threadIdx.x == 0) p.rowsum_out[blockIdx.x] = rs;
    }
}

template <typename Kern, typename Params>
cudaError_t launch_pdl(Kern kern, dim3 grid, dim3 block, size_t smem, bool pdl, cudaStream_t st, const Params& p) {
    cudaLaunchConfig_t lc = {};
    lc.gridDim = grid;
    lc.blockDim = block;
    lc.dynamicSmemBytes = smem;
    lc.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = attr;
    lc.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&lc, kern, p);
}

}  // namespace

cudaError_t launch_norm_quant(const NormQuantParams& p, bool pdl, cudaStream_t st) {
    const size_t smem = (size_t)p.n * sizeof(float);
    if (smem > 200 * 1024) return cudaErrorInvalidValue;
    if (p.rowsum_out && (p.n % 16 != 0 || !p.q)) return cudaErrorInvalidValue;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(norm_quant_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    return launch_pdl(norm_quant_kernel, dim3((unsigned)p.rows), dim3(kT), smem, pdl, st, p);
}

// ============================================================ rotary + KV append
namespace {

__global__ void __launch_bounds__(kT) rope_kv_kernel(const RopeKvParams p) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x;
    const int bs = p.shared_seq ? p.shared_seq - 1 : b;   // whose cache
    const int pos = p.pos[b];
    if (pos < 0 || pos >= p.Smax) return;
    const int half = p.Hd / 2;
    const float* row = p.table + (size_t)pos * p.Hd;   // [Hd/2][2]
    float* q = p.q + (size_t)b * p.Nh * p.Hd;
    float* k = p.k + (size_t)b * p.Nkv * p.Hd;
    const float* v = p.v + (size_t)b * p.Nkv * p.Hd;
    const int n_pairs = (p.Nh + p.Nkv) * half;
    for (int idx = threadIdx.x; idx < n_pairs; idx += kT) {
        const int head = idx / half, kk = idx % half;
        const bool is_k = head >= p.Nh;
        float* base = is_k ? k + (size_t)(head - p.Nh) * p.Hd : q + (size_t)head * p.Hd;
        const int i0 = p.neox ? kk : 2 * kk;
        const int i1 = p.neox ? kk + half : 2 * kk + 1;
        const float c = row[2 * kk], s = row[2 * kk + 1];
        const float v0 = base[i0], v1 = base[i1];
        const float a = v0 * c, bb = v1 * s;
        const float d = v0 * s, e = v1 * c;
        const float o0 = a - bb, o1 = d + e;
        base[i0] = o0;
        base[i1] = o1;
        if (is_k && p.kcache) {
            const size_t co = (((size_t)bs * p.Nkv + (head - p.Nh)) * p.Smax + pos) * p.Hd;
            p.kcache[co + i0] = f32_to_bf16_bits(o0);
            p.kcache[co + i1] = f32_to_bf16_bits(o1);
        }
    }
    if (!p.vcache) return;
    for (int idx = threadIdx.x; idx < p.Nkv * p.Hd; idx += kT) {
        const int g = idx / p.Hd, d = idx % p.Hd;
        const size_t co = (((size_t)bs * p.Nkv + g) * p.Smax + pos) * p.Hd;
        p.vcache[co + d] = f32_to_bf16_bits(v[idx]);
    }
}

}  // namespace

cudaError_t launch_rope_kv(const RopeKvParams& p, bool pdl, cudaStream_t st) {
    return launch_pdl(rope_kv_kernel, dim3((unsigned)p.B), dim3(kT), 0, pdl, st, p);
}

// ============================================================ split-KV GQA attention
// One CTA per (chunk, KV head, row); the arithmetic lives in attn.cuh (shared with the persistent
// decode kernel).  A second kernel merges the chunks left to right unless the caller gave arrival counters.
namespace {

template <int HD, int G, bool COMPACT>
__global__ void __launch_bounds__(kT, COMPACT ? (G <= 4 ? 3 : 2) : 1) attn_partial_kernel(const AttnParams p) {
    extern __shared__ __align__(128) uint8_t asmem[];
    using L = AttnSmem<HD, G, COMPACT>;
    uint64_t* bars = reinterpret_cast<uint64_t*>(asmem + L::kBarOff);
    __shared__ float redg[kMaxGroup * 8];
    __shared__ int is_last;

    const int tid = threadIdx.x;
    if (tid == 0) {
        mbar_init(&bars[0], 1);
        mbar_init(&bars[1], 1);
        mbar_fence_init();
    }
    const int c = blockIdx.x, g = blockIdx.y, b = blockIdx.z;
    const int bs = p.shared_seq ? p.shared_seq - 1 : b;   // whose cache
    {
        // Hints only, issued while the producer of q is still running: pull this CTA's K/V chunk and the
        // rotary row towards L2.  The position read here may be one step stale; nothing depends on it.
        const int pg = *reinterpret_cast<const volatile int*>(p.pos + b);
        const int s0g = c * kAttnChunk;
        if (pg >= 0 && pg < p.Smax && s0g <= pg + 1) {
            const int rows = min(kAttnChunk, pg + 2 - s0g);
            const size_t ho = ((size_t)bs * p.Nkv + g) * (size_t)p.Smax * HD + (size_t)s0g * HD;
            const int lines = rows * HD * 2 / 128;
            for (int i = tid; i < lines; i += kT) {
                asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char*>(p.kcache + ho) + (size_t)i * 128));
                asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char*>(p.vcache + ho) + (size_t)i * 128));
            }
            if (p.rope_table && tid < 8) {
                const int pr = min(pg + (tid >> 2), p.Smax - 1);
                asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char*>(p.rope_table + (size_t)pr * HD) + (tid & 3) * 128));
            }
        }
    }
    pdl_launch_dependents();
    pdl_wait();
    __syncthreads();
    const AttnItem it = attn_item<HD>(p, c, g, b, p.pos[b]);
    if (!it.active) return;
    if (tid == 0) attn_issue_kv<HD, G, COMPACT>(p, it, asmem);
    attn_compute<HD, G, COMPACT, 0>(p, it, asmem, redg, &is_last, 0);
}

// The tensor-core form (attn_mma.cuh), two or three CTAs per SM.
struct AttnMmaArgs {
    AttnParams a;
    alignas(64) CUtensorMap kmap;     // over the rows of a.kcache / a.vcache: [rows][HD] bf16, boxes of 64 x 256
    alignas(64) CUtensorMap vmap;
};
template <int HD, int G>
__global__ void __launch_bounds__(kT, AttnMmaSmem<HD, G>::kCtasPerSm) attn_mma_kernel(const __grid_constant__ AttnMmaArgs P) {
    extern __shared__ uint8_t asmem_raw[];
    uint8_t* asmem = asmem_raw + ((1024u - (smem_u32(asmem_raw) & 1023u)) & 1023u);   // the swizzle pattern wants it
    using L = AttnMmaSmem<HD, G>;
    const AttnParams& p = P.a;
    uint64_t* bars = reinterpret_cast<uint64_t*>(asmem + L::kBarOff);
    __shared__ float redg[kMaxGroup * 8];
    __shared__ int is_last;
    if (threadIdx.x == 0) {
        mbar_init(&bars[0], 1);
        mbar_init(&bars[1], 1);
        mbar_fence_init();
    }
    pdl_launch_dependents();
    pdl_wait();
    __syncthreads();
    const AttnItem it = attn_item<HD>(p, blockIdx.x, blockIdx.y, blockIdx.z, p.pos[blockIdx.z]);
    if (!it.active) return;
    attn_compute_mma<HD, G>(p, &P.kmap, &P.vmap, it, asmem, redg, &is_last);
}

template <int HD>
__global__ void __launch_bounds__(HD) attn_combine_kernel(const AttnParams p) {
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
    const int seq_len = p.pos[b] + 1;
    if (seq_len < 1 || seq_len > p.Smax) return;
    const int nc = (seq_len + kAttnChunk - 1) / kAttnChunk;
    const float* rec = p.scratch + ((size_t)b * p.Nh + h) * (size_t)p.max_chunks * (HD + 2);
    const int lane = d & 31;     // the block is HD threads (a multiple of 32), all of one head
    float M = rec[0], L = rec[1], O = rec[2 + d];
    for (int cb = 1; cb < nc; cb += 32) {
        const int nb = min(32, nc - cb);
        float mk = -CUDART_INF_F, lk = 0.0f;
        if (lane < nb) {
            mk = rec[(size_t)(cb + lane) * (HD + 2)];
            lk = rec[(size_t)(cb + lane) * (HD + 2) + 1];
        }
        float ak, bk, Mn;
        merge_factors(M, mk, lane, ak, bk, Mn);
        for (int k = 0; k < nb; ++k) {
            const float oc = rec[(size_t)(cb + k) * (HD + 2) + 2 + d];
            const float a = __shfl_sync(0xffffffffu, ak, k), bb = __shfl_sync(0xffffffffu, bk, k);
            const float lc = __shfl_sync(0xffffffffu, lk, k);
            L = fmaf(lc, bb, L * a);
            O = fmaf(oc, bb, O * a);
        }
        M = __shfl_sync(0xffffffffu, Mn, nb - 1);
    }
    p.out[((size_t)b * p.Nh + h) * HD + d] = O / L;
}

}  // namespace

size_t attention_scratch_floats(int B, int Nh, int Hd, int Smax) {
    const int mc = (Smax + kAttnChunk - 1) / kAttnChunk;
    return (size_t)B * Nh * mc * (Hd + 2);
}

namespace {
template <int HD, int G, bool COMPACT>
cudaError_t launch_attn_variant(const AttnParams& p, bool pdl, cudaStream_t st, int dev) {
    static bool attr_set[64] = {};
    if (!attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(attn_partial_kernel<HD, G, COMPACT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             AttnSmem<HD, G, COMPACT>::kBytes);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    const dim3 grid((unsigned)p.max_chunks, (unsigned)p.Nkv, (unsigned)p.B);
    return launch_pdl(attn_partial_kernel<HD, G, COMPACT>, grid, dim3(kT), AttnSmem<HD, G, COMPACT>::kBytes, pdl, st, p);
}
// False when the cache cannot be described by a tensor map (base not 16-byte aligned): the caller then takes
// the fixed-order kernel.
template <int HD>
bool attn_mma_maps(const AttnParams& p, AttnMmaArgs& args) {
    EncodeTiledFn enc = encode_tiled();
    if (!enc) return false;
    const long seqs = p.shared_seq ? p.shared_seq : p.B;
    const cuuint64_t dims[2] = {(cuuint64_t)HD, (cuuint64_t)(seqs * p.Nkv) * (cuuint64_t)p.Smax};
    const cuuint64_t strides[1] = {(cuuint64_t)HD * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)kAttnChunk};
    const cuuint32_t estr[2] = {1, 1};
    for (int i = 0; i < 2; ++i) {
        void* base = const_cast<uint16_t*>(i == 0 ? p.kcache : p.vcache);
        if (enc(i == 0 ? &args.kmap : &args.vmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return false;
    }
    return true;
}
template <int HD, int G>
cudaError_t launch_attn_mma(const AttnParams& p, bool pdl, cudaStream_t st, int dev, bool& taken) {
    AttnMmaArgs args;
    args.a = p;
    taken = attn_mma_maps<HD>(p, args);
    if (!taken) return cudaSuccess;
    static bool attr_set[64] = {};
    if (!attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(attn_mma_kernel<HD, G>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             AttnMmaSmem<HD, G>::kBytes);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    const dim3 grid((unsigned)p.max_chunks, (unsigned)p.Nkv, (unsigned)p.B);
    return launch_pdl(attn_mma_kernel<HD, G>, grid, dim3(kT), AttnMmaSmem<HD, G>::kBytes, pdl, st, args);
}
template <int HD, int G>
cudaError_t launch_attn_partial(const AttnParams& p, bool pdl, cudaStream_t st, int dev) {
    if (p.mma) {
        bool taken = false;
        const cudaError_t e = launch_attn_mma<HD, G>(p, pdl, st, dev, taken);
        if (taken || e != cudaSuccess) return e;
    }
    // more CTAs than SMs (token batches, prompt tiles): the one-buffer form, three CTAs per SM, so that grids of
    // up to 444 items still run as one wave
    const bool compact = (long)p.max_chunks * p.Nkv * p.B > 148;
    return compact ? launch_attn_variant<HD, G, true>(p, pdl, st, dev) : launch_attn_variant<HD, G, false>(p, pdl, st, dev);
}
template <int HD>
cudaError_t launch_attn_hd(const AttnParams& p, bool pdl, cudaStream_t st, int dev) {
    cudaError_t e;
    switch (p.Nh / p.Nkv) {
        case 1: e = launch_attn_partial<HD, 1>(p, pdl, st, dev); break;
        case 2: e = launch_attn_partial<HD, 2>(p, pdl, st, dev); break;
        case 4: e = launch_attn_partial<HD, 4>(p, pdl, st, dev); break;
        case 8: e = launch_attn_partial<HD, 8>(p, pdl, st, dev); break;
        default: return cudaErrorInvalidValue;
    }
    if (e != cudaSuccess || p.counters) return e;
    return launch_pdl(attn_combine_kernel<HD>, dim3((unsigned)p.Nh, (unsigned)p.B), dim3(HD), 0, pdl, st, p);
}
}  // namespace

cudaError_t launch_attention(const AttnParams& p, bool pdl, cudaStream_t st) {
    if (p.Nkv < 1 || p.Nh % p.Nkv != 0 || p.Nh / p.Nkv > kMaxGroup) return cudaErrorInvalidValue;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (p.Hd == 64) return launch_attn_hd<64>(p, pdl, st, dev);
    if (p.Hd == 128) return launch_attn_hd<128>(p, pdl, st, dev);
    return cudaErrorInvalidValue;
}

// ============================================================ bf16 lm_head, argmax, small ops
namespace {

struct LmHeadParams {
    const uint16_t* table;
    const float* x;
    float* logits;
    int V, H, B;
};

__device__ __forceinline__ uint4 ldg_stream16(const void* ptr) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(ptr));
    return v;
}

// A warp takes kLmVoc consecutive vocabulary rows at a time; lane l takes elements 256*i + 8*l + e of
// each (e ascending), fused multiply-adds, then an xor butterfly over the warp.  A CTA serves up to
// kLmRows batch rows (grid.x = groups of kLmRows batch rows, the fastest-varying index, so that the
// CTAs reading the same table rows for different batch groups run together and the table comes from
// HBM once).  Every (batch row, vocabulary row) pair has its own accumulator and sees the same
// sequence of operations whatever the batch size.  An activation value fetched from shared memory
// feeds kLmVoc multiply-adds, which keeps the kernel off the shared-memory limit at large batches.
constexpr int kLmRows = 8;
constexpr int kLmVoc = 4;
template <int ROWS>   // accumulator rows compiled in: 1 for a lone sequence (fewer registers), else kLmRows
__global__ void __launch_bounds__(kT) lm_head_bf16_kernel(const LmHeadParams p) {
    extern __shared__ __align__(16) float xs[];       // [rows][H]
    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int b0 = blockIdx.x * ROWS;
    const int rows = min(ROWS, p.B - b0);
    for (int i = tid; i < rows * p.H; i += kT) xs[i] = p.x[(size_t)b0 * p.H + i];
    __syncthreads();
    const int total_warps = gridDim.y * (kT / 32);
    for (int v0 = (blockIdx.y * (kT / 32) + warp) * kLmVoc; v0 < p.V; v0 += total_warps * kLmVoc) {
        const uint16_t* row[kLmVoc];
#pragma unroll
        for (int i = 0; i < kLmVoc; ++i) row[i] = p.table + (size_t)min(v0 + i, p.V - 1) * p.H;
        float acc[kLmVoc][ROWS];
#pragma unroll
        for (int i = 0; i < kLmVoc; ++i)
#pragma unroll
            for (int r = 0; r < ROWS; ++r) acc[i][r] = 0.0f;
        for (int base = 8 * lane; base < p.H; base += 256) {
            float wf[kLmVoc][8];
#pragma unroll
            for (int i = 0; i < kLmVoc; ++i) {
                const uint4 w = ldg_stream16(row[i] + base);
                wf[i][0] = bf16_bits_to_f32(w.x & 0xffffu); wf[i][1] = bf16_bits_to_f32(w.x >> 16);
                wf[i][2] = bf16_bits_to_f32(w.y & 0xffffu); wf[i][3] = bf16_bits_to_f32(w.y >> 16);
                wf[i][4] = bf16_bits_to_f32(w.z & 0xffffu); wf[i][5] = bf16_bits_to_f32(w.z >> 16);
                wf[i][6] = bf16_bits_to_f32(w.w & 0xffffu); wf[i][7] = bf16_bits_to_f32(w.w >> 16);
            }
#pragma unroll
            for (int r = 0; r < ROWS; ++r) {
                if (r < rows) {
                    const float4 xa = *reinterpret_cast<const float4*>(&xs[r * p.H + base]);
                    const float4 xb = *reinterpret_cast<const float4*>(&xs[r * p.H + base + 4]);
#pragma unroll
                    for (int i = 0; i < kLmVoc; ++i) {
                        float a = acc[i][r];
                        a = fmaf(wf[i][0], xa.x, a); a = fmaf(wf[i][1], xa.y, a); a = fmaf(wf[i][2], xa.z, a); a = fmaf(wf[i][3], xa.w, a);
                        a = fmaf(wf[i][4], xb.x, a); a = fmaf(wf[i][5], xb.y, a); a = fmaf(wf[i][6], xb.z, a); a = fmaf(wf[i][7], xb.w, a);
                        acc[i][r] = a;
                    }
                }
            }
        }
#pragma unroll
        for (int i = 0; i < kLmVoc; ++i) {
#pragma unroll
            for (int r = 0; r < ROWS; ++r) {
                if (r < rows) {
                    const float t = warp_sum_butterfly(acc[i][r]);
                    if (lane == 0 && v0 + i < p.V) p.logits[(size_t)(b0 + r) * p.V + v0 + i] = t;
                }
            }
        }
    }
}

struct ArgmaxParams {
    const float* logits;
    float* scratch;   // [B][kArgmaxParts][2]: value, index bits
    int* out;
    int V;
};

__device__ __forceinline__ void argmax_merge(float& v, int& i, float v2, int i2) {
    if (v2 > v || (v2 == v && i2 < i)) { v = v2; i = i2; }
}
__device__ __forceinline__ void argmax_block(float& v, int& i, float* sv, int* si) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float v2 = __shfl_xor_sync(0xffffffffu, v, o);
        const int i2 = __shfl_xor_sync(0xffffffffu, i, o);
        argmax_merge(v, i, v2, i2);
    }
    const int warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    if ((threadIdx.x & 31) == 0) { sv[warp] = v; si[warp] = i; }
    __syncthreads();
    if (threadIdx.x == 0)
        for (int w = 1; w < nw; ++w) argmax_merge(v, i, sv[w], si[w]);
}

__global__ void __launch_bounds__(kT) argmax_part_kernel(const ArgmaxParams p) {
    __shared__ float sv[kT / 32];
    __shared__ int si[kT / 32];
    pdl_launch_dependents();
    pdl_wait();
    const float* lg = p.logits + (size_t)blockIdx.y * p.V;
    float best = -CUDART_INF_F;
    int bi = 0x7fffffff;
    for (int i = blockIdx.x * kT + threadIdx.x; i < p.V; i += gridDim.x * kT) {
        const float v = lg[i];
        if (v > best) { best = v; bi = i; }
    }
    argmax_block(best, bi, sv, si);
    if (threadIdx.x == 0) {
        float* s = p.scratch + ((size_t)blockIdx.y * kArgmaxParts + blockIdx.x) * 2;
        s[0] = best;
        s[1] = __int_as_float(bi);
    }
}
__global__ void __launch_bounds__(kArgmaxParts) argmax_final_kernel(const ArgmaxParams p) {
    __shared__ float sv[kArgmaxParts / 32];
    __shared__ int si[kArgmaxParts / 32];
    pdl_launch_dependents();
    pdl_wait();
    const float* s = p.scratch + ((size_t)blockIdx.x * kArgmaxParts + threadIdx.x) * 2;
    float best = s[0];
    int bi = __float_as_int(s[1]);
    argmax_block(best, bi, sv, si);
    if (threadIdx.x == 0) p.out[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
}

struct EmbedParams { const uint16_t* table; const int* tokens; float* hidden; int H, V; };
__global__ void __launch_bounds__(kT) embed_kernel(const EmbedParams p) {
    pdl_launch_dependents();
    pdl_wait();
    int t = p.tokens[blockIdx.y];
    if (t < 0 || t >= p.V) t = 0;
    const int i = blockIdx.x * kT + threadIdx.x;
    if (i < p.H) p.hidden[(size_t)blockIdx.y * p.H + i] = bf16_bits_to_f32(p.table[(size_t)t * p.H + i]);
}
struct AddParams { float* x; const float* y; size_t n; };
__global__ void __launch_bounds__(kT) add_kernel(const AddParams p) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * kT + threadIdx.x;
    if (i < p.n) p.x[i] = p.x[i] + p.y[i];
}
struct IncParams { int* pos; int B; };
__global__ void inc_kernel(const IncParams p) {
    pdl_launch_dependents();
    pdl_wait();
    if ((int)threadIdx.x < p.B) p.pos[threadIdx.x] += 1;
}

}  // namespace

cudaError_t launch_lm_head_bf16(const uint16_t* table, const float* x, float* logits, int V, int H, int B,
                                int sm_count, bool pdl, cudaStream_t st) {
    if (H % 8 != 0) return cudaErrorInvalidValue;
    const int rows = B == 1 ? 1 : kLmRows;
    const size_t smem = (size_t)rows * H * sizeof(float);
    if (smem > 200 * 1024) return cudaErrorInvalidValue;
    auto kern = B == 1 ? lm_head_bf16_kernel<1> : lm_head_bf16_kernel<kLmRows>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    const int groups = (B + rows - 1) / rows;
    int gy = sm_count * (smem > 100 * 1024 ? 1 : (smem > 48 * 1024 ? 2 : 4)) / groups;   // CTAs per batch group
    const int need = (V + 8 * kLmVoc - 1) / (8 * kLmVoc);
    if (gy > need) gy = need;
    if (gy < 1) gy = 1;
    LmHeadParams p{table, x, logits, V, H, B};
    return launch_pdl(kern, dim3((unsigned)groups, (unsigned)gy), dim3(kT), smem, pdl, st, p);
}

cudaError_t launch_argmax(const float* logits, int V, int B, float* scratch, int* out, bool pdl, cudaStream_t st) {
    ArgmaxParams p{logits, scratch, out, V};
    cudaError_t e = launch_pdl(argmax_part_kernel, dim3(kArgmaxParts, (unsigned)B), dim3(kT), 0, pdl, st, p);
    if (e != cudaSuccess) return e;
    return launch_pdl(argmax_final_kernel, dim3((unsigned)B), dim3(kArgmaxParts), 0, pdl, st, p);
}

cudaError_t launch_embed(const uint16_t* table, const int* tokens, float* hidden, int H, int B, int V, bool pdl,
                         cudaStream_t st) {
    EmbedParams p{table, tokens, hidden, H, V};
    return launch_pdl(embed_kernel, dim3((unsigned)((H + kT - 1) / kT), (unsigned)B), dim3(kT), 0, pdl, st, p);
}
cudaError_t launch_add(float* x, const float* y, size_t n, bool pdl, cudaStream_t st) {
    AddParams p{x, y, n};
    return launch_pdl(add_kernel, dim3((unsigned)((n + kT - 1) / kT)), dim3(kT), 0, pdl, st, p);
}
namespace {
__global__ void select_kernel(const SelectParams p) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = threadIdx.x;
    if (b == 0 && p.step_word) *p.step_word += 1u;
    if (b >= p.B) return;
    const int ps = p.pos[b];
    int nxt = p.greedy[b];
    if (p.forced && ps + 1 < p.ctl[0] && ps + 1 < p.forced_stride) nxt = p.forced[(size_t)b * p.forced_stride + ps + 1];
    p.tokens[b] = nxt;
    if (p.log && ps >= 0 && ps < p.ctl[1] && ps < p.log_stride) p.log[(size_t)b * p.log_stride + ps] = nxt;
    p.pos[b] = ps + 1;
}
}  // namespace
cudaError_t launch_select(const SelectParams& p, bool pdl, cudaStream_t st) {
    if (p.B > 1024) return cudaErrorInvalidValue;
    return launch_pdl(select_kernel, dim3(1), dim3(p.B < 32 ? 32 : ((p.B + 31) / 32 * 32)), 0, pdl, st, p);
}
cudaError_t launch_inc(int* pos, int B, bool pdl, cudaStream_t st) {
    if (B > 1024) return cudaErrorInvalidValue;
    IncParams p{pos, B};
    return launch_pdl(inc_kernel, dim3(1), dim3(B < 32 ? 32 : ((B + 31) / 32 * 32)), 0, pdl, st, p);
}

}  // namespace terb

// ============================================================ attention for callers that cannot allocate
// Some hosts of this library may not allocate device memory at the point where they need
// attention: code running between cudaStreamBeginCapture and cudaStreamEndCapture, a real-time
// decode loop that has handed all of its memory budget out at start-up, or an embedding whose
// allocator is owned by another runtime and must not see foreign cudaMalloc calls.  The regular
// entry point asks them for a scratch buffer; this one brings its own, a fixed array that lives
// in the library's device image.  Every GPU that loads the library holds these 4 MiB until the
// process exits.
#include "handle.h"

#define TER_B200_STATIC_SCRATCH_FLOATS (1u << 20)   // 4 MiB; keep in step with include/ter_b200.h

static __device__ __align__(256) float g_attn_static_scratch[TER_B200_STATIC_SCRATCH_FLOATS];

// In host code `g_attn_static_scratch` is only a handle for the symbol, not a device address:
// the address is looked up once per device, with that device current, and remembered here.
static float* g_attn_static_ptr[64] = {};

extern "C" size_t ter_b200_attention_noalloc_max_floats(void) { return TER_B200_STATIC_SCRATCH_FLOATS; }

extern "C" int ter_b200_attention_noalloc(ter_b200_handle_t* h, const float* q_dev, const uint16_t* kcache_dev,
                                          const uint16_t* vcache_dev, const int* pos_dev, int B, int Nh, int Nkv,
                                          int Hd, int Smax, float* out_dev, void* stream) {
    using namespace terb;
    if (!h || !q_dev || !kcache_dev || !vcache_dev || !pos_dev || !out_dev) return TER_B200_E_NULL;
    if (B < 1 || Nkv < 1 || Nh < 1 || Nh % Nkv != 0 || (Nh / Nkv != 1 && Nh / Nkv != 2 && Nh / Nkv != 4 && Nh / Nkv != 8) || (Hd != 64 && Hd != 128) || Smax < 1)
        return TER_B200_E_SHAPE;
    // the partial records of this problem must fit the fixed array
    if (attention_scratch_floats(B, Nh, Hd, Smax) > (size_t)TER_B200_STATIC_SCRATCH_FLOATS) return TER_B200_E_SHAPE;
    if (h->device < 0 || h->device >= 64) return TER_B200_E_SHAPE;
    TERB_CUDA(h, cudaSetDevice(h->device));
    float* scratch = g_attn_static_ptr[h->device];
    if (!scratch) {
        // First call on this device: resolve the symbol.  Do this before any stream capture.
        void* ptr = nullptr;
        TERB_CUDA(h, cudaGetSymbolAddress(&ptr, g_attn_static_scratch));
        if (!ptr) return TER_B200_E_CUDA;
        scratch = static_cast<float*>(ptr);
        g_attn_static_ptr[h->device] = scratch;
    }
    AttnParams p{q_dev, kcache_dev, vcache_dev, pos_dev, scratch, out_dev, B, Nh, Nkv, Hd, Smax,
                 (Smax + kAttnChunk - 1) / kAttnChunk, nullptr, nullptr, nullptr, nullptr, nullptr, 0,
                 h->status_dev};
    TERB_CUDA(h, launch_attention(p, h->gemv_cfg.pdl != 0, pick_stream(h, stream)));
    h->launches += 2;
    return TER_B200_OK;
}
