// Device helpers shared by the glue kernels and the GEMV prologue: the fixed-order block
// reductions, the fixed exp(), and the row-wise "pre-op -> RMSNorm -> absmax int8" routine.
// Everything here is written with explicit fmaf() and compiled with -fmad=false, and runs with
// exactly 256 threads per CTA, so that its results depend on the data only.
#pragma once
#include <cuda_bf16.h>
#include <math_constants.h>

#include "common.cuh"
#include "glue.h"
#include "tagged.cuh"

namespace terb {
namespace {

constexpr int kT = 256;   // threads per CTA in every glue kernel

// exp(x) in fp32: n = rint(x*log2e); r = x - n*ln2 (two steps); degree-5 polynomial; * 2^n.
// Arguments are clamped to [-87, 88]; below -87 the result is 0.  Same operations, in the
// same order, as the CPU checker.
__device__ __forceinline__ float exp_fixed(float x) {
    if (!(x >= -87.0f)) return 0.0f;
    if (x > 88.0f) x = 88.0f;
    const float n = rintf(x * 1.44269504088896341f);
    float r = fmaf(n, -0.693145751953125f, x);
    r = fmaf(n, -1.42860682030941723212e-6f, r);
    float p = 1.9875691500e-4f;
    p = fmaf(p, r, 1.3981999507e-3f);
    p = fmaf(p, r, 8.3334519073e-3f);
    p = fmaf(p, r, 4.1665795894e-2f);
    p = fmaf(p, r, 1.6666665459e-1f);
    p = fmaf(p, r, 5.0000001201e-1f);
    const float r2 = r * r;
    float y = fmaf(p, r2, r);
    y = y + 1.0f;
    const int ni = (int)n;
    return y * __int_as_float((ni + 127) << 23);
}

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t b) { return __uint_as_float(b << 16); }
__device__ __forceinline__ uint16_t f32_to_bf16_bits(float f) {
    return __bfloat16_as_ushort(__float2bfloat16_rn(f));
}

__device__ __forceinline__ float warp_sum_butterfly(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = v + __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// Block order sum of one value per thread (256 threads).  red: 8 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum_butterfly(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = red[0];
#pragma unroll
    for (int w = 1; w < kT / 32; ++w) t = t + red[w];
    return t;
}
__device__ __forceinline__ float block_max(float v, float* red) {
    v = warp_max(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = red[0];
#pragma unroll
    for (int w = 1; w < kT / 32; ++w) t = fmaxf(t, red[w]);
    return t;
}

__device__ __forceinline__ int quant_one(float v, float scale) {
    int q = __float2int_rn(v * scale);
    return q > 127 ? 127 : (q < -128 ? -128 : q);
}

__device__ __forceinline__ float pre_op(int pre, float x, float u) {
    if (pre == PRE_SILU_MUL) {
        const float e = exp_fixed(-x);
        const float sg = x / (1.0f + e);
        return sg * u;
    }
    if (pre == PRE_RELU2_MUL) {
        const float r = x > 0.0f ? x * x : 0.0f;
        return r * u;
    }
    return x;
}

// One CTA (256 threads) processes row `row` of p.  vals: n floats of shared memory; red: 8 floats.
// q_out: where the int8 row goes (global or shared; null = no quantisation); returns the stored
// scale (1 / (127/amax)) in every thread.  normed (optional, global) receives the fp32 row.
__device__ __forceinline__ float block_norm_quant(const NormQuantParams& p, int row, float* vals, float* red,
                                                  int8_t* q_out, float* normed_out) {
    const int tid = threadIdx.x;
    const size_t off = (size_t)row * (size_t)p.n;
    const float* x = p.x + off;
    const float* u = p.u ? p.u + off : nullptr;
    const int n = p.n;

    float part = 0.0f;
    for (int base = 4 * tid; base < n; base += 4 * kT) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int i = base + e;
            if (i < n) {
                const float v = pre_op(p.pre, x[i], u ? u[i] : 0.0f);
                vals[i] = v;
                part = fmaf(v, v, part);
            }
        }
    }
    float amax = 0.0f;
    if (p.gamma) {
        const float ss = block_sum(part, red);
        const float mean = ss / (float)n;
        const float ri = 1.0f / sqrtf(mean + p.eps);
        for (int base = 4 * tid; base < n; base += 4 * kT) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int i = base + e;
                if (i < n) {
                    const float v = (vals[i] * ri) * p.gamma[i];
                    vals[i] = v;
                    amax = fmaxf(amax, fabsf(v));
                }
            }
        }
    } else {
        for (int base = 4 * tid; base < n; base += 4 * kT)
#pragma unroll
            for (int e = 0; e < 4; ++e)
                if (base + e < n) amax = fmaxf(amax, fabsf(vals[base + e]));
    }
    if (normed_out) {
        float* o = normed_out;
        for (int base = 4 * tid; base < n; base += 4 * kT)
#pragma unroll
            for (int e = 0; e < 4; ++e)
                if (base + e < n) o[base + e] = vals[base + e];
    }
    float stored = 0.0f;
    if (q_out) {
        amax = block_max(amax, red) + 1e-9f;
        const float scale = 127.0f / amax;
        stored = 1.0f / scale;
        int8_t* q = q_out;
        for (int base = 4 * tid; base < n; base += 4 * kT) {
            if (base + 3 < n && ((reinterpret_cast<uintptr_t>(q + base) & 3u) == 0)) {
                const int q0 = quant_one(vals[base], scale), q1 = quant_one(vals[base + 1], scale);
                const int q2 = quant_one(vals[base + 2], scale), q3 = quant_one(vals[base + 3], scale);
                *reinterpret_cast<uint32_t*>(q + base) =
                    (uint32_t)(q0 & 0xff) | ((uint32_t)(q1 & 0xff) << 8) | ((uint32_t)(q2 & 0xff) << 16) |
                    ((uint32_t)(q3 & 0xff) << 24);
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (base + e < n) q[base + e] = (int8_t)quant_one(vals[base + e], scale);
            }
        }
    }
    return stored;
}


// Single-barrier variants for one-shot use: each call must get its own 8-float slot of shared memory
// that nothing else writes between the call and the next __syncthreads of the kernel.
__device__ __forceinline__ float block_sum_once(float v, float* slot) {
    v = warp_sum_butterfly(v);
    if ((threadIdx.x & 31) == 0) slot[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = slot[0];
#pragma unroll
    for (int w = 1; w < kT / 32; ++w) t = t + slot[w];
    return t;
}
__device__ __forceinline__ float block_max_once(float v, float* slot) {
    v = warp_max(v);
    if ((threadIdx.x & 31) == 0) slot[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = slot[0];
#pragma unroll
    for (int w = 1; w < kT / 32; ++w) t = fmaxf(t, slot[w]);
    return t;
}

constexpr int kNqFastMax = 8192;   // rows up to this length are kept in registers (8 float4 per thread)

__device__ __forceinline__ bool norm_quant_fast_ok(const NormQuantParams& p, int row, const void* q_out,
                                                   const void* normed_out) {
    const size_t off = (size_t)row * (size_t)p.n;
    uintptr_t a = reinterpret_cast<uintptr_t>(p.x + off) | reinterpret_cast<uintptr_t>(normed_out);
    if (p.u) a |= reinterpret_cast<uintptr_t>(p.u + off);
    if (p.gamma) a |= reinterpret_cast<uintptr_t>(p.gamma);
    return p.n <= kNqFastMax && (p.n & 3) == 0 && (a & 15u) == 0 && (reinterpret_cast<uintptr_t>(q_out) & 3u) == 0;
}

// L2 prefetch of the (immutable) gain vector; a hint, safe to issue before griddepcontrol.wait.
__device__ __forceinline__ void norm_quant_prefetch_gamma(const NormQuantParams& p) {
    if (p.gamma)
        for (int i = threadIdx.x * 32; i < p.n; i += kT * 32)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(p.gamma + i));
}

// Same arithmetic, in the same order, as block_norm_quant, for rows of at most 8192 elements with
// 16-byte aligned pointers: the row lives in registers, x / up / gamma are fetched with one batch of
// independent 16-byte loads, and each reduction costs one barrier.  red16: 16 floats of shared memory.
// ts (optional): the row comes from a flag-in-data vector instead of p.x (persistent decode kernel: the
// values are polled until the producing CTAs have stored them); p.u must then be null.
// R: float4 slots per thread compiled in (the row has at most 1024*R elements).
// qsum: when not null, receives the sum of the int8 values THIS thread wrote (for the row sum of a token batch).
template <int R>
__device__ __forceinline__ float block_norm_quant_fast_r(const NormQuantParams& p, int row, float* red16,
                                                         int8_t* q_out, float* normed_out, const TaggedSrc* ts,
                                                         int* qsum = nullptr) {
    const int tid = threadIdx.x, n = p.n;
    const size_t off = (size_t)row * (size_t)n;
    const float4* x4 = reinterpret_cast<const float4*>(p.x + off);
    const float4* u4 = p.u ? reinterpret_cast<const float4*>(p.u + off) : nullptr;
    const float4* g4 = reinterpret_cast<const float4*>(p.gamma);
    float4 v[R], g[R];
    if (ts) {
        // all of this thread's words are requested first and validated afterwards: one round trip when the
        // producers are done, instead of one per word; only a word that is not there yet is polled
        uint4 w[2 * R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int idx = tid + kT * r;
            if (4 * idx < n) {
                w[2 * r] = ld_volatile16(ts->words + 2 * idx);
                w[2 * r + 1] = ld_volatile16(ts->words + 2 * idx + 1);
            }
            g[r] = (4 * idx < n && g4) ? g4[idx] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int idx = tid + kT * r;
            v[r] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (4 * idx < n) {
                if (w[2 * r].y != ts->seq || w[2 * r].w != ts->seq) w[2 * r] = poll_tagged(ts->words + 2 * idx, ts->seq, ts->ctx);
                if (w[2 * r + 1].y != ts->seq || w[2 * r + 1].w != ts->seq)
                    w[2 * r + 1] = poll_tagged(ts->words + 2 * idx + 1, ts->seq, ts->ctx);
                v[r] = make_float4(__uint_as_float(w[2 * r].x), __uint_as_float(w[2 * r].z), __uint_as_float(w[2 * r + 1].x),
                                   __uint_as_float(w[2 * r + 1].z));
            }
        }
    } else {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int idx = tid + kT * r;
            const bool valid = 4 * idx < n;
            v[r] = valid ? x4[idx] : make_float4(0.f, 0.f, 0.f, 0.f);
            g[r] = (valid && g4) ? g4[idx] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    if (u4) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int idx = tid + kT * r;
            if (4 * idx < n) {
                const float4 uu = u4[idx];
                v[r].x = pre_op(p.pre, v[r].x, uu.x);
                v[r].y = pre_op(p.pre, v[r].y, uu.y);
                v[r].z = pre_op(p.pre, v[r].z, uu.z);
                v[r].w = pre_op(p.pre, v[r].w, uu.w);
            }
        }
    }
    float amax = 0.0f;
    if (p.gamma) {
        float part = 0.0f;
#pragma unroll
        for (int r = 0; r < R; ++r)
            if (4 * (tid + kT * r) < n) {
                part = fmaf(v[r].x, v[r].x, part);
                part = fmaf(v[r].y, v[r].y, part);
                part = fmaf(v[r].z, v[r].z, part);
                part = fmaf(v[r].w, v[r].w, part);
            }
        const float ss = block_sum_once(part, red16);
        const float mean = ss / (float)n;
        const float ri = 1.0f / sqrtf(mean + p.eps);
#pragma unroll
        for (int r = 0; r < R; ++r) {
            v[r].x = (v[r].x * ri) * g[r].x;
            v[r].y = (v[r].y * ri) * g[r].y;
            v[r].z = (v[r].z * ri) * g[r].z;
            v[r].w = (v[r].w * ri) * g[r].w;
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r)
        if (4 * (tid + kT * r) < n)
            amax = fmaxf(fmaxf(fmaxf(amax, fabsf(v[r].x)), fabsf(v[r].y)), fmaxf(fabsf(v[r].z), fabsf(v[r].w)));
    if (normed_out) {
        float4* o = reinterpret_cast<float4*>(normed_out);
#pragma unroll
        for (int r = 0; r < R; ++r)
            if (4 * (tid + kT * r) < n) o[tid + kT * r] = v[r];
    }
    float stored = 0.0f;
    if (q_out) {
        amax = block_max_once(amax, red16 + 8) + 1e-9f;
        const float scale = 127.0f / amax;
        stored = 1.0f / scale;
        uint32_t* q4 = reinterpret_cast<uint32_t*>(q_out);
        int mine = 0;
#pragma unroll
        for (int r = 0; r < R; ++r)
            if (4 * (tid + kT * r) < n) {
                const int q0 = quant_one(v[r].x, scale), q1 = quant_one(v[r].y, scale);
                const int q2 = quant_one(v[r].z, scale), q3 = quant_one(v[r].w, scale);
                q4[tid + kT * r] = (uint32_t)(q0 & 0xff) | ((uint32_t)(q1 & 0xff) << 8) | ((uint32_t)(q2 & 0xff) << 16) |
                                   ((uint32_t)(q3 & 0xff) << 24);
                mine += (q0 + q1) + (q2 + q3);
            }
        if (qsum) *qsum = mine;
    }
    return stored;
}

// Dispatch on the row length, so that a short row does not pay for the slots of a long one.
__device__ __forceinline__ float block_norm_quant_fast(const NormQuantParams& p, int row, float* red16,
                                                       int8_t* q_out, float* normed_out,
                                                       const TaggedSrc* ts = nullptr, int* qsum = nullptr) {
    if (p.n <= 3072) return block_norm_quant_fast_r<3>(p, row, red16, q_out, normed_out, ts, qsum);
    return block_norm_quant_fast_r<kNqFastMax / (4 * kT)>(p, row, red16, q_out, normed_out, ts, qsum);
}

}  // namespace
}  // namespace terb
