// Split-KV GQA attention for token batches on the tensor cores (bf16 mma.sync m16n8k16, fp32 accumulators).
//
// Same split as attn.cuh: one CTA per (chunk of 256 positions, KV head, row), chunk records (m, l, o[HD]) in
// fp32, chunks merged left to right in fp32.  What differs is how the two contractions are summed:
//   scores   S[t][head] = sum_d K[t][d] * q[head][d]     A = K tile from the chunk buffer (ldmatrix),
//                                                        B = q split in three bf16 parts (hi + mid + lo = q exactly)
//   output   O[d][head] = sum_t V[t][d] * P[t][head]     A = V tile transposed on the way in (ldmatrix.trans),
//                                                        B = exp(s - m) split in three bf16 parts
// K and V are bf16 already, so every product is exact and only the order and rounding of the fp32 sums differs
// from the fixed-order kernel: results agree to a few units in the last place, not bit for bit.  The softmax
// itself (maximum, exponentials, their sum) is the fixed-order one.
//
// The chunk buffer holds rows of HD + 8 elements: the 16-byte pad spreads eight consecutive rows over all 32
// banks, which ldmatrix needs; each cached row therefore arrives by its own 1-D bulk copy.
#pragma once
#include "attn.cuh"

namespace terb {
namespace {

template <int HD, int G>
struct AttnMmaSmem {
    static constexpr int kRow = HD + 8;                              // elements per staged row
    static constexpr int kPRow = kAttnChunk + 8;                     // elements per probability row
    static constexpr int kChunkOff = 0;                              // K, then V: [256][kRow] bf16
    static constexpr int kQOff = kAttnChunk * kRow * 2;              // fp32 [G][HD]
    static constexpr int kScOff = kQOff + G * HD * 4;                // fp32 [G][256] scores
    static constexpr int kPOff = kScOff + G * kAttnChunk * 4;        // bf16 [3][G][kPRow] probability parts
    static constexpr int kBarOff = (kPOff + 3 * G * kPRow * 2 + 15) / 16 * 16;
    static constexpr int kBytes = kBarOff + 16;
};

// f = hi + mid + lo exactly (each part a bf16; 3 x 8 significant bits cover the 24 of an fp32)
__device__ __forceinline__ void split3(float f, uint16_t& hi, uint16_t& mid, uint16_t& lo) {
    hi = f32_to_bf16_bits(f);
    const float r1 = f - bf16_bits_to_f32(hi);
    mid = f32_to_bf16_bits(r1);
    const float r2 = r1 - bf16_bits_to_f32(mid);
    lo = f32_to_bf16_bits(r2);
}

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Rows [0, n) of a cache chunk into the padded buffer, one bulk copy per row; every thread calls it (row = thread).
template <int HD, int G>
__device__ __forceinline__ void attn_mma_copy_rows(uint16_t* buf, const uint16_t* src, int n, uint64_t* bar) {
    using L = AttnMmaSmem<HD, G>;
    const int tid = threadIdx.x;
    if (n <= 0) return;
    if (tid == 0) mbar_arrive_expect_tx(bar, (uint32_t)n * HD * 2u);
    __syncthreads();
    // the buffer may have been read or written by ordinary loads and stores before (K, then V, share it)
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (tid < n) bulk_g2s(buf + tid * L::kRow, src + (size_t)tid * HD, HD * 2u, bar);
}

// One item, all 256 threads.  Plain buffers (p.q, p.scratch, p.out); rotary and cache append fused when
// p.rope_table is set, exactly as in attn_compute.
template <int HD, int G>
__device__ __forceinline__ void attn_compute_mma(const AttnParams& p, const AttnItem& it, uint8_t* asmem, float* redg,
                                                 int* is_last) {
    using L = AttnMmaSmem<HD, G>;
    constexpr int RS = L::kRow;
    uint16_t* Cs = reinterpret_cast<uint16_t*>(asmem + L::kChunkOff);
    float* qs = reinterpret_cast<float*>(asmem + L::kQOff);
    float* scf = reinterpret_cast<float*>(asmem + L::kScOff);
    uint16_t* Ps = reinterpret_cast<uint16_t*>(asmem + L::kPOff);
    uint64_t* bars = reinterpret_cast<uint64_t*>(asmem + L::kBarOff);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (!it.active) return;
    const int g = it.g, b = it.b, c = it.c, pos = it.pos, s0 = it.s0, cnt = it.cnt, n_copy = it.n_copy;
    const bool owner = it.owner;
    const size_t head_off = it.head_off;

    attn_mma_copy_rows<HD, G>(Cs, p.kcache + head_off + (size_t)s0 * HD, n_copy, &bars[0]);

    const float* q = p.q + ((size_t)b * p.Nh + (size_t)g * G) * HD;
    if (it.fused) {
        const float* row = p.rope_table + (size_t)pos * HD;
        const int half = HD / 2;
        for (int idx = tid; idx < G * half; idx += kT) {
            const int hh = idx / half, kk = idx % half;
            const int i0 = p.neox ? kk : 2 * kk, i1 = p.neox ? kk + half : 2 * kk + 1;
            const float cs = row[2 * kk], sn = row[2 * kk + 1];
            const float v0 = q[hh * HD + i0], v1 = q[hh * HD + i1];
            const float a = v0 * cs, bb = v1 * sn;
            const float d = v0 * sn, e = v1 * cs;
            qs[hh * HD + i0] = a - bb;
            qs[hh * HD + i1] = d + e;
        }
        if (owner) {
            const float* kn = p.k_new + ((size_t)b * p.Nkv + g) * HD;
            const float* vn = p.v_new + ((size_t)b * p.Nkv + g) * HD;
            uint16_t* Kw = p.kcache_w + head_off + (size_t)pos * HD;
            uint16_t* Vw = p.vcache_w + head_off + (size_t)pos * HD;
            const int r = pos - s0;
            for (int kk = tid; kk < half; kk += kT) {
                const int i0 = p.neox ? kk : 2 * kk, i1 = p.neox ? kk + half : 2 * kk + 1;
                const float cs = row[2 * kk], sn = row[2 * kk + 1];
                const float v0 = kn[i0], v1 = kn[i1];
                const float a = v0 * cs, bb = v1 * sn;
                const float d = v0 * sn, e = v1 * cs;
                const uint16_t k0 = f32_to_bf16_bits(a - bb), k1 = f32_to_bf16_bits(d + e);
                Cs[r * RS + i0] = k0; Cs[r * RS + i1] = k1;
                Kw[i0] = k0; Kw[i1] = k1;
            }
            for (int d = tid; d < HD; d += kT) Vw[d] = f32_to_bf16_bits(vn[d]);
        }
    } else {
        for (int i = tid; i < G * HD; i += kT) qs[i] = q[i];
    }
    __syncthreads();
    if (n_copy > 0) mbar_wait_bounded(&bars[0], 0, p.status);

    // ---- scores: this warp's 32 positions x the group's heads
    const int n8 = lane >> 2, qd = lane & 3;     // fragment column (head) and pair index inside the fragment
    {
        uint32_t qb[HD / 16][3][2];
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks)
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                const int k = 16 * ks + 8 * hf + 2 * qd;
                float f0 = 0.0f, f1 = 0.0f;
                if (n8 < G) { f0 = qs[n8 * HD + k]; f1 = qs[n8 * HD + k + 1]; }
                uint16_t h0, m0, l0, h1, m1, l1;
                split3(f0, h0, m0, l0);
                split3(f1, h1, m1, l1);
                qb[ks][0][hf] = (uint32_t)h0 | ((uint32_t)h1 << 16);
                qb[ks][1][hf] = (uint32_t)m0 | ((uint32_t)m1 << 16);
                qb[ks][2][hf] = (uint32_t)l0 | ((uint32_t)l1 << 16);
            }
        const float inv_sqrt = 1.0f / sqrtf((float)HD);
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
            const int t0 = warp * 32 + mt * 16;
            float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            if (t0 < cnt) {
                const uint32_t a_base = smem_u32(Cs + (t0 + (lane & 15)) * RS + (lane >> 4) * 8);
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks) {
                    uint32_t a[4];
                    ldsm_x4(a_base + ks * 32, a);
                    mma_bf16(acc, a, qb[ks][2][0], qb[ks][2][1]);
                    mma_bf16(acc, a, qb[ks][1][0], qb[ks][1][1]);
                    mma_bf16(acc, a, qb[ks][0][0], qb[ks][0][1]);
                }
            }
            // acc[0..1]: position t0 + n8, heads 2qd, 2qd+1; acc[2..3]: position t0 + n8 + 8
            const int ta = t0 + n8, tb = ta + 8;
            if (2 * qd < G) {
                scf[(2 * qd) * kAttnChunk + ta] = ta < cnt ? acc[0] * inv_sqrt : -CUDART_INF_F;
                scf[(2 * qd) * kAttnChunk + tb] = tb < cnt ? acc[2] * inv_sqrt : -CUDART_INF_F;
            }
            if (2 * qd + 1 < G) {
                scf[(2 * qd + 1) * kAttnChunk + ta] = ta < cnt ? acc[1] * inv_sqrt : -CUDART_INF_F;
                scf[(2 * qd + 1) * kAttnChunk + tb] = tb < cnt ? acc[3] * inv_sqrt : -CUDART_INF_F;
            }
        }
    }
    __syncthreads();

    // ---- the buffer now takes V: cached rows by bulk copy, the new row from the projection output, zeros
    // up to the next multiple of 16 rows (a probability of 0 times stale bits could still give a NaN)
    attn_mma_copy_rows<HD, G>(Cs, p.vcache + head_off + (size_t)s0 * HD, n_copy, &bars[1]);
    if (owner) {
        const float* vn = p.v_new + ((size_t)b * p.Nkv + g) * HD;
        const int r = pos - s0;
        for (int d = tid; d < HD; d += kT) Cs[r * RS + d] = f32_to_bf16_bits(vn[d]);
    }
    {
        const int cnt16 = min(kAttnChunk, (cnt + 15) & ~15);
        for (int i = tid; i < (cnt16 - cnt) * (HD / 8); i += kT) {
            const int r = cnt + i / (HD / 8), cc = i % (HD / 8);
            *reinterpret_cast<uint4*>(Cs + r * RS + cc * 8) = make_uint4(0, 0, 0, 0);
        }
    }

    // ---- softmax of the chunk: the fixed-order maximum and sum (as in attn_compute)
    float* rec0 = p.scratch + (((size_t)b * p.Nh + (size_t)g * G) * p.max_chunks + c) * (HD + 2);
    const size_t rec_stride = (size_t)p.max_chunks * (HD + 2);
    float sv[G], mv[G];
#pragma unroll
    for (int hh = 0; hh < G; ++hh) {
        sv[hh] = scf[hh * kAttnChunk + tid];
        const float w = warp_max(sv[hh]);
        if (lane == 0) redg[hh * 8 + warp] = w;
    }
    __syncthreads();
#pragma unroll
    for (int hh = 0; hh < G; ++hh) {
        float t = redg[hh * 8];
#pragma unroll
        for (int w = 1; w < kT / 32; ++w) t = fmaxf(t, redg[hh * 8 + w]);
        mv[hh] = t;
    }
    __syncthreads();
#pragma unroll
    for (int hh = 0; hh < G; ++hh) {
        const float pt = tid < cnt ? exp_fixed(sv[hh] - mv[hh]) : 0.0f;
        uint16_t h, m, l;
        split3(pt, h, m, l);
        Ps[(0 * G + hh) * L::kPRow + tid] = h;
        Ps[(1 * G + hh) * L::kPRow + tid] = m;
        Ps[(2 * G + hh) * L::kPRow + tid] = l;
        const float w = warp_sum_butterfly(pt);
        if (lane == 0) redg[hh * 8 + warp] = w;
    }
    __syncthreads();
#pragma unroll
    for (int hh = 0; hh < G; ++hh) {
        if (tid == hh) {
            float t = redg[hh * 8];
#pragma unroll
            for (int w = 1; w < kT / 32; ++w) t = t + redg[hh * 8 + w];
            rec0[hh * rec_stride + 0] = mv[hh];
            rec0[hh * rec_stride + 1] = t;
        }
    }
    if (n_copy > 0) mbar_wait_bounded(&bars[1], 0, p.status);
    __syncthreads();    // the new row and the zero rows, written by other threads

    // ---- o[d][head]: warp w takes dims 16w .. 16w+15
    if (warp < HD / 16) {
        const int d0 = warp * 16;
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        const int steps = (cnt + 15) >> 4;
        const uint32_t a_base = smem_u32(Cs + ((lane & 7) + ((lane >> 4) << 3)) * RS + d0 + ((lane >> 3) & 1) * 8);
        const uint16_t* pb = Ps + (n8 < G ? n8 : 0) * L::kPRow + 2 * qd;
        for (int kt = 0; kt < steps; ++kt) {
            uint32_t a[4];
            ldsm_x4_trans(a_base + kt * 16 * RS * 2, a);
#pragma unroll
            for (int s = 2; s >= 0; --s) {
                uint32_t b0 = 0, b1 = 0;
                if (n8 < G) {
                    b0 = *reinterpret_cast<const uint32_t*>(pb + s * G * L::kPRow + kt * 16);
                    b1 = *reinterpret_cast<const uint32_t*>(pb + s * G * L::kPRow + kt * 16 + 8);
                }
                mma_bf16(acc, a, b0, b1);
            }
        }
        // acc[0..1]: dim d0 + n8, heads 2qd, 2qd+1; acc[2..3]: dim d0 + n8 + 8
        if (2 * qd < G) {
            rec0[(2 * qd) * rec_stride + 2 + d0 + n8] = acc[0];
            rec0[(2 * qd) * rec_stride + 2 + d0 + n8 + 8] = acc[2];
        }
        if (2 * qd + 1 < G) {
            rec0[(2 * qd + 1) * rec_stride + 2 + d0 + n8] = acc[1];
            rec0[(2 * qd + 1) * rec_stride + 2 + d0 + n8 + 8] = acc[3];
        }
    }

    attn_merge_last<HD, G>(p, it, is_last);
}

}  // namespace
}  // namespace terb
