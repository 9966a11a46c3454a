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
// A chunk of the cache arrives by tiled TMA copies (one tensor map over the rows of the cache, boxes of 64 dims
// x 256 positions, 128-byte swizzle): rows of 128 bytes whose eight 16-byte pieces are permuted by the row
// number, so that the eight rows of an ldmatrix fall into different banks.  The box always has 256 rows: rows
// past the item's positions hold whatever follows in the cache (or zeros past its end) and are masked.
#pragma once
#include "attn.cuh"
#include "umma.cuh"

namespace terb {
namespace {

template <int HD, int G>
struct AttnMmaSmem {
    static constexpr int kBoxBytes = kAttnChunk * 128;               // one box: 256 rows x 64 dims
    static constexpr int kBoxes = HD / 64;
    static constexpr int kPRow = kAttnChunk + 8;                     // elements per probability row
    static constexpr int kChunkOff = 0;                              // K, then V (1024-byte aligned)
    static constexpr int kScOff = kBoxes * kBoxBytes;                // fp32 [G][256] scores
    static constexpr int kQRow = HD + 8;                             // elements per row of a q part
    static constexpr int kQpOff = kScOff + G * kAttnChunk * 4;       // bf16 [3][G][kQRow] parts of q
    // the probability parts, bf16 [3][G][kPRow], take the place of the scores and of q once both are consumed
    static constexpr int kPOff = kScOff;
    static constexpr int kAuxA = G * kAttnChunk * 4 + 3 * G * kQRow * 2, kAuxB = 3 * G * kPRow * 2;
    static constexpr int kBarOff = (kScOff + (kAuxA > kAuxB ? kAuxA : kAuxB) + 15) / 16 * 16;
    static constexpr int kCtasPerSm = (kBarOff + 16 + 1024 + 1024) * 3 <= 227 * 1024 ? 3 : 2;
    static constexpr int kBytes = kBarOff + 16 + 1024;               // + slack to align the buffer
};

// Byte offset of element e of row r inside the swizzled chunk buffer.
__device__ __forceinline__ uint32_t attn_sw(int r, int e) {
    return (uint32_t)((e >> 6) * (kAttnChunk * 128) + r * 128 + ((((e >> 3) & 7) ^ (r & 7)) << 4) + (e & 7) * 2);
}

// f = hi + mid + lo exactly (each part a bf16; 3 x 8 significant bits cover the 24 of an fp32; the differences
// are exact, so any rounding of the parts does)
__device__ __forceinline__ uint16_t cvt_bf16(float f) {
    uint16_t r;
    asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(r) : "f"(f));
    return r;
}
__device__ __forceinline__ void split3(float f, uint16_t& hi, uint16_t& mid, uint16_t& lo) {
    hi = cvt_bf16(f);
    const float r1 = f - bf16_bits_to_f32(hi);
    mid = cvt_bf16(r1);
    const float r2 = r1 - bf16_bits_to_f32(mid);
    lo = cvt_bf16(r2);
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

// The 256 rows from cache row `row` on, all dims, into the chunk buffer.  ONE thread calls it.
template <int HD>
__device__ __forceinline__ void attn_mma_load_chunk(uint8_t* buf, const CUtensorMap* map, int row, uint64_t* bar) {
    mbar_arrive_expect_tx(bar, (uint32_t)(HD / 64) * kAttnChunk * 128u);
#pragma unroll
    for (int bx = 0; bx < HD / 64; ++bx)
        asm volatile(
            "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
            ::"r"(smem_u32(buf + bx * kAttnChunk * 128)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bx * 64), "r"(row),
              "r"(smem_u32(bar))
            : "memory");
}

// One lane of every warp polls, the others wait for it.
__device__ __forceinline__ void attn_mma_wait(uint64_t* bar, int* status) {
    if ((threadIdx.x & 31) == 0) mbar_wait_bounded(bar, 0, status);
    __syncwarp();
}

// One item, all 256 threads.  Plain buffers (p.q, p.scratch, p.out); rotary and cache append fused when
// p.rope_table is set, exactly as in attn_compute.  kmap / vmap: tensor maps over the rows of p.kcache / p.vcache.
template <int HD, int G>
__device__ __forceinline__ void attn_compute_mma(const AttnParams& p, const CUtensorMap* kmap, const CUtensorMap* vmap,
                                                 const AttnItem& it, uint8_t* asmem, float* redg, int* is_last) {
    using L = AttnMmaSmem<HD, G>;
    uint8_t* Cb = asmem + L::kChunkOff;
    float* scf = reinterpret_cast<float*>(asmem + L::kScOff);
    uint16_t* Ps = reinterpret_cast<uint16_t*>(asmem + L::kPOff);
    uint16_t* Qp = reinterpret_cast<uint16_t*>(asmem + L::kQpOff);
    uint64_t* bars = reinterpret_cast<uint64_t*>(asmem + L::kBarOff);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (!it.active) return;
    const int g = it.g, b = it.b, c = it.c, pos = it.pos, s0 = it.s0, cnt = it.cnt, n_copy = it.n_copy;
    const bool owner = it.owner;
    const size_t head_off = it.head_off;
    const int row0 = (int)(head_off / HD) + s0;        // first cache row of the chunk

    if (tid == 0 && n_copy > 0) attn_mma_load_chunk<HD>(Cb, kmap, row0, &bars[0]);

    const float* q = p.q + ((size_t)b * p.Nh + (size_t)g * G) * HD;
    uint16_t knew0 = 0, knew1 = 0;       // the new position's rotated K (owner CTA: threads < HD/2)
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
            uint16_t h, m, l;
            split3(a - bb, h, m, l);
            Qp[(0 * G + hh) * L::kQRow + i0] = h; Qp[(1 * G + hh) * L::kQRow + i0] = m; Qp[(2 * G + hh) * L::kQRow + i0] = l;
            split3(d + e, h, m, l);
            Qp[(0 * G + hh) * L::kQRow + i1] = h; Qp[(1 * G + hh) * L::kQRow + i1] = m; Qp[(2 * G + hh) * L::kQRow + i1] = l;
        }
        if (owner) {
            const float* kn = p.k_new + ((size_t)b * p.Nkv + g) * HD;
            const float* vn = p.v_new + ((size_t)b * p.Nkv + g) * HD;
            uint16_t* Kw = p.kcache_w + head_off + (size_t)pos * HD;
            uint16_t* Vw = p.vcache_w + head_off + (size_t)pos * HD;
            if (tid < half) {
                const int kk = tid;
                const int i0 = p.neox ? kk : 2 * kk, i1 = p.neox ? kk + half : 2 * kk + 1;
                const float cs = row[2 * kk], sn = row[2 * kk + 1];
                const float v0 = kn[i0], v1 = kn[i1];
                const float a = v0 * cs, bb = v1 * sn;
                const float d = v0 * sn, e = v1 * cs;
                knew0 = f32_to_bf16_bits(a - bb);
                knew1 = f32_to_bf16_bits(d + e);
                Kw[i0] = knew0; Kw[i1] = knew1;
            }
            for (int d = tid; d < HD; d += kT) Vw[d] = f32_to_bf16_bits(vn[d]);
        }
    } else {
        for (int i = tid; i < G * HD; i += kT) {
            const int hh = i / HD, d = i % HD;
            uint16_t h, m, l;
            split3(q[i], h, m, l);
            Qp[(0 * G + hh) * L::kQRow + d] = h; Qp[(1 * G + hh) * L::kQRow + d] = m; Qp[(2 * G + hh) * L::kQRow + d] = l;
        }
    }
    if (n_copy > 0) attn_mma_wait(&bars[0], p.status);
    if (owner && tid < HD / 2) {
        // after the copy has landed (its box covers this row too, with what the cache held before)
        const int r = pos - s0, kk = tid;
        const int i0 = p.neox ? kk : 2 * kk, i1 = p.neox ? kk + HD / 2 : 2 * kk + 1;
        *reinterpret_cast<uint16_t*>(Cb + attn_sw(r, i0)) = knew0;
        *reinterpret_cast<uint16_t*>(Cb + attn_sw(r, i1)) = knew1;
    }
    __syncthreads();

    // ---- scores: this warp's 32 positions x the group's heads
    const int n8 = lane >> 2, qd = lane & 3;     // fragment column (head) and pair index inside the fragment
    {
        const float inv_sqrt = 1.0f / sqrtf((float)HD);
        const uint32_t cb = smem_u32(Cb);
        // six independent accumulator chains: two tiles of 16 positions x three parts of q
        float acc[2][3][4];
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
            for (int s = 0; s < 3; ++s)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[mt][s][e] = 0.0f;
        const int tw = warp * 32;
        if (tw < cnt) {
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks) {
                // this lane's pieces of the three parts of q: head n8, dims 16ks + 2qd, +1 and 16ks + 8 + 2qd, +1
                uint32_t qb[3][2];
#pragma unroll
                for (int s = 0; s < 3; ++s) {
                    qb[s][0] = qb[s][1] = 0;
                    if (n8 < G) {
                        const uint16_t* qp = Qp + (s * G + n8) * L::kQRow + 16 * ks + 2 * qd;
                        qb[s][0] = *reinterpret_cast<const uint32_t*>(qp);
                        qb[s][1] = *reinterpret_cast<const uint32_t*>(qp + 8);
                    }
                }
#pragma unroll
                for (int mt = 0; mt < 2; ++mt) {
                    uint32_t a[4];
                    ldsm_x4(cb + attn_sw(tw + mt * 16 + (lane & 15), 16 * ks + (lane >> 4) * 8), a);
#pragma unroll
                    for (int s = 0; s < 3; ++s) mma_bf16(acc[mt][s], a, qb[s][0], qb[s][1]);
                }
            }
        }
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
            // element 0..1: position t0 + n8, heads 2qd, 2qd+1; element 2..3: position t0 + n8 + 8
            float r[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) r[e] = (acc[mt][2][e] + acc[mt][1][e]) + acc[mt][0][e];
            const int ta = tw + mt * 16 + n8, tb = ta + 8;
            if (2 * qd < G) {
                scf[(2 * qd) * kAttnChunk + ta] = ta < cnt ? r[0] * inv_sqrt : -CUDART_INF_F;
                scf[(2 * qd) * kAttnChunk + tb] = tb < cnt ? r[2] * inv_sqrt : -CUDART_INF_F;
            }
            if (2 * qd + 1 < G) {
                scf[(2 * qd + 1) * kAttnChunk + ta] = ta < cnt ? r[1] * inv_sqrt : -CUDART_INF_F;
                scf[(2 * qd + 1) * kAttnChunk + tb] = tb < cnt ? r[3] * inv_sqrt : -CUDART_INF_F;
            }
        }
    }
    __syncthreads();

    // ---- the buffer now takes V
    if (tid == 0 && n_copy > 0) {
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the buffer was read by ordinary loads
        attn_mma_load_chunk<HD>(Cb, vmap, row0, &bars[1]);
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
    if (n_copy > 0) attn_mma_wait(&bars[1], p.status);
    // after the copy: the new position's row from the projection output, and zeros from the item's last position
    // to the next multiple of 16 rows (a probability of 0 times stale bits could still give a NaN)
    if (owner) {
        const float* vn = p.v_new + ((size_t)b * p.Nkv + g) * HD;
        const int r = pos - s0;
        for (int d = tid; d < HD; d += kT) *reinterpret_cast<uint16_t*>(Cb + attn_sw(r, d)) = f32_to_bf16_bits(vn[d]);
    }
    {
        const int cnt16 = min(kAttnChunk, (cnt + 15) & ~15);
        for (int i = tid; i < (cnt16 - cnt) * (HD / 8); i += kT) {
            const int r = cnt + i / (HD / 8), cc = i % (HD / 8);
            *reinterpret_cast<uint4*>(Cb + attn_sw(r, cc * 8)) = make_uint4(0, 0, 0, 0);
        }
    }
    __syncthreads();

    // ---- o[d][head]: warp w takes dims 16w .. 16w+15; six accumulator chains (three parts x even / odd step)
    if (warp < HD / 16) {
        const int d0 = warp * 16;
        float acc[2][3][4];
#pragma unroll
        for (int par = 0; par < 2; ++par)
#pragma unroll
            for (int s = 0; s < 3; ++s)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[par][s][e] = 0.0f;
        const int steps = (cnt + 15) >> 4;
        const uint32_t cb = smem_u32(Cb);
        const int trow = (lane & 7) + ((lane >> 4) << 3), dcol = d0 + ((lane >> 3) & 1) * 8;
        const uint16_t* pb = Ps + (n8 < G ? n8 : 0) * L::kPRow + 2 * qd;
        for (int kt2 = 0; kt2 < steps; kt2 += 2) {
#pragma unroll
            for (int par = 0; par < 2; ++par) {
                const int kt = kt2 + par;
                if (kt < steps) {
                    uint32_t a[4];
                    ldsm_x4_trans(cb + attn_sw(kt * 16 + trow, dcol), a);
#pragma unroll
                    for (int s = 0; s < 3; ++s) {
                        uint32_t b0 = 0, b1 = 0;
                        if (n8 < G) {
                            b0 = *reinterpret_cast<const uint32_t*>(pb + s * G * L::kPRow + kt * 16);
                            b1 = *reinterpret_cast<const uint32_t*>(pb + s * G * L::kPRow + kt * 16 + 8);
                        }
                        mma_bf16(acc[par][s], a, b0, b1);
                    }
                }
            }
        }
        // element 0..1: dim d0 + n8, heads 2qd, 2qd+1; element 2..3: dim d0 + n8 + 8
        float r[4];
#pragma unroll
        for (int e = 0; e < 4; ++e)
            r[e] = ((acc[0][2][e] + acc[1][2][e]) + (acc[0][1][e] + acc[1][1][e])) + (acc[0][0][e] + acc[1][0][e]);
        if (2 * qd < G) {
            rec0[(2 * qd) * rec_stride + 2 + d0 + n8] = r[0];
            rec0[(2 * qd) * rec_stride + 2 + d0 + n8 + 8] = r[2];
        }
        if (2 * qd + 1 < G) {
            rec0[(2 * qd + 1) * rec_stride + 2 + d0 + n8] = r[1];
            rec0[(2 * qd + 1) * rec_stride + 2 + d0 + n8 + 8] = r[3];
        }
    }

    attn_merge_last<HD, G>(p, it, is_last);
}

}  // namespace
}  // namespace terb
