// Split-KV GQA attention over a bf16 cache as device functions, shared by the stand-alone attention
// kernel (glue_sm100.cu) and the persistent decode kernel (decode_sm100.cu).
//
// Chunked online softmax in a fixed order: the context is cut in chunks of 256 positions; one CTA
// computes, for one (sequence, KV head, chunk) and every query head of the group, the chunk maximum
// m, l = sum exp(s - m) (block order) and o[d] = sum_t exp(s_t - m) V[t][d] (t ascending, fused
// multiply-adds).  The chunks are merged left to right, by a second kernel or by the last CTA of a
// KV head to finish.  Score of one position: 8 lanes each take 8 consecutive dims of every 64, fused
// multiply-adds in ascending dim order, then an xor butterfly (4,2,1) over the 8 lanes.
//
// Reference kernels restated (formulas, not code): rope_k / kv_copy_k / attention_k
// (cuda/ter_cuda_forward_packed.cu:64-90,118-157; NEOX variant cuda/ter_cuda_forward_bitnet.cu:185-201).
#pragma once
#include "normq.cuh"

namespace terb {
namespace {

constexpr int kMaxGroup = 8;   // query heads per KV head

// Shared memory of one attention item: K chunk, V chunk (bf16 [256][HD] each, filled by one 1-D TMA
// bulk copy each), the group's query heads, the score / probability rows, barriers.
// COMPACT: K and V take turns in ONE chunk buffer (V is fetched once the scores are done), which
// halves the footprint so that two to five CTAs fit an SM: for large grids (token batches, prompt
// tiles), where throughput counts; the two-buffer form keeps both copies in flight for a lone step.
template <int HD, int G, bool COMPACT>
struct AttnSmem {
    static constexpr int kKOff = 0;
    static constexpr int kVOff = COMPACT ? 0 : kAttnChunk * HD * 2;
    static constexpr int kQOff = (COMPACT ? 1 : 2) * kAttnChunk * HD * 2;
    static constexpr int kScOff = kQOff + G * HD * 4;
    static constexpr int kRedOff = kScOff + G * kAttnChunk * 4;
    static constexpr int kBarOff = kRedOff + 64;
    static constexpr int kBytes = kBarOff + 16;
};

// One (chunk, KV head, row) work item and what follows from the row's position.
struct AttnItem {
    int c, g, b, bs;        // chunk, head group (= KV head unless the params deal a KV head's heads to several items), row,
                            // sequence whose cache is read
    int gk;                 // KV head
    int pos, seq_len, s0, cnt, n_copy;
    bool active, fused, owner;
    size_t head_off;
};

template <int HD>
__device__ __forceinline__ AttnItem attn_item(const AttnParams& p, int c, int g, int b, int pos) {
    AttnItem it;
    it.c = c; it.g = g; it.b = b;
    const int kvd = p.kv_div > 1 ? p.kv_div : 1;
    it.gk = g / kvd;
    it.bs = p.shared_seq ? p.shared_seq - 1 : b;
    it.pos = pos;
    it.seq_len = pos + 1;
    it.s0 = c * kAttnChunk;
    it.active = !(it.s0 >= it.seq_len || it.seq_len > p.Smax || pos < 0);
    it.cnt = min(kAttnChunk, it.seq_len - it.s0);
    it.fused = p.rope_table != nullptr;
    it.owner = it.fused && (pos >= it.s0) && (pos < it.s0 + kAttnChunk);   // this chunk holds the new row
    it.n_copy = it.owner ? it.cnt - 1 : it.cnt;                            // rows already in the cache
    it.head_off = ((size_t)it.bs * (p.Nkv / kvd) + it.gk) * (size_t)p.Smax * HD;
    return it;
}

// Starts the copies of the item's cached K rows (and V rows in the two-buffer form).  ONE thread calls it.
// The rows copied are older than the row's position, so the copies may start before the new q/k/v exist.
template <int HD, int G, bool COMPACT>
__device__ __forceinline__ void attn_issue_kv(const AttnParams& p, const AttnItem& it, uint8_t* asmem) {
    using L = AttnSmem<HD, G, COMPACT>;
    if (!it.active || it.n_copy <= 0) return;
    uint16_t* Ks = reinterpret_cast<uint16_t*>(asmem + L::kKOff);
    uint16_t* Vs = reinterpret_cast<uint16_t*>(asmem + L::kVOff);
    uint64_t* bars = reinterpret_cast<uint64_t*>(asmem + L::kBarOff);
    const uint32_t bytes = (uint32_t)it.n_copy * HD * 2u;
    mbar_arrive_expect_tx(&bars[0], bytes);
    bulk_g2s(Ks, p.kcache + it.head_off + (size_t)it.s0 * HD, bytes, &bars[0]);
    if (!COMPACT) {
        mbar_arrive_expect_tx(&bars[1], bytes);
        bulk_g2s(Vs, p.vcache + it.head_off + (size_t)it.s0 * HD, bytes, &bars[1]);
    }
}

// Rescaling factors of an ordered merge of up to 32 chunk records, prepared side by side: lane k of the warp
// passes the chunk maximum mk of its record (-inf beyond the last one); M is the running maximum before the first
// of them.  On return lane k holds a = exp(M_before_k - M_after_k) and b = exp(mk - M_after_k), the two factors
// a thread merging the records one after the other would compute for record k, and Mn = M_after_k.  The whole warp
// calls it.  Same operations on the same values; only the exponentials no longer wait for one another.
__device__ __forceinline__ void merge_factors(float M, float mk, int lane, float& a, float& b, float& Mn) {
    Mn = mk;                                             // inclusive prefix maximum over the lanes
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float up = __shfl_up_sync(0xffffffffu, Mn, o);
        if (lane >= o) Mn = fmaxf(Mn, up);
    }
    Mn = fmaxf(M, Mn);
    float Mp = __shfl_up_sync(0xffffffffu, Mn, 1);
    if (lane == 0) Mp = M;
    a = exp_fixed(Mp - Mn);
    b = exp_fixed(mk - Mn);
}

// Merge of the chunks by the last CTA of this (row, KV head) to finish, when the caller gave arrival
// counters; the order of the merge is fixed (chunk 0, 1, 2, ...) whoever performs it.  All threads call it.
template <int HD, int G>
__device__ __forceinline__ void attn_merge_last(const AttnParams& p, const AttnItem& it, int* is_last) {
    if (!p.counters) return;
    const int tid = threadIdx.x, b = it.b, g = it.g;
    const size_t rec_stride = (size_t)p.max_chunks * (HD + 2);
    const int nc = (it.seq_len + kAttnChunk - 1) / kAttnChunk;
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        int* cnt_p = p.counters + (size_t)b * p.Nkv + g;
        const int old = atomicAdd(cnt_p, 1);
        *is_last = (old == nc - 1);
        if (*is_last) *cnt_p = 0;          // ready for the next step
    }
    __syncthreads();
    if (*is_last) {
        __threadfence();
        const int lane = tid & 31;
        for (int idx = tid; idx < G * HD; idx += kT) {      // HD is a multiple of 32: a warp serves one head
            const int hh = idx / HD, d = idx % HD;
            const float* rec = p.scratch + ((size_t)b * p.Nh + (size_t)g * G + hh) * rec_stride;
            float M = __ldcg(rec), Lsum = __ldcg(rec + 1), O = __ldcg(rec + 2 + d);
            for (int cb = 1; cb < nc; cb += 32) {
                const int nb = min(32, nc - cb);
                float mk = -CUDART_INF_F, lk = 0.0f;
                if (lane < nb) {
                    const float* r = rec + (size_t)(cb + lane) * (HD + 2);
                    mk = __ldcg(r);
                    lk = __ldcg(r + 1);
                }
                float ak, bk, Mn;
                merge_factors(M, mk, lane, ak, bk, Mn);
                for (int k = 0; k < nb; ++k) {
                    const float oc = __ldcg(rec + (size_t)(cb + k) * (HD + 2) + 2 + d);
                    const float a = __shfl_sync(0xffffffffu, ak, k), bb = __shfl_sync(0xffffffffu, bk, k);
                    const float lc = __shfl_sync(0xffffffffu, lk, k);
                    Lsum = fmaf(lc, bb, Lsum * a);
                    O = fmaf(oc, bb, O * a);
                }
                M = __shfl_sync(0xffffffffu, Mn, nb - 1);
            }
            p.out[((size_t)b * p.Nh + (size_t)g * G + hh) * HD + d] = O / Lsum;
        }
    }
}

// Flag-in-data inputs and outputs of an item inside the persistent decode kernel (MODE 2 of attn_compute):
// q / k / v of the new position arrive as tagged vectors written by other CTAs; partial records and the
// attention output leave as tagged words; the rotary row and the chunk's (m, l) live in shared memory.
struct AttnTagged {
    TaggedSrc q, k, v;        // [Nh*Hd], [Nkv*Hd], [Nkv*Hd] of the one sequence
    const float* rope_row;    // shared memory: [Hd/2][2] of the position
    uint4* rec_t;             // [Nh][max_chunks][Hd/2 + 1] tagged partial records
    uint4* att_t;             // [Nh*Hd/2] tagged output
    uint32_t seq;             // generation of the records and of the output
    float* ml_s;              // shared memory, 2*G floats
#ifdef TERB_TRACE
    unsigned long long* trace;
#endif
};
#ifdef TERB_TRACE
#define ATR(k) do { if (MODE == 2 && tg && tg->trace && threadIdx.x == 0) tg->trace[k] = globaltimer_ns(); } while (0)
#else
#define ATR(k) do {} while (0)
#endif

// The item's arithmetic, by all 256 threads of the CTA, after attn_issue_kv.  When p.rope_table is set it
// also does what rope_kv_kernel does, for its own data only: it rotates the group's query heads on the fly
// (the q buffer is left untouched) and, in the CTA whose chunk contains the new position, rotates k, rounds
// k and v to bf16, appends them to the cache and uses them.  Otherwise q is taken as already rotated and
// the cache as already appended.
// parity: phase of the two copy barriers (0 for a kernel that uses them once).  redg: kMaxGroup*8 floats and
// is_last: one int of shared memory.
// MODE 0: plain buffers; the chunks are merged by a second kernel or, with p.counters, by the last CTA of a
// KV head to finish.  MODE 2 (persistent decode kernel, one sequence, not COMPACT): tagged inputs and
// outputs (tg); the CTA of chunk 0 merges, polling the other chunks' records in chunk order.
template <int HD, int G, bool COMPACT, int MODE>
__device__ __forceinline__ void attn_compute(const AttnParams& p, const AttnItem& it, uint8_t* asmem, float* redg,
                                             int* is_last, uint32_t parity, const AttnTagged* tg = nullptr) {
    using L = AttnSmem<HD, G, COMPACT>;
    uint16_t* Ks = reinterpret_cast<uint16_t*>(asmem + L::kKOff);
    uint16_t* Vs = reinterpret_cast<uint16_t*>(asmem + L::kVOff);
    float* qs = reinterpret_cast<float*>(asmem + L::kQOff);
    // scores, then probabilities: [head][position]; the throughput variant keeps [position][head] so that
    // one vector load gives a position's probabilities for all heads of the group
    float* scf = reinterpret_cast<float*>(asmem + L::kScOff);
    auto SC = [&](int hh, int t) -> float& { return COMPACT ? scf[t * G + hh] : scf[hh * kAttnChunk + t]; };
    uint64_t* bars = reinterpret_cast<uint64_t*>(asmem + L::kBarOff);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (!it.active) return;
    ATR(0);
    const int g = it.g, gk = it.gk, b = it.b, c = it.c, pos = it.pos, s0 = it.s0, cnt = it.cnt, n_copy = it.n_copy;
    const bool owner = it.owner;
    const bool cache_writer = p.kv_div <= 1 || g % p.kv_div == 0;   // one of the items of a KV head appends the new row
    const size_t head_off = it.head_off;
    const uint16_t* V = p.vcache + head_off;

    // query heads of the group (rotated here when fused)
    const float* q = p.q + ((size_t)b * p.Nh + (size_t)g * G) * HD;
    auto ldq = [&](int i) -> float {
        if constexpr (MODE == 2) return tagged_ld(tg->q, g * G * HD + i); else return q[i];
    };
    // a pair of elements of a tagged vector (base + i0, base + i1) with both requests in flight together
    auto ld_pair = [&](const TaggedSrc& src, int base, int i0, int i1, float& v0, float& v1) {
        const uint4* w0p = src.words + ((base + i0) >> 1);
        const uint4* w1p = src.words + ((base + i1) >> 1);
        uint4 w0 = ld_volatile16(w0p);
        uint4 w1 = w1p == w0p ? w0 : ld_volatile16(w1p);
        if (w0.y != src.seq || w0.w != src.seq) w0 = poll_tagged(w0p, src.seq, src.ctx);
        if (w1p == w0p) w1 = w0;
        else if (w1.y != src.seq || w1.w != src.seq) w1 = poll_tagged(w1p, src.seq, src.ctx);
        v0 = __uint_as_float(((base + i0) & 1) ? w0.z : w0.x);
        v1 = __uint_as_float(((base + i1) & 1) ? w1.z : w1.x);
    };
    if (it.fused) {
        const float* row = MODE == 2 ? tg->rope_row : p.rope_table + (size_t)pos * HD;
        const int half = HD / 2;
        for (int idx = tid; idx < G * half; idx += kT) {
            const int hh = idx / half, kk = idx % half;
            const int i0 = p.neox ? kk : 2 * kk, i1 = p.neox ? kk + half : 2 * kk + 1;
            const float cs = row[2 * kk], sn = row[2 * kk + 1];
            float v0, v1;
            if constexpr (MODE == 2) ld_pair(tg->q, g * G * HD + hh * HD, i0, i1, v0, v1);
            else { v0 = ldq(hh * HD + i0); v1 = ldq(hh * HD + i1); }
            const float a = v0 * cs, bb = v1 * sn;
            const float d = v0 * sn, e = v1 * cs;
            qs[hh * HD + i0] = a - bb;
            qs[hh * HD + i1] = d + e;
        }
        if (owner) {
            const float* kn = p.k_new + ((size_t)b * p.Nkv + gk) * HD;
            const float* vn = p.v_new + ((size_t)b * p.Nkv + gk) * HD;
            auto ldk = [&](int i) -> float {
                if constexpr (MODE == 2) return tagged_ld(tg->k, gk * HD + i); else return kn[i];
            };
            auto ldv = [&](int i) -> float {
                if constexpr (MODE == 2) return tagged_ld(tg->v, gk * HD + i); else return vn[i];
            };
            uint16_t* Kw = p.kcache_w + head_off + (size_t)pos * HD;
            uint16_t* Vw = p.vcache_w + head_off + (size_t)pos * HD;
            const int r = pos - s0;
            for (int kk = tid; kk < half; kk += kT) {
                const int i0 = p.neox ? kk : 2 * kk, i1 = p.neox ? kk + half : 2 * kk + 1;
                const float cs = row[2 * kk], sn = row[2 * kk + 1];
                float v0, v1;
                if constexpr (MODE == 2) ld_pair(tg->k, gk * HD, i0, i1, v0, v1);
                else { v0 = ldk(i0); v1 = ldk(i1); }
                const float a = v0 * cs, bb = v1 * sn;
                const float d = v0 * sn, e = v1 * cs;
                const uint16_t k0 = f32_to_bf16_bits(a - bb), k1 = f32_to_bf16_bits(d + e);
                Ks[r * HD + i0] = k0; Ks[r * HD + i1] = k1;
                if (cache_writer) { Kw[i0] = k0; Kw[i1] = k1; }
            }
            for (int d = tid; d < HD; d += kT) {
                const uint16_t vb = f32_to_bf16_bits(ldv(d));
                if (!COMPACT) Vs[r * HD + d] = vb;     // COMPACT: the buffer still holds K; written after the scores
                if (cache_writer) Vw[d] = vb;
            }
        }
    } else {
        for (int i = tid; i < G * HD; i += kT) qs[i] = ldq(i);
    }
    __syncthreads();
    ATR(1);
    if (n_copy > 0) mbar_wait_bounded(&bars[0], parity, p.status);
    ATR(2);

    const float inv_sqrt = 1.0f / sqrtf((float)HD);
    if constexpr (G * HD / 8 <= 64) {
        // The form below with this lane's slices of the query heads held in registers (the lane always
        // multiplies the same 8 dims of every 64): one 16-byte load per position and piece instead of one
        // per position, piece and head.  Same operations in the same order.
        const int sub = lane >> 3, j = lane & 7;
        float qr[G][HD / 8];
#pragma unroll
        for (int hh = 0; hh < G; ++hh)
#pragma unroll
            for (int pc = 0; pc < HD / 64; ++pc) {
                const float4 qa = *reinterpret_cast<const float4*>(&qs[hh * HD + pc * 64 + 8 * j]);
                const float4 qb = *reinterpret_cast<const float4*>(&qs[hh * HD + pc * 64 + 8 * j + 4]);
                qr[hh][pc * 8 + 0] = qa.x; qr[hh][pc * 8 + 1] = qa.y; qr[hh][pc * 8 + 2] = qa.z; qr[hh][pc * 8 + 3] = qa.w;
                qr[hh][pc * 8 + 4] = qb.x; qr[hh][pc * 8 + 5] = qb.y; qr[hh][pc * 8 + 6] = qb.z; qr[hh][pc * 8 + 7] = qb.w;
            }
#pragma unroll 2
        for (int itn = 0; itn < 8; ++itn) {
            const int t = warp * 32 + itn * 4 + sub;
            const bool valid = t < cnt;
            float kv[HD / 8];
#pragma unroll
            for (int pc = 0; pc < HD / 64; ++pc) {
                uint4 raw = make_uint4(0, 0, 0, 0);
                if (valid) raw = *reinterpret_cast<const uint4*>(Ks + t * HD + pc * 64 + 8 * j);
                kv[pc * 8 + 0] = bf16_bits_to_f32(raw.x & 0xffffu);
                kv[pc * 8 + 1] = bf16_bits_to_f32(raw.x >> 16);
                kv[pc * 8 + 2] = bf16_bits_to_f32(raw.y & 0xffffu);
                kv[pc * 8 + 3] = bf16_bits_to_f32(raw.y >> 16);
                kv[pc * 8 + 4] = bf16_bits_to_f32(raw.z & 0xffffu);
                kv[pc * 8 + 5] = bf16_bits_to_f32(raw.z >> 16);
                kv[pc * 8 + 6] = bf16_bits_to_f32(raw.w & 0xffffu);
                kv[pc * 8 + 7] = bf16_bits_to_f32(raw.w >> 16);
            }
            float acc[G];
#pragma unroll
            for (int hh = 0; hh < G; ++hh) {
                float a = 0.0f;
#pragma unroll
                for (int e = 0; e < HD / 8; ++e) a = fmaf(qr[hh][e], kv[e], a);
                acc[hh] = a;
            }
#pragma unroll
            for (int hh = 0; hh < G; ++hh) acc[hh] = acc[hh] + __shfl_xor_sync(0xffffffffu, acc[hh], 4);
#pragma unroll
            for (int hh = 0; hh < G; ++hh) acc[hh] = acc[hh] + __shfl_xor_sync(0xffffffffu, acc[hh], 2);
#pragma unroll
            for (int hh = 0; hh < G; ++hh) acc[hh] = acc[hh] + __shfl_xor_sync(0xffffffffu, acc[hh], 1);
            if (j == 0) {
#pragma unroll
                for (int hh = 0; hh < G; ++hh) SC(hh, t) = valid ? acc[hh] * inv_sqrt : -CUDART_INF_F;
            }
        }
    } else {
    const int sub = lane >> 3, j = lane & 7;
#pragma unroll 2
    for (int itn = 0; itn < 8; ++itn) {
        const int t = warp * 32 + itn * 4 + sub;
        const bool valid = t < cnt;
        float kv[HD / 8];   // this lane's dims: 8 per 64-dim piece
#pragma unroll
        for (int pc = 0; pc < HD / 64; ++pc) {
            uint4 raw = make_uint4(0, 0, 0, 0);
            if (valid) raw = *reinterpret_cast<const uint4*>(Ks + t * HD + pc * 64 + 8 * j);
            kv[pc * 8 + 0] = bf16_bits_to_f32(raw.x & 0xffffu);
            kv[pc * 8 + 1] = bf16_bits_to_f32(raw.x >> 16);
            kv[pc * 8 + 2] = bf16_bits_to_f32(raw.y & 0xffffu);
            kv[pc * 8 + 3] = bf16_bits_to_f32(raw.y >> 16);
            kv[pc * 8 + 4] = bf16_bits_to_f32(raw.z & 0xffffu);
            kv[pc * 8 + 5] = bf16_bits_to_f32(raw.z >> 16);
            kv[pc * 8 + 6] = bf16_bits_to_f32(raw.w & 0xffffu);
            kv[pc * 8 + 7] = bf16_bits_to_f32(raw.w >> 16);
        }
#pragma unroll
        for (int hh = 0; hh < G; ++hh) {
            float acc = 0.0f;
#pragma unroll
            for (int pc = 0; pc < HD / 64; ++pc) {
                const float4 qa = *reinterpret_cast<const float4*>(&qs[hh * HD + pc * 64 + 8 * j]);
                const float4 qb = *reinterpret_cast<const float4*>(&qs[hh * HD + pc * 64 + 8 * j + 4]);
                acc = fmaf(qa.x, kv[pc * 8 + 0], acc);
                acc = fmaf(qa.y, kv[pc * 8 + 1], acc);
                acc = fmaf(qa.z, kv[pc * 8 + 2], acc);
                acc = fmaf(qa.w, kv[pc * 8 + 3], acc);
                acc = fmaf(qb.x, kv[pc * 8 + 4], acc);
                acc = fmaf(qb.y, kv[pc * 8 + 5], acc);
                acc = fmaf(qb.z, kv[pc * 8 + 6], acc);
                acc = fmaf(qb.w, kv[pc * 8 + 7], acc);
            }
            acc = acc + __shfl_xor_sync(0xffffffffu, acc, 4);
            acc = acc + __shfl_xor_sync(0xffffffffu, acc, 2);
            acc = acc + __shfl_xor_sync(0xffffffffu, acc, 1);
            if (j == 0) SC(hh, t) = valid ? acc * inv_sqrt : -CUDART_INF_F;
        }
    }
    }
    __syncthreads();
    ATR(3);
    if (COMPACT) {
        // every score is computed: the chunk buffer now takes V (rows already in the cache by TMA, the
        // new row, in the CTA that owns it, from the projection output)
        if (tid == 0 && n_copy > 0) {
            const uint32_t bytes = (uint32_t)n_copy * HD * 2u;
            mbar_arrive_expect_tx(&bars[1], bytes);
            bulk_g2s(Vs, V + (size_t)s0 * HD, bytes, &bars[1]);
        }
        if (owner) {
            const float* vn = p.v_new + ((size_t)b * p.Nkv + g) * HD;
            const int r = pos - s0;
            for (int d = tid; d < HD; d += kT) Vs[r * HD + d] = f32_to_bf16_bits(vn[d]);
        }
    }

    float* rec0 = p.scratch + (((size_t)b * p.Nh + (size_t)g * G) * p.max_chunks + c) * (HD + 2);
    const size_t rec_stride = (size_t)p.max_chunks * (HD + 2);
    // chunk maximum and sum of exponentials of every head of the group: same values, in the same
    // order, as block_max / block_sum per head, with one barrier per reduction for all heads together
    float sv[kMaxGroup], mv[kMaxGroup];
#pragma unroll
    for (int hh = 0; hh < kMaxGroup; ++hh) {
        sv[hh] = -CUDART_INF_F;
        if (hh < G) {
            sv[hh] = SC(hh, tid);
            const float w = warp_max(sv[hh]);
            if (lane == 0) redg[hh * 8 + warp] = w;
        }
    }
    __syncthreads();
#pragma unroll
    for (int hh = 0; hh < kMaxGroup; ++hh) {
        mv[hh] = 0.0f;
        if (hh < G) {
            float t = redg[hh * 8];
#pragma unroll
            for (int w = 1; w < kT / 32; ++w) t = fmaxf(t, redg[hh * 8 + w]);
            mv[hh] = t;
        }
    }
    __syncthreads();
#pragma unroll
    for (int hh = 0; hh < kMaxGroup; ++hh) {
        if (hh < G) {
            const float pt = tid < cnt ? exp_fixed(sv[hh] - mv[hh]) : 0.0f;
            SC(hh, tid) = pt;
            const float w = warp_sum_butterfly(pt);
            if (lane == 0) redg[hh * 8 + warp] = w;
        }
    }
    __syncthreads();
#pragma unroll
    for (int hh = 0; hh < kMaxGroup; ++hh) {
        if (tid == hh && hh < G) {
            float t = redg[hh * 8];
#pragma unroll
            for (int w = 1; w < kT / 32; ++w) t = t + redg[hh * 8 + w];
            if constexpr (MODE == 2) {
                tg->ml_s[hh] = mv[hh];
                tg->ml_s[G + hh] = t;
            } else {
                rec0[hh * rec_stride + 0] = mv[hh];
                rec0[hh * rec_stride + 1] = t;
            }
        }
    }
    ATR(4);
    if (n_copy > 0) mbar_wait_bounded(&bars[1], parity, p.status);

    // o[hh][d] = sum_t p[t][hh] * V[t][d], ascending t
    if constexpr (MODE == 2) {
        // every (head, dim) pair of this thread at once (independent accumulators, each its own ascending
        // chain of fused multiply-adds), then the records go out as tagged words or are merged right here
        static_assert(!COMPACT, "tagged attention uses the two-buffer form");
        // one thread per (head, pair of adjacent dims): a 4-byte load brings both V values, a 16-byte load four
        // probabilities; each (head, dim) keeps its own ascending chain of fused multiply-adds
        constexpr int kPairs = G * HD / 2;
        constexpr int NI = (kPairs + kT - 1) / kT;
        float acc0[NI], acc1[NI];
        const float* prp[NI];
        const uint16_t* vp[NI];
#pragma unroll
        for (int i = 0; i < NI; ++i) {
            const int idx = tid + i * kT;
            const int hh = idx < kPairs ? idx / (HD / 2) : 0;
            acc0[i] = acc1[i] = 0.0f;
            prp[i] = scf + hh * kAttnChunk;
            vp[i] = Vs + 2 * (idx % (HD / 2));
        }
        if constexpr (G * HD <= kT / 2) {
            // Few chains (at most 128): one thread per (head, dim), so that twice as many warps share the
            // positions' loads and conversions (a chain is 3.25 instead of 5.25 instructions per position); the
            // values then go through the query buffer (free since the scores) to the thread of their dim pair.
            float a = 0.0f;
            if (tid < G * HD) {
                const float* pq = scf + (tid / HD) * kAttnChunk;
                const uint16_t* vq = Vs + (tid % HD);
                const int cnt4 = cnt & ~3;
                float4 pn = make_float4(0.f, 0.f, 0.f, 0.f);
                uint16_t wn[4] = {0, 0, 0, 0};
                auto load = [&](int t) {
                    pn = *reinterpret_cast<const float4*>(pq + t);
#pragma unroll
                    for (int k = 0; k < 4; ++k) wn[k] = vq[(t + k) * HD];
                };
                if (cnt4 > 0) load(0);
                for (int t = 0; t < cnt4; t += 4) {
                    const float4 pc = pn;
                    const float v0 = bf16_bits_to_f32(wn[0]), v1 = bf16_bits_to_f32(wn[1]);
                    const float v2 = bf16_bits_to_f32(wn[2]), v3 = bf16_bits_to_f32(wn[3]);
                    if (t + 4 < cnt4) load(t + 4);
                    a = fmaf(pc.x, v0, a);
                    a = fmaf(pc.y, v1, a);
                    a = fmaf(pc.z, v2, a);
                    a = fmaf(pc.w, v3, a);
                }
                for (int t = cnt4; t < cnt; ++t) a = fmaf(pq[t], bf16_bits_to_f32(vq[t * HD]), a);
                qs[tid] = a;
            }
        } else
        if (tid < kPairs) {
            // the loads of step t+4 are issued before the multiply-adds of step t (explicit double buffering:
            // with one or two warps per scheduler nothing else hides the shared-memory latency)
            const int cnt4 = cnt & ~3;
            float4 pr[NI];
            uint32_t w[NI][4];
            auto load = [&](int t) {
#pragma unroll
                for (int i = 0; i < NI; ++i) {
                    pr[i] = *reinterpret_cast<const float4*>(prp[i] + t);
#pragma unroll
                    for (int k = 0; k < 4; ++k) w[i][k] = *reinterpret_cast<const uint32_t*>(vp[i] + (t + k) * HD);
                }
            };
            if (cnt4 > 0) load(0);
            for (int t = 0; t < cnt4; t += 4) {
                float4 pc[NI];
                uint32_t wc[NI][4];
#pragma unroll
                for (int i = 0; i < NI; ++i) {
                    pc[i] = pr[i];
#pragma unroll
                    for (int k = 0; k < 4; ++k) wc[i][k] = w[i][k];
                }
                if (t + 4 < cnt4) load(t + 4);
#pragma unroll
                for (int i = 0; i < NI; ++i) {
                    acc0[i] = fmaf(pc[i].x, __uint_as_float(wc[i][0] << 16), acc0[i]);
                    acc1[i] = fmaf(pc[i].x, __uint_as_float(wc[i][0] & 0xffff0000u), acc1[i]);
                    acc0[i] = fmaf(pc[i].y, __uint_as_float(wc[i][1] << 16), acc0[i]);
                    acc1[i] = fmaf(pc[i].y, __uint_as_float(wc[i][1] & 0xffff0000u), acc1[i]);
                    acc0[i] = fmaf(pc[i].z, __uint_as_float(wc[i][2] << 16), acc0[i]);
                    acc1[i] = fmaf(pc[i].z, __uint_as_float(wc[i][2] & 0xffff0000u), acc1[i]);
                    acc0[i] = fmaf(pc[i].w, __uint_as_float(wc[i][3] << 16), acc0[i]);
                    acc1[i] = fmaf(pc[i].w, __uint_as_float(wc[i][3] & 0xffff0000u), acc1[i]);
                }
            }
            for (int t = cnt4; t < cnt; ++t) {
#pragma unroll
                for (int i = 0; i < NI; ++i) {
                    const uint32_t w0 = *reinterpret_cast<const uint32_t*>(vp[i] + t * HD);
                    acc0[i] = fmaf(prp[i][t], __uint_as_float(w0 << 16), acc0[i]);
                    acc1[i] = fmaf(prp[i][t], __uint_as_float(w0 & 0xffff0000u), acc1[i]);
                }
            }
        }
        __syncthreads();   // the chunk's (m, l) of every head are in tg->ml_s
        if constexpr (G * HD <= kT / 2) {
            if (tid < kPairs) { acc0[0] = qs[2 * tid]; acc1[0] = qs[2 * tid + 1]; }
        }
        ATR(5);
        const int nc = (it.seq_len + kAttnChunk - 1) / kAttnChunk;
        const uint32_t seq = tg->seq;
        constexpr int kRecWords = HD / 2 + 1;
#pragma unroll
        for (int i = 0; i < NI; ++i) {
            const int idx = tid + i * kT;
            if (idx < kPairs) {
                const int hh = idx / (HD / 2), dp = idx % (HD / 2);
                const int head = g * G + hh;
                uint4* rec = tg->rec_t + ((size_t)head * p.max_chunks) * kRecWords;
                if (c == 0) {
                    float M = tg->ml_s[hh], Lsum = tg->ml_s[G + hh], O0 = acc0[i], O1 = acc1[i];
                    // The other chunks' records, merged in chunk order.  All lanes of a warp serve the same head, so
                    // lane k prepares chunk cb + k: its header (m, l), the running maximum before and after it (a
                    // prefix maximum over the lanes) and the two rescaling factors; the ordered pass then takes them
                    // by shuffle.  Same operations on the same values as a thread doing all of it alone, but the
                    // exponentials of all chunks are evaluated side by side instead of one after the other.
                    for (int cb = 1; cb < nc; cb += 32) {
                        const int nb = min(32, nc - cb);
                        float mk = -CUDART_INF_F, lk = 0.0f;
                        if (lane < nb) {
                            const uint4* r = rec + (size_t)(cb + lane) * kRecWords;
                            uint4 w = ld_volatile16(r);
                            if (w.y != seq || w.w != seq) w = poll_tagged(r, seq, tg->q.ctx);
                            mk = __uint_as_float(w.x);
                            lk = __uint_as_float(w.z);
                        }
                        float ak, bk, Mn;
                        merge_factors(M, mk, lane, ak, bk, Mn);
                        for (int k0 = 0; k0 < nb; k0 += 4) {
                            uint4 w1[4];
#pragma unroll
                            for (int k = 0; k < 4; ++k)
                                if (k0 + k < nb) w1[k] = ld_volatile16(rec + (size_t)(cb + k0 + k) * kRecWords + 1 + dp);
#pragma unroll
                            for (int k = 0; k < 4; ++k)
                                if (k0 + k < nb) {
                                    const uint4* r = rec + (size_t)(cb + k0 + k) * kRecWords;
                                    if (w1[k].y != seq || w1[k].w != seq) w1[k] = poll_tagged(r + 1 + dp, seq, tg->q.ctx);
                                    const float a = __shfl_sync(0xffffffffu, ak, k0 + k), bb = __shfl_sync(0xffffffffu, bk, k0 + k);
                                    const float lc = __shfl_sync(0xffffffffu, lk, k0 + k);
                                    Lsum = fmaf(lc, bb, Lsum * a);
                                    O0 = fmaf(__uint_as_float(w1[k].x), bb, O0 * a);
                                    O1 = fmaf(__uint_as_float(w1[k].z), bb, O1 * a);
                                }
                        }
                        M = __shfl_sync(0xffffffffu, Mn, nb - 1);
                    }
                    st_volatile16(tg->att_t + ((size_t)head * HD) / 2 + dp, tag2(O0 / Lsum, O1 / Lsum, seq));
                } else {
                    uint4* r = rec + (size_t)c * kRecWords;
                    st_volatile16(r + 1 + dp, tag2(acc0[i], acc1[i], seq));
                    if (dp == 0) st_volatile16(r, tag2(tg->ml_s[hh], tg->ml_s[G + hh], seq));
                }
            }
        }
        ATR(6);
    } else if constexpr (COMPACT) {
        // throughput form: one thread per dim d keeps the G heads' accumulators; per position one vector
        // load of the G probabilities and one load of V[t][d] feed G multiply-adds
        if (tid < HD) {
            const int d = tid;
            float acc[G];
#pragma unroll
            for (int hh = 0; hh < G; ++hh) acc[hh] = 0.0f;
            const uint16_t* vp = Vs + d;
#pragma unroll 4
            for (int t = 0; t < cnt; ++t) {
                const float v = bf16_bits_to_f32(vp[t * HD]);
                float pr[G];
                if constexpr (G == 4) {
                    const float4 q4 = *reinterpret_cast<const float4*>(scf + t * 4);
                    pr[0] = q4.x; pr[1] = q4.y; pr[2] = q4.z; pr[3] = q4.w;
                } else if constexpr (G == 8) {
                    const float4 q4 = *reinterpret_cast<const float4*>(scf + t * 8);
                    const float4 q5 = *reinterpret_cast<const float4*>(scf + t * 8 + 4);
                    pr[0] = q4.x; pr[1] = q4.y; pr[2] = q4.z; pr[3] = q4.w;
                    pr[4] = q5.x; pr[5] = q5.y; pr[6] = q5.z; pr[7] = q5.w;
                } else if constexpr (G == 2) {
                    const float2 q2 = *reinterpret_cast<const float2*>(scf + t * 2);
                    pr[0] = q2.x; pr[1] = q2.y;
                } else {
#pragma unroll
                    for (int hh = 0; hh < G; ++hh) pr[hh] = scf[t * G + hh];
                }
#pragma unroll
                for (int hh = 0; hh < G; ++hh) acc[hh] = fmaf(pr[hh], v, acc[hh]);
            }
#pragma unroll
            for (int hh = 0; hh < G; ++hh) rec0[hh * rec_stride + 2 + d] = acc[hh];
        }
    } else {
        // latency form: one thread per (head, dim)
        for (int idx = tid; idx < G * HD; idx += kT) {
            const int hh = idx / HD, d = idx % HD;
            const float* pr = scf + hh * kAttnChunk;
            const uint16_t* vp = Vs + d;
            float acc = 0.0f;
#pragma unroll 8
            for (int t = 0; t < cnt; ++t) acc = fmaf(pr[t], bf16_bits_to_f32(vp[t * HD]), acc);
            rec0[hh * rec_stride + 2 + d] = acc;
        }
    }

    if constexpr (MODE != 2) attn_merge_last<HD, G>(p, it, is_last);
}

}  // namespace
}  // namespace terb
