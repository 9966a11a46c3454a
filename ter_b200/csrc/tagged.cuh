// Flag-in-data words: two floats travel with a sequence number in one 16-byte word {v0, seq, v1, seq}.
// A consumer polls the word itself until both 8-byte halves carry the number it expects, so a value
// needs no fence, no separate flag and no barrier to be handed from one CTA (or one GPU) to another:
// one store, one load.  Sequence numbers only grow; a buffer is rewritten only after everything that
// reads the previous generation has finished (the dataflow of a decode step guarantees it).
// Every poll is bounded: a wait that runs out publishes an abort mark for the step, records a status
// code, and all later polls of the CTA return at once.
#pragma once
#include "common.cuh"

namespace terb {

__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ uint4 ld_volatile16(const uint4* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_volatile16(uint4* p, const uint4& v) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ unsigned ld_volatile32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint4 tag2(float a, float b, uint32_t seq) {
    return make_uint4(__float_as_uint(a), seq, __float_as_uint(b), seq);
}

struct PollCtx {
    unsigned long long limit_ns;   // limit of one wait
    int* abort_s;                  // shared-memory flag of this CTA: a wait ran out, stop waiting
    unsigned* abort_g;             // global word: equals abort_val once some CTA of this step gave up
    unsigned abort_val;
    int* status;                   // device status word (DEV_TIMEOUT_FLAG)
    unsigned sleep_ns;             // pause between two looks at a word that is not there yet (0: none): thousands
                                   // of threads re-reading the same lines delay the very stores they wait for
};

// Returns the word once both halves carry `seq`; after an abort, whatever was read last.
__device__ __forceinline__ uint4 poll_tagged(const uint4* src, uint32_t seq, const PollCtx& c) {
    uint4 got = ld_volatile16(src);
    if (got.y == seq && got.w == seq) return got;
    if (*reinterpret_cast<volatile int*>(c.abort_s)) return got;
    const unsigned long long t0 = globaltimer_ns();
    for (unsigned spins = 1;; ++spins) {
        if (c.sleep_ns) __nanosleep(c.sleep_ns);
        got = ld_volatile16(src);
        if (got.y == seq && got.w == seq) return got;
        if ((spins & 63u) == 0) {
            if (*reinterpret_cast<volatile int*>(c.abort_s)) return got;
            if (ld_volatile32(c.abort_g) == c.abort_val) {
                *reinterpret_cast<volatile int*>(c.abort_s) = 1;
                return got;
            }
            if (globaltimer_ns() - t0 > c.limit_ns) {
                atomicExch(c.abort_g, c.abort_val);
                if (c.status) atomicExch(c.status, DEV_TIMEOUT_FLAG);
                *reinterpret_cast<volatile int*>(c.abort_s) = 1;
                return got;
            }
        }
    }
}

// A float vector in flag-in-data form and the generation a reader expects.
struct TaggedSrc {
    const uint4* words;    // element i is half (i & 1) of word i / 2
    uint32_t seq;
    PollCtx ctx;
};
__device__ __forceinline__ float tagged_ld(const TaggedSrc& s, int i) {
    const uint4 w = poll_tagged(s.words + (i >> 1), s.seq, s.ctx);
    return __uint_as_float((i & 1) ? w.z : w.x);
}
// elements 4*idx4 .. 4*idx4+3
__device__ __forceinline__ float4 tagged_ld4(const TaggedSrc& s, int idx4) {
    const uint4 a = poll_tagged(s.words + 2 * idx4, s.seq, s.ctx);
    const uint4 b = poll_tagged(s.words + 2 * idx4 + 1, s.seq, s.ctx);
    return make_float4(__uint_as_float(a.x), __uint_as_float(a.z), __uint_as_float(b.x), __uint_as_float(b.z));
}

}  // namespace terb
