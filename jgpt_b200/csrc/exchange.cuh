// Hand-over of small results between the CTAs of one cooperative launch without a grid barrier: (value, stamp)
// pairs written with one 8-byte store, polled by the readers until they carry the stamp they wait for.
// Aligned 8-byte accesses are single-copy atomic, so a pair is never seen half written; stamps grow from launch to
// launch, so nothing is ever reset.  Every wait is bounded and reports through the context's status word.
#pragma once

#include "common.cuh"

namespace jgpt {

constexpr unsigned kPollLimit = 1u << 21;  // re-reads before a waiting thread gives up (~1 s)

__device__ __forceinline__ unsigned ld_relaxed_u32(const unsigned *p) {
    unsigned v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// Two (value, stamp) pairs.  Each 8-byte half is written with one store, so a half is never seen torn.
__device__ __forceinline__ uint4 ld_pairs(const uint2 *p) {
    uint4 v;
    // L2 is the point of coherence and .cg reads go there; unlike volatile / relaxed reads they are coalesced (a warp's
    // 512 contiguous bytes are 4 requests, not 32: a 48 KB slab took 3.3 us with the strong forms)
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_pair(uint2 *p, float v, unsigned stamp) {
    asm volatile("st.relaxed.gpu.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(stamp) : "memory");
}

struct Poll {
    unsigned *abort_word;
    unsigned tag;  // this launch's value of the abort word
    int *status;
    int failed;
};

// v[i] = the two pairs at addr(i), i < cnt, re-read until both carry `stamp`.  On a timeout or an abort the values
// come back as zeros and pl.failed is set (the CTA leaves at its next block barrier).
template <int N, class AddrFn>
__device__ __forceinline__ void ll_load(uint4 (&v)[N], int cnt, unsigned stamp, Poll &pl, AddrFn addr) {
#pragma unroll
    for (int i = 0; i < N; i++) v[i] = i < cnt ? ld_pairs(addr(i)) : make_uint4(0u, stamp, 0u, stamp);
    unsigned polls = 0;
    for (;;) {
        bool ok = true;
#pragma unroll
        for (int i = 0; i < N; i++) ok = ok && v[i].y == stamp && v[i].w == stamp;
        if (ok) return;
        if ((++polls & 255u) == 0u) {
            if (ld_relaxed_u32(pl.abort_word) == pl.tag) break;
            if (polls > kPollLimit) {
                atomicOr(pl.status, DEV_STATUS_WAIT_TIMEOUT);
                atomicExch(pl.abort_word, pl.tag);
                break;
            }
        }
#pragma unroll
        for (int i = 0; i < N; i++)
            if (i < cnt && !(v[i].y == stamp && v[i].w == stamp)) v[i] = ld_pairs(addr(i));
    }
    pl.failed = 1;
#pragma unroll
    for (int i = 0; i < N; i++) v[i] = make_uint4(0u, stamp, 0u, stamp);
}

}  // namespace jgpt
