// Shared device/host helpers for the B200 scan kernels (sm_100a).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "../../include/b200scan.h"

namespace b200 {

// Head of every workspace that carries cross-tile state. The entry points zero it (together
// with the flag words that follow) on the caller's stream before each launch.
struct WsHeader {
    unsigned int ticket;  // next dynamic tile id
    unsigned int error;   // B200_ERR_* set by a kernel whose bounded wait gave up
    unsigned int pad[2];
};

// Upper bound on polls of one look-back flag (each poll sleeps ~40 ns): about a second, after
// which the tile records B200_ERR_TIMEOUT in the header and carries on with a zero carry so
// the kernel always terminates.
constexpr int kSpinLimit = 1 << 21;

// ---------------------------------------------------------------- element algebra
template <typename E>
struct Ops;

template <>
struct Ops<float> {
    static __device__ __forceinline__ float zero() { return 0.f; }
    static __device__ __forceinline__ float one() { return 1.f; }
    static __device__ __forceinline__ float mul(float a, float b) { return a * b; }
    // a * x + b
    static __device__ __forceinline__ float fma(float a, float x, float b) { return fmaf(a, x, b); }
    static __device__ __forceinline__ float conj(float a) { return a; }
    static __device__ __forceinline__ float add(float a, float b) { return a + b; }
};

template <>
struct Ops<float2> {  // complex64 as (re, im)
    static __device__ __forceinline__ float2 zero() { return make_float2(0.f, 0.f); }
    static __device__ __forceinline__ float2 one() { return make_float2(1.f, 0.f); }
    static __device__ __forceinline__ float2 mul(float2 a, float2 b) {
        return make_float2(fmaf(a.x, b.x, -a.y * b.y), fmaf(a.x, b.y, a.y * b.x));
    }
    static __device__ __forceinline__ float2 fma(float2 a, float2 x, float2 b) {
        return make_float2(fmaf(a.x, x.x, fmaf(-a.y, x.y, b.x)), fmaf(a.x, x.y, fmaf(a.y, x.x, b.y)));
    }
    static __device__ __forceinline__ float2 conj(float2 a) { return make_float2(a.x, -a.y); }
    static __device__ __forceinline__ float2 add(float2 a, float2 b) { return make_float2(a.x + b.x, a.y + b.y); }
};

// V consecutive elements moved with one 4/8/16-byte access.
template <typename E, int V>
struct alignas(sizeof(E) * V) Pack {
    E e[V];
};

// Streaming (evict-first) loads/stores: every sequence element crosses HBM once.
template <typename P>
__device__ __forceinline__ P ld_stream(const P* p) {
    P r;
    if constexpr (sizeof(P) == 4) {
        float t = __ldcs(reinterpret_cast<const float*>(p));
        memcpy(&r, &t, 4);
    } else if constexpr (sizeof(P) == 8) {
        float2 t = __ldcs(reinterpret_cast<const float2*>(p));
        memcpy(&r, &t, 8);
    } else {
        static_assert(sizeof(P) == 16, "pack must be 4, 8 or 16 bytes");
        float4 t = __ldcs(reinterpret_cast<const float4*>(p));
        memcpy(&r, &t, 16);
    }
    return r;
}

template <typename P>
__device__ __forceinline__ void st_stream(P* p, const P& v) {

    if constexpr (sizeof(P) == 4) {
        float t;
        memcpy(&t, &v, 4);
        __stcs(reinterpret_cast<float*>(p), t);
    } else if constexpr (sizeof(P) == 8) {
        float2 t;
        memcpy(&t, &v, 8);
        __stcs(reinterpret_cast<float2*>(p), t);
    } else {
        static_assert(sizeof(P) == 16, "pack must be 4, 8 or 16 bytes");
        float4 t;
        memcpy(&t, &v, 16);
        __stcs(reinterpret_cast<float4*>(p), t);
    }
}

// L2-coherent (L1-bypassing) accesses for data exchanged between CTAs.
template <typename P>
__device__ __forceinline__ P ld_cg(const P* p) {
    P r;
    if constexpr (sizeof(P) == 4) {
        float t = __ldcg(reinterpret_cast<const float*>(p));
        memcpy(&r, &t, 4);
    } else if constexpr (sizeof(P) == 8) {
        float2 t = __ldcg(reinterpret_cast<const float2*>(p));
        memcpy(&r, &t, 8);
    } else {
        static_assert(sizeof(P) == 16, "pack must be 4, 8 or 16 bytes");
        float4 t = __ldcg(reinterpret_cast<const float4*>(p));
        memcpy(&r, &t, 16);
    }
    return r;
}

template <typename P>
__device__ __forceinline__ void st_cg(P* p, const P& v) {
    if constexpr (sizeof(P) == 4) {
        float t;
        memcpy(&t, &v, 4);
        __stcg(reinterpret_cast<float*>(p), t);
    } else if constexpr (sizeof(P) == 8) {
        float2 t;
        memcpy(&t, &v, 8);
        __stcg(reinterpret_cast<float2*>(p), t);
    } else {
        static_assert(sizeof(P) == 16, "pack must be 4, 8 or 16 bytes");
        float4 t;
        memcpy(&t, &v, 16);
        __stcg(reinterpret_cast<float4*>(p), t);
    }
}

__device__ __forceinline__ unsigned int ld_acquire(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void st_release(unsigned int* p, unsigned int v) {
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Poll a look-back flag until it is non-zero or `limit` polls have passed (returns 0 then).
__device__ __forceinline__ unsigned int wait_flag(const unsigned int* p, int limit) {
    unsigned int f = ld_acquire(p);
    int spins = 0;
    while (f == 0u && spins < limit) {
        __nanosleep(40);
        f = ld_acquire(p);
        ++spins;
    }
    return f;
}

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

}  // namespace b200
