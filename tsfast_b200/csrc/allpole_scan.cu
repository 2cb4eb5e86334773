// All-pole IIR scan y_t = w_t - sum_{i=1..na} a_i y_{t-i} per lane (dynoNet G-block denominator),
// forward and reverse-time adjoint, float32, 1 <= na <= 16.
//
// Data layout: w, y, g [lanes, L] with TIME contiguous per lane; a, y0 [lanes, na]; the carried
// state is s[j] = y_{t-1-j} (newest first), which is also the layout of y0.
//
// One warp owns one lane and walks its sequence in tiles of 32*SEG steps, SEG = 32 consecutive
// steps per thread.  The recurrence is linear in (state, input), so a SEG-step segment maps its
// start state to its end state as s' = M s + r with M = (companion matrix)^SEG the same for every
// segment and r the segment's zero-state response.  Per tile:
//   1. each thread runs its SEG steps from a zero state (registers) to get r,
//   2. a warp-shuffle Kogge-Stone scan over the 32 segments composes the affine maps; step d
//      uses M^(2^d), and the carry from the previous tile enters through thread 0,
//   3. each thread re-runs its SEG steps from its true start state and the tile is stored.
// (Longer segments spread the cost of step 2 over more elements: SEG = 32 took the forward from
// 4.4 to 6.2 TB/s on B200.)
// The five powers M^(1,2,4,8,16) (in units of one segment) are built once per lane at kernel start by repeated squaring and
// kept in shared memory.  Powers and the composition of segment states are float64: with poles
// near the unit circle M has large entries that cancel, and a float32 composition loses ten times
// the accuracy of the sequential float32 loop, while float64 matches it (steps 1 and 3, i.e. all
// per-element work, stay float32).  Entries are clamped to +-1e300 so that 0 * overflow stays 0
// instead of becoming NaN; an unstable filter still runs to inf like the sequential loop.
//
// Memory pipeline: every warp keeps S-1 tiles in flight in a private shared-memory ring filled by
// coalesced 16-byte cp.async (4-byte when L or a pointer is not 16-byte aligned); chunks are
// padded by 16 bytes so that the per-thread 16-byte reads are bank-conflict free.  Results go
// back through the same buffer and leave as coalesced 16-byte stores.  No workspace, no atomics:
// the adjoint's grad_a is accumulated per thread in registers across all tiles and reduced with
// a fixed butterfly at the end, so results are bitwise reproducible.
#include <float.h>

#include <type_traits>

#include "common.cuh"

namespace b200 {

struct AllpoleArgs {
    const float* a;    // [lanes, na]
    const float* in;   // fwd: w        bwd: g
    const float* yin;  // bwd: forward output y
    const float* y0;   // may be null
    float* out;        // fwd: y        bwd: gw
    float* ga;         // bwd: [lanes, na]
    float* gy0;        // bwd: [lanes, na] or null
    long long lanes, L;
    // bwd, G-block use: when gP > 0 (pairs per batch row, gO outputs), lane (b, pair = j*gO + i) reads its
    // upstream gradient from row b*gO + i of `in` and its coefficients from row i*(gP/gO) + j of `a`
    long long gP, gO;
};

// Steps per thread (SEG, a template parameter: 16 or 32), hence 32*SEG steps per warp tile; a
// thread's chunk is padded by 4 floats in shared memory so that 16-byte reads are conflict free.

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
    const unsigned int d = static_cast<unsigned int>(__cvta_generic_to_shared(smem_dst));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async4(void* smem_dst, const void* gsrc) {
    const unsigned int d = static_cast<unsigned int>(__cvta_generic_to_shared(smem_dst));
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ double clamp_finite(double x) {
    if (x > 1e300) return 1e300;
    if (x < -1e300) return -1e300;
    return x;  // NaN passes through
}

// One recurrence step on the shift-register state: returns y = in - a.s and shifts y in.
template <int NA>
__device__ __forceinline__ float iir_step(const float (&a)[NA], float (&s)[NA], float in) {
    float acc = 0.f;
#pragma unroll
    for (int j = NA - 1; j >= 1; --j) acc = fmaf(a[j], s[j], acc);  // older taps first:
    const float y = in - fmaf(a[0], s[0], acc);                   // only a_1 y_{t-1} is on the critical path
#pragma unroll
    for (int j = NA - 1; j >= 1; --j) s[j] = s[j - 1];
    s[0] = y;
    return y;
}

template <int NA, bool BWD, int VEC, int W, int S, int MINB, int SEG>
__global__ void __launch_bounds__(32 * W, MINB) allpole_kernel(const AllpoleArgs p) {
    static_assert(VEC == 4 || VEC == 1, "pieces are 16 or 4 bytes");
    static_assert(SEG >= NA && SEG % 4 == 0, "a segment must hold the whole state");
    constexpr int kSeg = SEG, kTile = 32 * SEG, kChunk = SEG + 4, kStageF = 32 * kChunk;
    constexpr int NTENS = BWD ? 2 : 1;
    constexpr int PIECES = kTile / VEC;  // copy pieces per tile and tensor
    constexpr int PPC = kSeg / VEC;      // pieces per thread chunk

    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int w = threadIdx.x >> 5;
    const int lid = threadIdx.x & 31;
    const long long lane = (long long)blockIdx.x * W + w;
    if (lane >= p.lanes) return;  // warps never synchronise with each other

    // 7 matrices of doubles per warp, rounded up to an even count so that the float ring behind
    // them stays 16-byte aligned for every order and warp count
    constexpr int MDW = (7 * NA * NA + 1) & ~1;
    double* Md = reinterpret_cast<double*>(smem_raw) + w * MDW;  // squaring scratch (2 matrices)
    double* Mp = Md + 2 * NA * NA;                                // M^(2^d), d = 0..4
    float* ring = reinterpret_cast<float*>(reinterpret_cast<double*>(smem_raw) + W * MDW) +
                  w * (S * NTENS * kStageF);  // [S][NTENS][32][kChunk]

    const long long L = p.L;
    const long long C = (L + kTile - 1) / kTile;
    const long long in_row = (BWD && p.gP > 0) ? (lane / p.gP) * p.gO + (lane % p.gP) % p.gO : lane;
    const float* in = p.in + in_row * L;
    const float* yin = BWD ? p.yin + lane * L : nullptr;
    float* out = p.out + lane * L;

    // with the G-block row map the coefficients are the block's [O, I, na] tensor: pair j*O + i -> (i, j)
    const long long a_row = (BWD && p.gP > 0) ? ((lane % p.gP) % p.gO) * (p.gP / p.gO) + (lane % p.gP) / p.gO : lane;
    float a[NA];
#pragma unroll
    for (int j = 0; j < NA; ++j) a[j] = p.a[a_row * NA + j];

    auto phys0_of = [&](long long c) -> long long { return BWD ? (L - (c + 1) * kTile) : c * kTile; };
    auto issue = [&](long long c, int slot) {
        const long long ph = phys0_of(c);
        float* dst = ring + slot * (NTENS * kStageF);
#pragma unroll
        for (int q = 0; q < PIECES / 32; ++q) {
            const int gidx = q * 32 + lid;
            const long long t = ph + (long long)gidx * VEC;
            if (t >= 0 && t < L) {
                float* d = dst + (gidx / PPC) * kChunk + (gidx % PPC) * VEC;
                if constexpr (VEC == 4) {
                    cp_async16(d, in + t);
                    if constexpr (BWD) cp_async16(d + kStageF, yin + t);
                } else {
                    cp_async4(d, in + t);
                    if constexpr (BWD) cp_async4(d + kStageF, yin + t);
                }
            }
        }
    };

#pragma unroll
    for (int q = 0; q < S - 1; ++q) {
        if (q < C) issue(q, q);
        cp_commit();
    }

    // ---------------------------------------------------------------- M = companion^16 and its powers
    if (lid < NA) {
        double s[NA];
#pragma unroll
        for (int j = 0; j < NA; ++j) s[j] = (j == lid) ? 1.0 : 0.0;
        for (int t = 0; t < kSeg; ++t) {
            double acc = 0.0;
#pragma unroll
            for (int j = 0; j < NA; ++j) acc += (double)a[j] * s[j];
#pragma unroll
            for (int j = NA - 1; j >= 1; --j) s[j] = s[j - 1];
            s[0] = -acc;
        }
#pragma unroll
        for (int i = 0; i < NA; ++i) Md[i * NA + lid] = s[i];  // column `lid`
    }
    __syncwarp();
    {
        int cur = 0;
        for (int d = 0; d < 5; ++d) {
            const double* src = Md + cur * NA * NA;
            double* dst = Md + (cur ^ 1) * NA * NA;
            for (int e = lid; e < NA * NA; e += 32) {
                Mp[d * NA * NA + e] = clamp_finite(src[e]);
                if (d < 4) {
                    const int i = e / NA, j = e % NA;
                    double acc = 0.0;
                    for (int k = 0; k < NA; ++k) acc += src[i * NA + k] * src[k * NA + j];
                    dst[e] = acc;
                }
            }
            __syncwarp();
            cur ^= 1;
        }
    }

    double cin[NA];  // state carried into the current tile
    float acc_a[NA];
#pragma unroll
    for (int j = 0; j < NA; ++j) {
        cin[j] = (!BWD && p.y0 != nullptr) ? (double)p.y0[lane * NA + j] : 0.0;
        acc_a[j] = 0.f;
    }
    const int ch = BWD ? 31 - lid : lid;  // this thread's chunk, in physical order

    for (long long c = 0; c < C; ++c) {
        const int slot = (int)(c % S);
        const long long ph = phys0_of(c);
        float* stage = ring + slot * (NTENS * kStageF);
        cp_wait<S - 2>();
        __syncwarp();

        float v[kSeg], yv[BWD ? kSeg : 1];
        const long long tbase = ph + ch * kSeg;
#pragma unroll
        for (int q = 0; q < kSeg / 4; ++q) {
            const float4 t4 = *reinterpret_cast<const float4*>(stage + ch * kChunk + 4 * q);
            v[4 * q] = t4.x, v[4 * q + 1] = t4.y, v[4 * q + 2] = t4.z, v[4 * q + 3] = t4.w;
            if constexpr (BWD) {
                const float4 u4 = *reinterpret_cast<const float4*>(stage + kStageF + ch * kChunk + 4 * q);
                yv[4 * q] = u4.x, yv[4 * q + 1] = u4.y, yv[4 * q + 2] = u4.z, yv[4 * q + 3] = u4.w;
            }
        }
        const bool edge = ph < 0 || ph + kTile > L;
        if (edge) {  // edge tile only: steps outside the sequence get zero input
#pragma unroll
            for (int r = 0; r < kSeg; ++r) {
                const bool okr = (tbase + r) >= 0 && (tbase + r) < L;
                if (!okr) {
                    v[r] = 0.f;
                    if constexpr (BWD) yv[r] = 0.f;
                }
            }
        }
        __syncwarp();  // everyone has read this stage before the next tile's copies may land in it
        if (c + S - 1 < C) issue(c + S - 1, (int)((c + S - 1) % S));
        cp_commit();

        // 1. zero-state response of this thread's segment
        float s[NA];
#pragma unroll
        for (int j = 0; j < NA; ++j) s[j] = 0.f;
#pragma unroll
        for (int k = 0; k < kSeg; ++k) iir_step<NA>(a, s, v[BWD ? kSeg - 1 - k : k]);

        // 2. carry of the previous tile enters at thread 0; Kogge-Stone over the 32 segments (float64)
        double sd[NA];
#pragma unroll
        for (int j = 0; j < NA; ++j) sd[j] = (double)s[j];
        if (lid == 0) {
#pragma unroll
            for (int i = 0; i < NA; ++i) {
                double t = sd[i];
#pragma unroll
                for (int j = 0; j < NA; ++j) t = fma(Mp[i * NA + j], cin[j], t);
                sd[i] = t;
            }
        }
#pragma unroll
        for (int d = 0; d < 5; ++d) {
            double sp[NA];
#pragma unroll
            for (int j = 0; j < NA; ++j) sp[j] = __shfl_up_sync(0xffffffffu, sd[j], 1 << d);
            if (lid >= (1 << d)) {
                const double* M = Mp + d * NA * NA;
#pragma unroll
                for (int i = 0; i < NA; ++i) {
                    double t = sd[i];
#pragma unroll
                    for (int j = 0; j < NA; ++j) t = fma(M[i * NA + j], sp[j], t);
                    sd[i] = t;
                }
            }
        }
        float st[NA];
#pragma unroll
        for (int j = 0; j < NA; ++j) {
            const double up = __shfl_up_sync(0xffffffffu, sd[j], 1);
            st[j] = (float)(lid == 0 ? cin[j] : up);
        }
#pragma unroll
        for (int j = 0; j < NA; ++j) cin[j] = __shfl_sync(0xffffffffu, sd[j], 31);

        // 3. the true run of this segment (interior tiles take the copy without range checks)
        auto true_run = [&](auto edge_tag) {
            constexpr bool EDGE = decltype(edge_tag)::value;
#pragma unroll
            for (int k = 0; k < kSeg; ++k) {
                const int r = BWD ? kSeg - 1 - k : k;
                if constexpr (BWD) {  // grad_a_k += G_{t+1+k} * y_t with the state BEFORE the step
                    // (steps past the sequence are skipped: an unstable filter may have run its
                    // state to inf there, and inf * 0 must not reach the sum)
                    if (!EDGE || ((tbase + r) >= 0 && (tbase + r) < L)) {
#pragma unroll
                        for (int j = 0; j < NA; ++j) acc_a[j] = fmaf(st[j], yv[r], acc_a[j]);
                    }
                }
                v[r] = iir_step<NA>(a, st, v[r]);
            }
        };
        if (edge) {
            true_run(std::true_type{});
        } else {
            true_run(std::false_type{});
        }

        // stage the results in this thread's chunk and store the tile coalesced
#pragma unroll
        for (int q = 0; q < kSeg / 4; ++q)
            *reinterpret_cast<float4*>(stage + ch * kChunk + 4 * q) =
                make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
        __syncwarp();
#pragma unroll
        for (int q = 0; q < PIECES / 32; ++q) {
            const int gidx = q * 32 + lid;
            const long long t = ph + (long long)gidx * VEC;
            if (t >= 0 && t < L) {
                const float* sp = stage + (gidx / PPC) * kChunk + (gidx % PPC) * VEC;
                if constexpr (VEC == 4) {
                    __stcs(reinterpret_cast<float4*>(out + t), *reinterpret_cast<const float4*>(sp));
                } else {
                    __stcs(out + t, *sp);
                }
            }
        }
        __syncwarp();
    }
    cp_wait<0>();

    if constexpr (BWD) {
        // grad_a: fixed butterfly over the warp, then the initial-state terms from G_0..G_{na-1}
#pragma unroll
        for (int j = 0; j < NA; ++j) {
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) acc_a[j] += __shfl_xor_sync(0xffffffffu, acc_a[j], off);
        }
        __syncwarp();
        if (lid == 0) {
            float G[NA];
#pragma unroll
            for (int q = 0; q < NA; ++q) G[q] = q < L ? __ldcg(out + q) : 0.f;
#pragma unroll
            for (int i = 1; i <= NA; ++i) {
                float t = acc_a[i - 1];
                if (p.y0 != nullptr) {
#pragma unroll
                    for (int k = 1; k <= NA; ++k)
                        if (k <= i) t = fmaf(G[i - k], p.y0[lane * NA + k - 1], t);
                }
                p.ga[lane * NA + i - 1] = -t;
            }
            if (p.gy0 != nullptr) {
#pragma unroll
                for (int j = 0; j < NA; ++j) {
                    float t = 0.f;
#pragma unroll
                    for (int i = 1; i <= NA; ++i)
                        if (i >= j + 1) t = fmaf(a[i - 1], G[i - 1 - j], t);
                    p.gy0[lane * NA + j] = -t;
                }
            }
        }
    }
}

// ------------------------------------------------------------------------------- host side
#ifndef ALLPOLE_FWD_W
#define ALLPOLE_FWD_W 2  // lanes (warps) per CTA for orders up to 8, half of it above
#endif
#ifndef ALLPOLE_BWD_W
#define ALLPOLE_BWD_W 2
#endif
#ifndef ALLPOLE_FWD_S
#define ALLPOLE_FWD_S 2  // ring stages per warp
#endif
#ifndef ALLPOLE_BWD_S
#define ALLPOLE_BWD_S 3
#endif
#ifndef ALLPOLE_FWD_MINB
#define ALLPOLE_FWD_MINB 8  // CTAs per SM asked of the compiler (orders up to 8)
#endif
#ifndef ALLPOLE_BWD_MINB
#define ALLPOLE_BWD_MINB 6
#endif
#ifndef ALLPOLE_FWD_SEG
#define ALLPOLE_FWD_SEG 32  // steps per thread, forward
#endif
#ifndef ALLPOLE_BWD_SEG
#define ALLPOLE_BWD_SEG 32  // steps per thread, adjoint
#endif

template <int NA, bool BWD, int VEC>
static int launch_allpole(const AllpoleArgs& a, cudaStream_t st) {
    constexpr int W0 = BWD ? ALLPOLE_BWD_W : ALLPOLE_FWD_W;
    constexpr int W = (NA <= 8 || W0 == 1) ? W0 : W0 / 2;  // high orders: the matrix powers take the shared memory
    constexpr int S = BWD ? ALLPOLE_BWD_S : ALLPOLE_FWD_S;
    constexpr int NTENS = BWD ? 2 : 1;
    constexpr int SEG = BWD ? ALLPOLE_BWD_SEG : ALLPOLE_FWD_SEG;
    constexpr size_t smem =
        (size_t)W * (((7 * NA * NA + 1) & ~1) * sizeof(double) + (size_t)S * NTENS * 32 * (SEG + 4) * sizeof(float));
    constexpr int MINB = NA <= 8 ? (BWD ? ALLPOLE_BWD_MINB : ALLPOLE_FWD_MINB) : 1;
    auto kern = allpole_kernel<NA, BWD, VEC, W, S, MINB, SEG>;
    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return B200_ERR_LAUNCH;
        configured[dev] = true;
    }
    const long long grid = (a.lanes + W - 1) / W;
    if (grid > 0x7fffffffLL) return B200_ERR_UNSUPPORTED;
    kern<<<(unsigned int)grid, 32 * W, smem, st>>>(a);
    return cudaGetLastError() == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

template <bool BWD, int VEC>
static int dispatch_na(int na, const AllpoleArgs& a, cudaStream_t st) {
    switch (na) {
#define B200_NA_CASE(n) \
    case n:             \
        return launch_allpole<n, BWD, VEC>(a, st);
        B200_NA_CASE(1) B200_NA_CASE(2) B200_NA_CASE(3) B200_NA_CASE(4) B200_NA_CASE(5) B200_NA_CASE(6)
        B200_NA_CASE(7) B200_NA_CASE(8) B200_NA_CASE(9) B200_NA_CASE(10) B200_NA_CASE(11) B200_NA_CASE(12)
        B200_NA_CASE(13) B200_NA_CASE(14) B200_NA_CASE(15) B200_NA_CASE(16)
#undef B200_NA_CASE
        default:
            return B200_ERR_UNSUPPORTED;
    }
}

static int run_allpole(bool bwd, long long lanes, long long L, long long na, const void* a, const void* in,
                       const void* yin, const void* y0, void* out, void* ga, void* gy0, void* stream,
                       long long gP = 0, long long gO = 0) {
    if (lanes < 0 || L < 0 || na < 1) return B200_ERR_ARG;
    if (na > 16) return B200_ERR_UNSUPPORTED;
    if (lanes == 0) return B200_OK;
    if (!a || (bwd && !ga)) return B200_ERR_ARG;
    if (L > 0 && (!in || !out || (bwd && !yin))) return B200_ERR_ARG;
    if (bwd && y0 && !gy0) return B200_ERR_ARG;
    const uintptr_t por = (uintptr_t)a | (uintptr_t)in | (uintptr_t)yin | (uintptr_t)y0 | (uintptr_t)out |
                          (uintptr_t)ga | (uintptr_t)gy0;
    if (por % 4 != 0) return B200_ERR_ARG;
    AllpoleArgs p;
    p.a = static_cast<const float*>(a);
    p.in = static_cast<const float*>(in);
    p.yin = static_cast<const float*>(yin);
    p.y0 = static_cast<const float*>(y0);
    p.out = static_cast<float*>(out);
    p.ga = static_cast<float*>(ga);
    p.gy0 = y0 ? static_cast<float*>(gy0) : nullptr;
    p.lanes = lanes;
    p.L = L;
    p.gP = gP, p.gO = gO;
    const uintptr_t seq_or = (uintptr_t)in | (uintptr_t)yin | (uintptr_t)out;
    const bool vec = (L % 4 == 0) && (seq_or % 16 == 0);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (bwd) return vec ? dispatch_na<true, 4>((int)na, p, st) : dispatch_na<true, 1>((int)na, p, st);
    return vec ? dispatch_na<false, 4>((int)na, p, st) : dispatch_na<false, 1>((int)na, p, st);
}


// =============================================================================== fused G-block
// dynoNet's linear block for one (batch row, output channel): for every input channel j the FIR
// numerator w = b_ij * u_j (causal, NB taps, the carried input tail in front of the row), the
// all-pole denominator 1/A_ij on w, and the sum of the filtered signals over j.  Neither w nor
// (unless asked for) the per-pair outputs touch HBM: one warp owns (b, i), walks time in tiles of
// 1024 steps and, inside a tile, the input channels one after the other, adding each pair's
// output into 32 registers per thread.  The all-pole part is the scheme of allpole_kernel above
// (segment maps composed by a warp-shuffle Kogge-Stone scan in float64) with the matrix powers
// and the carried state of every pair kept in shared memory.
struct GBlockArgs {
    const float* ub;   // [B*I, pitch]: row (b, j) = carried tail (NB-1 samples) followed by u[b, :, j]
    const float* taps; // [O, I, NB] numerator taps b_0 .. b_{NB-1} (zero padded)
    const float* a;    // [O, I, na]
    const float* x0;   // [B, I*O, na] or null; pair index j*O + i
    float* y;          // [B, O, L]
    float* yp;         // [B, I*O, L] or null: the per-pair outputs (what the adjoint needs)
    float* xlast;      // [B, I*O, na]: last na outputs of every pair, newest first
    long long B, I, O, L, pitch;
    int split;         // one warp per pair instead of per (b, output): y is not written, yp must be
};

#ifndef GBLOCK_BW_W
#define GBLOCK_BW_W 1  // (batch row, input channel) warps per CTA of the numerator adjoint
#endif
#ifndef GBLOCK_BW_S
#define GBLOCK_BW_S 3
#endif
#ifndef GBLOCK_MINB
#define GBLOCK_MINB 4  // CTAs per SM asked of the compiler, forward
#endif
#ifndef GBLOCK_BW_MINB
#define GBLOCK_BW_MINB 4  // same, numerator adjoint
#endif

template <int NA, int NB, int VEC, int W, int S, int SEG>
__global__ void __launch_bounds__(32 * W, GBLOCK_MINB) gblock_fwd_kernel(const GBlockArgs p) {
    constexpr int kSeg = SEG, kTile = 32 * kSeg, kChunk = kSeg + 4;
    constexpr int kStageF = 33 * kChunk;  // 32 thread chunks + one for the NB-1 samples past the tile
    constexpr int PIECES = kTile / VEC, PPC = kSeg / VEC;
    constexpr int HALO = (NB - 1 + VEC - 1) / VEC;  // copy pieces past the tile
    constexpr int NU = kSeg + NB - 1;               // samples a thread's segment reads
    static_assert(NB >= 1 && NB - 1 <= kSeg, "the halo must fit one chunk");

    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int w = threadIdx.x >> 5, lid = threadIdx.x & 31;
    const long long widx = (long long)blockIdx.x * W + w;
    // normally a warp owns (b, i) and walks all inputs; in split mode (few outputs: not enough
    // (b, i) to fill the GPU) a warp owns one pair (b, j0, i) and only the per-pair outputs are written
    const long long OV = p.split ? p.I * p.O : p.O;
    if (widx >= p.B * OV) return;  // warps never synchronise with each other
    const long long b = widx / OV, iv = widx - b * OV;
    const long long i = p.split ? iv % p.O : iv;
    const int j0 = p.split ? (int)(iv / p.O) : 0;
    const int I = (int)p.I;          // inputs of the block (row and coefficient strides)
    const int nj = p.split ? 1 : I;  // inputs this warp walks
    const long long L = p.L, P = p.I * p.O;

    // per warp: doubles [2 NA^2 scratch | I x 5 NA^2 powers | I x NA carried states], then floats
    // [S ring stages | one stage for the summed output | I x NA previous-tile tails]
    const int dper = ((2 * NA * NA + I * (5 * NA * NA + NA)) + 1) & ~1;
    const int fper = S * kStageF + 32 * kChunk + ((I * NA + 3) & ~3);
    double* Md = reinterpret_cast<double*>(smem_raw) + (size_t)w * dper;
    double* Mp = Md + 2 * NA * NA;          // [I][5][NA*NA]
    double* cins = Mp + I * 5 * NA * NA;    // [I][NA]
    float* fbase = reinterpret_cast<float*>(reinterpret_cast<double*>(smem_raw) + (size_t)W * dper) + (size_t)w * fper;
    float* ring = fbase;                    // [S][33][kChunk]
    float* ysum = ring + S * kStageF;       // [32][kChunk]
    float* ptail = ysum + 32 * kChunk;      // [I][NA]

    const long long C = (L + kTile - 1) / kTile;
    const long long items = C * nj;  // item q = (tile q / nj, input channel j0 + q % nj)

    auto issue = [&](long long q, int slot) {
        const long long c = q / nj, j = j0 + (q - c * nj);
        const float* src = p.ub + (b * I + j) * p.pitch + c * kTile;
        const long long room = p.pitch - c * kTile;  // samples of the row from the tile start on
        float* dst = ring + slot * kStageF;
#pragma unroll
        for (int r = 0; r < PIECES / 32; ++r) {
            const int gidx = r * 32 + lid;
            if ((long long)gidx * VEC < room) {
                float* d = dst + (gidx / PPC) * kChunk + (gidx % PPC) * VEC;
                if constexpr (VEC == 4) cp_async16(d, src + gidx * VEC);
                else cp_async4(d, src + gidx * VEC);
            }
        }
        if (lid < HALO && (long long)(kTile + lid * VEC) < room) {
            float* d = dst + 32 * kChunk + lid * VEC;
            if constexpr (VEC == 4) cp_async16(d, src + kTile + lid * VEC);
            else cp_async4(d, src + kTile + lid * VEC);
        }
    };
#pragma unroll
    for (int q = 0; q < S - 1; ++q) {
        if (q < items) issue(q, q);
        cp_commit();
    }

    // ---------------------------------------------------------------- per pair: M^(2^d), start state
    for (int j = j0; j < j0 + nj; ++j) {
        const int jl = j - j0;  // index into this warp's shared-memory tables
        float aj[NA];
#pragma unroll
        for (int k = 0; k < NA; ++k) aj[k] = p.a[(i * p.I + j) * NA + k];
        if (lid < NA) {
            double s[NA];
#pragma unroll
            for (int k = 0; k < NA; ++k) s[k] = (k == lid) ? 1.0 : 0.0;
            for (int t = 0; t < kSeg; ++t) {
                double acc = 0.0;
#pragma unroll
                for (int k = 0; k < NA; ++k) acc += (double)aj[k] * s[k];
#pragma unroll
                for (int k = NA - 1; k >= 1; --k) s[k] = s[k - 1];
                s[0] = -acc;
            }
#pragma unroll
            for (int r = 0; r < NA; ++r) Md[r * NA + lid] = s[r];
            const long long pr = b * P + j * p.O + i;
            cins[jl * NA + lid] = p.x0 != nullptr ? (double)p.x0[pr * NA + lid] : 0.0;
            ptail[jl * NA + lid] = 0.f;
        }
        __syncwarp();
        int cur = 0;
        for (int d = 0; d < 5; ++d) {
            const double* src = Md + cur * NA * NA;
            double* dst = Md + (cur ^ 1) * NA * NA;
            for (int e = lid; e < NA * NA; e += 32) {
                Mp[(jl * 5 + d) * NA * NA + e] = clamp_finite(src[e]);
                if (d < 4) {
                    const int r = e / NA, cc = e % NA;
                    double acc = 0.0;
                    for (int k = 0; k < NA; ++k) acc += src[r * NA + k] * src[k * NA + cc];
                    dst[e] = acc;
                }
            }
            __syncwarp();
            cur ^= 1;
        }
    }

    float yacc[kSeg];
    long long q = 0;
    for (long long c = 0; c < C; ++c) {
        const long long t0 = c * kTile;
        const long long tbase = t0 + lid * kSeg;
        const bool edge = t0 + kTile > L;
#pragma unroll
        for (int r = 0; r < kSeg; ++r) yacc[r] = 0.f;
        for (int j = j0; j < j0 + nj; ++j, ++q) {
            const int jl = j - j0;
            const int slot = (int)(q % S);
            float* stage = ring + slot * kStageF;
            cp_wait<S - 2>();
            __syncwarp();

            // this thread's samples: its own chunk and the first NB-1 of the next one
            float uc[NU];
#pragma unroll
            for (int r = 0; r < kSeg / 4; ++r) {
                const float4 t4 = *reinterpret_cast<const float4*>(stage + lid * kChunk + 4 * r);
                uc[4 * r] = t4.x, uc[4 * r + 1] = t4.y, uc[4 * r + 2] = t4.z, uc[4 * r + 3] = t4.w;
            }
#pragma unroll
            for (int r = 0; r < (NB - 1 + 3) / 4; ++r) {
                const float4 t4 = *reinterpret_cast<const float4*>(stage + (lid + 1) * kChunk + 4 * r);
                const float t[4] = {t4.x, t4.y, t4.z, t4.w};
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (4 * r + e < NB - 1) uc[kSeg + 4 * r + e] = t[e];
            }
            __syncwarp();  // everyone has read this stage before the next item's copies may land
            if (q + S - 1 < items) issue(q + S - 1, (int)((q + S - 1) % S));
            cp_commit();

            float a[NA], bt[NB];
#pragma unroll
            for (int k = 0; k < NA; ++k) a[k] = p.a[(i * p.I + j) * NA + k];
#pragma unroll
            for (int k = 0; k < NB; ++k) bt[k] = p.taps[(i * p.I + j) * NB + k];

            // numerator: w_t = sum_k b_k u_buf[t + NB-1 - k]; steps past the sequence get zero
            float v[kSeg];
#pragma unroll
            for (int r = 0; r < kSeg; ++r) {
                float acc = 0.f;
#pragma unroll
                for (int k = NB - 1; k >= 0; --k) acc = fmaf(bt[k], uc[r + NB - 1 - k], acc);
                v[r] = (!edge || tbase + r < L) ? acc : 0.f;
            }

            // 1. zero-state response of this thread's segment
            float s[NA];
#pragma unroll
            for (int k = 0; k < NA; ++k) s[k] = 0.f;
#pragma unroll
            for (int k = 0; k < kSeg; ++k) iir_step<NA>(a, s, v[k]);

            // 2. carry of the previous tile enters at thread 0; Kogge-Stone over the 32 segments
            const double* Mj = Mp + jl * 5 * NA * NA;
            double cin[NA], sd[NA];
#pragma unroll
            for (int k = 0; k < NA; ++k) {
                cin[k] = cins[jl * NA + k];
                sd[k] = (double)s[k];
            }
            if (lid == 0) {
#pragma unroll
                for (int r = 0; r < NA; ++r) {
                    double t = sd[r];
#pragma unroll
                    for (int k = 0; k < NA; ++k) t = fma(Mj[r * NA + k], cin[k], t);
                    sd[r] = t;
                }
            }
#pragma unroll
            for (int d = 0; d < 5; ++d) {
                double sp[NA];
#pragma unroll
                for (int k = 0; k < NA; ++k) sp[k] = __shfl_up_sync(0xffffffffu, sd[k], 1 << d);
                if (lid >= (1 << d)) {
                    const double* M = Mj + d * NA * NA;
#pragma unroll
                    for (int r = 0; r < NA; ++r) {
                        double t = sd[r];
#pragma unroll
                        for (int k = 0; k < NA; ++k) t = fma(M[r * NA + k], sp[k], t);
                        sd[r] = t;
                    }
                }
            }
            float st[NA];
#pragma unroll
            for (int k = 0; k < NA; ++k) {
                const double up = __shfl_up_sync(0xffffffffu, sd[k], 1);
                st[k] = (float)(lid == 0 ? cin[k] : up);
            }
#pragma unroll
            for (int k = 0; k < NA; ++k) {
                const double e = __shfl_sync(0xffffffffu, sd[k], 31);
                if (lid == 0) cins[jl * NA + k] = e;
            }

            // 3. the true run of the segment; add the pair's output to the channel sum
#pragma unroll
            for (int k = 0; k < kSeg; ++k) {
                v[k] = iir_step<NA>(a, st, v[k]);
                yacc[k] += v[k];
            }

            // stage the pair's tile: per-pair store (if asked for) and the block's new state
#pragma unroll
            for (int r = 0; r < kSeg / 4; ++r)
                *reinterpret_cast<float4*>(stage + lid * kChunk + 4 * r) =
                    make_float4(v[4 * r], v[4 * r + 1], v[4 * r + 2], v[4 * r + 3]);
            __syncwarp();
            const long long pr = b * P + j * p.O + i;
            if (p.yp != nullptr) {
                float* out = p.yp + pr * L;
#pragma unroll
                for (int r = 0; r < PIECES / 32; ++r) {
                    const int gidx = r * 32 + lid;
                    const long long t = t0 + (long long)gidx * VEC;
                    if (t < L) {
                        const float* sp = stage + (gidx / PPC) * kChunk + (gidx % PPC) * VEC;
                        if constexpr (VEC == 4) __stcs(reinterpret_cast<float4*>(out + t), *reinterpret_cast<const float4*>(sp));
                        else __stcs(out + t, *sp);
                    }
                }
            }
            if (lid < NA) {  // x_last[k] = y_{L-1-k}; older ones come from the previous tile or x0
                if (c == C - 1) {
                    const long long t = L - 1 - lid;
                    float val;
                    if (t >= t0) {
                        const int x = (int)(t - t0);
                        val = stage[(x / kSeg) * kChunk + (x % kSeg)];
                    } else if (t >= 0) {
                        val = ptail[jl * NA + (int)(t0 - 1 - t)];
                    } else {
                        val = p.x0 != nullptr ? p.x0[pr * NA + (int)(-t - 1)] : 0.f;
                    }
                    p.xlast[pr * NA + lid] = val;
                }
            }
            __syncwarp();
            if (lid < NA && c < C - 1) {  // tail of a whole tile: y_{t0+1023-k}
                const int x = kTile - 1 - lid;
                ptail[jl * NA + lid] = stage[(x / kSeg) * kChunk + (x % kSeg)];
            }
            __syncwarp();
        }
        if (p.y == nullptr) continue;  // split mode: the caller sums the per-pair outputs
        // the channel's tile: stage and store coalesced
#pragma unroll
        for (int r = 0; r < kSeg / 4; ++r)
            *reinterpret_cast<float4*>(ysum + lid * kChunk + 4 * r) =
                make_float4(yacc[4 * r], yacc[4 * r + 1], yacc[4 * r + 2], yacc[4 * r + 3]);
        __syncwarp();
        float* out = p.y + (b * p.O + i) * L;
#pragma unroll
        for (int r = 0; r < PIECES / 32; ++r) {
            const int gidx = r * 32 + lid;
            const long long t = t0 + (long long)gidx * VEC;
            if (t < L) {
                const float* sp = ysum + (gidx / PPC) * kChunk + (gidx % PPC) * VEC;
                if constexpr (VEC == 4) __stcs(reinterpret_cast<float4*>(out + t), *reinterpret_cast<const float4*>(sp));
                else __stcs(out + t, *sp);
            }
        }
        __syncwarp();
    }
    cp_wait<0>();
}

// Adjoint of the G-block's numerator.  gw [B, I*O, L] is the gradient w.r.t. the numerator outputs
// (what the all-pole adjoint produces); one warp owns (batch row b, input channel j), walks time in
// 1024-step tiles and, inside a tile, the O pairs of its input:
//   gub[b, j, NB-1 + t] = sum_i sum_k taps[i,j,k] gw[b, j*O+i, t + k]     (input gradient, tail included)
//   gtaps[b, i, j, k]   = sum_t gw[b, j*O+i, t] ub[b, j, t + NB-1 - k]    (per batch row; summed by the caller)
// The input tile is fetched once per tile, every gw tile once; the tap sums are reduced over the warp
// with a fixed butterfly per (tile, output) and accumulated in shared memory ([O][NB]) in tile order, so
// results are reproducible.  One warp per CTA and 29 KB of shared memory each: all (b, j) warps of the
// benchmark shape are resident at once (seven per SM).
struct GBlockBwdArgs {
    const float* gw;    // [B, I*O, L]
    const float* ub;    // [B*I, pitch]
    const float* taps;  // [O, I, NB]
    float* gub;         // [B*I, pitch]; split mode: [B*I*O, pitch], one row per pair
    float* gtaps;       // [B, O, I, NB]
    long long B, I, O, L, pitch;
    int split;          // one warp per pair instead of per (b, input)
};

template <int NB, int VEC, int W, int S>
__global__ void __launch_bounds__(32 * W, GBLOCK_BW_MINB) gblock_num_bwd_kernel(const GBlockBwdArgs p) {
    constexpr int kSeg = 32, kTile = 32 * kSeg, kChunk = kSeg + 4, kStageF = 33 * kChunk;
    constexpr int PIECES = kTile / VEC, PPC = kSeg / VEC, HALO = (NB - 1 + VEC - 1) / VEC, NU = kSeg + NB - 1;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int w = threadIdx.x >> 5, lid = threadIdx.x & 31;
    const long long widx = (long long)blockIdx.x * W + w;
    // normally a warp owns (b, j) and walks all outputs; in split mode (few inputs: not enough (b, j)
    // to fill the GPU) a warp owns one pair and writes that pair's input-gradient row, which the
    // caller sums over the outputs
    const long long P = p.I * p.O;
    const long long IV = p.split ? P : p.I;
    if (widx >= p.B * IV) return;  // warps never synchronise with each other
    const long long b = widx / IV, jv = widx - b * IV;
    const long long j = p.split ? jv / p.O : jv;
    const int i0 = p.split ? (int)(jv % p.O) : 0;
    const int O = (int)p.O;              // outputs of the block (sizes the shared-memory tables)
    const int ni = p.split ? 1 : O;      // outputs this warp walks
    const long long L = p.L;
    const long long orow = p.split ? b * P + j * p.O + i0 : b * p.I + j;  // row of gub this warp writes

    // input tiles in flight: the S-1 items requested ahead span at most two tiles when a warp walks several
    // outputs per tile, three when it walks one (split mode)
    const int UB = p.split ? 3 : 2;
    const int fper = (S + UB) * kStageF + 32 * kChunk + O * NB;
    float* ring = reinterpret_cast<float*>(smem_raw) + (size_t)w * fper;  // [S] gw tiles
    float* ubuf = ring + S * kStageF;                                       // [UB] input tiles
    float* gstage = ubuf + UB * kStageF;                                    // [32][kChunk] output staging
    float* gbs = gstage + 32 * kChunk;                                      // [O][NB] tap sums (lane 0 adds the warp's sum per item)
    // tap sums start at zero; the tiles too, so that what a short last tile leaves uncopied is finite
    for (int e = lid; e < fper; e += 32) ring[e] = 0.f;
    __syncwarp();

    const long long C = (L + kTile - 1) / kTile;
    const long long items = C * ni;  // item q = (tile q / ni, output channel i0 + q % ni)
    auto copy_tile = [&](float* dst, const float* src, long long room) {
#pragma unroll
        for (int r = 0; r < PIECES / 32; ++r) {
            const int gidx = r * 32 + lid;
            if ((long long)gidx * VEC < room) {
                float* d = dst + (gidx / PPC) * kChunk + (gidx % PPC) * VEC;
                if constexpr (VEC == 4) cp_async16(d, src + gidx * VEC);
                else cp_async4(d, src + gidx * VEC);
            }
        }
        if (lid < HALO && (long long)(kTile + lid * VEC) < room) {
            float* d = dst + 32 * kChunk + lid * VEC;
            if constexpr (VEC == 4) cp_async16(d, src + kTile + lid * VEC);
            else cp_async4(d, src + kTile + lid * VEC);
        }
    };
    auto issue = [&](long long q, int slot) {
        const long long c = q / ni, i = i0 + (q - c * ni);
        // gw rows are L long (L % 4 == 0 when VEC == 4): whole pieces only below L
        copy_tile(ring + slot * kStageF, p.gw + (b * P + j * p.O + i) * L + c * kTile, L - c * kTile);
        if (i == i0) copy_tile(ubuf + (int)(c % UB) * kStageF, p.ub + (b * p.I + j) * p.pitch + c * kTile, p.pitch - c * kTile);
    };
#pragma unroll
    for (int q = 0; q < S - 1; ++q) {
        if (q < items) issue(q, q);
        cp_commit();
    }

    // gradient of the carried tail: gub[s] for s < NB-1 gathers gw[s - (NB-1) + k], k >= NB-1-s
    if (lid < NB - 1) {
        float acc = 0.f;
        for (int i = i0; i < i0 + ni; ++i) {
            const float* g = p.gw + (b * P + j * p.O + i) * L;
            const float* bt = p.taps + ((long long)i * p.I + j) * NB;
            for (int k = NB - 1 - lid; k < NB; ++k) {
                const long long t = lid - (NB - 1) + k;
                if (t < L) acc = fmaf(bt[k], g[t], acc);
            }
        }
        p.gub[orow * p.pitch + lid] = acc;
    }

    float* grow = p.gub + orow * p.pitch + (NB - 1);
    long long q = 0;
    for (long long c = 0; c < C; ++c) {
        const long long t0 = c * kTile, tbase = t0 + lid * kSeg;
        float uc[NU], guacc[kSeg];
#pragma unroll
        for (int r = 0; r < kSeg; ++r) guacc[r] = 0.f;
        for (int i = i0; i < i0 + ni; ++i, ++q) {
            float* stage = ring + (int)(q % S) * kStageF;
            cp_wait<S - 2>();
            __syncwarp();
            if (i == i0) {  // this tile's input samples: own chunk and the first NB-1 of the next one
                const float* ut = ubuf + (int)(c % UB) * kStageF;
#pragma unroll
                for (int r = 0; r < kSeg / 4; ++r) {
                    const float4 t4 = *reinterpret_cast<const float4*>(ut + lid * kChunk + 4 * r);
                    uc[4 * r] = t4.x, uc[4 * r + 1] = t4.y, uc[4 * r + 2] = t4.z, uc[4 * r + 3] = t4.w;
                }
#pragma unroll
                for (int r = 0; r < (NB - 1 + 3) / 4; ++r) {
                    const float4 t4 = *reinterpret_cast<const float4*>(ut + (lid + 1) * kChunk + 4 * r);
                    const float t[4] = {t4.x, t4.y, t4.z, t4.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        if (4 * r + e < NB - 1) uc[kSeg + 4 * r + e] = t[e];
                }
                if (tbase + NU > L + NB - 1) {  // past the row: leftovers of an earlier tile
#pragma unroll
                    for (int r = 0; r < NU; ++r)
                        if (tbase + r >= L + NB - 1) uc[r] = 0.f;
                }
            }
            float gc[NU];  // gw[tbase .. tbase + 32 + NB-1), zero past the sequence
#pragma unroll
            for (int r = 0; r < kSeg / 4; ++r) {
                const float4 t4 = *reinterpret_cast<const float4*>(stage + lid * kChunk + 4 * r);
                gc[4 * r] = t4.x, gc[4 * r + 1] = t4.y, gc[4 * r + 2] = t4.z, gc[4 * r + 3] = t4.w;
            }
#pragma unroll
            for (int r = 0; r < (NB - 1 + 3) / 4; ++r) {
                const float4 t4 = *reinterpret_cast<const float4*>(stage + (lid + 1) * kChunk + 4 * r);
                const float t[4] = {t4.x, t4.y, t4.z, t4.w};
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (4 * r + e < NB - 1) gc[kSeg + 4 * r + e] = t[e];
            }
            if (tbase + NU > L) {
#pragma unroll
                for (int r = 0; r < NU; ++r)
                    if (tbase + r >= L) gc[r] = 0.f;
            }
            __syncwarp();  // everyone has read this stage before the next item's copies may land
            if (q + S - 1 < items) issue(q + S - 1, (int)((q + S - 1) % S));
            cp_commit();

            float bt[NB];
#pragma unroll
            for (int k = 0; k < NB; ++k) bt[k] = p.taps[((long long)i * p.I + j) * NB + k];
#pragma unroll
            for (int r = 0; r < kSeg; ++r) {
                float acc = guacc[r];
#pragma unroll
                for (int k = 0; k < NB; ++k) acc = fmaf(bt[k], gc[r + k], acc);
                guacc[r] = acc;
            }
            float* gb = gbs + (i - i0) * NB;
#pragma unroll
            for (int k = 0; k < NB; ++k) {
                float acc = 0.f;
#pragma unroll
                for (int r = 0; r < kSeg; ++r) acc = fmaf(gc[r], uc[r + NB - 1 - k], acc);
                // the warp's sum in a fixed (butterfly) order, added to the running tap sum by lane 0
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
                if (lid == 0) gb[k] += acc;
            }
        }
        // the input gradient of this tile: staged, then stored as coalesced 4-byte rows (its
        // position NB-1 + t in the row is not 16-byte aligned)
#pragma unroll
        for (int r = 0; r < kSeg / 4; ++r)
            *reinterpret_cast<float4*>(gstage + lid * kChunk + 4 * r) =
                make_float4(guacc[4 * r], guacc[4 * r + 1], guacc[4 * r + 2], guacc[4 * r + 3]);
        __syncwarp();
#pragma unroll 8
        for (int r = 0; r < kSeg; ++r) {
            const int x = r * 32 + lid;
            if (t0 + x < L) __stcs(grow + t0 + x, gstage[(x / kSeg) * kChunk + (x % kSeg)]);
        }
        __syncwarp();
    }
    cp_wait<0>();
    __syncwarp();
    for (int e = lid; e < ni * NB; e += 32) {  // e = (i-i0)*NB + k
        const int i = i0 + e / NB, k = e % NB;
        p.gtaps[((b * p.O + i) * p.I + j) * NB + k] = gbs[e];
    }
}

template <int NB, int VEC>
static int launch_gblock_num_bwd(const GBlockBwdArgs& a, cudaStream_t st) {
    constexpr int W = GBLOCK_BW_W, S = GBLOCK_BW_S;
    const size_t fper = (size_t)(S + (a.split ? 3 : 2)) * 33 * 36 + 32 * 36 + (size_t)a.O * NB;
    const size_t smem = W * fper * sizeof(float);
    if (smem > 200 * 1024) return B200_ERR_UNSUPPORTED;
    auto kern = gblock_num_bwd_kernel<NB, VEC, W, S>;
    static size_t configured[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && configured[dev] < smem) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return B200_ERR_LAUNCH;
        configured[dev] = smem;
    }
    const long long grid = (a.B * (a.split ? a.I * a.O : a.I) + W - 1) / W;
    if (grid > 0x7fffffffLL) return B200_ERR_UNSUPPORTED;
    kern<<<(unsigned int)grid, 32 * W, smem, st>>>(a);
    return cudaGetLastError() == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

template <int VEC>
static int dispatch_gblock_num_bwd(int nb, const GBlockBwdArgs& a, cudaStream_t st) {
    switch (nb) {
        case 4: return launch_gblock_num_bwd<4, VEC>(a, st);
        case 8: return launch_gblock_num_bwd<8, VEC>(a, st);
        case 16: return launch_gblock_num_bwd<16, VEC>(a, st);
        default: return B200_ERR_UNSUPPORTED;
    }
}

// The G-block kernels read time-contiguous input rows: ub[b, j, :] = NB-nb zeros, the carried tail
// (nb-1 samples), u[b, :, j], zeros up to the pitch.  One thread per (batch row, position): it reads
// the I channels of its time step (contiguous) and writes one sample into each of the I rows, so
// that neighbouring threads read neighbouring input rows and write neighbouring samples.
__global__ void gblock_pack_rows_kernel(const float* __restrict__ u, const float* __restrict__ tail,
                                        float* __restrict__ ub, long long B, long long L, long long I, long long pitch,
                                        int NBp, int nb) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= B * pitch) return;
    const long long s_ = idx % pitch, b = idx / pitch;
    const float* src = nullptr;
    if (s_ >= NBp - 1) {
        const long long t = s_ - (NBp - 1);
        if (t < L) src = u + (b * L + t) * I;
    } else if (s_ >= NBp - nb && tail != nullptr) {
        src = tail + (b * (nb - 1) + (s_ - (NBp - nb))) * I;
    }
    float* dst = ub + b * I * pitch + s_;
    for (long long j = 0; j < I; ++j) dst[j * pitch] = src != nullptr ? src[j] : 0.f;
}

#ifndef GBLOCK_SEG
#define GBLOCK_SEG 32  // steps per thread of the forward (16 or 32)
#endif
#ifndef GBLOCK_W
#define GBLOCK_W 1  // (batch row, output channel) warps per CTA (1 measured 2.5 % faster than 2 at B=128, T=8192, 128 filters)
#endif
#ifndef GBLOCK_S
#define GBLOCK_S 2  // ring stages per warp (2 measured 5 % faster than 3 at B=128, T=8192, 128 filters)
#endif

template <int NA, int NB, int VEC>
static int launch_gblock(const GBlockArgs& a, cudaStream_t st) {
    constexpr int W = GBLOCK_W, S = GBLOCK_S, SEG = (NB - 1 <= GBLOCK_SEG) ? GBLOCK_SEG : 32;
    const int I = (int)a.I;
    const size_t dper = (size_t)(((2 * NA * NA + I * (5 * NA * NA + NA)) + 1) & ~1);
    const size_t fper = (size_t)S * 33 * (SEG + 4) + 32 * (SEG + 4) + (size_t)((I * NA + 3) & ~3);
    const size_t smem = W * (dper * sizeof(double) + fper * sizeof(float));
    if (smem > 200 * 1024) return B200_ERR_UNSUPPORTED;
    auto kern = gblock_fwd_kernel<NA, NB, VEC, W, S, SEG>;
    static size_t configured[64] = {0};  // largest size asked for so far, per device
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && configured[dev] < smem) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return B200_ERR_LAUNCH;
        configured[dev] = smem;
    }
    const long long grid = (a.B * (a.split ? a.I * a.O : a.O) + W - 1) / W;
    if (grid > 0x7fffffffLL) return B200_ERR_UNSUPPORTED;
    kern<<<(unsigned int)grid, 32 * W, smem, st>>>(a);
    return cudaGetLastError() == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

template <int NA, int VEC>
static int dispatch_gblock_nb(int nb, const GBlockArgs& a, cudaStream_t st) {
    switch (nb) {
        case 4: return launch_gblock<NA, 4, VEC>(a, st);
        case 8: return launch_gblock<NA, 8, VEC>(a, st);
        case 16: return launch_gblock<NA, 16, VEC>(a, st);
        default: return B200_ERR_UNSUPPORTED;
    }
}

template <int VEC>
static int dispatch_gblock(int na, int nb, const GBlockArgs& a, cudaStream_t st) {
    switch (na) {
        case 1: return dispatch_gblock_nb<1, VEC>(nb, a, st);
        case 2: return dispatch_gblock_nb<2, VEC>(nb, a, st);
        case 3: return dispatch_gblock_nb<3, VEC>(nb, a, st);
        case 4: return dispatch_gblock_nb<4, VEC>(nb, a, st);
        default: return B200_ERR_UNSUPPORTED;
    }
}

}  // namespace b200

extern "C" {
int b200_gblock_fwd(int64_t B, int64_t L, int64_t I, int64_t O, int64_t na, int64_t nb, int64_t pitch,
                    const void* ub, const void* taps, const void* a, const void* x0, void* y, void* y_pairs,
                    void* x_last, void* stream) {
    using namespace b200;
    if (B < 0 || L < 0 || I < 1 || O < 1 || na < 1 || nb < 1 || pitch < L + nb - 1) return B200_ERR_ARG;
    if (na > 4 || (nb != 4 && nb != 8 && nb != 16)) return B200_ERR_UNSUPPORTED;
    if (B == 0) return B200_OK;
    if (!ub || !taps || !a || !x_last || (L > 0 && !y && !y_pairs)) return B200_ERR_ARG;
    const uintptr_t por = (uintptr_t)ub | (uintptr_t)taps | (uintptr_t)a | (uintptr_t)x0 | (uintptr_t)y |
                          (uintptr_t)y_pairs | (uintptr_t)x_last;
    if (por % 4 != 0) return B200_ERR_ARG;
    GBlockArgs p;
    p.ub = static_cast<const float*>(ub);
    p.taps = static_cast<const float*>(taps);
    p.a = static_cast<const float*>(a);
    p.x0 = static_cast<const float*>(x0);
    p.y = static_cast<float*>(y);
    p.yp = static_cast<float*>(y_pairs);
    p.xlast = static_cast<float*>(x_last);
    p.B = B, p.I = I, p.O = O, p.L = L, p.pitch = pitch;
    p.split = y == nullptr ? 1 : 0;  // without y: one warp per pair, per-pair outputs only
    const uintptr_t seq_or = (uintptr_t)ub | (uintptr_t)y | (uintptr_t)y_pairs;
    const bool vec = (L % 4 == 0) && (pitch % 4 == 0) && (seq_or % 16 == 0);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (L == 0) {  // an empty chunk leaves the state as it was
        const size_t bytes = (size_t)B * I * O * na * sizeof(float);
        const cudaError_t e = x0 ? cudaMemcpyAsync(x_last, x0, bytes, cudaMemcpyDeviceToDevice, st)
                                 : cudaMemsetAsync(x_last, 0, bytes, st);
        return e == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
    }
    return vec ? dispatch_gblock<4>((int)na, (int)nb, p, st) : dispatch_gblock<1>((int)na, (int)nb, p, st);
}


int b200_allpole_fwd(int64_t lanes, int64_t L, int64_t na, const void* a, const void* w, const void* y0,
                     void* y, void* stream) {
    return b200::run_allpole(false, lanes, L, na, a, w, nullptr, y0, y, nullptr, nullptr, stream);
}

int b200_allpole_bwd(int64_t lanes, int64_t L, int64_t na, const void* g, const void* a, const void* y,
                     const void* y0, void* ga, void* gw, void* gy0, void* stream) {
    return b200::run_allpole(true, lanes, L, na, a, g, y, y0, gw, ga, gy0, stream);
}

size_t b200_gblock_bwd_workspace_bytes(int64_t B, int64_t L, int64_t I, int64_t O) {
    if (B <= 0 || L <= 0 || I <= 0 || O <= 0) return 256;
    return b200::align_up((size_t)B * I * O * L * sizeof(float), 256);
}

int b200_gblock_bwd(int64_t B, int64_t L, int64_t I, int64_t O, int64_t na, int64_t nb, int64_t pitch,
                    const void* gy, const void* ub, const void* taps, const void* a, const void* y_pairs,
                    const void* x0, void* gub, int64_t gub_per_filter, void* gtaps, void* ga, void* gx0,
                    void* workspace, size_t workspace_bytes, void* stream) {
    using namespace b200;
    const int64_t gub_rows = gub_per_filter ? B * I * O : B * I;
    if (B < 0 || L < 0 || I < 1 || O < 1 || na < 1 || nb < 1 || pitch < L + nb - 1) return B200_ERR_ARG;
    if (na > 4 || (nb != 4 && nb != 8 && nb != 16)) return B200_ERR_UNSUPPORTED;
    if (B == 0) return B200_OK;
    if (!ub || !taps || !a || !gub || !gtaps || !ga || (x0 && !gx0)) return B200_ERR_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (L == 0) {  // nothing flows through an empty chunk: zero gradients, the state passes through
        cudaError_t e = cudaMemsetAsync(gub, 0, (size_t)gub_rows * pitch * sizeof(float), st);
        if (e == cudaSuccess) e = cudaMemsetAsync(gtaps, 0, (size_t)B * O * I * nb * sizeof(float), st);
        if (e == cudaSuccess) e = cudaMemsetAsync(ga, 0, (size_t)B * I * O * na * sizeof(float), st);
        if (e == cudaSuccess && gx0) e = cudaMemsetAsync(gx0, 0, (size_t)B * I * O * na * sizeof(float), st);
        return e == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
    }
    if (!gy || !y_pairs) return B200_ERR_ARG;
    if (!workspace || ((uintptr_t)workspace % 256) != 0 || workspace_bytes < b200_gblock_bwd_workspace_bytes(B, L, I, O))
        return B200_ERR_WORKSPACE;
    // 1. denominator adjoint on every pair, upstream gradient and coefficients read through the row map
    int rc = run_allpole(true, B * I * O, L, na, a, gy, y_pairs, x0, workspace, ga, gx0, stream, I * O, O);
    if (rc != B200_OK) return rc;
    // 2. numerator adjoint
    GBlockBwdArgs p;
    p.gw = static_cast<const float*>(workspace);
    p.ub = static_cast<const float*>(ub);
    p.taps = static_cast<const float*>(taps);
    p.gub = static_cast<float*>(gub);
    p.gtaps = static_cast<float*>(gtaps);
    p.B = B, p.I = I, p.O = O, p.L = L, p.pitch = pitch;
    p.split = gub_per_filter ? 1 : 0;
    const uintptr_t por = (uintptr_t)ub | (uintptr_t)taps | (uintptr_t)gub | (uintptr_t)gtaps;
    if (por % 4 != 0) return B200_ERR_ARG;
    const bool vec = (L % 4 == 0) && (pitch % 4 == 0) && (((uintptr_t)ub | (uintptr_t)workspace) % 16 == 0);
    // positions of a row past NB-1 + L are not written by the kernel
    if (cudaMemsetAsync(gub, 0, (size_t)gub_rows * pitch * sizeof(float), st) != cudaSuccess) return B200_ERR_LAUNCH;
    return vec ? dispatch_gblock_num_bwd<4>((int)nb, p, st) : dispatch_gblock_num_bwd<1>((int)nb, p, st);
}

int b200_gblock_pack_rows(int64_t B, int64_t L, int64_t I, int64_t nb_padded, int64_t nb, int64_t pitch,
                          const void* u, const void* tail, void* ub, void* stream) {
    if (B < 0 || L < 0 || I < 1 || nb < 1 || nb_padded < nb || pitch < L + nb_padded - 1) return B200_ERR_ARG;
    const long long total = B * pitch;  // one thread per (batch row, position)
    if (total == 0) return B200_OK;
    if (!ub || (L > 0 && !u)) return B200_ERR_ARG;
    const long long blocks = (total + 255) / 256;
    if (blocks > 0x7fffffffLL) return B200_ERR_UNSUPPORTED;
    b200::gblock_pack_rows_kernel<<<(unsigned int)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const float*>(u), static_cast<const float*>(tail), static_cast<float*>(ub), B, L, I, pitch,
        (int)nb_padded, (int)nb);
    return cudaGetLastError() == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

}  // extern "C"
