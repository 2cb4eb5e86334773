// Diagonal linear scans x_t = a_t * x_{t-1} + v_t (S1: a constant per lane, S2: a per step),
// real float32 and complex64, forward and reverse-time adjoint, as one templated single-pass
// chunked scan with decoupled look-back.
//
// Data layout: sequences [M, L, N] with the state axis N contiguous, so a warp reading one
// time step of 32*V neighbouring lanes issues one fully coalesced 128..512-byte access.
//
// Tiling: a CTA owns TT = W*TS consecutive (logical) time steps of NL = 32*V lanes of one row
// m.  Warp w holds steps [w*TS, (w+1)*TS) of all NL lanes in registers (TS independent
// vector loads per tensor per thread, issued back to back), so a tile is read from HBM exactly
// once and never staged.  The scan runs in three levels over the monoid of affine maps
// (A, B): x -> A*x + B:
//   1. each thread folds its TS steps sequentially (registers),
//   2. warp 0 folds the W per-warp aggregates through shared memory,
//   3. tiles are chained along time by decoupled look-back: a tile publishes its aggregate
//      (flag 1), walks back over predecessors folding aggregates until it meets an inclusive
//      state (flag 2), then publishes its own inclusive state.
// Tiles take their index from an atomic ticket and the ticket order is time-major, so the
// predecessor of a tile always holds an earlier ticket: it is running or finished, and the
// bounded wait in wait_flag() can only run out if the GPU itself stalls.
//
// The adjoint is the same scan in reversed time (logical step s <-> t = L-1-s) over
// (conj(a_{t+1}), g_t), with the epilogue producing gv = G, glam and gx0.  For S1 the per-lane
// sum glam = sum_t G_t conj(x_{t-1}) is reduced deterministically: per-tile partials go to the
// workspace and the tile that finishes last adds them in time order.
#include "common.cuh"

namespace b200 {

struct DiagArgs {
    const void* coef;  // lam
    const void* val;   // fwd: v      bwd: g
    const void* xsrc;  // bwd: forward output x_1..x_L
    const void* x0;    // may be null
    void* out;         // fwd: out    bwd: gv
    void* gcoef;       // bwd: glam
    void* gx0;         // bwd: may be null
    long long M, L, N;
    long long C, J;  // time tiles, lane tiles
    WsHeader* hdr;
    unsigned int* flags;  // [C*M*J]
    unsigned int* done;   // [M*J]  (S1 backward)
    void* aggA;           // [C*M*J*NL]
    void* aggB;
    void* incl;
    void* part;  // [C*M*N]  (S1 backward)
};

template <typename E, bool VARY, bool BWD, int V, int TS, int W, int MINB>
__global__ void __launch_bounds__(32 * W, MINB) diag_scan_kernel(const DiagArgs p) {
    using O = Ops<E>;
    using P = Pack<E, V>;
    constexpr int NL = 32 * V;
    constexpr int TT = TS * W;

    __shared__ E sA[W][NL];
    __shared__ E sB[W][NL];
    __shared__ E sX[NL];
    __shared__ unsigned int sTicket;

    const int w = threadIdx.x >> 5;
    const int lid = threadIdx.x & 31;
    if (threadIdx.x == 0) sTicket = atomicAdd(&p.hdr->ticket, 1u);
    __syncthreads();

    const long long k = sTicket;
    const long long MJ = p.M * p.J;
    const long long c = k / MJ;
    const long long r = k - c * MJ;
    const long long m = r / p.J;
    const long long j = r - m * p.J;
    const long long n0 = j * NL + (long long)lid * V;
    const bool lane_ok = n0 < p.N;
    const long long s0 = c * TT + (long long)w * TS;  // first logical step of this thread
    const long long L = p.L, N = p.N;

    const E* coef = static_cast<const E*>(p.coef);
    const E* val = static_cast<const E*>(p.val);
    const E* xsrc = static_cast<const E*>(p.xsrc);
    const E* x0 = static_cast<const E*>(p.x0);
    const long long row0 = m * L;  // sequence element (m, t, n) sits at ((row0 + t) * N + n)

    P ones, zeros;
#pragma unroll
    for (int q = 0; q < V; ++q) {
        ones.e[q] = O::one();
        zeros.e[q] = O::zero();
    }

    // ---------------------------------------------------------------- loads (all up front)
    P ca[VARY ? TS : 1];
    P vb[TS];
    P xp[BWD ? TS : 1];
    if constexpr (!VARY) {
        ca[0] = lane_ok ? *reinterpret_cast<const P*>(coef + m * N + n0) : ones;
        if constexpr (BWD) {
#pragma unroll
            for (int q = 0; q < V; ++q) ca[0].e[q] = O::conj(ca[0].e[q]);
        }
    }
    // Element offset of this thread's step i is base + i * dstep; steps past the end of the
    // sequence (s >= L) are never dereferenced.
    const long long t0 = BWD ? (L - 1 - s0) : s0;
    const long long dstep = BWD ? -N : N;
    const long long base = (row0 + t0) * N + n0;
    const int nlive = lane_ok ? (int)max(0LL, min((long long)TS, L - s0)) : 0;  // live steps of this thread
#pragma unroll
    for (int i = 0; i < TS; ++i) {
        const bool ok = i < nlive;
        vb[i] = ok ? ld_stream(reinterpret_cast<const P*>(val + base + i * dstep)) : zeros;
        if constexpr (VARY) {
            if constexpr (!BWD) {
                ca[i] = ok ? ld_stream(reinterpret_cast<const P*>(coef + base + i * dstep)) : ones;
            } else {
                // adjoint coefficient conj(a_{t+1}); at t = L-1 (s = 0) it multiplies G_L = 0
                if (ok && (s0 + i) > 0) {
                    ca[i] = ld_stream(reinterpret_cast<const P*>(coef + base + i * dstep + N));
#pragma unroll
                    for (int q = 0; q < V; ++q) ca[i].e[q] = O::conj(ca[i].e[q]);
                } else {
                    ca[i] = ok ? zeros : ones;
                }
            }
        }
        if constexpr (BWD) {
            if (ok && (s0 + i) < L - 1) {  // t > 0
                xp[i] = ld_stream(reinterpret_cast<const P*>(xsrc + base + i * dstep - N));
            } else if (ok && x0 != nullptr) {
                xp[i] = *reinterpret_cast<const P*>(x0 + m * N + n0);
            } else {
                xp[i] = zeros;
            }
        }
    }

    // ---------------------------------------------------------------- level 1: thread fold
    E A[V], Bv[V];
#pragma unroll
    for (int q = 0; q < V; ++q) {
        A[q] = O::one();
        Bv[q] = O::zero();
    }
#pragma unroll
    for (int i = 0; i < TS; ++i) {
        const bool live = (s0 + i) < L;
#pragma unroll
        for (int q = 0; q < V; ++q) {
            const E cc = VARY ? ca[i].e[q] : (live ? ca[0].e[q] : O::one());
            Bv[q] = O::fma(cc, Bv[q], vb[i].e[q]);
            A[q] = O::mul(A[q], cc);
        }
    }
#pragma unroll
    for (int q = 0; q < V; ++q) {
        sA[w][lid * V + q] = A[q];
        sB[w][lid * V + q] = Bv[q];
    }
    __syncthreads();

    // ---------------------------------------------------------------- levels 2 and 3 (warp 0)
    if (w == 0) {
        E pa[V], pb[V];
#pragma unroll
        for (int q = 0; q < V; ++q) {
            pa[q] = O::one();
            pb[q] = O::zero();
        }
        // exclusive prefixes per warp replace the aggregates in shared memory
#pragma unroll
        for (int ww = 0; ww < W; ++ww) {
#pragma unroll
            for (int q = 0; q < V; ++q) {
                const E a = sA[ww][lid * V + q], b = sB[ww][lid * V + q];
                sA[ww][lid * V + q] = pa[q];
                sB[ww][lid * V + q] = pb[q];
                pb[q] = O::fma(a, pb[q], b);
                pa[q] = O::mul(a, pa[q]);
            }
        }
        const long long tile = (c * p.M + m) * p.J + j;
        P* aggA = static_cast<P*>(p.aggA) + tile * 32 + lid;
        P* aggB = static_cast<P*>(p.aggB) + tile * 32 + lid;
        P* incl = static_cast<P*>(p.incl) + tile * 32 + lid;
        const bool has_next = c + 1 < p.C;
        P xin = zeros;
        if (c == 0) {
            if constexpr (!BWD) {
                if (x0 != nullptr && lane_ok) xin = *reinterpret_cast<const P*>(x0 + m * N + n0);
            }
        } else {
            if (has_next) {
                P ta, tb;
#pragma unroll
                for (int q = 0; q < V; ++q) {
                    ta.e[q] = pa[q];
                    tb.e[q] = pb[q];
                }
                st_cg(aggA, ta);
                st_cg(aggB, tb);
                __threadfence();
                __syncwarp();
                if (lid == 0) st_release(p.flags + tile, 1u);
            }
            // look back: xin = fa * X + fb, X the state at the end of tile cc
            E fa[V], fb[V];
#pragma unroll
            for (int q = 0; q < V; ++q) {
                fa[q] = O::one();
                fb[q] = O::zero();
            }
            const long long stride = MJ;  // tiles between consecutive time tiles of one lane group
            long long pt = tile - stride;
            for (long long cc = c - 1; cc >= 0; --cc, pt -= stride) {
                const unsigned int f = wait_flag(p.flags + pt);
                if (f == 2u) {
                    const P X = ld_cg(static_cast<const P*>(p.incl) + pt * 32 + lid);
#pragma unroll
                    for (int q = 0; q < V; ++q) fb[q] = O::fma(fa[q], X.e[q], fb[q]);
                    break;
                }
                if (f == 0u) {  // gave up: flag the launch, keep going with what we have
                    atomicExch(&p.hdr->error, (unsigned int)B200_ERR_TIMEOUT);
                    break;
                }
                const P a = ld_cg(static_cast<const P*>(p.aggA) + pt * 32 + lid);
                const P b = ld_cg(static_cast<const P*>(p.aggB) + pt * 32 + lid);
#pragma unroll
                for (int q = 0; q < V; ++q) {
                    fb[q] = O::fma(fa[q], b.e[q], fb[q]);
                    fa[q] = O::mul(fa[q], a.e[q]);
                }
            }
#pragma unroll
            for (int q = 0; q < V; ++q) xin.e[q] = fb[q];
        }
        if (has_next) {
            P ti;
#pragma unroll
            for (int q = 0; q < V; ++q) ti.e[q] = O::fma(pa[q], xin.e[q], pb[q]);
            st_cg(incl, ti);
            __threadfence();
            __syncwarp();
            if (lid == 0) st_release(p.flags + tile, 2u);
        }
#pragma unroll
        for (int q = 0; q < V; ++q) sX[lid * V + q] = xin.e[q];
    }
    __syncthreads();

    // ---------------------------------------------------------------- apply carry, epilogue
    E x[V], acc[V];
#pragma unroll
    for (int q = 0; q < V; ++q) {
        x[q] = O::fma(sA[w][lid * V + q], sX[lid * V + q], sB[w][lid * V + q]);
        acc[q] = O::zero();
    }
    E* out = static_cast<E*>(p.out);
    E* gcoef = static_cast<E*>(p.gcoef);
    E* gx0 = static_cast<E*>(p.gx0);
#pragma unroll
    for (int i = 0; i < TS; ++i) {
        const bool live = (s0 + i) < L;
        const bool ok = i < nlive;
#pragma unroll
        for (int q = 0; q < V; ++q) {
            const E cc = VARY ? ca[i].e[q] : (live ? ca[0].e[q] : O::one());
            x[q] = O::fma(cc, x[q], vb[i].e[q]);
            vb[i].e[q] = x[q];
        }
        if (ok) st_stream(reinterpret_cast<P*>(out + base + i * dstep), vb[i]);
        if constexpr (BWD) {
            if constexpr (VARY) {
                P gl;
#pragma unroll
                for (int q = 0; q < V; ++q) gl.e[q] = O::mul(x[q], O::conj(xp[i].e[q]));
                if (ok) st_stream(reinterpret_cast<P*>(gcoef + base + i * dstep), gl);
            } else {
                if (live) {
#pragma unroll
                    for (int q = 0; q < V; ++q) acc[q] = O::fma(x[q], O::conj(xp[i].e[q]), acc[q]);
                }
            }
            if (ok && (s0 + i) == L - 1 && gx0 != nullptr) {  // t == 0
                P a0;
                if constexpr (VARY) {
                    a0 = *reinterpret_cast<const P*>(coef + row0 * N + n0);
#pragma unroll
                    for (int q = 0; q < V; ++q) a0.e[q] = O::conj(a0.e[q]);
                } else {
                    a0 = ca[0];
                }
                P gx;
#pragma unroll
                for (int q = 0; q < V; ++q) gx.e[q] = O::mul(a0.e[q], x[q]);
                *reinterpret_cast<P*>(gx0 + m * N + n0) = gx;
            }
        }
    }

    // ---------------------------------------------------------------- S1 adjoint: glam reduction
    if constexpr (BWD && !VARY) {
        __syncthreads();
#pragma unroll
        for (int q = 0; q < V; ++q) sA[w][lid * V + q] = acc[q];
        __syncthreads();
        if (w == 0) {
            P tot = zeros;
#pragma unroll
            for (int ww = 0; ww < W; ++ww) {
#pragma unroll
                for (int q = 0; q < V; ++q) tot.e[q] = O::add(tot.e[q], sA[ww][lid * V + q]);
            }
            if (p.C == 1) {
                if (lane_ok) *reinterpret_cast<P*>(gcoef + m * N + n0) = tot;
            } else {
                E* part = static_cast<E*>(p.part);
                if (lane_ok) st_cg(reinterpret_cast<P*>(part + (c * p.M + m) * N + n0), tot);
                __threadfence();
                __syncwarp();
                unsigned int prev = 0;
                if (lid == 0) prev = atomicAdd(p.done + m * p.J + j, 1u);
                prev = __shfl_sync(0xffffffffu, prev, 0);
                if (prev == (unsigned int)(p.C - 1)) {  // last tile of this lane group: add in time order
                    __threadfence();
                    if (lane_ok) {
                        P sum = zeros;
                        for (long long cc = 0; cc < p.C; ++cc) {
                            const P v = ld_cg(reinterpret_cast<const P*>(part + (cc * p.M + m) * N + n0));
#pragma unroll
                            for (int q = 0; q < V; ++q) sum.e[q] = O::add(sum.e[q], v.e[q]);
                        }
                        *reinterpret_cast<P*>(gcoef + m * N + n0) = sum;
                    }
                }
            }
        }
    }
}

// ------------------------------------------------------------------------------- host side
// Tile shape. A thread holds DIAG_*_BYTES of every streamed tensor in registers (the forward
// streams two tensors in and one out, the adjoint three in and two out), a CTA has DIAG_*_W
// warps along time, and DIAG_MINB CTAs are asked to fit one SM so that the loads of one tile
// overlap the fold and stores of another. The macros exist so that tuning builds can sweep them.
#ifndef DIAG_FWD_BYTES
#define DIAG_FWD_BYTES 128
#endif
#ifndef DIAG_BWD_BYTES
#define DIAG_BWD_BYTES 64
#endif
#ifndef DIAG_FWD_W
#define DIAG_FWD_W 8
#endif
#ifndef DIAG_BWD_W
#define DIAG_BWD_W 8
#endif
#ifndef DIAG_MINB
#define DIAG_MINB 2
#endif

template <typename E, int V, bool BWD>
struct Cfg {
    static constexpr int W = BWD ? DIAG_BWD_W : DIAG_FWD_W;
    static constexpr int TSraw = (BWD ? DIAG_BWD_BYTES : DIAG_FWD_BYTES) / (int)(sizeof(E) * V);
    static constexpr int TS = TSraw > 16 ? 16 : TSraw;  // narrow vectors: cap the unrolled steps
    static_assert(TS >= 1, "tile bytes too small for this vector width");
};

struct DiagPlan {
    int V, TS, W;
    long long C, J, tiles;
    size_t off_flags, off_done, zero_bytes, off_aggA, off_aggB, off_incl, off_part, total;
};

static DiagPlan make_plan(int dtype, int V, bool bwd, bool needs_part, long long M, long long L, long long N) {
    DiagPlan pl;
    const size_t esz = dtype == B200_C64 ? 8 : 4;
    pl.V = V;
    pl.W = bwd ? DIAG_BWD_W : DIAG_FWD_W;
    pl.TS = (bwd ? DIAG_BWD_BYTES : DIAG_FWD_BYTES) / (int)(esz * V);
    if (pl.TS > 16) pl.TS = 16;
    const long long NL = 32LL * V, TT = (long long)pl.TS * pl.W;
    pl.C = (L + TT - 1) / TT;
    pl.J = (N + NL - 1) / NL;
    pl.tiles = pl.C * M * pl.J;
    size_t off = sizeof(WsHeader);
    pl.off_flags = off;
    off += sizeof(unsigned int) * (size_t)pl.tiles;
    pl.off_done = off;
    off += sizeof(unsigned int) * (size_t)(M * pl.J);
    pl.zero_bytes = off;
    off = align_up(off, 256);
    const size_t agg = align_up((size_t)pl.tiles * NL * esz, 256);
    pl.off_aggA = off;
    off += agg;
    pl.off_aggB = off;
    off += agg;
    pl.off_incl = off;
    off += agg;
    pl.off_part = off;
    if (needs_part) off += align_up((size_t)(pl.C * M * N) * esz, 256);
    pl.total = off;
    return pl;
}

static int max_v(int dtype) { return dtype == B200_C64 ? 2 : 4; }

// Vector width: the widest access every pointer and the row pitch allow, unless a narrower one
// wastes fewer padded lanes (N = 64 real -> V = 2 so one warp spans exactly the row).
static int choose_v(int dtype, long long N, uintptr_t ptr_or) {
    const size_t esz = dtype == B200_C64 ? 8 : 4;
    int best = 1;
    long long best_pad = (N + 31) / 32 * 32;
    for (int V = 2; V <= max_v(dtype); V *= 2) {
        if (N % V != 0 || (ptr_or % (esz * V)) != 0) break;
        const long long NL = 32LL * V, pad = (N + NL - 1) / NL * NL;
        if (pad <= best_pad) {
            best = V;
            best_pad = pad;
        }
    }
    return best;
}

static size_t workspace_bytes(int dtype, bool bwd, bool needs_part, long long M, long long L, long long N) {
    size_t mx = 0;
    for (int V = 1; V <= max_v(dtype); V *= 2) {
        const DiagPlan pl = make_plan(dtype, V, bwd, needs_part, M, L, N);
        if (pl.total > mx) mx = pl.total;
    }
    return mx;
}

template <typename E, bool VARY, bool BWD, int V>
static int launch(const DiagArgs& a, const DiagPlan& pl, cudaStream_t st) {
    using C = Cfg<E, V, BWD>;
    diag_scan_kernel<E, VARY, BWD, V, C::TS, C::W, DIAG_MINB><<<(unsigned int)pl.tiles, 32 * C::W, 0, st>>>(a);
    return cudaGetLastError() == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

template <bool VARY, bool BWD>
static int dispatch(int dtype, const DiagArgs& a, const DiagPlan& pl, cudaStream_t st) {
    if (dtype == B200_F32) {
        switch (pl.V) {
            case 4: return launch<float, VARY, BWD, 4>(a, pl, st);
            case 2: return launch<float, VARY, BWD, 2>(a, pl, st);
            default: return launch<float, VARY, BWD, 1>(a, pl, st);
        }
    }
    switch (pl.V) {
        case 2: return launch<float2, VARY, BWD, 2>(a, pl, st);
        default: return launch<float2, VARY, BWD, 1>(a, pl, st);
    }
}

static int run(int dtype, bool vary, bool bwd, long long M, long long L, long long N, const void* coef,
               const void* val, const void* xsrc, const void* x0, void* out, void* gcoef, void* gx0,
               void* ws, size_t ws_bytes, void* stream) {
    if (dtype != B200_F32 && dtype != B200_C64) return B200_ERR_ARG;
    if (M < 0 || L < 0 || N < 0) return B200_ERR_ARG;
    if (M == 0 || L == 0 || N == 0) return B200_OK;
    if (!coef || !val || !out || (bwd && (!xsrc || !gcoef))) return B200_ERR_ARG;
    if (bwd && x0 && !gx0) return B200_ERR_ARG;
    const bool needs_part = bwd && !vary;
    if (!ws || ((uintptr_t)ws % 256) != 0 || ws_bytes < workspace_bytes(dtype, bwd, needs_part, M, L, N))
        return B200_ERR_WORKSPACE;
    uintptr_t por = (uintptr_t)coef | (uintptr_t)val | (uintptr_t)out | (uintptr_t)xsrc | (uintptr_t)x0 |
                    (uintptr_t)gcoef | (uintptr_t)gx0;
    const size_t esz = dtype == B200_C64 ? 8 : 4;
    if (por % esz != 0) return B200_ERR_ARG;
    const int V = choose_v(dtype, N, por);
    const DiagPlan pl = make_plan(dtype, V, bwd, needs_part, M, L, N);
    if (pl.tiles > 0x7fffffffLL) return B200_ERR_UNSUPPORTED;

    cudaStream_t st = static_cast<cudaStream_t>(stream);
    char* base = static_cast<char*>(ws);
    if (cudaMemsetAsync(base, 0, pl.zero_bytes, st) != cudaSuccess) return B200_ERR_LAUNCH;

    DiagArgs a;
    a.coef = coef;
    a.val = val;
    a.xsrc = xsrc;
    a.x0 = x0;
    a.out = out;
    a.gcoef = gcoef;
    a.gx0 = x0 ? gx0 : nullptr;
    a.M = M;
    a.L = L;
    a.N = N;
    a.C = pl.C;
    a.J = pl.J;
    a.hdr = reinterpret_cast<WsHeader*>(base);
    a.flags = reinterpret_cast<unsigned int*>(base + pl.off_flags);
    a.done = reinterpret_cast<unsigned int*>(base + pl.off_done);
    a.aggA = base + pl.off_aggA;
    a.aggB = base + pl.off_aggB;
    a.incl = base + pl.off_incl;
    a.part = base + pl.off_part;
    if (vary) return bwd ? dispatch<true, true>(dtype, a, pl, st) : dispatch<true, false>(dtype, a, pl, st);
    return bwd ? dispatch<false, true>(dtype, a, pl, st) : dispatch<false, false>(dtype, a, pl, st);
}

}  // namespace b200

extern "C" {

size_t b200_diag_workspace_bytes(int dtype, int backward, int64_t M, int64_t L, int64_t N) {
    if (M <= 0 || L <= 0 || N <= 0) return 256;
    return b200::workspace_bytes(dtype, backward != 0, backward != 0, M, L, N);
}

int b200_diag_fwd(int dtype, int64_t M, int64_t L, int64_t N, const void* lam, const void* v,
                  const void* x0, void* out, void* workspace, size_t workspace_bytes, void* stream) {
    return b200::run(dtype, false, false, M, L, N, lam, v, nullptr, x0, out, nullptr, nullptr, workspace,
                     workspace_bytes, stream);
}

int b200_diag_bwd(int dtype, int64_t M, int64_t L, int64_t N, const void* g, const void* lam,
                  const void* out, const void* x0, void* glam, void* gv, void* gx0, void* workspace,
                  size_t workspace_bytes, void* stream) {
    return b200::run(dtype, false, true, M, L, N, lam, g, out, x0, gv, glam, gx0, workspace, workspace_bytes,
                     stream);
}

size_t b200_sel_workspace_bytes(int dtype, int backward, int64_t B, int64_t L, int64_t N) {
    if (B <= 0 || L <= 0 || N <= 0) return 256;
    return b200::workspace_bytes(dtype, backward != 0, false, B, L, N);
}

int b200_sel_fwd(int dtype, int64_t B, int64_t L, int64_t N, const void* lam, const void* v,
                 const void* x0, void* out, void* workspace, size_t workspace_bytes, void* stream) {
    return b200::run(dtype, true, false, B, L, N, lam, v, nullptr, x0, out, nullptr, nullptr, workspace,
                     workspace_bytes, stream);
}

int b200_sel_bwd(int dtype, int64_t B, int64_t L, int64_t N, const void* g, const void* lam,
                 const void* out, const void* x0, void* glam, void* gv, void* gx0, void* workspace,
                 size_t workspace_bytes, void* stream) {
    return b200::run(dtype, true, true, B, L, N, lam, g, out, x0, gv, glam, gx0, workspace, workspace_bytes,
                     stream);
}

}  // extern "C"
