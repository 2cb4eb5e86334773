// Diagonal linear scans x_t = a_t * x_{t-1} + v_t (S1: a constant per lane, S2: a per step),
// real float32 and complex64, forward and reverse-time adjoint, as one templated single-pass
// chunked scan with decoupled look-back.
//
// Data layout: sequences [M, L, N] with the state axis N contiguous, so a warp touching one
// time step of 32*V neighbouring lanes moves one fully coalesced 128..512-byte segment.
//
// Tiling: a tile is TT = W*TS consecutive (logical) time steps of NL = 32*V lanes of one row m.
// Warp w of a CTA owns steps [w*TS, (w+1)*TS) of all NL lanes.
//
// Pipeline: CTAs are persistent.  Each takes tiles from an atomic ticket counter and keeps
// S-1 tiles ahead in flight: every thread copies ITS OWN slice of a future tile into a
// shared-memory ring with 4/8/16-byte cp.async, so no barrier guards the ring (a thread only
// ever reads what it copied itself) and HBM stays busy while the current tile is folded,
// chained and stored.  Each sequence element therefore crosses HBM exactly once.
//
// Scan: three levels over the monoid of affine maps (A, B): x -> A*x + B:
//   1. each thread folds its TS steps sequentially in registers,
//   2. warp 0 folds the W per-warp aggregates through shared memory,
//   3. tiles are chained along time by look-back over a FIXED window: every kAnchor-th time
//      tile is an anchor.  An anchor publishes only its inclusive state (flag 2), every other
//      tile only its aggregate (flag 1).  A tile walks back over its predecessors folding
//      their aggregates until it reaches the nearest anchor, waits for that anchor's inclusive
//      state and stops.  Which values a tile folds, and in which order, therefore depends on
//      its position alone and never on timing: two launches on the same input give the same
//      bits.  The serial chain along one lane group is one hand-over per anchor.
// Ticket order is time-major and every CTA works through its tickets in increasing order, so
// the unfinished tile with the smallest ticket is always being worked on and depends only on
// finished tiles: the chain cannot deadlock, and the bounded wait in wait_flag() can only run
// out if the GPU itself stalls (or, in the wait test, when a tile is told not to publish).
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
    long long tiles;
    WsHeader* hdr;
    unsigned int* flags;  // [C*M*J]
    unsigned int* done;   // [M*J]  (S1 backward)
    void* aggA;           // [C*M*J*NL]
    void* aggB;
    void* incl;
    void* part;  // [C*M*N]  (S1 backward)
    int spin_limit;       // polls of one flag before a wait gives up
    long long mute_tile;  // tile that publishes nothing (-1: none); only the bounded-wait test sets it
};

// Every kAnchor-th time tile hands over an inclusive state; the tiles between hand over aggregates.
constexpr int kAnchor = 4;

// cp.async of one pack (4, 8 or 16 bytes) from global to shared memory.
template <int BYTES>
__device__ __forceinline__ void cp_async(void* smem_dst, const void* gsrc) {
    const unsigned int d = static_cast<unsigned int>(__cvta_generic_to_shared(smem_dst));
    if constexpr (BYTES == 16) {
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gsrc) : "memory");
    } else if constexpr (BYTES == 8) {
        asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(d), "l"(gsrc) : "memory");
    } else {
        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(gsrc) : "memory");
    }
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Where a thread's slice of tile k lives.
struct TileCoord {
    long long c, m, j;  // time tile, row, lane tile
    long long n0;       // first lane of this thread
    long long s0;       // first logical step of this thread
    long long base;     // element offset of (m, t(s0), n0)
    long long dstep;    // element stride between consecutive logical steps
    int nlive;          // live steps of this thread (0 when its lanes are past N)
    bool lane_ok;
};

template <bool BWD, int V, int TS, int W>
__device__ __forceinline__ TileCoord tile_coord(const DiagArgs& p, long long k, int w, int lid) {
    TileCoord t;
    const long long MJ = p.M * p.J;
    t.c = k / MJ;
    const long long r = k - t.c * MJ;
    t.m = r / p.J;
    t.j = r - t.m * p.J;
    t.n0 = t.j * (32 * V) + (long long)lid * V;
    t.lane_ok = t.n0 < p.N;
    t.s0 = t.c * (TS * W) + (long long)w * TS;
    const long long t0 = BWD ? (p.L - 1 - t.s0) : t.s0;
    t.dstep = BWD ? -p.N : p.N;
    t.base = (t.m * p.L + t0) * p.N + t.n0;
    const long long left = p.L - t.s0;
    t.nlive = t.lane_ok ? (int)(left < 0 ? 0 : (left > TS ? TS : left)) : 0;
    return t;
}

template <typename E, bool VARY, bool BWD, int V, int TS, int W, int S, int MINB>
__global__ void __launch_bounds__(32 * W, MINB) diag_scan_kernel(const DiagArgs p) {
    using O = Ops<E>;
    using P = Pack<E, V>;
    constexpr int NL = 32 * V;
    constexpr int NTHR = 32 * W;
    constexpr int NT = (VARY ? 1 : 0) + 1 + (BWD ? 1 : 0);  // tensors streamed per tile
    constexpr int Q_VAL = 0, Q_COEF = 1, Q_XP = VARY ? 2 : 1;
    static_assert(S >= 2, "the ring needs at least two stages");

    extern __shared__ __align__(16) unsigned char ring_raw[];
    P* ring = reinterpret_cast<P*>(ring_raw);  // [S][NT][TS][NTHR], one pack per thread and step
    __shared__ E sA[2][W][NL];                 // double-buffered by tile parity
    __shared__ E sB[2][W][NL];
    __shared__ E sX[2][NL];
    __shared__ unsigned int sTick[S];

    const int tid = threadIdx.x;
    const int w = tid >> 5;
    const int lid = tid & 31;
    const int tick_thread = (W > 1) ? 32 : 0;  // keeps the ticket atomic off the look-back warp
    const long long L = p.L, N = p.N;

    const E* coef = static_cast<const E*>(p.coef);
    const E* val = static_cast<const E*>(p.val);
    const E* xsrc = static_cast<const E*>(p.xsrc);
    const E* x0 = static_cast<const E*>(p.x0);
    E* out = static_cast<E*>(p.out);
    E* gcoef = static_cast<E*>(p.gcoef);
    E* gx0 = static_cast<E*>(p.gx0);

    P ones, zeros;
#pragma unroll
    for (int q = 0; q < V; ++q) {
        ones.e[q] = O::one();
        zeros.e[q] = O::zero();
    }

    auto slot_ptr = [&](int slot, int q, int i) -> P* { return ring + ((slot * NT + q) * TS + i) * NTHR + tid; };

    // Start the copies of this thread's slice of tile k into ring stage `slot`.
    auto issue = [&](long long k, int slot) {
        const TileCoord tc = tile_coord<BWD, V, TS, W>(p, k, w, lid);
#pragma unroll
        for (int i = 0; i < TS; ++i) {
            if (i < tc.nlive) {
                const long long off = tc.base + i * tc.dstep;
                cp_async<sizeof(P)>(slot_ptr(slot, Q_VAL, i), val + off);
                if constexpr (VARY) {
                    if constexpr (!BWD) {
                        cp_async<sizeof(P)>(slot_ptr(slot, Q_COEF, i), coef + off);
                    } else {
                        if (tc.s0 + i > 0) cp_async<sizeof(P)>(slot_ptr(slot, Q_COEF, i), coef + off + N);
                    }
                }
                if constexpr (BWD) {
                    if (tc.s0 + i < L - 1) cp_async<sizeof(P)>(slot_ptr(slot, Q_XP, i), xsrc + off - N);
                }
            }
        }
    };

    // ---------------------------------------------------------------- prologue: S-1 tiles ahead
    if (tid == tick_thread) {
        for (int q = 0; q < S - 1; ++q) sTick[q] = atomicAdd(&p.hdr->ticket, 1u);
    }
    __syncthreads();
#pragma unroll
    for (int q = 0; q < S - 1; ++q) {
        const long long kq = sTick[q];
        if (kq < p.tiles) issue(kq, q);
        cp_async_commit();
    }

    for (int it = 0;; ++it) {
        const int slot = it % S;
        const int nslot = (it + S - 1) % S;  // stage of the tile fetched during this iteration
        const int par = it & 1;
        const long long k = sTick[slot];
        if (k >= p.tiles) break;
        if (tid == tick_thread) sTick[nslot] = atomicAdd(&p.hdr->ticket, 1u);

        const TileCoord tc = tile_coord<BWD, V, TS, W>(p, k, w, lid);
        const long long m = tc.m, n0 = tc.n0, s0 = tc.s0;
        const bool lane_ok = tc.lane_ok;
        const int nlive = tc.nlive;

        // ------------------------------------------------------------ ring -> registers
        cp_async_wait<S - 2>();
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
#pragma unroll
        for (int i = 0; i < TS; ++i) {
            const bool ok = i < nlive;
            vb[i] = ok ? *slot_ptr(slot, Q_VAL, i) : zeros;
            if constexpr (VARY) {
                if constexpr (!BWD) {
                    ca[i] = ok ? *slot_ptr(slot, Q_COEF, i) : ones;
                } else {
                    // adjoint coefficient conj(a_{t+1}); at t = L-1 (s = 0) it multiplies G_L = 0
                    if (ok && (s0 + i) > 0) {
                        ca[i] = *slot_ptr(slot, Q_COEF, i);
#pragma unroll
                        for (int q = 0; q < V; ++q) ca[i].e[q] = O::conj(ca[i].e[q]);
                    } else {
                        ca[i] = ok ? zeros : ones;
                    }
                }
            }
            if constexpr (BWD) {
                if (ok && (s0 + i) < L - 1) {  // t > 0
                    xp[i] = *slot_ptr(slot, Q_XP, i);
                } else if (ok && x0 != nullptr) {
                    xp[i] = *reinterpret_cast<const P*>(x0 + m * N + n0);
                } else {
                    xp[i] = zeros;
                }
            }
        }

        // ------------------------------------------------------------ level 1: thread fold
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
            sA[par][w][lid * V + q] = A[q];
            sB[par][w][lid * V + q] = Bv[q];
        }
        __syncthreads();

        // ------------------------------------------------------------ prefetch tile it+S-1
        {
            const long long kn = sTick[nslot];
            if (kn < p.tiles) issue(kn, nslot);
            cp_async_commit();
        }

        // ------------------------------------------------------------ levels 2 and 3 (warp 0)
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
                    const E a = sA[par][ww][lid * V + q], b = sB[par][ww][lid * V + q];
                    sA[par][ww][lid * V + q] = pa[q];
                    sB[par][ww][lid * V + q] = pb[q];
                    pb[q] = O::fma(a, pb[q], b);
                    pa[q] = O::mul(a, pa[q]);
                }
            }
            const long long tile = k;  // k == (c*M + m)*J + j by construction
            const long long stride = p.M * p.J;  // tiles between consecutive time tiles of one lane group
            const bool has_next = tc.c + 1 < p.C;
            const bool anchor = (tc.c % kAnchor) == 0;
            const bool muted = tile == p.mute_tile;
            P xin = zeros;
            if (tc.c == 0) {
                if constexpr (!BWD) {
                    if (x0 != nullptr && lane_ok) xin = *reinterpret_cast<const P*>(x0 + m * N + n0);
                }
            } else {
                if (has_next && !anchor && !muted) {  // successors fold this tile's aggregate
                    P ta, tb;
#pragma unroll
                    for (int q = 0; q < V; ++q) {
                        ta.e[q] = pa[q];
                        tb.e[q] = pb[q];
                    }
                    st_cg(static_cast<P*>(p.aggA) + tile * 32 + lid, ta);
                    st_cg(static_cast<P*>(p.aggB) + tile * 32 + lid, tb);
                    __threadfence();
                    __syncwarp();
                    if (lid == 0) st_release(p.flags + tile, 1u);
                }
                // look back to the nearest anchor: xin = fa * X + fb, X the anchor's inclusive state
                E fa[V], fb[V];
#pragma unroll
                for (int q = 0; q < V; ++q) {
                    fa[q] = O::one();
                    fb[q] = O::zero();
                }
                long long pt = tile - stride;
                for (long long cc = tc.c - 1; cc >= 0; --cc, pt -= stride) {
                    const unsigned int f = wait_flag(p.flags + pt, p.spin_limit);
                    if (f == 0u) {  // gave up: flag the launch, keep going with what we have
                        atomicExch(&p.hdr->error, (unsigned int)B200_ERR_TIMEOUT);
                        break;
                    }
                    if ((cc % kAnchor) == 0) {  // anchors only ever publish flag 2
                        const P X = ld_cg(static_cast<const P*>(p.incl) + pt * 32 + lid);
#pragma unroll
                        for (int q = 0; q < V; ++q) fb[q] = O::fma(fa[q], X.e[q], fb[q]);
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
            if (has_next && anchor && !muted) {
                P ti;
#pragma unroll
                for (int q = 0; q < V; ++q) ti.e[q] = O::fma(pa[q], xin.e[q], pb[q]);
                st_cg(static_cast<P*>(p.incl) + tile * 32 + lid, ti);
                __threadfence();
                __syncwarp();
                if (lid == 0) st_release(p.flags + tile, 2u);
            }
#pragma unroll
            for (int q = 0; q < V; ++q) sX[par][lid * V + q] = xin.e[q];
        }
        __syncthreads();

        // ------------------------------------------------------------ apply carry, epilogue
        E x[V], acc[V];
#pragma unroll
        for (int q = 0; q < V; ++q) {
            x[q] = O::fma(sA[par][w][lid * V + q], sX[par][lid * V + q], sB[par][w][lid * V + q]);
            acc[q] = O::zero();
        }
#pragma unroll
        for (int i = 0; i < TS; ++i) {
            const bool live = (s0 + i) < L;
            const bool ok = i < nlive;
            const long long off = tc.base + i * tc.dstep;
#pragma unroll
            for (int q = 0; q < V; ++q) {
                const E cc = VARY ? ca[i].e[q] : (live ? ca[0].e[q] : O::one());
                x[q] = O::fma(cc, x[q], vb[i].e[q]);
                vb[i].e[q] = x[q];
            }
            if (ok) st_stream(reinterpret_cast<P*>(out + off), vb[i]);
            if constexpr (BWD) {
                if constexpr (VARY) {
                    P gl;
#pragma unroll
                    for (int q = 0; q < V; ++q) gl.e[q] = O::mul(x[q], O::conj(xp[i].e[q]));
                    if (ok) st_stream(reinterpret_cast<P*>(gcoef + off), gl);
                } else {
                    if (live) {
#pragma unroll
                        for (int q = 0; q < V; ++q) acc[q] = O::fma(x[q], O::conj(xp[i].e[q]), acc[q]);
                    }
                }
                if (ok && (s0 + i) == L - 1 && gx0 != nullptr) {  // t == 0
                    P a0;
                    if constexpr (VARY) {
                        a0 = *reinterpret_cast<const P*>(coef + m * L * N + n0);
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

        // ------------------------------------------------------------ S1 adjoint: glam reduction
        if constexpr (BWD && !VARY) {
            __syncthreads();
#pragma unroll
            for (int q = 0; q < V; ++q) sA[par][w][lid * V + q] = acc[q];
            __syncthreads();
            if (w == 0) {
                P tot = zeros;
#pragma unroll
                for (int ww = 0; ww < W; ++ww) {
#pragma unroll
                    for (int q = 0; q < V; ++q) tot.e[q] = O::add(tot.e[q], sA[par][ww][lid * V + q]);
                }
                if (p.C == 1) {
                    if (lane_ok) *reinterpret_cast<P*>(gcoef + m * N + n0) = tot;
                } else {
                    E* part = static_cast<E*>(p.part);
                    if (lane_ok) st_cg(reinterpret_cast<P*>(part + (tc.c * p.M + m) * N + n0), tot);
                    __threadfence();
                    __syncwarp();
                    unsigned int prev = 0;
                    if (lid == 0) prev = atomicAdd(p.done + m * p.J + tc.j, 1u);
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
    cp_async_wait<0>();
}

// ===================================================================== streaming variant
// When a problem has at least as many independent chains (row m x lane tile j) as the GPU has
// room for CTAs, time needs no splitting across CTAs: one CTA owns one chain for all L steps and
// walks the time tiles in order, carrying the state in registers.  The same cp.async ring keeps
// S-1 tiles in flight, the W warps still split each tile in time and fold through shared memory
// (one barrier per tile), but there is no look-back, no flag and no workspace, and the S1
// adjoint's glam sum stays in registers until the end (fixed order, no atomics).
template <typename E, bool VARY, bool BWD, int V, int TS, int W, int S, int MINB>
__global__ void __launch_bounds__(32 * W, MINB) diag_stream_kernel(const DiagArgs p) {
    using O = Ops<E>;
    using P = Pack<E, V>;
    constexpr int NTHR = 32 * W;
    constexpr int NT = (VARY ? 1 : 0) + 1 + (BWD ? 1 : 0);
    constexpr int Q_VAL = 0, Q_COEF = 1, Q_XP = VARY ? 2 : 1;
    static_assert(S >= 2, "the ring needs at least two stages");

    extern __shared__ __align__(16) unsigned char ring_raw[];
    P* ring = reinterpret_cast<P*>(ring_raw);  // [S][NT][TS][NTHR]
    __shared__ P sA[2][W][32];                 // per-warp aggregates, double-buffered by tile parity
    __shared__ P sB[2][W][32];

    const int tid = threadIdx.x;
    const int w = tid >> 5;
    const int lid = tid & 31;
    const long long L = p.L, N = p.N;
    const long long m = blockIdx.x / p.J;
    const long long j = blockIdx.x - m * p.J;
    const long long n0 = j * (32 * V) + (long long)lid * V;
    const bool lane_ok = n0 < N;
    const long long dstep = BWD ? -N : N;

    const E* coef = static_cast<const E*>(p.coef);
    const E* val = static_cast<const E*>(p.val);
    const E* xsrc = static_cast<const E*>(p.xsrc);
    const E* x0 = static_cast<const E*>(p.x0);
    E* out = static_cast<E*>(p.out);
    E* gcoef = static_cast<E*>(p.gcoef);
    E* gx0 = static_cast<E*>(p.gx0);

    P ones, zeros;
#pragma unroll
    for (int q = 0; q < V; ++q) {
        ones.e[q] = O::one();
        zeros.e[q] = O::zero();
    }

    auto slot_ptr = [&](int slot, int q, int i) -> P* { return ring + ((slot * NT + q) * TS + i) * NTHR + tid; };
    // first logical step, live-step count and element offset of this thread's slice of time tile c
    auto first_step = [&](long long c) -> long long { return c * (TS * W) + (long long)w * TS; };
    auto live_steps = [&](long long s0) -> int {
        const long long left = L - s0;
        return lane_ok ? (int)(left < 0 ? 0 : (left > TS ? TS : left)) : 0;
    };
    auto base_of = [&](long long s0) -> long long { return (m * L + (BWD ? (L - 1 - s0) : s0)) * N + n0; };

    auto issue = [&](long long c, int slot) {
        const long long s0 = first_step(c);
        const int nlive = live_steps(s0);
        const long long base = base_of(s0);
#pragma unroll
        for (int i = 0; i < TS; ++i) {
            if (i < nlive) {
                const long long off = base + i * dstep;
                cp_async<sizeof(P)>(slot_ptr(slot, Q_VAL, i), val + off);
                if constexpr (VARY) {
                    if constexpr (!BWD) {
                        cp_async<sizeof(P)>(slot_ptr(slot, Q_COEF, i), coef + off);
                    } else {
                        if (s0 + i > 0) cp_async<sizeof(P)>(slot_ptr(slot, Q_COEF, i), coef + off + N);
                    }
                }
                if constexpr (BWD) {
                    if (s0 + i < L - 1) cp_async<sizeof(P)>(slot_ptr(slot, Q_XP, i), xsrc + off - N);
                }
            }
        }
    };

#pragma unroll
    for (int q = 0; q < S - 1; ++q) {
        if (q < p.C) issue(q, q);
        cp_async_commit();
    }

    P cl = ones;  // constant coefficient of this thread's lanes (S1)
    if constexpr (!VARY) {
        if (lane_ok) cl = *reinterpret_cast<const P*>(coef + m * N + n0);
        if constexpr (BWD) {
#pragma unroll
            for (int q = 0; q < V; ++q) cl.e[q] = O::conj(cl.e[q]);
        }
    }
    E xc[V], acc[V];  // carried state at the start of the current tile; running glam sum (S1 adjoint)
#pragma unroll
    for (int q = 0; q < V; ++q) {
        xc[q] = O::zero();
        acc[q] = O::zero();
    }
    if constexpr (!BWD) {
        if (x0 != nullptr && lane_ok) {
            const P t = *reinterpret_cast<const P*>(x0 + m * N + n0);
#pragma unroll
            for (int q = 0; q < V; ++q) xc[q] = t.e[q];
        }
    }

    for (long long c = 0; c < p.C; ++c) {
        const int slot = (int)(c % S);
        const int par = (int)(c & 1);
        const long long s0 = first_step(c);
        const int nlive = live_steps(s0);
        const long long base = base_of(s0);

        cp_async_wait<S - 2>();
        P ca[VARY ? TS : 1];
        P vb[TS];
        P xp[BWD ? TS : 1];
#pragma unroll
        for (int i = 0; i < TS; ++i) {
            const bool ok = i < nlive;
            vb[i] = ok ? *slot_ptr(slot, Q_VAL, i) : zeros;
            if constexpr (VARY) {
                if constexpr (!BWD) {
                    ca[i] = ok ? *slot_ptr(slot, Q_COEF, i) : ones;
                } else {
                    if (ok && (s0 + i) > 0) {
                        ca[i] = *slot_ptr(slot, Q_COEF, i);
#pragma unroll
                        for (int q = 0; q < V; ++q) ca[i].e[q] = O::conj(ca[i].e[q]);
                    } else {
                        ca[i] = ok ? zeros : ones;
                    }
                }
            }
            if constexpr (BWD) {
                if (ok && (s0 + i) < L - 1) {
                    xp[i] = *slot_ptr(slot, Q_XP, i);
                } else if (ok && x0 != nullptr) {
                    xp[i] = *reinterpret_cast<const P*>(x0 + m * N + n0);
                } else {
                    xp[i] = zeros;
                }
            }
        }

        // level 1: this thread's TS steps
        P A = ones, Bv = zeros;
#pragma unroll
        for (int i = 0; i < TS; ++i) {
            const bool live = (s0 + i) < L;
#pragma unroll
            for (int q = 0; q < V; ++q) {
                const E cc = VARY ? ca[i].e[q] : (live ? cl.e[q] : O::one());
                Bv.e[q] = O::fma(cc, Bv.e[q], vb[i].e[q]);
                A.e[q] = O::mul(A.e[q], cc);
            }
        }
        sA[par][w][lid] = A;
        sB[par][w][lid] = Bv;
        __syncthreads();

        if (c + S - 1 < p.C) issue(c + S - 1, (int)((c + S - 1) % S));
        cp_async_commit();

        // level 2: every thread folds the warps before it (its start state) and all of them (next carry)
        E x[V];
#pragma unroll
        for (int q = 0; q < V; ++q) x[q] = xc[q];
#pragma unroll
        for (int ww = 0; ww < W; ++ww) {
            const P a = sA[par][ww][lid], b = sB[par][ww][lid];
#pragma unroll
            for (int q = 0; q < V; ++q) xc[q] = O::fma(a.e[q], xc[q], b.e[q]);
            if (ww + 1 == w) {
#pragma unroll
                for (int q = 0; q < V; ++q) x[q] = xc[q];
            }
        }

        // apply and store
#pragma unroll
        for (int i = 0; i < TS; ++i) {
            const bool live = (s0 + i) < L;
            const bool ok = i < nlive;
            const long long off = base + i * dstep;
#pragma unroll
            for (int q = 0; q < V; ++q) {
                const E cc = VARY ? ca[i].e[q] : (live ? cl.e[q] : O::one());
                x[q] = O::fma(cc, x[q], vb[i].e[q]);
                vb[i].e[q] = x[q];
            }
            if (ok) st_stream(reinterpret_cast<P*>(out + off), vb[i]);
            if constexpr (BWD) {
                if constexpr (VARY) {
                    P gl;
#pragma unroll
                    for (int q = 0; q < V; ++q) gl.e[q] = O::mul(x[q], O::conj(xp[i].e[q]));
                    if (ok) st_stream(reinterpret_cast<P*>(gcoef + off), gl);
                } else {
                    if (live) {
#pragma unroll
                        for (int q = 0; q < V; ++q) acc[q] = O::fma(x[q], O::conj(xp[i].e[q]), acc[q]);
                    }
                }
                if (ok && (s0 + i) == L - 1 && gx0 != nullptr) {  // t == 0
                    P a0;
                    if constexpr (VARY) {
                        a0 = *reinterpret_cast<const P*>(coef + m * L * N + n0);
#pragma unroll
                        for (int q = 0; q < V; ++q) a0.e[q] = O::conj(a0.e[q]);
                    } else {
                        a0 = cl;
                    }
                    P gx;
#pragma unroll
                    for (int q = 0; q < V; ++q) gx.e[q] = O::mul(a0.e[q], x[q]);
                    *reinterpret_cast<P*>(gx0 + m * N + n0) = gx;
                }
            }
        }
    }
    cp_async_wait<0>();

    if constexpr (BWD && !VARY) {  // glam[m, lanes] = sum over warps, in warp order
        __syncthreads();
        P t;
#pragma unroll
        for (int q = 0; q < V; ++q) t.e[q] = acc[q];
        sA[0][w][lid] = t;
        __syncthreads();
        if (w == 0 && lane_ok) {
            P tot = zeros;
#pragma unroll
            for (int ww = 0; ww < W; ++ww) {
                const P v = sA[0][ww][lid];
#pragma unroll
                for (int q = 0; q < V; ++q) tot.e[q] = O::add(tot.e[q], v.e[q]);
            }
            *reinterpret_cast<P*>(gcoef + m * N + n0) = tot;
        }
    }
}

// ------------------------------------------------------------------------------- host side
// Tile shape. A thread holds DIAG_*_BYTES of every streamed tensor per tile (the forward
// streams two tensors in and one out, the adjoint three in and two out), a CTA has DIAG_*_W
// warps along time and a ring of DIAG_*_S tiles in shared memory, and DIAG_*_MINB CTAs are
// asked to fit one SM.  The macros exist so that tuning builds can sweep them.
#ifndef DIAG_FWD_BYTES
#define DIAG_FWD_BYTES 256
#endif
#ifndef DIAG_BWD_BYTES
#define DIAG_BWD_BYTES 128
#endif
#ifndef DIAG_FWD_W
#define DIAG_FWD_W 8
#endif
#ifndef DIAG_BWD_W
#define DIAG_BWD_W 8
#endif
#ifndef DIAG_FWD_S
#define DIAG_FWD_S 2
#endif
#ifndef DIAG_BWD_S
#define DIAG_BWD_S 2
#endif
#ifndef DIAG_FWD_MINB
#define DIAG_FWD_MINB 1
#endif
#ifndef DIAG_BWD_MINB
#define DIAG_BWD_MINB 1
#endif
#ifndef DIAG_MAX_VEC_BYTES
#define DIAG_MAX_VEC_BYTES 16  // widest access per thread and step
#endif

// Steps per thread: the byte budget, at most 16 (unrolled), and small enough that the ring of the
// widest instantiation (two streamed tensors forward, three in the adjoint) stays under 192 KB.
constexpr int diag_ts(int pack_bytes, bool bwd) {
    const int w = bwd ? DIAG_BWD_W : DIAG_FWD_W, st = bwd ? DIAG_BWD_S : DIAG_FWD_S, nt = bwd ? 3 : 2;
    int ts = (bwd ? DIAG_BWD_BYTES : DIAG_FWD_BYTES) / pack_bytes;
    const int cap = 196608 / (st * nt * 32 * w * pack_bytes);
    if (ts > cap) ts = cap;
    if (ts > 16) ts = 16;
    return ts < 1 ? 1 : ts;
}

template <typename E, int V, bool BWD>
struct Cfg {
    static constexpr int W = BWD ? DIAG_BWD_W : DIAG_FWD_W;
    static constexpr int S = BWD ? DIAG_BWD_S : DIAG_FWD_S;
    static constexpr int MINB = BWD ? DIAG_BWD_MINB : DIAG_FWD_MINB;
    static constexpr int TS = diag_ts((int)(sizeof(E) * V), BWD);
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
    pl.TS = diag_ts((int)(esz * V), bwd);
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

static int max_v(int dtype) { return DIAG_MAX_VEC_BYTES / (dtype == B200_C64 ? 8 : 4); }

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

// Number of SMs of the current device (queried once per device).
static int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

template <typename E, bool VARY, bool BWD, int V>
static int launch(const DiagArgs& a, const DiagPlan& pl, cudaStream_t st) {
    using C = Cfg<E, V, BWD>;
    constexpr int NT = (VARY ? 1 : 0) + 1 + (BWD ? 1 : 0);
    constexpr size_t ring = (size_t)C::S * NT * C::TS * (32 * C::W) * sizeof(E) * V;
    auto kern = diag_scan_kernel<E, VARY, BWD, V, C::TS, C::W, C::S, C::MINB>;
    static bool configured[64] = {false};  // per device: opt in to more than 48 KB of dynamic smem
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ring) != cudaSuccess)
            return B200_ERR_LAUNCH;
        configured[dev] = true;
    }
    static int per_sm = 0;  // resident CTAs per SM of this instantiation
    if (per_sm == 0) {
        int n = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, 32 * C::W, ring) != cudaSuccess || n < 1) n = 1;
        per_sm = n;
    }
    long long grid = (long long)sm_count() * per_sm;
    if (grid > pl.tiles) grid = pl.tiles;
    kern<<<(unsigned int)grid, 32 * C::W, ring, st>>>(a);
    return cudaGetLastError() == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

// Shape of the streaming variant (one CTA per chain): bytes of every streamed tensor a thread
// holds per tile, warps along time, ring stages, CTAs per SM asked of the compiler.
#ifndef STRM_FWD_BYTES
#define STRM_FWD_BYTES 128
#endif
#ifndef STRM_BWD_BYTES
#define STRM_BWD_BYTES 32
#endif
#ifndef STRM_FWD_W
#define STRM_FWD_W 4
#endif
#ifndef STRM_BWD_W
#define STRM_BWD_W 4
#endif
#ifndef STRM_FWD_S
#define STRM_FWD_S 4
#endif
#ifndef STRM_BWD_S
#define STRM_BWD_S 6
#endif
#ifndef STRM_FWD_MINB
#define STRM_FWD_MINB 1
#endif
#ifndef STRM_BWD_MINB
#define STRM_BWD_MINB 3
#endif

// complex64 streams 8-byte elements and is best with other shapes (measured at M=128, L=2000,
// N=256: adjoint 5.1 -> 6.3 TB/s, forward 5.6 -> 5.8 TB/s against the float32 shapes)
#ifndef STRM_C_FWD_BYTES
#define STRM_C_FWD_BYTES 64
#endif
#ifndef STRM_C_BWD_BYTES
#define STRM_C_BWD_BYTES 128
#endif
#ifndef STRM_C_FWD_W
#define STRM_C_FWD_W 8
#endif
#ifndef STRM_C_BWD_W
#define STRM_C_BWD_W 4
#endif
#ifndef STRM_C_FWD_S
#define STRM_C_FWD_S 4
#endif
#ifndef STRM_C_BWD_S
#define STRM_C_BWD_S 3
#endif
#ifndef STRM_C_FWD_MINB
#define STRM_C_FWD_MINB 1
#endif
#ifndef STRM_C_BWD_MINB
#define STRM_C_BWD_MINB 1
#endif

// The four (dtype, constant/varying coefficient) families stream 2..5 tensors of 4- or 8-byte
// elements, so each has its own shape (bytes per thread and tensor, warps, stages, CTAs per SM).
#ifndef STRM_S1_FWD_BYTES
#define STRM_S1_FWD_BYTES 64  // float32, constant coefficient: measured at M=128, L=2000, N=512 (5.5 -> 5.9 TB/s)
#define STRM_S1_FWD_W 8
#define STRM_S1_FWD_S 4
#define STRM_S1_FWD_MINB 1
#endif
#ifndef STRM_S1_BWD_BYTES
#define STRM_S1_BWD_BYTES 128  // (5.4 -> 6.0 TB/s)
#define STRM_S1_BWD_W 4
#define STRM_S1_BWD_S 3
#define STRM_S1_BWD_MINB 1
#endif
#ifndef STRM_CV_FWD_BYTES
#define STRM_CV_FWD_BYTES 128  // complex64, varying coefficient: measured at M=128, L=2000, N=256 (6.2 -> 6.4 TB/s)
#define STRM_CV_FWD_W 4
#define STRM_CV_FWD_S 4
#define STRM_CV_FWD_MINB 1
#endif
#ifndef STRM_CV_BWD_BYTES
#define STRM_CV_BWD_BYTES 64  // (6.0 -> 6.4 TB/s; 3.8 -> 6.0 TB/s at M=64, L=4096, N=128)
#define STRM_CV_BWD_W 4
#define STRM_CV_BWD_S 3
#define STRM_CV_BWD_MINB 3
#endif

#define B200_STRM_PICK(what)                                                                              \
    (CX ? (VARY ? (BWD ? STRM_CV_BWD_##what : STRM_CV_FWD_##what) : (BWD ? STRM_C_BWD_##what : STRM_C_FWD_##what)) \
        : (VARY ? (BWD ? STRM_BWD_##what : STRM_FWD_##what) : (BWD ? STRM_S1_BWD_##what : STRM_S1_FWD_##what)))

template <typename E, int V, bool BWD, bool VARY>
struct StreamCfg {
    static constexpr bool CX = sizeof(E) == 8;
    static constexpr int W = B200_STRM_PICK(W);
    static constexpr int S = B200_STRM_PICK(S);
    static constexpr int MINB = B200_STRM_PICK(MINB);
    static constexpr int BYTES = B200_STRM_PICK(BYTES);
    static constexpr int TSraw = BYTES / (int)(sizeof(E) * V);
    static constexpr int TS = TSraw > 16 ? 16 : (TSraw < 1 ? 1 : TSraw);
};

template <typename E, bool VARY, bool BWD, int V>
static int launch_stream(DiagArgs a, cudaStream_t st) {
    using C = StreamCfg<E, V, BWD, VARY>;
    constexpr int NT = (VARY ? 1 : 0) + 1 + (BWD ? 1 : 0);
    constexpr size_t ring = (size_t)C::S * NT * C::TS * (32 * C::W) * sizeof(E) * V;
    auto kern = diag_stream_kernel<E, VARY, BWD, V, C::TS, C::W, C::S, C::MINB>;
    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ring) != cudaSuccess)
            return B200_ERR_LAUNCH;
        configured[dev] = true;
    }
    const long long TT = (long long)C::TS * C::W;
    a.C = (a.L + TT - 1) / TT;
    a.J = (a.N + 32 * V - 1) / (32 * V);
    const long long chains = a.M * a.J;
    if (chains > 0x7fffffffLL) return B200_ERR_UNSUPPORTED;
    kern<<<(unsigned int)chains, 32 * C::W, ring, st>>>(a);
    return cudaGetLastError() == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

template <bool VARY, bool BWD>
static int dispatch_stream(int dtype, int V, const DiagArgs& a, cudaStream_t st) {
    if (dtype == B200_F32) {
        switch (V) {
            case 4: return launch_stream<float, VARY, BWD, 4>(a, st);
            case 2: return launch_stream<float, VARY, BWD, 2>(a, st);
            default: return launch_stream<float, VARY, BWD, 1>(a, st);
        }
    }
    switch (V) {
        case 2: return launch_stream<float2, VARY, BWD, 2>(a, st);
        default: return launch_stream<float2, VARY, BWD, 1>(a, st);
    }
}

// Streaming needs enough chains to fill the GPU.  Returns the vector width to stream with, or 0
// to use the look-back kernel: the widest V the pointers allow that leaves at least 1.5 chains
// per SM, else the widest that leaves one per SM.
static int stream_v(int dtype, long long M, long long N, uintptr_t ptr_or, int vcap = 0) {
    const size_t esz = dtype == B200_C64 ? 8 : 4;
    const long long sms = sm_count();
    int vmax = 1;
    for (int V = 2; V <= max_v(dtype); V *= 2) {
        if (N % V != 0 || (ptr_or % (esz * V)) != 0) break;
        vmax = V;
    }
    if (vcap >= 1 && vcap <= vmax && (vcap & (vcap - 1)) == 0) vmax = vcap;  // b200_diag_probe only
    for (int pass = 0; pass < 2; ++pass) {
        for (int V = vmax; V >= 1; V /= 2) {
            const long long chains = M * ((N + 32 * V - 1) / (32 * V));
            if (2 * chains >= (pass == 0 ? 3 : 2) * sms) return V;
        }
    }
    return 0;
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

// What the regular entry points never change: kernel choice left to the shape, full vector width,
// the one-second poll limit, every tile publishing.  b200_diag_probe passes other values.
struct RunOpts {
    int mode = 0;                 // 0 by shape, 1 look-back tiles, 2 streaming chains
    int vcap = 0;                 // cap on the vector width of the streaming kernel (0: none)
    int spin_limit = kSpinLimit;  // polls of one look-back flag
    long long mute_tile = -1;     // look-back tile that publishes nothing
};

static int run(int dtype, bool vary, bool bwd, long long M, long long L, long long N, const void* coef,
               const void* val, const void* xsrc, const void* x0, void* out, void* gcoef, void* gx0,
               void* ws, size_t ws_bytes, void* stream, const RunOpts& opt = RunOpts()) {
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
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    char* base = static_cast<char*>(ws);

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
    a.hdr = reinterpret_cast<WsHeader*>(base);
    a.spin_limit = opt.spin_limit > 0 ? opt.spin_limit : 1;
    a.mute_tile = opt.mute_tile;

    const int mode = opt.mode;
    const int sv = mode == 1 ? 0 : stream_v(dtype, M, N, por, opt.vcap);
    if (sv > 0 || mode == 2) {
        const int V = sv > 0 ? sv : choose_v(dtype, N, por);
        if (cudaMemsetAsync(base, 0, sizeof(WsHeader), st) != cudaSuccess) return B200_ERR_LAUNCH;
        a.C = a.J = a.tiles = 0;
        a.flags = a.done = nullptr;
        a.aggA = a.aggB = a.incl = a.part = nullptr;
        if (vary) return bwd ? dispatch_stream<true, true>(dtype, V, a, st) : dispatch_stream<true, false>(dtype, V, a, st);
        return bwd ? dispatch_stream<false, true>(dtype, V, a, st) : dispatch_stream<false, false>(dtype, V, a, st);
    }

    const int V = choose_v(dtype, N, por);
    const DiagPlan pl = make_plan(dtype, V, bwd, needs_part, M, L, N);
    if (pl.tiles > 0x7fffffffLL) return B200_ERR_UNSUPPORTED;
    if (cudaMemsetAsync(base, 0, pl.zero_bytes, st) != cudaSuccess) return B200_ERR_LAUNCH;
    a.C = pl.C;
    a.J = pl.J;
    a.tiles = pl.tiles;
    a.flags = reinterpret_cast<unsigned int*>(base + pl.off_flags);
    a.done = reinterpret_cast<unsigned int*>(base + pl.off_done);
    a.aggA = base + pl.off_aggA;
    a.aggB = base + pl.off_aggB;
    a.incl = base + pl.off_incl;
    a.part = base + pl.off_part;
    if (vary) return bwd ? dispatch<true, true>(dtype, a, pl, st) : dispatch<true, false>(dtype, a, pl, st);
    return bwd ? dispatch<false, true>(dtype, a, pl, st) : dispatch<false, false>(dtype, a, pl, st);
}

// ---------------------------------------------------------------- scratch for b200_diag_fwd_static
// Cross-tile state (tickets, flags, aggregates) of the look-back kernel for callers that cannot
// hand in a workspace.  It lives in the library image: every GPU that loads the library holds
// these 4 MiB until the process exits.  In host code `g_static_scratch` is only a handle for
// cudaGetSymbolAddress; the kernels get the device address that call returns.
constexpr size_t kStaticScratchBytes = size_t(4) << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// Device address of the scratch array on the current device (looked up once per device).
static void* static_scratch_addr(int* rc) {
    static void* addr[64] = {nullptr};
    int dev = 0;
    *rc = B200_OK;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        *rc = B200_ERR_LAUNCH;
        return nullptr;
    }
    if (addr[dev] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || p == nullptr) {
            *rc = B200_ERR_LAUNCH;
            return nullptr;
        }
        addr[dev] = p;
    }
    return addr[dev];
}

}  // namespace b200

extern "C" {

int b200_diag_fwd_static(int dtype, int64_t M, int64_t L, int64_t N, const void* lam, const void* v,
                         const void* x0, void* out, void* stream) {
    if (dtype != B200_F32 && dtype != B200_C64) return B200_ERR_ARG;
    if (M < 0 || L < 0 || N < 0) return B200_ERR_ARG;
    if (M == 0 || L == 0 || N == 0) return B200_OK;
    if (!lam || !v || !out) return B200_ERR_ARG;  // before any CUDA call, like the other entry points
    if (b200::workspace_bytes(dtype, false, false, M, L, N) > b200::kStaticScratchBytes) return B200_ERR_UNSUPPORTED;
    int rc = B200_OK;
    void* scratch = b200::static_scratch_addr(&rc);
    if (rc != B200_OK) return rc;
    b200::RunOpts opt;
    opt.mode = 1;  // the look-back kernel is the one whose state lives in the array
    return b200::run(dtype, false, false, M, L, N, lam, v, nullptr, x0, out, nullptr, nullptr, scratch,
                     b200::kStaticScratchBytes, stream, opt);
}

int b200_diag_static_status(void* stream) {
    int rc = B200_OK;
    void* scratch = b200::static_scratch_addr(&rc);
    if (rc != B200_OK) return rc;
    return b200_workspace_status(scratch, stream);
}

int b200_diag_probe(int mode, int vcap, int spin_limit, int64_t mute_tile, int dtype, int varying, int backward,
                    int64_t M, int64_t L, int64_t N, const void* lam, const void* val, const void* xsrc,
                    const void* x0, void* out, void* glam, void* gx0, void* workspace, size_t workspace_bytes,
                    void* stream) {
    if (mode < 0 || mode > 2 || spin_limit < 0) return B200_ERR_ARG;
    b200::RunOpts opt;
    opt.mode = mode;
    opt.vcap = vcap;
    if (spin_limit > 0) opt.spin_limit = spin_limit;
    opt.mute_tile = mute_tile;
    return b200::run(dtype, varying != 0, backward != 0, M, L, N, lam, val, xsrc, x0, out, glam, gx0, workspace,
                     workspace_bytes, stream, opt);
}

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
