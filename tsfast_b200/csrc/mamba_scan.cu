// Fused Mamba selective-scan section (S3), float32, forward and adjoint:
//   delta = softplus(draw);  h_t = exp(delta_t A) h_{t-1} + delta_t u_t B_t;
//   out_t = (h_t . C_t + Dp u_t) * z_t * sigmoid(z_t);  h_last = h_L.
// draw, u, z, out [B, L, D] (channel axis contiguous); A [D, N]; Bt, Ct [B, L, N]; Dp [D];
// h0, h_last [B, D, N].  Nothing [B, L, D, N]-sized ever touches HBM.
//
// Work split: one CTA owns one batch row and a block of DB channels for the whole sequence and
// walks time in tiles of kT steps.  A thread owns one channel and 4 of its N states (TPC threads
// per channel, neighbouring lanes), keeps them in registers and steps through time
// sequentially: the scan costs ONE exp per state and step, which is what bounds this kernel (the
// special-function unit, not HBM), so time is not split across threads (that would double the
// exps).  Per tile the raw inputs arrive through a cp.async ring (S-1 tiles in flight, every row
// a coalesced 128-byte segment), a cooperative pass turns draw into delta and z into the SiLU
// gate once per (t, d), then the state loop runs from shared memory and the gated outputs leave
// through a staging tile as coalesced 16-byte stores.
//
// Training: the forward also writes the state every kTB = 8 steps (chk [B, ceil(L/8), D, N], slot k =
// state after step 8(k+1) - 1), 1/8 of a full state store.  The adjoint walks the tiles in
// reverse: it recomputes the tile's 8 states per thread from the checkpoint into registers, then
// sweeps the tile backwards running G_t = gy_t C_t + lam_{t+1} G_{t+1} (the decays are evaluated
// again on the way back: two exps per state and step, which buys the registers/shared memory for
// four CTAs per SM, i.e. the whole grid of the benchmark shape in one wave).  Reductions over channels (grad_B, grad_C) are done in
// registers with a fixed reduce-scatter butterfly, across warps through shared memory and across
// channel blocks / batch rows through partial buffers summed in a fixed order: no atomics, so
// results are bitwise reproducible.
#include <initializer_list>

#include "common.cuh"

namespace b200 {

constexpr int kT = 16;       // steps per forward tile
constexpr int kTB = 8;       // checkpoint interval == steps per adjoint tile (its states live in registers)
constexpr int kNPT = 4;      // states per thread
constexpr float kLog2e = 1.4426950408889634f;

struct MambaArgs {
    const float *draw, *A, *Bt, *Ct, *u, *z, *Dp, *h0;
    float *out, *chk, *hlast;
    // adjoint only
    const float *gout, *ghlast;
    float *gdraw, *gu, *gz, *gh0;
    float *gA_part, *gDp_part, *gB_part, *gC_part;  // [B,D,N], [B,D], [ndb,B,L,N] x2
    long long B, L, D, N;
    long long ndb, NC, NCB;  // channel blocks per row, forward tiles, checkpoint slots (= adjoint tiles)
};

__device__ __forceinline__ void mcp16(void* smem_dst, const void* gsrc) {
    const unsigned int d = static_cast<unsigned int>(__cvta_generic_to_shared(smem_dst));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void mcp4(void* smem_dst, const void* gsrc) {
    const unsigned int d = static_cast<unsigned int>(__cvta_generic_to_shared(smem_dst));
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void mcp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void mcp_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ float ex2_fast(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// softplus with PyTorch's threshold (x > 20 -> x).  log1p(e) as a 6-term alternating series for
// e < 0.1 (truncation below 2e-7 relative) and log(1 + e) above, where rounding 1 + e costs at
// most 6e-7 relative: full float32 accuracy for two special-function ops.
__device__ __forceinline__ float softplus_f(float x) {
    // both branches are evaluated and selected (a warp nearly always holds inputs of both kinds)
    const float e = __expf(fminf(x, 20.f));
    float p = fmaf(e, -1.f / 6.f, 0.2f);
    p = fmaf(e, p, -0.25f);
    p = fmaf(e, p, 1.f / 3.f);
    p = fmaf(e, p, -0.5f);
    p = fmaf(e, p, 1.f);
    const float r = e < 0.1f ? e * p : __logf(1.f + e);
    return (x > 20.f || x != x) ? x : r;  // NaN passes through
}

// Sum v[0..G) over the TPC lanes of a channel group so that lane `ng` ends with the total of
// v[ng] in v[0] (G == TPC): log2(TPC) exchange steps moving G/2, G/4, ... values each.
template <int TPC>
__device__ __forceinline__ void group_reduce_scatter(float (&v)[TPC], int ng) {
#pragma unroll
    for (int off = TPC / 2; off >= 1; off >>= 1) {
        const bool upper = (ng & off) != 0;
#pragma unroll
        for (int i = 0; i < off; ++i) {
            const float send = upper ? v[i] : v[i + off];
            const float keep = upper ? v[i + off] : v[i];
            v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
        }
    }
}
__device__ __forceinline__ float sigmoid_f(float x) { return __fdividef(1.f, 1.f + __expf(-x)); }

// Copy a [rows x cols] float block (row pitch `pitch` in global memory, rows below `rows_live`
// and columns below `cols_live` only) into a dense [rows x ld] shared tile, cooperatively.
// VEC = 4 needs 16-byte aligned rows in both places and cols_live % 4 == 0.
template <int VEC, int NTHR>
__device__ __forceinline__ void copy_tile(float* dst, int ld, const float* src, long long pitch, int rows_live,
                                          int cols, int cols_live, int tid) {
    const int ppr = cols / VEC;  // pieces per row
    for (int e = tid; e < rows_live * ppr; e += NTHR) {
        const int r = e / ppr, c = (e - r * ppr) * VEC;
        if (c < cols_live) {
            if constexpr (VEC == 4) {
                mcp16(dst + r * ld + c, src + r * pitch + c);
            } else {
                mcp4(dst + r * ld + c, src + r * pitch + c);
            }
        }
    }
}

// Row pitch of the forward's [t][d] shared-memory tiles.  After a channel group's reduce-scatter
// lane `ng` of a channel works on step tg + ng, so the TPC lanes of a channel touch TPC consecutive
// rows at the same column; a pitch of 32/TPC (mod 32) words spreads those rows over distinct banks
// (the pad stays a multiple of 4 floats so that rows remain 16-byte copyable).
__host__ __device__ constexpr int mamba_ldd(int tpc, int db) { return tpc == 1 ? db : db + (32 / tpc > 4 ? 32 / tpc : 4); }

// ================================================================================ forward
template <int TPC, int DB, bool STORE_CHK, int VEC, int S>
__global__ void __launch_bounds__(DB* TPC) mamba_fwd_kernel(const MambaArgs p) {
    constexpr int NTHR = DB * TPC;
    constexpr int NPAD = kNPT * TPC;
    constexpr int LDD = mamba_ldd(TPC, DB);             // row pitch of the [t][d] tiles
    constexpr int STAGE = 3 * kT * LDD + 2 * kT * NPAD;  // floats per ring stage
    extern __shared__ __align__(16) float smem[];
    float* ring = smem;                  // [S][STAGE]
    float* outbuf = smem + S * STAGE;    // [2][kT][LDD]

    const int tid = threadIdx.x;
    const int dl = tid / TPC, ng = tid % TPC;
    const long long b = blockIdx.x / p.ndb;
    const long long d0 = (blockIdx.x - b * p.ndb) * DB;
    const long long d = d0 + dl;
    const int n0 = ng * kNPT;
    const long long L = p.L, D = p.D, N = p.N;
    const bool d_ok = d < D;
    const int dcols = (int)((D - d0) < DB ? (D - d0) : DB);

    for (int e = tid; e < S * STAGE + 2 * kT * LDD; e += NTHR) smem[e] = 0.f;  // pads must read as zero
    __syncthreads();

    // Whole tiles of a CTA whose rows are whole 16-byte pieces take a path with no index
    // arithmetic per tile: every thread copies the same pieces of every tile, so it keeps their
    // offsets (rows advance by 4 TPC per pass over the threads) and running tile offsets.
    const bool fastc = VEC == 4 && dcols == DB && N == NPAD;
    constexpr int PPR4 = DB / 4;                                // 16-byte pieces per [t][d] row
    constexpr int TD_PIECES = kT * PPR4, N_PIECES = kT * TPC;   // per tensor and tile
    constexpr int TD_PER = (TD_PIECES + NTHR - 1) / NTHR, N_PER = (N_PIECES + NTHR - 1) / NTHR;
    const int soff0 = (tid / PPR4) * LDD + (tid % PPR4) * 4;
    const long long goff0 = (long long)(tid / PPR4) * D + (tid % PPR4) * 4;
    const int soffn0 = (tid / TPC) * NPAD + (tid % TPC) * 4;
    const long long goffn0 = (long long)(tid / TPC) * N + (tid % TPC) * 4;
    long long ioff = b * L * D + d0, ioffn = b * L * N;  // next tile to fetch (tiles are fetched in order)
    long long ooff = b * L * D + d0;                     // next tile to store

    auto issue = [&](long long c, int slot) {
        const long long t0 = c * kT;
        const int rows = (int)((L - t0) < kT ? (L - t0) : kT);
        float* st = ring + slot * STAGE;
        if (fastc && rows == kT) {
#pragma unroll
            for (int j = 0; j < TD_PER; ++j) {
                if (TD_PIECES % NTHR == 0 || tid + j * NTHR < TD_PIECES) {
                    const long long g = ioff + goff0 + (long long)j * (4 * TPC) * D;
                    float* sd = st + soff0 + j * (4 * TPC) * LDD;
                    mcp16(sd, p.draw + g);
                    mcp16(sd + kT * LDD, p.u + g);
                    mcp16(sd + 2 * kT * LDD, p.z + g);
                }
            }
#pragma unroll
            for (int j = 0; j < N_PER; ++j) {
                if (N_PIECES % NTHR == 0 || tid + j * NTHR < N_PIECES) {
                    const long long g = ioffn + goffn0 + (long long)j * DB * N;
                    float* sd = st + 3 * kT * LDD + soffn0 + j * DB * NPAD;
                    mcp16(sd, p.Bt + g);
                    mcp16(sd + kT * NPAD, p.Ct + g);
                }
            }
            ioff += kT * D, ioffn += kT * N;
            return;
        }
        ioff += kT * D, ioffn += kT * N;
        const long long off = (b * L + t0) * D + d0;
        copy_tile<VEC, NTHR>(st, LDD, p.draw + off, D, rows, DB, dcols, tid);
        copy_tile<VEC, NTHR>(st + kT * LDD, LDD, p.u + off, D, rows, DB, dcols, tid);
        copy_tile<VEC, NTHR>(st + 2 * kT * LDD, LDD, p.z + off, D, rows, DB, dcols, tid);
        const long long offn = (b * L + t0) * N;
        copy_tile<VEC, NTHR>(st + 3 * kT * LDD, NPAD, p.Bt + offn, N, rows, NPAD, (int)N, tid);
        copy_tile<VEC, NTHR>(st + 3 * kT * LDD + kT * NPAD, NPAD, p.Ct + offn, N, rows, NPAD, (int)N, tid);
    };
    auto store_out = [&](long long c) {  // staged gated outputs of tile c -> global, coalesced
        const long long t0 = c * kT;
        const int rows = (int)((L - t0) < kT ? (L - t0) : kT);
        const float* ob = outbuf + (c & 1) * kT * LDD;
        if (fastc && rows == kT) {
#pragma unroll
            for (int j = 0; j < TD_PER; ++j) {
                if (TD_PIECES % NTHR == 0 || tid + j * NTHR < TD_PIECES) {
                    __stcs(reinterpret_cast<float4*>(p.out + ooff + goff0 + (long long)j * (4 * TPC) * D),
                           *reinterpret_cast<const float4*>(ob + soff0 + j * (4 * TPC) * LDD));
                }
            }
            ooff += kT * D;
            return;
        }
        ooff += kT * D;
        float* dst = p.out + (b * L + t0) * D + d0;
        constexpr int PPR = DB / VEC;
        for (int e = tid; e < rows * PPR; e += NTHR) {
            const int r = e / PPR, cc = (e - r * PPR) * VEC;
            if (cc < dcols) {
                if constexpr (VEC == 4) {
                    __stcs(reinterpret_cast<float4*>(dst + r * D + cc), *reinterpret_cast<const float4*>(ob + r * LDD + cc));
                } else {
                    __stcs(dst + r * D + cc, ob[r * LDD + cc]);
                }
            }
        }
    };

#pragma unroll
    for (int q = 0; q < S - 1; ++q) {
        if (q < p.NC) issue(q, q);
        mcp_commit();
    }

    float A2[kNPT], h[kNPT];
#pragma unroll
    for (int q = 0; q < kNPT; ++q) {
        const bool ok = d_ok && (n0 + q) < N;
        A2[q] = ok ? p.A[d * N + n0 + q] * kLog2e : 0.f;
        h[q] = (ok && p.h0 != nullptr) ? p.h0[(b * D + d) * N + n0 + q] : 0.f;
    }
    const float Dp = d_ok ? p.Dp[d] : 0.f;

    float* ckp = STORE_CHK ? p.chk + (b * p.NCB * D + d) * N + n0 : nullptr;  // next checkpoint slot
    int slot = 0, nslot = S - 1;  // stage of tile c and of the tile fetched while it is worked on
    for (long long c = 0; c < p.NC; ++c, slot = slot + 1 == S ? 0 : slot + 1, nslot = nslot + 1 == S ? 0 : nslot + 1) {
        float* st = ring + slot * STAGE;
        const int tlive = (int)((L - c * kT) < kT ? (L - c * kT) : kT);
        mcp_wait<S - 2>();
        __syncthreads();  // tile c has landed for everyone; tile c-1 is fully consumed and staged
        if (c + S - 1 < p.NC) issue(c + S - 1, nslot);
        mcp_commit();
        if (c > 0) store_out(c - 1);

        // once per (t, d): draw -> delta, z -> z * sigmoid(z)
        if (tlive == kT) {
#pragma unroll
            for (int j = 0; j < (kT * DB + NTHR - 1) / NTHR; ++j) {
                const int e = tid + j * NTHR;
                if ((kT * DB) % NTHR == 0 || e < kT * DB) {
                    const int o = (e / DB) * LDD + (e % DB);
                    st[o] = softplus_f(st[o]);
                    const float zz = st[2 * kT * LDD + o];
                    st[2 * kT * LDD + o] = zz * sigmoid_f(zz);
                }
            }
        } else {
            for (int e = tid; e < tlive * DB; e += NTHR) {
                const int o = (e / DB) * LDD + (e % DB);
                st[o] = softplus_f(st[o]);
                const float zz = st[2 * kT * LDD + o];
                st[2 * kT * LDD + o] = zz * sigmoid_f(zz);
            }
        }
        __syncthreads();

        float* ob = outbuf + (c & 1) * kT * LDD;
        const float* Bs = st + 3 * kT * LDD + n0;
        const float* Cs = Bs + kT * NPAD;
        // one time step of this thread's 4 states; returns its share of y_t = h_t . C_t
        auto state_step = [&](int t) -> float {
            const float delta = st[t * LDD + dl];
            const float du = delta * st[kT * LDD + t * LDD + dl];
            const float4 Bv = *reinterpret_cast<const float4*>(Bs + t * NPAD);
            const float4 Cv = *reinterpret_cast<const float4*>(Cs + t * NPAD);
            const float bq[kNPT] = {Bv.x, Bv.y, Bv.z, Bv.w}, cq[kNPT] = {Cv.x, Cv.y, Cv.z, Cv.w};
            float yp = 0.f;
#pragma unroll
            for (int q = 0; q < kNPT; ++q) {
                const float lam = ex2_fast(delta * A2[q]);
                h[q] = fmaf(lam, h[q], __fmul_rn(du, bq[q]));
                yp = fmaf(h[q], cq[q], yp);
            }
            return yp;
        };
        // gated output of step t for this thread's channel (kept in a register until the tile is
        // done: a shared-memory store inside the loop would pin every later load behind it)
        auto gated = [&](int t, float y) -> float {
            return (y + Dp * st[kT * LDD + t * LDD + dl]) * st[2 * kT * LDD + t * LDD + dl];
        };
        constexpr int G = (TPC >= 2 && TPC <= kT) ? TPC : 1;  // steps whose y sums are reduced together
        auto store_chk = [&](int t_done) {  // state after step t_done (tile-local) -> its checkpoint slot
            if constexpr (STORE_CHK) {
                if (d_ok) {
                    float* ck = ckp;  // slots are written in order, one every kTB steps
                    ckp += D * N;
                    if (VEC == 4 && n0 + kNPT <= N) {
                        *reinterpret_cast<float4*>(ck) = make_float4(h[0], h[1], h[2], h[3]);
                    } else {
#pragma unroll
                        for (int q = 0; q < kNPT; ++q)
                            if (n0 + q < N) ck[q] = h[q];
                    }
                }
            }
        };
        if (tlive == kT) {
            float yout[kT / G];
            float2 hp[2] = {make_float2(h[0], h[1]), make_float2(h[2], h[3])};
            const float2 A2p[2] = {make_float2(A2[0], A2[1]), make_float2(A2[2], A2[3])};
#pragma unroll
            for (int tg = 0; tg < kT; tg += G) {
                // decays and injections of the whole group first (independent work: G x 4 exps in
                // flight), then the short dependent chain through h
                // (sm_100 packed arithmetic: one instruction per PAIR of states)
                float2 lam[G][2], vin[G][2], cc[G][2];
#pragma unroll
                for (int k = 0; k < G; ++k) {
                    const int t = tg + k;
                    const float delta = st[t * LDD + dl];
                    const float du = delta * st[kT * LDD + t * LDD + dl];
                    const float4 Bv = *reinterpret_cast<const float4*>(Bs + t * NPAD);
                    const float4 Cv = *reinterpret_cast<const float4*>(Cs + t * NPAD);
                    cc[k][0] = make_float2(Cv.x, Cv.y), cc[k][1] = make_float2(Cv.z, Cv.w);
                    const float2 d2 = make_float2(delta, delta), du2 = make_float2(du, du);
                    const float2 e0 = __fmul2_rn(d2, A2p[0]), e1 = __fmul2_rn(d2, A2p[1]);
                    lam[k][0] = make_float2(ex2_fast(e0.x), ex2_fast(e0.y));
                    lam[k][1] = make_float2(ex2_fast(e1.x), ex2_fast(e1.y));
                    vin[k][0] = __fmul2_rn(du2, make_float2(Bv.x, Bv.y));
                    vin[k][1] = __fmul2_rn(du2, make_float2(Bv.z, Bv.w));
                }
                float yv[G];
#pragma unroll
                for (int k = 0; k < G; ++k) {
                    hp[0] = __ffma2_rn(lam[k][0], hp[0], vin[k][0]);
                    hp[1] = __ffma2_rn(lam[k][1], hp[1], vin[k][1]);
                    const float2 y2 = __ffma2_rn(hp[1], cc[k][1], __fmul2_rn(hp[0], cc[k][0]));
                    yv[k] = y2.x + y2.y;
                    if ((tg + k + 1) % kTB == 0) {
                        h[0] = hp[0].x, h[1] = hp[0].y, h[2] = hp[1].x, h[3] = hp[1].y;
                        store_chk(tg + k);
                    }
                }
                if constexpr (G > 1) {
                    group_reduce_scatter<G>(yv, ng);  // lane ng now owns step tg + ng
                    yout[tg / G] = gated(tg + ng, yv[0]);
                } else {
#pragma unroll
                    for (int off = 1; off < TPC; off <<= 1) yv[0] += __shfl_xor_sync(0xffffffffu, yv[0], off);
                    yout[tg / G] = gated(tg, yv[0]);
                }
            }
            h[0] = hp[0].x, h[1] = hp[0].y, h[2] = hp[1].x, h[3] = hp[1].y;
#pragma unroll
            for (int j = 0; j < kT / G; ++j) {
                if (G > 1 || ng == 0) ob[(j * G + (G > 1 ? ng : 0)) * LDD + dl] = yout[j];
            }
        } else {
            for (int t = 0; t < tlive; ++t) {
                float yp = state_step(t);
                if ((t + 1) % kTB == 0) store_chk(t);
#pragma unroll
                for (int off = 1; off < TPC; off <<= 1) yp += __shfl_xor_sync(0xffffffffu, yp, off);
                if (ng == 0) ob[t * LDD + dl] = gated(t, yp);
            }
        }
    }
    __syncthreads();
    if (p.NC > 0) store_out(p.NC - 1);
    mcp_wait<0>();
    if (d_ok) {
#pragma unroll
        for (int q = 0; q < kNPT; ++q)
            if (n0 + q < N) p.hlast[(b * D + d) * N + n0 + q] = h[q];
    }
}

// ================================================================================ adjoint
// One butterfly step of the channel reduction: lanes `OFF` apart exchange half of their CNT
// values and add, so the number of live values per lane halves (or, once a single value is
// left, plain exchange-and-add).  Upper lanes keep the upper half of the value indices.
template <int OFF, int CNT>
__device__ __forceinline__ void rs_step(float (&v)[8], int lane) {
    if constexpr (CNT > 1) {
        constexpr int H = CNT / 2;
        const bool upper = (lane & OFF) != 0;
#pragma unroll
        for (int i = 0; i < H; ++i) {
            const float send = upper ? v[i] : v[i + H];
            const float keep = upper ? v[i + H] : v[i];
            v[i] = keep + __shfl_xor_sync(0xffffffffu, send, OFF);
        }
    } else {
        v[0] += __shfl_xor_sync(0xffffffffu, v[0], OFF);
    }
}

template <int TPC, int DB, int VEC, int S>
__global__ void __launch_bounds__(DB* TPC, 4) mamba_bwd_kernel(const MambaArgs p) {
    constexpr int NTHR = DB * TPC;
    constexpr int NW = NTHR / 32;
    constexpr int NPAD = kNPT * TPC;
    constexpr int TD = kTB * DB;
    constexpr int STAGE = 4 * TD + 2 * kTB * NPAD + 4 * NTHR;  // draw,u,z,gout | Bt,Ct | checkpoint
    constexpr int G = (TPC >= 2 && TPC <= kTB) ? TPC : 1;       // steps whose channel sums are reduced together
    extern __shared__ __align__(16) float smem[];
    float* ring = smem;              // [S][STAGE]
    float* sigd = ring + S * STAGE;  // [kTB][DB]   sigmoid(draw)
    float* obuf = sigd + TD;         // [3][kTB][DB] staged gdraw, gu, gz
    float* red = obuf + 3 * TD;      // [NW][kTB][2][NPAD] per-warp grad_B / grad_C rows

    const int tid = threadIdx.x;
    const int lane = tid & 31, wid = tid >> 5;
    const int dl = tid / TPC, ng = tid % TPC;
    const long long b = blockIdx.x / p.ndb;
    const long long dblk = blockIdx.x - b * p.ndb;
    const long long d0 = dblk * DB;
    const long long d = d0 + dl;
    const int n0 = ng * kNPT;
    const long long L = p.L, D = p.D, N = p.N;
    const bool d_ok = d < D;
    const int dcols = (int)((D - d0) < DB ? (D - d0) : DB);

    for (int e = tid; e < S * STAGE + 4 * TD + NW * kTB * 2 * NPAD; e += NTHR) smem[e] = 0.f;
    __syncthreads();

    // Whole tiles of a CTA whose rows are whole 16-byte pieces take a path with no index
    // arithmetic per tile (same pieces for every tile, running offsets that step back one tile).
    const bool fastc = VEC == 4 && dcols == DB && N == NPAD;
    constexpr int PPR4 = DB / 4;
    constexpr int TD_PIECES = kTB * PPR4, N_PIECES = kTB * TPC;
    constexpr int TD_PER = (TD_PIECES + NTHR - 1) / NTHR, N_PER = (N_PIECES + NTHR - 1) / NTHR;
    const int soff0 = (tid / PPR4) * DB + (tid % PPR4) * 4;
    const long long goff0 = (long long)(tid / PPR4) * D + (tid % PPR4) * 4;
    const int soffn0 = (tid / TPC) * NPAD + (tid % TPC) * 4;
    const long long goffn0 = (long long)(tid / TPC) * N + (tid % TPC) * 4;
    // offsets of the next tile to fetch / to store (tiles are visited last to first, in order)
    long long ioff = (b * L + (p.NCB - 1) * kTB) * D + d0, ioffn = (b * L + (p.NCB - 1) * kTB) * N;
    long long ckoff = ((b * p.NCB + p.NCB - 2) * D + d) * N + n0;
    long long ooff = ioff, poff = ((dblk * p.B + b) * L + (p.NCB - 1) * kTB) * N;

    // tiles are visited from the last to the first: visit index i <-> tile c = NC-1-i
    auto issue = [&](long long c, int slot) {
        const long long t0 = c * kTB;
        const int rows = (int)((L - t0) < kTB ? (L - t0) : kTB);
        float* st = ring + slot * STAGE;
        if (fastc && rows == kTB) {
#pragma unroll
            for (int j = 0; j < TD_PER; ++j) {
                if (TD_PIECES % NTHR == 0 || tid + j * NTHR < TD_PIECES) {
                    const long long g = ioff + goff0 + (long long)j * (4 * TPC) * D;
                    float* sd = st + soff0 + j * (4 * TPC) * DB;
                    mcp16(sd, p.draw + g);
                    mcp16(sd + TD, p.u + g);
                    mcp16(sd + 2 * TD, p.z + g);
                    mcp16(sd + 3 * TD, p.gout + g);
                }
            }
#pragma unroll
            for (int j = 0; j < N_PER; ++j) {
                if (N_PIECES % NTHR == 0 || tid + j * NTHR < N_PIECES) {
                    const long long g = ioffn + goffn0 + (long long)j * DB * N;
                    float* sd = st + 4 * TD + soffn0 + j * DB * NPAD;
                    mcp16(sd, p.Bt + g);
                    mcp16(sd + kTB * NPAD, p.Ct + g);
                }
            }
            float* ck = st + 4 * TD + 2 * kTB * NPAD + 4 * tid;
            if (c > 0) {
                mcp16(ck, p.chk + ckoff);
            } else if (p.h0 != nullptr) {
                mcp16(ck, p.h0 + (b * D + d) * N + n0);
            }
            ioff -= kTB * D, ioffn -= kTB * N, ckoff -= D * N;
            return;
        }
        ioff -= kTB * D, ioffn -= kTB * N, ckoff -= D * N;
        const long long off = (b * L + t0) * D + d0;
        copy_tile<VEC, NTHR>(st, DB, p.draw + off, D, rows, DB, dcols, tid);
        copy_tile<VEC, NTHR>(st + TD, DB, p.u + off, D, rows, DB, dcols, tid);
        copy_tile<VEC, NTHR>(st + 2 * TD, DB, p.z + off, D, rows, DB, dcols, tid);
        copy_tile<VEC, NTHR>(st + 3 * TD, DB, p.gout + off, D, rows, DB, dcols, tid);
        const long long offn = (b * L + t0) * N;
        copy_tile<VEC, NTHR>(st + 4 * TD, NPAD, p.Bt + offn, N, rows, NPAD, (int)N, tid);
        copy_tile<VEC, NTHR>(st + 4 * TD + kTB * NPAD, NPAD, p.Ct + offn, N, rows, NPAD, (int)N, tid);
        // this thread's start state of the tile: checkpoint slot c-1, or h0 for the first tile
        float* ck = st + 4 * TD + 2 * kTB * NPAD + 4 * tid;
        const float* src = c > 0 ? p.chk + ((b * p.NCB + c - 1) * D + d) * N + n0
                                 : (p.h0 != nullptr ? p.h0 + (b * D + d) * N + n0 : nullptr);
        if (d_ok && src != nullptr) {
            if (VEC == 4 && n0 + kNPT <= N) {
                mcp16(ck, src);
            } else {
#pragma unroll
                for (int q = 0; q < kNPT; ++q)
                    if (n0 + q < N) mcp4(ck + q, src + q);
            }
        }
    };

#pragma unroll
    for (int q = 0; q < S - 1; ++q) {
        if (q < p.NCB) issue(p.NCB - 1 - q, q);
        mcp_commit();
    }

    float2 A1p[2], A2p[2], Gp[2], gAp[2], lamn[2];  // states in pairs: (n0, n0+1), (n0+2, n0+3)
    {
        float A1[kNPT], G0[kNPT];
#pragma unroll
        for (int q = 0; q < kNPT; ++q) {
            const bool ok = d_ok && (n0 + q) < N;
            A1[q] = ok ? p.A[d * N + n0 + q] : 0.f;
            G0[q] = (ok && p.ghlast != nullptr) ? p.ghlast[(b * D + d) * N + n0 + q] : 0.f;
        }
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            A1p[k] = make_float2(A1[2 * k], A1[2 * k + 1]);
            A2p[k] = make_float2(A1[2 * k] * kLog2e, A1[2 * k + 1] * kLog2e);
            Gp[k] = make_float2(G0[2 * k], G0[2 * k + 1]);
            gAp[k] = make_float2(0.f, 0.f);
            lamn[k] = make_float2(1.f, 1.f);  // passes ghlast into G_{L-1} unchanged
        }
    }
    const float Dp = d_ok ? p.Dp[d] : 0.f;
    float gDp = 0.f;
    const bool first_has_h0 = p.h0 != nullptr;

    int slot = 0, nslot = S - 1;  // stage of the tile worked on and of the tile fetched meanwhile
    for (long long i = 0; i < p.NCB; ++i, slot = slot + 1 == S ? 0 : slot + 1, nslot = nslot + 1 == S ? 0 : nslot + 1) {
        const long long c = p.NCB - 1 - i;
        float* st = ring + slot * STAGE;
        const int tlive = (int)((L - c * kTB) < kTB ? (L - c * kTB) : kTB);
        mcp_wait<S - 2>();
        __syncthreads();
        if (i + S - 1 < p.NCB) issue(p.NCB - 1 - (i + S - 1), nslot);
        mcp_commit();

        // once per (t, d): delta, sigmoid(draw), gy = gout*silu(z), gq = gout*d silu(z)/dz
        auto prep = [&](int e) {
            const float x = st[e];
            st[e] = softplus_f(x);
            sigd[e] = sigmoid_f(x);
            const float zz = st[2 * TD + e], go = st[3 * TD + e];
            const float sz = sigmoid_f(zz);
            st[2 * TD + e] = go * zz * sz;
            st[3 * TD + e] = go * sz * (1.f + zz * (1.f - sz));
        };
        if (tlive == kTB) {
#pragma unroll
            for (int j = 0; j < (TD + NTHR - 1) / NTHR; ++j) {
                if (TD % NTHR == 0 || tid + j * NTHR < TD) prep(tid + j * NTHR);
            }
        } else {
            for (int e = tid; e < tlive * DB; e += NTHR) prep(e);
        }
        __syncthreads();

        const float* Bs = st + 4 * TD + n0;
        const float* Cs = Bs + kTB * NPAD;
        // recompute the tile's states from its start state, kept in registers
        float2 hreg[kTB][2];
        {
            float h[kNPT];
            const float* ck = st + 4 * TD + 2 * kTB * NPAD + 4 * tid;
            const bool have = d_ok && (c > 0 || first_has_h0);
#pragma unroll
            for (int q = 0; q < kNPT; ++q) h[q] = (have && n0 + q < N) ? ck[q] : 0.f;
            float2 hp[2] = {make_float2(h[0], h[1]), make_float2(h[2], h[3])};
#pragma unroll
            for (int t = 0; t < kTB; ++t) {
                if (t < tlive) {
                    const float delta = st[t * DB + dl];
                    const float du = delta * st[TD + t * DB + dl];
                    const float4 Bv = *reinterpret_cast<const float4*>(Bs + t * NPAD);
                    const float2 d2 = make_float2(delta, delta), du2 = make_float2(du, du);
                    const float2 e0 = __fmul2_rn(d2, A2p[0]), e1 = __fmul2_rn(d2, A2p[1]);
                    hp[0] = __ffma2_rn(make_float2(ex2_fast(e0.x), ex2_fast(e0.y)), hp[0],
                                       __fmul2_rn(du2, make_float2(Bv.x, Bv.y)));
                    hp[1] = __ffma2_rn(make_float2(ex2_fast(e1.x), ex2_fast(e1.y)), hp[1],
                                       __fmul2_rn(du2, make_float2(Bv.z, Bv.w)));
                }
                hreg[t][0] = hp[0], hreg[t][1] = hp[1];
            }
        }

        // one step of the reverse sweep for this thread's 4 states: updates G, grad_A, the
        // per-warp grad_B / grad_C rows, and returns this thread's shares of y, grad_delta and the
        // B-weighted sum that goes into grad_u
        constexpr int CNT = TPC >= 32 ? 8 : (TPC == 16 ? 4 : (TPC == 8 ? 2 : 1));  // row values a lane ends up owning
        auto sweep_step = [&](int t, const float2 (&hv)[2], float& yp, float& gdp, float& gus, float (&rv)[CNT]) {
            const float delta = st[t * DB + dl];
            const float uu = st[TD + t * DB + dl];
            const float gy = st[2 * TD + t * DB + dl];
            const float du = delta * uu;
            const float4 Bv = *reinterpret_cast<const float4*>(Bs + t * NPAD);
            const float4 Cv = *reinterpret_cast<const float4*>(Cs + t * NPAD);
            const float2 b2[2] = {make_float2(Bv.x, Bv.y), make_float2(Bv.z, Bv.w)};
            const float2 c2[2] = {make_float2(Cv.x, Cv.y), make_float2(Cv.z, Cv.w)};
            const float2 gy2 = make_float2(gy, gy), du2 = make_float2(du, du);
            const float2 d2 = make_float2(delta, delta);
            float2 y2 = make_float2(0.f, 0.f), gd2 = y2, gu2 = y2;
            float vals[8];
#pragma unroll
            for (int k = 0; k < 2; ++k) {  // one pass per PAIR of states (sm_100 packed arithmetic)
                y2 = __ffma2_rn(hv[k], c2[k], y2);
                Gp[k] = __ffma2_rn(lamn[k], Gp[k], __fmul2_rn(gy2, c2[k]));
                // lam_t h_{t-1} = h_t - v_t, with v_t rounded exactly as in the recurrence (so 0 stays 0)
                // (scalar on purpose: the packed multiply-then-add may be contracted into one fma)
                const float2 lhp = make_float2(__fsub_rn(hv[k].x, __fmul_rn(du, b2[k].x)),
                                               __fsub_rn(hv[k].y, __fmul_rn(du, b2[k].y)));
                const float2 gb = __fmul2_rn(Gp[k], du2);   // grad_B contribution
                const float2 gc = __fmul2_rn(gy2, hv[k]);   // grad_C contribution
                vals[2 * k] = gb.x, vals[2 * k + 1] = gb.y;
                vals[4 + 2 * k] = gc.x, vals[4 + 2 * k + 1] = gc.y;
                const float2 P = __fmul2_rn(Gp[k], lhp);
                gAp[k] = __ffma2_rn(P, d2, gAp[k]);
                gd2 = __ffma2_rn(A1p[k], P, gd2);  // grad_delta = sum A (G lam h_prev) + u sum G B
                gu2 = __ffma2_rn(Gp[k], b2[k], gu2);
                const float2 e = __fmul2_rn(d2, A2p[k]);
                lamn[k] = make_float2(ex2_fast(e.x), ex2_fast(e.y));  // lam_t, needed by the step before
            }
            yp = y2.x + y2.y;
            gus = gu2.x + gu2.y;
            gdp = fmaf(uu, gus, gd2.x + gd2.y);
            // sum the 8 values over the channels of this warp; lanes end up owning distinct rows
            if constexpr (TPC <= 16) rs_step<16, 8>(vals, lane);
            if constexpr (TPC <= 8) rs_step<8, 4>(vals, lane);
            if constexpr (TPC <= 4) rs_step<4, 2>(vals, lane);
            if constexpr (TPC <= 2) rs_step<2, 1>(vals, lane);
            if constexpr (TPC <= 1) rs_step<1, 1>(vals, lane);
#pragma unroll
            for (int k = 0; k < CNT; ++k) rv[k] = vals[k];
        };
        // finish the per-(t, d) gradients of step t from the channel-group sums
        auto finish = [&](int t, float y_sum, float gd_sum, float gu_sum, float (&o)[3]) {
            const float delta = st[t * DB + dl];
            const float uu = st[TD + t * DB + dl];
            const float gy = st[2 * TD + t * DB + dl];
            o[0] = gd_sum * sigd[t * DB + dl];
            o[1] = fmaf(delta, gu_sum, gy * Dp);
            o[2] = st[3 * TD + t * DB + dl] * fmaf(Dp, uu, y_sum);
            gDp = fmaf(gy, uu, gDp);
        };

        // Results stay in registers until the sweep is over: a shared-memory store inside the
        // unrolled loop would keep the loads of later steps from being scheduled ahead of it.
        float redv[kTB][CNT];      // this lane's grad_B / grad_C row values per step
        float outv[kTB / G][3];    // gdraw, gu, gz of the steps this lane finishes
#pragma unroll
        for (int tg = kTB - G; tg >= 0; tg -= G) {
            float yv[G], gdv[G], guv[G];
#pragma unroll
            for (int k = G - 1; k >= 0; --k) {
                yv[k] = 0.f, gdv[k] = 0.f, guv[k] = 0.f;
                if (tg + k < tlive) sweep_step(tg + k, hreg[tg + k], yv[k], gdv[k], guv[k], redv[tg + k]);
            }
            if (tg < tlive) {
                if constexpr (G > 1) {
                    group_reduce_scatter<G>(yv, ng);  // lane ng now owns step tg + ng
                    group_reduce_scatter<G>(gdv, ng);
                    group_reduce_scatter<G>(guv, ng);
                    if (tg + ng < tlive) finish(tg + ng, yv[0], gdv[0], guv[0], outv[tg / G]);
                } else {
#pragma unroll
                    for (int off = 1; off < TPC; off <<= 1) {
                        yv[0] += __shfl_xor_sync(0xffffffffu, yv[0], off);
                        gdv[0] += __shfl_xor_sync(0xffffffffu, gdv[0], off);
                        guv[0] += __shfl_xor_sync(0xffffffffu, guv[0], off);
                    }
                    if (ng == 0) finish(tg, yv[0], gdv[0], guv[0], outv[tg / G]);
                }
            }
        }
        {
            int base = 0;  // index of the first row value this lane owns after the channel reduction
            if (TPC <= 16) base += (lane & 16) ? 4 : 0;
            if (TPC <= 8) base += (lane & 8) ? 2 : 0;
            if (TPC <= 4) base += (lane & 4) ? 1 : 0;
            const bool writer = TPC > 2 || (TPC == 2 ? (lane & 2) == 0 : (lane & 3) == 0);
#pragma unroll
            for (int t = 0; t < kTB; ++t) {
                if (writer && t < tlive) {
                    float* r = red + (wid * kTB + t) * 2 * NPAD;
#pragma unroll
                    for (int k = 0; k < CNT; ++k) {
                        const int idx = base + k;
                        r[(idx >> 2) * NPAD + n0 + (idx & 3)] = redv[t][k];
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < kTB / G; ++j) {
                const int t = j * G + (G > 1 ? ng : 0);
                if ((G > 1 || ng == 0) && t < tlive) {
                    obuf[t * DB + dl] = outv[j][0];
                    obuf[TD + t * DB + dl] = outv[j][1];
                    obuf[2 * TD + t * DB + dl] = outv[j][2];
                }
            }
        }
        __syncthreads();

        // staged per-(t,d) gradients -> global; per-warp grad_B/grad_C rows -> this block's partial
        if (fastc && tlive == kTB) {
#pragma unroll
            for (int j = 0; j < TD_PER; ++j) {
                if (TD_PIECES % NTHR == 0 || tid + j * NTHR < TD_PIECES) {
                    const long long g = ooff + goff0 + (long long)j * (4 * TPC) * D;
                    const float* ob = obuf + soff0 + j * (4 * TPC) * DB;
                    __stcs(reinterpret_cast<float4*>(p.gdraw + g), *reinterpret_cast<const float4*>(ob));
                    __stcs(reinterpret_cast<float4*>(p.gu + g), *reinterpret_cast<const float4*>(ob + TD));
                    __stcs(reinterpret_cast<float4*>(p.gz + g), *reinterpret_cast<const float4*>(ob + 2 * TD));
                }
            }
            // per-warp grad_B / grad_C rows -> this block's partial: element e = (t, which, n)
#pragma unroll
            for (int j = 0; j < (kTB * 2 * NPAD + NTHR - 1) / NTHR; ++j) {
                const int e = tid + j * NTHR;
                if ((kTB * 2 * NPAD) % NTHR == 0 || e < kTB * 2 * NPAD) {
                    const int t = e / (2 * NPAD), rem = e % (2 * NPAD);
                    float sacc = 0.f;
#pragma unroll
                    for (int ww = 0; ww < NW; ++ww) sacc += red[(ww * kTB + t) * 2 * NPAD + rem];
                    float* dst = rem < NPAD ? p.gB_part : p.gC_part;
                    dst[poff + t * NPAD + (rem % NPAD)] = sacc;
                }
            }
        } else {
            const long long t0 = c * kTB;
            constexpr int PPR = DB / VEC;
            float* dsts[3] = {p.gdraw, p.gu, p.gz};
#pragma unroll
            for (int k = 0; k < 3; ++k) {
                float* dst = dsts[k] + (b * L + t0) * D + d0;
                const float* ob = obuf + k * TD;
                for (int e = tid; e < tlive * PPR; e += NTHR) {
                    const int r = e / PPR, cc = (e - r * PPR) * VEC;
                    if (cc < dcols) {
                        if constexpr (VEC == 4) {
                            __stcs(reinterpret_cast<float4*>(dst + r * D + cc),
                                   *reinterpret_cast<const float4*>(ob + r * DB + cc));
                        } else {
                            __stcs(dst + r * D + cc, ob[r * DB + cc]);
                        }
                    }
                }
            }
            for (int e = tid; e < tlive * 2 * NPAD; e += NTHR) {
                const int t = e / (2 * NPAD), rem = e - t * 2 * NPAD;
                const int which = rem / NPAD, n = rem - which * NPAD;
                if (n < N) {
                    float sacc = 0.f;
#pragma unroll
                    for (int ww = 0; ww < NW; ++ww) sacc += red[(ww * kTB + t) * 2 * NPAD + rem];
                    float* dst = which == 0 ? p.gB_part : p.gC_part;
                    dst[((dblk * p.B + b) * L + t0 + t) * N + n] = sacc;
                }
            }
        }
        ooff -= kTB * D, poff -= kTB * N;
        // the next iteration's first barrier orders these reads before obuf/red are rewritten
    }
    mcp_wait<0>();

    // grad_Dp: every lane of a channel group summed the steps it finished
#pragma unroll
    for (int off = 1; off < TPC; off <<= 1) gDp += __shfl_xor_sync(0xffffffffu, gDp, off);
    if (d_ok) {
#pragma unroll
        for (int q = 0; q < kNPT; ++q) {
            if (n0 + q < N) {
                const float2 ga = gAp[q >> 1], gg = Gp[q >> 1], ll = lamn[q >> 1];
                p.gA_part[(b * D + d) * N + n0 + q] = (q & 1) ? ga.y : ga.x;
                if (p.gh0 != nullptr) p.gh0[(b * D + d) * N + n0 + q] = (q & 1) ? ll.y * gg.y : ll.x * gg.x;
            }
        }
        if (ng == 0) p.gDp_part[b * D + d] = gDp;
    }
}

// out[i] = sum_k in[k * stride + i], k ascending (fixed order)
__global__ void sum_leading_kernel(const float* __restrict__ in, float* __restrict__ out, long long count,
                                   long long stride, int K) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    float s = 0.f;
    for (int k = 0; k < K; ++k) s += in[k * stride + i];
    out[i] = s;
}

// ------------------------------------------------------------------------------- host side
#ifndef MAMBA_FWD_S
#define MAMBA_FWD_S 4  // ring stages of the forward
#endif
#ifndef MAMBA_BWD_S
#define MAMBA_BWD_S 3  // ring stages of the adjoint
#endif
#ifndef MAMBA_THREADS
#define MAMBA_THREADS 128  // threads per CTA (fewer when the state dimension is small enough)
#endif
// channels per CTA: MAMBA_THREADS / TPC, at least 4 so that rows stay 16-byte copyable
constexpr int mamba_db(int tpc) { return MAMBA_THREADS / tpc > 4 ? MAMBA_THREADS / tpc : 4; }

static int tpc_for(long long N) {  // threads per channel: 4 states each, power of two
    int t = 1;
    while ((long long)t * kNPT < N) t *= 2;
    return t;
}

template <typename K>
static int set_smem(K kern, size_t bytes, bool* configured) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) != cudaSuccess)
            return B200_ERR_LAUNCH;
        configured[dev] = true;
    }
    return B200_OK;
}

template <int TPC, bool STORE_CHK, int VEC>
static int launch_mamba_fwd(const MambaArgs& a, cudaStream_t st) {
    constexpr int DB = mamba_db(TPC), S = MAMBA_FWD_S, NTHR = DB * TPC;
    constexpr int LDD = mamba_ldd(TPC, DB);
    constexpr size_t smem = sizeof(float) * ((size_t)S * (3 * kT * LDD + 2 * kT * kNPT * TPC) + 2 * kT * LDD);
    auto kern = mamba_fwd_kernel<TPC, DB, STORE_CHK, VEC, S>;
    static bool configured[64] = {false};
    if (set_smem(kern, smem, configured) != B200_OK) return B200_ERR_LAUNCH;
    MambaArgs p = a;
    p.ndb = (a.D + DB - 1) / DB;
    const long long grid = a.B * p.ndb;
    if (grid > 0x7fffffffLL) return B200_ERR_UNSUPPORTED;
    kern<<<(unsigned int)grid, NTHR, smem, st>>>(p);
    return cudaGetLastError() == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

template <int TPC, int VEC>
static int launch_mamba_bwd(const MambaArgs& a, cudaStream_t st) {
    constexpr int DB = mamba_db(TPC), S = MAMBA_BWD_S, NPAD = kNPT * TPC, NTHR = DB * TPC, NW = NTHR / 32;
    constexpr size_t smem = sizeof(float) * ((size_t)S * (4 * kTB * DB + 2 * kTB * NPAD + 4 * NTHR) +
                                             4 * kTB * DB + NW * kTB * 2 * NPAD);
    auto kern = mamba_bwd_kernel<TPC, DB, VEC, S>;
    static bool configured[64] = {false};
    if (set_smem(kern, smem, configured) != B200_OK) return B200_ERR_LAUNCH;
    const long long grid = a.B * a.ndb;
    if (grid > 0x7fffffffLL) return B200_ERR_UNSUPPORTED;
    kern<<<(unsigned int)grid, NTHR, smem, st>>>(a);
    return cudaGetLastError() == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

#define B200_TPC_SWITCH(tpc, CALL)    \
    switch (tpc) {                    \
        case 1: return CALL(1);       \
        case 2: return CALL(2);       \
        case 4: return CALL(4);       \
        case 8: return CALL(8);       \
        case 16: return CALL(16);     \
        case 32: return CALL(32);     \
        default: return B200_ERR_UNSUPPORTED; \
    }

static int dispatch_mamba_fwd(int tpc, bool chk, bool vec, const MambaArgs& a, cudaStream_t st) {
    if (chk && vec) {
#define CALL(T) launch_mamba_fwd<T, true, 4>(a, st)
        B200_TPC_SWITCH(tpc, CALL)
#undef CALL
    } else if (chk) {
#define CALL(T) launch_mamba_fwd<T, true, 1>(a, st)
        B200_TPC_SWITCH(tpc, CALL)
#undef CALL
    } else if (vec) {
#define CALL(T) launch_mamba_fwd<T, false, 4>(a, st)
        B200_TPC_SWITCH(tpc, CALL)
#undef CALL
    } else {
#define CALL(T) launch_mamba_fwd<T, false, 1>(a, st)
        B200_TPC_SWITCH(tpc, CALL)
#undef CALL
    }
}

static int dispatch_mamba_bwd(int tpc, bool vec, const MambaArgs& a, cudaStream_t st) {
    if (vec) {
#define CALL(T) launch_mamba_bwd<T, 4>(a, st)
        B200_TPC_SWITCH(tpc, CALL)
#undef CALL
    } else {
#define CALL(T) launch_mamba_bwd<T, 1>(a, st)
        B200_TPC_SWITCH(tpc, CALL)
#undef CALL
    }
}

struct MambaWs {
    size_t off_gA, off_gDp, off_gB, off_gC, total;
    long long ndb;
};

static MambaWs mamba_ws(long long B, long long L, long long D, long long N) {
    MambaWs w;
    const int DB = mamba_db(tpc_for(N));
    w.ndb = (D + DB - 1) / DB;
    size_t off = 0;
    w.off_gA = off;
    off += align_up(sizeof(float) * (size_t)(B * D * N), 256);
    w.off_gDp = off;
    off += align_up(sizeof(float) * (size_t)(B * D), 256);
    w.off_gB = off;
    off += align_up(sizeof(float) * (size_t)(w.ndb * B * L * N), 256);
    w.off_gC = off;
    off += align_up(sizeof(float) * (size_t)(w.ndb * B * L * N), 256);
    w.total = off;
    return w;
}

static int sum_leading(const float* in, float* out, long long count, long long stride, long long K, cudaStream_t st) {
    if (count == 0) return B200_OK;
    const long long blocks = (count + 255) / 256;
    if (blocks > 0x7fffffffLL || K > 0x7fffffffLL) return B200_ERR_UNSUPPORTED;
    sum_leading_kernel<<<(unsigned int)blocks, 256, 0, st>>>(in, out, count, stride, (int)K);
    return cudaGetLastError() == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

static bool aligned16(std::initializer_list<const void*> ps) {
    for (const void* q : ps)
        if (((uintptr_t)q & 15) != 0) return false;
    return true;
}

}  // namespace b200

extern "C" {

int b200_mamba_chk_interval(void) { return b200::kTB; }

int b200_mamba_fwd(int64_t B, int64_t L, int64_t D, int64_t N, const void* draw, const void* A, const void* Bt,
                   const void* Ct, const void* u, const void* z, const void* Dp, const void* h0, void* out,
                   void* hlast, void* chk, void* stream) {
    using namespace b200;
    if (B < 0 || L < 0 || D < 0 || N < 1) return B200_ERR_ARG;
    if (N > 128) return B200_ERR_UNSUPPORTED;
    if (B == 0 || D == 0) return B200_OK;
    if (!A || !Dp || !hlast || (L > 0 && (!draw || !Bt || !Ct || !u || !z || !out))) return B200_ERR_ARG;
    MambaArgs a = {};
    a.draw = (const float*)draw, a.A = (const float*)A, a.Bt = (const float*)Bt, a.Ct = (const float*)Ct;
    a.u = (const float*)u, a.z = (const float*)z, a.Dp = (const float*)Dp, a.h0 = (const float*)h0;
    a.out = (float*)out, a.chk = (float*)chk, a.hlast = (float*)hlast;
    a.B = B, a.L = L, a.D = D, a.N = N;
    a.NC = (L + kT - 1) / kT;
    a.NCB = (L + kTB - 1) / kTB;
    const bool vec = D % 4 == 0 && N % 4 == 0 && aligned16({draw, Bt, Ct, u, z, out, chk});
    return dispatch_mamba_fwd(tpc_for(N), chk != nullptr, vec, a, static_cast<cudaStream_t>(stream));
}

size_t b200_mamba_bwd_workspace_bytes(int64_t B, int64_t L, int64_t D, int64_t N) {
    if (B <= 0 || L < 0 || D <= 0 || N < 1 || N > 128) return 256;
    const size_t t = b200::mamba_ws(B, L, D, N).total;
    return t ? t : 256;
}

int b200_mamba_bwd(int64_t B, int64_t L, int64_t D, int64_t N, const void* draw, const void* A, const void* Bt,
                   const void* Ct, const void* u, const void* z, const void* Dp, const void* h0, const void* chk,
                   const void* gout, const void* ghlast, void* gdraw, void* gA, void* gBt, void* gCt, void* gu,
                   void* gz, void* gDp, void* gh0, void* workspace, size_t workspace_bytes, void* stream) {
    using namespace b200;
    if (B < 0 || L < 0 || D < 0 || N < 1) return B200_ERR_ARG;
    if (N > 128) return B200_ERR_UNSUPPORTED;
    if (B == 0 || D == 0) return B200_OK;
    if (!A || !Dp || !gA || !gDp || (h0 && !gh0)) return B200_ERR_ARG;
    if (L > 0 && (!draw || !Bt || !Ct || !u || !z || !gout || !gdraw || !gBt || !gCt || !gu || !gz)) return B200_ERR_ARG;
    if (L > kTB && !chk) return B200_ERR_ARG;
    const MambaWs w = mamba_ws(B, L, D, N);
    if (!workspace || ((uintptr_t)workspace % 256) != 0 || workspace_bytes < w.total) return B200_ERR_WORKSPACE;
    char* base = static_cast<char*>(workspace);
    MambaArgs a = {};
    a.draw = (const float*)draw, a.A = (const float*)A, a.Bt = (const float*)Bt, a.Ct = (const float*)Ct;
    a.u = (const float*)u, a.z = (const float*)z, a.Dp = (const float*)Dp, a.h0 = (const float*)h0;
    a.chk = (float*)chk;
    a.gout = (const float*)gout, a.ghlast = (const float*)ghlast;
    a.gdraw = (float*)gdraw, a.gu = (float*)gu, a.gz = (float*)gz, a.gh0 = h0 ? (float*)gh0 : nullptr;
    a.gA_part = (float*)(base + w.off_gA), a.gDp_part = (float*)(base + w.off_gDp);
    a.gB_part = (float*)(base + w.off_gB), a.gC_part = (float*)(base + w.off_gC);
    a.B = B, a.L = L, a.D = D, a.N = N;
    a.ndb = w.ndb;
    a.NC = (L + kT - 1) / kT;
    a.NCB = (L + kTB - 1) / kTB;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool vec = D % 4 == 0 && N % 4 == 0 && aligned16({draw, Bt, Ct, u, z, gout, chk, h0, gdraw, gu, gz});
    int rc = dispatch_mamba_bwd(tpc_for(N), vec, a, st);
    if (rc != B200_OK) return rc;
    // fixed-order reductions of the partial buffers
    if ((rc = sum_leading(a.gA_part, (float*)gA, D * N, D * N, B, st)) != B200_OK) return rc;
    if ((rc = sum_leading(a.gDp_part, (float*)gDp, D, D, B, st)) != B200_OK) return rc;
    if ((rc = sum_leading(a.gB_part, (float*)gBt, B * L * N, B * L * N, w.ndb, st)) != B200_OK) return rc;
    return sum_leading(a.gC_part, (float*)gCt, B * L * N, B * L * N, w.ndb, st);
}

}  // extern "C"
