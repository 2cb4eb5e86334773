// Causal depthwise convolution + SiLU of the Mamba block, forward and adjoint, float32:
//   out[b,t,d] = silu(bias[d] + sum_{k<K} w[d,k] * X(b, t-(K-1)+k, d)),
//   X(s) = x[b,s,d] for s >= 0 and tail[b,d,s+K-1] for s < 0 (the carried left context).
// x is channel-last [B, L, D] with unit channel stride and arbitrary batch/time strides (the
// in_proj chunk view is read in place), tail [B, D, K-1], w [D, K], bias [D] or null; out dense.
//
// There is no recurrence, only a K-tap window along time, so the kernels are pure streams: a tile
// is one batch row, a segment of time steps and 128*VEC channels; a thread owns VEC neighbouring
// channels (one 8- or 16-byte access per row) and walks the segment in time with the last K-1
// inputs in registers, so every input row is read once (plus a K-1 row halo per segment) and every
// output row written once.  Rows are requested in batches, two batches alternating so that one is
// in flight while the other is worked on; full segments run without range checks (only a ragged
// last segment takes the checked path), pointers walk row by row.
// The adjoint recomputes the pre-activation (cheaper than saving it), forms
// gpre = gy * silu'(pre), emits gx[s] = sum_k w_k gpre[s+K-1-k] from a K-deep register window (a
// segment first runs the K-1 steps before it for their gpre and emits rows K-1 behind its own
// steps; the first segment's first K-1 rows are the tail gradient), and accumulates the weight and
// bias gradients per thread.  Its grid is persistent, so those stay in registers over all tiles of
// a CTA and are reduced through one partial per CTA, added in a fixed order.  No atomics.
#include <initializer_list>
#include <type_traits>

#include "common.cuh"

namespace b200 {

#ifndef CONV_SEGT
#define CONV_SEGT 64
#endif
#ifndef CONV_SEGB
#define CONV_SEGB 32
#endif
constexpr int kSegT = CONV_SEGT;  // time steps per forward CTA
constexpr int kSegB = CONV_SEGB;  // time steps per tile of the (persistent) adjoint
constexpr int kConvThreads = 128;
// Rows a thread requests per batch (two batches alternate, one in flight while the other is worked
// on) and the widest per-thread channel vector, per direction.  The adjoint keeps about 25
// registers per channel (weights, their gradients, two windows); 8-byte vectors fit twice the CTAs
// per SM and measured faster than 16-byte ones in both directions.
#ifndef CONV_FWD_U
#define CONV_FWD_U 8
#endif
#ifndef CONV_BWD_U
#define CONV_BWD_U 8
#endif
#ifndef CONV_BWD_CTAS
#define CONV_BWD_CTAS 4  // resident adjoint CTAs per SM (bounds its registers) = persistent CTAs per SM
#endif
#ifndef CONV_EDGE_U
#define CONV_EDGE_U 4
#endif
constexpr int kEdgeU = CONV_EDGE_U;  // rows per batch on the checked path of a ragged last segment
#ifndef CONV_FWD_VEC
#define CONV_FWD_VEC 2
#endif
#ifndef CONV_BWD_VEC
#define CONV_BWD_VEC 2
#endif

struct ConvArgs {
    const float* x;
    long long sxb, sxl;  // element strides of x along batch and time (channel stride is 1)
    const float *tail, *w, *bias;
    float* out;
    const float* gy;  // adjoint
    float *gx, *gtail, *gw_part, *gb_part;
    long long B, L, D;
    long long nseg, ndblk, ntiles;  // segments per sequence, channel blocks, tiles of the adjoint (B * nseg * ndblk)
};

template <int VEC>
struct VecT;
template <>
struct VecT<1> {
    float v[1];
};
template <>
struct alignas(8) VecT<2> {
    float v[2];
};
template <>
struct alignas(16) VecT<4> {
    float v[4];
};

template <int VEC>
__device__ __forceinline__ VecT<VEC> ldv(const float* p) {
    VecT<VEC> r;
    if constexpr (VEC == 4) {
        const float4 t = __ldcs(reinterpret_cast<const float4*>(p));
        r.v[0] = t.x, r.v[1] = t.y, r.v[2] = t.z, r.v[3] = t.w;
    } else if constexpr (VEC == 2) {
        const float2 t = __ldcs(reinterpret_cast<const float2*>(p));
        r.v[0] = t.x, r.v[1] = t.y;
    } else {
        r.v[0] = __ldcs(p);
    }
    return r;
}
template <int VEC>
__device__ __forceinline__ void stv(float* p, const VecT<VEC>& r) {
    if constexpr (VEC == 4) {
        __stcs(reinterpret_cast<float4*>(p), make_float4(r.v[0], r.v[1], r.v[2], r.v[3]));
    } else if constexpr (VEC == 2) {
        __stcs(reinterpret_cast<float2*>(p), make_float2(r.v[0], r.v[1]));
    } else {
        __stcs(p, r.v[0]);
    }
}

__device__ __forceinline__ float sigmoid_fast(float x) { return __fdividef(1.f, 1.f + __expf(-x)); }

// X(b, s, d..d+VEC): the virtual buffer cat(tail, x); zero outside [-(K-1), L)
template <int K, int VEC>
__device__ __forceinline__ VecT<VEC> load_x(const ConvArgs& p, long long b, long long s, long long d, bool d_ok) {
    VecT<VEC> r;
#pragma unroll
    for (int q = 0; q < VEC; ++q) r.v[q] = 0.f;
    if (!d_ok || s >= p.L || s < -(K - 1)) return r;
    if (s >= 0) return ldv<VEC>(p.x + b * p.sxb + s * p.sxl + d);
#pragma unroll
    for (int q = 0; q < VEC; ++q) r.v[q] = p.tail[(b * p.D + d + q) * (K - 1) + s + K - 1];
    return r;
}

// One output row of the forward: the pre-activation from the K-1 earlier rows in `win` and the
// current row, SiLU, and the window moves on (register renaming once the caller is unrolled).
template <int K, int VEC>
__device__ __forceinline__ VecT<VEC> conv_fwd_step(const float (&wgt)[K][VEC], const float (&bs)[VEC],
                                                   VecT<VEC> (&win)[K - 1 > 0 ? K - 1 : 1], const VecT<VEC>& cur) {
    VecT<VEC> o;
#pragma unroll
    for (int q = 0; q < VEC; ++q) {
        float pre = fmaf(wgt[K - 1][q], cur.v[q], bs[q]);
#pragma unroll
        for (int k = 0; k < K - 1; ++k) pre = fmaf(wgt[k][q], win[k].v[q], pre);
        o.v[q] = pre * sigmoid_fast(pre);
    }
#pragma unroll
    for (int k = 0; k + 1 < K - 1; ++k) win[k] = win[k + 1];
    if (K > 1) win[K - 2 > 0 ? K - 2 : 0] = cur;
    return o;
}

template <int K, int VEC>
__global__ void __launch_bounds__(kConvThreads) conv_silu_fwd_kernel(const ConvArgs p) {
    constexpr int kUnroll = CONV_FWD_U;
    long long bid = blockIdx.x;
    const long long dblk = bid % p.ndblk;
    bid /= p.ndblk;
    const long long seg = bid % p.nseg, b = bid / p.nseg;
    const long long d = (dblk * kConvThreads + threadIdx.x) * VEC;
    const bool d_ok = d < p.D;
    const long long t0 = seg * kSegT, t1 = (t0 + kSegT < p.L) ? t0 + kSegT : p.L;

    float wgt[K][VEC], bs[VEC];
#pragma unroll
    for (int q = 0; q < VEC; ++q) {
        bs[q] = (d_ok && p.bias != nullptr) ? p.bias[d + q] : 0.f;
#pragma unroll
        for (int k = 0; k < K; ++k) wgt[k][q] = d_ok ? p.w[(d + q) * K + k] : 0.f;
    }
    static_assert(kSegT % (2 * kUnroll) == 0, "whole pairs of batches per segment");
    VecT<VEC> win[K - 1 > 0 ? K - 1 : 1];  // X(t-K+1) .. X(t-1)

    // A full segment runs without range checks, tail lookups or per-row index arithmetic (this
    // kernel is bound by instruction issue and load latency, not by arithmetic): two row batches in
    // flight alternately, pointers walked row by row, and the last batch requests nothing beyond
    // the segment.  Only its K-1 context rows are looked up (the carried tail, for the first segment).
    if (t0 + kSegT <= p.L) {
        if (!d_ok) return;
        const long long sxl = p.sxl, sD = p.D;
        const float* xp = p.x + b * p.sxb + d + t0 * sxl;
        float* op = p.out + (b * p.L + t0) * p.D + d;
        if (t0 >= K - 1) {
#pragma unroll
            for (int i = 0; i < K - 1; ++i) win[i] = ldv<VEC>(xp + (i - (K - 1)) * sxl);
        } else {
#pragma unroll
            for (int i = 0; i < K - 1; ++i) win[i] = load_x<K, VEC>(p, b, t0 - (K - 1) + i, d, true);
        }
        VecT<VEC> ra[kUnroll], rb[kUnroll];
        auto fetch = [&](VecT<VEC>(&r)[kUnroll]) {
#pragma unroll
            for (int i = 0; i < kUnroll; ++i, xp += sxl) r[i] = ldv<VEC>(xp);
        };
        auto work = [&](const VecT<VEC>(&r)[kUnroll]) {
#pragma unroll
            for (int i = 0; i < kUnroll; ++i, op += sD) stv<VEC>(op, conv_fwd_step<K, VEC>(wgt, bs, win, r[i]));
        };
        fetch(ra);
        for (int it = 0; it < kSegT / (2 * kUnroll) - 1; ++it) {
            fetch(rb);
            work(ra);
            fetch(ra);
            work(rb);
        }
        fetch(rb);
        work(ra);
        work(rb);
        return;
    }

    // a ragged last segment
#pragma unroll
    for (int i = 0; i < K - 1; ++i) win[i] = load_x<K, VEC>(p, b, t0 - (K - 1) + i, d, d_ok);
    float* orow = p.out + b * p.L * p.D + d;  // row t of out at orow + t * D
    for (long long tb = t0; tb < t1; tb += kEdgeU) {
        VecT<VEC> cur[kEdgeU];
#pragma unroll
        for (int i = 0; i < kEdgeU; ++i) cur[i] = load_x<K, VEC>(p, b, tb + i, d, d_ok && tb + i < t1);
#pragma unroll
        for (int i = 0; i < kEdgeU; ++i) {
            if (tb + i < t1) {
                const VecT<VEC> o = conv_fwd_step<K, VEC>(wgt, bs, win, cur[i]);
                if (d_ok) stv<VEC>(orow + (tb + i) * p.D, o);
            }
        }
    }
}

// One step t of the adjoint: the window takes row X(t), the pre-activation is recomputed,
// gpre(t) = gy(t) * silu'(pre) enters the gradient window, the weight and bias gradients take
// their terms when the step is the segment's own, and gx(t-K+1) = sum_k w_k gpre(t-k) comes back.
template <int K, int VEC, bool OWN>
__device__ __forceinline__ VecT<VEC> conv_bwd_step(const float (&wgt)[K][VEC], const float (&bs)[VEC], VecT<VEC> (&win)[K],
                                                   float (&gwin)[K][VEC], float (&gw)[K][VEC], float (&gb)[VEC],
                                                   const VecT<VEC>& xrow, const VecT<VEC>& gyrow, bool live, bool own) {
#pragma unroll
    for (int k = 0; k < K - 1; ++k) win[k] = win[k + 1];
    win[K - 1] = xrow;
    VecT<VEC> gxo;
#pragma unroll
    for (int q = 0; q < VEC; ++q) {
        float pre = bs[q];
#pragma unroll
        for (int k = 0; k < K; ++k) pre = fmaf(wgt[k][q], win[k].v[q], pre);
        const float sg = sigmoid_fast(pre);
        float gp = gyrow.v[q] * sg * fmaf(pre, 1.f - sg, 1.f);
        if (!OWN) gp = live ? gp : 0.f;
#pragma unroll
        for (int k = K - 1; k > 0; --k) gwin[k][q] = gwin[k - 1][q];
        gwin[0][q] = gp;
        if (OWN || own) {
            gb[q] += gp;
#pragma unroll
            for (int k = 0; k < K; ++k) gw[k][q] = fmaf(gp, win[k].v[q], gw[k][q]);
        }
        float acc = wgt[0][q] * gwin[0][q];
#pragma unroll
        for (int k = 1; k < K; ++k) acc = fmaf(wgt[k][q], gwin[k][q], acc);
        gxo.v[q] = acc;
    }
    return gxo;
}

// A segment of the adjoint owns the weight / bias terms of its steps [t0, t1) and the input
// gradients gx[t0-(K-1), t1-(K-1)) (the last segment also the final K-1 rows): gx(s) needs
// gpre(s .. s+K-1), so a segment first runs the K-1 steps before t0 for their gpre alone and then
// every own step emits the row K-1 behind it.
//
// The grid is persistent: a few CTAs per SM, each walking the (batch, segment) tiles of ONE channel
// block in a fixed stride, so the last wave is not a partial one (segments are short for that),
// the weights are read once per CTA, and the weight / bias gradients stay in registers across the
// tiles: one partial per CTA instead of one per tile.
template <int K, int VEC, bool HAS_BIAS>
__global__ void __launch_bounds__(kConvThreads, CONV_BWD_CTAS) conv_silu_bwd_kernel(const ConvArgs p) {
    constexpr int kUnroll = CONV_BWD_U, kSeg = kSegB;
    static_assert(kSeg % (2 * kUnroll) == 0, "whole pairs of batches per segment");
    const long long dblk = blockIdx.x % p.ndblk;  // the grid is a multiple of ndblk: constant over this CTA's tiles
    const long long d = (dblk * kConvThreads + threadIdx.x) * VEC;
    if (d >= p.D) return;  // no barriers in this kernel

    float wgt[K][VEC], bs[VEC], gw[K][VEC], gb[VEC];
#pragma unroll
    for (int q = 0; q < VEC; ++q) {
        bs[q] = p.bias != nullptr ? p.bias[d + q] : 0.f;
        gb[q] = 0.f;
#pragma unroll
        for (int k = 0; k < K; ++k) wgt[k][q] = p.w[(d + q) * K + k], gw[k][q] = 0.f;
    }
    const long long sxl = p.sxl, sD = p.D;

    for (long long tile = blockIdx.x; tile < p.ntiles; tile += gridDim.x) {
        const long long rest = tile / p.ndblk;
        const long long seg = rest % p.nseg, b = rest / p.nseg;
        const long long t0 = seg * kSeg, t1 = (t0 + kSeg < p.L) ? t0 + kSeg : p.L;
        float gwin[K][VEC];  // gwin[j] = gpre[t - j]
#pragma unroll
        for (int q = 0; q < VEC; ++q)
#pragma unroll
            for (int k = 0; k < K; ++k) gwin[k][q] = 0.f;
        VecT<VEC> win[K];  // X(t-K+1) .. X(t)

        // A full segment runs without range checks or per-row index arithmetic: two row batches in flight alternately, pointers walked row by row, every own
        // step unconditional.  In the first segment the context is the carried tail (no gpre
        // before the sequence), and its first K-1 emitted rows, gx(-(K-1)) .. gx(-1), are the
        // gradient of that tail.
        if (t0 + kSeg <= p.L) {
            auto fast = [&](auto first_tag) {
                constexpr bool FIRST = decltype(first_tag)::value;
                const float* xp = p.x + b * p.sxb + d + t0 * sxl;
                const float* gyp = p.gy + (b * p.L + t0) * sD + d;
                float* gxp = p.gx + (b * p.L + t0) * sD + d - (K - 1) * sD;  // row t0 - (K-1): written from row 0 on only
                VecT<VEC> cx[2 * (K - 1)], cg[K - 1];  // context rows, all requested before the first use
#pragma unroll
                for (int i = 0; i < 2 * (K - 1); ++i) {
                    if constexpr (FIRST) cx[i] = load_x<K, VEC>(p, b, i - 2 * (K - 1), d, true);
                    else cx[i] = ldv<VEC>(xp + (i - 2 * (K - 1)) * sxl);
                }
#pragma unroll
                for (int i = 0; i < K - 1; ++i) {
                    if constexpr (FIRST) cg[i] = cx[0];  // unused: no gpre before the sequence
                    else cg[i] = ldv<VEC>(gyp + (i - (K - 1)) * sD);
                }
                VecT<VEC> xa[kUnroll], ga[kUnroll], xb[kUnroll], gbb[kUnroll];
                auto fetch = [&](VecT<VEC>(&xr)[kUnroll], VecT<VEC>(&gr)[kUnroll]) {
#pragma unroll
                    for (int i = 0; i < kUnroll; ++i, xp += sxl, gyp += sD) xr[i] = ldv<VEC>(xp), gr[i] = ldv<VEC>(gyp);
                };
                int n = 0;  // own steps done
                auto work = [&](const VecT<VEC>(&xr)[kUnroll], const VecT<VEC>(&gr)[kUnroll]) {
#pragma unroll
                    for (int i = 0; i < kUnroll; ++i, gxp += sD, ++n) {
                        const VecT<VEC> gxo = conv_bwd_step<K, VEC, true>(wgt, bs, win, gwin, gw, gb, xr[i], gr[i], true, true);
                        if (FIRST && n < K - 1) {
#pragma unroll
                            for (int q = 0; q < VEC; ++q) p.gtail[(b * p.D + d + q) * (K - 1) + n] = gxo.v[q];
                        } else {
                            stv<VEC>(gxp, gxo);
                        }
                    }
                };
                fetch(xa, ga);
#pragma unroll
                for (int i = 0; i < K - 1; ++i) win[i + 1] = cx[i];
#pragma unroll
                for (int i = 0; i < K - 1; ++i)
                    (void)conv_bwd_step<K, VEC, false>(wgt, bs, win, gwin, gw, gb, cx[K - 1 + i], cg[i], !FIRST, false);
                for (int it = 0; it < kSeg / (2 * kUnroll) - 1; ++it) {
                    fetch(xb, gbb);
                    work(xa, ga);
                    fetch(xa, ga);
                    work(xb, gbb);
                }
                fetch(xb, gbb);
                work(xa, ga);
                work(xb, gbb);
                if (t0 + kSeg == p.L) {  // the last segment: the final K-1 rows, from zero gpre beyond the end
                    VecT<VEC> zero;
#pragma unroll
                    for (int q = 0; q < VEC; ++q) zero.v[q] = 0.f;
#pragma unroll
                    for (int i = 0; i < K - 1; ++i, gxp += sD)
                        stv<VEC>(gxp, conv_bwd_step<K, VEC, false>(wgt, bs, win, gwin, gw, gb, zero, zero, false, false));
                }
            };
            if (t0 == 0) fast(std::true_type{});
            else fast(std::false_type{});
            continue;
        }

        // a ragged last segment (it also emits the final K-1 rows from zero gpre beyond the end;
        // when it is the first one too, the tail gradient comes from its first K-1 steps)
        float gfirst[K - 1 > 0 ? K - 1 : 1][VEC];
#pragma unroll
        for (int q = 0; q < VEC; ++q)
#pragma unroll
            for (int k = 0; k < K - 1; ++k) gfirst[k][q] = 0.f;
#pragma unroll
        for (int i = 0; i < K - 1; ++i) win[i + 1] = load_x<K, VEC>(p, b, t0 - 2 * (K - 1) + i, d, true);
        const long long tend = (t1 == p.L) ? t1 + (K - 1) : t1;
        const float* gyrow = p.gy + b * p.L * p.D + d;  // row t of gy / gx at + t * D
        float* gxrow = p.gx + b * p.L * p.D + d;
        for (long long tb = t0 - (K - 1); tb < tend; tb += kEdgeU) {
            VecT<VEC> cur[kEdgeU], gyv[kEdgeU];
#pragma unroll
            for (int i = 0; i < kEdgeU; ++i) {
                const long long t = tb + i;
                cur[i] = load_x<K, VEC>(p, b, t, d, t < tend);
#pragma unroll
                for (int q = 0; q < VEC; ++q) gyv[i].v[q] = 0.f;
                if (t >= 0 && t < p.L && t < tend) gyv[i] = ldv<VEC>(gyrow + t * p.D);
            }
#pragma unroll
            for (int i = 0; i < kEdgeU; ++i) {
                const long long t = tb + i;
                if (t < tend) {
                    const VecT<VEC> gxo = conv_bwd_step<K, VEC, false>(wgt, bs, win, gwin, gw, gb, cur[i], gyv[i],
                                                                       t >= 0 && t < p.L, t >= t0 && t < t1);
                    if (K > 1 && seg == 0) {
#pragma unroll
                        for (int k = 0; k < K - 1; ++k)
                            if (t == k) {
#pragma unroll
                                for (int q = 0; q < VEC; ++q) gfirst[k][q] = gwin[0][q];
                            }
                    }
                    const long long s_ = t - (K - 1);
                    if (s_ >= 0 && s_ >= t0 - (K - 1)) stv<VEC>(gxrow + s_ * p.D, gxo);
                }
            }
        }
        if (seg == 0) {  // gtail[j] = sum_{k<=j} w_k gpre[j-k]
#pragma unroll
            for (int q = 0; q < VEC; ++q)
#pragma unroll
                for (int j = 0; j < K - 1; ++j) {
                    float acc = 0.f;
#pragma unroll
                    for (int k = 0; k < K - 1; ++k)
                        if (k <= j) acc = fmaf(wgt[k][q], gfirst[j - k][q], acc);
                    p.gtail[(b * p.D + d + q) * (K - 1) + j] = acc;
                }
        }
    }
    const long long part = blockIdx.x / p.ndblk;
#pragma unroll
    for (int q = 0; q < VEC; ++q) {
#pragma unroll
        for (int k = 0; k < K; ++k) p.gw_part[(part * p.D + d + q) * K + k] = gw[k][q];
        if constexpr (HAS_BIAS) p.gb_part[part * p.D + d + q] = gb[q];
    }
}

// The partial weight and bias gradients, one set per CTA of the adjoint, added in a fixed order
// (reproducible): outputs [0, cw) are weight taps (partials cw apart), [cw, cw + cb) bias entries
// (partials cb apart).  32 lanes per output each add every 32nd partial, eight independent loads
// per round, then the 32 sub-sums are added in lane order; 32 outputs per block keep the reads of
// one partial coalesced.
__global__ void __launch_bounds__(1024) conv_sum_parts_kernel(const float* __restrict__ w_parts, const float* __restrict__ b_parts,
                                                              float* __restrict__ gw, float* __restrict__ gb, long long cw,
                                                              long long cb, int parts) {
    __shared__ float sh[32][33];
    const int o = threadIdx.x & 31, pl = threadIdx.x >> 5;
    long long i = (long long)blockIdx.x * 32 + o;
    const bool live = i < cw + cb;
    const bool is_w = i < cw;
    const float* in = is_w ? w_parts : b_parts;
    const long long stride = is_w ? cw : cb;
    if (!is_w) i -= cw;
    float s = 0.f;
    if (live) {
        int k = pl;
        for (; k + 224 < parts; k += 256) {
            float v[8];
#pragma unroll
            for (int r = 0; r < 8; ++r) v[r] = in[(k + 32 * r) * stride + i];
#pragma unroll
            for (int r = 0; r < 8; ++r) s += v[r];
        }
        for (; k < parts; k += 32) s += in[k * stride + i];
    }
    sh[pl][o] = s;
    __syncthreads();
    if (pl == 0 && live) {
        float t = 0.f;
#pragma unroll
        for (int q = 0; q < 32; ++q) t += sh[q][o];
        (is_w ? gw : gb)[i] = t;
    }
}

constexpr long long kMaxParts = 4096;  // >= resident adjoint CTAs of any GPU this runs on (SMs x CONV_BWD_CTAS)
static size_t conv_parts_bound(long long B, long long L) {
    const long long tiles = B * ((L + kSegB - 1) / kSegB);
    return (size_t)(tiles < kMaxParts ? tiles : kMaxParts);
}

static int conv_sm_count() {
    static int cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

// CTAs of the adjoint: every resident slot of the GPU, rounded down to whole channel-block groups
// (a CTA keeps one channel block), never more than there are tiles.
static long long conv_bwd_grid(const ConvArgs& a) {
    long long g = (long long)conv_sm_count() * CONV_BWD_CTAS;
    if (g > kMaxParts) g = kMaxParts;  // the workspace holds at most kMaxParts partial sets
    g -= g % a.ndblk;
    if (g < a.ndblk) g = a.ndblk;
    return g < a.ntiles ? g : a.ntiles;
}

template <int K, int VEC>
static int launch_conv(bool bwd, bool has_bias, const ConvArgs& a, cudaStream_t st) {
    const long long grid = bwd ? conv_bwd_grid(a) : a.B * a.nseg * a.ndblk;
    if (grid > 0x7fffffffLL) return B200_ERR_UNSUPPORTED;
    if (!bwd) {
        conv_silu_fwd_kernel<K, VEC><<<(unsigned int)grid, kConvThreads, 0, st>>>(a);
    } else if (has_bias) {
        conv_silu_bwd_kernel<K, VEC, true><<<(unsigned int)grid, kConvThreads, 0, st>>>(a);
    } else {
        conv_silu_bwd_kernel<K, VEC, false><<<(unsigned int)grid, kConvThreads, 0, st>>>(a);
    }
    return cudaGetLastError() == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

template <int VEC>
static int dispatch_conv_k(int K, bool bwd, bool has_bias, const ConvArgs& a, cudaStream_t st) {
    switch (K) {
        case 2: return launch_conv<2, VEC>(bwd, has_bias, a, st);
        case 3: return launch_conv<3, VEC>(bwd, has_bias, a, st);
        case 4: return launch_conv<4, VEC>(bwd, has_bias, a, st);
        case 5: return launch_conv<5, VEC>(bwd, has_bias, a, st);
        case 6: return launch_conv<6, VEC>(bwd, has_bias, a, st);
        case 7: return launch_conv<7, VEC>(bwd, has_bias, a, st);
        case 8: return launch_conv<8, VEC>(bwd, has_bias, a, st);
        default: return B200_ERR_UNSUPPORTED;
    }
}

// widest channel vector (4, 2 or 1 floats, at most `want`) that D, the strides and the pointers allow
static int conv_vec(int want, long long D, long long sxb, long long sxl, std::initializer_list<const void*> ps) {
    for (int v = want; v > 1; v /= 2) {
        bool ok = D % v == 0 && sxb % v == 0 && sxl % v == 0;
        for (const void* q : ps)
            if (((uintptr_t)q & (uintptr_t)(4 * v - 1)) != 0) ok = false;
        if (ok) return v;
    }
    return 1;
}

template <bool BWD>
static int dispatch_conv(int vec, int K, bool has_bias, const ConvArgs& a, cudaStream_t st) {
    switch (vec) {
        case 4: return dispatch_conv_k<4>(K, BWD, has_bias, a, st);
        case 2: return dispatch_conv_k<2>(K, BWD, has_bias, a, st);
        default: return dispatch_conv_k<1>(K, BWD, has_bias, a, st);
    }
}

static void conv_shape(ConvArgs& a, int vec, int seg) {
    a.nseg = (a.L + seg - 1) / seg;
    a.ndblk = (a.D + (long long)kConvThreads * vec - 1) / ((long long)kConvThreads * vec);
    a.ntiles = a.B * a.nseg * a.ndblk;
}

}  // namespace b200

extern "C" {

int b200_conv_silu_fwd(int64_t B, int64_t L, int64_t D, int64_t K, const void* x, int64_t x_stride_b,
                       int64_t x_stride_l, const void* tail, const void* w, const void* bias, void* out,
                       void* stream) {
    using namespace b200;
    if (B < 0 || L < 0 || D < 0) return B200_ERR_ARG;
    if (K < 2 || K > 8) return B200_ERR_UNSUPPORTED;
    if (B == 0 || L == 0 || D == 0) return B200_OK;
    if (!x || !tail || !w || !out) return B200_ERR_ARG;
    ConvArgs a = {};
    a.x = (const float*)x, a.sxb = x_stride_b, a.sxl = x_stride_l;
    a.tail = (const float*)tail, a.w = (const float*)w, a.bias = (const float*)bias, a.out = (float*)out;
    a.B = B, a.L = L, a.D = D;
    const int vec = conv_vec(CONV_FWD_VEC, D, x_stride_b, x_stride_l, {x, out});
    conv_shape(a, vec, kSegT);
    return dispatch_conv<false>(vec, (int)K, bias != nullptr, a, static_cast<cudaStream_t>(stream));
}

size_t b200_conv_silu_bwd_workspace_bytes(int64_t B, int64_t L, int64_t D, int64_t K) {
    if (B <= 0 || L <= 0 || D <= 0 || K < 2 || K > 8) return 256;
    // one partial set per CTA group of the adjoint: at most one per (batch, segment), and no more
    // than kMaxParts (the grid never exceeds the GPU's resident CTAs)
    const size_t parts = b200::conv_parts_bound(B, L);
    return b200::align_up(parts * D * K * sizeof(float), 256) + b200::align_up(parts * D * sizeof(float), 256);
}

int b200_conv_silu_bwd(int64_t B, int64_t L, int64_t D, int64_t K, const void* gy, const void* x,
                       int64_t x_stride_b, int64_t x_stride_l, const void* tail, const void* w,
                       const void* bias, void* gx, void* gtail, void* gw, void* gb, void* workspace,
                       size_t workspace_bytes, void* stream) {
    using namespace b200;
    if (B < 0 || L < 0 || D < 0) return B200_ERR_ARG;
    if (K < 2 || K > 8) return B200_ERR_UNSUPPORTED;
    if (B == 0 || L == 0 || D == 0) return B200_OK;
    if (!gy || !x || !tail || !w || !gx || !gtail || !gw || (bias && !gb)) return B200_ERR_ARG;
    if (!workspace || ((uintptr_t)workspace % 256) != 0 ||
        workspace_bytes < b200_conv_silu_bwd_workspace_bytes(B, L, D, K))
        return B200_ERR_WORKSPACE;
    ConvArgs a = {};
    a.x = (const float*)x, a.sxb = x_stride_b, a.sxl = x_stride_l;
    a.tail = (const float*)tail, a.w = (const float*)w, a.bias = (const float*)bias;
    a.gy = (const float*)gy, a.gx = (float*)gx, a.gtail = (float*)gtail;
    a.B = B, a.L = L, a.D = D;
    const int vec = conv_vec(CONV_BWD_VEC, D, x_stride_b, x_stride_l, {x, gy, gx});
    conv_shape(a, vec, kSegB);
    const size_t bound = conv_parts_bound(B, L);
    a.gw_part = (float*)workspace;
    a.gb_part = (float*)((char*)workspace + align_up(bound * D * K * sizeof(float), 256));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int rc = dispatch_conv<true>(vec, (int)K, bias != nullptr, a, st);
    if (rc != B200_OK) return rc;
    const long long parts = conv_bwd_grid(a) / a.ndblk;  // partial sets written: one per CTA group
    const long long cw = D * K, cb = bias ? D : 0;
    conv_sum_parts_kernel<<<(unsigned int)((cw + cb + 31) / 32), 1024, 0, st>>>(a.gw_part, a.gb_part, (float*)gw, (float*)gb, cw, cb,
                                                                              (int)parts);
    return cudaGetLastError() == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

}  // extern "C"
