// Causal depthwise convolution + SiLU of the Mamba block, forward and adjoint, float32:
//   out[b,t,d] = silu(bias[d] + sum_{k<K} w[d,k] * X(b, t-(K-1)+k, d)),
//   X(s) = x[b,s,d] for s >= 0 and tail[b,d,s+K-1] for s < 0 (the carried left context).
// x is channel-last [B, L, D] with unit channel stride and arbitrary batch/time strides (the
// in_proj chunk view is read in place), tail [B, D, K-1], w [D, K], bias [D] or null; out dense.
//
// There is no recurrence, only a K-tap window along time, so the kernel is a pure stream: a CTA
// owns one batch row, a segment of kSegT steps and 128*VEC channels; a thread owns VEC
// neighbouring channels (one 8- or 16-byte access per row) and walks its segment in time
// with the last K-1 inputs in registers, so every input row is read once (plus a K-1 row halo per
// segment) and every output row written once.  Rows are loaded in batches, the next batch requested before the current one is used.
// The adjoint recomputes the pre-activation (cheaper than saving it), forms
// gpre = gy * silu'(pre), emits gx[s] = sum_k w_k gpre[s+K-1-k] from a K-deep register window
// (each segment runs K-1 steps into the next one for that), and accumulates the weight and bias
// gradients per thread; those are reduced over (batch, segment) through partial buffers added in
// a fixed order, and the K-1 tail gradients come from the first segment.  No atomics.
#include <initializer_list>
#include <type_traits>

#include "common.cuh"

namespace b200 {

#ifndef CONV_SEGT
#define CONV_SEGT 64
#endif
constexpr int kSegT = CONV_SEGT;  // time steps per CTA segment
constexpr int kConvThreads = 128;
// Rows a thread loads per batch and the widest per-thread channel vector, per direction.  The
// adjoint keeps about 25 registers per channel (weights, their gradients, two windows); 8-byte
// vectors fit twice the CTAs per SM and measured faster than 16-byte ones in both directions
// (B=32, L=2048, D=512, K=4: forward 4.4 -> 4.9 TB/s, adjoint 2.2 -> 3.8 TB/s together with the
// prefetch of the next batch, the check-free interior path and the wider partial-sum kernel).
#ifndef CONV_FWD_U
#define CONV_FWD_U 8
#endif
#ifndef CONV_BWD_U
#define CONV_BWD_U 8
#endif
#ifndef CONV_FWD_PIPE
#define CONV_FWD_PIPE 1  // request the next batch of rows before working on the current one
#endif
#ifndef CONV_BWD_PIPE
#define CONV_BWD_PIPE 1
#endif
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
    long long nseg, ndblk;
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
    // A segment whose rows (left context and prefetch included) all lie inside the sequence takes
    // the same loop without range checks, tail lookups or per-row index arithmetic: this kernel is
    // bound by instruction issue, not by memory, and the checks were half of its instructions.
    static_assert(kSegT % kUnroll == 0, "whole batches per segment");
    const bool interior = t0 >= K - 1 && t0 + kSegT + kUnroll <= p.L;
    const float* xrow = p.x + b * p.sxb + d;   // row s of x at xrow + s * sxl
    float* orow = p.out + b * p.L * p.D + d;   // row t of out at orow + t * D
    auto body = [&](auto tag) {
        constexpr bool IN = decltype(tag)::value;
        auto row = [&](long long sidx, bool ok) -> VecT<VEC> {
            if constexpr (IN) return ldv<VEC>(xrow + sidx * p.sxl);
            else return load_x<K, VEC>(p, b, sidx, d, ok);
        };
        VecT<VEC> win[K - 1 > 0 ? K - 1 : 1];  // X(t-K+1) .. X(t-1)
#pragma unroll
        for (int i = 0; i < K - 1; ++i) win[i] = row(t0 - (K - 1) + i, d_ok);

        // rows of the next batch are requested before the current batch is worked on
        VecT<VEC> nxt[kUnroll];
        if constexpr (CONV_FWD_PIPE) {
#pragma unroll
            for (int i = 0; i < kUnroll; ++i) nxt[i] = row(t0 + i, d_ok && t0 + i < t1);
        }
        for (long long tb = t0; tb < t1; tb += kUnroll) {
            VecT<VEC> cur[kUnroll];
            if constexpr (CONV_FWD_PIPE) {
#pragma unroll
                for (int i = 0; i < kUnroll; ++i) cur[i] = nxt[i];
#pragma unroll
                for (int i = 0; i < kUnroll; ++i) nxt[i] = row(tb + kUnroll + i, d_ok && tb + kUnroll + i < t1);
            } else {
#pragma unroll
                for (int i = 0; i < kUnroll; ++i) cur[i] = row(tb + i, d_ok && tb + i < t1);
            }
#pragma unroll
            for (int i = 0; i < kUnroll; ++i) {
                if (IN || tb + i < t1) {
                    VecT<VEC> o;
#pragma unroll
                    for (int q = 0; q < VEC; ++q) {
                        float pre = fmaf(wgt[K - 1][q], cur[i].v[q], bs[q]);
#pragma unroll
                        for (int k = 0; k < K - 1; ++k) pre = fmaf(wgt[k][q], win[k].v[q], pre);
                        o.v[q] = pre * sigmoid_fast(pre);
                    }
                    if (IN || d_ok) stv<VEC>(orow + (tb + i) * p.D, o);
#pragma unroll
                    for (int k = 0; k + 1 < K - 1; ++k) win[k] = win[k + 1];
                    if (K > 1) win[K - 2 > 0 ? K - 2 : 0] = cur[i];
                }
            }
        }
    };
    if (interior) {
        if (d_ok) body(std::true_type{});
    } else {
        body(std::false_type{});
    }
}

template <int K, int VEC, bool HAS_BIAS>
__global__ void __launch_bounds__(kConvThreads) conv_silu_bwd_kernel(const ConvArgs p) {
    constexpr int kUnroll = CONV_BWD_U;
    long long bid = blockIdx.x;
    const long long dblk = bid % p.ndblk;
    bid /= p.ndblk;
    const long long seg = bid % p.nseg, b = bid / p.nseg;
    const long long d = (dblk * kConvThreads + threadIdx.x) * VEC;
    const bool d_ok = d < p.D;
    const long long t0 = seg * kSegT, t1 = (t0 + kSegT < p.L) ? t0 + kSegT : p.L;
    const long long tend = t1 + (K - 1);  // K-1 steps into the next segment: their gpre feeds this segment's gx

    float wgt[K][VEC], bs[VEC], gw[K][VEC], gb[VEC], gwin[K][VEC], gfirst[K - 1 > 0 ? K - 1 : 1][VEC];
#pragma unroll
    for (int q = 0; q < VEC; ++q) {
        bs[q] = (d_ok && p.bias != nullptr) ? p.bias[d + q] : 0.f;
        gb[q] = 0.f;
#pragma unroll
        for (int k = 0; k < K; ++k) {
            wgt[k][q] = d_ok ? p.w[(d + q) * K + k] : 0.f;
            gw[k][q] = 0.f;
            gwin[k][q] = 0.f;  // gwin[j] = gpre[t - j]
        }
#pragma unroll
        for (int k = 0; k < K - 1; ++k) gfirst[k][q] = 0.f;
    }
    // Segments whose rows (context, the K-1 steps into the next segment and the prefetch) all lie
    // inside the sequence run the same loop without range checks or per-row index arithmetic.
    const bool interior = t0 >= K - 1 && t0 + kSegT + (K - 1) + 2 * kUnroll <= p.L;
    const float* xrow = p.x + b * p.sxb + d;      // row s of x at xrow + s * sxl
    const float* gyrow = p.gy + b * p.L * p.D + d;  // row t of gy / gx at + t * D
    float* gxrow = p.gx + b * p.L * p.D + d;
    auto body = [&](auto tag) {
    constexpr bool IN = decltype(tag)::value;
    VecT<VEC> win[K];  // X(t-K+1) .. X(t)
#pragma unroll
    for (int i = 0; i < K - 1; ++i) {
        if constexpr (IN) win[i + 1] = ldv<VEC>(xrow + (t0 - (K - 1) + i) * p.sxl);
        else win[i + 1] = load_x<K, VEC>(p, b, t0 - (K - 1) + i, d, d_ok);
    }

    // rows of the next batch are requested before the current batch is worked on
    VecT<VEC> nx[kUnroll], ngy[kUnroll];
    auto fetch = [&](long long tb) {
#pragma unroll
        for (int i = 0; i < kUnroll; ++i) {
            const long long t = tb + i;
            if constexpr (IN) {
                nx[i] = ldv<VEC>(xrow + t * p.sxl);
                ngy[i] = ldv<VEC>(gyrow + t * p.D);
            } else {
                const bool live = d_ok && t < tend && t < p.L;
                nx[i] = load_x<K, VEC>(p, b, t, d, live);
#pragma unroll
                for (int q = 0; q < VEC; ++q) ngy[i].v[q] = 0.f;
                if (live) ngy[i] = ldv<VEC>(gyrow + t * p.D);
            }
        }
    };
    if constexpr (CONV_BWD_PIPE) fetch(t0);
    for (long long tb = t0; tb < tend; tb += kUnroll) {
        VecT<VEC> cur[kUnroll], gyv[kUnroll];
        if constexpr (!CONV_BWD_PIPE) fetch(tb);
#pragma unroll
        for (int i = 0; i < kUnroll; ++i) cur[i] = nx[i], gyv[i] = ngy[i];
        if constexpr (CONV_BWD_PIPE) fetch(tb + kUnroll);
#pragma unroll
        for (int i = 0; i < kUnroll; ++i) {
            const long long t = tb + i;
            if (t < tend) {
#pragma unroll
                for (int k = 0; k < K - 1; ++k) win[k] = win[k + 1];
                win[K - 1] = cur[i];
                const bool in_seq = IN || t < p.L, own = t < t1;
                VecT<VEC> gxo;
#pragma unroll
                for (int q = 0; q < VEC; ++q) {
                    float pre = bs[q];
#pragma unroll
                    for (int k = 0; k < K; ++k) pre = fmaf(wgt[k][q], win[k].v[q], pre);
                    const float sg = sigmoid_fast(pre);
                    const float gp = in_seq ? gyv[i].v[q] * sg * fmaf(pre, 1.f - sg, 1.f) : 0.f;
#pragma unroll
                    for (int k = K - 1; k > 0; --k) gwin[k][q] = gwin[k - 1][q];
                    gwin[0][q] = gp;
                    if (own) {
                        gb[q] += gp;
#pragma unroll
                        for (int k = 0; k < K; ++k) gw[k][q] = fmaf(gp, win[k].v[q], gw[k][q]);
                    }
                    float acc = 0.f;  // gx[t-K+1] = sum_k w_k gpre[t-k]
#pragma unroll
                    for (int k = 0; k < K; ++k) acc = fmaf(wgt[k][q], gwin[k][q], acc);
                    gxo.v[q] = acc;
                    if (!IN && K > 1 && seg == 0) {
#pragma unroll
                        for (int k = 0; k < K - 1; ++k)
                            if (t == k) gfirst[k][q] = gp;
                    }
                }
                const long long s = t - (K - 1);
                if (IN ? s >= t0 : (d_ok && s >= t0 && s < t1)) stv<VEC>(gxrow + s * p.D, gxo);
            }
        }
    }
    };
    if (interior) {
        if (d_ok) body(std::true_type{});
    } else {
        body(std::false_type{});
    }
    if (!d_ok) return;
    const long long part = b * p.nseg + seg;
#pragma unroll
    for (int q = 0; q < VEC; ++q) {
#pragma unroll
        for (int k = 0; k < K; ++k) p.gw_part[(part * p.D + d + q) * K + k] = gw[k][q];
        if constexpr (HAS_BIAS) p.gb_part[part * p.D + d + q] = gb[q];
        if (seg == 0) {  // gtail[j] = sum_{k<=j} w_k gpre[j-k]
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
}

// out[i] = sum_k in[k * stride + i] for many partials: 32 threads per output each add every 32nd
// partial in ascending order (independent loads, so many are in flight), then the 32 sub-sums are
// added in lane order: a fixed order, so the result is reproducible.  32 outputs per block keep
// the reads of one partial coalesced.
__global__ void __launch_bounds__(1024) conv_sum_parts_kernel(const float* __restrict__ in, float* __restrict__ out,
                                                              long long count, long long stride, int parts) {
    __shared__ float sh[32][33];
    const int o = threadIdx.x & 31, pl = threadIdx.x >> 5;
    const long long i = (long long)blockIdx.x * 32 + o;
    float s = 0.f;
    if (i < count) {
        int k = pl;
        for (; k + 96 < parts; k += 128) {  // four independent loads per round
            const float v0 = in[k * stride + i], v1 = in[(k + 32) * stride + i];
            const float v2 = in[(k + 64) * stride + i], v3 = in[(k + 96) * stride + i];
            s += v0, s += v1, s += v2, s += v3;
        }
        for (; k < parts; k += 32) s += in[k * stride + i];
    }
    sh[pl][o] = s;
    __syncthreads();
    if (pl == 0 && i < count) {
        float t = 0.f;
#pragma unroll
        for (int q = 0; q < 32; ++q) t += sh[q][o];
        out[i] = t;
    }
}

template <int K, int VEC>
static int launch_conv(bool bwd, bool has_bias, const ConvArgs& a, cudaStream_t st) {
    const long long grid = a.B * a.nseg * a.ndblk;
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

static void conv_shape(ConvArgs& a, int vec) {
    a.nseg = (a.L + kSegT - 1) / kSegT;
    a.ndblk = (a.D + (long long)kConvThreads * vec - 1) / ((long long)kConvThreads * vec);
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
    conv_shape(a, vec);
    return dispatch_conv<false>(vec, (int)K, bias != nullptr, a, static_cast<cudaStream_t>(stream));
}

size_t b200_conv_silu_bwd_workspace_bytes(int64_t B, int64_t L, int64_t D, int64_t K) {
    if (B <= 0 || L <= 0 || D <= 0 || K < 2 || K > 8) return 256;
    const size_t parts = (size_t)B * (size_t)((L + b200::kSegT - 1) / b200::kSegT);
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
    conv_shape(a, vec);
    const size_t parts = (size_t)B * (size_t)a.nseg;
    a.gw_part = (float*)workspace;
    a.gb_part = (float*)((char*)workspace + align_up(parts * D * K * sizeof(float), 256));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int rc = dispatch_conv<true>(vec, (int)K, bias != nullptr, a, st);
    if (rc != B200_OK) return rc;
    const long long cw = D * K;
    conv_sum_parts_kernel<<<(unsigned int)((cw + 31) / 32), 1024, 0, st>>>(a.gw_part, (float*)gw, cw, cw, (int)parts);
    if (bias) conv_sum_parts_kernel<<<(unsigned int)((D + 31) / 32), 1024, 0, st>>>(a.gb_part, (float*)gb, D, D, (int)parts);
    return cudaGetLastError() == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

}  // extern "C"
