// Pointwise glue of the LRU / S5 blocks around the scan, float32: the pre-norm LayerNorm over the
// feature axis and the gated residual  out = u + a * sigmoid(b)  (the GLU of the LRU block with
// a, b the two halves of one tensor; the "half GLU" of the S5 block with a = h and b a dense layer
// of h), each with its adjoint.  The rows are tokens (batch x time, hundreds of thousands), the
// feature axis is short (tens to a few hundred), so every kernel is one pass over HBM:
//   * LayerNorm: one warp per row, the row held in registers (two-pass mean / variance, as PyTorch
//     computes it), statistics saved for the adjoint; the adjoint adds the weight / bias gradients of
//     a CTA's rows in shared memory and writes one partial row per CTA, which rows_reduce_kernel
//     sums in a fixed order (no atomics, reproducible);
//   * gated residual: elementwise, four features per thread.
#include "common.cuh"

namespace b200 {

constexpr int kLnMaxPerLane = 16;  // features per lane held in registers: feature widths up to 512

// ------------------------------------------------------------------------------- LayerNorm forward
template <int PER>  // features per lane (row width D <= 32 * PER)
__global__ void __launch_bounds__(256) layernorm_fwd_kernel(const float* __restrict__ x, const float* __restrict__ gamma,
                                                             const float* __restrict__ beta, float* __restrict__ y,
                                                             float* __restrict__ mean_out, float* __restrict__ rstd_out,
                                                             long long M, int D, float eps) {
    const int lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= M) return;
    const float* xr = x + row * D;
    float v[PER];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int c = lane + 32 * i;
        v[i] = c < D ? __ldcs(xr + c) : 0.f;
        s += v[i];
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    const float mean = s / (float)D;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int c = lane + 32 * i;
        const float d = c < D ? v[i] - mean : 0.f;
        q = fmaf(d, d, q);
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) q += __shfl_xor_sync(0xffffffffu, q, off);
    const float rstd = rsqrtf(q / (float)D + eps);
    float* yr = y + row * D;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int c = lane + 32 * i;
        if (c < D) {
            const float g = gamma != nullptr ? gamma[c] : 1.f, b = beta != nullptr ? beta[c] : 0.f;
            __stcs(yr + c, fmaf((v[i] - mean) * rstd, g, b));
        }
    }
    if (lane == 0) {
        mean_out[row] = mean;
        rstd_out[row] = rstd;
    }
}

// ------------------------------------------------------------------------------- LayerNorm adjoint
// dx = rstd * (g*gamma - mean(g*gamma) - xhat * mean(g*gamma*xhat));  dgamma = sum_rows g*xhat;  dbeta = sum_rows g.
// A CTA walks its rows (grid-stride over warps); every lane keeps running column sums for its features,
// the warps of a CTA add them through shared memory and the CTA writes one partial row.
template <int PER>
__global__ void __launch_bounds__(256) layernorm_bwd_kernel(const float* __restrict__ g, const float* __restrict__ x,
                                                             const float* __restrict__ gamma, const float* __restrict__ mean_in,
                                                             const float* __restrict__ rstd_in, float* __restrict__ dx,
                                                             float* __restrict__ part, long long M, int D) {
    extern __shared__ float red[];  // [warps][2][32 * PER]
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    float gam[PER], dg[PER], db[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int c = lane + 32 * i;
        gam[i] = (c < D && gamma != nullptr) ? gamma[c] : 1.f;
        dg[i] = 0.f, db[i] = 0.f;
    }
    for (long long row = (long long)blockIdx.x * nw + wid; row < M; row += (long long)gridDim.x * nw) {
        const float mean = mean_in[row], rstd = rstd_in[row];
        const float* gr = g + row * D;
        const float* xr = x + row * D;
        float gv[PER], xh[PER];
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int c = lane + 32 * i;
            const bool ok = c < D;
            gv[i] = ok ? __ldcs(gr + c) : 0.f;
            xh[i] = ok ? (__ldcs(xr + c) - mean) * rstd : 0.f;
            const float gg = gv[i] * gam[i];
            s1 += gg;
            s2 = fmaf(gg, xh[i], s2);
            dg[i] = fmaf(gv[i], xh[i], dg[i]);
            db[i] += gv[i];
        }
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) {
            s1 += __shfl_xor_sync(0xffffffffu, s1, off);
            s2 += __shfl_xor_sync(0xffffffffu, s2, off);
        }
        const float m1 = s1 / (float)D, m2 = s2 / (float)D;
        float* dr = dx + row * D;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int c = lane + 32 * i;
            if (c < D) __stcs(dr + c, rstd * (gv[i] * gam[i] - m1 - xh[i] * m2));
        }
    }
    const int W = 32 * PER;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        red[(wid * 2 + 0) * W + lane + 32 * i] = dg[i];
        red[(wid * 2 + 1) * W + lane + 32 * i] = db[i];
    }
    __syncthreads();
    for (int e = threadIdx.x; e < 2 * W; e += blockDim.x) {
        const int which = e / W, c = e - which * W;
        float s = 0.f;
        for (int w = 0; w < nw; ++w) s += red[(w * 2 + which) * W + c];  // warps in order
        if (c < D) part[((long long)blockIdx.x * 2 + which) * D + c] = s;
    }
}

// out[e] = sum over partial rows of part[row][e], e in [0, width), in a fixed order: 32 lanes per
// output each add every 32nd partial (eight independent loads per round), then the 32 sub-sums are
// added in lane order; 32 outputs per block keep the reads of one partial row coalesced.  Entries
// below `split` go to out0, the rest to out1 (either may be null).
__global__ void __launch_bounds__(1024) rows_reduce_kernel(const float* __restrict__ part, int rows, int width, int split,
                                                           float* __restrict__ out0, float* __restrict__ out1) {
    __shared__ float sh[32][33];
    const int o = threadIdx.x & 31, pl = threadIdx.x >> 5;
    const int e = blockIdx.x * 32 + o;
    const bool live = e < width;
    const long long stride = width;
    float s = 0.f;
    if (live) {
        int k = pl;
        for (; k + 224 < rows; k += 256) {
            float v[8];
#pragma unroll
            for (int r = 0; r < 8; ++r) v[r] = part[(k + 32 * r) * stride + e];
#pragma unroll
            for (int r = 0; r < 8; ++r) s += v[r];
        }
        for (; k < rows; k += 32) s += part[k * stride + e];
    }
    sh[pl][o] = s;
    __syncthreads();
    if (pl == 0 && live) {
        float t = 0.f;
#pragma unroll
        for (int q = 0; q < 32; ++q) t += sh[q][o];
        float* dst = e < split ? out0 : out1;
        if (dst != nullptr) dst[e < split ? e : e - split] = t;
    }
}

// ------------------------------------------------------------------------------- column sums
// out[c] = sum over rows of x[m, c] (the bias gradient of a linear layer).  A CTA owns a contiguous
// slab of rows; a thread owns VEC neighbouring columns and every (256 / threads-per-row)-th row of
// the slab, eight rows in flight; the CTA's row groups are added in shared memory in a fixed order and
// one partial row per CTA goes to the workspace, which colsum_reduce_kernel adds in a fixed order.
template <int VEC>
__global__ void __launch_bounds__(256) colsum_kernel(const float* __restrict__ x, long long ldx, long long M, int D,
                                                     long long rows_per_cta, float* __restrict__ part) {
    extern __shared__ float sh[];  // [groups][D]
    const int tpr = (D + VEC - 1) / VEC;          // threads per row
    const int groups = 256 / tpr;                 // row groups of the CTA (>= 1: D <= 256 * VEC)
    const int grp = threadIdx.x / tpr, c = (threadIdx.x - grp * tpr) * VEC;
    const long long r0 = (long long)blockIdx.x * rows_per_cta;
    const long long r1 = r0 + rows_per_cta < M ? r0 + rows_per_cta : M;
    float acc[VEC];
#pragma unroll
    for (int q = 0; q < VEC; ++q) acc[q] = 0.f;
    if (grp < groups) {
        long long r = r0 + grp;
        for (; r + 7LL * groups < r1; r += 8LL * groups) {
            float v[8][VEC];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float* p = x + (r + (long long)i * groups) * ldx + c;
                if constexpr (VEC == 4) {
                    const float4 t = __ldcs(reinterpret_cast<const float4*>(p));
                    v[i][0] = t.x, v[i][1] = t.y, v[i][2] = t.z, v[i][3] = t.w;
                } else {
                    v[i][0] = __ldcs(p);
                }
            }
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int q = 0; q < VEC; ++q) acc[q] += v[i][q];
        }
        for (; r < r1; r += groups) {
            const float* p = x + r * ldx + c;
#pragma unroll
            for (int q = 0; q < VEC; ++q) acc[q] += p[q];
        }
#pragma unroll
        for (int q = 0; q < VEC; ++q) sh[grp * D + c + q] = acc[q];
    }
    __syncthreads();
    for (int e = threadIdx.x; e < D; e += 256) {
        float s = 0.f;
        for (int g = 0; g < groups; ++g) s += sh[g * D + e];
        part[(long long)blockIdx.x * D + e] = s;
    }
}

// ------------------------------------------------------------------------------- gated residual
__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

// out[m, c] = u[m, c] + a[m, c] * sigmoid(b[m, c]);  row pitches in floats; VEC = 4 needs 16-byte aligned rows
template <int VEC>
__global__ void gated_residual_fwd_kernel(const float* __restrict__ u, long long ldu, const float* __restrict__ a, long long lda,
                                          const float* __restrict__ b, long long ldb, float* __restrict__ out, long long ldo,
                                          long long M, int D) {
    const int per_row = D / VEC;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= M * per_row) return;
    const long long m = i / per_row;
    const int c = (int)(i - m * per_row) * VEC;
    if constexpr (VEC == 4) {
        const float4 uu = __ldcs(reinterpret_cast<const float4*>(u + m * ldu + c));
        const float4 aa = __ldcs(reinterpret_cast<const float4*>(a + m * lda + c));
        const float4 bb = __ldcs(reinterpret_cast<const float4*>(b + m * ldb + c));
        float4 o;
        o.x = fmaf(aa.x, sigmoidf_(bb.x), uu.x), o.y = fmaf(aa.y, sigmoidf_(bb.y), uu.y);
        o.z = fmaf(aa.z, sigmoidf_(bb.z), uu.z), o.w = fmaf(aa.w, sigmoidf_(bb.w), uu.w);
        __stcs(reinterpret_cast<float4*>(out + m * ldo + c), o);
    } else {
        out[m * ldo + c] = fmaf(a[m * lda + c], sigmoidf_(b[m * ldb + c]), u[m * ldu + c]);
    }
}

// ga = g * sigmoid(b);  gb = g * a * sigmoid(b) * (1 - sigmoid(b))      (the gradient of u is g itself)
template <int VEC>
__global__ void gated_residual_bwd_kernel(const float* __restrict__ g, long long ldg, const float* __restrict__ a, long long lda,
                                          const float* __restrict__ b, long long ldb, float* __restrict__ ga, long long ldga,
                                          float* __restrict__ gb, long long ldgb, long long M, int D) {
    const int per_row = D / VEC;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= M * per_row) return;
    const long long m = i / per_row;
    const int c = (int)(i - m * per_row) * VEC;
    auto one = [](float gg, float aa, float bb, float& oa, float& ob) {
        const float s = sigmoidf_(bb);
        oa = gg * s;
        ob = gg * aa * s * (1.f - s);
    };
    if constexpr (VEC == 4) {
        const float4 gg = __ldcs(reinterpret_cast<const float4*>(g + m * ldg + c));
        const float4 aa = __ldcs(reinterpret_cast<const float4*>(a + m * lda + c));
        const float4 bb = __ldcs(reinterpret_cast<const float4*>(b + m * ldb + c));
        float4 oa, ob;
        one(gg.x, aa.x, bb.x, oa.x, ob.x), one(gg.y, aa.y, bb.y, oa.y, ob.y);
        one(gg.z, aa.z, bb.z, oa.z, ob.z), one(gg.w, aa.w, bb.w, oa.w, ob.w);
        __stcs(reinterpret_cast<float4*>(ga + m * ldga + c), oa);
        __stcs(reinterpret_cast<float4*>(gb + m * ldgb + c), ob);
    } else {
        float oa, ob;
        one(g[m * ldg + c], a[m * lda + c], b[m * ldb + c], oa, ob);
        ga[m * ldga + c] = oa;
        gb[m * ldgb + c] = ob;
    }
}

static int ln_per(int D) { return D <= 32 ? 1 : D <= 64 ? 2 : D <= 128 ? 4 : D <= 256 ? 8 : 16; }
static int ln_bwd_ctas(long long M) {
    long long want = (M + 7) / 8;  // 8 warps per CTA
    const long long cap = 148 * 4;
    return (int)(want < cap ? (want < 1 ? 1 : want) : cap);
}
static bool vec4(const void* p, long long ld) { return ((uintptr_t)p & 15) == 0 && ld % 4 == 0; }
// CTAs of the column-sum kernel: every SM several times over, but at least 64 rows per CTA
static int colsum_ctas(long long M) {
    long long want = (M + 63) / 64;
    const long long cap = 148 * 8;
    return (int)(want < cap ? (want < 1 ? 1 : want) : cap);
}

}  // namespace b200

extern "C" {

int b200_layernorm_fwd(int64_t M, int64_t D, const void* x, const void* gamma, const void* beta, float eps, void* y,
                       void* mean, void* rstd, void* stream) {
    using namespace b200;
    if (M < 0 || D < 1) return B200_ERR_ARG;
    if (D > 32 * kLnMaxPerLane) return B200_ERR_UNSUPPORTED;
    if (M == 0) return B200_OK;
    if (!x || !y || !mean || !rstd) return B200_ERR_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const long long blocks = (M + 7) / 8;
    if (blocks > 0x7fffffffLL) return B200_ERR_UNSUPPORTED;
#define LN_FWD(P)                                                                                                         \
    layernorm_fwd_kernel<P><<<(unsigned int)blocks, 256, 0, st>>>((const float*)x, (const float*)gamma, (const float*)beta, \
                                                                   (float*)y, (float*)mean, (float*)rstd, M, (int)D, eps)
    switch (ln_per((int)D)) {
        case 1: LN_FWD(1); break;
        case 2: LN_FWD(2); break;
        case 4: LN_FWD(4); break;
        case 8: LN_FWD(8); break;
        default: LN_FWD(16); break;
    }
#undef LN_FWD
    return cudaGetLastError() == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

size_t b200_layernorm_bwd_workspace_bytes(int64_t M, int64_t D) {
    if (M <= 0 || D <= 0) return 256;
    return b200::align_up(sizeof(float) * 2 * (size_t)D * (size_t)b200::ln_bwd_ctas(M), 256);
}

int b200_layernorm_bwd(int64_t M, int64_t D, const void* g, const void* x, const void* gamma, const void* mean,
                       const void* rstd, void* dx, void* dgamma, void* dbeta, void* workspace, size_t workspace_bytes,
                       void* stream) {
    using namespace b200;
    if (M < 0 || D < 1) return B200_ERR_ARG;
    if (D > 32 * kLnMaxPerLane) return B200_ERR_UNSUPPORTED;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (M == 0) {
        if (dgamma && cudaMemsetAsync(dgamma, 0, sizeof(float) * D, st) != cudaSuccess) return B200_ERR_LAUNCH;
        if (dbeta && cudaMemsetAsync(dbeta, 0, sizeof(float) * D, st) != cudaSuccess) return B200_ERR_LAUNCH;
        return B200_OK;
    }
    if (!g || !x || !mean || !rstd || !dx) return B200_ERR_ARG;
    if (!workspace || ((uintptr_t)workspace % 256) != 0 || workspace_bytes < b200_layernorm_bwd_workspace_bytes(M, D))
        return B200_ERR_WORKSPACE;
    const int ctas = ln_bwd_ctas(M);
    const int per = ln_per((int)D);
    const size_t smem = sizeof(float) * 8 * 2 * 32 * per;
#define LN_BWD(P)                                                                                                          \
    layernorm_bwd_kernel<P><<<ctas, 256, smem, st>>>((const float*)g, (const float*)x, (const float*)gamma, (const float*)mean, \
                                                     (const float*)rstd, (float*)dx, (float*)workspace, M, (int)D)
    switch (per) {
        case 1: LN_BWD(1); break;
        case 2: LN_BWD(2); break;
        case 4: LN_BWD(4); break;
        case 8: LN_BWD(8); break;
        default: LN_BWD(16); break;
    }
#undef LN_BWD
    if (cudaGetLastError() != cudaSuccess) return B200_ERR_LAUNCH;
    rows_reduce_kernel<<<(unsigned int)((2 * D + 31) / 32), 1024, 0, st>>>((const float*)workspace, ctas, 2 * (int)D, (int)D,
                                                                           (float*)dgamma, (float*)dbeta);
    return cudaGetLastError() == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

size_t b200_colsum_workspace_bytes(int64_t M, int64_t D) {
    if (M <= 0 || D <= 0) return 256;
    return b200::align_up(sizeof(float) * (size_t)D * (size_t)b200::colsum_ctas(M), 256);
}

int b200_colsum(int64_t M, int64_t D, const void* x, int64_t ldx, void* out, void* workspace, size_t workspace_bytes,
                void* stream) {
    using namespace b200;
    if (M < 0 || D < 1 || !out) return B200_ERR_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (M == 0) return cudaMemsetAsync(out, 0, sizeof(float) * D, st) == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
    if (!x || ldx < D) return B200_ERR_ARG;
    const bool v4 = D % 4 == 0 && vec4(x, ldx);
    if (D > 256 * (v4 ? 4 : 1)) return B200_ERR_UNSUPPORTED;
    if (!workspace || ((uintptr_t)workspace % 256) != 0 || workspace_bytes < b200_colsum_workspace_bytes(M, D))
        return B200_ERR_WORKSPACE;
    const int ctas = colsum_ctas(M);
    const long long rows_per_cta = (M + ctas - 1) / ctas;
    const int tpr = (int)(v4 ? D / 4 : D), groups = 256 / tpr;
    const size_t smem = sizeof(float) * (size_t)groups * (size_t)D;
    if (v4)
        colsum_kernel<4><<<ctas, 256, smem, st>>>((const float*)x, ldx, M, (int)D, rows_per_cta, (float*)workspace);
    else
        colsum_kernel<1><<<ctas, 256, smem, st>>>((const float*)x, ldx, M, (int)D, rows_per_cta, (float*)workspace);
    if (cudaGetLastError() != cudaSuccess) return B200_ERR_LAUNCH;
    rows_reduce_kernel<<<(unsigned int)((D + 31) / 32), 1024, 0, st>>>((const float*)workspace, ctas, (int)D, (int)D, (float*)out,
                                                                       nullptr);
    return cudaGetLastError() == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

int b200_gated_residual_fwd(int64_t M, int64_t D, const void* u, int64_t ldu, const void* a, int64_t lda, const void* b,
                            int64_t ldb, void* out, int64_t ldo, void* stream) {
    using namespace b200;
    if (M < 0 || D < 1) return B200_ERR_ARG;
    if (M == 0) return B200_OK;
    if (!u || !a || !b || !out) return B200_ERR_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool v4 = D % 4 == 0 && vec4(u, ldu) && vec4(a, lda) && vec4(b, ldb) && vec4(out, ldo);
    const long long n = M * (v4 ? D / 4 : D), blocks = (n + 255) / 256;
    if (blocks > 0x7fffffffLL) return B200_ERR_UNSUPPORTED;
    if (v4)
        gated_residual_fwd_kernel<4><<<(unsigned int)blocks, 256, 0, st>>>((const float*)u, ldu, (const float*)a, lda, (const float*)b,
                                                                          ldb, (float*)out, ldo, M, (int)D);
    else
        gated_residual_fwd_kernel<1><<<(unsigned int)blocks, 256, 0, st>>>((const float*)u, ldu, (const float*)a, lda, (const float*)b,
                                                                          ldb, (float*)out, ldo, M, (int)D);
    return cudaGetLastError() == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

int b200_gated_residual_bwd(int64_t M, int64_t D, const void* g, int64_t ldg, const void* a, int64_t lda, const void* b,
                            int64_t ldb, void* ga, int64_t ldga, void* gb, int64_t ldgb, void* stream) {
    using namespace b200;
    if (M < 0 || D < 1) return B200_ERR_ARG;
    if (M == 0) return B200_OK;
    if (!g || !a || !b || !ga || !gb) return B200_ERR_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool v4 = D % 4 == 0 && vec4(g, ldg) && vec4(a, lda) && vec4(b, ldb) && vec4(ga, ldga) && vec4(gb, ldgb);
    const long long n = M * (v4 ? D / 4 : D), blocks = (n + 255) / 256;
    if (blocks > 0x7fffffffLL) return B200_ERR_UNSUPPORTED;
    if (v4)
        gated_residual_bwd_kernel<4><<<(unsigned int)blocks, 256, 0, st>>>((const float*)g, ldg, (const float*)a, lda, (const float*)b,
                                                                          ldb, (float*)ga, ldga, (float*)gb, ldgb, M, (int)D);
    else
        gated_residual_bwd_kernel<1><<<(unsigned int)blocks, 256, 0, st>>>((const float*)g, ldg, (const float*)a, lda, (const float*)b,
                                                                          ldb, (float*)ga, ldga, (float*)gb, ldgb, M, (int)D);
    return cudaGetLastError() == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

}  // extern "C"
