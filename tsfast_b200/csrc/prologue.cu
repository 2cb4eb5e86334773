// Parameter prologues of the LRU and S5 layers, forward and adjoint, float32 / complex64:
// everything between the stored parameters and what the projection GEMM and the scan consume,
//   LRU:  lam_j = exp(-exp(nu_j)) * e^{i exp(theta_j)},   W[2j] = e^{gamma_j} B_re[j],  W[2j+1] = e^{gamma_j} B_im[j]
//   S5:   (Lambda, step) -> (lam_bar, c) by zero-order hold or the bilinear map,  W[2j] + i W[2j+1] = c_j * B~[j]
// with W [2n, d] the input-projection weight in the interleaved (re, im) row order whose GEMM result
// has the memory layout of a complex [.., n] tensor.  These are parameter-sized (n, n x d): one warp
// owns one state row, lanes stride over the d input features; the adjoint's per-state sums over d are
// warp reductions in a fixed order.  In PyTorch the same math is a dozen tiny launches forward and
// twice that in the backward pass, per layer and step.
//
// Gradient convention (PyTorch's): for a complex value z = f(w) with f holomorphic, an incoming
// gradient g (= dL/dRe z + i dL/dIm z) becomes g * conj(f'(w)) on w.
#include "common.cuh"

namespace b200 {

struct cplx {
    float re, im;
};
__device__ __forceinline__ cplx cmul(cplx a, cplx b) { return {a.re * b.re - a.im * b.im, a.re * b.im + a.im * b.re}; }
__device__ __forceinline__ cplx cconj(cplx a) { return {a.re, -a.im}; }
__device__ __forceinline__ cplx cadd(cplx a, cplx b) { return {a.re + b.re, a.im + b.im}; }
__device__ __forceinline__ cplx cscale(cplx a, float s) { return {a.re * s, a.im * s}; }
__device__ __forceinline__ cplx cinv(cplx a) {
    const float d = 1.f / (a.re * a.re + a.im * a.im);
    return {a.re * d, -a.im * d};
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ------------------------------------------------------------------------------- LRU
__global__ void __launch_bounds__(256) lru_prologue_fwd_kernel(int n, int d, const float* __restrict__ nu_log,
                                                               const float* __restrict__ theta_log,
                                                               const float* __restrict__ gamma_log,
                                                               const float* __restrict__ B_re, const float* __restrict__ B_im,
                                                               float2* __restrict__ lam, float* __restrict__ W) {
    const int j = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (j >= n) return;
    if (lane == 0) {
        const float a = expf(-expf(nu_log[j])), ph = expf(theta_log[j]);
        float s, c;
        sincosf(ph, &s, &c);
        lam[j] = make_float2(a * c, a * s);
    }
    const float g = expf(gamma_log[j]);
    for (int k = lane; k < d; k += 32) {
        W[(size_t)(2 * j) * d + k] = g * B_re[(size_t)j * d + k];
        W[(size_t)(2 * j + 1) * d + k] = g * B_im[(size_t)j * d + k];
    }
}

__global__ void __launch_bounds__(256) lru_prologue_bwd_kernel(int n, int d, const float* __restrict__ nu_log,
                                                               const float* __restrict__ theta_log,
                                                               const float* __restrict__ gamma_log,
                                                               const float* __restrict__ B_re, const float* __restrict__ B_im,
                                                               const float2* __restrict__ glam, const float* __restrict__ gW,
                                                               float* __restrict__ g_nu, float* __restrict__ g_theta,
                                                               float* __restrict__ g_gamma, float* __restrict__ gB_re,
                                                               float* __restrict__ gB_im) {
    const int j = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (j >= n) return;
    if (lane == 0) {
        float gn = 0.f, gt = 0.f;
        if (glam != nullptr) {
            const float en = expf(nu_log[j]), a = expf(-en), ph = expf(theta_log[j]);
            float s, c;
            sincosf(ph, &s, &c);
            const float2 g = glam[j];
            gn = (g.x * c + g.y * s) * (-en * a);
            gt = (g.y * c - g.x * s) * a * ph;
        }
        g_nu[j] = gn, g_theta[j] = gt;
    }
    const float g = expf(gamma_log[j]);
    float acc = 0.f;
    if (gW != nullptr) {
        for (int k = lane; k < d; k += 32) {
            const float wr = gW[(size_t)(2 * j) * d + k], wi = gW[(size_t)(2 * j + 1) * d + k];
            const float br = B_re[(size_t)j * d + k], bi = B_im[(size_t)j * d + k];
            acc = fmaf(wr, br, fmaf(wi, bi, acc));
            gB_re[(size_t)j * d + k] = g * wr;
            gB_im[(size_t)j * d + k] = g * wi;
        }
    } else {
        for (int k = lane; k < d; k += 32) gB_re[(size_t)j * d + k] = 0.f, gB_im[(size_t)j * d + k] = 0.f;
    }
    acc = warp_sum(acc);
    if (lane == 0) g_gamma[j] = g * acc;
}

// phi1(z) = (e^z - 1) / z and its derivative (z e^z - e^z + 1) / z^2.  For small |z| = |lam| * step both
// closed forms cancel (the derivative to second order), so below |z| = 1/2 they are summed as power
// series (ten terms: the remainder is below 1e-10); ez = e^z.
__device__ __forceinline__ void phi1_pair(cplx z, cplx ez, cplx& phi, cplx& dphi) {
    if (z.re * z.re + z.im * z.im < 0.25f) {
        const float a[10] = {1.f, 1.f / 2, 1.f / 6, 1.f / 24, 1.f / 120, 1.f / 720, 1.f / 5040, 1.f / 40320, 1.f / 362880,
                             1.f / 3628800};
        const float b[10] = {1.f / 2, 1.f / 3, 1.f / 8, 1.f / 30, 1.f / 144, 1.f / 840, 1.f / 5760, 1.f / 45360, 1.f / 403200,
                             1.f / 3991680};
        phi = {a[9], 0.f}, dphi = {b[9], 0.f};
#pragma unroll
        for (int k = 8; k >= 0; --k) {
            phi = cadd(cmul(phi, z), {a[k], 0.f});
            dphi = cadd(cmul(dphi, z), {b[k], 0.f});
        }
    } else {
        const cplx inv = cinv(z);
        phi = cmul(cadd(ez, {-1.f, 0.f}), inv);
        dphi = cmul(cadd(ez, cscale(phi, -1.f)), inv);
    }
}

// ------------------------------------------------------------------------------- S5
struct S5Point {
    cplx lam, lam_bar, c;  // continuous eigenvalue (after the clip), discrete eigenvalue, input scale
    cplx dlb_dlam, dc_dlam, dlb_ds, dc_ds;  // derivatives (those by the real step s are complex numbers too)
    float s;
    bool clipped;
};

// mode 0: zero-order hold  lam_bar = exp(lam s), c = (lam_bar - 1) / lam (summed as a series for small lam s)
// mode 1: bilinear         bl = 1 / (1 - s/2 lam), lam_bar = bl (1 + s/2 lam), c = bl s
__device__ __forceinline__ S5Point s5_point(int mode, bool clip, float step_rescale, float lr, float li, float log_step) {
    S5Point q;
    q.clipped = clip && lr > -1e-4f;
    q.lam = {q.clipped ? -1e-4f : lr, li};
    q.s = step_rescale * expf(log_step);
    const cplx one = {1.f, 0.f};
    if (mode == 0) {
        const float m = expf(q.lam.re * q.s);
        float sn, cs;
        sincosf(q.lam.im * q.s, &sn, &cs);
        q.lam_bar = {m * cs, m * sn};
        // c = (lam_bar - 1) / lam = s phi1(lam s);  dc/dlam = s^2 phi1'(lam s);  dc/ds = lam_bar
        cplx phi, dphi;
        phi1_pair(cscale(q.lam, q.s), q.lam_bar, phi, dphi);
        q.c = cscale(phi, q.s);
        q.dlb_dlam = cscale(q.lam_bar, q.s);
        q.dlb_ds = cmul(q.lam, q.lam_bar);
        q.dc_dlam = cscale(dphi, q.s * q.s);
        q.dc_ds = q.lam_bar;
    } else {
        const float h = 0.5f * q.s;
        const cplx bl = cinv(cadd(one, cscale(q.lam, -h)));
        const cplx up = cadd(one, cscale(q.lam, h));
        q.lam_bar = cmul(bl, up);
        q.c = cscale(bl, q.s);
        const cplx bl2 = cmul(bl, bl);
        // d bl / d lam = h bl^2,  d bl / d h = lam bl^2
        const cplx t = cadd(bl, cmul(up, bl2));  // bl + (1 + h lam) bl^2
        q.dlb_dlam = cscale(t, h);
        q.dlb_ds = cscale(cmul(q.lam, t), 0.5f);
        q.dc_dlam = cscale(bl2, q.s * h);
        q.dc_ds = cadd(bl, cscale(cmul(q.lam, bl2), 0.5f * q.s));
    }
    return q;
}

__global__ void __launch_bounds__(256) s5_discretize_fwd_kernel(int p, int d, int mode, int clip, float step_rescale,
                                                                const float* __restrict__ L_re, const float* __restrict__ L_im,
                                                                const float* __restrict__ log_step,
                                                                const float* __restrict__ B_re, const float* __restrict__ B_im,
                                                                float2* __restrict__ lam_bar, float* __restrict__ W) {
    const int j = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (j >= p) return;
    const S5Point q = s5_point(mode, clip != 0, step_rescale, L_re[j], L_im[j], log_step[j]);
    if (lane == 0) lam_bar[j] = make_float2(q.lam_bar.re, q.lam_bar.im);
    for (int k = lane; k < d; k += 32) {
        const cplx b = {B_re[(size_t)j * d + k], B_im[(size_t)j * d + k]};
        const cplx w = cmul(q.c, b);
        W[(size_t)(2 * j) * d + k] = w.re;
        W[(size_t)(2 * j + 1) * d + k] = w.im;
    }
}

__global__ void __launch_bounds__(256) s5_discretize_bwd_kernel(int p, int d, int mode, int clip, float step_rescale,
                                                                const float* __restrict__ L_re, const float* __restrict__ L_im,
                                                                const float* __restrict__ log_step,
                                                                const float* __restrict__ B_re, const float* __restrict__ B_im,
                                                                const float2* __restrict__ glam_bar, const float* __restrict__ gW,
                                                                float* __restrict__ gL_re, float* __restrict__ gL_im,
                                                                float* __restrict__ g_log_step, float* __restrict__ gB_re,
                                                                float* __restrict__ gB_im) {
    const int j = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (j >= p) return;
    const S5Point q = s5_point(mode, clip != 0, step_rescale, L_re[j], L_im[j], log_step[j]);
    // gradient of the input scale c: sum_k gBbar[j,k] * conj(B~[j,k]);  gradient of B~: gBbar * conj(c)
    float gc_re = 0.f, gc_im = 0.f;
    const cplx cc = cconj(q.c);
    for (int k = lane; k < d; k += 32) {
        cplx g = {0.f, 0.f};
        if (gW != nullptr) g = {gW[(size_t)(2 * j) * d + k], gW[(size_t)(2 * j + 1) * d + k]};
        const cplx b = {B_re[(size_t)j * d + k], B_im[(size_t)j * d + k]};
        const cplx t = cmul(g, cconj(b));
        gc_re += t.re, gc_im += t.im;
        const cplx gb = cmul(g, cc);
        gB_re[(size_t)j * d + k] = gb.re;
        gB_im[(size_t)j * d + k] = gb.im;
    }
    gc_re = warp_sum(gc_re), gc_im = warp_sum(gc_im);
    if (lane == 0) {
        const cplx gc = {gc_re, gc_im};
        cplx gl = {0.f, 0.f};
        if (glam_bar != nullptr) gl = {glam_bar[j].x, glam_bar[j].y};
        const cplx glam = cadd(cmul(gl, cconj(q.dlb_dlam)), cmul(gc, cconj(q.dc_dlam)));
        const float gs = cmul(gl, cconj(q.dlb_ds)).re + cmul(gc, cconj(q.dc_ds)).re;
        gL_re[j] = q.clipped ? 0.f : glam.re;
        gL_im[j] = glam.im;
        g_log_step[j] = gs * q.s;
    }
}

static unsigned int warp_rows_grid(long long rows) { return (unsigned int)((rows + 7) / 8); }

}  // namespace b200

extern "C" {

int b200_lru_prologue_fwd(int64_t n, int64_t d, const void* nu_log, const void* theta_log, const void* gamma_log,
                          const void* B_re, const void* B_im, void* lam, void* W, void* stream) {
    using namespace b200;
    if (n < 0 || d < 0 || n > 0x3fffffff || d > 0x3fffffff) return B200_ERR_ARG;
    if (n == 0) return B200_OK;
    if (!nu_log || !theta_log || !gamma_log || !lam || (d > 0 && (!B_re || !B_im || !W))) return B200_ERR_ARG;
    lru_prologue_fwd_kernel<<<warp_rows_grid(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        (int)n, (int)d, (const float*)nu_log, (const float*)theta_log, (const float*)gamma_log, (const float*)B_re,
        (const float*)B_im, (float2*)lam, (float*)W);
    return cudaGetLastError() == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

int b200_lru_prologue_bwd(int64_t n, int64_t d, const void* nu_log, const void* theta_log, const void* gamma_log,
                          const void* B_re, const void* B_im, const void* glam, const void* gW, void* g_nu, void* g_theta,
                          void* g_gamma, void* gB_re, void* gB_im, void* stream) {
    using namespace b200;
    if (n < 0 || d < 0 || n > 0x3fffffff || d > 0x3fffffff) return B200_ERR_ARG;
    if (n == 0) return B200_OK;
    if (!nu_log || !theta_log || !gamma_log || !g_nu || !g_theta || !g_gamma || (d > 0 && (!B_re || !B_im || !gB_re || !gB_im)))
        return B200_ERR_ARG;
    lru_prologue_bwd_kernel<<<warp_rows_grid(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        (int)n, (int)d, (const float*)nu_log, (const float*)theta_log, (const float*)gamma_log, (const float*)B_re,
        (const float*)B_im, (const float2*)glam, (const float*)gW, (float*)g_nu, (float*)g_theta, (float*)g_gamma, (float*)gB_re,
        (float*)gB_im);
    return cudaGetLastError() == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

int b200_s5_discretize_fwd(int64_t p, int64_t d, int mode, int clip_eigs, float step_rescale, const void* Lambda_re,
                           const void* Lambda_im, const void* log_step, const void* B_re, const void* B_im, void* lam_bar,
                           void* W, void* stream) {
    using namespace b200;
    if (p < 0 || d < 0 || p > 0x3fffffff || d > 0x3fffffff) return B200_ERR_ARG;
    if (mode != 0 && mode != 1) return B200_ERR_UNSUPPORTED;
    if (p == 0) return B200_OK;
    if (!Lambda_re || !Lambda_im || !log_step || !lam_bar || (d > 0 && (!B_re || !B_im || !W))) return B200_ERR_ARG;
    s5_discretize_fwd_kernel<<<warp_rows_grid(p), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        (int)p, (int)d, mode, clip_eigs, step_rescale, (const float*)Lambda_re, (const float*)Lambda_im, (const float*)log_step,
        (const float*)B_re, (const float*)B_im, (float2*)lam_bar, (float*)W);
    return cudaGetLastError() == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

int b200_s5_discretize_bwd(int64_t p, int64_t d, int mode, int clip_eigs, float step_rescale, const void* Lambda_re,
                           const void* Lambda_im, const void* log_step, const void* B_re, const void* B_im,
                           const void* glam_bar, const void* gW, void* gLambda_re, void* gLambda_im, void* g_log_step,
                           void* gB_re, void* gB_im, void* stream) {
    using namespace b200;
    if (p < 0 || d < 0 || p > 0x3fffffff || d > 0x3fffffff) return B200_ERR_ARG;
    if (mode != 0 && mode != 1) return B200_ERR_UNSUPPORTED;
    if (p == 0) return B200_OK;
    if (!Lambda_re || !Lambda_im || !log_step || !gLambda_re || !gLambda_im || !g_log_step ||
        (d > 0 && (!B_re || !B_im || !gB_re || !gB_im)))
        return B200_ERR_ARG;
    s5_discretize_bwd_kernel<<<warp_rows_grid(p), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        (int)p, (int)d, mode, clip_eigs, step_rescale, (const float*)Lambda_re, (const float*)Lambda_im, (const float*)log_step,
        (const float*)B_re, (const float*)B_im, (const float2*)glam_bar, (const float*)gW, (float*)gLambda_re, (float*)gLambda_im,
        (float*)g_log_step, (float*)gB_re, (float*)gB_im);
    return cudaGetLastError() == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

}  // extern "C"
