/* TEST INFRASTRUCTURE - body of the CPU oracle, included once per precision.
 *
 * Included by scan_oracle.c with REAL (float|double), ORA(name) (symbol suffixing) and the
 * libm spellings EXP/LOG1P defined.  Every function is a plain sequential-in-time restatement
 * of the reference algorithm it cites (paths are relative to the tsfast project root).
 * Complex tensors are interleaved (re, im) pairs of REAL, the layout of torch.view_as_real.
 */

/* ------------------------------------------------------------------ S1: constant diagonal
 * x_t = lam * x_{t-1} + v_t per lane; lam [M,N], v/out [M,L,N], x0 [M,N] or NULL.
 * Follows tsfast/models/_core/scan.py:316-328 (sequential definition) and the single-sweep
 * form of tsfast/models/_core/scan_backends/diagonal_c.py:128-155 (fwd_chunk_impl). */
void ORA(diag_fwd)(int64_t M, int64_t L, int64_t N, int is_complex, const REAL* lam,
                   const REAL* v, const REAL* x0, REAL* out) {
    const int64_t S = is_complex ? 2 : 1;
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t m = 0; m < M; ++m) {
        for (int64_t n = 0; n < N; ++n) {
            const int64_t ln = m * N + n;
            if (is_complex) {
                const REAL ar = lam[2 * ln], ai = lam[2 * ln + 1];
                REAL xr = x0 ? x0[2 * ln] : (REAL)0, xi = x0 ? x0[2 * ln + 1] : (REAL)0;
                for (int64_t t = 0; t < L; ++t) {
                    const int64_t p = S * ((m * L + t) * N + n);
                    const REAL nr = ar * xr - ai * xi + v[p];
                    xi = ar * xi + ai * xr + v[p + 1];
                    xr = nr;
                    out[p] = xr;
                    out[p + 1] = xi;
                }
            } else {
                const REAL a = lam[ln];
                REAL x = x0 ? x0[ln] : (REAL)0;
                for (int64_t t = 0; t < L; ++t) {
                    const int64_t p = (m * L + t) * N + n;
                    x = a * x + v[p];
                    out[p] = x;
                }
            }
        }
    }
}

/* Adjoint of S1: G_t = g_t + conj(lam) G_{t+1}; gv = G; glam = sum_t G_t conj(x_{t-1});
 * gx0 = conj(lam) G_0 (written only when x0 != NULL).
 * Follows tsfast/models/_core/scan.py:118-134 and diagonal_c.py:172-221 (bwd_chunk_impl). */
void ORA(diag_bwd)(int64_t M, int64_t L, int64_t N, int is_complex, const REAL* g,
                   const REAL* lam, const REAL* out, const REAL* x0, REAL* glam, REAL* gv,
                   REAL* gx0) {
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t m = 0; m < M; ++m) {
        for (int64_t n = 0; n < N; ++n) {
            const int64_t ln = m * N + n;
            if (is_complex) {
                const REAL ar = lam[2 * ln], ai = -lam[2 * ln + 1]; /* conj(lam) */
                REAL Gr = 0, Gi = 0, sr = 0, si = 0;
                for (int64_t t = L - 1; t >= 0; --t) {
                    const int64_t p = 2 * ((m * L + t) * N + n);
                    const REAL nr = g[p] + ar * Gr - ai * Gi;
                    Gi = g[p + 1] + ar * Gi + ai * Gr;
                    Gr = nr;
                    gv[p] = Gr;
                    gv[p + 1] = Gi;
                    REAL xr, xi;
                    if (t > 0) {
                        xr = out[p - 2 * N];
                        xi = out[p - 2 * N + 1];
                    } else {
                        xr = x0 ? x0[2 * ln] : (REAL)0;
                        xi = x0 ? x0[2 * ln + 1] : (REAL)0;
                    }
                    sr += Gr * xr + Gi * xi; /* G * conj(x_prev) */
                    si += Gi * xr - Gr * xi;
                }
                glam[2 * ln] = sr;
                glam[2 * ln + 1] = si;
                if (x0) {
                    gx0[2 * ln] = ar * Gr - ai * Gi;
                    gx0[2 * ln + 1] = ar * Gi + ai * Gr;
                }
            } else {
                const REAL a = lam[ln];
                REAL G = 0, s = 0;
                for (int64_t t = L - 1; t >= 0; --t) {
                    const int64_t p = (m * L + t) * N + n;
                    G = g[p] + a * G;
                    gv[p] = G;
                    s += G * (t > 0 ? out[p - N] : (x0 ? x0[ln] : (REAL)0));
                }
                glam[ln] = s;
                if (x0) gx0[ln] = a * G;
            }
        }
    }
}

/* ------------------------------------------------------------------ S2: time-varying diagonal
 * x_t = lam_t * x_{t-1} + v_t; lam, v, out [B,L,N]; x0 [B,N] or NULL.
 * Follows tsfast/models/_core/scan.py:316-328 and scan_backends/selective_c.py:52-76 (sel_fwd);
 * the complex case follows the doubling-scan semantics of scan.py:157-170. */
void ORA(sel_fwd)(int64_t B, int64_t L, int64_t N, int is_complex, const REAL* lam,
                  const REAL* v, const REAL* x0, REAL* out) {
    /* one task per (row, 64-lane tile), time outermost inside the task so that every step
     * touches one contiguous run, as selective_c.py:44-76 does (TILE = 64) */
    const int64_t TILE = 64, nt = (N + TILE - 1) / TILE;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < B * nt; ++i) {
        const int64_t b = i / nt, n0 = (i % nt) * TILE;
        const int nw = (int)((N - n0) < TILE ? (N - n0) : TILE);
        REAL xr[64], xi[64];
        if (is_complex) {
            for (int j = 0; j < nw; ++j) {
                xr[j] = x0 ? x0[2 * (b * N + n0 + j)] : (REAL)0;
                xi[j] = x0 ? x0[2 * (b * N + n0 + j) + 1] : (REAL)0;
            }
            for (int64_t t = 0; t < L; ++t) {
                const int64_t p = 2 * ((b * L + t) * N + n0);
                for (int j = 0; j < nw; ++j) {
                    const REAL ar = lam[p + 2 * j], ai = lam[p + 2 * j + 1];
                    const REAL nr = ar * xr[j] - ai * xi[j] + v[p + 2 * j];
                    xi[j] = ar * xi[j] + ai * xr[j] + v[p + 2 * j + 1];
                    xr[j] = nr;
                    out[p + 2 * j] = xr[j];
                    out[p + 2 * j + 1] = xi[j];
                }
            }
        } else {
            for (int j = 0; j < nw; ++j) xr[j] = x0 ? x0[b * N + n0 + j] : (REAL)0;
            for (int64_t t = 0; t < L; ++t) {
                const int64_t p = (b * L + t) * N + n0;
                const REAL* lr = lam + p;
                const REAL* vr = v + p;
                REAL* orr = out + p;
                for (int j = 0; j < nw; ++j) {
                    xr[j] = lr[j] * xr[j] + vr[j];
                    orr[j] = xr[j];
                }
            }
        }
    }
}

/* Adjoint of S2: G_t = g_t + conj(a_{t+1}) G_{t+1}; gv = G; glam_t = G_t conj(x_{t-1});
 * gx0 = conj(a_0) G_0 (only when x0 != NULL).
 * Follows tsfast/models/_core/scan.py:173-195 and selective_c.py:78-120 (sel_bwd). */
void ORA(sel_bwd)(int64_t B, int64_t L, int64_t N, int is_complex, const REAL* g,
                  const REAL* lam, const REAL* out, const REAL* x0, REAL* glam, REAL* gv,
                  REAL* gx0) {
    const int64_t TILE = 64, nt = (N + TILE - 1) / TILE;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < B * nt; ++i) {
        const int64_t b = i / nt, n0 = (i % nt) * TILE;
        const int nw = (int)((N - n0) < TILE ? (N - n0) : TILE);
        REAL Gr[64], Gi[64];
        for (int j = 0; j < nw; ++j) Gr[j] = Gi[j] = 0;
        if (is_complex) {
            for (int64_t t = L - 1; t >= 0; --t) {
                const int64_t p = 2 * ((b * L + t) * N + n0);
                for (int j = 0; j < nw; ++j) {
                    const int64_t q = p + 2 * j, ln = b * N + n0 + j;
                    if (t + 1 < L) {
                        const REAL ar = lam[q + 2 * N], ai = -lam[q + 2 * N + 1];
                        const REAL nr = g[q] + ar * Gr[j] - ai * Gi[j];
                        Gi[j] = g[q + 1] + ar * Gi[j] + ai * Gr[j];
                        Gr[j] = nr;
                    } else {
                        Gr[j] = g[q];
                        Gi[j] = g[q + 1];
                    }
                    gv[q] = Gr[j];
                    gv[q + 1] = Gi[j];
                    REAL xr, xi;
                    if (t > 0) {
                        xr = out[q - 2 * N];
                        xi = out[q - 2 * N + 1];
                    } else {
                        xr = x0 ? x0[2 * ln] : (REAL)0;
                        xi = x0 ? x0[2 * ln + 1] : (REAL)0;
                    }
                    glam[q] = Gr[j] * xr + Gi[j] * xi;
                    glam[q + 1] = Gi[j] * xr - Gr[j] * xi;
                    if (t == 0 && x0) {
                        const REAL ar = lam[q], ai = -lam[q + 1];
                        gx0[2 * ln] = ar * Gr[j] - ai * Gi[j];
                        gx0[2 * ln + 1] = ar * Gi[j] + ai * Gr[j];
                    }
                }
            }
        } else {
            for (int64_t t = L - 1; t >= 0; --t) {
                const int64_t p = (b * L + t) * N + n0;
                const REAL* gr = g + p;
                REAL* gvr = gv + p;
                REAL* glr = glam + p;
                if (t + 1 < L) {
                    const REAL* ln_ = lam + p + N;
                    for (int j = 0; j < nw; ++j) Gr[j] = gr[j] + ln_[j] * Gr[j];
                } else {
                    for (int j = 0; j < nw; ++j) Gr[j] = gr[j];
                }
                for (int j = 0; j < nw; ++j) gvr[j] = Gr[j];
                if (t > 0) {
                    const REAL* op = out + p - N;
                    for (int j = 0; j < nw; ++j) glr[j] = Gr[j] * op[j];
                } else {
                    for (int j = 0; j < nw; ++j) glr[j] = Gr[j] * (x0 ? x0[b * N + n0 + j] : (REAL)0);
                    if (x0)
                        for (int j = 0; j < nw; ++j) gx0[b * N + n0 + j] = lam[p + j] * Gr[j];
                }
            }
        }
    }
}

/* ------------------------------------------------------------------ S3: fused Mamba section */
static inline REAL ORA(softplus)(REAL x) { return x > (REAL)20 ? x : LOG1P(EXP(x)); }
static inline REAL ORA(sigmoid)(REAL x) { return (REAL)1 / ((REAL)1 + EXP(-x)); }

/* h_t = exp(delta_t A) h_{t-1} + delta_t u_t B_t, delta = softplus(draw);
 * out_t = (h_t . C_t + Dp u_t) * z_t * sigmoid(z_t); hlast = h_L.
 * draw/u/z/out [B,L,D]; A [D,N]; Bt/Ct [B,L,N]; Dp [D]; h0/hlast [B,D,N] (h0 may be NULL).
 * Follows tsfast/models/architectures/mamba/backend_c.py:106-144 (mamba_fwd), with libm exp in
 * place of its polynomial fast_expf (backend_c.py:55-77). */
void ORA(mamba_fwd)(int64_t B, int64_t L, int64_t D, int64_t N, const REAL* draw, const REAL* A,
                    const REAL* Bt, const REAL* Ct, const REAL* u, const REAL* z, const REAL* Dp,
                    const REAL* h0, REAL* out, REAL* hlast) {
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t b = 0; b < B; ++b) {
        for (int64_t d = 0; d < D; ++d) {
            REAL h[256];
            const REAL* Ad = A + d * N;
            for (int64_t n = 0; n < N; ++n) h[n] = h0 ? h0[(b * D + d) * N + n] : (REAL)0;
            for (int64_t t = 0; t < L; ++t) {
                const REAL* Btt = Bt + (b * L + t) * N;
                const REAL* Ctt = Ct + (b * L + t) * N;
                const int64_t pd = (b * L + t) * D + d;
                const REAL delta = ORA(softplus)(draw[pd]);
                const REAL uu = u[pd], du = delta * uu;
                REAL acc = 0;
                for (int64_t n = 0; n < N; ++n) {
                    const REAL hv = EXP(delta * Ad[n]) * h[n] + du * Btt[n];
                    h[n] = hv;
                    acc += hv * Ctt[n];
                }
                const REAL zz = z[pd];
                out[pd] = (acc + Dp[d] * uu) * zz * ORA(sigmoid)(zz);
            }
            for (int64_t n = 0; n < N; ++n) hlast[(b * D + d) * N + n] = h[n];
        }
    }
}

/* Adjoint of S3 (formulas of mamba/backend_c.py:150-245 and mamba/mamba_triton.py:163-286):
 * gy = gout z sig(z); gz = gout y sig (1 + z (1 - sig)); G_t = gy_t C_t + lam_{t+1} G_{t+1}
 * (G_L = ghlast or 0); lam_t h_{t-1} = h_t - v_t; gC, gB reduced over d; gA, gDp over (b,t);
 * gdraw = gdelta * sigmoid(draw); gh0 = lam_1 G_1.  Each (b,d) task recomputes its full state
 * trajectory instead of walking checkpoints; the d-reductions go through per-d partial rows
 * summed in a fixed order, so the result is deterministic.
 * scratch_hs: B*D*L*N REALs is too large at benchmark sizes, so tasks allocate their own
 * L*N trajectory. gBt/gCt [B,L,N], gA [D,N], gDp [D], gh0 [B,D,N] or NULL. */
void ORA(mamba_bwd)(int64_t B, int64_t L, int64_t D, int64_t N, const REAL* draw, const REAL* A,
                    const REAL* Bt, const REAL* Ct, const REAL* u, const REAL* z, const REAL* Dp,
                    const REAL* h0, const REAL* gout, const REAL* ghlast, REAL* gdraw, REAL* gA,
                    REAL* gBt, REAL* gCt, REAL* gu, REAL* gz, REAL* gDp, REAL* gh0) {
    const int64_t BD = 8; /* channel block, as in backend_c.py:48 */
    const int64_t ndb = (D + BD - 1) / BD;
    REAL* gA_part = (REAL*)malloc(sizeof(REAL) * (size_t)(B * D * N));
    REAL* gDp_part = (REAL*)malloc(sizeof(REAL) * (size_t)(B * D));
    REAL* gB_part = (REAL*)calloc((size_t)(ndb * B * L * N), sizeof(REAL));
    REAL* gC_part = (REAL*)calloc((size_t)(ndb * B * L * N), sizeof(REAL));
#pragma omp parallel for collapse(2) schedule(dynamic)
    for (int64_t b = 0; b < B; ++b) {
        for (int64_t blk = 0; blk < ndb; ++blk) {
            REAL* hs = (REAL*)malloc(sizeof(REAL) * (size_t)(L * N));
            REAL* gBp = gB_part + (blk * B + b) * L * N;
            REAL* gCp = gC_part + (blk * B + b) * L * N;
            const int64_t d1 = (blk + 1) * BD < D ? (blk + 1) * BD : D;
            for (int64_t d = blk * BD; d < d1; ++d) {
                const REAL* Ad = A + d * N;
                REAL G[256], gAacc[256], hcur[256];
                REAL gDpacc = 0;
                for (int64_t n = 0; n < N; ++n) {
                    hcur[n] = h0 ? h0[(b * D + d) * N + n] : (REAL)0;
                    G[n] = ghlast ? ghlast[(b * D + d) * N + n] : (REAL)0;
                    gAacc[n] = 0;
                }
                for (int64_t t = 0; t < L; ++t) { /* recompute the state trajectory */
                    const REAL* Btt = Bt + (b * L + t) * N;
                    const int64_t pd = (b * L + t) * D + d;
                    const REAL delta = ORA(softplus)(draw[pd]);
                    const REAL du = delta * u[pd];
                    for (int64_t n = 0; n < N; ++n) {
                        hcur[n] = EXP(delta * Ad[n]) * hcur[n] + du * Btt[n];
                        hs[t * N + n] = hcur[n];
                    }
                }
                for (int64_t t = L - 1; t >= 0; --t) {
                    const REAL* Btt = Bt + (b * L + t) * N;
                    const REAL* Ctt = Ct + (b * L + t) * N;
                    const REAL* hv = hs + t * N;
                    const int64_t pd = (b * L + t) * D + d;
                    const REAL delta = ORA(softplus)(draw[pd]);
                    const REAL uu = u[pd], zz = z[pd], du = delta * uu;
                    REAL y = Dp[d] * uu;
                    for (int64_t n = 0; n < N; ++n) y += hv[n] * Ctt[n];
                    const REAL sig = ORA(sigmoid)(zz), go = gout[pd];
                    const REAL gy = go * zz * sig;
                    gz[pd] = go * y * sig * ((REAL)1 + zz * ((REAL)1 - sig));
                    gDpacc += gy * uu;
                    if (t + 1 < L) {
                        const REAL dn = ORA(softplus)(draw[pd + D]);
                        for (int64_t n = 0; n < N; ++n) G[n] = gy * Ctt[n] + EXP(dn * Ad[n]) * G[n];
                    } else {
                        for (int64_t n = 0; n < N; ++n) G[n] = gy * Ctt[n] + G[n];
                    }
                    REAL gdelta = 0, gus = 0;
                    for (int64_t n = 0; n < N; ++n) {
                        const REAL lam_hprev = hv[n] - du * Btt[n], gg = G[n];
                        gCp[t * N + n] += gy * hv[n];
                        gBp[t * N + n] += gg * du;
                        gAacc[n] += gg * lam_hprev * delta;
                        gdelta += gg * (Ad[n] * lam_hprev + uu * Btt[n]);
                        gus += gg * Btt[n];
                    }
                    gdraw[pd] = gdelta * ORA(sigmoid)(draw[pd]);
                    gu[pd] = delta * gus + gy * Dp[d];
                }
                gDp_part[b * D + d] = gDpacc;
                for (int64_t n = 0; n < N; ++n) gA_part[(b * D + d) * N + n] = gAacc[n];
                if (gh0) {
                    const REAL d0 = ORA(softplus)(draw[b * L * D + d]);
                    for (int64_t n = 0; n < N; ++n) gh0[(b * D + d) * N + n] = EXP(d0 * Ad[n]) * G[n];
                }
            }
            free(hs);
        }
    }
    /* fixed-order reductions (mamba_triton.py:450-459 sums the partial buffers the same way) */
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < D * N; ++i) {
        REAL s = 0;
        for (int64_t b = 0; b < B; ++b) s += gA_part[b * D * N + i];
        gA[i] = s;
    }
    for (int64_t d = 0; d < D; ++d) {
        REAL s = 0;
        for (int64_t b = 0; b < B; ++b) s += gDp_part[b * D + d];
        gDp[d] = s;
    }
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < B * L * N; ++i) {
        REAL sb = 0, sc = 0;
        for (int64_t k = 0; k < ndb; ++k) {
            sb += gB_part[k * B * L * N + i];
            sc += gC_part[k * B * L * N + i];
        }
        gBt[i] = sb;
        gCt[i] = sc;
    }
    free(gA_part);
    free(gDp_part);
    free(gB_part);
    free(gC_part);
}

/* ------------------------------------------------------------------ S4: all-pole IIR
 * y_t = w_t - sum_{i=1..na} a_i y_{t-i}, y_{-1-j} = y0[j] (newest first) or 0.
 * a, y0 [lanes,na]; w, y [lanes,L] (time contiguous).
 * Follows tsfast/models/architectures/dynonet/allpole_triton.py:71-95 (generated allpole_fwd). */
void ORA(allpole_fwd)(int64_t lanes, int64_t L, int64_t na, const REAL* a, const REAL* w,
                      const REAL* y0, REAL* y) {
#pragma omp parallel for schedule(static)
    for (int64_t ln = 0; ln < lanes; ++ln) {
        REAL s[16], c[16];
        for (int64_t k = 0; k < na; ++k) {
            c[k] = a[ln * na + k];
            s[k] = y0 ? y0[ln * na + k] : (REAL)0;
        }
        for (int64_t t = 0; t < L; ++t) {
            REAL acc = 0;
            for (int64_t k = 0; k < na; ++k) acc += c[k] * s[k];
            const REAL yt = w[ln * L + t] - acc;
            y[ln * L + t] = yt;
            for (int64_t k = na - 1; k > 0; --k) s[k] = s[k - 1];
            s[0] = yt;
        }
    }
}

/* Adjoint of S4: G_t = g_t - sum_i a_i G_{t+i}; gw = G;
 * grad_a_i = -sum_u G_{u+i} y_u - sum_{k=1..i} G_{i-k} y0[k-1];
 * grad_y0_j = -sum_{i=j+1..na} a_i G_{i-1-j} (only when y0 != NULL).
 * Follows allpole_triton.py:97-123 (generated allpole_bwd) and the head corrections of
 * allpole_triton.py:199-213. */
void ORA(allpole_bwd)(int64_t lanes, int64_t L, int64_t na, const REAL* g, const REAL* a,
                      const REAL* y, const REAL* y0, REAL* ga, REAL* gw, REAL* gy0) {
#pragma omp parallel for schedule(static)
    for (int64_t ln = 0; ln < lanes; ++ln) {
        REAL s[16], c[16], acc_a[16];
        for (int64_t k = 0; k < na; ++k) {
            c[k] = a[ln * na + k];
            s[k] = 0;
            acc_a[k] = 0;
        }
        for (int64_t t = L - 1; t >= 0; --t) {
            REAL acc = 0;
            for (int64_t k = 0; k < na; ++k) acc += c[k] * s[k];
            const REAL G = g[ln * L + t] - acc;
            gw[ln * L + t] = G;
            const REAL yu = y[ln * L + t];
            for (int64_t k = 0; k < na; ++k) acc_a[k] += s[k] * yu; /* s[k] = G_{t+1+k} */
            for (int64_t k = na - 1; k > 0; --k) s[k] = s[k - 1];
            s[0] = G;
        }
        for (int64_t i = 1; i <= na; ++i) {
            REAL v = acc_a[i - 1];
            if (y0)
                for (int64_t k = 1; k <= i; ++k)
                    if (i - k < L) v += gw[ln * L + (i - k)] * y0[ln * na + k - 1];
            ga[ln * na + i - 1] = -v;
        }
        if (y0) {
            for (int64_t j = 0; j < na; ++j) {
                REAL v = 0;
                for (int64_t i = j + 1; i <= na; ++i)
                    if (i - 1 - j < L) v += c[i - 1] * gw[ln * L + (i - 1 - j)];
                gy0[ln * na + j] = -v;
            }
        }
    }
}

/* ------------------------------------------------------------------ Mamba causal depthwise conv + SiLU
 * out[b,t,d] = silu(bias[d] + sum_k w[d,k] * X(b, t-(K-1)+k, d)), X(s) = x[b,s,d] for s >= 0 and
 * tail[b,d,s+K-1] for s < 0 (the carried left context).  x/out [B,L,D] dense, tail [B,D,K-1],
 * w [D,K], bias [D] or NULL.  Follows _causal_depthwise_silu of
 * tsfast/models/architectures/mamba/core.py:38-58 (the eager definition the fused Triton kernel
 * mamba/conv_triton.py:81-119 is tested against). */
static inline REAL ORA(conv_x)(const REAL* x, const REAL* tail, int64_t b, int64_t s, int64_t d, int64_t L,
                               int64_t D, int64_t K) {
    return s >= 0 ? x[(b * L + s) * D + d] : tail[(b * D + d) * (K - 1) + s + K - 1];
}

void ORA(conv_fwd)(int64_t B, int64_t L, int64_t D, int64_t K, const REAL* x, const REAL* tail,
                   const REAL* w, const REAL* bias, REAL* out) {
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t b = 0; b < B; ++b) {
        for (int64_t t = 0; t < L; ++t) {
            for (int64_t d = 0; d < D; ++d) {
                REAL p = bias ? bias[d] : (REAL)0;
                for (int64_t k = 0; k < K; ++k) p += w[d * K + k] * ORA(conv_x)(x, tail, b, t - (K - 1) + k, d, L, D, K);
                out[(b * L + t) * D + d] = p * ORA(sigmoid)(p);
            }
        }
    }
}

/* Adjoint (mamba/conv_triton.py:125-191,232-281): gpre = gy * sig(p) * (1 + p (1 - sig(p)));
 * gx[b,s,d] = sum_k w[d,k] gpre[b, s+K-1-k, d]; gtail[b,d,j] = sum_k w[d,k] gpre[b, j-k, d];
 * gw[d,k] = sum_{b,t} gpre[b,t,d] X(b, t-(K-1)+k, d); gb[d] = sum_{b,t} gpre (when bias != NULL). */
void ORA(conv_bwd)(int64_t B, int64_t L, int64_t D, int64_t K, const REAL* gy, const REAL* x,
                   const REAL* tail, const REAL* w, const REAL* bias, REAL* gx, REAL* gtail, REAL* gw,
                   REAL* gb) {
    REAL* gpre = (REAL*)malloc(sizeof(REAL) * (size_t)(B * L * D > 0 ? B * L * D : 1));
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t b = 0; b < B; ++b) {
        for (int64_t t = 0; t < L; ++t) {
            for (int64_t d = 0; d < D; ++d) {
                REAL p = bias ? bias[d] : (REAL)0;
                for (int64_t k = 0; k < K; ++k) p += w[d * K + k] * ORA(conv_x)(x, tail, b, t - (K - 1) + k, d, L, D, K);
                const REAL sg = ORA(sigmoid)(p);
                gpre[(b * L + t) * D + d] = gy[(b * L + t) * D + d] * sg * ((REAL)1 + p * ((REAL)1 - sg));
            }
        }
    }
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t b = 0; b < B; ++b) {
        for (int64_t s = 0; s < L; ++s) {
            for (int64_t d = 0; d < D; ++d) {
                REAL v = 0;
                for (int64_t k = 0; k < K; ++k) {
                    const int64_t t = s + K - 1 - k;
                    if (t < L) v += w[d * K + k] * gpre[(b * L + t) * D + d];
                }
                gx[(b * L + s) * D + d] = v;
            }
        }
    }
    for (int64_t b = 0; b < B; ++b)
        for (int64_t d = 0; d < D; ++d)
            for (int64_t j = 0; j < K - 1; ++j) {
                REAL v = 0;
                for (int64_t k = 0; k <= j; ++k)
                    if (j - k < L) v += w[d * K + k] * gpre[(b * L + (j - k)) * D + d];
                gtail[(b * D + d) * (K - 1) + j] = v;
            }
#pragma omp parallel for schedule(static)
    for (int64_t d = 0; d < D; ++d) {
        REAL sb = 0;
        for (int64_t k = 0; k < K; ++k) {
            REAL sw = 0;
            for (int64_t b = 0; b < B; ++b)
                for (int64_t t = 0; t < L; ++t)
                    sw += gpre[(b * L + t) * D + d] * ORA(conv_x)(x, tail, b, t - (K - 1) + k, d, L, D, K);
            gw[d * K + k] = sw;
        }
        if (gb) {
            for (int64_t b = 0; b < B; ++b)
                for (int64_t t = 0; t < L; ++t) sb += gpre[(b * L + t) * D + d];
            gb[d] = sb;
        }
    }
    free(gpre);
}
