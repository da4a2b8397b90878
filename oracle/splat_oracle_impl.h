/*
 * Body of the CPU oracle, included twice by splat_oracle.c with REAL = float and
 * REAL = double.  TEST INFRASTRUCTURE ONLY (see splat_oracle.c).
 *
 * Per-term arithmetic is done in REAL in the reference's operation order; sums
 * over gaussians / pixels are accumulated in double (torch sums pairwise, so a
 * double accumulator is the closest order-independent stand-in).
 */

/*
 * scales [M,2], rotations [M] -> inverse-covariance entries [M] each.
 * Follows src/igs/gs2d.py:549-580:
 *   R = [[cos,-sin],[sin,cos]]   (:551-557)
 *   S = diag(sx, sy)             (:561-563)
 *   RS = R S ; Sigma = RS RS^T   (:567-568)
 *   Minv = inverse(Sigma + eps I) (:572-573); entries [0,0], [0,1], [1,1] (:578-580)
 * The 2x2 inverse is the adjugate over the determinant (torch uses LU; same value
 * up to rounding).
 */
void SUF(oracle_cov_inv)(const REAL* scales, const REAL* rot, REAL eps, int64_t M,
                         REAL* c00, REAL* c01, REAL* c11) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < M; ++i) {
        REAL c = COS(rot[i]), s = SIN(rot[i]);
        REAL sx = scales[2 * i], sy = scales[2 * i + 1];
        /* RS = R * diag(sx, sy) */
        REAL rs00 = c * sx, rs01 = -s * sy;
        REAL rs10 = s * sx, rs11 = c * sy;
        /* Sigma = RS RS^T + eps I */
        REAL a = rs00 * rs00 + rs01 * rs01 + eps;
        REAL b = rs00 * rs10 + rs01 * rs11;
        REAL d = rs10 * rs10 + rs11 * rs11 + eps;
        REAL det = a * d - b * b;
        c00[i] = d / det;
        c01[i] = -b / det;
        c11[i] = a / det;
    }
}

/*
 * Reverse mode through oracle_cov_inv, written as the matrix chain autograd
 * walks (inverse -> add -> bmm -> bmm -> stack/cos/sin), not as a closed form:
 *   gM = [[g00, g01],[0, g11]]          (only [0,1] of the inverse is read, :579)
 *   gSigma = -M^T gM M^T                (inverse backward)
 *   gRS = (gSigma + gSigma^T) RS        (Sigma = RS RS^T)
 *   gR = gRS S^T ; gS = R^T gRS         (RS = R S)
 *   g_sx = gS[0,0]; g_sy = gS[1,1]; g_theta = sum_ij gR_ij dR_ij/dtheta
 */
void SUF(oracle_cov_inv_backward)(const REAL* scales, const REAL* rot, REAL eps, int64_t M,
                                  const REAL* g00, const REAL* g01, const REAL* g11,
                                  REAL* g_scales, REAL* g_rot) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < M; ++i) {
        REAL c = COS(rot[i]), s = SIN(rot[i]);
        REAL sx = scales[2 * i], sy = scales[2 * i + 1];
        REAL R[2][2] = {{c, -s}, {s, c}};
        REAL RS[2][2] = {{c * sx, -s * sy}, {s * sx, c * sy}};
        REAL Sg[2][2];
        for (int p = 0; p < 2; ++p)
            for (int q = 0; q < 2; ++q)
                Sg[p][q] = RS[p][0] * RS[q][0] + RS[p][1] * RS[q][1] + (p == q ? eps : (REAL)0);
        REAL det = Sg[0][0] * Sg[1][1] - Sg[0][1] * Sg[1][0];
        REAL Mi[2][2] = {{Sg[1][1] / det, -Sg[0][1] / det}, {-Sg[1][0] / det, Sg[0][0] / det}};
        REAL gM[2][2] = {{g00[i], g01[i]}, {(REAL)0, g11[i]}};
        /* T = M^T gM */
        REAL T[2][2], gSg[2][2];
        for (int p = 0; p < 2; ++p)
            for (int q = 0; q < 2; ++q) T[p][q] = Mi[0][p] * gM[0][q] + Mi[1][p] * gM[1][q];
        for (int p = 0; p < 2; ++p)
            for (int q = 0; q < 2; ++q) gSg[p][q] = -(T[p][0] * Mi[q][0] + T[p][1] * Mi[q][1]);
        REAL sym[2][2] = {{gSg[0][0] + gSg[0][0], gSg[0][1] + gSg[1][0]},
                          {gSg[1][0] + gSg[0][1], gSg[1][1] + gSg[1][1]}};
        REAL gRS[2][2];
        for (int p = 0; p < 2; ++p)
            for (int q = 0; q < 2; ++q) gRS[p][q] = sym[p][0] * RS[0][q] + sym[p][1] * RS[1][q];
        /* gR = gRS * diag(sx,sy)^T ; gS = R^T gRS (diagonal entries only) */
        REAL gR[2][2] = {{gRS[0][0] * sx, gRS[0][1] * sy}, {gRS[1][0] * sx, gRS[1][1] * sy}};
        g_scales[2 * i] = R[0][0] * gRS[0][0] + R[1][0] * gRS[1][0];
        g_scales[2 * i + 1] = R[0][1] * gRS[0][1] + R[1][1] * gRS[1][1];
        /* dR/dtheta = [[-s,-c],[c,-s]] */
        g_rot[i] = gR[0][0] * (-s) + gR[0][1] * (-c) + gR[1][0] * c + gR[1][1] * (-s);
    }
}

/*
 * Forward, src/igs/gs2d.py:296-323:
 *   w = exp(-0.5*(c00*dx^2 + c11*dy^2 + c01*(2*dx*dy))) * alpha   (:303-314)
 *   result += w * color ; weight_sum += w                          (:316-321)
 *   result /= (weight_sum + eps)                                   (:323)
 * wsum receives the sum WITHOUT eps, as saved for backward (:334).
 */
void SUF(oracle_forward)(const REAL* x, const REAL* y, const REAL* pos, const REAL* c00,
                         const REAL* c01, const REAL* c11, const REAL* alpha, const REAL* colors,
                         REAL eps, int B, int N, int H, int W, int C, REAL* out, REAL* wsum) {
    const int64_t HW = (int64_t)H * W;
#pragma omp parallel
    {
        double* acc = (double*)malloc(sizeof(double) * (size_t)(C > 0 ? C : 1));
#pragma omp for schedule(static) collapse(2)
        for (int b = 0; b < B; ++b) {
            for (int64_t p = 0; p < HW; ++p) {
                const REAL px = x[b * HW + p], py = y[b * HW + p];
                double s = 0.0;
                for (int c = 0; c < C; ++c) acc[c] = 0.0;
                for (int n = 0; n < N; ++n) {
                    const int64_t g = (int64_t)b * N + n;
                    REAL dx = px - pos[2 * g], dy = py - pos[2 * g + 1];
                    REAL dist = c00[g] * (dx * dx) + c11[g] * (dy * dy) + c01[g] * ((REAL)2 * dx * dy);
                    REAL w = EXP((REAL)-0.5 * dist) * alpha[g];
                    s += (double)w;
                    for (int c = 0; c < C; ++c) acc[c] += (double)(w * colors[g * C + c]);
                }
                REAL S = (REAL)s;
                wsum[b * HW + p] = S;
                for (int c = 0; c < C; ++c) out[((int64_t)b * C + c) * HW + p] = (REAL)acc[c] / (S + eps);
            }
        }
        free(acc);
    }
}

/*
 * Per-pixel upstream terms, src/igs/gs2d.py:369-371:
 *   S = weight_sum + eps
 *   gS = -(g*g).sum(c) / S^2     reference mode (mode 0)     (:370)
 *   gn = g / S                                              (:371)
 * mode 1 replaces gS with the derivative of out = R/S taken by autograd of the
 * dense formula (:24-44):  gS = -sum_c gn_c * out_c.
 */
static void SUF(pixel_terms)(const REAL* wsum, const REAL* out, const REAL* gout, REAL eps, int B,
                             int C, int64_t HW, int mode, REAL* gn, REAL* gS) {
#pragma omp parallel for schedule(static) collapse(2)
    for (int b = 0; b < B; ++b) {
        for (int64_t p = 0; p < HW; ++p) {
            REAL S = wsum[b * HW + p] + eps;
            REAL acc = 0;
            for (int c = 0; c < C; ++c) {
                int64_t i = ((int64_t)b * C + c) * HW + p;
                REAL g = gout[i];
                gn[i] = g / S;
                acc += (mode == 0) ? g * g : (g / S) * out[i];
            }
            gS[b * HW + p] = (mode == 0) ? -acc / (S * S) : -acc;
        }
    }
}

/*
 * Backward, src/igs/gs2d.py:374-453.  Outputs (any of gx, gy may be NULL to skip):
 *   gx, gy [B,H,W]; gpos [B,N,2]; g00,g01,g11 [B,N]; galpha [B,N]; gcolors [B,N,C]
 * `out` is only read in mode 1.
 */
void SUF(oracle_backward)(const REAL* x, const REAL* y, const REAL* pos, const REAL* c00,
                          const REAL* c01, const REAL* c11, const REAL* alpha, const REAL* colors,
                          const REAL* wsum, const REAL* out, const REAL* gout, REAL eps, int mode,
                          int B, int N, int H, int W, int C, REAL* gx, REAL* gy, REAL* gpos,
                          REAL* g00, REAL* g01, REAL* g11, REAL* galpha, REAL* gcolors) {
    const int64_t HW = (int64_t)H * W;
    REAL* gn = (REAL*)malloc(sizeof(REAL) * (size_t)((int64_t)B * C * HW + 1));
    REAL* gS = (REAL*)malloc(sizeof(REAL) * (size_t)((int64_t)B * HW + 1));
    SUF(pixel_terms)(wsum, out, gout, eps, B, C, HW, mode, gn, gS);

    /* per-gaussian sums over pixels */
#pragma omp parallel
    {
        double* dcol = (double*)malloc(sizeof(double) * (size_t)(C > 0 ? C : 1));
#pragma omp for schedule(static)
        for (int64_t g = 0; g < (int64_t)B * N; ++g) {
            const int b = (int)(g / N);
            const REAL gx0 = pos[2 * g], gy0 = pos[2 * g + 1];
            const REAL a00 = c00[g], a01 = c01[g], a11 = c11[g], al = alpha[g];
            double d_al = 0, d_px = 0, d_py = 0, d00 = 0, d01 = 0, d11 = 0;
            for (int c = 0; c < C; ++c) dcol[c] = 0.0;
            for (int64_t p = 0; p < HW; ++p) {
                REAL dx = x[b * HW + p] - gx0, dy = y[b * HW + p] - gy0;
                REAL dist = a00 * (dx * dx) + a11 * (dy * dy) + a01 * ((REAL)2 * dx * dy);  /* :393-397 */
                REAL e = EXP((REAL)-0.5 * dist);                                            /* :400 */
                REAL w = e * al;                                                            /* :403-405 */
                REAL A = 0;
                for (int c = 0; c < C; ++c) {
                    REAL gnc = gn[((int64_t)b * C + c) * HW + p];
                    A += gnc * colors[g * C + c];                                           /* :376-378 */
                    dcol[c] += (double)(gnc * w);                                           /* :406-408 */
                }
                REAL G = A + gS[b * HW + p];                                                /* :411-413 */
                d_al += (double)(G * e);                                                    /* :417-419 */
                REAL cf = G * w * (REAL)-0.5;                                               /* :422 */
                REAL gdx = cf * ((REAL)2 * a00 * dx + (REAL)2 * a01 * dy);                  /* :425-427 */
                REAL gdy = cf * ((REAL)2 * a11 * dy + (REAL)2 * a01 * dx);                  /* :428-430 */
                d_px -= (double)gdx;                                                        /* :437-442 */
                d_py -= (double)gdy;
                d00 += (double)(cf * (dx * dx));                                            /* :445-453 */
                d11 += (double)(cf * (dy * dy));
                d01 += (double)(cf * ((REAL)2 * dx * dy));
            }
            gpos[2 * g] = (REAL)d_px;
            gpos[2 * g + 1] = (REAL)d_py;
            g00[g] = (REAL)d00;
            g01[g] = (REAL)d01;
            g11[g] = (REAL)d11;
            galpha[g] = (REAL)d_al;
            for (int c = 0; c < C; ++c) gcolors[g * C + c] = (REAL)dcol[c];
        }
        free(dcol);
    }

    /* per-pixel sums over gaussians: gradients of the sample coordinates (:433-434) */
    if (gx && gy) {
#pragma omp parallel for schedule(static) collapse(2)
        for (int b = 0; b < B; ++b) {
            for (int64_t p = 0; p < HW; ++p) {
                const REAL px = x[b * HW + p], py = y[b * HW + p];
                double sx = 0, sy = 0;
                for (int n = 0; n < N; ++n) {
                    const int64_t g = (int64_t)b * N + n;
                    REAL dx = px - pos[2 * g], dy = py - pos[2 * g + 1];
                    REAL dist = c00[g] * (dx * dx) + c11[g] * (dy * dy) + c01[g] * ((REAL)2 * dx * dy);
                    REAL e = EXP((REAL)-0.5 * dist);
                    REAL w = e * alpha[g];
                    REAL A = 0;
                    for (int c = 0; c < C; ++c)
                        A += gn[((int64_t)b * C + c) * HW + p] * colors[g * C + c];
                    REAL cf = (A + gS[b * HW + p]) * w * (REAL)-0.5;
                    sx += (double)(cf * ((REAL)2 * c00[g] * dx + (REAL)2 * c01[g] * dy));
                    sy += (double)(cf * ((REAL)2 * c11[g] * dy + (REAL)2 * c01[g] * dx));
                }
                gx[b * HW + p] = (REAL)sx;
                gy[b * HW + p] = (REAL)sy;
            }
        }
    }
    free(gn);
    free(gS);
}
