/*
 * KLA scan oracle -- type-generic body. TEST INFRASTRUCTURE ONLY: a CPU
 * restatement of the reference algorithm used as the checker in tests, in the
 * smoke check and as the timed CPU baseline. Nothing in the product path may
 * call it.
 *
 * Included twice by kla_oracle.c with REAL = double / float and SUFFIX = f64 /
 * f32. Every function follows the reference's sequential definition of the
 * filter:
 *
 *   step      src/kla/ops/kla_ops.py:293-331   (kla_step)
 *   scan      src/kla/ops/kla_ops.py:334-362   (kla_scan_reference: a loop of
 *             kla_step over the sequence)
 *   floors    src/kla/ops/kla_ops.py:43-44, 181-185, 310-323 (EPS, P_MIN and
 *             where each clamp_min sits)
 *   adjoint   reverse-mode differentiation of exactly those statements, with
 *             torch's clamp_min subgradient (1 where input >= floor, else 0).
 *             The reference writes the same adjoint once by hand, in
 *             src/kla/ops/kernels/mps/fused_kla_scan.metal:212-323, in a
 *             different algebraic form (leaf coefficients A, C, den = C*lam'+1);
 *             this file differentiates the plain kla_step statements instead.
 *
 * Layout (all contiguous, row-major):
 *   v, lambda_v, y, y_var, dy, dyvar, dv, dlambda_v : [B, L, M]
 *   k, q, dk, dq                                    : [B, L, S]
 *   a, p, da, dp                                    : [M, S]
 *   lam0, eta0, lam_fin, eta_fin and their grads    : [B, M, S]
 */

#define CAT_(a, b) a##_##b
#define CAT(a, b) CAT_(a, b)
#define FN(name) CAT(name, SUFFIX)

/* One filter step for one (b, m, s) lane. kla_ops.py:310-327. */
static inline void FN(lane_step)(REAL lam_prev, REAL eta_prev, REAL phi, REAL r,
                                 REAL a, REAL a2, REAL p, REAL *lam, REAL *eta,
                                 REAL *inv_out)
{
    REAL den = a2 + p * lam_prev;           /* kla_ops.py:319 */
    if (den < (REAL)KLA_EPS) den = (REAL)KLA_EPS;
    REAL inv = (REAL)1 / den;
    *lam = lam_prev * inv + phi;            /* kla_ops.py:320 */
    *eta = (a * inv) * eta_prev + r;        /* kla_ops.py:321 */
    *inv_out = inv;
}

/*
 * Forward scan. lam0/eta0 may be NULL (unit prior, kla_ops.py:54-61).
 * floor_phi != 0 floors phi at EPS as kla_step does (kla_ops.py:310-312);
 * floor_phi == 0 leaves it unfloored as the default parallel path does
 * (kla_ops.py:238, rationale kla_ops.py:145-178).
 */
int FN(kla_oracle_fwd)(int64_t B, int64_t L, int64_t M, int64_t S,
                       const REAL *v, const REAL *lambda_v, const REAL *k,
                       const REAL *q, const REAL *a, const REAL *p,
                       const REAL *lam0, const REAL *eta0, int prior,
                       int floor_phi, REAL *y, REAL *y_var, REAL *lam_fin,
                       REAL *eta_fin)
{
    if (B < 0 || L < 0 || M < 0 || S < 0) return 1;
    int64_t BM = B * M;
#pragma omp parallel for schedule(static)
    for (int64_t bm = 0; bm < BM; ++bm) {
        int64_t b = bm / M, m = bm % M;
        REAL *lam = (REAL *)malloc(sizeof(REAL) * (size_t)(2 * S + 1));
        REAL *eta = lam + S;
        for (int64_t s = 0; s < S; ++s) {
            lam[s] = lam0 ? lam0[(b * M + m) * S + s] : (REAL)1;
            eta[s] = eta0 ? eta0[(b * M + m) * S + s] : (REAL)0;
        }
        for (int64_t t = 0; t < L; ++t) {
            REAL lv = lambda_v[(b * L + t) * M + m];
            REAL vl = v[(b * L + t) * M + m] * lv;   /* kla_ops.py:313 */
            const REAL *kt = k + (b * L + t) * S;
            const REAL *qt = q + (b * L + t) * S;
            REAL ys = 0, yvs = 0;
            for (int64_t s = 0; s < S; ++s) {
                REAL as = a[m * S + s];
                REAL ps = p[m * S + s];
                if (ps < (REAL)KLA_PMIN) ps = (REAL)KLA_PMIN;   /* :316 */
                REAL a2 = as * as;
                if (a2 < (REAL)KLA_EPS) a2 = (REAL)KLA_EPS;     /* :317 */
                REAL phi = lv * kt[s] * kt[s];
                if (floor_phi && phi < (REAL)KLA_EPS) phi = (REAL)KLA_EPS;
                REAL r = vl * kt[s];
                REAL inv;
                FN(lane_step)(lam[s], eta[s], phi, r, as, a2, ps, &lam[s],
                              &eta[s], &inv);
                REAL lc = lam[s] < (REAL)KLA_EPS ? (REAL)KLA_EPS : lam[s];
                REAL var = (REAL)1 / lc;                        /* :323 */
                REAL mean = eta[s] * var;                       /* :324 */
                if (prior) {                                    /* :325-327 */
                    mean = as * mean;
                    var = a2 * var + ps;
                }
                ys += mean * qt[s];                             /* :329 */
                yvs += var * qt[s] * qt[s];                     /* :330 */
            }
            y[(b * L + t) * M + m] = ys;
            y_var[(b * L + t) * M + m] = yvs;
        }
        for (int64_t s = 0; s < S; ++s) {
            lam_fin[(b * M + m) * S + s] = lam[s];
            eta_fin[(b * M + m) * S + s] = eta[s];
        }
        free(lam);
    }
    return 0;
}

/*
 * Backward scan: gradients of sum(dy*y) + sum(dyvar*y_var) + sum(dlam_fin*
 * lam_fin) + sum(deta_fin*eta_fin) with respect to every input. dyvar,
 * dlam_fin, deta_fin, lam0, eta0 may be NULL (zero / unit prior).
 */
int FN(kla_oracle_bwd)(int64_t B, int64_t L, int64_t M, int64_t S,
                       const REAL *v, const REAL *lambda_v, const REAL *k,
                       const REAL *q, const REAL *a, const REAL *p,
                       const REAL *lam0, const REAL *eta0, int prior,
                       int floor_phi, const REAL *dy, const REAL *dyvar,
                       const REAL *dlam_fin, const REAL *deta_fin, REAL *dv,
                       REAL *dlambda_v, REAL *dk, REAL *dq, REAL *da, REAL *dp,
                       REAL *dlam0, REAL *deta0)
{
    if (B < 0 || L < 0 || M < 0 || S < 0) return 1;
    memset(dk, 0, sizeof(REAL) * (size_t)(B * L * S));
    memset(dq, 0, sizeof(REAL) * (size_t)(B * L * S));
    memset(da, 0, sizeof(REAL) * (size_t)(M * S));
    memset(dp, 0, sizeof(REAL) * (size_t)(M * S));
    for (int64_t b = 0; b < B; ++b) {
#pragma omp parallel
        {
            /* thread-private partial sums of dk, dq over this thread's m */
            REAL *dk_loc = (REAL *)calloc((size_t)(2 * L * S + 1), sizeof(REAL));
            REAL *dq_loc = dk_loc + L * S;
            REAL *lam_h = (REAL *)malloc(sizeof(REAL) * (size_t)(2 * (L + 1) * S + 1));
            REAL *eta_h = lam_h + (L + 1) * S;
#pragma omp for schedule(static)
            for (int64_t m = 0; m < M; ++m) {
                /* replay: lam_h[t], eta_h[t] = state BEFORE step t */
                for (int64_t s = 0; s < S; ++s) {
                    lam_h[s] = lam0 ? lam0[(b * M + m) * S + s] : (REAL)1;
                    eta_h[s] = eta0 ? eta0[(b * M + m) * S + s] : (REAL)0;
                }
                for (int64_t t = 0; t < L; ++t) {
                    REAL lv = lambda_v[(b * L + t) * M + m];
                    REAL vl = v[(b * L + t) * M + m] * lv;
                    const REAL *kt = k + (b * L + t) * S;
                    for (int64_t s = 0; s < S; ++s) {
                        REAL as = a[m * S + s], ps = p[m * S + s];
                        if (ps < (REAL)KLA_PMIN) ps = (REAL)KLA_PMIN;
                        REAL a2 = as * as;
                        if (a2 < (REAL)KLA_EPS) a2 = (REAL)KLA_EPS;
                        REAL phi = lv * kt[s] * kt[s];
                        if (floor_phi && phi < (REAL)KLA_EPS) phi = (REAL)KLA_EPS;
                        REAL inv;
                        FN(lane_step)(lam_h[t * S + s], eta_h[t * S + s], phi,
                                      vl * kt[s], as, a2, ps,
                                      &lam_h[(t + 1) * S + s],
                                      &eta_h[(t + 1) * S + s], &inv);
                    }
                }
                /* reverse walk */
                for (int64_t s = 0; s < S; ++s) {
                    REAL as = a[m * S + s], ps_raw = p[m * S + s];
                    REAL ps = ps_raw < (REAL)KLA_PMIN ? (REAL)KLA_PMIN : ps_raw;
                    REAL a2_raw = as * as;
                    REAL a2 = a2_raw < (REAL)KLA_EPS ? (REAL)KLA_EPS : a2_raw;
                    REAL lam_bar = dlam_fin ? dlam_fin[(b * M + m) * S + s] : (REAL)0;
                    REAL eta_bar = deta_fin ? deta_fin[(b * M + m) * S + s] : (REAL)0;
                    REAL a_bar = 0, a2_bar = 0, p_bar = 0;
                    for (int64_t t = L - 1; t >= 0; --t) {
                        REAL lv = lambda_v[(b * L + t) * M + m];
                        REAL vv = v[(b * L + t) * M + m];
                        REAL vl = vv * lv;
                        REAL ks = k[(b * L + t) * S + s];
                        REAL qs = q[(b * L + t) * S + s];
                        REAL dyt = dy[(b * L + t) * M + m];
                        REAL dyvt = dyvar ? dyvar[(b * L + t) * M + m] : (REAL)0;
                        REAL lam_p = lam_h[t * S + s], eta_p = eta_h[t * S + s];
                        REAL lam_t = lam_h[(t + 1) * S + s];
                        REAL eta_t = eta_h[(t + 1) * S + s];
                        REAL den_raw = a2 + ps * lam_p;
                        REAL fd = den_raw >= (REAL)KLA_EPS ? (REAL)1 : (REAL)0;
                        REAL den = fd != 0 ? den_raw : (REAL)KLA_EPS;
                        REAL inv = (REAL)1 / den;
                        REAL alpha = as * inv;
                        REAL fl = lam_t >= (REAL)KLA_EPS ? (REAL)1 : (REAL)0;
                        REAL lc = fl != 0 ? lam_t : (REAL)KLA_EPS;
                        REAL var = (REAL)1 / lc;
                        REAL mean = eta_t * var;
                        REAL mean_o = prior ? as * mean : mean;
                        REAL var_o = prior ? a2 * var + ps : var;
                        /* read-out */
                        REAL mean_o_bar = dyt * qs;
                        REAL var_o_bar = dyvt * qs * qs;
                        dq_loc[t * S + s] += dyt * mean_o + (REAL)2 * dyvt * qs * var_o;
                        REAL mean_bar, var_bar;
                        if (prior) {
                            mean_bar = mean_o_bar * as;
                            a_bar += mean_o_bar * mean;
                            var_bar = var_o_bar * a2;
                            a2_bar += var_o_bar * var;
                            p_bar += var_o_bar;
                        } else {
                            mean_bar = mean_o_bar;
                            var_bar = var_o_bar;
                        }
                        /* mean = eta * var ; var = 1/max(lam, EPS) */
                        eta_bar += mean_bar * var;
                        var_bar += mean_bar * eta_t;
                        lam_bar += fl * (-var_bar * var * var);
                        /* eta = alpha*eta' + r ; alpha = a*inv */
                        REAL alpha_bar = eta_bar * eta_p;
                        REAL r_bar = eta_bar;
                        REAL eta_bar_prev = eta_bar * alpha;
                        a_bar += alpha_bar * inv;
                        REAL inv_bar = alpha_bar * as;
                        /* lam = lam'*inv + phi */
                        REAL phi_bar = lam_bar;
                        REAL lam_bar_prev = lam_bar * inv;
                        inv_bar += lam_bar * lam_p;
                        /* inv = 1/max(den_raw, EPS) ; den_raw = a2 + p*lam' */
                        REAL den_bar = fd * (-inv_bar * inv * inv);
                        a2_bar += den_bar;
                        p_bar += den_bar * lam_p;
                        lam_bar_prev += den_bar * ps;
                        /* phi = [max](lambda_v*k^2) ; r = (v*lambda_v)*k */
                        REAL phi_raw = lv * ks * ks;
                        REAL fphi = (!floor_phi || phi_raw >= (REAL)KLA_EPS) ? (REAL)1 : (REAL)0;
                        REAL dlv = fphi * phi_bar * ks * ks;
                        REAL dvl = r_bar * ks;
                        dk_loc[t * S + s] += fphi * phi_bar * (REAL)2 * lv * ks + r_bar * vl;
                        /* each (b,t,m) is owned by this thread: accumulate over s */
                        if (s == 0) {
                            dv[(b * L + t) * M + m] = 0;
                            dlambda_v[(b * L + t) * M + m] = 0;
                        }
                        dv[(b * L + t) * M + m] += dvl * lv;
                        dlambda_v[(b * L + t) * M + m] += dlv + dvl * vv;
                        lam_bar = lam_bar_prev;
                        eta_bar = eta_bar_prev;
                    }
                    REAL da2_da = a2_raw >= (REAL)KLA_EPS ? (REAL)2 * as : (REAL)0;
                    /* b is the serial outer loop and m is owned by one thread */
                    da[m * S + s] += a_bar + a2_bar * da2_da;
                    dp[m * S + s] += ps_raw >= (REAL)KLA_PMIN ? p_bar : (REAL)0;
                    dlam0[(b * M + m) * S + s] = lam_bar;
                    deta0[(b * M + m) * S + s] = eta_bar;
                }
            }
#pragma omp critical
            {
                for (int64_t i = 0; i < L * S; ++i) {
                    dk[b * L * S + i] += dk_loc[i];
                    dq[b * L * S + i] += dq_loc[i];
                }
            }
            free(dk_loc);
            free(lam_h);
        }
    }
    return 0;
}

/* Single decode step, kla_ops.py:293-331 (phi always floored there). */
int FN(kla_oracle_step)(int64_t B, int64_t M, int64_t S, const REAL *v,
                        const REAL *lambda_v, const REAL *k, const REAL *q,
                        const REAL *a, const REAL *p, const REAL *lam,
                        const REAL *eta, int prior, REAL *y, REAL *y_var,
                        REAL *lam_out, REAL *eta_out)
{
    return FN(kla_oracle_fwd)(B, 1, M, S, v, lambda_v, k, q, a, p, lam, eta,
                              prior, 1, y, y_var, lam_out, eta_out);
}

#undef FN
#undef CAT
#undef CAT_
