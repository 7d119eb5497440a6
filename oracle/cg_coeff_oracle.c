/*
 * TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * Plain-C restatement of the Clebsch-Gordan coefficient the reference project computes in
 *   CGNet/ClebschGordan/ClebschGordan.cpp:360-394   (ClebschGordan::slowCG, CPU, used by the Python twin)
 *   CGNet/cudaCG/cudaCG_sparse.cu:33-57             (_naiveCG, the device copy of the same formula)
 * with the log-factorial table of CGNet/cudaCG/cudaCG_utils.cu:83-90 (running sum of log(i) in double).
 *
 * The formula is Racah's closed form for <l1 m1; l2 m2 | l m>, evaluated in log space:
 *   sqrt((2l+1) (l+l1-l2)! (l-l1+l2)! (l1+l2-l)! / (l1+l2+l+1)!)
 *   * sqrt((l+m)! (l-m)! (l1-m1)! (l1+m1)! (l2-m2)! (l2+m2)!)
 *   * sum_t (-1)^t / ( t! (l1+l2-l-t)! (l1-m1-t)! (l2+m2-t)! (l-l2+m1+t)! (l-l1-m2+t)! )
 * The reference multiplies by plusminus(l1-l2+m)^2, which is +1 for every argument, so no extra phase appears here.
 *
 * Pinned against: the reference's own compiled module (oracle/_ref, `make ref`) and sympy's exact coefficients, by
 * tests/test_oracle.py and the fixtures under tests/golden/.
 *
 * Only tests/, the smoke test and bench.py's CPU-baseline leg may load this library.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>

static double *g_logfact = NULL;
static int g_logfact_n = 0;

static void ensure_logfact(int n) {
    if (n <= g_logfact_n) return;
    double *v = (double *)calloc((size_t)n, sizeof(double));
    for (int i = 2; i < n; ++i) v[i] = v[i - 1] + log((double)i);
    free(g_logfact);
    g_logfact = v;
    g_logfact_n = n;
}

static inline double lf(int n) { return n < 2 ? 0.0 : g_logfact[n]; }

/* <l1 m1; l2 m2 | l m1+m2>; zero when the arguments violate a selection rule. */
double cg_oracle_coeff(int l1, int l2, int l, int m1, int m2) {
    const int m = m1 + m2;
    if (l1 < 0 || l2 < 0 || l < 0) return 0.0;
    if (abs(m1) > l1 || abs(m2) > l2 || abs(m) > l) return 0.0;
    if (l < abs(l1 - l2) || l > l1 + l2) return 0.0;
    ensure_logfact(2 * (l1 + l2 + l) + 8);

    const int a = l2 - m1 - l, b = l1 + m2 - l;           /* lower limits of t (besides 0) */
    const int c = l1 + l2 - l, d = l1 - m1, e = l2 + m2;  /* upper limits of t */
    int lo = 0; if (a > lo) lo = a; if (b > lo) lo = b;
    int hi = c; if (d < hi) hi = d; if (e < hi) hi = e;

    double logA = 0.5 * (log(2.0 * l + 1.0) + lf(l + l1 - l2) + lf(l - l1 + l2) + lf(l1 + l2 - l) - lf(l1 + l2 + l + 1));
    logA += 0.5 * (lf(l + m) + lf(l - m) + lf(l1 - m1) + lf(l1 + m1) + lf(l2 - m2) + lf(l2 + m2));
    double s = 0.0;
    for (int t = lo; t <= hi; ++t) {
        const double logB = lf(t) + lf(c - t) + lf(d - t) + lf(e - t) + lf(t - a) + lf(t - b);
        const double term = exp(logA - logB);
        s += (t & 1) ? -term : term;
    }
    return s;
}

/* Dense (2l+1) x (2l1+1)(2l2+1) matrix, row m+l, column (m1+l1)(2l2+1)+(m2+l2): the layout the reference's
 * `ClebschGordan.precompute` hands to its Python twin (CGNet/ClebschGordan/CGmodule.cpp:85-99). */
void cg_oracle_dense(int l1, int l2, int l, double *out) {
    const int n1 = 2 * l1 + 1, n2 = 2 * l2 + 1, n = 2 * l + 1;
    for (int i = 0; i < n * n1 * n2; ++i) out[i] = 0.0;
    for (int m1 = -l1; m1 <= l1; ++m1)
        for (int m2 = -l2; m2 <= l2; ++m2) {
            const int m = m1 + m2;
            if (abs(m) > l) continue;
            out[(size_t)(m + l) * n1 * n2 + (size_t)(m1 + l1) * n2 + (m2 + l2)] = cg_oracle_coeff(l1, l2, l, m1, m2);
        }
}

/* Band table of one triple, (2l+1) x (2l2+1), entry [m+l][m2+l2] = <l1 m-m2; l2 m2 | l m>, zero outside |m-m2|<=l1:
 * the layout of the reference's device table (CGNet/cudaCG/cudaCG_sparse.cu:81-88). Values are cast to fp32 there. */
void cg_oracle_band(int l1, int l2, int l, float *out) {
    const int n2 = 2 * l2 + 1, n = 2 * l + 1;
    for (int m = -l; m <= l; ++m)
        for (int m2 = -l2; m2 <= l2; ++m2) {
            const int m1 = m - m2;
            out[(size_t)(m + l) * n2 + (m2 + l2)] = (abs(m1) <= l1) ? (float)cg_oracle_coeff(l1, l2, l, m1, m2) : 0.0f;
        }
}
