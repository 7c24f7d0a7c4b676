/*
 * accb_oracle.c -- CPU restatement of the collective-operation semantics of
 * accelerate-cuda, used ONLY as the checker in tests, in the smoke test and as
 * the timed CPU baseline of the benchmark.  It is test infrastructure: nothing
 * in the product library links, loads or calls it.
 *
 * PARITY UNPINNED: the reference repository holds no test-suite and no golden
 * vectors apart from three worked examples in doc comments
 * (Data/Array/Accelerate/CUDA/CodeGen/PrefixSum.hs:149-153,162-166,176-180);
 * those are checked in tests/test_oracle.py.  The CPU semantics proper live in
 * the third-party package `accelerate` 1.0 (git b6c1621c, pinned in
 * stack-8.0.yaml:8-11), which is not vendored; this file restates the
 * published denotational semantics (Data.List-style scans, folds, forward
 * permutation with a combination function, stencils with boundary
 * conditions) and anchors each function on the reference's own call sites.
 *
 * Float paths accumulate in double so that they can serve as the float64
 * oracle for the float32 kernels; integer paths wrap modulo 2^32 / 2^64 like
 * the device code does.
 *
 * Every function has a sequential form (one host core; the evaluation order
 * of Accelerate's interpreter) and, where it is timed as a baseline, an
 * OpenMP form selected with nthreads > 1.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

ORC_API int orc_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ------------------------------------------------------------------------
 * foldAll (+) 0 (zipWith (*) xs ys)
 * One Fold node whose delayed producer is xs[i]*ys[i]
 * (CodeGen.hs:104, CodeGen/Reduction.hs:152,162); the seed is combined on the
 * right as f(acc, seed) (Reduction.hs:203-215).
 * ---------------------------------------------------------------------- */
ORC_API double orc_dot_f32(const float *xs, const float *ys, int64_t n, double seed, int nthreads) {
    double acc = 0.0;
    if (nthreads <= 1) {
        for (int64_t i = 0; i < n; ++i) acc += (double)xs[i] * (double)ys[i];
    } else {
#pragma omp parallel for reduction(+ : acc) num_threads(nthreads) schedule(static)
        for (int64_t i = 0; i < n; ++i) acc += (double)xs[i] * (double)ys[i];
    }
    return acc + seed;
}

/* The float32 evaluation order of a sequential interpreter: used only to
 * show how far plain float32 accumulation drifts from the float64 oracle. */
ORC_API float orc_dot_f32_seq32(const float *xs, const float *ys, int64_t n, float seed) {
    float acc = 0.0f;
    for (int64_t i = 0; i < n; ++i) acc = acc + xs[i] * ys[i];
    return acc + seed;
}

ORC_API double orc_sum_f32(const float *xs, int64_t n, double seed) {
    double acc = 0.0;
    for (int64_t i = 0; i < n; ++i) acc += (double)xs[i];
    return acc + seed;
}

/* ------------------------------------------------------------------------
 * fold (+) seed over the innermost dimension of a rows x cols matrix
 * (CodeGen/Reduction.hs:221-367): out[row] = f(rowsum, seed) (:333-336);
 * an empty innermost dimension fills the output with the seed (:351-362).
 * ---------------------------------------------------------------------- */
ORC_API void orc_fold_rows_f32(const float *m, int64_t rows, int64_t cols, double seed, double *out,
                               int nthreads) {
#pragma omp parallel for num_threads(nthreads > 1 ? nthreads : 1) schedule(static) if (nthreads > 1)
    for (int64_t r = 0; r < rows; ++r) {
        double acc = 0.0;
        const float *p = m + r * cols;
        for (int64_t c = 0; c < cols; ++c) acc += (double)p[c];
        out[r] = acc + seed;
    }
}

ORC_API void orc_fold_rows_i32(const int32_t *m, int64_t rows, int64_t cols, int32_t seed, int32_t *out) {
    for (int64_t r = 0; r < rows; ++r) {
        uint32_t acc = 0;
        for (int64_t c = 0; c < cols; ++c) acc += (uint32_t)m[r * cols + c];
        out[r] = (int32_t)(acc + (uint32_t)seed);
    }
}

/* ------------------------------------------------------------------------
 * foldSeg (+) seed: `offs` is the exclusive scan of the segment lengths,
 * length nseg+1 (Execute.hs:320-324); one result per segment
 * (CodeGen/Reduction.hs:421-574), seed on the right (:567-574).
 * ---------------------------------------------------------------------- */
ORC_API void orc_fold_seg_i32(const int32_t *xs, const int32_t *offs, int64_t nseg, int32_t seed,
                              int32_t *out) {
    for (int64_t s = 0; s < nseg; ++s) {
        uint32_t acc = 0;
        for (int64_t i = offs[s]; i < offs[s + 1]; ++i) acc += (uint32_t)xs[i];
        out[s] = (int32_t)(acc + (uint32_t)seed);
    }
}

ORC_API void orc_fold_seg_f32(const float *xs, const int32_t *offs, int64_t nseg, double seed, double *out) {
    for (int64_t s = 0; s < nseg; ++s) {
        double acc = 0.0;
        for (int64_t i = offs[s]; i < offs[s + 1]; ++i) acc += (double)xs[i];
        out[s] = acc + seed;
    }
}

/* ------------------------------------------------------------------------
 * Scans (CodeGen/PrefixSum.hs:137-198, Execute.hs:326-362).
 *   scanl  f z xs : length n+1, out[0] = z, out[n] = total
 *   scanl1 f   xs : length n, inclusive
 *   scanl' f z xs : (init (scanl f z xs), last (scanl f z xs))
 *   scanr / scanr1 / scanr' : the mirror images (total at index 0).
 * Integer addition wraps modulo 2^32.
 * ---------------------------------------------------------------------- */
ORC_API void orc_scanl_i32(const int32_t *xs, int64_t n, int32_t z, int32_t *out /* n+1 */) {
    uint32_t acc = (uint32_t)z;
    out[0] = z;
    for (int64_t i = 0; i < n; ++i) {
        acc += (uint32_t)xs[i];
        out[i + 1] = (int32_t)acc;
    }
}

/* Blocked two-level parallel form of the same scan (timed baseline only). */
ORC_API void orc_scanl_i32_par(const int32_t *xs, int64_t n, int32_t z, int32_t *out, int nthreads) {
    if (nthreads <= 1 || n < (1 << 16)) {
        orc_scanl_i32(xs, n, z, out);
        return;
    }
    uint32_t *tot = (uint32_t *)calloc((size_t)nthreads + 1, sizeof(uint32_t));
    int64_t chunk = (n + nthreads - 1) / nthreads;
#pragma omp parallel num_threads(nthreads)
    {
#ifdef _OPENMP
        int t = omp_get_thread_num();
#else
        int t = 0;
#endif
        int64_t lo = t * chunk, hi = lo + chunk > n ? n : lo + chunk;
        uint32_t s = 0;
        for (int64_t i = lo; i < hi; ++i) s += (uint32_t)xs[i];
        tot[t + 1] = s;
#pragma omp barrier
#pragma omp single
        {
            tot[0] = (uint32_t)z;
            for (int k = 1; k <= nthreads; ++k) tot[k] += tot[k - 1];
        }
        uint32_t acc = tot[t];
        if (t == 0) out[0] = z;
        for (int64_t i = lo; i < hi; ++i) {
            acc += (uint32_t)xs[i];
            out[i + 1] = (int32_t)acc;
        }
    }
    free(tot);
}

ORC_API void orc_scanl1_i32(const int32_t *xs, int64_t n, int32_t *out /* n */) {
    uint32_t acc = 0;
    for (int64_t i = 0; i < n; ++i) {
        acc += (uint32_t)xs[i];
        out[i] = (int32_t)acc;
    }
}

ORC_API void orc_scanl_prime_i32(const int32_t *xs, int64_t n, int32_t z, int32_t *out /* n */,
                                 int32_t *total) {
    uint32_t acc = (uint32_t)z;
    for (int64_t i = 0; i < n; ++i) {
        out[i] = (int32_t)acc;
        acc += (uint32_t)xs[i];
    }
    *total = (int32_t)acc;
}

ORC_API void orc_scanr_i32(const int32_t *xs, int64_t n, int32_t z, int32_t *out /* n+1 */) {
    uint32_t acc = (uint32_t)z;
    out[n] = z;
    for (int64_t i = n - 1; i >= 0; --i) {
        acc += (uint32_t)xs[i];
        out[i] = (int32_t)acc;
    }
}

ORC_API void orc_scanr1_i32(const int32_t *xs, int64_t n, int32_t *out /* n */) {
    uint32_t acc = 0;
    for (int64_t i = n - 1; i >= 0; --i) {
        acc += (uint32_t)xs[i];
        out[i] = (int32_t)acc;
    }
}

ORC_API void orc_scanr_prime_i32(const int32_t *xs, int64_t n, int32_t z, int32_t *out /* n */,
                                 int32_t *total) {
    uint32_t acc = (uint32_t)z;
    for (int64_t i = n - 1; i >= 0; --i) {
        out[i] = (int32_t)acc;
        acc += (uint32_t)xs[i];
    }
    *total = (int32_t)acc;
}

/* float scans with a double running value: the float64 oracle */
ORC_API void orc_scanl_f32(const float *xs, int64_t n, double z, double *out /* n+1 */) {
    double acc = z;
    out[0] = z;
    for (int64_t i = 0; i < n; ++i) {
        acc += (double)xs[i];
        out[i + 1] = acc;
    }
}

/* ------------------------------------------------------------------------
 * permute (+) defaults (\i -> index1 (keys!i)) (fill n 1)
 * (CodeGen/IndexSpace.hs:160-213; host side Execute.hs:396-408): the defaults
 * are copied into the result first, then every source element is combined
 * into its destination; an `ignore` destination (here: key < 0) is skipped
 * (IndexSpace.hs:200,229-233).  With (+) on Int32 the order is immaterial.
 * `weights` may be NULL for the fused `fill 1` source.
 * ---------------------------------------------------------------------- */
ORC_API void orc_permute_add_i32(const int32_t *keys, const int32_t *weights, int64_t n,
                                 const int32_t *defaults, int64_t nbins, int32_t *out, int nthreads) {
    memcpy(out, defaults, (size_t)nbins * sizeof(int32_t));
    if (nthreads <= 1) {
        for (int64_t i = 0; i < n; ++i) {
            int32_t k = keys[i];
            if (k < 0 || k >= nbins) continue;
            out[k] = (int32_t)((uint32_t)out[k] + (uint32_t)(weights ? weights[i] : 1));
        }
        return;
    }
#pragma omp parallel num_threads(nthreads)
    {
        uint32_t *priv = (uint32_t *)calloc((size_t)nbins, sizeof(uint32_t));
#pragma omp for schedule(static)
        for (int64_t i = 0; i < n; ++i) {
            int32_t k = keys[i];
            if (k < 0 || k >= nbins) continue;
            priv[k] += (uint32_t)(weights ? weights[i] : 1);
        }
#pragma omp critical
        for (int64_t b = 0; b < nbins; ++b) out[b] = (int32_t)((uint32_t)out[b] + priv[b]);
        free(priv);
    }
}

/* ------------------------------------------------------------------------
 * Stencil boundary handling, one coordinate at a time
 * (CodeGen/Stencil/Extra.hs:200-226): returns the in-range coordinate, or -1
 * for the Constant boundary when the coordinate is outside (the whole tap is
 * then replaced by the constant, Extra.hs:122-128,191-196).
 *   mode 0 Clamp, 1 Mirror, 2 Wrap, 3 Constant
 * ---------------------------------------------------------------------- */
static inline int64_t orc_bound(int64_t i, int64_t sz, int mode) {
    switch (mode) {
        case 0: return i < 0 ? 0 : (i > sz - 1 ? sz - 1 : i);
        case 1: return i < 0 ? -i : (i >= sz ? sz - (i - sz + 2) : i);
        case 2: return i < 0 ? sz + i : (i >= sz ? i - sz : i);
        default: return (i < 0 || i >= sz) ? -1 : i;
    }
}

/* 2-D stencil with a (2ry+1) x (2rx+1) weight pattern, row-major taps
 * (CodeGen/Stencil.hs:55-114): out = sum_k w[k] * in[bound(y+dy), bound(x+dx)],
 * accumulated in double in row-major tap order. */
ORC_API void orc_stencil2d_f64(const double *in, int64_t h, int64_t w, const double *wt, int ry, int rx,
                               int mode, double cval, double *out, int nthreads) {
#pragma omp parallel for num_threads(nthreads > 1 ? nthreads : 1) schedule(static) if (nthreads > 1)
    for (int64_t y = 0; y < h; ++y) {
        for (int64_t x = 0; x < w; ++x) {
            double acc = 0.0;
            int k = 0;
            for (int dy = -ry; dy <= ry; ++dy) {
                for (int dx = -rx; dx <= rx; ++dx, ++k) {
                    int64_t yy = orc_bound(y + dy, h, mode), xx = orc_bound(x + dx, w, mode);
                    double v = (yy < 0 || xx < 0) ? cval : in[yy * w + xx];
                    acc += wt[k] * v;
                }
            }
            out[y * w + x] = acc;
        }
    }
}

ORC_API void orc_stencil2d_f32in(const float *in, int64_t h, int64_t w, const double *wt, int ry, int rx,
                                 int mode, double cval, double *out, int nthreads) {
#pragma omp parallel for num_threads(nthreads > 1 ? nthreads : 1) schedule(static) if (nthreads > 1)
    for (int64_t y = 0; y < h; ++y) {
        for (int64_t x = 0; x < w; ++x) {
            double acc = 0.0;
            int k = 0;
            for (int dy = -ry; dy <= ry; ++dy) {
                for (int dx = -rx; dx <= rx; ++dx, ++k) {
                    int64_t yy = orc_bound(y + dy, h, mode), xx = orc_bound(x + dx, w, mode);
                    double v = (yy < 0 || xx < 0) ? cval : (double)in[yy * w + xx];
                    acc += wt[k] * v;
                }
            }
            out[y * w + x] = acc;
        }
    }
}

/* `iters` applications of the same stencil, keeping double state between
 * iterations (the oracle of the iterated-blur configuration).  `tmp` and
 * `out` are h*w doubles; the result is left in `out`. */
ORC_API void orc_stencil2d_iter(const float *in, int64_t h, int64_t w, const double *wt, int ry, int rx,
                                int mode, double cval, int iters, double *tmp, double *out, int nthreads) {
    if (iters <= 0) {
        for (int64_t i = 0; i < h * w; ++i) out[i] = (double)in[i];
        return;
    }
    double *a = (iters % 2) ? out : tmp; /* first destination, chosen so the last lands in out */
    double *b = (iters % 2) ? tmp : out;
    orc_stencil2d_f32in(in, h, w, wt, ry, rx, mode, cval, a, nthreads);
    for (int it = 1; it < iters; ++it) {
        orc_stencil2d_f64(a, h, w, wt, ry, rx, mode, cval, b, nthreads);
        double *t = a;
        a = b;
        b = t;
    }
    /* after the loop the newest data is in `a`, which is `out` by construction */
}

/* Float32-state variant of one stencil step: what a float32 evaluator of the
 * same program computes (timed CPU baseline; one float rounding per tap). */
ORC_API void orc_stencil2d_f32(const float *in, int64_t h, int64_t w, const float *wt, int ry, int rx,
                               int mode, float cval, float *out, int nthreads) {
#pragma omp parallel for num_threads(nthreads > 1 ? nthreads : 1) schedule(static) if (nthreads > 1)
    for (int64_t y = 0; y < h; ++y) {
        for (int64_t x = 0; x < w; ++x) {
            float acc = 0.0f;
            int k = 0;
            for (int dy = -ry; dy <= ry; ++dy) {
                for (int dx = -rx; dx <= rx; ++dx, ++k) {
                    int64_t yy = orc_bound(y + dy, h, mode), xx = orc_bound(x + dx, w, mode);
                    float v = (yy < 0 || xx < 0) ? cval : in[yy * w + xx];
                    acc += wt[k] * v;
                }
            }
            out[y * w + x] = acc;
        }
    }
}

/* stencil2: binary stencil over the intersection of the two extents
 * (Execute.hs:433-435); out = sum w1[k]*a[..] + sum w2[k]*b[..]. */
ORC_API void orc_stencil2_2d(const float *a, int64_t ha, int64_t wa, const float *b, int64_t hb, int64_t wb,
                             const double *w1, const double *w2, int ry, int rx, int mode, double cval,
                             double *out) {
    int64_t h = ha < hb ? ha : hb, w = wa < wb ? wa : wb;
    for (int64_t y = 0; y < h; ++y)
        for (int64_t x = 0; x < w; ++x) {
            double acc = 0.0;
            int k = 0;
            for (int dy = -ry; dy <= ry; ++dy)
                for (int dx = -rx; dx <= rx; ++dx, ++k) {
                    int64_t ya = orc_bound(y + dy, ha, mode), xa = orc_bound(x + dx, wa, mode);
                    int64_t yb = orc_bound(y + dy, hb, mode), xb = orc_bound(x + dx, wb, mode);
                    double va = (ya < 0 || xa < 0) ? cval : (double)a[ya * wa + xa];
                    double vb = (yb < 0 || xb < 0) ? cval : (double)b[yb * wb + xb];
                    acc += w1[k] * va + w2[k] * vb;
                }
            out[y * w + x] = acc;
        }
}

/* ------------------------------------------------------------------------
 * Black-Scholes map (CodeGen/Mapping.hs:39-78 with a user function built from
 * exp/log/sqrt primitives, CodeGen/Arithmetic.hs:374-383, and erf/erfc
 * reached as a foreign scalar function, CodeGen.hs:793-805).  European call
 * and put under constant riskfree rate r and volatility v, in double.
 * ---------------------------------------------------------------------- */
static inline double orc_cnd(double d) { return 0.5 * erfc(-d * 0.70710678118654752440); }

ORC_API void orc_blackscholes(const float *spot, const float *strike, const float *years, int64_t n, double r,
                              double v, double *call, double *put, int nthreads) {
#pragma omp parallel for num_threads(nthreads > 1 ? nthreads : 1) schedule(static) if (nthreads > 1)
    for (int64_t i = 0; i < n; ++i) {
        double s = spot[i], k = strike[i], t = years[i];
        double sq = sqrt(t);
        double d1 = (log(s / k) + (r + 0.5 * v * v) * t) / (v * sq);
        double d2 = d1 - v * sq;
        double kexp = k * exp(-r * t);
        call[i] = s * orc_cnd(d1) - kexp * orc_cnd(d2);
        put[i] = kexp * orc_cnd(-d2) - s * orc_cnd(-d1);
    }
}

/* float32 evaluation of the same formula with the float libm (erff/expf/logf/
 * sqrtf), as a sequential float32 evaluator would do it (timed baseline). */
ORC_API void orc_blackscholes_f32(const float *spot, const float *strike, const float *years, int64_t n,
                                  float r, float v, float *call, float *put, int nthreads) {
#pragma omp parallel for num_threads(nthreads > 1 ? nthreads : 1) schedule(static) if (nthreads > 1)
    for (int64_t i = 0; i < n; ++i) {
        float s = spot[i], k = strike[i], t = years[i];
        float sq = sqrtf(t);
        float d1 = (logf(s / k) + (r + 0.5f * v * v) * t) / (v * sq);
        float d2 = d1 - v * sq;
        float kexp = k * expf(-r * t);
        float n1 = 0.5f * erfcf(-d1 * 0.70710678f), n2 = 0.5f * erfcf(-d2 * 0.70710678f);
        float m1 = 0.5f * erfcf(d1 * 0.70710678f), m2 = 0.5f * erfcf(d2 * 0.70710678f);
        call[i] = s * n1 - kexp * n2;
        put[i] = kexp * m2 - s * m1;
    }
}

/* ------------------------------------------------------------------------
 * backpermute / transform: out[i] = in[idx[i]] (CodeGen/IndexSpace.hs:96-141)
 * ---------------------------------------------------------------------- */
ORC_API void orc_backpermute_i32(const int32_t *in, const int32_t *idx, int64_t nout, int32_t *out) {
    for (int64_t i = 0; i < nout; ++i) out[i] = in[idx[i]];
}
