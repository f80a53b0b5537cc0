/*
 * mc_oracle.c -- CPU restatement of the ModernChainer CPU backend arithmetic
 * for the training-step path (forward ops, their backward formulas, Adam).
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA path is
 * compared against, and the timed CPU baseline.  Nothing in the shipped
 * library links, loads or calls it.
 *
 * Every function follows the accumulation type and loop order of the
 * reference function it cites (paths are relative to the reference project
 * root).  Plain C, row-major contiguous f32 unless stated.
 *
 * Parity pin: the reference is a Rust workspace that cannot be compiled in
 * this environment, and its tests hold only a handful of literal expected
 * values (Linear 0.678262, sum_all 36, accumulate 3.0/5.0, the GradScaler
 * arithmetic, the GELU closed form).  Those literals and a central-difference
 * gradcheck with the reference's own inputs and tolerances are checked in
 * tests/test_oracle_golden.py.  For GEMMs of >= 1,000,000 multiply-adds the
 * reference calls the third-party `gemm` crate 0.19.0 (crates/
 * modern-chainer-cpu/Cargo.toml:15), whose summation order is not visible:
 * bit-level parity for those is UNPINNED; here they are f32 products
 * accumulated in f64 and rounded once.
 *
 * Build: see oracle/Makefile (gcc -O2, and an -O3 -fopenmp build for timing).
 */
#define _GNU_SOURCE
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define MCO_OK 0
#define MCO_SHAPE_MISMATCH 1
#define MCO_BROADCAST 2
#define MCO_DTYPE_MISMATCH 3
#define MCO_UNSUPPORTED_DTYPE 4
#define MCO_INVALID_ARGUMENT 5
#define MCO_OUT_OF_BOUNDS 6
#define MCO_UNSUPPORTED 7

/* dtype tags shared with the CUDA library's header */
#define MCO_F32 0
#define MCO_I64 1
#define MCO_I32 2
#define MCO_U8 3
#define MCO_F16 4
#define MCO_BF16 5

/* crates/modern-chainer-cpu/src/kernels.rs:6 -- elementwise work is split over
 * threads above this many elements (values do not depend on it). */
#define PAR_THRESHOLD 32768

int mco_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ------------------------------------------------------------------ */
/* RNG and initialisers: crates/modern-chainer-core/src/rng.rs:14-56,   */
/* crates/modern-chainer-core/src/init.rs:6-11                          */
/* ------------------------------------------------------------------ */
typedef struct {
    uint64_t state;
    int has_spare;
    double spare;
} mco_rng;

void mco_rng_seed(mco_rng *r, uint64_t seed) {
    r->state = (seed * 0x9E3779B97F4A7C15ULL) | 1ULL;
    r->has_spare = 0;
    r->spare = 0.0;
}

uint64_t mco_rng_next_u64(mco_rng *r) {
    uint64_t x = r->state;
    x ^= x >> 12;
    x ^= x << 25;
    x ^= x >> 27;
    r->state = x;
    return x * 0x2545F4914F6CDD1DULL;
}

double mco_rng_next_f64(mco_rng *r) {
    return (double)(mco_rng_next_u64(r) >> 11) * (1.0 / (double)(1ULL << 53));
}

double mco_rng_normal(mco_rng *r) {
    if (r->has_spare) {
        r->has_spare = 0;
        return r->spare;
    }
    for (;;) {
        double u = 2.0 * mco_rng_next_f64(r) - 1.0;
        double v = 2.0 * mco_rng_next_f64(r) - 1.0;
        double s = u * u + v * v;
        if (s > 0.0 && s < 1.0) {
            double factor = sqrt(-2.0 * log(s) / s);
            r->spare = v * factor;
            r->has_spare = 1;
            return u * factor;
        }
    }
}

void mco_rng_normal_fill(mco_rng *r, int64_t n, double mean, double std, float *out) {
    for (int64_t i = 0; i < n; ++i) out[i] = (float)(mean + std * mco_rng_normal(r));
}

void mco_he_normal(int64_t n, int64_t fan_in, uint64_t seed, float *out) {
    double std = sqrt(2.0 / (double)(fan_in > 1 ? fan_in : 1));
    mco_rng r;
    mco_rng_seed(&r, seed);
    mco_rng_normal_fill(&r, n, 0.0, std, out);
}

/* ------------------------------------------------------------------ */
/* dtype conversion: crates/modern-chainer-core/src/dtype.rs:75-150     */
/* ------------------------------------------------------------------ */
static uint32_t f32_bits(float v) {
    uint32_t b;
    memcpy(&b, &v, 4);
    return b;
}
static float bits_f32(uint32_t b) {
    float v;
    memcpy(&v, &b, 4);
    return v;
}

/* round-to-nearest-even on the raw bits, NaN not special-cased (dtype.rs:136-146) */
uint16_t mco_f32_to_bf16_bits(float v) {
    uint32_t bits = f32_bits(v);
    uint32_t lsb = (bits >> 16) & 1u;
    uint32_t rounded = bits + 0x7FFFu + lsb;
    return (uint16_t)(rounded >> 16);
}
float mco_bf16_bits_to_f32(uint16_t b) { return bits_f32((uint32_t)b << 16); }

void mco_f32_to_bf16(const float *x, uint16_t *out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) out[i] = mco_f32_to_bf16_bits(x[i]);
}
void mco_bf16_to_f32(const uint16_t *x, float *out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) out[i] = mco_bf16_bits_to_f32(x[i]);
}
/* value-level bf16 rounding of an f32 array (used to emulate low-precision GEMM operands) */
void mco_round_bf16(const float *x, float *out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) out[i] = mco_bf16_bits_to_f32(mco_f32_to_bf16_bits(x[i]));
}

/* f32 -> f16 bits, dtype.rs:75-108: round to nearest even for results in the normal range,
 * overflow to inf, NaN to a quiet NaN (0x200 set), magnitudes below 2^-25 to a signed zero.
 * Results in the f16 subnormal range follow the reference's own arithmetic: it adds
 * 0xfff + bit(shift-1) before shifting by 14..24, which is round-half-even only for a shift
 * of 13, so for subnormal results it is close to truncation. */
uint16_t mco_f32_to_f16_bits(float v) {
    uint32_t bits = f32_bits(v);
    uint16_t sign = (uint16_t)((bits >> 16) & 0x8000u);
    int32_t exp = (int32_t)((bits >> 23) & 0xffu);
    uint32_t frac = bits & 0x7fffffu;
    if (exp == 0xff) return (uint16_t)(sign | 0x7c00u | (frac == 0 ? 0u : 0x200u));
    int32_t h_exp = exp - 112;
    if (h_exp >= 0x1f) return (uint16_t)(sign | 0x7c00u);
    if (h_exp <= 0) {
        if (h_exp < -10) return sign;
        uint32_t m = frac | 0x800000u;
        uint32_t shift = (uint32_t)(14 - h_exp);
        uint32_t rounding_bias = ((m >> (shift - 1)) & 1u) + 0xfffu;
        uint16_t h = (uint16_t)((m + rounding_bias) >> shift);
        return (uint16_t)(h | sign);
    }
    uint16_t h = (uint16_t)(sign | ((uint16_t)h_exp << 10) | (uint16_t)(frac >> 13));
    uint32_t rounding = (frac >> 12) & 1u;
    int sticky = (frac & 0xfffu) != 0;
    uint16_t lsb = h & 1u;
    if (rounding == 1 && (sticky || lsb == 1)) return (uint16_t)(h + 1);
    return h;
}
/* dtype.rs:110-134 */
float mco_f16_bits_to_f32(uint16_t b) {
    uint32_t sign = ((uint32_t)(b & 0x8000u)) << 16;
    uint32_t exp = (b >> 10) & 0x1fu, frac = b & 0x3ffu, out;
    if (exp == 0x1f) {
        out = sign | 0x7f800000u | (frac << 13);
    } else if (exp == 0) {
        if (frac == 0) {
            out = sign;
        } else {
            uint32_t e = 0, f = frac;
            while ((f & 0x400u) == 0) {
                f <<= 1;
                e += 1;
            }
            f &= 0x3ffu;
            out = sign | ((0x7fu - 14u - e) << 23) | (f << 13);
        }
    } else {
        out = sign | ((exp + 112u) << 23) | (frac << 13);
    }
    return bits_f32(out);
}
void mco_f32_to_f16(const float *x, uint16_t *out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) out[i] = mco_f32_to_f16_bits(x[i]);
}
void mco_f16_to_f32(const uint16_t *x, float *out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) out[i] = mco_f16_bits_to_f32(x[i]);
}
void mco_round_f16(const float *x, float *out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) out[i] = mco_f16_bits_to_f32(mco_f32_to_f16_bits(x[i]));
}

/* ------------------------------------------------------------------ */
/* elementwise maps: kernels.rs:21-153, 390-423, 1384-1401              */
/* ------------------------------------------------------------------ */
static int64_t numel(const int64_t *dims, int rank) {
    int64_t n = 1;
    for (int i = 0; i < rank; ++i) n *= dims[i];
    return n;
}

/* right-aligned NumPy-style broadcast of two shapes; returns status */
int mco_broadcast_shape(const int64_t *ad, int ar, const int64_t *bd, int br, int64_t *od, int *orank) {
    int r = ar > br ? ar : br;
    for (int i = 0; i < r; ++i) {
        int64_t a = (i >= r - ar) ? ad[i - (r - ar)] : 1;
        int64_t b = (i >= r - br) ? bd[i - (r - br)] : 1;
        if (a == b) od[i] = a;
        else if (a == 1) od[i] = b;
        else if (b == 1) od[i] = a;
        else return MCO_BROADCAST;
    }
    *orank = r;
    return MCO_OK;
}

/* kernels.rs:21-43 */
static int64_t broadcast_offset(const int64_t *od, int orank, const int64_t *id, int irank, int64_t linear) {
    int shift = orank > irank ? orank - irank : 0;
    int64_t stride[8];
    int64_t s = 1;
    for (int d = irank - 1; d >= 0; --d) {
        stride[d] = s;
        s *= id[d];
    }
    int64_t off = 0;
    for (int d = orank - 1; d >= 0; --d) {
        int64_t dim = od[d];
        int64_t coord = dim == 0 ? 0 : linear % dim;
        linear /= (dim > 1 ? dim : 1);
        if (d >= shift) {
            int k = d - shift;
            if (id[k] != 1) off += coord * stride[k];
        }
    }
    return off;
}

/* op: 0 add, 1 sub, 2 mul, 3 div.  out has the broadcast shape. kernels.rs:49-140 */
int mco_binary(int op, const float *a, const int64_t *ad, int ar, const float *b, const int64_t *bd, int br,
               float *out) {
    int64_t od[8];
    int orank;
    if (ar > 8 || br > 8) return MCO_INVALID_ARGUMENT;
    int st = mco_broadcast_shape(ad, ar, bd, br, od, &orank);
    if (st) return st;
    int64_t n = numel(od, orank);
    int same = (ar == br);
    for (int i = 0; same && i < ar; ++i) same = ad[i] == bd[i];
#pragma omp parallel for if (n >= PAR_THRESHOLD) schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        float x = same ? a[i] : a[broadcast_offset(od, orank, ad, ar, i)];
        float y = same ? b[i] : b[broadcast_offset(od, orank, bd, br, i)];
        float r;
        switch (op) {
        case 0: r = x + y; break;
        case 1: r = x - y; break;
        case 2: r = x * y; break;
        default: r = x / y; break;
        }
        out[i] = r;
    }
    return MCO_OK;
}

/* kernels.rs:390-393: the f64 factor is narrowed to f32 before the multiply */
void mco_scale(const float *x, double factor, float *out, int64_t n) {
    float f = (float)factor;
#pragma omp parallel for if (n >= PAR_THRESHOLD) schedule(static)
    for (int64_t i = 0; i < n; ++i) out[i] = x[i] * f;
}

/* kernels.rs:395-423 */
void mco_relu(const float *x, float *out, int64_t n) {
#pragma omp parallel for if (n >= PAR_THRESHOLD) schedule(static)
    for (int64_t i = 0; i < n; ++i) out[i] = x[i] > 0.0f ? x[i] : 0.0f; /* f32::max(x,0): NaN -> 0 */
}
void mco_relu_backward(const float *x, const float *g, float *out, int64_t n) {
#pragma omp parallel for if (n >= PAR_THRESHOLD) schedule(static)
    for (int64_t i = 0; i < n; ++i) out[i] = x[i] > 0.0f ? g[i] : 0.0f;
}

/* kernels.rs:1384-1389 */
void mco_gelu(const float *x, float *out, int64_t n) {
    const float k = sqrtf(2.0f / (float)M_PI);
#pragma omp parallel for if (n >= PAR_THRESHOLD) schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        float v = x[i];
        float v3 = v * v * v;
        out[i] = 0.5f * v * (1.0f + tanhf(k * (v + 0.044715f * v3)));
    }
}

/* crates/modern-chainer-autograd/src/ops.rs:646-676: the backward is composed
 * from f32 tensor ops; each line below is one of those ops on one element. */
void mco_gelu_backward(const float *x, const float *g, float *out, int64_t n) {
    const float c044 = (float)0.044715;
    const float k = (float)sqrt(2.0 / M_PI);
#pragma omp parallel for if (n >= PAR_THRESHOLD) schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        float v = x[i];
        float xx = v * v;
        float x3 = xx * v;
        float inner = v + x3 * c044;
        float c = inner * k;
        float e2 = expf(c * -2.0f);
        float denom = 1.0f + e2;
        float numer = 1.0f - e2;
        float th = numer / denom;
        float phi = (1.0f + th) * 0.5f;
        float sech = 1.0f - th * th;
        float dphi = sech * 0.5f;
        float three_x = v * 3.0f;
        float three_xx = three_x * v;
        float d_inner = 1.0f + three_xx * c044;
        float coeff = d_inner * k;
        float x_dphi = v * dphi;
        float local = phi + x_dphi * coeff;
        out[i] = g[i] * local;
    }
}

/* op: 0 exp, 1 log, 2 sigmoid, 3 sqrt, 4 silu, 5 abs, 6 neg. kernels.rs:142-153,833-835,1391-1401 */
void mco_unary(int op, const float *x, float *out, int64_t n) {
#pragma omp parallel for if (n >= PAR_THRESHOLD) schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        float v = x[i], r;
        switch (op) {
        case 0: r = expf(v); break;
        case 1: r = logf(v); break;
        case 2: r = 1.0f / (1.0f + expf(-v)); break;
        case 3: r = sqrtf(v); break;
        case 4: r = v / (1.0f + expf(-v)); break;
        case 5: r = fabsf(v); break;
        default: r = -v; break;
        }
        out[i] = r;
    }
}

/* ------------------------------------------------------------------ */
/* reductions: kernels.rs:332-388                                       */
/* ------------------------------------------------------------------ */
float mco_sum_all(const float *x, int64_t n) {
    double acc = 0.0;
    for (int64_t i = 0; i < n; ++i) acc += (double)x[i];
    return (float)acc;
}

/* sum `a` (shape ad) down to `td` (right-aligned; target dims are 1 or equal). */
int mco_sum_to(const float *a, const int64_t *ad, int ar, const int64_t *td, int tr, float *out) {
    if (tr > ar || ar > 8) return MCO_INVALID_ARGUMENT;
    int64_t tn = numel(td, tr);
    for (int64_t i = 0; i < tn; ++i) out[i] = 0.0f;
    if (tn == 0) return MCO_OK;
    if (ar == 2 && tr == 1 && td[0] == ad[1]) {
        for (int64_t r = 0; r < ad[0]; ++r)
            for (int64_t c = 0; c < ad[1]; ++c) out[c] += a[r * ad[1] + c];
        return MCO_OK;
    }
    int shift = ar - tr;
    int64_t ostr[8], s = 1;
    for (int d = tr - 1; d >= 0; --d) {
        ostr[d] = s;
        s *= td[d];
    }
    int64_t n = numel(ad, ar);
    for (int64_t lin = 0; lin < n; ++lin) {
        int64_t rest = lin, off = 0;
        for (int d = ar - 1; d >= 0; --d) {
            int64_t dim = ad[d];
            int64_t coord = dim == 0 ? 0 : rest % dim;
            rest /= (dim > 1 ? dim : 1);
            if (d >= shift) {
                int od = d - shift;
                if (td[od] != 1) off += coord * ostr[od];
            }
        }
        out[off] += a[lin];
    }
    return MCO_OK;
}

/* ------------------------------------------------------------------ */
/* GEMM family: kernels.rs:155-304, 552-645                             */
/* ------------------------------------------------------------------ */
static int naive_path(int64_t m, int64_t n, int64_t k) {
    double work = (double)m * (double)n * (double)k;
    return work < 1.0e6;
}

/* C[m,n] = A[m,k] * B[k,n].  fast!=0 uses an f32 blocked threaded kernel for
 * timing runs; otherwise big GEMMs accumulate in f64 (parity policy above). */
static int g_fast_gemm = 0;
void mco_set_fast_gemm(int on) { g_fast_gemm = on; }
/* In a build with OpenMP, mco_set_parallel(1) lets loops whose iterations are independent
 * (one output element, one (sample, head), one sample or one output channel per iteration)
 * run on several threads.  Every value is produced by the same operations in the same order
 * as with one thread, so results are bit-identical; it only makes full-size parity cases
 * affordable.  The reference runs these loops on one thread. */
static int g_par = 0;
void mco_set_parallel(int on) { g_par = on; }

/* generic strided big GEMM: C[i,j] = sum_d A[i*as0 + d*as1] * B[d*bs0 + j*bs1] */
static void big_gemm(int64_t m, int64_t n, int64_t k, const float *a, int64_t as0, int64_t as1, const float *b,
                     int64_t bs0, int64_t bs1, float *c) {
    if (!g_fast_gemm) {
        /* f32 products summed in f64 in index order d = 0..k-1, one rounding at the end.  Operands
         * are first copied so that d is contiguous, and four columns share one pass over a row of
         * A; neither changes any sum. */
        const float *ap = a, *bp = b;
        float *apk = NULL, *bpk = NULL;
        if (as1 != 1) {
            apk = (float *)malloc(sizeof(float) * (size_t)m * (size_t)k);
#pragma omp parallel for schedule(static)
            for (int64_t i = 0; i < m; ++i)
                for (int64_t d = 0; d < k; ++d) apk[i * k + d] = a[i * as0 + d * as1];
            ap = apk;
            as0 = k;
        }
        if (bs0 != 1) {
            bpk = (float *)malloc(sizeof(float) * (size_t)n * (size_t)k);
#pragma omp parallel for schedule(static)
            for (int64_t j = 0; j < n; ++j)
                for (int64_t d = 0; d < k; ++d) bpk[j * k + d] = b[d * bs0 + j * bs1];
            bp = bpk;
            bs1 = k;
        }
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < m; ++i) {
            const float *ar = ap + i * as0;
            int64_t j = 0;
            for (; j + 4 <= n; j += 4) {
                const float *b0 = bp + j * bs1, *b1 = b0 + bs1, *b2 = b1 + bs1, *b3 = b2 + bs1;
                double s0 = 0.0, s1 = 0.0, s2 = 0.0, s3 = 0.0;
                for (int64_t d = 0; d < k; ++d) {
                    float av = ar[d];
                    s0 += (double)(av * b0[d]);
                    s1 += (double)(av * b1[d]);
                    s2 += (double)(av * b2[d]);
                    s3 += (double)(av * b3[d]);
                }
                c[i * n + j] = (float)s0;
                c[i * n + j + 1] = (float)s1;
                c[i * n + j + 2] = (float)s2;
                c[i * n + j + 3] = (float)s3;
            }
            for (; j < n; ++j) {
                const float *b0 = bp + j * bs1;
                double acc = 0.0;
                for (int64_t d = 0; d < k; ++d) acc += (double)(ar[d] * b0[d]);
                c[i * n + j] = (float)acc;
            }
        }
        free(apk);
        free(bpk);
        return;
    }
    /* timing build: pack B to [k,n] row-major and A to [m,k] row-major, then a
     * cache-blocked i-k-j kernel the compiler vectorises over j. */
    float *bp = (float *)malloc(sizeof(float) * (size_t)k * (size_t)n);
    float *ap = (float *)malloc(sizeof(float) * (size_t)m * (size_t)k);
#pragma omp parallel for schedule(static)
    for (int64_t d = 0; d < k; ++d)
        for (int64_t j = 0; j < n; ++j) bp[d * n + j] = b[d * bs0 + j * bs1];
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < m; ++i)
        for (int64_t d = 0; d < k; ++d) ap[i * k + d] = a[i * as0 + d * as1];
    const int64_t BI = 48, BK = 256, BJ = 512;
#pragma omp parallel for schedule(dynamic) collapse(2)
    for (int64_t i0 = 0; i0 < m; i0 += BI)
        for (int64_t j0 = 0; j0 < n; j0 += BJ) {
            int64_t i1 = i0 + BI < m ? i0 + BI : m, j1 = j0 + BJ < n ? j0 + BJ : n;
            for (int64_t i = i0; i < i1; ++i)
                for (int64_t j = j0; j < j1; ++j) c[i * n + j] = 0.0f;
            for (int64_t d0 = 0; d0 < k; d0 += BK) {
                int64_t d1 = d0 + BK < k ? d0 + BK : k;
                for (int64_t i = i0; i < i1; ++i) {
                    float *crow = c + i * n;
                    for (int64_t d = d0; d < d1; ++d) {
                        float av = ap[i * k + d];
                        const float *brow = bp + d * n;
                        for (int64_t j = j0; j < j1; ++j) crow[j] += av * brow[j];
                    }
                }
            }
        }
    free(ap);
    free(bp);
}

/* kernels.rs:155-215 */
void mco_matmul(const float *a, const float *b, float *c, int64_t m, int64_t k, int64_t n) {
    if (naive_path(m, n, k)) {
        for (int64_t i = 0; i < m; ++i)
            for (int64_t j = 0; j < n; ++j) {
                float acc = 0.0f;
                for (int64_t d = 0; d < k; ++d) acc += a[i * k + d] * b[d * n + j];
                c[i * n + j] = acc;
            }
    } else {
        big_gemm(m, n, k, a, k, 1, b, n, 1, c);
    }
}

/* y[m,n] = x[m,k] * w[n,k]^T + bias[n]; bias added after the product. kernels.rs:218-304 */
void mco_linear(const float *x, const float *w, const float *bias, float *y, int64_t m, int64_t k, int64_t n) {
    double work = (double)m * (double)n * (double)k;
    if (work > 0 && work < 1.0e6) {
        for (int64_t i = 0; i < m; ++i)
            for (int64_t j = 0; j < n; ++j) {
                float acc = 0.0f;
                for (int64_t d = 0; d < k; ++d) acc += x[i * k + d] * w[j * k + d];
                y[i * n + j] = acc;
            }
    } else {
        big_gemm(m, n, k, x, k, 1, w, 1, k, y);
    }
    if (bias) {
        for (int64_t i = 0; i < m; ++i)
            for (int64_t j = 0; j < n; ++j) y[i * n + j] += bias[j];
    }
}

/* dx[m,k] = g[m,n] * w[n,k];  dw[n,k] = g^T * x;  db[n] = column sums of g.
 * kernels.rs:552-645 and the sum_to bias path (360-369). Any output may be NULL. */
void mco_linear_backward(const float *g, const float *x, const float *w, float *dx, float *dw, float *db, int64_t m,
                         int64_t k, int64_t n) {
    int naive = naive_path(m, n, k);
    if (dx) {
        if (naive) {
            for (int64_t i = 0; i < m; ++i)
                for (int64_t d = 0; d < k; ++d) {
                    float acc = 0.0f;
                    for (int64_t j = 0; j < n; ++j) acc += g[i * n + j] * w[j * k + d];
                    dx[i * k + d] = acc;
                }
        } else {
            big_gemm(m, k, n, g, n, 1, w, k, 1, dx);
        }
    }
    if (dw) {
        if (naive) {
            for (int64_t j = 0; j < n; ++j)
                for (int64_t d = 0; d < k; ++d) {
                    float acc = 0.0f;
                    for (int64_t i = 0; i < m; ++i) acc += g[i * n + j] * x[i * k + d];
                    dw[j * k + d] = acc;
                }
        } else {
            big_gemm(n, k, m, g, 1, n, x, k, 1, dw);
        }
    }
    if (db) {
        for (int64_t j = 0; j < n; ++j) db[j] = 0.0f;
        for (int64_t i = 0; i < m; ++i)
            for (int64_t j = 0; j < n; ++j) db[j] += g[i * n + j];
    }
}

/* ------------------------------------------------------------------ */
/* softmax / layer norm: kernels.rs:766-831, 1403-1496                  */
/* ------------------------------------------------------------------ */
void mco_softmax(const float *x, float *out, int64_t rows, int64_t cols) {
    for (int64_t r = 0; r < rows; ++r) {
        const float *s = x + r * cols;
        float *d = out + r * cols;
        float mx = -INFINITY;
        for (int64_t j = 0; j < cols; ++j) mx = s[j] > mx ? s[j] : mx;
        double sum = 0.0;
        for (int64_t j = 0; j < cols; ++j) sum += exp((double)(s[j] - mx));
        double inv = 1.0 / sum;
        for (int64_t j = 0; j < cols; ++j) d[j] = (float)(exp((double)(s[j] - mx)) * inv);
    }
}

void mco_softmax_backward(const float *x, const float *g, float *out, int64_t rows, int64_t cols) {
    float *p = (float *)malloc(sizeof(float) * (size_t)(cols > 0 ? cols : 1));
    for (int64_t r = 0; r < rows; ++r) {
        const float *s = x + r * cols;
        const float *gr = g + r * cols;
        float *d = out + r * cols;
        float mx = -INFINITY;
        for (int64_t j = 0; j < cols; ++j) mx = s[j] > mx ? s[j] : mx;
        double sum = 0.0;
        for (int64_t j = 0; j < cols; ++j) sum += exp((double)(s[j] - mx));
        for (int64_t j = 0; j < cols; ++j) p[j] = (float)(exp((double)(s[j] - mx)) / sum);
        float dot = 0.0f;
        for (int64_t j = 0; j < cols; ++j) dot += p[j] * gr[j];
        for (int64_t j = 0; j < cols; ++j) d[j] = p[j] * (gr[j] - dot);
    }
    free(p);
}

void mco_layer_norm(const float *x, const float *gamma, const float *beta, double eps, float *out, int64_t rows,
                    int64_t dim) {
    for (int64_t r = 0; r < rows; ++r) {
        const float *s = x + r * dim;
        float *d = out + r * dim;
        double mean = 0.0;
        for (int64_t i = 0; i < dim; ++i) mean += (double)s[i];
        mean /= (double)dim;
        double var = 0.0;
        for (int64_t i = 0; i < dim; ++i) {
            double t = (double)s[i] - mean;
            var += t * t;
        }
        var /= (double)dim;
        double inv = 1.0 / sqrt(var + eps);
        for (int64_t i = 0; i < dim; ++i)
            d[i] = (float)((((double)s[i] - mean) * inv) * (double)gamma[i] + (double)beta[i]);
    }
}

void mco_layer_norm_backward(const float *x, const float *gamma, const float *g, double eps, float *dx,
                             float *dgamma, float *dbeta, int64_t rows, int64_t dim) {
    float *norm = (float *)malloc(sizeof(float) * (size_t)(dim > 0 ? dim : 1));
    for (int64_t i = 0; i < dim; ++i) {
        dgamma[i] = 0.0f;
        dbeta[i] = 0.0f;
    }
    for (int64_t r = 0; r < rows; ++r) {
        const float *xs = x + r * dim;
        const float *gs = g + r * dim;
        double mean = 0.0;
        for (int64_t i = 0; i < dim; ++i) mean += (double)xs[i];
        mean /= (double)dim;
        double var = 0.0;
        for (int64_t i = 0; i < dim; ++i) {
            double t = (double)xs[i] - mean;
            var += t * t;
        }
        var /= (double)dim;
        double inv = 1.0 / sqrt(var + eps);
        for (int64_t i = 0; i < dim; ++i) norm[i] = (float)(((double)xs[i] - mean) * inv);
        float sum_dy = 0.0f, sum_dy_norm = 0.0f;
        for (int64_t i = 0; i < dim; ++i) {
            float dy = gs[i] * gamma[i];
            sum_dy += dy;
            sum_dy_norm += dy * norm[i];
            dgamma[i] += gs[i] * norm[i];
            dbeta[i] += gs[i];
        }
        for (int64_t i = 0; i < dim; ++i) {
            float dy = gs[i] * gamma[i];
            dx[r * dim + i] = (((float)dim * dy - sum_dy - norm[i] * sum_dy_norm) * (float)inv / (float)dim) * 1.0f;
        }
    }
    free(norm);
}

/* ------------------------------------------------------------------ */
/* softmax cross entropy: kernels.rs:425-549                            */
/* ------------------------------------------------------------------ */
static int label_at(const void *labels, int dtype, int64_t i, int64_t *out) {
    switch (dtype) {
    case MCO_I64: *out = ((const int64_t *)labels)[i]; return MCO_OK;
    case MCO_I32: *out = (int64_t)((const int32_t *)labels)[i]; return MCO_OK;
    case MCO_U8: *out = (int64_t)((const uint8_t *)labels)[i]; return MCO_OK;
    default: return MCO_UNSUPPORTED_DTYPE;
    }
}

/* The reference forward indexes row[label] unchecked (a Rust panic for label >= c);
 * this restatement reports OUT-OF-RANGE labels as InvalidArgument in both directions. */
int mco_softmax_cross_entropy(const float *x, const void *labels, int label_dtype, int64_t n, int64_t c,
                              float *loss_out) {
    if (n == 0) {
        *loss_out = 0.0f;
        return MCO_OK;
    }
    double loss = 0.0;
    for (int64_t i = 0; i < n; ++i) {
        int64_t lab;
        int st = label_at(labels, label_dtype, i, &lab);
        if (st) return st;
        if (lab < 0 || lab >= c) return MCO_INVALID_ARGUMENT;
    }
    for (int64_t i = 0; i < n; ++i) {
        int64_t lab;
        label_at(labels, label_dtype, i, &lab);
        const float *row = x + i * c;
        float mx = -INFINITY;
        for (int64_t j = 0; j < c; ++j) mx = row[j] > mx ? row[j] : mx;
        double sum = 0.0;
        for (int64_t j = 0; j < c; ++j) sum += exp((double)(row[j] - mx));
        loss += ((double)mx + log(sum)) - (double)row[lab];
    }
    *loss_out = (float)(loss / (double)n);
    return MCO_OK;
}

int mco_softmax_cross_entropy_backward(const float *x, const void *labels, int label_dtype, int64_t n, int64_t c,
                                       float *out) {
    if (n == 0) return MCO_OK;
    for (int64_t i = 0; i < n; ++i) {
        int64_t lab;
        int st = label_at(labels, label_dtype, i, &lab);
        if (st) return st;
        if (lab < 0 || lab >= c) return MCO_INVALID_ARGUMENT;
    }
    float inv_n = 1.0f / (float)n;
    for (int64_t i = 0; i < n; ++i) {
        int64_t lab;
        label_at(labels, label_dtype, i, &lab);
        const float *src = x + i * c;
        float *dst = out + i * c;
        float mx = -INFINITY;
        for (int64_t j = 0; j < c; ++j) mx = src[j] > mx ? src[j] : mx;
        double sum = 0.0;
        for (int64_t j = 0; j < c; ++j) sum += exp((double)(src[j] - mx));
        double inv_sum = 1.0 / sum;
        for (int64_t j = 0; j < c; ++j) dst[j] = (float)(exp((double)(src[j] - mx)) * inv_sum);
        dst[lab] -= 1.0f;
        for (int64_t j = 0; j < c; ++j) dst[j] *= inv_n;
    }
    return MCO_OK;
}

/* ------------------------------------------------------------------ */
/* embedding: kernels.rs:730-764, 1783-1815                             */
/* ------------------------------------------------------------------ */
int mco_embedding(const void *ids, int id_dtype, int64_t n, const float *weight, int64_t vocab, int64_t dim,
                  float *out) {
    for (int64_t i = 0; i < n; ++i) {
        int64_t id;
        int st = label_at(ids, id_dtype, i, &id);
        if (st) return st;
        if (id < 0 || id >= vocab) return MCO_INVALID_ARGUMENT;
        memcpy(out + i * dim, weight + id * dim, sizeof(float) * (size_t)dim);
    }
    return MCO_OK;
}

int mco_embedding_backward(const void *ids, int id_dtype, int64_t n, const float *g, int64_t vocab, int64_t dim,
                           float *out) {
    for (int64_t i = 0; i < vocab * dim; ++i) out[i] = 0.0f;
    for (int64_t i = 0; i < n; ++i) {
        int64_t id;
        int st = label_at(ids, id_dtype, i, &id);
        if (st) return st;
        if (id < 0 || id >= vocab) return MCO_INVALID_ARGUMENT;
        for (int64_t d = 0; d < dim; ++d) out[id * dim + d] += g[i * dim + d];
    }
    return MCO_OK;
}

/* ------------------------------------------------------------------ */
/* Adam: kernels.rs:648-728                                             */
/* ------------------------------------------------------------------ */
static float powi_f32(float base, int32_t e) {
    /* Rust f32::powi lowers to repeated squaring (compiler-rt __powisf2). */
    int neg = e < 0;
    uint32_t n = neg ? (uint32_t)(-(int64_t)e) : (uint32_t)e;
    float r = 1.0f, b = base;
    for (;;) {
        if (n & 1u) r *= b;
        n >>= 1;
        if (!n) break;
        b *= b;
    }
    return neg ? 1.0f / r : r;
}

void mco_adam_update(const float *p, const float *g, const float *m, const float *v, float *np_, float *nm_,
                     float *nv_, int64_t n, double lr_, double beta1, double beta2, double eps_, int32_t step) {
    float b1 = (float)beta1, b2 = (float)beta2;
    float omb1 = 1.0f - b1, omb2 = 1.0f - b2;
    float bc1 = 1.0f - powi_f32(b1, step);
    float bc2 = 1.0f - powi_f32(b2, step);
    float lr = (float)lr_, eps = (float)eps_;
#pragma omp parallel for if (n >= PAR_THRESHOLD) schedule(static, 4096)
    for (int64_t i = 0; i < n; ++i) {
        float gi = g[i];
        float nm = b1 * m[i] + omb1 * gi;
        float nv = b2 * v[i] + omb2 * gi * gi;
        float m_hat = nm / bc1;
        float v_hat = nv / bc2;
        nm_[i] = nm;
        nv_[i] = nv;
        np_[i] = p[i] - lr * m_hat / (sqrtf(v_hat) + eps);
    }
}

/* number of non-finite entries (crates/modern-chainer-optim/src/amp.rs:88-107 scans with !is_finite()) */
int64_t mco_count_non_finite(const float *g, int64_t n) {
    int64_t c = 0;
    for (int64_t i = 0; i < n; ++i) c += !isfinite(g[i]);
    return c;
}

/* ------------------------------------------------------------------ */
/* conv2d / max-pool: crates/modern-chainer-autograd/src/host_ops.rs    */
/* :57-180 and :359-476 (NCHW, one stride and one padding value)        */
/* ------------------------------------------------------------------ */
static int64_t out_extent(int64_t in, int64_t k, int64_t stride, int64_t pad) { return (in + 2 * pad - k) / stride + 1; }

void mco_conv2d(const float *x, const float *w, const float *bias, float *out, int64_t n, int64_t c, int64_t h,
                int64_t wd, int64_t o, int64_t kh, int64_t kw, int64_t stride, int64_t pad) {
    int64_t oh = out_extent(h, kh, stride, pad), ow = out_extent(wd, kw, stride, pad);
#pragma omp parallel for collapse(2) schedule(static) if (g_fast_gemm || g_par)
    for (int64_t ni = 0; ni < n; ++ni)
        for (int64_t oi = 0; oi < o; ++oi)
            for (int64_t y = 0; y < oh; ++y)
                for (int64_t xi = 0; xi < ow; ++xi) {
                    float sum = bias ? bias[oi] : 0.0f;
                    for (int64_t ci = 0; ci < c; ++ci)
                        for (int64_t ky = 0; ky < kh; ++ky)
                            for (int64_t kx = 0; kx < kw; ++kx) {
                                int64_t iy = y * stride + ky, ix = xi * stride + kx;
                                if (iy >= pad && ix >= pad && iy - pad < h && ix - pad < wd) {
                                    int64_t iv = ((ni * c + ci) * h + (iy - pad)) * wd + (ix - pad);
                                    int64_t ww = ((oi * c + ci) * kh + ky) * kw + kx;
                                    sum += x[iv] * w[ww];
                                }
                            }
                    out[((ni * o + oi) * oh + y) * ow + xi] = sum;
                }
}

void mco_conv2d_backward(const float *x, const float *w, const float *g, float *dx, float *dw, float *db, int64_t n,
                         int64_t c, int64_t h, int64_t wd, int64_t o, int64_t kh, int64_t kw, int64_t stride,
                         int64_t pad) {
    int64_t oh = out_extent(h, kh, stride, pad), ow = out_extent(wd, kw, stride, pad);
    memset(dx, 0, sizeof(float) * (size_t)(n * c * h * wd));
    memset(dw, 0, sizeof(float) * (size_t)(o * c * kh * kw));
    if (db) memset(db, 0, sizeof(float) * (size_t)o);
    /* The reference runs one loop nest (n, o, y, x, ci, ky, kx) that adds into dx, dw and db.
     * Here the same nest is walked twice: once per sample for dx (a sample's dx only receives
     * terms of that sample, in the order o, y, x, ...) and once per output channel for dw and db
     * (a channel's dw and db only receive terms of that channel, in the order n, y, x, ...).
     * Each accumulator sees its terms in the reference's order; the two walks can be threaded. */
#pragma omp parallel for schedule(static) if (g_fast_gemm || g_par)
    for (int64_t ni = 0; ni < n; ++ni)
        for (int64_t oi = 0; oi < o; ++oi)
            for (int64_t y = 0; y < oh; ++y)
                for (int64_t xi = 0; xi < ow; ++xi) {
                    float gv = g[((ni * o + oi) * oh + y) * ow + xi];
                    for (int64_t ci = 0; ci < c; ++ci)
                        for (int64_t ky = 0; ky < kh; ++ky)
                            for (int64_t kx = 0; kx < kw; ++kx) {
                                int64_t iy = y * stride + ky, ix = xi * stride + kx;
                                if (iy >= pad && ix >= pad && iy - pad < h && ix - pad < wd) {
                                    int64_t iv = ((ni * c + ci) * h + (iy - pad)) * wd + (ix - pad);
                                    int64_t wi = ((oi * c + ci) * kh + ky) * kw + kx;
                                    dx[iv] += gv * w[wi];
                                }
                            }
                }
#pragma omp parallel for schedule(static) if (g_fast_gemm || g_par)
    for (int64_t oi = 0; oi < o; ++oi)
        for (int64_t ni = 0; ni < n; ++ni)
            for (int64_t y = 0; y < oh; ++y)
                for (int64_t xi = 0; xi < ow; ++xi) {
                    float gv = g[((ni * o + oi) * oh + y) * ow + xi];
                    if (db) db[oi] += gv;
                    for (int64_t ci = 0; ci < c; ++ci)
                        for (int64_t ky = 0; ky < kh; ++ky)
                            for (int64_t kx = 0; kx < kw; ++kx) {
                                int64_t iy = y * stride + ky, ix = xi * stride + kx;
                                if (iy >= pad && ix >= pad && iy - pad < h && ix - pad < wd) {
                                    int64_t iv = ((ni * c + ci) * h + (iy - pad)) * wd + (ix - pad);
                                    int64_t wi = ((oi * c + ci) * kh + ky) * kw + kx;
                                    dw[wi] += gv * x[iv];
                                }
                            }
                }
}

void mco_max_pool2d(const float *x, float *out, int64_t n, int64_t c, int64_t h, int64_t w, int64_t kernel,
                    int64_t stride, int64_t pad) {
    int64_t oh = out_extent(h, kernel, stride, pad), ow = out_extent(w, kernel, stride, pad);
    for (int64_t nc = 0; nc < n * c; ++nc)
        for (int64_t y = 0; y < oh; ++y)
            for (int64_t xi = 0; xi < ow; ++xi) {
                float acc = -INFINITY;
                for (int64_t ky = 0; ky < kernel; ++ky)
                    for (int64_t kx = 0; kx < kernel; ++kx) {
                        int64_t iy = y * stride + ky, ix = xi * stride + kx;
                        if (iy >= pad && ix >= pad && iy - pad < h && ix - pad < w) {
                            float v = x[(nc * h + (iy - pad)) * w + (ix - pad)];
                            acc = (v > acc) ? v : acc; /* f32::max ignores NaN operands */
                        }
                    }
                out[(nc * oh + y) * ow + xi] = acc;
            }
}

/* host_ops.rs:422-470: the `break` leaves the inner (kx) loop only, so a later
 * ky row that also holds the window maximum receives the gradient too. */
void mco_max_pool2d_backward(const float *x, const float *g, float *dx, int64_t n, int64_t c, int64_t h, int64_t w,
                             int64_t kernel, int64_t stride, int64_t pad) {
    int64_t oh = out_extent(h, kernel, stride, pad), ow = out_extent(w, kernel, stride, pad);
    memset(dx, 0, sizeof(float) * (size_t)(n * c * h * w));
    for (int64_t nc = 0; nc < n * c; ++nc)
        for (int64_t y = 0; y < oh; ++y)
            for (int64_t xi = 0; xi < ow; ++xi) {
                float gv = g[(nc * oh + y) * ow + xi];
                float best = -INFINITY;
                for (int64_t ky = 0; ky < kernel; ++ky)
                    for (int64_t kx = 0; kx < kernel; ++kx) {
                        int64_t iy = y * stride + ky, ix = xi * stride + kx;
                        if (iy >= pad && ix >= pad && iy - pad < h && ix - pad < w) {
                            float v = x[(nc * h + (iy - pad)) * w + (ix - pad)];
                            best = (v > best) ? v : best;
                        }
                    }
                for (int64_t ky = 0; ky < kernel; ++ky)
                    for (int64_t kx = 0; kx < kernel; ++kx) {
                        int64_t iy = y * stride + ky, ix = xi * stride + kx;
                        if (iy >= pad && ix >= pad && iy - pad < h && ix - pad < w) {
                            int64_t idx = (nc * h + (iy - pad)) * w + (ix - pad);
                            if (x[idx] == best) {
                                dx[idx] += gv;
                                break;
                            }
                        }
                    }
            }
}

/* ------------------------------------------------------------------ */
/* multi-head attention: host_ops.rs:790-968.  q,k,v,out: [n, seq, dim] */
/* with head h in columns h*hd .. (h+1)*hd; all f32, sequential sums.   */
/* ------------------------------------------------------------------ */
static void attn_probs(const float *q, const float *k, float *probs, int64_t ni, int64_t hi, int64_t seq, int64_t dim,
                       int64_t hd, float scale, int causal) {
    for (int64_t qi = 0; qi < seq; ++qi) {
        float maxv = -INFINITY;
        float *row = probs + qi * seq;
        for (int64_t ki = 0; ki < seq; ++ki) {
            if (causal && ki > qi) {
                row[ki] = -INFINITY;
                continue;
            }
            float dot = 0.0f;
            for (int64_t d = 0; d < hd; ++d)
                dot += q[(ni * seq + qi) * dim + hi * hd + d] * k[(ni * seq + ki) * dim + hi * hd + d];
            float s = dot * scale;
            row[ki] = s;
            maxv = s > maxv ? s : maxv;
        }
        float sum = 0.0f;
        for (int64_t ki = 0; ki < seq; ++ki) {
            if (row[ki] > -INFINITY) {
                row[ki] = expf(row[ki] - maxv);
                sum += row[ki];
            } else {
                row[ki] = 0.0f;
            }
        }
        for (int64_t ki = 0; ki < seq; ++ki) {
            if (causal && ki > qi) row[ki] = 0.0f;
            else if (sum > 0.0f) row[ki] /= sum;
        }
    }
}

void mco_attention(const float *q, const float *k, const float *v, float *out, int64_t n, int64_t seq, int64_t dim,
                   int64_t heads, int causal) {
    int64_t hd = dim / heads;
    float scale = 1.0f / sqrtf((float)hd);
#pragma omp parallel for collapse(2) schedule(dynamic) if (g_fast_gemm || g_par)
    for (int64_t ni = 0; ni < n; ++ni)
        for (int64_t hi = 0; hi < heads; ++hi) {
            float *probs = (float *)malloc(sizeof(float) * (size_t)(seq * seq));
            attn_probs(q, k, probs, ni, hi, seq, dim, hd, scale, causal);
            for (int64_t qi = 0; qi < seq; ++qi)
                for (int64_t d = 0; d < hd; ++d) {
                    float acc = 0.0f;
                    for (int64_t ki = 0; ki < seq; ++ki)
                        acc += probs[qi * seq + ki] * v[(ni * seq + ki) * dim + hi * hd + d];
                    out[(ni * seq + qi) * dim + hi * hd + d] = acc;
                }
            free(probs);
        }
}

void mco_attention_backward(const float *q, const float *k, const float *v, const float *gout, float *dq, float *dk,
                            float *dv, int64_t n, int64_t seq, int64_t dim, int64_t heads, int causal) {
    int64_t hd = dim / heads;
    float scale = 1.0f / sqrtf((float)hd);
#pragma omp parallel for collapse(2) schedule(dynamic) if (g_fast_gemm || g_par)
    for (int64_t ni = 0; ni < n; ++ni)
        for (int64_t hi = 0; hi < heads; ++hi) {
            float *probs = (float *)malloc(sizeof(float) * (size_t)(seq * seq));
            float *dp = (float *)malloc(sizeof(float) * (size_t)(seq * seq));
            float *ds = (float *)malloc(sizeof(float) * (size_t)(seq * seq));
            attn_probs(q, k, probs, ni, hi, seq, dim, hd, scale, causal);
            for (int64_t qi = 0; qi < seq; ++qi) {
                for (int64_t ki = 0; ki < seq; ++ki) {
                    float dot = 0.0f;
                    for (int64_t d = 0; d < hd; ++d)
                        dot += gout[(ni * seq + qi) * dim + hi * hd + d] * v[(ni * seq + ki) * dim + hi * hd + d];
                    dp[qi * seq + ki] = dot;
                }
                float row = 0.0f;
                for (int64_t ki = 0; ki < seq; ++ki) row += probs[qi * seq + ki] * dp[qi * seq + ki];
                for (int64_t ki = 0; ki < seq; ++ki) ds[qi * seq + ki] = probs[qi * seq + ki] * (dp[qi * seq + ki] - row);
            }
            for (int64_t ki = 0; ki < seq; ++ki)
                for (int64_t d = 0; d < hd; ++d) {
                    float acc = 0.0f;
                    for (int64_t qi = 0; qi < seq; ++qi)
                        acc += probs[qi * seq + ki] * gout[(ni * seq + qi) * dim + hi * hd + d];
                    dv[(ni * seq + ki) * dim + hi * hd + d] = acc;
                }
            for (int64_t qi = 0; qi < seq; ++qi)
                for (int64_t d = 0; d < hd; ++d) {
                    float acc = 0.0f;
                    for (int64_t ki = 0; ki < seq; ++ki) acc += ds[qi * seq + ki] * k[(ni * seq + ki) * dim + hi * hd + d];
                    dq[(ni * seq + qi) * dim + hi * hd + d] = acc * scale;
                }
            for (int64_t ki = 0; ki < seq; ++ki)
                for (int64_t d = 0; d < hd; ++d) {
                    float acc = 0.0f;
                    for (int64_t qi = 0; qi < seq; ++qi) acc += ds[qi * seq + ki] * q[(ni * seq + qi) * dim + hi * hd + d];
                    dk[(ni * seq + ki) * dim + hi * hd + d] = acc * scale;
                }
            free(probs);
            free(dp);
            free(ds);
        }
}
