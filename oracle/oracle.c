/* CPU oracle in C for the 4-bit quantize -> dequantize -> matmul path.
 *
 * TEST INFRASTRUCTURE ONLY: a second, independent restatement (plain loops) of the
 * reference's pure-PyTorch CPU algorithm, mps_bitsandbytes/functional.py.  It serves
 * (1) as the multi-threaded CPU baseline the benchmark times beside the GPU kernels,
 * (2) to cross-check the numpy oracle on sizes where numpy is slow, and
 * (3) to derive and prove, exhaustively, the shortcuts the CUDA quantiser uses
 *     (decision thresholds instead of a 16-way search; reciprocal-based division).
 * The shipped library never links or loads it.
 *
 * Parity status: PINNED through tests/test_oracle_golden.py, which checks these
 * functions against outputs of the reference itself (tests/golden/).
 *
 * Build: gcc -O2 -fopenmp -shared -fPIC -ffp-contract=off -o _build/liboracle.so oracle.c -lm
 * (-ffp-contract=off: no fused multiply-add may replace a rounded multiply and add.)
 */
#include <fenv.h>
#include <math.h>
#include <omp.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* mps_bitsandbytes/functional.py:21-26 */
static const float NF4[16] = {
    -1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f,
    -0.28444138169288635f, -0.18477343022823334f, -0.09105003625154495f, 0.0f,
    0.07958029955625534f, 0.16093020141124725f, 0.24611230194568634f, 0.33791524171829224f,
    0.44070982933044434f, 0.5626170039176941f, 0.7229568362236023f, 1.0f};
/* mps_bitsandbytes/functional.py:29-32 */
static const float FP4[16] = {
    0.0f, 0.0625f, 0.125f, 0.25f, 0.375f, 0.5f, 0.75f, 1.0f,
    -0.0f, -0.0625f, -0.125f, -0.25f, -0.375f, -0.5f, -0.75f, -1.0f};

static const float *code_of(int qt) { return qt == 0 ? NF4 : FP4; }

/* argmin_i |v - code[i]|, first index on ties (functional.py:242-243). */
static inline int nearest16(float v, const float *code) {
    int best = 0;
    float bd = fabsf(v - code[0]);
    for (int i = 1; i < 16; ++i) {
        float d = fabsf(v - code[i]);
        if (d < bd) { bd = d; best = i; }
    }
    return best;
}

int64_t o_padded_k(int64_t K, int64_t bs) {            /* functional.py:219-221 */
    int64_t kp = ((K + bs - 1) / bs) * bs;
    if (kp % 2) kp += bs;
    return kp;
}

/* functional.py:216-255.  A: fp32 [rows, cols] (fp16/bf16 inputs are widened exactly by
 * the caller).  packed: [rows, Kp/2]; absmax: [rows, Kp/bs]. qt: 0 = nf4, 1 = fp4. */
void o_quantize_4bit(const float *A, int64_t rows, int64_t cols, int64_t bs, int qt,
                     uint8_t *packed, float *absmax) {
    const float *code = code_of(qt);
    const int64_t Kp = o_padded_k(cols, bs), nb = Kp / bs;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        uint8_t *idx = (uint8_t *)malloc((size_t)Kp);
        for (int64_t b = 0; b < nb; ++b) {
            float am = 0.0f;
            for (int64_t j = 0; j < bs; ++j) {
                int64_t k = b * bs + j;
                float x = k < cols ? A[r * cols + k] : 0.0f;
                float a = fabsf(x);
                if (a > am || a != a) am = a;
            }
            if (am < 1e-8f) am = 1e-8f;                  /* clamp(min=1e-8), :232 */
            absmax[r * nb + b] = am;
            for (int64_t j = 0; j < bs; ++j) {
                int64_t k = b * bs + j;
                float x = k < cols ? A[r * cols + k] : 0.0f;
                idx[k] = (uint8_t)nearest16(x / am, code);  /* :239-243 */
            }
        }
        for (int64_t j = 0; j < Kp / 2; ++j)
            packed[r * (Kp / 2) + j] = (uint8_t)(idx[2 * j] | (idx[2 * j + 1] << 4)); /* :251 */
        free(idx);
    }
}

/* functional.py:348-386: fp32 values code[idx] * absmax, [rows, cols]. */
void o_dequantize_4bit(const uint8_t *packed, const float *absmax, int64_t rows, int64_t cols,
                       int64_t bs, int qt, float *out) {
    const float *code = code_of(qt);
    const int64_t Kp = o_padded_k(cols, bs), nb = Kp / bs;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t k = 0; k < cols; ++k) {
            uint8_t byte = packed[r * (Kp / 2) + k / 2];
            int idx = (k & 1) ? (byte >> 4) : (byte & 15);
            out[r * cols + k] = code[idx] * absmax[r * nb + k / bs];
        }
}

/* functional.py:591-594 as used for double-quantised absmax: q * (absmax2 / 127). */
void o_dequantize_absmax(const int8_t *q, const float *absmax2, int64_t n, float *out) {
    for (int64_t i = 0; i < n; ++i) out[i] = (float)q[i] * (absmax2[i / 256] / 127.0f);
}

/* functional.py:752-773 on fp16 data: every call first materialises the whole weight in
 * fp16 (the reference's CPU hot spot), then y = x @ W^T with fp32 accumulation, rounded
 * to fp16.  x: [M,K] fp16, y: [M,N] fp16, absmax fp32 [N, nb] (already expanded). */
void o_matmul_4bit_f16(const _Float16 *x, const uint8_t *packed, const float *absmax,
                       int64_t M, int64_t N, int64_t K, int64_t bs, int qt,
                       const _Float16 *bias, _Float16 *y, _Float16 *wscratch) {
    const float *code = code_of(qt);
    const int64_t Kp = o_padded_k(K, bs), nb = Kp / bs;
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        _Float16 *w = wscratch + n * K;
        for (int64_t k = 0; k < K; ++k) {
            uint8_t byte = packed[n * (Kp / 2) + k / 2];
            int idx = (k & 1) ? (byte >> 4) : (byte & 15);
            w[k] = (_Float16)(code[idx] * absmax[n * nb + k / bs]);
        }
    }
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        const _Float16 *w = wscratch + n * K;
        for (int64_t m = 0; m < M; ++m) {
            const _Float16 *xr = x + m * K;
            float acc[8] = {0};
            int64_t k = 0;
            for (; k + 8 <= K; k += 8)
                for (int j = 0; j < 8; ++j) acc[j] += (float)xr[k + j] * (float)w[k + j];
            float s = 0.0f;
            for (; k < K; ++k) s += (float)xr[k] * (float)w[k];
            for (int j = 0; j < 8; ++j) s += acc[j];
            if (bias) s += (float)bias[n];
            y[m * N + n] = (_Float16)s;
        }
    }
}

/* ------------------------------------------------------------------------------------
 * Decision thresholds.  For two neighbouring codes lo < hi (by value) the 16-way search
 * prefers `lo_first ? lo : hi` on a tie of the ROUNDED fp32 distances.  Both rounded
 * distances are monotone in v, so there is one float t with: v <= t picks lo, v > t
 * picks hi.  o_threshold finds it by bisection over the float bit patterns.
 * ---------------------------------------------------------------------------------- */
static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
/* order-preserving map float <-> uint32 */
static inline uint32_t ord(float f) { uint32_t u = f2u(f); return (u & 0x80000000u) ? ~u : (u | 0x80000000u); }
static inline float unord(uint32_t o) { return u2f((o & 0x80000000u) ? (o & 0x7FFFFFFFu) : ~o); }

float o_threshold(float lo, float hi, int lo_first) {
    uint32_t a = ord(lo), b = ord(hi);                  /* at a: lo wins; at b: hi wins */
    while (b - a > 1) {
        uint32_t m = a + (b - a) / 2;
        float v = unord(m);
        float dl = fabsf(v - lo), dh = fabsf(v - hi);
        int hi_wins = lo_first ? (dh < dl) : (dh <= dl);
        if (hi_wins) b = m; else a = m;
    }
    return unord(a);
}

/* NF4: codes ascend with the index, ties go to the lower index.  t[i] separates i | i+1. */
void o_nf4_thresholds(float *t) {
    for (int i = 0; i < 15; ++i) t[i] = o_threshold(NF4[i], NF4[i + 1], 1);
}
/* FP4 on |v|: magnitudes ascend with index 0..7; ties go to the lower magnitude (for
 * negative v: index 8+j beats 8+j+1, and index 0 beats 9).  t[i] separates i | i+1. */
void o_fp4_thresholds(float *t) {
    for (int i = 0; i < 7; ++i) t[i] = o_threshold(FP4[i], FP4[i + 1], 1);
}

/* The threshold form of the search, exactly as the CUDA kernel evaluates it. */
int o_nearest_by_threshold(float v, int qt, const float *t) {
    if (qt == 0) {
        int idx = 0;
        for (int i = 0; i < 15; ++i) idx += (v > t[i]);
        return idx;
    }
    float a = fabsf(v);
    int m = 0;
    for (int i = 0; i < 7; ++i) m += (a > t[i]);
    return (v < 0.0f && m != 0) ? m + 8 : m;
}

/* Exhaustive proof over the 16-bit input formats.  is_bf16 = 0: fp16, 1: bf16.
 * For every finite block maximum a > 0 and every finite x with |x| <= a, compares
 *   reference: nearest16(x / a)           (IEEE division, 16-way search)
 *   kernel   : threshold search on q', q' = fma(fma(-q, a, x), r, q), q = x * r, r = 1/a
 * Only block maxima in [a_min, a_max] are visited (outside it the kernel divides).
 * Returns the number of (x, a) pairs whose code differs (0 proves equivalence). */
static float widen16(uint32_t h, int is_bf16) {
    if (is_bf16) return u2f(h << 16);
    _Float16 f; uint16_t b = (uint16_t)h; memcpy(&f, &b, 2); return (float)f;
}
int64_t o_prove_quantizer(int qt, int is_bf16, int64_t a_stride, float a_min, float a_max) {
    float t[15];
    if (qt == 0) o_nf4_thresholds(t); else o_fp4_thresholds(t);
    const float *code = code_of(qt);
    int64_t bad = 0;
#pragma omp parallel for schedule(dynamic, 64) reduction(+ : bad)
    for (int64_t ai = 1; ai < 0x8000; ai += a_stride) {
        float a = widen16((uint32_t)ai, is_bf16);
        if (!(a > 0.0f) || isinf(a) || isnan(a) || a < a_min || a > a_max) continue;
        float r = 1.0f / a;
        for (uint32_t xi = 0; xi < 0x10000; ++xi) {
            float x = widen16(xi, is_bf16);
            if (isnan(x) || fabsf(x) > a) continue;
            int ref = nearest16(x / a, code);
            float q = x * r;
            float q2 = fmaf(fmaf(-q, a, x), r, q);
            int got = o_nearest_by_threshold(q2, qt, t);
            bad += (ref != got);
        }
    }
    return bad;
}

/* Threshold search vs 16-way search on every float in +-window ulps around every
 * threshold and on n_random floats in [-1, 1]; returns the number of disagreements. */
int64_t o_prove_thresholds(int qt, int window, int64_t n_random) {
    float t[15];
    int nt = qt == 0 ? 15 : 7;
    if (qt == 0) o_nf4_thresholds(t); else o_fp4_thresholds(t);
    const float *code = code_of(qt);
    int64_t bad = 0;
    for (int i = 0; i < nt; ++i)
        for (int s = -1; s <= 1; s += 2) {
            uint32_t c = ord(s < 0 ? -t[i] : t[i]);
            for (int d = -window; d <= window; ++d) {
                float v = unord(c + d);
                bad += nearest16(v, code) != o_nearest_by_threshold(v, qt, t);
            }
        }
    uint64_t st = 88172645463325252ull;
    for (int64_t i = 0; i < n_random; ++i) {
        st ^= st << 13; st ^= st >> 7; st ^= st << 17;
        float v = (float)((double)(st >> 11) / 9007199254740992.0 * 2.0 - 1.0);
        bad += nearest16(v, code) != o_nearest_by_threshold(v, qt, t);
    }
    return bad;
}

/* The bucket form of the NF4 search used by the fast CUDA quantiser: g = trunc(fma(v, 8, 8)) clamped to 0..15,
 * code = (thresholds below bucket g) + (v > first threshold of g) + (v > second).  Compared with the plain
 * threshold search on EVERY float whose ordered key is a multiple of `stride` (stride 1: all 2^32 bit patterns
 * except NaN, values outside [-1, 1] included); returns the number of disagreements. */
int64_t o_prove_nf4_buckets(int64_t stride) {
    float t[15];
    o_nf4_thresholds(t);
    const float inf = INFINITY;
    const float ta[16] = {inf, t[0], inf, t[1], t[2], t[3], t[4], t[6], t[7], t[9], t[10], t[11], t[12], t[13], t[14], inf};
    float tb[16];
    for (int g = 0; g < 16; ++g) tb[g] = inf;
    tb[6] = t[5]; tb[8] = t[8];
    const uint64_t base = 0xFEDCBA9764321100ull;
    int64_t bad = 0;
#pragma omp parallel for schedule(static) reduction(+ : bad)
    for (int64_t k = 0; k < 0x100000000ll; k += stride) {
        const float v = unord((uint32_t)k);
        if (isnan(v)) continue;
        const float f = fmaf(v, 8.0f, 8.0f);
        int g = f >= 2147483648.0f ? 2147483647 : (f <= -2147483648.0f ? (-2147483647 - 1) : (int)f);   /* cvt.rzi.s32.f32 saturates */
        g = g < 0 ? 0 : (g > 15 ? 15 : g);
        const int got = (int)((base >> (4 * g)) & 15u) + (v > ta[g]) + (v > tb[g]);
        bad += (got != o_nearest_by_threshold(v, 0, t));
    }
    return bad;
}

/* The NF4 search as the streaming CUDA quantiser does it: [-1, 1] in 32 buckets of width 1/16, none of which holds
 * more than one of the fifteen thresholds; the bucket is the low six bits of fma_rz(v, 16, 2^23 + 16) =
 * floor(16 v + 16) - no conversion, no clamp (32, reached by v = 1 only, uses bucket 31's entry) - and
 * code = (thresholds below the bucket) + (v > the bucket's threshold).  Checked against the plain threshold search on
 * every float of [-1, 1] whose ordered key is a multiple of `stride` (the quotient x / absmax of a block never leaves
 * that interval); returns the number of disagreements (2^40 added if the rounding mode could not be set, 2^41 if a
 * bucket holds two thresholds). */
int64_t o_prove_nf4_buckets32_rz(int64_t stride) {
    float t[15];
    o_nf4_thresholds(t);
    float tg[32];
    int base[32];
    int64_t bad = 0;
    for (int g = 0; g < 32; ++g) {
        const float lo = -1.0f + (float)g / 16.0f, hi = -1.0f + (float)(g + 1) / 16.0f;   /* exact */
        int below = 0, inside = 0;
        tg[g] = INFINITY;
        for (int i = 0; i < 15; ++i) {
            if (t[i] < lo) ++below;
            else if (t[i] < hi) { tg[g] = t[i]; ++inside; }
        }
        base[g] = below;
        if (inside > 1) bad += 1ll << 41;
    }
#pragma omp parallel reduction(+ : bad)
    {
        const int old_mode = fegetround();
        fesetround(FE_TOWARDZERO);
        {   /* the rounding mode must really be in force: a tiny negative v lands in bucket 15, not 16 */
            volatile float tiny = -1e-30f;
            const float f0 = fmaf(tiny, 16.0f, 8388624.0f);
            uint32_t b0;
            memcpy(&b0, &f0, 4);
            if ((b0 & 63u) != 15u) bad += 1ll << 40;
        }
#pragma omp for schedule(static)
        for (int64_t k = 0; k < 0x100000000ll; k += stride) {
            const float v = unord((uint32_t)k);
            if (isnan(v) || v < -1.0f || v > 1.0f) continue;
            volatile float vv = v;                                   /* keeps the fma out of constant folding */
            const float f = fmaf(vv, 16.0f, 8388624.0f);
            uint32_t bits;
            memcpy(&bits, &f, 4);
            if ((bits & 0xFFFFFFC0u) != 0x4B000000u) { bad += 1; continue; }   /* the kernel adds bits << 8 to the table address unmasked */
            int g = (int)(bits & 63u);
            if (g > 32) { bad += 1; continue; }
            if (g == 32) g = 31;
            const int got = base[g] + (v > tg[g]);
            bad += (got != o_nearest_by_threshold(v, 0, t));
        }
        fesetround(old_mode);
    }
    return bad;
}

/* The FP4 search of the streaming CUDA quantiser: the magnitude a = |v| in 16 buckets of width 1/16, none of which
 * holds more than one of the seven thresholds; bucket = low five bits of fma_rz(a, 16, 2^23) = floor(16 a) (16, reached
 * by a = 1 only, uses bucket 15's entry); m = (thresholds below the bucket) + (a > the bucket's threshold); the sign
 * as in the threshold form.  Every float of [-1, 1] whose ordered key is a multiple of `stride`. */
int64_t o_prove_fp4_buckets16_rz(int64_t stride) {
    float t[15];
    o_fp4_thresholds(t);
    float tg[16];
    int base[16];
    int64_t bad = 0;
    for (int g = 0; g < 16; ++g) {
        const float lo = (float)g / 16.0f, hi = (float)(g + 1) / 16.0f;   /* exact */
        int below = 0, inside = 0;
        tg[g] = INFINITY;
        for (int i = 0; i < 7; ++i) {
            if (t[i] < lo) ++below;
            else if (t[i] < hi) { tg[g] = t[i]; ++inside; }
        }
        base[g] = below;
        if (inside > 1) bad += 1ll << 41;
    }
#pragma omp parallel reduction(+ : bad)
    {
        const int old_mode = fegetround();
        fesetround(FE_TOWARDZERO);
        {   /* the rounding mode must really be in force: just below 1/16 stays in bucket 0 */
            volatile float edge = 0.0624999963f;
            const float f0 = fmaf(edge, 16.0f, 8388608.0f);
            uint32_t b0;
            memcpy(&b0, &f0, 4);
            if ((b0 & 31u) != 0u) bad += 1ll << 40;
        }
#pragma omp for schedule(static)
        for (int64_t k = 0; k < 0x100000000ll; k += stride) {
            const float v = unord((uint32_t)k);
            if (isnan(v) || v < -1.0f || v > 1.0f) continue;
            volatile float aa = fabsf(v);
            const float a = aa;
            const float f = fmaf(aa, 16.0f, 8388608.0f);
            uint32_t bits;
            memcpy(&bits, &f, 4);
            if ((bits & 0xFFFFFFE0u) != 0x4B000000u) { bad += 1; continue; }   /* bits << 8 is used unmasked */
            int g = (int)(bits & 31u);
            if (g > 16) { bad += 1; continue; }
            if (g == 16) g = 15;
            const int m = base[g] + (a > tg[g]);
            const int got = (v < 0.0f && m != 0) ? m + 8 : m;
            bad += (got != o_nearest_by_threshold(v, 1, t));
        }
        fesetround(old_mode);
    }
    return bad;
}

/* Thread count of the OpenMP loops above.  A launcher may export OMP_NUM_THREADS=1 (torch.distributed.run does); the
 * timed CPU baseline sets the count explicitly and reports what it got.  n <= 0: query only. */
int o_threads(int n) {
    if (n > 0) omp_set_num_threads(n);
    return omp_get_max_threads();
}
