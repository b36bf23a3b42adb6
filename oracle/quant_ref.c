/* Plain-C restatement of cinnamon's FP8 quantisers.  TEST INFRASTRUCTURE ONLY:
 * a checker for the CUDA library and for the Python restatement beside it;
 * never linked into, or called from, the shipped package.
 *
 * Follows src/kernels.py of shyampathak22/cinnamon:
 *   row-wise  1x128 tiles   lines 41-71   (amax, floor 1e-4, /448, x/scale, clamp, e4m3 RNE)
 *   block-wise 128x128      lines 97-132
 * Divisions are IEEE round-to-nearest (build with -ffp-contract=off, no -ffast-math);
 * the GPU's approximate div.full.f32 cannot be restated on a CPU.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

/* fp32 -> e4m3fn code, round-to-nearest-even, finite saturation at 448, NaN -> 0x7F
 * (semantics of cvt.rn.satfinite.e4m3x2.f32, the cast at src/kernels.py:62,123). */
uint8_t oracle_e4m3_encode1(float v) {
    uint32_t bits = f2u(v);
    uint8_t sign = (uint8_t)((bits >> 24) & 0x80);
    uint32_t mag = bits & 0x7FFFFFFFu;
    if (mag > 0x7F800000u) return 0x7F;
    float a = fabsf(v);
    if (a >= 448.0f) return sign | 0x7E;
    if (a < 0.015625f) {                       /* subnormal: units of 2^-9, ties to even */
        double t = (double)a * 512.0;
        return sign | (uint8_t)nearbyint(t);   /* default rounding mode = nearest-even */
    }
    uint32_t lsb = (mag >> 20) & 1u;
    uint32_t r = (mag + 0x7FFFFu + lsb) & ~0xFFFFFu;
    int32_t e = (int32_t)(r >> 23) - 127 + 7;
    uint32_t m = (r >> 20) & 7u;
    uint32_t code = ((uint32_t)e << 3) | m;
    if (code > 0x7E) code = 0x7E;
    return sign | (uint8_t)code;
}

void oracle_e4m3_encode(const float *v, uint8_t *out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) out[i] = oracle_e4m3_encode1(v[i]);
}

static float scale_from_amax(float amax, int round_scale) {
    if (!(amax > 1e-4f)) amax = 1e-4f;                 /* :53 / :114 */
    float s = amax / 448.0f;                           /* :57 / :118 */
    if (round_scale) {                                 /* :55 / :116 */
        float lg = (float)log2((double)s);
        s = ldexpf(1.0f, (int)ceilf(lg));
    }
    return s;
}

static uint8_t quant1(float x, float s) {
    float y = x / s;                                   /* :60 */
    y = fmaxf(y, -448.0f);                             /* PTX max/min drop NaN, as fmaxf/fminf do */
    y = fminf(y, 448.0f);
    return oracle_e4m3_encode1(y);
}

/* x: M x N fp32 with row pitch ld (elements).  q: M x N.  scales: M x ceil(N/128). */
void oracle_quant_rowwise_f32(const float *x, int64_t M, int64_t N, int64_t ld,
                              uint8_t *q, float *scales, int round_scale) {
    int64_t nb = (N + 127) / 128;
    for (int64_t r = 0; r < M; ++r)
        for (int64_t b = 0; b < nb; ++b) {
            int64_t c0 = b * 128, c1 = c0 + 128 < N ? c0 + 128 : N;
            float amax = 0.0f;
            for (int64_t c = c0; c < c1; ++c) { float a = fabsf(x[r * ld + c]); if (a > amax) amax = a; }
            float s = scale_from_amax(amax, round_scale);
            scales[r * nb + b] = s;
            for (int64_t c = c0; c < c1; ++c) q[r * N + c] = quant1(x[r * ld + c], s);
        }
}

/* 128 x 128 blocks; scales: ceil(M/128) x ceil(N/128). */
void oracle_quant_blockwise_f32(const float *x, int64_t M, int64_t N, int64_t ld,
                                uint8_t *q, float *scales, int round_scale) {
    int64_t mb = (M + 127) / 128, nb = (N + 127) / 128;
    for (int64_t bi = 0; bi < mb; ++bi)
        for (int64_t bj = 0; bj < nb; ++bj) {
            int64_t r1 = bi * 128 + 128 < M ? bi * 128 + 128 : M;
            int64_t c1 = bj * 128 + 128 < N ? bj * 128 + 128 : N;
            float amax = 0.0f;
            for (int64_t r = bi * 128; r < r1; ++r)
                for (int64_t c = bj * 128; c < c1; ++c) { float a = fabsf(x[r * ld + c]); if (a > amax) amax = a; }
            float s = scale_from_amax(amax, round_scale);
            scales[bi * nb + bj] = s;
            for (int64_t r = bi * 128; r < r1; ++r)
                for (int64_t c = bj * 128; c < c1; ++c) q[r * N + c] = quant1(x[r * ld + c], s);
        }
}
