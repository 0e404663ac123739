/* CPU oracle of the quantizer rules in plain C. TEST INFRASTRUCTURE ONLY: the tests load it with ctypes to check
 * oracle/rules.py (PyTorch) and the CUDA kernels against a second, independent restatement that does its own E4M3
 * rounding bit by bit instead of relying on a library conversion. The product never links or calls it.
 *
 * Rules restated (paths relative to the reference project):
 *   amax, NaN-propagating ............ zig/fp8.zig:33-52
 *   scale = amax / 448, 1 if 0 ........ zig/fp8.zig:54-60, tests/test_fp8_gemm.py:202-206
 *   E8M0 byte of the quotient ......... zig/fp8.zig:63-70, tests/test_fp8_gemm.py:207-211
 *   codes = e4m3(x / scale) ........... zig/fp8.zig:95-114, tests/test_fp8_gemm.py:214-215
 * Parity: pinned through tests/test_oracle_golden.py (same golden vectors as oracle/rules.py).
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

static uint32_t bits_of(float v) {
    uint32_t b;
    memcpy(&b, &v, 4);
    return b;
}

static float float_of(uint32_t b) {
    float v;
    memcpy(&v, &b, 4);
    return v;
}

/* Nearest-even E4M3 (fn) code of an FP32 value, magnitudes above 448 saturate, NaN gives 0x7F | sign. */
uint8_t zck_oracle_e4m3(float v) {
    uint32_t b = bits_of(v);
    uint8_t sign = (uint8_t)((b >> 24) & 0x80);
    uint32_t mag = b & 0x7FFFFFFFu;
    if (mag > 0x7F800000u) return (uint8_t)(sign | 0x7F); /* NaN */
    float a = float_of(mag);
    if (a >= 448.0f) return (uint8_t)(sign | 0x7E);        /* saturate (also +-inf) */
    if (a < 0.0009765625f) return sign;                      /* below half of the least subnormal 2^-9 ... */
    /* value = q * step with step = 2^(e-3), e = max(exponent, -6): round q to nearest even */
    int exponent;
    (void)frexpf(a, &exponent); /* a = f * 2^exponent, f in [0.5, 1) -> binade exponent-1 */
    int e = exponent - 1;
    if (e < -6) e = -6;
    float step = ldexpf(1.0f, e - 3);
    float q = a / step;            /* exact: a power-of-two division */
    float r = nearbyintf(q);       /* ties to even in the default rounding mode */
    float rounded = r * step;
    if (rounded >= 512.0f) return (uint8_t)(sign | 0x7E);
    /* encode `rounded` (a representable E4M3 value, possibly in the next binade) */
    if (rounded == 0.0f) return sign;
    int e2;
    float f = frexpf(rounded, &e2); /* rounded = f * 2^e2 */
    int binade = e2 - 1;
    if (binade < -6) { /* subnormal: mantissa counts multiples of 2^-9 */
        return (uint8_t)(sign | (uint8_t)(rounded * 512.0f));
    }
    uint32_t mant = (uint32_t)((f * 2.0f - 1.0f) * 8.0f);
    return (uint8_t)(sign | ((uint32_t)(binade + 7) << 3) | mant);
}

static float amax_update(float amax, float x) {
    float a = fabsf(x);
    if (isnan(amax) || isnan(a)) return NAN;
    return a > amax ? a : amax;
}

float zck_oracle_scale_f32(float amax) {
    float q = amax / 448.0f;
    return q == 0.0f ? 1.0f : q;
}

uint8_t zck_oracle_scale_e8m0(float amax) {
    uint32_t mag = bits_of(amax / 448.0f) & 0x7FFFFFFFu;
    uint32_t up = (mag + 0x7FFFFFu) >> 23;
    if (up > 254u) up = 254u;
    uint32_t byte = mag <= 0x00400000u ? 0u : up;
    if (mag == 0u) byte = 127u;
    if (mag >= 0x7F800000u) byte = 255u;
    return (uint8_t)byte;
}

float zck_oracle_e8m0_value(uint8_t byte) {
    if (byte == 255u) return NAN;
    return float_of(byte == 0u ? 0x00400000u : (uint32_t)byte << 23);
}

/* quantize_fp8_rows on FP32 input: x[m][k] row-major, codes[m][k], scales laid out as scales[g * m + row]
 * (FP32 values, or E8M0 bytes when e8m0 != 0). */
void zck_oracle_quantize_rows(const float* x, uint32_t m, uint32_t k, uint8_t* codes, void* scales, int e8m0) {
    uint32_t groups = k / 128;
    for (uint32_t row = 0; row < m; ++row) {
        for (uint32_t g = 0; g < groups; ++g) {
            const float* src = x + (size_t)row * k + (size_t)g * 128;
            float amax = 0.0f;
            for (int i = 0; i < 128; ++i) amax = amax_update(amax, src[i]);
            float divisor;
            if (e8m0) {
                uint8_t byte = zck_oracle_scale_e8m0(amax);
                ((uint8_t*)scales)[(size_t)g * m + row] = byte;
                divisor = zck_oracle_e8m0_value(byte);
            } else {
                divisor = zck_oracle_scale_f32(amax);
                ((float*)scales)[(size_t)g * m + row] = divisor;
            }
            for (int i = 0; i < 128; ++i) codes[(size_t)row * k + (size_t)g * 128 + i] = zck_oracle_e4m3(src[i] / divisor);
        }
    }
}

/* quantize_fp8_tiles on FP32 input: one scale per 128 x 128 tile at scales[tile_row * (k/128) + tile_col]; rows past
 * n do not count. */
void zck_oracle_quantize_tiles(const float* w, uint32_t n, uint32_t k, uint8_t* codes, void* scales, int e8m0) {
    uint32_t tile_rows = (n + 127) / 128, tile_cols = k / 128;
    for (uint32_t tr = 0; tr < tile_rows; ++tr) {
        for (uint32_t tc = 0; tc < tile_cols; ++tc) {
            uint32_t r0 = tr * 128, r1 = r0 + 128 < n ? r0 + 128 : n;
            float amax = 0.0f;
            for (uint32_t r = r0; r < r1; ++r)
                for (int i = 0; i < 128; ++i) amax = amax_update(amax, w[(size_t)r * k + (size_t)tc * 128 + i]);
            float divisor;
            if (e8m0) {
                uint8_t byte = zck_oracle_scale_e8m0(amax);
                ((uint8_t*)scales)[(size_t)tr * tile_cols + tc] = byte;
                divisor = zck_oracle_e8m0_value(byte);
            } else {
                divisor = zck_oracle_scale_f32(amax);
                ((float*)scales)[(size_t)tr * tile_cols + tc] = divisor;
            }
            for (uint32_t r = r0; r < r1; ++r)
                for (int i = 0; i < 128; ++i) {
                    size_t at = (size_t)r * k + (size_t)tc * 128 + i;
                    codes[at] = zck_oracle_e4m3(w[at] / divisor);
                }
        }
    }
}
