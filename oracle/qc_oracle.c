/*
 * CPU oracle for the quantization-cast hot path.
 *
 * THIS IS TEST INFRASTRUCTURE, NOT PRODUCT CODE.  Only the test-suite, the smoke check and the
 * CPU-baseline leg of the benchmark may load this library; the shipped CUDA path never does.
 *
 * It restates, in scalar C with integer bit arithmetic, the algorithms that the reference project
 * (vkuzo/quant_cast_bench) defines as plain PyTorch in
 *     quant_cast_bench/quant_cast_gold/recipes.py   ("G" below)
 *     quant_cast_bench/quant_cast_gold/utils.py     ("GU" below)
 * Each function cites the reference lines it follows.  Parity of this file with the reference is
 * pinned by golden vectors generated from the reference itself (tests/golden/make_golden.py runs
 * G on CPU and stores inputs + outputs; tests/test_oracle_golden.py replays them through this file).
 *
 * Pieces that the reference does not contain and that are therefore NOT pinned by it
 * ("extensions"): the e5m2 element format, the FLOOR scale mode of mxfp8, and the Philox-keyed
 * stochastic-rounding stream (the reference draws its dither from a float-uniform generator of a
 * newer PyTorch; only the dither/truncate/encode step G:1392-1406 is followed here).  Philox4x32-10
 * itself is pinned by the published Random123 known-answer vectors.
 *
 * Third-party arithmetic of record: PyTorch's fp32 -> float8_e4m3fn / float8_e5m2 conversions
 * (round to nearest even).  They are restated in f32_to_fp8() and pinned against PyTorch in the
 * golden-vector tests.  One deliberate difference: this oracle SATURATES to the largest finite
 * value (e4m3: +-448, e5m2: +-57344) where PyTorch's e4m3 cast yields NaN above 464 and its e5m2
 * cast yields Inf; inputs that reach that range cannot occur when the scale was computed from the
 * same tensor.
 *
 * Build: gcc -O2 -fopenmp -ffp-contract=off -fno-fast-math -shared -fPIC (see oracle/build.py).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define QC_FMT_E4M3 0
#define QC_FMT_E5M2 1

#define QC_ROWWISE 1   /* 1x32 blocks along the last dim, outputs in the input frame      */
#define QC_COLWISE 2   /* 32x1 blocks down the rows, outputs in the transposed frame      */
#define QC_SWIZZLE 4   /* block scales in the 32x4x4 blocked layout instead of row-major  */
#define QC_FLOOR   8   /* mxfp8: FLOOR scale mode instead of RCEIL                        */
#define QC_SR      16  /* nvfp4: stochastic rounding of the fp4 values                    */

/* ------------------------------------------------------------------------------------------ */
/* bit helpers                                                                                */
/* ------------------------------------------------------------------------------------------ */
static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline float bf16_to_f32(uint16_t h) { return u2f((uint32_t)h << 16); }
static inline uint16_t bf16_abs(uint16_t h) { return (uint16_t)(h & 0x7FFFu); }

/*
 * fp32 -> 8-bit float, round to nearest even, saturating to the largest finite value.
 * ebits/mbits/bias describe the target; max_code is the largest finite magnitude code
 * (e4m3fn: 0x7E = 448, e5m2: 0x7B = 57344).  NaN -> 0x7F with the sign dropped.
 * Restates PyTorch's `.to(torch.float8_e4m3fn)` / `.to(torch.float8_e5m2)` as used at
 * G:306, G:567, G:1190, G:1259 for every value whose magnitude does not overflow.
 */
static inline uint8_t f32_to_fp8(float f, int mbits, int bias, uint32_t max_code)
{
    uint32_t u = f2u(f);
    uint32_t sign = (u >> 31) << 7;
    uint32_t a = u & 0x7FFFFFFFu;
    if (a > 0x7F800000u) return 0x7F;                       /* NaN */
    int e = (int)(a >> 23) - 127;                           /* unbiased fp32 exponent */
    uint32_t code;
    if (e < 1 - bias) {
        /* target subnormal (or zero): count quanta of 2^(1-bias-mbits), ties to even */
        float scaled = u2f(a) * u2f((uint32_t)(127 + bias - 1 + mbits) << 23);
        code = (uint32_t)lrintf(scaled);                    /* default rounding mode = RNE */
    } else {
        int shift = 23 - mbits;
        uint32_t mant = a & 0x7FFFFFu;
        code = ((uint32_t)(e + bias) << mbits) | (mant >> shift);
        uint32_t rem = mant & ((1u << shift) - 1u);
        uint32_t half = 1u << (shift - 1);
        if (rem > half || (rem == half && (code & 1u))) code++;
    }
    if (code > max_code) code = max_code;
    return (uint8_t)(sign | code);
}

static inline uint8_t f32_to_fp8_fmt(float f, int fmt)
{
    return fmt == QC_FMT_E5M2 ? f32_to_fp8(f, 2, 15, 0x7B) : f32_to_fp8(f, 3, 7, 0x7E);
}

static inline float fp8_max_fmt(int fmt) { return fmt == QC_FMT_E5M2 ? 57344.0f : 448.0f; }

/* `tensor / python_scalar` of the gold recipes.  Eager PyTorch computes it as one IEEE division on the CPU, and as a
 * multiplication with the fp32 reciprocal of the scalar on a CUDA device (aten/src/ATen/native/cuda/
 * BinaryDivTrueKernel.cu: "a * (1 / b)" when b is a host scalar).  qco_set_recip_div(1) selects the second form for
 * every such division below (amax / 448, amax / 57344, amax / 2688, block amax / 6); the default is the first. */
static int g_recip_div = 0;
void qco_set_recip_div(int on) { g_recip_div = on != 0; }
int qco_get_recip_div(void) { return g_recip_div; }
static inline float div_by_const(float a, float c)
{
    if (g_recip_div) {
        volatile float inv = 1.0f / c;   /* rounded to fp32 before the product */
        return a * inv;
    }
    return a / c;
}

/* e4m3fn byte -> fp32 (exact).  Inverse of the cast at G:1259 as read back at G:1261. */
static inline float e4m3_to_f32(uint8_t b)
{
    uint32_t sign = (uint32_t)(b & 0x80) << 24;
    uint32_t e = (b >> 3) & 0xF, m = b & 7;
    if (e == 0xF && m == 7) return u2f(sign | 0x7FC00000u);
    if (e == 0) return u2f(sign | f2u((float)m * 0.001953125f)); /* m * 2^-9 */
    return u2f(sign | ((e + 120u) << 23) | (m << 20));
}

/*
 * fp32 -> fp4 e2m1 code (sign in bit 3), round to nearest even, saturating at +-6.
 * Follows GU:15-57 (f32_to_f4_unpacked): sign split, >= 6.0 saturates to code 7, values below 1.0
 * are rounded on the 0.5 grid, the rest on the e2m1 normal grid; a negative value that rounds to
 * zero keeps its sign (code 8).
 */
static inline uint8_t f32_to_e2m1(float f)
{
    uint32_t u = f2u(f);
    uint8_t sign = (uint8_t)((u >> 31) << 3);
    uint32_t a = u & 0x7FFFFFFFu;
    float af = u2f(a);
    uint32_t code;
    if (af >= 6.0f) {
        code = 7;
    } else if (af < 1.0f) {
        code = (uint32_t)lrintf(af * 2.0f);                 /* quanta of 0.5, ties to even */
    } else {
        int e = (int)(a >> 23) - 127;                       /* 0, 1 or 2 */
        uint32_t mant = a & 0x7FFFFFu;
        code = ((uint32_t)(e + 1) << 1) | (mant >> 22);
        uint32_t rem = mant & 0x3FFFFFu;
        if (rem > 0x200000u || (rem == 0x200000u && (code & 1u))) code++;
    }
    return (uint8_t)(sign | code);
}

/*
 * amax -> e8m0 byte, RCEIL.  Follows G:494-528 (_amax_to_e8m0_rceil): descale = fp32(amax) *
 * fp32(1/448), then the biased exponent is bumped when any mantissa bit is set (for fp32
 * subnormals: only above 2^-127); non-finite -> 255.
 */
static inline uint8_t amax_to_e8m0_rceil(float amax)
{
    const float inv448 = u2f(0x3B124925u);                  /* fp32(1.0/448.0) */
    float descale = amax * inv448;
    uint32_t b = f2u(descale);
    if ((b & 0x7F800000u) == 0x7F800000u) return 255;
    uint32_t e = (b >> 23) & 0xFF, m = b & 0x7FFFFFu;
    uint32_t up = (e == 0) ? (m > 0x400000u) : (m != 0);
    return (uint8_t)(e + up);
}

/*
 * amax -> e8m0 byte, FLOOR (extension; not in the reference).  OCP MX v1.0 section 6.3: shared
 * exponent = floor(log2(amax)) - emax_elem, emax_elem = 8 for e4m3, clamped at the bottom of the
 * e8m0 range; non-finite -> 255.  The exponent is read from the fp32 exponent field.
 */
static inline uint8_t amax_to_e8m0_floor(float amax)
{
    uint32_t b = f2u(amax);
    uint32_t e = (b >> 23) & 0xFF;
    if (e == 0xFF) return 255;
    return (uint8_t)(e > 8 ? e - 8 : 0);
}

/*
 * e8m0 byte -> fp32 reciprocal 2^(127-byte).  Follows G:538-558: biased 254-byte shifted into the
 * exponent field; byte 254 -> the subnormal 2^-127; byte 255 -> NaN.
 * In FLOOR mode the scale is first clamped to the smallest normal (byte 0 acts as byte 1), which
 * is what dividing by max(2^(byte-127), 2^-126) gives.
 */
static inline float e8m0_to_recip(uint8_t byte, int floor_mode)
{
    uint32_t bb = byte;
    if (floor_mode && bb == 0) bb = 1;
    uint32_t r = (254u - bb) & 0xFFu;
    if (r == 0) return u2f(0x00400000u);
    if (r == 255) return u2f(0x7F800001u);
    return u2f(r << 23);
}

/*
 * Offset of block-scale (r, c) inside the 32x4x4 blocked layout whose grid has ncb column blocks.
 * Follows G:1000-1037 (_to_blocked_4d): atoms of 128 rows x 4 cols become 32 x 16 bytes.
 */
static inline size_t blocked_offset(size_t r, size_t c, size_t ncb)
{
    size_t br = r / 128, rr = r % 128, bc = c / 4, c4 = c % 4;
    return ((br * ncb + bc) * 32 + (rr % 32)) * 16 + (rr / 32) * 4 + c4;
}

static inline size_t blocked_bytes(size_t rows, size_t cols)
{
    return ((rows + 127) / 128) * ((cols + 3) / 4) * 512;
}

/* Philox4x32-10 (Salmon et al., SC'11).  ctr = 128-bit counter, key = 64-bit key. */
static inline void philox4x32_10(uint32_t c[4], uint32_t k0, uint32_t k1)
{
    for (int r = 0; r < 10; r++) {
        uint64_t p0 = (uint64_t)0xD2511F53u * c[0];
        uint64_t p1 = (uint64_t)0xCD9E8D57u * c[2];
        uint32_t n0 = (uint32_t)(p1 >> 32) ^ c[1] ^ k0;
        uint32_t n1 = (uint32_t)p1;
        uint32_t n2 = (uint32_t)(p0 >> 32) ^ c[3] ^ k1;
        uint32_t n3 = (uint32_t)p0;
        c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
}

/* exported for the known-answer test */
void qco_philox4x32_10(const uint32_t ctr[4], const uint32_t key[2], uint32_t out[4])
{
    uint32_t c[4] = {ctr[0], ctr[1], ctr[2], ctr[3]};
    philox4x32_10(c, key[0], key[1]);
    memcpy(out, c, 16);
}

/*
 * 22-bit dither of element `flat` (row-major index in the whole tensor): Philox counter =
 * (flat >> 2) + offset, key = seed, word = output lane (flat & 3), dither = low 22 bits.  This is
 * the keying of experiments/prng_match/api.py:64-84 (counter = flat index >> 2, four consecutive
 * elements share one Philox call, low bits of the raw word are the dither).
 */
static inline uint32_t sr_dither22(uint64_t flat, uint64_t seed, uint64_t offset)
{
    uint64_t g = (flat >> 2) + offset;
    uint32_t c[4] = {(uint32_t)g, (uint32_t)(g >> 32), 0, 0};
    philox4x32_10(c, (uint32_t)seed, (uint32_t)(seed >> 32));
    return c[flat & 3] & 0x3FFFFFu;
}

/* exported element-wise helpers so the tests can pin the scalar conversions exhaustively */
void qco_f32_to_fp8(const float *in, int64_t n, int fmt, uint8_t *out)
{
    for (int64_t i = 0; i < n; i++) out[i] = f32_to_fp8_fmt(in[i], fmt);
}
void qco_f32_to_e2m1(const float *in, int64_t n, uint8_t *out)
{
    for (int64_t i = 0; i < n; i++) out[i] = f32_to_e2m1(in[i]);
}
void qco_e4m3_to_f32(const uint8_t *in, int64_t n, float *out)
{
    for (int64_t i = 0; i < n; i++) out[i] = e4m3_to_f32(in[i]);
}
void qco_amax_to_e8m0(const float *amax, int64_t n, int floor_mode, uint8_t *out)
{
    for (int64_t i = 0; i < n; i++)
        out[i] = floor_mode ? amax_to_e8m0_floor(amax[i]) : amax_to_e8m0_rceil(amax[i]);
}
void qco_e8m0_to_recip(const uint8_t *in, int64_t n, int floor_mode, float *out)
{
    for (int64_t i = 0; i < n; i++) out[i] = e8m0_to_recip(in[i], floor_mode);
}
/*
 * fp32 -> bf16 stochastic rounding (sr_bf16_f G:1841-1851, sr_bf16_global_f G:1887-1914, _sr_bf16_dither G:1828-1838):
 * out = bf16((bits(x) + rand16) & 0xFFFF0000).  rand16 of the element with flat index g in its parent tensor
 * (g = (global_row + i) * num_col + global_col + j) = 16-bit piece g & 7 of the 128 bits of Philox4x32-10 at counter
 * (g >> 3) + offset: piece k is half (k & 1), low half first, of word k >> 1 -- eight elements per Philox call (the
 * reference's own draw comes from a module that the installed PyTorch lacks, so the stream is this backend's).
 */
void qco_sr_f32_to_bf16(const uint32_t *xbits, int64_t M, int64_t N, uint64_t seed, uint64_t offset, int64_t global_row,
                        int64_t global_col, int64_t num_col, uint16_t *out)
{
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < M; i++)
        for (int64_t j = 0; j < N; j++) {
            uint64_t flat = (uint64_t)(global_row + i) * (uint64_t)num_col + (uint64_t)(global_col + j);
            uint64_t g = (flat >> 3) + offset;
            uint32_t c[4] = {(uint32_t)g, (uint32_t)(g >> 32), 0, 0};
            philox4x32_10(c, (uint32_t)seed, (uint32_t)(seed >> 32));
            uint32_t k = (uint32_t)(flat & 7), rand16 = (c[k >> 1] >> (16 * (k & 1))) & 0xFFFFu;
            out[i * N + j] = (uint16_t)((xbits[i * N + j] + rand16) >> 16);
        }
}

void qco_sr_dither22(int64_t first, int64_t n, uint64_t seed, uint64_t offset, uint32_t *out)
{
    for (int64_t i = 0; i < n; i++) out[i] = sr_dither22((uint64_t)(first + i), seed, offset);
}

/* (H, W) row-major 1-byte scales -> blocked layout, padding written as 0.  G:1000-1037. */
void qco_to_blocked(const uint8_t *scale, int64_t H, int64_t W, uint8_t *out)
{
    size_t ncb = (size_t)(W + 3) / 4;
    memset(out, 0, blocked_bytes((size_t)H, (size_t)W));
    for (int64_t r = 0; r < H; r++)
        for (int64_t c = 0; c < W; c++)
            out[blocked_offset((size_t)r, (size_t)c, ncb)] = scale[r * W + c];
}

/* ------------------------------------------------------------------------------------------ */
/* amax and the per-tensor scales                                                             */
/* ------------------------------------------------------------------------------------------ */

/* max |x| over n bf16 values, returned as the bf16 bit pattern of the maximum magnitude */
static uint16_t amax_bf16_bits(const uint16_t *x, int64_t n)
{
    uint16_t best = 0;
#pragma omp parallel for reduction(max : best) schedule(static)
    for (int64_t i = 0; i < n; i++) {
        uint16_t a = bf16_abs(x[i]);
        if (a > best) best = a;
    }
    return best;
}

/* |x| amax as fp32 (exact: a bf16 magnitude).  First half of G:1179-1183 and of G:1243-1246. */
void qco_amax_bf16(const uint16_t *x, int64_t n, float *out)
{
    *out = bf16_to_f32(amax_bf16_bits(x, n));
}

/* amax -> fp8 per-tensor scale: clamp to bf16(1e-12) IN BF16, widen, divide by the format max.
 * G:1179-1183 (float8_tensorwise_scale). */
void qco_fp8_scale_from_amax(float amax, int fmt, float *scale)
{
    const float tiny = u2f(0x2B8D0000u);                    /* bf16(1e-12) widened */
    float a = amax < tiny ? tiny : amax;
    *scale = div_by_const(a, fp8_max_fmt(fmt));
}

void qco_fp8_tensorwise_scale(const uint16_t *x, int64_t n, int fmt, float *scale)
{
    float amax;
    qco_amax_bf16(x, n, &amax);
    qco_fp8_scale_from_amax(amax, fmt, scale);
}

/* max |x| of every 128x128 block divided by `div` (2688: nvfp4_blocked_outer_scale G:1601-1606), (M/128, N/128) */
int qco_amax_block128x128(const uint16_t *x, int64_t M, int64_t N, float div, float *out)
{
    if (M % 128 || N % 128) return -1;
    int64_t nbc = N / 128;
#pragma omp parallel for schedule(static)
    for (int64_t bi = 0; bi < (M / 128) * nbc; bi++) {
        int64_t br = bi / nbc, bc = bi % nbc;
        uint16_t best = 0;
        for (int r = 0; r < 128; r++)
            for (int c = 0; c < 128; c++) {
                uint16_t a = bf16_abs(x[(br * 128 + r) * N + bc * 128 + c]);
                if (a > best) best = a;
            }
        out[bi] = div_by_const(bf16_to_f32(best), div);
    }
    return 0;
}

/* amax -> nvfp4 per-tensor outer scale = amax / (448 * 6), no clamp.  G:1243-1246. */
void qco_nvfp4_scale_from_amax(float amax, float *scale) { *scale = div_by_const(amax, 2688.0f); }

void qco_nvfp4_gs_scale(const uint16_t *x, int64_t n, float *scale)
{
    float amax;
    qco_amax_bf16(x, n, &amax);
    qco_nvfp4_scale_from_amax(amax, scale);
}

/* ------------------------------------------------------------------------------------------ */
/* fp8 casts                                                                                  */
/* ------------------------------------------------------------------------------------------ */

/* q = fp8(x_f32 * (1/scale)).  G:1186-1191 (float8_tensorwise_f). */
void qco_fp8_tensorwise_cast(const uint16_t *x, int64_t n, const float *scale, int fmt, uint8_t *q)
{
    float inv = 1.0f / *scale;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; i++) q[i] = f32_to_fp8_fmt(bf16_to_f32(x[i]) * inv, fmt);
}

/* one scale per row, amax over all columns.  G:301-307 (rowwise_fp8_f). */
void qco_fp8_rowwise(const uint16_t *x, int64_t M, int64_t N, int fmt, uint8_t *q, float *scale)
{
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < M; r++) {
        const uint16_t *xr = x + r * N;
        uint16_t best = 0;
        for (int64_t c = 0; c < N; c++) {
            uint16_t a = bf16_abs(xr[c]);
            if (a > best) best = a;
        }
        float s;
        qco_fp8_scale_from_amax(bf16_to_f32(best), fmt, &s);
        scale[r] = s;
        float inv = 1.0f / s;
        for (int64_t c = 0; c < N; c++) q[r * N + c] = f32_to_fp8_fmt(bf16_to_f32(xr[c]) * inv, fmt);
    }
}

/* per-row scale only.  G:389-393 (rowwise_precalc_scale). */
void qco_fp8_rowwise_scale(const uint16_t *x, int64_t M, int64_t N, int fmt, float *scale)
{
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < M; r++) {
        uint16_t best = 0;
        for (int64_t c = 0; c < N; c++) {
            uint16_t a = bf16_abs(x[r * N + c]);
            if (a > best) best = a;
        }
        qco_fp8_scale_from_amax(bf16_to_f32(best), fmt, &scale[r]);
    }
}

/* q = fp8(x_f32 / scale[row]) -- a true division, not a reciprocal multiply.  G:396-399. */
void qco_fp8_rowwise_precalc(const uint16_t *x, int64_t M, int64_t N, const float *scale, int fmt,
                             uint8_t *q)
{
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < M; r++)
        for (int64_t c = 0; c < N; c++)
            q[r * N + c] = f32_to_fp8_fmt(bf16_to_f32(x[r * N + c]) / scale[r], fmt);
}

/* one scale per column, outputs transposed: q (N, M), scale (N).  G:339-349 (colwise_fp8_f). */
void qco_fp8_colwise(const uint16_t *x, int64_t M, int64_t N, int fmt, uint8_t *q, float *scale)
{
    uint16_t *best = (uint16_t *)calloc((size_t)N, 2);
    for (int64_t r = 0; r < M; r++)
        for (int64_t c = 0; c < N; c++) {
            uint16_t a = bf16_abs(x[r * N + c]);
            if (a > best[c]) best[c] = a;
        }
#pragma omp parallel for schedule(static)
    for (int64_t c = 0; c < N; c++) {
        float s;
        qco_fp8_scale_from_amax(bf16_to_f32(best[c]), fmt, &s);
        scale[c] = s;
        float inv = 1.0f / s;
        for (int64_t r = 0; r < M; r++)
            q[c * M + r] = f32_to_fp8_fmt(bf16_to_f32(x[r * N + c]) * inv, fmt);
    }
    free(best);
}

/* per-column scale only, as a row of N values.  G:438-442 (colwise_precalc_scale). */
void qco_fp8_colwise_scale(const uint16_t *x, int64_t M, int64_t N, int fmt, float *scale)
{
    uint16_t *best = (uint16_t *)calloc((size_t)N, 2);
    for (int64_t r = 0; r < M; r++)
        for (int64_t c = 0; c < N; c++) {
            uint16_t a = bf16_abs(x[r * N + c]);
            if (a > best[c]) best[c] = a;
        }
    for (int64_t c = 0; c < N; c++) qco_fp8_scale_from_amax(bf16_to_f32(best[c]), fmt, &scale[c]);
    free(best);
}

/* q (N, M) = fp8(x_f32 / scale[col]) -- a true division, transposed output.  G:445-449. */
void qco_fp8_colwise_precalc(const uint16_t *x, int64_t M, int64_t N, const float *scale, int fmt,
                             uint8_t *q)
{
#pragma omp parallel for schedule(static)
    for (int64_t c = 0; c < N; c++)
        for (int64_t r = 0; r < M; r++)
            q[c * M + r] = f32_to_fp8_fmt(bf16_to_f32(x[r * N + c]) / scale[c], fmt);
}

/*
 * fp8 e4m3 with one fp32 scale per bm x bn block ("deepseek" recipes): scale = clamp(amax) / 448,
 * q = e4m3(x * (1 / scale)).
 *   bm = 1,   bn = 128: deepseek_1x128_f        G:103-110   q (M, N),  scale (M, N/128)
 *   bm = 128, bn = 128: deepseek_128x128_f      G:141-161   q (M, N),  scale (M/128, N/128)
 *   bm = 128, bn = 1, transposed != 0: deepseek_1x128_dim_m_f  G:194-214   q (N, M), scale (N, M/128)
 * deepseek_1x128_dim_km_f (G:251-277) is the first and the third on one fp32 view of x; there the
 * amax is clamped in fp32 (clamp_f32 != 0: 1e-12 as fp32), elsewhere in bf16 (bf16(1e-12)).
 */
int qco_fp8_blockwise(const uint16_t *x, int64_t M, int64_t N, int64_t bm, int64_t bn, int clamp_f32,
                      int transposed, uint8_t *q, float *scale)
{
    if (bm <= 0 || bn <= 0 || M % bm || N % bn) return -1;
    int64_t nbr = M / bm, nbc = N / bn;
    const float tiny = clamp_f32 ? 1e-12f : u2f(0x2B8D0000u);
#pragma omp parallel for schedule(static)
    for (int64_t bi = 0; bi < nbr * nbc; bi++) {
        int64_t br = bi / nbc, bc = bi % nbc;
        uint16_t best = 0;
        for (int64_t r = 0; r < bm; r++)
            for (int64_t c = 0; c < bn; c++) {
                uint16_t a = bf16_abs(x[(br * bm + r) * N + bc * bn + c]);
                if (a > best) best = a;
            }
        float amax = bf16_to_f32(best);
        float s = div_by_const(amax < tiny ? tiny : amax, 448.0f);
        float inv = 1.0f / s;
        scale[transposed ? bc * nbr + br : br * nbc + bc] = s;
        for (int64_t r = 0; r < bm; r++)
            for (int64_t c = 0; c < bn; c++) {
                int64_t R = br * bm + r, C = bc * bn + c;
                q[transposed ? C * M + R : R * N + C] = f32_to_fp8(bf16_to_f32(x[R * N + C]) * inv, 3, 7, 0x7E);
            }
    }
    return 0;
}

/* ------------------------------------------------------------------------------------------ */
/* mxfp8                                                                                      */
/* ------------------------------------------------------------------------------------------ */

/*
 * mxfp8 with 32-element blocks and e8m0 scales, element format e4m3.
 *   QC_ROWWISE: qk (M, N), sk (M, N/32)               G:561-568  (mxfp8_f)
 *   QC_COLWISE: qm (N, M), sm (N, M/32), transposed   G:656-671  (mxfp8_dim_m_f)
 *   both:                                             G:701-719  (mxfp8_dim_km_f)
 *   QC_SWIZZLE: each scale in the blocked layout      G:1051-1053, G:1092-1094, G:1134-1139
 *   QC_FLOOR:   FLOOR scale mode (extension)
 * Rowwise needs N % 32 == 0; colwise needs M % 32 == 0.  Unused outputs may be NULL.
 */
int qco_mxfp8(const uint16_t *x, int64_t M, int64_t N, int flags, uint8_t *qk, uint8_t *sk,
              uint8_t *qm, uint8_t *sm)
{
    int fl = (flags & QC_FLOOR) != 0, swz = (flags & QC_SWIZZLE) != 0;
    if ((flags & QC_ROWWISE) && N % 32) return -1;
    if ((flags & QC_COLWISE) && M % 32) return -1;
    if (flags & QC_ROWWISE) {
        int64_t nb = N / 32;
        size_t ncb = (size_t)(nb + 3) / 4;
        if (swz) memset(sk, 0, blocked_bytes((size_t)M, (size_t)nb));
#pragma omp parallel for schedule(static)
        for (int64_t r = 0; r < M; r++)
            for (int64_t b = 0; b < nb; b++) {
                const uint16_t *xb = x + r * N + b * 32;
                uint16_t best = 0;
                for (int i = 0; i < 32; i++) {
                    uint16_t a = bf16_abs(xb[i]);
                    if (a > best) best = a;
                }
                float amax = bf16_to_f32(best);
                uint8_t e = fl ? amax_to_e8m0_floor(amax) : amax_to_e8m0_rceil(amax);
                float rcp = e8m0_to_recip(e, fl);
                sk[swz ? blocked_offset((size_t)r, (size_t)b, ncb) : (size_t)(r * nb + b)] = e;
                for (int i = 0; i < 32; i++)
                    qk[r * N + b * 32 + i] = f32_to_fp8(bf16_to_f32(xb[i]) * rcp, 3, 7, 0x7E);
            }
    }
    if (flags & QC_COLWISE) {
        int64_t mb = M / 32;
        size_t ncb = (size_t)(mb + 3) / 4;
        if (swz) memset(sm, 0, blocked_bytes((size_t)N, (size_t)mb));
#pragma omp parallel for schedule(static)
        for (int64_t b = 0; b < mb; b++) {
            uint8_t tile[32];
            for (int64_t c = 0; c < N; c++) {
                uint16_t best = 0;
                for (int i = 0; i < 32; i++) {
                    uint16_t a = bf16_abs(x[(b * 32 + i) * N + c]);
                    if (a > best) best = a;
                }
                float amax = bf16_to_f32(best);
                uint8_t e = fl ? amax_to_e8m0_floor(amax) : amax_to_e8m0_rceil(amax);
                float rcp = e8m0_to_recip(e, fl);
                sm[swz ? blocked_offset((size_t)c, (size_t)b, ncb) : (size_t)(c * mb + b)] = e;
                for (int i = 0; i < 32; i++)
                    tile[i] = f32_to_fp8(bf16_to_f32(x[(b * 32 + i) * N + c]) * rcp, 3, 7, 0x7E);
                memcpy(qm + c * M + b * 32, tile, 32);
            }
        }
    }
    return 0;
}

/*
 * mxfp4 (mxfp4_f G:607-617): 1x32 blocks, RCEIL e8m0 scale with descale = amax * fp32(1/6) (G:504 with
 * max_pos = 6), elements e2m1 (GU:15-57) packed even -> low nibble (GU:87-92).  q (M, N/2), s (M, N/32)
 * plain or blocked.
 */
int qco_mxfp4(const uint16_t *x, int64_t M, int64_t N, int flags, uint8_t *q, uint8_t *s)
{
    if (N % 32) return -1;
    int swz = (flags & QC_SWIZZLE) != 0;
    int64_t nb = N / 32;
    size_t ncb = (size_t)(nb + 3) / 4;
    const float inv6 = u2f(0x3E2AAAABu);                    /* fp32(1.0 / 6.0) */
    if (swz) memset(s, 0, blocked_bytes((size_t)M, (size_t)nb));
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < M; r++)
        for (int64_t b = 0; b < nb; b++) {
            const uint16_t *xb = x + r * N + b * 32;
            uint16_t best = 0;
            for (int i = 0; i < 32; i++) {
                uint16_t a = bf16_abs(xb[i]);
                if (a > best) best = a;
            }
            uint32_t bits = f2u(bf16_to_f32(best) * inv6);
            uint8_t e;
            if ((bits & 0x7F800000u) == 0x7F800000u) e = 255;
            else {
                uint32_t ex = (bits >> 23) & 0xFF, m = bits & 0x7FFFFFu;
                e = (uint8_t)(ex + ((ex == 0) ? (m > 0x400000u) : (m != 0)));
            }
            float rcp = e8m0_to_recip(e, 0);
            s[swz ? blocked_offset((size_t)r, (size_t)b, ncb) : (size_t)(r * nb + b)] = e;
            for (int i = 0; i < 32; i += 2) {
                uint8_t lo = f32_to_e2m1(bf16_to_f32(xb[i]) * rcp), hi = f32_to_e2m1(bf16_to_f32(xb[i + 1]) * rcp);
                q[r * (N / 2) + b * 16 + i / 2] = (uint8_t)(lo | (hi << 4));
            }
        }
    return 0;
}

/*
 * mxfp8 with one RCEIL e8m0 scale per 32x32 block (mxfp8_32x32_f G:753-773): q (M, N) in the
 * layout of x, s the plain (M/32, N/32) grid.  The expanded / blocked / transposed forms of the
 * other 32x32 recipes (G:809-815, G:856-862, G:900-910, G:946-959) are index permutations of these
 * two outputs, done by the caller.
 */
int qco_mxfp8_32x32(const uint16_t *x, int64_t M, int64_t N, uint8_t *q, uint8_t *s)
{
    if (M % 32 || N % 32) return -1;
    int64_t mb = M / 32, nb = N / 32;
#pragma omp parallel for schedule(static)
    for (int64_t bi = 0; bi < mb * nb; bi++) {
        int64_t br = bi / nb, bc = bi % nb;
        uint16_t best = 0;
        for (int r = 0; r < 32; r++)
            for (int c = 0; c < 32; c++) {
                uint16_t a = bf16_abs(x[(br * 32 + r) * N + bc * 32 + c]);
                if (a > best) best = a;
            }
        uint8_t e = amax_to_e8m0_rceil(bf16_to_f32(best));
        float rcp = e8m0_to_recip(e, 0);
        s[bi] = e;
        for (int r = 0; r < 32; r++)
            for (int c = 0; c < 32; c++) {
                int64_t i = (br * 32 + r) * N + bc * 32 + c;
                q[i] = f32_to_fp8(bf16_to_f32(x[i]) * rcp, 3, 7, 0x7E);
            }
    }
    return 0;
}

/* ------------------------------------------------------------------------------------------ */
/* nvfp4                                                                                      */
/* ------------------------------------------------------------------------------------------ */

/* One 1x16 block given 16 fp32 values (already widened) and the outer scale.  Writes 8 packed
 * bytes and returns the e4m3 inner-scale byte.  G:1502-1515 (nvfp4_gs_f) with the pack order of
 * GU:87-92 (even index -> low nibble).  With sr != 0 the fp4 values are stochastically rounded as
 * at G:1392-1406: add a 22-bit dither to the fp32 bits, clear the low 22 bits, then encode. */
static inline uint8_t nvfp4_block(const float v[16], float amax, float outer, uint8_t out[8],
                                  int sr, uint64_t flat0, int64_t flat_stride, uint64_t seed,
                                  uint64_t offset)
{
    float inner_f = div_by_const(amax, 6.0f) / outer;
    if (inner_f < 0.015625f) inner_f = 0.015625f;
    if (inner_f > 448.0f) inner_f = 448.0f;
    uint8_t inner = f32_to_fp8(inner_f, 3, 7, 0x7E);
    float recip = (1.0f / outer) / e4m3_to_f32(inner);
    uint8_t code[16];
    for (int i = 0; i < 16; i++) {
        float d = v[i] * recip;
        if (d < -6.0f) d = -6.0f;
        if (d > 6.0f) d = 6.0f;
        if (sr) {
            uint32_t dither = sr_dither22(flat0 + (uint64_t)(i * flat_stride), seed, offset);
            d = u2f((f2u(d) + dither) & 0xFFC00000u);
        }
        code[i] = f32_to_e2m1(d);
    }
    for (int i = 0; i < 8; i++) out[i] = (uint8_t)(code[2 * i] | (code[2 * i + 1] << 4));
    return inner;
}

/*
 * nvfp4 along the last dim: q (M, N/2) packed, inner scale (M, N/16) e4m3, row-major or blocked.
 * outer: one fp32 (outer_per_row == 0) or one per row (outer_per_row != 0).
 * G:1494-1517 (nvfp4_gs_f), G:1249-1266 (nvfp4_gs_swizzle_f), G:1409-1426 (..._sr_f).
 * The stochastic-rounding stream is indexed by the row-major position of the element in x.
 */
int qco_nvfp4(const uint16_t *x, int64_t M, int64_t N, const float *outer, int outer_per_row,
              int flags, uint64_t seed, uint64_t offset, uint8_t *q, uint8_t *s)
{
    if (N % 16) return -1;
    if (outer_per_row == 2 && (M % 128 || N % 128)) return -1;
    int swz = (flags & QC_SWIZZLE) != 0, sr = (flags & QC_SR) != 0;
    int64_t nb = N / 16;
    size_t ncb = (size_t)(nb + 3) / 4;
    if (swz) memset(s, 0, blocked_bytes((size_t)M, (size_t)nb));
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < M; r++) {
        float o = outer_per_row == 1 ? outer[r] : outer[0];
        for (int64_t b = 0; b < nb; b++) {
            /* outer_per_row == 2: one outer scale per 128x128 block, nvfp4_blocked_outer_f G:1609-1634 */
            if (outer_per_row == 2) o = outer[(r / 128) * (N / 128) + b / 8];
            const uint16_t *xb = x + r * N + b * 16;
            float v[16];
            uint16_t best = 0;
            for (int i = 0; i < 16; i++) {
                uint16_t a = bf16_abs(xb[i]);
                if (a > best) best = a;
                v[i] = bf16_to_f32(xb[i]);
            }
            uint8_t inner = nvfp4_block(v, bf16_to_f32(best), o, q + r * (N / 2) + b * 8, sr,
                                        (uint64_t)(r * N + b * 16), 1, seed, offset);
            s[swz ? blocked_offset((size_t)r, (size_t)b, ncb) : (size_t)(r * nb + b)] = inner;
        }
    }
    return 0;
}

/*
 * Transposed nvfp4: the result of the cast above applied to x.t().contiguous() (the call made at
 * test/test_quant_cast_gold.py:104), computed without materialising the transpose:
 * q (N, M/2), inner scale over the (N, M/16) frame.  16x1 blocks run down the rows of x.
 * The stochastic-rounding stream is indexed by the row-major position in the TRANSPOSED frame.
 */
int qco_nvfp4_t(const uint16_t *x, int64_t M, int64_t N, const float *outer, int flags,
                uint64_t seed, uint64_t offset, uint8_t *q, uint8_t *s)
{
    if (M % 16) return -1;
    int swz = (flags & QC_SWIZZLE) != 0, sr = (flags & QC_SR) != 0;
    int64_t mb = M / 16;
    size_t ncb = (size_t)(mb + 3) / 4;
    if (swz) memset(s, 0, blocked_bytes((size_t)N, (size_t)mb));
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < mb; b++)
        for (int64_t c = 0; c < N; c++) {
            float v[16];
            uint16_t best = 0;
            for (int i = 0; i < 16; i++) {
                uint16_t h = x[(b * 16 + i) * N + c];
                uint16_t a = bf16_abs(h);
                if (a > best) best = a;
                v[i] = bf16_to_f32(h);
            }
            uint8_t inner = nvfp4_block(v, bf16_to_f32(best), outer[0], q + c * (M / 2) + b * 8, sr,
                                        (uint64_t)(c * M + b * 16), 1, seed, offset);
            s[swz ? blocked_offset((size_t)c, (size_t)b, ncb) : (size_t)(c * mb + b)] = inner;
        }
    return 0;
}

/*
 * 16x16 randomised Hadamard transform along the last dim (hadamard_rht_f G:1784-1789 with
 * rht = diag(sign) @ H / 4, hadamard_rht_matrix G:1778-1781; H the Sylvester-Walsh matrix
 * H[i][j] = (-1)^popcount(i & j), G:1753-1775):
 *     y[16 b + j] = bf16( sum_i x[16 b + i] * sign[i] * H[i][j] / 4 ),   fp32 accumulation.
 * The reference evaluates this as a bf16 matmul, whose fp32 accumulation order belongs to the GEMM
 * library that runs it.  This restatement fixes the order: the four-stage in-place butterfly
 * (strides 1, 2, 4, 8; (a, b) -> (a + b, a - b)), then the exact scaling by 1/4 and ONE rounding to
 * bf16 (nearest even).  Whenever the 16-term sums are exact in fp32 -- inputs of one block within a
 * 2^12 magnitude range, in practice all activations -- every order gives the same bits; the golden
 * vectors from the reference's CPU run confirm it for those inputs.
 * sign_mask: bit i set -> sign[i] = -1.
 */
static inline uint16_t f32_to_bf16_rne(float f)
{
    uint32_t u = f2u(f);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x40u);
    return (uint16_t)((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
}

static void rht16(const uint16_t *x, int64_t stride, uint32_t sign_mask, uint16_t *y)
{
    float t[16];
    for (int i = 0; i < 16; i++) t[i] = bf16_to_f32((uint16_t)(x[i * stride] ^ (((sign_mask >> i) & 1u) << 15)));
    for (int s = 1; s < 16; s <<= 1)
        for (int i = 0; i < 16; i++)
            if (!(i & s)) {
                float a = t[i], b = t[i | s];
                t[i] = a + b;
                t[i | s] = a - b;
            }
    for (int j = 0; j < 16; j++) y[j] = f32_to_bf16_rne(t[j] * 0.25f);
}

int qco_hadamard_rht(const uint16_t *x, int64_t rows, int64_t cols, uint32_t sign_mask, uint16_t *y)
{
    if (cols % 16) return -1;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; r++)
        for (int64_t b = 0; b < cols / 16; b++) rht16(x + r * cols + b * 16, 1, sign_mask, y + r * cols + b * 16);
    return 0;
}

/* y (N, M) = RHT along M of x.t(): the tensor the dim-m half of G:1324-1333 quantises, without the
 * transposed copy of x. */
int qco_hadamard_rht_t(const uint16_t *x, int64_t M, int64_t N, uint32_t sign_mask, uint16_t *y)
{
    if (M % 16) return -1;
#pragma omp parallel for schedule(static)
    for (int64_t c = 0; c < N; c++)
        for (int64_t b = 0; b < M / 16; b++) rht16(x + (b * 16) * N + c, N, sign_mask, y + c * M + b * 16);
    return 0;
}

/* torchrun exports OMP_NUM_THREADS=1; the CPU baseline asks for all host threads explicitly */
void qco_set_num_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int qco_num_threads(void)
{
    int n = 1;
#ifdef _OPENMP
#pragma omp parallel
    {
#pragma omp single
        n = omp_get_num_threads();
    }
#endif
    return n;
}
