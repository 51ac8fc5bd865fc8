// fp8 casts and the tensor-wide amax, sm_100a.
//
// All kernels here are HBM-bound streams: 128-bit coalesced loads, packed cvt.rn.satfinite stores,
// grids sized from the SM count.  Numerics follow G = quant_cast_bench/quant_cast_gold/recipes.py of
// vkuzo/quant_cast_bench: float8_tensorwise_scale G:1179-1183, float8_tensorwise_f G:1186-1191,
// rowwise_fp8_f G:301-307, rowwise_precalc_f G:396-399, nvfp4_gs_scale G:1243-1246.
#include "common.cuh"
#include "host_util.h"
#include "xchg.cuh"

#ifndef QCC_AMAX_LD
#define QCC_AMAX_LD ld_nc_v4
#endif

namespace qcc {

// ---------------------------------------------------------------------------------------------
// amax: per-CTA partial maxima, then a one-CTA finish
// ---------------------------------------------------------------------------------------------
constexpr int AMAX_THREADS = 256;

__device__ __forceinline__ uint32_t warp_max_u32(uint32_t v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = max(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    return v;
}

#ifndef QCC_AMAX_U
#define QCC_AMAX_U 8
#endif
#ifndef QCC_AMAX_CTAS
#define QCC_AMAX_CTAS 6
#endif
constexpr int AMAX_U = QCC_AMAX_U;            // 16-byte loads in flight per thread
constexpr int AMAX_CTAS_PER_SM = QCC_AMAX_CTAS;

// partial[blockIdx.x] = max |x| over this CTA's grid-stride share, as fp32 bits
__global__ void __launch_bounds__(AMAX_THREADS, AMAX_CTAS_PER_SM) amax_partial_kernel(const uint16_t *__restrict__ x, int64_t n,
                                                                                   uint32_t *__restrict__ partial)
{
    const int64_t nvec = n >> 3;  // 16-byte chunks
    const uint4 *xv = reinterpret_cast<const uint4 *>(x);
    uint32_t acc0 = 0, acc1 = 0, acc2 = 0, acc3 = 0;
    const int64_t stride = (int64_t)gridDim.x * AMAX_THREADS;
    int64_t i = (int64_t)blockIdx.x * AMAX_THREADS + threadIdx.x;
    for (; i + (AMAX_U - 1) * stride < nvec; i += AMAX_U * stride) {
        uint4 v[AMAX_U];
#pragma unroll
        for (int u = 0; u < AMAX_U; u++) v[u] = QCC_AMAX_LD(xv + i + u * stride);
#pragma unroll
        for (int u = 0; u < AMAX_U; u += 2) {
            acc0 = absmax2_acc(absmax2_acc(acc0, v[u].x), v[u].y); acc1 = absmax2_acc(absmax2_acc(acc1, v[u].z), v[u].w);
            acc2 = absmax2_acc(absmax2_acc(acc2, v[u + 1].x), v[u + 1].y); acc3 = absmax2_acc(absmax2_acc(acc3, v[u + 1].z), v[u + 1].w);
        }
    }
    for (; i < nvec; i += stride) {
        uint4 a = QCC_AMAX_LD(xv + i);
        acc0 = absmax2_acc(absmax2_acc(acc0, a.x), a.y); acc1 = absmax2_acc(absmax2_acc(acc1, a.z), a.w);
    }
    uint32_t acc = absmax2(absmax2(acc0, acc1), absmax2(acc2, acc3));
    uint32_t m = f2u(hmax_halves_f32(acc));
    // scalar tail (n % 8 elements), handled by the first thread of the grid
    if (blockIdx.x == 0 && threadIdx.x == 0)
        for (int64_t t = nvec << 3; t < n; t++) m = max(m, ((uint32_t)x[t] & 0x7FFFu) << 16);
    m = warp_max_u32(m);
    __shared__ uint32_t s[AMAX_THREADS / 32];
    if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x < 32) {
        m = threadIdx.x < AMAX_THREADS / 32 ? s[threadIdx.x] : 0u;
        m = warp_max_u32(m);
        if (threadIdx.x == 0) partial[blockIdx.x] = m;
    }
}

// Built-in scratch of qcc_amax_bf16_noalloc: the per-CTA partial maxima of one call.  It lives in
// the library image, so every GPU that loads the library keeps these 8 KB until the process exits.
static __device__ __align__(256) uint32_t g_amax_noalloc_scratch[AMAX_MAX_CTAS];

// mode: QCC_AMAX_*, with QCC_RECIP_DIV or-ed in when given
__device__ __forceinline__ float amax_finish(float amax, int mode, int fmt)
{
    const bool recip = mode & QCC_RECIP_DIV;
    mode &= ~QCC_RECIP_DIV;
    if (mode == QCC_AMAX_FP8_SCALE)
        return fmt == QCC_FMT_E5M2 ? fp8_scale_from_amax<QCC_FMT_E5M2>(amax, recip) : fp8_scale_from_amax<QCC_FMT_E4M3>(amax, recip);
    if (mode == QCC_AMAX_NVFP4_SCALE) return div_by_const(amax, 2688.0f, recip);
    return amax;
}

__global__ void __launch_bounds__(AMAX_THREADS) amax_finish_kernel(const uint32_t *__restrict__ partial, int count,
                                                                  int mode, int fmt, float *__restrict__ out)
{
    uint32_t m = 0;
    for (int i = threadIdx.x; i < count; i += AMAX_THREADS) m = max(m, partial[i]);
    m = warp_max_u32(m);
    __shared__ uint32_t s[AMAX_THREADS / 32];
    if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x < 32) {
        m = threadIdx.x < AMAX_THREADS / 32 ? s[threadIdx.x] : 0u;
        m = warp_max_u32(m);
        if (threadIdx.x == 0) out[0] = amax_finish(u2f(m), mode, fmt);
    }
}

__global__ void scale_from_amax_kernel(const float *__restrict__ amax, int mode, int fmt, float *__restrict__ out)
{
    out[0] = amax_finish(amax[0], mode, fmt);
}

// One launch.  A one-shot grid: every CTA reduces its own AMAX1_U x 4 KB piece of x and merges the result into one
// word (atomic max on the bits of a non-negative float, skipped when the word already holds as much).
// XCHG false: the CTAs also take a ticket and the one that draws the last ticket writes out[0] and leaves the two
// control words (ctl[0] = ticket, ctl[1] = running maximum) zero for the next call.
// XCHG true: the word is the accumulator of this rank's amax exchange (ctl = the exchange state); the first
// consumer publishes it, so the CTAs wait for nothing.
#ifndef QCC_AMAX1_U
#define QCC_AMAX1_U 8
#endif
constexpr int AMAX1_U = QCC_AMAX1_U;

template <bool XCHG>
__global__ void __launch_bounds__(AMAX_THREADS) amax_oneshot_kernel(const uint16_t *__restrict__ x, int64_t n,
                                                                   uint32_t *__restrict__ ctl, int mode, int fmt,
                                                                   float *__restrict__ out)
{
    uint32_t seen = 0;
    if (XCHG) {
        pdl_trigger();
        seen = xchg_producer_begin(ctl);
    }
    const int64_t nvec = n >> 3;
    const uint4 *xv = reinterpret_cast<const uint4 *>(x);
    const int64_t base = (int64_t)blockIdx.x * (AMAX_THREADS * AMAX1_U) + threadIdx.x;
    uint4 v[AMAX1_U];
#pragma unroll
    for (int u = 0; u < AMAX1_U; u++) {
        const int64_t i = base + (int64_t)u * AMAX_THREADS;
        v[u] = i < nvec ? QCC_AMAX_LD(xv + i) : make_uint4(0, 0, 0, 0);
    }
    uint32_t acc0 = 0, acc1 = 0;
#pragma unroll
    for (int u = 0; u < AMAX1_U; u++) {
        acc0 = absmax2_acc(absmax2_acc(acc0, v[u].x), v[u].y);
        acc1 = absmax2_acc(absmax2_acc(acc1, v[u].z), v[u].w);
    }
    uint32_t m = f2u(hmax_halves_f32(absmax2(acc0, acc1)));
    if (blockIdx.x == 0 && threadIdx.x == 0)
        for (int64_t t = nvec << 3; t < n; t++) m = max(m, ((uint32_t)x[t] & 0x7FFFu) << 16);
    __shared__ uint32_t s[AMAX_THREADS / 32];
    if (XCHG) {
        xchg_producer_merge(ctl, m, seen, s);
        return;
    }
    if (!cta_max_ticket(m, ctl, s)) return;
    if (threadIdx.x == 0 && out) out[0] = amax_finish(u2f(m), mode, fmt);
}

// ---------------------------------------------------------------------------------------------
// tensorwise cast: 16 elements per thread per step (two 16-byte loads, one 16-byte store)
// ---------------------------------------------------------------------------------------------
template <int FMT>
__device__ __forceinline__ uint4 cast16(uint4 a, uint4 b, float inv)
{
    uint4 o;
    o.x = cvt_fp8x4<FMT>(bf16lo(a.x) * inv, bf16hi(a.x) * inv, bf16lo(a.y) * inv, bf16hi(a.y) * inv);
    o.y = cvt_fp8x4<FMT>(bf16lo(a.z) * inv, bf16hi(a.z) * inv, bf16lo(a.w) * inv, bf16hi(a.w) * inv);
    o.z = cvt_fp8x4<FMT>(bf16lo(b.x) * inv, bf16hi(b.x) * inv, bf16lo(b.y) * inv, bf16hi(b.y) * inv);
    o.w = cvt_fp8x4<FMT>(bf16lo(b.z) * inv, bf16hi(b.z) * inv, bf16lo(b.w) * inv, bf16hi(b.w) * inv);
    return o;
}
template <int FMT>
__device__ __forceinline__ uint2 cast8(uint4 a, float inv)
{
    uint2 o;
    o.x = cvt_fp8x4<FMT>(bf16lo(a.x) * inv, bf16hi(a.x) * inv, bf16lo(a.y) * inv, bf16hi(a.y) * inv);
    o.y = cvt_fp8x4<FMT>(bf16lo(a.z) * inv, bf16hi(a.z) * inv, bf16lo(a.w) * inv, bf16hi(a.w) * inv);
    return o;
}

#ifndef QCC_TW_THREADS
#define QCC_TW_THREADS 256
#endif
#ifndef QCC_TW_UNROLL
#define QCC_TW_UNROLL 1
#endif
constexpr int TW_THREADS = QCC_TW_THREADS;
constexpr int TW_UNROLL = QCC_TW_UNROLL;  // 16-element groups per thread (1 measured best: 7.0 TB/s)

// SRC: where the scale comes from.  QCC_SRC_SCALE: scale[0] is the scale; QCC_SRC_AMAX: scale[0] is a raw amax, the
// kernel forms max(amax, bf16(1e-12)) / fp8_max itself and its first CTA writes the scale to scale_out.
template <int FMT, int SRC>
__global__ void __launch_bounds__(TW_THREADS) fp8_tensorwise_kernel(const uint16_t *__restrict__ x, int64_t n,
                                                                   const float *__restrict__ scale,
                                                                   float *__restrict__ scale_out, uint8_t *__restrict__ q, int recip_div)
{
    const int64_t ngrp = n >> 4;  // groups of 16 elements
    const uint4 *xv = reinterpret_cast<const uint4 *>(x);
    uint4 *qv = reinterpret_cast<uint4 *>(q);
    const int64_t base = (int64_t)blockIdx.x * (TW_THREADS * TW_UNROLL) + threadIdx.x;
    uint4 a[TW_UNROLL], b[TW_UNROLL];
#pragma unroll
    for (int u = 0; u < TW_UNROLL; u++) {
        int64_t g = base + (int64_t)u * TW_THREADS;
        if (g < ngrp) { a[u] = ld_nc_v4(xv + 2 * g); b[u] = ld_nc_v4(xv + 2 * g + 1); }
    }
    float sc = __ldg(scale);
    if (SRC == QCC_SRC_AMAX) {
        sc = fp8_scale_from_amax<FMT>(sc, recip_div != 0);
        if (blockIdx.x == 0 && threadIdx.x == 0 && scale_out) scale_out[0] = sc;
    }
    const float inv = __fdiv_rn(1.0f, sc);
#pragma unroll
    for (int u = 0; u < TW_UNROLL; u++) {
        int64_t g = base + (int64_t)u * TW_THREADS;
        if (g < ngrp) st_out(qv + g, cast16<FMT>(a[u], b[u], inv));
    }
    // scalar tail: the last n % 16 elements
    if (blockIdx.x == 0 && threadIdx.x < (n & 15)) {
        int64_t t = (ngrp << 4) + threadIdx.x;
        q[t] = (uint8_t)cvt_fp8x2<FMT>(u2f((uint32_t)x[t] << 16) * inv, 0.0f);
    }
}

// A plain copy with the access pattern of the streaming casts (one-shot grid, two 16-byte loads in flight per thread,
// evict-first stores): the yardstick the benchmarks hold the casts against at each size.
__global__ void __launch_bounds__(TW_THREADS) stream_copy_kernel(const uint4 *__restrict__ src, uint4 *__restrict__ dst, int64_t nvec)
{
    const int64_t i = (int64_t)blockIdx.x * (TW_THREADS * 2) + threadIdx.x;
    uint4 a = make_uint4(0, 0, 0, 0), b = a;
    if (i < nvec) a = ld_nc_v4(src + i);
    if (i + TW_THREADS < nvec) b = ld_nc_v4(src + i + TW_THREADS);
    if (i < nvec) st_out(dst + i, a);
    if (i + TW_THREADS < nvec) st_out(dst + i + TW_THREADS, b);
}

// The same yardstick for casts that write fewer bytes than they read: every 16-byte piece of dst is the XOR of R
// consecutive 16-byte pieces of src -- the loads and stores of a 2-byte -> 1-byte cast (R = 2: a thread reads 32 contiguous
// bytes, as the tensorwise cast does) or of a 2-byte -> half-byte cast (R = 4: 64 contiguous bytes, as the nvfp4 stream
// does), without their arithmetic.
template <int R, int U>
__global__ void __launch_bounds__(TW_THREADS) stream_fold_kernel(const uint4 *__restrict__ src, uint4 *__restrict__ dst, int64_t nout)
{
    const int64_t base = (int64_t)blockIdx.x * (TW_THREADS * U) + threadIdx.x;
    uint4 v[U][R];
#pragma unroll
    for (int u = 0; u < U; u++) {
        const int64_t o = base + (int64_t)u * TW_THREADS;
#pragma unroll
        for (int r = 0; r < R; r++) v[u][r] = o < nout ? ld_v4(src + o * R + r) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < U; u++) {
        const int64_t o = base + (int64_t)u * TW_THREADS;
        uint4 a = v[u][0];
#pragma unroll
        for (int r = 1; r < R; r++) { a.x ^= v[u][r].x; a.y ^= v[u][r].y; a.z ^= v[u][r].z; a.w ^= v[u][r].w; }
        if (o < nout) st_out(dst + o, a);
    }
}

// ---------------------------------------------------------------------------------------------
// rowwise cast: TPR threads share a row and keep it in registers (CH 16-byte chunks each), so x is
// read from HBM exactly once.  PRECALC: per-row scale supplied, true division.
// ---------------------------------------------------------------------------------------------
constexpr int RW_THREADS = 256;

template <int FMT, int TPR, int CH, bool PRECALC>
__global__ void __launch_bounds__(RW_THREADS, (TPR == 256 && CH == 8) ? 5 : 1) fp8_rowwise_kernel(const uint16_t *__restrict__ x, int64_t M, int64_t N,
                                                                const float *__restrict__ scale_in,
                                                                uint8_t *__restrict__ q, float *__restrict__ scale_out, int recip_div)
{
    constexpr int ROWS = RW_THREADS / TPR;
    const int tr = threadIdx.x % TPR;
    const int lr = threadIdx.x / TPR;
    const int64_t row = (int64_t)blockIdx.x * ROWS + lr;
    const bool row_ok = row < M;
    const int64_t nchunk = N >> 3;
    const uint4 *xr = reinterpret_cast<const uint4 *>(x + (row_ok ? row : 0) * N);
    uint4 v[CH];
#pragma unroll
    for (int c = 0; c < CH; c++) {
        int64_t k = tr + (int64_t)c * TPR;
        v[c] = (row_ok && k < nchunk) ? ld_nc_v4(xr + k) : make_uint4(0, 0, 0, 0);
    }
    float s;
    if (PRECALC) {
        s = row_ok ? __ldg(scale_in + row) : 1.0f;
    } else {
        uint32_t acc = 0;
#pragma unroll
        for (int c = 0; c < CH; c++) acc = absmax2(absmax2(absmax2(absmax2(acc, v[c].x), v[c].y), v[c].z), v[c].w);
        uint32_t m = f2u(hmax_halves_f32(acc));
        constexpr int W = TPR < 32 ? TPR : 32;
#pragma unroll
        for (int o = W / 2; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
        if (TPR > 32) {
            __shared__ uint32_t sm[RW_THREADS / 32];
            if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = m;
            __syncthreads();
            constexpr int WPR = TPR / 32 > 0 ? TPR / 32 : 1;
            m = 0;
#pragma unroll
            for (int w = 0; w < WPR; w++) m = max(m, sm[lr * WPR + w]);
        }
        s = fp8_scale_from_amax<FMT>(u2f(m), recip_div != 0);
        if (row_ok && tr == 0) scale_out[row] = s;
    }
    if (q == nullptr || !row_ok) return;
    uint2 *qr = reinterpret_cast<uint2 *>(q + row * N);
    if (PRECALC) {
#pragma unroll
        for (int c = 0; c < CH; c++) {
            int64_t k = tr + (int64_t)c * TPR;
            if (k < nchunk) {
                uint4 a = v[c];
                uint2 o;
                o.x = cvt_fp8x4<FMT>(__fdiv_rn(bf16lo(a.x), s), __fdiv_rn(bf16hi(a.x), s), __fdiv_rn(bf16lo(a.y), s),
                                     __fdiv_rn(bf16hi(a.y), s));
                o.y = cvt_fp8x4<FMT>(__fdiv_rn(bf16lo(a.z), s), __fdiv_rn(bf16hi(a.z), s), __fdiv_rn(bf16lo(a.w), s),
                                     __fdiv_rn(bf16hi(a.w), s));
                st_out(qr + k, o);
            }
        }
    } else {
        const float inv = __fdiv_rn(1.0f, s);
#pragma unroll
        for (int c = 0; c < CH; c++) {
            int64_t k = tr + (int64_t)c * TPR;
            if (k < nchunk) st_out(qr + k, cast8<FMT>(v[c], inv));
        }
    }
}

// Any N (also N % 8 != 0 or rows longer than the register-resident variants): one CTA per row, two
// passes over the row (the second pass is served by L2).
template <int FMT, bool PRECALC>
__global__ void __launch_bounds__(RW_THREADS) fp8_rowwise_generic_kernel(const uint16_t *__restrict__ x, int64_t M,
                                                                        int64_t N, const float *__restrict__ scale_in,
                                                                        uint8_t *__restrict__ q,
                                                                        float *__restrict__ scale_out, int recip_div)
{
    const int64_t row = blockIdx.x;
    const uint16_t *xr = x + row * N;
    float s;
    __shared__ uint32_t sm[RW_THREADS / 32];
    if (PRECALC) {
        s = __ldg(scale_in + row);
    } else {
        uint32_t m = 0;
        for (int64_t c = threadIdx.x; c < N; c += RW_THREADS) m = max(m, ((uint32_t)xr[c] & 0x7FFFu) << 16);
        m = warp_max_u32(m);
        if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = m;
        __syncthreads();
        m = 0;
#pragma unroll
        for (int w = 0; w < RW_THREADS / 32; w++) m = max(m, sm[w]);
        s = fp8_scale_from_amax<FMT>(u2f(m), recip_div != 0);
        if (threadIdx.x == 0) scale_out[row] = s;
    }
    if (q == nullptr) return;
    const float inv = __fdiv_rn(1.0f, s);
    for (int64_t c = threadIdx.x; c < N; c += RW_THREADS) {
        float f = u2f((uint32_t)xr[c] << 16);
        float d = PRECALC ? __fdiv_rn(f, s) : f * inv;
        q[row * N + c] = (uint8_t)cvt_fp8x2<FMT>(d, 0.0f);
    }
}

template <int FMT, bool PRECALC>
static int launch_rowwise(const void *x, int64_t M, int64_t N, const float *scale_in, void *q, float *scale_out,
                          int recip_div, cudaStream_t st)
{
    const uint16_t *xp = (const uint16_t *)x;
    uint8_t *qp = (uint8_t *)q;
#define QCC_RW(TPR, CH)                                                                                      \
    do {                                                                                                     \
        constexpr int ROWS = RW_THREADS / (TPR);                                                             \
        unsigned grid = (unsigned)((M + ROWS - 1) / ROWS);                                                   \
        fp8_rowwise_kernel<FMT, TPR, CH, PRECALC><<<grid, RW_THREADS, 0, st>>>(xp, M, N, scale_in, qp, scale_out, recip_div); \
        return (int)cudaGetLastError();                                                                      \
    } while (0)
    if (N % 8 == 0 && N <= 16384 && M <= 0x7FFFFFFF) {
        const int64_t chunks = N / 8;
        if (chunks <= 32) QCC_RW(32, 1);
        if (chunks <= 64) QCC_RW(32, 2);
        if (chunks <= 128) QCC_RW(32, 4);
        if (chunks <= 256) QCC_RW(64, 4);
        if (chunks <= 512) QCC_RW(128, 4);
        if (chunks <= 1024) QCC_RW(256, 4);
        QCC_RW(256, 8);
    }
#undef QCC_RW
    if (M > 0x7FFFFFFF) return QCC_ERR_SHAPE;
    fp8_rowwise_generic_kernel<FMT, PRECALC><<<(unsigned)M, RW_THREADS, 0, st>>>(xp, M, N, scale_in, qp, scale_out, recip_div);
    return (int)cudaGetLastError();
}


// ---------------------------------------------------------------------------------------------
// colwise cast: one scale per column, transposed outputs q (N, M), scale (N, 1).
// colwise_fp8_f G:339-349, colwise_precalc_f G:445-449.  The kernels here are the two-launch form: column maxima into
// a caller-supplied scratch of N words (atomic max on the bit patterns: exact and order independent), then a tile
// kernel that casts and transposes.  It serves the cast with given scales and matrices too tall for the one-launch
// form of colwise.cu, which is tried first.
// ---------------------------------------------------------------------------------------------
// rows per CTA of the column-maximum pass: 256 measured best at 16384^2 (211 us for both passes against 231 us
// with 64, 128 or 512 rows)
constexpr int CW_AMAX_ROWS = 256;
constexpr int CW_AMAX_THREADS = 256;

__global__ void __launch_bounds__(CW_AMAX_THREADS) fp8_colwise_amax_kernel(const uint16_t *__restrict__ x, int M, int N,
                                                              uint32_t *__restrict__ amax_bits)
{
    const int chunk = blockIdx.x * CW_AMAX_THREADS + threadIdx.x;       // 8 adjacent columns
    if (chunk * 8 >= N) return;
    const int r0 = blockIdx.y * CW_AMAX_ROWS;
    const int r1 = min(M, r0 + CW_AMAX_ROWS);
    const uint4 *p = reinterpret_cast<const uint4 *>(x + (size_t)r0 * N) + chunk;
    const size_t stride = (size_t)N >> 3;
    uint32_t a0 = 0, a1 = 0, a2 = 0, a3 = 0;
    int r = r0;
    for (; r + 8 <= r1; r += 8) {
        uint4 v[8];
#pragma unroll
        for (int u = 0; u < 8; u++) v[u] = ld_nc_v4(p + (size_t)(r - r0 + u) * stride);
#pragma unroll
        for (int u = 0; u < 8; u++) {
            a0 = absmax2_acc(a0, v[u].x); a1 = absmax2_acc(a1, v[u].y);
            a2 = absmax2_acc(a2, v[u].z); a3 = absmax2_acc(a3, v[u].w);
        }
    }
    for (; r < r1; r++) {
        const uint4 v = ld_nc_v4(p + (size_t)(r - r0) * stride);
        a0 = absmax2_acc(a0, v.x); a1 = absmax2_acc(a1, v.y); a2 = absmax2_acc(a2, v.z); a3 = absmax2_acc(a3, v.w);
    }
    uint32_t *dst = amax_bits + chunk * 8;
    const uint32_t acc[4] = {a0, a1, a2, a3};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        atomicMax(dst + 2 * i, acc[i] << 16);
        atomicMax(dst + 2 * i + 1, acc[i] & 0xFFFF0000u);
    }
}

// scale[c] = max(amax_c, bf16(1e-12)) / fp8_max from the finished column maxima
template <int FMT>
__global__ void colwise_scale_kernel(const uint32_t *__restrict__ amax_bits, float *__restrict__ scale, int N, int recip_div)
{
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c < N) scale[c] = fp8_scale_from_amax<FMT>(u2f(amax_bits[c]), recip_div != 0);
}

constexpr int CW_PANEL = 64 * 128;                // one 64-column panel of a 64-row tile
constexpr int CW_Q_OFF = 2 * CW_PANEL;            // staging: 4 sub-tiles x 32 rows x 64 B
constexpr int CW_BAR_OFF = CW_Q_OFF + 4 * 32 * 64;
constexpr int CW_ALLOC = CW_BAR_OFF + 32 + 1024;     // four barriers

// One 64-row x 128-column tile by one CTA of two warps; warp b owns the 32-row slab b, lane = four adjacent columns.
// PRECALC: per-column scale given, true division (G:448); otherwise scale = f(column amax), multiply by 1/scale.
// The caller has issued the two TMA loads of the tile on `bar`; `parity` is the phase to wait for.
template <int FMT, bool PRECALC>
__device__ __forceinline__ void colwise_cast_tile(uint32_t base, uint64_t *bar, uint32_t parity, const uint32_t *amax_bits,
                                                  const float *__restrict__ scale_in, uint8_t *__restrict__ q,
                                                  float *__restrict__ scale_out, int M, int N, int tile_m, int tile_n,
                                                  bool recip_div)
{
    const int b = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float sc[4];   // multiplier (or divisor when PRECALC) of the four columns
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const int Cn = tile_n * 128 + 4 * lane + k;
        float s = 1.0f;
        if (Cn < N) {
            if (PRECALC) {
                s = __ldg(scale_in + Cn);
            } else {
                s = fp8_scale_from_amax<FMT>(u2f(__ldcg(amax_bits + Cn)), recip_div);
                if (tile_m == 0 && b == 0) scale_out[Cn] = s;
            }
        }
        sc[k] = PRECALC ? s : __fdiv_rn(1.0f, s);
    }
    mbar_wait(bar, parity, 5u);
    const uint32_t pbase = base + (lane >> 4) * CW_PANEL + (b * 32) * 128 + (lane & 1) * 8;
    const uint32_t j = (lane & 15) >> 1;
    const uint32_t qs = base + CW_Q_OFF;
    const uint32_t key = (lane >> 1) & 3;
    uint32_t o[4][8];
#pragma unroll
    for (int q4 = 0; q4 < 8; q4++) {
        uint2 w[4];
#pragma unroll
        for (int i = 0; i < 4; i++) w[i] = lds_v2(pbase + (4 * q4 + i) * 128 + ((j ^ ((4 * q4 + i) & 7)) << 4));
        if (PRECALC) {
            o[0][q4] = cvt_fp8x4<FMT>(__fdiv_rn(bf16lo(w[0].x), sc[0]), __fdiv_rn(bf16lo(w[1].x), sc[0]), __fdiv_rn(bf16lo(w[2].x), sc[0]), __fdiv_rn(bf16lo(w[3].x), sc[0]));
            o[1][q4] = cvt_fp8x4<FMT>(__fdiv_rn(bf16hi(w[0].x), sc[1]), __fdiv_rn(bf16hi(w[1].x), sc[1]), __fdiv_rn(bf16hi(w[2].x), sc[1]), __fdiv_rn(bf16hi(w[3].x), sc[1]));
            o[2][q4] = cvt_fp8x4<FMT>(__fdiv_rn(bf16lo(w[0].y), sc[2]), __fdiv_rn(bf16lo(w[1].y), sc[2]), __fdiv_rn(bf16lo(w[2].y), sc[2]), __fdiv_rn(bf16lo(w[3].y), sc[2]));
            o[3][q4] = cvt_fp8x4<FMT>(__fdiv_rn(bf16hi(w[0].y), sc[3]), __fdiv_rn(bf16hi(w[1].y), sc[3]), __fdiv_rn(bf16hi(w[2].y), sc[3]), __fdiv_rn(bf16hi(w[3].y), sc[3]));
        } else {
            o[0][q4] = scale_cvt_fp8x4<FMT>(bf16lo(w[0].x), bf16lo(w[1].x), bf16lo(w[2].x), bf16lo(w[3].x), sc[0]);
            o[1][q4] = scale_cvt_fp8x4<FMT>(bf16hi(w[0].x), bf16hi(w[1].x), bf16hi(w[2].x), bf16hi(w[3].x), sc[1]);
            o[2][q4] = scale_cvt_fp8x4<FMT>(bf16lo(w[0].y), bf16lo(w[1].y), bf16lo(w[2].y), bf16lo(w[3].y), sc[2]);
            o[3][q4] = scale_cvt_fp8x4<FMT>(bf16hi(w[0].y), bf16hi(w[1].y), bf16hi(w[2].y), bf16hi(w[3].y), sc[3]);
        }
    }
    // staging as in the mxfp8 tile kernel: sub-tile k = columns {4 l + k}, 64-byte rows, chunk c at c ^ ((l >> 1) & 3)
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const uint32_t rowp = qs + k * 2048 + lane * 64;
        sts_v4(rowp + (((2 * b) ^ key) << 4), make_uint4(o[k][0], o[k][1], o[k][2], o[k][3]));
        sts_v4(rowp + (((2 * b + 1) ^ key) << 4), make_uint4(o[k][4], o[k][5], o[k][6], o[k][7]));
    }
    __syncthreads();
    const int jj = lane & 3;
    const int mcol = tile_m * 64 + jj * 16;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int kk = 2 * b + (i >> 2);
        const int l = (i & 3) * 8 + (lane >> 2);
        const int Cn = tile_n * 128 + 4 * l + kk;
        const uint4 v = lds_v4(qs + kk * 2048 + l * 64 + ((jj ^ ((l >> 1) & 3)) << 4));
        if (Cn < N && mcol < M) *reinterpret_cast<uint4 *>(q + (size_t)Cn * M + mcol) = v;
    }
}

// One CTA per tile: the cast with given scales, or the second pass of the two-launch form.
template <int FMT, bool PRECALC>
__global__ void __launch_bounds__(64, 8)
fp8_colwise_cast_kernel(const __grid_constant__ CUtensorMap tm_x, const uint32_t *__restrict__ amax_bits,
                        const float *__restrict__ scale_in, uint8_t *__restrict__ q, float *__restrict__ scale_out, int M,
                        int N, int tiles_n, int recip_div)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *sbase = smem_raw + (base - smem_u32(smem_raw));
    uint64_t *bar = reinterpret_cast<uint64_t *>(sbase + CW_BAR_OFF);
    const int tile_m = blockIdx.x / tiles_n, tile_n = blockIdx.x - tile_m * tiles_n;
    if (threadIdx.x == 0) {
        mbar_init(bar, 1);
        fence_barrier_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        mbar_expect_tx(bar, 2 * CW_PANEL);
        tma_load_2d(sbase, &tm_x, bar, tile_n * 128, tile_m * 64);
        tma_load_2d(sbase + CW_PANEL, &tm_x, bar, tile_n * 128 + 64, tile_m * 64);
    }
    colwise_cast_tile<FMT, PRECALC>(base, bar, 0, amax_bits, scale_in, q, scale_out, M, N, tile_m, tile_n, recip_div != 0);
}

template <int FMT, bool PRECALC>
static int launch_colwise(const void *x, int64_t M, int64_t N, const float *scale_in, void *q, float *scale_out,
                          uint32_t *amax_bits, int recip_div, cudaStream_t st)
{
    CUtensorMap tx;
    uint64_t dims[2] = {(uint64_t)N, (uint64_t)M};
    uint64_t strides[1] = {(uint64_t)N * 2};
    uint32_t box[2] = {64, 64};
    int e = make_tensor_map(&tx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (e) return e;
    if (!PRECALC && q != nullptr) {
        // one launch with the panel resident in shared memory where the shape allows it (colwise.cu)
        const int rc = qcc_colwise_resident(x, M, N, FMT | (recip_div ? QCC_RECIP_DIV : 0), q, scale_out, amax_bits, st);
        if (rc != 1) return rc;
    }
    if (!PRECALC) {
        cudaError_t ce = cudaMemsetAsync(amax_bits, 0, (size_t)N * 4, st);
        if (ce != cudaSuccess) return (int)ce;
        dim3 grid((unsigned)((N / 8 + CW_AMAX_THREADS - 1) / CW_AMAX_THREADS), (unsigned)((M + CW_AMAX_ROWS - 1) / CW_AMAX_ROWS));
        fp8_colwise_amax_kernel<<<grid, CW_AMAX_THREADS, 0, st>>>((const uint16_t *)x, (int)M, (int)N, amax_bits);
        ce = cudaGetLastError();
        if (ce != cudaSuccess) return (int)ce;
        if (q == nullptr) {     // the scales alone (colwise_precalc_scale G:438-442): one read of x, no cast
            colwise_scale_kernel<FMT><<<(unsigned)((N + 255) / 256), 256, 0, st>>>(amax_bits, scale_out, (int)N, recip_div);
            return (int)cudaGetLastError();
        }
    }
    auto kern = fp8_colwise_cast_kernel<FMT, PRECALC>;
    static PerDeviceFlag configured;
    const int dev = current_device_slot();
    if (dev < 0) return QCC_ERR_ARG;
    if (!configured.get(dev)) {
        cudaError_t ce = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, CW_ALLOC);
        if (ce != cudaSuccess) return (int)ce;
        ce = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
        if (ce != cudaSuccess) return (int)ce;
        configured.set(dev);
    }
    const int tiles_n = (int)((N + 127) / 128), tiles_m = (int)((M + 63) / 64);
    const long long num_tiles = (long long)tiles_n * tiles_m;
    if (num_tiles > 0x7FFFFFFF) return QCC_ERR_SHAPE;
    kern<<<(unsigned)num_tiles, 64, CW_ALLOC, st>>>(tx, amax_bits, scale_in, (uint8_t *)q, scale_out, (int)M, (int)N, tiles_n, recip_div);
    return (int)cudaGetLastError();
}

}  // namespace qcc

using namespace qcc;

// per-translation-unit error words of the tiled kernels
extern "C" int qcc_mxfp8_device_error(unsigned int *out);
extern "C" int qcc_nvfp4_device_error(unsigned int *out);
extern "C" int qcc_block128_device_error(unsigned int *out);
extern "C" int qcc_colwise_device_error(unsigned int *out);
extern "C" int qcc_xchg_device_error(unsigned int *out);

extern "C" {

int qcc_version(void) { return 100; }

int qcc_device_error(unsigned int *out)
{
    unsigned int a = 0, b = 0, c = 0;
    int e = read_clear_device_error(&a);
    if (e) return e;
    if ((e = qcc_mxfp8_device_error(&b)) != 0) return e;
    if ((e = qcc_nvfp4_device_error(&c)) != 0) return e;
    unsigned int d = 0;
    if ((e = qcc_block128_device_error(&d)) != 0) return e;
    c = c > d ? c : d;
    if ((e = qcc_colwise_device_error(&d)) != 0) return e;
    c = c > d ? c : d;
    if ((e = qcc_xchg_device_error(&d)) != 0) return e;
    c = c > d ? c : d;
    if (out) *out = a > b ? (a > c ? a : c) : (b > c ? b : c);
    return 0;
}

int qcc_sm_count(void) { return sm_count(); }

int qcc_copy2d_async(void *dst, size_t dst_pitch, const void *src, size_t src_pitch, size_t width_bytes, size_t rows,
                     int to_host, void *stream)
{
    if (!dst || !src) return QCC_ERR_ARG;
    if (width_bytes == 0 || rows == 0) return 0;
    return (int)cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, width_bytes, rows,
                                  to_host ? cudaMemcpyDeviceToHost : cudaMemcpyHostToDevice, (cudaStream_t)stream);
}

int qcc_stream_copy(const void *src, void *dst, size_t bytes, void *stream)
{
    if (bytes == 0) return 0;
    if (!src || !dst) return QCC_ERR_ARG;
    if (bytes % 16 != 0) return QCC_ERR_SHAPE;
    if (!aligned16(src) || !aligned16(dst)) return QCC_ERR_ALIGN;
    const int64_t nvec = (int64_t)(bytes / 16);
    const int64_t grid = (nvec + TW_THREADS * 2 - 1) / (TW_THREADS * 2);
    if (grid > 0x7FFFFFFF) return QCC_ERR_SHAPE;
    stream_copy_kernel<<<(unsigned)grid, TW_THREADS, 0, (cudaStream_t)stream>>>((const uint4 *)src, (uint4 *)dst, nvec);
    return (int)cudaGetLastError();
}

int qcc_stream_fold(const void *src, void *dst, size_t bytes_in, int ratio, void *stream)
{
    if (bytes_in == 0) return 0;
    if (!src || !dst || (ratio != 2 && ratio != 4)) return QCC_ERR_ARG;
    if (bytes_in % (16 * (size_t)ratio) != 0) return QCC_ERR_SHAPE;
    if (!aligned16(src) || !aligned16(dst)) return QCC_ERR_ALIGN;
    const int64_t nout = (int64_t)(bytes_in / 16 / ratio);
    const int u = ratio == 2 ? 2 : 1;
    const int64_t grid = (nout + TW_THREADS * u - 1) / (TW_THREADS * u);
    if (grid > 0x7FFFFFFF) return QCC_ERR_SHAPE;
    if (ratio == 2)
        stream_fold_kernel<2, 2><<<(unsigned)grid, TW_THREADS, 0, (cudaStream_t)stream>>>((const uint4 *)src, (uint4 *)dst, nout);
    else
        stream_fold_kernel<4, 1><<<(unsigned)grid, TW_THREADS, 0, (cudaStream_t)stream>>>((const uint4 *)src, (uint4 *)dst, nout);
    return (int)cudaGetLastError();
}

size_t qcc_amax_workspace_bytes(void) { return (size_t)(AMAX_MAX_CTAS + 64) * sizeof(uint32_t); }

int qcc_amax_workspace_init(void *workspace, size_t workspace_bytes, void *stream)
{
    if (!workspace) return QCC_ERR_ARG;
    if (workspace_bytes < qcc_amax_workspace_bytes()) return QCC_ERR_WORKSPACE;
    return (int)cudaMemsetAsync(workspace, 0, qcc_amax_workspace_bytes(), (cudaStream_t)stream);
}

static int amax_oneshot_grid(int64_t n, unsigned *grid)
{
    const int64_t per_cta = (int64_t)AMAX_THREADS * AMAX1_U;
    const int64_t want = ((n >> 3) + per_cta - 1) / per_cta;
    if (want > 0x7FFFFFFF) return QCC_ERR_SHAPE;
    *grid = (unsigned)(want < 1 ? 1 : want);
    return 0;
}

int qcc_amax_bf16(const void *x, int64_t n, int mode, int fmt, float *out, void *workspace, size_t workspace_bytes,
                  void *stream)
{
    const bool one_launch = (mode & QCC_AMAX_ONE_LAUNCH) != 0;
    mode &= ~QCC_AMAX_ONE_LAUNCH;
    if (!x || !out || !workspace || n < 0) return QCC_ERR_ARG;
    if (!amax_mode_ok(mode) || (fmt != QCC_FMT_E4M3 && fmt != QCC_FMT_E5M2)) return QCC_ERR_ARG;
    if (!aligned16(x)) return QCC_ERR_ALIGN;
    if (workspace_bytes < qcc_amax_workspace_bytes()) return QCC_ERR_WORKSPACE;
    cudaStream_t st = (cudaStream_t)stream;
    if (one_launch) {
        unsigned grid1 = 0;
        int rc = amax_oneshot_grid(n, &grid1);
        if (rc) return rc;
        amax_oneshot_kernel<false><<<grid1, AMAX_THREADS, 0, st>>>((const uint16_t *)x, n, (uint32_t *)workspace + AMAX_MAX_CTAS,
                                                                  mode, fmt, out);
        return (int)cudaGetLastError();
    }
    int64_t want = ((n >> 3) + AMAX_THREADS * AMAX_U - 1) / (AMAX_THREADS * AMAX_U);
    int64_t cap = (int64_t)sm_count() * AMAX_CTAS_PER_SM;
    if (cap > AMAX_MAX_CTAS) cap = AMAX_MAX_CTAS;
    int grid = (int)(want < 1 ? 1 : (want > cap ? cap : want));
    amax_partial_kernel<<<grid, AMAX_THREADS, 0, st>>>((const uint16_t *)x, n, (uint32_t *)workspace);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    amax_finish_kernel<<<1, AMAX_THREADS, 0, st>>>((const uint32_t *)workspace, grid, mode, fmt, out);
    return (int)cudaGetLastError();
}

int qcc_amax_bf16_xchg(const void *x, int64_t n, void *state, void *stream)
{
    if (!x || !state || n < 0) return QCC_ERR_ARG;
    if (!aligned16(x)) return QCC_ERR_ALIGN;
    unsigned grid1 = 0;
    int rc = amax_oneshot_grid(n, &grid1);
    if (rc) return rc;
    amax_oneshot_kernel<true><<<grid1, AMAX_THREADS, 0, (cudaStream_t)stream>>>((const uint16_t *)x, n, static_cast<uint32_t *>(state),
                                                                                QCC_AMAX_RAW, QCC_FMT_E4M3, nullptr);
    return (int)cudaGetLastError();
}

int qcc_amax_bf16_noalloc(const void *x, int64_t n, int mode, int fmt, float *out, void *stream)
{
    if (!x || !out || n < 0) return QCC_ERR_ARG;
    if (!amax_mode_ok(mode) || (fmt != QCC_FMT_E4M3 && fmt != QCC_FMT_E5M2)) return QCC_ERR_ARG;
    if (!aligned16(x)) return QCC_ERR_ALIGN;
    if (n > QCC_AMAX_NOALLOC_MAX_ELEMS) return QCC_ERR_TOO_LARGE;
    // In host code the array's name is only a handle: the device address has to be asked for, once per
    // device, with that device current.  The first call on a device does it here.
    // The address stays valid for the life of the device's primary context.  Host threads that make their first call
    // on a device at the same time all store the same address (the slots are atomics), so the race is harmless.
    static std::atomic<uint32_t *> scratch[QCC_MAX_DEVICES];
    const int dev = current_device_slot();
    if (dev < 0) return QCC_ERR_ARG;
    cudaError_t e;
    uint32_t *scratch_dev = scratch[dev].load(std::memory_order_acquire);
    if (!scratch_dev) {
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, g_amax_noalloc_scratch);
        if (e != cudaSuccess) return (int)e;
        scratch_dev = static_cast<uint32_t *>(p);
        scratch[dev].store(scratch_dev, std::memory_order_release);
    }
    cudaStream_t st = (cudaStream_t)stream;
    int64_t want = ((n >> 3) + AMAX_THREADS * AMAX_U - 1) / (AMAX_THREADS * AMAX_U);
    int64_t cap = (int64_t)sm_count() * AMAX_CTAS_PER_SM;
    if (cap > AMAX_MAX_CTAS) cap = AMAX_MAX_CTAS;
    int grid = (int)(want < 1 ? 1 : (want > cap ? cap : want));
    // every slot the finish reads is written by this launch, so nothing has to be cleared
    amax_partial_kernel<<<grid, AMAX_THREADS, 0, st>>>((const uint16_t *)x, n, scratch_dev);
    e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    amax_finish_kernel<<<1, AMAX_THREADS, 0, st>>>(scratch_dev, grid, mode, fmt, out);
    return (int)cudaGetLastError();
}

int qcc_scale_from_amax(const float *amax, int mode, int fmt, float *out, void *stream)
{
    if (!amax || !out) return QCC_ERR_ARG;
    if (!amax_mode_ok(mode) || (fmt != QCC_FMT_E4M3 && fmt != QCC_FMT_E5M2)) return QCC_ERR_ARG;
    scale_from_amax_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(amax, mode, fmt, out);
    return (int)cudaGetLastError();
}

static int fp8_tensorwise_entry(const void *x, int64_t n, const float *src, int src_kind, int fmt, void *q, float *scale_out,
                               void *stream)
{
    if (!src) return QCC_ERR_ARG;
    const int recip_div = take_recip_div(fmt);
    if (fmt != QCC_FMT_E4M3 && fmt != QCC_FMT_E5M2) return QCC_ERR_ARG;
    if (n == 0 && src_kind == QCC_SRC_SCALE) return 0;
    if (!x || !q || n < 0) return QCC_ERR_ARG;
    if (!aligned16(x) || !aligned16(q)) return QCC_ERR_ALIGN;
    cudaStream_t st = (cudaStream_t)stream;
    const int64_t per_cta = (int64_t)TW_THREADS * TW_UNROLL * 16;
    int64_t grid = (n + per_cta - 1) / per_cta;
    if (grid > 0x7FFFFFFF) return QCC_ERR_SHAPE;
    if (grid < 1) grid = 1;
    const uint16_t *xp = (const uint16_t *)x;
#define QCC_TW(FMT_, SRC_) fp8_tensorwise_kernel<FMT_, SRC_><<<(unsigned)grid, TW_THREADS, 0, st>>>(xp, n, src, scale_out, (uint8_t *)q, recip_div)
    if (fmt == QCC_FMT_E5M2) {
        if (src_kind == QCC_SRC_SCALE) QCC_TW(QCC_FMT_E5M2, QCC_SRC_SCALE); else QCC_TW(QCC_FMT_E5M2, QCC_SRC_AMAX);
    } else {
        if (src_kind == QCC_SRC_SCALE) QCC_TW(QCC_FMT_E4M3, QCC_SRC_SCALE); else QCC_TW(QCC_FMT_E4M3, QCC_SRC_AMAX);
    }
#undef QCC_TW
    return (int)cudaGetLastError();
}

int qcc_fp8_tensorwise_from_amax(const void *x, int64_t n, const float *amax, int fmt, void *q, float *scale_out, void *stream)
{
    return fp8_tensorwise_entry(x, n, amax, QCC_SRC_AMAX, fmt, q, scale_out, stream);
}

int qcc_fp8_tensorwise(const void *x, int64_t n, const float *scale, int fmt, void *q, void *stream)
{
    if (n == 0) return 0;
    if (!scale) return QCC_ERR_ARG;
    return fp8_tensorwise_entry(x, n, scale, QCC_SRC_SCALE, fmt, q, nullptr, stream);
}

int qcc_fp8_rowwise(const void *x, int64_t M, int64_t N, int fmt, void *q, float *scale, void *stream)
{
    if (M == 0 || N == 0) return 0;
    if (!x || !scale || M < 0 || N < 0) return QCC_ERR_ARG;
    const int recip_div = take_recip_div(fmt);
    if (fmt != QCC_FMT_E4M3 && fmt != QCC_FMT_E5M2) return QCC_ERR_ARG;
    if (N % 8 == 0 && (!aligned16(x) || (q && !aligned16(q)))) return QCC_ERR_ALIGN;
    if (M == 0 || N == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    return fmt == QCC_FMT_E5M2 ? launch_rowwise<QCC_FMT_E5M2, false>(x, M, N, nullptr, q, scale, recip_div, st)
                               : launch_rowwise<QCC_FMT_E4M3, false>(x, M, N, nullptr, q, scale, recip_div, st);
}

int qcc_nvfp4_per_token_scale(const void *x, int64_t M, int64_t N, int flags, float *scale, void *stream)
{
    if (M == 0 || N == 0) return 0;
    if (!x || !scale || M < 0 || N < 0 || (flags & ~QCC_RECIP_DIV)) return QCC_ERR_ARG;
    if (N % 8 == 0 && !aligned16(x)) return QCC_ERR_ALIGN;
    return launch_rowwise<FMT_NVFP4_OUTER, false>(x, M, N, nullptr, nullptr, scale, (flags & QCC_RECIP_DIV) ? 1 : 0, (cudaStream_t)stream);
}

int qcc_fp8_rowwise_precalc(const void *x, int64_t M, int64_t N, const float *scale, int fmt, void *q, void *stream)
{
    if (M == 0 || N == 0) return 0;
    if (!x || !scale || !q || M < 0 || N < 0) return QCC_ERR_ARG;
    if (fmt != QCC_FMT_E4M3 && fmt != QCC_FMT_E5M2) return QCC_ERR_ARG;
    if (N % 8 == 0 && (!aligned16(x) || !aligned16(q))) return QCC_ERR_ALIGN;
    if (M == 0 || N == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    return fmt == QCC_FMT_E5M2 ? launch_rowwise<QCC_FMT_E5M2, true>(x, M, N, scale, q, nullptr, 0, st)
                               : launch_rowwise<QCC_FMT_E4M3, true>(x, M, N, scale, q, nullptr, 0, st);
}

size_t qcc_fp8_colwise_workspace_bytes(int64_t M, int64_t N)
{
    (void)M;
    if (N <= 0) return 0;
    return (size_t)N * 4 + 128 + 128 * (1 + (size_t)((N + 63) / 64));   // column maxima, then one counter per panel on a 128-byte line of its own
}

int qcc_fp8_colwise(const void *x, int64_t M, int64_t N, int fmt, void *q, float *scale, void *workspace,
                    size_t workspace_bytes, void *stream)
{
    if (M == 0 || N == 0) return 0;
    if (!x || !scale || !workspace || M < 0 || N < 0) return QCC_ERR_ARG;
    const int recip_div = take_recip_div(fmt);
    if (fmt != QCC_FMT_E4M3 && fmt != QCC_FMT_E5M2) return QCC_ERR_ARG;
    if (N % 8 != 0 || M % 16 != 0 || M > 0x7FFFFF00 || N > 0x7FFFFF00 || (M + CW_AMAX_ROWS - 1) / CW_AMAX_ROWS > 65535)
        return QCC_ERR_SHAPE;
    if (!aligned16(x) || (q && !aligned16(q)) || !aligned16(workspace)) return QCC_ERR_ALIGN;
    if (workspace_bytes < qcc_fp8_colwise_workspace_bytes(M, N)) return QCC_ERR_WORKSPACE;
    cudaStream_t st = (cudaStream_t)stream;
    return fmt == QCC_FMT_E5M2 ? launch_colwise<QCC_FMT_E5M2, false>(x, M, N, nullptr, q, scale, (uint32_t *)workspace, recip_div, st)
                               : launch_colwise<QCC_FMT_E4M3, false>(x, M, N, nullptr, q, scale, (uint32_t *)workspace, recip_div, st);
}

int qcc_fp8_colwise_precalc(const void *x, int64_t M, int64_t N, const float *scale, int fmt, void *q, void *stream)
{
    if (M == 0 || N == 0) return 0;
    if (!x || !q || !scale || M < 0 || N < 0) return QCC_ERR_ARG;
    if (fmt != QCC_FMT_E4M3 && fmt != QCC_FMT_E5M2) return QCC_ERR_ARG;
    if (N % 8 != 0 || M % 16 != 0 || M > 0x7FFFFF00 || N > 0x7FFFFF00) return QCC_ERR_SHAPE;
    if (!aligned16(x) || !aligned16(q)) return QCC_ERR_ALIGN;
    cudaStream_t st = (cudaStream_t)stream;
    return fmt == QCC_FMT_E5M2 ? launch_colwise<QCC_FMT_E5M2, true>(x, M, N, scale, q, nullptr, nullptr, 0, st)
                               : launch_colwise<QCC_FMT_E4M3, true>(x, M, N, scale, q, nullptr, nullptr, 0, st);
}

}  // extern "C"
