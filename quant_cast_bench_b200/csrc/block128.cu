// fp8 e4m3 with one fp32 scale per 1x128, 128x1 or 128x128 block (the "deepseek" recipes) for sm_100a.
//
//  * 1x128 along the rows: a flat stream.  A thread owns 32 consecutive elements (four 16-byte loads), four
//    lanes share a block: two shuffles give the block maximum, every lane forms scale and reciprocal, two
//    16-byte stores per thread and one scale store per block.
//  * 128x1 down the rows (outputs transposed) and both directions from one read: a one-shot tile kernel, one
//    CTA per 128x128 tile fetched by TMA (two 64-column boxes, 128-byte swizzle, bounded mbarrier wait).  Four
//    column warps each hold a 32-row slab in registers (lane = four adjacent columns), exchange their column
//    maxima through shared memory, quantise and stage the transposed bytes in a swizzled tile that leaves as
//    coalesced 16-byte stores; with both directions the same warps then quantise along the rows (lane = row).
//  * 128x128: one CTA of 128 threads per block, the block held in registers (16 x 16 bytes per thread), one
//    CTA-wide maximum, 8-byte stores.
//
// Numerics: G = quant_cast_bench/quant_cast_gold/recipes.py of vkuzo/quant_cast_bench.  deepseek_1x128_f
// G:103-110, deepseek_128x128_f G:141-161, deepseek_1x128_dim_m_f G:194-214, deepseek_1x128_dim_km_f G:251-277:
// scale = clamp(amax, 1e-12) / 448 (IEEE division; with QCC_RECIP_DIV the product with fl(1 / 448) that CUDA eager
// computes), q = e4m3(x * (1 / scale)).  The clamp happens in bf16 in the
// first three (bf16(1e-12) = 0x2B8D) and in fp32 in the fused recipe (G:264, G:268), which only shows in the
// scale of an all-zero block.
#include "common.cuh"
#include "host_util.h"

namespace qcc {

template <bool CLAMP_F32>
__device__ __forceinline__ float block_scale(float amax, bool recip_div)
{
    const float a = fmaxf(amax, CLAMP_F32 ? 1e-12f : u2f(0x2B8D0000u));
    return div_by_const(a, 448.0f, recip_div);
}

// ---------------------------------------------------------------------------------------------
// 1x128 along the rows: flat stream
// ---------------------------------------------------------------------------------------------
constexpr int B1_THREADS = 256;

template <bool CLAMP_F32>
__global__ void __launch_bounds__(B1_THREADS)
fp8_1x128_stream_kernel(const uint16_t *__restrict__ x, uint32_t n_seg, uint8_t *__restrict__ q, float *__restrict__ scale,
                        int recip_div)
{
    const uint32_t si = blockIdx.x * B1_THREADS + threadIdx.x;   // 32-element segment; four per block
    const bool ok = si < n_seg;
    uint4 c[4] = {};
    if (ok) {
        const uint4 *p = reinterpret_cast<const uint4 *>(x) + (size_t)si * 4;
#pragma unroll
        for (int i = 0; i < 4; i++) c[i] = ld_v4(p + i);
    }
    uint32_t m = f2u(amax_of_block(c));                          // non-negative floats order like integers
    m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, 1));
    m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, 2));
    const float s = block_scale<CLAMP_F32>(u2f(m), recip_div != 0);
    const float inv = __fdiv_rn(1.0f, s);
    uint4 o0, o1;
    quant_row_block(c, inv, o0, o1);
    if (ok) {
        uint4 *dst = reinterpret_cast<uint4 *>(q) + (size_t)si * 2;
        st_out(dst, o0);
        st_out(dst + 1, o1);
        if ((threadIdx.x & 3) == 0) scale[si >> 2] = s;
    }
}

// ---------------------------------------------------------------------------------------------
// 128x128 blocks: register tile
// ---------------------------------------------------------------------------------------------
// AMAX_ONLY: no cast; scale receives the block maximum divided by `amax_div` (1: the maximum itself, 2688: the
// per-block nvfp4 outer scale of nvfp4_blocked_outer_scale, G:1601-1606, which takes no clamp).
template <bool AMAX_ONLY>
__global__ void __launch_bounds__(128, 4)
fp8_128x128_kernel(const uint16_t *__restrict__ x, int N, int tiles_n, uint8_t *__restrict__ q, float *__restrict__ scale,
                   float amax_div, int recip_div)
{
    __shared__ uint32_t s_max[4];
    const int tile_m = blockIdx.x / tiles_n, tile_n = blockIdx.x - tile_m * tiles_n;
    const int t = threadIdx.x, chunk = t & 15, r0 = t >> 4;
    const size_t origin = (size_t)tile_m * 128 * N + (size_t)tile_n * 128 + chunk * 8;
    uint4 v[16];
#pragma unroll
    for (int i = 0; i < 16; i++) v[i] = ld_nc_v4(reinterpret_cast<const uint4 *>(x + origin + (size_t)(i * 8 + r0) * N));
    uint32_t a0 = 0, a1 = 0;
#pragma unroll
    for (int i = 0; i < 16; i++) {
        a0 = absmax2_acc(absmax2_acc(a0, v[i].x), v[i].y);
        a1 = absmax2_acc(absmax2_acc(a1, v[i].z), v[i].w);
    }
    uint32_t m = f2u(hmax_halves_f32(absmax2(a0, a1)));
    m = __reduce_max_sync(0xFFFFFFFFu, m);
    if ((t & 31) == 0) s_max[t >> 5] = m;
    __syncthreads();
    m = max(max(s_max[0], s_max[1]), max(s_max[2], s_max[3]));
    if (AMAX_ONLY) {
        if (t == 0) scale[blockIdx.x] = div_by_const(u2f(m), amax_div, recip_div != 0);
        return;
    }
    const float s = block_scale<false>(u2f(m), recip_div != 0);
    const float inv = __fdiv_rn(1.0f, s);
    uint8_t *qo = q + origin;
#pragma unroll
    for (int i = 0; i < 16; i++) {
        uint2 o;
        o.x = scale_cvt_fp8x4<QCC_FMT_E4M3>(bf16lo(v[i].x), bf16hi(v[i].x), bf16lo(v[i].y), bf16hi(v[i].y), inv);
        o.y = scale_cvt_fp8x4<QCC_FMT_E4M3>(bf16lo(v[i].z), bf16hi(v[i].z), bf16lo(v[i].w), bf16hi(v[i].w), inv);
        st_out(reinterpret_cast<uint2 *>(qo + (size_t)(i * 8 + r0) * N), o);
    }
    if (t == 0) scale[blockIdx.x] = s;
}

// ---------------------------------------------------------------------------------------------
// 128x1 down the rows (transposed outputs), optionally with 1x128 along the rows: tile kernel
// ---------------------------------------------------------------------------------------------
constexpr int BT_PANEL = 128 * 128;                 // one 64-column panel: 128 rows x 128 B
constexpr int BT_X_OFF = 0;
constexpr int BT_QM_OFF = 2 * BT_PANEL;             // transposed staging: 4 sub-tiles x 32 output rows x 128 B
constexpr int BT_AM_OFF = BT_QM_OFF + 4 * 32 * 128; // column maxima of the four slabs: 4 x 32 lanes x 8 B
constexpr int BT_BAR_OFF = BT_AM_OFF + 1024;
constexpr int BT_QK_OFF = BT_QM_OFF;                // rowwise staging (fused form): reuses the transposed staging
constexpr int BT_ALLOC = BT_BAR_OFF + 64 + 1024;

// 16 bf16 in two 16-byte chunks -> 16 e4m3 bytes
__device__ __forceinline__ uint4 quant16(uint4 a, uint4 b, float inv)
{
    uint4 o;
    o.x = scale_cvt_fp8x4<QCC_FMT_E4M3>(bf16lo(a.x), bf16hi(a.x), bf16lo(a.y), bf16hi(a.y), inv);
    o.y = scale_cvt_fp8x4<QCC_FMT_E4M3>(bf16lo(a.z), bf16hi(a.z), bf16lo(a.w), bf16hi(a.w), inv);
    o.z = scale_cvt_fp8x4<QCC_FMT_E4M3>(bf16lo(b.x), bf16hi(b.x), bf16lo(b.y), bf16hi(b.y), inv);
    o.w = scale_cvt_fp8x4<QCC_FMT_E4M3>(bf16lo(b.z), bf16hi(b.z), bf16lo(b.w), bf16hi(b.w), inv);
    return o;
}

// RECIP: QCC_RECIP_DIV, as a template parameter because the kernel sits at its register limit.
template <bool DO_K, bool CLAMP_F32, bool RECIP>
__global__ void __launch_bounds__(128, 4)
fp8_block128_tile_kernel(const __grid_constant__ CUtensorMap tm_x, uint8_t *__restrict__ qk, float *__restrict__ sk,
                         uint8_t *__restrict__ qm, float *__restrict__ sm, int M, int N, int tiles_n)
{
    constexpr bool recip_div = RECIP;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *sbase = smem_raw + (base - smem_u32(smem_raw));
    uint64_t *bar = reinterpret_cast<uint64_t *>(sbase + BT_BAR_OFF);
    const int tile_m = blockIdx.x / tiles_n, tile_n = blockIdx.x - tile_m * tiles_n;
    const int b = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        mbar_init(bar, 1);
        fence_barrier_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        mbar_expect_tx(bar, 2 * BT_PANEL);
        tma_load_2d(sbase + BT_X_OFF, &tm_x, bar, tile_n * 128, tile_m * 128);
        tma_load_2d(sbase + BT_X_OFF + BT_PANEL, &tm_x, bar, tile_n * 128 + 64, tile_m * 128);
    }
    mbar_wait(bar, 0, 5u);

    // ---------------------------------------------------------------------- along the row: lane = row
    auto row_phase = [&](const int rw) {
        const int row_t = rw * 32 + lane;
        const int R = tile_m * 128 + row_t;
        const uint32_t xrow = base + BT_X_OFF + row_t * 128;
        const uint32_t key7 = lane & 7;
        uint32_t a0 = 0, a1 = 0;
#pragma unroll
        for (int ch = 0; ch < 16; ch++) {
            const uint4 v = lds_v4(xrow + (ch >> 3) * BT_PANEL + ((((uint32_t)ch & 7u) ^ key7) << 4));
            a0 = absmax2_acc(absmax2_acc(a0, v.x), v.y);
            a1 = absmax2_acc(absmax2_acc(a1, v.z), v.w);
        }
        const float s = block_scale<CLAMP_F32>(hmax_halves_f32(absmax2(a0, a1)), recip_div);
        const float inv = __fdiv_rn(1.0f, s);
        const uint32_t qrow = base + BT_QK_OFF + row_t * 128;
#pragma unroll
        for (int oc = 0; oc < 8; oc++) {
            const uint32_t prow = xrow + (oc >> 2) * BT_PANEL;
            const uint32_t j0 = (oc & 3) * 2;
            const uint4 va = lds_v4(prow + ((j0 ^ key7) << 4));
            const uint4 vb = lds_v4(prow + (((j0 + 1) ^ key7) << 4));
            sts_v4(qrow + (((uint32_t)oc ^ key7) << 4), quant16(va, vb, inv));
        }
        __syncwarp();
        {
            const uint32_t j = lane & 7;
            const int col = tile_n * 128 + j * 16;
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const int rt = rw * 32 + i * 4 + (lane >> 3);
                const int Rr = tile_m * 128 + rt;
                const uint4 v = lds_v4(base + BT_QK_OFF + rt * 128 + ((j ^ ((uint32_t)rt & 7u)) << 4));
                if (Rr < M && col < N) *reinterpret_cast<uint4 *>(qk + (size_t)Rr * N + col) = v;
            }
        }
        if (R < M) sk[(size_t)R * (N >> 7) + tile_n] = s;
    };

    // ---------------------------------------------------------------------- down the rows: lane = 4 columns
    const uint32_t pbase = base + BT_X_OFF + (lane >> 4) * BT_PANEL + (b * 32) * 128 + (lane & 1) * 8;
    const uint32_t j = (lane & 15) >> 1;
    uint2 w[32];
    uint32_t a0 = 0, a1 = 0;
#pragma unroll
    for (int r = 0; r < 32; r++) {
        w[r] = lds_v2(pbase + r * 128 + ((j ^ (r & 7)) << 4));
        a0 = absmax2_acc(a0, w[r].x);
        a1 = absmax2_acc(a1, w[r].y);
    }
    // the block runs over all four slabs: exchange the slab maxima
    const uint32_t ams = base + BT_AM_OFF;
    asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(ams + b * 256 + lane * 8), "r"(a0), "r"(a1) : "memory");
    named_barrier(1, 128);
#pragma unroll
    for (int bb = 0; bb < 4; bb++) {
        const uint2 o = lds_v2(ams + bb * 256 + lane * 8);
        a0 = absmax2(a0, o.x);
        a1 = absmax2(a1, o.y);
    }
    float s[4], inv[4];
    {
        const float am[4] = {u2f(a0 << 16), u2f(a0 & 0xFFFF0000u), u2f(a1 << 16), u2f(a1 & 0xFFFF0000u)};
#pragma unroll
        for (int kk = 0; kk < 4; kk++) {
            s[kk] = block_scale<CLAMP_F32>(am[kk], recip_div);
            inv[kk] = __fdiv_rn(1.0f, s[kk]);
        }
    }
    // staging: sub-tile kk holds columns {4 l + kk}, one 128-byte row (the tile's 128 m) per column;
    // 16-byte chunk c of row l sits at position c ^ (l & 7).  Slab b is chunks 2b and 2b + 1.
    const uint32_t qms = base + BT_QM_OFF;
    const uint32_t key = lane & 7;
#pragma unroll
    for (int kk = 0; kk < 4; kk++) {
        uint32_t o[8];
#pragma unroll
        for (int q4 = 0; q4 < 8; q4++) {
            const uint2 r0 = w[4 * q4], r1 = w[4 * q4 + 1], r2 = w[4 * q4 + 2], r3 = w[4 * q4 + 3];
            const float sc = inv[kk];
            if (kk == 0)
                o[q4] = scale_cvt_fp8x4<QCC_FMT_E4M3>(bf16lo(r0.x), bf16lo(r1.x), bf16lo(r2.x), bf16lo(r3.x), sc);
            else if (kk == 1)
                o[q4] = scale_cvt_fp8x4<QCC_FMT_E4M3>(bf16hi(r0.x), bf16hi(r1.x), bf16hi(r2.x), bf16hi(r3.x), sc);
            else if (kk == 2)
                o[q4] = scale_cvt_fp8x4<QCC_FMT_E4M3>(bf16lo(r0.y), bf16lo(r1.y), bf16lo(r2.y), bf16lo(r3.y), sc);
            else
                o[q4] = scale_cvt_fp8x4<QCC_FMT_E4M3>(bf16hi(r0.y), bf16hi(r1.y), bf16hi(r2.y), bf16hi(r3.y), sc);
        }
        const uint32_t rowp = qms + kk * 4096 + lane * 128;
        sts_v4(rowp + (((uint32_t)(2 * b) ^ key) << 4), make_uint4(o[0], o[1], o[2], o[3]));
        sts_v4(rowp + (((uint32_t)(2 * b + 1) ^ key) << 4), make_uint4(o[4], o[5], o[6], o[7]));
    }
    named_barrier(1, 128);
    // write-out: warp b takes sub-tile b; eight lanes move one 128-byte row
    {
        const uint32_t jj = lane & 7;
        const int mcol = tile_m * 128 + jj * 16;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int l = i * 4 + (lane >> 3);
            const int Cn = tile_n * 128 + 4 * l + b;
            const uint4 v = lds_v4(qms + b * 4096 + l * 128 + ((jj ^ ((uint32_t)l & 7u)) << 4));
            if (Cn < N && mcol < M) *reinterpret_cast<uint4 *>(qm + (size_t)Cn * M + mcol) = v;
        }
    }
    if (b == 0) {
#pragma unroll
        for (int kk = 0; kk < 4; kk++) {
            const int Cn = tile_n * 128 + 4 * lane + kk;
            if (Cn < N) sm[(size_t)Cn * (M >> 7) + tile_m] = s[kk];
        }
    }
    if (DO_K) {
        // the same four warps take the rows once the staging tile has been drained (four extra warps for this half
        // left 3 CTAs per SM and idled while the column warps finished)
        __syncthreads();
        row_phase(b);
    }
}

template <bool DO_K, bool CLAMP_F32, bool RECIP>
static int launch_block128_tile_r(const CUtensorMap &tx, uint8_t *qk, float *sk, uint8_t *qm, float *sm, int M, int N, cudaStream_t st)
{
    auto kern = fp8_block128_tile_kernel<DO_K, CLAMP_F32, RECIP>;
    constexpr int ALLOC = BT_ALLOC;
    static PerDeviceFlag configured;
    const int dev = current_device_slot();
    if (dev < 0) return QCC_ERR_ARG;
    if (!configured.get(dev)) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, ALLOC);
        if (e != cudaSuccess) return (int)e;
        e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
        if (e != cudaSuccess) return (int)e;
        configured.set(dev);
    }
    const int tiles_n = (N + 127) / 128, tiles_m = M / 128;
    const long long num_tiles = (long long)tiles_n * tiles_m;
    if (num_tiles > 0x7FFFFFFF) return QCC_ERR_SHAPE;
    kern<<<(unsigned)num_tiles, 128, ALLOC, st>>>(tx, qk, sk, qm, sm, M, N, tiles_n);
    return (int)cudaGetLastError();
}

template <bool DO_K, bool CLAMP_F32>
static int launch_block128_tile(const CUtensorMap &tx, uint8_t *qk, float *sk, uint8_t *qm, float *sm, int M, int N, int recip_div,
                                cudaStream_t st)
{
    return recip_div ? launch_block128_tile_r<DO_K, CLAMP_F32, true>(tx, qk, sk, qm, sm, M, N, st)
                     : launch_block128_tile_r<DO_K, CLAMP_F32, false>(tx, qk, sk, qm, sm, M, N, st);
}

}  // namespace qcc

using namespace qcc;

extern "C" int qcc_block128_device_error(unsigned int *out) { return read_clear_device_error(out); }

extern "C" int qcc_fp8_block128(const void *x, int64_t M, int64_t N, int flags, void *qk, float *sk, void *qm, float *sm,
                                void *stream)
{
    const int recip_div = take_recip_div(flags);
    const bool row = flags & QCC_ROWWISE, col = flags & QCC_COLWISE;
    if (M == 0 || N == 0) return 0;
    if (!x || (!row && !col) || (flags & ~(QCC_ROWWISE | QCC_COLWISE))) return QCC_ERR_ARG;
    if ((row && (!qk || !sk)) || (col && (!qm || !sm))) return QCC_ERR_ARG;
    if (M < 0 || N < 0 || M > 0x7FFFFF00 || N > 0x7FFFFF00) return QCC_ERR_SHAPE;
    if ((row && N % 128 != 0) || (col && (M % 128 != 0 || N % 8 != 0))) return QCC_ERR_SHAPE;
    if (!aligned16(x) || (row && !aligned16(qk)) || (col && !aligned16(qm))) return QCC_ERR_ALIGN;
    cudaStream_t st = (cudaStream_t)stream;
    if (!col) {
        if (M * (N / 32) >= (1ll << 32) - B1_THREADS) return QCC_ERR_SHAPE;
        const uint32_t n_seg = (uint32_t)(M * (N / 32));
        fp8_1x128_stream_kernel<false><<<(n_seg + B1_THREADS - 1) / B1_THREADS, B1_THREADS, 0, st>>>(
            (const uint16_t *)x, n_seg, (uint8_t *)qk, sk, recip_div);
        return (int)cudaGetLastError();
    }
    CUtensorMap tx;
    uint64_t dims[2] = {(uint64_t)N, (uint64_t)M};
    uint64_t strides[1] = {(uint64_t)N * 2};
    uint32_t box[2] = {64, 128};
    int e = make_tensor_map(&tx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (e) return e;
    if (row) return launch_block128_tile<true, true>(tx, (uint8_t *)qk, sk, (uint8_t *)qm, sm, (int)M, (int)N, recip_div, st);
    return launch_block128_tile<false, false>(tx, nullptr, nullptr, (uint8_t *)qm, sm, (int)M, (int)N, recip_div, st);
}

extern "C" int qcc_fp8_block128x128(const void *x, int64_t M, int64_t N, int flags, void *q, float *scale, void *stream)
{
    if (M == 0 || N == 0) return 0;
    if (!x || !q || !scale || (flags & ~QCC_RECIP_DIV)) return QCC_ERR_ARG;
    if (M < 0 || N < 0 || M % 128 != 0 || N % 128 != 0 || N > 0x7FFFFF00 || (M / 128) * (N / 128) > 0x7FFFFFFF) return QCC_ERR_SHAPE;
    if (!aligned16(x) || !aligned16(q)) return QCC_ERR_ALIGN;
    const int tiles_n = (int)(N / 128);
    fp8_128x128_kernel<false><<<(unsigned)((M / 128) * tiles_n), 128, 0, (cudaStream_t)stream>>>(
        (const uint16_t *)x, (int)N, tiles_n, (uint8_t *)q, scale, 1.0f, (flags & QCC_RECIP_DIV) ? 1 : 0);
    return (int)cudaGetLastError();
}

extern "C" int qcc_amax_block128x128(const void *x, int64_t M, int64_t N, int mode, float *out, void *stream)
{
    if (M == 0 || N == 0) return 0;
    const int recip_div = take_recip_div(mode);
    if (!x || !out || (mode != QCC_AMAX_RAW && mode != QCC_AMAX_NVFP4_SCALE)) return QCC_ERR_ARG;
    if (M < 0 || N < 0 || M % 128 != 0 || N % 128 != 0 || N > 0x7FFFFF00 || (M / 128) * (N / 128) > 0x7FFFFFFF) return QCC_ERR_SHAPE;
    if (!aligned16(x)) return QCC_ERR_ALIGN;
    const int tiles_n = (int)(N / 128);
    fp8_128x128_kernel<true><<<(unsigned)((M / 128) * tiles_n), 128, 0, (cudaStream_t)stream>>>(
        (const uint16_t *)x, (int)N, tiles_n, nullptr, out, mode == QCC_AMAX_NVFP4_SCALE ? 2688.0f : 1.0f, recip_div);
    return (int)cudaGetLastError();
}
