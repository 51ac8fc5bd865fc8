// mxfp8 (1x32 / 32x1 blocks, e8m0 scales, e4m3 elements) for sm_100a: one tiled kernel for the
// rowwise, the colwise (transposed) and the fused two-direction cast.
//
// Data movement is all TMA: a CTA owns a tile of 128 rows x (128 * G) columns of x.  The tile is
// fetched as 64-column x 32-row boxes (cp.async.bulk.tensor, 128-byte swizzle) that complete on one
// mbarrier per 32-row slab, so warps start as soon as their slab has landed.  Four "row" warps per
// 128-column group quantise along the row (lane = row, four 1x32 blocks each) and four "column"
// warps quantise down the rows (lane = four adjacent columns, one 32x1 block each).  Both write
// their bytes into 128-byte-swizzled staging tiles in shared memory -- every shared access of a
// quarter warp lands in eight distinct 16-byte bank groups -- and the staged tiles leave through
// TMA stores: (32 rows x 128 B) boxes for the rowwise output and, for the transposed output, a
// rank-3 view (m, column % 4, column / 4) of the (N, M) matrix so that one box is the 32 columns
// {4 l + k} a warp produced with all their 128 consecutive m.  Out-of-range parts of edge tiles are
// zero-filled on load and clipped on store by the TMA unit.
//
// Numerics: G = quant_cast_bench/quant_cast_gold/recipes.py of vkuzo/quant_cast_bench.
// mxfp8_f G:561-568, mxfp8_dim_m_f G:656-671, mxfp8_dim_km_f G:701-719, the blocked scale layout
// G:1000-1037 (swizzled variants G:1051-1053, G:1092-1094, G:1134-1139), e8m0 math G:494-558.
#include "common.cuh"
#include "host_util.h"

namespace qcc {

constexpr int MX_THREADS = 256;
constexpr int MX_TILE_M = 128;
constexpr int MX_GROUP_N = 128;          // columns per warp group
constexpr int MX_PANEL_BYTES = 128 * 128; // one 64-column panel of the tile: 128 rows x 128 B
constexpr int MX_SLAB_BYTES = 32 * 128;   // 32 rows of a panel / of a staging tile

template <int RG, int CG>
struct MxSmem {
    static constexpr int G = RG > CG ? RG : CG;
    static constexpr int X_OFF = 0;
    static constexpr int QK_OFF = X_OFF + G * 2 * MX_PANEL_BYTES;
    static constexpr int QM_OFF = QK_OFF + RG * MX_PANEL_BYTES;
    static constexpr int SM_OFF = QM_OFF + CG * MX_PANEL_BYTES;
    static constexpr int BAR_OFF = SM_OFF + CG * 512;
    static constexpr int BYTES = BAR_OFF + G * 4 * 8;
    static constexpr int ALLOC = BYTES + 1024;  // slack to align the base to 1024 B
};

// 32 fp32-scaled values of one row block -> 32 e4m3 bytes, given the four 16-byte chunks
__device__ __forceinline__ void quant_row_block(const uint4 c[4], float rcp, uint4 &o0, uint4 &o1)
{
    o0.x = cvt_fp8x4<QCC_FMT_E4M3>(bf16lo(c[0].x) * rcp, bf16hi(c[0].x) * rcp, bf16lo(c[0].y) * rcp, bf16hi(c[0].y) * rcp);
    o0.y = cvt_fp8x4<QCC_FMT_E4M3>(bf16lo(c[0].z) * rcp, bf16hi(c[0].z) * rcp, bf16lo(c[0].w) * rcp, bf16hi(c[0].w) * rcp);
    o0.z = cvt_fp8x4<QCC_FMT_E4M3>(bf16lo(c[1].x) * rcp, bf16hi(c[1].x) * rcp, bf16lo(c[1].y) * rcp, bf16hi(c[1].y) * rcp);
    o0.w = cvt_fp8x4<QCC_FMT_E4M3>(bf16lo(c[1].z) * rcp, bf16hi(c[1].z) * rcp, bf16lo(c[1].w) * rcp, bf16hi(c[1].w) * rcp);
    o1.x = cvt_fp8x4<QCC_FMT_E4M3>(bf16lo(c[2].x) * rcp, bf16hi(c[2].x) * rcp, bf16lo(c[2].y) * rcp, bf16hi(c[2].y) * rcp);
    o1.y = cvt_fp8x4<QCC_FMT_E4M3>(bf16lo(c[2].z) * rcp, bf16hi(c[2].z) * rcp, bf16lo(c[2].w) * rcp, bf16hi(c[2].w) * rcp);
    o1.z = cvt_fp8x4<QCC_FMT_E4M3>(bf16lo(c[3].x) * rcp, bf16hi(c[3].x) * rcp, bf16lo(c[3].y) * rcp, bf16hi(c[3].y) * rcp);
    o1.w = cvt_fp8x4<QCC_FMT_E4M3>(bf16lo(c[3].z) * rcp, bf16hi(c[3].z) * rcp, bf16lo(c[3].w) * rcp, bf16hi(c[3].w) * rcp);
}

template <int RG, int CG, bool SWZ, bool FLOOR>
__global__ void __launch_bounds__(MX_THREADS)
mxfp8_tile_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_qk,
                  const __grid_constant__ CUtensorMap tm_qm, uint8_t *__restrict__ sk, uint8_t *__restrict__ sm, int M,
                  int N)
{
    using L = MxSmem<RG, CG>;
    constexpr int G = L::G;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem_raw + (base - smem_u32(smem_raw)) + L::BAR_OFF);

    const int tile_n = blockIdx.x, tile_m = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
#pragma unroll
        for (int i = 0; i < G * 4; i++) mbar_init(&bars[i], 1);
        fence_barrier_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
#pragma unroll
        for (int b = 0; b < 4; b++) {
#pragma unroll
            for (int g = 0; g < G; g++) {
                const int col0 = (tile_n * G + g) * MX_GROUP_N;
                if (col0 >= N) continue;
                uint64_t *bar = &bars[g * 4 + b];
                mbar_expect_tx(bar, 2 * MX_SLAB_BYTES);
                uint8_t *dst = smem_raw + (base - smem_u32(smem_raw)) + L::X_OFF + g * 2 * MX_PANEL_BYTES + b * MX_SLAB_BYTES;
                tma_load_2d(dst, &tm_x, bar, col0, tile_m * MX_TILE_M + b * 32);
                tma_load_2d(dst + MX_PANEL_BYTES, &tm_x, bar, col0 + 64, tile_m * MX_TILE_M + b * 32);
            }
        }
    }

    const bool is_row = warp < 4 * RG;
    const int role = is_row ? warp : warp - 4 * RG;
    const int g = role >> 2, b = role & 3;
    const int grp = tile_n * G + g;               // 128-column group index in the whole matrix
    if (grp * MX_GROUP_N >= N) return;            // this group lies entirely right of the matrix
    const uint32_t xs = base + L::X_OFF + g * 2 * MX_PANEL_BYTES;
    const int nb = N >> 5, mb = M >> 5;           // scale columns of the two frames

    mbar_wait(&bars[g * 4 + b], 0, 1u);

    if (is_row) {
        // ------------------------------------------------------------------ along the row
        const int row_t = b * 32 + lane;          // row inside the tile
        const uint32_t key = lane & 7;
        const uint32_t xrow = xs + row_t * 128;
        const uint32_t qrow = base + L::QK_OFF + g * MX_PANEL_BYTES + row_t * 128;
        uint32_t sbytes = 0;
#pragma unroll
        for (int kb = 0; kb < 4; kb++) {
            const uint32_t prow = xrow + (kb >> 1) * MX_PANEL_BYTES;
            const uint32_t j0 = (kb & 1) * 4;
            uint4 c[4];
#pragma unroll
            for (int i = 0; i < 4; i++) c[i] = lds_v4(prow + (((j0 + i) ^ key) << 4));
            uint32_t a0 = 0, a1 = 0;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                a0 = absmax2(absmax2(a0, c[i].x), c[i].y);
                a1 = absmax2(absmax2(a1, c[i].z), c[i].w);
            }
            const float amax = hmax_halves_f32(absmax2(a0, a1));
            const uint32_t e = e8m0_from_amax<FLOOR>(amax);
            const float rcp = e8m0_recip<FLOOR>(e);
            sbytes |= e << (8 * kb);
            uint4 o0, o1;
            quant_row_block(c, rcp, o0, o1);
            sts_v4(qrow + (((2 * kb) ^ key) << 4), o0);
            sts_v4(qrow + (((2 * kb + 1) ^ key) << 4), o1);
        }
        // scales: four consecutive bytes (row, 4 * grp .. 4 * grp + 3) in either layout
        const int R = tile_m * MX_TILE_M + row_t;
        const int C = grp * 4;
        if (SWZ) {
            const uint32_t ncb = (nb + 3) >> 2;
            const size_t off = ((size_t)tile_m * ncb + grp) * 512u + lane * 16u + b * 4u;
            *reinterpret_cast<uint32_t *>(sk + off) = sbytes;
        } else if (R < M) {
            uint8_t *dst = sk + (size_t)R * nb + C;
            if ((nb & 3) == 0) {
                *reinterpret_cast<uint32_t *>(dst) = sbytes;
            } else {
#pragma unroll
                for (int kb = 0; kb < 4; kb++)
                    if (C + kb < nb) dst[kb] = (uint8_t)(sbytes >> (8 * kb));
            }
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0 && tile_m * MX_TILE_M + b * 32 < M) {
            tma_store_2d(&tm_qk, reinterpret_cast<const void *>(smem_raw + (base - smem_u32(smem_raw)) + L::QK_OFF +
                                                               g * MX_PANEL_BYTES + b * MX_SLAB_BYTES),
                         grp * MX_GROUP_N, tile_m * MX_TILE_M + b * 32);
            tma_commit();
            tma_wait_read_all();
        }
    } else {
        // ------------------------------------------------------------------ down the rows
        const uint32_t pbase = xs + (lane >> 4) * MX_PANEL_BYTES + (b * 32) * 128 + (lane & 1) * 8;
        const uint32_t j = (lane & 15) >> 1;
        uint32_t a0 = 0, a1 = 0;
#pragma unroll
        for (int r = 0; r < 32; r++) {
            uint2 w = lds_v2(pbase + r * 128 + ((j ^ (r & 7)) << 4));
            a0 = absmax2(a0, w.x);
            a1 = absmax2(a1, w.y);
        }
        float rcp[4];
        uint32_t e[4];
        {
            const float am[4] = {u2f(a0 << 16), u2f(a0 & 0xFFFF0000u), u2f(a1 << 16), u2f(a1 & 0xFFFF0000u)};
#pragma unroll
            for (int k = 0; k < 4; k++) {
                e[k] = e8m0_from_amax<FLOOR>(am[k]);
                rcp[k] = e8m0_recip<FLOOR>(e[k]);
            }
        }
        uint32_t out[4][8];
#pragma unroll
        for (int w = 0; w < 8; w++) {
            uint2 r0 = lds_v2(pbase + (4 * w + 0) * 128 + ((j ^ ((4 * w + 0) & 7)) << 4));
            uint2 r1 = lds_v2(pbase + (4 * w + 1) * 128 + ((j ^ ((4 * w + 1) & 7)) << 4));
            uint2 r2 = lds_v2(pbase + (4 * w + 2) * 128 + ((j ^ ((4 * w + 2) & 7)) << 4));
            uint2 r3 = lds_v2(pbase + (4 * w + 3) * 128 + ((j ^ ((4 * w + 3) & 7)) << 4));
            out[0][w] = cvt_fp8x4<QCC_FMT_E4M3>(bf16lo(r0.x) * rcp[0], bf16lo(r1.x) * rcp[0], bf16lo(r2.x) * rcp[0], bf16lo(r3.x) * rcp[0]);
            out[1][w] = cvt_fp8x4<QCC_FMT_E4M3>(bf16hi(r0.x) * rcp[1], bf16hi(r1.x) * rcp[1], bf16hi(r2.x) * rcp[1], bf16hi(r3.x) * rcp[1]);
            out[2][w] = cvt_fp8x4<QCC_FMT_E4M3>(bf16lo(r0.y) * rcp[2], bf16lo(r1.y) * rcp[2], bf16lo(r2.y) * rcp[2], bf16lo(r3.y) * rcp[2]);
            out[3][w] = cvt_fp8x4<QCC_FMT_E4M3>(bf16hi(r0.y) * rcp[3], bf16hi(r1.y) * rcp[3], bf16hi(r2.y) * rcp[3], bf16hi(r3.y) * rcp[3]);
        }
        // staging: sub-tile k holds columns {4 l + k}, one 128-byte row per column, swizzled on l
        const uint32_t qms = base + L::QM_OFF + g * MX_PANEL_BYTES;
        const uint32_t key = lane & 7;
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const uint32_t rowp = qms + k * MX_SLAB_BYTES + lane * 128;
            sts_v4(rowp + (((2 * b) ^ key) << 4), make_uint4(out[k][0], out[k][1], out[k][2], out[k][3]));
            sts_v4(rowp + (((2 * b + 1) ^ key) << 4), make_uint4(out[k][4], out[k][5], out[k][6], out[k][7]));
        }
        // scale bytes of this slab into the staging block (layout = the one written to memory)
        uint8_t *sms = smem_raw + (base - smem_u32(smem_raw)) + L::SM_OFF + g * 512;
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const int c = 4 * lane + k;
            const int off = SWZ ? ((c & 31) * 16 + (c >> 5) * 4 + b) : (c * 4 + b);
            sms[off] = (uint8_t)e[k];
        }
        fence_proxy_async();
        named_barrier(1 + g, 128);
        if (lane == 0) {
            tma_store_3d(&tm_qm, reinterpret_cast<const void *>(smem_raw + (base - smem_u32(smem_raw)) + L::QM_OFF +
                                                               g * MX_PANEL_BYTES + b * MX_SLAB_BYTES),
                         tile_m * MX_TILE_M, b, grp * 32);
            tma_commit();
        }
        if (SWZ) {
            // one 512-byte atom: rows = columns of x in this group, 4 scale columns = the 4 slabs
            if (b == 0) {
                const uint32_t ncb = (mb + 3) >> 2;
                const size_t off = ((size_t)grp * ncb + tile_m) * 512u + lane * 16u;
                *reinterpret_cast<uint4 *>(sm + off) = *reinterpret_cast<const uint4 *>(sms + lane * 16);
            }
        } else {
            const int c = b * 32 + lane;            // column inside the group
            const int Cn = grp * MX_GROUP_N + c;
            if (Cn < N) {
                const uint32_t v = *reinterpret_cast<const uint32_t *>(sms + c * 4);
                uint8_t *dst = sm + (size_t)Cn * mb + tile_m * 4;
                if ((mb & 3) == 0) {
                    *reinterpret_cast<uint32_t *>(dst) = v;
                } else {
#pragma unroll
                    for (int kk = 0; kk < 4; kk++)
                        if (tile_m * 4 + kk < mb) dst[kk] = (uint8_t)(v >> (8 * kk));
                }
            }
        }
        if (lane == 0) tma_wait_read_all();
    }
}

template <int RG, int CG, bool SWZ, bool FLOOR>
static int launch_mx(const CUtensorMap &tx, const CUtensorMap &tqk, const CUtensorMap &tqm, uint8_t *sk, uint8_t *sm,
                     int M, int N, cudaStream_t st)
{
    using L = MxSmem<RG, CG>;
    auto kern = mxfp8_tile_kernel<RG, CG, SWZ, FLOOR>;
    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::ALLOC);
        if (e != cudaSuccess) return (int)e;
        configured[dev] = true;
    }
    dim3 grid((unsigned)((N + L::G * MX_GROUP_N - 1) / (L::G * MX_GROUP_N)), (unsigned)((M + MX_TILE_M - 1) / MX_TILE_M));
    kern<<<grid, MX_THREADS, L::ALLOC, st>>>(tx, tqk, tqm, sk, sm, M, N);
    return (int)cudaGetLastError();
}

}  // namespace qcc

using namespace qcc;

extern "C" int qcc_mxfp8_device_error(unsigned int *out) { return read_clear_device_error(out); }

extern "C" int qcc_mxfp8(const void *x, int64_t M, int64_t N, int flags, void *qk, void *sk, void *qm, void *sm,
                         void *stream)
{
    const bool row = flags & QCC_ROWWISE, col = flags & QCC_COLWISE;
    if (M == 0 || N == 0) return 0;
    if (!x || (!row && !col) || (flags & ~(QCC_ROWWISE | QCC_COLWISE | QCC_SWIZZLE | QCC_FLOOR))) return QCC_ERR_ARG;
    if ((row && (!qk || !sk)) || (col && (!qm || !sm))) return QCC_ERR_ARG;
    if (M < 0 || N < 0 || M > 0x7FFFFF00 || N > 0x7FFFFF00) return QCC_ERR_SHAPE;
    if (N % 32 != 0 || (col && M % 32 != 0)) return QCC_ERR_SHAPE;
    if (!aligned16(x) || (row && !aligned16(qk)) || (col && !aligned16(qm))) return QCC_ERR_ALIGN;
    if ((row && !aligned16(sk)) || (col && !aligned16(sm))) return QCC_ERR_ALIGN;
    if (M == 0 || N == 0) return 0;
    if ((M + 127) / 128 > 65535) return QCC_ERR_SHAPE;
    cudaStream_t st = (cudaStream_t)stream;

    CUtensorMap tx, tqk, tqm;
    {
        uint64_t dims[2] = {(uint64_t)N, (uint64_t)M};
        uint64_t strides[1] = {(uint64_t)N * 2};
        uint32_t box[2] = {64, 32};
        int e = make_tensor_map(&tx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (e) return e;
    }
    tqk = tx;
    tqm = tx;
    if (row) {
        uint64_t dims[2] = {(uint64_t)N, (uint64_t)M};
        uint64_t strides[1] = {(uint64_t)N};
        uint32_t box[2] = {128, 32};
        int e = make_tensor_map(&tqk, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, qk, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (e) return e;
    }
    if (col) {
        // (N, M) bytes seen as (column / 4, column % 4, m): a box is 32 columns of equal residue
        uint64_t dims[3] = {(uint64_t)M, 4, (uint64_t)N / 4};
        uint64_t strides[2] = {(uint64_t)M, (uint64_t)M * 4};
        uint32_t box[3] = {128, 1, 32};
        int e = make_tensor_map(&tqm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, qm, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (e) return e;
    }
    const bool swz = flags & QCC_SWIZZLE, fl = flags & QCC_FLOOR;
    uint8_t *skp = (uint8_t *)sk, *smp = (uint8_t *)sm;
#define QCC_MX(RG, CG)                                                                                         \
    (swz ? (fl ? launch_mx<RG, CG, true, true>(tx, tqk, tqm, skp, smp, (int)M, (int)N, st)                     \
               : launch_mx<RG, CG, true, false>(tx, tqk, tqm, skp, smp, (int)M, (int)N, st))                   \
         : (fl ? launch_mx<RG, CG, false, true>(tx, tqk, tqm, skp, smp, (int)M, (int)N, st)                    \
               : launch_mx<RG, CG, false, false>(tx, tqk, tqm, skp, smp, (int)M, (int)N, st)))
    if (row && col) return QCC_MX(1, 1);
    if (row) return QCC_MX(2, 0);
    return QCC_MX(0, 2);
#undef QCC_MX
}
