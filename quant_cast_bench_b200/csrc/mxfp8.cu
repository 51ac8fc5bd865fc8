// mxfp8 (1x32 / 32x1 blocks, e8m0 scales, e4m3 elements) for sm_100a.
//
// Two kernels:
//
//  * rowwise only: a flat stream.  A thread owns one 1x32 block (four 16-byte loads, two 16-byte
//    stores, one scale byte); x, q and the plain scales are addressed by the flat block index.
//
//  * colwise (transposed) and the fused two-direction cast: a one-shot tile kernel, one CTA of
//    four warps per 64-row x 128-column tile of x and five to six CTAs resident per SM, so that
//    loads, conversion and stores of different tiles overlap the way they do in a plain streaming
//    kernel.  The tile arrives by TMA (two 64-column x 64-row boxes, 128-byte swizzle, one
//    mbarrier).  Two "row" warps quantise along the row (lane = row of a 32-row slab, four 1x32
//    blocks each) and two "column" warps quantise down the rows (lane = four adjacent columns of a
//    slab, one 32x1 block each, held in registers).  Both write their bytes into swizzled staging
//    tiles in shared memory -- every shared access of a quarter warp lands in eight distinct
//    16-byte bank groups -- and the staged tiles leave as coalesced 16-byte global stores, a
//    quarter warp per 128-byte row segment of the rowwise output and four lanes per 64-byte row
//    segment of the transposed output.  (Measured on B200: TMA stores top out near 6.0 TB/s where
//    plain stores reach 7.2 TB/s, and a persistent one-CTA-per-SM pipeline of the same work was
//    20 % slower than this one-shot grid.)  Out-of-range parts of edge tiles are zero-filled by
//    the TMA load and masked on store.  The wait on the mbarrier is bounded and records an error
//    code instead of hanging.
//
// Numerics: G = quant_cast_bench/quant_cast_gold/recipes.py of vkuzo/quant_cast_bench.
// mxfp8_f G:561-568, mxfp8_dim_m_f G:656-671, mxfp8_dim_km_f G:701-719, the blocked scale layout
// G:1000-1037 (swizzled variants G:1051-1053, G:1092-1094, G:1134-1139), e8m0 math G:494-558.
#include "common.cuh"
#include "host_util.h"
#include "xchg.cuh"

namespace qcc {

// ---------------------------------------------------------------------------------------------
// rowwise stream
// ---------------------------------------------------------------------------------------------
#ifndef QCC_RS_THREADS
#define QCC_RS_THREADS 256
#endif
#ifndef QCC_RS_UNROLL
#define QCC_RS_UNROLL 2
#endif
constexpr int RS_THREADS = QCC_RS_THREADS;
constexpr int RS_UNROLL = QCC_RS_UNROLL;

// Tables of the token-group casts (all null for the plain casts).  Rows are rows of the OUTPUT frame.
//   row_map[r]  row -> row inside the 128-padded, stacked groups (-1: not in any group)
//   mb_a[b]     32-row block b -> byte offset of its scale column inside its group's blocked matrix
//               (group base + (column / 4) * 512 + column % 4), 0xFFFFFFFF: not in any group
//   mb_b[b]     bytes between consecutive 128-row blocks of that group's blocked matrix
// and, when the cast also pads every group to a multiple of 32 rows (the input then has src_rows unpadded rows):
//   blk_src[b]    first source row of output block b (src_rows, i.e. past the end, where there is none)
//   blk_valid[b]  how many of its 32 rows come from the input; the others are zero
struct GroupTables {
    const int32_t *row_map;
    const uint32_t *mb_a;
    const uint32_t *mb_b;
    const int32_t *blk_src;
    const int32_t *blk_valid;
    int src_rows;
    // stacked matrices (per-expert weights) cast by one launch: rows of one matrix (a multiple of 128) and the bytes
    // of one matrix's transposed scale grid; 0 when x is a single matrix
    int rows_per_mat;
    uint32_t sm_bytes_per_mat;
};

// Scale byte of block `bi` of the flat stream: plain (M, N/32) or blocked.  Called by every lane of the warp.
template <bool SWZ>
__device__ __forceinline__ void stream_scale_store(uint8_t *__restrict__ s, uint32_t bi, bool ok, uint32_t e, uint32_t nb,
                                                   const FastDiv32 &div_nb, const int32_t *__restrict__ row_map)
{
    if (!SWZ) {
        if (ok) s[bi] = (uint8_t)e;
    } else if ((nb & 3) == 0) {
        // four consecutive lanes hold the four scale columns of one (row, column block): one 4-byte store
        uint32_t v = e | (__shfl_down_sync(0xFFFFFFFFu, e, 1) << 8);
        v |= __shfl_down_sync(0xFFFFFFFFu, v, 2) << 16;
        if (ok && (threadIdx.x & 3) == 0) {
            uint32_t row = div_nb.div(bi);
            const uint32_t cb = bi - row * nb;
            int32_t dst = (int32_t)row;
            if (row_map) dst = __ldg(row_map + row);      // token groups: row inside the padded, stacked groups
            if (dst >= 0) *reinterpret_cast<uint32_t *>(s + blocked_offset((uint32_t)dst, cb, nb >> 2)) = v;
        }
    } else if (ok) {
        uint32_t row = div_nb.div(bi);
        const uint32_t cb = bi - row * nb;
        int32_t dst = (int32_t)row;
        if (row_map) dst = __ldg(row_map + row);
        if (dst >= 0) s[blocked_offset((uint32_t)dst, cb, (nb + 3) >> 2)] = (uint8_t)e;
    }
}

// Where the cast also delivers max |x| (every block maximum is in registers anyway).  AMAX 1: ctl = two zeroed
// control words (ticket, running maximum) and out receives the raw amax from the CTA that finishes last.  AMAX 2:
// ctl = this rank's amax-exchange state, whose accumulator the CTAs merge into; the first consumer publishes it.
struct AmaxSink {
    uint32_t *ctl;
    float *out;
};

// AMAX: 0 the cast alone; 1 / 2 also the tensor's amax (see AmaxSink).
template <bool SWZ, bool FLOOR, int AMAX = 0>
#ifndef QCC_RS_MINCTAS
#define QCC_RS_MINCTAS 5
#endif
__global__ void __launch_bounds__(RS_THREADS, QCC_RS_MINCTAS)    // (the amax forms would take 52 registers: 4 CTAs per SM instead of 5)
mxfp8_rowwise_stream_kernel(const uint16_t *__restrict__ x, uint32_t nblocks, uint32_t nb, FastDiv32 div_nb,
                            uint8_t *__restrict__ q, uint8_t *__restrict__ s, GroupTables g, AmaxSink sink)
{
    const int32_t *__restrict__ row_map = g.row_map;
    const uint4 *xv = reinterpret_cast<const uint4 *>(x);
    uint4 *qv = reinterpret_cast<uint4 *>(q);
    const uint32_t base = blockIdx.x * (RS_THREADS * RS_UNROLL) + threadIdx.x;
    uint32_t seen = 0;
    if (AMAX == 2) {
        pdl_trigger();      // the exchange warp (and the cast behind it) may be launched once every CTA has got this far
        seen = xchg_producer_begin(sink.ctl);
    }
    uint4 c[RS_UNROLL][4];
#pragma unroll
    for (int u = 0; u < RS_UNROLL; u++) {
        const uint32_t bi = base + u * RS_THREADS;
        size_t src = bi;                      // block index inside x
        bool have = bi < nblocks;
        if (have && g.blk_src) {              // padded token groups: the row comes from another place, or is padding
            const uint32_t row = div_nb.div(bi);
            const uint32_t rb = row >> 5, ri = row & 31u;
            have = (int32_t)ri < __ldg(g.blk_valid + rb);
            src = (size_t)((uint32_t)__ldg(g.blk_src + rb) + ri) * nb + (bi - row * nb);
        }
        if (have) {
#pragma unroll
            for (int i = 0; i < 4; i++) c[u][i] = ld_v4(xv + 4 * src + i);
        } else {
#pragma unroll
            for (int i = 0; i < 4; i++) c[u][i] = make_uint4(0, 0, 0, 0);
        }
    }
    uint32_t mx = 0;
#pragma unroll
    for (int u = 0; u < RS_UNROLL; u++) {
        const uint32_t bi = base + u * RS_THREADS;
        const bool ok = bi < nblocks;
        const float am = amax_of_block(c[u]);
        if (AMAX) mx = max(mx, f2u(am));          // non-negative floats order like their bits
        const uint32_t e = e8m0_from_amax<FLOOR>(am);
        const float rcp = e8m0_recip<FLOOR>(e);
        uint4 o0, o1;
        quant_row_block(c[u], rcp, o0, o1);
        if (ok) {
            st_out(qv + 2 * (size_t)bi, o0);
            st_out(qv + 2 * (size_t)bi + 1, o1);
        }
        stream_scale_store<SWZ>(s, bi, ok, e, nb, div_nb, row_map);
    }
    if (AMAX) {
        __shared__ uint32_t red[RS_THREADS / 32];
        if (AMAX == 2) {
            xchg_producer_merge(sink.ctl, mx, seen, red);
        } else if (cta_max_ticket(mx, sink.ctl, red)) {
            if (threadIdx.x == 0 && sink.out) sink.out[0] = u2f(mx);
        }
    }
}

// mxfp4 (gold mxfp4_f G:607-617): the same 1x32 blocks and RCEIL e8m0 scale, descaled by 6 instead of 448,
// elements as e2m1 packed two per byte (even element in the low nibble).
template <bool SWZ>
__global__ void __launch_bounds__(RS_THREADS)
mxfp4_rowwise_stream_kernel(const uint16_t *__restrict__ x, uint32_t nblocks, uint32_t nb, FastDiv32 div_nb,
                            uint8_t *__restrict__ q, uint8_t *__restrict__ s)
{
    const uint4 *xv = reinterpret_cast<const uint4 *>(x);
    uint4 *qv = reinterpret_cast<uint4 *>(q);
    const uint32_t bi = blockIdx.x * RS_THREADS + threadIdx.x;
    const bool ok = bi < nblocks;
    uint4 c[4] = {};
    if (ok) {
#pragma unroll
        for (int i = 0; i < 4; i++) c[i] = ld_v4(xv + 4 * (size_t)bi + i);
    }
    const uint32_t e = e8m0_rceil_of(amax_of_block(c), 0x3E2AAAABu);   // fp32(1 / 6)
    const float rcp = e8m0_recip<false>(e);
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        float v[8] = {bf16lo(c[i].x) * rcp, bf16hi(c[i].x) * rcp, bf16lo(c[i].y) * rcp, bf16hi(c[i].y) * rcp,
                      bf16lo(c[i].z) * rcp, bf16hi(c[i].z) * rcp, bf16lo(c[i].w) * rcp, bf16hi(c[i].w) * rcp};
        o[i] = cvt_e2m1x8(v);
    }
    if (ok) st_out(qv + bi, make_uint4(o[0], o[1], o[2], o[3]));
    stream_scale_store<SWZ>(s, bi, ok, e, nb, div_nb, nullptr);
}

// ---------------------------------------------------------------------------------------------
// one-shot tile kernel: one CTA per 64-row x 128-column tile, many CTAs resident per SM
// ---------------------------------------------------------------------------------------------
// Tile order.  CTAs are dispatched in tile-number order and those resident at any moment work on
// consecutive numbers, so the numbering decides which cache lines are touched together.  Tiles are
// numbered down groups of QCC_MX_GROUP_M tile rows, column by column; with the default of 1 the
// sweep is row-major, which measured best on B200 (the 128-byte segments of x rows and of the
// rowwise output written at the same time are neighbours; taller groups favour the transposed
// output instead).

#ifndef QCC_MX_GROUP_M
#define QCC_MX_GROUP_M 1
#endif
__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int &tile_m, int &tile_n)
{
    constexpr int GM = QCC_MX_GROUP_M;
    const int per_group = GM * tiles_n;
    const int g = t / per_group;
    const int r = t - g * per_group;
    const int h = min(GM, tiles_m - g * GM);
    tile_n = r / h;
    tile_m = g * GM + (r - tile_n * h);
}

constexpr int T64_ROWS = 64;
constexpr int T64_PANEL = T64_ROWS * 128;          // one 64-column panel: 64 rows x 128 B

template <bool DO_K, bool DO_M>
struct T64 {
    static constexpr int THREADS = 32 * ((DO_K ? 2 : 0) + (DO_M ? 2 : 0));
    static constexpr int MIN_CTAS = DO_K ? (DO_M ? 6 : 10) : 8;               // register cap: measured best on B200
    static constexpr int X_OFF = 0;
    static constexpr int QK_OFF = 2 * T64_PANEL;                              // 64 rows x 128 B
    static constexpr int QM_OFF = QK_OFF + (DO_K ? T64_ROWS * 128 : 0);       // 4 sub-tiles x 32 rows x 64 B
    static constexpr int SM_OFF = QM_OFF + (DO_M ? 4 * 32 * 64 : 0);          // 128 columns x 2 scale bytes
    static constexpr int BAR_OFF = SM_OFF + 256;
    static constexpr int BYTES = BAR_OFF + 16;
    static constexpr int ALLOC = BYTES + 1024;
};

// B32: one scale per 32x32 block (gold mxfp8_32x32_f and its layouts, G:753-984): the block maximum is the
// maximum over the 32 lanes of a row warp, or over the eight lanes (32 columns) of a column warp; both give the
// same byte, which is then stored once per row / per column in the expanded 1x32 and 32x1 scale frames.  The
// rowwise form (DO_M false) can also write the transposed frame's scales (sm non-null) without the transposed data.
// PAD (token groups padded by the cast itself): the two 32-row slabs of a tile are fetched from their own source rows
// and the rows past a group's end read as zero.
// BATCHED (blocked scales, no groups): x is E matrices of g.rows_per_mat rows stacked; loads and rowwise outputs
// address the stack as one tall matrix (its blocked scale grid is the E grids one after the other), the transposed
// outputs go to matrix e's own (N, rows_per_mat) frame and scale grid.
template <bool DO_K, bool DO_M, bool SWZ, bool FLOOR, bool B32, bool PAD, bool BATCHED>
__global__ void __launch_bounds__(T64<DO_K, DO_M>::THREADS, T64<DO_K, DO_M>::MIN_CTAS)
mxfp8_tile64_kernel(const __grid_constant__ CUtensorMap tm_x, uint8_t *__restrict__ qk, uint8_t *__restrict__ sk,
                    uint8_t *__restrict__ qm, uint8_t *__restrict__ sm, int M, int N, int tiles_m, int tiles_n, GroupTables g)
{
    using L = T64<DO_K, DO_M>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *sbase = smem_raw + (base - smem_u32(smem_raw));
    uint64_t *bar = reinterpret_cast<uint64_t *>(sbase + L::BAR_OFF);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int tile_m, tile_n;
    tile_coords((int)blockIdx.x, tiles_m, tiles_n, tile_m, tile_n);

    if (threadIdx.x == 0) {
        mbar_init(bar, 1);
        fence_barrier_init();
    }
    __syncthreads();
    const int nblk = (M + 31) >> 5;
    if (threadIdx.x == 0) {
        mbar_expect_tx(bar, 2 * T64_PANEL);
        if (PAD) {
            // padded token groups: each 32-row slab of the tile has its own source rows (the tensor map's box is 32 rows)
#pragma unroll
            for (int sl = 0; sl < 2; sl++) {
                const int ob = tile_m * 2 + sl;
                const int src = ob < nblk ? __ldg(g.blk_src + ob) : g.src_rows;   // past the end: zero fill
                tma_load_2d(sbase + L::X_OFF + sl * 4096, &tm_x, bar, tile_n * 128, src);
                tma_load_2d(sbase + L::X_OFF + T64_PANEL + sl * 4096, &tm_x, bar, tile_n * 128 + 64, src);
            }
        } else {
            tma_load_2d(sbase + L::X_OFF, &tm_x, bar, tile_n * 128, tile_m * T64_ROWS);
            tma_load_2d(sbase + L::X_OFF + T64_PANEL, &tm_x, bar, tile_n * 128 + 64, tile_m * T64_ROWS);
        }
    }
    const bool is_row = DO_K && warp < 2;
    const int b = warp & 1;                        // 32-row slab of this warp
    const int nb = N >> 5, mb = M >> 5;
    const uint32_t xs = base + L::X_OFF;
    // rows of this warp's slab that hold input (the rest of a padded token group's last block reads as zero)
    int valid = 32;
    if (PAD) valid = (tile_m * 2 + b) < nblk ? __ldg(g.blk_valid + tile_m * 2 + b) : 0;
    mbar_wait(bar, 0, 4u);

    if (is_row) {
        // ------------------------------------------------------------------ along the row
        const int row_t = b * 32 + lane;
        const uint32_t key = lane & 7;
        const uint32_t xrow = xs + row_t * 128;
        const uint32_t qrow = base + L::QK_OFF + row_t * 128;
        uint32_t sbytes = 0;
#pragma unroll
        for (int kb = 0; kb < 4; kb++) {
            const uint32_t prow = xrow + (kb >> 1) * T64_PANEL;
            const uint32_t j0 = (kb & 1) * 4;
            uint4 c[4];
#pragma unroll
            for (int i = 0; i < 4; i++) c[i] = lds_v4(prow + (((j0 + i) ^ key) << 4));
            if (PAD && lane >= valid) c[0] = c[1] = c[2] = c[3] = make_uint4(0, 0, 0, 0);
            float am = amax_of_block(c);
            if (B32) am = u2f(__reduce_max_sync(0xFFFFFFFFu, f2u(am)));   // non-negative floats order like integers
            const uint32_t e = e8m0_from_amax<FLOOR>(am);
            const float rcp = e8m0_recip<FLOOR>(e);
            sbytes |= e << (8 * kb);
            uint4 o0, o1;
            quant_row_block(c, rcp, o0, o1);
            sts_v4(qrow + (((2 * kb) ^ key) << 4), o0);
            sts_v4(qrow + (((2 * kb + 1) ^ key) << 4), o1);
        }
        __syncwarp();
        {
            const int j = lane & 7;
            const int col = tile_n * 128 + j * 16;
            const uint32_t slab = base + L::QK_OFF + b * 32 * 128;
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const int r = i * 4 + (lane >> 3);
                const int R = tile_m * T64_ROWS + b * 32 + r;
                const uint4 v = lds_v4(slab + r * 128 + ((j ^ (r & 7)) << 4));
                if (R < M && col < N) *reinterpret_cast<uint4 *>(qk + (size_t)R * N + col) = v;
            }
        }
        const int R = tile_m * T64_ROWS + row_t;
        const int C = tile_n * 4;
        if (SWZ) {
            const uint32_t ncb = (nb + 3) >> 2;
            int32_t Rd = R;
            if (g.row_map) Rd = R < M ? __ldg(g.row_map + R) : -1;   // token groups: row inside the stacked groups
            if (Rd >= 0) {
                const uint32_t rr = (uint32_t)Rd & 127u;
                const size_t off = ((size_t)(Rd >> 7) * ncb + tile_n) * 512u + (rr & 31u) * 16u + (rr >> 5) * 4u;
                *reinterpret_cast<uint32_t *>(sk + off) = sbytes;  // padding rows carry zeros (zero-filled x)
            }
        } else if (B32) {
            // plain (M / 32, N / 32) grid: one writer per 32-row slab
            if (lane == 0 && R < M) {
                uint8_t *dst = sk + (size_t)(R >> 5) * nb + C;
#pragma unroll
                for (int kb = 0; kb < 4; kb++)
                    if (C + kb < nb) dst[kb] = (uint8_t)(sbytes >> (8 * kb));
            }
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
        if (B32 && SWZ && !DO_M && sm != nullptr) {
            // scales of the transposed frame (N, M / 32), expanded over the 32 columns of each block
            const uint32_t ncb_m = (uint32_t)(mb + 3) >> 2;
            const uint32_t mblk = (uint32_t)tile_m * 2 + b;
            const uint32_t byte = (sbytes >> (8 * (lane >> 3))) & 0xFFu;
            const size_t atom = ((size_t)tile_n * ncb_m + (mblk >> 2)) * 512u + (mblk & 3u);
#pragma unroll
            for (int cc = 0; cc < 4; cc++) {
                const uint32_t c = 4 * lane + cc;
                sm[atom + (c & 31u) * 16u + (c >> 5) * 4u] = (uint8_t)byte;
            }
        }
    } else if constexpr (DO_M) {
        // ------------------------------------------------------------------ down the rows
        const uint32_t pbase = xs + (lane >> 4) * T64_PANEL + (b * 32) * 128 + (lane & 1) * 8;
        const uint32_t j = (lane & 15) >> 1;
        uint2 w[32];
        uint32_t a0 = 0, a1 = 0;
#pragma unroll
        for (int r = 0; r < 32; r++) {
            w[r] = lds_v2(pbase + r * 128 + ((j ^ (r & 7)) << 4));
            if (PAD && r >= valid) w[r] = make_uint2(0, 0);
            a0 = absmax2_acc(a0, w[r].x);
            a1 = absmax2_acc(a1, w[r].y);
        }
        float rcp[4];
        uint32_t e[4];
        {
            float am[4] = {u2f(a0 << 16), u2f(a0 & 0xFFFF0000u), u2f(a1 << 16), u2f(a1 & 0xFFFF0000u)};
            if (B32) {
                // 32 columns = this lane's four and those of the seven other lanes of its group of eight
                uint32_t m = max(max(f2u(am[0]), f2u(am[1])), max(f2u(am[2]), f2u(am[3])));
                m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, 1));
                m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, 2));
                m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, 4));
                am[0] = am[1] = am[2] = am[3] = u2f(m);
            }
#pragma unroll
            for (int kk = 0; kk < 4; kk++) {
                e[kk] = e8m0_from_amax<FLOOR>(am[kk]);
                rcp[kk] = e8m0_recip<FLOOR>(e[kk]);
            }
        }
        // staging: sub-tile kk holds columns {4 l + kk}, one 64-byte row (the tile's 64 m) per column;
        // 16-byte chunk c of row l sits at position c ^ ((l >> 1) & 3)
        const uint32_t qms = base + L::QM_OFF;
        const uint32_t key = (lane >> 1) & 3;
#pragma unroll
        for (int kk = 0; kk < 4; kk++) {
            uint32_t o[8];
#pragma unroll
            for (int q4 = 0; q4 < 8; q4++) {
                const uint2 r0 = w[4 * q4], r1 = w[4 * q4 + 1], r2 = w[4 * q4 + 2], r3 = w[4 * q4 + 3];
                const float sc = rcp[kk];
                if (kk == 0)
                    o[q4] = scale_cvt_fp8x4<QCC_FMT_E4M3>(bf16lo(r0.x), bf16lo(r1.x), bf16lo(r2.x), bf16lo(r3.x), sc);
                else if (kk == 1)
                    o[q4] = scale_cvt_fp8x4<QCC_FMT_E4M3>(bf16hi(r0.x), bf16hi(r1.x), bf16hi(r2.x), bf16hi(r3.x), sc);
                else if (kk == 2)
                    o[q4] = scale_cvt_fp8x4<QCC_FMT_E4M3>(bf16lo(r0.y), bf16lo(r1.y), bf16lo(r2.y), bf16lo(r3.y), sc);
                else
                    o[q4] = scale_cvt_fp8x4<QCC_FMT_E4M3>(bf16hi(r0.y), bf16hi(r1.y), bf16hi(r2.y), bf16hi(r3.y), sc);
            }
            const uint32_t rowp = qms + kk * 2048 + lane * 64;
            sts_v4(rowp + (((2 * b) ^ key) << 4), make_uint4(o[0], o[1], o[2], o[3]));
            sts_v4(rowp + (((2 * b + 1) ^ key) << 4), make_uint4(o[4], o[5], o[6], o[7]));
        }
        uint8_t *sms = sbase + L::SM_OFF;
#pragma unroll
        for (int kk = 0; kk < 4; kk++) sms[(4 * lane + kk) * 2 + b] = (uint8_t)e[kk];
        named_barrier(1, 64);
        // frame of the transposed outputs: the whole matrix, or matrix e of a stack
        int tm = tile_m, Mq = M;
        uint8_t *qmp = qm, *smp = sm;
        if (BATCHED) {
            const int tpm = g.rows_per_mat >> 6;
            const int e = tile_m / tpm;
            tm = tile_m - e * tpm;
            Mq = g.rows_per_mat;
            qmp = qm + (size_t)e * N * Mq;
            smp = sm + (size_t)e * g.sm_bytes_per_mat;
        }
        // write-out: col warp b takes sub-tiles 2b and 2b+1; four lanes move one 64-byte row segment
        {
            const int jj = lane & 3;
            const int mcol = tm * T64_ROWS + jj * 16;
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const int kk = 2 * b + (i >> 2);
                const int l = (i & 3) * 8 + (lane >> 2);
                const int Cn = tile_n * 128 + 4 * l + kk;
                const uint4 v = lds_v4(qms + kk * 2048 + l * 64 + ((jj ^ ((l >> 1) & 3)) << 4));
                if (Cn < N && mcol < Mq) *reinterpret_cast<uint4 *>(qmp + (size_t)Cn * Mq + mcol) = v;
            }
        }
        // scales: thread (b, lane) writes the two bytes (m-blocks 2 tile_m, 2 tile_m + 1) of columns 2t, 2t+1
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int c = (b * 32 + lane) * 2 + h;
            const int Cn = tile_n * 128 + c;
            const uint16_t v = *reinterpret_cast<const uint16_t *>(sms + c * 2);
            if (SWZ && g.mb_a) {
                // token groups: every 32-row block of x has its own place (group base, column inside the group)
                const int m0 = tile_m * 2;
                const uint32_t a0 = m0 < mb ? __ldg(g.mb_a + m0) : 0xFFFFFFFFu;
                const uint32_t a1 = m0 + 1 < mb ? __ldg(g.mb_a + m0 + 1) : 0xFFFFFFFFu;
                const uint32_t b0 = m0 < mb ? __ldg(g.mb_b + m0) : 0u, b1 = m0 + 1 < mb ? __ldg(g.mb_b + m0 + 1) : 0u;
                const uint32_t lane_off = (c & 31) * 16u + (c >> 5) * 4u;
                if (Cn < N) {
                    if (a0 != 0xFFFFFFFFu && a1 == a0 + 1u && b1 == b0 && (a0 & 1u) == 0u) {
                        // both blocks in one group, in neighbouring scale columns of one atom: one 2-byte store
                        *reinterpret_cast<uint16_t *>(sm + (size_t)a0 + (size_t)tile_n * b0 + lane_off) = v;
                    } else {
                        if (a0 != 0xFFFFFFFFu) sm[(size_t)a0 + (size_t)tile_n * b0 + lane_off] = (uint8_t)v;
                        if (a1 != 0xFFFFFFFFu) sm[(size_t)a1 + (size_t)tile_n * b1 + lane_off] = (uint8_t)(v >> 8);
                    }
                }
            } else if (SWZ) {
                const uint32_t ncb = (uint32_t)((Mq >> 5) + 3) >> 2;
                const size_t off = ((size_t)tile_n * ncb + (tm >> 1)) * 512u + (c & 31) * 16u + (c >> 5) * 4u + (tm & 1) * 2u;
                *reinterpret_cast<uint16_t *>(smp + off) = v;      // padding columns carry zeros (zero-filled x)
            } else if (Cn < N) {
                uint8_t *dst = sm + (size_t)Cn * mb + tile_m * 2;
                if ((mb & 1) == 0) {
                    *reinterpret_cast<uint16_t *>(dst) = v;       // both blocks inside, address even
                } else {
                    if (tile_m * 2 < mb) dst[0] = (uint8_t)v;
                    if (tile_m * 2 + 1 < mb) dst[1] = (uint8_t)(v >> 8);
                }
            }
        }
    }
}

template <bool DO_K, bool DO_M, bool SWZ, bool FLOOR, bool B32 = false, bool PAD = false, bool BATCHED = false>
static int launch_t64(const CUtensorMap &tx, uint8_t *qk, uint8_t *sk, uint8_t *qm, uint8_t *sm, int M, int N, cudaStream_t st,
                      GroupTables g)
{
    using L = T64<DO_K, DO_M>;
    auto kern = mxfp8_tile64_kernel<DO_K, DO_M, SWZ, FLOOR, B32, PAD, BATCHED>;
    static PerDeviceFlag configured;          // one per template instance
    int dev = current_device_slot();
    if (dev < 0) return QCC_ERR_ARG;
    if (!configured.get(dev)) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::ALLOC);
        if (e != cudaSuccess) return (int)e;
        e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
        if (e != cudaSuccess) return (int)e;
        configured.set(dev);
    }
    // With blocked scales the tiles must cover whole 128-row atoms so that the padding gets its zeros:
    // a tile that lies entirely below the matrix loads zero-filled data and stores nothing but scales.
    const int tiles_n = (N + 127) / 128;
    // (the token-group casts clear their scale buffers up front instead)
    const int tiles_m = (SWZ && !g.row_map) ? 2 * ((M + 127) / 128) : (M + T64_ROWS - 1) / T64_ROWS;
    const long long num_tiles = (long long)tiles_n * tiles_m;
    if (num_tiles > 0x7FFFFFFF) return QCC_ERR_SHAPE;
    kern<<<(unsigned)num_tiles, L::THREADS, L::ALLOC, st>>>(tx, qk, sk, qm, sm, M, N, tiles_m, tiles_n, g);
    return (int)cudaGetLastError();
}

}  // namespace qcc

using namespace qcc;

extern "C" int qcc_mxfp8_device_error(unsigned int *out) { return read_clear_device_error(out); }

static int mxfp8_entry(const void *x, int64_t M, int64_t N, int flags, void *qk, void *sk, void *qm, void *sm,
                       void *stream, GroupTables g, int amax_mode = 0, const AmaxSink *sink_p = nullptr)
{
    AmaxSink sink{};
    if (amax_mode) sink = *sink_p;
    const bool row = flags & QCC_ROWWISE, col = flags & QCC_COLWISE;
    if (M == 0 || N == 0) return 0;
    if (!x || (!row && !col) || (flags & ~(QCC_ROWWISE | QCC_COLWISE | QCC_SWIZZLE | QCC_FLOOR | QCC_BLOCK32))) return QCC_ERR_ARG;
    const bool b32 = flags & QCC_BLOCK32;
    // 32x32 blocks: the transposed data may be left out when only its scales are wanted (with the rowwise outputs)
    if ((row && (!qk || !sk)) || (col && (!sm || (!qm && !(b32 && row))))) return QCC_ERR_ARG;
    if (b32 && ((flags & QCC_FLOOR) || g.row_map || (col && !(flags & QCC_SWIZZLE)))) return QCC_ERR_ARG;
    if (b32 && M % 32 != 0) return QCC_ERR_SHAPE;
    if (M < 0 || N < 0 || M > 0x7FFFFF00 || N > 0x7FFFFF00) return QCC_ERR_SHAPE;
    if (N % 32 != 0 || (col && M % 32 != 0)) return QCC_ERR_SHAPE;
    if (!aligned16(x) || (row && !aligned16(qk)) || (col && qm && !aligned16(qm))) return QCC_ERR_ALIGN;
    if ((row && !aligned16(sk)) || (col && !aligned16(sm))) return QCC_ERR_ALIGN;
    cudaStream_t st = (cudaStream_t)stream;
    const bool swz = flags & QCC_SWIZZLE, fl = flags & QCC_FLOOR;
    uint8_t *skp = (uint8_t *)sk, *smp = (uint8_t *)sm;

    if (b32) {
        CUtensorMap t64;
        uint64_t dims[2] = {(uint64_t)N, (uint64_t)M};
        uint64_t strides[1] = {(uint64_t)N * 2};
        uint32_t box[2] = {64, 64};
        int e = make_tensor_map(&t64, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (e) return e;
        uint8_t *qkp = (uint8_t *)qk, *qmp = (uint8_t *)qm;
        if (!col)
            return swz ? launch_t64<true, false, true, false, true>(t64, qkp, skp, nullptr, nullptr, (int)M, (int)N, st, g)
                       : launch_t64<true, false, false, false, true>(t64, qkp, skp, nullptr, nullptr, (int)M, (int)N, st, g);
        if (!row) return launch_t64<false, true, true, false, true>(t64, nullptr, nullptr, qmp, smp, (int)M, (int)N, st, g);
        if (!qm) return launch_t64<true, false, true, false, true>(t64, qkp, skp, nullptr, smp, (int)M, (int)N, st, g);
        return launch_t64<true, true, true, false, true>(t64, qkp, skp, qmp, smp, (int)M, (int)N, st, g);
    }

    if (!col) {
        const int64_t nb = N / 32;
        if (M * nb >= (1ll << 32) - 2 * RS_THREADS * RS_UNROLL) return QCC_ERR_SHAPE;
        const uint32_t nblocks = (uint32_t)(M * nb);
        FastDiv32 dv;
        dv.init((uint32_t)nb);
        if (swz && !g.row_map && ((M & 127) != 0 || (nb & 3) != 0)) {
            blocked_zero_pad_kernel<<<sm_count() * 4, 256, 0, st>>>(skp, (uint32_t)M, (uint32_t)nb);
            cudaError_t e = cudaGetLastError();
            if (e != cudaSuccess) return (int)e;
        }
        const unsigned grid = (nblocks + RS_THREADS * RS_UNROLL - 1) / (RS_THREADS * RS_UNROLL);
        const uint16_t *xp = (const uint16_t *)x;
        uint8_t *qp = (uint8_t *)qk;
#define QCC_RS(SWZ_, FL_, AM_) \
    mxfp8_rowwise_stream_kernel<SWZ_, FL_, AM_><<<grid, RS_THREADS, 0, st>>>(xp, nblocks, (uint32_t)nb, dv, qp, skp, g, sink)
#define QCC_RS_AM(SWZ_, FL_) \
    do { if (amax_mode == 0) QCC_RS(SWZ_, FL_, 0); else if (amax_mode == 1) QCC_RS(SWZ_, FL_, 1); else QCC_RS(SWZ_, FL_, 2); } while (0)
        if (swz) {
            if (fl) QCC_RS_AM(true, true); else QCC_RS_AM(true, false);
        } else {
            if (fl) QCC_RS_AM(false, true); else QCC_RS_AM(false, false);
        }
#undef QCC_RS_AM
#undef QCC_RS
        return (int)cudaGetLastError();
    }

    uint8_t *qkp = (uint8_t *)qk, *qmp = (uint8_t *)qm;
    {
        CUtensorMap t64;
        // padded token groups: M counts output rows, the input has g.src_rows of them and is fetched by 32-row boxes
        uint64_t dims[2] = {(uint64_t)N, (uint64_t)(g.blk_src ? g.src_rows : M)};
        uint64_t strides[1] = {(uint64_t)N * 2};
        uint32_t box[2] = {64, g.blk_src ? 32u : 64u};
        int e = make_tensor_map(&t64, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (e) return e;
#define QCC_T64(DO_K)                                                                                        \
    (swz ? (fl ? launch_t64<DO_K, true, true, true>(t64, qkp, skp, qmp, smp, (int)M, (int)N, st, g)             \
               : launch_t64<DO_K, true, true, false>(t64, qkp, skp, qmp, smp, (int)M, (int)N, st, g))           \
         : (fl ? launch_t64<DO_K, true, false, true>(t64, qkp, skp, qmp, smp, (int)M, (int)N, st, g)            \
               : launch_t64<DO_K, true, false, false>(t64, qkp, skp, qmp, smp, (int)M, (int)N, st, g)))
        if (g.rows_per_mat) {   // stacked matrices (blocked scales only)
            if (row) return fl ? launch_t64<true, true, true, true, false, false, true>(t64, qkp, skp, qmp, smp, (int)M, (int)N, st, g)
                               : launch_t64<true, true, true, false, false, false, true>(t64, qkp, skp, qmp, smp, (int)M, (int)N, st, g);
            return fl ? launch_t64<false, true, true, true, false, false, true>(t64, qkp, skp, qmp, smp, (int)M, (int)N, st, g)
                      : launch_t64<false, true, true, false, false, false, true>(t64, qkp, skp, qmp, smp, (int)M, (int)N, st, g);
        }
        if (g.blk_src) {   // padded token groups (blocked scales only)
            if (row) return fl ? launch_t64<true, true, true, true, false, true>(t64, qkp, skp, qmp, smp, (int)M, (int)N, st, g)
                               : launch_t64<true, true, true, false, false, true>(t64, qkp, skp, qmp, smp, (int)M, (int)N, st, g);
            return fl ? launch_t64<false, true, true, true, false, true>(t64, qkp, skp, qmp, smp, (int)M, (int)N, st, g)
                      : launch_t64<false, true, true, false, false, true>(t64, qkp, skp, qmp, smp, (int)M, (int)N, st, g);
        }
        if (row) return QCC_T64(true);
        return QCC_T64(false);
#undef QCC_T64
    }
}

extern "C" int qcc_mxfp8(const void *x, int64_t M, int64_t N, int flags, void *qk, void *sk, void *qm, void *sm,
                         void *stream)
{
    return mxfp8_entry(x, M, N, flags, qk, sk, qm, sm, stream, GroupTables{nullptr, nullptr, nullptr, nullptr, nullptr, 0, 0, 0});
}

// The rowwise cast that also delivers max |x| (raw, fp32): x is read once for both.  workspace: as for qcc_amax_bf16
// with QCC_AMAX_ONE_LAUNCH (prepared by qcc_amax_workspace_init).
extern "C" int qcc_mxfp8_amax(const void *x, int64_t M, int64_t N, int flags, void *qk, void *sk, float *amax_out,
                              void *workspace, size_t workspace_bytes, void *stream)
{
    if ((flags & (QCC_COLWISE | QCC_BLOCK32)) || !(flags & QCC_ROWWISE) || !amax_out || !workspace) return QCC_ERR_ARG;
    if (workspace_bytes < qcc_amax_workspace_bytes()) return QCC_ERR_WORKSPACE;
    if (M <= 0 || N <= 0) return QCC_ERR_SHAPE;
    AmaxSink sink{};
    sink.ctl = static_cast<uint32_t *>(workspace) + AMAX_MAX_CTAS;
    sink.out = amax_out;
    return mxfp8_entry(x, M, N, flags, qk, sk, nullptr, nullptr, stream,
                       GroupTables{nullptr, nullptr, nullptr, nullptr, nullptr, 0, 0, 0}, 1, &sink);
}

// The same as a producer of this rank's amax exchange: the amax goes into the exchange state's accumulator.
extern "C" int qcc_mxfp8_amax_xchg(const void *x, int64_t M, int64_t N, int flags, void *qk, void *sk, void *state, void *stream)
{
    if ((flags & (QCC_COLWISE | QCC_BLOCK32)) || !(flags & QCC_ROWWISE) || !state) return QCC_ERR_ARG;
    if (M <= 0 || N <= 0) return QCC_ERR_SHAPE;
    AmaxSink sink{};
    sink.ctl = static_cast<uint32_t *>(state);
    return mxfp8_entry(x, M, N, flags, qk, sk, nullptr, nullptr, stream,
                       GroupTables{nullptr, nullptr, nullptr, nullptr, nullptr, 0, 0, 0}, 2, &sink);
}

// E independent (M, N) matrices stacked in x (per-expert weights): one launch per matrix, issued from here so that
// the caller pays one call instead of E.  Outputs are stacked the same way; blocked scale grids are per matrix.
extern "C" int qcc_mxfp8_batched(const void *x, int64_t E, int64_t M, int64_t N, int flags, void *qk, void *sk, void *qm,
                                 void *sm, void *stream)
{
    if (E < 0) return QCC_ERR_ARG;
    if (E == 0 || M == 0 || N == 0) return 0;
    const bool swz = flags & QCC_SWIZZLE, b32 = flags & QCC_BLOCK32;
    const int64_t nb = N / 32, mb = M / 32;
    const size_t sk_bytes = b32 && !swz ? (size_t)mb * nb
                                        : swz ? (size_t)((M + 127) / 128) * ((nb + 3) / 4) * 512 : (size_t)M * nb;
    const size_t sm_bytes = swz ? (size_t)((N + 127) / 128) * ((mb + 3) / 4) * 512 : (size_t)N * mb;
    // every slice must start 16-byte aligned
    if ((((size_t)M * N) & 15) || (sk && (sk_bytes & 15)) || (sm && (sm_bytes & 15))) return QCC_ERR_SHAPE;
    // One launch for the whole stack where the stacked outputs are those of one tall matrix: always for the plain
    // rowwise cast, for blocked scales when every matrix is whole 128-row atoms (the transposed outputs then go to
    // their own frames inside the kernel).
    const bool col = flags & QCC_COLWISE;
    const int64_t ME = E * M;
    if (!b32 && ME <= 0x7FFFFF00 && sm_bytes < (1ull << 32)) {
        if (!col && (!swz || M % 128 == 0)) return qcc_mxfp8(x, ME, N, flags, qk, sk, nullptr, nullptr, stream);
        if (col && swz && M % 128 == 0)
            return mxfp8_entry(x, ME, N, flags, qk, sk, qm, sm, stream,
                               GroupTables{nullptr, nullptr, nullptr, nullptr, nullptr, 0, (int)M, (uint32_t)sm_bytes});
    }
    for (int64_t e = 0; e < E; e++) {
        const int rc = qcc_mxfp8((const uint16_t *)x + (size_t)e * M * N, M, N, flags,
                                 qk ? (uint8_t *)qk + (size_t)e * M * N : nullptr, sk ? (uint8_t *)sk + e * sk_bytes : nullptr,
                                 qm ? (uint8_t *)qm + (size_t)e * M * N : nullptr, sm ? (uint8_t *)sm + e * sm_bytes : nullptr,
                                 stream);
        if (rc) return rc;
    }
    return 0;
}

// ---------------------------------------------------------------------------------------------
// token groups (MoE activations): blocked scales per group
// ---------------------------------------------------------------------------------------------
namespace qcc {

constexpr int GROUPS_MAX = 4096;
constexpr int GROUPS_MAX_PAD = 2048;                // the padding form keeps two more per-group arrays in shared memory
constexpr unsigned int QCC_DEVERR_GROUPS = 16u;   // reported by qcc_device_error

// offs[g] = end row of group g in x (ascending, last = src_rows).  Fills the tables of GroupTables for an output frame
// of M rows.  PAD false: the groups are multiples of 32 rows already and M = src_rows.  PAD true: every group is
// padded to a multiple of 32 rows on the way (torch_pad_token_groups of torchao / _pad_token_groups of the reference,
// experiments/quantize_tensor_api/moe_utils.py:35-59), M is the upper bound ceil32(src_rows + G * 32) and
// padded_offs[g] receives the group ends of the padded frame.
// Every CTA recomputes the (short) prefix sums over the groups, then fills its share of the tables.
template <bool PAD>
__global__ void __launch_bounds__(256) group_tables_kernel(const int32_t *__restrict__ offs, int G, int M, int src_rows,
                                                          int padded_c, int32_t *__restrict__ row_map,
                                                          uint32_t *__restrict__ mb_a, uint32_t *__restrict__ mb_b,
                                                          int32_t *__restrict__ blk_src, int32_t *__restrict__ blk_valid,
                                                          int32_t *__restrict__ padded_offs)
{
    constexpr int GMAX = PAD ? GROUPS_MAX_PAD : GROUPS_MAX;
    __shared__ int32_t s_end[GMAX];       // group ends in the output frame
    __shared__ int32_t s_prow[GMAX];      // first row of the group inside the stacked, 128-padded groups
    __shared__ uint32_t s_pcol[GMAX];     // first scale column of the group after padding each group to 4
    __shared__ int32_t s_shift[PAD ? GMAX : 1];   // source row minus output row inside the group
    __shared__ int32_t s_size[PAD ? GMAX : 1];    // rows the group really has
    for (int i = threadIdx.x; i < G; i += blockDim.x) s_end[i] = offs[i];
    __syncthreads();
    int bad = 0;
    if (threadIdx.x == 0) {
        int32_t prow = 0, start = 0, pstart = 0;
        uint32_t pcol = 0;
        for (int i = 0; i < G; i++) {
            const int32_t end = s_end[i];
            const int32_t size = end - start;
            bad |= (size < 0) | (end > src_rows) | (PAD ? 0 : (end & 31));
            const int32_t psize = PAD ? ((max(size, 0) + 31) & ~31) : size;
            s_prow[i] = prow;
            s_pcol[i] = pcol;
            if (PAD) {
                s_shift[i] = start - pstart;
                s_size[i] = size;
                s_end[i] = pstart + psize;
            }
            if (size > 0) {
                prow += ((psize + 127) >> 7) << 7;
                pcol += (uint32_t)((((psize >> 5) + 3) >> 2) << 2);
                start = end;
                pstart += psize;
            }
        }
        // the padding form consumes every input row; without padding rows after the last group simply belong to none
        bad |= (PAD ? (start != src_rows) : 0) | (pstart > M);
        if (bad && blockIdx.x == 0) atomicMax(&g_qcc_error, QCC_DEVERR_GROUPS);
    }
    // offsets that are not ascending (multiples of 32) ending at the last row: no scale is written at all
    const int total = __syncthreads_or(bad) ? 0 : s_end[G - 1];
    if (PAD && padded_offs && blockIdx.x == 0)
        for (int i = threadIdx.x; i < G; i += blockDim.x) padded_offs[i] = total ? s_end[i] : 0;
    for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < M; r += gridDim.x * blockDim.x) {
        int32_t dst = -1, src = src_rows, nvalid = 0;
        uint32_t a = 0xFFFFFFFFu, bstride = 0;
        if (r < total) {
            int lo = 0, hi = G - 1;                 // first group whose end is above r
            while (lo < hi) {
                const int mid = (lo + hi) >> 1;
                if (s_end[mid] > r) hi = mid; else lo = mid + 1;
            }
            const int start = lo > 0 ? s_end[lo - 1] : 0;
            const int size = s_end[lo] - start;
            dst = s_prow[lo] + (r - start);
            const uint32_t cg = (uint32_t)(r - start) >> 5;
            const uint32_t ncb = (uint32_t)(((size >> 5) + 3) >> 2);
            a = s_pcol[lo] * (uint32_t)padded_c + (cg >> 2) * 512u + (cg & 3u);
            bstride = ncb * 512u;
            if (PAD) {
                src = r + s_shift[lo];
                nvalid = min(32, max(0, s_size[lo] - (r - start)));
            }
        }
        row_map[r] = dst;
        if ((r & 31) == 0) {
            mb_a[r >> 5] = a;
            mb_b[r >> 5] = bstride;
            if (PAD) { blk_src[r >> 5] = src; blk_valid[r >> 5] = nvalid; }
        }
    }
}

// PAD: out (rows_padded, row_bytes) = the rows of x moved to their padded places, zeros elsewhere.
// !PAD (the inverse, _unpad_token_groups of moe_main.py:54-68): out (unpadded rows) = the real rows of the padded x.
// One 16-byte piece per thread, indexed in the padded frame.
template <bool PAD>
__global__ void __launch_bounds__(256) pad_rows_kernel(const uint4 *__restrict__ x, uint4 *__restrict__ out, int rows_padded,
                                                      uint32_t vec_per_row, FastDiv32 div_vec,
                                                      const int32_t *__restrict__ blk_src, const int32_t *__restrict__ blk_valid)
{
    const uint64_t total = (uint64_t)rows_padded * vec_per_row;
    for (uint64_t i = (uint64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (uint64_t)gridDim.x * 256) {
        // i < 2^32 is checked by the launcher
        const uint32_t row = div_vec.div((uint32_t)i);
        const uint32_t v = (uint32_t)i - row * vec_per_row;
        const uint32_t rb = row >> 5, ri = row & 31u;
        const bool real = (int32_t)ri < __ldg(blk_valid + rb);
        const size_t other = (size_t)((uint32_t)__ldg(blk_src + rb) + ri) * vec_per_row + v;   // place in the unpadded frame
        if (PAD) {
            uint4 val = make_uint4(0, 0, 0, 0);
            if (real) val = ld_nc_v4(x + other);
            st_out(out + i, val);
        } else if (real) {
            st_out(out + other, ld_nc_v4(x + i));
        }
    }
}

}  // namespace qcc

extern "C" size_t qcc_mxfp8_grouped_workspace_bytes(int64_t M)
{
    return (size_t)(M * 4 + 2 * ((M + 31) / 32) * 4 + 64);
}

extern "C" int qcc_mxfp8_grouped(const void *x, int64_t M, int64_t N, int flags, const int32_t *offs, int64_t G, void *qk,
                                 void *sk, void *qm, void *sm, void *workspace, size_t workspace_bytes, void *stream)
{
    const bool row = flags & QCC_ROWWISE, col = flags & QCC_COLWISE;
    if (M == 0 || N == 0) return 0;
    if (!offs || !workspace || G <= 0 || !(flags & QCC_SWIZZLE)) return QCC_ERR_ARG;
    if (G > GROUPS_MAX || M % 32 != 0 || M > 0x7FFFFF00) return QCC_ERR_SHAPE;
    if (row && N % 128 != 0) return QCC_ERR_SHAPE;   // (M + G * 128, N / 32) holds whole 4-column atoms only
    if (workspace_bytes < qcc_mxfp8_grouped_workspace_bytes(M)) return QCC_ERR_WORKSPACE;
    if (!aligned16(workspace)) return QCC_ERR_ALIGN;
    cudaStream_t st = (cudaStream_t)stream;
    const int64_t nb = N / 32, mb = M / 32, padded_c = ((N + 127) / 128) * 128;
    if ((uint64_t)padded_c * (uint64_t)(mb + G * 4) >= (1ull << 32)) return QCC_ERR_SHAPE;
    int32_t *row_map = (int32_t *)workspace;
    uint32_t *mb_a = (uint32_t *)(row_map + M);
    uint32_t *mb_b = mb_a + mb;
    cudaError_t e;
    if (row && sk && (e = cudaMemsetAsync(sk, 0, (size_t)(M + G * 128) * nb, st)) != cudaSuccess) return (int)e;
    if (col && sm && (e = cudaMemsetAsync(sm, 0, (size_t)padded_c * (mb + G * 4), st)) != cudaSuccess) return (int)e;
    int grid = (int)((M + 255) / 256);
    if (grid > sm_count()) grid = sm_count();
    group_tables_kernel<false><<<grid, 256, 0, st>>>(offs, (int)G, (int)M, (int)M, (int)padded_c, row_map, mb_a, mb_b, nullptr,
                                                    nullptr, nullptr);
    if ((e = cudaGetLastError()) != cudaSuccess) return (int)e;
    return mxfp8_entry(x, M, N, flags, qk, sk, qm, sm, stream, GroupTables{row_map, mb_a, mb_b, nullptr, nullptr, 0, 0, 0});
}

// ---- token groups of any size: pad to multiples of 32 rows and cast in one pass -----------------------------------
extern "C" int64_t qcc_padded_token_rows(int64_t M, int64_t G) { return ((M + G * 32 + 31) / 32) * 32; }

extern "C" size_t qcc_token_pad_workspace_bytes(int64_t M, int64_t G)
{
    const int64_t R = qcc_padded_token_rows(M, G);
    return (size_t)(R * 4 + 4 * (R / 32) * 4 + 64);
}

namespace {
struct PadTables {
    int32_t *row_map, *blk_src, *blk_valid;
    uint32_t *mb_a, *mb_b;
};
// carves the workspace and launches the table kernel for the padded frame of R rows
int build_pad_tables(const int32_t *offs, int64_t G, int64_t M, int64_t R, int64_t padded_c, int32_t *padded_offs,
                     void *workspace, cudaStream_t st, PadTables &t)
{
    t.row_map = (int32_t *)workspace;
    t.mb_a = (uint32_t *)(t.row_map + R);
    t.mb_b = t.mb_a + R / 32;
    t.blk_src = (int32_t *)(t.mb_b + R / 32);
    t.blk_valid = t.blk_src + R / 32;
    int grid = (int)((R + 255) / 256);
    if (grid > sm_count()) grid = sm_count();
    group_tables_kernel<true><<<grid, 256, 0, st>>>(offs, (int)G, (int)R, (int)M, (int)padded_c, t.row_map, t.mb_a, t.mb_b,
                                                   t.blk_src, t.blk_valid, padded_offs);
    return (int)cudaGetLastError();
}
}  // namespace

static int pad_or_unpad(const void *x, int64_t M, int64_t row_bytes, const int32_t *offs, int64_t G, void *out,
                        int32_t *padded_offs, void *workspace, size_t workspace_bytes, void *stream, bool unpad)
{
    if (M == 0) {
        // no tokens at all: the padded frame (32 G rows) is all padding, the unpadded one is empty
        if (!offs || G <= 0 || row_bytes <= 0 || (!unpad && !out)) return QCC_ERR_ARG;
        if (G > GROUPS_MAX_PAD || row_bytes % 16 != 0) return QCC_ERR_SHAPE;
        cudaError_t ce = cudaSuccess;
        if (!unpad) ce = cudaMemsetAsync(out, 0, (size_t)qcc_padded_token_rows(0, G) * row_bytes, (cudaStream_t)stream);
        if (ce == cudaSuccess && padded_offs) ce = cudaMemsetAsync(padded_offs, 0, (size_t)G * sizeof(int32_t), (cudaStream_t)stream);
        return (int)ce;
    }
    if (!x || !offs || !out || !workspace || G <= 0 || M < 0 || row_bytes <= 0) return QCC_ERR_ARG;
    if (G > GROUPS_MAX_PAD || row_bytes % 16 != 0 || M > 0x7FFFF000) return QCC_ERR_SHAPE;
    const int64_t R = qcc_padded_token_rows(M, G);
    if (R * (row_bytes / 16) >= (1ll << 32)) return QCC_ERR_SHAPE;
    if (workspace_bytes < qcc_token_pad_workspace_bytes(M, G)) return QCC_ERR_WORKSPACE;
    if (!aligned16(x) || !aligned16(out) || !aligned16(workspace)) return QCC_ERR_ALIGN;
    cudaStream_t st = (cudaStream_t)stream;
    PadTables t;
    int e = build_pad_tables(offs, G, M, R, 128, padded_offs, workspace, st, t);
    if (e) return e;
    FastDiv32 dv;
    dv.init((uint32_t)(row_bytes / 16));
    const uint64_t total = (uint64_t)R * (uint64_t)(row_bytes / 16);
    uint64_t grid = (total + 255) / 256;
    const uint64_t cap = (uint64_t)sm_count() * 32;
    if (grid > cap) grid = cap;
    if (unpad)
        pad_rows_kernel<false><<<(unsigned)grid, 256, 0, st>>>((const uint4 *)x, (uint4 *)out, (int)R, (uint32_t)(row_bytes / 16),
                                                              dv, t.blk_src, t.blk_valid);
    else
        pad_rows_kernel<true><<<(unsigned)grid, 256, 0, st>>>((const uint4 *)x, (uint4 *)out, (int)R, (uint32_t)(row_bytes / 16),
                                                             dv, t.blk_src, t.blk_valid);
    return (int)cudaGetLastError();
}

extern "C" int qcc_pad_token_groups(const void *x, int64_t M, int64_t row_bytes, const int32_t *offs, int64_t G, void *out,
                                    int32_t *padded_offs, void *workspace, size_t workspace_bytes, void *stream)
{
    return pad_or_unpad(x, M, row_bytes, offs, G, out, padded_offs, workspace, workspace_bytes, stream, false);
}

extern "C" int qcc_unpad_token_groups(const void *padded, int64_t M, int64_t row_bytes, const int32_t *offs, int64_t G,
                                      void *out, void *workspace, size_t workspace_bytes, void *stream)
{
    return pad_or_unpad(padded, M, row_bytes, offs, G, out, nullptr, workspace, workspace_bytes, stream, true);
}

extern "C" int qcc_mxfp8_grouped_pad(const void *x, int64_t M, int64_t N, int flags, const int32_t *offs, int64_t G,
                                     void *qk, void *sk, void *qm, void *sm, int32_t *padded_offs, void *workspace,
                                     size_t workspace_bytes, void *stream)
{
    const bool row = flags & QCC_ROWWISE, col = flags & QCC_COLWISE;
    if (N == 0) return 0;
    if (!offs || !workspace || G <= 0 || M < 0 || !(flags & QCC_SWIZZLE)) return QCC_ERR_ARG;
    if (G > GROUPS_MAX_PAD || M > 0x7FFFF000) return QCC_ERR_SHAPE;
    if (row && N % 128 != 0) return QCC_ERR_SHAPE;
    if (workspace_bytes < qcc_token_pad_workspace_bytes(M, G)) return QCC_ERR_WORKSPACE;
    if (!aligned16(workspace)) return QCC_ERR_ALIGN;
    cudaStream_t st = (cudaStream_t)stream;
    const int64_t R = qcc_padded_token_rows(M, G);
    const int64_t nb = N / 32, mb = R / 32, padded_c = ((N + 127) / 128) * 128;
    if ((uint64_t)padded_c * (uint64_t)(mb + G * 4) >= (1ull << 32)) return QCC_ERR_SHAPE;
    cudaError_t ce;
    if (row && sk && (ce = cudaMemsetAsync(sk, 0, (size_t)(R + G * 128) * nb, st)) != cudaSuccess) return (int)ce;
    if (col && sm && (ce = cudaMemsetAsync(sm, 0, (size_t)padded_c * (mb + G * 4), st)) != cudaSuccess) return (int)ce;
    if (M == 0) {
        // a rank that received no tokens (expert parallelism): the padded frame is all padding -- zero elements, zero
        // scales, every padded group empty -- as the pad-then-cast route gives for an empty input
        if (row && qk && (ce = cudaMemsetAsync(qk, 0, (size_t)R * N, st)) != cudaSuccess) return (int)ce;
        if (col && qm && (ce = cudaMemsetAsync(qm, 0, (size_t)R * N, st)) != cudaSuccess) return (int)ce;
        if (padded_offs && (ce = cudaMemsetAsync(padded_offs, 0, (size_t)G * sizeof(int32_t), st)) != cudaSuccess) return (int)ce;
        return 0;
    }
    if (!x) return QCC_ERR_ARG;
    PadTables t;
    int e = build_pad_tables(offs, G, M, R, padded_c, padded_offs, workspace, st, t);
    if (e) return e;
    return mxfp8_entry(x, R, N, flags, qk, sk, qm, sm, stream,
                       GroupTables{t.row_map, t.mb_a, t.mb_b, t.blk_src, t.blk_valid, (int)M, 0, 0});
}

extern "C" int qcc_mxfp4(const void *x, int64_t M, int64_t N, int flags, void *q, void *s, void *stream)
{
    if (M == 0 || N == 0) return 0;
    if (!x || !q || !s || (flags & ~QCC_SWIZZLE)) return QCC_ERR_ARG;
    if (M < 0 || N < 0 || N % 32 != 0) return QCC_ERR_SHAPE;
    if (!aligned16(x) || !aligned16(q) || !aligned16(s)) return QCC_ERR_ALIGN;
    const int64_t nb = N / 32;
    if (M * nb >= (1ll << 32) - RS_THREADS || M > 0x7FFFFFFF) return QCC_ERR_SHAPE;
    cudaStream_t st = (cudaStream_t)stream;
    const uint32_t nblocks = (uint32_t)(M * nb);
    FastDiv32 dv;
    dv.init((uint32_t)nb);
    const bool swz = flags & QCC_SWIZZLE;
    if (swz && ((M & 127) != 0 || (nb & 3) != 0)) {
        blocked_zero_pad_kernel<<<sm_count() * 4, 256, 0, st>>>((uint8_t *)s, (uint32_t)M, (uint32_t)nb);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return (int)e;
    }
    const unsigned grid = (nblocks + RS_THREADS - 1) / RS_THREADS;
    if (swz) mxfp4_rowwise_stream_kernel<true><<<grid, RS_THREADS, 0, st>>>((const uint16_t *)x, nblocks, (uint32_t)nb, dv, (uint8_t *)q, (uint8_t *)s);
    else mxfp4_rowwise_stream_kernel<false><<<grid, RS_THREADS, 0, st>>>((const uint16_t *)x, nblocks, (uint32_t)nb, dv, (uint8_t *)q, (uint8_t *)s);
    return (int)cudaGetLastError();
}
