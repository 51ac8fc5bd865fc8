// nvfp4 (1x16 blocks, e4m3 block scales under an fp32 outer scale, e2m1 elements packed two per
// byte) for sm_100a.
//
//  * rowwise: a flat stream -- a thread owns one 16-element block (two 16-byte loads, one 8-byte
//    store of packed nibbles, one scale byte); x, q and the plain scales are addressed by the flat
//    block index, only the blocked scale layout and per-row outer scales need (row, column).
//  * transposed: a one-shot tile kernel like the mxfp8 one.  A CTA of four warps owns 128 rows x 128
//    columns of x, fetched by TMA (two 64-column x 128-row boxes, 128-byte swizzle, one mbarrier with
//    a bounded wait); five CTAs are resident per SM.  Warp b quantises the 32-row slab b down the rows
//    (lane = four adjacent columns, two 16x1 blocks each) and writes 16 packed bytes per column into
//    a swizzled staging tile whose rows are output rows; the tile leaves as coalesced 16-byte stores,
//    four lanes per 64-byte row segment, and the block scales as whole 512-byte atoms.
//
// Numerics: G = quant_cast_bench/quant_cast_gold/recipes.py, GU = quant_cast_gold/utils.py of
// vkuzo/quant_cast_bench.  nvfp4_gs_f G:1494-1517, nvfp4_gs_swizzle_f G:1249-1266,
// nvfp4_gs_swizzle_sr_f G:1392-1426, fp4 encode GU:15-57, nibble order GU:87-92, blocked layout
// G:1000-1037; the transposed cast is nvfp4_gs_swizzle_f(x.t().contiguous(), s) of
// test/test_quant_cast_gold.py:104.
#include "common.cuh"
#include "host_util.h"

namespace qcc {

// One block: 16 bf16 in two uint4 -> 8 packed bytes and the inner scale byte.
template <bool SR>
__device__ __forceinline__ uint32_t nvfp4_quant16(uint4 a, uint4 b, float outer, float inv_outer, const float *lut,
                                                 uint64_t flat0, uint64_t seed, uint64_t offset, uint2 &packed, bool recip_div)
{
    uint32_t acc = absmax2(absmax2(absmax2(absmax2(0u, a.x), a.y), absmax2(a.z, a.w)),
                           absmax2(absmax2(b.x, b.y), absmax2(b.z, b.w)));
    float recip;
    const uint32_t byte = lut ? nvfp4_inner_lut(hmax_halves_f32(acc), outer, lut, recip, recip_div)
                              : nvfp4_inner(hmax_halves_f32(acc), outer, inv_outer, recip, recip_div);
    float v[16] = {bf16lo(a.x), bf16hi(a.x), bf16lo(a.y), bf16hi(a.y), bf16lo(a.z), bf16hi(a.z), bf16lo(a.w), bf16hi(a.w),
                   bf16lo(b.x), bf16hi(b.x), bf16lo(b.y), bf16hi(b.y), bf16lo(b.z), bf16hi(b.z), bf16lo(b.w), bf16hi(b.w)};
#pragma unroll
    for (int i = 0; i < 16; i += 2) mul2(v[i], v[i + 1], recip, v[i], v[i + 1]);   // packed fp32x2 multiply
    // the clamp to +-6 of G:1513 is what the saturating conversion does; it only has to be explicit
    // ahead of the dither
    if (SR) {
#pragma unroll
        for (int i = 0; i < 16; i++) v[i] = fminf(fmaxf(v[i], -6.0f), 6.0f);
#pragma unroll
        for (int g4 = 0; g4 < 4; g4++) {
            uint4 w = sr_words((flat0 >> 2) + g4, seed, offset);
            v[4 * g4 + 0] = sr_dither(v[4 * g4 + 0], w.x);
            v[4 * g4 + 1] = sr_dither(v[4 * g4 + 1], w.y);
            v[4 * g4 + 2] = sr_dither(v[4 * g4 + 2], w.z);
            v[4 * g4 + 3] = sr_dither(v[4 * g4 + 3], w.w);
        }
    }
    packed.x = cvt_e2m1x8(v);
    packed.y = cvt_e2m1x8(v + 8);
    return byte;
}

#ifndef QCC_NV_THREADS
#define QCC_NV_THREADS 256
#endif
#ifndef QCC_NV_UNROLL
#define QCC_NV_UNROLL 2
#endif
constexpr int NV_THREADS = QCC_NV_THREADS;
constexpr int NV_UNROLL = QCC_NV_UNROLL;

// The per-tensor outer scale.  SRC QCC_SRC_SCALE: outer[0] is the scale; QCC_SRC_AMAX: outer[0] is the raw amax and
// the scale is amax / 2688 (nvfp4_gs_scale G:1243-1246, folded into the cast), which the first CTA also writes to
// outer_out.  QCC_SRC_SCALE_PDL: as QCC_SRC_SCALE in a launch that overlaps the kernel that writes outer[0]: call after
// the thread has issued its loads of x; one thread waits for that kernel, reads the value past L1 and hands it to the
// CTA through shared memory (one barrier).  Called by all threads.
// Kernel option word `opts`: bit 0 walk the tensor from its end (QCC_REVERSE), bit 1 divisions by a constant as
// multiplications with its reciprocal (QCC_RECIP_DIV).
#define QCC_SRC_SCALE_PDL 2
constexpr int NV_OPT_REV = 1, NV_OPT_RECIP = 2;
template <int SRC>
__device__ __forceinline__ float nvfp4_outer_of_cta(const float *__restrict__ outer, float *__restrict__ outer_out, bool recip_div)
{
    if (SRC == QCC_SRC_SCALE) return __ldg(outer);
    if (SRC == QCC_SRC_SCALE_PDL) {
        __shared__ float sh;
        if (threadIdx.x == 0) {
            pdl_wait();
            sh = ld_cg_f32(outer);
        }
        __syncthreads();
        return sh;
    }
    const float o = div_by_const(__ldg(outer), 2688.0f, recip_div);
    if (blockIdx.x == 0 && threadIdx.x == 0 && outer_out) outer_out[0] = o;
    return o;
}

// OUTER: 0 one outer scale for the tensor, 1 one per row (per token, G:1567-1571), 2 one per 128x128 block
// (nvfp4_blocked_outer_f G:1609-1634; outer is then the (M/128, N/128) grid); SRC (OUTER 0 only): see above
template <bool SWZ, bool SR, int OUTER, int SRC = QCC_SRC_SCALE>
__global__ void __launch_bounds__(NV_THREADS)
nvfp4_rowwise_kernel(const uint16_t *__restrict__ x, uint32_t nblocks, uint32_t nb, FastDiv32 div_nb,
                     const float *__restrict__ outer, const uint64_t *__restrict__ key, uint8_t *__restrict__ q,
                     uint8_t *__restrict__ s, float *__restrict__ outer_out, int opts)
{
    const bool rev = opts & NV_OPT_REV, recip_div = opts & NV_OPT_RECIP;
    const uint4 *xv = reinterpret_cast<const uint4 *>(x);
    uint2 *qv = reinterpret_cast<uint2 *>(q);
    uint64_t seed = 0, offset = 0;
    if (SR) { seed = key[0]; offset = key[1]; }
    float o_all = 0.f, inv_all = 0.f;
    // (a shared-memory table of the second division, as the transposed kernel uses, measured slower here:
    // its loads compete with the scale shuffles for the same issue queue)
    const float *lut = nullptr;
    const uint32_t base = (rev ? gridDim.x - 1u - blockIdx.x : blockIdx.x) * (NV_THREADS * NV_UNROLL) + threadIdx.x;
    uint4 a[NV_UNROLL], b[NV_UNROLL];
#pragma unroll
    for (int u = 0; u < NV_UNROLL; u++) {
        const uint32_t bi = base + u * NV_THREADS;
        if (bi < nblocks) {
            a[u] = ld_v4(xv + 2 * (size_t)bi);
            b[u] = ld_v4(xv + 2 * (size_t)bi + 1);
        } else {
            a[u] = b[u] = make_uint4(0, 0, 0, 0);
        }
    }
    if (OUTER == 0) {
        o_all = nvfp4_outer_of_cta<SRC>(outer, outer_out, recip_div);
        inv_all = __fdiv_rn(1.0f, o_all);
    }
    // every lane runs the whole body (the shuffles below need the full warp); stores are predicated
#pragma unroll
    for (int u = 0; u < NV_UNROLL; u++) {
        const uint32_t bi = base + u * NV_THREADS;
        const bool ok = bi < nblocks;
        uint32_t row = 0, cb = 0;
        if (SWZ || OUTER != 0) { row = div_nb.div(ok ? bi : 0u); cb = (ok ? bi : 0u) - row * nb; }
        float o = o_all, inv = inv_all;
        if (OUTER == 1) { o = __ldg(outer + row); inv = __fdiv_rn(1.0f, o); }
        if (OUTER == 2) { o = __ldg(outer + (size_t)(row >> 7) * (nb >> 3) + (cb >> 3)); inv = __fdiv_rn(1.0f, o); }
        uint2 packed;
        const uint32_t byte = nvfp4_quant16<SR>(a[u], b[u], o, inv, lut, (uint64_t)bi * 16u, seed, offset, packed, recip_div);
        if (ok) st_out(qv + bi, packed);
        if (SWZ) {
            // four consecutive lanes hold the four scale columns of one (row, column block)
            uint32_t v = byte | (__shfl_down_sync(0xFFFFFFFFu, byte, 1) << 8);
            v |= __shfl_down_sync(0xFFFFFFFFu, v, 2) << 16;
            if ((nb & 3) == 0) {
                if (ok && (threadIdx.x & 3) == 0) *reinterpret_cast<uint32_t *>(s + blocked_offset(row, cb, nb >> 2)) = v;
            } else if (ok) {
                s[blocked_offset(row, cb, (nb + 3) >> 2)] = (uint8_t)byte;
            }
        } else if (ok) {
            s[bi] = (uint8_t)byte;
        }
    }
}

// The common case -- blocked scales, round to nearest, one outer scale, N % 64 == 0 -- with two adjacent blocks per thread: 64
// contiguous input bytes (four 16-byte loads that share sectors through L1), one 16-byte store of packed nibbles,
// and one blocked-offset computation per four scale bytes (a lane pair) instead of per byte.  (Four blocks per
// thread measured 33 % slower: 128-byte strides between lanes defeat coalescing.)
template <int SRC>
__global__ void __launch_bounds__(NV_THREADS)
nvfp4_rowwise_pair_kernel(const uint16_t *__restrict__ x, uint32_t npairs, uint32_t nb, FastDiv32 div_np,
                          const float *__restrict__ outer, uint8_t *__restrict__ q, uint8_t *__restrict__ s,
                          float *__restrict__ outer_out, int opts)
{
    const bool rev = opts & NV_OPT_REV, recip_div = opts & NV_OPT_RECIP;
    // rev: CTAs walk the tensor from its end (CTAs are dispatched in index order), so a cast that follows another pass
    // over the same tensor starts with the part that pass left in L2
    const uint32_t cta = rev ? gridDim.x - 1u - blockIdx.x : blockIdx.x;
    const uint32_t pi = cta * NV_THREADS + threadIdx.x;   // blocks 2 pi and 2 pi + 1 of the flat stream
    const bool ok = pi < npairs;
    uint4 c[4] = {};
    if (ok) {
        const uint4 *p = reinterpret_cast<const uint4 *>(x) + 4 * (size_t)pi;
#pragma unroll
        for (int i = 0; i < 4; i++) c[i] = ld_v4(p + i);
    }
    const float o = nvfp4_outer_of_cta<SRC>(outer, outer_out, recip_div);
    const float inv = __fdiv_rn(1.0f, o);
    uint2 p0, p1;
    const uint32_t b0 = nvfp4_quant16<false>(c[0], c[1], o, inv, nullptr, 0, 0, 0, p0, recip_div);
    const uint32_t b1 = nvfp4_quant16<false>(c[2], c[3], o, inv, nullptr, 0, 0, 0, p1, recip_div);
    if (ok) st_out(reinterpret_cast<uint4 *>(q) + pi, make_uint4(p0.x, p0.y, p1.x, p1.y));
    // an even lane and its neighbour hold the four scale columns of one (row, column block)
    const uint32_t b01 = b0 | (b1 << 8);
    const uint32_t v = b01 | (__shfl_down_sync(0xFFFFFFFFu, b01, 1) << 16);
    if (ok && (threadIdx.x & 1) == 0) {
        const uint32_t np = nb >> 1;
        const uint32_t row = div_np.div(pi);
        const uint32_t cb = (pi - row * np) << 1;
        *reinterpret_cast<uint32_t *>(s + blocked_offset(row, cb, nb >> 2)) = v;
    }
}

// The same cast for M % 128 == 0, N % 128 == 0 with the CTAs laid over 128-row x 128-column tiles instead of the flat
// stream: a tile is two whole 512-byte atoms of the blocked scale layout, so the scale bytes go through 1 KB of shared
// memory and leave as 64 contiguous 16-byte stores per CTA.  In the flat form every lane pair's 4-byte store lands in an
// atom of its own (the four bytes of a row, 512 bytes from the next pair's): four times as many store transactions as
// the packed data itself needs.  Thread = (row of the upper or lower 64-row half, 32-column pair of blocks); a warp
// reads 256 contiguous bytes of each of 8 rows.
#ifndef QCC_NV_ATOM_MIN_BLOCKS
#define QCC_NV_ATOM_MIN_BLOCKS 0
#endif
template <int SRC>
__global__ void __launch_bounds__(NV_THREADS)
nvfp4_rowwise_atom_kernel(const uint16_t *__restrict__ x, uint32_t tiles_n, uint32_t N, const float *__restrict__ outer,
                          uint8_t *__restrict__ q, uint8_t *__restrict__ s, float *__restrict__ outer_out, int opts)
{
    const bool rev = opts & NV_OPT_REV, recip_div = opts & NV_OPT_RECIP;
    __shared__ __align__(16) uint8_t stage[2 * 512];
    const uint32_t cta = rev ? gridDim.x - 1u - blockIdx.x : blockIdx.x;
    const uint32_t tile_m = cta / tiles_n, tile_n = cta - tile_m * tiles_n;
    const uint32_t pr = threadIdx.x & 3u, rr = threadIdx.x >> 2;
    uint4 c[2][4];
#pragma unroll
    for (int u = 0; u < 2; u++) {
        const size_t row = (size_t)tile_m * 128u + rr + 64u * u;
        const uint4 *p = reinterpret_cast<const uint4 *>(x + row * N + tile_n * 128u + pr * 32u);
#pragma unroll
        for (int i = 0; i < 4; i++) c[u][i] = ld_v4(p + i);
    }
    const float o = nvfp4_outer_of_cta<SRC>(outer, outer_out, recip_div);
    const float inv = __fdiv_rn(1.0f, o);
#pragma unroll
    for (int u = 0; u < 2; u++) {
        const uint32_t r = rr + 64u * u;                       // row inside the tile
        const size_t row = (size_t)tile_m * 128u + r;
        uint2 p0, p1;
        const uint32_t b0 = nvfp4_quant16<false>(c[u][0], c[u][1], o, inv, nullptr, 0, 0, 0, p0, recip_div);
        const uint32_t b1 = nvfp4_quant16<false>(c[u][2], c[u][3], o, inv, nullptr, 0, 0, 0, p1, recip_div);
        st_out(reinterpret_cast<uint4 *>(q + row * (N >> 1) + tile_n * 64u + pr * 16u), make_uint4(p0.x, p0.y, p1.x, p1.y));
        *reinterpret_cast<uint16_t *>(stage + (pr >> 1) * 512u + (r & 31u) * 16u + (r >> 5) * 4u + (pr & 1u) * 2u) =
            (uint16_t)(b0 | (b1 << 8));
    }
    __syncthreads();
    if (threadIdx.x < 64) {
        const uint32_t a = threadIdx.x >> 5, i = threadIdx.x & 31u;
        const size_t off = ((size_t)tile_m * (N >> 6) + tile_n * 2u + a) * 512u + i * 16u;
        *reinterpret_cast<uint4 *>(s + off) = *reinterpret_cast<const uint4 *>(stage + a * 512u + i * 16u);
    }
}

// ---------------------------------------------------------------------------------------------
// transposed cast: one-shot tile kernel
// ---------------------------------------------------------------------------------------------
constexpr int NVT_TILE_M = 128;
constexpr int NVT_PANEL_BYTES = NVT_TILE_M * 128;  // one 64-column panel: 128 rows x 128 B
constexpr int NVT_X_OFF = 0;
constexpr int NVT_Q_OFF = 2 * NVT_PANEL_BYTES;     // staging: 4 sub-tiles x 32 rows x 64 B
constexpr int NVT_S_OFF = NVT_Q_OFF + 4 * 32 * 64; // 128 columns x 8 block scales
constexpr int NVT_LUT_OFF = NVT_S_OFF + 1024;      // 128 multipliers, one per inner-scale byte
constexpr int NVT_BAR_OFF = NVT_LUT_OFF + 512;
constexpr int NVT_QK_OFF = NVT_Q_OFF;              // rowwise staging (fused form): reuses the transposed staging
constexpr int NVT_ALLOC = NVT_BAR_OFF + 512 + 1024;

// Row-major tile order (column tiles fastest), as in the mxfp8 tile kernel.  The four warps quantise down the
// rows (transposed outputs q, s); with DO_K they then also quantise along the rows of the same tile (outputs qk, sk),
// so both orientations come from one read of x.
// RHT: the 16-row blocks going down the rows pass through the 16-point randomised Hadamard transform before they
// are quantised -- the dim-m half of nvfp4_gs_swizzle_dim_k_dim_m_rht_f (G:1324-1333) and of its stochastic form
// (G:1429-1438); the rowwise half is not transformed and has its own outer scale and Philox key.

// RECIP: QCC_RECIP_DIV, as a template parameter because the kernel sits at its register limit.
template <bool DO_K, bool SWZ, bool SR, bool RHT, bool RECIP>
__global__ void __launch_bounds__(128, (RHT && SR) ? 4 : 5)
nvfp4_transposed_kernel(const __grid_constant__ CUtensorMap tm_x, const float *__restrict__ outer_p,
                        const float *__restrict__ outer_k_p, const uint64_t *__restrict__ key,
                        const uint64_t *__restrict__ key_k, const uint16_t *__restrict__ rht, uint8_t *__restrict__ q,
                        uint8_t *__restrict__ s, uint8_t *__restrict__ qk, uint8_t *__restrict__ sk, int M, int N,
                        int tiles_n)
{
    constexpr bool recip_div = RECIP;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *sbase = smem_raw + (base - smem_u32(smem_raw));
    uint64_t *bar = reinterpret_cast<uint64_t *>(sbase + NVT_BAR_OFF);
    const int tile_m = blockIdx.x / tiles_n, tile_n = blockIdx.x - tile_m * tiles_n;
    const int b = threadIdx.x >> 5, lane = threadIdx.x & 31;   // warp b owns the 32-row slab b

    if (threadIdx.x == 0) {
        mbar_init(bar, 1);
        fence_barrier_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        mbar_expect_tx(bar, 2 * NVT_PANEL_BYTES);
        tma_load_2d(sbase + NVT_X_OFF, &tm_x, bar, tile_n * 128, tile_m * NVT_TILE_M);
        tma_load_2d(sbase + NVT_X_OFF + NVT_PANEL_BYTES, &tm_x, bar, tile_n * 128 + 64, tile_m * NVT_TILE_M);
    }
    const float outer = __ldg(outer_p);
    const float inv_outer = __fdiv_rn(1.0f, outer);
    float *lut = reinterpret_cast<float *>(sbase + NVT_LUT_OFF);
    nvfp4_fill_recip_lut(lut, inv_outer);
    const uint32_t sgn = RHT ? rht_sign_mask(rht) : 0u;
    __syncthreads();
    uint64_t seed = 0, offset = 0;
    if (SR) { seed = key[0]; offset = key[1]; }
    const int mb16 = M >> 4;   // scale columns of the transposed frame
    const int halfM = M >> 1;  // bytes per output row

    mbar_wait(bar, 0, 2u);

    // ---------------------------------------------------------------------- along the row (fused form)
    auto row_phase = [&](const int rw, const float outer_k, const float inv_outer_k, const uint64_t seed_k,
                         const uint64_t offset_k) {
        const int row_t = rw * 32 + lane;
        const int R = tile_m * NVT_TILE_M + row_t;
        const int nb16 = N >> 4, halfN = N >> 1;
        const uint32_t xrow = base + NVT_X_OFF + row_t * 128;
        const uint32_t key7 = lane & 7;
        const uint32_t key2 = ((row_t >> 1) & 3) << 1;       // staging swizzle on 8-byte units, pairs kept together
        const uint32_t qrow = base + NVT_QK_OFF + row_t * 64;
        uint32_t sb[2] = {0u, 0u};
#pragma unroll
        for (int kb = 0; kb < 8; kb++) {
            const uint32_t prow = xrow + (kb >> 2) * NVT_PANEL_BYTES;
            const uint32_t j0 = (kb & 3) * 2;
            const uint4 a4 = lds_v4(prow + (((j0) ^ key7) << 4));
            const uint4 b4 = lds_v4(prow + (((j0 + 1) ^ key7) << 4));
            uint2 packed;
            const uint64_t flat0 = (uint64_t)R * (uint64_t)N + (uint64_t)(tile_n * 128 + kb * 16);
            uint32_t byte = nvfp4_quant16<SR>(a4, b4, outer_k, inv_outer_k, lut, flat0, seed_k, offset_k, packed, recip_div);
            const bool ok = R < M && (tile_n * 8 + kb) < nb16;
            sb[kb >> 2] |= (ok ? byte : 0u) << (8 * (kb & 3));
            asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(qrow + ((kb ^ key2) << 3)), "r"(packed.x), "r"(packed.y) : "memory");
        }
        __syncwarp();
        {
            const int jj = lane & 3;
            const int cbyte = tile_n * 64 + jj * 16;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int r = i * 8 + (lane >> 2);
                const int rt = rw * 32 + r;
                const int Rr = tile_m * NVT_TILE_M + rt;
                const uint4 v = lds_v4(base + NVT_QK_OFF + rt * 64 + ((jj ^ ((rt >> 1) & 3)) << 4));
                if (Rr < M && cbyte < halfN) *reinterpret_cast<uint4 *>(qk + (size_t)Rr * halfN + cbyte) = v;
            }
        }
        if (SWZ) {
            const uint32_t ncb = (nb16 + 3) >> 2;
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const uint32_t bc = tile_n * 2 + h;
                if (bc < ncb)
                    *reinterpret_cast<uint32_t *>(sk + ((size_t)tile_m * ncb + bc) * 512u + lane * 16u + rw * 4u) = sb[h];
            }
        } else if (R < M) {
            uint8_t *dst = sk + (size_t)R * nb16 + tile_n * 8;
            if ((nb16 & 7) == 0) {
                *reinterpret_cast<uint2 *>(dst) = make_uint2(sb[0], sb[1]);
            } else {
#pragma unroll
                for (int kb = 0; kb < 8; kb++)
                    if (tile_n * 8 + kb < nb16) dst[kb] = (uint8_t)(sb[kb >> 2] >> (8 * (kb & 3)));
            }
        }
    };

    const uint32_t pbase = base + NVT_X_OFF + (lane >> 4) * NVT_PANEL_BYTES + (b * 32) * 128 + (lane & 1) * 8;
    const uint32_t j = (lane & 15) >> 1;
    uint4 outw[4];  // per column: 32 rows -> 16 packed bytes
    uint32_t sc[4][2];
#pragma unroll
    for (int h = 0; h < 2; h++) {
        uint2 w[16];
        uint32_t a0 = 0, a1 = 0;
        if (RHT) {
            uint32_t wx[16], wy[16];
#pragma unroll
            for (int r = 0; r < 16; r++) {
                const int rr = 16 * h + r;
                const uint2 v2 = lds_v2(pbase + rr * 128 + ((j ^ (rr & 7)) << 4));
                wx[r] = v2.x;
                wy[r] = v2.y;
            }
            rht16_bf16x2(wx, sgn);
            rht16_bf16x2(wy, sgn);
#pragma unroll
            for (int r = 0; r < 16; r++) {
                w[r] = make_uint2(wx[r], wy[r]);
                a0 = absmax2_acc(a0, wx[r]);
                a1 = absmax2_acc(a1, wy[r]);
            }
        } else {
#pragma unroll
            for (int r = 0; r < 16; r++) {
                const int rr = 16 * h + r;
                w[r] = lds_v2(pbase + rr * 128 + ((j ^ (rr & 7)) << 4));
                a0 = absmax2_acc(a0, w[r].x);
                a1 = absmax2_acc(a1, w[r].y);
            }
        }
        const float am[4] = {u2f(a0 << 16), u2f(a0 & 0xFFFF0000u), u2f(a1 << 16), u2f(a1 & 0xFFFF0000u)};
#pragma unroll
        for (int k = 0; k < 4; k++) {
            float recip;
            sc[k][h] = nvfp4_inner_lut(am[k], outer, lut, recip, recip_div);
            float v[16];
#pragma unroll
            for (int r = 0; r < 16; r += 2) {
                const uint32_t w0 = (k < 2) ? w[r].x : w[r].y, w1 = (k < 2) ? w[r + 1].x : w[r + 1].y;
                mul2((k & 1) ? bf16hi(w0) : bf16lo(w0), (k & 1) ? bf16hi(w1) : bf16lo(w1), recip, v[r], v[r + 1]);
            }
            if (SR) {
#pragma unroll
                for (int r = 0; r < 16; r++) v[r] = fminf(fmaxf(v[r], -6.0f), 6.0f);
                // flat index in the transposed frame: column * M + m
                const uint64_t col = (uint64_t)tile_n * 128 + 4 * lane + k;
                const uint64_t flat0 = col * (uint64_t)M + (uint64_t)tile_m * NVT_TILE_M + b * 32 + 16 * h;
#pragma unroll
                for (int g4 = 0; g4 < 4; g4++) {
                    uint4 rw = sr_words((flat0 >> 2) + g4, seed, offset);
                    v[4 * g4 + 0] = sr_dither(v[4 * g4 + 0], rw.x);
                    v[4 * g4 + 1] = sr_dither(v[4 * g4 + 1], rw.y);
                    v[4 * g4 + 2] = sr_dither(v[4 * g4 + 2], rw.z);
                    v[4 * g4 + 3] = sr_dither(v[4 * g4 + 3], rw.w);
                }
            }
            const uint32_t p0 = cvt_e2m1x8(v), p1 = cvt_e2m1x8(v + 8);
            if (h == 0) { outw[k].x = p0; outw[k].y = p1; } else { outw[k].z = p0; outw[k].w = p1; }
        }
    }
    // staging: sub-tile k holds columns {4 l + k}, one 64-byte row (the tile's 128 m, two per byte) per
    // column; 16-byte chunk c of row l sits at position c ^ ((l >> 1) & 3).  Slab b is chunk b.
    const uint32_t qs = base + NVT_Q_OFF;
    const uint32_t key4 = (lane >> 1) & 3;
#pragma unroll
    for (int k = 0; k < 4; k++) sts_v4(qs + k * 2048 + lane * 64 + ((b ^ key4) << 4), outw[k]);
    // block scales of this slab -> staging, zero outside the matrix
    uint8_t *ss = sbase + NVT_S_OFF;
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const int c = 4 * lane + k;
        const bool col_ok = tile_n * 128 + c < N;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int blk = 2 * b + h;                       // 0..7 inside the tile
            const bool ok = col_ok && (tile_m * 8 + blk < mb16);
            const int off = SWZ ? ((blk >> 2) * 512 + (c & 31) * 16 + (c >> 5) * 4 + (blk & 3)) : (c * 8 + blk);
            ss[off] = ok ? (uint8_t)sc[k][h] : (uint8_t)0;
        }
    }
    named_barrier(1, 128);   // the four column warps
    // write-out: warp b takes sub-tile b; four lanes move one 64-byte row segment
    {
        const int jj = lane & 3;
        const int mbyte = tile_m * (NVT_TILE_M / 2) + jj * 16;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int l = i * 8 + (lane >> 2);
            const int Cn = tile_n * 128 + 4 * l + b;
            const uint4 v = lds_v4(qs + b * 2048 + l * 64 + ((jj ^ ((l >> 1) & 3)) << 4));
            if (Cn < N && mbyte < halfM) *reinterpret_cast<uint4 *>(q + (size_t)Cn * halfM + mbyte) = v;
        }
    }
    if (SWZ) {
        // two consecutive 512-byte atoms (row block = tile_n, column blocks 2 tile_m and 2 tile_m + 1)
        if (threadIdx.x < 64) {
            const int t = threadIdx.x;
            const uint32_t ncb = (mb16 + 3) >> 2;
            const uint32_t atom = t >> 5;
            if ((uint32_t)tile_m * 2 + atom < ncb) {
                const size_t off = ((size_t)tile_n * ncb + tile_m * 2 + atom) * 512u + (t & 31) * 16u;
                *reinterpret_cast<uint4 *>(s + off) = *reinterpret_cast<const uint4 *>(ss + t * 16);
            }
        }
    } else {
        const int t = threadIdx.x;
        const int Cn = tile_n * 128 + t;
        if (Cn < N) {
            uint8_t *dst = s + (size_t)Cn * mb16 + tile_m * 8;
            if ((mb16 & 7) == 0) {
                *reinterpret_cast<uint2 *>(dst) = *reinterpret_cast<const uint2 *>(ss + t * 8);
            } else {
                const uint8_t *src = ss + t * 8;
                for (int kk = 0; kk < 8; kk++)
                    if (tile_m * 8 + kk < mb16) dst[kk] = src[kk];
            }
        }
    }
    if (DO_K) {
        // The same four warps, after their column work (four more warps for this half measured 14 % slower: they sit
        // idle while the column warps finish, and eight warps at 80 registers allow 3 CTAs per SM instead of 5).
        float outer_k = outer, inv_outer_k = inv_outer;
        uint64_t seed_k = 0, offset_k = 0;
        if (SR) { seed_k = key_k[0]; offset_k = key_k[1]; }
        __syncthreads();                     // the staging tile and the multiplier table are about to be reused
        if (RHT) {                           // the two halves have their own outer scales
            outer_k = __ldg(outer_k_p);
            inv_outer_k = __fdiv_rn(1.0f, outer_k);
            nvfp4_fill_recip_lut(lut, inv_outer_k);
            __syncthreads();
        }
        row_phase(b, outer_k, inv_outer_k, seed_k, offset_k);
    }
}

// rht must be diag(sign) @ H / 4 in bf16: entry (i, j) = +-0.25 with the sign of row i times (-1)^popcount(i & j)
__global__ void rht_check_kernel(const uint16_t *__restrict__ rht)
{
    const uint32_t i = threadIdx.x >> 4, jx = threadIdx.x & 15;
    const uint32_t row_sign = __ldg(rht + i * 16) & 0x8000u;
    const uint32_t want = (0x3E80u | row_sign) ^ ((__popc(i & jx) & 1u) << 15);
    if (__ldg(rht + threadIdx.x) != want) atomicMax(&g_qcc_error, QCC_DEVERR_RHT);
}

int launch_rht_check(const void *rht, cudaStream_t st)
{
    rht_check_kernel<<<1, 256, 0, st>>>((const uint16_t *)rht);
    return (int)cudaGetLastError();
}

}  // namespace qcc

using namespace qcc;

extern "C" int qcc_nvfp4_device_error(unsigned int *out) { return read_clear_device_error(out); }

// outer_kind: 0..2 as `outer_per_row` of qcc_nvfp4; 3 = outer points at a raw amax
static int nvfp4_rowwise_entry(const void *x, int64_t M, int64_t N, const void *outer_src, int outer_kind, int flags,
                               const uint64_t *philox_key, void *q, void *s, float *outer_out, void *stream)
{
    if (M == 0 || N == 0) return 0;
    if (!x || !outer_src || !q || !s || (flags & ~(QCC_SWIZZLE | QCC_SR | QCC_PDL | QCC_REVERSE | QCC_RECIP_DIV))) return QCC_ERR_ARG;
    if ((flags & QCC_SR) && !philox_key) return QCC_ERR_ARG;
    if (M < 0 || N < 0 || N % 16 != 0) return QCC_ERR_SHAPE;
    if (!aligned16(x) || !aligned16(q) || !aligned16(s)) return QCC_ERR_ALIGN;
    const int64_t nb = N / 16;
    if (M * nb >= (1ll << 32) - 2 * NV_THREADS * NV_UNROLL || nb > 0x7FFFFFFF || M > 0x7FFFFFFF) return QCC_ERR_SHAPE;
    cudaStream_t st = (cudaStream_t)stream;
    const uint32_t nblocks = (uint32_t)(M * nb);
    FastDiv32 dv;
    dv.init((uint32_t)nb);
    const unsigned grid = (nblocks + NV_THREADS * NV_UNROLL - 1) / (NV_THREADS * NV_UNROLL);
    if (outer_kind < 0 || outer_kind > 3) return QCC_ERR_ARG;
    const int src = outer_kind == 3 ? QCC_SRC_AMAX : QCC_SRC_SCALE;
    const int outer_per_row = outer_kind <= 2 ? outer_kind : 0;
    const bool swz = flags & QCC_SWIZZLE, sr = flags & QCC_SR, pr = outer_per_row == 1;
    if (src != QCC_SRC_SCALE && sr) return QCC_ERR_ARG;
    // the overlapped form exists for the common case only: blocked scales, one outer scale, round to nearest
    const int rev = ((flags & QCC_REVERSE) ? NV_OPT_REV : 0) | ((flags & QCC_RECIP_DIV) ? NV_OPT_RECIP : 0);   // the kernels' option word
    const bool pdl = (flags & QCC_PDL) && swz && !sr && outer_kind == 0 && (nb & 3) == 0;
    if (outer_per_row == 2 && (sr || M % 128 != 0 || N % 128 != 0)) return sr ? QCC_ERR_ARG : QCC_ERR_SHAPE;
    const uint16_t *xp = (const uint16_t *)x;
    uint8_t *qp = (uint8_t *)q, *sp = (uint8_t *)s;
    const float *outer = (const float *)outer_src;
    if (swz && ((M & 127) != 0 || (nb & 3) != 0)) {
        blocked_zero_pad_kernel<<<sm_count() * 4, 256, 0, st>>>(sp, (uint32_t)M, (uint32_t)nb);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return (int)e;
    }
#ifndef QCC_NV_PAIR_MIN_BLOCKS
#define QCC_NV_PAIR_MIN_BLOCKS 0
#endif
#ifndef QCC_NV_NO_ATOM
    if (swz && !sr && outer_per_row == 0 && !pdl && (M & 127) == 0 && (N & 127) == 0 && nblocks >= (uint32_t)QCC_NV_ATOM_MIN_BLOCKS) {
        const uint32_t tiles_n = (uint32_t)(N >> 7);
        const unsigned agrid = (unsigned)((M >> 7) * tiles_n);
        if (src == QCC_SRC_SCALE)
            nvfp4_rowwise_atom_kernel<QCC_SRC_SCALE><<<agrid, NV_THREADS, 0, st>>>(xp, tiles_n, (uint32_t)N, outer, qp, sp, outer_out, rev);
        else
            nvfp4_rowwise_atom_kernel<QCC_SRC_AMAX><<<agrid, NV_THREADS, 0, st>>>(xp, tiles_n, (uint32_t)N, outer, qp, sp, outer_out, rev);
        return (int)cudaGetLastError();
    }
#endif
    if (swz && !sr && outer_per_row == 0 && (nb & 3) == 0 && nblocks >= (uint32_t)QCC_NV_PAIR_MIN_BLOCKS) {   // (the plain layout gains nothing from pairing)
        const uint32_t npairs = nblocks >> 1;
        FastDiv32 dp;
        dp.init((uint32_t)(nb >> 1));
        const unsigned pgrid = (npairs + NV_THREADS - 1) / NV_THREADS;
#define QCC_NVP(SRC_) \
    nvfp4_rowwise_pair_kernel<SRC_><<<pgrid, NV_THREADS, 0, st>>>(xp, npairs, (uint32_t)nb, dp, outer, qp, sp, outer_out, rev)
        if (pdl) {
            cudaError_t le = launch_maybe_pdl(nvfp4_rowwise_pair_kernel<QCC_SRC_SCALE_PDL>, dim3(pgrid), dim3(NV_THREADS), 0, st, true, xp,
                                              npairs, (uint32_t)nb, dp, outer, qp, sp, outer_out, rev);
            return (int)le;
        }
        if (src == QCC_SRC_SCALE) QCC_NVP(QCC_SRC_SCALE);
        else QCC_NVP(QCC_SRC_AMAX);
#undef QCC_NVP
        return (int)cudaGetLastError();
    }
#define QCC_NV(SWZ_, SR_, PR_, SRC_) \
    nvfp4_rowwise_kernel<SWZ_, SR_, PR_, SRC_><<<grid, NV_THREADS, 0, st>>>(xp, nblocks, (uint32_t)nb, dv, outer, philox_key, qp, sp, \
                                                                            outer_out, rev)
    if (src != QCC_SRC_SCALE) {
        if (swz) QCC_NV(true, false, 0, QCC_SRC_AMAX); else QCC_NV(false, false, 0, QCC_SRC_AMAX);
    } else if (outer_per_row == 2) {
        if (swz) QCC_NV(true, false, 2, QCC_SRC_SCALE); else QCC_NV(false, false, 2, QCC_SRC_SCALE);
    } else if (swz) {
        if (sr) { if (pr) QCC_NV(true, true, 1, QCC_SRC_SCALE); else QCC_NV(true, true, 0, QCC_SRC_SCALE); }
        else    { if (pr) QCC_NV(true, false, 1, QCC_SRC_SCALE); else QCC_NV(true, false, 0, QCC_SRC_SCALE); }
    } else {
        if (sr) { if (pr) QCC_NV(false, true, 1, QCC_SRC_SCALE); else QCC_NV(false, true, 0, QCC_SRC_SCALE); }
        else    { if (pr) QCC_NV(false, false, 1, QCC_SRC_SCALE); else QCC_NV(false, false, 0, QCC_SRC_SCALE); }
    }
#undef QCC_NV
    return (int)cudaGetLastError();
}

extern "C" int qcc_nvfp4(const void *x, int64_t M, int64_t N, const float *outer, int outer_per_row, int flags,
                         const uint64_t *philox_key, void *q, void *s, void *stream)
{
    if (outer_per_row < 0 || outer_per_row > 2) return (M == 0 || N == 0) ? 0 : QCC_ERR_ARG;
    return nvfp4_rowwise_entry(x, M, N, outer, outer_per_row, flags, philox_key, q, s, nullptr, stream);
}

extern "C" int qcc_nvfp4_from_amax(const void *x, int64_t M, int64_t N, const float *amax, int flags, void *q, void *s,
                                   float *outer_out, void *stream)
{
    return nvfp4_rowwise_entry(x, M, N, amax, 3, flags, nullptr, q, s, outer_out, stream);
}

struct NvtArgs {
    const float *outer, *outer_k;          // down the rows / along the rows (fused forms)
    const uint64_t *key, *key_k;
    const uint16_t *rht;                   // non-null: transform down the rows
    uint8_t *q, *s, *qk, *sk;
    int recip_div = 0;                     // QCC_RECIP_DIV given
};

template <bool DO_K, bool SWZ, bool SR, bool RHT, bool RECIP>
static int launch_nvt_r(const CUtensorMap &tx, const NvtArgs &a, int M, int N, cudaStream_t st)
{
    auto kern = nvfp4_transposed_kernel<DO_K, SWZ, SR, RHT, RECIP>;
    static PerDeviceFlag configured;
    const int dev = current_device_slot();
    if (dev < 0) return QCC_ERR_ARG;
    if (!configured.get(dev)) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, NVT_ALLOC);
        if (e != cudaSuccess) return (int)e;
        e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
        if (e != cudaSuccess) return (int)e;
        configured.set(dev);
    }
    const int tiles_n = (N + 127) / 128, tiles_m = (M + NVT_TILE_M - 1) / NVT_TILE_M;
    const long long num_tiles = (long long)tiles_n * tiles_m;
    if (num_tiles > 0x7FFFFFFF) return QCC_ERR_SHAPE;
    kern<<<(unsigned)num_tiles, 128, NVT_ALLOC, st>>>(tx, a.outer, a.outer_k, a.key, a.key_k, a.rht, a.q, a.s, a.qk, a.sk, M, N,
                                                     tiles_n);
    return (int)cudaGetLastError();
}

template <bool DO_K, bool SWZ, bool SR, bool RHT>
static int launch_nvt(const CUtensorMap &tx, const NvtArgs &a, int M, int N, cudaStream_t st)
{
    return a.recip_div ? launch_nvt_r<DO_K, SWZ, SR, RHT, true>(tx, a, M, N, st) : launch_nvt_r<DO_K, SWZ, SR, RHT, false>(tx, a, M, N, st);
}

template <bool DO_K, bool RHT>
static int launch_nvt_flags(const CUtensorMap &tx, const NvtArgs &a, bool swz, bool sr, int M, int N, cudaStream_t st)
{
    constexpr bool SR_OK = !DO_K;          // the fused form is round-to-nearest (see qcc_nvfp4_rht)
    if (sr && !SR_OK) return QCC_ERR_ARG;
    if (swz) return (sr && SR_OK) ? launch_nvt<DO_K, true, SR_OK, RHT>(tx, a, M, N, st) : launch_nvt<DO_K, true, false, RHT>(tx, a, M, N, st);
    return (sr && SR_OK) ? launch_nvt<DO_K, false, SR_OK, RHT>(tx, a, M, N, st) : launch_nvt<DO_K, false, false, RHT>(tx, a, M, N, st);
}

static int nvfp4_tile_entry(const void *x, int64_t M, int64_t N, const NvtArgs &args, int flags, bool both, void *stream)
{
    if (M == 0 || N == 0) return 0;
    NvtArgs a = args;
    a.recip_div = (flags & QCC_RECIP_DIV) ? 1 : 0;
    if (!x || !a.outer || !a.q || !a.s || (both && (!a.qk || !a.sk || !a.outer_k)) || (flags & ~(QCC_SWIZZLE | QCC_SR | QCC_RECIP_DIV)))
        return QCC_ERR_ARG;
    if ((flags & QCC_SR) && (!a.key || (both && !a.key_k))) return QCC_ERR_ARG;
    if (M < 0 || N < 0 || M > 0x7FFFFF00 || N > 0x7FFFFF00) return QCC_ERR_SHAPE;
    // output rows of M / 2 bytes are written in 16-byte pieces: M % 32 == 0; the TMA load needs N % 8 == 0
    if (M % 32 != 0 || N % 8 != 0 || (both && N % 32 != 0)) return QCC_ERR_SHAPE;
    if (!aligned16(x) || !aligned16(a.q) || !aligned16(a.s) || (both && (!aligned16(a.qk) || !aligned16(a.sk)))) return QCC_ERR_ALIGN;
    cudaStream_t st = (cudaStream_t)stream;
    CUtensorMap tx;
    {
        uint64_t dims[2] = {(uint64_t)N, (uint64_t)M};
        uint64_t strides[1] = {(uint64_t)N * 2};
        uint32_t box[2] = {64, 128};
        int e = make_tensor_map(&tx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (e) return e;
    }
    const bool swz = flags & QCC_SWIZZLE, sr = flags & QCC_SR;
    if (a.rht) {
        int e = launch_rht_check(a.rht, st);
        if (e) return e;
        return both ? launch_nvt_flags<true, true>(tx, a, swz, sr, (int)M, (int)N, st)
                    : launch_nvt_flags<false, true>(tx, a, swz, sr, (int)M, (int)N, st);
    }
    return both ? launch_nvt_flags<true, false>(tx, a, swz, sr, (int)M, (int)N, st)
                : launch_nvt_flags<false, false>(tx, a, swz, sr, (int)M, (int)N, st);
}

extern "C" int qcc_nvfp4_transposed(const void *x, int64_t M, int64_t N, const float *outer, int flags,
                                    const uint64_t *philox_key, void *q, void *s, void *stream)
{
    NvtArgs a = {outer, nullptr, philox_key, nullptr, nullptr, (uint8_t *)q, (uint8_t *)s, nullptr, nullptr};
    return nvfp4_tile_entry(x, M, N, a, flags, false, stream);
}

extern "C" int qcc_nvfp4_both(const void *x, int64_t M, int64_t N, const float *outer, int flags, void *qk, void *sk,
                              void *qm, void *sm, void *stream)
{
    if (flags & QCC_SR) return QCC_ERR_ARG;   // one key cannot serve two streams; the transform form takes two
    NvtArgs a = {outer, outer, nullptr, nullptr, nullptr, (uint8_t *)qm, (uint8_t *)sm, (uint8_t *)qk, (uint8_t *)sk};
    return nvfp4_tile_entry(x, M, N, a, flags, true, stream);
}

extern "C" int qcc_nvfp4_rht(const void *x, int64_t M, int64_t N, const float *outer_k, const float *outer_m,
                             const void *rht, int flags, const uint64_t *key_k, const uint64_t *key_m, void *qk, void *sk,
                             void *qm, void *sm, void *stream)
{
    if (!rht) return QCC_ERR_ARG;
    const bool both = qk != nullptr || sk != nullptr;
    if (both && (flags & QCC_SR)) {
        // With stochastic rounding both halves are bound by the Philox arithmetic, and the fused kernel (128 registers,
        // 4 CTAs per SM) measured 7 % slower than the rowwise stream cast followed by the tile kernel for the dim-m half.
        if (M % 32 != 0 || N % 32 != 0) return QCC_ERR_SHAPE;
        int e = qcc_nvfp4(x, M, N, outer_k, 0, flags, key_k, qk, sk, stream);
        if (e) return e;
        NvtArgs m_only = {outer_m, nullptr, key_m, nullptr, (const uint16_t *)rht, (uint8_t *)qm, (uint8_t *)sm, nullptr, nullptr};
        return nvfp4_tile_entry(x, M, N, m_only, flags, false, stream);
    }
    NvtArgs a = {outer_m, outer_k, key_m, key_k, (const uint16_t *)rht, (uint8_t *)qm, (uint8_t *)sm, (uint8_t *)qk, (uint8_t *)sk};
    return nvfp4_tile_entry(x, M, N, a, flags, both, stream);
}
