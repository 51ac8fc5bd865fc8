// 16-point randomised Hadamard transform of bf16 data for sm_100a: the standalone transform along the rows
// (hadamard_rht_f, quant_cast_gold/recipes.py:1784-1789 of vkuzo/quant_cast_bench) and the maximum of
// |RHT(x.t())| that gives the dim-m outer scale of the two-orientation nvfp4 cast (recipes.py:1364-1365).
// The transform itself (butterfly order, rounding) is rht16_bf16x2 / rht16_bf16_row of common.cuh; the cast
// that applies it down the rows lives with the nvfp4 tile kernel.
#include "common.cuh"
#include "host_util.h"

namespace qcc {

constexpr int RHT_THREADS = 256;

// One thread per 16-element block of a row: two 16-byte loads, two 16-byte stores.
__global__ void __launch_bounds__(RHT_THREADS)
hadamard_rht_rows_kernel(const uint4 *__restrict__ x, uint4 *__restrict__ y, uint32_t n_blocks,
                         const uint16_t *__restrict__ rht)
{
    const uint32_t sgn = rht_sign_mask(rht);
    const uint32_t bi = blockIdx.x * RHT_THREADS + threadIdx.x;
    if (bi >= n_blocks) return;
    const uint4 a = ld_nc_v4(x + 2 * (size_t)bi), b = ld_nc_v4(x + 2 * (size_t)bi + 1);
    uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    rht16_bf16_row(w, sgn);
    st_out(y + 2 * (size_t)bi, make_uint4(w[0], w[1], w[2], w[3]));
    st_out(y + 2 * (size_t)bi + 1, make_uint4(w[4], w[5], w[6], w[7]));
}

// max |RHT(x.t())|: a warp takes 16 rows x 128 columns (lane = four adjacent columns), transforms down the rows
// and keeps the packed bf16 maximum; one atomic max per CTA on the bits of a non-negative fp32.
#ifndef QCC_RHTA_MINCTAS
#define QCC_RHTA_MINCTAS 3   // 80 registers (a few spilled words) and 3 CTAs per SM: 6 % faster than 101 registers and 2
#endif
#ifndef QCC_RHTA_CTAS_PER_SM
#define QCC_RHTA_CTAS_PER_SM 16
#endif
__global__ void __launch_bounds__(RHT_THREADS, QCC_RHTA_MINCTAS)
rht_t_amax_kernel(const uint16_t *__restrict__ x, int M, int N, const uint16_t *__restrict__ rht,
                  unsigned int *__restrict__ out_bits)
{
    __shared__ uint32_t s_max[RHT_THREADS / 32];
    const uint32_t sgn = rht_sign_mask(rht);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int col_groups = (N + 127) >> 7;
    const long long items = (long long)(M >> 4) * col_groups;
    uint32_t acc = 0;
    for (long long it = (long long)blockIdx.x * (RHT_THREADS / 32) + warp; it < items;
         it += (long long)gridDim.x * (RHT_THREADS / 32)) {
        const int rb = (int)(it / col_groups), cg = (int)(it - (long long)rb * col_groups);
        const int c = cg * 128 + lane * 4;
        if (c < N) {   // N % 4 == 0: the four columns are inside together
            const uint16_t *p = x + (size_t)rb * 16 * N + c;
            uint32_t wx[16], wy[16];
#pragma unroll
            for (int r = 0; r < 16; r++) {
                const uint2 v = __ldg(reinterpret_cast<const uint2 *>(p + (size_t)r * N));
                wx[r] = v.x;
                wy[r] = v.y;
            }
            rht16_bf16x2(wx, sgn);
            rht16_bf16x2(wy, sgn);
#pragma unroll
            for (int r = 0; r < 16; r++) acc = absmax2_acc(absmax2_acc(acc, wx[r]), wy[r]);
        }
    }
    uint32_t m = f2u(hmax_halves_f32(acc));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const uint32_t other = __shfl_xor_sync(0xFFFFFFFFu, m, o);
        m = other > m ? other : m;
    }
    if (lane == 0) s_max[warp] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int i = 1; i < RHT_THREADS / 32; i++) m = s_max[i] > m ? s_max[i] : m;
        atomicMax(out_bits, m);
    }
}

__global__ void rht_amax_finish_kernel(float *out, int mode)
{
    if ((mode & ~QCC_RECIP_DIV) == QCC_AMAX_NVFP4_SCALE) out[0] = div_by_const(out[0], 2688.0f, mode & QCC_RECIP_DIV);   // 448 * 6, no clamp (G:1365)
}

}  // namespace qcc

using namespace qcc;

extern "C" int qcc_hadamard_rht(const void *x, int64_t M, int64_t N, const void *rht, void *y, void *stream)
{
    if (M == 0 || N == 0) return 0;
    if (!x || !rht || !y) return QCC_ERR_ARG;
    if (M < 0 || N < 0 || N % 16 != 0 || M * (N / 16) >= (1ll << 32) - RHT_THREADS) return QCC_ERR_SHAPE;
    if (!aligned16(x) || !aligned16(y)) return QCC_ERR_ALIGN;
    cudaStream_t st = (cudaStream_t)stream;
    int e = launch_rht_check(rht, st);
    if (e) return e;
    const uint32_t n_blocks = (uint32_t)(M * (N / 16));
    hadamard_rht_rows_kernel<<<(n_blocks + RHT_THREADS - 1) / RHT_THREADS, RHT_THREADS, 0, st>>>(
        (const uint4 *)x, (uint4 *)y, n_blocks, (const uint16_t *)rht);
    return (int)cudaGetLastError();
}

extern "C" int qcc_nvfp4_rht_amax(const void *x, int64_t M, int64_t N, const void *rht, int mode, float *out, void *stream)
{
    if (!x || !rht || !out || ((mode & ~QCC_RECIP_DIV) != QCC_AMAX_RAW && (mode & ~QCC_RECIP_DIV) != QCC_AMAX_NVFP4_SCALE)) return QCC_ERR_ARG;
    if (M <= 0 || N <= 0 || M % 16 != 0 || N % 4 != 0 || M > 0x7FFFFF00 || N > 0x7FFFFF00) return QCC_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(x) & 7u) != 0) return QCC_ERR_ALIGN;
    cudaStream_t st = (cudaStream_t)stream;
    int e = launch_rht_check(rht, st);
    if (e) return e;
    cudaError_t ce = cudaMemsetAsync(out, 0, sizeof(float), st);
    if (ce != cudaSuccess) return (int)ce;
    const long long items = (M / 16) * ((N + 127) / 128);
    long long grid = (items + RHT_THREADS / 32 - 1) / (RHT_THREADS / 32);
    const long long cap = (long long)sm_count() * QCC_RHTA_CTAS_PER_SM;
    if (grid > cap) grid = cap;
    rht_t_amax_kernel<<<(unsigned)grid, RHT_THREADS, 0, st>>>((const uint16_t *)x, (int)M, (int)N, (const uint16_t *)rht,
                                                            (unsigned int *)out);
    if ((ce = cudaGetLastError()) != cudaSuccess) return (int)ce;
    rht_amax_finish_kernel<<<1, 1, 0, st>>>(out, mode);
    return (int)cudaGetLastError();
}
