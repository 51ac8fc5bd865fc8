// fp32 -> bf16 stochastic rounding for sm_100a: the reference's `fp32_to_bf16_sr` and
// `fp32_to_bf16_sr_global_offsets` recipes (sr_bf16_f G:1841-1851, sr_bf16_global_f G:1887-1914 of
// quant_cast_bench/quant_cast_gold/recipes.py in vkuzo/quant_cast_bench).
//
// Gold: out = bf16((bits(x) + rand16) & 0xFFFF0000) with rand16 uniform in [0, 2^16) (_sr_bf16_dither G:1828-1838): the
// 16 mantissa bits bf16 drops are dithered, then truncated.  The reference draws rand16 from torch.func._random's
// stateless Philox, a module of PyTorch builds newer than the installed one, so the VALUES of the draw are this
// backend's own definition: the element with flat index g (row-major in the PARENT tensor:
// g = (global_row + i) * num_col + global_col + j, the keying of the `_global_offsets` recipe; the plain recipe is the
// case global_row = global_col = 0, num_col = N) takes 16-bit piece g & 7 of the 128 bits of
// Philox4x32-10(counter = (g >> 3) + offset, key = seed) -- piece k = half (k & 1) of word (k >> 1), low half first.
// Eight elements share one Philox call because a bf16 dither needs only 16 bits; with a whole 32-bit word per element
// the kernel ran at the rate of the integer multiplier (305 us at 16384^2) instead of the memory's.  Keyed on the global
// index, the cast of a tile equals that tile of the cast of the whole tensor.
//
// A stream kernel: a thread owns 8 consecutive elements of a row (two 16-byte loads, one 16-byte store) and, where rows
// start on a multiple of eight flat indices, one Philox call serves them; otherwise every element makes its own call.
#include "common.cuh"
#include "host_util.h"

namespace qcc {

constexpr int SRB_THREADS = 256;

__device__ __forceinline__ uint32_t sr_bf16_bits(uint32_t xbits, uint32_t word) { return (xbits + (word & 0xFFFFu)) >> 16; }

#ifndef QCC_SRB_UNROLL
#define QCC_SRB_UNROLL 4
#endif
constexpr int SRB_UNROLL = QCC_SRB_UNROLL;          // 8-element pieces per thread (their loads are all issued first)

template <bool ALIGNED>
__global__ void __launch_bounds__(SRB_THREADS)
sr_f32_to_bf16_kernel(const float *__restrict__ x, uint32_t pieces, uint32_t chunks, FastDiv32 div_chunks, int64_t N,
                      const uint64_t *__restrict__ key, int64_t global_row, int64_t global_col, int64_t num_col,
                      uint16_t *__restrict__ out)
{
    const uint64_t seed = key[0], offset = key[1];
    const uint32_t base = blockIdx.x * (SRB_THREADS * SRB_UNROLL) + threadIdx.x;   // 8-element piece; `chunks` of them per row
    uint4 a[SRB_UNROLL], b[SRB_UNROLL];
    int64_t row[SRB_UNROLL], c0[SRB_UNROLL];
    bool vec[SRB_UNROLL];
#pragma unroll
    for (int u = 0; u < SRB_UNROLL; u++) {
        const uint32_t t = base + u * SRB_THREADS;
        const uint32_t r32 = div_chunks.div(t < pieces ? t : 0u);
        row[u] = r32;
        c0[u] = (int64_t)((t < pieces ? t : 0u) - r32 * chunks) << 3;
        vec[u] = ALIGNED && t < pieces && c0[u] + 8 <= N;
        if (vec[u]) {
            const float *xr = x + row[u] * N + c0[u];
            a[u] = ld_nc_v4(xr);
            b[u] = ld_nc_v4(xr + 4);
        }
    }
#pragma unroll
    for (int u = 0; u < SRB_UNROLL; u++) {
        const uint32_t t = base + u * SRB_THREADS;
        if (t >= pieces) continue;
        uint16_t *orow = out + row[u] * N + c0[u];
        const uint64_t g0 = (uint64_t)(global_row + row[u]) * (uint64_t)num_col + (uint64_t)(global_col + c0[u]);
        if (vec[u]) {
            const uint4 w = sr_words(g0 >> 3, seed, offset);
            uint4 o;
            o.x = sr_bf16_bits(a[u].x, w.x) | (sr_bf16_bits(a[u].y, w.x >> 16) << 16);
            o.y = sr_bf16_bits(a[u].z, w.y) | (sr_bf16_bits(a[u].w, w.y >> 16) << 16);
            o.z = sr_bf16_bits(b[u].x, w.z) | (sr_bf16_bits(b[u].y, w.z >> 16) << 16);
            o.w = sr_bf16_bits(b[u].z, w.w) | (sr_bf16_bits(b[u].w, w.w >> 16) << 16);
            st_out(reinterpret_cast<uint4 *>(orow), o);
            continue;
        }
        const float *xr = x + row[u] * N + c0[u];
        for (int j = 0; j < 8 && c0[u] + j < N; j++) {
            const uint64_t g = g0 + (uint64_t)j;
            const uint4 w = sr_words(g >> 3, seed, offset);
            const uint32_t k = (uint32_t)(g & 7u), word = (k >> 1) == 0 ? w.x : (k >> 1) == 1 ? w.y : (k >> 1) == 2 ? w.z : w.w;
            orow[j] = (uint16_t)sr_bf16_bits(f2u(xr[j]), word >> (16u * (k & 1u)));
        }
    }
}

}  // namespace qcc

using namespace qcc;

extern "C" int qcc_sr_f32_to_bf16(const void *x, int64_t M, int64_t N, const uint64_t *philox_key, int64_t global_row,
                                  int64_t global_col, int64_t num_col, void *out, void *stream)
{
    if (M == 0 || N == 0) return 0;
    if (!x || !out || !philox_key || M < 0 || N < 0 || global_row < 0 || global_col < 0 || num_col < global_col + N) return QCC_ERR_ARG;
    const int64_t chunks = (N + 7) >> 3;
    if (chunks > 0x7FFFFFFF || M * chunks >= (1ll << 32) - SRB_THREADS * SRB_UNROLL) return QCC_ERR_SHAPE;
    const uint32_t pieces = (uint32_t)(M * chunks);
    FastDiv32 dv;
    dv.init((uint32_t)chunks);
    const unsigned grid = (pieces + SRB_THREADS * SRB_UNROLL - 1) / (SRB_THREADS * SRB_UNROLL);
    // the vector form: rows start on a multiple of eight flat indices and of 16 bytes
    const bool aligned = (N & 7) == 0 && (num_col & 7) == 0 && (global_col & 7) == 0 && aligned16(x) && aligned16(out);
    cudaStream_t st = (cudaStream_t)stream;
    if (aligned)
        sr_f32_to_bf16_kernel<true><<<grid, SRB_THREADS, 0, st>>>((const float *)x, pieces, (uint32_t)chunks, dv, N, philox_key, global_row, global_col,
                                                                 num_col, (uint16_t *)out);
    else
        sr_f32_to_bf16_kernel<false><<<grid, SRB_THREADS, 0, st>>>((const float *)x, pieces, (uint32_t)chunks, dv, N, philox_key, global_row, global_col,
                                                                  num_col, (uint16_t *)out);
    return (int)cudaGetLastError();
}
