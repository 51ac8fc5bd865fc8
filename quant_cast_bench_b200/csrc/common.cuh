// Shared device helpers for the sm_100a quantization-cast kernels: packed conversions (PTX cvt),
// e8m0 / e4m3 scale arithmetic in integer bit math, the 32x4x4 blocked scale layout, Philox4x32-10,
// and thin wrappers over the TMA / mbarrier PTX used by the tiled kernels.
//
// Numerics follow the gold recipes of vkuzo/quant_cast_bench
// (quant_cast_bench/quant_cast_gold/recipes.py = "G", quant_cast_gold/utils.py = "GU").
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/quant_cast_cuda.h"

namespace qcc {

// ---------------------------------------------------------------------------------------------
// bit helpers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float u2f(uint32_t u) { return __uint_as_float(u); }
__device__ __forceinline__ uint32_t f2u(float f) { return __float_as_uint(f); }

// bf16x2 word -> the two fp32 values (low half = even element)
__device__ __forceinline__ float bf16lo(uint32_t w) { return u2f(w << 16); }
__device__ __forceinline__ float bf16hi(uint32_t w) { return u2f(w & 0xFFFF0000u); }

// |a|, |b| packed maximum of two bf16x2 words (magnitudes), result is a non-negative bf16x2
__device__ __forceinline__ uint32_t absmax2(uint32_t acc, uint32_t w)
{
    __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162 *>(&acc);
    __nv_bfloat162 b = *reinterpret_cast<__nv_bfloat162 *>(&w);
    __nv_bfloat162 r = __hmax2(__habs2(a), __habs2(b));
    return *reinterpret_cast<uint32_t *>(&r);
}
// same, for an accumulator that is already non-negative
__device__ __forceinline__ uint32_t absmax2_acc(uint32_t acc, uint32_t w)
{
    __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162 *>(&acc);
    __nv_bfloat162 b = *reinterpret_cast<__nv_bfloat162 *>(&w);
    __nv_bfloat162 r = __hmax2(a, __habs2(b));
    return *reinterpret_cast<uint32_t *>(&r);
}
// max of the two halves of a non-negative bf16x2, widened to fp32 (exact)
__device__ __forceinline__ float hmax_halves_f32(uint32_t acc)
{
    uint32_t lo = acc << 16, hi = acc & 0xFFFF0000u;   // non-negative floats order like integers
    return u2f(lo > hi ? lo : hi);
}

// ---------------------------------------------------------------------------------------------
// packed conversions
// ---------------------------------------------------------------------------------------------
// two fp32 -> two fp8 in a 16-bit word; `lo` lands in the low byte.  RNE, saturate to max finite.
template <int FMT>
__device__ __forceinline__ uint32_t cvt_fp8x2(float lo, float hi)
{
    uint16_t r;
    if (FMT == QCC_FMT_E5M2)
        asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    else
        asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    return r;
}
// (a * s, b * s) with one packed fp32x2 multiply (sm_100), each lane rounded to nearest like a scalar multiply
__device__ __forceinline__ void mul2(float a, float b, float s, float &oa, float &ob)
{
#ifdef QCC_NO_F32X2
    oa = a * s;
    ob = b * s;
#else
    asm("{\n.reg .b64 x, y, z;\n"
        "mov.b64 x, {%2, %3};\n"
        "mov.b64 y, {%4, %4};\n"
        "mul.rn.f32x2 z, x, y;\n"
        "mov.b64 {%0, %1}, z;\n}\n"
        : "=f"(oa), "=f"(ob)
        : "f"(a), "f"(b), "f"(s));
#endif
}
// four fp32, all scaled by s -> four fp8 bytes in one word, element 0 in the lowest byte
template <int FMT>
__device__ __forceinline__ uint32_t scale_cvt_fp8x4(float a, float b, float c, float d, float s)
{
    float sa, sb, sc, sd;
    mul2(a, b, s, sa, sb);
    mul2(c, d, s, sc, sd);
    return cvt_fp8x2<FMT>(sa, sb) | (cvt_fp8x2<FMT>(sc, sd) << 16);
}
// four fp32 -> four fp8 bytes in one word, element 0 in the lowest byte
template <int FMT>
__device__ __forceinline__ uint32_t cvt_fp8x4(float a, float b, float c, float d)
{
    return cvt_fp8x2<FMT>(a, b) | (cvt_fp8x2<FMT>(c, d) << 16);
}
// 32 fp32-scaled values of one row block -> 32 e4m3 bytes, given the four 16-byte chunks
__device__ __forceinline__ void quant_row_block(const uint4 c[4], float rcp, uint4 &o0, uint4 &o1)
{
    o0.x = scale_cvt_fp8x4<QCC_FMT_E4M3>(bf16lo(c[0].x), bf16hi(c[0].x), bf16lo(c[0].y), bf16hi(c[0].y), rcp);
    o0.y = scale_cvt_fp8x4<QCC_FMT_E4M3>(bf16lo(c[0].z), bf16hi(c[0].z), bf16lo(c[0].w), bf16hi(c[0].w), rcp);
    o0.z = scale_cvt_fp8x4<QCC_FMT_E4M3>(bf16lo(c[1].x), bf16hi(c[1].x), bf16lo(c[1].y), bf16hi(c[1].y), rcp);
    o0.w = scale_cvt_fp8x4<QCC_FMT_E4M3>(bf16lo(c[1].z), bf16hi(c[1].z), bf16lo(c[1].w), bf16hi(c[1].w), rcp);
    o1.x = scale_cvt_fp8x4<QCC_FMT_E4M3>(bf16lo(c[2].x), bf16hi(c[2].x), bf16lo(c[2].y), bf16hi(c[2].y), rcp);
    o1.y = scale_cvt_fp8x4<QCC_FMT_E4M3>(bf16lo(c[2].z), bf16hi(c[2].z), bf16lo(c[2].w), bf16hi(c[2].w), rcp);
    o1.z = scale_cvt_fp8x4<QCC_FMT_E4M3>(bf16lo(c[3].x), bf16hi(c[3].x), bf16lo(c[3].y), bf16hi(c[3].y), rcp);
    o1.w = scale_cvt_fp8x4<QCC_FMT_E4M3>(bf16lo(c[3].z), bf16hi(c[3].z), bf16lo(c[3].w), bf16hi(c[3].w), rcp);
}

__device__ __forceinline__ float amax_of_block(const uint4 c[4])
{
    uint32_t a0 = absmax2(c[0].x, c[0].y), a1 = absmax2(c[0].z, c[0].w);
#pragma unroll
    for (int i = 1; i < 4; i++) {
        a0 = absmax2_acc(absmax2_acc(a0, c[i].x), c[i].y);
        a1 = absmax2_acc(absmax2_acc(a1, c[i].z), c[i].w);
    }
    __nv_bfloat162 x = *reinterpret_cast<__nv_bfloat162 *>(&a0), y = *reinterpret_cast<__nv_bfloat162 *>(&a1);
    __nv_bfloat162 m = __hmax2(x, y);
    return hmax_halves_f32(*reinterpret_cast<uint32_t *>(&m));
}

// e4m3 byte -> fp32 (exact)
__device__ __forceinline__ float e4m3_to_f32(uint32_t byte)
{
    uint32_t h2;
    uint16_t b = (uint16_t)byte;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(b));
    __half lo = __ushort_as_half((unsigned short)(h2 & 0xFFFFu));
    return __half2float(lo);
}
// eight fp32 -> eight fp4 e2m1 nibbles in one word, element 0 in the lowest nibble (GU:87-92).
// RNE, saturating at +-6; a negative value that rounds to zero keeps its sign (GU:52-56).
__device__ __forceinline__ uint32_t cvt_e2m1x8(const float v[8])
{
    uint32_t r;
    asm("{\n"
        ".reg .b8 b0, b1, b2, b3;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n"
        "mov.b32 %0, {b0, b1, b2, b3};\n"
        "}\n"
        : "=r"(r)
        : "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]));
    return r;
}

// ---------------------------------------------------------------------------------------------
// scale arithmetic
// ---------------------------------------------------------------------------------------------
// fp32(1/448) exactly as PyTorch rounds the Python double 1.0/448 to fp32 (G:503)
#define QCC_INV448_BITS 0x3B124925u

// amax (>= 0, an exact bf16 magnitude widened to fp32) -> e8m0 byte, RCEIL.  G:494-528:
// descale = amax * fp32(1/448); byte = biased exponent, +1 if any mantissa bit is set (for an
// fp32 subnormal: only above 2^-127); Inf/NaN -> 255.
// (inv_max_bits: fp32(1 / max_pos) of the element format, G:494-504: 1/448 for e4m3, 1/6 for e2m1)
__device__ __forceinline__ uint32_t e8m0_rceil_of(float amax, uint32_t inv_max_bits)
{
    uint32_t b = f2u(__fmul_rn(amax, u2f(inv_max_bits)));
    uint32_t add = b < 0x00800000u ? 0x3FFFFFu : 0x7FFFFFu;
    return min((b + add) >> 23, 255u);
}
__device__ __forceinline__ uint32_t e8m0_rceil(float amax) { return e8m0_rceil_of(amax, QCC_INV448_BITS); }
// FLOOR mode (OCP MX v1.0 6.3, not in the reference): exponent field of amax minus emax(e4m3)=8,
// clamped at 0; Inf/NaN -> 255.
__device__ __forceinline__ uint32_t e8m0_floor(float amax)
{
    uint32_t e = (f2u(amax) >> 23) & 0xFFu;
    return e == 0xFFu ? 255u : (e > 8u ? e - 8u : 0u);
}
// e8m0 byte -> fp32 reciprocal 2^(127-byte).  G:538-558: byte 254 -> subnormal 2^-127, 255 -> NaN.
// FLOOR clamps the scale to the smallest normal first (byte 0 behaves as byte 1).
template <bool FLOOR>
__device__ __forceinline__ float e8m0_recip(uint32_t byte)
{
    if (FLOOR) byte = max(byte, 1u);
    uint32_t r = (254u - byte) & 0xFFu;
    uint32_t bits = r << 23;
    bits = r == 0u ? 0x00400000u : bits;
    bits = r == 255u ? 0x7F800001u : bits;
    return u2f(bits);
}
template <bool FLOOR>
__device__ __forceinline__ uint32_t e8m0_from_amax(float amax)
{
    return FLOOR ? e8m0_floor(amax) : e8m0_rceil(amax);
}

// a / c for a constant c, the way the gold recipes get `tensor / python_scalar`: one IEEE division when they run on
// the CPU; under CUDA eager PyTorch multiplies by the fp32 reciprocal of the scalar instead (aten's
// BinaryDivTrueKernel.cu: "a * (1 / b)" when b is a host scalar), which differs in the last bit for about half of
// all operands.  `recip` (QCC_RECIP_DIV) selects the second form.
__device__ __forceinline__ float div_by_const(float a, float c, bool recip)
{
    return recip ? __fmul_rn(a, __fdiv_rn(1.0f, c)) : __fdiv_rn(a, c);
}

// fp8 per-tensor / per-row scale from an amax: clamp at bf16(1e-12) (the clamp happens in bf16 in
// the reference, G:304, G:1182), then the division by the format maximum.
// FMT_NVFP4_OUTER (library internal): not an fp8 format -- the row kernels then deliver the nvfp4 per-token outer scale,
// amax / (448 * 6) without a clamp (nvfp4_gs_per_token_scale G:1569-1573), and are launched without a cast.
constexpr int FMT_NVFP4_OUTER = 2;
template <int FMT>
__device__ __forceinline__ float fp8_scale_from_amax(float amax, bool recip)
{
    if (FMT == FMT_NVFP4_OUTER) return div_by_const(amax, 2688.0f, recip);
    float a = fmaxf(amax, u2f(0x2B8D0000u));
    return div_by_const(a, FMT == QCC_FMT_E5M2 ? 57344.0f : 448.0f, recip);
}

// nvfp4 inner (per-16) scale byte and the data multiplier.  G:1505-1513:
// inner = e4m3(clamp((amax / 6) / outer, 2^-6, 448)); recip = (1 / outer) / fp32(inner).
__device__ __forceinline__ uint32_t nvfp4_inner(float amax, float outer, float inv_outer, float &recip, bool recip_div)
{
    // A zero dividend sends the IEEE division down its slow path, and a warp whose lanes hold blocks of different rows
    // pays for it whenever ONE of them is an all-zero block.  0 / 6 / outer is 0 for any finite outer > 0, so there a
    // stand-in is divided and its quotient replaced by 0; for any other outer the division runs as written.
    const bool shortcut = !(amax > 0.0f) && outer > 0.0f && outer < __int_as_float(0x7F800000);
    float f = __fdiv_rn(div_by_const(shortcut ? 1.0f : amax, 6.0f, recip_div), outer);
    f = shortcut ? 0.0f : f;
    f = fminf(fmaxf(f, 0.015625f), 448.0f);
    uint32_t byte = cvt_fp8x2<QCC_FMT_E4M3>(f, 0.0f) & 0xFFu;
    recip = __fdiv_rn(inv_outer, e4m3_to_f32(byte));
    return byte;
}

// Same with the second division read from a 128-entry table in shared memory: for a per-tensor outer
// scale the multiplier (1 / outer) / fp32(inner) depends on the inner byte only, so a CTA divides once
// per possible byte (nvfp4_fill_recip_lut) instead of once per block.  Entry i is the IEEE quotient for
// byte i, hence bit-identical to nvfp4_inner.
__device__ __forceinline__ void nvfp4_fill_recip_lut(float *lut, float inv_outer)
{
    if (threadIdx.x < 128) lut[threadIdx.x] = __fdiv_rn(inv_outer, e4m3_to_f32(threadIdx.x));
}
__device__ __forceinline__ uint32_t nvfp4_inner_lut(float amax, float outer, const float *lut, float &recip, bool recip_div)
{
    // A zero dividend sends the IEEE division down its slow path (measured: 1 % all-zero rows cost the fused
    // two-orientation cast 20 %); 0 / 6 / outer is 0 for any finite outer > 0, so a stand-in is divided and its
    // quotient replaced by 0.
    float f = __fdiv_rn(div_by_const(amax > 0.0f ? amax : 1.0f, 6.0f, recip_div), outer);
    f = amax > 0.0f ? f : 0.0f;
    f = fminf(fmaxf(f, 0.015625f), 448.0f);
    uint32_t byte = cvt_fp8x2<QCC_FMT_E4M3>(f, 0.0f) & 0xFFu;
    recip = lut[byte & 127u];
    return byte;
}

// ---------------------------------------------------------------------------------------------
// 16-point randomised Hadamard transform (hadamard_rht_f G:1784-1789 with rht = diag(sign) @ H / 4)
// ---------------------------------------------------------------------------------------------
// y[j] = bf16( (1/4) sum_i sign[i] x[i] (-1)^popcount(i & j) ): in-place fp32 butterfly over strides 1, 2, 4, 8
// ((a, b) -> (a + b, a - b)), exact scaling by 1/4, one rounding to bf16.  The reference's bf16 matmul leaves
// the fp32 accumulation order to its GEMM library; this order is the one the CPU oracle restates.
constexpr unsigned int QCC_DEVERR_RHT = 17u;   // rht is not diag(+-1) @ H16 / 4

// packed fp32 pairs (sm_100 f32x2 arithmetic): two independent lanes, each rounded like the scalar operation
__device__ __forceinline__ uint64_t pack2(float lo, float hi)
{
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b)
{
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t sub2(uint64_t a, uint64_t b)
{
    uint64_t r;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
// (lo / 4, hi / 4) rounded to bf16, lo in the low half
__device__ __forceinline__ uint32_t quarter_to_bf16x2(uint64_t v)
{
    uint32_t r;
    asm("{\n.reg .b64 q, z;\n.reg .f32 lo, hi;\n"
        "mov.b64 q, {0f3E800000, 0f3E800000};\n"
        "mul.rn.f32x2 z, %1, q;\n"
        "mov.b64 {lo, hi}, z;\n"
        "cvt.rn.bf16x2.f32 %0, hi, lo;\n}\n"
        : "=r"(r)
        : "l"(v));
    return r;
}

// Sign mask of the transform from its matrix: bit i set where row i is negated (column 0 of H is all ones).
// Call with all 32 lanes of the warp.
__device__ __forceinline__ uint32_t rht_sign_mask(const uint16_t *__restrict__ rht)
{
    const uint32_t e = __ldg(rht + (threadIdx.x & 15) * 16);
    return __ballot_sync(0xFFFFFFFFu, (e >> 15) & 1u) & 0xFFFFu;
}

// Transform of two independent 16-vectors held as the low and high halves of w[0..15] (bf16x2 words), in place.
__device__ __forceinline__ void rht16_bf16x2(uint32_t (&w)[16], uint32_t sgn)
{
    uint64_t t[16];
#pragma unroll
    for (int i = 0; i < 16; i++) {
        const uint32_t word = w[i] ^ (((sgn >> i) & 1u) * 0x80008000u);
        t[i] = pack2(bf16lo(word), bf16hi(word));
    }
#pragma unroll
    for (int s = 1; s < 16; s <<= 1) {
#pragma unroll
        for (int i = 0; i < 16; i++) {
            if (!(i & s)) {
                const uint64_t a = t[i], b = t[i | s];
                t[i] = add2(a, b);
                t[i | s] = sub2(a, b);
            }
        }
    }
#pragma unroll
    for (int j = 0; j < 16; j++) w[j] = quarter_to_bf16x2(t[j]);
}

// Transform of one 16-vector of consecutive elements (eight bf16x2 words), in place.
__device__ __forceinline__ void rht16_bf16_row(uint32_t (&w)[8], uint32_t sgn)
{
    float t[16];
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const uint32_t word = w[i] ^ (((sgn >> (2 * i)) & 1u) << 15) ^ (((sgn >> (2 * i + 1)) & 1u) << 31);
        t[2 * i] = bf16lo(word);
        t[2 * i + 1] = bf16hi(word);
    }
#pragma unroll
    for (int s = 1; s < 16; s <<= 1) {
#pragma unroll
        for (int i = 0; i < 16; i++) {
            if (!(i & s)) {
                const float a = t[i], b = t[i | s];
                t[i] = __fadd_rn(a, b);
                t[i | s] = __fsub_rn(a, b);
            }
        }
    }
#pragma unroll
    for (int j = 0; j < 8; j++) w[j] = quarter_to_bf16x2(pack2(t[2 * j], t[2 * j + 1]));
}

// Offset of block scale (r, c) in the 32x4x4 blocked layout with `ncb` column blocks (G:1000-1037)
__device__ __forceinline__ size_t blocked_offset(uint32_t r, uint32_t c, uint32_t ncb)
{
    uint32_t br = r >> 7, rr = r & 127u, bc = c >> 2, c4 = c & 3u;
    return ((size_t)br * ncb + bc) * 512u + (rr & 31u) * 16u + (rr >> 5) * 4u + c4;
}

// n / d for n < 2^32 by multiply-shift (d >= 1); built on the host, passed by value to a kernel
struct FastDiv32 {
    uint32_t mul, shift;
    void init(uint32_t div)
    {
        shift = 0;
        while ((1ull << shift) < div) shift++;
        mul = (uint32_t)(((1ull << 32) * ((1ull << shift) - div)) / div + 1);
    }
    __device__ __forceinline__ uint32_t div(uint32_t n) const { return (uint32_t)(((uint64_t)__umulhi(n, mul) + n) >> shift); }
};

// Zero the padding of a blocked scale grid that a stream over the real blocks does not visit: rows
// H..ceil128(H) and scale columns W..ceil4(W).
static __global__ void blocked_zero_pad_kernel(uint8_t *__restrict__ s, uint32_t H, uint32_t W)
{
    const uint32_t Hp = ((H + 127) >> 7) << 7, Wp = ((W + 3) >> 2) << 2, ncb = Wp >> 2;
    const uint64_t total = (uint64_t)Hp * Wp;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t r = (uint32_t)(i / Wp), cc = (uint32_t)(i % Wp);
        if (r >= H || cc >= W) s[blocked_offset(r, cc, ncb)] = 0;
    }
}

// ---------------------------------------------------------------------------------------------
// Philox4x32-10 and the stochastic-rounding dither
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint4 philox4x32_10(uint4 c, uint32_t k0, uint32_t k1)
{
#pragma unroll
    for (int r = 0; r < 10; r++) {
        // (separate high / low multiplies measured 10 % faster here than one 64-bit product per word)
        uint32_t hi0 = __umulhi(0xD2511F53u, c.x), lo0 = 0xD2511F53u * c.x;
        uint32_t hi1 = __umulhi(0xCD9E8D57u, c.z), lo1 = 0xCD9E8D57u * c.z;
        c = make_uint4(hi1 ^ c.y ^ k0, lo1, hi0 ^ c.w ^ k1, lo0);
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    return c;
}
// the same with one 64-bit product per word (IMAD.WIDE): half as many multiplies
__device__ __forceinline__ uint4 philox4x32_10_wide(uint4 c, uint32_t k0, uint32_t k1)
{
#pragma unroll
    for (int r = 0; r < 10; r++) {
        const uint64_t p0 = (uint64_t)0xD2511F53u * c.x, p1 = (uint64_t)0xCD9E8D57u * c.z;
        c = make_uint4((uint32_t)(p1 >> 32) ^ c.y ^ k0, (uint32_t)p1, (uint32_t)(p0 >> 32) ^ c.w ^ k1, (uint32_t)p0);
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    return c;
}
// the four 32-bit words for elements [4g, 4g+4) of the flat stream (g = flat index >> 2)
__device__ __forceinline__ uint4 sr_words(uint64_t g, uint64_t seed, uint64_t offset)
{
    g += offset;
#ifdef QCC_PHILOX_WIDE
    return philox4x32_10_wide(make_uint4((uint32_t)g, (uint32_t)(g >> 32), 0u, 0u), (uint32_t)seed, (uint32_t)(seed >> 32));
#else
    return philox4x32_10(make_uint4((uint32_t)g, (uint32_t)(g >> 32), 0u, 0u), (uint32_t)seed,
                         (uint32_t)(seed >> 32));
#endif
}
// G:1401-1405: add a 22-bit dither into the mantissa bits fp4 discards, then truncate them
__device__ __forceinline__ float sr_dither(float d, uint32_t word)
{
    return u2f((f2u(d) + (word & 0x3FFFFFu)) & 0xFFC00000u);
}

// ---------------------------------------------------------------------------------------------
// device-side error word (bounded waits record a code here instead of hanging)
// ---------------------------------------------------------------------------------------------
// One copy per translation unit; qcc_device_error() collects them.
static __device__ unsigned int g_qcc_error = 0;

static inline int read_clear_device_error(unsigned int *out)
{
    unsigned int v = 0, zero = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, g_qcc_error, sizeof(v));
    if (e != cudaSuccess) return (int)e;
    if (v) {
        e = cudaMemcpyToSymbol(g_qcc_error, &zero, sizeof(zero));
        if (e != cudaSuccess) return (int)e;
    }
    *out = v;
    return 0;
}

// ---------------------------------------------------------------------------------------------
// TMA load / mbarrier wrappers (cluster size 1, every CTA fetches its own tile; outputs leave by plain coalesced
// stores, which measured faster than TMA stores on B200)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
// Wait for phase `parity` with an iteration cap; on timeout record the code and carry on (the caller
// then works on whatever is in shared memory, but never hangs).
__device__ __forceinline__ void mbar_wait(uint64_t *bar, uint32_t parity, unsigned int err_code)
{
    uint32_t a = smem_u32(bar);
    for (uint32_t it = 0; it < (1u << 24); it++) {
        uint32_t done;
        asm volatile(
            "{\n.reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(done)
            : "r"(a), "r"(parity)
            : "memory");
        if (done) return;
    }
    atomicMax(&g_qcc_error, err_code);
}
__device__ __forceinline__ void fence_barrier_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, uint64_t *bar, int x, int y)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void named_barrier(int id, int threads)
{
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// Programmatic dependent launch (a launch flagged QCC_PDL may begin while the kernel before it on the stream is still
// draining; it must not touch that kernel's results before pdl_wait()).  pdl_trigger() in the earlier kernel lets the
// flagged launch begin as soon as every CTA of the earlier kernel has started.  Both are no-ops in launches that are
// not part of such a pair.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// a per-tensor scalar that an overlapped predecessor wrote: read past L1 (which may hold what an earlier kernel saw)
__device__ __forceinline__ float ld_cg_f32(const float *p)
{
    float v;
    asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
    return v;
}

// Output stores of the streaming kernels: evict-first (st.global.cs) unless built with QCC_PLAIN_STORES
template <class T>
__device__ __forceinline__ void st_out(T *p, T v)
{
#ifdef QCC_PLAIN_STORES
    *p = v;
#else
    __stcs(p, v);
#endif
}

// 16-byte vector access
__device__ __forceinline__ uint4 ld_nc_v4(const void *p)
{
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}
// 16-byte load that allocates in L1: for threads that read several neighbouring 16-byte pieces of the
// same sectors with separate instructions (measured +9 % on the 64-bytes-per-thread streams)
__device__ __forceinline__ uint4 ld_v4(const void *p)
{
    uint4 r;
    asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}
__device__ __forceinline__ uint4 lds_v4(uint32_t addr)
{
    uint4 r;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "r"(addr));
    return r;
}
__device__ __forceinline__ uint2 lds_v2(uint32_t addr)
{
    uint2 r;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(r.x), "=r"(r.y) : "r"(addr));
    return r;
}
__device__ __forceinline__ void sts_v4(uint32_t addr, uint4 v)
{
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

}  // namespace qcc
