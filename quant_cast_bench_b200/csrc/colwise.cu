// fp8 colwise cast in one launch that reads x from HBM once, sm_100a.
//
// colwise_fp8_f (quant_cast_bench/quant_cast_gold/recipes.py:339-349 of vkuzo/quant_cast_bench) needs the maximum of a
// whole column before the first byte of it can be cast, so x is read twice; what can be chosen is where the second
// read comes from.  The matrix is cut into panels of 64 * strips columns (all M rows; about 8 MB), small enough that
// the panels between a panel's two reads stay in L2.  One persistent CTA per SM owns a run of up to CWR_TILES 64 x 64
// tiles of one 64-column strip of every panel, and per step i
//     1. reduces its tiles of panel i (TMA loads from HBM, two buffers) to 64 column maxima, which warp 0 merges into
//        the global maxima (64 atomics per CTA) before it adds one to the panel's counter;
//     2. casts its tiles of panel i - lag (TMA loads again, now L2 hits, two more buffers) with the final maxima,
//        transposes them in place and writes them out;
//     3. issues the loads of both streams two steps ahead.
// A signal takes 2 to 3 us from one SM through L2 to all others, longer than a step (about 2 us); with the cast
// lag = 4 or 5 steps behind the maxima, the counter a cast depends on was completed long before, and the wait for it
// (bounded) costs nothing.  That wait, the read of the final maxima and their turn into reciprocal scales are done a
// step ahead by a warp of their own, so that the cast warps never see an L2 latency.
//
// Warp roles (16 warps): 0 merges and signals (it joins the others only at the barrier that hands it the partial
// maxima); 1..4 compute partial maxima, then cast; 1..14 cast, two warps per tile; 15 prepares the next step's scales.
//
// CTAs wait on one another, so all of them must be resident: the grid is the SM count with one CTA per SM (the
// shared-memory footprint allows no second one), launched cooperatively.  All waits are bounded in time and report
// through the device error word.
#include "common.cuh"
#include "host_util.h"

namespace qcc {

constexpr int CWR_TILES = 7;                       // 64 x 64 tiles per CTA and panel
constexpr int CWR_NBUF = 4;                        // two buffers for the maxima stream, two for the cast stream
constexpr int CWR_LAG = 5;                         // a panel is cast this many steps after its maxima (measured best of 2..7
                                                   // at 64 panels; 4 with fewer than 40 panels); the load prologue needs >= 2
static_assert(CWR_LAG >= 3, "the cast stream's first loads are issued in steps lag - 2 and lag - 1");
constexpr int CWR_TILE_BYTES = 64 * 128;
constexpr int CWR_BUF_BYTES = CWR_TILES * CWR_TILE_BYTES;
constexpr int CWR_WARPS = 16;
constexpr int CWR_XWARPS = 4;                                  // warps that reduce the tiles to partial maxima
constexpr int CWR_RED_OFF = CWR_NBUF * CWR_BUF_BYTES;          // 2 x [CWR_XWARPS][8 column chunks] uint4
constexpr int CWR_RCP_OFF = CWR_RED_OFF + 2 * CWR_XWARPS * 8 * 16;   // 2 x 64 reciprocal scales
constexpr int CWR_BAR_OFF = CWR_RCP_OFF + 2 * 64 * 4;
constexpr int CWR_ALLOC = CWR_BAR_OFF + 64 + 1024;             // 1024: the buffers start on a 1024-byte boundary
constexpr int CWR_THREADS = 32 * CWR_WARPS;
static_assert(CWR_ALLOC <= 232448, "shared memory of one CTA");
static_assert(CWR_WARPS >= 1 + 2 * CWR_TILES, "one control warp and two cast warps per tile");
constexpr unsigned int QCC_DEVERR_COLWISE_TMA = 7;             // a panel's loads did not arrive
constexpr unsigned int QCC_DEVERR_COLWISE_WAIT = 18;           // a panel's counter did not fill up

__device__ __forceinline__ void red_release_add(uint32_t *p, uint32_t v)
{
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_u32(const uint32_t *p)
{
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint64_t global_timer_ns()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
// Waits of this kernel give up after 50 ms of wall time, and at once when a wait of the same launch has given up before
// (`abort_word`, cleared with the counters before every launch): a launch that goes wrong ends within a fraction of a
// second.  The code of the first failure also goes to the device error word, which stays set until it is read.
constexpr uint64_t CWR_WAIT_NS = 50ull * 1000 * 1000;
__device__ __forceinline__ void give_up(uint32_t *abort_word, unsigned int err_code)
{
    atomicMax(abort_word, err_code);
    atomicMax(&g_qcc_error, err_code);
}
__device__ __forceinline__ void mbar_wait_timed(uint64_t *bar, uint32_t parity, uint32_t *abort_word, unsigned int err_code)
{
    const uint32_t a = smem_u32(bar);
    const uint64_t start = global_timer_ns();
    for (uint32_t n = 1;; n++) {
        uint32_t ok;
        asm volatile(
            "{\n.reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(ok)
            : "r"(a), "r"(parity)
            : "memory");
        if (ok) return;
        if (n & 15) continue;                                   // a try_wait itself blocks for a while: look up rarely
        if (*(volatile uint32_t *)abort_word != 0) return;
        if (global_timer_ns() - start > CWR_WAIT_NS) break;
    }
    give_up(abort_word, err_code);
}
__device__ __forceinline__ uint64_t l2_policy_evict_first()
{
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last()
{
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ void tma_load_2d_hint(void *dst, const CUtensorMap *map, uint64_t *bar, int x, int y, uint64_t pol)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y), "l"(pol)
        : "memory");
}
__device__ __forceinline__ void st_v4_evict_first(void *p, uint4 v, uint64_t pol)
{
    asm volatile("st.global.L2::cache_hint.v4.u32 [%0], {%1,%2,%3,%4}, %5;" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w), "l"(pol) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// done[32 p]: CTAs that have merged their maxima of panel p (one counter per 128-byte line: they are polled);
// done[32 np]: the launch's abort word.
template <int FMT>
__global__ void __launch_bounds__(CWR_THREADS, 1)
fp8_colwise_resident_kernel(const __grid_constant__ CUtensorMap tm_x, uint32_t *amax_bits, uint32_t *done,
                            uint8_t *__restrict__ q, float *__restrict__ scale_out, int M, int N, int strips, int np, int lag,
                            int recip_div)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *sbase = smem_raw + (base - smem_u32(smem_raw));
    uint4 *s_red = reinterpret_cast<uint4 *>(sbase + CWR_RED_OFF);
    float *s_rcp = reinterpret_cast<float *>(sbase + CWR_RCP_OFF);
    uint64_t *bar = reinterpret_cast<uint64_t *>(sbase + CWR_BAR_OFF);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    uint32_t *abort_word = done + 32 * np;
    const uint64_t pol_first = l2_policy_evict_first();

    // this CTA: one 64-column strip of every panel, a run of row tiles of it
    const int strip = blockIdx.x % strips, rank = blockIdx.x / strips;
    const int n_rank = ((int)gridDim.x - strip + strips - 1) / strips;
    const int tiles_m = (M + 63) >> 6;
    const int t0 = (int)(((long long)rank * tiles_m) / n_rank), t1 = (int)(((long long)(rank + 1) * tiles_m) / n_rank);
    const int nt = t1 - t0;                                                 // <= CWR_TILES (checked on the host)

    if (tid == 0) {
#pragma unroll
        for (int k = 0; k < CWR_NBUF; k++) mbar_init(bar + k, 1);
        fence_barrier_init();
    }
    __syncthreads();
    // one thread: loads of panel p into buffer b (0, 1: maxima stream; 2, 3: cast stream) on barrier b
    uint32_t issued0 = 0, issued1 = 0, issued2 = 0, issued3 = 0;   // (thread 32) loads posted per buffer
    uint32_t abort_seen = 0;                  // (thread 32) the launch's abort word as read at the top of the step
    auto issue = [&](int p, int b) {
        const int col0 = (p * strips + strip) * 64;
        if (col0 >= N || nt == 0) return;
        if (abort_seen != 0) return;                             // a wait of this launch has given up: post nothing more
        if (b == 0) issued0++; else if (b == 1) issued1++; else if (b == 2) issued2++; else issued3++;
        mbar_expect_tx(bar + b, (uint32_t)nt * CWR_TILE_BYTES);
        // L2: keep what the maxima stream brings in, let go of what the cast stream has re-read (measured: 192 -> 172 us
        // at 16384^2; with the outputs written evict-first as well 167 us)
        const uint64_t pol = b < 2 ? l2_policy_evict_last() : pol_first;
        for (int k = 0; k < nt; k++)
            tma_load_2d_hint(sbase + b * CWR_BUF_BYTES + k * CWR_TILE_BYTES, &tm_x, bar + b, col0, (t0 + k) * 64, pol);
    };
    if (tid == 32)
        for (int p = 0; p < 2 && p < np; p++) issue(p, p);

    for (int i = 0; i < np + lag; i++) {
        const int p = i - lag;                                              // the panel cast in this step
        if (tid == 32) abort_seen = *(volatile uint32_t *)abort_word;       // read now, used at the end of the step
        const int col0_x = (i * strips + strip) * 64, col0_c = (p * strips + strip) * 64;
        const bool have_x = i < np && col0_x < N && nt > 0;
        const bool have_c = p >= 0 && col0_c < N && nt > 0;
        uint4 *red = s_red + (i & 1) * (CWR_XWARPS * 8);
        if (warp == 0) {
            // ---- control warp: merge the partial maxima of panel i into the global ones, then signal
            named_barrier(1, 32 * (1 + CWR_XWARPS));
            if (i < np) {
                if (have_x && lane < 8) {
                    uint4 m = red[lane];
#pragma unroll
                    for (int w = 1; w < CWR_XWARPS; w++) {
                        const uint4 o = red[w * 8 + lane];
                        m.x = absmax2_acc(m.x, o.x); m.y = absmax2_acc(m.y, o.y); m.z = absmax2_acc(m.z, o.z); m.w = absmax2_acc(m.w, o.w);
                    }
                    const int col = col0_x + lane * 8;
                    if (col < N) {
                        uint32_t *dst = amax_bits + col;
                        const uint32_t acc[4] = {m.x, m.y, m.z, m.w};
#pragma unroll
                        for (int k = 0; k < 4; k++) {
                            atomicMax(dst + 2 * k, acc[k] << 16);
                            atomicMax(dst + 2 * k + 1, acc[k] & 0xFFFF0000u);
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) red_release_add(done + 32 * i, 1u);
            }
            continue;                                                           // warp 0 takes no part in the other barrier
        }
        // ---- 1. partial maxima of panel i: warp w = 1 .. CWR_XWARPS takes 64 / CWR_XWARPS rows of every tile,
        //         lane = (16-byte column chunk cg, rows rg, rg + 4, ...)
        if (warp <= CWR_XWARPS) {
            if (have_x) {
                constexpr int RW = 64 / CWR_XWARPS;                             // rows per warp
                const int bx = i & 1;
                const int cg = lane & 7, rg = lane >> 3;
                uint32_t a0 = 0, a1 = 0, a2 = 0, a3 = 0;
                mbar_wait_timed(bar + bx, (uint32_t)(i >> 1) & 1u, abort_word, QCC_DEVERR_COLWISE_TMA);
                const uint32_t src = base + bx * CWR_BUF_BYTES + (RW * (warp - 1) + rg) * 128;
                for (int k = 0; k < nt; k++) {
#pragma unroll
                    for (int r = 0; r < RW / 4; r++) {
                        const uint4 v = lds_v4(src + k * CWR_TILE_BYTES + 4 * r * 128 + ((cg ^ ((rg + 4 * r) & 7)) << 4));
                        a0 = absmax2_acc(a0, v.x); a1 = absmax2_acc(a1, v.y); a2 = absmax2_acc(a2, v.z); a3 = absmax2_acc(a3, v.w);
                    }
                }
#pragma unroll
                for (int d = 8; d <= 16; d <<= 1) {
                    a0 = absmax2_acc(a0, __shfl_xor_sync(0xFFFFFFFFu, a0, d)); a1 = absmax2_acc(a1, __shfl_xor_sync(0xFFFFFFFFu, a1, d));
                    a2 = absmax2_acc(a2, __shfl_xor_sync(0xFFFFFFFFu, a2, d)); a3 = absmax2_acc(a3, __shfl_xor_sync(0xFFFFFFFFu, a3, d));
                }
                if (lane < 8) red[(warp - 1) * 8 + cg] = make_uint4(a0, a1, a2, a3);
            }
            named_barrier(1, 32 * (1 + CWR_XWARPS));                            // also: warp 0 has read the scratch of two steps ago
        }
        if (warp == CWR_WARPS - 1) {
            // ---- scale warp: when the counter of the panel cast in the NEXT step (signalled lag - 1 steps ago) shows
            //      every CTA, turn its 64 final maxima into reciprocal scales for the cast warps
            const int pn = p + 1, col0_n = (pn * strips + strip) * 64;
            if (pn >= 0 && pn < np && col0_n < N && nt > 0) {
                if (lane == 0) {
                    const uint64_t start = global_timer_ns();
                    while (ld_acquire_u32(done + 32 * pn) < gridDim.x) {
                        if (*(volatile uint32_t *)abort_word != 0) break;
                        if (global_timer_ns() - start > CWR_WAIT_NS) {
                            give_up(abort_word, QCC_DEVERR_COLWISE_WAIT);
                            break;
                        }
                        __nanosleep(100);
                    }
                }
                __syncwarp();
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const int c = lane + 32 * h, Cn = col0_n + c;
                    float s = 1.0f;
                    if (Cn < N) {
                        s = fp8_scale_from_amax<FMT>(u2f(__ldcg(amax_bits + Cn)), recip_div != 0);
                        if (t0 == 0) scale_out[Cn] = s;                         // the owner of row tile 0
                    }
                    s_rcp[(pn & 1) * 64 + c] = __fdiv_rn(1.0f, s);
                }
            }
        }
        else if (have_c && (warp - 1) >> 1 < nt) {
            // ---- 2. cast of panel p: warps 2 t + 1 and 2 t + 2 cast the upper and the lower 32-row slab of tile t;
            //         lane = (l16: four adjacent columns, rh: 16-row half of the slab)
            const int tk = (warp - 1) >> 1, hb = (warp - 1) & 1;
            const int l16 = lane & 15, rh = lane >> 4;
            const float4 sc = *reinterpret_cast<const float4 *>(s_rcp + (p & 1) * 64 + 4 * l16);
            mbar_wait_timed(bar + 2 + (p & 1), (uint32_t)(p >> 1) & 1u, abort_word, QCC_DEVERR_COLWISE_TMA);
            const uint32_t slab = base + (2 + (p & 1)) * CWR_BUF_BYTES + tk * CWR_TILE_BYTES + hb * 4096;
            const uint32_t pbase = slab + (rh * 16) * 128 + (l16 & 1) * 8;
            const uint32_t j = l16 >> 1;
            uint32_t o[4][4];
#pragma unroll
            for (int q4 = 0; q4 < 4; q4++) {
                uint2 w[4];
#pragma unroll
                for (int r = 0; r < 4; r++) w[r] = lds_v2(pbase + (4 * q4 + r) * 128 + ((j ^ ((4 * q4 + r) & 7)) << 4));
                o[0][q4] = scale_cvt_fp8x4<FMT>(bf16lo(w[0].x), bf16lo(w[1].x), bf16lo(w[2].x), bf16lo(w[3].x), sc.x);
                o[1][q4] = scale_cvt_fp8x4<FMT>(bf16hi(w[0].x), bf16hi(w[1].x), bf16hi(w[2].x), bf16hi(w[3].x), sc.y);
                o[2][q4] = scale_cvt_fp8x4<FMT>(bf16lo(w[0].y), bf16lo(w[1].y), bf16lo(w[2].y), bf16lo(w[3].y), sc.z);
                o[3][q4] = scale_cvt_fp8x4<FMT>(bf16hi(w[0].y), bf16hi(w[1].y), bf16hi(w[2].y), bf16hi(w[3].y), sc.w);
            }
            __syncwarp();                                                       // the slab has been read: transpose in place
            // staging in the slab's own memory: sub-tile k = columns {4 l16 + k}: 16 rows of 32 bytes (the 32 rows of the
            // slab, as fp8); of the two 16-byte chunks of row l16, chunk c sits at c ^ ((l16 >> 2) & 1)
            const uint32_t key = (l16 >> 2) & 1;
#pragma unroll
            for (int k = 0; k < 4; k++)
                sts_v4(slab + k * 512 + l16 * 32 + ((rh ^ key) << 4), make_uint4(o[k][0], o[k][1], o[k][2], o[k][3]));
            __syncwarp();
            const int jj = lane & 1;
            const int mcol = (t0 + tk) * 64 + hb * 32 + jj * 16;
#pragma unroll
            for (int it = 0; it < 4; it++) {
                const int slot = it * 16 + (lane >> 1);
                const int k = slot >> 4, l = slot & 15;
                const int Cn = col0_c + 4 * l + k;
                const uint4 v = lds_v4(slab + k * 512 + l * 32 + ((jj ^ ((l >> 2) & 1)) << 4));
                if (Cn < N && mcol < M) st_v4_evict_first(q + (size_t)Cn * M + mcol, v, pol_first);
            }
        }
        named_barrier(2, 32 * (CWR_WARPS - 1));                                 // both buffers of this step are free
        // ---- 3. next loads: panel i + 2 for its maxima (from HBM), panel p + 2 for its cast (from L2)
        if (tid == 32) {
            fence_proxy_async_smem();
            if (i + 2 < np) issue(i + 2, i & 1);
            if (p + 2 >= 0 && p + 2 < np) issue(p + 2, 2 + (p & 1));
        }
    }
    // After a wait has given up the consumers no longer wait for their loads, so copies may still be in flight into this
    // CTA's shared memory: the issuing thread waits (bounded) for the last phase of every buffer before the CTA ends.
    if (tid == 32 && *(volatile uint32_t *)abort_word != 0) {
        const uint32_t issued[CWR_NBUF] = {issued0, issued1, issued2, issued3};
        static_assert(CWR_NBUF == 4, "four buffers");
#pragma unroll
        for (int b = 0; b < CWR_NBUF; b++) {
            if (issued[b] == 0) continue;
            const uint32_t a = smem_u32(bar + b), parity = (issued[b] - 1u) & 1u;
            const uint64_t start = global_timer_ns();
            for (;;) {
                uint32_t ok;
                asm volatile(
                    "{\n.reg .pred p;\n"
                    "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
                    "selp.u32 %0, 1, 0, p;\n}\n"
                    : "=r"(ok)
                    : "r"(a), "r"(parity)
                    : "memory");
                if (ok || global_timer_ns() - start > CWR_WAIT_NS) break;
            }
        }
    }
}

// Largest number of 64-column strips per panel (<= 16) for which a CTA's run of row tiles fits its buffers; 0: none.
static int resident_strips(int64_t M, int64_t N, int grid)
{
    const int64_t tiles_m = (M + 63) / 64;
    int best = 0;
    for (int s = 1; s <= 16 && s <= grid && (int64_t)(s - 1) * 64 < N; s++)
        if ((tiles_m + grid / s - 1) / (grid / s) <= CWR_TILES) best = s;
    return best;
}

template <int FMT>
static int launch_resident(const CUtensorMap &tx, uint32_t *amax_bits, uint32_t *done, void *q, float *scale_out, int64_t M,
                           int64_t N, int strips, int np, int grid, int recip_div, cudaStream_t st)
{
    auto kern = fp8_colwise_resident_kernel<FMT>;
    static PerDeviceFlag configured, cooperative;
    const int dev = current_device_slot();
    if (dev < 0) return QCC_ERR_ARG;
    if (!configured.get(dev)) {
        int coop = 0;
        if (cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev) == cudaSuccess && coop) cooperative.set(dev);
        cudaError_t ce = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, CWR_ALLOC);
        if (ce != cudaSuccess) return (int)ce;
        configured.set(dev);
    }
    if (!cooperative.get(dev)) return 1;                      // no cooperative launches here: two-launch form
    uint8_t *qp = (uint8_t *)q;
    int Mi = (int)M, Ni = (int)N;
    int lag = np >= 40 ? CWR_LAG : CWR_LAG - 1;               // few panels: the steps that only drain the pipeline weigh more
    void *args[] = {(void *)&tx, &amax_bits, &done, &qp, &scale_out, &Mi, &Ni, &strips, &np, &lag, &recip_div};
    const cudaError_t ce = cudaLaunchCooperativeKernel((const void *)kern, dim3((unsigned)grid), dim3(CWR_THREADS), args, CWR_ALLOC, st);
    if (ce == cudaErrorCooperativeLaunchTooLarge || ce == cudaErrorNotSupported || ce == cudaErrorLaunchOutOfResources) {
        cudaGetLastError();                                   // fewer SMs available than the device reports, or the context
        return 1;                                             // refuses the launch form: the two-launch form works there
    }
    return (int)ce;
}

}  // namespace qcc

using namespace qcc;

// Returns 1 when the shape does not fit the resident form (the caller then takes the two-pass form), 0 on success,
// else an error.  amax_bits: N words followed by 128 + 128 * (1 + ceil(N / 64)) bytes for the panel counters and the
// abort word.
int qcc_colwise_resident(const void *x, int64_t M, int64_t N, int fmt, void *q, float *scale_out, uint32_t *amax_bits,
                         cudaStream_t st)
{
    const int recip_div = take_recip_div(fmt);   // the caller passes QCC_RECIP_DIV inside fmt
    const int grid = sm_count();
    const int strips = resident_strips(M, N, grid);
    if (strips == 0) return 1;
    CUtensorMap tx;
    uint64_t dims[2] = {(uint64_t)N, (uint64_t)M};
    uint64_t strides[1] = {(uint64_t)N * 2};
    uint32_t box[2] = {64, 64};
    int e = make_tensor_map(&tx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (e) return e;
    const int np = (int)((N + 64 * strips - 1) / (64 * strips));
    uint32_t *done = (uint32_t *)(((uintptr_t)(amax_bits + N) + 127) & ~(uintptr_t)127);
    cudaError_t ce = cudaMemsetAsync(amax_bits, 0, (size_t)((uint8_t *)(done + 32 * (np + 1)) - (uint8_t *)amax_bits), st);
    if (ce != cudaSuccess) return (int)ce;
    return fmt == QCC_FMT_E5M2 ? launch_resident<QCC_FMT_E5M2>(tx, amax_bits, done, q, scale_out, M, N, strips, np, grid, recip_div, st)
                               : launch_resident<QCC_FMT_E4M3>(tx, amax_bits, done, q, scale_out, M, N, strips, np, grid, recip_div, st);
}

extern "C" int qcc_colwise_device_error(unsigned int *out) { return read_clear_device_error(out); }
