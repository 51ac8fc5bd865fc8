/*
 * quant_cast_cuda -- C ABI of the sm_100a quantization-cast kernels.
 *
 * Every entry point takes plain device pointers and sizes plus the CUDA stream to launch on
 * (a cudaStream_t passed as void*; NULL = the legacy default stream).  Nothing here allocates device
 * memory, synchronises the device, or keeps mutable host state: outputs and scratch are supplied
 * by the caller and launches are asynchronous.
 *
 * Return value: 0 on success; a negative QCC_ERR_* for a rejected argument (nothing was launched);
 * a positive value is the cudaError_t of a failed launch.
 *
 * Each function replaces the body of one gold recipe of vkuzo/quant_cast_bench; the citation gives
 * the reference definition ("G" = quant_cast_bench/quant_cast_gold/recipes.py).  A backend recipe
 * file in the style of quant_cast_bench/quant_cast_triton/recipes.py:48-65 binds these through
 * ctypes (see quant_cast_bench_b200/quant_cast_cuda/recipes.py).
 *
 * Common conventions: x is a contiguous row-major (M, N) bf16 matrix; pointers must be 16-byte
 * aligned; outputs are contiguous; one-byte scales are raw bytes (e8m0 / e4m3 bit patterns); the
 * "blocked" scale layout is the (ceil(H/128), ceil(W/4), 32, 16) grid of G:1000-1037 with padding
 * written as zero.
 */
#ifndef QUANT_CAST_CUDA_H
#define QUANT_CAST_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element formats of the fp8 casts */
#define QCC_FMT_E4M3 0 /* torch.float8_e4m3fn, max 448 */
#define QCC_FMT_E5M2 1 /* torch.float8_e5m2, max 57344 (not in the reference; same recipe, other dtype) */

/* flags of the block-scaled casts */
#define QCC_ROWWISE 1  /* blocks along the last dim; outputs in the frame of x                       */
#define QCC_COLWISE 2  /* blocks down the rows; outputs in the transposed (N, M) frame               */
#define QCC_SWIZZLE 4  /* block scales in the blocked 32x4x4 layout instead of plain row-major      */
#define QCC_FLOOR 8    /* mxfp8: FLOOR scale mode (OCP MX v1.0) instead of RCEIL                     */
#define QCC_SR 16      /* nvfp4: stochastic rounding of the fp4 values, Philox4x32-10 keyed          */
#define QCC_BLOCK32 32 /* mxfp8: one scale per 32x32 block instead of per 1x32 / 32x1 block        */
#define QCC_REVERSE 0x400 /* qcc_nvfp4 / qcc_nvfp4_from_amax: walk the tensor from its end.  Results do not change; a cast
                             that follows another pass over the same tensor (its amax, its mxfp8 cast) then begins with
                             the rows that pass touched last, which are still in L2.                                   */
#define QCC_PDL 0x200  /* qcc_nvfp4 (blocked scales, one outer scale, round to nearest): programmatic dependent launch --
                          the cast may start, and load x, while the kernel before it on the stream (the one that writes
                          the outer scale, i.e. qcc_xchg_resolve) is still running; it waits for that kernel before it
                          reads the scale.  Only for a launch directly behind the kernel that writes `outer`.        */

/* How a tensor is divided by a constant (amax / 448, amax / 57344, amax / 2688, block amax / 6).  The gold recipes
 * write `tensor / python_scalar`: PyTorch's CPU kernels compute that as one IEEE division, its CUDA kernels as a
 * multiplication with the fp32 reciprocal of the scalar (aten/src/ATen/native/cuda/BinaryDivTrueKernel.cu), and the two
 * differ in the last bit for about half of all operands.  Default: the IEEE division (the gold recipes on the CPU).
 * With QCC_RECIP_DIV: a * fl(1 / c), bit-identical to the gold recipes run eagerly on a CUDA device.  Accepted in the
 * `mode` of the amax entry points (qcc_amax_bf16, qcc_amax_bf16_noalloc, qcc_scale_from_amax, qcc_xchg_resolve,
 * qcc_amax_block128x128, qcc_nvfp4_rht_amax), in the `fmt` of qcc_fp8_tensorwise_from_amax, qcc_fp8_rowwise and
 * qcc_fp8_colwise, and in the `flags` of qcc_fp8_block128, qcc_fp8_block128x128, qcc_nvfp4_per_token_scale and every
 * qcc_nvfp4* cast.  Casts that
 * only multiply (mxfp8, mxfp4, a cast by a given scale) have no such division and do not take it. */
#define QCC_RECIP_DIV 0x800

/* what the amax entry points write (their `mode`) */
#define QCC_AMAX_RAW 0        /* the amax itself, fp32                                   */
#define QCC_AMAX_FP8_SCALE 1  /* max(amax, bf16(1e-12)) / fp8_max     G:1179-1183        */
#define QCC_AMAX_NVFP4_SCALE 2 /* amax / (448 * 6)                    G:1243-1246        */

/* OR'ed into `mode` of qcc_amax_bf16: the workspace was prepared by qcc_amax_workspace_init and has since been used
 * by amax calls only, issued in stream order -> one launch instead of two */
#define QCC_AMAX_ONE_LAUNCH 0x100

/* where a cast takes its per-tensor scale from (library internal; see qcc_*_from_amax) */
#define QCC_SRC_SCALE 0 /* a device fp32 holding the scale                                                   */
#define QCC_SRC_AMAX 1  /* a device fp32 holding the raw amax; the cast forms the scale in its prologue      */

/* amax exchange between the GPUs of one box */
#define QCC_XCHG_MAX_RANKS 16
#define QCC_XCHG_STATE_BYTES 1024
#define QCC_XCHG_HANDLE_BYTES 64

/* argument errors */
#define QCC_ERR_SHAPE -1     /* a dimension violates the divisibility the cast needs */
#define QCC_ERR_ALIGN -2     /* a pointer is not 16-byte aligned                     */
#define QCC_ERR_ARG -3       /* NULL pointer, unknown format or flag combination     */
#define QCC_ERR_WORKSPACE -4 /* scratch buffer too small                             */
#define QCC_ERR_DRIVER -5    /* the CUDA driver entry point for tensor maps is missing */
#define QCC_ERR_TOO_LARGE -6 /* the input exceeds what a fixed-size built-in buffer supports */

/* Library version (major * 100 + minor). */
int qcc_version(void);

/* Reads and clears the device-side error word of the current device.  Non-zero: a kernel gave up a
 * bounded wait on a TMA barrier (codes 1..15), or qcc_mxfp8_grouped was given group offsets that are
 * not ascending multiples of 32 inside M (code 16; the scale buffers then hold zeros only), or a
 * transform matrix that is not diag(+-1) @ H16 / 4 was passed to one of the qcc_*rht* calls (code 17;
 * the outputs then follow the signs of its first column), or a cast tile of qcc_fp8_colwise gave up waiting for the
 * column maxima of its panel (code 18).  Synchronises the device. */
int qcc_device_error(unsigned int *out);

/* Number of SMs of the current device (cached per device). */
int qcc_sm_count(void);

/* Strided copy between (pinned) host memory and the device on `stream`: `rows` rows of `width_bytes`
 * bytes, row starts `dst_pitch` / `src_pitch` bytes apart; to_host != 0 copies device -> host, else
 * host -> device.  Used by the host-buffer casters to place the transposed outputs of a row chunk into
 * the columns of the full host matrix (no counterpart in the reference, which keeps data on the GPU). */
int qcc_copy2d_async(void *dst, size_t dst_pitch, const void *src, size_t src_pitch, size_t width_bytes,
                     size_t rows, int to_host, void *stream);

/* dst[0..bytes) = src[0..bytes) by a kernel with the access pattern of the streaming casts (bytes % 16 == 0): the
 * bandwidth yardstick of the benchmarks -- what a kernel that only moves data reaches at a given size on this GPU.
 * (No counterpart in the reference, whose yardstick is an eager relu, benchmarks/benchmark.py:41-60.) */
int qcc_stream_copy(const void *src, void *dst, size_t bytes, void *stream);

/* The yardstick for casts that write fewer bytes than they read: piece i (16 bytes) of dst = XOR of pieces ratio * i ...
 * ratio * i + ratio - 1 of src; ratio 2 or 4, bytes_in % (16 * ratio) == 0, dst holds bytes_in / ratio bytes.  The loads
 * and stores of an fp8 / mxfp8 cast (2: two bytes in, one out) or of an nvfp4 cast (4: two bytes in, half a byte out)
 * without their arithmetic. */
int qcc_stream_fold(const void *src, void *dst, size_t bytes_in, int ratio, void *stream);

/* ---------------------------------------------------------------------------------------------
 * amax and per-tensor scales
 * ------------------------------------------------------------------------------------------- */

/* Bytes of scratch qcc_amax_bf16 needs (independent of n). */
size_t qcc_amax_workspace_bytes(void);

/* Clears a workspace (one small memset on `stream`) so that it can be used with QCC_AMAX_ONE_LAUNCH.  Every such
 * call leaves the workspace cleared again, so this is needed once per workspace, not once per call.  Calls that
 * share a workspace must not overlap on the GPU. */
int qcc_amax_workspace_init(void *workspace, size_t workspace_bytes, void *stream);

/*
 * out[0] = f(max |x[i]|) over n bf16 values, f selected by `mode` (QCC_AMAX_*), `fmt` used by
 * QCC_AMAX_FP8_SCALE only.  Two launches: per-CTA partial maxima into `workspace` (any contents), then a
 * one-CTA finish.  With mode | QCC_AMAX_ONE_LAUNCH: one launch of a one-shot grid whose CTAs merge their maxima
 * into one word of the (prepared) workspace; the CTA that finishes last writes out[0].  The maximum is exact
 * (a bf16 magnitude), so any partition of x gives the same
 * result.  Replaces float8_tensorwise_scale (G:1179-1183) and nvfp4_gs_scale (G:1243-1246).
 */
int qcc_amax_bf16(const void *x, int64_t n, int mode, int fmt, float *out, void *workspace,
                  size_t workspace_bytes, void *stream);

/*
 * Same result as qcc_amax_bf16, for callers that cannot hand over scratch memory.
 * (No counterpart in the reference; an addition of this library.)
 *
 * Some hosts of these kernels are not allowed to allocate device memory at the point where they
 * need the amax: code running inside a region that forbids cudaMalloc (a pre-sized memory pool that
 * is already exhausted or frozen, a real-time or interrupt-like path, a plugin that only receives
 * its input and output buffers from the framework that calls it).  For them the per-CTA partial
 * maxima go into an 8 KB buffer that is part of the library image, so the call needs nothing but
 * x and out.  Nothing here calls cudaMalloc, cudaFree or any allocating routine.
 *
 * Limits and rules:
 *  - n may be at most QCC_AMAX_NOALLOC_MAX_ELEMS (2^32 bf16 values, 8 GiB); larger inputs are
 *    rejected with QCC_ERR_TOO_LARGE and nothing is launched.
 *  - Every GPU that loads the library holds the 8 KB until the process exits.
 *  - The first call on each device looks the buffer's device address up (cudaGetSymbolAddress with
 *    that device current); make that first call outside of any stream capture.
 *  - All calls on one device share the buffer.  Two calls whose kernels may run at the same time
 *    (different streams, or different host threads on different streams) race on it and can return
 *    a wrong amax; serialise them on one stream or use qcc_amax_bf16 with separate workspaces.
 *    The buffer keeps the last call's partial maxima; each call overwrites every slot it reads, so
 *    no clearing is needed between calls.
 */
#define QCC_AMAX_NOALLOC_MAX_ELEMS (1ll << 32)
int qcc_amax_bf16_noalloc(const void *x, int64_t n, int mode, int fmt, float *out, void *stream);

/* out[0] = f(amax[0]) for an amax that is already reduced (e.g. after an all-reduce over shards);
 * same `mode` / `fmt` as above.  One tiny launch. */
int qcc_scale_from_amax(const float *amax, int mode, int fmt, float *out, void *stream);

/* ---------------------------------------------------------------------------------------------
 * amax exchange: the tensor-wide amax of a row-sharded tensor, one process per GPU of one box
 *
 * (No counterpart in the reference, which is single GPU.  It does the job of ncclAllReduce(MAX) on the per-shard
 * amax over peer memory, without a collective call and without a second stream.)
 *
 * A PRODUCER (qcc_amax_bf16_xchg, or the cast qcc_mxfp8_amax_xchg, which has every block maximum in registers anyway)
 * leaves the shard's amax in the rank's own exchange state; its CTAs wait for nothing.  qcc_xchg_resolve, one warp
 * launched next on the same stream, stores that value, tagged with the exchange number, into every rank's state over
 * NVLink (plain 8-byte peer stores), reads the `world` tagged values from its own memory, waits for any that have not
 * arrived (bounded by the state's timeout; code 19 of qcc_device_error), and writes f(global amax) for the casts that
 * follow.  The maximum is exact and order independent, so every rank derives the bits a single GPU would.
 *
 * Rules: every rank owns one state of QCC_XCHG_STATE_BYTES in device memory.  Set-up, once: qcc_xchg_alloc (or own
 * memory + qcc_xchg_state_init), qcc_xchg_ipc_export, hand the 64 handle bytes to the other ranks' processes by any
 * host channel, qcc_xchg_ipc_open on each; states[0..world) then holds the addresses, valid on this GPU, of all
 * ranks' states, states[rank] being the rank's own.  With several GPUs in one process the peers' states are used
 * directly (peer access enabled by the caller).  All ranks must issue the same sequence of producing calls, each
 * followed by one publishing resolve before the rank's next producing call, all on one stream.
 * ------------------------------------------------------------------------------------------- */
typedef struct qcc_xchg_ref {
    void *const *states; /* [world] device addresses of the ranks' states as seen from this GPU */
    int world;           /* 1..QCC_XCHG_MAX_RANKS                                             */
    int rank;            /* this rank                                                         */
    int publish;         /* qcc_xchg_resolve: bit flags.  QCC_XCHG_PUBLISH: hand this rank's amax to all ranks first (the
                            normal call); without it only read an exchange that was published before.  QCC_XCHG_PDL:
                            launch directly behind the producing kernel as a programmatic dependent launch (the warp
                            starts while that kernel drains and waits for its completion on the device) */
} qcc_xchg_ref;
#define QCC_XCHG_PUBLISH 1
#define QCC_XCHG_PDL 2

int qcc_xchg_alloc(void **state);   /* cudaMalloc + clear, timeout 1 s; set-up path, the only allocating call */
int qcc_xchg_free(void *state);
int qcc_xchg_state_init(void *state, unsigned int timeout_us, void *stream);   /* clear caller-owned memory */
int qcc_xchg_ipc_export(void *state, void *handle /* QCC_XCHG_HANDLE_BYTES */);
int qcc_xchg_ipc_open(const void *handle, void **peer_state);
int qcc_xchg_ipc_close(void *peer_state);

/* Producer: max |x| of this rank's shard into the rank's own state; one launch, no CTA waits for anything. */
int qcc_amax_bf16_xchg(const void *x, int64_t n, void *state, void *stream);

/* The publishing half of qcc_xchg_resolve on its own (one warp that waits for nothing; ref->publish is ignored):
 * for driving several ranks' states from one stream, where every rank must have published before any rank waits. */
int qcc_xchg_publish(const qcc_xchg_ref *ref, void *stream);

/* out[0] = f(maximum over the ranks of the exchange), f by `mode` / `fmt` as in qcc_amax_bf16.  One warp. */
int qcc_xchg_resolve(const qcc_xchg_ref *ref, int mode, int fmt, float *out, void *stream);

/* ---------------------------------------------------------------------------------------------
 * fp8 casts
 * ------------------------------------------------------------------------------------------- */

/* q[i] = fp8(float(x[i]) * (1 / scale[0])), saturating.  float8_tensorwise_f, G:1186-1191. */
int qcc_fp8_tensorwise(const void *x, int64_t n, const float *scale, int fmt, void *q, void *stream);

/* The same cast from a raw amax (device fp32, e.g. max-reduced over shards): the scale
 * max(amax, bf16(1e-12)) / fp8_max of G:1179-1183 is formed in the kernel's prologue and also written to scale_out
 * (device, may be NULL) -- float8_tensorwise_scale's division folded into float8_tensorwise_f. */
int qcc_fp8_tensorwise_from_amax(const void *x, int64_t n, const float *amax, int fmt, void *q, float *scale_out,
                                 void *stream);

/* One scale per row: scale[r] = max(amax_r, bf16(1e-12)) / fp8_max, q = fp8(x * (1 / scale[r])).
 * rowwise_fp8_f, G:301-307.  q may be NULL to get the scales only (rowwise_precalc_scale,
 * G:389-393). */
int qcc_fp8_rowwise(const void *x, int64_t M, int64_t N, int fmt, void *q, float *scale, void *stream);

/* q = fp8(float(x) / scale[r]) with a caller-supplied per-row scale; a true division.
 * rowwise_precalc_f, G:396-399. */
int qcc_fp8_rowwise_precalc(const void *x, int64_t M, int64_t N, const float *scale, int fmt, void *q,
                            void *stream);

/* One scale per column (amax over all rows), outputs transposed: q (N, M), scale[c] for column c.
 * colwise_fp8_f, G:339-349.  workspace: qcc_fp8_colwise_workspace_bytes(M, N) bytes of scratch, 16-byte aligned
 * (column maxima and the panel counters of the launch; cleared by the call).  One persistent launch: x is cut into
 * column panels that stay in L2 between their maximum pass and their cast, so HBM sees x once; matrices with more
 * than 448 rows per SM (66304 rows on 148 SMs) take two launches and read x twice.
 * Needs N % 8 == 0 and M % 16 == 0. */
size_t qcc_fp8_colwise_workspace_bytes(int64_t M, int64_t N);
int qcc_fp8_colwise(const void *x, int64_t M, int64_t N, int fmt, void *q, float *scale, void *workspace,
                    size_t workspace_bytes, void *stream);

/* q (N, M) = fp8(float(x) / scale[c]) with a caller-supplied per-column scale; a true division.
 * colwise_precalc_f, G:445-449. */
int qcc_fp8_colwise_precalc(const void *x, int64_t M, int64_t N, const float *scale, int fmt, void *q,
                            void *stream);

/*
 * fp8 e4m3 with one fp32 scale per 128-element block: scale = clamp(amax, 1e-12) / 448, q = e4m3(x * (1 / scale)).
 *   QCC_ROWWISE: qk (M, N), sk (M, N/128) fp32 -- 1x128 blocks along the rows   deepseek_1x128_f        G:103-110
 *   QCC_COLWISE: qm (N, M), sm (N, M/128) fp32 -- 128x1 blocks down the rows,
 *                outputs transposed                                             deepseek_1x128_dim_m_f  G:194-214
 *   both:        one read of x, four outputs                                    deepseek_1x128_dim_km_f G:251-277
 * The amax is clamped in bf16 (bf16(1e-12)) for a single direction and in fp32 for the fused form, as in the
 * reference; the two differ only in the scale of an all-zero block.
 * QCC_ROWWISE needs N % 128 == 0; QCC_COLWISE needs M % 128 == 0 and N % 8 == 0.
 */
int qcc_fp8_block128(const void *x, int64_t M, int64_t N, int flags, void *qk, float *sk, void *qm, float *sm,
                     void *stream);

/* 128x128 blocks: q (M, N), scale (M/128, N/128) fp32 (deepseek_128x128_f G:141-161).  M % 128 == 0, N % 128 == 0. */
int qcc_fp8_block128x128(const void *x, int64_t M, int64_t N, int flags /* 0 or QCC_RECIP_DIV */, void *q, float *scale,
                         void *stream);

/* out (M/128, N/128) fp32 = max |x| of every 128x128 block (QCC_AMAX_RAW) or that maximum / 2688
 * (QCC_AMAX_NVFP4_SCALE: nvfp4_blocked_outer_scale G:1601-1606).  M % 128 == 0, N % 128 == 0. */
int qcc_amax_block128x128(const void *x, int64_t M, int64_t N, int mode, float *out, void *stream);

/* ---------------------------------------------------------------------------------------------
 * mxfp8: 32-element blocks, e8m0 scales, e4m3 elements
 * ------------------------------------------------------------------------------------------- */

/*
 * flags & QCC_ROWWISE: qk (M, N) e4m3 and sk, the (M, N/32) scales      mxfp8_f            G:561-568
 * flags & QCC_COLWISE: qm (N, M) e4m3 and sm, the (N, M/32) scales      mxfp8_dim_m_f      G:656-671
 * both:                one read of x, four outputs                      mxfp8_dim_km_f     G:701-719
 * flags & QCC_SWIZZLE: sk / sm in the blocked layout                    G:1051-1053, G:1092-1094,
 *                                                                       G:1134-1139
 * flags & QCC_FLOOR:   FLOOR scale mode (extension, not in the reference)
 * Needs N % 32 == 0, and M % 32 == 0 when QCC_COLWISE is set.  Outputs of a direction that is not
 * requested may be NULL.
 *
 * flags & QCC_BLOCK32: one RCEIL scale per 32x32 block of x, shared by both orientations (needs M % 32 == 0):
 *   QCC_ROWWISE alone, no QCC_SWIZZLE: qk (M, N) and sk the plain (M/32, N/32) grid   mxfp8_32x32_f         G:753-773
 *   QCC_ROWWISE | QCC_SWIZZLE: sk = the block scales repeated over their 32 rows, i.e. the (M, N/32) frame
 *                              of the 1x32 cast, blocked                              mxfp8_32x32_swizzle_f G:809-815
 *   QCC_COLWISE | QCC_SWIZZLE: qm (N, M) and sm over the (N, M/32) frame, blocked     mxfp8_32x32_dim_m_swizzle_f G:856-862
 *   both | QCC_SWIZZLE: all four                                                      mxfp8_32x32_dim_km_swizzle_f G:900-910
 *   both | QCC_SWIZZLE with qm == NULL: qk, sk and sm only      mxfp8_32x32_qdata_dim_k_scale_dim_km_swizzle_f G:946-959
 * QCC_FLOOR is not available with QCC_BLOCK32.
 */
int qcc_mxfp8(const void *x, int64_t M, int64_t N, int flags, void *qk, void *sk, void *qm, void *sm,
              void *stream);

/* The rowwise cast of qcc_mxfp8 (flags: QCC_ROWWISE, optionally QCC_SWIZZLE / QCC_FLOOR) that also delivers
 * amax_out[0] = max |x| (raw fp32) from the same read of x -- for a tensor that is cast to mxfp8 and to nvfp4
 * (nvfp4_gs_scale G:1243-1246 needs the amax) this saves the separate amax pass.  workspace: as for qcc_amax_bf16
 * with QCC_AMAX_ONE_LAUNCH.  The _xchg form is a producer of the rank's amax exchange instead: the amax goes into
 * `state`, and its CTAs wait for nothing (the form above takes a ticket per CTA so that the last one can write
 * amax_out). */
int qcc_mxfp8_amax(const void *x, int64_t M, int64_t N, int flags, void *qk, void *sk, float *amax_out,
                   void *workspace, size_t workspace_bytes, void *stream);
int qcc_mxfp8_amax_xchg(const void *x, int64_t M, int64_t N, int flags, void *qk, void *sk, void *state, void *stream);

/*
 * E independent (M, N) matrices stacked in x, e.g. per-expert weights (the 3-D branch of quantize_tensor,
 * experiments/quantize_tensor_api/api.py:171-190, with _to_blocked_per_group_3d of moe_utils.py:84-90): the casts of
 * qcc_mxfp8 applied to every matrix, outputs stacked, scale grids per matrix.  One call: a single launch for the
 * whole stack when the scales are plain and only rowwise outputs are asked for, or when the scales are blocked and
 * M % 128 == 0 (every matrix is whole scale atoms; the transposed outputs are placed per matrix inside the kernel);
 * otherwise one launch per matrix.
 */
int qcc_mxfp8_batched(const void *x, int64_t E, int64_t M, int64_t N, int flags, void *qk, void *sk, void *qm, void *sm,
                      void *stream);

/*
 * mxfp4 (mxfp4_f G:607-617): 1x32 blocks along the rows, RCEIL e8m0 scale of amax / 6, elements e2m1 packed two
 * per byte (even element in the low nibble).  q (M, N/2) bytes, s the (M, N/32) scales, plain or (QCC_SWIZZLE)
 * blocked.  N % 32 == 0.
 */
int qcc_mxfp4(const void *x, int64_t M, int64_t N, int flags, void *q, void *s, void *stream);

/*
 * mxfp8 of token groups (MoE activations): x is (M, N) with G groups of consecutive rows, offs[g] = end row
 * of group g (device int32, ascending, every group a multiple of 32 rows; rows after the last group belong to no
 * group and get no scale).  Element bytes are those of
 * qcc_mxfp8; the blocked scales are laid out per group, as the grouped block-scaled GEMM reads them
 * (experiments/quantize_tensor_api/api.py:301-411, moe_utils.py:62-128 of the reference):
 *   sk: (M + G * 128, N / 32) bytes -- each group's (rows, N/32) scales blocked on their own, padded to 128
 *       rows, stacked in group order (_to_blocked_2d_m_groups);
 *   sm: ceil128(N) * (M / 32 + G * 4) bytes -- each group's (N, rows/32) transposed scales blocked on their
 *       own, columns padded to 4, stored group after group (_to_blocked_2d_k_groups).
 * flags must contain QCC_SWIZZLE; QCC_ROWWISE needs N % 128 == 0 (as the reference's reshape does).  workspace: qcc_mxfp8_grouped_workspace_bytes(M) bytes of scratch.  At most
 * 4096 groups.  Both scale buffers are cleared by the call.  offs lives on the device, so it is checked
 * there: offsets that are not ascending multiples of 32 within M leave the scale buffers zero and
 * set code 16 in the word qcc_device_error reads (the data outputs do not depend on the groups).
 */
size_t qcc_mxfp8_grouped_workspace_bytes(int64_t M);
int qcc_mxfp8_grouped(const void *x, int64_t M, int64_t N, int flags, const int32_t *offs, int64_t G, void *qk,
                      void *sk, void *qm, void *sm, void *workspace, size_t workspace_bytes, void *stream);

/*
 * Token groups of ANY size (offs[g] = end row of group g, ascending, last = M): what the reference does in two steps --
 * pad every group with zero rows to a multiple of 32 (_pad_token_groups, experiments/quantize_tensor_api/
 * moe_utils.py:35-59, used by moe_main.py:178-188), then quantize_tensor_grouped* -- without the padded bf16 copy.
 * The padded frame has R = qcc_padded_token_rows(M, G) = ceil32(M + 32 G) rows (the reference's upper bound, so no
 * size has to come back from the device); rows after the last padded group are zero.
 *   qcc_pad_token_groups:  out (R, row_bytes) = the padded rows themselves (any element type, row_bytes % 16 == 0);
 *   qcc_mxfp8_grouped_pad: the outputs of qcc_mxfp8_grouped on that padded matrix: qk (R, N), sk (R + 128 G, N/32),
 *                          qm (N, R), sm (ceil128(N), R/32 + 4 G); x is read once, from its unpadded rows.
 * padded_offs (device int32[G], may be NULL): group ends in the padded frame, the `offs` of the grouped GEMM.
 * workspace: qcc_token_pad_workspace_bytes(M, G) bytes.  At most 2048 groups.  Offsets that are not ascending or do
 * not end at M: code 16 in the device error word, scales zero, padded_offs zero.
 */
int64_t qcc_padded_token_rows(int64_t M, int64_t G);
size_t qcc_token_pad_workspace_bytes(int64_t M, int64_t G);
int qcc_pad_token_groups(const void *x, int64_t M, int64_t row_bytes, const int32_t *offs, int64_t G, void *out,
                         int32_t *padded_offs, void *workspace, size_t workspace_bytes, void *stream);
/* The inverse of qcc_pad_token_groups (_unpad_token_groups, moe_main.py:54-68): out (M, row_bytes) = the real rows of
 * `padded` (qcc_padded_token_rows(M, G) rows); offs are the UNPADDED group ends, as above. */
int qcc_unpad_token_groups(const void *padded, int64_t M, int64_t row_bytes, const int32_t *offs, int64_t G, void *out,
                           void *workspace, size_t workspace_bytes, void *stream);
int qcc_mxfp8_grouped_pad(const void *x, int64_t M, int64_t N, int flags, const int32_t *offs, int64_t G, void *qk,
                          void *sk, void *qm, void *sm, int32_t *padded_offs, void *workspace, size_t workspace_bytes,
                          void *stream);

/* ---------------------------------------------------------------------------------------------
 * nvfp4: 16-element blocks, e4m3 block scales relative to an fp32 outer scale, e2m1 elements
 * packed two per byte (even element in the low nibble)
 * ------------------------------------------------------------------------------------------- */

/*
 * Rowwise: q (M, N/2) bytes, s the (M, N/16) e4m3 scales (plain or blocked).
 *   nvfp4_gs_f G:1494-1517, nvfp4_gs_swizzle_f G:1249-1266, nvfp4_gs_swizzle_sr_f G:1409-1426.
 * outer: device fp32; outer_per_row == 0 -> one value for the tensor, 1 -> one per row (the per-token
 * form of G:1567-1571), 2 -> one per 128x128 block, the (M/128, N/128) grid of nvfp4_blocked_outer_f
 * (G:1609-1634; needs M % 128 == 0, N % 128 == 0, no QCC_SR).  philox_key: device uint64[2] = {seed, offset}, read only when
 * QCC_SR is set; element (r, c) uses counter ((r * N + c) >> 2) + offset, output word (r * N + c) & 3,
 * and its low 22 bits as the dither of G:1401-1405.  Needs N % 16 == 0.
 */
int qcc_nvfp4(const void *x, int64_t M, int64_t N, const float *outer, int outer_per_row, int flags,
              const uint64_t *philox_key, void *q, void *s, void *stream);

/* fp32 -> bf16 with stochastic rounding: out = bf16((bits(x) + rand16) & 0xFFFF0000), rand16 uniform in [0, 2^16)
 * (sr_bf16_f G:1841-1851, sr_bf16_global_f G:1887-1914; _sr_bf16_dither G:1828-1838).  x (M, N) fp32, out (M, N) bf16.
 * Element (i, j) has the flat index g = (global_row + i) * num_col + global_col + j in its parent tensor and takes 16-bit
 * piece g & 7 (half (g & 1) of word (g & 7) >> 1, low half first) of Philox4x32-10(counter = (g >> 3) + offset, key =
 * seed), philox_key = device uint64 {seed, offset}: the cast of a tile equals that tile of the cast of the whole tensor.  global_row = global_col = 0,
 * num_col = N is the plain recipe.  num_col >= global_col + N. */
int qcc_sr_f32_to_bf16(const void *x, int64_t M, int64_t N, const uint64_t *philox_key, int64_t global_row, int64_t global_col,
                       int64_t num_col, void *out, void *stream);

/* scale (M, 1) fp32 = max |x| of every row / 2688, no clamp: the per-token outer scale that qcc_nvfp4 takes with
 * outer_per_row = 1 (nvfp4_gs_per_token_scale, G:1569-1573).  flags: 0 or QCC_RECIP_DIV.  One read of x. */
int qcc_nvfp4_per_token_scale(const void *x, int64_t M, int64_t N, int flags, float *scale, void *stream);

/* qcc_nvfp4 (one outer scale for the tensor, round to nearest; flags: QCC_SWIZZLE or 0) from a raw amax (device
 * fp32): outer = amax / 2688 (nvfp4_gs_scale G:1243-1246) is formed in the kernel's prologue and also written to
 * outer_out (device, may be NULL). */
int qcc_nvfp4_from_amax(const void *x, int64_t M, int64_t N, const float *amax, int flags, void *q, void *s,
                        float *outer_out, void *stream);

/*
 * Transposed: the outputs that the rowwise cast gives on x.t().contiguous() (the call of
 * test/test_quant_cast_gold.py:104), without materialising the transpose: q (N, M/2), s over the
 * (N, M/16) frame.  The stochastic-rounding stream is indexed in the transposed frame.
 * Needs M % 32 == 0 (output rows of M/2 bytes are written in 16-byte pieces) and N % 8 == 0; outer
 * is a single value.
 */
int qcc_nvfp4_transposed(const void *x, int64_t M, int64_t N, const float *outer, int flags,
                         const uint64_t *philox_key, void *q, void *s, void *stream);

/*
 * Both orientations from one read of x: (qk, sk) are the outputs of qcc_nvfp4 (one per-tensor outer
 * scale, round to nearest), (qm, sm) those of qcc_nvfp4_transposed -- the pair of casts an nvfp4 linear
 * layer makes of one operand (test/test_quant_cast_gold.py:103-104).  flags: QCC_SWIZZLE or 0.
 * Needs M % 32 == 0 and N % 32 == 0.
 */
int qcc_nvfp4_both(const void *x, int64_t M, int64_t N, const float *outer, int flags, void *qk, void *sk,
                   void *qm, void *sm, void *stream);

/* ---------------------------------------------------------------------------------------------
 * 16-point randomised Hadamard transform (RHT) and the nvfp4 casts built on it
 * ------------------------------------------------------------------------------------------- */

/*
 * rht: device, 16x16 bf16, row-major, = diag(sign) @ H / 4 with H the Sylvester-Walsh matrix
 * (hadamard_rht_matrix G:1778-1781); only such matrices are supported (checked on the device, code 17 of
 * qcc_device_error).  y[16 b + j] = bf16(sum_i x[16 b + i] * rht[i][j]) with fp32 accumulation in a fixed
 * order: butterfly over strides 1, 2, 4, 8, then the exact scaling by 1/4 and one rounding.  The reference
 * evaluates the same sum as a bf16 matmul whose accumulation order is its GEMM library's; the results agree
 * bit for bit whenever the 16-term sums are exact in fp32 (block values within a 2^12 magnitude range).
 */

/* y (M, N) bf16 = the transform of x along the rows (hadamard_rht_f G:1784-1789).  N % 16 == 0. */
int qcc_hadamard_rht(const void *x, int64_t M, int64_t N, const void *rht, void *y, void *stream);

/*
 * out[0] = max |RHT(x.t())| (transform down the rows of x, 16-row blocks), as QCC_AMAX_RAW, or divided by
 * 2688 as QCC_AMAX_NVFP4_SCALE: the dim-m outer scale of G:1364-1365 without materialising the transposed,
 * transformed tensor.  M % 16 == 0, N % 4 == 0.
 */
int qcc_nvfp4_rht_amax(const void *x, int64_t M, int64_t N, const void *rht, int mode, float *out, void *stream);

/*
 * nvfp4 in both orientations from one read of x, the dim-m half through the transform
 * (nvfp4_gs_swizzle_dim_k_dim_m_rht_f G:1324-1333; with QCC_SR nvfp4_gs_swizzle_dim_k_dim_m_rht_sr_f
 * G:1429-1438):
 *   (qk, sk) = qcc_nvfp4(x, outer_k)                       -- no transform
 *   (qm, sm) = nvfp4 along M of RHT(x.t()) under outer_m   -- q (N, M/2), scales over the (N, M/16) frame
 * Round to nearest: one read of x, the four warps of a tile first transform and quantise down the rows, then quantise
 * along the rows of the same tile.  With QCC_SR: two launches (both halves are bound by the Philox arithmetic and the
 * fused kernel measured slower).  qk == sk == NULL gives the dim-m half alone.  flags: QCC_SWIZZLE, QCC_SR (key_k / key_m: device uint64[2]
 * each, the stream of a half indexed by the row-major position in that half's own frame).
 * Needs M % 32 == 0, N % 8 == 0, and N % 32 == 0 when the dim-k half is requested.
 */
int qcc_nvfp4_rht(const void *x, int64_t M, int64_t N, const float *outer_k, const float *outer_m, const void *rht,
                  int flags, const uint64_t *key_k, const uint64_t *key_m, void *qk, void *sk, void *qm, void *sm,
                  void *stream);

#ifdef __cplusplus
}
#endif
#endif /* QUANT_CAST_CUDA_H */
