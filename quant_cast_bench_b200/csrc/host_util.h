// Host-side helpers shared by the launchers: device properties, alignment checks and the tensor-map
// encoder obtained from the driver at run time (no link-time dependency on libcuda).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

namespace qcc {

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// QCC_RECIP_DIV rides in the `fmt`, `mode` or `flags` argument of an entry point: take_recip_div strips it from the
// argument and returns 1 when it was set; amax_mode_ok checks an amax `mode` that may still carry it.
inline int take_recip_div(int &arg)
{
    const int r = (arg & QCC_RECIP_DIV) ? 1 : 0;
    arg &= ~QCC_RECIP_DIV;
    return r;
}
inline bool amax_mode_ok(int mode)
{
    mode &= ~QCC_RECIP_DIV;
    return mode >= QCC_AMAX_RAW && mode <= QCC_AMAX_NVFP4_SCALE;
}

// Per-device host-side caches ("this kernel's attributes are set on device d", "the address of this symbol on device
// d").  Host threads may make their first call on a device at the same time: every writer stores the same value, and
// the flags are atomics, so the only cost of that race is doing the set-up twice.  Devices 0..63; current_device_slot()
// returns -1 for any other ordinal and the entry points then reject the call.
constexpr int QCC_MAX_DEVICES = 64;
struct PerDeviceFlag {
    std::atomic<unsigned char> v[QCC_MAX_DEVICES];
    PerDeviceFlag() { for (auto &e : v) e.store(0, std::memory_order_relaxed); }
    bool get(int dev) const { return v[dev].load(std::memory_order_acquire) != 0; }
    void set(int dev) { v[dev].store(1, std::memory_order_release); }
};
inline int current_device_slot()
{
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= QCC_MAX_DEVICES) return -1;
    return dev;
}

// SM count of the current device, cached per device ordinal.
inline int sm_count()
{
    static std::atomic<int> cache[QCC_MAX_DEVICES];
    const int dev = current_device_slot();
    if (dev < 0) return 148;
    int n = cache[dev].load(std::memory_order_relaxed);
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cache[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}

typedef CUresult (*encode_tiled_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                    const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline encode_tiled_fn get_encode_tiled()
{
    static encode_tiled_fn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<encode_tiled_fn>(p);
        tried = true;
    }
    return fn;
}

// Tensor map over a row-major tensor of up to 3 dims (dim 0 contiguous).  strides[i] = byte stride of
// dim i+1.  Returns 0, QCC_ERR_DRIVER, or 1000 + CUresult.
inline int make_tensor_map(CUtensorMap *map, CUtensorMapDataType dt, int rank, const void *base, const uint64_t *dims,
                           const uint64_t *strides, const uint32_t *box, CUtensorMapSwizzle swz)
{
    encode_tiled_fn enc = get_encode_tiled();
    if (!enc) return -5;
    cuuint64_t gd[3];
    cuuint64_t gs[2];
    cuuint32_t bx[3];
    cuuint32_t es[3] = {1, 1, 1};
    for (int i = 0; i < rank; i++) { gd[i] = dims[i]; bx[i] = box[i]; }
    for (int i = 0; i + 1 < rank; i++) gs[i] = strides[i];
    CUresult r = enc(map, dt, (cuuint32_t)rank, const_cast<void *>(base), gd, gs, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 1000 + (int)r;
}

// Kernel launch with the programmatic-stream-serialization attribute when `pdl` is set (the kernel may then start while
// its predecessor on the stream drains and must call pdl_wait() before reading that predecessor's results).
template <class... KArgs, class... Args>
inline cudaError_t launch_maybe_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool pdl, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

// Launches the one-CTA check that `rht` (device, 16x16 bf16) is diag(+-1) @ H16 / 4; a matrix of another form
// sets code 17 in the device error word (defined with the nvfp4 kernels).
int launch_rht_check(const void *rht, cudaStream_t st);

}  // namespace qcc

// fp8 colwise cast with the panel resident in shared memory (colwise.cu).  1: the shape does not fit that form.
int qcc_colwise_resident(const void *x, int64_t M, int64_t N, int fmt, void *q, float *scale_out, uint32_t *amax_bits,
                         cudaStream_t st);

