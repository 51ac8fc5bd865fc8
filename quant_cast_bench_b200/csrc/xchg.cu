// Amax exchange between the GPUs of one box: set-up of the per-rank state (allocation, CUDA IPC handles for the
// other ranks' processes) and the stand-alone consumer.  The producing and consuming device code is in xchg.cuh and
// runs inside the amax and cast kernels.  No counterpart in the reference (single GPU).
#include "common.cuh"
#include "host_util.h"
#include "xchg.cuh"

namespace qcc {

// out[0] = f(maximum over the ranks of the last exchange), f as in qcc_amax_bf16
__global__ void xchg_resolve_kernel(uint32_t *state, XchgPeers peers, int publish, int mode, int fmt, float *__restrict__ out)
{
    pdl_trigger();          // a cast flagged QCC_PDL may start loading its input now; it waits for this kernel's result
    pdl_wait();             // launched with QCC_XCHG_PDL: the producing kernel may still be draining
    const uint32_t e = (publish & QCC_XCHG_PUBLISH) ? xchg_publish(state, peers) : xchg_current(state);
    const float am = xchg_resolve(state, peers.world, e);
    if (threadIdx.x != 0) return;
    float r = am;
    const bool recip = mode & QCC_RECIP_DIV;   // mode: QCC_AMAX_*, with QCC_RECIP_DIV or-ed in when given
    if ((mode & ~QCC_RECIP_DIV) == QCC_AMAX_FP8_SCALE)
        r = fmt == QCC_FMT_E5M2 ? fp8_scale_from_amax<QCC_FMT_E5M2>(am, recip) : fp8_scale_from_amax<QCC_FMT_E4M3>(am, recip);
    else if ((mode & ~QCC_RECIP_DIV) == QCC_AMAX_NVFP4_SCALE)
        r = div_by_const(am, 2688.0f, recip);
    out[0] = r;
}

// publish alone: hands this rank's amax to all ranks and waits for nothing
__global__ void xchg_publish_kernel(uint32_t *state, XchgPeers peers) { xchg_publish(state, peers); }

}  // namespace qcc

using namespace qcc;

static_assert(sizeof(cudaIpcMemHandle_t) <= QCC_XCHG_HANDLE_BYTES, "handle buffer too small");
static_assert(XCHG_SLOT_BYTE_OFF + 2 * QCC_XCHG_MAX_RANKS * 8 <= QCC_XCHG_STATE_BYTES, "state too small");

extern "C" {

int qcc_xchg_device_error(unsigned int *out) { return read_clear_device_error(out); }

int qcc_xchg_state_init(void *state, unsigned int timeout_us, void *stream)
{
    if (!state || timeout_us == 0) return QCC_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e = cudaMemsetAsync(state, 0, QCC_XCHG_STATE_BYTES, st);
    if (e != cudaSuccess) return (int)e;
    return (int)cudaMemcpyAsync(static_cast<uint32_t *>(state) + XCHG_W_TIMEOUT, &timeout_us, sizeof(timeout_us),
                                cudaMemcpyHostToDevice, st);
}

int qcc_xchg_alloc(void **state)
{
    if (!state) return QCC_ERR_ARG;
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, QCC_XCHG_STATE_BYTES);
    if (e != cudaSuccess) return (int)e;
    int rc = qcc_xchg_state_init(p, 1000000u, nullptr);
    if (rc == 0) rc = (int)cudaStreamSynchronize(nullptr);
    if (rc) {
        cudaFree(p);
        return rc;
    }
    *state = p;
    return 0;
}

int qcc_xchg_free(void *state) { return state ? (int)cudaFree(state) : 0; }

int qcc_xchg_ipc_export(void *state, void *handle)
{
    if (!state || !handle) return QCC_ERR_ARG;
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, state);
    if (e != cudaSuccess) return (int)e;
    memset(handle, 0, QCC_XCHG_HANDLE_BYTES);
    memcpy(handle, &h, sizeof(h));
    return 0;
}

int qcc_xchg_ipc_open(const void *handle, void **peer_state)
{
    if (!handle || !peer_state) return QCC_ERR_ARG;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void *p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return (int)e;
    *peer_state = p;
    return 0;
}

int qcc_xchg_ipc_close(void *peer_state) { return peer_state ? (int)cudaIpcCloseMemHandle(peer_state) : 0; }

int qcc_xchg_publish(const qcc_xchg_ref *ref, void *stream)
{
    if (!ref) return QCC_ERR_ARG;
    XchgPeers peers;
    int rc = make_xchg_peers(&peers, ref->states, ref->world, ref->rank);
    if (rc) return rc;
    xchg_publish_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(static_cast<uint32_t *>(ref->states[ref->rank]), peers);
    return (int)cudaGetLastError();
}

int qcc_xchg_resolve(const qcc_xchg_ref *ref, int mode, int fmt, float *out, void *stream)
{
    if (!ref || !out) return QCC_ERR_ARG;
    if (!amax_mode_ok(mode) || (fmt != QCC_FMT_E4M3 && fmt != QCC_FMT_E5M2))
        return QCC_ERR_ARG;
    XchgPeers peers;
    int rc = make_xchg_peers(&peers, ref->states, ref->world, ref->rank);
    if (rc) return rc;
    return (int)launch_maybe_pdl(xchg_resolve_kernel, dim3(1), dim3(32), 0, (cudaStream_t)stream, (ref->publish & QCC_XCHG_PDL) != 0,
                                 static_cast<uint32_t *>(ref->states[ref->rank]), peers, ref->publish, mode, fmt, out);
}

}  // extern "C"
