"""ctypes binding of libquant_cast_cuda.so (the C ABI declared in include/quant_cast_cuda.h).

There is no fallback: if the library has not been built, or no CUDA device is present, every cast
raises.  Build with `python -m quant_cast_bench_b200.build`.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(os.path.dirname(_HERE), "lib", "libquant_cast_cuda.so")

# constants of include/quant_cast_cuda.h
FMT_E4M3, FMT_E5M2 = 0, 1
ROWWISE, COLWISE, SWIZZLE, FLOOR, SR, BLOCK32 = 1, 2, 4, 8, 16, 32
PDL, REVERSE = 0x200, 0x400
XCHG_PUBLISH, XCHG_PDL = 1, 2
AMAX_RAW, AMAX_FP8_SCALE, AMAX_NVFP4_SCALE = 0, 1, 2
AMAX_ONE_LAUNCH = 0x100
RECIP_DIV = 0x800   # QCC_RECIP_DIV: `tensor / constant` as PyTorch's CUDA kernels compute it, tensor * fl(1 / constant)
XCHG_MAX_RANKS, XCHG_STATE_BYTES, XCHG_HANDLE_BYTES = 16, 1024, 64
ERRORS = {
    -1: "shape: a dimension violates the divisibility this cast needs",
    -2: "alignment: a tensor is not 16-byte aligned",
    -3: "argument: missing tensor, unknown format or flag combination",
    -4: "workspace too small",
    -5: "the CUDA driver does not provide cuTensorMapEncodeTiled",
    -6: "input too large for the library's built-in fixed-size buffer",
}

_vp, _i64, _int, _sz = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_size_t
SIGNATURES = {
    "qcc_version": (_int, []),
    "qcc_device_error": (_int, [ctypes.POINTER(ctypes.c_uint)]),
    "qcc_sm_count": (_int, []),
    "qcc_copy2d_async": (_int, [_vp, _sz, _vp, _sz, _sz, _sz, _int, _vp]),
    "qcc_stream_copy": (_int, [_vp, _vp, _sz, _vp]),
    "qcc_stream_fold": (_int, [_vp, _vp, _sz, _int, _vp]),
    "qcc_amax_workspace_bytes": (_sz, []),
    "qcc_amax_workspace_init": (_int, [_vp, _sz, _vp]),
    "qcc_amax_bf16": (_int, [_vp, _i64, _int, _int, _vp, _vp, _sz, _vp]),
    "qcc_xchg_alloc": (_int, [ctypes.POINTER(_vp)]),
    "qcc_xchg_free": (_int, [_vp]),
    "qcc_xchg_state_init": (_int, [_vp, ctypes.c_uint, _vp]),
    "qcc_xchg_ipc_export": (_int, [_vp, _vp]),
    "qcc_xchg_ipc_open": (_int, [_vp, ctypes.POINTER(_vp)]),
    "qcc_xchg_ipc_close": (_int, [_vp]),
    "qcc_amax_bf16_xchg": (_int, [_vp, _i64, _vp, _vp]),
    "qcc_xchg_publish": (_int, [_vp, _vp]),
    "qcc_xchg_resolve": (_int, [_vp, _int, _int, _vp, _vp]),
    "qcc_fp8_tensorwise_from_amax": (_int, [_vp, _i64, _vp, _int, _vp, _vp, _vp]),
    "qcc_mxfp8_amax": (_int, [_vp, _i64, _i64, _int, _vp, _vp, _vp, _vp, _sz, _vp]),
    "qcc_mxfp8_amax_xchg": (_int, [_vp, _i64, _i64, _int, _vp, _vp, _vp, _vp]),
    "qcc_nvfp4_from_amax": (_int, [_vp, _i64, _i64, _vp, _int, _vp, _vp, _vp, _vp]),
    "qcc_amax_bf16_noalloc": (_int, [_vp, _i64, _int, _int, _vp, _vp]),
    "qcc_scale_from_amax": (_int, [_vp, _int, _int, _vp, _vp]),
    "qcc_fp8_tensorwise": (_int, [_vp, _i64, _vp, _int, _vp, _vp]),
    "qcc_fp8_rowwise": (_int, [_vp, _i64, _i64, _int, _vp, _vp, _vp]),
    "qcc_fp8_rowwise_precalc": (_int, [_vp, _i64, _i64, _vp, _int, _vp, _vp]),
    "qcc_fp8_colwise_workspace_bytes": (_sz, [_i64, _i64]),
    "qcc_fp8_colwise": (_int, [_vp, _i64, _i64, _int, _vp, _vp, _vp, _sz, _vp]),
    "qcc_fp8_colwise_precalc": (_int, [_vp, _i64, _i64, _vp, _int, _vp, _vp]),
    "qcc_mxfp8": (_int, [_vp, _i64, _i64, _int, _vp, _vp, _vp, _vp, _vp]),
    "qcc_padded_token_rows": (_i64, [_i64, _i64]),
    "qcc_token_pad_workspace_bytes": (_sz, [_i64, _i64]),
    "qcc_pad_token_groups": (_int, [_vp, _i64, _i64, _vp, _i64, _vp, _vp, _vp, _sz, _vp]),
    "qcc_unpad_token_groups": (_int, [_vp, _i64, _i64, _vp, _i64, _vp, _vp, _sz, _vp]),
    "qcc_mxfp8_grouped_pad": (_int, [_vp, _i64, _i64, _int, _vp, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "qcc_mxfp8_batched": (_int, [_vp, _i64, _i64, _i64, _int, _vp, _vp, _vp, _vp, _vp]),
    "qcc_mxfp4": (_int, [_vp, _i64, _i64, _int, _vp, _vp, _vp]),
    "qcc_mxfp8_grouped_workspace_bytes": (_sz, [_i64]),
    "qcc_mxfp8_grouped": (_int, [_vp, _i64, _i64, _int, _vp, _i64, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "qcc_nvfp4": (_int, [_vp, _i64, _i64, _vp, _int, _int, _vp, _vp, _vp, _vp]),
    "qcc_nvfp4_transposed": (_int, [_vp, _i64, _i64, _vp, _int, _vp, _vp, _vp, _vp]),
    "qcc_nvfp4_both": (_int, [_vp, _i64, _i64, _vp, _int, _vp, _vp, _vp, _vp, _vp]),
    "qcc_fp8_block128": (_int, [_vp, _i64, _i64, _int, _vp, _vp, _vp, _vp, _vp]),
    "qcc_sr_f32_to_bf16": (_int, [_vp, _i64, _i64, _vp, _i64, _i64, _i64, _vp, _vp]),
    "qcc_nvfp4_per_token_scale": (_int, [_vp, _i64, _i64, _int, _vp, _vp]),
    "qcc_fp8_block128x128": (_int, [_vp, _i64, _i64, _int, _vp, _vp, _vp]),
    "qcc_amax_block128x128": (_int, [_vp, _i64, _i64, _int, _vp, _vp]),
    "qcc_hadamard_rht": (_int, [_vp, _i64, _i64, _vp, _vp, _vp]),
    "qcc_nvfp4_rht_amax": (_int, [_vp, _i64, _i64, _vp, _int, _vp, _vp]),
    "qcc_nvfp4_rht": (_int, [_vp, _i64, _i64, _vp, _vp, _vp, _int, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
}

CHECK_DEVICE = os.environ.get("QCC_CHECK_DEVICE", "0") not in ("", "0")   # see raise_on_device_error



class XchgRef(ctypes.Structure):
    """qcc_xchg_ref of include/quant_cast_cuda.h"""
    _fields_ = [("states", ctypes.POINTER(ctypes.c_void_p)), ("world", ctypes.c_int), ("rank", ctypes.c_int),
                ("publish", ctypes.c_int)]


_lib = None
launch_count = 0  # kernels launched through this binding (the benchmark resets and reads it)


def load():
    """Load the shared library and declare every entry point; raises if it is missing."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: the CUDA library has not been built "
                "(python -m quant_cast_bench_b200.build). quant_cast_cuda has no CPU fallback."
            )
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError if the .so does not export a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


# ---- how the casts divide by a constant ------------------------------------------------------------------------
# The gold recipes write `amax / 448.0`, `amax / 2688.0`, `block_amax / 6.0`.  Run eagerly on the CPU PyTorch computes
# an IEEE division there; run eagerly on a CUDA device it multiplies by the fp32 reciprocal of the scalar (aten's
# BinaryDivTrueKernel.cu), and the two results differ in the last bit for about half of all operands.  "ieee" (default)
# makes the casts bit-identical to the gold recipes on the CPU, "cuda_eager" to the gold recipes on a CUDA device.
_SCALAR_DIVISIONS = ("ieee", "cuda_eager")
_scalar_division = os.environ.get("QCC_SCALAR_DIVISION", "ieee")
if _scalar_division not in _SCALAR_DIVISIONS:
    raise ValueError(f"QCC_SCALAR_DIVISION must be one of {_SCALAR_DIVISIONS}, not {_scalar_division!r}")


def set_scalar_division(mode):
    """Process-wide choice of how `amax / constant` is computed by every cast that follows: "ieee" or "cuda_eager"
    (see above).  Returns the previous setting."""
    global _scalar_division
    if mode not in _SCALAR_DIVISIONS:
        raise ValueError(f"scalar division must be one of {_SCALAR_DIVISIONS}, not {mode!r}")
    prev, _scalar_division = _scalar_division, mode
    return prev


def get_scalar_division():
    return _scalar_division


class scalar_division:
    """Context manager: `with scalar_division("cuda_eager"): ...`."""

    def __init__(self, mode):
        self.mode = mode

    def __enter__(self):
        self.prev = set_scalar_division(self.mode)
        return self

    def __exit__(self, *exc):
        set_scalar_division(self.prev)
        return False


def div_flag():
    """The bit the C entry points take for the current setting (0 or RECIP_DIV)."""
    return RECIP_DIV if _scalar_division == "cuda_eager" else 0


def check(rc, what):
    if rc == 0:
        if CHECK_DEVICE:
            raise_on_device_error(what)
        return
    if rc < 0:
        raise ValueError(f"{what}: {ERRORS.get(rc, rc)}")
    raise RuntimeError(f"{what}: CUDA error {rc}")


DEVICE_ERRORS = {
    16: "token-group offsets are not ascending multiples of 32 ending at M",
    17: "the transform matrix is not diag(+-1) @ H16 / 4",
    18: "a colwise fp8 cast gave up waiting for the column maxima of a panel",
    19: "a wait for another rank's amax (amax exchange) ran out",
}


def device_error():
    """Reads and clears the device-side error word of the current CUDA device (synchronises): 0 when no kernel
    reported anything, 1..15 a TMA barrier wait that ran out, 16 invalid token-group offsets, 17 an unsupported transform matrix, 18 a colwise cast
    that gave up waiting for the column maxima of a panel, 19 a wait for another rank's amax that ran out."""
    v = ctypes.c_uint(0)
    rc = load().qcc_device_error(ctypes.byref(v))       # (not through check(): that is what calls this under QCC_CHECK_DEVICE)
    if rc:
        raise RuntimeError(f"device_error: CUDA error {rc}")
    return int(v.value)


def raise_on_device_error(what="quant_cast_cuda"):
    """Opt-in check after a cast (synchronises the device): raises RuntimeError when a kernel of this library
    recorded an error -- a bounded wait that ran out leaves wrong bytes in the outputs without failing the launch.
    `QCC_CHECK_DEVICE=1` in the environment makes every recipe call do this."""
    code = device_error()
    if code:
        raise RuntimeError(f"{what}: device error {code}: {DEVICE_ERRORS.get(code, 'a TMA barrier wait ran out')}")


