"""The casts as NATIVE PyTorch operators: `torch.ops.quant_cast_cuda_native.*`, registered from C++ (TORCH_LIBRARY in
csrc/torch_binding.cpp, built into lib/libquant_cast_torch.so by `python -m quant_cast_bench_b200.build --torch`).

The same six operator families as `torch_ops.py` (which registers them from Python over ctypes and needs no C++ build),
with CUDA and Meta implementations in C++: they trace under `torch.compile` / `torch.export`, and a C++ program that links
libquant_cast_torch.so can call them through the dispatcher without Python.  Importing this module loads the library;
`<gold recipe name>_native(...)` below give the operators the gold signatures.  No CPU implementation exists.
"""
import os

import torch

from . import _lib as L

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(os.path.dirname(HERE), "lib", "libquant_cast_torch.so")


def load():
    """Load the operator library (once).  Raises when it has not been built."""
    if not hasattr(load, "done"):
        if not os.path.exists(LIB):
            raise FileNotFoundError(f"{LIB} is missing: build it with `python -m quant_cast_bench_b200.build --torch`")
        torch.ops.load_library(LIB)
        load.done = True
    return torch.ops.quant_cast_cuda_native


ops = load()


def _recip():
    return L.div_flag() != 0


def float8_tensorwise_scale_native(x, fmt="e4m3"):
    return ops.amax(x, "fp8", fmt, _recip())


def nvfp4_gs_scale_native(x):
    return ops.amax(x, "nvfp4", "e4m3", _recip())


def amax_native(x):
    return ops.amax(x, "raw", "e4m3", False)


def float8_tensorwise_native(x, scale, fmt="e4m3", **kwargs):
    return (ops.fp8_tensorwise(x, scale, fmt),)


def rowwise_fp8_native(x, fmt="e4m3", **kwargs):
    return tuple(ops.fp8_rowwise(x, fmt, _recip()))


def colwise_fp8_native(x, fmt="e4m3", **kwargs):
    return tuple(ops.fp8_colwise(x, fmt, _recip()))


def _mx(rowwise, colwise, swizzle):
    def fn(x, mode="rceil", **kwargs):
        return tuple(ops.mxfp8(x, rowwise, colwise, swizzle, mode))
    return fn


mxfp8_native, mxfp8_swizzle_native = _mx(True, False, False), _mx(True, False, True)
mxfp8_dim_m_native, mxfp8_dim_m_swizzle_native = _mx(False, True, False), _mx(False, True, True)
mxfp8_dim_km_native, mxfp8_dim_km_swizzle_native = _mx(True, True, False), _mx(True, True, True)


def nvfp4_gs_native(x, outer_scale, **kwargs):
    return tuple(ops.nvfp4(x, outer_scale, False, False, _recip()))


def nvfp4_gs_swizzle_native(x, outer_scale, **kwargs):
    return tuple(ops.nvfp4(x, outer_scale, True, False, _recip()))


def nvfp4_gs_swizzle_t_native(x, outer_scale, **kwargs):
    return tuple(ops.nvfp4(x, outer_scale, True, True, _recip()))


def nvfp4_gs_swizzle_sr_native(x, outer_scale, key, **kwargs):
    return tuple(ops.nvfp4_sr(x, outer_scale, key, True, False, _recip()))


def nvfp4_gs_swizzle_t_sr_native(x, outer_scale, key, **kwargs):
    return tuple(ops.nvfp4_sr(x, outer_scale, key, True, True, _recip()))


def nvfp4_gs_swizzle_both_native(x, outer_scale, **kwargs):
    return tuple(ops.nvfp4_both(x, outer_scale, True, _recip()))


def nvfp4_blocked_outer_native(x, outer_blocked, **kwargs):
    return tuple(ops.nvfp4(x, outer_blocked, True, False, _recip()))


def rowwise_precalc_native(x, scale, fmt="e4m3", **kwargs):
    return (ops.fp8_rowwise_precalc(x, scale, fmt),)


def colwise_precalc_native(x, scale, fmt="e4m3", **kwargs):
    return (ops.fp8_colwise_precalc(x, scale, fmt),)


def deepseek_1x128_native(x, **kwargs):
    return tuple(ops.fp8_block128(x, True, False, _recip()))


def deepseek_1x128_dim_m_native(x, **kwargs):
    return tuple(ops.fp8_block128(x, False, True, _recip()))


def deepseek_1x128_dim_km_native(x, **kwargs):
    return tuple(ops.fp8_block128(x, True, True, _recip()))


def deepseek_128x128_native(x, **kwargs):
    return tuple(ops.fp8_block128x128(x, _recip()))


def mxfp8_32x32_native(x, **kwargs):
    return tuple(ops.mxfp8_32x32(x, True, False, False, True))


def mxfp8_32x32_swizzle_native(x, **kwargs):
    return tuple(ops.mxfp8_32x32(x, True, False, True, True))


def mxfp8_32x32_dim_m_swizzle_native(x, **kwargs):
    return tuple(ops.mxfp8_32x32(x, False, True, True, True))


def mxfp8_32x32_dim_km_swizzle_native(x, **kwargs):
    return tuple(ops.mxfp8_32x32(x, True, True, True, True))


def mxfp8_32x32_qdata_dim_k_scale_dim_km_swizzle_native(x, **kwargs):
    return tuple(ops.mxfp8_32x32(x, True, True, True, False))


def mxfp4_native(x, swizzle=False, **kwargs):
    return tuple(ops.mxfp4(x, swizzle))


def nvfp4_gs_per_token_scale_native(x):
    return ops.nvfp4_per_token_scale(x, _recip())


def sr_bf16_global_native(x, key, global_row=0, global_col=0, num_col=None, **kwargs):
    return (ops.sr_f32_to_bf16(x, key, int(global_row), int(global_col), -1 if num_col is None else int(num_col)),)


def sr_bf16_native(x, key, **kwargs):
    return (ops.sr_f32_to_bf16(x, key, 0, 0, -1),)


# (gold function name in the golden vectors, operator-backed function, aux input): the other recipe families
MORE_NATIVE = [
    ("rowwise_precalc_f", rowwise_precalc_native, "row_scale"), ("colwise_precalc_f", colwise_precalc_native, "col_scale"),
    ("deepseek_1x128_f", deepseek_1x128_native, None), ("deepseek_1x128_dim_m_f", deepseek_1x128_dim_m_native, None),
    ("deepseek_1x128_dim_km_f", deepseek_1x128_dim_km_native, None), ("deepseek_128x128_f", deepseek_128x128_native, None),
    ("mxfp8_32x32_f", mxfp8_32x32_native, None), ("mxfp8_32x32_swizzle_f", mxfp8_32x32_swizzle_native, None),
    ("mxfp8_32x32_dim_m_swizzle_f", mxfp8_32x32_dim_m_swizzle_native, None),
    ("mxfp8_32x32_dim_km_swizzle_f", mxfp8_32x32_dim_km_swizzle_native, None),
    ("mxfp8_32x32_qdata_dim_k_scale_dim_km_swizzle_f", mxfp8_32x32_qdata_dim_k_scale_dim_km_swizzle_native, None),
    ("mxfp4_f", mxfp4_native, None), ("nvfp4_blocked_outer_f", nvfp4_blocked_outer_native, "blocked_outer"),
    ("nvfp4_gs_f_per_token", nvfp4_gs_native, "per_token"), ("nvfp4_gs_swizzle_t_f", nvfp4_gs_swizzle_t_native, "outer"),
]

# (gold recipe name, operator-backed function): the recipes of BASELINE configurations 1-4
NATIVE_RECIPES = [
    ("fp8_tensorwise_precalc_scale", float8_tensorwise_native), ("fp8_rowwise", rowwise_fp8_native), ("fp8_colwise", colwise_fp8_native),
    ("mxfp8", mxfp8_native), ("mxfp8_swizzle", mxfp8_swizzle_native), ("mxfp8_dim_m", mxfp8_dim_m_native),
    ("mxfp8_dim_m_swizzle", mxfp8_dim_m_swizzle_native), ("mxfp8_dim_km", mxfp8_dim_km_native),
    ("mxfp8_dim_km_swizzle", mxfp8_dim_km_swizzle_native), ("nvfp4", nvfp4_gs_native), ("nvfp4_swizzle", nvfp4_gs_swizzle_native),
]
