"""The casts as registered PyTorch operators: `torch.ops.quant_cast_cuda.*`.

A thin layer over the same C ABI as `recipes.py` (which stays the dependency-free ctypes route): every operator calls
the recipe function of the same family, and carries a fake (meta) implementation that gives the gold shapes and dtype
views, so the casts can be traced -- `torch.compile(fullgraph=True)`, `torch.export`, FakeTensor shape propagation --
like the reference's Triton backend, whose kernels Inductor can see through
(quant_cast_triton/recipes.py:48-65 of vkuzo/quant_cast_bench).  Importing this module registers the operators:

    quant_cast_cuda::amax(x, kind, fmt)                  -> fp32 scalar      kind: "raw" | "fp8" | "nvfp4"
    quant_cast_cuda::fp8_tensorwise(x, scale, fmt)       -> q
    quant_cast_cuda::fp8_rowwise(x, fmt)                 -> (q, scale (M, 1))
    quant_cast_cuda::fp8_colwise(x, fmt)                 -> (q (N, M), scale (N, 1))
    quant_cast_cuda::mxfp8(x, rowwise, colwise, swizzle, mode) -> [qk, sk][qm, sm]  (the requested directions, in that order)
    quant_cast_cuda::nvfp4(x, outer_scale, swizzle, transposed)          -> (q, inner scales)
    quant_cast_cuda::nvfp4_sr(x, outer_scale, key, swizzle, transposed)  -> (q, inner scales)

and `<gold recipe name>_op(...)` below give them the gold signatures (`mxfp8_dim_km_swizzle_op(x)` ...).
There is still no CPU implementation: on a CPU tensor the operators raise.
"""
from typing import List, Tuple

import torch
from torch.library import custom_op

from . import _lib as L
from . import recipes as R

_F8 = {"e4m3": torch.float8_e4m3fn, "e5m2": torch.float8_e5m2}


def _check_2d(x):
    torch._check(x.dim() == 2, lambda: "x must be 2-D")
    return x.shape


@custom_op("quant_cast_cuda::amax", mutates_args=(), device_types="cuda")
def amax(x: torch.Tensor, kind: str, fmt: str) -> torch.Tensor:
    if kind == "raw":
        return R.amax_cuda(x)
    return R.float8_tensorwise_scale_cuda(x, fmt) if kind == "fp8" else R.nvfp4_gs_scale_cuda(x)


@amax.register_fake
def _(x, kind, fmt):
    return x.new_empty((), dtype=torch.float32)


@custom_op("quant_cast_cuda::fp8_tensorwise", mutates_args=(), device_types="cuda")
def fp8_tensorwise(x: torch.Tensor, scale: torch.Tensor, fmt: str) -> torch.Tensor:
    return R.float8_tensorwise_cuda(x, scale, fmt)[0]


@fp8_tensorwise.register_fake
def _(x, scale, fmt):
    return x.new_empty(x.shape, dtype=_F8[fmt])


@custom_op("quant_cast_cuda::fp8_rowwise", mutates_args=(), device_types="cuda")
def fp8_rowwise(x: torch.Tensor, fmt: str) -> Tuple[torch.Tensor, torch.Tensor]:
    return R.rowwise_fp8_cuda(x, fmt)


@fp8_rowwise.register_fake
def _(x, fmt):
    M, N = _check_2d(x)
    return x.new_empty((M, N), dtype=_F8[fmt]), x.new_empty((M, 1), dtype=torch.float32)


@custom_op("quant_cast_cuda::fp8_colwise", mutates_args=(), device_types="cuda")
def fp8_colwise(x: torch.Tensor, fmt: str) -> Tuple[torch.Tensor, torch.Tensor]:
    return R.colwise_fp8_cuda(x, fmt)


@fp8_colwise.register_fake
def _(x, fmt):
    M, N = _check_2d(x)
    return x.new_empty((N, M), dtype=_F8[fmt]), x.new_empty((N, 1), dtype=torch.float32)


@custom_op("quant_cast_cuda::mxfp8", mutates_args=(), device_types="cuda")
def mxfp8(x: torch.Tensor, rowwise: bool, colwise: bool, swizzle: bool, mode: str) -> List[torch.Tensor]:
    flags = (L.ROWWISE if rowwise else 0) | (L.COLWISE if colwise else 0) | (L.SWIZZLE if swizzle else 0) | R._mode(mode)
    return list(R._mxfp8(x, flags))


@mxfp8.register_fake
def _(x, rowwise, colwise, swizzle, mode):
    M, N = _check_2d(x)
    e8 = torch.float8_e8m0fnu
    outs = []
    if rowwise:
        outs += [x.new_empty((M, N), dtype=torch.float8_e4m3fn),
                 x.new_empty(R.blocked_shape(M, N // 32) if swizzle else (M, N // 32), dtype=e8)]
    if colwise:
        outs += [x.new_empty((N, M), dtype=torch.float8_e4m3fn),
                 x.new_empty(R.blocked_shape(N, M // 32) if swizzle else (N, M // 32), dtype=e8)]
    return outs


def _nvfp4_fake(x, swizzle, transposed):
    M, N = _check_2d(x)
    rows, cols = (N, M) if transposed else (M, N)
    return (x.new_empty((rows, cols // 2), dtype=torch.float4_e2m1fn_x2),
            x.new_empty(R.blocked_shape(rows, cols // 16) if swizzle else (rows, cols // 16), dtype=torch.float8_e4m3fn))


@custom_op("quant_cast_cuda::nvfp4", mutates_args=(), device_types="cuda")
def nvfp4(x: torch.Tensor, outer_scale: torch.Tensor, swizzle: bool, transposed: bool) -> Tuple[torch.Tensor, torch.Tensor]:
    return R._nvfp4(x, outer_scale, L.SWIZZLE if swizzle else 0, None, transposed)


@nvfp4.register_fake
def _(x, outer_scale, swizzle, transposed):
    return _nvfp4_fake(x, swizzle, transposed)


@custom_op("quant_cast_cuda::nvfp4_sr", mutates_args=(), device_types="cuda")
def nvfp4_sr(x: torch.Tensor, outer_scale: torch.Tensor, key: torch.Tensor, swizzle: bool,
             transposed: bool) -> Tuple[torch.Tensor, torch.Tensor]:
    return R._nvfp4(x, outer_scale, (L.SWIZZLE if swizzle else 0) | L.SR, key, transposed)


@nvfp4_sr.register_fake
def _(x, outer_scale, key, swizzle, transposed):
    return _nvfp4_fake(x, swizzle, transposed)


# ---- the gold signatures over the operators (same names as recipes.py with `_op` for `_cuda`)
def float8_tensorwise_scale_op(x, fmt="e4m3"):
    return torch.ops.quant_cast_cuda.amax(x, "fp8", fmt)


def nvfp4_gs_scale_op(x):
    return torch.ops.quant_cast_cuda.amax(x, "nvfp4", "e4m3")


def float8_tensorwise_op(x, scale, fmt="e4m3", **kwargs):
    return (torch.ops.quant_cast_cuda.fp8_tensorwise(x, scale, fmt),)


def rowwise_fp8_op(x, fmt="e4m3", **kwargs):
    return tuple(torch.ops.quant_cast_cuda.fp8_rowwise(x, fmt))


def colwise_fp8_op(x, fmt="e4m3", **kwargs):
    return tuple(torch.ops.quant_cast_cuda.fp8_colwise(x, fmt))


def _mx(rowwise, colwise, swizzle):
    def fn(x, mode="rceil", **kwargs):
        return tuple(torch.ops.quant_cast_cuda.mxfp8(x, rowwise, colwise, swizzle, mode))
    return fn


mxfp8_op, mxfp8_swizzle_op = _mx(True, False, False), _mx(True, False, True)
mxfp8_dim_m_op, mxfp8_dim_m_swizzle_op = _mx(False, True, False), _mx(False, True, True)
mxfp8_dim_km_op, mxfp8_dim_km_swizzle_op = _mx(True, True, False), _mx(True, True, True)


def nvfp4_gs_op(x, outer_scale, **kwargs):
    return tuple(torch.ops.quant_cast_cuda.nvfp4(x, outer_scale, False, False))


def nvfp4_gs_swizzle_op(x, outer_scale, **kwargs):
    return tuple(torch.ops.quant_cast_cuda.nvfp4(x, outer_scale, True, False))


def nvfp4_gs_swizzle_t_op(x, outer_scale, **kwargs):
    return tuple(torch.ops.quant_cast_cuda.nvfp4(x, outer_scale, True, True))


def nvfp4_gs_swizzle_sr_op(x, outer_scale, key, **kwargs):
    return tuple(torch.ops.quant_cast_cuda.nvfp4_sr(x, outer_scale, key, True, False))


# (gold recipe name, operator-backed function): the recipes of BASELINE configurations 1-5
OP_RECIPES = [
    ("fp8_tensorwise_precalc_scale", float8_tensorwise_op), ("fp8_rowwise", rowwise_fp8_op), ("fp8_colwise", colwise_fp8_op),
    ("mxfp8", mxfp8_op), ("mxfp8_swizzle", mxfp8_swizzle_op), ("mxfp8_dim_m", mxfp8_dim_m_op),
    ("mxfp8_dim_m_swizzle", mxfp8_dim_m_swizzle_op), ("mxfp8_dim_km", mxfp8_dim_km_op),
    ("mxfp8_dim_km_swizzle", mxfp8_dim_km_swizzle_op), ("nvfp4", nvfp4_gs_op), ("nvfp4_swizzle", nvfp4_gs_swizzle_op),
]
