"""`quantize_tensor` / `quantize_tensor_bidirectional` over the CUDA casts.

Same keyword surface, enums, return values and error behaviour as the proposed user-facing API of
vkuzo/quant_cast_bench (experiments/quantize_tensor_api/api.py:76-298), which dispatches
`(scaling_type, orientation, swizzle_type)` to that project's Triton recipes; here every supported
combination lands on a kernel of this package.  On top of the reference's table this backend also takes:
the transposed and the bidirectional nvfp4 casts, stochastic rounding for nvfp4 (`random_key` = uint64
[seed, offset], see `philox_key`), and `InnerScaleCalc.E8M0_FLOOR`.

3-D `(E, M, K)` inputs are quantised per expert (scaling never crosses the E dimension, blocked scales
are per expert and returned flattened as `(E, flat_len)`), one launch per expert into slices of the
stacked outputs.  BlockWise32x32 (one scale per 32x32 block, `skip_transposed_qdata` in the bidirectional call)
and mxfp4 (fp4 data under an E8M0 scale) follow the reference's table as well.

`quantize_tensor_grouped` / `quantize_tensor_grouped_bidirectional` (api.py:301-411) cast a `(total_M, C)`
activation whose rows form token groups ending at `offs`: the data is cast as one matrix, the blocked
scales are laid out per group (moe_utils.py:62-128).  One kernel writes data and grouped scales; the
reference re-lays the scales out afterwards.
"""
from enum import IntEnum

import torch
from torch import Tensor

try:  # core enum (NO_SWIZZLE = 0, SWIZZLE_32_4_4 = 1) where this torch has it
    from torch.nn.functional import SwizzleType
except ImportError:  # pragma: no cover
    class SwizzleType(IntEnum):
        NO_SWIZZLE = 0
        SWIZZLE_32_4_4 = 1

try:
    from enum import StrEnum
except ImportError:  # pragma: no cover
    from enum import Enum

    class StrEnum(str, Enum):
        pass

from . import _lib as L
from . import recipes as R


class ScalingType(IntEnum):
    """Mirrors torch.nn.functional.ScalingType values (api.py:36-48)."""
    TensorWise = 0
    RowWise = 1
    BlockWise1x16 = 2
    BlockWise1x32 = 3
    BlockWise1x128 = 4
    BlockWise128x128 = 5
    BlockWise32x32 = 6


class QuantOrientation(StrEnum):
    NATURAL = "natural"          # block maps to (M, K) as given
    TRANSPOSED = "transposed"    # block maps to the (K, M) view; outputs written transposed-contiguous


class RoundingMode(StrEnum):
    RTNE = "rtne"
    STOCHASTIC = "stochastic"


class InnerScaleCalc(StrEnum):
    E8M0_RCEIL = "e8m0_rceil"
    E8M0_FLOOR = "e8m0_floor"    # addition of this backend (OCP MX FLOOR mode)
    E4M3_NVFP4 = "e4m3_nvfp4"


def _is_swz(swizzle_type):
    if swizzle_type == SwizzleType.SWIZZLE_32_4_4:
        return True
    if swizzle_type == SwizzleType.NO_SWIZZLE:
        return False
    raise ValueError(f"unsupported swizzle_type={swizzle_type!r}; supported: NO_SWIZZLE, SWIZZLE_32_4_4")


def _mx_flags(inner_scale_calc, swz):
    return (L.SWIZZLE if swz else 0) | (L.FLOOR if inner_scale_calc == InnerScaleCalc.E8M0_FLOOR else 0)


def _per_expert(x, flags):
    """mxfp8 of every (M, K) slice of a contiguous (E, M, K) tensor into stacked outputs."""
    if not (x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous()):
        raise ValueError("per-expert casts take a contiguous CUDA bf16 (E, M, K) tensor (quant_cast_cuda has no CPU path)")
    E, M, K = x.shape
    dev, u8 = x.device, torch.uint8
    swz = bool(flags & L.SWIZZLE)
    row, col = bool(flags & L.ROWWISE), bool(flags & L.COLWISE)
    qk = torch.empty((E, M, K), dtype=u8, device=dev) if row else None
    qm = torch.empty((E, K, M), dtype=u8, device=dev) if col else None
    nk = R.blocked_shape(M, K // 32) if swz else (M, K // 32)
    nm = R.blocked_shape(K, M // 32) if swz else (K, M // 32)
    sk = torch.empty((E,) + tuple(nk), dtype=u8, device=dev) if row else None
    sm = torch.empty((E,) + tuple(nm), dtype=u8, device=dev) if col else None
    assert M % 32 == 0 or not col, f"the transposed cast needs M % 32 == 0, got M={M}"
    assert K % 32 == 0, f"mxfp8 needs K % 32 == 0, got K={K}"
    with R._on_device(dev):
        L.check(L.load().qcc_mxfp8_batched(R._p(x), E, M, K, flags, R._p(qk), R._p(sk), R._p(qm), R._p(sm), R._stream(x)),
                "mxfp8_batched")
    L.launch_count += E
    f8, e8 = torch.float8_e4m3fn, torch.float8_e8m0fnu
    outs = []
    if row:
        outs += [qk.view(f8), (sk.reshape(E, -1) if swz else sk).view(e8)]
    if col:
        outs += [qm.view(f8), (sm.reshape(E, -1) if swz else sm).view(e8)]
    return tuple(outs)


def quantize_tensor(input: Tensor, *, qdata_dtype: torch.dtype = torch.float8_e4m3fn,
                    inner_scale_calc: InnerScaleCalc = InnerScaleCalc.E8M0_RCEIL,
                    scaling_type: ScalingType = ScalingType.BlockWise1x32,
                    orientation: QuantOrientation = QuantOrientation.NATURAL,
                    swizzle_type=SwizzleType.SWIZZLE_32_4_4, rounding_mode: RoundingMode = RoundingMode.RTNE,
                    random_key: Tensor | None = None, outer_scale: Tensor | None = None) -> tuple[Tensor, Tensor]:
    """One-orientation block-scaled cast: returns (qdata, scale).  See the module docstring for the table.
    `input` must be bfloat16 (the reference's API documents bf16 or fp32 input; this backend's kernels read bf16 only --
    cast fp32 activations with `.to(torch.bfloat16)` first, which is also what the gold recipes' bf16 amax assumes)."""
    assert input.dim() in (2, 3), f"only 2D or 3D input supported, got {input.dim()}D"
    swz = _is_swz(swizzle_type)
    sr = rounding_mode == RoundingMode.STOCHASTIC
    if sr != (random_key is not None):
        raise ValueError("rounding_mode=STOCHASTIC needs random_key, and random_key is only used by it")

    if qdata_dtype == torch.float4_e2m1fn_x2:
        assert input.dim() == 2, "fp4 quantization is only supported for 2D input"
        assert input.is_contiguous(), "input must be contiguous"
        if inner_scale_calc == InnerScaleCalc.E8M0_RCEIL:   # mxfp4 (api.py:124-135)
            assert outer_scale is None, "outer_scale is only used by nvfp4 quantization"
            if sr:
                raise NotImplementedError("stochastic rounding is implemented for nvfp4 only")
            if scaling_type != ScalingType.BlockWise1x32 or orientation != QuantOrientation.NATURAL:
                raise ValueError(f"unsupported (scaling_type, orientation)=({scaling_type!r}, {orientation!r}) for mxfp4; "
                                 "supported: (BlockWise1x32, NATURAL)")
            return R.mxfp4_cuda(input, swizzle=swz)
        if inner_scale_calc != InnerScaleCalc.E4M3_NVFP4:
            raise ValueError(f"float4_e2m1fn_x2 qdata takes inner_scale_calc=E8M0_RCEIL (mxfp4) or E4M3_NVFP4, got {inner_scale_calc!r}")
        assert outer_scale is not None, "nvfp4 quantization requires a precomputed outer_scale"
        if scaling_type != ScalingType.BlockWise1x16:
            raise ValueError(f"unsupported scaling_type={scaling_type!r} for nvfp4; supported: BlockWise1x16")
        flags = (L.SWIZZLE if swz else 0) | (L.SR if sr else 0)
        if outer_scale.ndim == 2:
            assert outer_scale.shape == (input.shape[0], 1), (
                f"per-token nvfp4 outer_scale must be (M, 1)=({input.shape[0]}, 1), got {tuple(outer_scale.shape)}")
            if orientation != QuantOrientation.NATURAL:
                raise ValueError("per-token nvfp4 supports orientation=NATURAL only")
        return R._nvfp4(input, outer_scale, flags, key=random_key, transposed=orientation == QuantOrientation.TRANSPOSED)

    assert qdata_dtype == torch.float8_e4m3fn, f"only float8_e4m3fn or float4_e2m1fn_x2 qdata supported, got {qdata_dtype}"
    if inner_scale_calc not in (InnerScaleCalc.E8M0_RCEIL, InnerScaleCalc.E8M0_FLOOR):
        raise ValueError(f"float8_e4m3fn qdata takes an E8M0 inner scale, got {inner_scale_calc!r}")
    assert outer_scale is None, "outer_scale is only used by nvfp4 (float4_e2m1fn_x2) quantization"
    if sr:
        raise NotImplementedError("stochastic rounding is implemented for nvfp4 only")
    if scaling_type == ScalingType.BlockWise32x32:   # api.py:203-206 plus the swizzled layouts of the gold index
        assert input.dim() == 2 and input.is_contiguous(), "32x32 blocks take a contiguous 2D input"
        if inner_scale_calc != InnerScaleCalc.E8M0_RCEIL:
            raise ValueError("32x32 blocks take inner_scale_calc=E8M0_RCEIL")
        if orientation == QuantOrientation.NATURAL:
            return R._mxfp8_32x32(input, True, False, swz)
        if orientation == QuantOrientation.TRANSPOSED and swz:
            return R._mxfp8_32x32(input, False, True, True)
        raise ValueError(f"unsupported (orientation, swizzle_type)=({orientation!r}, {swizzle_type!r}) for BlockWise32x32; "
                         "supported: NATURAL with either layout, TRANSPOSED with SWIZZLE_32_4_4")
    if scaling_type != ScalingType.BlockWise1x32:
        raise ValueError(f"unsupported scaling_type={scaling_type!r} for mxfp8; supported: BlockWise1x32, BlockWise32x32")
    if orientation == QuantOrientation.NATURAL:
        direction = L.ROWWISE
    elif orientation == QuantOrientation.TRANSPOSED:
        direction = L.COLWISE
    else:
        raise ValueError(f"orientation={orientation!r} is not supported; supported: NATURAL, TRANSPOSED")
    flags = direction | _mx_flags(inner_scale_calc, swz)
    if input.dim() == 3:
        if not swz:
            raise ValueError("quantize_tensor with 3D (E, N, K) input supports only SWIZZLE_32_4_4")
        return _per_expert(input.contiguous(), flags)
    assert input.is_contiguous(), "input must be contiguous"
    return R._mxfp8(input, flags)


def quantize_tensor_bidirectional(input: Tensor, *, qdata_dtype: torch.dtype = torch.float8_e4m3fn,
                                  inner_scale_calc: InnerScaleCalc = InnerScaleCalc.E8M0_RCEIL,
                                  scaling_type: ScalingType = ScalingType.BlockWise1x32,
                                  swizzle_type=SwizzleType.SWIZZLE_32_4_4, skip_transposed_qdata: bool = False,
                                  rounding_mode: RoundingMode = RoundingMode.RTNE, random_key: Tensor | None = None,
                                  outer_scale: Tensor | None = None):
    """Both orientations from one read of `input`: returns (qk, sk, qm, sm)."""
    assert input.dim() in (2, 3), f"only 2D or 3D input supported, got {input.dim()}D"
    if rounding_mode == RoundingMode.STOCHASTIC or random_key is not None:
        raise NotImplementedError("stochastic rounding is not implemented for the bidirectional casts")
    swz = _is_swz(swizzle_type)
    if skip_transposed_qdata and (scaling_type != ScalingType.BlockWise32x32 or not swz or qdata_dtype != torch.float8_e4m3fn):
        raise ValueError("skip_transposed_qdata is only supported for (BlockWise32x32, SWIZZLE_32_4_4) float8_e4m3fn")
    if qdata_dtype == torch.float4_e2m1fn_x2:
        assert input.dim() == 2 and input.is_contiguous(), "nvfp4 bidirectional takes a contiguous 2D input"
        if inner_scale_calc != InnerScaleCalc.E4M3_NVFP4 or scaling_type != ScalingType.BlockWise1x16:
            raise ValueError("nvfp4 bidirectional takes inner_scale_calc=E4M3_NVFP4 and scaling_type=BlockWise1x16")
        assert outer_scale is not None and outer_scale.numel() == 1, "nvfp4 bidirectional needs a per-tensor outer_scale"
        return R._nvfp4_both(input, outer_scale, L.SWIZZLE if swz else 0)
    assert qdata_dtype == torch.float8_e4m3fn, f"only float8_e4m3fn or float4_e2m1fn_x2 qdata supported, got {qdata_dtype}"
    if inner_scale_calc not in (InnerScaleCalc.E8M0_RCEIL, InnerScaleCalc.E8M0_FLOOR):
        raise ValueError(f"float8_e4m3fn qdata takes an E8M0 inner scale, got {inner_scale_calc!r}")
    assert outer_scale is None, "outer_scale is only used by nvfp4 (float4_e2m1fn_x2) quantization"
    if scaling_type == ScalingType.BlockWise32x32:   # api.py:281-285; with the transposed data: gold G:900-910
        assert input.dim() == 2 and input.is_contiguous(), "32x32 blocks take a contiguous 2D input"
        if inner_scale_calc != InnerScaleCalc.E8M0_RCEIL or not swz:
            raise ValueError("32x32 blocks take inner_scale_calc=E8M0_RCEIL and swizzle_type=SWIZZLE_32_4_4 here")
        return R._mxfp8_32x32(input, True, True, True, transposed_data=not skip_transposed_qdata)
    if scaling_type != ScalingType.BlockWise1x32:
        raise ValueError(f"unsupported scaling_type={scaling_type!r}; supported: BlockWise1x32, BlockWise32x32")
    flags = L.ROWWISE | L.COLWISE | _mx_flags(inner_scale_calc, swz)
    if input.dim() == 3:
        if not swz:
            raise ValueError("quantize_tensor_bidirectional with 3D (E, N, K) input supports only SWIZZLE_32_4_4")
        return _per_expert(input.contiguous(), flags)
    assert input.is_contiguous(), "input must be contiguous"
    return R._mxfp8(input, flags)


def _grouped(x, offs, flags):
    lib = L.load()
    assert x.dim() == 2, f"grouped casts take a 2D (total_M, C) input, got {x.dim()}D"
    x = x.contiguous()
    R._check_x(x)
    M, C = x.shape
    assert C % 32 == 0 and M % 32 == 0, f"grouped mxfp8 needs total_M % 32 == 0 and C % 32 == 0, got {(M, C)}"
    assert offs.dim() == 1 and offs.device == x.device, "offs: 1-D tensor of group ends on the input's device"
    offs = offs.to(torch.int32).contiguous()
    G = offs.numel()
    dev, u8 = x.device, torch.uint8
    row, col = bool(flags & L.ROWWISE), bool(flags & L.COLWISE)
    assert not row or C % 128 == 0, f"the natural orientation of a grouped cast needs C % 128 == 0, got C={C}"
    qk = torch.empty((M, C), dtype=u8, device=dev) if row else None
    sk = torch.empty((M + G * 128, C // 32), dtype=u8, device=dev) if row else None
    qm = torch.empty((C, M), dtype=u8, device=dev) if col else None
    sm = torch.empty((-(-C // 128) * 128, M // 32 + G * 4), dtype=u8, device=dev) if col else None
    nws = lib.qcc_mxfp8_grouped_workspace_bytes(M)
    ws = torch.empty(max(nws, 16), dtype=u8, device=dev)
    with R._on_device(dev):
        L.check(lib.qcc_mxfp8_grouped(R._p(x), M, C, flags, R._p(offs), G, R._p(qk), R._p(sk), R._p(qm), R._p(sm),
                                      R._p(ws), nws, R._stream(x)), "mxfp8_grouped")
    L.launch_count += 1
    f8, e8 = torch.float8_e4m3fn, torch.float8_e8m0fnu
    outs = []
    if row:
        outs += [qk.view(f8), sk.view(e8)]
    if col:
        outs += [qm.view(f8), sm.view(e8)]
    return tuple(outs)


def _check_grouped(qdata_dtype, inner_scale_calc, scaling_type, swizzle_type, rounding_mode, random_key, outer_scale, who):
    assert qdata_dtype == torch.float8_e4m3fn, f"only float8_e4m3fn qdata supported, got {qdata_dtype}"
    if inner_scale_calc not in (InnerScaleCalc.E8M0_RCEIL, InnerScaleCalc.E8M0_FLOOR):
        raise ValueError(f"float8_e4m3fn qdata takes an E8M0 inner scale, got {inner_scale_calc!r}")
    assert outer_scale is None, f"outer_scale is not supported by {who}"
    if rounding_mode == RoundingMode.STOCHASTIC or random_key is not None:
        raise NotImplementedError("stochastic rounding is not implemented for the grouped casts")
    if scaling_type != ScalingType.BlockWise1x32 or not _is_swz(swizzle_type):
        raise ValueError(f"unsupported (scaling_type, swizzle_type)=({scaling_type!r}, {swizzle_type!r}); "
                         f"{who} supports only (BlockWise1x32, SWIZZLE_32_4_4)")


def quantize_tensor_grouped(input: Tensor, offs: Tensor, *, qdata_dtype: torch.dtype = torch.float8_e4m3fn,
                            inner_scale_calc: InnerScaleCalc = InnerScaleCalc.E8M0_RCEIL,
                            scaling_type: ScalingType = ScalingType.BlockWise1x32,
                            orientation: QuantOrientation = QuantOrientation.NATURAL,
                            swizzle_type=SwizzleType.SWIZZLE_32_4_4, rounding_mode: RoundingMode = RoundingMode.RTNE,
                            random_key: Tensor | None = None, outer_scale: Tensor | None = None) -> tuple[Tensor, Tensor]:
    """One-orientation cast of token groups (api.py:301-359).  `offs[g]` is the row where group g ends; every
    group size must be a multiple of 32 (the caller pads).  NATURAL: (q (M, C), scales (M + G*128, C/32));
    TRANSPOSED: (q (C, M), scales (ceil128(C), M/32 + G*4))."""
    _check_grouped(qdata_dtype, inner_scale_calc, scaling_type, swizzle_type, rounding_mode, random_key, outer_scale,
                   "quantize_tensor_grouped")
    if orientation == QuantOrientation.NATURAL:
        direction = L.ROWWISE
    elif orientation == QuantOrientation.TRANSPOSED:
        direction = L.COLWISE
    else:
        raise ValueError(f"orientation={orientation!r} is not supported; supported: NATURAL, TRANSPOSED")
    return _grouped(input, offs, direction | _mx_flags(inner_scale_calc, True))


def quantize_tensor_grouped_bidirectional(input: Tensor, offs: Tensor, *, qdata_dtype: torch.dtype = torch.float8_e4m3fn,
                                          inner_scale_calc: InnerScaleCalc = InnerScaleCalc.E8M0_RCEIL,
                                          scaling_type: ScalingType = ScalingType.BlockWise1x32,
                                          swizzle_type=SwizzleType.SWIZZLE_32_4_4, skip_transposed_qdata: bool = False,
                                          rounding_mode: RoundingMode = RoundingMode.RTNE,
                                          random_key: Tensor | None = None, outer_scale: Tensor | None = None):
    """Both orientations of the grouped cast from one read of `input` (api.py:362-411):
    (q_nat, sb_nat, q_t, sb_t)."""
    _check_grouped(qdata_dtype, inner_scale_calc, scaling_type, swizzle_type, rounding_mode, random_key, outer_scale,
                   "quantize_tensor_grouped_bidirectional")
    if skip_transposed_qdata:
        raise NotImplementedError("skip_transposed_qdata is not supported by quantize_tensor_grouped_bidirectional")
    return _grouped(input, offs, L.ROWWISE | L.COLWISE | _mx_flags(inner_scale_calc, True))


def pad_token_groups(input: Tensor, offs: Tensor):
    """`_pad_token_groups` of the reference (experiments/quantize_tensor_api/moe_utils.py:35-59) as one kernel and
    without the host sync on the group sizes: every group's rows moved to the start of its 32-row-aligned slot of a
    zero matrix with ceil32(total_M + 32 G) rows.  Returns (padded_tokens, padded_start_offsets, padded_offsets)."""
    lib = L.load()
    assert input.dim() == 2 and input.is_cuda, "a 2D CUDA tensor"
    x = input.contiguous()
    M, C = x.shape
    row_bytes = C * x.element_size()
    assert row_bytes % 16 == 0, f"rows must be a multiple of 16 bytes, got {row_bytes}"
    offs32 = offs.to(torch.int32).contiguous()
    G = offs32.numel()
    rows_out = lib.qcc_padded_token_rows(M, G)
    out = torch.empty((rows_out, C), dtype=x.dtype, device=x.device)
    padded_offs = torch.empty(G, dtype=torch.int32, device=x.device)
    nws = lib.qcc_token_pad_workspace_bytes(M, G)
    ws = torch.empty(nws, dtype=torch.uint8, device=x.device)
    with R._on_device(x.device):
        L.check(lib.qcc_pad_token_groups(R._p(x), M, row_bytes, R._p(offs32), G, R._p(out), R._p(padded_offs), R._p(ws), nws,
                                         R._stream(x)), "pad_token_groups")
    L.launch_count += 2
    sizes = torch.diff(offs32, prepend=offs32.new_zeros(1))
    padded_sizes = (sizes + 31) // 32 * 32
    return out, padded_offs - padded_sizes, padded_offs


def unpad_token_groups(padded: Tensor, offs: Tensor):
    """`_unpad_token_groups` (moe_main.py:54-68): the (total_M, C) rows of a tensor in the padded frame of
    `pad_token_groups`; `offs` are the unpadded group ends."""
    lib = L.load()
    assert padded.dim() == 2 and padded.is_cuda, "a 2D CUDA tensor"
    p = padded.contiguous()
    offs32 = offs.to(torch.int32).contiguous()
    G = offs32.numel()
    C = p.shape[1]
    row_bytes = C * p.element_size()
    # total_M is the last offset; it fixes the output shape, so it is read back once (the reference does the same)
    M = int(offs32[-1].item())
    assert p.shape[0] == lib.qcc_padded_token_rows(M, G), "padded must have qcc_padded_token_rows(total_M, G) rows"
    out = torch.empty((M, C), dtype=p.dtype, device=p.device)
    nws = lib.qcc_token_pad_workspace_bytes(M, G)
    ws = torch.empty(nws, dtype=torch.uint8, device=p.device)
    with R._on_device(p.device):
        L.check(lib.qcc_unpad_token_groups(R._p(p), M, row_bytes, R._p(offs32), G, R._p(out), R._p(ws), nws, R._stream(p)),
                "unpad_token_groups")
    L.launch_count += 2
    return out


def _grouped_pad(x, offs, flags):
    lib = L.load()
    assert x.dim() == 2, f"grouped casts take a 2D (total_M, C) input, got {x.dim()}D"
    x = x.contiguous()
    R._check_x(x)
    M, C = x.shape
    row, col = bool(flags & L.ROWWISE), bool(flags & L.COLWISE)
    assert C % 32 == 0 and (not row or C % 128 == 0), f"needs C % 32 == 0 (C % 128 == 0 for the natural orientation), got C={C}"
    assert offs.dim() == 1 and offs.device == x.device, "offs: 1-D tensor of group ends on the input's device"
    offs32 = offs.to(torch.int32).contiguous()
    G = offs32.numel()
    Rr = lib.qcc_padded_token_rows(M, G)
    dev, u8 = x.device, torch.uint8
    qk = torch.empty((Rr, C), dtype=u8, device=dev) if row else None
    sk = torch.empty((Rr + G * 128, C // 32), dtype=u8, device=dev) if row else None
    qm = torch.empty((C, Rr), dtype=u8, device=dev) if col else None
    sm = torch.empty((-(-C // 128) * 128, Rr // 32 + G * 4), dtype=u8, device=dev) if col else None
    padded_offs = torch.empty(G, dtype=torch.int32, device=dev)
    nws = lib.qcc_token_pad_workspace_bytes(M, G)
    ws = torch.empty(nws, dtype=u8, device=dev)
    with R._on_device(dev):
        L.check(lib.qcc_mxfp8_grouped_pad(R._p(x), M, C, flags, R._p(offs32), G, R._p(qk), R._p(sk), R._p(qm), R._p(sm),
                                          R._p(padded_offs), R._p(ws), nws, R._stream(x)), "mxfp8_grouped_pad")
    L.launch_count += 2
    f8, e8 = torch.float8_e4m3fn, torch.float8_e8m0fnu
    outs = []
    if row:
        outs += [qk.view(f8), sk.view(e8)]
    if col:
        outs += [qm.view(f8), sm.view(e8)]
    return tuple(outs) + (padded_offs,)


def quantize_tensor_grouped_padded(input: Tensor, offs: Tensor, *, orientation: QuantOrientation = QuantOrientation.NATURAL,
                                   inner_scale_calc: InnerScaleCalc = InnerScaleCalc.E8M0_RCEIL):
    """`quantize_tensor_grouped(*_pad_token_groups(input, offs)[::2])` in one pass over the unpadded input (the call
    pattern of moe_main.py:178-188): token groups of any size; returns (qdata, blocked scales, padded_offsets)."""
    if inner_scale_calc not in (InnerScaleCalc.E8M0_RCEIL, InnerScaleCalc.E8M0_FLOOR):
        raise ValueError(f"float8_e4m3fn qdata takes an E8M0 inner scale, got {inner_scale_calc!r}")
    if orientation not in (QuantOrientation.NATURAL, QuantOrientation.TRANSPOSED):
        raise ValueError(f"orientation={orientation!r} is not supported; supported: NATURAL, TRANSPOSED")
    direction = L.ROWWISE if orientation == QuantOrientation.NATURAL else L.COLWISE
    return _grouped_pad(input, offs, direction | _mx_flags(inner_scale_calc, True))


def quantize_tensor_grouped_padded_bidirectional(input: Tensor, offs: Tensor, *,
                                                 inner_scale_calc: InnerScaleCalc = InnerScaleCalc.E8M0_RCEIL):
    """Both orientations of the padded grouped cast from one read: (q_nat, sb_nat, q_t, sb_t, padded_offsets)."""
    if inner_scale_calc not in (InnerScaleCalc.E8M0_RCEIL, InnerScaleCalc.E8M0_FLOOR):
        raise ValueError(f"float8_e4m3fn qdata takes an E8M0 inner scale, got {inner_scale_calc!r}")
    return _grouped_pad(input, offs, L.ROWWISE | L.COLWISE | _mx_flags(inner_scale_calc, True))

