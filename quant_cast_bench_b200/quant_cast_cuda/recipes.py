"""CUDA implementations of the quant_cast_gold recipes.

Mirrors the backend recipe files of vkuzo/quant_cast_bench (quant_cast_triton/recipes.py:48-65,
:1796-1835): every `<name>_cuda(*inputs, **kwargs) -> tuple[Tensor, ...]` takes the positional inputs
of the gold `pt_ref_fn` of the same recipe (quant_cast_gold/recipes.py), accepts and ignores the
tile kwargs `global_row / global_col / num_col`, allocates its outputs with torch.empty on x.device,
returns the gold shapes and dtype views, reads scalar aux inputs on the device (no host sync), and
launches on the current CUDA stream.  `ALL_RECIPES` lists `(gold recipe name, QuantCastCudaRecipe)`.

Functions without a gold counterpart are marked "extension": e5m2 (`fmt="e5m2"`), the FLOOR scale
mode (`mode="floor"`), the transposed nvfp4 cast, and Philox-keyed stochastic rounding.
"""
from dataclasses import dataclass
from typing import Callable, Optional

import torch

from . import _lib as L

_FMT = {"e4m3": L.FMT_E4M3, "e5m2": L.FMT_E5M2, torch.float8_e4m3fn: L.FMT_E4M3, torch.float8_e5m2: L.FMT_E5M2}
_FP8_DTYPE = {L.FMT_E4M3: torch.float8_e4m3fn, L.FMT_E5M2: torch.float8_e5m2}


def _fmt(fmt):
    if fmt not in _FMT:
        raise ValueError(f"unknown fp8 format {fmt!r}; use 'e4m3' or 'e5m2'")
    return _FMT[fmt]


def _mode(mode):
    if mode not in ("rceil", "floor"):
        raise ValueError(f"unknown mxfp8 scale mode {mode!r}; use 'rceil' or 'floor'")
    return L.FLOOR if mode == "floor" else 0


def _check_x(x, name="x"):
    if not (isinstance(x, torch.Tensor) and x.is_cuda):
        raise ValueError(f"{name} must be a CUDA tensor (quant_cast_cuda has no CPU path)")
    assert x.dtype == torch.bfloat16, f"{name} must be bfloat16, got {x.dtype}"
    assert x.is_contiguous() and x.dim() == 2, f"{name} must be a contiguous 2-D tensor"
    return x


def _p(t):
    return t.data_ptr() if t is not None else None


def _stream(x):
    return torch.cuda.current_stream(x.device).cuda_stream


class _on_device:
    """`with torch.cuda.device(...)` only when the tensor's device is not already current (the context
    manager costs more host time than a whole launch)."""

    def __init__(self, dev):
        self.ctx = None if dev.index is None or dev.index == torch.cuda.current_device() else torch.cuda.device(dev)

    def __enter__(self):
        if self.ctx is not None:
            self.ctx.__enter__()

    def __exit__(self, *exc):
        if self.ctx is not None:
            self.ctx.__exit__(*exc)
        return False


def _cdiv(a, b):
    return (a + b - 1) // b


def blocked_shape(rows, cols):
    """Shape of the 32x4x4 blocked scale grid of a (rows, cols) block-scale matrix (gold G:1000-1037)."""
    return (_cdiv(rows, 128), _cdiv(cols, 4), 32, 16)


def philox_key(seed, offset=0, device="cuda"):
    """A Philox4x32-10 key as the stochastic-rounding casts take it: uint64 [seed, offset] on the device."""
    t = torch.tensor([int(seed) & 0x7FFFFFFFFFFFFFFF, int(offset)], dtype=torch.int64, device=device)
    return t.view(torch.uint64)


def stream_copy_cuda(src, dst):
    """dst = src by this library's plain copy kernel (same access pattern as the streaming casts): the yardstick the
    benchmarks hold the casts against.  Tensors of equal byte size, contiguous, a multiple of 16 bytes."""
    lib = L.load()
    assert src.is_cuda and dst.is_cuda and src.is_contiguous() and dst.is_contiguous()
    nbytes = src.numel() * src.element_size()
    assert nbytes == dst.numel() * dst.element_size(), "source and destination differ in size"
    with _on_device(src.device):
        L.check(lib.qcc_stream_copy(_p(src), _p(dst), nbytes, _stream(src)), "stream_copy")
    L.launch_count += 1
    return dst


def stream_fold_cuda(src, dst, ratio):
    """dst = XOR-fold of src, `ratio` (2 or 4) 16-byte pieces into one: the data movement of a cast that writes
    1/ratio of what it reads, without the arithmetic -- the yardstick for the fp8 / mxfp8 casts (2) and nvfp4 (4)."""
    lib = L.load()
    assert src.is_cuda and dst.is_cuda and src.is_contiguous() and dst.is_contiguous()
    nbytes = src.numel() * src.element_size()
    assert nbytes == ratio * dst.numel() * dst.element_size(), "dst must hold 1/ratio of the bytes of src"
    with _on_device(src.device):
        L.check(lib.qcc_stream_fold(_p(src), _p(dst), nbytes, ratio, _stream(src)), "stream_fold")
    L.launch_count += 1
    return dst


# --------------------------------------------------------------------------------------------
# amax and per-tensor scales
# --------------------------------------------------------------------------------------------
_amax_ws_cache = {}   # (device index, stream handle) -> prepared workspace


def new_amax_workspace(device, stream=None):
    """A workspace for the one-launch amax (`workspace=` of the amax functions and of `mxfp8_*_amax_cuda`): cleared once
    here, left cleared by every call that uses it.  Calls that share one must not overlap on the GPU."""
    lib = L.load()
    device = torch.device(device)
    n = lib.qcc_amax_workspace_bytes()
    ws = torch.empty(n, dtype=torch.uint8, device=device)
    st = stream if stream is not None else torch.cuda.current_stream(device).cuda_stream
    with _on_device(device):
        L.check(lib.qcc_amax_workspace_init(_p(ws), n, st), "amax_workspace_init")
    return ws


def _amax_workspace(x):
    """The cached workspace of (device, current stream), or None while the stream is being captured into a CUDA
    graph and nothing is cached for it (memory allocated during a capture belongs to that graph)."""
    key = (x.device.index, _stream(x))
    ws = _amax_ws_cache.get(key)
    if ws is None and not torch.cuda.is_current_stream_capturing():
        ws = _amax_ws_cache[key] = new_amax_workspace(x.device)
    return ws


def _amax(x, mode, fmt=L.FMT_E4M3, workspace=None):
    lib = L.load()
    assert x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous()
    out = torch.empty((), dtype=torch.float32, device=x.device)
    ws = workspace if workspace is not None else _amax_workspace(x)
    ws_bytes = lib.qcc_amax_workspace_bytes()
    with _on_device(x.device):
        if ws is not None:     # one launch
            L.check(lib.qcc_amax_bf16(_p(x), x.numel(), mode | L.AMAX_ONE_LAUNCH | L.div_flag(), fmt, _p(out), _p(ws), ws_bytes, _stream(x)), "amax")
            L.launch_count += 1
        else:                  # two launches, any workspace contents
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=x.device)
            L.check(lib.qcc_amax_bf16(_p(x), x.numel(), mode | L.div_flag(), fmt, _p(out), _p(ws), ws_bytes, _stream(x)), "amax")
            L.launch_count += 2
    return out


def amax_cuda(x, workspace=None):
    """max |x| as a 0-dim fp32 tensor (exact: a bf16 magnitude)."""
    return _amax(x, L.AMAX_RAW, workspace=workspace)


def scale_from_amax_cuda(amax, kind, fmt="e4m3"):
    """Per-tensor scale from an already reduced amax: kind 'fp8' -> max(amax, bf16(1e-12)) / fp8_max,
    kind 'nvfp4' -> amax / 2688.  Used after the all-reduce of per-shard amaxes."""
    lib = L.load()
    mode = {"fp8": L.AMAX_FP8_SCALE, "nvfp4": L.AMAX_NVFP4_SCALE, "raw": L.AMAX_RAW}[kind]
    a = amax.reshape(-1)[:1].contiguous().float()
    out = torch.empty((), dtype=torch.float32, device=amax.device)
    with _on_device(amax.device):
        L.check(lib.qcc_scale_from_amax(_p(a), mode | L.div_flag(), _fmt(fmt), _p(out), _stream(amax)), "scale_from_amax")
    L.launch_count += 1
    return out


def float8_tensorwise_scale_cuda(x, fmt="e4m3", workspace=None):
    """gold float8_tensorwise_scale (G:1179-1183): 0-dim fp32 scale = max(amax, bf16(1e-12)) / fp8_max."""
    return _amax(x, L.AMAX_FP8_SCALE, _fmt(fmt), workspace=workspace)


def nvfp4_gs_scale_cuda(x, workspace=None):
    """gold nvfp4_gs_scale (G:1243-1246): 0-dim fp32 outer scale = amax / (448 * 6)."""
    return _amax(x, L.AMAX_NVFP4_SCALE, workspace=workspace)


# --------------------------------------------------------------------------------------------
# fp8
# --------------------------------------------------------------------------------------------
def float8_tensorwise_cuda(x, scale, fmt="e4m3", **kwargs):
    """gold float8_tensorwise_f (G:1186-1191): (qdata,) = fp8(x * (1 / scale))."""
    lib = L.load()
    _check_x(x)
    f = _fmt(fmt)
    assert scale.device == x.device and scale.dtype == torch.float32 and scale.numel() == 1
    q = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    with _on_device(x.device):
        L.check(lib.qcc_fp8_tensorwise(_p(x), x.numel(), _p(scale), f, _p(q), _stream(x)), "fp8_tensorwise")
    L.launch_count += 1
    return (q.view(_FP8_DTYPE[f]),)


def float8_tensorwise_from_amax_cuda(x, amax, fmt="e4m3"):
    """float8_tensorwise_scale + float8_tensorwise_f (G:1179-1191) for an amax that is already known (e.g. reduced over
    shards): the division amax -> scale happens in the cast's prologue.  Returns (qdata, scale)."""
    lib = L.load()
    _check_x(x)
    f = _fmt(fmt)
    assert amax.device == x.device and amax.dtype == torch.float32 and amax.numel() == 1
    q = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    scale = torch.empty((), dtype=torch.float32, device=x.device)
    with _on_device(x.device):
        L.check(lib.qcc_fp8_tensorwise_from_amax(_p(x), x.numel(), _p(amax), f | L.div_flag(), _p(q), _p(scale), _stream(x)),
                "fp8_tensorwise_from_amax")
    L.launch_count += 1
    return q.view(_FP8_DTYPE[f]), scale


def rowwise_fp8_cuda(x, fmt="e4m3", **kwargs):
    """gold rowwise_fp8_f (G:301-307): (qdata (M, N), scale (M, 1) fp32)."""
    lib = L.load()
    _check_x(x)
    f = _fmt(fmt)
    M, N = x.shape
    q = torch.empty((M, N), dtype=torch.uint8, device=x.device)
    s = torch.empty((M, 1), dtype=torch.float32, device=x.device)
    with _on_device(x.device):
        L.check(lib.qcc_fp8_rowwise(_p(x), M, N, f | L.div_flag(), _p(q), _p(s), _stream(x)), "fp8_rowwise")
    L.launch_count += 1
    return q.view(_FP8_DTYPE[f]), s


def rowwise_precalc_scale_cuda(x, fmt="e4m3"):
    """gold rowwise_precalc_scale (G:389-393): (M, 1) fp32 per-row scale."""
    lib = L.load()
    _check_x(x)
    M, N = x.shape
    s = torch.empty((M, 1), dtype=torch.float32, device=x.device)
    with _on_device(x.device):
        L.check(lib.qcc_fp8_rowwise(_p(x), M, N, _fmt(fmt) | L.div_flag(), None, _p(s), _stream(x)), "fp8_rowwise_scale")
    L.launch_count += 1
    return s


def rowwise_precalc_cuda(x, scale, fmt="e4m3", **kwargs):
    """gold rowwise_precalc_f (G:396-399): (qdata,) = fp8(x / scale) with a given (M, 1) scale."""
    lib = L.load()
    _check_x(x)
    f = _fmt(fmt)
    M, N = x.shape
    assert scale.device == x.device and scale.dtype == torch.float32 and scale.numel() == M and scale.is_contiguous()
    q = torch.empty((M, N), dtype=torch.uint8, device=x.device)
    with _on_device(x.device):
        L.check(lib.qcc_fp8_rowwise_precalc(_p(x), M, N, _p(scale), f, _p(q), _stream(x)), "fp8_rowwise_precalc")
    L.launch_count += 1
    return (q.view(_FP8_DTYPE[f]),)


def colwise_fp8_cuda(x, fmt="e4m3", **kwargs):
    """gold colwise_fp8_f (G:339-349): (qdata (N, M), scale (N, 1) fp32), one scale per column, transposed."""
    lib = L.load()
    _check_x(x)
    f = _fmt(fmt)
    M, N = x.shape
    assert N % 8 == 0 and M % 16 == 0, f"colwise fp8 needs N % 8 == 0 and M % 16 == 0, got {M}x{N}"
    q = torch.empty((N, M), dtype=torch.uint8, device=x.device)
    s = torch.empty((N, 1), dtype=torch.float32, device=x.device)
    ws_bytes = int(lib.qcc_fp8_colwise_workspace_bytes(M, N))
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=x.device)
    with _on_device(x.device):
        L.check(lib.qcc_fp8_colwise(_p(x), M, N, f | L.div_flag(), _p(q), _p(s), _p(ws), ws_bytes, _stream(x)), "fp8_colwise")
    L.launch_count += 2
    return q.view(_FP8_DTYPE[f]), s


def colwise_precalc_scale_cuda(x, fmt="e4m3"):
    """gold colwise_precalc_scale (G:438-442): (1, N) fp32 per-column scale -- the column maxima pass alone (one read
    of x, no cast)."""
    lib = L.load()
    _check_x(x)
    M, N = x.shape
    assert N % 8 == 0 and M % 16 == 0, f"colwise fp8 needs N % 8 == 0 and M % 16 == 0, got {M}x{N}"
    s = torch.empty((1, N), dtype=torch.float32, device=x.device)
    ws_bytes = int(lib.qcc_fp8_colwise_workspace_bytes(M, N))
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=x.device)
    with _on_device(x.device):
        L.check(lib.qcc_fp8_colwise(_p(x), M, N, _fmt(fmt) | L.div_flag(), None, _p(s), _p(ws), ws_bytes, _stream(x)), "fp8_colwise_scale")
    L.launch_count += 2
    return s


def colwise_precalc_cuda(x, scale, fmt="e4m3", **kwargs):
    """gold colwise_precalc_f (G:445-449): (qdata (N, M),) = fp8(x / scale) with a given (1, N) scale."""
    lib = L.load()
    _check_x(x)
    f = _fmt(fmt)
    M, N = x.shape
    assert N % 8 == 0 and M % 16 == 0, f"colwise fp8 needs N % 8 == 0 and M % 16 == 0, got {M}x{N}"
    assert scale.device == x.device and scale.dtype == torch.float32 and scale.numel() == N and scale.is_contiguous()
    q = torch.empty((N, M), dtype=torch.uint8, device=x.device)
    with _on_device(x.device):
        L.check(lib.qcc_fp8_colwise_precalc(_p(x), M, N, _p(scale), f, _p(q), _stream(x)), "fp8_colwise_precalc")
    L.launch_count += 1
    return (q.view(_FP8_DTYPE[f]),)


# --------------------------------------------------------------------------------------------
# mxfp8
# --------------------------------------------------------------------------------------------
def _mxfp8(x, flags):
    lib = L.load()
    _check_x(x)
    M, N = x.shape
    assert N % 32 == 0, f"mxfp8 needs N % 32 == 0, got N={N}"
    if flags & L.COLWISE:
        assert M % 32 == 0, f"mxfp8 dim-m needs M % 32 == 0, got M={M}"
    swz = bool(flags & L.SWIZZLE)
    dev = x.device
    qk = sk = qm = sm = None
    if flags & L.ROWWISE:
        qk = torch.empty((M, N), dtype=torch.uint8, device=dev)
        sk = torch.empty(blocked_shape(M, N // 32) if swz else (M, N // 32), dtype=torch.uint8, device=dev)
    if flags & L.COLWISE:
        qm = torch.empty((N, M), dtype=torch.uint8, device=dev)
        sm = torch.empty(blocked_shape(N, M // 32) if swz else (N, M // 32), dtype=torch.uint8, device=dev)
    with _on_device(dev):
        L.check(lib.qcc_mxfp8(_p(x), M, N, flags, _p(qk), _p(sk), _p(qm), _p(sm), _stream(x)), "mxfp8")
    L.launch_count += 1
    outs = []
    if flags & L.ROWWISE:
        outs += [qk.view(torch.float8_e4m3fn), sk.view(torch.float8_e8m0fnu)]
    if flags & L.COLWISE:
        outs += [qm.view(torch.float8_e4m3fn), sm.view(torch.float8_e8m0fnu)]
    return tuple(outs)


def mxfp8_with_amax_cuda(x, swizzle=True, mode="rceil", workspace=None):
    """mxfp8_f / mxfp8_swizzle_f (G:561-568, G:1051-1053) and max |x| from ONE read of x: (qdata, scale, amax) with amax
    the raw 0-dim fp32 maximum that nvfp4_gs_scale (G:1243-1246) or float8_tensorwise_scale would reduce again."""
    lib = L.load()
    _check_x(x)
    M, N = x.shape
    assert N % 32 == 0, f"mxfp8 needs N % 32 == 0, got N={N}"
    flags = L.ROWWISE | (L.SWIZZLE if swizzle else 0) | _mode(mode)
    dev = x.device
    ws = workspace if workspace is not None else _amax_workspace(x)
    if ws is None:
        raise RuntimeError("mxfp8_with_amax_cuda needs workspace=new_amax_workspace(device) when called during a CUDA graph capture")
    qk = torch.empty((M, N), dtype=torch.uint8, device=dev)
    sk = torch.empty(blocked_shape(M, N // 32) if swizzle else (M, N // 32), dtype=torch.uint8, device=dev)
    amax = torch.empty((), dtype=torch.float32, device=dev)
    with _on_device(dev):
        L.check(lib.qcc_mxfp8_amax(_p(x), M, N, flags, _p(qk), _p(sk), _p(amax), _p(ws), ws.numel(), _stream(x)), "mxfp8_amax")
    L.launch_count += 1
    return qk.view(torch.float8_e4m3fn), sk.view(torch.float8_e8m0fnu), amax


def mxfp4_cuda(x, swizzle=False, **kwargs):
    """gold mxfp4_f (G:607-617): 1x32 blocks, e8m0 RCEIL scale of amax / 6, fp4 e2m1 data packed two per byte:
    (qdata (M, N/2), scale (M, N/32)); swizzle=True gives the blocked scale layout (extension)."""
    lib = L.load()
    _check_x(x)
    M, N = x.shape
    assert N % 32 == 0, f"mxfp4 needs N % 32 == 0, got N={N}"
    q = torch.empty((M, N // 2), dtype=torch.uint8, device=x.device)
    s = torch.empty(blocked_shape(M, N // 32) if swizzle else (M, N // 32), dtype=torch.uint8, device=x.device)
    with _on_device(x.device):
        L.check(lib.qcc_mxfp4(_p(x), M, N, L.SWIZZLE if swizzle else 0, _p(q), _p(s), _stream(x)), "mxfp4")
    L.launch_count += 1
    return q.view(torch.float4_e2m1fn_x2), s.view(torch.float8_e8m0fnu)


def _fp8_block128(x, row, col):
    lib = L.load()
    _check_x(x)
    M, N = x.shape
    if row:
        assert N % 128 == 0, f"1x128 blocks need N % 128 == 0, got N={N}"
    if col:
        assert M % 128 == 0 and N % 8 == 0, f"128x1 blocks need M % 128 == 0 and N % 8 == 0, got {M}x{N}"
    dev = x.device
    qk = torch.empty((M, N), dtype=torch.uint8, device=dev) if row else None
    sk = torch.empty((M, N // 128), dtype=torch.float32, device=dev) if row else None
    qm = torch.empty((N, M), dtype=torch.uint8, device=dev) if col else None
    sm = torch.empty((N, M // 128), dtype=torch.float32, device=dev) if col else None
    flags = (L.ROWWISE if row else 0) | (L.COLWISE if col else 0)
    with _on_device(dev):
        L.check(lib.qcc_fp8_block128(_p(x), M, N, flags | L.div_flag(), _p(qk), _p(sk), _p(qm), _p(sm), _stream(x)), "fp8_block128")
    L.launch_count += 1
    outs = []
    if row:
        outs += [qk.view(torch.float8_e4m3fn), sk]
    if col:
        outs += [qm.view(torch.float8_e4m3fn), sm]
    return tuple(outs)


def deepseek_1x128_cuda(x, **kwargs):
    """gold deepseek_1x128_f (G:103-110): (qdata (M, N) e4m3, scale (M, N/128) fp32)."""
    return _fp8_block128(x, True, False)


def deepseek_1x128_dim_m_cuda(x, **kwargs):
    """gold deepseek_1x128_dim_m_f (G:194-214): 128x1 blocks, (qdata (N, M), scale (N, M/128))."""
    return _fp8_block128(x, False, True)


def deepseek_1x128_dim_km_cuda(x, **kwargs):
    """gold deepseek_1x128_dim_km_f (G:251-277): both from one read (the amax clamp is in fp32 there)."""
    return _fp8_block128(x, True, True)


def deepseek_128x128_cuda(x, **kwargs):
    """gold deepseek_128x128_f (G:141-161): (qdata (M, N), scale (M/128, N/128) fp32)."""
    lib = L.load()
    _check_x(x)
    M, N = x.shape
    assert M % 128 == 0 and N % 128 == 0, f"128x128 blocks need M % 128 == 0 and N % 128 == 0, got {M}x{N}"
    q = torch.empty((M, N), dtype=torch.uint8, device=x.device)
    s = torch.empty((M // 128, N // 128), dtype=torch.float32, device=x.device)
    with _on_device(x.device):
        L.check(lib.qcc_fp8_block128x128(_p(x), M, N, L.div_flag(), _p(q), _p(s), _stream(x)), "fp8_block128x128")
    L.launch_count += 1
    return q.view(torch.float8_e4m3fn), s


def _mxfp8_32x32(x, row, col, swz, transposed_data=True):
    """32x32 blocks: one e8m0 scale per block, shared by both orientations (QCC_BLOCK32)."""
    lib = L.load()
    _check_x(x)
    M, N = x.shape
    assert M % 32 == 0 and N % 32 == 0, f"mxfp8 32x32 needs M % 32 == 0 and N % 32 == 0, got {M}x{N}"
    dev, u8 = x.device, torch.uint8
    qk = torch.empty((M, N), dtype=u8, device=dev) if row else None
    sk = torch.empty(blocked_shape(M, N // 32) if swz else (M // 32, N // 32), dtype=u8, device=dev) if row else None
    qm = torch.empty((N, M), dtype=u8, device=dev) if col and transposed_data else None
    sm = torch.empty(blocked_shape(N, M // 32), dtype=u8, device=dev) if col else None
    flags = L.BLOCK32 | (L.ROWWISE if row else 0) | (L.COLWISE if col else 0) | (L.SWIZZLE if swz else 0)
    with _on_device(dev):
        L.check(lib.qcc_mxfp8(_p(x), M, N, flags, _p(qk), _p(sk), _p(qm), _p(sm), _stream(x)), "mxfp8 32x32")
    L.launch_count += 1
    f8, e8 = torch.float8_e4m3fn, torch.float8_e8m0fnu
    outs = []
    if row:
        outs += [qk.view(f8), sk.view(e8)]
    if col:
        outs += ([qm.view(f8)] if transposed_data else []) + [sm.view(e8)]
    return tuple(outs)


def mxfp8_32x32_cuda(x, **kwargs):
    """gold mxfp8_32x32_f (G:753-773): (qdata (M, N), scale (M/32, N/32))."""
    return _mxfp8_32x32(x, True, False, False)


def mxfp8_32x32_swizzle_cuda(x, **kwargs):
    """gold mxfp8_32x32_swizzle_f (G:809-815): scale repeated over the 32 rows of its block, blocked (M, N/32) frame."""
    return _mxfp8_32x32(x, True, False, True)


def mxfp8_32x32_dim_m_swizzle_cuda(x, **kwargs):
    """gold mxfp8_32x32_dim_m_swizzle_f (G:856-862): (qdata (N, M), blocked scale over the (N, M/32) frame)."""
    return _mxfp8_32x32(x, False, True, True)


def mxfp8_32x32_dim_km_swizzle_cuda(x, **kwargs):
    """gold mxfp8_32x32_dim_km_swizzle_f (G:900-910): (qk, sk, qm, sm) from one read."""
    return _mxfp8_32x32(x, True, True, True)


def mxfp8_32x32_qdata_dim_k_scale_dim_km_swizzle_cuda(x, **kwargs):
    """gold mxfp8_32x32_qdata_dim_k_scale_dim_km_swizzle_f (G:946-959): (qk, sk, sm), no transposed data."""
    return _mxfp8_32x32(x, True, True, True, transposed_data=False)


def mxfp8_cuda(x, mode="rceil", **kwargs):
    """gold mxfp8_f (G:561-568): (qdata (M, N) e4m3, scale (M, N/32) e8m0)."""
    return _mxfp8(x, L.ROWWISE | _mode(mode))


def mxfp8_swizzle_cuda(x, mode="rceil", **kwargs):
    """gold mxfp8_swizzle_f (G:1051-1053): scale as the (ceil(M/128), ceil(N/128), 32, 16) blocked grid."""
    return _mxfp8(x, L.ROWWISE | L.SWIZZLE | _mode(mode))


def mxfp8_dim_m_cuda(x, mode="rceil", **kwargs):
    """gold mxfp8_dim_m_f (G:656-671): (qdata (N, M), scale (N, M/32)), 32x1 blocks, transposed."""
    return _mxfp8(x, L.COLWISE | _mode(mode))


def mxfp8_dim_m_swizzle_cuda(x, mode="rceil", **kwargs):
    """gold mxfp8_dim_m_swizzle_f (G:1092-1094)."""
    return _mxfp8(x, L.COLWISE | L.SWIZZLE | _mode(mode))


def mxfp8_dim_km_cuda(x, mode="rceil", **kwargs):
    """gold mxfp8_dim_km_f (G:701-719): (qk, sk, qm, sm) from one read of x."""
    return _mxfp8(x, L.ROWWISE | L.COLWISE | _mode(mode))


def mxfp8_dim_km_swizzle_cuda(x, mode="rceil", **kwargs):
    """gold mxfp8_dim_km_swizzle_f (G:1134-1139)."""
    return _mxfp8(x, L.ROWWISE | L.COLWISE | L.SWIZZLE | _mode(mode))


# --------------------------------------------------------------------------------------------
# nvfp4
# --------------------------------------------------------------------------------------------
def _nvfp4(x, outer_scale, flags, key=None, transposed=False):
    lib = L.load()
    _check_x(x)
    M, N = x.shape
    dev = x.device
    assert outer_scale.device == x.device and outer_scale.dtype == torch.float32, "outer_scale must be a CUDA fp32 tensor"
    per_row = int(outer_scale.ndim == 2)
    o = outer_scale.contiguous()
    if per_row:
        assert o.numel() == M and not transposed, "per-token outer scale must be (M, 1)"
    else:
        assert o.numel() == 1
    if flags & L.SR:
        assert key is not None and key.device == x.device and key.numel() >= 2 and key.element_size() == 8, (
            "stochastic rounding needs a uint64 [seed, offset] key on the device (see philox_key)")
    swz = bool(flags & L.SWIZZLE)
    with _on_device(dev):
        if transposed:
            assert M % 32 == 0 and N % 8 == 0, f"transposed nvfp4 needs M % 32 == 0 and N % 8 == 0, got {M}x{N}"
            q = torch.empty((N, M // 2), dtype=torch.uint8, device=dev)
            s = torch.empty(blocked_shape(N, M // 16) if swz else (N, M // 16), dtype=torch.uint8, device=dev)
            L.check(lib.qcc_nvfp4_transposed(_p(x), M, N, _p(o), flags | L.div_flag(), _p(key), _p(q), _p(s), _stream(x)), "nvfp4_t")
        else:
            assert N % 16 == 0, f"nvfp4 needs N % 16 == 0, got N={N}"
            q = torch.empty((M, N // 2), dtype=torch.uint8, device=dev)
            s = torch.empty(blocked_shape(M, N // 16) if swz else (M, N // 16), dtype=torch.uint8, device=dev)
            L.check(lib.qcc_nvfp4(_p(x), M, N, _p(o), per_row, flags | L.div_flag(), _p(key), _p(q), _p(s), _stream(x)), "nvfp4")
    L.launch_count += 1
    return q.view(torch.float4_e2m1fn_x2), s.view(torch.float8_e4m3fn)


def sr_bf16_global_cuda(x, key, global_row=0, global_col=0, num_col=None, **kwargs):
    """gold sr_bf16_global_f (G:1887-1914): fp32 -> bf16 with stochastic rounding, the draw keyed on each element's
    position in the parent tensor (`global_row`, `global_col`, `num_col`, as the reference's tiling framework passes
    them), so the cast of a tile equals that tile of the cast of the whole tensor.  key: `philox_key(seed)`.  The
    VALUES of the draw are this backend's Philox4x32-10 stream (the reference's comes from `torch.func._random`)."""
    lib = L.load()
    assert x.is_cuda and x.dtype == torch.float32 and x.dim() == 2 and x.is_contiguous(), "SR bf16 expects a contiguous 2-D CUDA fp32 tensor"
    assert key is not None and key.device == x.device and key.numel() >= 2 and key.element_size() == 8, "key: philox_key(...) on the device"
    M, N = x.shape
    nc = N if num_col is None else int(num_col)
    out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    with _on_device(x.device):
        L.check(lib.qcc_sr_f32_to_bf16(_p(x), M, N, _p(key), int(global_row), int(global_col), nc, _p(out), _stream(x)), "sr_f32_to_bf16")
    L.launch_count += 1
    return (out,)


def sr_bf16_cuda(x, key, **kwargs):
    """gold sr_bf16_f (G:1841-1851): the same cast keyed on the layout of the tensor it is given (tile-local)."""
    return sr_bf16_global_cuda(x, key)


def nvfp4_gs_per_token_scale_cuda(x):
    """Per-token fp32 outer scale, (M, 1): row amax / (448 * 6) without a clamp (nvfp4_gs_per_token_scale, G:1569-1573).
    `nvfp4_gs_cuda(x, scale)` / `nvfp4_gs_swizzle_cuda(x, scale)` take it as the outer scale.  (An all-zero row gets
    scale 0, which the cast divides by, as in the reference.)"""
    lib = L.load()
    assert x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.is_contiguous()
    M, N = x.shape
    s = torch.empty((M, 1), dtype=torch.float32, device=x.device)
    with _on_device(x.device):
        L.check(lib.qcc_nvfp4_per_token_scale(_p(x), M, N, L.div_flag(), _p(s), _stream(x)), "nvfp4_per_token_scale")
    L.launch_count += 1
    return s


def nvfp4_from_amax_cuda(x, amax, swizzle=True):
    """nvfp4_gs_scale + nvfp4_gs_f / nvfp4_gs_swizzle_f (G:1243-1266, G:1494-1517) for an amax that is already known:
    outer = amax / 2688 is formed in the cast's prologue.  Returns (qdata, inner scales, outer scale)."""
    lib = L.load()
    _check_x(x)
    M, N = x.shape
    assert N % 16 == 0, f"nvfp4 needs N % 16 == 0, got N={N}"
    assert amax.device == x.device and amax.dtype == torch.float32 and amax.numel() == 1
    dev = x.device
    q = torch.empty((M, N // 2), dtype=torch.uint8, device=dev)
    s_ = torch.empty(blocked_shape(M, N // 16) if swizzle else (M, N // 16), dtype=torch.uint8, device=dev)
    outer = torch.empty((), dtype=torch.float32, device=dev)
    with _on_device(dev):
        L.check(lib.qcc_nvfp4_from_amax(_p(x), M, N, _p(amax), (L.SWIZZLE if swizzle else 0) | L.div_flag(), _p(q), _p(s_), _p(outer),
                                        _stream(x)), "nvfp4_from_amax")
    L.launch_count += 1
    return q.view(torch.float4_e2m1fn_x2), s_.view(torch.float8_e4m3fn), outer


def nvfp4_blocked_outer_scale_cuda(x, blk=128):
    """gold nvfp4_blocked_outer_scale (G:1601-1606): max |x| / 2688 of every 128x128 block, (M/128, N/128) fp32."""
    lib = L.load()
    _check_x(x)
    M, N = x.shape
    assert blk == 128 and M % 128 == 0 and N % 128 == 0, f"needs 128x128 blocks tiling the input, got {M}x{N}"
    out = torch.empty((M // 128, N // 128), dtype=torch.float32, device=x.device)
    with _on_device(x.device):
        L.check(lib.qcc_amax_block128x128(_p(x), M, N, L.AMAX_NVFP4_SCALE | L.div_flag(), _p(out), _stream(x)), "amax_block128x128")
    L.launch_count += 1
    return out


def nvfp4_blocked_outer_cuda(x, outer_blocked, **kwargs):
    """gold nvfp4_blocked_outer_f (G:1609-1634): nvfp4 with one outer scale per 128x128 block, blocked inner scales."""
    lib = L.load()
    _check_x(x)
    M, N = x.shape
    assert M % 128 == 0 and N % 128 == 0, f"needs 128x128 blocks tiling the input, got {M}x{N}"
    assert outer_blocked.device == x.device and outer_blocked.dtype == torch.float32 and outer_blocked.shape == (M // 128, N // 128), (
        "outer_blocked: (M/128, N/128) fp32 on the device")
    q = torch.empty((M, N // 2), dtype=torch.uint8, device=x.device)
    s = torch.empty(blocked_shape(M, N // 16), dtype=torch.uint8, device=x.device)
    with _on_device(x.device):
        L.check(lib.qcc_nvfp4(_p(x), M, N, _p(outer_blocked.contiguous()), 2, L.SWIZZLE | L.div_flag(), None, _p(q), _p(s), _stream(x)),
                "nvfp4 blocked outer")
    L.launch_count += 1
    return q.view(torch.float4_e2m1fn_x2), s.view(torch.float8_e4m3fn)


def nvfp4_gs_cuda(x, outer_scale, **kwargs):
    """gold nvfp4_gs_f (G:1494-1517): (qdata (M, N/2) packed fp4, inner (M, N/16) e4m3); outer_scale a
    0-dim / (1,) per-tensor value or an (M, 1) per-token column."""
    return _nvfp4(x, outer_scale, 0)


def nvfp4_gs_swizzle_cuda(x, outer_scale, **kwargs):
    """gold nvfp4_gs_swizzle_f (G:1249-1266): inner scale as the blocked (.., .., 32, 16) grid."""
    return _nvfp4(x, outer_scale, L.SWIZZLE)


def nvfp4_gs_swizzle_sr_cuda(x, outer_scale, key, **kwargs):
    """gold nvfp4_gs_swizzle_sr_f (G:1409-1426) with the dither drawn from Philox4x32-10 keyed by
    `key` = uint64 [seed, offset] (extension: the gold draws from torch.func._random.uniform)."""
    return _nvfp4(x, outer_scale, L.SWIZZLE | L.SR, key=key)


def nvfp4_gs_t_cuda(x, outer_scale, **kwargs):
    """Extension: nvfp4_gs_f(x.t().contiguous(), outer_scale) without materialising the transpose."""
    return _nvfp4(x, outer_scale, 0, transposed=True)


def nvfp4_gs_swizzle_t_cuda(x, outer_scale, **kwargs):
    """Extension: nvfp4_gs_swizzle_f(x.t().contiguous(), outer_scale), the transposed operand of
    test/test_quant_cast_gold.py:104, without materialising the transpose."""
    return _nvfp4(x, outer_scale, L.SWIZZLE, transposed=True)


def nvfp4_gs_swizzle_t_sr_cuda(x, outer_scale, key, **kwargs):
    """Extension: stochastic-rounding variant of nvfp4_gs_swizzle_t_cuda (stream indexed in the
    transposed frame)."""
    return _nvfp4(x, outer_scale, L.SWIZZLE | L.SR, key=key, transposed=True)


def _nvfp4_both(x, outer_scale, flags):
    lib = L.load()
    _check_x(x)
    M, N = x.shape
    dev = x.device
    assert outer_scale.device == x.device and outer_scale.dtype == torch.float32 and outer_scale.numel() == 1
    assert M % 32 == 0 and N % 32 == 0, f"fused nvfp4 needs M % 32 == 0 and N % 32 == 0, got {M}x{N}"
    swz = bool(flags & L.SWIZZLE)
    qk = torch.empty((M, N // 2), dtype=torch.uint8, device=dev)
    sk = torch.empty(blocked_shape(M, N // 16) if swz else (M, N // 16), dtype=torch.uint8, device=dev)
    qm = torch.empty((N, M // 2), dtype=torch.uint8, device=dev)
    sm = torch.empty(blocked_shape(N, M // 16) if swz else (N, M // 16), dtype=torch.uint8, device=dev)
    with _on_device(dev):
        L.check(lib.qcc_nvfp4_both(_p(x), M, N, _p(outer_scale.contiguous()), flags | L.div_flag(), _p(qk), _p(sk), _p(qm), _p(sm),
                                   _stream(x)), "nvfp4_both")
    L.launch_count += 1
    f4, e4 = torch.float4_e2m1fn_x2, torch.float8_e4m3fn
    return qk.view(f4), sk.view(e4), qm.view(f4), sm.view(e4)


def nvfp4_gs_both_cuda(x, outer_scale, **kwargs):
    """Extension: nvfp4_gs_f(x, s) and nvfp4_gs_f(x.t().contiguous(), s) from one read of x:
    (qk (M, N/2), sk (M, N/16), qm (N, M/2), sm (N, M/16))."""
    return _nvfp4_both(x, outer_scale, 0)


def nvfp4_gs_swizzle_both_cuda(x, outer_scale, **kwargs):
    """Extension: the two casts an nvfp4 linear layer makes of one operand
    (test/test_quant_cast_gold.py:103-104: nvfp4_gs_swizzle_f of x and of x.t().contiguous()) from one read."""
    return _nvfp4_both(x, outer_scale, L.SWIZZLE)


# --------------------------------------------------------------------------------------------
# randomised Hadamard transform and the nvfp4 casts on it
# --------------------------------------------------------------------------------------------
def hadamard_rht_matrix_cuda(sign_vector, device="cuda", dtype=torch.bfloat16):
    """gold hadamard_rht_matrix (G:1778-1781): diag(sign) @ H / 4, H[i][j] = (-1)^popcount(i & j)."""
    i = torch.arange(16, device=device)
    par = i.view(-1, 1) & i.view(1, -1)
    par = (par ^ (par >> 1) ^ (par >> 2) ^ (par >> 3)) & 1
    h = (1.0 - 2.0 * par.float()) / 4.0
    return (sign_vector.to(device=device, dtype=torch.float32).view(-1, 1) * h).to(dtype)


def _check_rht(rht, x):
    assert rht.is_cuda and rht.device == x.device and rht.dtype == torch.bfloat16 and rht.shape == (16, 16), (
        "rht: a (16, 16) bf16 tensor on x's device, built with hadamard_rht_matrix")
    return rht.contiguous()


def hadamard_rht_cuda(x, rht, **kwargs):
    """gold hadamard_rht_f (G:1784-1789): the transform along the last dim, bf16 out (1-tuple).  Only matrices
    of the form diag(+-1) @ H16 / 4 are supported; the fp32 accumulation order is the butterfly's."""
    lib = L.load()
    _check_x(x)
    M, N = x.shape
    assert N % 16 == 0, f"hadamard_rht needs N % 16 == 0, got N={N}"
    rht = _check_rht(rht, x)
    y = torch.empty_like(x)
    with _on_device(x.device):
        L.check(lib.qcc_hadamard_rht(_p(x), M, N, _p(rht), _p(y), _stream(x)), "hadamard_rht")
    L.launch_count += 2
    return (y,)


def nvfp4_rht_outer_scale_m_cuda(x, rht):
    """The dim-m outer scale of G:1364-1365: max |RHT(x.t())| / 2688, from one read of x (0-dim fp32)."""
    lib = L.load()
    _check_x(x)
    M, N = x.shape
    assert M % 16 == 0 and N % 4 == 0, f"needs M % 16 == 0 and N % 4 == 0, got {M}x{N}"
    rht = _check_rht(rht, x)
    out = torch.empty((), dtype=torch.float32, device=x.device)
    with _on_device(x.device):
        L.check(lib.qcc_nvfp4_rht_amax(_p(x), M, N, _p(rht), L.AMAX_NVFP4_SCALE | L.div_flag(), _p(out), _stream(x)), "nvfp4_rht_amax")
    L.launch_count += 3
    return out


def _nvfp4_rht(x, outer_scale_k, outer_scale_m, rht, flags, key_k=None, key_m=None, both=True):
    lib = L.load()
    _check_x(x)
    M, N = x.shape
    dev = x.device
    for o in (outer_scale_k, outer_scale_m) if both else (outer_scale_m,):
        assert o.is_cuda and o.dtype == torch.float32 and o.numel() == 1, "outer scales: one fp32 value each, on the device"
    assert M % 32 == 0 and N % (32 if both else 8) == 0, f"nvfp4 with RHT needs M % 32 == 0 and N % 32 == 0, got {M}x{N}"
    rht = _check_rht(rht, x)
    if flags & L.SR:
        for k in (key_k, key_m) if both else (key_m,):
            assert k is not None and k.is_cuda and k.dtype == torch.uint64 and k.numel() == 2, "keys: philox_key(...) on the device"
    swz = bool(flags & L.SWIZZLE)
    u8 = torch.uint8
    qk = torch.empty((M, N // 2), dtype=u8, device=dev) if both else None
    sk = torch.empty(blocked_shape(M, N // 16) if swz else (M, N // 16), dtype=u8, device=dev) if both else None
    qm = torch.empty((N, M // 2), dtype=u8, device=dev)
    sm = torch.empty(blocked_shape(N, M // 16) if swz else (N, M // 16), dtype=u8, device=dev)
    with _on_device(dev):
        L.check(lib.qcc_nvfp4_rht(_p(x), M, N, _p(outer_scale_k.contiguous()) if both else None, _p(outer_scale_m.contiguous()),
                                  _p(rht), flags | L.div_flag(), _p(key_k), _p(key_m), _p(qk), _p(sk), _p(qm), _p(sm), _stream(x)), "nvfp4_rht")
    L.launch_count += 3 if (both and flags & L.SR) else 2
    f4, e4 = torch.float4_e2m1fn_x2, torch.float8_e4m3fn
    if both:
        return qk.view(f4), sk.view(e4), qm.view(f4), sm.view(e4)
    return qm.view(f4), sm.view(e4)


def nvfp4_gs_swizzle_dim_k_dim_m_rht_cuda(x, outer_scale_k, outer_scale_m, rht, **kwargs):
    """gold nvfp4_gs_swizzle_dim_k_dim_m_rht_f (G:1324-1333): (qk, sk) plain nvfp4 of x, (qm, sm) nvfp4 along M of
    RHT(x.t()), both with blocked scales, from one read of x."""
    return _nvfp4_rht(x, outer_scale_k, outer_scale_m, rht, L.SWIZZLE)


def nvfp4_gs_swizzle_dim_k_dim_m_rht_sr_cuda(x, outer_scale_k, outer_scale_m, rht, key_k, key_m, **kwargs):
    """gold nvfp4_gs_swizzle_dim_k_dim_m_rht_sr_f (G:1429-1438): the same with stochastic rounding of both fp4 casts
    (keys: philox_key(seed); the reference's torch.func._random keys are not available to this backend)."""
    return _nvfp4_rht(x, outer_scale_k, outer_scale_m, rht, L.SWIZZLE | L.SR, key_k, key_m)


def nvfp4_gs_swizzle_dim_m_rht_cuda(x, outer_scale_m, rht, **kwargs):
    """Extension: the dim-m half alone, nvfp4_gs_swizzle_f(RHT(x.t().contiguous()), outer_scale_m)."""
    return _nvfp4_rht(x, None, outer_scale_m, rht, L.SWIZZLE, both=False)


# --------------------------------------------------------------------------------------------
# recipe records
# --------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class QuantCastCudaRecipe:
    """A gold recipe plus its CUDA implementation (`cuda_fn`, same `(inputs) -> outputs` signature as
    `pt_ref_fn`).  Same fields as QuantCastSingleKernelGold (quant_cast_gold/recipes.py:63-88) plus
    `cuda_fn`, built with `from_gold` like the other backends' recipe classes.  When the reference
    package is not importable the gold fields are None and only `cuda_fn` / `example_input_fn` are set."""

    pt_ref_fn: Optional[Callable]
    correctness_fn: Optional[Callable]
    example_input_fn: Optional[Callable]
    perf_description: str
    cuda_fn: Optional[Callable] = None

    @classmethod
    def from_gold(cls, gold, cuda_fn: Callable) -> "QuantCastCudaRecipe":
        return cls(
            pt_ref_fn=gold.pt_ref_fn,
            correctness_fn=gold.correctness_fn,
            example_input_fn=gold.example_input_fn,
            perf_description=gold.perf_description,
            cuda_fn=cuda_fn,
        )


def _x(M, K):
    return torch.randn(M, K, dtype=torch.bfloat16, device="cuda")


def _inputs_x(M, K):
    return (_x(M, K),)


def _inputs_tensorwise(M, K):
    x = _x(M, K)
    return (x, float8_tensorwise_scale_cuda(x))


def _inputs_rowwise_precalc(M, K):
    x = _x(M, K)
    return (x, rowwise_precalc_scale_cuda(x))


def _inputs_colwise_precalc(M, K):
    x = _x(M, K)
    return (x, colwise_precalc_scale_cuda(x))


def _inputs_nvfp4(M, K):
    x = _x(M, K)
    return (x, nvfp4_gs_scale_cuda(x))


def _inputs_nvfp4_blocked_outer(M, K):
    x = _x(M, K)
    return (x, nvfp4_blocked_outer_scale_cuda(x))


def _rht_matrix(x):
    return hadamard_rht_matrix_cuda(torch.tensor([1, -1] * 8), x.device, x.dtype)


def _inputs_rht(M, K):
    x = _x(M, K)
    return (x, _rht_matrix(x))


def _inputs_nvfp4_rht(M, K):
    x = _x(M, K)
    rht = _rht_matrix(x)
    return (x, nvfp4_gs_scale_cuda(x), nvfp4_rht_outer_scale_m_cuda(x, rht), rht)


def _inputs_nvfp4_rht_sr(M, K):
    return _inputs_nvfp4_rht(M, K) + (philox_key(0, device="cuda"), philox_key(1, device="cuda"))


def _inputs_sr_bf16(M, K):
    # a constant strictly between two bf16 grid points, as the reference's unbiasedness check wants (G:1872-1876)
    return (torch.full((M, K), 1.0 + 0.003, dtype=torch.float32, device="cuda"), philox_key(0, device="cuda"))


# (gold recipe name, gold attribute in quant_cast_gold.recipes, cuda fn, input builder, description)
_TABLE = [
    ("fp8_tensorwise_precalc_scale", "Float8TensorwiseGold", float8_tensorwise_cuda, _inputs_tensorwise, "elementwise"),
    ("fp8_rowwise_precalc_scale", "RowwisePrecalcGold", rowwise_precalc_cuda, _inputs_rowwise_precalc, "elementwise"),
    ("fp8_colwise_precalc_scale", "ColwisePrecalcGold", colwise_precalc_cuda, _inputs_colwise_precalc, "elementwise"),
    ("mxfp8", "Mxfp8Gold", mxfp8_cuda, _inputs_x, "(1,32) block"),
    ("mxfp8_swizzle", "Mxfp8SwizzleGold", mxfp8_swizzle_cuda, _inputs_x, "(1,32) block, swizzle"),
    ("fp8_deepseek_1x128", "Deepseek1x128Gold", deepseek_1x128_cuda, _inputs_x, "(1,128) block"),
    ("mxfp8_dim_m", "Mxfp8DimMGold", mxfp8_dim_m_cuda, _inputs_x, "(32,1) block, t-contig"),
    ("mxfp8_dim_m_swizzle", "Mxfp8DimMSwizzleGold", mxfp8_dim_m_swizzle_cuda, _inputs_x, "(32,1) block, t-contig, swizzle"),
    ("fp8_deepseek_1x128_dim_m", "Deepseek1x128DimMGold", deepseek_1x128_dim_m_cuda, _inputs_x, "(128,1) block, t-contig"),
    ("mxfp8_dim_km", "Mxfp8DimKmGold", mxfp8_dim_km_cuda, _inputs_x, "(1,32) dim-k + (32,1) dim-m, one pass, t-contig"),
    ("mxfp8_dim_km_swizzle", "Mxfp8DimKmSwizzleGold", mxfp8_dim_km_swizzle_cuda, _inputs_x,
     "(1,32) dim-k + (32,1) dim-m, one pass, t-contig, swizzle"),
    ("fp8_deepseek_1x128_dim_km", "Deepseek1x128DimKmGold", deepseek_1x128_dim_km_cuda, _inputs_x,
     "(1,128) dim-k + (128,1) dim-m, one pass, t-contig"),
    ("mxfp8_32x32", "Mxfp832x32Gold", mxfp8_32x32_cuda, _inputs_x, "(32,32) block"),
    ("mxfp8_32x32_swizzle", "Mxfp832x32SwizzleGold", mxfp8_32x32_swizzle_cuda, _inputs_x, "(32,32) block, swizzle"),
    ("mxfp8_32x32_dim_m_swizzle", "Mxfp832x32DimMSwizzleGold", mxfp8_32x32_dim_m_swizzle_cuda, _inputs_x,
     "(32,32) block, t-contig, swizzle"),
    ("mxfp8_32x32_dim_km_swizzle", "Mxfp832x32DimKMSwizzleGold", mxfp8_32x32_dim_km_swizzle_cuda, _inputs_x,
     "(32,32) block, one pass, t-contig, swizzle"),
    ("mxfp8_32x32_qdata_dim_k_scale_dim_km_swizzle", "Mxfp832x32QdataDimKScaleDimKMSwizzleGold",
     mxfp8_32x32_qdata_dim_k_scale_dim_km_swizzle_cuda, _inputs_x, "(32,32) block, one pass, dim-k qdata + km scales, swizzle"),
    ("fp8_deepseek_128x128", "Deepseek128x128Gold", deepseek_128x128_cuda, _inputs_x, "(128,128) block"),
    ("fp8_rowwise", "RowwiseFp8Gold", rowwise_fp8_cuda, _inputs_x, "(1,-1) block"),
    ("fp8_colwise", "ColwiseFp8Gold", colwise_fp8_cuda, _inputs_x, "(-1,1) block, t-contig"),
    ("nvfp4", "Nvfp4GsGold", nvfp4_gs_cuda, _inputs_nvfp4, "(1,16) block, fp4 qdata, no swizzle"),
    ("nvfp4_swizzle", "Nvfp4GsSwizzleGold", nvfp4_gs_swizzle_cuda, _inputs_nvfp4, "(1,16) block, fp4 qdata, swizzle"),
    ("nvfp4_swizzle_dim_k_dim_m_rht", "Nvfp4GsSwizzle_DimK_DimMRHT_Gold", nvfp4_gs_swizzle_dim_k_dim_m_rht_cuda, _inputs_nvfp4_rht,
     "(1,16) block, fp4 qdata, swizzle; dim-k (no RHT) + dim-m (RHT), two outer scales"),
    ("nvfp4_swizzle_dim_k_sr_dim_m_rht_sr", "Nvfp4GsSwizzle_DimKSR_DimMRHTSR_Gold", nvfp4_gs_swizzle_dim_k_dim_m_rht_sr_cuda,
     _inputs_nvfp4_rht_sr, "(1,16) block, fp4 qdata (stochastic rounding), swizzle; dim-k (no RHT) + dim-m (RHT), two outer scales"),
    ("nvfp4_blocked_outer", "Nvfp4BlockedOuterGold", nvfp4_blocked_outer_cuda, _inputs_nvfp4_blocked_outer,
     "(1,16) block, fp4 qdata, swizzle, 128x128-blocked outer scale"),
    ("bf16_rht", "HadamardRht", hadamard_rht_cuda, _inputs_rht, "elementwise RHT"),
    ("fp32_to_bf16_sr", "SrF32ToBf16", sr_bf16_cuda, _inputs_sr_bf16, ""),
    ("fp32_to_bf16_sr_global_offsets", "SrF32ToBf16Global", sr_bf16_global_cuda, _inputs_sr_bf16, "elementwise SR with stateless RNG"),
]


def _build_recipes():
    try:  # the reference package, when this backend is dropped in beside it
        from quant_cast_bench.quant_cast_gold import recipes as gold
    except Exception:
        gold = None
    out = []
    for name, gold_attr, fn, inputs, desc in _TABLE:
        g = getattr(gold, gold_attr, None) if gold is not None else None
        if g is not None:
            out.append((name, QuantCastCudaRecipe.from_gold(g, fn)))
        else:
            out.append((name, QuantCastCudaRecipe(None, None, inputs, desc, fn)))
    return out


# Order follows quant_cast_gold.ALL_RECIPES (G:1929-1973), restricted to the recipes this backend implements.
ALL_RECIPES = _build_recipes()

__all__ = [n for n in dir() if n.endswith("_cuda")] + ["ALL_RECIPES", "QuantCastCudaRecipe", "blocked_shape", "philox_key",
                                                          "new_amax_workspace"]
