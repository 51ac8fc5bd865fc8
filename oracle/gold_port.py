"""Python face of the CPU oracle (oracle/qc_oracle.c): functions with the names, signatures and
output layouts of the reference's gold recipes, computed on CPU tensors by the C restatement.

THIS IS TEST INFRASTRUCTURE.  Only tests/, the smoke check and the CPU-baseline leg of the benchmark
may import it; the product package must never do so.

Reference functions mirrored (quant_cast_bench/quant_cast_gold/recipes.py = "G"):
  float8_tensorwise_scale G:1179-1183, float8_tensorwise_f G:1186-1191, rowwise_fp8_f G:301-307,
  rowwise_precalc_scale G:389-393, rowwise_precalc_f G:396-399, colwise_fp8_f G:339-349,
  colwise_precalc_scale G:438-442, colwise_precalc_f G:445-449,
  mxfp8_f G:561-568, mxfp8_swizzle_f G:1051-1053, mxfp8_dim_m_f G:656-671,
  mxfp8_dim_m_swizzle_f G:1092-1094, mxfp8_dim_km_f G:701-719, mxfp8_dim_km_swizzle_f G:1134-1139,
  nvfp4_gs_scale G:1243-1246, nvfp4_gs_f G:1494-1517, nvfp4_gs_swizzle_f G:1249-1266,
  nvfp4_gs_swizzle_sr_f G:1409-1426, _to_blocked_4d G:1000-1037.
Extensions without a reference counterpart take `fmt="e5m2"`, `mode="floor"`, or a Philox key.
"""
import ctypes

import torch

from . import build as _build

FMT = {"e4m3": 0, "e5m2": 1}
FP8_DTYPE = {"e4m3": torch.float8_e4m3fn, "e5m2": torch.float8_e5m2}
ROWWISE, COLWISE, SWIZZLE, FLOOR, SR = 1, 2, 4, 8, 16

_lib = None


def lib():
    global _lib
    if _lib is None:
        path = _build.build()
        _lib = ctypes.CDLL(path)
        _lib.qco_mxfp8.restype = ctypes.c_int
        _lib.qco_nvfp4.restype = ctypes.c_int
        _lib.qco_nvfp4_t.restype = ctypes.c_int
        _lib.qco_num_threads.restype = ctypes.c_int
        _lib.qco_hadamard_rht.restype = ctypes.c_int
        _lib.qco_mxfp8_32x32.restype = ctypes.c_int
        _lib.qco_mxfp4.restype = ctypes.c_int
        _lib.qco_fp8_blockwise.restype = ctypes.c_int
        _lib.qco_amax_block128x128.restype = ctypes.c_int
        _lib.qco_hadamard_rht_t.restype = ctypes.c_int
        _lib.qco_get_recip_div.restype = ctypes.c_int
    return _lib


def set_scalar_division(mode: str) -> str:
    """How `tensor / python_scalar` of the gold recipes is restated: "ieee" (default; eager PyTorch on the CPU) or
    "cuda_eager" (eager PyTorch on a CUDA device multiplies by the fp32 reciprocal of the scalar).  Returns the
    previous setting."""
    assert mode in ("ieee", "cuda_eager"), mode
    prev = "cuda_eager" if lib().qco_get_recip_div() else "ieee"
    lib().qco_set_recip_div(int(mode == "cuda_eager"))
    return prev


class scalar_division:
    """`with scalar_division("cuda_eager"): ...`"""

    def __init__(self, mode):
        self.mode = mode

    def __enter__(self):
        self.prev = set_scalar_division(self.mode)
        return self

    def __exit__(self, *exc):
        set_scalar_division(self.prev)
        return False


def _div_const(t, c):
    """t / c for a fp32 tensor t and a Python scalar c, under the current setting."""
    if lib().qco_get_recip_div():
        return t * (torch.tensor(1.0, dtype=torch.float32) / torch.tensor(float(c), dtype=torch.float32))
    return t / c


def num_threads() -> int:
    return lib().qco_num_threads()


def set_num_threads(n: int) -> None:
    lib().qco_set_num_threads(int(n))


def _p(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)


def _i64(v):
    return ctypes.c_int64(int(v))


def _u64(v):
    return ctypes.c_uint64(int(v) & 0xFFFFFFFFFFFFFFFF)


def _check_x(x):
    assert x.device.type == "cpu" and x.dtype == torch.bfloat16 and x.is_contiguous(), "oracle wants contiguous CPU bf16"
    return x


def _cdiv(a, b):
    return (a + b - 1) // b


def blocked_shape(rows, cols):
    return (_cdiv(rows, 128), _cdiv(cols, 4), 32, 16)


def key_words(key):
    """(seed, offset) of a Philox key given as a 2-element uint64 tensor, a (seed, offset) pair or an int."""
    if isinstance(key, torch.Tensor):
        k = key.reshape(-1).cpu().view(torch.int64).tolist()
        return k[0], (k[1] if len(k) > 1 else 0)
    if isinstance(key, (tuple, list)):
        return int(key[0]), int(key[1])
    return int(key), 0


# ------------------------------------------------------------------ scalar helpers (for KATs)
def f32_to_fp8(v, fmt="e4m3"):
    v = v.contiguous().float()
    out = torch.empty(v.shape, dtype=torch.uint8)
    lib().qco_f32_to_fp8(_p(v), _i64(v.numel()), FMT[fmt], _p(out))
    return out


def f32_to_e2m1(v):
    v = v.contiguous().float()
    out = torch.empty(v.shape, dtype=torch.uint8)
    lib().qco_f32_to_e2m1(_p(v), _i64(v.numel()), _p(out))
    return out


def e4m3_to_f32(b):
    b = b.contiguous().view(torch.uint8)
    out = torch.empty(b.shape, dtype=torch.float32)
    lib().qco_e4m3_to_f32(_p(b), _i64(b.numel()), _p(out))
    return out


def amax_to_e8m0(amax, mode="rceil"):
    a = amax.contiguous().float()
    out = torch.empty(a.shape, dtype=torch.uint8)
    lib().qco_amax_to_e8m0(_p(a), _i64(a.numel()), int(mode == "floor"), _p(out))
    return out


def e8m0_to_recip(b, mode="rceil"):
    b = b.contiguous().view(torch.uint8)
    out = torch.empty(b.shape, dtype=torch.float32)
    lib().qco_e8m0_to_recip(_p(b), _i64(b.numel()), int(mode == "floor"), _p(out))
    return out


def philox4x32_10(ctr, key):
    c = (ctypes.c_uint32 * 4)(*ctr)
    k = (ctypes.c_uint32 * 2)(*key)
    o = (ctypes.c_uint32 * 4)()
    lib().qco_philox4x32_10(c, k, o)
    return list(o)


def sr_dither22(first, n, key):
    seed, off = key_words(key)
    out = torch.empty(n, dtype=torch.int32)
    lib().qco_sr_dither22(_i64(first), _i64(n), _u64(seed), _u64(off), _p(out))
    return out


def sr_bf16_global_f(x, key, global_row=0, global_col=0, num_col=None, **kwargs):
    """fp32 -> bf16 stochastic rounding keyed on the element's position in its parent tensor (sr_bf16_global_f,
    G:1887-1914); `sr_bf16_f` (G:1841-1851) is the case of a tile that is the whole tensor.  Returns `(out,)`."""
    assert x.dtype == torch.float32 and x.dim() == 2 and x.is_contiguous()
    M, N = x.shape
    seed, off = key_words(key)
    out = torch.empty((M, N), dtype=torch.bfloat16)
    lib().qco_sr_f32_to_bf16(_p(x), _i64(M), _i64(N), _u64(seed), _u64(off), _i64(global_row), _i64(global_col),
                             _i64(N if num_col is None else num_col), _p(out))
    return (out,)


def sr_bf16_f(x, key, **kwargs):
    return sr_bf16_global_f(x, key)


def to_blocked_4d(scale):
    """G:1000-1037: (H, W) one-byte scales -> (ceil(H/128), ceil(W/4), 32, 16), padding 0."""
    H, W = scale.shape
    s = scale.contiguous().view(torch.uint8)
    out = torch.empty(blocked_shape(H, W), dtype=torch.uint8)
    lib().qco_to_blocked(_p(s), _i64(H), _i64(W), _p(out))
    return out.view(scale.dtype)


# ------------------------------------------------------------------ amax / per-tensor scales
def amax_bf16(x):
    _check_x(x)
    out = torch.empty((), dtype=torch.float32)
    lib().qco_amax_bf16(_p(x), _i64(x.numel()), _p(out))
    return out


def float8_tensorwise_scale(x, fmt="e4m3"):
    _check_x(x)
    out = torch.empty((), dtype=torch.float32)
    lib().qco_fp8_tensorwise_scale(_p(x), _i64(x.numel()), FMT[fmt], _p(out))
    return out


def fp8_scale_from_amax(amax, fmt="e4m3"):
    out = torch.empty((), dtype=torch.float32)
    lib().qco_fp8_scale_from_amax(ctypes.c_float(float(amax)), FMT[fmt], _p(out))
    return out


def nvfp4_gs_scale(x):
    _check_x(x)
    out = torch.empty((), dtype=torch.float32)
    lib().qco_nvfp4_gs_scale(_p(x), _i64(x.numel()), _p(out))
    return out


def nvfp4_gs_per_token_scale(x):
    """(M, 1) fp32: row amax / (448 * 6), no clamp.  nvfp4_gs_per_token_scale, G:1569-1573."""
    _check_x(x)
    return _div_const(x.abs().to(torch.float32).amax(dim=-1, keepdim=True), 448.0 * 6.0)


def nvfp4_scale_from_amax(amax):
    out = torch.empty((), dtype=torch.float32)
    lib().qco_nvfp4_scale_from_amax(ctypes.c_float(float(amax)), _p(out))
    return out


# ------------------------------------------------------------------ fp8
def float8_tensorwise_f(x, scale, fmt="e4m3", **kwargs):
    _check_x(x)
    s = scale.detach().reshape(-1)[:1].float().contiguous()
    q = torch.empty(x.shape, dtype=torch.uint8)
    lib().qco_fp8_tensorwise_cast(_p(x), _i64(x.numel()), _p(s), FMT[fmt], _p(q))
    return (q.view(FP8_DTYPE[fmt]),)


def rowwise_fp8_f(x, fmt="e4m3", **kwargs):
    _check_x(x)
    M, N = x.shape
    q = torch.empty((M, N), dtype=torch.uint8)
    s = torch.empty((M, 1), dtype=torch.float32)
    lib().qco_fp8_rowwise(_p(x), _i64(M), _i64(N), FMT[fmt], _p(q), _p(s))
    return q.view(FP8_DTYPE[fmt]), s


def rowwise_precalc_scale(x, fmt="e4m3"):
    _check_x(x)
    M, N = x.shape
    s = torch.empty((M, 1), dtype=torch.float32)
    lib().qco_fp8_rowwise_scale(_p(x), _i64(M), _i64(N), FMT[fmt], _p(s))
    return s


def rowwise_precalc_f(x, scale, fmt="e4m3", **kwargs):
    _check_x(x)
    M, N = x.shape
    s = scale.float().contiguous()
    assert s.numel() == M
    q = torch.empty((M, N), dtype=torch.uint8)
    lib().qco_fp8_rowwise_precalc(_p(x), _i64(M), _i64(N), _p(s), FMT[fmt], _p(q))
    return (q.view(FP8_DTYPE[fmt]),)


def colwise_fp8_f(x, fmt="e4m3", **kwargs):
    _check_x(x)
    M, N = x.shape
    q = torch.empty((N, M), dtype=torch.uint8)
    s = torch.empty((N, 1), dtype=torch.float32)
    lib().qco_fp8_colwise(_p(x), _i64(M), _i64(N), FMT[fmt], _p(q), _p(s))
    return q.view(FP8_DTYPE[fmt]), s


def colwise_precalc_scale(x, fmt="e4m3"):
    """G:438-442: (1, N) fp32 per-column scale."""
    _check_x(x)
    M, N = x.shape
    s = torch.empty((1, N), dtype=torch.float32)
    lib().qco_fp8_colwise_scale(_p(x), _i64(M), _i64(N), FMT[fmt], _p(s))
    return s


def colwise_precalc_f(x, scale, fmt="e4m3", **kwargs):
    """G:445-449: (qdata (N, M),) = fp8(x / scale) with a given (1, N) scale."""
    _check_x(x)
    M, N = x.shape
    s = scale.float().contiguous()
    assert s.numel() == N
    q = torch.empty((N, M), dtype=torch.uint8)
    lib().qco_fp8_colwise_precalc(_p(x), _i64(M), _i64(N), _p(s), FMT[fmt], _p(q))
    return (q.view(FP8_DTYPE[fmt]),)


# ------------------------------------------------------------------ mxfp8
def _mxfp8(x, flags):
    _check_x(x)
    M, N = x.shape
    swz = bool(flags & SWIZZLE)
    qk = sk = qm = sm = None
    if flags & ROWWISE:
        qk = torch.empty((M, N), dtype=torch.uint8)
        sk = torch.empty(blocked_shape(M, N // 32) if swz else (M, N // 32), dtype=torch.uint8)
    if flags & COLWISE:
        qm = torch.empty((N, M), dtype=torch.uint8)
        sm = torch.empty(blocked_shape(N, M // 32) if swz else (N, M // 32), dtype=torch.uint8)
    rc = lib().qco_mxfp8(_p(x), _i64(M), _i64(N), flags, _p(qk), _p(sk), _p(qm), _p(sm))
    assert rc == 0, "mxfp8: rowwise needs N % 32 == 0, colwise needs M % 32 == 0"
    outs = []
    if flags & ROWWISE:
        outs += [qk.view(torch.float8_e4m3fn), sk.view(torch.float8_e8m0fnu)]
    if flags & COLWISE:
        outs += [qm.view(torch.float8_e4m3fn), sm.view(torch.float8_e8m0fnu)]
    return tuple(outs)


def _mode(mode):
    return FLOOR if mode == "floor" else 0


def mxfp8_f(x, mode="rceil", **kwargs):
    return _mxfp8(x, ROWWISE | _mode(mode))


def mxfp8_swizzle_f(x, mode="rceil", **kwargs):
    return _mxfp8(x, ROWWISE | SWIZZLE | _mode(mode))


def mxfp8_dim_m_f(x, mode="rceil", **kwargs):
    return _mxfp8(x, COLWISE | _mode(mode))


def mxfp8_dim_m_swizzle_f(x, mode="rceil", **kwargs):
    return _mxfp8(x, COLWISE | SWIZZLE | _mode(mode))


def mxfp8_dim_km_f(x, mode="rceil", **kwargs):
    return _mxfp8(x, ROWWISE | COLWISE | _mode(mode))


def mxfp8_dim_km_swizzle_f(x, mode="rceil", **kwargs):
    return _mxfp8(x, ROWWISE | COLWISE | SWIZZLE | _mode(mode))


# ------------------------------------------------------------------ nvfp4
# ------------------------------------------------------------------ fp8 with 1x128 / 128x128 blocks
def _fp8_blockwise(x, bm, bn, clamp_f32=False, transposed=False):
    _check_x(x)
    M, N = x.shape
    q = torch.empty((N, M) if transposed else (M, N), dtype=torch.uint8)
    sshape = (N // bn, M // bm) if transposed else (M // bm, N // bn)
    s = torch.empty(sshape, dtype=torch.float32)
    rc = lib().qco_fp8_blockwise(_p(x), _i64(M), _i64(N), _i64(bm), _i64(bn), int(clamp_f32), int(transposed), _p(q), _p(s))
    assert rc == 0, f"blocks of {bm}x{bn} must tile the {M}x{N} input"
    return q.view(torch.float8_e4m3fn), s


def deepseek_1x128_f(x, **kwargs):
    """G:103-110"""
    return _fp8_blockwise(x, 1, 128)


def deepseek_128x128_f(x, **kwargs):
    """G:141-161"""
    return _fp8_blockwise(x, 128, 128)


def deepseek_1x128_dim_m_f(x, **kwargs):
    """G:194-214"""
    return _fp8_blockwise(x, 128, 1, transposed=True)


def deepseek_1x128_dim_km_f(x, **kwargs):
    """G:251-277 (amax clamped in fp32 there)"""
    return _fp8_blockwise(x, 1, 128, clamp_f32=True) + _fp8_blockwise(x, 128, 1, clamp_f32=True, transposed=True)


def mxfp4_f(x, swizzle=False, **kwargs):
    """gold mxfp4_f (G:607-617): (qdata (M, N/2) packed fp4, scale (M, N/32) e8m0); swizzle=True: blocked scale."""
    _check_x(x)
    M, N = x.shape
    q = torch.empty((M, N // 2), dtype=torch.uint8)
    s = torch.empty(blocked_shape(M, N // 32) if swizzle else (M, N // 32), dtype=torch.uint8)
    rc = lib().qco_mxfp4(_p(x), _i64(M), _i64(N), SWIZZLE if swizzle else 0, _p(q), _p(s))
    assert rc == 0, "mxfp4 needs N % 32 == 0"
    return q.view(torch.float4_e2m1fn_x2), s.view(torch.float8_e8m0fnu)


# ------------------------------------------------------------------ mxfp8, 32x32 blocks
def mxfp8_32x32_f(x, **kwargs):
    """gold mxfp8_32x32_f (G:753-773): (qdata (M, N) e4m3, scale (M/32, N/32) e8m0)."""
    _check_x(x)
    M, N = x.shape
    q = torch.empty((M, N), dtype=torch.uint8)
    s = torch.empty((M // 32, N // 32), dtype=torch.uint8)
    rc = lib().qco_mxfp8_32x32(_p(x), _i64(M), _i64(N), _p(q), _p(s))
    assert rc == 0, "mxfp8_32x32 needs M % 32 == 0 and N % 32 == 0"
    return q.view(torch.float8_e4m3fn), s.view(torch.float8_e8m0fnu)


def _expand_k(s):   # (M/32, N/32) -> blocked (M, N/32): every block scale repeated over its 32 rows
    return to_blocked_4d(s.view(torch.uint8).repeat_interleave(32, dim=0)).view(torch.float8_e8m0fnu)


def _expand_m(s):   # (M/32, N/32) -> blocked (N, M/32): repeated over its 32 columns, transposed
    return to_blocked_4d(s.view(torch.uint8).repeat_interleave(32, dim=1).t().contiguous()).view(torch.float8_e8m0fnu)


def mxfp8_32x32_swizzle_f(x, **kwargs):
    """G:809-815"""
    q, s = mxfp8_32x32_f(x)
    return q, _expand_k(s)


def mxfp8_32x32_dim_m_swizzle_f(x, **kwargs):
    """G:856-862"""
    q, s = mxfp8_32x32_f(x)
    return q.view(torch.uint8).t().contiguous().view(torch.float8_e4m3fn), _expand_m(s)


def mxfp8_32x32_dim_km_swizzle_f(x, **kwargs):
    """G:900-910"""
    q, s = mxfp8_32x32_f(x)
    return q, _expand_k(s), q.view(torch.uint8).t().contiguous().view(torch.float8_e4m3fn), _expand_m(s)


def mxfp8_32x32_qdata_dim_k_scale_dim_km_swizzle_f(x, **kwargs):
    """G:946-959"""
    q, s = mxfp8_32x32_f(x)
    return q, _expand_k(s), _expand_m(s)


def _nvfp4(x, outer_scale, flags, key=None, transposed=False, outer_mode=None):
    _check_x(x)
    M, N = x.shape
    o = outer_scale.detach().float().contiguous().reshape(-1)
    per_row = int(outer_scale.ndim == 2)
    if outer_mode is not None:
        per_row = outer_mode
    if per_row == 1:
        assert o.numel() == M and not transposed
    seed, off = key_words(key) if key is not None else (0, 0)
    swz = bool(flags & SWIZZLE)
    if transposed:
        q = torch.empty((N, M // 2), dtype=torch.uint8)
        s = torch.empty(blocked_shape(N, M // 16) if swz else (N, M // 16), dtype=torch.uint8)
        rc = lib().qco_nvfp4_t(_p(x), _i64(M), _i64(N), _p(o), flags, _u64(seed), _u64(off), _p(q), _p(s))
    else:
        q = torch.empty((M, N // 2), dtype=torch.uint8)
        s = torch.empty(blocked_shape(M, N // 16) if swz else (M, N // 16), dtype=torch.uint8)
        rc = lib().qco_nvfp4(_p(x), _i64(M), _i64(N), _p(o), per_row, flags, _u64(seed), _u64(off), _p(q), _p(s))
    assert rc == 0, "nvfp4: the blocked dim must be a multiple of 16"
    return q.view(torch.float4_e2m1fn_x2), s.view(torch.float8_e4m3fn)


def nvfp4_gs_f(x, outer_scale, **kwargs):
    return _nvfp4(x, outer_scale, 0)


def nvfp4_gs_swizzle_f(x, outer_scale, **kwargs):
    return _nvfp4(x, outer_scale, SWIZZLE)


def nvfp4_blocked_outer_scale(x):
    """G:1601-1606: per-128x128-block outer scale, (M/128, N/128) fp32."""
    _check_x(x)
    M, N = x.shape
    out = torch.empty((M // 128, N // 128), dtype=torch.float32)
    rc = lib().qco_amax_block128x128(_p(x), _i64(M), _i64(N), ctypes.c_float(2688.0), _p(out))
    assert rc == 0
    return out


def nvfp4_blocked_outer_f(x, outer_blocked, **kwargs):
    """G:1609-1634"""
    assert outer_blocked.shape == (x.shape[0] // 128, x.shape[1] // 128)
    return _nvfp4(x, outer_blocked, SWIZZLE, outer_mode=2)


def nvfp4_gs_swizzle_sr_f(x, outer_scale, key, **kwargs):
    return _nvfp4(x, outer_scale, SWIZZLE | SR, key=key)


def nvfp4_gs_t_f(x, outer_scale, **kwargs):
    """== nvfp4_gs_f(x.t().contiguous(), outer_scale)"""
    return _nvfp4(x, outer_scale, 0, transposed=True)


def nvfp4_gs_swizzle_t_f(x, outer_scale, **kwargs):
    """== nvfp4_gs_swizzle_f(x.t().contiguous(), outer_scale) (test/test_quant_cast_gold.py:104)"""
    return _nvfp4(x, outer_scale, SWIZZLE, transposed=True)


def nvfp4_gs_swizzle_t_sr_f(x, outer_scale, key, **kwargs):
    return _nvfp4(x, outer_scale, SWIZZLE | SR, key=key, transposed=True)


# ------------------------------------------------------------------ randomised Hadamard transform
def hadamard_rht_matrix(sign_vector, dtype=torch.bfloat16):
    """diag(sign) @ H / 4 with H[i][j] = (-1)^popcount(i & j) (G:1753-1781)."""
    i = torch.arange(16)
    par = (i.view(-1, 1) & i.view(1, -1))
    par = (par ^ (par >> 1) ^ (par >> 2) ^ (par >> 3)) & 1
    h = (1.0 - 2.0 * par.float()) / 4.0
    return (sign_vector.float().view(-1, 1) * h).to(dtype)


def rht_sign_mask(rht):
    """Bit i set where row i of `rht` carries sign -1; asserts that rht is diag(sign) @ H / 4."""
    sign = torch.where(rht[:, 0].float() < 0, -1.0, 1.0)
    assert torch.equal(hadamard_rht_matrix(sign, rht.dtype), rht.cpu()), "rht must be diag(+-1) @ H16 / 4"
    return int(sum(1 << i for i in range(16) if sign[i] < 0))


def hadamard_rht_f(x, rht, **kwargs):
    """gold hadamard_rht_f (G:1784-1789): RHT along the last dim, bf16 out (1-tuple)."""
    _check_x(x)
    y = torch.empty_like(x)
    rc = lib().qco_hadamard_rht(_p(x), _i64(x.shape[0]), _i64(x.shape[1]), ctypes.c_uint32(rht_sign_mask(rht)), _p(y))
    assert rc == 0, "hadamard_rht: last dim must be a multiple of 16"
    return (y,)


def hadamard_rht_t(x, rht):
    """RHT(x.t().contiguous()) along M: the (N, M) tensor the dim-m half of G:1324-1333 quantises."""
    _check_x(x)
    M, N = x.shape
    y = torch.empty((N, M), dtype=x.dtype)
    rc = lib().qco_hadamard_rht_t(_p(x), _i64(M), _i64(N), ctypes.c_uint32(rht_sign_mask(rht)), _p(y))
    assert rc == 0, "hadamard_rht_t: M must be a multiple of 16"
    return y


def nvfp4_rht_outer_scale_m(x, rht):
    """The dim-m outer scale of _nvfp4_gs_swizzle_dim_k_dim_m_rht_inputs (G:1364-1365)."""
    return _div_const(hadamard_rht_t(x, rht).abs().to(torch.float32).amax(), 448.0 * 6.0)


def nvfp4_gs_swizzle_dim_k_dim_m_rht_f(x, outer_scale_k, outer_scale_m, rht, **kwargs):
    """G:1324-1333: (qk, sk) plain nvfp4 of x; (qm, sm) nvfp4 of RHT(x.t()) along M."""
    return nvfp4_gs_swizzle_f(x, outer_scale_k) + nvfp4_gs_swizzle_f(hadamard_rht_t(x, rht), outer_scale_m)


def nvfp4_gs_swizzle_dim_k_dim_m_rht_sr_f(x, outer_scale_k, outer_scale_m, rht, key_k, key_m, **kwargs):
    """G:1429-1438: the same with stochastic rounding of both fp4 casts, one Philox key per direction."""
    return (nvfp4_gs_swizzle_sr_f(x, outer_scale_k, key_k)
            + nvfp4_gs_swizzle_sr_f(hadamard_rht_t(x, rht), outer_scale_m, key_m))


# ------------------------------------------------------------------ token groups (MoE activations)
def to_blocked_2d_m_groups(scales, offs):
    """Blocked layout of (M, W) scales whose rows form token groups ending at `offs`: each group is blocked on
    its own, padded to 128 rows, and the groups are stacked; result (M + G * 128, W).
    Follows experiments/quantize_tensor_api/moe_utils.py:62-81 (_to_blocked_2d_m_groups)."""
    s = scales.contiguous().view(torch.uint8)
    M, W = s.shape
    assert W % 4 == 0
    ends = [int(v) for v in offs.tolist()]
    out = torch.zeros((M + len(ends) * 128) * W, dtype=torch.uint8)
    ncb = W // 4
    start, prow = 0, 0
    cols = torch.arange(W)
    for end in ends:
        size = end - start
        if size == 0:
            continue
        r = torch.arange(size).view(-1, 1) + prow
        off = ((r // 128) * ncb + cols // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + cols % 4
        out[off.reshape(-1)] = s[start:end].reshape(-1)
        prow += _cdiv(size, 128) * 128
        start = end
    return out.view(M + len(ends) * 128, W).view(scales.dtype)


def to_blocked_2d_k_groups(scales, offs):
    """Blocked layout of (H, W) scales whose COLUMNS form groups ending at `offs` (in scale columns): each group
    (H, w_g) is blocked on its own, columns padded to 4, and stored group after group; result
    (ceil128(H), W + G * 4).  Follows moe_utils.py:93-128 (_to_blocked_2d_k_groups)."""
    s = scales.contiguous().view(torch.uint8)
    H, W = s.shape
    Hp = _cdiv(H, 128) * 128
    ends = [int(v) for v in offs.tolist()]
    out = torch.zeros(Hp * (W + len(ends) * 4), dtype=torch.uint8)
    start, pcol = 0, 0
    r = torch.arange(H).view(-1, 1)
    for end in ends:
        size = end - start
        if size == 0:
            continue
        ncb = _cdiv(size, 4)
        c = torch.arange(size)
        off = pcol * Hp + ((r // 128) * ncb + c // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + c % 4
        out[off.reshape(-1)] = s[:, start:end].reshape(-1)
        pcol += ncb * 4
        start = end
    return out.view(Hp, W + len(ends) * 4).view(scales.dtype)


def pad_token_groups(x, offs, alignment=32):
    """moe_utils.py:35-59 (_pad_token_groups): each group's rows at the start of its `alignment`-aligned slot of a zero
    matrix with ceil(total + G * alignment) rows.  Returns (padded, padded_start_offsets, padded_offsets)."""
    ends = [int(v) for v in offs.tolist()]
    M, C = x.shape
    G = len(ends)
    rows_out = _cdiv(M + G * alignment, alignment) * alignment
    out = torch.zeros((rows_out, C), dtype=x.dtype)
    starts, pends = [], []
    start = pstart = 0
    for end in ends:
        size = end - start
        psize = _cdiv(size, alignment) * alignment
        out[pstart:pstart + size] = x[start:end]
        starts.append(pstart)
        pstart += psize
        pends.append(pstart)
        start = end
    return out, torch.tensor(starts, dtype=torch.int32), torch.tensor(pends, dtype=torch.int32)


def quantize_grouped(x, offs, mode="rceil"):
    """(q (M, C), sk grouped, q_t (C, M), sm grouped): api.py:301-411 (quantize_tensor_grouped_bidirectional)."""
    qk, sk, qm, sm = _mxfp8(x, ROWWISE | COLWISE | _mode(mode))
    return qk, to_blocked_2d_m_groups(sk, offs), qm, to_blocked_2d_k_groups(sm, offs // 32)
