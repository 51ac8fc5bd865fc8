"""Parity of the CUDA casts with the CPU oracle and with golden vectors of the reference's gold
recipes, bit for bit.  Same skeleton as the reference's backend tests
(test/test_quant_cast_triton.py:59-107 of vkuzo/quant_cast_bench: same output count, shapes, dtypes,
then raw equality, at an aligned shape and at ragged shapes that force blocked-layout padding) --
but without the tolerance fallback: every non-stochastic output must match exactly, and the
stochastic one must too because checker and kernel share the Philox stream definition.
"""

import pytest
import torch

from helpers import assert_same_bits, golden_cases, golden_n_outputs, golden_out, golden_x, same_outputs
from oracle import gold_port as O
from quant_cast_bench_b200 import quant_cast_cuda as Q
from quant_cast_bench_b200.quant_cast_cuda import _lib as L
from quant_cast_bench_b200.workloads import make_input

pytestmark = pytest.mark.gpu

# aligned shape + the reference's two ragged shapes + shapes crossing tile / atom boundaries
SHAPES = [(512, 512), (96, 160), (128, 160), (32, 32), (160, 416), (384, 96), (1024, 2048), (2080, 1056)]
ONE_INPUT = ["rowwise_fp8", "mxfp8", "mxfp8_swizzle", "mxfp8_dim_m", "mxfp8_dim_m_swizzle", "mxfp8_dim_km",
             "mxfp8_dim_km_swizzle"]


def cuda_fn(name):
    return getattr(Q, name + "_cuda")


def oracle_fn(name):
    return getattr(O, name + "_f")


@pytest.fixture(autouse=True)
def _no_device_error():
    """After every test: the recipe layer's own check (what QCC_CHECK_DEVICE=1 does after every call) must find that no
    kernel gave up a bounded wait."""
    yield
    L.raise_on_device_error("after the test")


def _x(M, N, seed=0, **kw):
    return make_input(M, N, seed, **kw)


DEEPSEEK = ["deepseek_1x128", "deepseek_128x128", "deepseek_1x128_dim_m", "deepseek_1x128_dim_km"]


@pytest.mark.parametrize("tag", [t for t in golden_cases() if golden_n_outputs(t, "deepseek_1x128_f")])
@pytest.mark.parametrize("fn", DEEPSEEK)
def test_golden_deepseek(tag, fn):
    x = golden_x(tag).cuda()
    outs = cuda_fn(fn)(x)
    assert len(outs) == golden_n_outputs(tag, fn + "_f") > 0
    for i, o in enumerate(outs):
        assert_same_bits(o, golden_out(tag, fn + "_f", i), f"{fn}[{i}] {tag}")


@pytest.mark.parametrize("shape", [(128, 128), (256, 384), (1024, 2048), (2176, 1152)])
@pytest.mark.parametrize("fn", DEEPSEEK)
def test_deepseek_matches_oracle(fn, shape):
    x = _x(*shape, seed=shape[1] + 11)
    same_outputs(cuda_fn(fn)(x.cuda()), oracle_fn(fn)(x), f"{fn} {shape}")


@pytest.mark.parametrize("tag", [t for t in golden_cases() if golden_n_outputs(t, "nvfp4_blocked_outer_f")])
def test_golden_nvfp4_blocked_outer(tag):
    x = golden_x(tag).cuda()
    ob = Q.nvfp4_blocked_outer_scale_cuda(x)
    assert_same_bits(ob, golden_out(tag, "nvfp4_blocked_outer_scale", 0), "blocked outer scale")
    for i, o in enumerate(Q.nvfp4_blocked_outer_cuda(x, ob)):
        assert_same_bits(o, golden_out(tag, "nvfp4_blocked_outer_f", i), f"nvfp4_blocked_outer[{i}] {tag}")


@pytest.mark.parametrize("shape", [(128, 128), (256, 384), (1024, 2048), (2176, 1152)])
def test_nvfp4_blocked_outer_matches_oracle(shape):
    x = _x(*shape, seed=31, zero_row_p=0.0)
    ob = Q.nvfp4_blocked_outer_scale_cuda(x.cuda())
    assert_same_bits(ob, O.nvfp4_blocked_outer_scale(x), "blocked outer scale")
    same_outputs(Q.nvfp4_blocked_outer_cuda(x.cuda(), ob), O.nvfp4_blocked_outer_f(x, ob.cpu()), f"blocked outer {shape}")


@pytest.mark.parametrize("tag", golden_cases())
def test_golden_mxfp4(tag):
    x = golden_x(tag).cuda()
    for i, o in enumerate(Q.mxfp4_cuda(x)):
        assert_same_bits(o, golden_out(tag, "mxfp4_f", i), f"mxfp4[{i}] {tag}")


@pytest.mark.parametrize("shape", SHAPES)
def test_mxfp4_matches_oracle(shape):
    x = _x(*shape, seed=17)
    for swz in (False, True):
        same_outputs(Q.mxfp4_cuda(x.cuda(), swizzle=swz), O.mxfp4_f(x, swizzle=swz), f"mxfp4 {shape} swizzle={swz}")


def test_deepseek_ragged_and_zero_blocks():
    """1x128 takes any row count, 128x1 any multiple of 8 columns; an all-zero input takes the clamp of each recipe."""
    x = _x(96, 256, seed=2)
    same_outputs(Q.deepseek_1x128_cuda(x.cuda()), O.deepseek_1x128_f(x), "1x128 at 96 rows")
    x = _x(256, 200, seed=3)
    same_outputs(Q.deepseek_1x128_dim_m_cuda(x.cuda()), O.deepseek_1x128_dim_m_f(x), "128x1 at 200 columns")
    z = torch.zeros(256, 256, dtype=torch.bfloat16)
    for fn in DEEPSEEK:
        same_outputs(cuda_fn(fn)(z.cuda()), oracle_fn(fn)(z), f"{fn} zeros")
    with pytest.raises(AssertionError):
        Q.deepseek_1x128_cuda(_x(128, 160).cuda())
    with pytest.raises(AssertionError):
        Q.deepseek_128x128_cuda(_x(96, 256).cuda())


B32 = ["mxfp8_32x32", "mxfp8_32x32_swizzle", "mxfp8_32x32_dim_m_swizzle", "mxfp8_32x32_dim_km_swizzle",
       "mxfp8_32x32_qdata_dim_k_scale_dim_km_swizzle"]


@pytest.mark.parametrize("tag", golden_cases())
@pytest.mark.parametrize("fn", B32)
def test_golden_32x32(tag, fn):
    x = golden_x(tag).cuda()
    outs = cuda_fn(fn)(x)
    assert len(outs) == golden_n_outputs(tag, fn + "_f") > 0
    for i, o in enumerate(outs):
        assert_same_bits(o, golden_out(tag, fn + "_f", i), f"{fn}[{i}] {tag}")


@pytest.mark.parametrize("shape", [(512, 512), (96, 160), (128, 160), (32, 32), (160, 416), (384, 96), (1024, 2048), (2080, 1056)])
@pytest.mark.parametrize("fn", B32)
def test_32x32_matches_oracle(fn, shape):
    x = _x(*shape, seed=shape[0] + 7)
    same_outputs(cuda_fn(fn)(x.cuda()), oracle_fn(fn)(x), f"{fn} {shape}")


def test_32x32_outputs_fully_written():
    """Blocked scale padding is zero whatever the buffers held before (ragged shape: 160 rows, 13 column blocks)."""
    x = _x(160, 416, seed=3)
    xc = x.cuda()
    for fill in (0x00, 0xFF):
        junk = [torch.full((1 << 22,), fill, dtype=torch.uint8, device="cuda") for _ in range(4)]
        del junk
        same_outputs(Q.mxfp8_32x32_dim_km_swizzle_cuda(xc), O.mxfp8_32x32_dim_km_swizzle_f(x), f"fill {fill}")
        same_outputs(Q.mxfp8_32x32_qdata_dim_k_scale_dim_km_swizzle_cuda(xc), O.mxfp8_32x32_qdata_dim_k_scale_dim_km_swizzle_f(x), f"fill {fill}")


# ---------------------------------------------------------------------------- golden vectors
@pytest.mark.parametrize("tag", golden_cases())
@pytest.mark.parametrize("fn", ONE_INPUT)
def test_golden_single_input(tag, fn):
    x = golden_x(tag).cuda()
    outs = cuda_fn(fn)(x)
    gname = fn + "_f"
    assert len(outs) == golden_n_outputs(tag, gname)
    for i, o in enumerate(outs):
        assert_same_bits(o, golden_out(tag, gname, i), f"{fn}[{i}] {tag}")


@pytest.mark.parametrize("tag", golden_cases())
def test_golden_fp8_tensorwise_and_precalc(tag):
    x = golden_x(tag).cuda()
    s = Q.float8_tensorwise_scale_cuda(x)
    assert s.shape == () and s.dtype == torch.float32
    assert_same_bits(s.reshape(1), golden_out(tag, "float8_tensorwise_scale", 0), "scale")
    (q,) = Q.float8_tensorwise_cuda(x, s)
    assert q.dtype == torch.float8_e4m3fn
    assert_same_bits(q, golden_out(tag, "float8_tensorwise_f", 0), "q")
    ps = Q.rowwise_precalc_scale_cuda(x)
    assert_same_bits(ps, golden_out(tag, "rowwise_precalc_scale", 0), "row scale")
    assert_same_bits(Q.rowwise_precalc_cuda(x, ps)[0], golden_out(tag, "rowwise_precalc_f", 0), "precalc q")


@pytest.mark.parametrize("tag", golden_cases())
def test_golden_nvfp4(tag):
    x = golden_x(tag).cuda()
    gs = Q.nvfp4_gs_scale_cuda(x)
    assert_same_bits(gs.reshape(1), golden_out(tag, "nvfp4_gs_scale", 0), "outer")
    for fn in ("nvfp4_gs", "nvfp4_gs_swizzle", "nvfp4_gs_swizzle_t", "nvfp4_gs_t"):
        outs = cuda_fn(fn)(x, gs)
        assert outs[0].dtype == torch.float4_e2m1fn_x2 and outs[1].dtype == torch.float8_e4m3fn
        for i, o in enumerate(outs):
            assert_same_bits(o, golden_out(tag, fn + "_f", i), f"{fn}[{i}] {tag}")
    pt = golden_out(tag, "nvfp4_per_token_scale", 0).view(torch.float32).cuda()
    mine = Q.nvfp4_gs_per_token_scale_cuda(x)
    assert mine.shape == (x.shape[0], 1) and mine.dtype == torch.float32
    assert_same_bits(mine.clamp(min=2.0 ** -100), pt, "per-token outer scale")      # (the stored one is clamped)
    for i, o in enumerate(Q.nvfp4_gs_cuda(x, pt)):
        assert_same_bits(o, golden_out(tag, "nvfp4_gs_f_per_token", i), f"per-token[{i}] {tag}")


# ---------------------------------------------------------------------------- oracle, many shapes
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: f"{s[0]}x{s[1]}")
@pytest.mark.parametrize("fn", ONE_INPUT)
def test_matches_oracle(fn, shape):
    x = _x(*shape, seed=shape[0] + shape[1])
    kw = {"global_row": 0, "global_col": 0, "num_col": shape[1]}  # tile kwargs are accepted and ignored
    same_outputs(cuda_fn(fn)(x.cuda(), **kw), oracle_fn(fn)(x), f"{fn} {shape}")


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: f"{s[0]}x{s[1]}")
@pytest.mark.parametrize("fn", [f for f in ONE_INPUT if f.startswith("mxfp8")])
def test_mxfp8_floor_mode(fn, shape):
    x = _x(*shape, seed=7)
    same_outputs(cuda_fn(fn)(x.cuda(), mode="floor"), oracle_fn(fn)(x, mode="floor"), f"{fn} floor {shape}")


@pytest.mark.parametrize("fmt", ["e4m3", "e5m2"])
@pytest.mark.parametrize("shape", SHAPES + [(17, 100), (3, 7), (5, 20000), (64, 16384)], ids=lambda s: f"{s[0]}x{s[1]}")
def test_fp8_family(fmt, shape):
    x = _x(*shape, seed=11, spread=8.0)
    xc = x.cuda()
    s = Q.float8_tensorwise_scale_cuda(xc, fmt)
    so = O.float8_tensorwise_scale(x, fmt)
    assert_same_bits(s, so, "tensorwise scale")
    same_outputs(Q.float8_tensorwise_cuda(xc, s, fmt), O.float8_tensorwise_f(x, so, fmt), f"tensorwise {fmt}")
    same_outputs(Q.rowwise_fp8_cuda(xc, fmt), O.rowwise_fp8_f(x, fmt), f"rowwise {fmt}")
    ps = Q.rowwise_precalc_scale_cuda(xc, fmt)
    assert_same_bits(ps, O.rowwise_precalc_scale(x, fmt), "row scale")
    same_outputs(Q.rowwise_precalc_cuda(xc, ps, fmt), O.rowwise_precalc_f(x, ps.cpu(), fmt), f"precalc {fmt}")


@pytest.mark.parametrize("fmt", ["e4m3", "e5m2"])
@pytest.mark.parametrize("shape", [(512, 512), (96, 160), (128, 160), (16, 8), (2080, 1056), (4096, 264)], ids=lambda s: f"{s[0]}x{s[1]}")
def test_fp8_colwise(fmt, shape):
    x = _x(*shape, seed=13, spread=8.0)
    xc = x.cuda()
    same_outputs(Q.colwise_fp8_cuda(xc, fmt), O.colwise_fp8_f(x, fmt), f"colwise {fmt} {shape}")
    cs = Q.colwise_precalc_scale_cuda(xc, fmt)
    assert_same_bits(cs, O.colwise_precalc_scale(x, fmt), "column scale")
    same_outputs(Q.colwise_precalc_cuda(xc, cs, fmt), O.colwise_precalc_f(x, cs.cpu(), fmt), f"colwise precalc {fmt} {shape}")


@pytest.mark.parametrize("tag", golden_cases())
def test_golden_fp8_colwise(tag):
    x = golden_x(tag).cuda()
    q, s = Q.colwise_fp8_cuda(x)
    assert_same_bits(q, golden_out(tag, "colwise_fp8_f", 0), "colwise q")
    assert_same_bits(s, golden_out(tag, "colwise_fp8_f", 1), "colwise scale")
    cs = golden_out(tag, "colwise_precalc_scale", 0).view(torch.float32).cuda()
    assert_same_bits(Q.colwise_precalc_cuda(x, cs)[0], golden_out(tag, "colwise_precalc_f", 0), "colwise precalc q")


def test_fp8_all_zero_and_tiny():
    x = torch.zeros(64, 256, dtype=torch.bfloat16)
    x[3, 5] = 1e-30
    xc = x.cuda()
    s = Q.float8_tensorwise_scale_cuda(xc)
    assert_same_bits(s, O.float8_tensorwise_scale(x), "scale of ~zero tensor (bf16 clamp at 1e-12)")
    same_outputs(Q.rowwise_fp8_cuda(xc), O.rowwise_fp8_f(x), "rowwise zero rows")
    for fn in ONE_INPUT[1:]:
        same_outputs(cuda_fn(fn)(xc), oracle_fn(fn)(x), f"{fn} zeros")


@pytest.mark.parametrize("shape", [(512, 512), (128, 192), (96, 160), (128, 160), (160, 416), (1024, 2048), (2080, 1056)],
                         ids=lambda s: f"{s[0]}x{s[1]}")
def test_nvfp4_matches_oracle(shape):
    x = _x(*shape, seed=5)
    xc = x.cuda()
    gs = Q.nvfp4_gs_scale_cuda(xc)
    gso = O.nvfp4_gs_scale(x)
    assert_same_bits(gs, gso, "outer scale")
    for fn in ("nvfp4_gs", "nvfp4_gs_swizzle", "nvfp4_gs_t", "nvfp4_gs_swizzle_t"):
        same_outputs(cuda_fn(fn)(xc, gs), oracle_fn(fn)(x, gso), f"{fn} {shape}")
    if shape[0] % 32 == 0 and shape[1] % 32 == 0:   # both orientations from one read
        same_outputs(Q.nvfp4_gs_swizzle_both_cuda(xc, gs), O.nvfp4_gs_swizzle_f(x, gso) + O.nvfp4_gs_swizzle_t_f(x, gso),
                     f"fused swizzle {shape}")
        same_outputs(Q.nvfp4_gs_both_cuda(xc, gs), O.nvfp4_gs_f(x, gso) + O.nvfp4_gs_t_f(x, gso), f"fused plain {shape}")
    # per-token outer scale (M, 1)
    amax_rows = x.float().abs().amax(dim=1, keepdim=True).clamp(min=2.0 ** -100)
    pt = amax_rows / 2688.0
    same_outputs(Q.nvfp4_gs_cuda(xc, pt.cuda()), O.nvfp4_gs_f(x, pt), f"per-token {shape}")


def test_all_bf16_values_through_every_conversion():
    """Every finite bf16 bit pattern goes through the fp8, e8m0 and fp4 paths (ties, subnormals,
    signed zeros, saturation), with several scales."""
    bits = torch.arange(0, 1 << 16, dtype=torch.int32)
    finite = (bits & 0x7F80) != 0x7F80
    v = bits[finite].to(torch.int16).view(torch.bfloat16)           # 65024 values
    n = 128 * 512                                                    # pad with zeros to 128 rows
    v = torch.cat([v, torch.zeros(n - v.numel(), dtype=torch.bfloat16)])
    x = v.reshape(128, 512).contiguous()
    g = torch.Generator().manual_seed(3)
    xs = x.flatten()[torch.randperm(n, generator=g)].reshape(-1, 512).contiguous()  # mixed magnitudes per block
    for t in (x, xs):
        tc = t.cuda()
        for fmt in ("e4m3", "e5m2"):
            for scale in (1.0, 0.37, 3.1e-5, 2.0 ** 40, 1.7e30):
                s = torch.tensor(scale, dtype=torch.float32)
                # the checker saturates like the kernel, so overflowing products are compared too
                same_outputs(Q.float8_tensorwise_cuda(tc, s.cuda(), fmt), O.float8_tensorwise_f(t, s, fmt), f"{fmt} {scale}")
        for fn in ONE_INPUT:
            same_outputs(cuda_fn(fn)(tc), oracle_fn(fn)(t), fn)
            if fn.startswith("mxfp8"):
                same_outputs(cuda_fn(fn)(tc, mode="floor"), oracle_fn(fn)(t, mode="floor"), fn + " floor")
        for outer in (1.0, 2.0 ** -20, 3.3e3, 7.7e-12, 1.1e25):
            o = torch.tensor(outer, dtype=torch.float32)
            for fn in ("nvfp4_gs", "nvfp4_gs_swizzle", "nvfp4_gs_t", "nvfp4_gs_swizzle_t"):
                same_outputs(cuda_fn(fn)(tc, o.cuda()), oracle_fn(fn)(t, o), f"{fn} outer={outer}")
            same_outputs(Q.nvfp4_gs_swizzle_both_cuda(tc, o.cuda()), O.nvfp4_gs_swizzle_f(t, o) + O.nvfp4_gs_swizzle_t_f(t, o),
                         f"fused outer={outer}")


def test_fp4_ties_round_to_even():
    """Scaled values exactly on e2m1 midpoints: outer = 1/6 and a block amax of 6 make recip == 1."""
    vals = [0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -0.25, -0.75, -2.5, -5.0, 6.0, 0.0, -0.0, 0.5, 1.0]
    x = torch.tensor(vals, dtype=torch.bfloat16).repeat(32, 4).contiguous()   # (32, 64)
    outer = torch.tensor(1.0 / 6.0, dtype=torch.float32)
    q, s = Q.nvfp4_gs_cuda(x.cuda(), outer.cuda())
    qo, so = O.nvfp4_gs_f(x, outer)
    assert_same_bits(q, qo, "fp4 ties")
    assert_same_bits(s, so, "inner")
    nib = q.view(torch.uint8).cpu()[0, :8]
    lo = (nib & 15).tolist()
    hi = (nib >> 4).tolist()
    got = [c for pair in zip(lo, hi) for c in pair]
    # 0.25->0, 0.75->1.0, 1.25->1.0, 1.75->2, 2.5->2, 3.5->4, 5->4, negatives mirror, -0.25 -> -0
    assert got == [0, 2, 2, 4, 4, 6, 6, 8, 10, 12, 14, 7, 0, 8, 1, 2]


# ---------------------------------------------------------------------------- stochastic rounding
@pytest.mark.parametrize("shape", [(128, 256), (96, 160), (1024, 2048)], ids=lambda s: f"{s[0]}x{s[1]}")
def test_sr_bit_exact_against_oracle_stream(shape):
    x = _x(*shape, seed=9, spread=0.0, outlier_p=1e-3, outlier_mul=50.0, zero_row_p=0.0)
    xc = x.cuda()
    gs = Q.nvfp4_gs_scale_cuda(xc)
    for seed, off in ((0, 0), (12345, 0), (2 ** 40 + 17, 2 ** 33 + 5)):
        key = Q.philox_key(seed, off)
        same_outputs(Q.nvfp4_gs_swizzle_sr_cuda(xc, gs, key), O.nvfp4_gs_swizzle_sr_f(x, gs.cpu(), (seed, off)), f"sr {seed}")
        if shape[0] % 32 == 0:
            same_outputs(Q.nvfp4_gs_swizzle_t_sr_cuda(xc, gs, key), O.nvfp4_gs_swizzle_t_sr_f(x, gs.cpu(), (seed, off)),
                         f"sr transposed {seed}")
    # scales and layout do not depend on the rounding mode
    q_sr, s_sr = Q.nvfp4_gs_swizzle_sr_cuda(xc, gs, Q.philox_key(1))
    q_rn, s_rn = Q.nvfp4_gs_swizzle_cuda(xc, gs)
    assert_same_bits(s_sr, s_rn, "sr scales == rne scales")
    assert q_sr.shape == q_rn.shape and q_sr.dtype == q_rn.dtype


def _fp4_decode(q):
    lut = torch.tensor([0, 0.5, 1, 1.5, 2, 3, 4, 6, -0.0, -0.5, -1, -1.5, -2, -3, -4, -6], device=q.device)
    b = q.view(torch.uint8).long()
    return torch.stack([lut[b & 15], lut[b >> 4]], dim=-1).flatten(-2)


def test_sr_unbiased_over_seeds():
    """Mean of the dequantised values over 16 seeds approaches x (relative error of the mean <= 1e-3),
    every draw lands on one of the two fp4 neighbours, and the draw frequency matches the distance
    (the property test of the reference: quant_cast_gold/recipes.py:1854-1869 and
    experiments/stochastic_rounding_api/test_vs_gold.py:116-176)."""
    M, N = 1024, 2048
    x = _x(M, N, seed=21, spread=0.0, outlier_p=1e-3, outlier_mul=50.0, zero_row_p=0.0).cuda()
    gs = Q.nvfp4_gs_scale_cuda(x)
    q_rn, s = Q.nvfp4_gs_swizzle_cuda(x, gs)
    qp, sp = Q.nvfp4_gs_cuda(x, gs)   # plain-layout scales to dequantise with
    inner = sp.float().repeat_interleave(16, dim=1)
    recip_scale = inner * gs
    acc = torch.zeros(M, N, device="cuda", dtype=torch.float64)
    n_seeds = 16
    for seed in range(n_seeds):
        q, s_sr = Q.nvfp4_gs_swizzle_sr_cuda(x, gs, Q.philox_key(seed))
        assert_same_bits(s_sr, s, "scales")
        acc += (_fp4_decode(q) * recip_scale).double()
    mean = acc / n_seeds
    xf = x.double()
    # aggregate relative error of the mean
    rel = (mean - xf).abs().sum() / xf.abs().sum()
    rne = ((_fp4_decode(q_rn) * recip_scale).double() - xf).abs().sum() / xf.abs().sum()
    assert rel < rne, f"SR mean error {rel:.4g} should beat RNE error {rne:.4g}"
    signed = ((mean - xf).sum() / xf.abs().sum()).abs()
    assert signed <= 1e-3, f"relative bias of the SR mean {signed:.3g} > 1e-3"
    # P(round up) on a constant probe: value 1.25 between fp4 neighbours 1.0 and 1.5 -> 50 %; 1.125 -> 25 %.
    # Below 1.0 the recipe double-rounds (dither on the fp32 mantissa, then RNE onto the 0.5 grid;
    # quant_cast_gold/recipes.py:1398-1400): 0.625 dithers to 0.5 or 0.75 with equal chance and 0.75
    # ties to 1.0, so P(1.0) is 50 %, not 25 %.
    for v, p_up, lo, hi in ((1.25, 0.5, 1.0, 1.5), (1.125, 0.25, 1.0, 1.5), (2.25, 0.25, 2.0, 3.0), (0.625, 0.5, 0.5, 1.0)):
        probe = torch.full((256, 1024), v, dtype=torch.bfloat16, device="cuda")
        probe[:, ::16] = 6.0   # block amax 6 with outer 1/6 -> recip == 1
        outer = torch.tensor(1.0 / 6.0, device="cuda")
        q, _ = Q.nvfp4_gs_swizzle_sr_cuda(probe, outer, Q.philox_key(99))
        d = _fp4_decode(q)
        body = d[:, torch.arange(1024, device="cuda") % 16 != 0]
        assert set(body.unique().tolist()) <= {lo, hi}
        frac = (body == hi).double().mean().item()
        assert abs(frac - p_up) < 0.01, f"P(up) for {v}: {frac:.4f} vs {p_up}"


# ---------------------------------------------------------------------------- unwritten bytes / padding
@pytest.mark.parametrize("fill", [0x00, 0xFF])
def test_outputs_fully_written_with_guard_bytes(fill):
    """Call the C ABI on pre-filled buffers (ragged shape -> blocked-layout padding): every output byte
    must equal the oracle's whatever the buffer held before, and the guard bytes after each buffer
    stay untouched."""
    lib = L.load()
    M, N = 160, 416
    x = _x(M, N, seed=2)
    xc = x.cuda()
    stream = torch.cuda.current_stream().cuda_stream
    GUARD = 256

    def buf(nbytes):
        t = torch.full((nbytes + GUARD,), fill, dtype=torch.uint8, device="cuda")
        t[nbytes:] = 0xA5
        return t

    def check(t, want, what):
        n = want.numel() * want.element_size()
        assert_same_bits(t[:n].cpu(), want.contiguous().view(torch.uint8).flatten(), what)
        assert bool((t[n:] == 0xA5).all()), f"{what}: guard bytes overwritten"

    for flags, ofn in ((L.ROWWISE | L.COLWISE | L.SWIZZLE, O.mxfp8_dim_km_swizzle_f), (L.ROWWISE | L.COLWISE, O.mxfp8_dim_km_f)):
        want = ofn(x)
        bufs = [buf(w.numel()) for w in want]
        rc = lib.qcc_mxfp8(xc.data_ptr(), M, N, flags, *[b.data_ptr() for b in bufs], stream)
        assert rc == 0
        for b, w, n in zip(bufs, want, ("qk", "sk", "qm", "sm")):
            check(b, w, f"mxfp8 flags={flags} {n}")
    gs = O.nvfp4_gs_scale(x)
    gsc = gs.cuda()
    for tr, flags, ofn in ((False, L.SWIZZLE, O.nvfp4_gs_swizzle_f), (True, L.SWIZZLE, O.nvfp4_gs_swizzle_t_f),
                           (False, 0, O.nvfp4_gs_f), (True, 0, O.nvfp4_gs_t_f)):
        want = ofn(x, gs)
        bufs = [buf(w.numel()) for w in want]
        if tr:
            rc = lib.qcc_nvfp4_transposed(xc.data_ptr(), M, N, gsc.data_ptr(), flags, None, bufs[0].data_ptr(), bufs[1].data_ptr(), stream)
        else:
            rc = lib.qcc_nvfp4(xc.data_ptr(), M, N, gsc.data_ptr(), 0, flags, None, bufs[0].data_ptr(), bufs[1].data_ptr(), stream)
        assert rc == 0
        for b, w, n in zip(bufs, want, ("q", "s")):
            check(b, w, f"nvfp4 transposed={tr} flags={flags} {n}")


# ---------------------------------------------------------------------------- errors
def test_rejected_arguments():
    x = torch.randn(64, 48, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(AssertionError):
        Q.mxfp8_cuda(x)                       # N % 32 != 0
    with pytest.raises(AssertionError):
        Q.mxfp8_dim_m_cuda(torch.randn(48, 64, dtype=torch.bfloat16, device="cuda"))  # M % 32 != 0
    with pytest.raises(AssertionError):
        Q.mxfp8_cuda(x.t())                   # not contiguous
    with pytest.raises(ValueError):
        Q.mxfp8_cuda(x.cpu())                 # no CPU path
    with pytest.raises(ValueError):
        Q.float8_tensorwise_cuda(x, torch.ones((), device="cuda"), fmt="e3m4")
    lib = L.load()
    assert lib.qcc_mxfp8(x.data_ptr(), 64, 48, L.ROWWISE, x.data_ptr(), x.data_ptr(), None, None, None) == -1
    assert lib.qcc_mxfp8(x.data_ptr() + 2, 64, 64, L.ROWWISE, x.data_ptr(), x.data_ptr(), None, None, None) == -2
    assert lib.qcc_mxfp8(None, 64, 64, L.ROWWISE, x.data_ptr(), x.data_ptr(), None, None, None) == -3
    assert lib.qcc_amax_bf16(x.data_ptr(), 10, 0, 0, x.data_ptr(), x.data_ptr(), 16, None) == -4
    # empty input is a no-op
    e = torch.empty(0, 64, dtype=torch.bfloat16, device="cuda")
    q, s = Q.mxfp8_cuda(e)
    assert q.shape == (0, 64) and s.shape == (0, 2)


def test_rejected_arguments_of_the_block_and_transform_entries():
    """Every entry point returns its error code before anything is launched: -1 shape, -2 alignment, -3 argument,
    -4 workspace."""
    lib = L.load()
    x = torch.randn(256, 256, dtype=torch.bfloat16, device="cuda")
    p = x.data_ptr()
    B32 = L.BLOCK32
    assert lib.qcc_mxfp8(p, 48, 64, L.ROWWISE | B32, p, p, None, None, None) == -1               # M % 32 with 32x32 blocks
    assert lib.qcc_mxfp8(p, 64, 64, L.ROWWISE | B32 | L.FLOOR, p, p, None, None, None) == -3     # FLOOR with 32x32 blocks
    assert lib.qcc_mxfp8(p, 64, 64, L.COLWISE | B32, None, None, p, p, None) == -3               # transposed 32x32 needs SWIZZLE
    assert lib.qcc_mxfp8(p, 64, 64, L.ROWWISE | L.COLWISE | L.SWIZZLE, p, p, None, p, None) == -3  # qm may be NULL with BLOCK32 only
    assert lib.qcc_mxfp4(p, 64, 48, 0, p, p, None) == -1
    assert lib.qcc_mxfp4(p, 64, 64, L.ROWWISE, p, p, None) == -3                                  # only QCC_SWIZZLE is a valid flag
    assert lib.qcc_fp8_block128(p, 128, 160, L.ROWWISE, p, p, None, None, None) == -1             # N % 128
    assert lib.qcc_fp8_block128(p, 96, 128, L.COLWISE, None, None, p, p, None) == -1              # M % 128
    assert lib.qcc_fp8_block128(p, 128, 128, 0, p, p, p, p, None) == -3
    assert lib.qcc_fp8_block128(p, 128, 128, L.ROWWISE, p + 4, p, None, None, None) == -2
    assert lib.qcc_fp8_block128x128(p, 128, 192, 0, p, p, None) == -1
    assert lib.qcc_fp8_block128x128(p, 128, 128, L.SWIZZLE, p, p, None) == -3                      # only QCC_RECIP_DIV is a valid flag
    assert lib.qcc_amax_block128x128(p, 128, 128, 1, p, None) == -3                                # FP8_SCALE is not a mode here
    assert lib.qcc_nvfp4(p, 128, 128, p, 3, 0, None, p, p, None) == -3                             # outer mode 0..2
    assert lib.qcc_nvfp4(p, 96, 128, p, 2, L.SWIZZLE, None, p, p, None) == -1                      # blocked outer needs M % 128
    assert lib.qcc_nvfp4(p, 128, 128, p, 2, L.SWIZZLE | L.SR, p, p, p, None) == -3                 # no SR with a blocked outer
    assert lib.qcc_hadamard_rht(p, 64, 40, p, p, None) == -1
    assert lib.qcc_hadamard_rht(p, 64, 64, None, p, None) == -3
    assert lib.qcc_nvfp4_rht_amax(p, 40, 64, p, 0, p, None) == -1
    assert lib.qcc_nvfp4_rht_amax(p, 64, 64, p, 1, p, None) == -3
    assert lib.qcc_nvfp4_rht(p, 48, 64, p, p, p, L.SWIZZLE, None, None, p, p, p, p, None) == -1
    assert lib.qcc_nvfp4_rht(p, 64, 64, p, p, None, L.SWIZZLE, None, None, p, p, p, p, None) == -3
    assert lib.qcc_nvfp4_rht(p, 64, 64, p, p, p, L.SWIZZLE | L.SR, None, None, p, p, p, p, None) == -3   # SR without keys
    offs = torch.tensor([64], dtype=torch.int32, device="cuda")
    need = lib.qcc_mxfp8_grouped_workspace_bytes(64)
    assert lib.qcc_mxfp8_grouped(p, 64, 128, L.ROWWISE | L.SWIZZLE, offs.data_ptr(), 1, p, p, None, None, p, need - 1, None) == -4
    assert lib.qcc_mxfp8_grouped(p, 64, 128, L.ROWWISE, offs.data_ptr(), 1, p, p, None, None, p, need, None) == -3   # needs SWIZZLE
    assert lib.qcc_mxfp8_grouped(p, 64, 96, L.ROWWISE | L.SWIZZLE, offs.data_ptr(), 1, p, p, None, None, p, need, None) == -1
    assert lib.qcc_mxfp8_grouped(p, 64, 128, L.ROWWISE | L.SWIZZLE, offs.data_ptr(), 5000, p, p, None, None, p, need, None) == -1
    torch.cuda.synchronize()
    assert L.device_error() == 0


@pytest.mark.parametrize("swizzle", [True, False])
def test_host_buffer_caster_matches_oracle(swizzle):
    """The chunked, pipelined host-buffer call returns the bytes of the one-shot cast."""
    from quant_cast_bench_b200.quant_cast_cuda.host_api import HostMxfp8Caster
    M, N = 1024, 384
    x = _x(M, N, seed=17)
    xp = x.pin_memory()
    caster = HostMxfp8Caster(M, N, "cuda", swizzle=swizzle, chunk_rows=256)
    want = O.mxfp8_dim_km_swizzle_f(x) if swizzle else O.mxfp8_dim_km_f(x)
    for _ in range(2):   # buffers are reused by the second call
        got = caster.cast(xp)
        same_outputs(got, want, f"host caster swizzle={swizzle}")


def test_recipe_index_mirrors_reference_backends():
    names = [n for n, _ in Q.ALL_RECIPES]
    assert names == ["fp8_tensorwise_precalc_scale", "fp8_rowwise_precalc_scale", "fp8_colwise_precalc_scale", "mxfp8", "mxfp8_swizzle", "fp8_deepseek_1x128", "mxfp8_dim_m",
                     "mxfp8_dim_m_swizzle", "fp8_deepseek_1x128_dim_m", "mxfp8_dim_km", "mxfp8_dim_km_swizzle", "fp8_deepseek_1x128_dim_km",
                     "mxfp8_32x32", "mxfp8_32x32_swizzle",
                     "mxfp8_32x32_dim_m_swizzle", "mxfp8_32x32_dim_km_swizzle", "mxfp8_32x32_qdata_dim_k_scale_dim_km_swizzle",
                     "fp8_deepseek_128x128", "fp8_rowwise", "fp8_colwise", "nvfp4", "nvfp4_swizzle",
                     "nvfp4_swizzle_dim_k_dim_m_rht", "nvfp4_swizzle_dim_k_sr_dim_m_rht_sr", "nvfp4_blocked_outer", "bf16_rht",
                     "fp32_to_bf16_sr", "fp32_to_bf16_sr_global_offsets"]
    for name, r in Q.ALL_RECIPES:
        inputs = r.example_input_fn(256, 256)
        outs = r.cuda_fn(*inputs, global_row=0, global_col=0, num_col=256)
        assert isinstance(outs, tuple) and all(o.is_cuda for o in outs)


@pytest.mark.gpu
@pytest.mark.parametrize("n", [16, 4096 + 16, 1 << 20, (1 << 22) + 48])
def test_stream_copy_yardstick(n):
    """The benchmarks' plain-copy kernel copies exactly (sizes around the 8 KB per-CTA step)."""
    src = torch.randint(0, 256, (n,), dtype=torch.uint8, device="cuda")
    dst = torch.zeros(n + 32, dtype=torch.uint8, device="cuda")
    Q.stream_copy_cuda(src, dst[:n])
    assert torch.equal(dst[:n], src) and int(dst[n:].sum()) == 0
    assert L.load().qcc_stream_copy(src.data_ptr(), dst.data_ptr(), 24, None) == -1


@pytest.mark.gpu
@pytest.mark.parametrize("ratio", [2, 4])
@pytest.mark.parametrize("nout", [1, 511, 512, 1 << 16, (1 << 18) + 3])
def test_stream_fold_yardstick(ratio, nout):
    """The benchmarks' fold kernel: piece i of dst is the XOR of `ratio` consecutive 16-byte pieces of src."""
    src = torch.randint(0, 256, (nout * ratio, 16), dtype=torch.uint8, device="cuda")
    dst = torch.zeros(nout * 16 + 32, dtype=torch.uint8, device="cuda")
    Q.stream_fold_cuda(src, dst[:nout * 16], ratio)
    want = src.view(nout, ratio, 16)[:, 0]
    for r in range(1, ratio):
        want = want ^ src.view(nout, ratio, 16)[:, r]
    assert torch.equal(dst[:nout * 16].view(nout, 16), want) and int(dst[nout * 16:].sum()) == 0
    lib = L.load()
    assert lib.qcc_stream_fold(src.data_ptr(), dst.data_ptr(), 16 * ratio, 3, None) == -3
    assert lib.qcc_stream_fold(src.data_ptr(), dst.data_ptr(), 16 * ratio + 16, ratio, None) == -1
