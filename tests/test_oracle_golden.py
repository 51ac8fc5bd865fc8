"""The CPU oracle (oracle/qc_oracle.c) against golden vectors produced by the reference's gold
recipes (tests/golden/make_golden.py), bit for bit.  Runs without a GPU."""
import os

import pytest
import torch

from helpers import assert_same_bits, golden, golden_cases, golden_n_outputs, golden_out, golden_rht, golden_x
from oracle import gold_port as O

ONE_INPUT = ["rowwise_fp8_f", "colwise_fp8_f", "mxfp4_f", "mxfp8_f", "mxfp8_swizzle_f", "mxfp8_dim_m_f",
             "mxfp8_dim_m_swizzle_f", "mxfp8_dim_km_f", "mxfp8_dim_km_swizzle_f"]


@pytest.mark.parametrize("tag", golden_cases())
@pytest.mark.parametrize("fn", ONE_INPUT)
def test_single_input_recipes(tag, fn):
    x = golden_x(tag)
    outs = getattr(O, fn)(x)
    assert len(outs) == golden_n_outputs(tag, fn)
    for i, o in enumerate(outs):
        assert_same_bits(o, golden_out(tag, fn, i), f"{fn}[{i}] {tag}")


DEEPSEEK = ["deepseek_1x128_f", "deepseek_128x128_f", "deepseek_1x128_dim_m_f", "deepseek_1x128_dim_km_f"]


@pytest.mark.parametrize("tag", [t for t in golden_cases() if golden_n_outputs(t, "deepseek_1x128_f")])
@pytest.mark.parametrize("fn", DEEPSEEK)
def test_deepseek_recipes(tag, fn):
    x = golden_x(tag)
    outs = getattr(O, fn)(x)
    assert len(outs) == golden_n_outputs(tag, fn) > 0
    for i, o in enumerate(outs):
        assert_same_bits(o, golden_out(tag, fn, i), f"{fn}[{i}] {tag}")


@pytest.mark.parametrize("tag", [t for t in golden_cases() if golden_n_outputs(t, "nvfp4_blocked_outer_f")])
def test_nvfp4_blocked_outer(tag):
    x = golden_x(tag)
    ob = O.nvfp4_blocked_outer_scale(x)
    assert_same_bits(ob, golden_out(tag, "nvfp4_blocked_outer_scale", 0), "blocked outer scale")
    for i, o in enumerate(O.nvfp4_blocked_outer_f(x, ob)):
        assert_same_bits(o, golden_out(tag, "nvfp4_blocked_outer_f", i), f"nvfp4_blocked_outer[{i}] {tag}")


def test_deepseek_clamp_variants():
    """An all-zero block takes the clamp: bf16(1e-12) in the single-direction recipes, fp32(1e-12) in dim_km."""
    x = torch.zeros(128, 128, dtype=torch.bfloat16)
    s_bf16 = O.deepseek_1x128_f(x)[1][0, 0]
    s_f32 = O.deepseek_1x128_dim_km_f(x)[1][0, 0]
    assert s_bf16 == torch.tensor(1e-12).to(torch.bfloat16).float() / 448.0
    assert s_f32 == torch.tensor(1e-12, dtype=torch.float32) / 448.0
    assert s_bf16 != s_f32


B32 = ["mxfp8_32x32_f", "mxfp8_32x32_swizzle_f", "mxfp8_32x32_dim_m_swizzle_f", "mxfp8_32x32_dim_km_swizzle_f",
       "mxfp8_32x32_qdata_dim_k_scale_dim_km_swizzle_f"]


@pytest.mark.parametrize("tag", golden_cases())
@pytest.mark.parametrize("fn", B32)
def test_mxfp8_32x32_recipes(tag, fn):
    x = golden_x(tag)
    outs = getattr(O, fn)(x)
    assert len(outs) == golden_n_outputs(tag, fn) > 0
    for i, o in enumerate(outs):
        assert_same_bits(o, golden_out(tag, fn, i), f"{fn}[{i}] {tag}")


@pytest.mark.parametrize("tag", golden_cases())
def test_fp8_tensorwise(tag):
    x = golden_x(tag)
    s = O.float8_tensorwise_scale(x)
    assert_same_bits(s.reshape(1), golden_out(tag, "float8_tensorwise_scale", 0), "scale")
    assert_same_bits(O.float8_tensorwise_f(x, s)[0], golden_out(tag, "float8_tensorwise_f", 0), "q")


@pytest.mark.parametrize("tag", golden_cases())
def test_fp8_rowwise_precalc(tag):
    x = golden_x(tag)
    ps = O.rowwise_precalc_scale(x)
    assert_same_bits(ps, golden_out(tag, "rowwise_precalc_scale", 0), "scale")
    assert_same_bits(O.rowwise_precalc_f(x, ps)[0], golden_out(tag, "rowwise_precalc_f", 0), "q")


@pytest.mark.parametrize("tag", golden_cases())
def test_fp8_colwise_precalc(tag):
    x = golden_x(tag)
    cs = O.colwise_precalc_scale(x)
    assert_same_bits(cs, golden_out(tag, "colwise_precalc_scale", 0), "scale")
    assert_same_bits(O.colwise_precalc_f(x, cs)[0], golden_out(tag, "colwise_precalc_f", 0), "q")


@pytest.mark.parametrize("tag", golden_cases())
def test_nvfp4(tag):
    x = golden_x(tag)
    gs = O.nvfp4_gs_scale(x)
    assert_same_bits(gs.reshape(1), golden_out(tag, "nvfp4_gs_scale", 0), "outer")
    for fn in ("nvfp4_gs_f", "nvfp4_gs_swizzle_f", "nvfp4_gs_swizzle_t_f", "nvfp4_gs_t_f"):
        for i, o in enumerate(getattr(O, fn)(x, gs)):
            assert_same_bits(o, golden_out(tag, fn, i), f"{fn}[{i}] {tag}")
    pt = golden_out(tag, "nvfp4_per_token_scale", 0).view(torch.float32)
    assert_same_bits(O.nvfp4_gs_per_token_scale(x).clamp(min=2.0 ** -100), pt, "per-token outer scale")   # (the stored one is clamped)
    for i, o in enumerate(O.nvfp4_gs_f(x, pt)):
        assert_same_bits(o, golden_out(tag, "nvfp4_gs_f_per_token", i), f"per-token[{i}] {tag}")


def test_scalar_casts_match_pytorch():
    g = golden()
    for fmt in ("e4m3", "e5m2"):
        v = torch.from_numpy(g[f"kat/{fmt}_in"].copy()).view(torch.float32)
        assert_same_bits(O.f32_to_fp8(v, fmt), torch.from_numpy(g[f"kat/{fmt}_out"].copy()), fmt)
    # the installed PyTorch must still agree with the stored table (arithmetic of record)
    v = torch.from_numpy(g["kat/e4m3_in"].copy()).view(torch.float32)
    assert_same_bits(v.to(torch.float8_e4m3fn), torch.from_numpy(g["kat/e4m3_out"].copy()), "torch e4m3")


def test_fp4_encoder():
    g = golden()
    v = torch.from_numpy(g["kat/e2m1_in"].copy()).view(torch.float32)
    assert_same_bits(O.f32_to_e2m1(v), torch.from_numpy(g["kat/e2m1_out"].copy()), "e2m1")
    # ties to even on every midpoint of the e2m1 grid, and the sign of a negative zero result
    mids = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -0.25, -1e-30, 6.5, -9.0])
    assert O.f32_to_e2m1(mids).tolist() == [0, 2, 2, 4, 4, 6, 6, 8, 8, 7, 15]


def test_e4m3_decode_e8m0_and_blocked_layout():
    g = golden()
    codes = torch.arange(256, dtype=torch.uint8)
    want = torch.from_numpy(g["kat/e4m3_decode"].copy())
    got = O.e4m3_to_f32(codes).view(torch.int32)
    finite = torch.tensor([c not in (0x7F, 0xFF) for c in range(256)])
    assert torch.equal(got[finite], want[finite])
    am = torch.from_numpy(g["kat/rceil_in"].copy()).view(torch.float32)
    assert_same_bits(O.amax_to_e8m0(am), torch.from_numpy(g["kat/rceil_out"].copy()), "rceil")
    assert_same_bits(O.e8m0_to_recip(codes), torch.from_numpy(g["kat/recip_out"].copy()), "recip")
    for H, W in ((128, 4), (96, 5), (300, 9)):
        sc = torch.from_numpy(g[f"kat/blocked_{H}x{W}_in"].copy())
        assert_same_bits(O.to_blocked_4d(sc), torch.from_numpy(g[f"kat/blocked_{H}x{W}_out"].copy()), "blocked")
    assert g["kat/bf16_clamp_min"].view("uint16")[0] == 0x2B8D


@pytest.mark.parametrize("tag", golden_cases())
def test_hadamard_rht(tag):
    """The transform and the two-orientation nvfp4 cast on it (gold G:1324-1333, G:1784-1789).  The gold matmul's
    accumulation order is the GEMM library's; the restatement's fixed butterfly order gives the same bits here."""
    x, rht = golden_x(tag), golden_rht(tag)
    assert_same_bits(O.hadamard_rht_matrix(torch.where(rht[:, 0].float() < 0, -1.0, 1.0)), rht, "rht matrix")
    assert_same_bits(O.hadamard_rht_f(x, rht)[0], golden_out(tag, "hadamard_rht_f", 0), f"rht {tag}")
    gs = O.nvfp4_gs_scale(x)
    gs_m = O.nvfp4_rht_outer_scale_m(x, rht)
    assert_same_bits(gs_m.reshape(1), golden_out(tag, "nvfp4_rht_outer_scale_m", 0), "outer m")
    fn = "nvfp4_gs_swizzle_dim_k_dim_m_rht_f"
    for i, o in enumerate(O.nvfp4_gs_swizzle_dim_k_dim_m_rht_f(x, gs, gs_m, rht)):
        assert_same_bits(o, golden_out(tag, fn, i), f"{fn}[{i}] {tag}")


def test_token_group_layouts():
    g = golden()
    for name in ("a", "b", "c"):
        offs = torch.from_numpy(g[f"kat/mgroups_{name}_offs"].copy())
        sc = torch.from_numpy(g[f"kat/mgroups_{name}_in"].copy())
        assert_same_bits(O.to_blocked_2d_m_groups(sc, offs), torch.from_numpy(g[f"kat/mgroups_{name}_out"].copy()), f"m groups {name}")
        sct = torch.from_numpy(g[f"kat/kgroups_{name}_in"].copy())
        assert_same_bits(O.to_blocked_2d_k_groups(sct, offs // 32), torch.from_numpy(g[f"kat/kgroups_{name}_out"].copy()), f"k groups {name}")


def test_pad_token_groups():
    g = golden()
    for name in ("a", "b", "c"):
        x = torch.from_numpy(g[f"kat/padgroups_{name}_in"].copy()).view(torch.bfloat16)
        offs = torch.from_numpy(g[f"kat/padgroups_{name}_offs"].copy())
        padded, starts, ends = O.pad_token_groups(x, offs)
        assert_same_bits(padded, torch.from_numpy(g[f"kat/padgroups_{name}_out"].copy()), f"padded {name}")
        assert starts.tolist() == g[f"kat/padgroups_{name}_starts"].tolist()
        assert ends.tolist() == g[f"kat/padgroups_{name}_ends"].tolist()


def test_philox_known_answers():
    """Random123 known-answer vectors for Philox4x32-10."""
    kat = [
        ([0] * 4, [0] * 2, [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]),
        ([0xFFFFFFFF] * 4, [0xFFFFFFFF] * 2, [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]),
        ([0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344], [0xA4093822, 0x299F31D0],
         [0xD16CFE09, 0x94FDCCEB, 0x5001E420, 0x24126EA1]),
    ]
    for ctr, key, want in kat:
        assert O.philox4x32_10(ctr, key) == want
    # stream convention: element i uses counter i>>2, lane i&3, low 22 bits
    d = O.sr_dither22(0, 8, (0, 0)).tolist()
    w0 = O.philox4x32_10([0, 0, 0, 0], [0, 0])
    w1 = O.philox4x32_10([1, 0, 0, 0], [0, 0])
    assert d == [w & 0x3FFFFF for w in w0 + w1]


def test_floor_mode_definition():
    """FLOOR (extension): byte = max(fp32 exponent field of amax - 8, 0); data multiplied by the
    exact power-of-two reciprocal and saturated at +-448."""
    am = torch.tensor([0.0, 2.0 ** -130, 1.0, 1.99, 2.0, 448.0, 500.0, 3.0e38])
    assert O.amax_to_e8m0(am, "floor").tolist() == [0, 0, 119, 119, 120, 127, 127, 246]
    x = torch.zeros(1, 32, dtype=torch.bfloat16)
    x[0, 0] = 500.0  # floor scale 2^0 -> 500 saturates to 448
    x[0, 1] = -3.0
    q, s = O.mxfp8_f(x, mode="floor")
    assert s.view(torch.uint8).item() == 127
    assert q.view(torch.uint8)[0, :2].tolist() == [0x7E, 0xC4]


def _reference_checkout():
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
    import make_golden
    return make_golden.default_reference()


@pytest.mark.skipif(_reference_checkout() is None, reason="reference checkout not present ($QCC_REFERENCE_ROOT)")
def test_against_live_reference():
    """Where the reference checkout is present, run its gold recipes directly on fresh inputs."""
    import make_golden
    G, _ = make_golden.import_gold(_reference_checkout())
    for (M, N, seed) in [(256, 256, 11), (384, 128, 12), (32, 2048, 13)]:
        x = make_golden.make_input(M, N, seed, spread=8.0)
        for fn in ONE_INPUT:
            for i, (a, b) in enumerate(zip(getattr(O, fn)(x), getattr(G, fn)(x))):
                assert_same_bits(a, b, f"{fn}[{i}] {M}x{N}")
        gs = G.nvfp4_gs_scale(x)
        for fn in ("nvfp4_gs_f", "nvfp4_gs_swizzle_f"):
            for i, (a, b) in enumerate(zip(getattr(O, fn)(x, gs), getattr(G, fn)(x, gs))):
                assert_same_bits(a, b, f"{fn}[{i}] {M}x{N}")
        for i, (a, b) in enumerate(zip(O.nvfp4_gs_swizzle_t_f(x, gs), G.nvfp4_gs_swizzle_f(x.t().contiguous(), gs))):
            assert_same_bits(a, b, f"nvfp4_t[{i}] {M}x{N}")
