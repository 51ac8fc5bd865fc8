"""`tensor / python_scalar` of the gold recipes on the CPU and on a CUDA device.

Eager PyTorch computes `amax / 448.0` as one IEEE division on the CPU and as `amax * fl(1 / 448)` on a CUDA device
(aten/src/ATen/native/cuda/BinaryDivTrueKernel.cu), so the reference's gold recipes give slightly different scales --
and a few different quantised bytes -- depending on where they run.  The casts follow the CPU form by default and the
CUDA form under `scalar_division("cuda_eager")`; both are pinned here:

  * the CPU form by tests/golden/gold_vectors.npz (the other test files),
  * the CUDA form by tests/golden/gold_vectors_cuda.npz, which `tests/golden/make_golden.py --device cuda` wrote on a
    B200 from the same inputs, and -- where the reference package is installed under oracle/_ref -- by running its
    gold recipes on the test's own GPU.
"""
import os

import numpy as np
import pytest
import torch

from helpers import assert_same_bits, golden, golden_cases, golden_rht, golden_x
from oracle import gold_port as O
from quant_cast_bench_b200.quant_cast_cuda import _lib as L

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN_CUDA = os.path.join(HERE, "golden", "gold_vectors_cuda.npz")
_gc = None


def golden_cuda():
    global _gc
    if _gc is None:
        _gc = np.load(GOLDEN_CUDA)
    return _gc


needs_cuda_golden = pytest.mark.skipif(not os.path.exists(GOLDEN_CUDA), reason="tests/golden/gold_vectors_cuda.npz not generated")


def want(key):
    """The gold output `key` as a CUDA device computes it: from the CUDA file when it differs from the CPU file."""
    gc = golden_cuda()
    if key in gc.files:
        return torch.from_numpy(gc[key].copy())
    assert key in set(str(k) for k in gc["same_as_cpu"]), f"{key} is in neither list of the CUDA file"
    return torch.from_numpy(golden()[key].copy())


def chain(ns, suffix, x, tag, rht, per_token, dev):
    """Every division-affected recipe on one input, keyed like the golden files.  `ns` + `suffix` name the
    implementation: (oracle.gold_port, "") or (quant_cast_cuda, "_cuda")."""
    f = lambda name: getattr(ns, name + suffix)           # noqa: E731
    g = lambda name: getattr(ns, name[:-2] + suffix if suffix else name)   # noqa: E731  gold "<name>_f" -> "<name>_cuda"
    out = {}
    s = f("float8_tensorwise_scale")(x)
    out["float8_tensorwise_scale/0"] = s.reshape(1)
    out["float8_tensorwise_f/0"] = g("float8_tensorwise_f")(x, s)[0]
    ps = f("rowwise_precalc_scale")(x)
    out["rowwise_precalc_scale/0"] = ps
    out["rowwise_precalc_f/0"] = g("rowwise_precalc_f")(x, ps)[0]
    cs = f("colwise_precalc_scale")(x)
    out["colwise_precalc_scale/0"] = cs
    out["colwise_precalc_f/0"] = g("colwise_precalc_f")(x, cs)[0]
    single = ["rowwise_fp8_f", "colwise_fp8_f", "mxfp8_f", "mxfp8_dim_km_swizzle_f"]
    M, N = x.shape
    if M % 128 == 0 and N % 128 == 0:
        single += ["deepseek_1x128_f", "deepseek_128x128_f", "deepseek_1x128_dim_m_f", "deepseek_1x128_dim_km_f"]
        ob = f("nvfp4_blocked_outer_scale")(x)
        ob = torch.where(ob == 0, torch.full_like(ob, 2.0 ** -100), ob)
        out["nvfp4_blocked_outer_scale/0"] = ob
        for i, o in enumerate(g("nvfp4_blocked_outer_f")(x, ob)):
            out[f"nvfp4_blocked_outer_f/{i}"] = o
    for name in single:
        for i, o in enumerate(g(name)(x)):
            out[f"{name}/{i}"] = o
    gs = f("nvfp4_gs_scale")(x)
    out["nvfp4_gs_scale/0"] = gs.reshape(1)
    for name in ("nvfp4_gs_f", "nvfp4_gs_swizzle_f", "nvfp4_gs_swizzle_t_f", "nvfp4_gs_t_f"):
        for i, o in enumerate(g(name)(x, gs)):
            out[f"{name}/{i}"] = o
    gs_m = f("nvfp4_rht_outer_scale_m")(x, rht)
    out["nvfp4_rht_outer_scale_m/0"] = gs_m.reshape(1)
    for i, o in enumerate(g("nvfp4_gs_swizzle_dim_k_dim_m_rht_f")(x, gs, gs_m, rht)):
        out[f"nvfp4_gs_swizzle_dim_k_dim_m_rht_f/{i}"] = o
    for i, o in enumerate(g("nvfp4_gs_f")(x, per_token.to(dev))):
        out[f"nvfp4_gs_f_per_token/{i}"] = o
    out["nvfp4_per_token_scale/0"] = f("nvfp4_gs_per_token_scale")(x).clamp(min=2.0 ** -100)   # the files store it clamped
    return out


# ---------------------------------------------------------------------------- host side, no GPU
def test_setting_and_flag():
    assert L.get_scalar_division() == "ieee" and L.div_flag() == 0
    with L.scalar_division("cuda_eager"):
        assert L.get_scalar_division() == "cuda_eager" and L.div_flag() == L.RECIP_DIV == 0x800
        with L.scalar_division("ieee"):
            assert L.div_flag() == 0
        assert L.div_flag() == L.RECIP_DIV
    assert L.get_scalar_division() == "ieee"
    with pytest.raises(ValueError):
        L.set_scalar_division("fast")
    assert L.get_scalar_division() == "ieee"


def test_oracle_forms_differ_as_pytorch_documents():
    """a * fl(1 / c) against a / c: the oracle's two forms are the two PyTorch expressions, and they do differ."""
    g = torch.Generator().manual_seed(3)
    x = torch.randn(256, 512, generator=g).to(torch.bfloat16)
    amax = x.abs().amax(dim=1, keepdim=True).clamp(min=1e-12).float()
    _, s_ieee = O.rowwise_fp8_f(x)
    with O.scalar_division("cuda_eager"):
        _, s_cuda = O.rowwise_fp8_f(x)
        gs_cuda = O.nvfp4_gs_scale(x)
    assert torch.equal(s_ieee, amax / 448.0)
    inv = torch.tensor(1.0, dtype=torch.float32) / torch.tensor(448.0, dtype=torch.float32)
    assert torch.equal(s_cuda, amax * inv)
    assert 0 < int((s_ieee != s_cuda).sum()) < s_ieee.numel()
    inv2688 = torch.tensor(1.0, dtype=torch.float32) / torch.tensor(2688.0, dtype=torch.float32)
    assert torch.equal(gs_cuda, x.abs().amax().float() * inv2688)
    assert torch.equal(O.rowwise_fp8_f(x)[1], s_ieee)            # the setting was restored


@needs_cuda_golden
@pytest.mark.parametrize("tag", golden_cases())
def test_oracle_cuda_eager_matches_gold_run_on_a_cuda_device(tag):
    x = golden_x(tag)
    pt = want(f"{tag}/nvfp4_per_token_scale/0").view(torch.float32)
    with O.scalar_division("cuda_eager"):
        outs = chain(O, "", x, tag, golden_rht(tag), pt, "cpu")
    for key, o in outs.items():
        assert_same_bits(o, want(f"{tag}/{key}"), f"{key} {tag}")


@needs_cuda_golden
def test_cuda_file_lists_what_differs():
    """The device form changes the fp8 scales and the outer scales; the mxfp8 family has no such division."""
    gc = golden_cuda()
    differs = {k.split("/", 1)[1] for k in gc.files if "/" in k}
    same = {str(k).split("/", 1)[1] for k in gc["same_as_cpu"]}
    assert "rowwise_fp8_f/1" in differs and "rowwise_precalc_scale/0" in differs and "colwise_fp8_f/1" in differs
    for k in ("mxfp8_f/0", "mxfp8_f/1", "mxfp8_swizzle_f/1", "mxfp8_dim_km_swizzle_f/2", "mxfp4_f/0", "hadamard_rht_f/0"):
        assert k in same and k not in differs, k


# ---------------------------------------------------------------------------- on the GPU
def _c2_like(M, N, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, N, generator=g) * torch.exp2((torch.rand(M, 1, generator=g) * 2 - 1) * 10.0)
    x = torch.where(torch.rand(M, N, generator=g) < 1e-3, x * 100.0, x)
    x[torch.rand(M, generator=g) < 0.01] = 0
    return x.to(torch.bfloat16)


@pytest.mark.gpu
@needs_cuda_golden
@pytest.mark.parametrize("tag", golden_cases())
def test_kernels_cuda_eager_match_gold_run_on_a_cuda_device(tag):
    from quant_cast_bench_b200 import quant_cast_cuda as Q
    x = golden_x(tag).cuda()
    pt = want(f"{tag}/nvfp4_per_token_scale/0").view(torch.float32)
    with L.scalar_division("cuda_eager"):
        outs = chain(Q, "_cuda", x, tag, golden_rht(tag).cuda(), pt, "cuda")
    for key, o in outs.items():
        assert_same_bits(o, want(f"{tag}/{key}"), f"{key} {tag}")


@pytest.mark.gpu
@pytest.mark.parametrize("shape,seed", [((128, 256), 0), ((384, 1024), 1), ((1024, 7168), 2), ((2048, 16384), 3), ((96, 160), 4)])
def test_kernels_cuda_eager_match_the_oracle(shape, seed):
    from quant_cast_bench_b200 import quant_cast_cuda as Q
    x = _c2_like(*shape, seed)
    rht = O.hadamard_rht_matrix(torch.tensor([1, -1, -1, 1] * 4, dtype=torch.bfloat16))
    pt = (x.abs().float().amax(dim=1, keepdim=True) / 2688.0).clamp(min=2.0 ** -100)
    with O.scalar_division("cuda_eager"):
        ref = chain(O, "", x, "", rht, pt, "cpu")
    with L.scalar_division("cuda_eager"):
        got = chain(Q, "_cuda", x.cuda(), "", rht.cuda(), pt, "cuda")
    assert ref.keys() == got.keys()
    for key in ref:
        assert_same_bits(got[key], ref[key], f"{key} {shape}")
    # and the default form still differs from it where a division is involved
    s_default = Q.rowwise_precalc_scale_cuda(x.cuda())
    assert not torch.equal(s_default.cpu(), ref["rowwise_precalc_scale/0"])


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["ieee", "cuda_eager"])
def test_e5m2_forms_match_the_oracle_in_both_settings(mode):
    """The e5m2 extension divides by 57344 the same two ways."""
    from quant_cast_bench_b200 import quant_cast_cuda as Q
    x = _c2_like(256, 768, 21)
    xc = x.cuda()
    with O.scalar_division(mode), L.scalar_division(mode):
        assert_same_bits(Q.float8_tensorwise_scale_cuda(xc, "e5m2").reshape(1), O.float8_tensorwise_scale(x, "e5m2").reshape(1), "scale")
        for name in ("rowwise_fp8", "colwise_fp8"):
            got = getattr(Q, name + "_cuda")(xc, "e5m2")
            ref = getattr(O, name + "_f")(x, "e5m2")
            for i, (a, b) in enumerate(zip(got, ref)):
                assert_same_bits(a, b, f"{name} e5m2 [{i}] {mode}")


@pytest.mark.gpu
def test_from_amax_and_exchange_forms_follow_the_setting():
    """The casts that form their scale from a raw amax in their prologue take the same flag."""
    from quant_cast_bench_b200 import quant_cast_cuda as Q
    x = _c2_like(512, 1024, 11).cuda()
    with L.scalar_division("cuda_eager"):
        amax = Q.amax_cuda(x)
        q1, s1 = Q.float8_tensorwise_from_amax_cuda(x, amax)
        s_ref = Q.float8_tensorwise_scale_cuda(x)
        assert_same_bits(s1.reshape(1), s_ref.reshape(1), "scale from amax")
        assert_same_bits(q1, Q.float8_tensorwise_cuda(x, s_ref)[0], "q from amax")
        outs = Q.nvfp4_from_amax_cuda(x, amax)
        gs = Q.nvfp4_gs_scale_cuda(x)
        assert_same_bits(outs[2].reshape(1), gs.reshape(1), "outer from amax")
        for a, b in zip(outs[:2], Q.nvfp4_gs_swizzle_cuda(x, gs)):
            assert_same_bits(a, b, "nvfp4 from amax")
        assert_same_bits(Q.scale_from_amax_cuda(amax, "nvfp4").reshape(1), gs.reshape(1), "scale_from_amax")
        inv = torch.tensor(1.0, dtype=torch.float32) / torch.tensor(2688.0, dtype=torch.float32)
        assert torch.equal(gs.cpu(), amax.cpu() * inv)


@pytest.mark.gpu
def test_kernels_cuda_eager_match_the_reference_gold_on_this_gpu():
    """The reference's own test pattern (test/test_quant_cast_triton.py:70-107): its gold recipe and this backend on the
    same CUDA tensor, bit for bit.  Needs the reference installed under oracle/_ref."""
    from oracle import ref_gold
    if not ref_gold.available():
        pytest.skip("the reference package is not installed under oracle/_ref")
    G = ref_gold.gold()
    from quant_cast_bench_b200 import quant_cast_cuda as Q
    from quant_cast_bench_b200.quant_cast_cuda import recipes as R
    gold_index = dict(G.ALL_RECIPES)
    checked = 0
    for shape, seed in (((512, 512), 0), ((1024, 7168), 1)):
        x = _c2_like(*shape, seed).cuda()
        with L.scalar_division("cuda_eager"):
            assert_same_bits(Q.float8_tensorwise_scale_cuda(x).reshape(1), G.float8_tensorwise_scale(x).reshape(1), "tensorwise scale")
            assert_same_bits(Q.nvfp4_gs_scale_cuda(x).reshape(1), G.nvfp4_gs_scale(x).reshape(1), "nvfp4 outer scale")
            assert_same_bits(Q.rowwise_precalc_scale_cuda(x), G.rowwise_precalc_scale(x), "row scales")
            assert_same_bits(Q.colwise_precalc_scale_cuda(x).reshape(-1), G.colwise_precalc_scale(x).reshape(-1), "column scales")
            assert_same_bits(Q.nvfp4_blocked_outer_scale_cuda(x), G.nvfp4_blocked_outer_scale(x), "blocked outer scales")
            assert_same_bits(Q.nvfp4_gs_per_token_scale_cuda(x), G.nvfp4_gs_per_token_scale(x), "per-token outer scales")
            rht = R._rht_matrix(x)
            # The gold transform is a bf16 matmul, which on the GPU runs on the tensor cores: their accumulation aligns
            # the 16 addends to the largest exponent and drops bits below it, so where the sum nearly cancels the gold
            # result on the device is off by an ulp or two from the exact sum that a CPU matmul and this backend's fp32
            # butterfly both give (rows of very different magnitude make that frequent; N(0, 1) data makes it about one
            # element in 10^5).  The transformed outputs are therefore compared by count, everything else bit for bit.
            xe = torch.randn(*shape, generator=torch.Generator().manual_seed(100 + seed)).to(torch.bfloat16).cuda()
            for name, rec in R.ALL_RECIPES:
                if "sr" in name.split("_") or name not in gold_index:
                    continue
                if name == "fp8_tensorwise_precalc_scale":
                    inputs = (x, G.float8_tensorwise_scale(x))
                elif name == "fp8_rowwise_precalc_scale":
                    inputs = (x, G.rowwise_precalc_scale(x))
                elif name == "fp8_colwise_precalc_scale":
                    inputs = (x, G.colwise_precalc_scale(x))
                elif name in ("nvfp4", "nvfp4_swizzle"):
                    inputs = (x, G.nvfp4_gs_scale(x))
                elif name == "nvfp4_blocked_outer":
                    ob = G.nvfp4_blocked_outer_scale(x)
                    inputs = (x, torch.where(ob == 0, torch.full_like(ob, 2.0 ** -100), ob))
                elif name == "bf16_rht":
                    inputs = (xe, rht)
                elif name == "nvfp4_swizzle_dim_k_dim_m_rht":
                    (xt,) = G.hadamard_rht_f(xe.t().contiguous(), rht)
                    inputs = (xe, G.nvfp4_gs_scale(xe), xt.abs().to(torch.float32).amax() / (G.F8E4M3_MAX * G.F4_E2M1_MAX), rht)
                else:
                    inputs = (x,)
                want_outs = gold_index[name].pt_ref_fn(*inputs)
                got_outs = rec.cuda_fn(*inputs)
                assert len(want_outs) == len(got_outs), name
                for i, (a, b) in enumerate(zip(got_outs, want_outs)):
                    if name == "bf16_rht" or (name == "nvfp4_swizzle_dim_k_dim_m_rht" and i >= 2):
                        a8, b8 = a.contiguous().view(torch.uint8), b.contiguous().view(torch.uint8)
                        assert a8.shape == b8.shape, f"{name}[{i}] {shape}"
                        assert int((a8 != b8).sum()) <= max(2, a8.numel() // 20000), f"{name}[{i}] {shape}"
                    else:
                        assert_same_bits(a, b.contiguous(), f"{name}[{i}] {shape}")
                checked += 1
    assert checked >= 40
