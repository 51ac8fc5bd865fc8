"""The casts as native PyTorch operators (torch.ops.quant_cast_cuda_native.*, registered from C++ in
csrc/torch_binding.cpp and built into lib/libquant_cast_torch.so).

CPU: the library loads, its Meta implementations give the shapes and dtype views the gold recipes return (checked
against the golden vectors' shapes), a CPU tensor is refused.  GPU: the golden vectors of the reference replayed through
the operators, bit for bit; both forms of the constant division; a cast traced by torch.compile(fullgraph=True)."""
import os

import pytest
import torch

from helpers import assert_same_bits, golden_cases, golden_n_outputs, golden_out, golden_x, same_outputs
from quant_cast_bench_b200 import build as qbuild

qbuild.build_torch_binding()          # in-tree, a few seconds; no GPU needed
from quant_cast_bench_b200.quant_cast_cuda import _lib as L  # noqa: E402
from quant_cast_bench_b200.quant_cast_cuda import native_ops as N  # noqa: E402
from test_torch_ops import GOLD_FN, _inputs  # noqa: E402


def test_library_is_built_in_tree_and_registers_the_operators():
    assert os.path.exists(N.LIB) and os.path.dirname(N.LIB).endswith(os.path.join("quant_cast_bench_b200", "lib"))
    for name in ("amax", "fp8_tensorwise", "fp8_rowwise", "fp8_colwise", "mxfp8", "nvfp4"):
        op = getattr(torch.ops.quant_cast_cuda_native, name)
        assert "Tensor x" in str(op.default._schema), name
    assert "recip_div=False" in str(torch.ops.quant_cast_cuda_native.fp8_rowwise.default._schema)


@pytest.mark.parametrize("name,fn", N.NATIVE_RECIPES)
def test_meta_implementations_give_the_gold_shapes(name, fn):
    gold_fn, aux = GOLD_FN[name]
    for tag in golden_cases():
        if golden_n_outputs(tag, gold_fn) == 0:
            continue
        meta = tuple(t.to("meta") for t in _inputs(tag, aux, "cpu"))
        outs = fn(*meta)
        assert len(outs) == golden_n_outputs(tag, gold_fn)
        for i, o in enumerate(outs):
            want = golden_out(tag, gold_fn, i)
            assert o.device.type == "meta" and tuple(o.shape) == tuple(want.shape), (name, tag, i)
            assert o.numel() * o.element_size() == want.numel() * want.element_size(), (name, tag, i)


def _more_inputs(tag, aux, device):
    x = golden_x(tag).to(device)
    key = {"row_scale": "rowwise_precalc_scale", "col_scale": "colwise_precalc_scale", "blocked_outer": "nvfp4_blocked_outer_scale",
           "per_token": "nvfp4_per_token_scale", "outer": "nvfp4_gs_scale"}.get(aux)
    if key is None:
        return (x,)
    a = golden_out(tag, key, 0).view(torch.float32)
    return (x, (a.reshape(()) if aux == "outer" else a).to(device))


@pytest.mark.parametrize("gold_fn,fn,aux", N.MORE_NATIVE)
def test_meta_shapes_of_the_other_families(gold_fn, fn, aux):
    ran = 0
    for tag in golden_cases():
        n = golden_n_outputs(tag, gold_fn)
        if n == 0:
            continue
        outs = fn(*(t.to("meta") for t in _more_inputs(tag, aux, "cpu")))
        assert len(outs) == n, (gold_fn, tag)
        for i, o in enumerate(outs):
            want = golden_out(tag, gold_fn, i)
            assert tuple(o.shape) == tuple(want.shape) and o.numel() * o.element_size() == want.numel() * want.element_size(), (gold_fn, tag, i)
        ran += 1
    assert ran > 0


@pytest.mark.gpu
@pytest.mark.parametrize("gold_fn,fn,aux", N.MORE_NATIVE)
def test_the_other_families_match_the_golden_vectors(gold_fn, fn, aux):
    ran = 0
    for tag in golden_cases():
        n = golden_n_outputs(tag, gold_fn)
        if n == 0:
            continue
        outs = fn(*_more_inputs(tag, aux, "cuda"))
        for i, o in enumerate(outs):
            assert_same_bits(o, golden_out(tag, gold_fn, i), f"{gold_fn}[{i}] {tag}")
        ran += 1
    assert ran > 0


@pytest.mark.gpu
def test_stochastic_and_two_orientation_forms_match_the_ctypes_route():
    from quant_cast_bench_b200 import quant_cast_cuda as Q
    x = torch.randn(256, 512, device="cuda", dtype=torch.bfloat16)
    gs = Q.nvfp4_gs_scale_cuda(x)
    key = Q.philox_key(7, device="cuda")
    for a, b in zip(N.nvfp4_gs_swizzle_sr_native(x, gs, key), Q.nvfp4_gs_swizzle_sr_cuda(x, gs, key)):
        assert_same_bits(a, b, "nvfp4 sr")
    for a, b in zip(N.nvfp4_gs_swizzle_t_sr_native(x, gs, key), Q.nvfp4_gs_swizzle_t_sr_cuda(x, gs, key)):
        assert_same_bits(a, b, "nvfp4 transposed sr")
    for a, b in zip(N.nvfp4_gs_swizzle_both_native(x, gs), Q.nvfp4_gs_swizzle_both_cuda(x, gs)):
        assert_same_bits(a, b, "nvfp4 both")
    for a, b in zip(N.mxfp4_native(x, swizzle=True), Q.mxfp4_cuda(x, swizzle=True)):
        assert_same_bits(a, b, "mxfp4 blocked")


@pytest.mark.gpu
def test_per_token_scale_and_stochastic_bf16_match_the_ctypes_route():
    from quant_cast_bench_b200 import quant_cast_cuda as Q
    x = torch.randn(200, 328, device="cuda", dtype=torch.bfloat16)
    assert_same_bits(N.nvfp4_gs_per_token_scale_native(x), Q.nvfp4_gs_per_token_scale_cuda(x), "per-token scale")
    xf = torch.randn(96, 200, device="cuda")
    key = Q.philox_key(3, 9, device="cuda")
    assert_same_bits(N.sr_bf16_native(xf, key)[0], Q.sr_bf16_cuda(xf, key)[0], "sr bf16")
    assert_same_bits(N.sr_bf16_global_native(xf, key, global_row=4, global_col=16, num_col=512)[0],
                     Q.sr_bf16_global_cuda(xf, key, global_row=4, global_col=16, num_col=512)[0], "sr bf16 global")
    m = N.sr_bf16_native(xf.to("meta"), key.to("meta"))[0]
    assert m.device.type == "meta" and m.dtype == torch.bfloat16 and tuple(m.shape) == (96, 200)


def test_operators_have_no_cpu_implementation_and_check_their_arguments():
    with pytest.raises(NotImplementedError):
        torch.ops.quant_cast_cuda_native.mxfp8(torch.zeros(32, 32, dtype=torch.bfloat16), True, False, False, "rceil")
    x = torch.empty(64, 64, dtype=torch.bfloat16, device="meta")
    with pytest.raises(RuntimeError, match="mode must be"):
        torch.ops.quant_cast_cuda_native.mxfp8(x, True, False, False, "nearest")
    with pytest.raises(RuntimeError, match="fmt must be"):
        torch.ops.quant_cast_cuda_native.fp8_rowwise(x, "e3m4")


@pytest.mark.gpu
@pytest.mark.parametrize("name,fn", N.NATIVE_RECIPES)
def test_operators_match_the_golden_vectors(name, fn):
    gold_fn, aux = GOLD_FN[name]
    ran = 0
    for tag in golden_cases():
        n = golden_n_outputs(tag, gold_fn)
        if n == 0:
            continue
        outs = fn(*_inputs(tag, aux, "cuda"))
        want = [golden_out(tag, gold_fn, i) for i in range(n)]
        got = [o.view(torch.uint8) if o.element_size() == 1 else o for o in outs]
        same_outputs(got, [w if w.dtype == torch.uint8 else w.view(torch.float32) for w in want], f"{name} {tag}")
        ran += 1
    assert ran > 0


@pytest.mark.gpu
def test_scales_and_both_division_forms_match_the_ctypes_route():
    from quant_cast_bench_b200 import quant_cast_cuda as Q
    g = torch.Generator().manual_seed(5)
    x = (torch.randn(384, 1024, generator=g) * torch.exp2(torch.rand(384, 1, generator=g) * 12 - 6)).to(torch.bfloat16).cuda()
    for mode in ("ieee", "cuda_eager"):
        with L.scalar_division(mode):
            assert_same_bits(N.float8_tensorwise_scale_native(x).reshape(1), Q.float8_tensorwise_scale_cuda(x).reshape(1), f"fp8 scale {mode}")
            assert_same_bits(N.nvfp4_gs_scale_native(x).reshape(1), Q.nvfp4_gs_scale_cuda(x).reshape(1), f"nvfp4 scale {mode}")
            for a, b in zip(N.rowwise_fp8_native(x), Q.rowwise_fp8_cuda(x)):
                assert_same_bits(a, b, f"rowwise {mode}")
            for a, b in zip(N.colwise_fp8_native(x, "e5m2"), Q.colwise_fp8_cuda(x, "e5m2")):
                assert_same_bits(a, b, f"colwise e5m2 {mode}")
            gs = Q.nvfp4_gs_scale_cuda(x)
            for a, b in zip(N.nvfp4_gs_swizzle_t_native(x, gs), Q.nvfp4_gs_swizzle_t_cuda(x, gs)):
                assert_same_bits(a, b, f"nvfp4 transposed {mode}")
    assert_same_bits(N.amax_native(x).reshape(1), Q.amax_cuda(x).reshape(1), "amax")
    with L.scalar_division("cuda_eager"):
        s_dev = N.rowwise_fp8_native(x)[1]
    assert not torch.equal(s_dev, N.rowwise_fp8_native(x)[1])     # the two forms do differ on this input


@pytest.mark.gpu
def test_a_cast_traces_under_torch_compile():
    from quant_cast_bench_b200 import quant_cast_cuda as Q
    x = torch.randn(256, 512, device="cuda", dtype=torch.bfloat16)

    def f(t):
        t = t * 2.0
        qk, sk, qm, sm = N.mxfp8_dim_km_swizzle_native(t)
        outer = N.nvfp4_gs_scale_native(t)
        q4, s4 = N.nvfp4_gs_swizzle_native(t, outer)
        return qk, sk, qm, sm, q4, s4

    got = torch.compile(f, fullgraph=True)(x)
    x2 = x * 2.0
    want = (*Q.mxfp8_dim_km_swizzle_cuda(x2), *Q.nvfp4_gs_swizzle_cuda(x2, Q.nvfp4_gs_scale_cuda(x2)))
    for g_, w in zip(got, want):
        assert g_.dtype == w.dtype and torch.equal(g_.view(torch.uint8), w.view(torch.uint8))


@pytest.mark.gpu
def test_operators_are_callable_from_cpp_without_python(tmp_path):
    """tests/cpp/native_op_from_cpp.cpp: a C++ program that links the operator library, finds the operator in the
    dispatcher and compares its outputs with the C ABI called directly."""
    import subprocess
    from torch.utils import cpp_extension as ext
    src = os.path.join(os.path.dirname(os.path.abspath(__file__)), "cpp", "native_op_from_cpp.cpp")
    exe = str(tmp_path / "native_op_from_cpp")
    lib_dir = os.path.dirname(N.LIB)
    cmd = ["g++", "-O1", "-std=c++17", src, "-o", exe, f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    cmd += [f"-I{p}" for p in ext.include_paths("cuda")]
    cmd += [f"-L{p}" for p in ext.library_paths("cuda")] + [f"-L{lib_dir}"]
    cmd += ["-Wl,--no-as-needed", "-lquant_cast_torch", "-lquant_cast_cuda", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch",
            "-lcudart"]
    cmd += [f"-Wl,-rpath,{p}" for p in ext.library_paths("cuda") + [lib_dir]]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, (r.stdout + r.stderr)[-2000:]
    assert "equals the C ABI: ok" in r.stdout
