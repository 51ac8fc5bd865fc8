"""The casts as registered PyTorch operators (torch.ops.quant_cast_cuda.*).

CPU: the fake (meta) implementations give the shapes and dtype views the gold recipes return (checked against the
golden vectors' shapes); a CPU tensor is refused.  GPU: the golden vectors of the reference replayed through the
operators, bit for bit, and a cast traced by torch.compile(fullgraph=True)."""
import pytest
import torch

from helpers import golden_cases, golden_n_outputs, golden_out, golden_x, same_outputs
from quant_cast_bench_b200.quant_cast_cuda import torch_ops as T

# gold function name in the golden file -> operator-backed function and the aux inputs it takes
GOLD_FN = {
    "fp8_tensorwise_precalc_scale": ("float8_tensorwise_f", "scale"), "fp8_rowwise": ("rowwise_fp8_f", None),
    "fp8_colwise": ("colwise_fp8_f", None), "mxfp8": ("mxfp8_f", None), "mxfp8_swizzle": ("mxfp8_swizzle_f", None),
    "mxfp8_dim_m": ("mxfp8_dim_m_f", None), "mxfp8_dim_m_swizzle": ("mxfp8_dim_m_swizzle_f", None),
    "mxfp8_dim_km": ("mxfp8_dim_km_f", None), "mxfp8_dim_km_swizzle": ("mxfp8_dim_km_swizzle_f", None),
    "nvfp4": ("nvfp4_gs_f", "outer"), "nvfp4_swizzle": ("nvfp4_gs_swizzle_f", "outer"),
}
DT = {"uint8": torch.uint8, "int32": torch.int32}


def _inputs(tag, aux, device):
    x = golden_x(tag).to(device)
    if aux == "scale":
        return (x, golden_out(tag, "float8_tensorwise_scale", 0).view(torch.float32).reshape(()).to(device))
    if aux == "outer":
        return (x, golden_out(tag, "nvfp4_gs_scale", 0).view(torch.float32).reshape(()).to(device))
    return (x,)


@pytest.mark.parametrize("name,fn", T.OP_RECIPES)
def test_fake_implementations_give_the_gold_shapes(name, fn):
    gold_fn, aux = GOLD_FN[name]
    for tag in golden_cases():
        if golden_n_outputs(tag, gold_fn) == 0:
            continue
        meta = tuple(t.to("meta") for t in _inputs(tag, aux, "cpu"))
        outs = fn(*meta)
        assert len(outs) == golden_n_outputs(tag, gold_fn)
        for i, o in enumerate(outs):
            want = golden_out(tag, gold_fn, i)
            assert o.device.type == "meta" and o.numel() * o.element_size() == want.numel() * want.element_size(), (name, tag, i)
            assert tuple(o.shape) == tuple(want.shape), (name, tag, i)


def test_operators_have_no_cpu_implementation():
    with pytest.raises(NotImplementedError):
        torch.ops.quant_cast_cuda.mxfp8(torch.zeros(32, 32, dtype=torch.bfloat16), True, False, False, "rceil")


@pytest.mark.gpu
@pytest.mark.parametrize("name,fn", T.OP_RECIPES)
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
def test_a_cast_traces_under_torch_compile():
    from quant_cast_bench_b200 import quant_cast_cuda as Q
    x = torch.randn(256, 512, device="cuda", dtype=torch.bfloat16)

    def f(t):
        t = t * 2.0
        qk, sk, qm, sm = T.mxfp8_dim_km_swizzle_op(t)
        outer = T.nvfp4_gs_scale_op(t)
        q4, s4 = T.nvfp4_gs_swizzle_op(t, outer)
        return qk, sk, qm, sm, q4, s4

    got = torch.compile(f, fullgraph=True)(x)
    x2 = x * 2.0
    want = (*Q.mxfp8_dim_km_swizzle_cuda(x2), *Q.nvfp4_gs_swizzle_cuda(x2, Q.nvfp4_gs_scale_cuda(x2)))
    for g, w in zip(got, want):
        assert g.dtype == w.dtype and torch.equal(g.view(torch.uint8), w.view(torch.uint8))
