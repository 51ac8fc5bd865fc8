"""Consumer check: the quantized bytes and the 32x4x4 blocked scales are what the block-scaled GEMM of the GPU
consumes.  Mirrors the reference's end-to-end test (test/test_quant_cast_gold.py:90-194: quantize both operands,
multiply with the scaled GEMM, compare with the bf16 product by SQNR), here through torch._scaled_mm."""
import pytest
import torch

from quant_cast_bench_b200 import quant_cast_cuda as Q

pytestmark = pytest.mark.gpu


def _sqnr(ref, got):
    return (20 * torch.log10(torch.linalg.vector_norm(ref) / torch.linalg.vector_norm(ref - got))).item()


def _scaled_mm(a, b_t, sa, sb, **kw):
    try:
        return torch._scaled_mm(a, b_t, scale_a=sa, scale_b=sb, out_dtype=torch.bfloat16, **kw)
    except (RuntimeError, NotImplementedError, TypeError) as e:  # this torch build lacks the block-scaled path
        pytest.skip(f"torch._scaled_mm does not take these operands here: {str(e).splitlines()[0][:120]}")


def test_mxfp8_blocked_scales_feed_scaled_mm():
    torch.manual_seed(0)
    M, K, N = 256, 512, 384
    a = torch.randn(M, K, dtype=torch.bfloat16, device="cuda")
    b = torch.randn(N, K, dtype=torch.bfloat16, device="cuda")
    qa, sa = Q.mxfp8_swizzle_cuda(a)
    qb, sb = Q.mxfp8_swizzle_cuda(b)
    y = _scaled_mm(qa, qb.t(), sa.flatten(), sb.flatten())
    ref = a.float() @ b.float().t()
    assert _sqnr(ref, y.float()) > 25.0
    # the transposed output of the two-direction cast is the same operand for the other GEMM of a linear layer:
    # (K, M) quantised along M feeds a product over M
    c = torch.randn(M, N, dtype=torch.bfloat16, device="cuda")       # e.g. grad_output
    _, _, qa_t, sa_t = Q.mxfp8_dim_km_swizzle_cuda(a)                # (K, M) blocks along M
    _, _, qc_t, sc_t = Q.mxfp8_dim_km_swizzle_cuda(c)                # (N, M) blocks along M
    y2 = _scaled_mm(qc_t, qa_t.t(), sc_t.flatten(), sa_t.flatten())  # (N, K) = c^T a
    ref2 = c.float().t() @ a.float()
    assert _sqnr(ref2, y2.float()) > 25.0


def test_nvfp4_blocked_scales_feed_scaled_mm():
    torch.manual_seed(1)
    M, K, N = 256, 512, 384
    a = torch.randn(M, K, dtype=torch.bfloat16, device="cuda")
    b = torch.randn(N, K, dtype=torch.bfloat16, device="cuda")
    ga, gb = Q.nvfp4_gs_scale_cuda(a), Q.nvfp4_gs_scale_cuda(b)
    qa, sa = Q.nvfp4_gs_swizzle_cuda(a, ga)
    qb, sb = Q.nvfp4_gs_swizzle_cuda(b, gb)
    y = _scaled_mm(qa, qb.t(), sa.flatten(), sb.flatten())
    ref = a.float() @ b.float().t()
    got = y.float() * (ga * gb)      # the per-tensor outer scales are applied outside the GEMM
    assert _sqnr(ref, got) > 12.0


def _scaled_grouped_mm(a, b, sa, sb, offs):
    if not hasattr(torch, "_scaled_grouped_mm"):
        pytest.skip("this torch build has no torch._scaled_grouped_mm")
    try:
        return torch._scaled_grouped_mm(a, b, sa, sb, offs=offs, out_dtype=torch.bfloat16)
    except (RuntimeError, NotImplementedError, TypeError) as e:
        pytest.skip(f"torch._scaled_grouped_mm does not take these operands here: {str(e).splitlines()[0][:160]}")


def test_grouped_casts_feed_the_grouped_gemm():
    """The MoE flow of the reference (experiments/quantize_tensor_api/moe_main.py:71-162): token groups of any size,
    padded and cast in one pass, multiplied per expert by torch._scaled_grouped_mm; forward (2d-3d) and weight
    gradient (2d-2d), each against the bf16 product of the same groups."""
    from quant_cast_bench_b200.quant_cast_cuda import quantize_tensor_api as A
    torch.manual_seed(2)
    E, K, N = 4, 256, 384
    ends = [100, 100, 333, 512]                      # one empty group, ragged sizes
    M = ends[-1]
    act = torch.randn(M, K, dtype=torch.bfloat16, device="cuda")
    weight_t = torch.randn(E, K, N, dtype=torch.bfloat16, device="cuda")
    offs = torch.tensor(ends, dtype=torch.int32, device="cuda")

    qa, sa, padded_offs = A.quantize_tensor_grouped_padded(act, offs)                       # (Mp, K), M-groups scales
    wq, ws = A.quantize_tensor(weight_t, orientation=A.QuantOrientation.TRANSPOSED)          # (E, N, K), per-expert scales
    out = _scaled_grouped_mm(qa, wq.transpose(-2, -1), sa, ws, padded_offs)                  # (Mp, N)
    pends = padded_offs.cpu().tolist()
    start, pstart = 0, 0
    for e, end in enumerate(ends):
        size = end - start
        if size:
            ref = act[start:end].float() @ weight_t[e].float()
            got = out[pstart:pstart + size].float()
            assert _sqnr(ref, got) > 25.0, f"forward, expert {e}"
        start, pstart = end, pends[e]

    # weight gradient: grad_output^T @ act per group, both operands cast along the (padded) token dimension
    go = torch.randn(M, N, dtype=torch.bfloat16, device="cuda")
    go_t, go_ts, po2 = A.quantize_tensor_grouped_padded(go, offs, orientation=A.QuantOrientation.TRANSPOSED)   # (N, Mp)
    ia_t, ia_ts, _ = A.quantize_tensor_grouped_padded(act, offs, orientation=A.QuantOrientation.TRANSPOSED)    # (K, Mp)
    gw = _scaled_grouped_mm(go_t, ia_t.transpose(-2, -1), go_ts, ia_ts, po2)                                   # (E, N, K)
    start = 0
    for e, end in enumerate(ends):
        if end > start:
            ref = go[start:end].float().t() @ act[start:end].float()
            assert _sqnr(ref, gw[e].float()) > 25.0, f"weight gradient, expert {e}"
        start = end
