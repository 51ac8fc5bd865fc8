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
