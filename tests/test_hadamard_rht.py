"""The 16-point randomised Hadamard transform and the two-orientation nvfp4 cast on it (gold recipes
`bf16_rht`, `nvfp4_swizzle_dim_k_dim_m_rht`, `nvfp4_swizzle_dim_k_sr_dim_m_rht_sr`;
quant_cast_gold/recipes.py:1324-1438, 1778-1810 of vkuzo/quant_cast_bench) against golden vectors of the
reference and against the CPU oracle, bit for bit.  Kernel and oracle share the accumulation order of the
transform, so they must agree on any input, also where that order matters."""
import pytest
import torch

from helpers import assert_same_bits, golden_cases, golden_out, golden_rht, golden_x, same_outputs
from oracle import gold_port as O
from quant_cast_bench_b200 import quant_cast_cuda as Q
from quant_cast_bench_b200.quant_cast_cuda import _lib as L
from quant_cast_bench_b200.workloads import make_input

pytestmark = pytest.mark.gpu

SIGNS = [[1, -1] * 8, [1, 1, -1, 1, -1, -1, -1, 1, 1, -1, 1, 1, -1, 1, -1, -1], [1] * 16, [-1] * 16]


@pytest.fixture(autouse=True)
def _no_device_error():
    yield
    assert L.device_error() == 0


def _rht(sign):
    return O.hadamard_rht_matrix(torch.tensor(sign, dtype=torch.float32))


def test_matrix_builder():
    for sign in SIGNS:
        assert_same_bits(Q.hadamard_rht_matrix_cuda(torch.tensor(sign)), _rht(sign), "rht matrix")


@pytest.mark.parametrize("tag", golden_cases())
def test_golden(tag):
    x, rht = golden_x(tag), golden_rht(tag)
    xc, rc = x.cuda(), rht.cuda()
    assert_same_bits(Q.hadamard_rht_cuda(xc, rc)[0], golden_out(tag, "hadamard_rht_f", 0), f"rht {tag}")
    gs = Q.nvfp4_gs_scale_cuda(xc)
    gs_m = Q.nvfp4_rht_outer_scale_m_cuda(xc, rc)
    assert_same_bits(gs_m.reshape(1), golden_out(tag, "nvfp4_rht_outer_scale_m", 0), "outer m")
    fn = "nvfp4_gs_swizzle_dim_k_dim_m_rht_f"
    outs = Q.nvfp4_gs_swizzle_dim_k_dim_m_rht_cuda(xc, gs, gs_m, rc)
    assert len(outs) == 4
    for i, o in enumerate(outs):
        assert_same_bits(o, golden_out(tag, fn, i), f"{fn}[{i}] {tag}")
    same_outputs(Q.nvfp4_gs_swizzle_dim_m_rht_cuda(xc, gs_m, rc), outs[2:], "dim-m half alone")


@pytest.mark.parametrize("shape", [(512, 512), (96, 160), (32, 32), (160, 416), (384, 96), (1024, 2048), (2080, 1056)])
@pytest.mark.parametrize("wide", [False, True])
def test_matches_oracle(shape, wide):
    M, N = shape
    x = make_input(M, N, seed=M + N)
    if wide:   # block values 2^40 apart: the sums are inexact in fp32 and the accumulation order shows
        g = torch.Generator().manual_seed(5)
        x = (x.float() * torch.exp2(torch.randint(-20, 20, (M, N), generator=g).float())).to(torch.bfloat16)
    xc = x.cuda()
    for sign in SIGNS[:2] if wide else SIGNS:
        rht = _rht(sign)
        rc = rht.cuda()
        assert_same_bits(Q.hadamard_rht_cuda(xc, rc)[0], O.hadamard_rht_f(x, rht)[0], f"rht {sign}")
        gs = Q.nvfp4_gs_scale_cuda(xc)
        gs_m = Q.nvfp4_rht_outer_scale_m_cuda(xc, rc)
        assert_same_bits(gs_m.reshape(1), O.nvfp4_rht_outer_scale_m(x, rht).reshape(1), "outer m")
        same_outputs(Q.nvfp4_gs_swizzle_dim_k_dim_m_rht_cuda(xc, gs, gs_m, rc),
                     O.nvfp4_gs_swizzle_dim_k_dim_m_rht_f(x, gs.cpu(), gs_m.cpu(), rht), f"rht cast {sign}")
        same_outputs(Q.nvfp4_gs_swizzle_dim_m_rht_cuda(xc, gs_m, rc),
                     O.nvfp4_gs_swizzle_f(O.hadamard_rht_t(x, rht), gs_m.cpu()), f"dim-m alone {sign}")


@pytest.mark.parametrize("shape", [(256, 256), (96, 160), (1024, 512)])
def test_stochastic_rounding_streams(shape):
    x = make_input(*shape, seed=3, spread=0.0, outlier_p=1e-3, outlier_mul=50.0, zero_row_p=0.0)
    xc = x.cuda()
    rht = _rht(SIGNS[1])
    rc = rht.cuda()
    gs = Q.nvfp4_gs_scale_cuda(xc)
    gs_m = Q.nvfp4_rht_outer_scale_m_cuda(xc, rc)
    for (sk_, ok_), (sm_, om_) in (((0, 0), (1, 0)), ((2 ** 40 + 17, 2 ** 33 + 5), (77, 123))):
        got = Q.nvfp4_gs_swizzle_dim_k_dim_m_rht_sr_cuda(xc, gs, gs_m, rc, Q.philox_key(sk_, ok_), Q.philox_key(sm_, om_))
        want = O.nvfp4_gs_swizzle_dim_k_dim_m_rht_sr_f(x, gs.cpu(), gs_m.cpu(), rht, (sk_, ok_), (sm_, om_))
        same_outputs(got, want, f"rht sr {sk_} {sm_}")
    # the dim-k half is the plain stochastic cast; scales do not depend on the rounding mode
    got = Q.nvfp4_gs_swizzle_dim_k_dim_m_rht_sr_cuda(xc, gs, gs_m, rc, Q.philox_key(5), Q.philox_key(6))
    same_outputs(got[:2], Q.nvfp4_gs_swizzle_sr_cuda(xc, gs, Q.philox_key(5)), "dim-k half")
    rne = Q.nvfp4_gs_swizzle_dim_k_dim_m_rht_cuda(xc, gs, gs_m, rc)
    assert_same_bits(got[1], rne[1], "sk")
    assert_same_bits(got[3], rne[3], "sm")


def test_round_trip_sqnr():
    """The reference's own acceptance test for these recipes (G:1336-1353): dequantise both halves, invert the
    transform of the dim-m half with rht.t(), SQNR above 12 dB."""
    M, N = 512, 1024
    xc = torch.randn(M, N, dtype=torch.bfloat16, generator=torch.Generator().manual_seed(0)).cuda()
    rc = Q.hadamard_rht_matrix_cuda(torch.tensor(SIGNS[0]))
    gs, gs_m = Q.nvfp4_gs_scale_cuda(xc), Q.nvfp4_rht_outer_scale_m_cuda(xc, rc)
    qk, sk, qm, sm = Q.nvfp4_gs_swizzle_dim_k_dim_m_rht_cuda(xc, gs, gs_m, rc)
    lut = torch.tensor([0, 0.5, 1, 1.5, 2, 3, 4, 6, -0.0, -0.5, -1, -1.5, -2, -3, -4, -6], device="cuda")

    def dequant(q, s, rows, cols, outer):
        b = q.view(torch.uint8).long()
        v = torch.stack([lut[b & 15], lut[b >> 4]], dim=-1).reshape(rows, cols // 16, 16)
        nrb, ncb = s.shape[0], s.shape[1]
        plain = s.view(torch.uint8).view(nrb, ncb, 32, 4, 4).permute(0, 3, 2, 1, 4).reshape(nrb * 128, ncb * 4)
        inner = plain[:rows, :cols // 16].view(torch.float8_e4m3fn).float()
        return (v * inner.unsqueeze(-1) * outer).reshape(rows, cols)

    def sqnr(a, b):
        return 10 * torch.log10(a.pow(2).sum() / (a - b).pow(2).sum())

    xf = xc.float()
    assert sqnr(xf, dequant(qk, sk, M, N, gs)) > 12.0
    y = dequant(qm, sm, N, M, gs_m)
    x_hat = (y.reshape(N, M // 16, 16) @ rc.float().t()).reshape(N, M).t()
    assert sqnr(xf, x_hat) > 12.0


def test_unsupported_matrix_is_reported():
    xc = make_input(64, 64, seed=0).cuda()
    bad = _rht(SIGNS[0]).clone()
    bad[3, 5] = 0.5
    Q.hadamard_rht_cuda(xc, bad.cuda())
    assert L.device_error() == 17
    with pytest.raises(AssertionError):
        Q.hadamard_rht_cuda(xc, bad.float().cuda())
    with pytest.raises(AssertionError):
        Q.hadamard_rht_cuda(make_input(64, 40, seed=0).cuda(), _rht(SIGNS[0]).cuda())
