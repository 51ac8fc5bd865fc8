"""The benchmark configurations at their FULL sizes.  The CPU oracle cannot cast 10^9 elements in test time, so
the full-size outputs are checked through properties that do not depend on the size:

* row-tile invariance (the tiling contract of flex_tile_map/recipes.py:137-179 of vkuzo/quant_cast_bench): the
  bytes that a 128-row slab of the input produces inside the full-size outputs equal the oracle's outputs for
  that slab alone -- bit for bit, at the first, a middle and the last slab (per-tensor scales are handed over);
* the reference's own acceptance test: dequantised outputs recover the input above the SQNR floor of the
  recipe (quant_cast_gold/recipes.py:129 fp8 20 dB, :590 mxfp8 15 dB, :1294 nvfp4 12 dB);
* determinism: a second call returns the same bytes;
* the blocked scale grids hold zeros in every padding slot.
"""
import pytest
import torch

from helpers import assert_same_bits
from oracle import gold_port as O
from quant_cast_bench_b200 import quant_cast_cuda as Q
from quant_cast_bench_b200.workloads import config_input_device

pytestmark = pytest.mark.gpu


def _slabs(M):
    return [0, (M // 2 // 128) * 128, M - 128]


def _sqnr(x, y):
    return float(20 * torch.log10(torch.linalg.vector_norm(x) / torch.linalg.vector_norm(x - y)))


def _unblock(s, H, W):
    """(nrb, ncb, 32, 16) blocked grid -> (H, W) bytes, on the device."""
    nrb, ncb = s.shape[0], s.shape[1]
    return s.view(torch.uint8).view(nrb, ncb, 32, 4, 4).permute(0, 3, 2, 1, 4).reshape(nrb * 128, ncb * 4)[:H, :W]


def _e8m0(b):
    return torch.exp2(b.float() - 127.0)


def _sqnr_rows(x, dequant_rows, chunk=4096):
    """SQNR over the whole matrix, accumulated over row chunks to bound the fp32 temporaries."""
    num = den = 0.0
    for r0 in range(0, x.shape[0], chunk):
        xf = x[r0:r0 + chunk].float()
        num += float(xf.pow(2).sum(dtype=torch.float64))
        den += float((xf - dequant_rows(r0, min(r0 + chunk, x.shape[0]))).pow(2).sum(dtype=torch.float64))
    return 10 * torch.log10(torch.tensor(num / den)).item()


def test_c1_fp8_4096():
    x = config_input_device("c1_fp8_4096", "cuda")
    M, N = x.shape
    s = Q.float8_tensorwise_scale_cuda(x)
    (q,) = Q.float8_tensorwise_cuda(x, s)
    qr, sr = Q.rowwise_fp8_cuda(x)
    assert_same_bits(s.reshape(1), O.float8_tensorwise_scale(x.cpu()).reshape(1), "tensor scale at full size")
    for r0 in _slabs(M):
        xs = x[r0:r0 + 128].cpu()
        assert_same_bits(q[r0:r0 + 128], O.float8_tensorwise_f(xs, s.cpu())[0], f"tensorwise slab {r0}")
        wq, ws = O.rowwise_fp8_f(xs)
        assert_same_bits(qr[r0:r0 + 128], wq, f"rowwise slab {r0}")
        assert_same_bits(sr[r0:r0 + 128], ws, f"rowwise scale slab {r0}")
    assert _sqnr(x.float(), qr.float() * sr) > 20.0
    assert torch.equal(Q.rowwise_fp8_cuda(x)[0].view(torch.uint8), qr.view(torch.uint8))
    assert int(q.view(torch.uint8).bitwise_and(0x7F).max()) <= 0x7E     # saturating: never the NaN code


@pytest.mark.parametrize("mode", ["rceil", "floor"])
def test_c2_mxfp8_16384(mode):
    x = config_input_device("c2_mxfp8_16384", "cuda")
    M, N = x.shape
    qk, sk, qm, sm = Q.mxfp8_dim_km_swizzle_cuda(x, mode=mode)
    pk, psk, pm, psm = Q.mxfp8_dim_km_cuda(x, mode=mode)
    for r0 in _slabs(M):
        want = O.mxfp8_dim_km_swizzle_f(x[r0:r0 + 128].cpu(), mode=mode)
        assert_same_bits(qk[r0:r0 + 128], want[0], f"qk slab {r0}")
        assert_same_bits(sk[r0 // 128], want[1][0], f"sk slab {r0}")
        assert_same_bits(qm[:, r0:r0 + 128], want[2], f"qm slab {r0}")
        assert_same_bits(sm[:, r0 // 128], want[3][:, 0], f"sm slab {r0}")
    # the plain layouts carry the same bytes as the blocked ones
    assert torch.equal(pk.view(torch.uint8), qk.view(torch.uint8)) and torch.equal(pm.view(torch.uint8), qm.view(torch.uint8))
    assert torch.equal(_unblock(sk, M, N // 32), psk.view(torch.uint8))
    assert torch.equal(_unblock(sm, N, M // 32), psm.view(torch.uint8))
    # single-direction casts give the same outputs as the fused one
    q1, s1 = Q.mxfp8_swizzle_cuda(x, mode=mode)
    assert torch.equal(q1.view(torch.uint8), qk.view(torch.uint8)) and torch.equal(s1.view(torch.uint8), sk.view(torch.uint8))
    q2, s2 = Q.mxfp8_dim_m_swizzle_cuda(x, mode=mode)
    assert torch.equal(q2.view(torch.uint8), qm.view(torch.uint8)) and torch.equal(s2.view(torch.uint8), sm.view(torch.uint8))
    del q1, s1, q2, s2, pk, pm
    if mode == "rceil":
        sc = _e8m0(psk.view(torch.uint8))
        assert _sqnr_rows(x, lambda a, b: (qk[a:b].float().view(b - a, N // 32, 32) * sc[a:b].unsqueeze(-1)).view(b - a, N)) > 15.0
        scm = _e8m0(psm.view(torch.uint8))      # (N, M/32)
        xt_sqnr = _sqnr_rows(x, lambda a, b: (qm[:, a:b].float().view(N, (b - a) // 32, 32)
                                              * scm[:, a // 32:b // 32].unsqueeze(-1)).view(N, b - a).t())
        assert xt_sqnr > 15.0


def test_c3_nvfp4_8192():
    x = config_input_device("c3_nvfp4_8192", "cuda")
    M, N = x.shape
    gs = Q.nvfp4_gs_scale_cuda(x)
    assert_same_bits(gs.reshape(1), O.nvfp4_gs_scale(x.cpu()).reshape(1), "outer scale at full size")
    q, s = Q.nvfp4_gs_swizzle_cuda(x, gs)
    qt, st = Q.nvfp4_gs_swizzle_t_cuda(x, gs)
    qp, sp = Q.nvfp4_gs_cuda(x, gs)
    for r0 in _slabs(M):
        xs = x[r0:r0 + 128].cpu()
        wq, ws = O.nvfp4_gs_swizzle_f(xs, gs.cpu())
        assert_same_bits(q[r0:r0 + 128], wq, f"q slab {r0}")
        assert_same_bits(s[r0 // 128], ws[0], f"s slab {r0}")
        wqt, wst = O.nvfp4_gs_swizzle_t_f(xs, gs.cpu())
        assert_same_bits(qt[:, r0 // 2:r0 // 2 + 64], wqt, f"transposed q slab {r0}")
        assert_same_bits(st[:, r0 // 64:r0 // 64 + 2], wst, f"transposed s slab {r0}")
    assert torch.equal(qp.view(torch.uint8), q.view(torch.uint8))
    assert torch.equal(_unblock(s, M, N // 16), sp.view(torch.uint8))
    lut = torch.tensor([0, 0.5, 1, 1.5, 2, 3, 4, 6, -0.0, -0.5, -1, -1.5, -2, -3, -4, -6], device="cuda")
    b = qp.view(torch.uint8).long()
    v = torch.stack([lut[b & 15], lut[b >> 4]], dim=-1).reshape(M, N // 16, 16)
    x_hat = (v * sp.float().unsqueeze(-1) * gs).reshape(M, N)
    assert _sqnr(x.float(), x_hat) > 12.0


def test_c4_moe_131072x7168():
    x = config_input_device("c4_moe_131072x7168", "cuda")
    M, N = x.shape
    gs = Q.nvfp4_gs_scale_cuda(x)
    q8, s8 = Q.mxfp8_swizzle_cuda(x)
    q4, s4 = Q.nvfp4_gs_swizzle_cuda(x, gs)
    for r0 in _slabs(M):
        xs = x[r0:r0 + 128].cpu()
        w8 = O.mxfp8_swizzle_f(xs)
        assert_same_bits(q8[r0:r0 + 128], w8[0], f"mxfp8 slab {r0}")
        assert_same_bits(s8[r0 // 128], w8[1][0], f"mxfp8 scale slab {r0}")
        w4 = O.nvfp4_gs_swizzle_f(xs, gs.cpu())
        assert_same_bits(q4[r0:r0 + 128], w4[0], f"nvfp4 slab {r0}")
        assert_same_bits(s4[r0 // 128], w4[1][0], f"nvfp4 scale slab {r0}")
    del q8, s8, q4, s4
    # both orientations of the whole activation (3.8 GB of outputs): halves concatenate to the whole
    qk, sk, qm, sm = Q.mxfp8_dim_km_swizzle_cuda(x)
    h = M // 2
    ak, ask, am, asm_ = Q.mxfp8_dim_km_swizzle_cuda(x[:h])
    assert torch.equal(qk[:h].view(torch.uint8), ak.view(torch.uint8)) and torch.equal(sk[:h // 128].view(torch.uint8), ask.view(torch.uint8))
    assert torch.equal(qm[:, :h].view(torch.uint8), am.view(torch.uint8))
    assert torch.equal(sm[:, :h // 128].view(torch.uint8), asm_.view(torch.uint8))
    # N / 32 = 224 scale columns = 56 whole atoms; M / 32 = 4096: no padding anywhere, N = 7168 = 56 * 128
    assert sk.shape == (M // 128, N // 128, 32, 16) and sm.shape == (N // 128, M // 128, 32, 16)


def test_c5_nvfp4_sr_8192x16384():
    x = config_input_device("c5_nvfp4_sr_8192x16384", "cuda")
    M, N = x.shape
    gs = Q.nvfp4_gs_scale_cuda(x)
    q0, s0 = Q.nvfp4_gs_swizzle_cuda(x, gs)
    lut = torch.tensor([0, 0.5, 1, 1.5, 2, 3, 4, 6, -0.0, -0.5, -1, -1.5, -2, -3, -4, -6], device="cuda")
    inner = _unblock(s0, M, N // 16).view(torch.float8_e4m3fn).float()
    mean = torch.zeros(M, N, device="cuda")
    for seed in range(16):
        q, s = Q.nvfp4_gs_swizzle_sr_cuda(x, gs, Q.philox_key(seed))
        assert torch.equal(s.view(torch.uint8), s0.view(torch.uint8)), "scales must not depend on the rounding mode"
        if seed < 2:   # bit-exact against the oracle's stream on the first and the last slab
            for r0 in (0, M - 128):
                # the stream is indexed by the position in the whole tensor: offset = first element / 4
                want = O.nvfp4_gs_swizzle_sr_f(x[r0:r0 + 128].cpu(), gs.cpu(), (seed, r0 * N // 4))
                assert_same_bits(q[r0:r0 + 128], want[0], f"sr slab {r0} seed {seed}")
        b = q.view(torch.uint8).long()
        v = torch.stack([lut[b & 15], lut[b >> 4]], dim=-1).reshape(M, N // 16, 16)
        mean += (v * inner.unsqueeze(-1) * gs).reshape(M, N)
    mean /= 16
    xf = x.float()
    rel = float((mean - xf).sum().abs() / xf.abs().sum())
    assert rel <= 1e-3, f"mean error of 16 seeds {rel:.2e}"


def test_addressing_beyond_2_31_elements():
    """131072 x 16384 = 2^31 elements (4 GiB of bf16): byte offsets of every output pass 2^31, element offsets of the
    input pass 2^31 - 1.  Slabs at the far end must still match the oracle."""
    from quant_cast_bench_b200.workloads import make_input_device
    M, N = 131072, 16384
    x = make_input_device(M, N, seed=9, device="cuda", spread=4.0, outlier_p=0.0, zero_row_p=0.0)
    qk, sk, qm, sm = Q.mxfp8_dim_km_swizzle_cuda(x)
    for r0 in (0, M - 128):
        want = O.mxfp8_dim_km_swizzle_f(x[r0:r0 + 128].cpu())
        assert_same_bits(qk[r0:r0 + 128], want[0], f"qk slab {r0}")
        assert_same_bits(sk[r0 // 128], want[1][0], f"sk slab {r0}")
        assert_same_bits(qm[:, r0:r0 + 128], want[2], f"qm slab {r0}")
        assert_same_bits(sm[:, r0 // 128], want[3][:, 0], f"sm slab {r0}")
    del qk, sk, qm, sm
    gs = Q.nvfp4_gs_scale_cuda(x)
    q4, s4 = Q.nvfp4_gs_swizzle_cuda(x, gs)
    qt, st = Q.nvfp4_gs_swizzle_t_cuda(x, gs)
    r0 = M - 128
    xs = x[r0:].cpu()
    w = O.nvfp4_gs_swizzle_f(xs, gs.cpu())
    assert_same_bits(q4[r0:], w[0], "nvfp4 last slab")
    assert_same_bits(s4[r0 // 128], w[1][0], "nvfp4 scale last slab")
    wt = O.nvfp4_gs_swizzle_t_f(xs, gs.cpu())
    assert_same_bits(qt[:, r0 // 2:], wt[0], "nvfp4 transposed last slab")
    assert_same_bits(st[:, r0 // 64:], wt[1], "nvfp4 transposed scale last slab")
    (q8,) = Q.float8_tensorwise_cuda(x, Q.float8_tensorwise_scale_cuda(x))
    assert_same_bits(q8[r0:], O.float8_tensorwise_f(xs, Q.float8_tensorwise_scale_cuda(x).cpu())[0], "tensorwise last slab")
    # shapes past the 32-bit block counters are refused before anything is launched (no memory is touched: the
    # pointers only have to be non-null and aligned)
    from quant_cast_bench_b200.quant_cast_cuda import _lib as L
    lib = L.load()
    p = x.data_ptr()
    big_m = (1 << 32) // (N // 32) + 128
    assert lib.qcc_mxfp8(p, big_m, N, L.ROWWISE, p, p, None, None, None) == -1          # QCC_ERR_SHAPE
    assert lib.qcc_nvfp4(p, (1 << 32) // (N // 16) + 128, N, p, 0, 0, None, p, p, None) == -1
    assert lib.qcc_fp8_block128(p, big_m, N, L.ROWWISE, p, p, None, None, None) == -1


@pytest.mark.parametrize("config", ["c2_mxfp8_16384", "c3_nvfp4_8192", "c4_moe_131072x7168"])
def test_fp8_colwise_full_size(config):
    """fp8 colwise is invariant under COLUMN slabs (every column has its own scale): 128 columns of the full-size
    outputs equal the oracle's outputs for those columns alone, all rows included."""
    x = config_input_device(config, "cuda")
    M, N = x.shape
    q, s = Q.colwise_fp8_cuda(x)
    q2, s2 = Q.colwise_fp8_cuda(x)
    assert torch.equal(q.view(torch.uint8), q2.view(torch.uint8)) and torch.equal(s, s2), "colwise is not deterministic"
    for c0 in (0, (N // 2 // 128) * 128, N - 128):
        qo, so = O.colwise_fp8_f(x[:, c0:c0 + 128].contiguous().cpu())
        assert_same_bits(q[c0:c0 + 128], qo, f"colwise q, columns {c0}..")
        assert_same_bits(s[c0:c0 + 128], so, f"colwise scale, columns {c0}..")
    # every column's scale by gold's formula (the division on the CPU: torch's CUDA kernel multiplies by 1/448 instead)
    amax = x.abs().amax(dim=0).clamp(min=1e-12).float().cpu()
    assert torch.equal(s.reshape(-1).cpu(), amax / 448.0)
