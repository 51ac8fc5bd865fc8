"""The `quantize_tensor` dispatch against the CPU oracle: every supported (scaling, orientation, swizzle)
combination of the reference's table (experiments/quantize_tensor_api/api.py:76-298, tested there by
test_dense.py) plus the additions of this backend, and the errors for unsupported ones."""
import pytest
import torch

from helpers import same_outputs, assert_same_bits
from oracle import gold_port as O
from quant_cast_bench_b200 import quant_cast_cuda as Q
from quant_cast_bench_b200.quant_cast_cuda import quantize_tensor_api as A
from quant_cast_bench_b200.quant_cast_cuda import _lib as L
from quant_cast_bench_b200.workloads import make_input

pytestmark = pytest.mark.gpu
SW, NOSW = A.SwizzleType.SWIZZLE_32_4_4, A.SwizzleType.NO_SWIZZLE
NAT, TR = A.QuantOrientation.NATURAL, A.QuantOrientation.TRANSPOSED


def test_mxfp8_table():
    x = make_input(256, 384, seed=3)
    xc = x.cuda()
    for orient, swz, ofn in ((NAT, NOSW, O.mxfp8_f), (NAT, SW, O.mxfp8_swizzle_f), (TR, NOSW, O.mxfp8_dim_m_f), (TR, SW, O.mxfp8_dim_m_swizzle_f)):
        same_outputs(A.quantize_tensor(xc, orientation=orient, swizzle_type=swz), ofn(x), f"{orient} {swz}")
        same_outputs(A.quantize_tensor(xc, orientation=orient, swizzle_type=swz, inner_scale_calc=A.InnerScaleCalc.E8M0_FLOOR),
                     ofn(x, mode="floor"), f"floor {orient} {swz}")
    same_outputs(A.quantize_tensor_bidirectional(xc, swizzle_type=SW), O.mxfp8_dim_km_swizzle_f(x), "bidirectional swizzle")
    same_outputs(A.quantize_tensor_bidirectional(xc, swizzle_type=NOSW), O.mxfp8_dim_km_f(x), "bidirectional plain")


def test_nvfp4_table():
    x = make_input(256, 384, seed=4)
    xc = x.cuda()
    gs = Q.nvfp4_gs_scale_cuda(xc)
    kw = dict(qdata_dtype=torch.float4_e2m1fn_x2, inner_scale_calc=A.InnerScaleCalc.E4M3_NVFP4, scaling_type=A.ScalingType.BlockWise1x16)
    same_outputs(A.quantize_tensor(xc, outer_scale=gs, swizzle_type=SW, **kw), O.nvfp4_gs_swizzle_f(x, gs.cpu()), "nvfp4 swizzle")
    same_outputs(A.quantize_tensor(xc, outer_scale=gs, swizzle_type=NOSW, **kw), O.nvfp4_gs_f(x, gs.cpu()), "nvfp4 plain")
    same_outputs(A.quantize_tensor(xc, outer_scale=gs, swizzle_type=SW, orientation=TR, **kw), O.nvfp4_gs_swizzle_t_f(x, gs.cpu()), "nvfp4 transposed")
    pt = (x.float().abs().amax(dim=1, keepdim=True).clamp(min=2.0 ** -100) / 2688.0)
    same_outputs(A.quantize_tensor(xc, outer_scale=pt.cuda(), swizzle_type=NOSW, **kw), O.nvfp4_gs_f(x, pt), "nvfp4 per-token")
    key = Q.philox_key(7)
    same_outputs(A.quantize_tensor(xc, outer_scale=gs, swizzle_type=SW, rounding_mode=A.RoundingMode.STOCHASTIC, random_key=key, **kw),
                 O.nvfp4_gs_swizzle_sr_f(x, gs.cpu(), (7, 0)), "nvfp4 stochastic")
    same_outputs(A.quantize_tensor_bidirectional(xc, outer_scale=gs, swizzle_type=SW, **kw),
                 O.nvfp4_gs_swizzle_f(x, gs.cpu()) + O.nvfp4_gs_swizzle_t_f(x, gs.cpu()), "nvfp4 bidirectional")


def test_32x32_and_mxfp4_table():
    x = make_input(256, 384, seed=6)
    xc = x.cuda()
    b32 = dict(scaling_type=A.ScalingType.BlockWise32x32)
    same_outputs(A.quantize_tensor(xc, swizzle_type=NOSW, **b32), O.mxfp8_32x32_f(x), "32x32 plain")
    same_outputs(A.quantize_tensor(xc, swizzle_type=SW, **b32), O.mxfp8_32x32_swizzle_f(x), "32x32 swizzle")
    same_outputs(A.quantize_tensor(xc, swizzle_type=SW, orientation=TR, **b32), O.mxfp8_32x32_dim_m_swizzle_f(x), "32x32 transposed")
    same_outputs(A.quantize_tensor_bidirectional(xc, **b32), O.mxfp8_32x32_dim_km_swizzle_f(x), "32x32 bidirectional")
    same_outputs(A.quantize_tensor_bidirectional(xc, skip_transposed_qdata=True, **b32),
                 O.mxfp8_32x32_qdata_dim_k_scale_dim_km_swizzle_f(x), "32x32 skip transposed qdata")
    with pytest.raises(ValueError):
        A.quantize_tensor(xc, swizzle_type=NOSW, orientation=TR, **b32)
    with pytest.raises(ValueError):
        A.quantize_tensor_bidirectional(xc, skip_transposed_qdata=True)
    fp4 = dict(qdata_dtype=torch.float4_e2m1fn_x2, inner_scale_calc=A.InnerScaleCalc.E8M0_RCEIL)
    same_outputs(A.quantize_tensor(xc, swizzle_type=NOSW, **fp4), O.mxfp4_f(x), "mxfp4")
    same_outputs(A.quantize_tensor(xc, swizzle_type=SW, **fp4), O.mxfp4_f(x, swizzle=True), "mxfp4 swizzle")
    with pytest.raises(ValueError):
        A.quantize_tensor(xc, orientation=TR, **fp4)


@pytest.mark.parametrize("E,M,K", [(3, 160, 256),      # ragged experts: one launch per expert
                                   (4, 256, 384),      # whole 128-row atoms: the stack is cast by one launch
                                   (5, 128, 160),      # ... with a ragged column count
                                   (2, 1024, 2048)])
def test_per_expert_3d(E, M, K):
    x = make_input(E * M, K, seed=5).reshape(E, M, K)
    xc = x.cuda()
    q, s = A.quantize_tensor(xc)
    assert q.shape == (E, M, K) and s.shape[0] == E and s.dim() == 2
    qt, st = A.quantize_tensor(xc, orientation=TR)
    qk, sk, qm, sm = A.quantize_tensor_bidirectional(xc)
    for e in range(E):
        wq, ws = O.mxfp8_swizzle_f(x[e].contiguous())
        assert_same_bits(q[e], wq, f"expert {e} q")
        assert_same_bits(s[e], ws.reshape(-1), f"expert {e} scale")
        wqt, wst = O.mxfp8_dim_m_swizzle_f(x[e].contiguous())
        assert_same_bits(qt[e], wqt, f"expert {e} transposed q")
        assert_same_bits(st[e], wst.reshape(-1), f"expert {e} transposed scale")
        assert_same_bits(qk[e], wq, "bidir qk"); assert_same_bits(sk[e], ws.reshape(-1), "bidir sk")
        assert_same_bits(qm[e], wqt, "bidir qm"); assert_same_bits(sm[e], wst.reshape(-1), "bidir sm")
    fl = A.InnerScaleCalc.E8M0_FLOOR
    qk, sk, qm, sm = A.quantize_tensor_bidirectional(xc, inner_scale_calc=fl)
    for e in range(E):
        want = O.mxfp8_dim_km_swizzle_f(x[e].contiguous(), mode="floor")
        for got, w in zip((qk[e], sk[e], qm[e], sm[e]), want):
            assert_same_bits(got, w.reshape(got.shape), f"floor expert {e}")


def test_unsupported_combinations_raise():
    x = torch.randn(64, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError):
        A.quantize_tensor(x, scaling_type=A.ScalingType.BlockWise128x128)
    with pytest.raises(ValueError):
        A.quantize_tensor(x, rounding_mode=A.RoundingMode.STOCHASTIC)
    with pytest.raises(AssertionError):
        A.quantize_tensor(x, qdata_dtype=torch.float4_e2m1fn_x2, inner_scale_calc=A.InnerScaleCalc.E4M3_NVFP4,
                          scaling_type=A.ScalingType.BlockWise1x16)            # no outer_scale
    with pytest.raises(ValueError):   # only with 32x32 blocks
        A.quantize_tensor_bidirectional(x, skip_transposed_qdata=True)
    with pytest.raises(ValueError):
        A.quantize_tensor(x.reshape(1, 64, 64), swizzle_type=NOSW)


@pytest.mark.parametrize("M,C,ends", [
    (512, 256, [128, 256, 512]),              # groups on 128-row boundaries
    (384, 384, [32, 32, 160, 384]),           # ragged groups and an empty one
    (256, 160, [64, 256]),                    # C not a multiple of 128: transposed orientation only
    (1024, 512, [0, 96, 96, 608, 1024]),      # empty first group, groups that straddle 128-row atoms
])
def test_token_groups(M, C, ends):
    """quantize_tensor_grouped{,_bidirectional} (experiments/quantize_tensor_api/api.py:301-411): data as the
    ungrouped cast, scales blocked per group (moe_utils.py:62-128; the layout functions are pinned against the
    reference's in the CPU suite)."""
    x = make_input(M, C, seed=M + C)
    xc = x.cuda()
    offs = torch.tensor(ends, dtype=torch.int32)
    for mode, calc in (("rceil", A.InnerScaleCalc.E8M0_RCEIL), ("floor", A.InnerScaleCalc.E8M0_FLOOR)):
        if C % 128:
            wq, ws = O.mxfp8_dim_m_f(x, mode=mode)
            same_outputs(A.quantize_tensor_grouped(xc, offs.cuda(), orientation=TR, inner_scale_calc=calc),
                         (wq, O.to_blocked_2d_k_groups(ws, offs // 32)), f"grouped transposed {mode}")
            with pytest.raises(AssertionError):
                A.quantize_tensor_grouped(xc, offs.cuda(), inner_scale_calc=calc)
            continue
        want = O.quantize_grouped(x, offs, mode)
        got = A.quantize_tensor_grouped_bidirectional(xc, offs.cuda(), inner_scale_calc=calc)
        same_outputs(got, want, f"grouped bidirectional {mode}")
        same_outputs(A.quantize_tensor_grouped(xc, offs.cuda(), inner_scale_calc=calc), want[:2], f"grouped natural {mode}")
        same_outputs(A.quantize_tensor_grouped(xc, offs.cuda(), orientation=TR, inner_scale_calc=calc), want[2:],
                     f"grouped transposed {mode}")


def test_token_groups_errors():
    xc = make_input(128, 128, seed=1).cuda()
    offs = torch.tensor([128], dtype=torch.int32).cuda()
    with pytest.raises(ValueError):
        A.quantize_tensor_grouped(xc, offs, swizzle_type=NOSW)
    with pytest.raises(NotImplementedError):
        A.quantize_tensor_grouped_bidirectional(xc, offs, skip_transposed_qdata=True)
    # offsets live on the device and are checked there: bad ones (a group that is not a multiple of 32 rows,
    # a last end other than total_M, descending ends) write no scale and raise the device error word
    want_q = O.mxfp8_f(make_input(128, 128, seed=1))[0]
    for ends in ([48, 128], [96, 64, 128], [128, 160]):
        assert L.device_error() == 0
        q, s = A.quantize_tensor_grouped(xc, torch.tensor(ends, dtype=torch.int32).cuda())
        assert L.device_error() == 16, ends
        assert_same_bits(q, want_q, f"data with bad offsets {ends}")
        assert int(s.view(torch.uint8).max()) == 0
    assert L.device_error() == 0


PAD_CASES = [
    (100, 128, [7, 7, 40, 100]),          # ragged groups, an empty one
    (0, 128, [0, 0, 0]),                  # a rank that received no tokens (expert parallelism)
    (64, 256, [64]),                      # one aligned group
    (131, 128, [1, 33, 131]),             # a one-row group
    (1000, 384, [0, 250, 250, 777, 1000]),
    (4096, 512, [1000, 2047, 2048, 4096]),
]


@pytest.mark.parametrize("M,C,ends", PAD_CASES)
def test_pad_token_groups(M, C, ends):
    """The padded copy itself (moe_utils.py:35-59), for bf16 and for a 16-byte-row byte tensor."""
    x = make_input(M, C, seed=M)
    offs = torch.tensor(ends, dtype=torch.int32)
    want, wstarts, wends = O.pad_token_groups(x, offs)
    got, starts, pends = A.pad_token_groups(x.cuda(), offs.cuda())
    assert_same_bits(got, want, "padded tokens")
    assert starts.cpu().tolist() == wstarts.tolist() and pends.cpu().tolist() == wends.tolist()
    assert_same_bits(A.unpad_token_groups(got, offs.cuda()), x, "unpad(pad(x))")
    assert L.device_error() == 0


@pytest.mark.parametrize("M,C,ends", PAD_CASES)
def test_token_groups_padded_by_the_cast(M, C, ends):
    """quantize_tensor_grouped(_pad_token_groups(x, offs)) in one pass: same bytes as padding first."""
    x = make_input(M, C, seed=M + 1)
    offs = torch.tensor(ends, dtype=torch.int32)
    padded, _, pends = O.pad_token_groups(x, offs)
    for mode, calc in (("rceil", A.InnerScaleCalc.E8M0_RCEIL), ("floor", A.InnerScaleCalc.E8M0_FLOOR)):
        want = O.quantize_grouped(padded, pends, mode)
        got = A.quantize_tensor_grouped_padded_bidirectional(x.cuda(), offs.cuda(), inner_scale_calc=calc)
        same_outputs(got[:4], want, f"padded grouped bidirectional {mode}")
        assert got[4].cpu().tolist() == pends.tolist()
        nat = A.quantize_tensor_grouped_padded(x.cuda(), offs.cuda(), inner_scale_calc=calc)
        same_outputs(nat[:2], want[:2], f"padded grouped natural {mode}")
        tr = A.quantize_tensor_grouped_padded(x.cuda(), offs.cuda(), orientation=TR, inner_scale_calc=calc)
        same_outputs(tr[:2], want[2:], f"padded grouped transposed {mode}")
        # and equal to the two-step route through this backend
        p2, _, po2 = A.pad_token_groups(x.cuda(), offs.cuda())
        same_outputs(A.quantize_tensor_grouped_bidirectional(p2, po2, inner_scale_calc=calc), got[:4], "two-step route")
    assert L.device_error() == 0


def test_padded_groups_bad_offsets():
    xc = make_input(128, 128, seed=1).cuda()
    for ends in ([64, 32, 128], [64, 100], [64, 200]):
        out = A.quantize_tensor_grouped_padded(xc, torch.tensor(ends, dtype=torch.int32).cuda())
        assert L.device_error() == 16, ends
        assert int(out[1].view(torch.uint8).max()) == 0 and out[2].cpu().tolist() == [0] * len(ends)
