"""Seeded sweeps over odd shapes: every cast against the CPU oracle, bit for bit, at sizes that put tile, atom and
group boundaries in unusual places (the reference's tests use 512x512, 96x160 and 128x160 only)."""
import random

import pytest
import torch

from helpers import same_outputs
from oracle import gold_port as O
from quant_cast_bench_b200 import quant_cast_cuda as Q
from quant_cast_bench_b200.quant_cast_cuda import _lib as L
from quant_cast_bench_b200.quant_cast_cuda import quantize_tensor_api as A
from quant_cast_bench_b200.workloads import make_input

pytestmark = pytest.mark.gpu


def _shapes(seed, n, m_step, n_step, m_max=700, n_max=1200):
    rng = random.Random(seed)
    return [(rng.randrange(1, m_max // m_step + 1) * m_step, rng.randrange(1, n_max // n_step + 1) * n_step) for _ in range(n)]


@pytest.fixture(autouse=True)
def _no_device_error():
    yield
    assert L.device_error() == 0


@pytest.mark.parametrize("shape", _shapes(1, 12, 1, 32), ids=str)
def test_rowwise_casts_any_row_count(shape):
    x = make_input(*shape, seed=sum(shape))
    xc = x.cuda()
    for fn in ("rowwise_fp8", "mxfp8", "mxfp8_swizzle", "mxfp4"):
        same_outputs(getattr(Q, fn + "_cuda")(xc), getattr(O, fn + "_f")(x), f"{fn} {shape}")
    gs = Q.nvfp4_gs_scale_cuda(xc)
    same_outputs(Q.nvfp4_gs_cuda(xc, gs), O.nvfp4_gs_f(x, gs.cpu()), f"nvfp4 {shape}")
    same_outputs(Q.nvfp4_gs_swizzle_cuda(xc, gs), O.nvfp4_gs_swizzle_f(x, gs.cpu()), f"nvfp4 swizzle {shape}")
    s = Q.float8_tensorwise_scale_cuda(xc)
    same_outputs(Q.float8_tensorwise_cuda(xc, s), O.float8_tensorwise_f(x, s.cpu()), f"tensorwise {shape}")


@pytest.mark.parametrize("shape", _shapes(2, 12, 32, 32), ids=str)
def test_transposing_casts(shape):
    x = make_input(*shape, seed=sum(shape) + 1)
    xc = x.cuda()
    for fn in ("mxfp8_dim_m", "mxfp8_dim_m_swizzle", "mxfp8_dim_km", "mxfp8_dim_km_swizzle", "mxfp8_32x32", "mxfp8_32x32_swizzle",
               "mxfp8_32x32_dim_m_swizzle", "mxfp8_32x32_dim_km_swizzle", "mxfp8_32x32_qdata_dim_k_scale_dim_km_swizzle"):
        same_outputs(getattr(Q, fn + "_cuda")(xc), getattr(O, fn + "_f")(x), f"{fn} {shape}")
    for mode in ("floor",):
        same_outputs(Q.mxfp8_dim_km_swizzle_cuda(xc, mode=mode), O.mxfp8_dim_km_swizzle_f(x, mode=mode), f"floor {shape}")
    gs = Q.nvfp4_gs_scale_cuda(xc)
    same_outputs(Q.nvfp4_gs_swizzle_t_cuda(xc, gs), O.nvfp4_gs_swizzle_t_f(x, gs.cpu()), f"nvfp4 transposed {shape}")
    same_outputs(Q.nvfp4_gs_swizzle_both_cuda(xc, gs), O.nvfp4_gs_swizzle_f(x, gs.cpu()) + O.nvfp4_gs_swizzle_t_f(x, gs.cpu()),
                 f"nvfp4 both {shape}")
    same_outputs(Q.colwise_fp8_cuda(xc), O.colwise_fp8_f(x), f"colwise {shape}")


@pytest.mark.parametrize("shape", _shapes(3, 8, 128, 128, 640, 1024), ids=str)
def test_128_blocks(shape):
    x = make_input(*shape, seed=sum(shape) + 2)
    xc = x.cuda()
    for fn in ("deepseek_1x128", "deepseek_1x128_dim_m", "deepseek_1x128_dim_km", "deepseek_128x128"):
        same_outputs(getattr(Q, fn + "_cuda")(xc), getattr(O, fn + "_f")(x), f"{fn} {shape}")
    ob = Q.nvfp4_blocked_outer_scale_cuda(xc)
    ob = torch.where(ob == 0, torch.full_like(ob, 2.0 ** -100), ob)
    same_outputs(Q.nvfp4_blocked_outer_cuda(xc, ob), O.nvfp4_blocked_outer_f(x, ob.cpu()), f"blocked outer {shape}")


@pytest.mark.parametrize("seed", range(10))
def test_random_token_groups(seed):
    rng = random.Random(100 + seed)
    G = rng.randrange(1, 9)
    sizes = [rng.choice([0, 1, 5, 31, 32, 33, 64, 100, 127, 128, 200]) for _ in range(G)]
    if sum(sizes) == 0:
        sizes[-1] = 17
    M = sum(sizes)
    C = rng.choice([128, 256, 384])
    ends, acc = [], 0
    for sz in sizes:
        acc += sz
        ends.append(acc)
    x = make_input(M, C, seed=seed)
    offs = torch.tensor(ends, dtype=torch.int32)
    padded, _, pends = O.pad_token_groups(x, offs)
    want = O.quantize_grouped(padded, pends)
    got = A.quantize_tensor_grouped_padded_bidirectional(x.cuda(), offs.cuda())
    same_outputs(got[:4], want, f"groups {sizes} C={C}")
    assert got[4].cpu().tolist() == pends.tolist()
    pt, _, po = A.pad_token_groups(x.cuda(), offs.cuda())
    same_outputs((pt,), (padded,), "padded copy")
    same_outputs((A.unpad_token_groups(pt, offs.cuda()),), (x,), "unpad")


@pytest.mark.parametrize("shape", [(66304, 128), (66320, 64), (40000, 200), (16, 8), (9472, 1096), (148 * 7 * 64, 72)], ids=str)
def test_colwise_tall_and_ragged(shape):
    """fp8 colwise at the edges of its one-launch form: the tallest matrix it takes (66304 rows = 148 SMs x 7 tiles of
    64 rows), one that is 16 rows taller (two-launch form), a last panel that is cut by the matrix edge, and row counts
    that leave some CTAs without tiles."""
    x = make_input(*shape, seed=shape[0] + shape[1])
    xc = x.cuda()
    for fmt in ("e4m3", "e5m2"):
        same_outputs(Q.colwise_fp8_cuda(xc, fmt), O.colwise_fp8_f(x, fmt), f"colwise {fmt} {shape}")
