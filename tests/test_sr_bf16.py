"""fp32 -> bf16 stochastic rounding (`fp32_to_bf16_sr`, `fp32_to_bf16_sr_global_offsets`; gold sr_bf16_f G:1841-1851,
sr_bf16_global_f G:1887-1914).

The reference draws its dither from `torch.func._random`, which the installed PyTorch does not have, so the VALUES of the
draw are this backend's own Philox4x32-10 stream (pinned by the Random123 known-answer vectors elsewhere); what the
reference defines -- the dither-then-truncate arithmetic, the two-neighbours / unbiasedness property its own
correctness function checks, and tile invariance of the globally keyed form -- is checked here for the oracle (CPU)
and for the kernel against the oracle (GPU), bit for bit."""
import pytest
import torch

from helpers import assert_same_bits
from oracle import gold_port as O


def _key(seed, offset=0):
    return torch.tensor([seed, offset], dtype=torch.int64)


def test_oracle_is_the_gold_arithmetic_on_the_backends_philox_words():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(37, 52, generator=g) * 100
    key = _key(11, 5)
    (out,) = O.sr_bf16_f(x, key)
    n = x.numel()
    words = torch.tensor([O.philox4x32_10([c + 5, 0, 0, 0], [11, 0]) for c in range((n + 7) // 8)], dtype=torch.int64)   # counter = call index + offset, key = seed: one call per eight elements
    pieces = torch.stack([words & 0xFFFF, words >> 16], dim=-1).reshape(-1)[:n]             # low half first, word by word
    rand16 = pieces.to(torch.int32).reshape(x.shape)
    want = ((x.contiguous().view(torch.int32) + rand16) & -65536).view(torch.float32).to(torch.bfloat16)   # _sr_bf16_dither, G:1828-1838
    assert_same_bits(out, want, "oracle vs gold arithmetic")


def test_oracle_two_neighbours_and_unbiased():
    """The reference's own check (_sr_bf16_unbiased_correctness, G:1854-1869) on its own example input."""
    v = 1.0 + 0.003
    x = torch.full((512, 512), v, dtype=torch.float32)
    (out,) = O.sr_bf16_f(x, _key(0))
    lo, hi = 1.0, 1.0 + 2.0 ** -7
    assert set(out.float().unique().tolist()) == {lo, hi}
    assert abs(out.float().mean().item() - v) < 1e-3


def test_oracle_global_keying_is_tile_invariant():
    g = torch.Generator().manual_seed(1)
    x = torch.randn(96, 160, generator=g)
    key = _key(3, 1000)
    (whole,) = O.sr_bf16_global_f(x, key)
    for r0, r1, c0, c1 in ((0, 32, 0, 64), (32, 96, 64, 160), (17, 50, 3, 99)):
        (tile,) = O.sr_bf16_global_f(x[r0:r1, c0:c1].contiguous(), key, global_row=r0, global_col=c0, num_col=160)
        assert_same_bits(tile, whole[r0:r1, c0:c1].contiguous(), f"tile {r0}:{r1}, {c0}:{c1}")
    (local,) = O.sr_bf16_f(x[17:50, 3:99].contiguous(), key)            # keyed on the tile's own layout: a different draw
    assert not torch.equal(local, whole[17:50, 3:99])


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(64, 64), (128, 1024), (33, 100), (5, 7), (1024, 2048), (1, 8)])
def test_kernel_matches_the_oracle(shape):
    from quant_cast_bench_b200 import quant_cast_cuda as Q
    g = torch.Generator().manual_seed(shape[0] * 131 + shape[1])
    x = torch.randn(*shape, generator=g) * torch.exp2(torch.randint(-30, 30, shape, generator=g).float())
    x.view(-1)[::97] = 0.0
    if x.numel() > 40:
        x.view(-1)[5] = float("inf"); x.view(-1)[6] = float("-inf"); x.view(-1)[7] = float("nan"); x.view(-1)[8] = 1e-42; x.view(-1)[9] = -3.4e38
    for seed, off in ((0, 0), (123456789, 7), (2 ** 40 + 3, 2 ** 33)):
        key_h = _key(seed, off)
        key_d = Q.philox_key(seed, off, device="cuda")
        (got,) = Q.sr_bf16_cuda(x.cuda(), key_d)
        assert got.dtype == torch.bfloat16 and got.shape == x.shape
        assert_same_bits(got, O.sr_bf16_f(x, key_h)[0], f"sr_bf16 {shape} seed {seed}")


@pytest.mark.gpu
def test_kernel_global_offsets_and_tile_invariance():
    from quant_cast_bench_b200 import quant_cast_cuda as Q
    g = torch.Generator().manual_seed(2)
    x = torch.randn(256, 384, generator=g)
    xc = x.cuda()
    key_h, key_d = _key(9, 77), Q.philox_key(9, 77, device="cuda")
    (whole,) = Q.sr_bf16_global_cuda(xc, key_d, global_row=0, global_col=0, num_col=384)
    assert_same_bits(whole, O.sr_bf16_global_f(x, key_h)[0], "whole tensor")
    for r0, r1, c0, c1 in ((0, 128, 0, 128), (128, 256, 128, 384), (64, 192, 8, 264), (31, 77, 3, 200), (200, 256, 381, 384)):
        tile = xc[r0:r1, c0:c1].contiguous()
        (t,) = Q.sr_bf16_global_cuda(tile, key_d, global_row=r0, global_col=c0, num_col=384)
        assert_same_bits(t, whole[r0:r1, c0:c1].contiguous(), f"tile {r0}:{r1}, {c0}:{c1}")
    # a parent wider than the tensor, and the reference's calling convention through the recipe record
    (t,) = Q.sr_bf16_global_cuda(xc, key_d, global_row=5, global_col=12, num_col=1000)
    assert_same_bits(t, O.sr_bf16_global_f(x, key_h, global_row=5, global_col=12, num_col=1000)[0], "offset parent")
    rec = dict(Q.ALL_RECIPES)["fp32_to_bf16_sr_global_offsets"]
    (t2,) = rec.cuda_fn(xc, key_d, global_row=0, global_col=0, num_col=384)
    assert_same_bits(t2, whole, "through the recipe record")


@pytest.mark.gpu
def test_kernel_two_neighbours_and_unbiased_on_the_reference_example():
    from quant_cast_bench_b200 import quant_cast_cuda as Q
    for name in ("fp32_to_bf16_sr", "fp32_to_bf16_sr_global_offsets"):
        rec = dict(Q.ALL_RECIPES)[name]
        x = torch.full((1024, 1024), 1.0 + 0.003, dtype=torch.float32, device="cuda")     # the reference's example input (G:1872-1876)
        key = Q.philox_key(0, device="cuda")
        (out,) = rec.cuda_fn(x, key, global_row=0, global_col=0, num_col=1024)
        v = float(x.flatten()[0])
        assert set(out.float().unique().tolist()) == {1.0, 1.0 + 2.0 ** -7}
        assert abs(out.float().mean().item() - v) < 1e-3
    lib_rc = Q.sr_bf16_cuda                      # argument checks
    with pytest.raises(AssertionError):
        lib_rc(torch.zeros(4, 4, device="cuda", dtype=torch.bfloat16), Q.philox_key(0, device="cuda"))
