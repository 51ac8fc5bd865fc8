"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

No dataset is involved: the reference benchmarks on `torch.randn` (benchmarks/benchmark.py:64-66 of
vkuzo/quant_cast_bench) and the configurations below only add per-row dynamic range, sparse outliers
and all-zero rows.  Inputs are generated in row chunks on the CPU generator of the given seed (so the
same bytes can be handed to a CPU checker) and moved to `device`.
"""
import torch

# name -> (M, N, per-row log2 spread, outlier probability, outlier multiplier, zero-row fraction)
CONFIGS = {
    "c1_fp8_4096": (4096, 4096, 8.0, 0.0, 1.0, 0.0),
    "c2_mxfp8_16384": (16384, 16384, 10.0, 1e-3, 100.0, 0.01),
    "c3_nvfp4_8192": (8192, 8192, 10.0, 1e-3, 100.0, 0.01),
    "c4_moe_131072x7168": (131072, 7168, 6.0, 0.0, 1.0, 0.0),
    "c5_nvfp4_sr_8192x16384": (8192, 16384, 0.0, 1e-3, 50.0, 0.0),
}


def make_input(M, N, seed=0, spread=10.0, outlier_p=1e-3, outlier_mul=100.0, zero_row_p=0.01, device="cpu",
               row_offset=0, chunk_rows=4096):
    """bf16 (M, N): N(0,1) * 2^U(-spread, spread) per row, a fraction `outlier_p` of elements multiplied by
    `outlier_mul`, a fraction `zero_row_p` of rows all zero.  Row r of the result depends only on
    (seed, row_offset + r), so a row shard equals the matching rows of the whole tensor."""
    out = torch.empty((M, N), dtype=torch.bfloat16, device=device)
    for r0 in range(0, M, chunk_rows):
        r1 = min(M, r0 + chunk_rows)
        rows = []
        for blk in range((row_offset + r0) // chunk_rows, (row_offset + r1 - 1) // chunk_rows + 1):
            g = torch.Generator().manual_seed(seed * 1000003 + blk)
            x = torch.randn(chunk_rows, N, generator=g)
            if spread > 0:
                x = x * torch.exp2((torch.rand(chunk_rows, 1, generator=g) * 2 - 1) * spread)
            if outlier_p > 0:
                x = torch.where(torch.rand(chunk_rows, N, generator=g) < outlier_p, x * outlier_mul, x)
            if zero_row_p > 0:
                x[torch.rand(chunk_rows, generator=g) < zero_row_p] = 0
            lo = max(row_offset + r0, blk * chunk_rows) - blk * chunk_rows
            hi = min(row_offset + r1, (blk + 1) * chunk_rows) - blk * chunk_rows
            rows.append(x[lo:hi].to(torch.bfloat16))
        out[r0:r1] = torch.cat(rows).to(device)
    return out


def config_input(name, seed=0, device="cpu", rows=None, row_offset=0):
    """Input of a named configuration; `rows` / `row_offset` select a row shard."""
    M, N, spread, p, mul, z = CONFIGS[name]
    return make_input(rows if rows is not None else M, N, seed, spread, p, mul, z, device, row_offset)


def make_input_device(M, N, seed, device, spread=10.0, outlier_p=1e-3, outlier_mul=100.0, zero_row_p=0.01, row_offset=0,
                      chunk_rows=2048):
    """The same distribution drawn by the device's generator (full-size inputs in seconds instead of minutes).  Every
    `chunk_rows`-row chunk has its own seed, so a row shard (offset and size multiples of `chunk_rows`) holds the
    same values whatever the number of shards.  Not the same bytes as `make_input`."""
    assert M % chunk_rows == 0 and row_offset % chunk_rows == 0
    x = torch.empty((M, N), dtype=torch.bfloat16, device=device)
    g = torch.Generator(device=device)
    for r0 in range(0, M, chunk_rows):
        g.manual_seed(seed * 1000003 + (row_offset + r0) // chunk_rows)
        t = torch.randn(chunk_rows, N, generator=g, device=device)
        if spread > 0:
            t *= torch.exp2((torch.rand(chunk_rows, 1, generator=g, device=device) * 2 - 1) * spread)
        if outlier_p > 0:
            t = torch.where(torch.rand(chunk_rows, N, generator=g, device=device) < outlier_p, t * outlier_mul, t)
        if zero_row_p > 0:
            t[torch.rand(chunk_rows, generator=g, device=device) < zero_row_p] = 0
        x[r0:r0 + chunk_rows] = t.to(torch.bfloat16)
    return x


def config_input_device(name, device, seed=0):
    M, N, spread, p, mul, z = CONFIGS[name]
    return make_input_device(M, N, seed, device, spread, p, mul, z)

