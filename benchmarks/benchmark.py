"""Memory-bandwidth sweep of the CUDA casts: `python benchmarks/benchmark.py --mode cuda`.

Same CLI surface and table / CSV schema as benchmarks/benchmark.py of vkuzo/quant_cast_bench
(flags --M --K --recipe_name_filter --mode --csv; bytes moved = sum of numel * element_size over
inputs and outputs, B:35-38; rows `kernel,mode,gpu_time_ms,gbps,mem_bw_pct` upserted into the CSV,
B:233-261; percentage against 8000 GB/s, B:22).  Timing: CUDA events around each launch with a
256 MB write in between to flush L2 (the reference flushes the same way inside
do_bench_using_profiling), median over --iters repetitions.  `--extensions` adds the casts without a
reference recipe (e5m2, FLOOR, transposed nvfp4, stochastic rounding, the amax reductions).
"""
import argparse
import csv as _csv
import os
import statistics
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from quant_cast_bench_b200 import quant_cast_cuda as Q  # noqa: E402

B200_PEAK_BW_GBPS = 8000.0
_BENCH_SKIP = {"mxfp8", "fp8_rowwise_precalc_scale"}   # as the reference's _BENCH_SKIP


def _bytes_moved(inputs, outputs):
    tensors = [t for t in (*inputs, *outputs) if isinstance(t, torch.Tensor)]
    return sum(t.numel() * t.element_size() for t in tensors)


def _time(run, iters, flush):
    for _ in range(3):
        run()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        run()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    return statistics.median(ts)


def _extensions(x):
    s = Q.float8_tensorwise_scale_cuda(x)
    s5 = Q.float8_tensorwise_scale_cuda(x, "e5m2")
    gs = Q.nvfp4_gs_scale_cuda(x)
    key = Q.philox_key(0, device=x.device)
    rht = Q.hadamard_rht_matrix_cuda(torch.tensor([1, -1] * 8), x.device)
    gs_m = Q.nvfp4_rht_outer_scale_m_cuda(x, rht)
    y = torch.empty_like(x)
    yb = y.view(torch.uint8).reshape(-1)
    n = x.numel()
    return [
        # the yardsticks: kernels that only move data, with the streaming casts' access pattern
        ("yardstick_copy", (x,), lambda: (Q.stream_copy_cuda(x, y),)),
        ("yardstick_fold_2_to_1", (x,), lambda: (Q.stream_fold_cuda(x, yb[:n], 2),)),
        ("yardstick_fold_4_to_1", (x,), lambda: (Q.stream_fold_cuda(x, yb[:n // 2], 4),)),
        ("amax_fp8_scale", (x,), lambda: (Q.float8_tensorwise_scale_cuda(x),)),
        ("amax_nvfp4_scale", (x,), lambda: (Q.nvfp4_gs_scale_cuda(x),)),
        ("fp8_tensorwise_e5m2", (x, s5), lambda: Q.float8_tensorwise_cuda(x, s5, "e5m2")),
        ("fp8_rowwise_e5m2", (x,), lambda: Q.rowwise_fp8_cuda(x, "e5m2")),
        ("mxfp8_floor", (x,), lambda: Q.mxfp8_cuda(x, mode="floor")),
        ("mxfp8_swizzle_floor", (x,), lambda: Q.mxfp8_swizzle_cuda(x, mode="floor")),
        ("mxfp8_dim_m_swizzle_floor", (x,), lambda: Q.mxfp8_dim_m_swizzle_cuda(x, mode="floor")),
        ("mxfp8_dim_km_swizzle_floor", (x,), lambda: Q.mxfp8_dim_km_swizzle_cuda(x, mode="floor")),
        ("nvfp4_swizzle_both", (x, gs), lambda: Q.nvfp4_gs_swizzle_both_cuda(x, gs)),
        ("nvfp4_t", (x, gs), lambda: Q.nvfp4_gs_t_cuda(x, gs)),
        ("nvfp4_swizzle_t", (x, gs), lambda: Q.nvfp4_gs_swizzle_t_cuda(x, gs)),
        ("nvfp4_swizzle_sr", (x, gs, key), lambda: Q.nvfp4_gs_swizzle_sr_cuda(x, gs, key)),
        ("nvfp4_rht_outer_scale_m", (x, rht), lambda: (Q.nvfp4_rht_outer_scale_m_cuda(x, rht),)),
        ("nvfp4_swizzle_dim_m_rht", (x, gs_m, rht), lambda: Q.nvfp4_gs_swizzle_dim_m_rht_cuda(x, gs_m, rht)),
    ]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--M", type=int, default=16384)
    ap.add_argument("--K", type=int, default=16384)
    ap.add_argument("--recipe_name_filter", default=None)
    ap.add_argument("--recipe_name_exact", default=None, help="run the one recipe of exactly this name")
    ap.add_argument("--mode", default="cuda")
    ap.add_argument("--csv", default=None)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--extensions", action="store_true")
    ap.add_argument("--include_skipped", action="store_true", help="also run the recipes the reference sweep skips")
    ap.add_argument("--scalar_division", default=None, choices=("ieee", "cuda_eager"),
                    help="how amax / 448 and the like are computed: as the gold recipes do on the CPU (default) or on a CUDA device")
    args = ap.parse_args()
    if args.scalar_division:
        Q.set_scalar_division(args.scalar_division)
    assert args.mode == "cuda", "this harness drives the CUDA backend only (--mode cuda)"
    assert torch.cuda.is_available(), "no CUDA device"
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    rows, csv_rows = [], []
    tile_kwargs = {"global_row": 0, "global_col": 0, "num_col": args.K}

    def wanted(name):
        if args.recipe_name_exact is not None:
            return name == args.recipe_name_exact
        return args.recipe_name_filter is None or args.recipe_name_filter in name

    cases = []
    for name, recipe in Q.ALL_RECIPES:
        if (name in _BENCH_SKIP and not args.include_skipped) or not wanted(name):
            continue
        torch.manual_seed(0)
        inputs = recipe.example_input_fn(args.M, args.K)
        cases.append((name, inputs, (lambda r=recipe, i=inputs: r.cuda_fn(*i, **tile_kwargs)), recipe.perf_description))
    if args.extensions:
        torch.manual_seed(0)
        x = torch.randn(args.M, args.K, dtype=torch.bfloat16, device="cuda")
        cases += [(n, i, f, "extension") for n, i, f in _extensions(x) if wanted(n)]
    if not cases:
        raise ValueError(f"no recipe matched {args.recipe_name_exact or args.recipe_name_filter!r}")

    for name, inputs, run, desc in cases:
        outputs = run()
        nbytes = _bytes_moved(inputs, outputs)
        ms = _time(run, args.iters, flush)
        gbps = nbytes / (ms * 1e-3) / 1e9
        pct = gbps / B200_PEAK_BW_GBPS * 100
        rows.append((name, f"{ms:.4f}", f"{gbps:.1f}", f"{pct:.1f}%", desc))
        csv_rows.append((name, args.mode, ms, gbps, pct))

    print(f"shape: ({args.M}, {args.K})  mode: {args.mode}")
    w = max(len(r[0]) for r in rows)
    print(f"{'recipe':<{w}}  {'gpu_time_ms':>11}  {'gbps':>8}  {'pct_peak':>8}  perf_description")
    for r in rows:
        print(f"{r[0]:<{w}}  {r[1]:>11}  {r[2]:>8}  {r[3]:>8}  {r[4]}")

    if args.csv is not None:
        header = ["kernel", "mode", "gpu_time_ms", "gbps", "mem_bw_pct"]
        merged, index = [], {}
        if os.path.exists(args.csv):
            with open(args.csv, newline="") as f:
                reader = _csv.reader(f)
                next(reader, None)
                for r in reader:
                    if len(r) >= len(header):
                        index[(r[0], r[1])] = len(merged)
                        merged.append(r[: len(header)])
        for kernel, md, ms, gbps, pct in csv_rows:
            row = [kernel, md, f"{ms:.4f}", f"{gbps:.1f}", f"{pct:.2f}"]
            if (kernel, md) in index:
                merged[index[(kernel, md)]] = row
            else:
                index[(kernel, md)] = len(merged)
                merged.append(row)
        with open(args.csv, "w", newline="") as f:
            wr = _csv.writer(f)
            wr.writerow(header)
            wr.writerows(merged)
        print(f"wrote {len(merged)} rows to {args.csv} ({len(csv_rows)} upserted for mode {args.mode!r})")


if __name__ == "__main__":
    main()
