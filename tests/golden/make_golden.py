"""Generate tests/golden/gold_vectors.npz by running the REFERENCE's gold recipes on CPU.

Run where a checkout of the reference project is available:
    python tests/golden/make_golden.py --reference /path/to/quant_cast_bench_checkout
(default: $QCC_REFERENCE_ROOT, else a checkout named `reference` beside this repository)
The reference imports `torch.func._random` (a module of newer PyTorch builds) at import time; it is
only used by the stochastic-rounding recipes, which are not part of the stored vectors, so an empty
stand-in module is registered before the import.  Nothing from the reference is copied: only the
inputs fed to it and the bytes it returned are stored.

With `--device cuda` (on a machine with a GPU) the same recipes run eagerly on the CUDA device instead and the
result goes to tests/golden/gold_vectors_cuda.npz:
    python tests/golden/make_golden.py --reference oracle/_ref --device cuda
Eager PyTorch computes `tensor / python_scalar` as an IEEE division on the CPU and as a multiplication with the
fp32 reciprocal of the scalar on a CUDA device, so the recipes that divide an amax by 448, 2688 or 6 give slightly
different bytes there.  That file stores only the outputs that differ from the CPU file (same keys), and under
`same_as_cpu` the names of those that do not.

Stored per case `<shape>_<seed>`: the bf16 input bits and, for every gold recipe on the hot path,
the raw bytes of each output (fp8 / e8m0 / packed fp4 as uint8, fp32 scales as their int32 bits).
Also stored: scalar known-answer tables for PyTorch's fp32->e4m3/e5m2 casts, the reference's fp4
encoder, its e8m0 RCEIL rounding and reciprocal, and its blocked-layout permutation.
"""
import argparse
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def default_reference():
    """$QCC_REFERENCE_ROOT, else a checkout named `reference` beside this repository, else None."""
    repo = os.path.dirname(os.path.dirname(HERE))
    for c in (os.environ.get("QCC_REFERENCE_ROOT"), os.path.join(os.path.dirname(repo), "reference")):
        if c and os.path.isfile(os.path.join(c, "quant_cast_bench", "quant_cast_gold", "recipes.py")):
            return c
    return None


def import_gold(ref_root):
    stub = types.ModuleType("torch.func._random")
    stub.uniform = None
    stub.key = None
    sys.modules["torch.func._random"] = stub
    sys.path.insert(0, ref_root)
    from quant_cast_bench.quant_cast_gold import recipes as G
    from quant_cast_bench.quant_cast_gold import utils as GU
    return G, GU


def make_input(M, N, seed, spread=10.0, outlier_p=1e-3, outlier_mul=100.0, zero_row_p=0.01):
    """Same distribution family as the benchmark configs: N(0,1) * 2^U(-spread, spread) per row,
    sparse outliers, some all-zero rows."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, N, generator=g)
    x = x * torch.exp2((torch.rand(M, 1, generator=g) * 2 - 1) * spread)
    x = torch.where(torch.rand(M, N, generator=g) < outlier_p, x * outlier_mul, x)
    x[torch.rand(M, generator=g) < zero_row_p] = 0
    x[M // 2] = 0  # at least one all-zero row in every case
    return x.to(torch.bfloat16)


def raw(t):
    t = t.detach().cpu()
    if t.dtype == torch.float32:
        return t.contiguous().view(torch.int32).numpy()
    if t.dtype == torch.bfloat16:
        return t.contiguous().view(torch.int16).numpy()
    return t.contiguous().view(torch.uint8).numpy()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=default_reference())
    ap.add_argument("--device", default="cpu", choices=("cpu", "cuda"))
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    dev = args.device
    if args.out is None:
        args.out = os.path.join(HERE, "gold_vectors.npz" if dev == "cpu" else "gold_vectors_cuda.npz")
    if not args.reference:
        raise SystemExit("no reference checkout: pass --reference or set QCC_REFERENCE_ROOT")
    G, GU = import_gold(args.reference)
    out = {}

    cases = [(128, 128, 0), (96, 160, 1), (128, 160, 2), (160, 320, 4), (256, 256, 5)]
    names = []
    for M, N, seed in cases:
        x = make_input(M, N, seed).to(dev)
        tag = f"{M}x{N}_s{seed}"
        names.append(tag)
        out[f"{tag}/x"] = raw(x)
        s = G.float8_tensorwise_scale(x)
        out[f"{tag}/float8_tensorwise_scale/0"] = raw(s.reshape(1))
        out[f"{tag}/float8_tensorwise_f/0"] = raw(G.float8_tensorwise_f(x, s)[0])
        ps = G.rowwise_precalc_scale(x)
        out[f"{tag}/rowwise_precalc_scale/0"] = raw(ps)
        out[f"{tag}/rowwise_precalc_f/0"] = raw(G.rowwise_precalc_f(x, ps)[0])
        cs = G.colwise_precalc_scale(x)
        out[f"{tag}/colwise_precalc_scale/0"] = raw(cs)
        out[f"{tag}/colwise_precalc_f/0"] = raw(G.colwise_precalc_f(x, cs)[0])
        for fn in ("rowwise_fp8_f", "colwise_fp8_f", "mxfp8_f", "mxfp8_swizzle_f", "mxfp8_dim_m_f",
                   "mxfp8_dim_m_swizzle_f", "mxfp8_dim_km_f", "mxfp8_dim_km_swizzle_f"):
            for i, o in enumerate(getattr(G, fn)(x)):
                out[f"{tag}/{fn}/{i}"] = raw(o)
        if M % 128 == 0 and N % 128 == 0:   # 1x128 / 128x128 blocks with fp32 scales (G:103-277)
            for fn in ("deepseek_1x128_f", "deepseek_128x128_f", "deepseek_1x128_dim_m_f", "deepseek_1x128_dim_km_f"):
                for i, o in enumerate(getattr(G, fn)(x)):
                    out[f"{tag}/{fn}/{i}"] = raw(o)
            ob = G.nvfp4_blocked_outer_scale(x)
            ob = torch.where(ob == 0, torch.full_like(ob, 2.0 ** -100), ob)   # an all-zero block: outer 0 divides 0 by 0
            out[f"{tag}/nvfp4_blocked_outer_scale/0"] = raw(ob)
            for i, o in enumerate(G.nvfp4_blocked_outer_f(x, ob)):
                out[f"{tag}/nvfp4_blocked_outer_f/{i}"] = raw(o)
        if M % 32 == 0:   # 32x32 blocks (G:753-959)
            for fn in ("mxfp8_32x32_f", "mxfp8_32x32_swizzle_f", "mxfp8_32x32_dim_m_swizzle_f", "mxfp8_32x32_dim_km_swizzle_f",
                       "mxfp8_32x32_qdata_dim_k_scale_dim_km_swizzle_f"):
                for i, o in enumerate(getattr(G, fn)(x)):
                    out[f"{tag}/{fn}/{i}"] = raw(o)
        for i, o in enumerate(G.mxfp4_f(x)):
            out[f"{tag}/mxfp4_f/{i}"] = raw(o)
        gs = G.nvfp4_gs_scale(x)
        out[f"{tag}/nvfp4_gs_scale/0"] = raw(gs.reshape(1))
        for fn in ("nvfp4_gs_f", "nvfp4_gs_swizzle_f"):
            for i, o in enumerate(getattr(G, fn)(x, gs)):
                out[f"{tag}/{fn}/{i}"] = raw(o)
        # transposed variant = the same recipe on x.t().contiguous() (test/test_quant_cast_gold.py:104)
        for i, o in enumerate(G.nvfp4_gs_swizzle_f(x.t().contiguous(), gs)):
            out[f"{tag}/nvfp4_gs_swizzle_t_f/{i}"] = raw(o)
        for i, o in enumerate(G.nvfp4_gs_f(x.t().contiguous(), gs)):
            out[f"{tag}/nvfp4_gs_t_f/{i}"] = raw(o)
        # randomised Hadamard transform and the two-orientation nvfp4 cast built on it (G:1324-1372, G:1778-1810)
        sign = torch.tensor([1, -1] * 8 if seed % 2 == 0 else [1, 1, -1, 1, -1, -1, -1, 1, 1, -1, 1, 1, -1, 1, -1, -1],
                            dtype=torch.bfloat16)
        rht = G.hadamard_rht_matrix(sign, dev, torch.bfloat16)
        out[f"{tag}/rht"] = raw(rht)
        out[f"{tag}/hadamard_rht_f/0"] = raw(G.hadamard_rht_f(x, rht)[0])
        (x_t_rht,) = G.hadamard_rht_f(x.t().contiguous(), rht)
        gs_m = x_t_rht.abs().to(torch.float32).amax() / (G.F8E4M3_MAX * G.F4_E2M1_MAX)
        out[f"{tag}/nvfp4_rht_outer_scale_m/0"] = raw(gs_m.reshape(1))
        for i, o in enumerate(G.nvfp4_gs_swizzle_dim_k_dim_m_rht_f(x, gs, gs_m, rht)):
            out[f"{tag}/nvfp4_gs_swizzle_dim_k_dim_m_rht_f/{i}"] = raw(o)
        pt = G.nvfp4_gs_per_token_scale(x).clamp(min=2.0 ** -100)
        out[f"{tag}/nvfp4_per_token_scale/0"] = raw(pt)
        for i, o in enumerate(G.nvfp4_gs_f(x, pt)):
            out[f"{tag}/nvfp4_gs_f_per_token/{i}"] = raw(o)
    out["cases"] = np.array(names)
    if dev != "cpu":
        # keep what the device computes differently, name the rest
        cpu = np.load(os.path.join(HERE, "gold_vectors.npz"))
        same, kept = [], {"cases": out["cases"]}
        for k, v in out.items():
            if k == "cases" or k.endswith("/x") or k.endswith("/rht"):
                assert k == "cases" or np.array_equal(v, cpu[k]), k   # same inputs as the CPU file
                continue
            if v.shape == cpu[k].shape and np.array_equal(v, cpu[k]):
                same.append(k)
            else:
                kept[k] = v
        kept["same_as_cpu"] = np.array(same)
        np.savez_compressed(args.out, **kept)
        print(f"wrote {args.out}: {len(kept) - 2} outputs differ from the CPU file, {len(same)} do not; "
              f"{os.path.getsize(args.out)/1e6:.2f} MB, torch {torch.__version__}, {torch.cuda.get_device_name(0)}")
        for k in sorted(kept):
            if k not in ("cases", "same_as_cpu"):
                print("  differs:", k, int((kept[k] != cpu[k]).sum()) if kept[k].shape == cpu[k].shape else "shape", "of", kept[k].size)
        return

    # ---- scalar known-answer tables -------------------------------------------------------------
    g = torch.Generator().manual_seed(1234)
    bits = torch.randint(0, 2 ** 32, (20000,), generator=g, dtype=torch.int64)
    # every e4m3 / e5m2 / e2m1 grid point and midpoint, and their fp32 neighbours
    grid = []
    for dt in (torch.float8_e4m3fn, torch.float8_e5m2):
        vals = torch.arange(256, dtype=torch.uint8).view(dt).float()
        vals = vals[torch.isfinite(vals)].unique()
        mids = (vals[1:] + vals[:-1]) / 2
        grid += [vals, mids]
    grid.append(torch.tensor([0.0, 0.25, 0.5, 0.75, 1.0, 1.25, 1.5, 1.75, 2.0, 2.5, 3.0, 3.5, 4.0, 5.0, 6.0, 7.0]))
    grid = torch.cat(grid)
    grid = torch.cat([grid, -grid])
    gb = grid.view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    near = torch.cat([gb - 1, gb, gb + 1]) & 0xFFFFFFFF
    allbits = torch.cat([bits, near])
    allbits = torch.where(allbits >= 2 ** 31, allbits - 2 ** 32, allbits).to(torch.int32)
    v = allbits.view(torch.float32)
    v = v[torch.isfinite(v)]
    v4 = v[v.abs() <= 464.0]
    out["kat/e4m3_in"] = raw(v4)
    out["kat/e4m3_out"] = raw(v4.to(torch.float8_e4m3fn))
    v5 = v[v.abs() < 61440.0]
    out["kat/e5m2_in"] = raw(v5)
    out["kat/e5m2_out"] = raw(v5.to(torch.float8_e5m2))
    small = torch.cat([v, torch.empty(8000).uniform_(-8, 8, generator=g)])
    out["kat/e2m1_in"] = raw(small)
    out["kat/e2m1_out"] = raw(GU.f32_to_f4_unpacked(small.clone()))
    codes = torch.arange(256, dtype=torch.uint8)
    dec = codes.view(torch.float8_e4m3fn).float()
    out["kat/e4m3_decode"] = raw(dec)
    am = v[v >= 0]
    am = torch.cat([am, torch.tensor([448.0 * 2.0 ** k for k in range(-126, 120)])])
    out["kat/rceil_in"] = raw(am)
    out["kat/rceil_out"] = raw(G._amax_to_e8m0_rceil(am))
    out["kat/recip_out"] = raw(G._e8m0_scale_to_reciprocal_fp32(codes.view(torch.float8_e8m0fnu)))
    for H, W in ((128, 4), (96, 5), (300, 9)):
        sc = torch.randint(0, 256, (H, W), generator=g, dtype=torch.uint8)
        out[f"kat/blocked_{H}x{W}_in"] = raw(sc)
        out[f"kat/blocked_{H}x{W}_out"] = raw(G._to_blocked_4d(sc))
    # token-group blocked layouts (experiments/quantize_tensor_api/moe_utils.py)
    from experiments.quantize_tensor_api import moe_utils as MU
    for name, M, W, offs in (("a", 160, 8, [32, 32, 96, 160]), ("b", 384, 12, [128, 160, 384]), ("c", 64, 4, [64])):
        sc = torch.randint(1, 256, (M, W), generator=g, dtype=torch.uint8)
        o = torch.tensor(offs, dtype=torch.int32)
        out[f"kat/mgroups_{name}_in"] = raw(sc)
        out[f"kat/mgroups_{name}_offs"] = o.numpy()
        out[f"kat/mgroups_{name}_out"] = raw(MU._to_blocked_2d_m_groups(sc, o))
        sct = torch.randint(1, 256, (W * 16, M // 32), generator=g, dtype=torch.uint8)   # (C, M/32) transposed scales
        out[f"kat/kgroups_{name}_in"] = raw(sct)
        out[f"kat/kgroups_{name}_out"] = raw(MU._to_blocked_2d_k_groups(sct, o // 32))
    for name, M, C, offs in (("a", 100, 16, [7, 7, 40, 100]), ("b", 64, 8, [64]), ("c", 131, 24, [1, 33, 131])):
        xin = torch.randn(M, C, generator=g).to(torch.bfloat16)
        o = torch.tensor(offs, dtype=torch.int32)
        padded, pstarts, pends = MU._pad_token_groups(xin, o)
        out[f"kat/padgroups_{name}_in"] = raw(xin)
        out[f"kat/padgroups_{name}_offs"] = o.numpy()
        out[f"kat/padgroups_{name}_out"] = raw(padded)
        out[f"kat/padgroups_{name}_starts"] = pstarts.to(torch.int32).numpy()
        out[f"kat/padgroups_{name}_ends"] = pends.to(torch.int32).numpy()
    out["kat/bf16_clamp_min"] = raw(torch.zeros(1, dtype=torch.bfloat16).clamp(min=1e-12))

    np.savez_compressed(args.out, **out)
    print(f"wrote {args.out}: {len(out)} arrays, {os.path.getsize(args.out)/1e6:.2f} MB, torch {torch.__version__}")


if __name__ == "__main__":
    main()
