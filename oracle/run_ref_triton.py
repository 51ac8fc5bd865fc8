"""Launch one Triton kernel of the reference (installed under oracle/_ref) a few times -- a small, fixed workload for a
profiler capture of the reference's own GPU code next to this backend's.

    python oracle/run_ref_triton.py mxfp8_swizzle [--M 16384] [--N 16384] [--launches 3] [--gblock 128 --warps 4]

Test and benchmark infrastructure only, like everything under oracle/.  Without --gblock the recipe goes through the
reference's public function and its autotuner (hundreds of launches while it tunes: not what a capture wants); with
--gblock / --warps the `mxfp8_swizzle` kernel (quant_cast_triton/recipes.py:1359-1400) is launched directly with that
configuration -- `GBLOCK 128, 4 warps` is what its autotuner picks at 16384 x 16384 on a B200.  After the reference's
launches the same input goes through this backend's recipe as often, and the two results are compared.
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from oracle import ref_gold  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("recipe")
    ap.add_argument("--M", type=int, default=16384)
    ap.add_argument("--N", type=int, default=16384)
    ap.add_argument("--launches", type=int, default=3)
    ap.add_argument("--gblock", type=int, default=None)
    ap.add_argument("--warps", type=int, default=4)
    args = ap.parse_args()
    import triton
    T = ref_gold.triton_recipes()
    from quant_cast_bench_b200 import quant_cast_cuda as Q
    torch.manual_seed(0)
    M, N = args.M, args.N
    x = torch.randn(M, N, dtype=torch.bfloat16, device="cuda")
    if args.gblock is not None:
        assert args.recipe == "mxfp8_swizzle", "a fixed configuration is wired for mxfp8_swizzle only"
        y = torch.empty_like(x, dtype=torch.float8_e4m3fn)
        ngc = N // 32
        nrb, ncb = (M + 127) // 128, (ngc + 3) // 4
        n_slots = nrb * ncb * 512
        s_u8 = torch.empty(nrb, ncb, 32, 16, dtype=torch.uint8, device="cuda")
        kern = T._mxfp8_swizzle_kernel.fn       # the JIT function under the autotuner
        for _ in range(args.launches):
            kern[(triton.cdiv(n_slots, args.gblock),)](x, y, s_u8, n_slots, M, N, ngc, ncb, GBLOCK=args.gblock, num_warps=args.warps)
        theirs = (y, s_u8)
    else:
        fn = dict(T.ALL_RECIPES)[args.recipe].triton_fn
        for _ in range(args.launches):
            theirs = fn(x)
    torch.cuda.synchronize()
    ours_fn = dict(Q.ALL_RECIPES)[args.recipe].cuda_fn
    for _ in range(args.launches):
        ours = ours_fn(x)
    torch.cuda.synchronize()
    same = all(torch.equal(a.contiguous().view(torch.uint8).reshape(-1), b.contiguous().view(torch.uint8).reshape(-1)) for a, b in zip(ours, theirs))
    print(f"{args.recipe} {M}x{N}: outputs of the reference's kernel and of this backend equal: {same}")


if __name__ == "__main__":
    main()
