"""The recipe index against the reference's own (CPU; needs the reference checkout, skipped elsewhere): every
entry names a gold recipe of quant_cast_gold.ALL_RECIPES under the same name and in the same relative order, and
`from_gold` carries the gold record's fields over, as the reference's backends do
(quant_cast_triton/recipes.py:48-65, :1796-1835 of vkuzo/quant_cast_bench)."""
import importlib
import os
import sys

import pytest

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
import make_golden  # noqa: E402

REFERENCE = make_golden.default_reference()      # $QCC_REFERENCE_ROOT, or a checkout named `reference` beside the repository
pytestmark = pytest.mark.skipif(REFERENCE is None, reason="reference checkout not present ($QCC_REFERENCE_ROOT)")


def test_names_order_and_gold_fields():
    G, _ = make_golden.import_gold(REFERENCE)           # stubs torch.func._random, puts the reference on sys.path
    from quant_cast_bench_b200.quant_cast_cuda import recipes as R
    R = importlib.reload(R)                             # now quant_cast_gold is importable: records come from gold
    try:
        gold_names = [n for n, _ in G.ALL_RECIPES]
        gold_by_name = dict(G.ALL_RECIPES)
        ours = R.ALL_RECIPES
        names = [n for n, _ in ours]
        assert len(names) == len(set(names))
        for n in names:
            assert n in gold_by_name, f"{n} is not a gold recipe name"
        assert names == [n for n in gold_names if n in set(names)], "same relative order as quant_cast_gold.ALL_RECIPES"
        for n, rec in ours:
            g = gold_by_name[n]
            assert rec.pt_ref_fn is g.pt_ref_fn and rec.correctness_fn is g.correctness_fn
            assert rec.example_input_fn is g.example_input_fn and rec.perf_description == g.perf_description
            assert callable(rec.cuda_fn)
        # what is left out of the index, and only that
        assert sorted(set(gold_names) - set(names)) == ["debug_relu", "mxfp8_bias"]
    finally:
        for m in [m for m in sys.modules if m == "quant_cast_bench" or m.startswith("quant_cast_bench.")]:
            del sys.modules[m]
        if REFERENCE in sys.path:
            sys.path.remove(REFERENCE)
        importlib.reload(R)
