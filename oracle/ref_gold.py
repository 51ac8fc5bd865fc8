"""Access to the reference project installed under oracle/_ref/ (see oracle/build.py --ref).

Test and benchmark infrastructure only: the product package never imports this.  The benchmark's comparison legs
use it to run the reference's own code next to this backend -- its gold recipes eagerly on the host CPU
(quant_cast_gold/recipes.py) and its Triton kernels on the GPU (quant_cast_triton/recipes.py).

The reference imports `torch.func._random` at import time, a module of PyTorch builds newer than the installed one;
only its stochastic-rounding recipes use it, so an empty stand-in module is registered before the import.
"""
import os
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")


def available():
    return os.path.exists(os.path.join(REF_DIR, "quant_cast_bench", "quant_cast_gold", "recipes.py"))


def _prepare():
    if not available():
        raise ImportError("oracle/_ref is empty: run `python oracle/build.py --ref <reference checkout>`")
    if "torch.func._random" not in sys.modules:
        try:
            import torch.func._random  # noqa: F401
        except Exception:
            stub = types.ModuleType("torch.func._random")
            stub.uniform = None
            stub.key = None
            sys.modules["torch.func._random"] = stub
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)


def gold():
    """The reference's quant_cast_gold.recipes module."""
    _prepare()
    from quant_cast_bench.quant_cast_gold import recipes
    return recipes


def triton_recipes():
    """The reference's quant_cast_triton.recipes module (needs a GPU and Triton to run its kernels)."""
    _prepare()
    from quant_cast_bench.quant_cast_triton import recipes
    return recipes


def cute_recipes():
    """The reference's quant_cast_cute.recipes module (needs nvidia-cutlass-dsl of the version it was written for)."""
    _prepare()
    from quant_cast_bench.quant_cast_cute import recipes
    return recipes
