"""quant_cast_cuda: the CUDA backend of the quant-cast recipes (a sibling of quant_cast_triton /
quant_cast_cute in vkuzo/quant_cast_bench)."""
from .recipes import *  # noqa: F401,F403
from .recipes import ALL_RECIPES, QuantCastCudaRecipe  # noqa: F401
from ._lib import get_scalar_division, scalar_division, set_scalar_division  # noqa: F401
