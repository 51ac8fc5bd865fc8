"""quant_cast_cuda: the CUDA backend of the quant-cast recipes (a sibling of quant_cast_triton /
quant_cast_cute in vkuzo/quant_cast_bench)."""
from .recipes import *  # noqa: F401,F403
from .recipes import ALL_RECIPES, QuantCastCudaRecipe  # noqa: F401
