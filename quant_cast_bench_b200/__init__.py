"""B200-native quantization-cast backend: hand-written sm_100a CUDA kernels behind a C ABI
(include/quant_cast_cuda.h) and a Python recipe layer with the signatures of the quant_cast_gold
recipes of vkuzo/quant_cast_bench."""

__version__ = "0.1.0"
