"""Casts on a GPU that is not the process's current device (needs two GPUs).

Every entry point works on the device its tensors live on: the Python layers switch to it for the launch, the library
keeps its per-device host state (kernel attributes, SM count, the built-in amax buffer's address) per ordinal."""
import pytest
import torch

from helpers import assert_same_bits
from oracle import gold_port as O
from quant_cast_bench_b200.workloads import make_input

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")]


def test_casts_on_a_second_device():
    from quant_cast_bench_b200 import build as qbuild
    from quant_cast_bench_b200 import quant_cast_cuda as Q
    from quant_cast_bench_b200.quant_cast_cuda import _lib as L
    qbuild.build_torch_binding()
    from quant_cast_bench_b200.quant_cast_cuda import native_ops as N
    torch.cuda.set_device(0)
    x = make_input(256, 512, seed=9)
    for dev in ("cuda:1", "cuda:0", "cuda:1"):          # back and forth: the per-device set-up happens once each
        xc = x.to(dev)
        assert torch.cuda.current_device() == 0
        outs = {
            "mxfp8_dim_km_swizzle": (Q.mxfp8_dim_km_swizzle_cuda(xc), O.mxfp8_dim_km_swizzle_f(x)),
            "rowwise": (Q.rowwise_fp8_cuda(xc), O.rowwise_fp8_f(x)),
            "colwise": (Q.colwise_fp8_cuda(xc), O.colwise_fp8_f(x)),
            "deepseek_dim_km": (Q.deepseek_1x128_dim_km_cuda(xc), O.deepseek_1x128_dim_km_f(x)),
            "native mxfp8_dim_km_swizzle": (N.mxfp8_dim_km_swizzle_native(xc), O.mxfp8_dim_km_swizzle_f(x)),
            "native colwise": (N.colwise_fp8_native(xc), O.colwise_fp8_f(x)),
        }
        gs = Q.nvfp4_gs_scale_cuda(xc)
        assert gs.device == xc.device
        assert_same_bits(gs.reshape(1), O.nvfp4_gs_scale(x).reshape(1), f"outer scale on {dev}")
        outs["nvfp4_swizzle_t"] = (Q.nvfp4_gs_swizzle_t_cuda(xc, gs), O.nvfp4_gs_swizzle_t_f(x, gs.cpu()))
        outs["native nvfp4_swizzle"] = (N.nvfp4_gs_swizzle_native(xc, gs), O.nvfp4_gs_swizzle_f(x, gs.cpu()))
        for name, (got, want) in outs.items():
            assert len(got) == len(want), name
            for i, (a, b) in enumerate(zip(got, want)):
                assert a.device == xc.device, name
                assert_same_bits(a, b, f"{name}[{i}] on {dev}")
        # the allocation-free amax keeps one built-in buffer per device
        lib = L.load()
        out = torch.zeros((), dtype=torch.float32, device=dev)
        with torch.cuda.device(xc.device):
            assert lib.qcc_amax_bf16_noalloc(xc.data_ptr(), xc.numel(), L.AMAX_RAW, L.FMT_E4M3, out.data_ptr(),
                                             torch.cuda.current_stream().cuda_stream) == 0
        assert float(out) == float(x.float().abs().max())
        torch.cuda.synchronize(dev)
    assert torch.cuda.current_device() == 0
    for d in (0, 1):
        with torch.cuda.device(d):
            assert L.device_error() == 0

