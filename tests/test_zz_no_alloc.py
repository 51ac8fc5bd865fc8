"""The allocation-free amax entry point against the regular one.

qcc_amax_bf16_noalloc exists for hosts that cannot allocate device memory where they need the amax
(inside a region that forbids cudaMalloc, or a plugin that is only handed its input and output
buffers): its scratch is an 8 KB buffer inside the library image.  Here it is called through the C
ABI on buffers that exist before the call, twice in a row on different inputs -- the second input is
smaller and quieter, so partial maxima left over from the first call would show -- and every result
must equal bit for bit what qcc_amax_bf16 gives with a caller-supplied workspace, and what the CPU oracle computes
from the same bytes (max |x|, float8_tensorwise_scale G:1179-1183, nvfp4_gs_scale G:1243-1246).

The file name sorts last so that a run that stops at the first failure has already run everything else.
"""
import pytest
import torch

from quant_cast_bench_b200.quant_cast_cuda import _lib as L
from quant_cast_bench_b200.workloads import make_input

pytestmark = pytest.mark.gpu


def _reference(lib, x, mode, fmt, stream):
    out = torch.empty(1, dtype=torch.float32, device="cuda")
    nbytes = lib.qcc_amax_workspace_bytes()
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    assert lib.qcc_amax_bf16(x.data_ptr(), x.numel(), mode, fmt, out.data_ptr(), ws.data_ptr(), nbytes, stream) == 0
    return out


def _oracle(x_cpu, mode, fmt):
    from oracle import gold_port as O
    if mode == L.AMAX_RAW:
        return O.amax_bf16(x_cpu)
    if mode == L.AMAX_FP8_SCALE:
        return O.float8_tensorwise_scale(x_cpu, "e5m2" if fmt == L.FMT_E5M2 else "e4m3")
    return O.nvfp4_gs_scale(x_cpu)


def test_noalloc_amax_matches_regular_entry_point_twice_in_a_row():
    lib = L.load()
    stream = torch.cuda.current_stream().cuda_stream
    big_cpu = make_input(2048, 4096, seed=31, spread=8.0)                # many CTAs, large values
    small_cpu = (make_input(64, 256, seed=32, spread=0.0, outlier_p=0.0, zero_row_p=0.0) * 1e-3).to(torch.bfloat16)
    big, small = big_cpu.cuda(), small_cpu.cuda()
    outs = torch.empty(2, dtype=torch.float32, device="cuda")            # allocated before the calls under test
    for mode, fmt in ((L.AMAX_RAW, L.FMT_E4M3), (L.AMAX_FP8_SCALE, L.FMT_E4M3), (L.AMAX_FP8_SCALE, L.FMT_E5M2),
                      (L.AMAX_NVFP4_SCALE, L.FMT_E4M3)):
        want = [_reference(lib, t, mode, fmt, stream) for t in (big, small)]
        rc0 = lib.qcc_amax_bf16_noalloc(big.data_ptr(), big.numel(), mode, fmt, outs.data_ptr(), stream)
        rc1 = lib.qcc_amax_bf16_noalloc(small.data_ptr(), small.numel(), mode, fmt, outs.data_ptr() + 4, stream)
        assert rc0 == 0 and rc1 == 0
        torch.cuda.synchronize()
        assert torch.equal(outs[0:1].view(torch.int32), want[0].view(torch.int32)), f"first call, mode {mode}"
        assert torch.equal(outs[1:2].view(torch.int32), want[1].view(torch.int32)), f"second call, mode {mode}"
        for i, t in enumerate((big_cpu, small_cpu)):
            assert torch.equal(outs[i:i + 1].cpu().view(torch.int32), _oracle(t, mode, fmt).reshape(1).view(torch.int32)), (
                f"call {i} against the CPU oracle, mode {mode}")
    assert float(outs[1]) > 0


def test_noalloc_amax_rejects_oversized_and_bad_arguments():
    lib = L.load()
    x = torch.zeros(64, dtype=torch.bfloat16, device="cuda")
    out = torch.empty(1, dtype=torch.float32, device="cuda")
    assert lib.qcc_amax_bf16_noalloc(x.data_ptr(), (1 << 32) + 1, 0, 0, out.data_ptr(), None) == -6
    assert lib.qcc_amax_bf16_noalloc(None, 64, 0, 0, out.data_ptr(), None) == -3
    assert lib.qcc_amax_bf16_noalloc(x.data_ptr() + 2, 8, 0, 0, out.data_ptr(), None) == -2
    assert -6 in L.ERRORS
