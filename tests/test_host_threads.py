"""Several host threads cast at the same time, each on a stream of its own: the entry points keep no shared mutable
state beyond per-device caches that every thread fills with the same values."""
import threading

import pytest
import torch

from helpers import assert_same_bits
from oracle import gold_port as O
from quant_cast_bench_b200.workloads import make_input


@pytest.mark.gpu
def test_four_threads_four_streams():
    from quant_cast_bench_b200 import quant_cast_cuda as Q
    from quant_cast_bench_b200.quant_cast_cuda import _lib as L
    xs = [make_input(128 * (t + 1), 256 * (t + 1), seed=70 + t) for t in range(4)]
    want = []
    for x in xs:
        gs = O.nvfp4_gs_scale(x)
        want.append((O.mxfp8_dim_km_swizzle_f(x), O.rowwise_fp8_f(x), O.nvfp4_gs_swizzle_f(x, gs), O.nvfp4_gs_swizzle_t_f(x, gs), gs))
    errors, got = [], [None] * 4
    start = threading.Barrier(4)

    def work(t):
        try:
            torch.cuda.set_device(0)
            stream = torch.cuda.Stream()
            xc = xs[t].cuda()
            torch.cuda.synchronize()
            start.wait()
            with torch.cuda.stream(stream):
                for _ in range(25):
                    gs = Q.nvfp4_gs_scale_cuda(xc)
                    res = (Q.mxfp8_dim_km_swizzle_cuda(xc), Q.rowwise_fp8_cuda(xc), Q.nvfp4_gs_swizzle_cuda(xc, gs),
                           Q.nvfp4_gs_swizzle_t_cuda(xc, gs), gs)
            stream.synchronize()
            got[t] = res
        except Exception as exc:      # noqa: BLE001
            errors.append((t, repr(exc)))

    threads = [threading.Thread(target=work, args=(t,)) for t in range(4)]
    for th in threads:
        th.start()
    for th in threads:
        th.join()
    assert not errors, errors
    for t in range(4):
        for group_got, group_want in zip(got[t][:4], want[t][:4]):
            for a, b in zip(group_got, group_want):
                assert_same_bits(a, b, f"thread {t}")
        assert_same_bits(got[t][4].reshape(1), want[t][4].reshape(1), f"outer scale, thread {t}")
    assert L.device_error() == 0
