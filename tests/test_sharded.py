"""Row sharding with the amax all-reduce on CPU ranks (gloo, world size 2): the sharded outputs, put back
together, are bit-identical to the unsharded ones.  The cast functions are the CPU checker's, so only the
sharding layer (shard bounds, the MAX all-reduce, scale derivation, reassembly rules) is under test here; the
same layer over the CUDA kernels is covered by the `gpu` test at the bottom."""
import os
import socket
from types import SimpleNamespace

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import assert_same_bits
from quant_cast_bench_b200.quant_cast_cuda import sharded
from quant_cast_bench_b200.workloads import make_input

M, N = 512, 256


def oracle_ops():
    from oracle import gold_port as O
    def scale_from_amax(amax, kind, fmt="e4m3"):
        return O.fp8_scale_from_amax(float(amax), fmt) if kind == "fp8" else O.nvfp4_scale_from_amax(float(amax))
    return SimpleNamespace(
        amax=O.amax_bf16, scale_from_amax=scale_from_amax,
        float8_tensorwise=O.float8_tensorwise_f, rowwise_fp8=O.rowwise_fp8_f, mxfp8=O._mxfp8,
        nvfp4=lambda x, outer, flags, key, transposed: O._nvfp4(x, outer, flags, key, transposed))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        r0, r1 = sharded.shard_rows(M, world, rank)
        x = make_input(r1 - r0, N, seed=5, row_offset=r0, chunk_rows=128)
        if rank == 1:
            x[3, 7] = 3.0e4      # the global maximum lives on one rank only
        c = sharded.ShardedCaster(ops=oracle_ops())
        res = {}
        res["tw_q"], res["tw_scale"] = c.fp8_tensorwise(x)
        res["nv_q"], res["nv_s"], res["nv_outer"] = c.nvfp4(x, flags=4)
        res["nvt_q"], res["nvt_s"], _ = c.nvfp4(x, flags=4, transposed=True)
        (res["qk"], res["sk"], res["qm"], res["sm"]) = c.mxfp8(x, 1 | 2 | 4)
        mx, nv = c.mxfp8_then_nvfp4(x)
        res["pipe_mx_q"], res["pipe_nv_q"] = mx[0], nv[0]
        torch.save({k: (v.view(torch.uint8) if v.element_size() == 1 else v) for k, v in res.items()},
                   os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_two_cpu_ranks_match_unsharded(tmp_path):
    from oracle import gold_port as O
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    parts = [torch.load(os.path.join(tmp_path, f"rank{r}.pt")) for r in range(world)]
    x = make_input(M, N, seed=5, chunk_rows=128)
    x[M // 2 + 3, 7] = 3.0e4
    scale = O.float8_tensorwise_scale(x)
    for p in parts:
        assert_same_bits(p["tw_scale"], scale, "tensorwise scale on every rank")
    assert_same_bits(sharded.concat_rowwise([p["tw_q"] for p in parts]), O.float8_tensorwise_f(x, scale)[0].view(torch.uint8), "tensorwise q")
    outer = O.nvfp4_gs_scale(x)
    q, s = O.nvfp4_gs_swizzle_f(x, outer)
    assert_same_bits(parts[0]["nv_outer"], outer, "nvfp4 outer scale")
    assert_same_bits(sharded.concat_rowwise([p["nv_q"] for p in parts]), q.view(torch.uint8), "nvfp4 q")
    assert_same_bits(sharded.concat_rowwise([p["nv_s"] for p in parts]), s.view(torch.uint8), "nvfp4 blocked scales")
    qt, st = O.nvfp4_gs_swizzle_t_f(x, outer)
    assert_same_bits(sharded.concat_transposed([p["nvt_q"] for p in parts]), qt.view(torch.uint8), "nvfp4 transposed q")
    assert_same_bits(sharded.concat_transposed([p["nvt_s"] for p in parts]), st.view(torch.uint8), "nvfp4 transposed scales")
    qk, sk, qm, sm = O.mxfp8_dim_km_swizzle_f(x)
    assert_same_bits(sharded.concat_rowwise([p["qk"] for p in parts]), qk.view(torch.uint8), "qk")
    assert_same_bits(sharded.concat_rowwise([p["sk"] for p in parts]), sk.view(torch.uint8), "sk")
    assert_same_bits(sharded.concat_transposed([p["qm"] for p in parts]), qm.view(torch.uint8), "qm")
    assert_same_bits(sharded.concat_transposed([p["sm"] for p in parts]), sm.view(torch.uint8), "sm")
    assert_same_bits(sharded.concat_rowwise([p["pipe_mx_q"] for p in parts]), O.mxfp8_swizzle_f(x)[0].view(torch.uint8), "overlapped mxfp8")
    assert_same_bits(sharded.concat_rowwise([p["pipe_nv_q"] for p in parts]), q.view(torch.uint8), "overlapped nvfp4")


def test_shard_bounds_and_rejections():
    assert sharded.shard_rows(131072, 8, 3) == (3 * 16384, 4 * 16384)
    with pytest.raises(ValueError):
        sharded.shard_rows(1000, 8, 0)
    c = sharded.ShardedCaster(ops=oracle_ops())
    with pytest.raises(ValueError):
        c.fp8_tensorwise(torch.zeros(100, 64, dtype=torch.bfloat16))


@pytest.mark.gpu
def test_shards_on_one_gpu_match_whole_tensor():
    """Tile / shard invariance of the CUDA kernels (the INDUCTOR == MANUAL_TILE property of the reference's
    test/test_flex_tile_map.py:98-134): casting four row shards separately, with the global amax, gives the
    bytes of the whole-tensor cast."""
    from quant_cast_bench_b200 import quant_cast_cuda as Q
    x = make_input(1024, 512, seed=8).cuda()
    gs = Q.nvfp4_gs_scale_cuda(x)
    s8 = Q.float8_tensorwise_scale_cuda(x)
    shards = [x[i * 256:(i + 1) * 256].contiguous() for i in range(4)]
    amax = torch.stack([Q.amax_cuda(t) for t in shards]).max()
    assert_same_bits(Q.scale_from_amax_cuda(amax, "nvfp4"), gs, "outer from shard amaxes")
    assert_same_bits(Q.scale_from_amax_cuda(amax, "fp8"), s8, "fp8 scale from shard amaxes")
    whole = Q.mxfp8_dim_km_swizzle_cuda(x)
    parts = [Q.mxfp8_dim_km_swizzle_cuda(t) for t in shards]
    for i, cat in enumerate((sharded.concat_rowwise, sharded.concat_rowwise, sharded.concat_transposed, sharded.concat_transposed)):
        assert_same_bits(cat([p[i] for p in parts]), whole[i].view(torch.uint8), f"mxfp8 output {i}")
    wq, ws = Q.nvfp4_gs_swizzle_cuda(x, gs)
    pq = [Q.nvfp4_gs_swizzle_cuda(t, gs) for t in shards]
    assert_same_bits(sharded.concat_rowwise([p[0] for p in pq]), wq.view(torch.uint8), "nvfp4 q")
    assert_same_bits(sharded.concat_rowwise([p[1] for p in pq]), ws.view(torch.uint8), "nvfp4 scales")
    tq, ts = Q.nvfp4_gs_swizzle_t_cuda(x, gs)
    pt = [Q.nvfp4_gs_swizzle_t_cuda(t, gs) for t in shards]
    assert_same_bits(sharded.concat_transposed([p[0] for p in pt]), tq.view(torch.uint8), "nvfp4 transposed q")
    assert_same_bits(sharded.concat_transposed([p[1] for p in pt]), ts.view(torch.uint8), "nvfp4 transposed scales")
