"""One-launch amax, casts that form their per-tensor scale themselves, and the amax exchange over peer memory.

All comparisons are bit-exact against the CPU oracle (amax / scale: nvfp4_gs_scale G:1243-1246,
float8_tensorwise_scale G:1179-1183 of quant_cast_gold/recipes.py; casts: the gold functions fed with the oracle's
scale).  The exchange is exercised on one GPU with several rank states in the same memory: every producing and
every publishing call of the emulated ranks is issued before any consuming call, on one stream, so no kernel ever
waits for a later one (a rank's first consumer normally publishes itself; with one rank that path runs as it is).  The wait that runs out (a rank that never publishes) is tested with a 20 ms limit: the kernel returns, the
outputs are flagged by code 19 of the device error word, the context stays usable.  Two real GPUs, when the box
has them, run the same casts as two processes (NCCL all-reduce and peer exchange) against the one-GPU result.
"""
import ctypes
import os
import socket
import subprocess
import sys

import pytest
import torch

from helpers import assert_same_bits
from quant_cast_bench_b200.quant_cast_cuda import _lib as L
from quant_cast_bench_b200.workloads import make_input

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(autouse=True)
def _no_device_error():
    yield
    assert L.device_error() == 0


def _stream():
    return torch.cuda.current_stream().cuda_stream


@pytest.mark.parametrize("shape", [(1, 8), (3, 5), (64, 256), (257, 1024), (2048, 4096), (4096, 4100)])
def test_one_launch_amax_matches_oracle_and_two_launch_form(shape):
    from oracle import gold_port as O
    from quant_cast_bench_b200 import quant_cast_cuda as Q
    x = make_input(shape[0], shape[1], seed=3 + shape[1], spread=6.0)
    xc = x.cuda()
    ws = Q.new_amax_workspace(xc.device)
    for _ in range(3):                                     # the workspace is left clean by every call
        assert_same_bits(Q.amax_cuda(xc, workspace=ws), O.amax_bf16(x), "raw amax")
    assert_same_bits(Q.nvfp4_gs_scale_cuda(xc, workspace=ws), O.nvfp4_gs_scale(x), "nvfp4 outer scale")
    for fmt in ("e4m3", "e5m2"):
        assert_same_bits(Q.float8_tensorwise_scale_cuda(xc, fmt, workspace=ws), O.float8_tensorwise_scale(x, fmt), fmt)
    # the cached per-stream workspace (no argument) and the two-launch form with an uninitialised workspace
    assert_same_bits(Q.amax_cuda(xc), O.amax_bf16(x), "cached workspace")
    lib = L.load()
    out = torch.empty(1, dtype=torch.float32, device="cuda")
    n = lib.qcc_amax_workspace_bytes()
    dirty = torch.full((n,), 0xFF, dtype=torch.uint8, device="cuda")
    assert lib.qcc_amax_bf16(xc.data_ptr(), xc.numel(), L.AMAX_RAW, 0, out.data_ptr(), dirty.data_ptr(), n, _stream()) == 0
    assert_same_bits(out.reshape(()), O.amax_bf16(x), "two launches")


def test_amax_of_zeros_and_after_a_larger_tensor():
    from quant_cast_bench_b200 import quant_cast_cuda as Q
    ws = Q.new_amax_workspace("cuda")
    big = make_input(512, 512, seed=1, spread=8.0).cuda()
    zero = torch.zeros(128, 64, dtype=torch.bfloat16, device="cuda")
    assert float(Q.amax_cuda(big, workspace=ws)) > 0
    assert float(Q.amax_cuda(zero, workspace=ws)) == 0.0   # nothing left over from the first call


@pytest.mark.parametrize("shape", [(128, 128), (96, 160), (256, 7168), (1024, 2048)])
@pytest.mark.parametrize("swizzle", [True, False])
def test_casts_that_form_their_scale_match_the_two_step_recipes(shape, swizzle):
    from oracle import gold_port as O
    from quant_cast_bench_b200 import quant_cast_cuda as Q
    x = make_input(shape[0], shape[1], seed=11, spread=6.0)
    xc = x.cuda()
    # mxfp8 + amax from one read
    for mode in ("rceil", "floor"):
        q, s, amax = Q.mxfp8_with_amax_cuda(xc, swizzle=swizzle, mode=mode)
        want = O.mxfp8_swizzle_f(x, mode=mode) if swizzle else O.mxfp8_f(x, mode=mode)
        assert_same_bits(q, want[0], "mxfp8 q")
        assert_same_bits(s, want[1], "mxfp8 scales")
        assert_same_bits(amax, O.amax_bf16(x), "amax out of the cast")
    # nvfp4 with outer = amax / 2688 formed in the prologue
    q, s, outer = Q.nvfp4_from_amax_cuda(xc, amax, swizzle=swizzle)
    want_outer = O.nvfp4_gs_scale(x)
    want = O.nvfp4_gs_swizzle_f(x, want_outer) if swizzle else O.nvfp4_gs_f(x, want_outer)
    assert_same_bits(outer, want_outer, "outer scale")
    assert_same_bits(q, want[0], "nvfp4 q")
    assert_same_bits(s, want[1], "nvfp4 scales")
    for fmt in ("e4m3", "e5m2"):
        q8, sc = Q.float8_tensorwise_from_amax_cuda(xc, amax, fmt)
        want_sc = O.float8_tensorwise_scale(x, fmt)
        assert_same_bits(sc, want_sc, "fp8 scale")
        assert_same_bits(q8, O.float8_tensorwise_f(x, want_sc, fmt)[0], "fp8 q")


class _Ranks:
    """`world` exchange states in this GPU's memory, as the C ABI sees the ranks of a box."""

    def __init__(self, world, timeout_us=1_000_000):
        self.lib = L.load()
        self.world = world
        self.mem = torch.empty(world * L.XCHG_STATE_BYTES, dtype=torch.uint8, device="cuda")
        ptrs = [self.mem.data_ptr() + r * L.XCHG_STATE_BYTES for r in range(world)]
        for p in ptrs:
            assert self.lib.qcc_xchg_state_init(p, timeout_us, _stream()) == 0
        self.ptrs = ptrs
        self.states = (ctypes.c_void_p * world)(*ptrs)
        self.pending = [False] * world

    def ref(self, rank):
        r = L.XchgRef(ctypes.cast(self.states, ctypes.POINTER(ctypes.c_void_p)), self.world, rank, int(self.pending[rank]))
        self.pending[rank] = False
        return ctypes.byref(r)

    def publish_amax(self, rank, x):
        assert self.lib.qcc_amax_bf16_xchg(x.data_ptr(), x.numel(), self.ptrs[rank], _stream()) == 0
        self.pending[rank] = True

    def publish_with_mxfp8(self, rank, x, swizzle=True):
        from quant_cast_bench_b200.quant_cast_cuda.recipes import blocked_shape
        M, N = x.shape
        q = torch.empty((M, N), dtype=torch.uint8, device="cuda")
        s = torch.empty(blocked_shape(M, N // 32) if swizzle else (M, N // 32), dtype=torch.uint8, device="cuda")
        flags = L.ROWWISE | (L.SWIZZLE if swizzle else 0)
        assert self.lib.qcc_mxfp8_amax_xchg(x.data_ptr(), M, N, flags, q.data_ptr(), s.data_ptr(), self.ptrs[rank], _stream()) == 0
        self.pending[rank] = True
        return q, s

    def publish(self, rank):
        assert self.lib.qcc_xchg_publish(self.ref(rank), _stream()) == 0

    def resolve(self, rank, mode=L.AMAX_RAW, fmt=0):
        out = torch.empty((), dtype=torch.float32, device="cuda")
        assert self.lib.qcc_xchg_resolve(self.ref(rank), mode, fmt, out.data_ptr(), _stream()) == 0
        return out

    def nvfp4(self, rank, x, swizzle=True):
        from quant_cast_bench_b200 import quant_cast_cuda as Q
        outer = self.resolve(rank, L.AMAX_NVFP4_SCALE)
        q, s = (Q.nvfp4_gs_swizzle_cuda if swizzle else Q.nvfp4_gs_cuda)(x, outer)
        return q, s, outer

    def fp8(self, rank, x, fmt=0):
        from quant_cast_bench_b200 import quant_cast_cuda as Q
        scale = self.resolve(rank, L.AMAX_FP8_SCALE, fmt)
        return Q.float8_tensorwise_cuda(x, scale, "e5m2" if fmt else "e4m3")[0], scale


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_exchange_of_emulated_ranks_matches_the_unsharded_casts(world):
    from oracle import gold_port as O
    from quant_cast_bench_b200.quant_cast_cuda import sharded
    M, N = 128 * world * 2, 512
    ranks = _Ranks(world)
    for it in range(5):                                     # both slot sets, several exchange numbers
        x = make_input(M, N, seed=40 + it, spread=6.0)
        x[(it * 37) % M, 5] = 2.0 ** (it + 3)               # the maximum moves from shard to shard
        shards = [x[r * (M // world):(r + 1) * (M // world)].contiguous().cuda() for r in range(world)]
        fused = it % 2 == 1
        mx = []
        for r in range(world):                              # all producers first ...
            if fused:
                mx.append(ranks.publish_with_mxfp8(r, shards[r]))
            else:
                ranks.publish_amax(r, shards[r])
        if world > 1:
            for r in range(world):                          # ... every rank hands its value over (no waiting) ...
                ranks.publish(r)
        want_outer = O.nvfp4_gs_scale(x)
        wq, ws = O.nvfp4_gs_swizzle_f(x, want_outer)
        nv = [ranks.nvfp4(r, shards[r]) for r in range(world)]   # ... then the resolves (with one rank the first one publishes)
        for r in range(world):
            assert_same_bits(nv[r][2], want_outer, f"outer scale on rank {r}")
            assert_same_bits(ranks.resolve(r), O.amax_bf16(x), f"raw amax on rank {r}")
        assert_same_bits(sharded.concat_rowwise([n[0] for n in nv]), wq.view(torch.uint8), "nvfp4 q")
        assert_same_bits(sharded.concat_rowwise([n[1] for n in nv]), ws.view(torch.uint8), "nvfp4 scales")
        if fused:
            gq, gs = O.mxfp8_swizzle_f(x)
            assert_same_bits(sharded.concat_rowwise([m[0] for m in mx]), gq.view(torch.uint8), "mxfp8 q")
            assert_same_bits(sharded.concat_rowwise([m[1] for m in mx]), gs.view(torch.uint8), "mxfp8 scales")
        want_scale = O.float8_tensorwise_scale(x)
        f8 = [ranks.fp8(r, shards[r]) for r in range(world)]
        assert_same_bits(f8[0][1], want_scale, "fp8 scale")
        assert_same_bits(sharded.concat_rowwise([f[0] for f in f8]), O.float8_tensorwise_f(x, want_scale)[0].view(torch.uint8), "fp8 q")


def test_sharded_caster_with_peer_exchange_on_one_rank():
    """World size 1: the producing cast, the consumer that publishes to itself, a second consumer of the same exchange."""
    from oracle import gold_port as O
    from quant_cast_bench_b200.quant_cast_cuda import sharded
    x = make_input(512, 1024, seed=9, spread=6.0)
    xc = x.cuda()
    c = sharded.ShardedCaster(exchange="peer")
    outer = O.nvfp4_gs_scale(x)
    for fuse in (True, False, True):
        mx, nv = c.mxfp8_then_nvfp4(xc, fuse_amax=fuse)
        s8 = c.xchg.global_scale("fp8")                   # second reader of the same exchange: no publishing
        q8 = c.ops.float8_tensorwise(xc, s8, "e4m3")[0]
        for got, want in zip(mx, O.mxfp8_swizzle_f(x)):
            assert_same_bits(got, want, "mxfp8")
        for got, want in zip(nv, (*O.nvfp4_gs_swizzle_f(x, outer), outer)):
            assert_same_bits(got, want, "nvfp4")
        assert_same_bits(s8, O.float8_tensorwise_scale(x), "fp8 scale")
        assert_same_bits(q8, O.float8_tensorwise_f(x, O.float8_tensorwise_scale(x))[0], "fp8 q")
    q8, s8 = c.fp8_tensorwise(xc * 2)
    assert_same_bits(s8, O.float8_tensorwise_scale(x * 2), "fp8 scale after another producer")
    assert_same_bits(c.global_amax(xc), O.amax_bf16(x), "global amax")
    c.xchg.close()


@pytest.mark.parametrize("pdl", [True, False])
def test_overlapped_launches_see_each_steps_own_scale(pdl):
    """The exchange warp and the nvfp4 cast start while the kernel before them drains (programmatic dependent launch)
    and pick the scale up on the device: consecutive steps on tensors of very different magnitude, issued eagerly
    and replayed from one CUDA graph, must each be cast under their own outer scale."""
    from oracle import gold_port as O
    from quant_cast_bench_b200.quant_cast_cuda import sharded
    base = make_input(1024, 2048, seed=21, spread=4.0)
    xs = [(base * k).to(torch.bfloat16) for k in (1.0, 64.0, 1.0 / 128.0, 8.0)]
    xc = [x.cuda() for x in xs]
    want = []
    for x in xs:
        outer = O.nvfp4_gs_scale(x)
        want.append((*O.mxfp8_swizzle_f(x), *O.nvfp4_gs_swizzle_f(x, outer), outer))
    c = sharded.ShardedCaster(exchange="peer", pdl=pdl)

    def check(outs, what):
        for (mx, nv), w in zip(outs, want):
            for got, ref in zip((*mx, *nv), w):
                assert_same_bits(got, ref, what)

    check([c.mxfp8_then_nvfp4(x) for x in xc], "eager")
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        outs = [c.mxfp8_then_nvfp4(x) for x in xc]
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    check(outs, "graph replay")
    c.xchg.close()


@pytest.mark.parametrize("rows,chunk", [(512, 128), (1024, 384), (256, 8192)])
def test_host_shard_caster_matches_the_one_shot_casts(rows, chunk):
    """Pinned host shard in, pinned host outputs back, cast in row chunks with the amax accumulating over the chunks:
    the same bytes as the one-shot casts of the oracle."""
    from oracle import gold_port as O
    from quant_cast_bench_b200.quant_cast_cuda import sharded
    from quant_cast_bench_b200.quant_cast_cuda.host_api import HostShardCaster
    N = 1024
    x = make_input(rows, N, seed=rows, spread=6.0)
    x[rows - 3, 11] = 7.0e3                                   # the maximum sits in the last chunk
    xh = x.pin_memory()
    xchg = sharded.AmaxExchange()
    hc = HostShardCaster(rows, N, "cuda", xchg, chunk_rows=chunk)
    outer = O.nvfp4_gs_scale(x)
    want = (*O.mxfp8_swizzle_f(x), *O.nvfp4_gs_swizzle_f(x, outer), outer)
    for _ in range(2):                                        # buffers and exchange state are reused
        got = hc.cast(xh)
        for g, w in zip(got, want):
            assert_same_bits(g, w, "host shard caster")
    xchg.close()


def test_host_shard_caster_two_slots_in_flight():
    """submit / result with two slots: five different shards go through in turn, two in flight at any time; every one
    comes back with the bytes of its own one-shot casts (its own amax, not a neighbour's)."""
    from oracle import gold_port as O
    from quant_cast_bench_b200.quant_cast_cuda import sharded
    from quant_cast_bench_b200.quant_cast_cuda.host_api import HostShardCaster
    rows, N = 512, 1024
    xs = []
    for k in range(5):
        x = make_input(rows, N, seed=40 + k, spread=6.0)
        x[(37 * k) % rows, 5] = 1.0e3 * (k + 1)               # a different maximum, in a different chunk, every time
        xs.append(x)
    xh = [x.pin_memory() for x in xs]
    xchg = sharded.AmaxExchange()
    hc = HostShardCaster(rows, N, "cuda", xchg, chunk_rows=128, slots=2)

    def check(k, got):
        outer = O.nvfp4_gs_scale(xs[k])
        want = (*O.mxfp8_swizzle_f(xs[k]), *O.nvfp4_gs_swizzle_f(xs[k], outer), outer)
        for g, w in zip(got, want):
            assert_same_bits(g, w, f"shard {k}")
    hc.submit(xh[0], 0)
    hc.submit(xh[1], 1)
    for k in range(2, 5):
        check(k - 2, hc.result(k & 1))
        hc.submit(xh[k], k & 1)
    check(3, hc.result(1))
    check(4, hc.result(0))
    check(0, hc.cast(xh[0]))                                   # the blocking form still works on the same object
    xchg.close()


def test_a_rank_that_never_publishes_runs_the_wait_out():
    ranks = _Ranks(2, timeout_us=20_000)
    x = make_input(128, 256, seed=2).cuda()
    ranks.publish_amax(0, x)                 # rank 1 stays silent
    out = ranks.resolve(0)                   # publishes rank 0's value, then waits 20 ms for rank 1's
    torch.cuda.synchronize()
    assert L.device_error() == 19
    assert float(out) == float(x.float().abs().max())       # what had arrived
    # the state remembers the failure: later waits return at once; the context is intact
    ranks.publish_amax(0, x)
    ranks.resolve(0)
    torch.cuda.synchronize()
    L.device_error()                         # cleared for the fixture
    assert float((x.float() * 2).sum()) == float(x.float().sum()) * 2


def test_exchange_argument_errors():
    lib = L.load()
    ranks = _Ranks(2)
    x = torch.zeros(64, 64, dtype=torch.bfloat16, device="cuda")
    out = torch.empty(1, dtype=torch.float32, device="cuda")
    states = ctypes.cast(ranks.states, ctypes.POINTER(ctypes.c_void_p))
    assert lib.qcc_amax_bf16_xchg(x.data_ptr(), x.numel(), None, None) == -3
    assert lib.qcc_amax_bf16_xchg(None, 8, ranks.ptrs[0], None) == -3
    assert lib.qcc_amax_bf16_xchg(x.data_ptr() + 2, 8, ranks.ptrs[0], None) == -2
    for bad in (L.XchgRef(states, 2, 2, 0), L.XchgRef(states, 17, 0, 0), L.XchgRef(states, 0, 0, 0), L.XchgRef(None, 2, 0, 0)):
        assert lib.qcc_xchg_resolve(ctypes.byref(bad), 0, 0, out.data_ptr(), None) == -3
        assert lib.qcc_xchg_publish(ctypes.byref(bad), None) == -3
    assert lib.qcc_xchg_resolve(None, 0, 0, out.data_ptr(), None) == -3
    assert lib.qcc_nvfp4_from_amax(x.data_ptr(), 64, 64, None, 0, x.data_ptr(), x.data_ptr(), None, None) == -3
    assert lib.qcc_nvfp4_from_amax(x.data_ptr(), 64, 64, out.data_ptr(), L.SR, x.data_ptr(), x.data_ptr(), None, None) == -3
    assert lib.qcc_fp8_tensorwise_from_amax(x.data_ptr(), 64, None, 0, x.data_ptr(), None, None) == -3
    assert lib.qcc_mxfp8_amax_xchg(x.data_ptr(), 64, 64, L.ROWWISE | L.COLWISE, x.data_ptr(), x.data_ptr(), ranks.ptrs[0], None) == -3
    n = lib.qcc_amax_workspace_bytes()
    assert lib.qcc_amax_workspace_init(None, n, None) == -3
    assert lib.qcc_amax_workspace_init(x.data_ptr(), n - 1, None) == -4


_WORKER = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from quant_cast_bench_b200.quant_cast_cuda import sharded, _lib as L
from quant_cast_bench_b200.workloads import make_input
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
M, N = 1024, 512
r0, r1 = sharded.shard_rows(M, world, rank)
x = make_input(r1 - r0, N, seed=5, row_offset=r0, chunk_rows=128)
if rank == world - 1:
    x[3, 7] = 3.0e4
x = x.cuda()
res = {}
for name in ("nccl", "peer"):
    c = sharded.ShardedCaster(exchange=name)
    for it in range(3):
        mx, nv = c.mxfp8_then_nvfp4(x)
        q8, s8 = c.fp8_tensorwise(x)
    res[name] = [t.view(torch.uint8).cpu() if t.element_size() == 1 else t.cpu() for t in (*mx, *nv, q8, s8)]
    if c.xchg is not None:
        torch.cuda.synchronize(); dist.barrier(); c.xchg.close()
torch.cuda.synchronize()
assert L.device_error() == 0
torch.save(res, os.path.join(sys.argv[2], f"rank{rank}.pt"))
dist.barrier()
dist.destroy_process_group()
"""


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_ranks_nccl_and_peer_exchange_match_one_gpu(tmp_path):
    from quant_cast_bench_b200 import quant_cast_cuda as Q
    from quant_cast_bench_b200.quant_cast_cuda import sharded
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    script = tmp_path / "worker.py"
    script.write_text(_WORKER)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
                        "127.0.0.1", "--master-port", str(port), str(script), ROOT, str(tmp_path)], env=env,
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    parts = [torch.load(tmp_path / f"rank{k}.pt") for k in range(2)]
    M, N = 1024, 512
    x = make_input(M, N, seed=5, chunk_rows=128)
    x[M // 2 + 3, 7] = 3.0e4
    xc = x.cuda()
    gs = Q.nvfp4_gs_scale_cuda(xc)
    want = [*Q.mxfp8_swizzle_cuda(xc), *Q.nvfp4_gs_swizzle_cuda(xc, gs), gs,
            Q.float8_tensorwise_cuda(xc, Q.float8_tensorwise_scale_cuda(xc))[0], Q.float8_tensorwise_scale_cuda(xc)]
    for name in ("nccl", "peer"):
        got = [[p[name][i] for p in parts] for i in range(7)]
        for i in (0, 1, 2, 3, 5):
            assert_same_bits(sharded.concat_rowwise(got[i]), want[i].view(torch.uint8), f"{name} output {i}")
        for i in (4, 6):
            for k in range(2):
                assert_same_bits(got[i][k], want[i], f"{name} scale {i} on rank {k}")
