"""Row-sharded casts over the GPUs of one box: one process per GPU, `torch.distributed` for the plumbing.

A (M, N) matrix is split into contiguous row shards whose heights are multiples of 128, so every 1x32 /
1x16 / 32x1 block and every 128x4 scale atom lies inside one shard (the tiling rules of the reference's
flex_tile_map/recipes.py:137-179).  Rowwise outputs of the shards concatenate on dim 0 (blocked scale grids
on their first axis), transposed outputs on dim 1 (blocked grids on their second axis).  mxfp8 and rowwise
fp8 need no communication.  The per-tensor scales of fp8 tensorwise and nvfp4 need the global amax: each
rank reduces its shard, ONE all-reduce(MAX) of a single fp32 crosses NVLink, and every rank derives the scale
with the same IEEE division -- max is exact and order independent, so sharded outputs are bit-identical to
the single-GPU ones.

`ops` is the set of cast functions to run on a shard; by default the CUDA recipes.  Tests on CPU ranks (gloo)
pass a checker-backed set to exercise the sharding logic without GPUs.
"""
from types import SimpleNamespace

import torch
import torch.distributed as dist

from . import _lib as L
from .recipes import _FMT, _stream, blocked_shape


def shard_rows(M, world_size, rank, multiple=128):
    """[r0, r1) of `rank`: equal shards, each a multiple of `multiple` rows."""
    if M % (world_size * multiple) != 0:
        raise ValueError(f"M={M} must be a multiple of world_size * {multiple} = {world_size * multiple}")
    rows = M // world_size
    return rank * rows, (rank + 1) * rows


def cuda_ops():
    from . import recipes as R
    return SimpleNamespace(
        amax=R.amax_cuda, scale_from_amax=R.scale_from_amax_cuda, float8_tensorwise=R.float8_tensorwise_cuda,
        rowwise_fp8=R.rowwise_fp8_cuda, mxfp8=R._mxfp8, nvfp4=R._nvfp4,
        float8_tensorwise_from_amax=R.float8_tensorwise_from_amax_cuda, nvfp4_from_amax=R.nvfp4_from_amax_cuda)


def new_amax_group(ranks=None):
    """A process group for the amax all-reduce.  Under NCCL its stream gets high priority: the all-reduce kernel
    becomes ready together with a cast that fills every SM, and at default priority it is scheduled only once that
    cast's grid has drained, which puts the collective's latency (about 30 us over 8 GPUs) after the cast instead of
    under it.  Collective: every rank of the default group must call it."""
    if dist.get_backend() == "nccl":
        opts = dist.ProcessGroupNCCL.Options(is_high_priority_stream=True)
        return dist.new_group(ranks, backend="nccl", pg_options=opts)
    return dist.new_group(ranks)


class AmaxExchange:
    """The amax exchange of `include/quant_cast_cuda.h` for one process per GPU: every rank allocates its state,
    the CUDA IPC handles travel through the process group (host side, once), and from then on a producing kernel
    leaves the shard's amax in the rank's state and a one-warp kernel hands it to every rank over NVLink (plain peer
    stores), takes the maximum of the ranks' values in its own memory and writes the scale the casts read -- no
    collective call, nothing on another stream.  Constructing one is a collective call (every rank of `group`).
    World size 1 works without a process group.

    Protocol per tensor: one producer (`amax` or `mxfp8_with_amax`), then `global_scale(kind)`."""

    def __init__(self, group=None, device=None, timeout_s=1.0, local=False):
        """local=True: an exchange of this rank with itself (no peers, not a collective call) -- the same kernels
        giving the shard's own amax."""
        import ctypes
        self._ct = ctypes
        self.lib = L.load()
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.world = dist.get_world_size(group) if dist.is_initialized() and not local else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() and not local else 0
        if self.world > L.XCHG_MAX_RANKS:
            raise ValueError(f"the amax exchange serves at most {L.XCHG_MAX_RANKS} ranks, got {self.world}")
        state = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            L.check(self.lib.qcc_xchg_alloc(ctypes.byref(state)), "xchg_alloc")
            if timeout_s != 1.0:
                L.check(self.lib.qcc_xchg_state_init(state, max(1, int(timeout_s * 1e6)), None), "xchg_state_init")
                torch.cuda.synchronize()
            self.own = state.value
            self.opened = []
            ptrs = [None] * self.world
            ptrs[self.rank] = self.own
            if self.world > 1:
                handle = ctypes.create_string_buffer(L.XCHG_HANDLE_BYTES)
                L.check(self.lib.qcc_xchg_ipc_export(state, handle), "xchg_ipc_export")
                handles = [None] * self.world
                dist.all_gather_object(handles, bytes(handle.raw), group=group)
                for r, h in enumerate(handles):
                    if r == self.rank:
                        continue
                    peer = ctypes.c_void_p()
                    L.check(self.lib.qcc_xchg_ipc_open(ctypes.create_string_buffer(h, L.XCHG_HANDLE_BYTES), ctypes.byref(peer)),
                            f"xchg_ipc_open(rank {r})")
                    ptrs[r] = peer.value
                    self.opened.append(peer.value)
                dist.barrier(group=group)     # every rank has mapped every state before anyone publishes
        self.states = (ctypes.c_void_p * self.world)(*ptrs)
        self._refs = {p: L.XchgRef(self._ct.cast(self.states, self._ct.POINTER(self._ct.c_void_p)), self.world, self.rank, p)
                      for p in range(4)}
        self._pending = False         # a producer has run and its value has not been published yet

    def _ref(self, pdl=False):
        ref = self._refs[(L.XCHG_PUBLISH if self._pending else 0) | (L.XCHG_PDL if pdl else 0)]
        self._pending = False
        return self._ct.byref(ref)

    def close(self):
        """Unmaps the peers' states and frees the own one (call on every rank, after the work that uses the exchange
        has finished on all of them)."""
        if self.own is None:
            return
        with torch.cuda.device(self.device):
            torch.cuda.synchronize()
            for p in self.opened:
                self.lib.qcc_xchg_ipc_close(self._ct.c_void_p(p))
            self.lib.qcc_xchg_free(self._ct.c_void_p(self.own))
        self.own, self.opened = None, []

    # ---- producers (one launch each; the shard's amax stays in this rank's state until the first consumer)
    def amax(self, x_shard):
        L.check(self.lib.qcc_amax_bf16_xchg(x_shard.data_ptr(), x_shard.numel(), self.own, _stream(x_shard)), "amax_xchg")
        L.launch_count += 1
        self._pending = True

    def mxfp8_with_amax(self, x_shard, swizzle=True, mode="rceil"):
        """The rowwise mxfp8 cast of the shard, which also leaves the shard's amax in the exchange: (qdata, scale)."""
        M, N = x_shard.shape
        dev = x_shard.device
        flags = L.ROWWISE | (L.SWIZZLE if swizzle else 0) | (L.FLOOR if mode == "floor" else 0)
        qk = torch.empty((M, N), dtype=torch.uint8, device=dev)
        sk = torch.empty(blocked_shape(M, N // 32) if swizzle else (M, N // 32), dtype=torch.uint8, device=dev)
        L.check(self.lib.qcc_mxfp8_amax_xchg(x_shard.data_ptr(), M, N, flags, qk.data_ptr(), sk.data_ptr(), self.own,
                                            _stream(x_shard)), "mxfp8_amax_xchg")
        L.launch_count += 1
        self._pending = True
        return qk.view(torch.float8_e4m3fn), sk.view(torch.float8_e8m0fnu)

    # ---- the exchange itself
    def global_scale(self, kind, fmt="e4m3", pdl=False):
        """f(max over ranks) of the last producing call as a 0-dim fp32: kind 'raw' | 'fp8' | 'nvfp4'.  One warp; the
        first call after a producer publishes this rank's value to all ranks, later calls only read.  pdl=True (only
        directly behind the producing launch on the stream): programmatic dependent launch -- the warp is already
        resident when the producer's last CTA retires."""
        mode = {"raw": L.AMAX_RAW, "fp8": L.AMAX_FP8_SCALE, "nvfp4": L.AMAX_NVFP4_SCALE}[kind]
        out = torch.empty((), dtype=torch.float32, device=self.device)
        L.check(self.lib.qcc_xchg_resolve(self._ref(pdl), mode | L.div_flag(), _FMT[fmt], out.data_ptr(),
                                         torch.cuda.current_stream(self.device).cuda_stream), "xchg_resolve")
        L.launch_count += 1
        return out


class ShardedCaster:
    """Casts of one row shard per rank.

    exchange: how the tensor-wide amax travels.  "nccl": one all_reduce(MAX) of a single fp32 over `group` (with more
    than one rank and group=None the group is created with `new_amax_group()`, so constructing a caster is then a
    collective call).  "peer": the amax exchange over peer memory (`AmaxExchange`; CUDA ranks of one box only; also a
    collective constructor).  Both give the bits a single GPU gives.  "local": no exchange at all -- every rank scales
    by its own shard's amax (what a sharded cast costs without the collective; NOT the unsharded result)."""

    def __init__(self, group=None, ops=None, exchange="nccl", pdl=True):
        self.pdl = pdl            # overlap the launches of mxfp8_then_nvfp4 on the peer path (programmatic dependent launch)
        self.reverse_second_pass = True
        if exchange not in ("nccl", "peer", "local"):
            raise ValueError(f"unknown exchange {exchange!r}; use 'nccl', 'peer' or 'local'")
        self.xchg = AmaxExchange(group, local=exchange == "local") if exchange in ("peer", "local") else None
        if exchange == "nccl" and group is None and dist.is_initialized() and dist.get_world_size() > 1:
            group = new_amax_group()
        self.group = group
        self.ops = ops if ops is not None else cuda_ops()
        self.world = dist.get_world_size(group) if dist.is_initialized() and exchange != "local" else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() and exchange != "local" else 0

    def check_shard(self, x_shard):
        if x_shard.dim() != 2 or x_shard.shape[0] % 128 != 0:
            raise ValueError(f"a row shard must be 2-D with a multiple of 128 rows, got {tuple(x_shard.shape)}")
        return x_shard

    # ---- the one collective
    def global_amax(self, x_shard, async_op=False):
        """max |x| over all shards as a 0-dim fp32 tensor; with async_op the (tensor, work) pair."""
        if self.xchg is not None:
            self.xchg.amax(x_shard)
            amax = self.xchg.global_scale("raw")
            return (amax.reshape(1), None) if async_op else amax
        amax = self.ops.amax(x_shard).reshape(1)
        work = None
        if self.world > 1:
            work = dist.all_reduce(amax, op=dist.ReduceOp.MAX, group=self.group, async_op=async_op)
        return (amax, work) if async_op else amax.reshape(())

    # ---- casts
    def mxfp8(self, x_shard, flags):
        """Any mxfp8 cast of the shard (flags as in include/quant_cast_cuda.h); no communication."""
        return self.ops.mxfp8(self.check_shard(x_shard), flags)

    def rowwise_fp8(self, x_shard, fmt="e4m3"):
        return self.ops.rowwise_fp8(self.check_shard(x_shard), fmt)

    def fp8_tensorwise(self, x_shard, fmt="e4m3"):
        """(qdata_shard, scale): scale from the global amax."""
        self.check_shard(x_shard)
        if self.xchg is not None:
            self.xchg.amax(x_shard)
            scale = self.xchg.global_scale("fp8", fmt)
            (q,) = self.ops.float8_tensorwise(x_shard, scale, fmt)
            return q, scale
        amax = self.global_amax(x_shard)
        if hasattr(self.ops, "float8_tensorwise_from_amax"):
            return self.ops.float8_tensorwise_from_amax(x_shard, amax, fmt)
        scale = self.ops.scale_from_amax(amax, "fp8", fmt)
        (q,) = self.ops.float8_tensorwise(x_shard, scale, fmt)
        return q, scale

    def nvfp4(self, x_shard, flags=4, transposed=False):
        """(qdata_shard, inner_scales_shard, outer_scale): outer scale from the global amax."""
        self.check_shard(x_shard)
        if self.xchg is not None:
            self.xchg.amax(x_shard)
            outer = self.xchg.global_scale("nvfp4")
            q, s = self.ops.nvfp4(x_shard, outer, flags, None, transposed)
            return q, s, outer
        amax = self.global_amax(x_shard)
        if not transposed and not (flags & ~L.SWIZZLE) and hasattr(self.ops, "nvfp4_from_amax"):
            return self.ops.nvfp4_from_amax(x_shard, amax, bool(flags & L.SWIZZLE))
        outer = self.ops.scale_from_amax(amax, "nvfp4")
        q, s = self.ops.nvfp4(x_shard, outer, flags, None, transposed)
        return q, s, outer

    def mxfp8_then_nvfp4(self, x_shard, mx_flags=1 | 4, nv_flags=4, fuse_amax=None):
        """Both casts of an activation shard (the MoE configuration): (mxfp8 outputs, (qdata, inner scales, outer scale)).

        exchange "nccl": local amax, all-reduce started, the mxfp8 cast (which does not depend on it) runs while the 4
        bytes are in flight, then nvfp4 with the scale formed in its prologue.
        exchange "peer", fuse_amax False: amax kernel -> mxfp8 -> exchange (one warp) -> nvfp4.
        exchange "peer", fuse_amax True (default there, rowwise mxfp8 only): the mxfp8 cast itself delivers the amax, so
        x is read twice instead of three times: mxfp8 -> exchange (one warp) -> nvfp4."""
        self.check_shard(x_shard)
        plain_nv = not (nv_flags & ~L.SWIZZLE)
        if self.xchg is not None:
            if fuse_amax is None:
                fuse_amax = not (mx_flags & (L.COLWISE | L.BLOCK32))
            if fuse_amax:
                mx = self.xchg.mxfp8_with_amax(x_shard, bool(mx_flags & L.SWIZZLE), "floor" if mx_flags & L.FLOOR else "rceil")
            else:
                self.xchg.amax(x_shard)
                mx = self.ops.mxfp8(x_shard, mx_flags)
            # the exchange warp and the nvfp4 cast are dependent launches: the warp is resident before the mxfp8 kernel
            # has drained, the cast loads x while the warp exchanges and waits for the outer scale on the device
            # (inside a CUDA graph the launch latency is hidden anyway and the extra barrier of the overlapped form costs
            # more than it saves)
            pdl = self.pdl and plain_nv and bool(nv_flags & L.SWIZZLE) and not torch.cuda.is_current_stream_capturing()
            outer = self.xchg.global_scale("nvfp4", pdl=pdl)
            # second pass over the shard: from its end, where the first pass left it in L2 (worth 1.5 % on a 235 MB shard,
            # nothing on larger ones: little of the tail survives the first pass's own output stream)
            extra = (L.PDL if pdl else 0) | (L.REVERSE if self.reverse_second_pass else 0)
            q, s = self.ops.nvfp4(x_shard, outer, nv_flags | extra, None, False)
            return mx, (q, s, outer)
        amax, work = self.global_amax(x_shard, async_op=True)
        mx = self.ops.mxfp8(x_shard, mx_flags)
        if work is not None:
            work.wait()
        if plain_nv and hasattr(self.ops, "nvfp4_from_amax"):
            return mx, self.ops.nvfp4_from_amax(x_shard, amax.reshape(()), bool(nv_flags & L.SWIZZLE))
        outer = self.ops.scale_from_amax(amax.reshape(()), "nvfp4")
        q, s = self.ops.nvfp4(x_shard, outer, nv_flags, None, False)
        return mx, (q, s, outer)


def concat_rowwise(parts):
    """Reassemble rowwise outputs (and blocked grids of rowwise scales) of consecutive row shards."""
    return torch.cat([p.view(torch.uint8) if p.element_size() == 1 else p for p in parts], dim=0)


def concat_transposed(parts):
    """Reassemble transposed outputs (dim 1) and blocked grids of transposed scales (their second axis)."""
    return torch.cat([p.view(torch.uint8) if p.element_size() == 1 else p for p in parts], dim=1)
