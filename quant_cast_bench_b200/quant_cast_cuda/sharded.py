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
        rowwise_fp8=R.rowwise_fp8_cuda, mxfp8=R._mxfp8, nvfp4=R._nvfp4)


def new_amax_group(ranks=None):
    """A process group for the amax all-reduce.  Under NCCL its stream gets high priority: the all-reduce kernel
    becomes ready together with a cast that fills every SM, and at default priority it is scheduled only once that
    cast's grid has drained, which puts the collective's latency (about 30 us over 8 GPUs) after the cast instead of
    under it.  Collective: every rank of the default group must call it."""
    if dist.get_backend() == "nccl":
        opts = dist.ProcessGroupNCCL.Options(is_high_priority_stream=True)
        return dist.new_group(ranks, backend="nccl", pg_options=opts)
    return dist.new_group(ranks)


class ShardedCaster:
    """`group=None` with more than one rank creates the group with `new_amax_group()`, so constructing a caster is
    then a collective call."""

    def __init__(self, group=None, ops=None):
        if group is None and dist.is_initialized() and dist.get_world_size() > 1:
            group = new_amax_group()
        self.group = group
        self.ops = ops if ops is not None else cuda_ops()
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0

    def check_shard(self, x_shard):
        if x_shard.dim() != 2 or x_shard.shape[0] % 128 != 0:
            raise ValueError(f"a row shard must be 2-D with a multiple of 128 rows, got {tuple(x_shard.shape)}")
        return x_shard

    # ---- the one collective
    def global_amax(self, x_shard, async_op=False):
        """max |x| over all shards as a 0-dim fp32 tensor; with async_op the (tensor, work) pair."""
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
        scale = self.ops.scale_from_amax(self.global_amax(x_shard), "fp8", fmt)
        (q,) = self.ops.float8_tensorwise(x_shard, scale, fmt)
        return q, scale

    def nvfp4(self, x_shard, flags=4, transposed=False):
        """(qdata_shard, inner_scales_shard, outer_scale): outer scale from the global amax."""
        self.check_shard(x_shard)
        outer = self.ops.scale_from_amax(self.global_amax(x_shard), "nvfp4")
        q, s = self.ops.nvfp4(x_shard, outer, flags, None, transposed)
        return q, s, outer

    def mxfp8_then_nvfp4(self, x_shard, mx_flags=1 | 4, nv_flags=4):
        """Both casts of an activation shard (the MoE configuration): the amax all-reduce is started first and
        the mxfp8 cast, which does not depend on it, runs while the 4 bytes are in flight."""
        self.check_shard(x_shard)
        amax, work = self.global_amax(x_shard, async_op=True)
        mx = self.ops.mxfp8(x_shard, mx_flags)
        if work is not None:
            work.wait()
        outer = self.ops.scale_from_amax(amax.reshape(()), "nvfp4")
        q, s = self.ops.nvfp4(x_shard, outer, nv_flags, None, False)
        return mx, (q, s, outer)


def concat_rowwise(parts):
    """Reassemble rowwise outputs (and blocked grids of rowwise scales) of consecutive row shards."""
    return torch.cat([p.view(torch.uint8) if p.element_size() == 1 else p for p in parts], dim=0)


def concat_transposed(parts):
    """Reassemble transposed outputs (dim 1) and blocked grids of transposed scales (their second axis)."""
    return torch.cat([p.view(torch.uint8) if p.element_size() == 1 else p for p in parts], dim=1)
