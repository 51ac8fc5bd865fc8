"""Host-buffer entry to the mxfp8 two-direction cast: pinned host bf16 in, pinned host outputs back.

This is the call a user with data in host memory makes.  The caster owns device staging buffers and the
pinned output buffers, so repeated casts allocate nothing.  A cast is pipelined over row chunks on three
streams: while chunk i is being cast, chunk i+1 travels host -> device and the outputs of chunk i-1 travel
device -> host (PCIe is full duplex), so the call takes about max(H2D, D2H) instead of their sum.  Row
chunks are multiples of 128 rows, so every block and every 128x4 scale atom lies inside one chunk and the
chunked result is bit-identical to the one-shot cast: rowwise outputs of a chunk are row slabs of the
host outputs; transposed outputs are column slabs, placed with strided copies.
"""
import torch

from . import _lib as L
from .recipes import blocked_shape


class HostMxfp8Caster:
    """mxfp8_dim_km(_swizzle) for an (M, N) bf16 matrix that lives in (pinned) host memory."""

    def __init__(self, M, N, device, swizzle=True, mode="rceil", chunk_rows=1024):
        assert M % 128 == 0 and N % 32 == 0, "host caster wants M % 128 == 0 and N % 32 == 0"
        self.M, self.N, self.device = M, N, torch.device(device)
        self.swizzle = swizzle
        self.flags = L.ROWWISE | L.COLWISE | (L.SWIZZLE if swizzle else 0) | (L.FLOOR if mode == "floor" else 0)
        rc = min(chunk_rows, M)
        while M % rc or rc % 128:
            rc -= 128
        self.rc = rc
        dev = self.device
        sk_c = blocked_shape(rc, N // 32) if swizzle else (rc, N // 32)
        sm_c = blocked_shape(N, rc // 32) if swizzle else (N, rc // 32)
        self.x_dev = [torch.empty((rc, N), dtype=torch.bfloat16, device=dev) for _ in range(2)]
        self.out_dev = [[torch.empty(s, dtype=torch.uint8, device=dev) for s in ((rc, N), sk_c, (N, rc), sm_c)]
                        for _ in range(2)]
        sk_shape = blocked_shape(M, N // 32) if swizzle else (M, N // 32)
        sm_shape = blocked_shape(N, M // 32) if swizzle else (N, M // 32)
        self.host = [torch.empty(s, dtype=torch.uint8, pin_memory=True) for s in ((M, N), sk_shape, (N, M), sm_shape)]
        self.dtypes = [torch.float8_e4m3fn, torch.float8_e8m0fnu, torch.float8_e4m3fn, torch.float8_e8m0fnu]
        with torch.cuda.device(dev):
            self.s_h2d, self.s_cmp, self.s_d2h = (torch.cuda.Stream() for _ in range(3))
        self.bytes_in = M * N * 2
        self.bytes_out = sum(h.numel() for h in self.host)

    def cast(self, x_host):
        """x_host: contiguous (M, N) bf16 host tensor (pinned for full copy speed).  Returns (qk, sk, qm, sm)
        as views of this object's pinned host buffers (overwritten by the next cast); complete on return."""
        lib = L.load()
        M, N, rc = self.M, self.N, self.rc
        assert x_host.shape == (M, N) and x_host.dtype == torch.bfloat16 and x_host.is_contiguous()
        qk_h, sk_h, qm_h, sm_h = self.host
        n_chunks = M // rc
        with torch.cuda.device(self.device):
            cur = torch.cuda.current_stream()
            for s in (self.s_h2d, self.s_cmp, self.s_d2h):
                s.wait_stream(cur)
            x_free = [None, None]     # event: the cast that read x_dev[b] is done
            out_free = [None, None]   # event: the copies out of out_dev[b] are done
            for i in range(n_chunks):
                b = i & 1
                r0 = i * rc
                with torch.cuda.stream(self.s_h2d):
                    if x_free[b] is not None:
                        self.s_h2d.wait_event(x_free[b])
                    self.x_dev[b].copy_(x_host[r0:r0 + rc], non_blocking=True)
                    x_ready = torch.cuda.Event()
                    x_ready.record(self.s_h2d)
                qk_d, sk_d, qm_d, sm_d = self.out_dev[b]
                with torch.cuda.stream(self.s_cmp):
                    self.s_cmp.wait_event(x_ready)
                    if out_free[b] is not None:
                        self.s_cmp.wait_event(out_free[b])
                    L.check(lib.qcc_mxfp8(self.x_dev[b].data_ptr(), rc, N, self.flags, qk_d.data_ptr(), sk_d.data_ptr(),
                                          qm_d.data_ptr(), sm_d.data_ptr(), self.s_cmp.cuda_stream), "mxfp8")
                    L.launch_count += 1
                    done = torch.cuda.Event()
                    done.record(self.s_cmp)
                    x_free[b] = done
                with torch.cuda.stream(self.s_d2h):
                    self.s_d2h.wait_event(done)
                    st = self.s_d2h.cuda_stream
                    qk_h[r0:r0 + rc].copy_(qk_d, non_blocking=True)                       # row slab
                    if self.swizzle:
                        sk_h[r0 // 128:(r0 + rc) // 128].copy_(sk_d, non_blocking=True)   # first-axis slab
                        w = (rc // 128) * 512                                             # second-axis slab
                        L.check(lib.qcc_copy2d_async(sm_h.data_ptr() + (r0 // 128) * 512, (M // 128) * 512, sm_d.data_ptr(),
                                                     w, w, sm_d.shape[0], 1, st), "copy2d sm")
                    else:
                        sk_h[r0:r0 + rc].copy_(sk_d, non_blocking=True)
                        w = rc // 32
                        L.check(lib.qcc_copy2d_async(sm_h.data_ptr() + r0 // 32, M // 32, sm_d.data_ptr(), w, w, N, 1, st),
                                "copy2d sm")
                    L.check(lib.qcc_copy2d_async(qm_h.data_ptr() + r0, M, qm_d.data_ptr(), rc, rc, N, 1, st), "copy2d qm")
                    ev = torch.cuda.Event()
                    ev.record(self.s_d2h)
                    out_free[b] = ev
            self.s_d2h.synchronize()
        return tuple(h.view(dt) for h, dt in zip(self.host, self.dtypes))


class HostShardCaster:
    """mxfp8_swizzle + nvfp4_swizzle (tensor-wide outer scale) of one rank's (rows, N) bf16 row shard that lives in
    pinned host memory; outputs come back to pinned host memory.  The MoE-activation flow of a row-sharded tensor.

    One call: the shard travels host -> device in row chunks; each chunk is cast to mxfp8 as it arrives by the kernel
    that also accumulates the shard's amax, and its mxfp8 outputs leave device -> host while the next chunk arrives.
    After the last chunk one warp exchanges the amax with the other ranks (`AmaxExchange`, peer memory) and forms the
    outer scale; the nvfp4 cast then runs chunk by chunk over the shard, which stayed on the device, with its outputs
    leaving behind it.  Chunks are multiples of 128 rows, so the result equals the one-shot casts bit for bit."""

    def __init__(self, rows, N, device, exchange, chunk_rows=8192, slots=1):
        assert rows % 128 == 0 and N % 64 == 0, "host shard caster wants rows % 128 == 0 and N % 64 == 0"
        assert slots >= 1
        self.rows, self.N, self.device, self.xchg = rows, N, torch.device(device), exchange
        rc = min(chunk_rows, rows)
        while rows % rc or rc % 128:
            rc -= 128
        self.rc = rc
        dev, u8 = self.device, torch.uint8
        shapes = ((rows, N), blocked_shape(rows, N // 32), (rows, N // 2), blocked_shape(rows, N // 16))
        # One slot = the device and pinned host buffers of one shard in flight.  With two slots `submit` can take the
        # next shard while the nvfp4 outputs of the one before are still leaving (see submit / result).
        self.slot = [{"x_dev": torch.empty((rows, N), dtype=torch.bfloat16, device=dev),
                      "out_dev": [torch.empty(sh, dtype=u8, device=dev) for sh in shapes],
                      "outer_dev": torch.empty((), dtype=torch.float32, device=dev),
                      "host": [torch.empty(sh, dtype=u8, pin_memory=True) for sh in shapes],
                      "outer_host": torch.empty((), dtype=torch.float32, pin_memory=True),
                      "read_done": None, "done": None} for _ in range(slots)]
        s0 = self.slot[0]
        self.x_dev, self.out_dev, self.outer_dev, self.host, self.outer_host = (s0["x_dev"], s0["out_dev"], s0["outer_dev"], s0["host"],
                                                                               s0["outer_host"])
        self.dtypes = [torch.float8_e4m3fn, torch.float8_e8m0fnu, torch.float4_e2m1fn_x2, torch.float8_e4m3fn]
        with torch.cuda.device(dev):
            self.s_h2d, self.s_cmp, self.s_d2h = (torch.cuda.Stream() for _ in range(3))
        self.bytes_in = rows * N * 2
        self.bytes_out = sum(h.numel() for h in self.host) + 4

    def cast(self, x_host):
        """x_host: contiguous (rows, N) bf16 host tensor (pinned for full copy speed).  Returns (mx_q, mx_scales, nv_q,
        nv_scales, outer_scale) as views of this object's pinned host buffers; complete on return."""
        self.submit(x_host, 0)
        return self.result(0)

    def result(self, slot=0):
        """Waits for the shard submitted into `slot` and returns its five outputs (views of the slot's pinned buffers,
        valid until the slot is submitted to again)."""
        sl = self.slot[slot]
        assert sl["done"] is not None, "nothing was submitted into this slot"
        sl["done"].synchronize()
        return tuple(h.view(dt) for h, dt in zip(sl["host"], self.dtypes)) + (sl["outer_host"],)

    def submit(self, x_host, slot=0):
        """Queues the whole flow for one shard into `slot` and returns without waiting.  With two slots used in turn
        (submit(a, 0); submit(b, 1); result(0); submit(c, 0); ...) the input copy of a shard overlaps the departure of the
        nvfp4 outputs of the shard before it, which a single shard cannot overlap with anything because they need the
        amax of ALL its rows.  Every rank of the exchange must submit in the same order.  The caller must have taken
        `result(slot)` of the slot's previous shard (its pinned output buffers are overwritten)."""
        lib = L.load()
        rows, N, rc = self.rows, self.N, self.rc
        assert x_host.shape == (rows, N) and x_host.dtype == torch.bfloat16 and x_host.is_contiguous()
        sl = self.slot[slot]
        x_dev, outer_dev, outer_host = sl["x_dev"], sl["outer_dev"], sl["outer_host"]
        mq_d, ms_d, nq_d, ns_d = sl["out_dev"]
        mq_h, ms_h, nq_h, ns_h = sl["host"]
        n_chunks = rows // rc
        ab = rc // 128                       # 128-row scale atoms rows per chunk
        flags = L.ROWWISE | L.SWIZZLE
        with torch.cuda.device(self.device):
            cur = torch.cuda.current_stream()
            for s in (self.s_h2d, self.s_cmp, self.s_d2h):
                s.wait_stream(cur)
            if sl["read_done"] is not None:      # the slot's previous shard: its last cast has read x_dev ...
                self.s_h2d.wait_event(sl["read_done"])
            if sl["done"] is not None:           # ... and its outputs have left the device buffers
                self.s_cmp.wait_event(sl["done"])
            for i in range(n_chunks):
                r0 = i * rc
                with torch.cuda.stream(self.s_h2d):
                    x_dev[r0:r0 + rc].copy_(x_host[r0:r0 + rc], non_blocking=True)
                    arrived = torch.cuda.Event()
                    arrived.record(self.s_h2d)
                with torch.cuda.stream(self.s_cmp):
                    self.s_cmp.wait_event(arrived)
                    L.check(lib.qcc_mxfp8_amax_xchg(x_dev[r0:r0 + rc].data_ptr(), rc, N, flags, mq_d[r0:r0 + rc].data_ptr(),
                                                    ms_d[i * ab:(i + 1) * ab].data_ptr(), self.xchg.own, self.s_cmp.cuda_stream),
                            "mxfp8_amax_xchg")
                    L.launch_count += 1
                    done = torch.cuda.Event()
                    done.record(self.s_cmp)
                with torch.cuda.stream(self.s_d2h):
                    self.s_d2h.wait_event(done)
                    mq_h[r0:r0 + rc].copy_(mq_d[r0:r0 + rc], non_blocking=True)
                    ms_h[i * ab:(i + 1) * ab].copy_(ms_d[i * ab:(i + 1) * ab], non_blocking=True)
            with torch.cuda.stream(self.s_cmp):
                self.xchg._pending = True
                L.check(lib.qcc_xchg_resolve(self.xchg._ref(), L.AMAX_NVFP4_SCALE | L.div_flag(), L.FMT_E4M3, outer_dev.data_ptr(),
                                             self.s_cmp.cuda_stream), "xchg_resolve")
                L.launch_count += 1
                for i in range(n_chunks):
                    r0 = i * rc
                    L.check(lib.qcc_nvfp4(x_dev[r0:r0 + rc].data_ptr(), rc, N, outer_dev.data_ptr(), 0, L.SWIZZLE | L.div_flag(), None,
                                          nq_d[r0:r0 + rc].data_ptr(), ns_d[i * ab:(i + 1) * ab].data_ptr(), self.s_cmp.cuda_stream),
                            "nvfp4")
                    L.launch_count += 1
                    done = torch.cuda.Event()
                    done.record(self.s_cmp)
                    with torch.cuda.stream(self.s_d2h):
                        self.s_d2h.wait_event(done)
                        nq_h[r0:r0 + rc].copy_(nq_d[r0:r0 + rc], non_blocking=True)
                        ns_h[i * ab:(i + 1) * ab].copy_(ns_d[i * ab:(i + 1) * ab], non_blocking=True)
                        if i == 0:
                            outer_host.copy_(outer_dev, non_blocking=True)
                sl["read_done"] = done                      # the last nvfp4 chunk: x_dev may be overwritten after it
            sl["done"] = torch.cuda.Event()
            sl["done"].record(self.s_d2h)
        return slot
