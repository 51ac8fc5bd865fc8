"""Host-buffer entry to the mxfp8 two-direction cast: pinned host bf16 in, pinned host outputs back.

This is the call a user with data in host memory makes; it owns the device staging buffers and the
pinned output buffers, so repeated casts allocate nothing.  Each cast copies x to the device,
launches the CUDA cast and copies the four outputs back; it returns after the outputs are complete.
"""
import torch

from . import _lib as L
from .recipes import blocked_shape


class HostMxfp8Caster:
    """mxfp8_dim_km(_swizzle) for an (M, N) bf16 matrix that lives in (pinned) host memory."""

    def __init__(self, M, N, device, swizzle=True, mode="rceil"):
        assert M % 32 == 0 and N % 32 == 0
        self.M, self.N, self.device = M, N, torch.device(device)
        self.flags = L.ROWWISE | L.COLWISE | (L.SWIZZLE if swizzle else 0) | (L.FLOOR if mode == "floor" else 0)
        sk_shape = blocked_shape(M, N // 32) if swizzle else (M, N // 32)
        sm_shape = blocked_shape(N, M // 32) if swizzle else (N, M // 32)
        shapes = [(M, N), sk_shape, (N, M), sm_shape]
        self.x_dev = torch.empty((M, N), dtype=torch.bfloat16, device=self.device)
        self.dev = [torch.empty(s, dtype=torch.uint8, device=self.device) for s in shapes]
        self.host = [torch.empty(s, dtype=torch.uint8, pin_memory=True) for s in shapes]
        self.dtypes = [torch.float8_e4m3fn, torch.float8_e8m0fnu, torch.float8_e4m3fn, torch.float8_e8m0fnu]

    def cast(self, x_host):
        """x_host: contiguous (M, N) bf16 host tensor (pinned for full copy speed).  Returns
        (qk, sk, qm, sm) as views of this object's pinned host buffers (overwritten by the next cast)."""
        lib = L.load()
        assert x_host.shape == (self.M, self.N) and x_host.dtype == torch.bfloat16 and x_host.is_contiguous()
        with torch.cuda.device(self.device):
            stream = torch.cuda.current_stream(self.device)
            self.x_dev.copy_(x_host, non_blocking=True)
            L.check(lib.qcc_mxfp8(self.x_dev.data_ptr(), self.M, self.N, self.flags, self.dev[0].data_ptr(),
                                  self.dev[1].data_ptr(), self.dev[2].data_ptr(), self.dev[3].data_ptr(),
                                  stream.cuda_stream), "mxfp8")
            L.launch_count += 1
            for h, d in zip(self.host, self.dev):
                h.copy_(d, non_blocking=True)
            stream.synchronize()
        return tuple(h.view(dt) for h, dt in zip(self.host, self.dtypes))
