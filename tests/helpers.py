"""Shared test helpers: golden-vector access, raw-byte comparison, seeded inputs."""
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "gold_vectors.npz")
_golden = None


def golden():
    global _golden
    if _golden is None:
        _golden = np.load(GOLDEN)
    return _golden


def golden_cases():
    return [str(c) for c in golden()["cases"]]


def golden_x(tag):
    return torch.from_numpy(golden()[f"{tag}/x"].copy()).view(torch.bfloat16)


def golden_rht(tag):
    """The 16x16 bf16 transform matrix of a golden case."""
    return torch.from_numpy(golden()[f"{tag}/rht"].copy()).view(torch.bfloat16)


def golden_out(tag, fn, i):
    return torch.from_numpy(golden()[f"{tag}/{fn}/{i}"].copy())


def golden_n_outputs(tag, fn):
    n = 0
    while f"{tag}/{fn}/{n}" in golden().files:
        n += 1
    return n


def raw(t):
    """Raw bits of a tensor in the layout the golden file uses."""
    t = t.detach().cpu().contiguous()
    if t.dtype in (torch.int32, torch.int16, torch.uint8):
        return t
    if t.dtype == torch.float32:
        return t.view(torch.int32)
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16)
    return t.view(torch.uint8)


def assert_same_bits(got, want, what=""):
    g, w = raw(got), raw(want) if isinstance(want, torch.Tensor) else want
    assert tuple(g.shape) == tuple(w.shape), f"{what}: shape {tuple(g.shape)} != {tuple(w.shape)}"
    assert g.dtype == w.dtype, f"{what}: raw dtype {g.dtype} != {w.dtype}"
    if not torch.equal(g, w):
        bad = (g != w).nonzero()
        first = tuple(bad[0].tolist()) if bad.numel() else ()
        raise AssertionError(
            f"{what}: {bad.shape[0]} of {g.numel()} elements differ; first at {first}: "
            f"got {g[first].item():#x} want {w[first].item():#x}"
        )


def same_outputs(got, want, what=""):
    assert len(got) == len(want), f"{what}: {len(got)} outputs != {len(want)}"
    for i, (g, w) in enumerate(zip(got, want)):
        assert g.dtype == w.dtype, f"{what}[{i}]: dtype {g.dtype} != {w.dtype}"
        assert_same_bits(g, w, f"{what}[{i}]")
