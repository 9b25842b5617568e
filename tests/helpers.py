"""Shared input builders for the GPU parity tests."""
import numpy as np
import torch

import spira_oracle as O


def cloud(seed, n, lo=32, hi=96, zhi=None):
    rng = np.random.default_rng(seed)
    c = rng.integers(lo, hi, size=(n, 3))
    if zhi is not None:
        c[:, 2] = rng.integers(lo, zhi, size=n)
    return np.unique(c, axis=0).astype(np.int32)[rng.permutation(len(np.unique(c, axis=0)))]


def surface(seed, n=20000):
    """A wavy sheet plus a slab: surface-like occupancy with ~9 neighbours per voxel."""
    rng = np.random.default_rng(seed)
    x = rng.uniform(0, 160, n)
    y = rng.uniform(0, 160, n)
    z = 20 + 8 * np.sin(x / 17.0) + 6 * np.cos(y / 11.0)
    c = np.stack([x, y, z], axis=1)
    c2 = np.stack([rng.uniform(40, 80, n // 4), np.full(n // 4, 50.0), rng.uniform(0, 40, n // 4)], axis=1)
    c = np.floor(np.concatenate([c, c2])).astype(np.int64) + 32
    c = np.unique(c, axis=0)
    return c[rng.permutation(len(c))].astype(np.int32)


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def keys_to_torch(keys):
    """uint32/uint64 numpy keys -> int32/int64 torch tensor with the same bits (on the GPU)."""
    return torch.from_numpy(keys.view(np.int32 if keys.dtype.itemsize == 4 else np.int64).copy()).cuda()


def keys_from_torch(t):
    a = t.cpu().numpy()
    return a.view(np.uint32 if a.dtype.itemsize == 4 else np.uint64)


def assert_features_close(got, want, rtol=1e-2, atol=1e-3):
    """Tolerance of the feature path: 1e-2 relative / 1e-3 absolute (fp16 in/out, fp32 accumulate)."""
    g = got.float().cpu()
    w = want.float().cpu()
    assert g.shape == w.shape
    bad = (g - w).abs() > atol + rtol * w.abs()
    assert not bad.any(), f"{int(bad.sum())} / {bad.numel()} elements out of tolerance; max abs err {(g - w).abs().max().item():.4g}"
