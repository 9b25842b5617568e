"""Seeded synthetic voxel scenes standing in for the reference's licensed datasets.

The reference evaluates on SemanticKITTI / Waymo (outdoor LiDAR, 0.1 m voxels,
``datasets/prepare_kitti.py:29``) and ScanNet (indoor, 0.02 m voxels,
``datasets/prepare_scannet.py:24``).  None of them can be shipped, so every workload here
is generated from ``numpy.random.default_rng(seed)`` with the same voxel sizes, extents
and surface-like (geometrically continuous) occupancy.

All generators return ``int32 [N, 3]`` (x, y, z) coordinates without a batch column (the
reference has none, ``csrc/spira/cuda/kernels/compress.cuh:17-22``), de-duplicated, shuffled
like ``scripts/loaders.py:18`` and shifted by a fixed ``MARGIN`` per axis instead of the
loader's min->0 shift (``scripts/loaders.py:21-22``).  ``MARGIN`` is a multiple of the
largest network stride (16) and larger than the largest kernel reach, so no packed-key
neighbour query ever under- or overflows a bit field.
"""
from __future__ import annotations

import numpy as np

MARGIN = 32


def _finish(cells: np.ndarray, rng: np.random.Generator, limit: int | None = None) -> np.ndarray:
    """De-duplicate (keeping first-seen order), optionally trim the tail, shift and shuffle."""
    cells = np.asarray(cells, dtype=np.int64)
    _, first = np.unique(cells, axis=0, return_index=True)
    cells = cells[np.sort(first)]
    if limit is not None:
        if len(cells) < limit:
            raise ValueError(f"generator produced {len(cells)} voxels, fewer than the requested {limit}")
        cells = cells[:limit]
    cells = cells - cells.min(axis=0, keepdims=True) + MARGIN
    cells = cells[rng.permutation(len(cells))]
    return np.ascontiguousarray(cells, dtype=np.int32)


def _plane_patch(rng, centre, size, grid):
    """All voxels of a bounded, densely sampled planar patch with a random orientation."""
    n = rng.normal(size=3)
    n /= np.linalg.norm(n)
    a = np.cross(n, [1.0, 0.0, 0.0] if abs(n[0]) < 0.9 else [0.0, 1.0, 0.0])
    a /= np.linalg.norm(a)
    b = np.cross(n, a)
    u = np.arange(-size / 2, size / 2, 0.35)
    uu, vv = np.meshgrid(u, u, indexing="ij")
    pts = centre[None, :] + uu.reshape(-1, 1) * a[None, :] + vv.reshape(-1, 1) * b[None, :]
    pts = np.floor(pts).astype(np.int64)
    ok = np.all((pts >= 0) & (pts < grid), axis=1)
    return pts[ok]


def _sphere_shell(rng, centre, radius, grid):
    n = int(4 * np.pi * radius * radius * 10)
    d = rng.normal(size=(n, 3))
    d /= np.linalg.norm(d, axis=1, keepdims=True)
    pts = np.floor(centre[None, :] + radius * d).astype(np.int64)
    ok = np.all((pts >= 0) & (pts < grid), axis=1)
    return pts[ok]


def planes_and_spheres(seed: int = 0, n_voxels: int = 50_000, grid: int = 512) -> np.ndarray:
    """Single-layer workload: 8 random plane patches + 4 random sphere shells in a ``grid``^3 box.

    The union is trimmed to exactly ``n_voxels`` by dropping trailing voxels of the last
    shape (never by random thinning, which would destroy surface continuity).  z reaches
    ~``grid`` so 64-bit packed keys are required when ``grid`` > 224 (8-bit z field).
    """
    rng = np.random.default_rng(seed)
    lim = grid - 2 * MARGIN
    parts = []
    for _ in range(4):
        r = rng.uniform(17.0, 21.0)
        c = rng.uniform(r + 1, lim - r - 1, size=3)
        parts.append(_sphere_shell(rng, c, r, lim))
    for _ in range(8):
        c = rng.uniform(60, lim - 60, size=3)
        parts.append(_plane_patch(rng, c, 75.0, lim))
    return _finish(np.concatenate(parts), rng, n_voxels)


def _box_surface(rng, lo, hi, step):
    """Dense surface samples of an axis-aligned box [lo, hi]."""
    pts = []
    for ax in range(3):
        o = [i for i in range(3) if i != ax]
        u = np.arange(lo[o[0]], hi[o[0]] + step, step)
        v = np.arange(lo[o[1]], hi[o[1]] + step, step)
        uu, vv = np.meshgrid(u, v, indexing="ij")
        for w in (lo[ax], hi[ax]):
            p = np.empty((uu.size, 3))
            p[:, ax] = w
            p[:, o[0]] = uu.ravel()
            p[:, o[1]] = vv.ravel()
            pts.append(p)
    return np.concatenate(pts)


def _ring_sweep(rng, half_extent, z_ground, n_beams=64, shift=(0.0, 0.0)):
    """Ground returns of a spinning ``n_beams`` LiDAR: concentric rings around the sensor."""
    sensor_h = 1.73
    elev = np.deg2rad(np.linspace(-24.8, -0.9, n_beams))
    radii = sensor_h / np.tan(-elev)
    radii = radii[radii < half_extent * 1.35]
    pts = []
    for r in radii:
        n = max(64, int(2 * np.pi * r / 0.04))
        az = np.linspace(0, 2 * np.pi, n, endpoint=False) + rng.uniform(0, 0.01)
        p = np.stack([r * np.cos(az) + shift[0], r * np.sin(az) + shift[1],
                      np.full(n, z_ground) + rng.normal(0, 0.015, n)], axis=1)
        pts.append(p)
    return np.concatenate(pts)


def lidar_scene(seed: int = 1, half_extent: float = 51.2, z_range=(-4.0, 2.0), voxel: float = 0.1,
                n_boxes: int = 30, sweeps: int = 1, ground_half: float = 9.5) -> np.ndarray:
    """LiDAR-like outdoor scene: ring pattern + dense ground patch + random boxes (~120k voxels).

    ``sweeps`` > 1 stacks several ring patterns with small random ego shifts (multi-sweep
    aggregation, as in the SECOND-style workload).
    """
    rng = np.random.default_rng(seed)
    z_ground = -1.73
    pts = []
    for s in range(sweeps):
        shift = (0.0, 0.0) if s == 0 else tuple(rng.normal(0, 0.6, 2))
        pts.append(_ring_sweep(rng, half_extent, z_ground, shift=shift))
    g = np.arange(-ground_half, ground_half, voxel / 2)
    gx, gy = np.meshgrid(g, g, indexing="ij")
    pts.append(np.stack([gx.ravel(), gy.ravel(), np.full(gx.size, z_ground)], axis=1))
    for _ in range(n_boxes):
        size = rng.uniform([1.4, 1.2, 1.0], [3.4, 1.9, 1.7])
        c = np.append(rng.uniform(-half_extent * 0.85, half_extent * 0.85, 2), z_ground + size[2] / 2)
        pts.append(_box_surface(rng, c - size / 2, c + size / 2, voxel / 2))
    p = np.concatenate(pts)
    ok = (np.abs(p[:, 0]) < half_extent) & (np.abs(p[:, 1]) < half_extent) & (p[:, 2] >= z_range[0]) & (p[:, 2] < z_range[1])
    cells = np.floor(p[ok] / voxel).astype(np.int64)
    return _finish(cells, rng)


def room_scene(seed: int = 5, size=(8.0, 8.0, 3.0), voxel: float = 0.02, n_boxes: int = 20) -> np.ndarray:
    """Indoor room: floor, ceiling, 4 walls, furniture boxes, voxelised at 0.02 m (~250k voxels)."""
    rng = np.random.default_rng(seed)
    size = np.asarray(size)
    shell = np.floor(_box_surface(rng, np.zeros(3), size - voxel, voxel / 2) / voxel + 1e-6).astype(np.int64)
    # a scan never covers a whole room: keep one third of the shell, in 0.8 m blocks
    block = shell // 40
    shell = shell[(block[:, 0] + block[:, 1] + block[:, 2]) % 3 == 0]
    pts = []
    for _ in range(n_boxes):
        s = rng.uniform([0.3, 0.3, 0.3], [0.8, 0.65, 0.75])
        lo = np.append(rng.uniform(0.1, size[:2] - s[:2] - 0.1), 0.0)
        pts.append(_box_surface(rng, lo, lo + s, voxel / 2))
    cells = np.concatenate([shell, np.floor(np.concatenate(pts) / voxel + 1e-6).astype(np.int64)])
    return _finish(cells, rng)


def multisweep_scene(seed: int = 10) -> np.ndarray:
    """SECOND-style input: 5 stacked ring sweeps, x,y in [-75,75] m, z in [-2,4] m (~300k voxels)."""
    return lidar_scene(seed, half_extent=75.0, z_range=(-2.0, 4.0), sweeps=5, n_boxes=42, ground_half=14.0)


def features(n: int, channels: int, seed: int, kind: str = "normal") -> np.ndarray:
    rng = np.random.default_rng(seed + 7919)
    x = rng.normal(size=(n, channels)) if kind == "normal" else rng.uniform(0.0, 1.0, size=(n, channels))
    return x.astype(np.float16)
