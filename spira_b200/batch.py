"""Several scenes per launch: a batch is ONE sparse tensor whose scenes lie side by side.

The reference has no batch dimension (``csrc/spira/cuda/kernels/compress.cuh:17-22`` packs ``[N, 3]`` coordinates
without a batch column) and runs one scene at a time (``scripts/end_to_end_experiment.py:191-207``).  A sparse convolution
is local, so scenes that are shifted apart by more than the reach of the deepest layer never interact: placing B
scenes on a grid in the x / y plane turns every kernel of the engine -- sort, down-sampling, map search, grouping,
both convolution dataflows -- into a B-scene launch without touching it.  The deep levels of a network, which hold
only a few thousand voxels of one scene and leave most SMs idle, get B times the tiles per launch, and the host-side
cost of a step is paid once per batch.

The shift of every scene is a multiple of ``align`` (the largest stride of the network), so down-sampled coordinates
of a scene keep their relative positions and the batch computes, row for row, what the scenes compute on their own
(output-stationary layers: bit for bit).
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch

__all__ = ["merge_scenes", "scene_ids", "split_rows"]


def _grid(n_scenes: int) -> Tuple[int, int]:
    nx = 1
    while nx * nx < n_scenes:
        nx += 1
    return nx, (n_scenes + nx - 1) // nx


def merge_scenes(coordinates: Sequence[torch.Tensor], features: Sequence[torch.Tensor], *, gap: int = 64, align: int = 64,
                 double: bool = False):
    """``B`` scenes (``[N_b, 3] int32`` coordinates, ``[N_b, C]`` features) -> one scene.

    Scene ``b`` moves to cell ``(b % nx, b // nx)`` of a grid in x / y whose pitch is the largest scene extent plus
    ``gap`` voxels, rounded up to a multiple of ``align`` (choose ``align`` as a multiple of the network's largest
    stride and ``gap`` beyond its largest kernel reach).  Returns ``(coordinates, features, pitch, (nx, ny))``; raises
    if the grid does not fit the key layout (12 bits per axis for 32-bit keys, 24 for 64-bit keys)."""
    if len(coordinates) != len(features) or len(coordinates) == 0:
        raise ValueError("merge_scenes needs as many feature tensors as coordinate tensors, and at least one")
    extent = 0
    for c in coordinates:
        if c.dim() != 2 or c.shape[1] != 3:
            raise ValueError("coordinates must be [N, 3]")
        if c.shape[0]:
            extent = max(extent, int(c[:, :2].max().item()) + 1)
    pitch = (extent + gap + align - 1) // align * align
    nx, ny = _grid(len(coordinates))
    limit = 1 << (24 if double else 12)
    if max(nx, ny) * pitch > limit:
        raise ValueError(f"{len(coordinates)} scenes of extent {extent} need {max(nx, ny) * pitch} cells per axis; the "
                         f"{'64' if double else '32'}-bit key layout holds {limit}")
    shifted = []
    for b, c in enumerate(coordinates):
        shift = torch.tensor([(b % nx) * pitch, (b // nx) * pitch, 0], dtype=c.dtype, device=c.device)
        shifted.append(c + shift)
    return torch.cat(shifted), torch.cat(list(features)), pitch, (nx, ny)


def scene_ids(coordinates: torch.Tensor, pitch: int, grid: Tuple[int, int]) -> torch.Tensor:
    """Scene index of every row of a merged ``[N, 3]`` coordinate tensor (any stride level: cells are ``pitch`` wide)."""
    return (coordinates[:, 0] // pitch + (coordinates[:, 1] // pitch) * grid[0]).to(torch.int64)


def split_rows(rows: torch.Tensor, ids: torch.Tensor, n_scenes: int) -> List[torch.Tensor]:
    """Rows of a merged result per scene, each in the order the scene has on its own (sorted keys keep their relative
    order under the shift)."""
    return [rows[ids == b] for b in range(n_scenes)]
