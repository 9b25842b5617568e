"""CPU restatement of the reference's kernel-map + sparse-convolution hot path.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this module; it is the
checker used by ``tests/``, by the smoke entry and by the CPU-baseline leg of ``bench.py``.

The reference (SPIN-Research-Group/Spira) has no CPU implementation of this path
(``source/spira/nn/functional/indexing.py:27`` raises for non-CUDA tensors) and ships no
golden vectors, so this file restates the algorithm of its CUDA sources in numpy / torch-CPU.
Parity pin: the restatement is compared on the GPU box against the reference's own native
module built from its unmodified sources (``oracle/build_ref.py`` -> ``oracle/_ref/_C.so``);
fixtures produced that way are committed under ``tests/golden/``.

Every function cites the reference lines it follows (paths relative to the reference root).
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import numpy as np

# ----------------------------------------------------------------------------------------------
# packed keys -- source/csrc/spira/compress_layout.h:12-44
# ----------------------------------------------------------------------------------------------
LAYOUT = {
    4: dict(dtype=np.uint32, zb=8, yb=12, xb=12),
    8: dict(dtype=np.uint64, zb=16, yb=24, xb=24),
}


def _lay(width: int):
    L = LAYOUT[width]
    return L["dtype"], L["zb"], L["zb"] + L["yb"], L


def pack(coords: np.ndarray, width: int = 4) -> np.ndarray:
    """key = x << X_SHIFT | y << Y_SHIFT | z, z least significant, no range masking.

    Follows ``source/csrc/spira/cuda/kernels/compress.cuh:18-22`` (int32 -> unsigned cast, shift, or).
    """
    dt, ys, xs, _ = _lay(width)
    c = np.asarray(coords, dtype=np.int32).astype(np.int64).astype(dt)  # two's-complement cast like static_cast<CT>
    return (c[:, 0] << dt(xs)) | (c[:, 1] << dt(ys)) | c[:, 2]


def unpack(keys: np.ndarray) -> np.ndarray:
    """Inverse of :func:`pack` (``compress.cuh:35-44``)."""
    width = keys.dtype.itemsize
    dt, ys, xs, L = _lay(width)
    k = keys.view(dt)
    x = (k >> dt(xs)) & dt((1 << L["xb"]) - 1)
    y = (k >> dt(ys)) & dt((1 << L["yb"]) - 1)
    z = k & dt((1 << L["zb"]) - 1)
    return np.stack([x, y, z], axis=1).astype(np.int32)


def flat_sort(coords: np.ndarray, double: bool = False) -> Tuple[np.ndarray, np.ndarray]:
    """Packed keys sorted ascending as unsigned + the int32 permutation.

    ``source/csrc/spira/cuda/functions/arg_sort_coodrinates.cu:35-88`` (Compress, FillRange,
    radix SortPairs over all key bits -- a stable sort).
    """
    keys = pack(coords, 8 if double else 4)
    idx = np.argsort(keys, kind="stable").astype(np.int32)
    return keys[idx], idx


def stride_mask(stride: Sequence[int], width: int):
    """Mask clearing the low log2(stride) bits of each field.

    ``source/csrc/spira/torch/cuda_arg_sort_coordinates.cu:86-89`` -- strides must be powers of two.
    """
    dt, ys, xs, L = _lay(width)
    xm = ((1 << L["xb"]) - 1) & ~(int(stride[0]) - 1)
    ym = ((1 << L["yb"]) - 1) & ~(int(stride[1]) - 1)
    zm = ((1 << L["zb"]) - 1) & ~(int(stride[2]) - 1)
    return dt((xm << xs) | (ym << ys) | zm)


def downsample(keys: np.ndarray, stride: Sequence[int]) -> np.ndarray:
    """unique(sort(key & mask)): ``cuda_arg_sort_coordinates.cu:68-105``; coordinates stay in level-0 units."""
    width = keys.dtype.itemsize
    dt = LAYOUT[width]["dtype"]
    return np.unique(keys.view(dt) & stride_mask(stride, width))


def streamed_output_generate(keys: np.ndarray, strides: Sequence[Sequence[int]]) -> List[np.ndarray]:
    """Every level is derived from the level-0 keys (``cuda_arg_sort_coordinates.cu:107-200``)."""
    return [downsample(keys, s) for s in strides]


# ----------------------------------------------------------------------------------------------
# offsets -- source/csrc/spira/torch/cuda_sparse_convolution_mapping.cu:10-49
# ----------------------------------------------------------------------------------------------
def axis_range(k: int) -> Tuple[int, int]:
    lo = -(k // 2) if k % 2 == 1 else -(k // 2) + 1
    return lo, k // 2


def xy_offsets(kernel_size: Sequence[int], src_stride: Sequence[int], width: int) -> np.ndarray:
    """Packed xy offsets (x-major, then y) with z preset to kz_min*sz; wrapping unsigned arithmetic."""
    dt, ys, xs, _ = _lay(width)
    bits = 8 * width
    x0, x1 = axis_range(kernel_size[0])
    y0, y1 = axis_range(kernel_size[1])
    z0, _ = axis_range(kernel_size[2])
    out = []
    for ix in range(x0, x1 + 1):
        for iy in range(y0, y1 + 1):
            v = ix * src_stride[0] * (1 << xs) + iy * src_stride[1] * (1 << ys) + z0 * src_stride[2]
            out.append(v % (1 << bits))
    return np.asarray(out, dtype=dt)


def n_offsets(kernel_size: Sequence[int]) -> Tuple[int, int]:
    return kernel_size[0] * kernel_size[1], kernel_size[2]


def aligned(n: int) -> int:
    """T_al = ceil(T/128)*128 (``cuda_sparse_convolution_mapping.cu:223``)."""
    return (n + 127) // 128 * 128


# ----------------------------------------------------------------------------------------------
# kernel-map search -- source/csrc/spira/cuda/kernels/query_sorted.cuh:8-163
# ----------------------------------------------------------------------------------------------
def search_hits(src: np.ndarray, tgt: np.ndarray, kernel_size, src_stride, emulate_reference_walk: bool = False) -> np.ndarray:
    """hits[o, iz, t] = index of the source matching tgt[t] + off[o] + iz*sz (wrapping), or -1.

    Default: exact lookup of every wrapped query (what the z-walk of ``query_sorted.cuh:35-54``
    computes whenever the first query of a column does not wrap past the last source).
    ``emulate_reference_walk=True`` additionally reproduces the walk's one systematic miss:
    when ``lower_bound`` of the first query of a column returns ``num_sources`` the
    ``index < num_sources`` guard (``query_sorted.cuh:47-49``) reports every later z-step of
    that column as -1 even if the wrapped query comes back into range.
    """
    width = src.dtype.itemsize
    dt = LAYOUT[width]["dtype"]
    src = src.view(dt)
    tgt = tgt.view(dt)
    S = len(src)
    off = xy_offsets(kernel_size, src_stride, width)
    nxy, kz = n_offsets(kernel_size)
    sz = dt(src_stride[2])
    hits = np.full((nxy, kz, len(tgt)), -1, dtype=np.int32)
    if S == 0 or len(tgt) == 0:
        return hits
    with np.errstate(over="ignore"):
        for o in range(nxy):
            q = tgt + off[o]
            dead = None
            for iz in range(kz):
                i = np.searchsorted(src, q, side="left")
                ok = i < S
                hit = ok & (src[np.minimum(i, S - 1)] == q)
                if emulate_reference_walk:
                    if iz == 0:
                        dead = ~ok
                    else:
                        hit &= ~dead
                hits[o, iz] = np.where(hit, i, -1)
                q = q + sz
    return hits


def kernel_map(src, tgt, kernel_size, src_stride, layout: str = "os", emulate_reference_walk: bool = False) -> np.ndarray:
    """Dense int32 map padded to T_al rows with -1.

    ``layout='os'``: ``[T_al, K]``, column ``iz*nxy + o`` (``query_sorted.cuh:150,159``).
    ``layout='ws'``: ``[K, T_al]``, row ``kz*o + iz`` (``query_sorted.cuh:42,52``).
    """
    hits = search_hits(src, tgt, kernel_size, src_stride, emulate_reference_walk)
    nxy, kz, T = hits.shape
    Tal = aligned(T)
    if layout == "ws":
        m = np.full((nxy * kz, Tal), -1, dtype=np.int32)
        m[:, :T] = hits.reshape(nxy * kz, T)
        return m
    m = np.full((Tal, kz * nxy), -1, dtype=np.int32)
    m[:T] = hits.transpose(2, 1, 0).reshape(T, kz * nxy)
    return m


def triples(dense: np.ndarray, layout: str, kernel_size) -> np.ndarray:
    """Sorted (in, out, natural offset index k=(ix*ky+iy)*kz+iz) triples of a dense map."""
    nxy, kz = n_offsets(kernel_size)
    if layout == "ws":
        k, t = np.nonzero(dense >= 0)
        i = dense[k, t]
    else:
        t, c = np.nonzero(dense >= 0)
        i = dense[t, c]
        k = (c % nxy) * kz + c // nxy
    tr = np.stack([i.astype(np.int64), t.astype(np.int64), k.astype(np.int64)], axis=1)
    return tr[np.lexsort((tr[:, 2], tr[:, 1], tr[:, 0]))]


def ws_structures(dense_ws: np.ndarray, num_sources: int, num_targets: int, quantum: int = 128):
    """Post-processing of a ``[K, T_al]`` map for the fused weight-stationary dataflow.

    ``source/csrc/spira/cuda/functions/query_sorted_index.cu:146-209`` (full) and ``:290-348``
    (half: submanifold and odd K -> only the first (K+1)/2 rows are compacted,
    ``cuda_sparse_convolution_mapping.cu:269``); prefix sums follow
    ``source/csrc/spira/cuda/kernels/quantifier_wstat.cuh:8-44``.
    Returns ``(nbmaps[2, nnz] (row 0 = in, row 1 = out), nbsizes, naddrs, qnaddrs, mapsize, qmapsize)``.
    """
    K = dense_ws.shape[0]
    half = (num_sources == num_targets) and (K % 2 == 1)
    rows = (K + 1) // 2 if half else K
    ins, outs, sizes = [], [], []
    for k in range(rows):
        t = np.nonzero(dense_ws[k] >= 0)[0]
        ins.append(dense_ws[k, t])
        outs.append(t.astype(np.int32))
        sizes.append(len(t))
    nbsizes = np.asarray(sizes, dtype=np.int32)
    naddrs = np.concatenate([[0], np.cumsum(nbsizes)]).astype(np.int32)
    q = (nbsizes + quantum - 1) // quantum * quantum
    qnaddrs = np.concatenate([[0], np.cumsum(q)]).astype(np.int32)
    nbmaps = np.stack([np.concatenate(ins), np.concatenate(outs)]).astype(np.int32)
    return nbmaps, nbsizes, naddrs, qnaddrs, int(naddrs[-1]), int(qnaddrs[-1])


def gs_masks(dense_ws: np.ndarray, num_sources: int, num_targets: int):
    """source_masks[K,S], target_masks[K,T]: rank of a pair inside its offset's list, -1 elsewhere.

    ``source/csrc/spira/cuda/kernels/generate_masks_from_kernel_map.cuh:9-62``.
    """
    K = dense_ws.shape[0]
    sm = np.full((K, num_sources), -1, dtype=np.int32)
    tm = np.full((K, num_targets), -1, dtype=np.int32)
    sizes = np.zeros(K, dtype=np.int32)
    for k in range(K):
        t = np.nonzero(dense_ws[k, :num_targets] >= 0)[0]
        r = np.arange(len(t), dtype=np.int32)
        sm[k, dense_ws[k, t]] = r
        tm[k, t] = r
        sizes[k] = len(t)
    return sm, tm, sizes


def gs_masks_half(rows_map: np.ndarray, rows_masks: int, num_sources: int, num_targets: int):
    """Mask format of a mirrored map: ``rows_map`` holds the listed rows (the first half of ``rows_masks`` rows, centre
    included when ``rows_masks`` is odd).  The pair (s, t) with rank r of listed row o is written to row o as in
    :func:`gs_masks` and to the mirrored row ``rows_masks - 1 - o`` with the roles exchanged, unless o is its own image.

    ``source/csrc/spira/cuda/kernels/generate_masks_from_kernel_map.cuh:36-62``."""
    listed = rows_map.shape[0]
    sm = np.full((rows_masks, num_sources), -1, dtype=np.int32)
    tm = np.full((rows_masks, num_targets), -1, dtype=np.int32)
    sizes = np.zeros(listed, dtype=np.int32)
    for o in range(listed):
        t = np.nonzero(rows_map[o, :num_targets] >= 0)[0]
        s_ = rows_map[o, t]
        r = np.arange(len(t), dtype=np.int32)
        sm[o, s_] = r
        tm[o, t] = r
        if 2 * o + 1 != rows_masks:
            sm[rows_masks - 1 - o, t] = r
            tm[rows_masks - 1 - o, s_] = r
        sizes[o] = len(t)
    return sm, tm, sizes


def l1_permutation(kernel_size: Sequence[int], dataflow: int):
    """``position[k]`` of natural offset ``k = (ix*ky + iy)*kz + iz`` in the row order of the hybrid dataflows 3-8: offsets
    with L1 norm below ``(dataflow - 1) // 2`` first, the others behind them, both in natural order.  The number of
    dense rows is what the reference reads from ``position[0]``.

    ``source/csrc/spira/torch/cuda_sparse_convolution_mapping.cu:159-209`` (``generate_indexes_L1``) and ``:682`` / ``:788``."""
    threshold = (int(dataflow) - 1) // 2
    l1 = []
    (x0, x1), (y0, y1), (z0, z1) = (axis_range(k) for k in kernel_size)
    for x in range(x0, x1 + 1):
        for y in range(y0, y1 + 1):
            for z in range(z0, z1 + 1):
                l1.append(abs(x) + abs(y) + abs(z))
    front = sum(1 for v in l1 if v < threshold)
    position, f, b = [], 0, front
    for v in l1:
        if v < threshold:
            position.append(f)
            f += 1
        else:
            position.append(b)
            b += 1
    return np.asarray(position, dtype=np.int32), int(position[0])


def hybrid_structures(dense_ws: np.ndarray, num_sources: int, num_targets: int, kernel_size, dataflow: int):
    """The 9-tuple slots of a hybrid dataflow (3-8) from the natural-order ``[K, T_al]`` map.

    Rows are permuted to L1-norm order (``BinarySearch_kz_hybrid``, ``source/csrc/spira/cuda/kernels/query_sorted.cuh:58-113``);
    the first half of the rows behind the ``dense`` leading ones is compacted into pair lists for odd dataflows
    (``query_sorted_index.cu:777-908``) or ranked into mirrored masks for even ones (``:647-775``); dataflows above 4 return
    the leading rows transposed, ``[T_al, dense]`` (``cuda_sparse_convolution_mapping.cu:770-773,884-887``).
    Returns a dict with ``map`` and, by parity of the dataflow, ``nbmaps / nbsizes / naddrs / qnaddrs / sizes`` or
    ``smask / tmask / nbsizes``, plus ``permuted`` (the whole permuted map) and ``dense``."""
    K = dense_ws.shape[0]
    position, dense = l1_permutation(kernel_size, dataflow)
    permuted = np.empty_like(dense_ws)
    permuted[position] = dense_ws
    half = (K - dense) // 2
    rows = permuted[dense:dense + half]
    out = dict(permuted=permuted, dense=dense,
               map=np.ascontiguousarray(permuted[:dense].T) if dataflow > 4 else permuted)
    if dataflow % 2 == 1:
        ins, outs, sizes = [], [], []
        for o in range(half):
            t = np.nonzero(rows[o] >= 0)[0]
            ins.append(rows[o, t])
            outs.append(t.astype(np.int32))
            sizes.append(len(t))
        nbsizes = np.asarray(sizes, dtype=np.int32)
        naddrs = np.concatenate([[0], np.cumsum(nbsizes)]).astype(np.int32)
        q = (nbsizes + 127) // 128 * 128
        qnaddrs = np.concatenate([[0], np.cumsum(q)]).astype(np.int32)
        cat = (lambda parts: np.concatenate(parts) if parts else np.zeros(0, dtype=np.int32))
        out.update(nbmaps=np.stack([cat(ins), cat(outs)]).astype(np.int32), nbsizes=nbsizes, naddrs=naddrs, qnaddrs=qnaddrs,
                   sizes=np.asarray([naddrs[-1], qnaddrs[-1]], dtype=np.int32))
    else:
        sm, tm, sizes = gs_masks_half(rows, K - dense, num_sources, num_targets)
        out.update(smask=sm, tmask=tm, nbsizes=sizes)
    return out


def natural_weights_from_l1(weights, kernel_size, dataflow: int):
    """The kernel tensor in natural offset order that means what ``weights`` means in the L1-norm order a hybrid dataflow
    reads (``scripts/models/convert_weights.py:30-55``): ``w_nat[k] = weights[position[k]]``."""
    import torch
    position, _ = l1_permutation(kernel_size, dataflow)
    return torch.as_tensor(weights)[torch.as_tensor(position.astype(np.int64))]


def convert_transposed_os(out_in_map: np.ndarray, num_inputs: int) -> np.ndarray:
    """Invert a ``[T_al, K]`` out->in map into ``[S_al, K]`` in->out, same column.

    ``source/csrc/spira/cuda/kernels/convert_transposed_os.cuh:7-13``,
    ``source/csrc/spira/torch/cuda_sparse_convolution_mapping.cu:1809-1830``.
    """
    K = out_in_map.shape[1]
    res = np.full((aligned(num_inputs), K), -1, dtype=np.int32)
    t, c = np.nonzero(out_in_map >= 0)
    res[out_in_map[t, c], c] = t
    return res


# ----------------------------------------------------------------------------------------------
# feature compute -- out[t] = sum_k feats[map[t,k]] @ W[k], fp32 accumulate, one rounding to fp16
# (source/csrc/spira/cuda/kernels/output_stat.cuh:451,637)
# ----------------------------------------------------------------------------------------------
def conv_from_pairs(feats, weights, in_idx, out_idx, k_idx, num_targets: int):
    """torch-CPU gather-GEMM-scatter over explicit (in, out, weight index) triples."""
    import torch

    feats = torch.as_tensor(feats)
    weights = torch.as_tensor(weights)
    out = torch.zeros(num_targets, weights.shape[2], dtype=torch.float32)
    in_idx = torch.as_tensor(np.asarray(in_idx, dtype=np.int64))
    out_idx = torch.as_tensor(np.asarray(out_idx, dtype=np.int64))
    k_idx = np.asarray(k_idx)
    f32 = feats.float()
    for k in np.unique(k_idx):
        sel = torch.as_tensor(np.nonzero(k_idx == k)[0])
        out.index_add_(0, out_idx[sel], f32[in_idx[sel]] @ weights[int(k)].float())
    return out.to(feats.dtype)


def conv_os(feats, weights, out_in_map: np.ndarray, num_targets: int):
    """Output-stationary call: column c of the map uses ``weights[c]``
    (``source/csrc/spira/cuda/functions/sparse_convolution.cu:1354-1393``)."""
    t, c = np.nonzero(out_in_map[:num_targets] >= 0)
    return conv_from_pairs(feats, weights, out_in_map[t, c], t, c, num_targets)


def conv_ws(feats, weights, dense_ws: np.ndarray, num_targets: int):
    """Weight-stationary call: row k of the map uses ``weights[k]``."""
    k, t = np.nonzero(dense_ws[:, :num_targets] >= 0)
    return conv_from_pairs(feats, weights, dense_ws[k, t], t, k, num_targets)


def conv_ws_transposed(feats, weights, dense_ws: np.ndarray, num_sources_of_map: int):
    """Transposed layer on the map of its non-transposed twin: roles of in/out are swapped and
    the SAME weight row is used (``source/spira/nn/conv.py:341-348``, ``weight_stat.cuh:786-798``
    keep ``widx`` for the non-mirrored half)."""
    k, t = np.nonzero(dense_ws >= 0)
    return conv_from_pairs(feats, weights, t, dense_ws[k, t], k, num_sources_of_map)


# ----------------------------------------------------------------------------------------------
# engine-native structures without a counterpart in the reference: specified here, checked on the GPU
# ----------------------------------------------------------------------------------------------
def group_os_map(out_in_map: np.ndarray, num_targets: int):
    """Rows of an output-stationary map ``[T_al, K]`` (K <= 32) sorted by presence mask.

    Key of row t: ``(K - popcount(mask)) << 19 | (mask >> max(0, K - 19))`` for K <= 27 (fullest rows first, rows whose
    masks agree in the 19 highest offsets adjacent), else ``~mask``; the sort is stable, so rows with the same key keep
    their spatial order.  Returns
    ``(grouped_map [T_al, K], row_of [T_al], tile_masks [T_al / 128] uint32, stats (n128, n256))`` where padding rows
    are -1, ``tile_masks[i]`` has bit k set if some row of tile i has a neighbour at offset k, and the stats count the
    non-empty (tile, offset) pairs for 128- and 256-row tiles.  The convolution over the grouped map writes output row
    ``row_of[i]`` for grouped row i and equals the convolution over the original map.
    """
    Tal, K = out_in_map.shape
    assert K <= 32 and Tal % 128 == 0 and num_targets <= Tal
    present = out_in_map[:num_targets] >= 0
    mask = (present.astype(np.uint64) << np.arange(K, dtype=np.uint64)).sum(1)
    if K <= 27:
        key = ((K - present.sum(1)).astype(np.uint64) << np.uint64(19)) | (mask >> np.uint64(max(0, K - 19)))
    else:
        key = (~mask) & np.uint64(0xFFFFFFFF)
    order = np.argsort(key, kind="stable").astype(np.int32)
    row_of = np.full(Tal, -1, dtype=np.int32)
    row_of[:num_targets] = order
    grouped = np.full((Tal, K), -1, dtype=np.int32)
    grouped[:num_targets] = out_in_map[order]
    tiles = (grouped >= 0).reshape(Tal // 128, 128, K).any(1)
    tile_masks = (tiles.astype(np.uint64) << np.arange(K, dtype=np.uint64)).sum(1).astype(np.uint32)
    pairs = tiles if tiles.shape[0] % 2 == 0 else np.concatenate([tiles, np.zeros((1, K), bool)])
    n256 = int(pairs.reshape(-1, 2, K).any(1).sum())
    return grouped, row_of, tile_masks, (int(tiles.sum()), n256)


def conv_os_grouped(feats, weights, grouped_map: np.ndarray, row_of: np.ndarray, num_targets: int):
    """Convolution over a grouped map: row i of the result of :func:`conv_os` on ``grouped_map`` lands in output row
    ``row_of[i]``."""
    import torch
    rows = conv_os(feats, weights, grouped_map, num_targets)
    out = torch.empty_like(rows)
    out[torch.from_numpy(row_of[:num_targets].astype(np.int64))] = rows
    return out
