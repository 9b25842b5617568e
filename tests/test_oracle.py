"""CPU checks of the oracle itself: every piece against an independent brute-force statement."""
import itertools

import numpy as np
import pytest
import torch

import spira_oracle as O


def random_cloud(rng, n, lo, hi):
    c = rng.integers(lo, hi, size=(n, 3))
    return np.unique(c, axis=0).astype(np.int32)


@pytest.mark.parametrize("width", [4, 8])
def test_pack_roundtrip_and_order(width):
    rng = np.random.default_rng(0)
    hi = 250 if width == 4 else 60000
    c = random_cloud(rng, 2000, 0, hi)
    k = O.pack(c, width)
    assert k.dtype == (np.uint32 if width == 4 else np.uint64)
    np.testing.assert_array_equal(O.unpack(k), c)
    # z is the least significant field: sorting keys == lexicographic (x, y, z)
    order = np.lexsort((c[:, 2], c[:, 1], c[:, 0]))
    np.testing.assert_array_equal(np.argsort(k, kind="stable"), order)


def test_pack_bit_layout():
    assert O.pack(np.array([[1, 2, 3]], np.int32), 4)[0] == (1 << 20) | (2 << 8) | 3
    assert O.pack(np.array([[1, 2, 3]], np.int32), 8)[0] == (1 << 40) | (2 << 16) | 3
    # no range masking: z = 256 spills into y for the 32-bit layout
    assert O.pack(np.array([[0, 0, 256]], np.int32), 4)[0] == 1 << 8


def test_flat_sort_is_stable_with_duplicates():
    c = np.array([[5, 5, 5], [1, 1, 1], [5, 5, 5], [0, 0, 9]], np.int32)
    keys, idx = O.flat_sort(c)
    np.testing.assert_array_equal(idx, [3, 1, 0, 2])
    assert idx.dtype == np.int32


@pytest.mark.parametrize("stride", [(2, 2, 2), (4, 4, 4), (8, 8, 16), (1, 2, 4)])
def test_downsample_against_floor_division(stride):
    rng = np.random.default_rng(1)
    c = random_cloud(rng, 3000, 32, 200)
    keys, _ = O.flat_sort(c)
    down = O.downsample(keys, stride)
    want = np.unique((c // np.array(stride)) * np.array(stride), axis=0)
    np.testing.assert_array_equal(O.unpack(down), want[np.lexsort((want[:, 2], want[:, 1], want[:, 0]))])
    assert np.all(np.diff(down.astype(np.int64)) > 0)


def test_offsets_order_and_even_kernels():
    off = O.xy_offsets((3, 3, 3), (1, 1, 1), 4)
    want = [((ix << 20) + (iy << 8) - 1) % 2**32 for ix in (-1, 0, 1) for iy in (-1, 0, 1)]
    np.testing.assert_array_equal(off, np.array(want, np.uint32))
    assert O.axis_range(2) == (0, 1) and O.axis_range(3) == (-1, 1) and O.axis_range(5) == (-2, 2) and O.axis_range(4) == (-1, 2)
    off2 = O.xy_offsets((2, 2, 2), (4, 4, 4), 8)
    np.testing.assert_array_equal(off2, np.array([(ix * 4 << 40) + (iy * 4 << 16) for ix in (0, 1) for iy in (0, 1)], np.uint64))


def brute_map(src_c, tgt_c, ks, stride):
    """dict lookup per (target, offset): the geometric definition of a kernel map."""
    table = {tuple(c): i for i, c in enumerate(src_c.tolist())}
    rx, ry, rz = (range(O.axis_range(k)[0], O.axis_range(k)[1] + 1) for k in ks)
    out = []
    for t, c in enumerate(tgt_c.tolist()):
        for k, (dx, dy, dz) in enumerate(itertools.product(rx, ry, rz)):
            s = table.get((c[0] + dx * stride[0], c[1] + dy * stride[1], c[2] + dz * stride[2]))
            if s is not None:
                out.append((s, t, k))
    return np.array(sorted(out), dtype=np.int64).reshape(-1, 3)


@pytest.mark.parametrize("ks,width", [((3, 3, 3), 4), ((5, 5, 5), 4), ((2, 2, 2), 4), ((3, 3, 3), 8), ((3, 1, 5), 4)])
def test_submanifold_map_against_brute_force(ks, width):
    rng = np.random.default_rng(2)
    c = random_cloud(rng, 700, 32, 44)
    keys, idx = O.flat_sort(c, double=(width == 8))
    cs = c[idx]
    for layout in ("os", "ws"):
        dense = O.kernel_map(keys, keys, ks, (1, 1, 1), layout)
        K = ks[0] * ks[1] * ks[2]
        assert dense.shape == ((O.aligned(len(keys)), K) if layout == "os" else (K, O.aligned(len(keys))))
        np.testing.assert_array_equal(O.triples(dense, layout, ks), brute_map(cs, cs, ks, (1, 1, 1)))


@pytest.mark.parametrize("ks", [(3, 3, 3), (2, 2, 2)])
def test_strided_map_against_brute_force(ks):
    rng = np.random.default_rng(3)
    c = random_cloud(rng, 900, 32, 50)
    keys, idx = O.flat_sort(c)
    down = O.downsample(keys, (2, 2, 2))
    dense = O.kernel_map(keys, down, ks, (1, 1, 1), "ws")
    np.testing.assert_array_equal(O.triples(dense, "ws", ks), brute_map(c[idx], O.unpack(down), ks, (1, 1, 1)))
    # second level: sources at stride 2, offsets scaled by the source stride
    down2 = O.downsample(keys, (4, 4, 4))
    dense2 = O.kernel_map(down, down2, ks, (2, 2, 2), "os")
    np.testing.assert_array_equal(O.triples(dense2, "os", ks), brute_map(O.unpack(down), O.unpack(down2), ks, (2, 2, 2)))


def test_reference_walk_emulation_differs_only_at_the_origin_column():
    # a voxel in the (0, 0, .) column at z = 0: the first query of the centre column underflows
    c = np.array([[0, 0, 0], [0, 0, 1], [0, 1, 0], [3, 3, 3]], np.int32)
    keys, _ = O.flat_sort(c)
    exact = O.kernel_map(keys, keys, (3, 3, 3), (1, 1, 1), "ws")
    walk = O.kernel_map(keys, keys, (3, 3, 3), (1, 1, 1), "ws", emulate_reference_walk=True)
    assert exact[13, 0] == 0 and walk[13, 0] == -1            # centre entry of the origin voxel is lost by the walk
    lost = (exact != walk)
    assert lost.sum() > 0 and np.all(walk[lost] == -1)
    # with a margin the two agree everywhere
    keys2, _ = O.flat_sort(c + 32)
    np.testing.assert_array_equal(O.kernel_map(keys2, keys2, (3, 3, 3), (1, 1, 1), "ws"),
                                  O.kernel_map(keys2, keys2, (3, 3, 3), (1, 1, 1), "ws", emulate_reference_walk=True))


def test_ws_structures_half_and_full():
    rng = np.random.default_rng(4)
    c = random_cloud(rng, 500, 32, 42)
    keys, _ = O.flat_sort(c)
    dense = O.kernel_map(keys, keys, (3, 3, 3), (1, 1, 1), "ws")
    nbmaps, nbsizes, naddrs, qnaddrs, mapsize, qmapsize = O.ws_structures(dense, len(keys), len(keys))
    assert len(nbsizes) == 14 and nbsizes[13] == len(keys)      # half list, centre row = identity
    assert mapsize == nbsizes.sum() and qmapsize % 128 == 0 and nbmaps.shape == (2, mapsize)
    # symmetry that the half list relies on: (s, t, k) in map  <=>  (t, s, K-1-k) in map
    tr = O.triples(dense, "ws", (3, 3, 3))
    mirrored = np.stack([tr[:, 1], tr[:, 0], 26 - tr[:, 2]], axis=1)
    np.testing.assert_array_equal(mirrored[np.lexsort((mirrored[:, 2], mirrored[:, 1], mirrored[:, 0]))], tr)
    down = O.downsample(keys, (2, 2, 2))
    dense2 = O.kernel_map(keys, down, (3, 3, 3), (1, 1, 1), "ws")
    nb2, sizes2, *_ = O.ws_structures(dense2, len(keys), len(down))
    assert len(sizes2) == 27 and nb2.shape[1] == (dense2 >= 0).sum()


def test_masks_and_transposed_inverse():
    rng = np.random.default_rng(5)
    c = random_cloud(rng, 400, 32, 42)
    keys, _ = O.flat_sort(c)
    down = O.downsample(keys, (2, 2, 2))
    ws = O.kernel_map(keys, down, (2, 2, 2), (1, 1, 1), "ws")
    sm, tm, sizes = O.gs_masks(ws, len(keys), len(down))
    for k in range(8):
        assert sorted(sm[k][sm[k] >= 0].tolist()) == list(range(sizes[k])) == sorted(tm[k][tm[k] >= 0].tolist())
    os_map = O.kernel_map(keys, down, (2, 2, 2), (1, 1, 1), "os")
    inv = O.convert_transposed_os(os_map, len(keys))
    assert inv.shape == (O.aligned(len(keys)), 8)
    t, col = np.nonzero(os_map >= 0)
    np.testing.assert_array_equal(inv[os_map[t, col], col], t)
    assert (inv >= 0).sum() == len(t)       # stride-2, kernel-2: every fine voxel has exactly one parent per column hit


@pytest.mark.parametrize("ks", [(3, 3, 3), (2, 2, 2)])
def test_conv_oracle_against_dense_conv3d(ks):
    """Pins offset order <-> weight index: weight k = (ix*ky + iy)*kz + iz multiplies the source at target + offset."""
    rng = np.random.default_rng(6)
    G = 10
    c = random_cloud(rng, 300, 0, G) + 32
    keys, idx = O.flat_sort(c)
    cs = c[idx] - 32
    cin, cout = 5, 7
    feats = rng.normal(size=(len(cs), cin)).astype(np.float32)
    w = (rng.normal(size=(ks[0] * ks[1] * ks[2], cin, cout)) * 0.2).astype(np.float32)
    ws = O.kernel_map(keys, keys, ks, (1, 1, 1), "ws")
    got = O.conv_ws(torch.from_numpy(feats), torch.from_numpy(w), ws, len(cs)).numpy()
    dense = torch.zeros(1, cin, G, G, G)
    dense[0, :, cs[:, 0], cs[:, 1], cs[:, 2]] = torch.from_numpy(feats).T
    wt = torch.from_numpy(w).reshape(ks[0], ks[1], ks[2], cin, cout).permute(4, 3, 0, 1, 2).contiguous()
    lo = [-O.axis_range(k)[0] for k in ks]
    hi = [O.axis_range(k)[1] for k in ks]
    padded = torch.nn.functional.pad(dense, (lo[2], hi[2], lo[1], hi[1], lo[0], hi[0]))
    full = torch.nn.functional.conv3d(padded, wt)[0]
    want = full[:, cs[:, 0], cs[:, 1], cs[:, 2]].T.numpy()
    np.testing.assert_allclose(got, want, rtol=1e-4, atol=1e-4)
    # the output-stationary call on the z-major map with z-major weights gives the same features
    os_map = O.kernel_map(keys, keys, ks, (1, 1, 1), "os")
    nxy, kz = O.n_offsets(ks)
    perm = [(col % nxy) * kz + col // nxy for col in range(nxy * kz)]
    got_os = O.conv_os(torch.from_numpy(feats), torch.from_numpy(w[perm]), os_map, len(cs)).numpy()
    np.testing.assert_allclose(got_os, want, rtol=1e-4, atol=1e-4)


def test_transposed_conv_oracle_is_adjoint():
    rng = np.random.default_rng(7)
    c = random_cloud(rng, 300, 32, 44)
    keys, _ = O.flat_sort(c)
    down = O.downsample(keys, (2, 2, 2))
    ws = O.kernel_map(keys, down, (3, 3, 3), (1, 1, 1), "ws")
    cin, cout = 4, 4
    w = torch.from_numpy(rng.normal(size=(27, cin, cout)).astype(np.float32))
    x = torch.from_numpy(rng.normal(size=(len(keys), cin)).astype(np.float32))
    y = torch.from_numpy(rng.normal(size=(len(down), cout)).astype(np.float32))
    fwd = O.conv_ws(x, w, ws, len(down))
    bwd = O.conv_ws_transposed(y, w.transpose(1, 2).contiguous(), ws, len(keys))
    # <conv(x), y> == <x, conv_T(y)> when the transposed layer uses the transposed weight matrices
    np.testing.assert_allclose((fwd * y).sum().item(), (x * bwd).sum().item(), rtol=1e-3)


def test_grouped_map_is_a_row_permutation_and_convolves_to_the_same_result():
    import torch
    from helpers import surface
    c = surface(31, 3000)
    keys, _ = O.flat_sort(c)
    dense = O.kernel_map(keys, keys, (3, 3, 3), (1, 1, 1), "os")
    T = len(keys)
    g, row_of, masks, (n128, n256) = O.group_os_map(dense, T)
    assert sorted(row_of[:T].tolist()) == list(range(T)) and (row_of[T:] == -1).all()
    assert np.array_equal(g[:T], dense[row_of[:T]]) and (g[T:] == -1).all()
    pop = (g[:T] >= 0).sum(1)
    assert (np.diff(pop) <= 0).all()                                  # fullest rows first
    before = (dense.reshape(-1, 128, 27) >= 0).any(1).sum()
    assert n128 == sum(bin(int(m)).count("1") for m in masks) and n128 < before and n256 <= n128
    rng = np.random.default_rng(0)
    f = torch.from_numpy(rng.normal(size=(T, 16)).astype(np.float16))
    w = torch.from_numpy((rng.normal(size=(27, 16, 16)) / 20).astype(np.float16))
    assert torch.equal(O.conv_os(f, w, dense, T), O.conv_os_grouped(f, w, g, row_of, T))
