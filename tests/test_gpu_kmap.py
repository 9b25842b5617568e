"""GPU parity: kernel maps through the C-ABI vs the oracle -- bit exact, dense maps and derived structures."""
import numpy as np
import pytest
import torch

import spira_oracle as O
from helpers import cloud, surface, dev, keys_from_torch, keys_to_torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def C(lib):
    from spira_b200.nn.functional import _C
    return _C


def build(C, src, tgt, ks, stride, dataflow):
    return C.cuda_binary_search(keys_to_torch(src), keys_to_torch(tgt), ks, stride, dataflow)


@pytest.mark.parametrize("ks", [(3, 3, 3), (5, 5, 5), (2, 2, 2), (3, 3, 1), (1, 1, 3), (3, 5, 2)])
@pytest.mark.parametrize("double", [False, True])
def test_submanifold_dense_maps(C, ks, double):
    c = surface(11)
    keys, _ = O.flat_sort(c, double)
    for df, layout in ((0, "os"), (1, "ws")):
        m = build(C, keys, keys, ks, (1, 1, 1), df)
        assert m[0] == len(keys) and m[1] == len(keys)
        np.testing.assert_array_equal(m[2].cpu().numpy(), O.kernel_map(keys, keys, ks, (1, 1, 1), layout))


@pytest.mark.parametrize("n", [1, 2, 127, 128, 129, 300])
def test_ragged_sizes(C, n):
    c = cloud(n, n, 32, 40)
    keys, _ = O.flat_sort(c)
    for df, layout in ((0, "os"), (1, "ws")):
        m = build(C, keys, keys, (3, 3, 3), (1, 1, 1), df)
        np.testing.assert_array_equal(m[2].cpu().numpy(), O.kernel_map(keys, keys, (3, 3, 3), (1, 1, 1), layout))


@pytest.mark.parametrize("ks", [(3, 3, 3), (2, 2, 2)])
def test_strided_chain(C, ks):
    """Down-sampling maps level l -> l+1 and submanifold maps at every level, built in ONE streamed call."""
    c = surface(12, 40000)
    keys, _ = O.flat_sort(c)
    strides = [(2, 2, 2), (4, 4, 4), (8, 8, 8)]
    levels = [keys] + O.streamed_output_generate(keys, strides)
    kernel_sizes = [(3, 3, 3), ks, (3, 3, 3), ks, (3, 3, 3), ks, (3, 3, 3)]
    source_strides = [(1, 1, 1), (1, 1, 1), (2, 2, 2), (2, 2, 2), (4, 4, 4), (4, 4, 4), (8, 8, 8)]
    dataflows = [0, 1, 1, 0, 2, 1, 0]
    maps = C.cuda_binary_search_streamed([keys_to_torch(v) for v in levels], kernel_sizes, source_strides, dataflows)
    assert len(maps) == 7
    for i, m in enumerate(maps):
        src, tgt = levels[i // 2], levels[(i + 1) // 2]
        layout = "os" if dataflows[i] == 0 else "ws"
        want = O.kernel_map(src, tgt, kernel_sizes[i], source_strides[i], layout)
        np.testing.assert_array_equal(m[2].cpu().numpy(), want, err_msg=f"map {i}")
        assert (m[0], m[1]) == (len(src), len(tgt))


def test_wrapping_queries_match_exact_lookup(C):
    """Voxels at the origin and at the top of the fields: queries under/overflow; the engine answers with the
    exact lookup of the wrapped key (the oracle's default), for every tile position."""
    rng = np.random.default_rng(13)
    c = np.concatenate([rng.integers(0, 3, size=(60, 3)), rng.integers(0, 3, size=(60, 3)) + [4093, 4093, 253],
                        rng.integers(100, 140, size=(3000, 3))])
    c = np.unique(c, axis=0).astype(np.int32)
    keys, _ = O.flat_sort(c)
    for df, layout in ((0, "os"), (1, "ws")):
        m = build(C, keys, keys, (3, 3, 3), (1, 1, 1), df)
        np.testing.assert_array_equal(m[2].cpu().numpy(), O.kernel_map(keys, keys, (3, 3, 3), (1, 1, 1), layout))


def test_huge_window_falls_back_to_global_search(C):
    """A sparse target set over a dense source set: the per-tile source windows exceed the staging capacity."""
    c = cloud(14, 60000, 32, 80)
    keys, _ = O.flat_sort(c)
    tgt = keys[::400].copy()
    m = build(C, keys, tgt, (3, 3, 3), (1, 1, 1), 1)
    np.testing.assert_array_equal(m[2].cpu().numpy(), O.kernel_map(keys, tgt, (3, 3, 3), (1, 1, 1), "ws"))


@pytest.mark.parametrize("sub", [True, False])
def test_weight_stationary_lists(C, sub):
    c = surface(15)
    keys, _ = O.flat_sort(c)
    tgt = keys if sub else O.downsample(keys, (2, 2, 2))
    m = build(C, keys, tgt, (3, 3, 3), (1, 1, 1), 1)
    dense = m[2].cpu().numpy()
    nbmaps, nbsizes, naddrs, qnaddrs, mapsize, qmapsize = O.ws_structures(dense, len(keys), len(tgt))
    np.testing.assert_array_equal(m[3].cpu().numpy(), nbmaps)
    np.testing.assert_array_equal(m[4].cpu().numpy(), nbsizes)
    np.testing.assert_array_equal(m[5].cpu().numpy(), naddrs)
    np.testing.assert_array_equal(m[6].cpu().numpy(), qnaddrs)
    assert (m[7], m[8]) == (mapsize, qmapsize)
    assert m[4].shape[0] == (14 if sub else 27)
    counts = m[2]._sb["counts"].cpu().numpy()
    np.testing.assert_array_equal(counts, (dense >= 0).reshape(27, -1, 128).sum(axis=2))


def test_mask_format(C):
    c = surface(16)
    keys, _ = O.flat_sort(c)
    tgt = O.downsample(keys, (2, 2, 2))
    m = build(C, keys, tgt, (2, 2, 2), (1, 1, 1), 2)
    sm, tm, sizes = O.gs_masks(m[2].cpu().numpy(), len(keys), len(tgt))
    np.testing.assert_array_equal(m[3].cpu().numpy(), sm)
    np.testing.assert_array_equal(m[4].cpu().numpy(), tm)
    np.testing.assert_array_equal(m[5].cpu().numpy(), sizes)


def test_transposed_inverse_and_transpose(C):
    c = surface(17)
    keys, _ = O.flat_sort(c)
    tgt = O.downsample(keys, (2, 2, 2))
    m = build(C, keys, tgt, (3, 3, 3), (1, 1, 1), 0)
    inv = C.cuda_convert_transposed_os(m[2], len(keys))
    np.testing.assert_array_equal(inv.cpu().numpy(), O.convert_transposed_os(m[2].cpu().numpy(), len(keys)))
    np.testing.assert_array_equal(C.transpose_map(m[2]).cpu().numpy(), m[2].cpu().numpy().T)
    nz = C.cuda_binary_search_no_small_z(keys_to_torch(keys), keys_to_torch(tgt), (3, 3, 3), (1, 1, 1))
    np.testing.assert_array_equal(nz[2].cpu().numpy(), O.kernel_map(keys, tgt, (3, 3, 3), (1, 1, 1), "ws").T)


def test_empty_and_invalid(C):
    e = torch.empty(0, dtype=torch.int32, device="cuda")
    k = keys_to_torch(O.flat_sort(cloud(1, 50, 32, 40))[0])
    m = C.cuda_binary_search(k, e, (3, 3, 3), (1, 1, 1), 0)
    assert m[2].shape == (0, 27)
    m = C.cuda_binary_search(e, k, (3, 3, 3), (1, 1, 1), 1)
    assert (m[2].cpu().numpy() == -1).all() and m[7] == 0
    with pytest.raises(RuntimeError):
        C.cuda_binary_search(k, k, (9, 9, 9), (1, 1, 1), 0)      # more than 64 xy offsets
    with pytest.raises(RuntimeError):
        C.cuda_binary_search(k, k, (3, 3, 3), (1, 1, 1), 11)


def test_lidar_scene_all_map_kinds(C):
    """One full-size LiDAR-like scene (~125k voxels): 3^3, 5^3, stride-2 down and its transposed reuse."""
    from spira_b200 import scenes
    c = scenes.lidar_scene(1)
    keys, _ = O.flat_sort(c)
    down = O.downsample(keys, (2, 2, 2))
    tk, td = keys_to_torch(keys), keys_to_torch(down)
    maps = C.cuda_binary_search_streamed([tk, td], [(3, 3, 3), (3, 3, 3)], [(1, 1, 1), (1, 1, 1)], [0, 1])
    np.testing.assert_array_equal(maps[0][2].cpu().numpy(), O.kernel_map(keys, keys, (3, 3, 3), (1, 1, 1), "os"))
    np.testing.assert_array_equal(maps[1][2].cpu().numpy(), O.kernel_map(keys, down, (3, 3, 3), (1, 1, 1), "ws"))
    m5 = C.cuda_binary_search(tk, tk, (5, 5, 5), (1, 1, 1), 0)
    np.testing.assert_array_equal(m5[2].cpu().numpy(), O.kernel_map(keys, keys, (5, 5, 5), (1, 1, 1), "os"))
    # transposed up-sampling reuses the down-sampling map with the roles exchanged
    m0 = C.cuda_binary_search(tk, td, (3, 3, 3), (1, 1, 1), 0)
    inv = C.cuda_convert_transposed_os(m0[2], len(keys))
    np.testing.assert_array_equal(inv.cpu().numpy(), O.convert_transposed_os(m0[2].cpu().numpy(), len(keys)))
