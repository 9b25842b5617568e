"""GPU: size-independent properties at the full size of the headline workload (one ~125 k-voxel LiDAR-like scene with
the channel widths of the MinkUNet18-style network), where the CPU oracle would take minutes per case.

Keys: sortedness, uniqueness, idempotence and nesting of the down-sampling.  Maps: the two layouts hold the same pair
set, a submanifold map is its own mirror image, inverting twice returns the map, grouping is a row permutation.
Features: exact homogeneity under powers of two, additivity within fp16 rounding, both dataflows agree, zero in gives
zero out, the fused epilogue equals the separate passes."""
import numpy as np
import pytest
import torch

import spira_oracle as O
from helpers import keys_to_torch, keys_from_torch, assert_features_close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def C(lib):
    from spira_b200.nn.functional import _C
    yield _C
    _C.check_status()


@pytest.fixture(scope="module")
def scene(C):
    from spira_b200 import scenes
    c = scenes.lidar_scene(11)
    keys, perm = C.cuda_flatten_sort(torch.from_numpy(c).cuda(), False)
    return c, keys, perm


def test_sorted_keys_are_a_sorted_permutation_of_the_packed_input(C, scene):
    c, keys, perm = scene
    k = keys_from_torch(keys)
    assert (np.diff(k.astype(np.int64)) > 0).all()                     # strictly ascending: sorted and unique
    packed = O.pack(c, 4)
    assert np.array_equal(packed[perm.cpu().numpy()], k)
    assert np.array_equal(np.sort(perm.cpu().numpy()), np.arange(len(c)))
    np.testing.assert_array_equal(O.unpack(k), c[perm.cpu().numpy()])


def test_downsampling_is_sorted_unique_idempotent_and_nested(C, scene):
    _, keys, _ = scene
    levels = C.cuda_streamed_output_generate(keys, [(2, 2, 2), (4, 4, 4), (8, 8, 8), (16, 16, 16)])
    sizes = [keys.shape[0]] + [lv.shape[0] for lv in levels]
    assert all(a > b > 0 for a, b in zip(sizes[:-1], sizes[1:]))
    for lv, s in zip(levels, (2, 4, 8, 16)):
        k = keys_from_torch(lv)
        assert (np.diff(k.astype(np.int64)) > 0).all()
        assert (O.unpack(k) % s == 0).all()
        again = C.cuda_downsample(lv, s, s, s)                               # idempotent
        assert torch.equal(again, lv)
    for coarse, fine, s in zip(levels[1:], levels[:-1], (4, 8, 16)):
        assert torch.equal(C.cuda_downsample(fine, s, s, s), coarse)        # a level can be derived from the one before
    # every level-0 voxel has its coarse cell in level 1 and every level-1 cell has a voxel
    k0 = keys_from_torch(keys)
    assert np.array_equal(np.unique(k0 & O.stride_mask((2, 2, 2), 4)), keys_from_torch(levels[0]))


def _pairs(dense, layout, T, kernel_size):
    t = O.triples(dense, layout, kernel_size)
    return t[np.lexsort((t[:, 2], t[:, 1], t[:, 0]))]


def test_both_layouts_hold_the_same_pairs_and_a_submanifold_map_mirrors_itself(C, scene):
    _, keys, _ = scene
    T = keys.shape[0]
    m_os = C.cuda_binary_search(keys, keys, (3, 3, 3), (1, 1, 1), 0)
    m_ws = C.cuda_binary_search(keys, keys, (3, 3, 3), (1, 1, 1), 1)
    d_os, d_ws = m_os[2].cpu().numpy(), m_ws[2].cpu().numpy()
    assert np.array_equal(_pairs(d_os, "os", T, (3, 3, 3)), _pairs(d_ws, "ws", T, (3, 3, 3)))
    # natural order (ws rows): offset k and offset 26 - k are opposite, so (s -> t at k) implies (t -> s at 26 - k)
    k, t = np.nonzero(d_ws[:, :T] >= 0)
    s = d_ws[k, t]
    assert (d_ws[26 - k, s] == t).all()
    assert (d_ws[13, :T] == np.arange(T)).all()                              # the centre offset maps every voxel to itself
    # the counts the search reports equal the number of pairs, and the list sizes follow from them
    assert int(C.map_counts(m_ws[2]).sum()) == len(k) == int(C.map_counts(m_os[2]).sum())
    assert m_ws[7] == int((d_ws[:14, :T] >= 0).sum())                        # mirrored lists hold rows 0..13 only


def test_inverting_a_strided_map_twice_returns_it(C, scene):
    _, keys, _ = scene
    down = C.cuda_downsample(keys, 2, 2, 2)
    S, T = keys.shape[0], down.shape[0]
    m = C.cuda_binary_search(keys, down, (3, 3, 3), (1, 1, 1), 0)
    inv = C.cuda_convert_transposed_os(m[2], S)                              # [S_al, K]: for every source, its target per offset
    back = C.cuda_convert_transposed_os(inv, T)
    assert torch.equal(back[:T], m[2][:T])
    d, i = m[2].cpu().numpy(), inv.cpu().numpy()
    t, k = np.nonzero(d[:T] >= 0)
    assert (i[d[t, k], k] == t).all() and int((i >= 0).sum()) == len(t)


def test_grouping_is_a_row_permutation_at_full_size(C, scene):
    _, keys, _ = scene
    T = keys.shape[0]
    m = C.cuda_binary_search(keys, keys, (3, 3, 3), (1, 1, 1), 0)
    g = C.grouped_twin(m[2])
    row_of = g.row_of[:T].long()
    assert torch.equal(torch.sort(row_of).values, torch.arange(T, device="cuda"))
    assert torch.equal(g.map[:T], m[2][row_of])
    assert bool((g.row_of[T:] == -1).all()) and bool((g.map[T:] == -1).all())
    pop = (g.map[:T] >= 0).sum(1)
    assert bool((pop[1:] <= pop[:-1]).all())
    n128, n256 = g.stats.cpu().tolist()
    before = int((m[2].view(-1, 128, 27) >= 0).any(1).sum())
    assert n128 < 0.5 * before and n256 <= n128


@pytest.mark.parametrize("cin,cout,dataflow", [(32, 32, 0), (96, 96, 0), (128, 96, 0), (96, 96, 1), (256, 128, 1)])
def test_convolution_is_homogeneous_additive_and_maps_zero_to_zero(C, scene, cin, cout, dataflow):
    _, keys, _ = scene
    n = keys.shape[0]
    m = C.cuda_binary_search(keys, keys, (3, 3, 3), (1, 1, 1), dataflow)
    g = torch.Generator(device="cuda").manual_seed(cin + cout + dataflow)
    x1 = (torch.randn(n, cin, device="cuda", generator=g) * 0.5).half()
    x2 = (torch.randn(n, cin, device="cuda", generator=g) * 0.5).half()
    w = (torch.randn(27, cin, cout, device="cuda", generator=g) / (27 * cin) ** 0.5).half()
    run = (lambda x: C.conv_os(n, n, m[2], x, w)) if dataflow == 0 else (lambda x: C.conv_ws(n, n, x, w, m[2]._sb["ws"]))
    y1, y2 = run(x1), run(x2)
    assert torch.isfinite(y1).all() and float(y1.float().abs().mean()) > 1e-3
    if dataflow == 0:
        big = y1.abs() > 2e-4                                                # (fp16 subnormals round on a fixed grid)
        assert torch.equal(run(x1 * 4)[big], (y1 * 4)[big])                  # exact: a power of two commutes with every rounding
        assert torch.equal(run(x1), y1)                                      # and the output-stationary path is deterministic
    else:
        assert_features_close(run(x1 * 4), y1 * 4, rtol=4e-3, atol=4e-3)     # the order of the fp32 reductions varies
    assert int(torch.count_nonzero(run(torch.zeros_like(x1)))) == 0
    y12 = run((x1.float() + x2.float()).half())
    assert_features_close(y12, (y1.float() + y2.float()), rtol=1e-2, atol=4e-3)


def test_both_dataflows_agree_at_full_size(C, scene):
    _, keys, _ = scene
    n = keys.shape[0]
    m0 = C.cuda_binary_search(keys, keys, (3, 3, 3), (1, 1, 1), 0)
    m1 = C.cuda_binary_search(keys, keys, (3, 3, 3), (1, 1, 1), 1)
    g = torch.Generator(device="cuda").manual_seed(5)
    x = (torch.randn(n, 64, device="cuda", generator=g) * 0.5).half()
    w_nat = (torch.randn(27, 64, 96, device="cuda", generator=g) / (27 * 64) ** 0.5).half()
    # the output-stationary map numbers its columns z-major, the weight-stationary rows are in natural order
    col_of_nat = torch.tensor([(k % 3) * 9 + k // 3 for k in range(27)], device="cuda")
    w_os = torch.empty_like(w_nat)
    w_os[col_of_nat] = w_nat
    y_os = C.conv_os(n, n, m0[2], x, w_os)
    y_ws = C.conv_ws(n, n, x, w_nat, m1[2]._sb["ws"])
    assert_features_close(y_os, y_ws, rtol=1e-2, atol=2e-3)


def test_fused_epilogue_equals_separate_passes_at_full_size(C, scene):
    _, keys, _ = scene
    n = keys.shape[0]
    m = C.cuda_binary_search(keys, keys, (3, 3, 3), (1, 1, 1), 0)
    g = torch.Generator(device="cuda").manual_seed(9)
    x = (torch.randn(n, 96, device="cuda", generator=g) * 0.5).half()
    w = (torch.randn(27, 96, 96, device="cuda", generator=g) / (27 * 96) ** 0.5).half()
    res = torch.randn(n, 96, device="cuda", generator=g).half()
    scale = torch.rand(96, device="cuda", generator=g) + 0.5
    shift = torch.randn(96, device="cuda", generator=g)
    plain = C.conv_os(n, n, m[2], x, w)
    fused = C.conv_os(n, n, m[2], x, w, scale=scale, shift=shift, residual=res, relu=True)
    want = torch.relu(plain.float() * scale + shift + res.float())
    assert_features_close(fused, want, rtol=1e-2, atol=4e-3)
