"""GPU parity: feature compute through the C-ABI vs the torch-CPU oracle.

Tolerance: 1e-2 relative / 1e-3 absolute (fp16 in/out, fp32 accumulate, one rounding)."""
import numpy as np
import pytest
import torch

import spira_oracle as O
from helpers import surface, cloud, dev, keys_to_torch, assert_features_close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def C(lib):
    from spira_b200.nn.functional import _C
    yield _C
    _C.check_status()


@pytest.fixture(scope="module")
def scene():
    c = surface(21, 24000)
    keys, _ = O.flat_sort(c)
    down = O.downsample(keys, (2, 2, 2))
    return keys, down


def tensors(n, cin, cout, K, seed):
    rng = np.random.default_rng(seed)
    f = rng.normal(size=(n, cin)).astype(np.float16)
    w = (rng.normal(size=(K, cin, cout)) / np.sqrt(K * cin)).astype(np.float16)
    return torch.from_numpy(f), torch.from_numpy(w)


CHANNELS = [(16, 16), (32, 32), (64, 64), (32, 64), (96, 96), (128, 128), (192, 96), (256, 256), (384, 256), (64, 48),
            (24, 16), (4, 32), (3, 32), (5, 16), (32, 19)]


@pytest.mark.parametrize("cin,cout", CHANNELS)
def test_output_stationary_submanifold(C, scene, cin, cout):
    keys, _ = scene
    n = len(keys)
    m = C.cuda_binary_search(keys_to_torch(keys), keys_to_torch(keys), (3, 3, 3), (1, 1, 1), 0)
    f, w = tensors(n, cin, cout, 27, cin * 1000 + cout)
    got = C.cuda_sparse_convolution_forward_os(n, n, m[2], f.cuda(), w.cuda())
    want = O.conv_os(f, w, m[2].cpu().numpy(), n)
    assert_features_close(got, want)
    C.check_status()


@pytest.mark.parametrize("cin,cout", [(64, 64), (4, 32)])
def test_simt_kernel_agrees(C, scene, cin, cout):
    keys, _ = scene
    n = len(keys)
    m = C.cuda_binary_search(keys_to_torch(keys), keys_to_torch(keys), (3, 3, 3), (1, 1, 1), 0)
    f, w = tensors(n, cin, cout, 27, 5)
    got = C.conv_os(n, n, m[2], f.cuda(), w.cuda(), force_simt=True)
    assert_features_close(got, O.conv_os(f, w, m[2].cpu().numpy(), n))


@pytest.mark.parametrize("cin,cout", [(16, 16), (32, 32), (64, 64), (128, 64), (96, 128), (256, 256), (4, 32), (24, 48)])
def test_weight_stationary_submanifold_mirrored(C, scene, cin, cout):
    keys, _ = scene
    n = len(keys)
    m = C.cuda_binary_search(keys_to_torch(keys), keys_to_torch(keys), (3, 3, 3), (1, 1, 1), 1)
    f, w = tensors(n, cin, cout, 27, cin * 7 + cout)
    got = C.cuda_sparse_convolution_forward_ws_merged(n, n, f.cuda(), w.cuda(), m[5], m[6], m[3], m[7], m[8], False)
    want = O.conv_ws(f, w, m[2].cpu().numpy(), n)
    assert_features_close(got, want)
    C.check_status()


@pytest.mark.parametrize("ks", [(3, 3, 3), (2, 2, 2)])
@pytest.mark.parametrize("cin,cout", [(32, 64), (64, 64), (4, 16)])
def test_strided_and_transposed(C, scene, ks, cin, cout):
    keys, down = scene
    S, T = len(keys), len(down)
    K = ks[0] * ks[1] * ks[2]
    tk, td = keys_to_torch(keys), keys_to_torch(down)
    f, w = tensors(S, cin, cout, K, 31)
    m_os = C.cuda_binary_search(tk, td, ks, (1, 1, 1), 0)
    m_ws = C.cuda_binary_search(tk, td, ks, (1, 1, 1), 1)
    dense_ws = m_ws[2].cpu().numpy()
    want = O.conv_ws(f, w, dense_ws, T)
    # the z-major map pairs column c with weight row c: permute natural weights to z-major for the OS call
    nxy, kz = O.n_offsets(ks)
    perm = [(col % nxy) * kz + col // nxy for col in range(K)]
    got_os = C.cuda_sparse_convolution_forward_os(S, T, m_os[2], f.cuda(), w[perm].contiguous().cuda())
    assert_features_close(got_os, want)
    got_ws = C.cuda_sparse_convolution_forward_ws_merged(S, T, f.cuda(), w.cuda(), m_ws[5], m_ws[6], m_ws[3], m_ws[7], m_ws[8], False)
    assert_features_close(got_ws, want)
    # transposed layer on the same maps: coarse -> fine
    g, wt = tensors(T, cout, cin, K, 32)
    want_t = O.conv_ws_transposed(g, wt, dense_ws, S)
    got_t = C.cuda_sparse_convolution_forward_ws_merged(T, S, g.cuda(), wt.cuda(), m_ws[5], m_ws[6], m_ws[3], m_ws[7], m_ws[8], True)
    assert_features_close(got_t, want_t)
    inv = C.cuda_convert_transposed_os(m_os[2], S)
    got_t_os = C.cuda_sparse_convolution_forward_os(T, S, inv, g.cuda(), wt[perm].contiguous().cuda())
    assert_features_close(got_t_os, want_t)
    C.check_status()


def test_large_kernel_volume(C):
    """5^3 = 125 offsets: the map slab is single-buffered and chunks straddle offsets (c_in = 32)."""
    c = surface(22, 6000)
    keys, _ = O.flat_sort(c)
    n = len(keys)
    tk = keys_to_torch(keys)
    f, w = tensors(n, 32, 32, 125, 33)
    m = C.cuda_binary_search(tk, tk, (5, 5, 5), (1, 1, 1), 0)
    assert_features_close(C.cuda_sparse_convolution_forward_os(n, n, m[2], f.cuda(), w.cuda()), O.conv_os(f, w, m[2].cpu().numpy(), n))
    m1 = C.cuda_binary_search(tk, tk, (5, 5, 5), (1, 1, 1), 1)
    got = C.cuda_sparse_convolution_forward_ws_merged(n, n, f.cuda(), w.cuda(), m1[5], m1[6], m1[3], m1[7], m1[8], False)
    assert_features_close(got, O.conv_ws(f, w, m1[2].cpu().numpy(), n))
    C.check_status()


@pytest.mark.parametrize("n", [1, 100, 128, 129, 257])
def test_ragged_tiles(C, n):
    c = cloud(n + 40, n, 32, 38)
    keys, _ = O.flat_sort(c)
    n = len(keys)
    tk = keys_to_torch(keys)
    f, w = tensors(n, 64, 64, 27, 34)
    m = C.cuda_binary_search(tk, tk, (3, 3, 3), (1, 1, 1), 0)
    assert_features_close(C.cuda_sparse_convolution_forward_os(n, n, m[2], f.cuda(), w.cuda()), O.conv_os(f, w, m[2].cpu().numpy(), n))
    m1 = C.cuda_binary_search(tk, tk, (3, 3, 3), (1, 1, 1), 1)
    got = C.cuda_sparse_convolution_forward_ws_merged(n, n, f.cuda(), w.cuda(), m1[5], m1[6], m1[3], m1[7], m1[8], False)
    assert_features_close(got, O.conv_ws(f, w, m1[2].cpu().numpy(), n))
    C.check_status()


def test_isolated_voxels_have_only_the_centre(C):
    """No neighbours at all: every tile still produces its (centre-only) output; empty offsets are skipped."""
    c = (np.stack(np.meshgrid(np.arange(12), np.arange(12), np.arange(6), indexing="ij"), -1).reshape(-1, 3) * 4 + 32).astype(np.int32)
    keys, _ = O.flat_sort(c)
    n = len(keys)
    f, w = tensors(n, 64, 64, 27, 35)
    m = C.cuda_binary_search(keys_to_torch(keys), keys_to_torch(keys), (3, 3, 3), (1, 1, 1), 0)
    got = C.cuda_sparse_convolution_forward_os(n, n, m[2], f.cuda(), w.cuda())
    want = (f.float() @ w[13].float()).half()          # z-major column 13 is still the centre
    assert_features_close(got, want)


@pytest.mark.parametrize("mode", ["os", "ws"])
def test_fused_epilogue(C, scene, mode):
    keys, _ = scene
    n = len(keys)
    tk = keys_to_torch(keys)
    f, w = tensors(n, 64, 64, 27, 36)
    rng = np.random.default_rng(36)
    bias = torch.from_numpy(rng.normal(size=64).astype(np.float16))
    scale = torch.from_numpy(rng.uniform(0.5, 1.5, 64).astype(np.float32))
    shift = torch.from_numpy(rng.normal(size=64).astype(np.float32))
    res = torch.from_numpy(rng.normal(size=(n, 64)).astype(np.float16))
    kw = dict(bias=bias.cuda(), scale=scale.cuda(), shift=shift.cuda(), residual=res.cuda(), relu=True)
    if mode == "os":
        m = C.cuda_binary_search(tk, tk, (3, 3, 3), (1, 1, 1), 0)
        got = C.conv_os(n, n, m[2], f.cuda(), w.cuda(), **kw)
        acc = O.conv_from_pairs(f.float(), w.float(), *_pairs_os(m[2].cpu().numpy(), n), n)
    else:
        m = C.cuda_binary_search(tk, tk, (3, 3, 3), (1, 1, 1), 1)
        got = C.conv_ws(n, n, f.cuda(), w.cuda(), m[2]._sb["ws"], **kw)
        d = m[2].cpu().numpy()
        k, t = np.nonzero(d[:, :n] >= 0)
        acc = O.conv_from_pairs(f.float(), w.float(), d[k, t], t, k, n)
    want = torch.relu((acc + bias.float()) * scale + shift + res.float()).half()
    assert_features_close(got, want)


def _pairs_os(m, n):
    t, c = np.nonzero(m[:n] >= 0)
    return m[t, c], t, c


def test_module_level_dataflows_agree(C, scene):
    """SparseConv through the cache: dataflow 0, 1, 2 and force_os give the same features (weights permuted to
    the order each map implies), stride-2 and transposed included."""
    import spira_b200 as sp
    from spira_b200 import nn as spnn
    keys, _ = scene
    n = len(keys)
    f, _ = tensors(n, 32, 32, 27, 37)
    x = sp.SparseTensor(keys_to_torch(keys), f.cuda())
    torch.manual_seed(0)
    net = torch.nn.Sequential(spnn.SparseConv(32, 64, 3), spnn.SparseConv(64, 64, 3, stride=2), spnn.SparseConv(64, 32, 3, stride=2, transposed=True)).cuda().half()
    outs = {}
    for df, force_os in ((1, False), (2, False), (1, True), (2, True)):
        cache = spnn.KernelMapCache()
        sp.set_kernel_map_cache(net, cache)
        for layer in net:
            layer._tunable_config["map_dataflow"], layer._tunable_config["force_os"] = df, force_os
        with torch.no_grad():
            outs[(df, force_os)] = net(x)._features
    base = outs[(1, False)]
    for k, v in outs.items():
        assert_features_close(v, base)
    C.check_status()


# ---- grouped output-stationary maps (rows sorted by neighbour pattern) ------------------------------------------------
def test_grouping_reorders_the_map_without_changing_it(C, scene):
    keys, down = scene
    for src, tgt, stride in ((keys, keys, (1, 1, 1)), (keys, down, (1, 1, 1))):
        m = C.cuda_binary_search(keys_to_torch(src), keys_to_torch(tgt), (3, 3, 3), stride, 0)
        T = len(tgt)
        g = C.grouped_twin(m[2])
        assert g is not None
        dense = m[2].cpu().numpy()
        want_map, want_rows, want_masks, want_stats = O.group_os_map(dense, T)
        assert np.array_equal(g.map.cpu().numpy(), want_map)
        assert np.array_equal(g.row_of.cpu().numpy(), want_rows)
        assert np.array_equal(g.tile_masks.cpu().numpy().view(np.uint32), want_masks)
        assert tuple(g.stats.cpu().tolist()) == want_stats
        Tal = dense.shape[0]
        tm = (want_map >= 0).reshape(-1, 128, 27).any(1)
        # grouping pays: far fewer (tile, offset) pairs have to be visited than in target order
        assert tm.sum() < 0.8 * (dense[:Tal].reshape(-1, 128, 27) >= 0).any(1).sum()


@pytest.mark.parametrize("cin,cout", [(32, 32), (64, 64), (96, 96), (128, 96), (128, 128), (256, 256), (64, 48), (24, 16),
                                      (4, 32), (3, 32), (5, 16), (8, 64)])      # (the last four: network stems)
def test_grouped_convolution_is_bit_identical(C, scene, cin, cout):
    keys, down = scene
    rng = np.random.default_rng(cin + cout)
    for src, tgt in ((keys, keys), (keys, down)):
        S, T = len(src), len(tgt)
        m = C.cuda_binary_search(keys_to_torch(src), keys_to_torch(tgt), (3, 3, 3), (1, 1, 1), 0)
        assert C.grouped_twin(m[2]) is not None
        f, w = tensors(S, cin, cout, 27, cin * 7 + cout)
        res = torch.from_numpy(rng.normal(size=(T, cout)).astype(np.float16)).cuda()
        scale = torch.from_numpy(rng.uniform(0.5, 1.5, cout).astype(np.float32)).cuda()
        shift = torch.from_numpy(rng.normal(size=cout).astype(np.float32)).cuda()
        for kw in ({}, dict(scale=scale, shift=shift, residual=res, relu=True)):
            a = C.conv_os(S, T, m[2], f.cuda(), w.cuda(), grouped=True, splits=1, **kw)
            b = C.conv_os(S, T, m[2], f.cuda(), w.cuda(), grouped=False, splits=1, **kw)
            assert torch.equal(a, b)
        assert_features_close(C.conv_os(S, T, m[2], f.cuda(), w.cuda()), O.conv_os(f, w, m[2].cpu().numpy(), T))
    C.check_status()


@pytest.mark.parametrize("n", [1, 700, 2000, 9000])
@pytest.mark.parametrize("cin,cout", [(64, 64), (128, 128), (256, 256), (96, 48)])
def test_split_output_stationary_agrees_and_is_deterministic(C, n, cin, cout):
    """Tiles shared among 2, 4 or 8 CTAs: same sums as one CTA per tile up to the order of the fp32 additions
    (compared with the oracle and with the unsplit call at the usual tolerance), the same bits on every run, tile
    counters back at zero."""
    keys, _ = O.flat_sort(surface(n + 3, n))
    n = len(keys)
    down = O.downsample(keys, (2, 2, 2))
    rng = np.random.default_rng(n + cin)
    for src, tgt, ks in ((keys, keys, (3, 3, 3)), (keys, down, (2, 2, 2))):
        S, T = len(src), len(tgt)
        K = ks[0] ** 3
        m = C.cuda_binary_search(keys_to_torch(src), keys_to_torch(tgt), ks, (1, 1, 1), 0)
        limit, _ = C.os_split_plan(T, K, cin, cout)
        f, w = tensors(S, cin, cout, K, cin + cout + n)
        res = torch.from_numpy(rng.normal(size=(T, cout)).astype(np.float16)).cuda()
        scale = torch.from_numpy(rng.uniform(0.5, 1.5, cout).astype(np.float32)).cuda()
        shift = torch.from_numpy(rng.normal(size=cout).astype(np.float32)).cuda()
        bias = torch.from_numpy(rng.normal(size=cout).astype(np.float16)).cuda()
        want = O.conv_os(f, w, m[2].cpu().numpy(), T)
        for splits in (2, 4, 8):
            if splits > limit:
                with pytest.raises(RuntimeError):
                    C.conv_os(S, T, m[2], f.cuda(), w.cuda(), splits=splits)
                continue
            for grouped in (True, False):
                got = C.conv_os(S, T, m[2], f.cuda(), w.cuda(), grouped=grouped, splits=splits)
                assert_features_close(got, want)
                assert torch.equal(got, C.conv_os(S, T, m[2], f.cuda(), w.cuda(), grouped=grouped, splits=splits))
                kw = dict(bias=bias, scale=scale, shift=shift, residual=res, relu=True)
                a = C.conv_os(S, T, m[2], f.cuda(), w.cuda(), grouped=grouped, splits=splits, **kw)
                b = C.conv_os(S, T, m[2], f.cuda(), w.cuda(), grouped=grouped, splits=1, **kw)
                assert_features_close(a, b.float().cpu())
                assert float((ulp_distance(a, b) <= 1).float().mean()) > 0.99      # (cancellation against the residual aside)
            scratch = C.split_scratch(torch.device("cuda", 0), 1024)
            assert int(scratch[:1024].max()) == 0
        if limit >= 4:      # the opt-in default: the largest split the layer takes
            C.OS_SPLIT = True
            try:
                auto = C.cuda_sparse_convolution_forward_os(S, T, m[2], f.cuda(), w.cuda())
            finally:
                C.OS_SPLIT = False
            assert torch.equal(auto, C.conv_os(S, T, m[2], f.cuda(), w.cuda(), splits=limit))
    C.check_status()


@pytest.mark.parametrize("ca,cb,cout", [(32, 32, 64), (64, 32, 96), (96, 32, 96), (128, 64, 128), (256, 128, 256), (8, 24, 32)])
def test_two_sources_equal_the_convolution_of_the_concatenation(C, scene, ca, cb, cout):
    """[a | b] read as two sources: bit-identical to the same kernel on torch.cat (output-stationary: same order of
    additions), within tolerance of the oracle; weight-stationary within tolerance (its fp32 reductions are unordered)."""
    keys, down = scene
    rng = np.random.default_rng(ca * 100 + cb)
    for src, tgt, ks in ((keys, keys, (3, 3, 3)), (keys, down, (2, 2, 2))):
        S, T = len(src), len(tgt)
        K = ks[0] ** 3
        f, w = tensors(S, ca + cb, cout, K, ca + cb + cout)
        fa, fb = f[:, :ca].contiguous().cuda(), f[:, ca:].contiguous().cuda()
        res = torch.from_numpy(rng.normal(size=(T, cout)).astype(np.float16)).cuda()
        scale = torch.from_numpy(rng.uniform(0.5, 1.5, cout).astype(np.float32)).cuda()
        shift = torch.from_numpy(rng.normal(size=cout).astype(np.float32)).cuda()
        kw = dict(scale=scale, shift=shift, residual=res, relu=True)
        m0 = C.cuda_binary_search(keys_to_torch(src), keys_to_torch(tgt), ks, (1, 1, 1), 0)
        want = O.conv_os(f, w, m0[2].cpu().numpy(), T)
        for grouped in (True, False):
            got = C.conv_os(S, T, m0[2], fa, w.cuda(), sources_b=fb, grouped=grouped, splits=1)
            assert torch.equal(got, C.conv_os(S, T, m0[2], f.cuda(), w.cuda(), grouped=grouped, splits=1))
            assert_features_close(got, want)
            got = C.conv_os(S, T, m0[2], fa, w.cuda(), sources_b=fb, grouped=grouped, splits=1, **kw)
            assert torch.equal(got, C.conv_os(S, T, m0[2], f.cuda(), w.cuda(), grouped=grouped, splits=1, **kw))
        m1 = C.cuda_binary_search(keys_to_torch(src), keys_to_torch(tgt), ks, (1, 1, 1), 1)
        w_nat = w.cuda()
        got = C.conv_ws(S, T, fa, w_nat, m1[2]._sb["ws"], sources_b=fb)
        assert_features_close(got, C.conv_ws(S, T, f.cuda(), w_nat, m1[2]._sb["ws"]).float().cpu())
    C.check_status()


@pytest.mark.parametrize("n", [1, 127, 128, 5000, 40001])
@pytest.mark.parametrize("ca,cb,cout", [(64, 0, 128), (128, 64, 128), (256, 128, 256), (96, 32, 96), (32, 0, 64), (96, 0, 48),
                                        (160, 32, 240), (40, 24, 64)])
def test_identity_map_layer_matches_the_matrix_product(C, n, ca, cb, cout):
    """A 1x1x1 layer through the identity map (no map tensor), one or two sources, with the fused epilogue, against the
    fp32 matrix product: on the dense TMA kernel (channel counts in whole 32-channel boxes; the last case is not) and,
    with that kernel switched off, on the output-stationary kernel.  The two kernels add the same products in the same
    order, so their results are equal."""
    rng = np.random.default_rng(n + ca)
    f = torch.from_numpy(rng.normal(size=(n, ca + cb)).astype(np.float16))
    w = torch.from_numpy((rng.normal(size=(1, ca + cb, cout)) / np.sqrt(ca + cb)).astype(np.float16))
    bias = torch.from_numpy(rng.normal(size=cout).astype(np.float16))
    scale = torch.from_numpy(rng.uniform(0.5, 1.5, cout).astype(np.float32))
    shift = torch.from_numpy(rng.normal(size=cout).astype(np.float32))
    res = torch.from_numpy(rng.normal(size=(n, cout)).astype(np.float16))
    want = f.float() @ w[0].float() + bias.float()
    fa = f[:, :ca].contiguous().cuda()
    fb = f[:, ca:].contiguous().cuda() if cb else None
    results = []
    assert C.get_option("identity_tma") == 1
    for tma in (1, 0):
        C.set_option("identity_tma", tma)
        try:
            got = [C.conv_identity(fa, w.cuda(), sources_b=fb, bias=bias.cuda()),
                   C.conv_identity(fa, w.cuda(), sources_b=fb, bias=bias.cuda(), residual=res.cuda(), relu=True),
                   C.conv_identity(fa, w.cuda(), sources_b=fb, scale=scale.cuda(), shift=shift.cuda(), relu=True)]
        finally:
            C.set_option("identity_tma", 1)
        assert_features_close(got[0], want)
        assert_features_close(got[1], torch.relu(want + res.float()))
        assert_features_close(got[2], torch.relu((f.float() @ w[0].float()) * scale + shift))
        results.append(got)
    for a, b in zip(*results):
        assert torch.equal(a, b)
    C.check_status()


def test_two_sources_are_checked(C, scene):
    keys, _ = scene
    n = len(keys)
    m0 = C.cuda_binary_search(keys_to_torch(keys), keys_to_torch(keys), (3, 3, 3), (1, 1, 1), 0)
    f, w = tensors(n, 64, 64, 27, 1)
    with pytest.raises(RuntimeError):       # 60 + 4 channels: not multiples of 8
        C.conv_os(n, n, m0[2], f[:, :60].contiguous().cuda(), w.cuda(), sources_b=f[:, 60:].contiguous().cuda())
    with pytest.raises(RuntimeError):       # channel counts do not add up
        C.conv_os(n, n, m0[2], f[:, :32].contiguous().cuda(), w.cuda(), sources_b=f[:, :16].contiguous().cuda())
    with pytest.raises(RuntimeError):       # rows differ
        C.conv_os(n, n, m0[2], f[:, :32].contiguous().cuda(), w.cuda(), sources_b=f[:100, 32:].contiguous().cuda())


def test_split_plan_limits(C):
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    assert C.os_split_plan(128 * (sms // 8), 27, 256, 256)[0] == 8
    assert C.os_split_plan(128 * (sms // 8) + 1, 27, 256, 256)[0] == 4
    assert C.os_split_plan(128 * (sms // 2) + 1, 27, 256, 256)[0] == 1
    assert C.os_split_plan(1000, 27, 96, 48) == (2, 1024 + 1024 * 2 * 48 * 4)       # 48 / 4 is not a multiple of 8
    assert C.os_split_plan(1000, 27, 4, 32)[0] == 1                                  # not tensor-core eligible
    assert C.os_split_plan(1000, 1, 64, 64)[0] == 1                                  # one chunk: nothing to share


def test_grouping_rejects_wide_kernels(C, lib):
    import ctypes
    from spira_b200._lib import GroupDesc
    n = ctypes.c_size_t()
    assert lib.spira_b200_kmap_group_workspace(1000, ctypes.byref(n)) == 0 and n.value > 0
    buf = torch.zeros(1 << 20, dtype=torch.int32, device="cuda")
    d = (GroupDesc * 1)()
    d[0].map_os = d[0].grouped_map = d[0].row_of = d[0].tile_masks = d[0].stats = buf.data_ptr()
    d[0].num_targets, d[0].K = 1000, 125
    rc = lib.spira_b200_kmap_group(d, 1, buf.data_ptr(), n.value, None)
    assert rc != 0 and b"32" in lib.spira_b200_last_error()


# ---- weight-stationary convolution as one cooperative launch over the persistent zero scratch --------------------------
@pytest.mark.parametrize("cin,cout", [(32, 32), (64, 64), (96, 96), (128, 128), (256, 256), (64, 48)])
def test_fused_weight_stationary_call_agrees_and_leaves_zeros(C, scene, cin, cout):
    """Same sums as the three-launch call; the order of the fp32 reductions differs from run to run in both, so the
    comparison allows the last bits of fp16."""
    keys, down = scene
    rng = np.random.default_rng(cin * 3 + cout)
    for src, tgt, swap in ((keys, keys, False), (keys, down, False), (keys, down, True)):
        m = C.cuda_binary_search(keys_to_torch(src), keys_to_torch(tgt), (3, 3, 3), (1, 1, 1), 1)
        lists = m[2]._sb["ws"]
        S, T = (len(tgt), len(src)) if swap else (len(src), len(tgt))       # a transposed layer exchanges the roles
        f, w = tensors(S, cin, cout, 27, cin * 11 + cout)
        res = torch.from_numpy(rng.normal(size=(T, cout)).astype(np.float16)).cuda()
        scale = torch.from_numpy(rng.uniform(0.5, 1.5, cout).astype(np.float32)).cuda()
        shift = torch.from_numpy(rng.normal(size=cout).astype(np.float32)).cuda()
        for kw in ({}, dict(scale=scale, shift=shift, residual=res, relu=True)):
            for _ in range(2):                   # twice: the second call finds the scratch as the first one left it
                a = C.conv_ws(S, T, f.cuda(), w.cuda(), lists, swap=swap, fused=True, **kw)
            b = C.conv_ws(S, T, f.cuda(), w.cuda(), lists, swap=swap, fused=False, **kw)
            assert torch.allclose(a.float(), b.float(), rtol=4e-3, atol=4e-3)
        scratch = C.zero_scratch(torch.device("cuda", torch.cuda.current_device()), 1)
        assert int(torch.count_nonzero(scratch)) == 0
    C.check_status()


def test_fused_weight_stationary_call_without_pairs(C):
    """A map with no pair at all still converts the (zero) scratch: the output is the epilogue of zero."""
    a = np.array([[40, 40, 40], [80, 80, 80]], dtype=np.int32)
    ka, _ = O.flat_sort(a)
    b = np.array([[200, 200, 100]], dtype=np.int32)
    kb, _ = O.flat_sort(b)
    m = C.cuda_binary_search(keys_to_torch(ka), keys_to_torch(kb), (3, 3, 3), (1, 1, 1), 1)
    f, w = tensors(2, 32, 32, 27, 1)
    bias = torch.full((32,), 0.5, dtype=torch.float16).cuda()
    got = C.conv_ws(2, 1, f.cuda(), w.cuda(), m[2]._sb["ws"], bias=bias, fused=True)
    assert torch.equal(got, torch.full((1, 32), 0.5, dtype=torch.float16).cuda())
    C.check_status()


# ---- kernel variants selected by run-time options give the same results ----------------------------------------------
def ulp_distance(a, b):
    """Distance of two fp16 tensors in units in the last place (0 = bit-equal up to the sign of zero)."""
    def ordered(t):
        bits = t.contiguous().view(torch.int16).to(torch.int32)
        return torch.where(bits < 0, -(bits & 0x7FFF), bits)
    return (ordered(a) - ordered(b)).abs()


@pytest.mark.parametrize("option,value", [("os_n256", 0), ("os_n256_min_targets", 1 << 30), ("gather_tma", 1), ("pdl", 0),
                                          ("ws_cooperative_launch", 1)])
def test_kernel_variants_agree_with_the_default(C, scene, option, value):
    keys, down = scene
    tk, td = keys_to_torch(keys), keys_to_torch(down)
    n, nd = len(keys), len(down)
    m_os = C.cuda_binary_search(tk, tk, (3, 3, 3), (1, 1, 1), 0)
    m_dn = C.cuda_binary_search(tk, td, (3, 3, 3), (1, 1, 1), 0)
    m_ws = C.cuda_binary_search(tk, tk, (3, 3, 3), (1, 1, 1), 1)
    cases = []
    for cin, cout in ((64, 64), (96, 96), (128, 96), (32, 128), (4, 32), (5, 16), (3, 64)):
        f, w = tensors(n, cin, cout, 27, cin + 3 * cout)
        cases.append((f.cuda(), w.cuda()))

    rng = np.random.default_rng(5)
    extras = {}
    for _, w in cases:
        cout = w.shape[2]
        if cout not in extras:       # bias, BatchNorm affine and a residual for the fused epilogue
            extras[cout] = (torch.from_numpy(rng.normal(size=cout).astype(np.float16)).cuda(),
                            torch.from_numpy(rng.uniform(0.5, 1.5, size=cout).astype(np.float32)).cuda(),
                            torch.from_numpy(rng.normal(size=cout).astype(np.float32)).cuda(),
                            torch.from_numpy(rng.normal(size=(n, cout)).astype(np.float16)).cuda())

    def run_all():
        out = []
        for f, w in cases:
            bias, scale, shift, res = extras[w.shape[2]]
            out.append(C.conv_os(n, n, m_os[2], f, w, grouped=True))
            out.append(C.conv_os(n, n, m_os[2], f, w, grouped=False))
            out.append(C.conv_os(n, nd, m_dn[2], f, w, relu=True))
            out.append(C.conv_ws(n, n, f, w, m_ws[2]._sb["ws"]))
            out.append(C.conv_os(n, n, m_os[2], f, w, bias=bias, scale=scale, shift=shift, residual=res, relu=True))
            out.append(C.conv_os(n, n, m_os[2], f, w, residual=res, grouped=False))
        return out

    default = C.get_option(option)
    want = run_all()
    C.set_option(option, value)
    try:
        got = run_all()
    finally:
        C.set_option(option, default)
    for i, (g, w) in enumerate(zip(got, want)):
        if i % 6 == 3 or option == "gather_tma":     # atomics order varies; the TMA producer pads every offset to whole chunks
            assert torch.allclose(g.float(), w.float(), rtol=4e-3, atol=4e-3)
        elif option in ("pdl", "ws_cooperative_launch"):      # how a kernel is launched changes nothing it computes
            assert torch.equal(g, w)
        else:
            # Both output-stationary kernels apply bias, affine, residual and ReLU to the fp32 accumulator and round once;
            # they multiply the same chunks in the same order, with the operand roles exchanged.
            assert int(ulp_distance(g, w).max()) <= 1, f"case {i}: {int((ulp_distance(g, w) > 0).sum())} values differ"
    C.check_status()


@pytest.mark.parametrize("n,cin,cout,bias", [(1, 8, 1, True), (255, 96, 19, True), (256, 96, 19, False), (25001, 64, 20, True),
                                             (4097, 32, 32, True), (1000, 256, 13, False), (777, 16, 8, True), (3000, 24, 5, True),
                                             (100, 512, 32, True), (17, 40, 19, False)])
def test_pointwise_head_matches_fp32_matmul(C, n, cin, cout, bias):
    """The 1x1x1 head kernel against a float32 product of the same fp16 inputs, rounded once (the reference computes
    this layer with torch.mm, spira/nn/conv.py:312-316): tolerance 2e-3 relative / 1e-3 absolute."""
    g = torch.Generator(device="cuda").manual_seed(n + cin + cout)
    x = (torch.randn(n, cin, device="cuda", generator=g) * 0.7).half()
    w = (torch.randn(cin, cout, device="cuda", generator=g) / cin ** 0.5).half()
    b = torch.randn(cout, device="cuda", generator=g).half() if bias else None
    got = C.pointwise(x, w, b)
    assert got is not None and got.shape == (n, cout) and got.dtype == torch.float16
    want = x.float() @ w.float() + (b.float() if bias else 0.0)
    assert_features_close(got, want, rtol=2e-3, atol=1e-3)
    torch.cuda.synchronize()


def test_pointwise_head_declines_what_it_does_not_cover(C, lib):
    x = torch.zeros(10, 96, device="cuda").half()
    assert C.pointwise(x, torch.zeros(96, 64, device="cuda").half(), None) is None          # too many output channels
    assert C.pointwise(x[:, :4].contiguous(), torch.zeros(4, 8, device="cuda").half(), None) is None   # c_in not a multiple of 8
    assert C.pointwise(torch.zeros(10, 1024, device="cuda").half(), torch.zeros(1024, 32, device="cuda").half(), None) is None
    assert C.pointwise(x.float(), torch.zeros(96, 8, device="cuda"), None) is None           # fp16 only
    out = torch.empty(10, 64, device="cuda").half()
    rc = lib.spira_b200_pointwise(x.data_ptr(), x.data_ptr(), None, 10, 96, 64, out.data_ptr(), None)
    assert rc == -3 and b"pointwise" in lib.spira_b200_last_error()
    assert C.pointwise(x[:0], torch.zeros(96, 8, device="cuda").half(), None).shape == (0, 8)
