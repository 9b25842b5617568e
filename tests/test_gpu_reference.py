"""GPU parity against the reference's OWN kernels: its native module, built from its unmodified sources by
``oracle/build_ref.py`` into ``oracle/_ref/_C.so``, is loaded next to this engine and fed the same inputs.
Maps must be bit exact as sorted (in, out, offset) triples; features within 1e-2 relative / 1e-3 absolute."""
import importlib.util
from pathlib import Path

import numpy as np
import pytest
import torch

import spira_oracle as O
from helpers import surface, keys_to_torch, keys_from_torch, assert_features_close

pytestmark = pytest.mark.gpu

REF_SO = Path(__file__).resolve().parents[1] / "oracle" / "_ref" / "_C.so"


@pytest.fixture(scope="module")
def ref():
    if not REF_SO.exists():
        pytest.skip("reference module not built (oracle/build_ref.py needs the reference checkout)")
    spec = importlib.util.spec_from_file_location("_C", str(REF_SO))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture(scope="module")
def C(lib):
    from spira_b200.nn.functional import _C
    return _C


@pytest.fixture(scope="module")
def scene():
    from spira_b200 import scenes
    c = scenes.lidar_scene(2)
    return torch.from_numpy(c).cuda()


@pytest.mark.parametrize("double", [False, True])
def test_sort_and_downsample(ref, C, scene, double):
    rk, ri = ref.cuda_flatten_sort(scene, double)
    k, i = C.cuda_flatten_sort(scene, double)
    assert torch.equal(rk, k) and torch.equal(ri, i)
    assert torch.equal(ref.cuda_unflatten(rk), C.cuda_unflatten(k))
    strides = [(2, 2, 2), (4, 4, 4), (8, 8, 8), (16, 16, 16)]
    for a, b in zip(ref.cuda_streamed_output_generate(rk, strides), C.cuda_streamed_output_generate(k, strides)):
        assert torch.equal(a, b)
    assert torch.equal(ref.cuda_downsample(rk, 2, 2, 2), C.cuda_downsample(k, 2, 2, 2))


def padded(t):
    """Same values in a buffer with slack at the end: the reference's search reads ``sources[num_sources]`` when a
    query is larger than every source key (csrc/spira/cuda/kernels/query_sorted.cuh:42,48); keep that read inside
    the allocation."""
    big = torch.empty(t.shape[0] + 64, dtype=t.dtype, device=t.device)
    big[:t.shape[0]] = t
    big[t.shape[0]:] = 0
    return big[:t.shape[0]]


def _triples(m, layout, ks):
    return O.triples(m.cpu().numpy(), layout, ks)


@pytest.mark.parametrize("ks,strided", [((3, 3, 3), False), ((5, 5, 5), False), ((3, 3, 3), True), ((2, 2, 2), True)])
def test_kernel_maps_bit_exact(ref, C, scene, ks, strided):
    keys = padded(C.cuda_flatten_sort(scene, False)[0])
    tgt = C.cuda_downsample(keys, 2, 2, 2) if strided else keys
    for df, layout in ((0, "os"), (1, "ws")):
        r = ref.cuda_binary_search(keys, tgt, ks, (1, 1, 1), df)
        m = C.cuda_binary_search(keys, tgt, ks, (1, 1, 1), df)
        assert (r[0], r[1]) == (m[0], m[1])
        assert torch.equal(r[2], m[2]), "dense map differs from the reference's"
        np.testing.assert_array_equal(_triples(r[2], layout, ks), _triples(m[2], layout, ks))
        if df == 1:
            for slot in (3, 4, 5, 6):
                assert torch.equal(r[slot], m[slot]), f"slot {slot}"
            assert (r[7], r[8]) == (m[7], m[8])
    if strided:
        r = ref.cuda_binary_search(keys, tgt, ks, (1, 1, 1), 0)
        assert torch.equal(ref.cuda_convert_transposed_os(r[2], keys.shape[0]), C.cuda_convert_transposed_os(r[2], keys.shape[0]))


def test_streamed_builder_matches(ref, C, scene):
    keys, _ = C.cuda_flatten_sort(scene, False)
    strides = [(2, 2, 2), (4, 4, 4)]
    voxels = [padded(v) for v in [keys] + C.cuda_streamed_output_generate(keys, strides)]
    ks = [(3, 3, 3)] * 5
    ss = [(1, 1, 1), (1, 1, 1), (2, 2, 2), (2, 2, 2), (4, 4, 4)]
    df = [0, 1, 1, 0, 1]
    for r, m in zip(ref.cuda_binary_search_streamed(voxels, ks, ss, df), C.cuda_binary_search_streamed(voxels, ks, ss, df)):
        assert torch.equal(r[2], m[2])


@pytest.mark.parametrize("cin,cout", [(64, 64), (32, 64), (128, 128), (4, 32)])
def test_features_against_reference_kernels(ref, C, scene, cin, cout):
    keys = padded(C.cuda_flatten_sort(scene, False)[0])
    n = keys.shape[0]
    g = torch.Generator(device="cpu").manual_seed(cin + cout)
    f = torch.randn(n, cin, generator=g).half().cuda()
    w = (torch.randn(27, cin, cout, generator=g) / np.sqrt(27 * cin)).half().cuda()
    r0 = ref.cuda_binary_search(keys, keys, (3, 3, 3), (1, 1, 1), 0)
    want = ref.cuda_sparse_convolution_forward_os(n, n, r0[2], f, w)        # fp32 accumulate in the reference too
    assert_features_close(C.cuda_sparse_convolution_forward_os(n, n, r0[2], f, w), want)
    # weight-stationary on the reference's own pair lists; weights in natural order -> permute the z-major OS result
    r1 = ref.cuda_binary_search(keys, keys, (3, 3, 3), (1, 1, 1), 1)
    perm = torch.tensor([(c % 9) * 3 + c // 9 for c in range(27)])
    want_nat = ref.cuda_sparse_convolution_forward_os(n, n, r0[2], f, w[perm.cuda()].contiguous())
    got = C.cuda_sparse_convolution_forward_ws_merged(n, n, f, w, r1[5], r1[6], r1[3], r1[7], r1[8], False)
    assert_features_close(got, want_nat)
    C.check_status()


# ---- mask format and hybrid dataflows: every slot of the reference's 9-tuple, and the forward calls that consume them ----
def _assert_same_tuple(r, m, what):
    assert (r[0], r[1]) == (m[0], m[1]), what
    assert r[2].shape == m[2].shape and torch.equal(r[2], m[2]), f"{what}: map"
    for slot in (3, 4, 5, 6):
        assert (r[slot] is None) == (m[slot] is None), f"{what}: slot {slot} presence"
        if r[slot] is not None:
            assert r[slot].shape == m[slot].shape and torch.equal(r[slot], m[slot]), f"{what}: slot {slot}"
    assert (r[7], r[8]) == (m[7], m[8]), f"{what}: list sizes"


@pytest.mark.parametrize("ks", [(3, 3, 3), (5, 5, 5)])
@pytest.mark.parametrize("df", [2, 3, 4, 5, 6, 7, 8])
def test_mask_and_hybrid_maps_bit_exact(ref, C, scene, ks, df):
    keys = padded(C.cuda_flatten_sort(scene, False)[0])
    r = ref.cuda_binary_search(keys, keys, ks, (1, 1, 1), df)
    m = C.cuda_binary_search(keys, keys, ks, (1, 1, 1), df)
    _assert_same_tuple(r, m, f"dataflow {df}, kernel {ks}")
    # and against the CPU restatement
    host = keys.cpu().numpy().view(np.uint32)
    ws = O.kernel_map(host, host, ks, (1, 1, 1), "ws")
    if df >= 3:
        h = O.hybrid_structures(ws, len(host), len(host), ks, df)
        assert np.array_equal(m[2].cpu().numpy(), h["map"])


def test_strided_mask_format_bit_exact(ref, C, scene):
    keys = padded(C.cuda_flatten_sort(scene, False)[0])
    down = C.cuda_downsample(keys, 2, 2, 2)
    _assert_same_tuple(ref.cuda_binary_search(keys, down, (3, 3, 3), (1, 1, 1), 2),
                       C.cuda_binary_search(keys, down, (3, 3, 3), (1, 1, 1), 2), "dataflow 2, strided")


@pytest.mark.parametrize("df", [2, 3, 4, 5, 6, 7, 8])
@pytest.mark.parametrize("cin,cout", [(32, 64), (64, 96)])
def test_mask_and_hybrid_forward_calls(ref, C, scene, df, cin, cout):
    """The mask-format and hybrid calls fed with the REFERENCE's own map structures (nothing of this engine attached to
    them), against the oracle and the reference's output-stationary kernel on the same mathematical layer."""
    keys = padded(C.cuda_flatten_sort(scene, False)[0])
    n = keys.shape[0]
    g = torch.Generator(device="cpu").manual_seed(df * 1000 + cin + cout)
    f = torch.randn(n, cin, generator=g).half().cuda()
    w = (torch.randn(27, cin, cout, generator=g) / np.sqrt(27 * cin)).half().cuda()      # in the order dataflow `df` reads
    r = ref.cuda_binary_search(keys, keys, (3, 3, 3), (1, 1, 1), df)
    if df == 2:
        got = C.cuda_sparse_convolution_forward_ws(n, n, 16, 16, 4, -1, f, w, r[3], r[4], r[5])
        w_nat = w
    elif df % 2 == 1:
        got = C.cuda_sparse_convolution_forward_hs_merged(n, n, f, w, r[5], r[6], r[3], None if df == 3 else r[2], r[7], r[8], False)
        w_nat = O.natural_weights_from_l1(w.cpu(), (3, 3, 3), df).cuda()
    else:
        got = C.cuda_sparse_convolution_forward_hs(n, n, 16, 16, 4, -1, f, w, r[3], r[4], r[5], None if df == 4 else r[2])
        w_nat = O.natural_weights_from_l1(w.cpu(), (3, 3, 3), df).cuda()
    # the same layer through the reference's output-stationary kernel (fp32 accumulation): z-major order of w_nat
    r0 = ref.cuda_binary_search(keys, keys, (3, 3, 3), (1, 1, 1), 0)
    zmajor_of_nat = torch.tensor([(c % 9) * 3 + c // 9 for c in range(27)]).cuda()
    want = ref.cuda_sparse_convolution_forward_os(n, n, r0[2], f, w_nat[zmajor_of_nat].contiguous())
    assert_features_close(got, want, rtol=1e-2, atol=2e-3)        # (the hybrid sum rounds its dense part once more)
    C.check_status()


def test_strided_and_transposed_mask_format_calls(ref, C, scene):
    keys = padded(C.cuda_flatten_sort(scene, False)[0])
    down = C.cuda_downsample(keys, 2, 2, 2)
    n, nd = keys.shape[0], down.shape[0]
    g = torch.Generator(device="cpu").manual_seed(77)
    w = (torch.randn(27, 32, 64, generator=g) / np.sqrt(27 * 32)).half().cuda()
    r = ref.cuda_binary_search(keys, down, (3, 3, 3), (1, 1, 1), 2)
    host_map = r[2].cpu().numpy()
    f = torch.randn(n, 32, generator=g).half().cuda()
    got = C.cuda_sparse_convolution_forward_ws(n, nd, 16, 16, 4, -1, f, w, r[3], r[4], r[5])
    assert_features_close(got, O.conv_ws(f.cpu(), w.cpu(), host_map, nd))
    # the transposed layer hands the masks over exchanged (spira/nn/conv.py:353-360)
    wt = (torch.randn(27, 64, 32, generator=g) / np.sqrt(27 * 64)).half().cuda()
    fd = torch.randn(nd, 64, generator=g).half().cuda()
    got_t = C.cuda_sparse_convolution_forward_ws(nd, n, 16, 16, 4, -1, fd, wt, r[4], r[3], r[5])
    assert_features_close(got_t, O.conv_ws_transposed(fd.cpu(), wt.cpu(), host_map, n))
    C.check_status()


def test_layers_run_the_hybrid_dataflows(ref, C, scene):
    """``SparseConv`` with ``map_dataflow`` 3-8 (kernel tensor in L1-norm order), alone and with a fused epilogue."""
    import spira_b200 as sp
    from spira_b200 import nn as spnn
    coords = scene[:40000].contiguous()
    torch.manual_seed(5)
    feats = torch.randn(coords.shape[0], 32).half().cuda()
    x = sp.SparseTensor(coords, feats).order()
    keys = x._coordinates.cpu().numpy().view(np.uint32)
    dense = O.kernel_map(keys, keys, (3, 3, 3), (1, 1, 1), "ws")
    for df in (3, 4, 5, 6, 7, 8):
        conv = spnn.SparseConv(32, 64, 3, bias=True).cuda().half()
        conv._tunable_config["map_dataflow"] = df
        cache = spnn.KernelMapCache()
        sp.set_kernel_map_cache(conv, cache)
        w_nat = O.natural_weights_from_l1(conv.kernel.data.cpu(), (3, 3, 3), df)
        want = O.conv_ws(x._features.cpu(), w_nat, dense, len(keys)).float() + conv.bias.data.float().cpu()
        with torch.no_grad():
            assert_features_close(conv(x)._features, want.half(), rtol=1e-2, atol=2e-3)
            res = torch.randn(len(keys), 64).half().cuda()
            conv.set_fused_epilogue(torch.full((64,), 0.5).cuda(), torch.full((64,), 0.25).cuda(), True)
            got = conv(x, residual=res)._features
        assert_features_close(got, torch.relu(want * 0.5 + 0.25 + res.float().cpu()).half(), rtol=1e-2, atol=3e-3)
    C.check_status()
