"""GPU parity: packing, sorting and down-sampling through the C-ABI vs the oracle (bit exact)."""
import numpy as np
import pytest
import torch

import spira_oracle as O
from helpers import cloud, dev, keys_from_torch, keys_to_torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def C(lib):
    from spira_b200.nn.functional import _C
    return _C


@pytest.mark.parametrize("double", [False, True])
@pytest.mark.parametrize("n", [1, 127, 128, 129, 5000, 200_000])
def test_flatten_sort(C, n, double):
    rng = np.random.default_rng(n)
    hi = 60000 if double else 250
    c = rng.integers(0, hi, size=(n, 3)).astype(np.int32)       # duplicates on purpose: the sort is stable
    keys, perm = C.cuda_flatten_sort(dev(c), double)
    want_k, want_i = O.flat_sort(c, double)
    np.testing.assert_array_equal(keys_from_torch(keys), want_k)
    np.testing.assert_array_equal(perm.cpu().numpy(), want_i)
    assert keys.dtype == (torch.int64 if double else torch.int32) and perm.dtype == torch.int32
    back = C.cuda_unflatten(keys)
    np.testing.assert_array_equal(back.cpu().numpy(), c[want_i])


def test_flatten_sort_empty(C):
    keys, perm = C.cuda_flatten_sort(torch.empty((0, 3), dtype=torch.int32, device="cuda"), False)
    assert keys.numel() == 0 and perm.numel() == 0


def test_order_permutes_features(C):
    import spira_b200 as sp
    c = cloud(3, 4000)
    f = np.random.default_rng(3).normal(size=(len(c), 4)).astype(np.float16)
    x = sp.SparseTensor(dev(c), dev(f)).order()
    want_k, want_i = O.flat_sort(c)
    np.testing.assert_array_equal(keys_from_torch(x._coordinates), want_k)
    np.testing.assert_array_equal(x._features.cpu().numpy(), f[want_i])
    f5 = np.random.default_rng(4).normal(size=(len(c), 5)).astype(np.float16)   # 10-byte rows: 2-byte path
    x5 = sp.SparseTensor(dev(c), dev(f5)).order()
    np.testing.assert_array_equal(x5._features.cpu().numpy(), f5[want_i])


@pytest.mark.parametrize("double", [False, True])
def test_streamed_output_generate(C, double):
    c = cloud(5, 30000, 32, 160, zhi=90)
    keys, _ = O.flat_sort(c, double)
    strides = [(2, 2, 2), (4, 4, 4), (8, 8, 8), (16, 16, 16), (8, 8, 16), (1, 2, 4)]
    got = C.cuda_streamed_output_generate(keys_to_torch(keys), strides)
    want = O.streamed_output_generate(keys, strides)
    assert len(got) == len(strides)
    for g, w in zip(got, want):
        np.testing.assert_array_equal(keys_from_torch(g), w)
    one = C.cuda_downsample(keys_to_torch(keys), 2, 2, 2)
    np.testing.assert_array_equal(keys_from_torch(one), want[0])


def test_bad_arguments_raise(C):
    with pytest.raises(RuntimeError):
        C.cuda_flatten_sort(torch.zeros((4, 2), dtype=torch.int32, device="cuda"))
    with pytest.raises(RuntimeError):
        C.cuda_downsample(torch.zeros(4, dtype=torch.int32, device="cuda"), 3, 2, 2)     # not a power of two
    with pytest.raises(NotImplementedError):
        C.cuda_unflatten(torch.zeros(4, dtype=torch.int32))


@pytest.mark.parametrize("double", [False, True])
@pytest.mark.parametrize("strides", [[(2, 2, 2), (4, 4, 4), (8, 8, 8), (16, 16, 16)], [(2, 2, 1), (2, 4, 2), (4, 4, 2), (4, 8, 4)],
                                     [(1, 1, 2)], [(1, 1, 1), (2, 2, 2)]])
def test_sort_free_downsampling_of_sorted_keys(C, double, strides):
    """Strides that double level by level take the path without a sort; it must agree with the oracle, with the
    sorting path, and fall back to the sorting path when the input is not sorted."""
    c = cloud(7, 40000, 32, 200, zhi=120)
    keys, _ = O.flat_sort(c, double)
    assert C._strides_double(strides)
    want = O.streamed_output_generate(keys, strides)
    got = C.cuda_streamed_output_generate(keys_to_torch(keys), strides)
    for g, w in zip(got, want):
        np.testing.assert_array_equal(keys_from_torch(g), w)
    C.SORT_FREE_DOWNSAMPLE = False
    try:
        ref = C.cuda_streamed_output_generate(keys_to_torch(keys), strides)
    finally:
        C.SORT_FREE_DOWNSAMPLE = True
    for g, r in zip(got, ref):
        assert torch.equal(g, r)
    shuffled = keys[np.random.default_rng(1).permutation(len(keys))]
    again = C.cuda_streamed_output_generate(keys_to_torch(shuffled), strides)
    for g, w in zip(again, want):
        np.testing.assert_array_equal(keys_from_torch(g), w)


def test_sort_free_downsampling_rejects_other_strides(C, lib):
    import ctypes
    n = ctypes.c_size_t()
    assert lib.spira_b200_downsample_sorted_workspace(100, 4, ctypes.byref(n)) == 0
    buf = torch.zeros(4096, dtype=torch.int32, device="cuda")
    strides = (ctypes.c_int32 * 3)(4, 4, 4)
    outs = (ctypes.c_void_p * 1)(buf.data_ptr())
    rc = lib.spira_b200_downsample_sorted(buf.data_ptr(), 100, 4, 1, strides, outs, buf.data_ptr(), buf.data_ptr(), n.value, None, None)
    assert rc != 0
