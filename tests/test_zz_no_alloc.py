"""GPU: the allocation-free weight-stationary entry point against the regular one, through the C ABI.

``spira_b200_conv_ws_static`` keeps its fp32 scratch in a fixed array inside the library, for hosts that may not
allocate while serving requests (a server with a device-memory budget fixed at start-up, or an embedder without an
allocator to borrow from).  It must give the same features as ``spira_b200_conv_ws`` -- twice in a row, because the
shared array still holds the previous call's partial sums when the second call starts -- and refuse problems larger
than its built-in scratch.  This file is collected last so that a failure here cannot hide any other test."""
import ctypes as C

import numpy as np
import pytest
import torch

import spira_oracle as O
from helpers import surface, keys_to_torch, assert_features_close

pytestmark = pytest.mark.gpu


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def test_static_scratch_matches_caller_scratch(lib):
    from spira_b200 import _lib
    from spira_b200.nn.functional import _C
    c = surface(41, 9000)
    keys, _ = O.flat_sort(c)
    n = len(keys)
    tk = keys_to_torch(keys)
    m = _C.cuda_binary_search(tk, tk, (3, 3, 3), (1, 1, 1), 1)
    lists = m[2]._sb["ws"]
    rng = np.random.default_rng(41)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    status = _C.status_word("cuda")
    for cin, cout in ((64, 64), (32, 96)):
        feats = torch.from_numpy(rng.normal(size=(n, cin)).astype(np.float16)).cuda()
        w = torch.from_numpy((rng.normal(size=(27, cin, cout)) / np.sqrt(27 * cin)).astype(np.float16)).cuda()
        packed = _C.packed_weights(w, _lib.PACK_WS)
        common = (_ptr(feats), _ptr(w), _ptr(packed), None, _ptr(lists.in_idx), _ptr(lists.out_idx), _ptr(lists.naddrs),
                  _ptr(lists.qnaddrs), lists.rows, lists.qmapsize // 128, 1 if lists.mirror else 0, 0, n, n, 27, cin, cout)
        want = torch.empty((n, cout), dtype=torch.float16, device="cuda")
        accum = torch.empty((n, cout), dtype=torch.float32, device="cuda")
        _lib.call("spira_b200_conv_ws", *common, _ptr(accum), _ptr(want), _ptr(status), stream)
        for attempt in range(2):      # the second call starts from the first call's leftovers in the shared array
            got = torch.full((n, cout), float("nan"), dtype=torch.float16, device="cuda")
            _lib.call("spira_b200_conv_ws_static", *common, _ptr(got), _ptr(status), stream)
            torch.cuda.synchronize()
            assert_features_close(got, want)
        assert_features_close(want, O.conv_ws(feats.cpu(), w.cpu(), m[2].cpu().numpy(), n))
    _C.check_status()


def test_static_scratch_rejects_oversized_problems(lib):
    from spira_b200 import _lib
    too_many = _lib.STATIC_SCRATCH_FLOATS // 64 + 1
    one = torch.zeros(16, dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match="built-in scratch"):
        _lib.call("spira_b200_conv_ws_static", _ptr(one), _ptr(one), None, None, _ptr(one), _ptr(one), _ptr(one), _ptr(one), 1, 0,
                  0, 0, 1, too_many, 27, 64, 64, _ptr(one), None, None)
