"""GPU: the bounded waits of the tensor-core kernels, exercised without faulting anything.

A fused weight-stationary launch ends with a grid barrier: every CTA adds itself to a device-wide arrival counter and
waits until the counter reaches the value the host computed for this launch.  Here the host is told to ask for a value
that cannot be reached (``ws_barrier_skew_once``) and the wait limit is lowered to a few milliseconds, so the wait runs
out: the kernel must return on its own with the status word set, ``check_status`` must raise, bring the host's count
back in step with the device's and hand out a fresh zero scratch, and the next call must be correct again.  Nothing
traps, nothing is left spinning.  Collected late, so that a failure here cannot hide the other tests."""
import ctypes as C

import numpy as np
import pytest
import torch

import spira_oracle as O
from helpers import surface, keys_to_torch, assert_features_close

pytestmark = pytest.mark.gpu


def test_grid_barrier_wait_runs_out_and_the_engine_recovers(lib):
    from spira_b200.nn.functional import _C
    c = surface(17, 6000)
    keys, _ = O.flat_sort(c)
    n = len(keys)
    tk = keys_to_torch(keys)
    m = _C.cuda_binary_search(tk, tk, (3, 3, 3), (1, 1, 1), 1)
    rng = np.random.default_rng(17)
    feats = torch.from_numpy(rng.normal(size=(n, 64)).astype(np.float16)).cuda()
    w = torch.from_numpy((rng.normal(size=(27, 64, 64)) / np.sqrt(27 * 64)).astype(np.float16)).cuda()
    want = O.conv_ws(feats.cpu(), w.cpu(), m[2].cpu().numpy(), n)
    assert_features_close(_C.conv_ws(n, n, feats, w, m[2]._sb["ws"], fused=True), want)
    _C.check_status()

    default = _C.get_option("wait_limit_us")
    _C.set_option("wait_limit_us", 5000)
    _C.set_option("ws_barrier_skew_once", 1 << 20)        # one launch whose barrier target lies out of reach
    try:
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        _C.conv_ws(n, n, feats, w, m[2]._sb["ws"], fused=True)
        t1.record()
        torch.cuda.synchronize()                          # returns: the kernel gave up by itself
        assert t0.elapsed_time(t1) < 1000.0
        assert int(_C.status_word("cuda").item()) == 1
        with pytest.raises(RuntimeError, match="gave up on an internal wait"):
            _C.check_status()
    finally:
        _C.set_option("wait_limit_us", default)
    assert _C.get_option("ws_barrier_skew_once") == 0
    # the host's arrival count is back in step and the scratch is a fresh zero buffer: normal service
    for _ in range(2):
        assert_features_close(_C.conv_ws(n, n, feats, w, m[2]._sb["ws"], fused=True), want)
    _C.check_status()


def test_fused_calls_of_a_device_stay_on_one_stream(lib):
    from spira_b200 import _lib
    from spira_b200.nn.functional import _C
    c = surface(18, 3000)
    keys, _ = O.flat_sort(c)
    n = len(keys)
    tk = keys_to_torch(keys)
    m = _C.cuda_binary_search(tk, tk, (3, 3, 3), (1, 1, 1), 1)
    rng = np.random.default_rng(18)
    feats = torch.from_numpy(rng.normal(size=(n, 32)).astype(np.float16)).cuda()
    w = torch.from_numpy((rng.normal(size=(27, 32, 32)) / np.sqrt(27 * 32)).astype(np.float16)).cuda()
    want = _C.conv_ws(n, n, feats, w, m[2]._sb["ws"], fused=True)
    torch.cuda.synchronize()
    other = torch.cuda.Stream()
    with torch.cuda.stream(other):
        with pytest.raises(RuntimeError, match="another stream"):
            _C.conv_ws(n, n, feats, w, m[2]._sb["ws"], fused=True)
        # the plain call has no such limit
        assert_features_close(_C.conv_ws(n, n, feats, w, m[2]._sb["ws"], fused=False), want, rtol=4e-3, atol=4e-3)
        # after a resync the device may be bound to the new stream
        _lib.call("spira_b200_ws_barrier_resync")
        assert_features_close(_C.conv_ws(n, n, feats, w, m[2]._sb["ws"], fused=True), want, rtol=4e-3, atol=4e-3)
    torch.cuda.synchronize()
    _lib.call("spira_b200_ws_barrier_resync")
    assert_features_close(_C.conv_ws(n, n, feats, w, m[2]._sb["ws"], fused=True), want, rtol=4e-3, atol=4e-3)
    _C.check_status()
