"""CPU: host-side logic that needs no GPU -- stride rules of the sort-free down-sampling, the selector's cost model,
the lazily materialised result tuples."""
import pytest


def test_strides_that_double_level_by_level():
    from spira_b200.nn.functional import _C
    assert _C._strides_double([(2, 2, 2), (4, 4, 4), (8, 8, 8)])
    assert _C._strides_double([(1, 1, 2), (2, 1, 2), (2, 2, 4)])
    assert not _C._strides_double([(4, 4, 4)])                       # 1 -> 4 skips a level
    assert not _C._strides_double([(2, 2, 2), (8, 8, 8)])
    assert not _C._strides_double([(2, 2, 2), (1, 2, 2)])            # strides never shrink
    assert not _C._strides_double([(3, 3, 3)])


def test_selector_model_orders_the_obvious_cases():
    from spira_b200.utils.helpers import estimate_layer_us, choose_dataflow
    # big surface-dense level, narrow layer: output-stationary (no atomics); tiny deep level, wide layer: weight-stationary
    os_us, ws_us = estimate_layer_us(96, 96, 27, 127363, 1042915)
    assert os_us < ws_us
    os_us, ws_us = estimate_layer_us(256, 256, 27, 1961, 13223)
    assert ws_us < os_us
    assert choose_dataflow(96, 96, 27, 127363, 1042915, None) == 0
    assert choose_dataflow(256, 256, 27, 1961, 13223, None) == 1
    assert choose_dataflow(4, 32, 27, 127363, 1042915, None) == 0     # the tensor-core kernels cannot tile a 4-channel stem
    # a transposed output-stationary layer also pays for its inverse map
    a, _ = estimate_layer_us(96, 96, 27, 127363, 271937, submanifold=False, transposed=False)
    b, _ = estimate_layer_us(96, 96, 27, 127363, 271937, submanifold=False, transposed=True)
    assert b > a
    # more pairs never make a layer cheaper
    for df in (0, 1):
        small = estimate_layer_us(64, 64, 27, 14014, 50000)[df]
        large = estimate_layer_us(64, 64, 27, 14014, 150000)[df]
        assert large >= small


def test_weight_stationary_result_tuple_fills_its_list_slots_on_demand():
    from spira_b200.nn.functional import _C

    class Lists:
        nbmaps, nbsizes, naddrs, qnaddrs = "nbmaps", "nbsizes", "naddrs", "qnaddrs"
    t = _C._WsTuple((10, 7, "map", Lists()))
    assert len(t) == 9 and t[0] == 10 and t[1] == 7 and t[2] == "map"
    assert t[3] == "nbmaps" and t[4] == "nbsizes" and t[5] == "naddrs" and t[6] == "qnaddrs" and t[-3] == "qnaddrs"
    assert t[7] is None and t[8] is None
    assert list(t) == [10, 7, "map", "nbmaps", "nbsizes", "naddrs", "qnaddrs", None, None]
    assert t[2:5] == ("map", "nbmaps", "nbsizes")
    s, tt, m, *rest = t
    assert (s, tt, m) == (10, 7, "map") and rest[0] == "nbmaps"


def test_cache_entries_of_the_network_wide_build_keep_list_slots_empty():
    from spira_b200.nn import KernelMapCache
    from spira_b200.nn.functional import _C

    class Lists:
        nbmaps = nbsizes = naddrs = qnaddrs = "x"
    e = KernelMapCache._entry(_C._WsTuple((3, 2, "map", Lists())))
    assert e == [False, 3, 2, "map", None, None, None, None, None, None]
    assert KernelMapCache._entry((3, 2, "map", 1, 2, 3, 4, 5, 6)) == [False, 3, 2, "map", 1, 2, 3, 4, 5, 6]


def test_grouping_is_weighed_against_its_cost():
    from spira_b200.utils.helpers import estimate_layer_us, grouping_cost_us
    # five wide layers on one 127 k-voxel map save far more than the sort costs; two 16-channel layers on 300 k do not
    saved = 5 * (estimate_layer_us(96, 96, 27, 127363, 1042915, 25985, grouped=False)[0]
                 - estimate_layer_us(96, 96, 27, 127363, 1042915, 25985, grouped=True)[0])
    assert saved > grouping_cost_us(127363)
    saved = 2 * (estimate_layer_us(16, 16, 27, 300000, 2400000, 2343 * 27, grouped=False)[0]
                 - estimate_layer_us(16, 16, 27, 300000, 2400000, 2343 * 27, grouped=True)[0])
    assert saved < grouping_cost_us(300000)
    assert estimate_layer_us(96, 96, 27, 127363, 1042915, 25985, grouped=False)[0] > estimate_layer_us(96, 96, 27, 127363, 1042915, 25985)[0]
    # kernels wider than 32 offsets are never grouped: the flag changes nothing
    assert estimate_layer_us(64, 64, 125, 50000, 900000, 40000, grouped=True) == estimate_layer_us(64, 64, 125, 50000, 900000, 40000, grouped=False)


def test_concurrent_builds_never_expose_a_partial_library(tmp_path):
    """Several ranks of one node call build() at the same moment.  With a stand-in compiler that writes its output in
    two halves, the library path must only ever hold a complete file, and every process must return successfully."""
    import os
    import subprocess
    import sys
    import time
    from pathlib import Path
    root = Path(__file__).resolve().parents[1]
    fake = tmp_path / "fake_nvcc"
    fake.write_text("#!/bin/sh\n"
                    "out=\"\"; shared=0\n"
                    "while [ $# -gt 0 ]; do case \"$1\" in -o) out=\"$2\"; shift;; -shared) shared=1;; esac; shift; done\n"
                    "if [ $shared = 1 ]; then printf FIRSTHALF > \"$out\"; sleep 0.3; printf SECONDHALF >> \"$out\"; else printf obj > \"$out\"; fi\n")
    fake.chmod(0o755)
    lib = tmp_path / "libfake.so"
    code = ("import sys; sys.path.insert(0, %r)\n"
            "from pathlib import Path\n"
            "from spira_b200 import build\n"
            "build.build(force=True, lib=Path(%r), objdir=Path(%r))\n" % (str(root), str(lib), str(tmp_path / "obj")))
    env = dict(os.environ, NVCC=str(fake))
    procs = [subprocess.Popen([sys.executable, "-c", code], env=env) for _ in range(4)]
    seen = set()
    while any(p.poll() is None for p in procs):
        if lib.exists():
            seen.add(lib.read_bytes())
        time.sleep(0.01)
    assert all(p.returncode == 0 for p in procs)
    assert lib.read_bytes() == b"FIRSTHALFSECONDHALF"
    assert seen <= {b"FIRSTHALFSECONDHALF"}
    assert not list(tmp_path.glob("*.tmp"))
