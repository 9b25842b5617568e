"""CPU: the oracle against golden vectors produced by the REFERENCE's own kernels.

``tests/golden/reference_vectors.npz`` was written by ``tests/golden/make_golden.py`` on a B200 from the reference's
native module (its unmodified sources, built by ``oracle/build_ref.py``).  Integer results must match bit for bit;
features within 1e-2 relative / 1e-3 absolute."""
from pathlib import Path

import numpy as np
import pytest
import torch

import spira_oracle as O

GOLD = Path(__file__).resolve().parent / "golden" / "reference_vectors.npz"


@pytest.fixture(scope="module")
def g():
    assert GOLD.exists(), "golden vectors missing: run tests/golden/make_golden.py on a GPU box"
    return np.load(GOLD)


def u(a):
    return a.view(np.uint32 if a.dtype.itemsize == 4 else np.uint64)


@pytest.mark.parametrize("tag", ["u32", "u64"])
def test_sort_unflatten_downsample(g, tag):
    keys, perm = O.flat_sort(g["coords"], double=(tag == "u64"))
    np.testing.assert_array_equal(keys, u(g[f"{tag}_keys"]))
    np.testing.assert_array_equal(perm, g[f"{tag}_perm"])
    np.testing.assert_array_equal(O.unpack(keys), g[f"{tag}_unflat"])
    for s in [(2, 2, 2), (4, 4, 4), (8, 8, 16)]:
        np.testing.assert_array_equal(O.downsample(keys, s), u(g[f"{tag}_down_{s[0]}_{s[1]}_{s[2]}"]))


CASES = {"sub3": ("k", "k", (3, 3, 3), (1, 1, 1)), "sub5": ("k", "k", (5, 5, 5), (1, 1, 1)),
         "down3": ("k", "d2", (3, 3, 3), (1, 1, 1)), "down2": ("k", "d2", (2, 2, 2), (1, 1, 1)),
         "lvl2": ("d2", "d4", (3, 3, 3), (2, 2, 2))}


@pytest.mark.parametrize("tag", ["u32", "u64"])
@pytest.mark.parametrize("name", list(CASES))
def test_kernel_maps_and_lists(g, tag, name):
    sets = {"k": u(g[f"{tag}_keys"]), "d2": u(g[f"{tag}_down_2_2_2"]), "d4": u(g[f"{tag}_down_4_4_4"])}
    s, t, ks, st = CASES[name]
    src, tgt = sets[s], sets[t]
    np.testing.assert_array_equal(O.kernel_map(src, tgt, ks, st, "os"), g[f"{tag}_{name}_os"])
    ws = O.kernel_map(src, tgt, ks, st, "ws")
    np.testing.assert_array_equal(ws, g[f"{tag}_{name}_ws"])
    # the walk emulation agrees as well: the inputs keep a margin, no query underflows
    np.testing.assert_array_equal(O.kernel_map(src, tgt, ks, st, "ws", emulate_reference_walk=True), ws)
    nbmaps, nbsizes, naddrs, qnaddrs, mapsize, qmapsize = O.ws_structures(ws, len(src), len(tgt))
    np.testing.assert_array_equal(nbmaps, g[f"{tag}_{name}_nbmaps"])
    np.testing.assert_array_equal(nbsizes, g[f"{tag}_{name}_nbsizes"])
    np.testing.assert_array_equal(naddrs, g[f"{tag}_{name}_naddrs"])
    np.testing.assert_array_equal(qnaddrs, g[f"{tag}_{name}_qnaddrs"])
    np.testing.assert_array_equal([mapsize, qmapsize], g[f"{tag}_{name}_sizes"])
    if name == "down3":
        np.testing.assert_array_equal(O.convert_transposed_os(g[f"{tag}_{name}_os"], len(src)), g[f"{tag}_{name}_inverse"])
        sm, tm, _ = O.gs_masks(ws, len(src), len(tgt))
        np.testing.assert_array_equal(sm, g[f"{tag}_{name}_smask"])
        np.testing.assert_array_equal(tm, g[f"{tag}_{name}_tmask"])


def test_features(g):
    f, w = torch.from_numpy(g["feats"]), torch.from_numpy(g["weights"])
    n = f.shape[0]
    got = O.conv_os(f, w, g["u32_sub3_os"], n).float()
    want = torch.from_numpy(g["conv_os_on_os_map"]).float()
    assert ((got - want).abs() <= 1e-3 + 1e-2 * want.abs()).all()
    # the reference's fused weight-stationary kernel accumulates in fp16 with fp16 atomics
    # (csrc/spira/cuda/kernels/weight_stat.cuh:835,914): compare with a correspondingly looser bound
    got_ws = O.conv_ws(f, w, g["u32_sub3_ws"], n).float()
    want_ws = torch.from_numpy(g["conv_ws_merged"]).float()
    assert ((got_ws - want_ws).abs() <= 2e-2 + 2e-2 * want_ws.abs()).all()
