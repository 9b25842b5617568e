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


@pytest.mark.parametrize("tag", ["u32", "u64"])
@pytest.mark.parametrize("name", ["sub3", "sub5"])
@pytest.mark.parametrize("df", [2, 3, 4, 5, 6, 7, 8])
def test_mirrored_masks_and_hybrid_maps(g, tag, name, df):
    if f"{tag}_{name}_df{df}_map" not in g.files:
        pytest.skip("golden vectors predate the hybrid dataflows: regenerate with tests/golden/make_golden.py on a GPU box")
    keys = u(g[f"{tag}_keys"])
    ks = CASES[name][2]
    ws = O.kernel_map(keys, keys, ks, (1, 1, 1), "ws")
    n = len(keys)
    got = {}
    if df == 2:
        K = ws.shape[0]
        sm, tm, sizes = O.gs_masks_half(ws[:(K + 1) // 2], K, n, n)
        got = {"map": ws, 3: sm, 4: tm, 5: sizes}
    else:
        h = O.hybrid_structures(ws, n, n, ks, df)
        got["map"] = h["map"]
        if df % 2 == 1:
            got.update({3: h["nbmaps"], 4: h["nbsizes"], 5: h["naddrs"], 6: h["qnaddrs"], "sizes": h["sizes"]})
        else:
            got.update({3: h["smask"], 4: h["tmask"], 5: h["nbsizes"]})
    np.testing.assert_array_equal(got["map"], g[f"{tag}_{name}_df{df}_map"])
    for slot in (3, 4, 5, 6):
        key = f"{tag}_{name}_df{df}_slot{slot}"
        assert (key in g.files) == (slot in got), f"slot {slot} presence"
        if slot in got:
            np.testing.assert_array_equal(got[slot], g[key])
    if "sizes" in got:
        np.testing.assert_array_equal(got["sizes"], g[f"{tag}_{name}_df{df}_sizes"])


@pytest.mark.parametrize("df", [2, 3, 4, 5, 6, 7, 8])
def test_mask_and_hybrid_features(g, df):
    if f"conv_df{df}" not in g.files:
        pytest.skip("golden vectors predate the hybrid dataflows: regenerate with tests/golden/make_golden.py on a GPU box")
    f, w = torch.from_numpy(g["feats"]), torch.from_numpy(g["weights"])
    n = f.shape[0]
    # the hybrid calls read the kernel tensor in L1-norm order, dataflow 2 in natural order
    w_nat = w if df == 2 else O.natural_weights_from_l1(w, (3, 3, 3), df)
    got = O.conv_ws(f, w_nat, g["u32_sub3_ws"], n).float()
    want = torch.from_numpy(g[f"conv_df{df}"]).float()
    # the reference sums these dataflows in fp16 (cuBLAS Hgemm outputs, fp16 scatter sums and atomics)
    assert ((got - want).abs() <= 2e-2 + 2e-2 * want.abs()).all()


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
