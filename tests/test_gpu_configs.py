"""GPU: parity on the exact benchmark configurations, at full size.

* single layer: 50,000-voxel plane / sphere scene in a 512^3 grid, 64-bit keys, one 3^3 layer 64 -> 64;
* indoor network: the ~270 k-voxel room scene, 3 input channels, 20-class head;
* SECOND-style backbone: a ~300 k-voxel multi-sweep scene, 5 input channels;
* whole networks: the same scene and weights through the REFERENCE's own Python package driving its own native module
  (``oracle/reference_module.py``) and through this engine -- eager, and fused + compiled with the selector's dataflows;
* the reference's model file (``scripts/models/spira/sparse_unet.py``, 2^3 resampling) imported unchanged on top of
  this engine through ``install_as_spira()``.

Maps must be bit exact; features within 1e-2 relative / 1e-3 absolute of the oracle and of the reference's
output-stationary kernel (fp32 accumulation in both); whole-network logits within 2e-2 of the largest logit (every
layer of the reference rounds three times -- convolution, BatchNorm, ReLU -- where the fused engine rounds once)."""
import contextlib
import sys

import numpy as np
import pytest
import torch

import spira_oracle as O
import reference_module as R
from helpers import assert_features_close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref():
    if not R.available():
        pytest.skip("reference module not built (oracle/build_ref.py needs the reference checkout)")
    return R.load_native()


@pytest.fixture(scope="module")
def ref_sp():
    if not R.package_available():
        pytest.skip("the reference's Python package is not staged (oracle/build_ref.py needs the reference checkout)")
    return R.load_package()


@pytest.fixture(scope="module")
def C(lib):
    from spira_b200.nn.functional import _C
    return _C


def padded(t):
    """Same values with slack behind them: the reference's search reads ``sources[num_sources]``
    (csrc/spira/cuda/kernels/query_sorted.cuh:42,48)."""
    big = torch.zeros(t.shape[0] + 64, dtype=t.dtype, device=t.device)
    big[:t.shape[0]] = t
    return big[:t.shape[0]]


def safe_scene(c):
    """Drops one voxel when the key tensor would end exactly on an allocator block boundary (see :func:`padded`): the
    reference's own Python cannot pad its tensors."""
    return c[:-1] if len(c) % 64 == 0 else c


def natural_from_zmajor(w, ks):
    """The kernel tensor that means, read in natural offset order (dataflows 1 and 2), what ``w`` means read in z-major
    order (dataflow 0): ``w_nat[(o * kz + iz)] = w[iz * nxy + o]`` (scripts/models/convert_weights.py:19-28)."""
    nxy, kz = ks[0] * ks[1], ks[2]
    nat_of_col = torch.tensor([(col % nxy) * kz + col // nxy for col in range(nxy * kz)], device=w.device)
    out = torch.empty_like(w)
    out[nat_of_col] = w
    return out


# ---- single layer, 64-bit keys ----------------------------------------------------------------------------------------
def test_single_layer_configuration_64_bit_keys(ref, C):
    from spira_b200 import scenes
    c = scenes.planes_and_spheres(0)
    assert c.shape == (50_000, 3) and c[:, 2].max() > 255        # needs the 16-bit z field of 64-bit keys
    coords = torch.from_numpy(c).cuda()
    keys, perm = C.cuda_flatten_sort(coords, True)
    rk, rp = ref.cuda_flatten_sort(coords, True)
    assert torch.equal(keys, rk) and torch.equal(perm, rp)
    ok, op = O.flat_sort(c, double=True)
    assert np.array_equal(keys.cpu().numpy().view(np.uint64), ok) and np.array_equal(perm.cpu().numpy(), op)
    n = len(c)
    src = padded(keys)
    feats = torch.from_numpy(scenes.features(n, 64, 0)).cuda()
    rng = np.random.default_rng(0)
    w = torch.from_numpy((rng.normal(size=(27, 64, 64)) / np.sqrt(27 * 64)).astype(np.float16)).cuda()
    m0, m1 = C.cuda_binary_search(src, src, (3, 3, 3), (1, 1, 1), 0), C.cuda_binary_search(src, src, (3, 3, 3), (1, 1, 1), 1)
    r0, r1 = ref.cuda_binary_search(src, src, (3, 3, 3), (1, 1, 1), 0), ref.cuda_binary_search(src, src, (3, 3, 3), (1, 1, 1), 1)
    assert torch.equal(m0[2], r0[2]) and torch.equal(m1[2], r1[2])
    for slot in (3, 4, 5, 6):
        assert torch.equal(m1[slot], r1[slot]), f"list slot {slot}"
    assert (m1[7], m1[8]) == (r1[7], r1[8])
    assert np.array_equal(m0[2].cpu().numpy(), O.kernel_map(ok, ok, (3, 3, 3), (1, 1, 1), "os"))
    assert np.array_equal(m1[2].cpu().numpy(), O.kernel_map(ok, ok, (3, 3, 3), (1, 1, 1), "ws"))
    # features: output-stationary (z-major weight order) vs the oracle and the reference's kernel
    got0 = C.cuda_sparse_convolution_forward_os(n, n, m0[2], feats, w)
    assert_features_close(got0, O.conv_os(feats.cpu(), w.cpu(), m0[2].cpu().numpy(), n))
    assert_features_close(got0, ref.cuda_sparse_convolution_forward_os(n, n, r0[2], feats, w))
    # weight-stationary (natural weight order): the same mathematical layer needs the permuted kernel tensor
    w_nat = natural_from_zmajor(w, (3, 3, 3))
    got1 = C.cuda_sparse_convolution_forward_ws_merged(n, n, feats, w_nat, m1[5], m1[6], m1[3], m1[7], m1[8], False)
    assert_features_close(got1, O.conv_ws(feats.cpu(), w_nat.cpu(), m1[2].cpu().numpy(), n))
    assert_features_close(got1, got0)
    C.check_status()


# ---- indoor and SECOND-style configurations: every map of the network, stems with 3 / 5 channels, the 20-class head ----
def _network_maps(C, ref, coords_np, n_down):
    from spira_b200 import models
    coords = torch.from_numpy(coords_np).cuda()
    keys, perm = C.cuda_flatten_sort(coords, False)
    ks, ss, ts = models.map_schedule(n_down, 3, 3)
    levels = C.cuda_streamed_output_generate(keys, ts)
    rlevels = ref.cuda_streamed_output_generate(keys, ts)
    for a, b in zip(levels, rlevels):
        assert torch.equal(a, b)
    voxels = [padded(v) for v in [keys] + levels]
    for df in (0, 1):
        mine = C.cuda_binary_search_streamed(voxels, ks, ss[:-1], [df] * len(ks))
        theirs = ref.cuda_binary_search_streamed(voxels, ks, ss[:-1], [df] * len(ks))
        for i, (m, r) in enumerate(zip(mine, theirs)):
            assert (m[0], m[1]) == (r[0], r[1])
            assert torch.equal(m[2], r[2]), f"map {i} (dataflow {df}) differs from the reference's"
            if df == 1:
                for slot in (3, 4, 5, 6):
                    assert torch.equal(m[slot], r[slot]), f"map {i} list slot {slot}"
                assert (m[7], m[8]) == (r[7], r[8])
    return keys, perm, voxels


def _stem_against_oracle(C, keys, perm, feats_np, cin, cout, seed):
    n = keys.shape[0]
    f = torch.from_numpy(feats_np).cuda()[perm.long()].contiguous()
    rng = np.random.default_rng(seed)
    w = torch.from_numpy((rng.normal(size=(27, cin, cout)) / np.sqrt(27 * cin)).astype(np.float16)).cuda()
    host = keys.cpu().numpy().view(np.uint32)
    dense_os = O.kernel_map(host, host, (3, 3, 3), (1, 1, 1), "os")
    m0 = C.cuda_binary_search(keys, keys, (3, 3, 3), (1, 1, 1), 0)
    assert np.array_equal(m0[2].cpu().numpy(), dense_os)
    want = O.conv_os(f.cpu(), w.cpu(), dense_os, n)
    assert_features_close(C.conv_os(n, n, m0[2], f, w, grouped=True), want)
    assert_features_close(C.conv_os(n, n, m0[2], f, w, grouped=False), want)
    return f


def test_indoor_configuration(ref, C):
    from spira_b200 import scenes
    c = scenes.room_scene(5)
    assert 200_000 < len(c) < 350_000 and c[:, 2].max() < 256
    keys, perm, _ = _network_maps(C, ref, c, 3)
    f = _stem_against_oracle(C, keys, perm, scenes.features(len(c), 3, 5, "uniform"), 3, 32, 5)
    # the 20-class head: a 1x1x1 layer with bias on 32 channels
    n = keys.shape[0]
    rng = np.random.default_rng(6)
    x = torch.from_numpy(rng.normal(size=(n, 32)).astype(np.float16)).cuda()
    w = torch.from_numpy((rng.normal(size=(32, 20)) / np.sqrt(32)).astype(np.float16)).cuda()
    b = torch.from_numpy(rng.normal(size=20).astype(np.float16)).cuda()
    got = C.pointwise(x, w, b)
    assert got is not None
    assert_features_close(got, (x.float() @ w.float() + b.float()).half())
    C.check_status()


def test_second_configuration(ref, C):
    from spira_b200 import scenes
    c = scenes.multisweep_scene(10)
    assert 250_000 < len(c) < 400_000
    keys, perm, _ = _network_maps(C, ref, c, 3)
    _stem_against_oracle(C, keys, perm, scenes.features(len(c), 5, 10), 5, 16, 10)
    C.check_status()


# ---- whole networks: the reference's Python + native module against this engine ----------------------------------------
def _randomise_batchnorm(model, seed):
    g = torch.Generator().manual_seed(seed)
    for m in model.modules():
        if isinstance(m, torch.nn.BatchNorm1d):
            m.weight.data = torch.empty(m.num_features).uniform_(0.8, 1.2, generator=g)
            m.bias.data = torch.empty(m.num_features).normal_(0, 0.1, generator=g)
            m.running_mean.data = torch.empty(m.num_features).normal_(0, 0.1, generator=g)
            m.running_var.data = torch.empty(m.num_features).uniform_(0.8, 1.2, generator=g)


def _set_dataflow(model, df):
    for m in model.modules():
        if hasattr(m, "_tunable_config"):
            m._tunable_config["map_dataflow"] = df
            m._tunable_config["force_os"] = False


WORKLOADS = {"minkunet": ("lidar_scene", 1, 4, "normal", 4), "indoor": ("room_scene", 5, 3, "uniform", 3),
             "second": ("multisweep_scene", 10, 5, "normal", 3)}


@pytest.mark.parametrize("kind", ["minkunet", "indoor", "second"])
def test_whole_network_against_the_reference_python(ref_sp, C, kind, tmp_path):
    import spira_b200 as sp
    from spira_b200 import models, scenes, nn as spnn
    scene_fn, seed, cin, feat_kind, n_down = WORKLOADS[kind]
    c = safe_scene(getattr(scenes, scene_fn)(seed))
    coords = torch.from_numpy(c).cuda()
    feats = torch.from_numpy(scenes.features(len(c), cin, seed, feat_kind)).cuda()
    ks, ss, ts = models.map_schedule(n_down, 3, 3)

    torch.manual_seed(11)
    mine = {"minkunet": lambda: models.minkunet18(4, 19, 3), "indoor": lambda: models.indoor_resunet(3, 20),
            "second": lambda: models.second_backbone(5)}[kind]()
    _randomise_batchnorm(mine, 12)
    mine = mine.cuda().half().eval()
    theirs = R.build_network(kind, ref_sp).cuda().half().eval()
    theirs.load_state_dict(mine.state_dict())

    # reference: its own SparseTensor / KernelMapCache / SparseConv on its own kernels, output-stationary (fp32 accumulation)
    _set_dataflow(theirs, 0)
    rcache = ref_sp.nn.KernelMapCache()
    ref_sp.set_kernel_map_cache(theirs, rcache)
    rx = ref_sp.SparseTensor(coordinates=coords.clone(), features=feats.clone()).order()
    rcache.add_all_kernel_maps(rx._coordinates, ks, ss, ts, (1, 1, 1), [0] * len(ks))
    with torch.no_grad():
        want = theirs(rx)._features.float()
    scale = max(want.abs().max().item(), 1.0)

    def close(got, what):
        err = (got.float() - want).abs()
        assert err.max().item() <= 2e-2 * scale, f"{kind}, {what}: max |diff| {err.max().item():.4g} of scale {scale:.4g}"
        assert err.mean().item() <= 2e-3 * scale, f"{kind}, {what}: mean |diff| {err.mean().item():.4g}"

    # this engine, eager, the same dataflow everywhere
    cache = spnn.KernelMapCache()
    sp.set_kernel_map_cache(mine, cache)
    _set_dataflow(mine, 0)
    x = sp.SparseTensor(coords.clone(), feats.clone()).order()
    assert torch.equal(x._coordinates, rx._coordinates) and torch.equal(x._features, rx._features)
    cache.add_all_kernel_maps(x._coordinates, ks, ss, ts, (1, 1, 1), [0] * len(ks))
    with torch.no_grad():
        close(mine(x)._features, "eager, output-stationary")

    # this engine as the benchmark runs it: fused epilogues, the selector's dataflow per layer group, recorded tape.
    # A layer the selector moves to the weight-stationary dataflow reads its kernel tensor in natural offset order.
    sp.fuse(mine)

    def loader():
        yield sp.SparseTensor(coords.clone(), feats.clone()).order()
    _, chosen = sp.tune(mine, loader(), cache, n_samples=1, save_dir=str(tmp_path), tune_tag=kind, force_retune=True,
                        return_dataflows=True)
    for m in mine.modules():
        if isinstance(m, spnn.SparseConv) and not m.is_trivial and m._tunable_config["map_dataflow"] != 0:
            m.kernel.data = natural_from_zmajor(m.kernel.data, m.kernel_size)
    strides = [tuple(b // a for a, b in zip(ss[i], ss[i + 1])) for i in range(len(ks))]
    dataflows = [chosen.get((ss[i], ks[i], strides[i]), 0) for i in range(len(ks))]
    x = sp.SparseTensor(coords.clone(), feats.clone()).order()
    cache.reset()
    cache.add_all_kernel_maps(x._coordinates, ks, ss, ts, (1, 1, 1), dataflows)
    compiled = sp.compile_model(mine, x, cache)
    for _ in range(2):
        x = sp.SparseTensor(coords.clone(), feats.clone()).order()
        cache.reset()
        cache.add_all_kernel_maps(x._coordinates, ks, ss, ts, (1, 1, 1), dataflows)
        close(compiled(x)._features, f"fused + compiled, dataflows {sorted(set(dataflows))}")
    C.check_status()


# ---- the reference's model file, unchanged, on this engine ---------------------------------------------------------------
@contextlib.contextmanager
def engine_registered_as_spira():
    """Temporarily makes ``import spira`` resolve to this engine (what a user of the reference does once at start-up)."""
    import spira_b200 as sp
    saved = {k: v for k, v in sys.modules.items() if k == "spira" or k.startswith("spira.")}
    for k in saved:
        del sys.modules[k]
    try:
        sp.install_as_spira()
        yield
    finally:
        for k in [k for k in sys.modules if k == "spira" or k.startswith("spira.")]:
            del sys.modules[k]
        sys.modules.update(saved)


def test_reference_model_definition_runs_unchanged_on_this_engine(ref_sp, C):
    import spira_b200 as sp
    from spira_b200 import models, scenes, nn as spnn
    with engine_registered_as_spira():
        zoo = R.load_models("spira_models_on_this_engine")
    assert zoo.SparseResUNet42.__module__.startswith("spira_models_on_this_engine")
    torch.manual_seed(3)
    mine = zoo.SparseResUNet42(in_channels=4)             # 2^3 stride-2 resampling, sparse_unet.py:112-119
    assert isinstance(mine.stem[0], spnn.SparseConv)
    _randomise_batchnorm(mine, 4)
    mine = mine.cuda().half().eval()
    theirs = R.load_models().SparseResUNet42(in_channels=4).cuda().half().eval()
    assert isinstance(theirs.stem[0], ref_sp.nn.SparseConv)
    theirs.load_state_dict(mine.state_dict())

    c = safe_scene(scenes.lidar_scene(2))
    coords = torch.from_numpy(c).cuda()
    feats = torch.from_numpy(scenes.features(len(c), 4, 2)).cuda()
    ks, ss, ts = models.map_schedule(4, 3, 2)            # the schedule of scripts/end_to_end_experiment.py:107-112
    outs = []
    for pkg, model in ((ref_sp, theirs), (sp, mine)):
        _set_dataflow(model, 0)
        cache = pkg.nn.KernelMapCache()
        pkg.set_kernel_map_cache(model, cache)
        x = pkg.SparseTensor(coordinates=coords.clone(), features=feats.clone()).order()
        cache.add_all_kernel_maps(x._coordinates, ks, ss, ts, (1, 1, 1), [0] * len(ks))
        with torch.no_grad():
            outs.append(model(x))
    assert len(outs[0]) == len(outs[1]) == 9              # stem, four encoder stages, four decoder stages
    for a, b in zip(outs[0], outs[1]):
        assert a._stride == b._stride and torch.equal(a._coordinates, b._coordinates)
        scale = max(a._features.float().abs().max().item(), 1.0)
        err = (a._features.float() - b._features.float()).abs()
        assert err.max().item() <= 2e-2 * scale and err.mean().item() <= 2e-3 * scale
    C.check_status()
