"""GPU: whole networks through the public API -- network-wide map precompute, both dataflows, the selector."""
import numpy as np
import pytest
import torch

import spira_oracle as O
from helpers import assert_features_close

pytestmark = pytest.mark.gpu


def run(model, cache, coords, feats, schedule, dataflow):
    import spira_b200 as sp
    x = sp.SparseTensor(coords.clone(), feats.clone()).order()
    ks, ss, ts = schedule
    cache.reset()
    cache.add_all_kernel_maps(x._coordinates, ks, ss, ts, (1, 1, 1), [dataflow] * len(ks))
    for m in model.modules():
        if hasattr(m, "_tunable_config"):
            m._tunable_config["map_dataflow"] = dataflow
    with torch.no_grad():
        return model(x), x


@pytest.mark.parametrize("resample_kernel", [3, 2])
def test_minkunet_dataflows_agree(lib, resample_kernel):
    import spira_b200 as sp
    from spira_b200 import models, scenes, nn as spnn
    from spira_b200.nn.functional import _C
    torch.manual_seed(0)
    c = scenes.lidar_scene(3)[:60000]
    coords = torch.from_numpy(c).cuda()
    feats = torch.from_numpy(scenes.features(len(c), 4, 3)).cuda()
    model = models.minkunet18(4, 19, resample_kernel).cuda().half().eval()
    cache = spnn.KernelMapCache()
    sp.set_kernel_map_cache(model, cache)
    sched = models.map_schedule(4, 3, resample_kernel)
    y0, x0 = run(model, cache, coords, feats, sched, 0)
    assert y0._features.shape == (len(c), 19) and torch.isfinite(y0._features).all()
    # dataflow 0 reads the kernel parameter in z-major order, dataflow 1 in natural order: permute once so that
    # both runs use the same mathematical weights
    nxy, kz = (resample_kernel ** 2, resample_kernel)
    for m in model.modules():
        if isinstance(m, spnn.SparseConv) and not m.is_trivial:
            nxy, kz = m.kernel_size[0] * m.kernel_size[1], m.kernel_size[2]
            K = nxy * kz
            nat_of_col = torch.tensor([(col % nxy) * kz + col // nxy for col in range(K)], device="cuda")
            w_nat = torch.empty_like(m.kernel.data)
            w_nat[nat_of_col] = m.kernel.data
            m.kernel.data = w_nat
    y1, _ = run(model, cache, coords, feats, sched, 1)
    scale = y0._features.float().abs().max().item()
    assert (y0._features.float() - y1._features.float()).abs().max().item() <= 2e-2 * max(scale, 1.0)
    _C.check_status()
    # the first stem layer against the torch-CPU oracle
    stem = model.stem[0][0]
    keys = x0._coordinates.cpu().numpy().view(np.uint32)
    dense = O.kernel_map(keys, keys, (3, 3, 3), (1, 1, 1), "ws")
    want = O.conv_ws(x0._features.cpu(), stem.kernel.data.cpu(), dense, len(keys))
    got = stem(x0)._features
    assert_features_close(got, want)


def test_selector_and_backbone(lib, tmp_path):
    import spira_b200 as sp
    from spira_b200 import models, scenes, nn as spnn
    c = scenes.lidar_scene(4)[:50000]
    model = models.second_backbone(5).cuda().half().eval()
    cache = spnn.KernelMapCache()
    sp.set_kernel_map_cache(model, cache)

    def loader():
        for s in range(3):
            yield sp.SparseTensor(torch.from_numpy(c).cuda(), torch.from_numpy(scenes.features(len(c), 5, s)).cuda()).order()

    model, chosen = sp.tune(model, loader(), cache, n_samples=2, save_dir=str(tmp_path), tune_tag="t", force_retune=True,
                            return_dataflows=True, verify=True)
    assert len(chosen) >= 4 and all(v in (0, 1) for v in chosen.values())
    x = next(loader())
    with torch.no_grad():
        y = model(x)
    assert torch.isfinite(y._features).all() and y._stride == (8, 8, 8)
    # reload from the stored file
    model2, chosen2 = sp.tune(model, loader(), cache, save_dir=str(tmp_path), tune_tag="t", return_dataflows=True)
    assert chosen2 == chosen


def test_fused_epilogues_match_the_module_by_module_result(lib):
    """spira_b200.fuse(): BatchNorm(eval) + ReLU + residual add inside the convolution kernels vs separate passes."""
    import copy
    import spira_b200 as sp
    from spira_b200 import models, scenes, nn as spnn
    from spira_b200.nn.functional import _C
    torch.manual_seed(1)
    c = scenes.lidar_scene(2)[:40000]
    coords = torch.from_numpy(c).cuda()
    feats = torch.from_numpy(scenes.features(len(c), 4, 5)).cuda()
    model = models.minkunet18(4, 19, 3).cuda().half().eval()
    for m in model.modules():                      # non-trivial BatchNorm statistics
        if isinstance(m, spnn.BatchNorm):
            m.running_mean.normal_(0, 0.2)
            m.running_var.uniform_(0.5, 1.5)
            m.weight.data.uniform_(0.8, 1.2)
            m.bias.data.normal_(0, 0.1)
    sched = models.map_schedule(4, 3, 3)
    for dataflow in (0, 1):
        cache = spnn.KernelMapCache()
        sp.set_kernel_map_cache(model, cache)
        y_ref, _ = run(model, cache, coords, feats, sched, dataflow)
        fused = sp.fuse(copy.deepcopy(model))
        n_fused = sum(1 for m in fused.modules() if isinstance(m, spnn.SparseConv) and m._fused is not None)
        assert n_fused == 42
        cache2 = spnn.KernelMapCache()
        sp.set_kernel_map_cache(fused, cache2)
        y_fused, _ = run(fused, cache2, coords, feats, sched, dataflow)
        scale = y_ref._features.float().abs().max().item()
        assert (y_ref._features.float() - y_fused._features.float()).abs().max().item() <= 3e-2 * max(scale, 1.0)
    _C.check_status()


def test_compiled_replay_matches_eager(lib):
    """compile_model(): the recorded tape replayed on OTHER scenes gives what the eager modules give."""
    import spira_b200 as sp
    from spira_b200 import models, scenes, nn as spnn
    from spira_b200.nn.functional import _C
    torch.manual_seed(2)
    model = sp.fuse(models.minkunet18(4, 19, 3).cuda().half().eval())
    cache = spnn.KernelMapCache()
    sp.set_kernel_map_cache(model, cache)
    sched = models.map_schedule(4, 3, 3)
    full = scenes.lidar_scene(4)

    def prepare(n, seed, dataflows):
        x = sp.SparseTensor(torch.from_numpy(full[:n]).cuda(), torch.from_numpy(scenes.features(n, 4, seed)).cuda()).order()
        cache.reset()
        cache.add_all_kernel_maps(x._coordinates, *sched, (1, 1, 1), dataflows)
        return x

    for dataflows in ([0] * 9, [0, 1, 0, 1, 0, 1, 1, 1, 1]):
        for i, m in enumerate(mod for mod in model.modules() if isinstance(mod, spnn.SparseConv)):
            pass
        # per-layer dataflow follows the map of its group
        def set_flows():
            for mod in model.modules():
                if isinstance(mod, spnn.SparseConv):
                    mod._tunable_config["map_dataflow"] = 0
        set_flows()
        if any(dataflows):
            ks, ss, ts = sched
            flow_of = {}
            for i in range(len(ks)):
                stride_ratio = tuple(b // a for a, b in zip(ss[i], ss[i + 1]))
                flow_of[(ss[i], ks[i], stride_ratio)] = dataflows[i]
            hooks = []
            def hook(mod, inp, out):
                st = inp[0]._stride
                eff = tuple(a // b for a, b in zip(st, mod.stride)) if mod.transposed else st
                mod._tunable_config["map_dataflow"] = flow_of.get((eff, mod.kernel_size, mod.stride), 0)
            x0 = prepare(30000, 0, [1] * 9)
            for mod in model.modules():
                if isinstance(mod, spnn.SparseConv):
                    mod._tunable_config["map_dataflow"] = 1
                    hooks.append(mod.register_forward_hook(hook))
            with torch.no_grad():
                model(x0)
            for h in hooks:
                h.remove()
        import spira_b200.compile as spc
        x = prepare(30000, 1, dataflows)
        spc.NATIVE_TAPE = False
        try:
            replay = sp.compile_model(model, x, cache)        # operator by operator from Python
        finally:
            spc.NATIVE_TAPE = True
        native = sp.compile_model(model, x, cache)            # one spira_b200_run_tape call per scene
        assert replay.native is None and native.native is not None, native.native_error
        for n, seed in ((30000, 1), (52000, 2), (17000, 3)):
            x = prepare(n, seed, dataflows)
            with torch.no_grad():
                want = model(x)
            scale = want._features.float().abs().max().item()
            got = replay(x)
            assert got._stride == want._stride and got._features.shape == want._features.shape
            tol = 0.0 if not any(dataflows) else 2e-2 * max(scale, 1.0)     # OS is deterministic; WS sums with atomics
            assert (got._features.float() - want._features.float()).abs().max().item() <= tol
            # the native tape runs the 1x1x1 shortcuts on the engine's own kernel instead of the library GEMM (one
            # rounding instead of two) and reads concatenations as two sources: equal up to those roundings
            got = native(x)
            assert got._stride == want._stride and got._features.shape == want._features.shape
            tol = (5e-3 if not any(dataflows) else 2e-2) * max(scale, 1.0)
            assert (got._features.float() - want._features.float()).abs().max().item() <= tol
            again = native(x)
            if not any(dataflows):
                assert torch.equal(again._features, got._features)
    _C.check_status()


def test_native_tape_declines_what_it_does_not_cover(lib):
    """A pass with an operator outside the tape executor (an unfused BatchNorm) replays from Python, with the reason kept."""
    import spira_b200 as sp
    from spira_b200 import models, scenes, nn as spnn
    torch.manual_seed(0)
    model = models.minkunet18(4, 19, 3).cuda().half().eval()            # not fused: BatchNorm / ReLU stay torch operators
    cache = spnn.KernelMapCache()
    sp.set_kernel_map_cache(model, cache)
    sched = models.map_schedule(4, 3, 3)
    c = scenes.lidar_scene(2)[:20000]
    x = sp.SparseTensor(torch.from_numpy(c).cuda(), torch.from_numpy(scenes.features(len(c), 4, 0)).cuda()).order()
    cache.add_all_kernel_maps(x._coordinates, *sched, (1, 1, 1), [0] * 9)
    for m in model.modules():
        if hasattr(m, "_tunable_config"):
            m._tunable_config["map_dataflow"] = 0
    compiled = sp.compile_model(model, x, cache)
    assert compiled.native is None and "torch operator" in compiled.native_error
    with torch.no_grad():
        want = model(x)
    assert torch.equal(compiled(x)._features, want._features)


@pytest.mark.parametrize("dataflow", [0, 1, 2])
def test_rebuilding_maps_every_scene_releases_the_previous_ones(lib, dataflow):
    """A serving loop resets the cache and rebuilds all maps per scene: device memory must return to the same level
    (the map structures hold no reference cycle that would keep a scene's lists alive)."""
    import gc
    import spira_b200 as sp
    from spira_b200 import models, scenes, nn as spnn
    c = scenes.lidar_scene(5)[:30000]
    coords = torch.from_numpy(c).cuda()
    feats = torch.from_numpy(scenes.features(len(c), 4, 5)).cuda()
    model = models.minkunet18(4, 19, 3).cuda().half().eval()
    cache = spnn.KernelMapCache()
    sp.set_kernel_map_cache(model, cache)
    sched = models.map_schedule(4, 3, 3)
    gc.collect()
    gc.disable()
    try:
        levels = []
        for _ in range(6):
            y, _x = run(model, cache, coords, feats, sched, dataflow)
            del y, _x
            cache.reset()
            torch.cuda.synchronize()
            levels.append(torch.cuda.memory_allocated())
    finally:
        gc.enable()
    assert levels[-1] == levels[1], levels


def test_inverse_maps_of_transposed_layers_are_prebuilt_from_the_second_scene_on(lib):
    import spira_b200 as sp
    from spira_b200 import models, scenes, nn as spnn
    torch.manual_seed(1)
    c = scenes.lidar_scene(6)[:40000]
    coords = torch.from_numpy(c).cuda()
    feats = torch.from_numpy(scenes.features(len(c), 4, 6)).cuda()
    model = models.minkunet18(4, 19, 3).cuda().half().eval()
    cache = spnn.KernelMapCache()
    sp.set_kernel_map_cache(model, cache)
    sched = models.map_schedule(4, 3, 3)
    y0, _ = run(model, cache, coords, feats, sched, 0)          # inverses built on demand, their keys remembered
    assert len(cache._inverse_keys) == 4
    x = sp.SparseTensor(coords.clone(), feats.clone()).order()
    ks, ss, ts = sched
    cache.reset()
    cache.add_all_kernel_maps(x._coordinates, ks, ss, ts, (1, 1, 1), [0] * len(ks))
    inv = [v for k, v in cache._derived.items() if k[1] == "inverted"]
    assert len(inv) == 4 and all(v._sb["grouped"] is not None for v in inv if v.shape[0] >= 1024)
    with torch.no_grad():
        y1 = model(x)
    assert torch.equal(y0._features, y1._features)


def test_group_policy_switches_the_grouping_off_per_map(lib):
    import spira_b200 as sp
    from spira_b200 import models, scenes, nn as spnn
    torch.manual_seed(2)
    c = scenes.lidar_scene(7)[:30000]
    coords = torch.from_numpy(c).cuda()
    feats = torch.from_numpy(scenes.features(len(c), 4, 7)).cuda()
    model = models.minkunet18(4, 19, 3).cuda().half().eval()
    cache = spnn.KernelMapCache()
    sp.set_kernel_map_cache(model, cache)
    sched = models.map_schedule(4, 3, 3)
    y0, _ = run(model, cache, coords, feats, sched, 0)
    key0 = ((1, 1, 1), (1, 1, 1), (3, 3, 3))
    assert cache._kernel_maps_cache[key0][3]._sb["grouped"] is not None
    cache.set_group_policy({k: False for k in cache._kernel_maps_cache})
    y1, _ = run(model, cache, coords, feats, sched, 0)
    assert all(e[3]._sb["grouped"] is None for e in cache._kernel_maps_cache.values())
    assert torch.equal(y0._features, y1._features)        # grouping never changes a result


@pytest.mark.parametrize("dataflow", [0, 1])
def test_network_on_64_bit_keys_matches_32_bit_keys(lib, dataflow):
    """The key width changes how coordinates are packed, not which voxels neighbour which: the same scene ordered with
    64-bit keys yields the same voxel order, the same maps and therefore the same features."""
    import spira_b200 as sp
    from spira_b200 import models, scenes, nn as spnn
    from spira_b200.nn.functional import _C
    torch.manual_seed(1)
    c = scenes.lidar_scene(5)[:40000]
    coords = torch.from_numpy(c).cuda()
    feats = torch.from_numpy(scenes.features(len(c), 4, 5)).cuda()
    model = models.minkunet18(4, 19, 2).cuda().half().eval()
    cache = spnn.KernelMapCache()
    sp.set_kernel_map_cache(model, cache)
    ks, ss, ts = models.map_schedule(4, 3, 2)
    for m in model.modules():
        if hasattr(m, "_tunable_config"):
            m._tunable_config["map_dataflow"] = dataflow
    outs = []
    for double in (False, True):
        x = sp.SparseTensor(coords.clone(), feats.clone(), double=double).order()
        assert x._coordinates.dtype == (torch.int64 if double else torch.int32)
        cache.reset()
        cache.add_all_kernel_maps(x._coordinates, ks, ss, ts, (1, 1, 1), [dataflow] * len(ks))
        with torch.no_grad():
            outs.append((model(x)._features.clone(), x._features.clone()))
    (y32, x32), (y64, x64) = outs
    assert torch.equal(x32, x64)                                             # same voxel order
    if dataflow == 0:
        assert torch.equal(y32, y64)                                         # deterministic path: bit-identical
    else:
        assert_features_close(y64, y32, rtol=1e-2, atol=4e-3)
    _C.check_status()


def test_two_map_builds_in_flight_keep_their_own_level_sizes(lib):
    """Two caches start their network-wide builds before either reads its level sizes back: every pending build owns
    its pinned landing buffer, so neither sees the other scene's sizes."""
    from spira_b200 import models, scenes, nn as spnn
    from spira_b200.nn.functional import _C
    ks, ss, ts = models.map_schedule(3, 3, 3)
    scenes_k, caches = [], []
    for seed, n in ((7, 30000), (8, 9000)):
        c = scenes.lidar_scene(seed)[:n]
        keys, _ = _C.cuda_flatten_sort(torch.from_numpy(c).cuda(), False)
        scenes_k.append(keys)
    for keys in scenes_k:                    # both builds are pending now
        cache = spnn.KernelMapCache()
        cache.add_all_kernel_maps(keys, ks, ss, ts, (1, 1, 1), [0] * len(ks))
        assert cache._pending is not None
        caches.append(cache)
    for keys, cache in zip(scenes_k, caches):
        host = keys.cpu().numpy().view(np.uint32)
        for stride in ts:
            want = O.downsample(host, stride)
            got = cache._coordinates_cache[stride].cpu().numpy().view(np.uint32)
            assert np.array_equal(got, want), f"level {stride} of a scene with {len(host)} voxels"
    _C.check_status()


@pytest.mark.parametrize("kind", ["second", "minkunet"])
def test_batched_scenes_compute_what_the_scenes_compute_alone(lib, kind):
    """Three scenes merged into one sparse tensor (``spira_b200.batch``) against the same scenes one at a time.
    The all-convolution backbone on the output-stationary dataflow must agree bit for bit; the U-Net (library GEMMs for
    its 1x1x1 shortcuts, whose kernel choice depends on the row count) and the weight-stationary dataflow within tolerance."""
    import spira_b200 as sp
    from spira_b200 import batch, models, scenes, nn as spnn
    from spira_b200.nn.functional import _C
    torch.manual_seed(21)
    cin, n_down = (5, 3) if kind == "second" else (4, 4)
    model = (models.second_backbone(5) if kind == "second" else models.minkunet18(4, 19, 3)).cuda().half().eval()
    cache = spnn.KernelMapCache()
    sp.set_kernel_map_cache(model, cache)
    sched = models.map_schedule(n_down, 3, 3)
    parts = [(scenes.lidar_scene(s)[:n], s) for s, n in ((31, 30000), (32, 17000), (33, 42000))]
    cs = [torch.from_numpy(c).cuda() for c, _ in parts]
    fs = [torch.from_numpy(scenes.features(len(c), cin, s)).cuda() for c, s in parts]
    mc, mf, pitch, grid = batch.merge_scenes(cs, fs)
    for dataflow in (0, 1):
        alone = [run(model, cache, c, f, sched, dataflow)[0] for c, f in zip(cs, fs)]
        y, x = run(model, cache, mc, mf, sched, dataflow)
        stride = y._stride[0]
        ids = batch.scene_ids(_C.cuda_unflatten(y._coordinates), pitch, grid)
        for b, (got, want) in enumerate(zip(batch.split_rows(y._features, ids, len(cs)), alone)):
            assert got.shape == want._features.shape, f"scene {b}: {tuple(got.shape)} rows vs {tuple(want._features.shape)}"
            if kind == "second" and dataflow == 0:
                assert torch.equal(got, want._features), f"scene {b} differs between the batch and its own run"
            else:
                scale = max(want._features.float().abs().max().item(), 1.0)
                assert (got.float() - want._features.float()).abs().max().item() <= 2e-2 * scale
    _C.check_status()
