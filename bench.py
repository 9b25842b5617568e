#!/usr/bin/env python
"""Benchmark of the sparse-convolution hot path on synthetic LiDAR-like scenes.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload minkunet|indoor|second]

One step = one whole scene through the reference's timed region (scripts/end_to_end_experiment.py:191-207):
``SparseTensor.order()`` + network-wide kernel-map build (``KernelMapCache.add_all_kernel_maps``) + the network's
forward pass.  Default workload: MinkUNet18-style network, fp16, random init, one ~125k-voxel scene per step
(the headline workload).  With N > 1 (launched by torch.distributed.run) every rank owns one GPU and its own
scenes; nothing is exchanged on the data path, so scaling is weak and ``value`` = scenes of all ranks / slowest rank.

``--impl reference`` is the stock reference: its own Python package (``SparseTensor``, ``KernelMapCache``, ``SparseConv``,
``tune`` over all nine dataflows) driving its own native module, both taken from ``oracle/_ref`` (built and staged from the
unmodified sources by ``oracle/build_ref.py``), on a network assembled from the reference's own blocks.
``--impl reference-kernels`` runs the same native module behind this repository's Python glue and model classes instead.
The reference has no CPU implementation of this path; if its module is unavailable the arm times the CPU oracle port.

Prints ONE JSON line (rank 0).
"""
from __future__ import annotations

import argparse
import contextlib
import functools
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

import numpy as np
import torch

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return {k: float(d[k]) for k in FALLBACK_PEAKS}, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


# ------------------------------------------------------------------------------------------------
# workloads
# ------------------------------------------------------------------------------------------------
def make_workload(name: str):
    from spira_b200 import models, scenes
    if name == "minkunet":
        return dict(model=lambda: models.minkunet18(4, 19, 3), n_down=4, channels=4, feat_kind="normal",
                    scene=lambda seed: scenes.lidar_scene(seed), seeds=[1, 2, 3, 4],
                    label="MinkUNet18-style (32|32-64-128-256|256-128-96-96, 3^3, 19 classes), 1 LiDAR-like scene ~125k voxels per step")
    if name == "indoor":
        return dict(model=lambda: models.indoor_resunet(3, 20), n_down=3, channels=3, feat_kind="uniform",
                    scene=lambda seed: scenes.room_scene(seed), seeds=[5, 6],
                    label="SparseResUNet-style indoor network (32-64-128-256), 1 room scene ~270k voxels per step")
    if name == "second":
        return dict(model=lambda: models.second_backbone(5), n_down=3, channels=5, feat_kind="normal",
                    scene=lambda seed: scenes.multisweep_scene(seed), seeds=[10, 11],
                    label="SECOND-style backbone (16-32-64-128), 1 multi-sweep scene ~300k voxels per step")
    raise SystemExit(f"unknown workload {name}")


# ------------------------------------------------------------------------------------------------
# the reference (test infrastructure under oracle/: only the reference arm touches it)
# ------------------------------------------------------------------------------------------------
def reference_tools():
    """``oracle/reference_module.py``: loaders for the reference's native module, Python package and model blocks."""
    sys.path.insert(0, str(ROOT / "oracle"))
    import reference_module
    return reference_module


def schedule(n_down: int, kernel: int = 3, resample_kernel: int = 3):
    """(kernel_sizes, source_strides, target_strides) of ``KernelMapCache.add_all_kernel_maps`` for a network with
    ``n_down`` stride-2 levels, in the builder's alternating order (scripts/end_to_end_experiment.py:107-112)."""
    kernel_sizes, source_strides, target_strides = [], [(1, 1, 1)], []
    s = 1
    for level in range(n_down + 1):
        kernel_sizes.append((kernel,) * 3)
        source_strides.append((s,) * 3)
        if level < n_down:
            kernel_sizes.append((resample_kernel,) * 3)
            s *= 2
            source_strides.append((s,) * 3)
            target_strides.append((s,) * 3)
    return kernel_sizes, source_strides, target_strides


class StockReferenceEngine:
    """The reference as its users run it: its own Python package on its own native module, a network assembled from its
    own blocks, dataflows chosen by its own ``spira.tune`` (spira/utils/helpers.py:388-618)."""

    def __init__(self, workload_name, workload, device):
        self.R = reference_tools()
        self.sp = self.R.load_package()
        torch.manual_seed(0)
        self.model = self.R.build_network(workload_name, self.sp).to(device).half().eval()
        self.cache = self.sp.nn.KernelMapCache()
        self.sp.set_kernel_map_cache(self.model, self.cache)
        self.ks, self.ss, self.ts = schedule(workload["n_down"], 3, 3)
        self.layer_strides = [tuple(b // a for a, b in zip(self.ss[i], self.ss[i + 1])) for i in range(len(self.ks))]
        self.dataflows = [0] * len(self.ks)
        self.tune_note = None

    def tune(self, dev_scenes, save_dir, n_samples=5):
        """``spira.tune`` as scripts/end_to_end_experiment.py:122-151 calls it.  The tuner needs more than three samples
        (it discards the first three of every configuration, helpers.py:236), so the scenes are cycled.  Layers with 3 or
        5 input channels cannot run the mask-format dataflows (the gather tile sizes must be multiples of four,
        spira/nn/conv.py:261): if the full search fails, it is repeated without them."""
        sp = self.sp

        def loader():
            i = 0
            while True:
                c, f = dev_scenes[i % len(dev_scenes)]
                yield sp.SparseTensor(features=f.clone(), coordinates=c.clone()).order()
                i += 1

        last = None
        for options, gs in ((None, True), ([0, 1, 3, 5, 7], False), ([0, 1], False)):
            self.cache.reset()  # (the tuner's structure pass runs on whatever maps a failed attempt left behind)
            if not gs:          # a restricted search starts from a dataflow every layer can run
                for m in self.model.modules():
                    if hasattr(m, "_tunable_config"):
                        m._tunable_config["map_dataflow"], m._tunable_config["force_os"] = 0, False
            try:
                _, chosen = sp.tune(model=self.model, data_loader=loader(), kernel_map_cache=self.cache, map_dataflow_options=options,
                                    test_force_os=True, n_samples=n_samples, force_retune=True, save_dir=save_dir, verbose=False,
                                    allow_gs_tuning=gs, return_dataflows=True)
            except (RuntimeError, ValueError, KeyError) as e:
                last = e
                try:
                    sp.nn.functional.cuda_reset_error()
                except Exception:
                    pass
                continue
            self.dataflows = [chosen.get((self.ss[i], self.ks[i], self.layer_strides[i]), 0) for i in range(len(self.ks))]
            self.tune_note = {"tuner": "spira.tune (reference)", "map_dataflow_options": options or list(range(9)),
                              "per_group": {str(k): v for k, v in chosen.items()}}
            return
        raise RuntimeError(f"the reference's tuner failed on every option set: {last}")

    def step(self, coords, feats):
        x = self.sp.SparseTensor(features=feats, coordinates=coords).order()
        self.cache.reset()
        self.cache.add_all_kernel_maps(x._coordinates, self.ks, self.ss, self.ts, (1, 1, 1), self.dataflows)
        with torch.no_grad():
            return self.model(x)._features


# ------------------------------------------------------------------------------------------------
# engine
# ------------------------------------------------------------------------------------------------
class Engine:
    def __init__(self, workload, device, dataflows=None):
        import spira_b200 as sp
        from spira_b200 import models, nn as spnn
        self.sp = sp
        torch.manual_seed(0)
        self.model = workload["model"]().to(device).half().eval()
        self.cache = spnn.KernelMapCache()
        sp.set_kernel_map_cache(self.model, self.cache)
        self.ks, self.ss, self.ts = models.map_schedule(workload["n_down"], 3, 3)
        self.layer_strides = []
        for i in range(len(self.ks)):
            self.layer_strides.append(tuple(b // a for a, b in zip(self.ss[i], self.ss[i + 1])))
        self.compiled = None
        self.set_uniform_dataflow(0)
        if dataflows is not None:
            self.dataflows = dataflows

    def set_uniform_dataflow(self, df: int):
        self.dataflows = [df] * len(self.ks)
        for m in self.model.modules():
            if hasattr(m, "_tunable_config"):
                m._tunable_config["map_dataflow"] = df
                m._tunable_config["force_os"] = False

    def apply_groups(self, chosen):
        """chosen: {(effective_stride, kernel_size, stride): dataflow} from ``tune`` -> per-map list, like
        scripts/end_to_end_experiment.py:138-151."""
        self.dataflows = [chosen.get((self.ss[i], self.ks[i], self.layer_strides[i]), 0) for i in range(len(self.ks))]

    def step(self, coords, feats):
        x = self.sp.SparseTensor(coords, feats).order()
        self.cache.reset()
        self.cache.add_all_kernel_maps(x._coordinates, self.ks, self.ss, self.ts, (1, 1, 1), self.dataflows)
        if self.compiled is not None:
            return self.compiled(x)._features
        with torch.no_grad():
            return self.model(x)._features

    def compile(self, coords, feats):
        """Records the operator tape once (spira_b200.compile_model); later steps replay it."""
        x = self.sp.SparseTensor(coords, feats).order()
        self.cache.reset()
        self.cache.add_all_kernel_maps(x._coordinates, self.ks, self.ss, self.ts, (1, 1, 1), self.dataflows)
        self.compiled = self.sp.compile_model(self.model, x, self.cache)


def tune_reference_groups(engine, dev, start_df):
    """Greedy per-group dataflow choice for the reference arm, by measurement (two whole-model steps per trial)."""
    from spira_b200.nn import SparseConv
    convs = {n: m for n, m in engine.model.named_modules() if isinstance(m, SparseConv) and not m.is_trivial}
    seen = {}

    def hook(module, inputs, output, name):
        s = inputs[0]._stride
        eff = tuple(a // b for a, b in zip(s, module.stride)) if module.transposed else tuple(s)
        seen[name] = (eff, module.kernel_size, module.stride)

    handles = [m.register_forward_hook(functools.partial(hook, name=n)) for n, m in convs.items()]
    engine.step(*dev[0])
    for h in handles:
        h.remove()
    groups = sorted(set(seen.values()))
    if not groups:
        return None
    current = {g: start_df for g in groups}

    def apply(cfg):
        for n, m in convs.items():
            m._tunable_config["map_dataflow"] = cfg[seen[n]]
            m._tunable_config["force_os"] = False
        engine.apply_groups(cfg)
        engine.dataflows = [cfg.get((engine.ss[i], engine.ks[i], engine.layer_strides[i]), start_df) for i in range(len(engine.ks))]

    def timed():
        engine.step(*dev[0])
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(2):
            engine.step(*dev[i % len(dev)])
        b.record()
        b.synchronize()
        return a.elapsed_time(b)

    apply(current)
    base = timed()
    for g in groups:
        for alt in (0, 1, 2):
            if alt == current[g]:
                continue
            trial = dict(current)
            trial[g] = alt
            try:
                apply(trial)
                t = timed()
            except RuntimeError:
                ref_mod_reset()
                continue
            if t < 0.98 * base:
                current, base = trial, t
    apply(current)
    # the mask-format kernels (even dataflows) also have a padding threshold per group (reference: helpers.py:468-560
    # sweeps 52 values); a coarse sweep here
    for g in groups:
        if current[g] % 2 != 0 or current[g] == 0:
            continue
        members = [m for n, m in convs.items() if seen[n] == g]
        best_thr = members[0]._tunable_config["threshold"]
        for thr in (0.0, 0.5, 1.0, 2.0, None):
            for m in members:
                m._tunable_config["threshold"] = thr
            try:
                t = timed()
            except RuntimeError:
                ref_mod_reset()
                continue
            if t < 0.98 * base:
                base, best_thr = t, thr
        for m in members:
            m._tunable_config["threshold"] = best_thr
    return current


def ref_mod_reset():
    import spira_b200.nn.functional as F
    try:
        F._C.cuda_reset_error()
    except Exception:
        pass


# ------------------------------------------------------------------------------------------------
# measurement helpers
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows, self.proc = [], None
        self.index = index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([v.strip() for v in line.split(",")])

    def wait_first(self, timeout_s: float = 5.0):
        """Blocks until nvidia-smi has delivered its first sample (it needs a few hundred ms to come up)."""
        t_end = time.time() + timeout_s
        while self.proc is not None and not self.rows and time.time() < t_end:
            time.sleep(0.01)
        self.rows.clear()          # (that sample was taken on an idle device)

    def n_samples(self) -> int:
        return len(self.rows)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except Exception:
                continue
            for n, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm),
                "window": "timed loops, then the same steps until three samples (one per 100 ms) were taken under load"}


def flush_l2(buf):
    buf.add_(1)     # read + write of a buffer twice the size of L2


def timed_loop(step_fn, n_steps, warmup, l2buf, dist_ctx, drain_fn=None):
    import gc
    # serving hygiene, both arms alike: the long-lived objects (model, tapes, scenes) leave the collector's view, so that
    # a full collection cannot land in the middle of a timed step (it costs tens of milliseconds with torch loaded).
    # Done before the warm-up, so that the timed steps follow the warm-up steps directly and start on a busy device
    torch.cuda.synchronize()
    gc.collect()
    gc.freeze()
    for i in range(warmup):
        step_fn(i)
    torch.cuda.synchronize()
    if dist_ctx:
        torch.distributed.barrier()
    evs = []
    wall0 = time.perf_counter()
    enqueue = 0.0
    for i in range(n_steps):
        flush_l2(l2buf)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        c0 = time.perf_counter()
        step_fn(warmup + i)
        if drain_fn is not None and i == n_steps - 1:
            drain_fn()          # work a step left on another stream ends inside the timed region of the last step
        enqueue += time.perf_counter() - c0
        b.record()
        evs.append((a, b))
    torch.cuda.synchronize()
    wall = (time.perf_counter() - wall0, enqueue)
    if dist_ctx:
        torch.distributed.barrier()
    from spira_b200 import sharding
    gc.unfreeze()
    per_step = [a.elapsed_time(b) for a, b in evs]
    dev_ = torch.device("cuda")
    return {"median_ms": sharding.max_over_ranks(statistics.median(per_step), dev_),
            "rank_median_ms": [round(v, 4) for v in sharding.all_ranks(statistics.median(per_step), dev_)],
            "rank_enqueue_ms": [round(v, 4) for v in sharding.all_ranks(enqueue * 1e3 / n_steps, dev_)],
            "mean_ms": sharding.max_over_ranks(sum(per_step) / len(per_step), dev_),
            "steps": per_step, "enqueue_ms": wall[1] * 1e3 / n_steps, "wall_s": wall[0]}


def profile_kernels(engine, scene):
    """One extra, untimed step with CUDA events around every call into the native library."""
    from spira_b200 import _lib
    records = []

    def hook(name, args, run):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if "_conv_" in name:
            # a convolution call is idempotent: two untimed runs put the GPU behind the host, so that the events around
            # the third bracket the kernel and not the Python call (a small layer's kernel is shorter than that)
            run()
            run()
        a.record()
        run()
        b.record()
        records.append((name, args, a, b))

    conv_meta = []

    def fwd_hook(module, inputs, output):
        if module.is_trivial:
            return
        x = inputs[0]
        conv_meta.append(dict(cin=module.in_channels, cout=module.out_channels, K=int(np.prod(module.kernel_size)),
                              S=x._features.shape[0], T=output._features.shape[0], transposed=module.transposed,
                              in_stride=x._stride, out_stride=output._stride, ksize=module.kernel_size))

    from spira_b200.nn import SparseConv
    handles = [m.register_forward_hook(fwd_hook) for m in engine.model.modules() if isinstance(m, SparseConv)]
    _lib.profile_hook = hook
    compiled, engine.compiled = engine.compiled, None      # module hooks only fire on the eager path
    try:
        engine.step(*scene)
        torch.cuda.synchronize()
    finally:
        engine.compiled = compiled
        _lib.profile_hook = None
        for h in handles:
            h.remove()
    # nnz of every layer's map from the search's hit counters
    for meta in conv_meta:
        s, t = meta["in_stride"], meta["out_stride"]
        key = (t, s, meta["ksize"]) if meta["transposed"] else (s, t, meta["ksize"])
        entry = engine.cache._kernel_maps_cache.get(key)
        sb = getattr(entry[3], "_sb", None) if entry is not None else None
        from spira_b200.nn.functional import _C as _native
        counts = _native.map_counts(entry[3]) if (sb is not None and hasattr(_native, "map_counts")) else (sb or {}).get("counts")
        meta["nnz"] = int(counts.sum().item()) if counts is not None else None
    out = {}
    conv_calls = [(n, args, a.elapsed_time(b)) for n, args, a, b in records if n in ("spira_b200_conv_os", "spira_b200_conv_os_grouped", "spira_b200_conv_ws", "spira_b200_conv_ws_fused")]
    for n, args, a, b in records:
        d = out.setdefault(n, dict(calls=0, ms=0.0))
        d["calls"] += 1
        d["ms"] += a.elapsed_time(b)
    layers = []
    for meta, (n, args, ms) in zip(conv_meta, conv_calls):
        if meta["nnz"] is None:
            continue
        flops = 2.0 * meta["nnz"] * meta["cin"] * meta["cout"]
        map_bytes = meta["K"] * meta["T"] * 4 if "conv_os" in n else meta["nnz"] * 8
        byts = meta["S"] * meta["cin"] * 2 + meta["K"] * meta["cin"] * meta["cout"] * 2 + meta["T"] * meta["cout"] * 2 + map_bytes
        layers.append(dict(meta, kernel=n, ms=ms, flops=flops, bytes=byts))
    return out, layers


def kernel_source_sha() -> str:
    """Hash of the CUDA sources of the library, comments and white space excluded: a captured DRAM-traffic figure is only
    valid for the code it was captured from."""
    import hashlib
    import re
    h = hashlib.sha256()
    for f in sorted((ROOT / "spira_b200" / "csrc").glob("*.cu*")):
        text = f.read_text()
        text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)       # block comments
        text = re.sub(r"//[^\n]*", " ", text)                     # line comments (no string literal of the sources holds "//")
        h.update(f.name.encode())
        h.update(" ".join(text.split()).encode())
    return h.hexdigest()[:16]


def captured_traffic(kernel: str, workload: str):
    """DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of ``kernel`` on ``workload`` from the ncu
    capture recorded in ``profiles/dram_traffic.json``, or None when there is no capture of the CURRENT kernel sources."""
    p = ROOT / "profiles" / "dram_traffic.json"
    if not p.exists():
        return None
    try:
        table = json.loads(p.read_text())
    except Exception:
        return None
    sha = kernel_source_sha()
    for e in table.get("captures", []):
        if e.get("kernel") == kernel and e.get("workload") == workload and e.get("source_sha") == sha:
            return int(e["dram_bytes_per_launch"])
    return None


def roofline_of(layers, pk, pk_kind, peak_key):
    """achieved / peak of a set of layers from their live CUDA-event times: FLOPs against the tensor peak or algorithmic
    bytes against the HBM peak, whichever ideal time is larger."""
    t_ms = sum(l["ms"] for l in layers)
    flops = sum(l["flops"] for l in layers)
    byts = sum(l["bytes"] for l in layers)
    ideal_tensor_ms = flops / (pk[peak_key] * 1e12) * 1e3
    ideal_hbm_ms = byts / (pk["hbm_gbs"] * 1e9) * 1e3
    common = {"peak_source": f"of {pk_kind}", "launches": len(layers), "kernel_ms": round(t_ms, 4),
              "algorithmic_flops": int(flops), "algorithmic_bytes": int(byts),
              "tflops": round(flops / (t_ms * 1e-3) / 1e12, 2), "gbs": round(byts / (t_ms * 1e-3) / 1e9, 1)}
    if ideal_hbm_ms >= ideal_tensor_ms:
        ach = byts / (t_ms * 1e-3) / 1e9
        return dict({"bound": "hbm", "achieved": round(ach, 1), "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": round(ach / pk["hbm_gbs"], 4)}, **common)
    ach = flops / (t_ms * 1e-3) / 1e12
    return dict({"bound": "tensor", "achieved": round(ach, 2), "peak": pk[peak_key], "unit": "TFLOP/s", "frac": round(ach / pk[peak_key], 4)}, **common)


def roofline_from_layers(layers, pk, pk_kind, workload_label):
    """Roofline of the DOMINANT kernel of a step (largest share of the measured convolution time) with its own achieved /
    peak; ``conv_class`` carries the aggregate over all sparse-convolution launches and ``per_kernel`` the shares."""
    if not layers:
        return None
    from spira_b200 import _lib
    lib = _lib.load()
    by_kernel = {}
    for l in layers:
        ws = 0 if "conv_os" in l["kernel"] else 1
        kid = lib.spira_b200_conv_kernel_choice(ws, l["K"], l["cin"], l["cout"], l["T"])
        by_kernel.setdefault(_lib.KERNEL_NAMES.get(kid, "unknown"), []).append(l)
    total_ms = sum(l["ms"] for l in layers)
    name, group = max(by_kernel.items(), key=lambda kv: sum(l["ms"] for l in kv[1]))
    # the kernels run inside a long step: the sustained figure is the denominator
    roof = roofline_of(group, pk, pk_kind, "bf16_tflops_sustained")
    roof["kernel"] = name
    roof["share_of_conv_time"] = round(sum(l["ms"] for l in group) / total_ms, 3)
    traffic = captured_traffic(name, workload_label)
    roof["traffic"] = traffic
    roof["traffic_source"] = None if traffic is None else "profiles/dram_traffic.json (ncu capture of the current kernel sources, mean per launch)"
    roof["per_kernel"] = {k: {"launches": len(v), "ms": round(sum(l["ms"] for l in v), 4),
                              "frac": roofline_of(v, pk, pk_kind, "bf16_tflops_sustained")["frac"]} for k, v in by_kernel.items()}
    roof["conv_class"] = roofline_of(layers, pk, pk_kind, "bf16_tflops_sustained")
    roof["kernel_ms_per_step"] = round(total_ms, 4)
    return roof


# ------------------------------------------------------------------------------------------------
# CPU baseline: the oracle port on the host cores
# ------------------------------------------------------------------------------------------------
def cpu_scene_pass(coords_np, layers, budget_s=25.0):
    """Sort + all kernel maps (numpy) + every sparse-convolution layer as torch-CPU gather-GEMM-scatter.
    Stops adding layers when the time budget is spent and scales by the share of FLOPs done."""
    sys.path.insert(0, str(ROOT / "oracle"))
    import spira_oracle as O
    t0 = time.perf_counter()
    keys, _ = O.flat_sort(coords_np)
    level_keys = {(1, 1, 1): keys}
    dense = {}
    done_flops, total_flops = 0.0, sum(l["flops"] for l in layers)
    n_done = 0
    for l in layers:
        s, t = (l["out_stride"], l["in_stride"]) if l["transposed"] else (l["in_stride"], l["out_stride"])
        for st in (s, t):
            if st not in level_keys:
                level_keys[st] = O.downsample(keys, st)
        key = (s, t, l["ksize"])
        if key not in dense:
            dense[key] = O.kernel_map(level_keys[s], level_keys[t], l["ksize"], s, "ws")
        d = dense[key]
        n_in = len(level_keys[t]) if l["transposed"] else len(level_keys[s])
        n_out = len(level_keys[s]) if l["transposed"] else len(level_keys[t])
        feats = torch.zeros(n_in, l["cin"], dtype=torch.float16)
        w = torch.zeros(l["K"], l["cin"], l["cout"], dtype=torch.float16)
        if l["transposed"]:
            O.conv_ws_transposed(feats, w, d, n_out)
        else:
            O.conv_ws(feats, w, d, n_out)
        done_flops += l["flops"]
        n_done += 1
        if time.perf_counter() - t0 > budget_s:
            break
    elapsed = time.perf_counter() - t0
    share = done_flops / total_flops if total_flops else 1.0
    return elapsed / max(share, 1e-9), elapsed, n_done, share


# ------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)     # (scenes of ~2 ms: 32 steps keep one slow step from moving the mean)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-kernels"])
    ap.add_argument("--no-batched", action="store_true", help="skip the B-scenes-per-launch throughput reported as batched")
    ap.add_argument("--no-batch16", action="store_true", help="skip the 16-scene sharded SECOND-style batch reported as c4_batch16")
    ap.add_argument("--workload", default="minkunet", choices=["minkunet", "indoor", "second", "layer", "kmap"])
    ap.add_argument("--no-group", action="store_true", help="output-stationary maps keep their target order (no grouping by neighbour pattern)")
    ap.add_argument("--no-defer", action="store_true", help="add_all_kernel_maps completes all maps before it returns")
    ap.add_argument("--n256-min-targets", type=int, default=-1, help="layers with fewer targets use 128-target tiles (-1 = library default)")
    ap.add_argument("--no-n256", action="store_true", help="output-stationary layers always use the targets-as-M kernel")
    ap.add_argument("--gather", default="default", choices=["default", "tma", "cpasync"], help="row-gather engine of the tensor-core kernels")
    ap.add_argument("--cin", type=int, default=64)
    ap.add_argument("--cout", type=int, default=64)
    ap.add_argument("--ksize", type=int, default=3, choices=[3, 1], help="layer workload: 3 = submanifold 3^3 layer, 1 = 1x1x1 layer (no map)")
    ap.add_argument("--scene", default="c0", choices=["c0", "lidar"], help="layer workload: 50k-voxel plane/sphere scene or a LiDAR scene")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--dataflow", default="auto", choices=["auto", "0", "1"], help="auto = per-group selector (tune); 0/1 = uniform")
    ap.add_argument("--no-compile", action="store_true", help="run the eager module path instead of the recorded tape (ours arm)")
    ap.add_argument("--tape", default="auto", choices=["auto", "native", "replay"],
                    help="forward replay of the ours arm: the library's tape executor, the Python replay, or whichever runs whole steps faster on this box")
    ap.add_argument("--no-native-tape", action="store_true", help="replay the recorded tape operator by operator from Python instead of one spira_b200_run_tape call per scene (ours arm)")
    ap.add_argument("--no-pdl", action="store_true", help="launch every kernel the ordinary way (no programmatic dependent launch)")
    ap.add_argument("--no-identity-tma", action="store_true", help="1x1x1 layers of the native tape run on the output-stationary kernel through the identity map instead of the dense TMA kernel")
    ap.add_argument("--no-fuse", action="store_true", help="keep BatchNorm / ReLU / residual adds as separate passes (ours arm)")
    ap.add_argument("--dump-layers", default=None, help="write the per-layer timing table of the profiled step to this JSON file")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dist_ctx = world > 1
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if dist_ctx:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.distributed.init_process_group("nccl", device_id=device)
    n_gpus = world

    pk, pk_kind = peaks()
    if args.impl == "ours" and args.no_group:
        from spira_b200.nn.functional import _C as native_
        native_.GROUP_OS = False
    if args.impl == "ours" and args.no_defer:
        from spira_b200.nn.functional import _C as native_
        native_.DEFER_MAPS = False
    if args.impl == "ours" and args.n256_min_targets >= 0:
        from spira_b200.nn.functional import _C as native_
        native_.set_option("os_n256_min_targets", args.n256_min_targets)
    if args.impl == "ours" and args.no_n256:
        from spira_b200.nn.functional import _C as native_
        native_.set_option("os_n256", 0)
    if args.impl == "ours" and args.gather != "default":
        from spira_b200 import build
        build.build()
        from spira_b200.nn.functional import _C as native
        native.set_option("gather_tma", 1 if args.gather == "tma" else 0)
    if args.workload in ("layer", "kmap"):
        if args.impl != "ours":
            if rank == 0:
                if reference_tools().available():
                    line = {"layer": run_layer_reference, "kmap": run_kmap_reference}[args.workload](args, device, pk, pk_kind)
                    line.update(n_gpus=n_gpus, impl="reference")
                else:
                    line = {"impl": "reference", "unavailable": "the reference's native module is not built (oracle/_ref/_C.so missing)"}
                print(json.dumps(line))
            if dist_ctx:
                torch.distributed.destroy_process_group()
            return
        from spira_b200 import build, _lib
        build.build()
        _lib.load()
        if args.no_identity_tma:
            _lib.call("spira_b200_set_option", b"identity_tma", 0)
        line = {"layer": run_layer, "kmap": run_kmap}[args.workload](args, device, pk, pk_kind)
        line["n_gpus"] = n_gpus
        if rank == 0:
            print(json.dumps(line))
        if dist_ctx:
            torch.distributed.destroy_process_group()
        return
    wl = make_workload(args.workload)
    if args.impl != "ours" and not reference_tools().available():
        if rank == 0:
            run_reference_port(args, wl, n_gpus)
        if dist_ctx:
            torch.distributed.destroy_process_group()
        return
    if args.impl == "ours":
        from spira_b200 import build, _lib
        build.build()
        _lib.load()
        if args.no_pdl:
            _lib.call("spira_b200_set_option", b"pdl", 0)
        if args.no_identity_tma:
            _lib.call("spira_b200_set_option", b"identity_tma", 0)

    host, dev = load_scenes(wl, [s + 100 * rank for s in wl["seeds"]], device)
    n_vox = [len(h[0]) for h in host]
    engine, chosen_note = make_engine(args, args.workload, wl, device, dev, rank)
    l2buf = torch.zeros(256 * 1024 * 1024 // 4, dtype=torch.float32, device=device)
    from spira_b200 import _lib

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        sampler.wait_first()
    m = measure(engine, host, dev, args, l2buf, dist_ctx, device)
    if rank == 0:
        # the timed loops are a few tens of milliseconds: the same steps keep running until the sampler (one sample
        # per 100 ms) has seen the device under this load at least three times
        t_end, i = time.time() + 3.0, 0
        while sampler.n_samples() < 3 and time.time() < t_end:
            engine.step(*dev[i % len(dev)])
            i += 1
        torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None

    line = {
        "metric": "MinkUNet scene throughput (scene latency = ms_per_step)" if args.workload == "minkunet" else f"{args.workload} scene throughput",
        "value": round(n_gpus * 1e3 / m["median_ms"], 3), "unit": "scenes/s", "n_gpus": n_gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(m["median_ms"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16 (fp32 accumulate); u32 packed keys", "data": "synthetic",
        "config": {"workload": wl["label"], "voxels_per_scene": n_vox, "scenes_per_rank": len(dev),
                   "timed_region": "order() + add_all_kernel_maps() + model forward, per scene",
                   "statistic": "median of the K per-step device times, slowest rank (the mean is in mean_ms_per_step); both arms alike",
                   "l2": "256 MiB buffer rewritten between timed steps",
                   "setup": "tune / compile, then every scene once untimed (allocator priming), then the W warm-up steps",
                   "dataflows": chosen_note, "sharding": "independent scenes per GPU, no collective",
                   "fused_epilogue": bool(args.impl == "ours" and not args.no_fuse),
                   "recorded_tape": bool(args.impl == "ours" and not args.no_compile),
                   "native_tape": bool(getattr(getattr(engine, "compiled", None), "use_native", False)),
                   "tape_choice_ms": getattr(engine, "tape_choice", None)},
        "e2e": {"value": round(n_gpus * 1e3 / m["e2e_median_ms"], 3), "unit": "scenes/s", "ms_per_step": round(m["e2e_median_ms"], 4),
                "mean_ms_per_step": round(m["e2e_mean_ms"], 4), "h2d_bytes_per_step": m["h2d"], "d2h_bytes_per_step": m["d2h"]},
        "mean_ms_per_step": round(m["mean_ms"], 4),
        "gpu_launches": m["launches"] if args.impl == "ours" else 0,
        "host_enqueue_ms_per_step": round(m["enqueue_ms"], 4),
        "ms_per_step_per_rank": m["rank_median_ms"], "host_enqueue_ms_per_rank": m["rank_enqueue_ms"],
        "step_ms_min_median_max": [round(min(m["steps"]), 4), round(statistics.median(m["steps"]), 4), round(max(m["steps"]), 4)],
        "step_ms_first": [round(v, 4) for v in m["steps"][:8]],
        "clocks": clocks,
    }
    if args.impl != "ours":
        line["impl"] = args.impl
        line["cpu_baseline"] = {"value": line["value"], "unit": "scenes/s", "cores": 0, "kind": "reference",
                                "sample": "the reference's own CUDA kernels (its unmodified sources built for sm_100) on the GPU: it has no CPU path"}
    else:
        # roofline of the dominant kernel + secondary metrics, measured live with CUDA events
        per_call, layers = profile_kernels(engine, dev[0])
        line["roofline"] = roofline_from_layers(layers, pk, pk_kind, wl["label"])
        if args.dump_layers and rank == 0:
            Path(args.dump_layers).parent.mkdir(parents=True, exist_ok=True)
            Path(args.dump_layers).write_text(json.dumps([{k: (list(v) if isinstance(v, tuple) else v) for k, v in l.items()} for l in layers], indent=0))
        km = per_call.get("spira_b200_kmap_search")
        if km:
            maps_bytes = 0
            for key, entry in engine.cache._kernel_maps_cache.items():
                S, T = entry[1], entry[2]
                K = int(np.prod(key[2]))
                maps_bytes += (S + T) * 4 + K * ((T + 127) // 128 * 128) * 4
            line["kernel_map_build"] = {"search_kernel_ms": round(km["ms"], 4), "maps": len(engine.cache._kernel_maps_cache),
                                        "algorithmic_bytes": maps_bytes, "gbs": round(maps_bytes / (km["ms"] * 1e-3) / 1e9, 1),
                                        "frac_of_hbm_peak": round(maps_bytes / (km["ms"] * 1e-3) / 1e9 / pk["hbm_gbs"], 4)}
        line["native_calls_ms"] = {k.replace("spira_b200_", ""): round(v["ms"], 4) for k, v in per_call.items()}
        if rank == 0 and n_gpus == 1 and not args.no_cpu_baseline:
            # bounded sample: whole scenes (the layer shapes of scene 0 on the coordinates of every scene in turn) until
            # about ten seconds of CPU work are done
            scenes_done, cpu_s, n_done, share = 0.0, 0.0, 0, 1.0
            while cpu_s < 10.0 and scenes_done < 64:
                est, spent, n_done, share = cpu_scene_pass(host[int(scenes_done) % len(host)][0].numpy(), layers)
                cpu_s += spent
                scenes_done += share
                if share < 1.0:
                    break
            line["cpu_baseline"] = {"value": round(scenes_done / cpu_s, 5), "unit": "scenes/s", "cores": torch.get_num_threads(), "kind": "port",
                                    "sample": f"oracle port: sort + kernel maps (numpy) + {n_done}/{len(layers)} conv layers "
                                              f"(torch-CPU gather-GEMM-scatter) per scene, {scenes_done:.2f} scenes in {cpu_s:.1f} s; BN/ReLU omitted"}
    del engine
    if not args.no_batched:
        line["batched"] = run_batched(args, args.workload, wl, device, rank, n_gpus, dev, l2buf, dist_ctx)
    if not args.no_batch16:
        line["c4_batch16"] = run_batch16(args, device, rank, world, dist_ctx, l2buf)
    if rank == 0:
        print(json.dumps(line))
    if dist_ctx:
        torch.distributed.destroy_process_group()


def load_scenes(wl, seeds, device):
    """Scenes resident on the device AND in pinned host memory (for the end-to-end number).  A scene whose key tensor
    would end exactly on an allocator block boundary loses its last voxel, both arms alike: the reference's search reads
    one key past its source array (csrc/spira/cuda/kernels/query_sorted.cuh:42,48)."""
    from spira_b200 import scenes as sc
    host, dev = [], []
    for s in seeds:
        c = wl["scene"](s)
        if len(c) % 64 == 0:
            c = c[:-1]
        f = sc.features(len(c), wl["channels"], s, wl["feat_kind"])
        hc, hf = torch.from_numpy(c).pin_memory(), torch.from_numpy(f).pin_memory()
        host.append((hc, hf))
        dev.append((hc.to(device), hf.to(device)))
    return host, dev


def make_engine(args, workload_name, wl, device, dev, rank):
    """The engine of the chosen arm with its dataflows selected: (engine, note for the JSON line)."""
    if args.impl == "reference":
        engine = StockReferenceEngine(workload_name, wl, device)
        engine.tune(dev, os.path.join(tempfile.gettempdir(), f"spira_ref_tune_{workload_name}_r{rank}"))
        return engine, engine.tune_note
    if args.impl == "reference-kernels":
        R = reference_tools()
        ref_mod = R.ReferenceModule()
        R.install_native(ref_mod)
    engine = Engine(wl, device)
    if args.impl == "ours" and not args.no_fuse:
        import spira_b200 as sp_
        sp_.fuse(engine.model)
    chosen_note = None
    if args.impl == "ours" and args.dataflow != "auto":
        engine.set_uniform_dataflow(int(args.dataflow))
        chosen_note = {"uniform_map_dataflow": int(args.dataflow)}
    elif args.impl == "ours":
        import spira_b200 as sp

        def loader():
            for c, f in dev:
                yield sp.SparseTensor(c, f).order()
        _, chosen = sp.tune(engine.model, loader(), engine.cache, n_samples=2, save_dir=os.path.join(tempfile.gettempdir(), "spira_b200_tune"),
                            tune_tag=f"{workload_name}_r{rank}", force_retune=True, return_dataflows=True, verify=False)
        engine.apply_groups(chosen)
        chosen_note = {str(k): v for k, v in chosen.items()}
    else:
        # the reference's kernels behind this repository's glue: the best UNIFORM dataflow of 0/1/2 first
        best = None
        for df in (0, 1, 2):
            try:
                engine.set_uniform_dataflow(df)
                for i in range(2):
                    engine.step(*dev[i % len(dev)])
                torch.cuda.synchronize()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                for i in range(2):
                    engine.step(*dev[i % len(dev)])
                b.record(); b.synchronize()
                t = a.elapsed_time(b)
            except RuntimeError as e:
                ref_mod.cuda_reset_error()
                continue
            if best is None or t < best[1]:
                best = (df, t)
        engine.set_uniform_dataflow(best[0])
        chosen_note = {"uniform_map_dataflow": best[0]}
        # then per layer group: every group tries the other dataflows on whole-model runs and keeps what is faster
        try:
            tuned = tune_reference_groups(engine, dev, best[0])
            if tuned is not None:
                chosen_note = {"per_group": {str(k): v for k, v in tuned.items()}, "start": best[0]}
        except RuntimeError:
            ref_mod.cuda_reset_error()
            engine.set_uniform_dataflow(best[0])
    if args.impl == "ours" and not args.no_compile:
        if args.no_native_tape:
            import spira_b200.compile as spc
            spc.NATIVE_TAPE = False
        engine.compile(*dev[0])
        engine.tape_choice = None
        if engine.compiled.native is not None and args.tape == "auto":
            # part of the setup, like the dataflow selection: whole steps timed with the forward replayed from Python and
            # through the library's tape executor; the faster one stays (which one that is depends on the host)
            took = {}
            for mode in (True, False, True, False):
                engine.compiled.use_native = mode
                for i in range(3):
                    engine.step(*dev[i % len(dev)])
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                for i in range(12):
                    engine.step(*dev[i % len(dev)])
                torch.cuda.synchronize()
                took.setdefault(mode, []).append((time.perf_counter() - t0) / 12 * 1e3)
            # the library's executor stays unless the Python replay is clearly faster: it runs the whole step on the
            # engine's own kernels (no concatenation copies, no library GEMMs) and keeps the host at a fraction of the work
            engine.compiled.use_native = min(took[True]) <= 1.03 * min(took[False])
            engine.tape_choice = {"native_ms": round(min(took[True]), 4), "replay_ms": round(min(took[False]), 4),
                                  "rule": "native unless the Python replay is more than 3 % faster"}
        elif engine.compiled.native is not None:
            engine.compiled.use_native = args.tape == "native"
    return engine, chosen_note


def measure(engine, host, dev, args, l2buf, dist_ctx, device):
    """The two timed loops of an arm: scenes resident in HBM, then end to end through pinned host buffers."""
    from spira_b200 import _lib

    def step_resident(i):
        c, f = dev[i % len(dev)]
        return engine.step(c, f)

    stage_c = [torch.empty_like(d[0]) for d in dev]
    stage_f = [torch.empty_like(d[1]) for d in dev]
    out_host = {}
    d2h_bytes = [0]

    # End to end, both arms alike: the inputs of a step come from pinned host memory (H2D on the compute stream, inside
    # the step) and its logits go back to pinned host memory.  The D2H copy runs on a copy stream behind an event, so that
    # the next step's kernels do not queue behind it; the timed region ends after the last copy has landed (the loop's
    # final synchronize).  Every copy is accounted for: a step's end marker waits for the copy of the step before it, and
    # the last step's marker waits for its own.
    copy_stream = torch.cuda.Stream(device=device)
    pending_out = {}

    h2d = {}        # step number -> event: its inputs have been copied to the staging buffers (issued one step ahead)

    def upload(i, stream_ctx):
        j = i % len(dev)
        with stream_ctx:
            stage_c[j].copy_(host[j][0], non_blocking=True)
            stage_f[j].copy_(host[j][1], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
        h2d[i] = ev

    def step_e2e(i):
        j = i % len(dev)
        main = torch.cuda.current_stream()
        if i not in h2d:                     # first step of a loop: nothing was uploaded ahead
            upload(i, contextlib.nullcontext())
        main.wait_event(h2d.pop(i))
        # the next step's inputs travel while this step computes (its staging buffers belong to another scene)
        if len(dev) > 1:
            h2d.clear()
            mark = torch.cuda.Event()
            mark.record(main)                # everything enqueued so far (the steps that last read those buffers) comes first
            copy_stream.wait_event(mark)
            upload(i + 1, torch.cuda.stream(copy_stream))
        y = engine.step(stage_c[j], stage_f[j])
        if j not in out_host:
            out_host[j] = torch.empty(y.shape, dtype=y.dtype).pin_memory()
        main = torch.cuda.current_stream()
        if "done" in pending_out:
            main.wait_event(pending_out["done"])     # the previous step's copy ends inside this step's timed region
        ready = torch.cuda.Event()
        ready.record()
        copy_stream.wait_event(ready)
        with torch.cuda.stream(copy_stream):
            out_host[j].copy_(y, non_blocking=True)
            done = torch.cuda.Event()
            done.record()
        y.record_stream(copy_stream)
        pending_out["done"] = done
        d2h_bytes[0] = y.numel() * y.element_size()
        return y

    def drain_e2e():
        torch.cuda.current_stream().wait_stream(copy_stream)

    # set-up, both arms alike: every scene of the rank runs once through both entry points, so that the caching
    # allocator has seen every tensor size before the W warm-up steps (a first-time size costs a cudaMalloc)
    for i in range(len(dev)):
        step_resident(i)
        step_e2e(i)
    torch.cuda.synchronize()
    launches0 = _lib.launch_count
    res = timed_loop(step_resident, args.steps, args.warmup, l2buf, dist_ctx)
    launches = _lib.launch_count - launches0
    e2e = timed_loop(step_e2e, args.steps, args.warmup, l2buf, dist_ctx, drain_e2e)
    return {"median_ms": res["median_ms"], "mean_ms": res["mean_ms"], "steps": res["steps"], "enqueue_ms": res["enqueue_ms"],
            "rank_median_ms": res["rank_median_ms"], "rank_enqueue_ms": res["rank_enqueue_ms"],
            "e2e_median_ms": e2e["median_ms"], "e2e_mean_ms": e2e["mean_ms"], "launches": launches,
            "h2d": int(np.mean([h[0].numel() * 4 + h[1].numel() * 2 for h in host])), "d2h": int(d2h_bytes[0])}


def run_batched(args, workload_name, wl, device, rank, n_gpus, dev, l2buf, dist_ctx):
    """Throughput with the rank's scenes merged into ONE sparse tensor per step (``spira_b200.batch.merge_scenes``: the
    scenes lie side by side, far enough apart never to interact), so that every launch of the step works on all of
    them: value = scenes of all ranks per second, from the median device time of a step.  Both arms alike."""
    from spira_b200 import batch
    coords, feats, pitch, grid = batch.merge_scenes([c for c, _ in dev], [f for _, f in dev])
    if coords.shape[0] % 64 == 0:          # (see load_scenes)
        coords, feats = coords[:-1].contiguous(), feats[:-1].contiguous()
    merged = [(coords, feats)]
    engine, note = make_engine(args, workload_name, wl, device, merged, rank)
    for _ in range(2):
        engine.step(coords, feats)
    torch.cuda.synchronize()
    res = timed_loop(lambda i: engine.step(coords, feats), max(4, args.steps // 2), args.warmup, l2buf, dist_ctx)
    B = len(dev)
    return {"value": round(n_gpus * B * 1e3 / res["median_ms"], 2), "unit": "scenes/s", "scenes_per_step": B,
            "ms_per_step": round(res["median_ms"], 4), "voxels_per_step": int(coords.shape[0]), "grid": list(grid), "pitch": pitch,
            "dataflows": note}


def run_batch16(args, device, rank, world, dist_ctx, l2buf):
    """Sixteen multi-sweep scenes (seeds 10-25) through the SECOND-style backbone, scene i on rank i mod G
    (``spira_b200.sharding.assign_scenes``), no collective on the data path: scenes/s = 16 / the slowest rank's device time
    for its share, after one untimed pass over the same scenes."""
    from spira_b200 import sharding
    wl = make_workload("second")
    mine = sharding.assign_scenes(16, world, rank)
    host, dev = load_scenes(wl, [10 + i for i in mine], device)
    engine, note = make_engine(args, "second", wl, device, dev[:2], rank)
    for c, f in dev:                       # untimed pass: allocator priming and warm-up
        engine.step(c, f)
    torch.cuda.synchronize()
    if dist_ctx:
        torch.distributed.barrier()
    flush_l2(l2buf)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for c, f in dev:
        engine.step(c, f)
    b.record()
    torch.cuda.synchronize()
    if dist_ctx:
        torch.distributed.barrier()
    local_ms = a.elapsed_time(b)
    worst = sharding.max_over_ranks(local_ms, torch.device("cuda"))
    return {"value": round(16 / (worst / 1e3), 2), "unit": "scenes/s", "scenes": 16, "scenes_on_rank0": len(mine),
            "slowest_rank_ms": round(worst, 3), "workload": wl["label"], "voxels_per_scene_rank0": [len(h[0]) for h in host],
            "assignment": "scene i -> rank i mod n_gpus", "dataflows": note}


def _time_calls(fn, steps, warmup, l2buf):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    evs = []
    for _ in range(steps):
        flush_l2(l2buf)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); fn(); b.record()
        evs.append((a, b))
    torch.cuda.synchronize()
    t = [a.elapsed_time(b) for a, b in evs]
    return sum(t) / len(t), min(t)


def run_pointwise_layer(args, device, pk, pk_kind, n, feats, rng):
    """Single 1x1x1 layer c_in -> c_out over the voxels of the scene (no kernel map: row t of the output reads row t of
    the input), with a BatchNorm-style epilogue.  The layer is bound by HBM: it reads n*c_in*2 and writes n*c_out*2 bytes.
    A launch takes ~15 us, less than the Python wrapper needs to prepare one, so a timed step is one pass of prepared
    descriptor calls over SIX input / output sets (together larger than the L2: every launch reads rows that left the
    cache several launches ago); the figures are per launch."""
    import ctypes
    from spira_b200 import _lib
    from spira_b200.nn.functional import _C
    w = torch.from_numpy((rng.normal(size=(1, args.cin, args.cout)) / np.sqrt(args.cin)).astype(np.float16)).to(device)
    scale = torch.from_numpy(rng.uniform(0.5, 1.5, args.cout).astype(np.float32)).to(device)
    shift = torch.from_numpy(rng.normal(size=args.cout).astype(np.float32)).to(device)
    l2buf = torch.zeros(256 * 1024 * 1024 // 4, dtype=torch.float32, device=device)
    packed = _C.packed_weights(w, _C.PACK_OS)
    if packed is None:
        raise RuntimeError(f"a 1x1x1 layer {args.cin} -> {args.cout} is outside the tensor-core kernels")
    ep, keep = _C._epilogue(None, scale, shift, None, False)
    n_sets = 6
    sets = []
    for i in range(n_sets):
        f = feats if i == 0 else feats.clone()
        out = torch.empty((n, args.cout), dtype=torch.float16, device=device)
        d = _lib.ConvDesc(dataflow=0, K=1, c_in=args.cin, c_out=args.cout, c_in_a=args.cin, num_sources=n, num_targets=n,
                          feats=f.data_ptr(), packed=packed.data_ptr(), out=out.data_ptr())
        d.epilogue = ctypes.pointer(ep)
        sets.append((f, out, d))

    def one_pass():
        for _, _, d in sets:
            _C.conv_desc_call(d, device)

    pass_ms, pass_min_ms = _time_calls(one_pass, args.steps, args.warmup, l2buf)
    mean_ms, min_ms = pass_ms / n_sets, pass_min_ms / n_sets
    _C.check_status()
    want = torch.mm(feats, w[0]).float() * scale + shift
    err = (sets[-1][1].float() - want).abs().max().item()
    if not err <= 2e-2 * max(1.0, want.abs().max().item()):
        raise RuntimeError(f"1x1x1 layer: result differs from the matrix product by {err}")
    flops = 2.0 * n * args.cin * args.cout
    byts = n * args.cin * 2 + args.cin * args.cout * 2 + n * args.cout * 2
    ach = byts / (mean_ms * 1e-3) / 1e9
    dense = _C.get_option("identity_tma") == 1 and args.cin % 32 == 0
    kernel = "dense_tc_kernel" if dense else "conv_tc_kernel<OS>"
    workload_label = f"single 1x1x1 layer {args.cin}->{args.cout}, {n} voxels ({args.scene})"
    roof = {"bound": "hbm", "achieved": round(ach, 1), "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": round(ach / pk["hbm_gbs"], 4),
            "traffic": captured_traffic(kernel, workload_label), "kernel": kernel, "peak_source": f"of {pk_kind}",
            "algorithmic_bytes": int(byts), "algorithmic_flops": int(flops),
            "fastest_pass": {"ms_per_launch": round(min_ms, 5), "gbs": round(byts / (min_ms * 1e-3) / 1e9, 1)}}
    return {"metric": "1x1x1 layer GB/s (bytes = n*(c_in + c_out)*2 + weights)", "value": round(ach, 1), "unit": "GB/s",
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(mean_ms, 5), "min_ms": round(min_ms, 5), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16 (fp32 accumulate)", "data": "synthetic",
            "config": {"workload": workload_label, "launches_per_step": n_sets,
                       "l2": "six input/output sets (340 MB at 128->96 over 127 k voxels) visited in turn, and a 256 MiB buffer rewritten between timed steps"},
            "roofline": roof, "gpu_launches": args.steps * n_sets}


def run_layer(args, device, pk, pk_kind):
    """Single-layer workload: one submanifold 3^3 layer, c_in -> c_out, 50,000 voxels in a 512^3 grid (64-bit keys)."""
    from spira_b200 import scenes as sc, _lib
    from spira_b200.nn.functional import _C
    if args.scene == "c0":
        c, double = sc.planes_and_spheres(0), True
    else:
        c, double = sc.lidar_scene(1), False
    n = len(c)
    keys, perm = _C.cuda_flatten_sort(torch.from_numpy(c).to(device), double)
    feats = torch.from_numpy(sc.features(n, args.cin, 0)).to(device)
    rng = np.random.default_rng(0)
    if args.ksize == 1:
        return run_pointwise_layer(args, device, pk, pk_kind, n, feats, rng)
    w = torch.from_numpy((rng.normal(size=(27, args.cin, args.cout)) / np.sqrt(27 * args.cin)).astype(np.float16)).to(device)
    df = 1 if args.dataflow == "1" else 0
    m = _C.cuda_binary_search(keys, keys, (3, 3, 3), (1, 1, 1), df)
    nnz = int(m[2]._sb["counts"].sum().item())
    l2buf = torch.zeros(256 * 1024 * 1024 // 4, dtype=torch.float32, device=device)
    if df == 0:
        fn = lambda: _C.conv_os(n, n, m[2], feats, w)
    else:
        fn = lambda: _C.conv_ws(n, n, feats, w, m[2]._sb["ws"])
    mean_ms, min_ms = _time_calls(fn, args.steps, args.warmup, l2buf)
    _C.check_status()
    map_ms, _ = _time_calls(lambda: _C.cuda_binary_search(keys, keys, (3, 3, 3), (1, 1, 1), df), args.steps, args.warmup, l2buf)
    flops = 2.0 * nnz * args.cin * args.cout
    byts = n * args.cin * 2 + 27 * args.cin * args.cout * 2 + n * args.cout * 2 + (27 * n * 4 if df == 0 else nnz * 8)
    t_tensor, t_hbm = flops / (pk["bf16_tflops"] * 1e12), byts / (pk["hbm_gbs"] * 1e9)
    if t_hbm >= t_tensor:
        ach = byts / (mean_ms * 1e-3) / 1e9
        roof = {"bound": "hbm", "achieved": round(ach, 1), "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": round(ach / pk["hbm_gbs"], 4), "traffic": None}
    else:
        ach = flops / (mean_ms * 1e-3) / 1e12
        roof = {"bound": "tensor", "achieved": round(ach, 2), "peak": pk["bf16_tflops"], "unit": "TFLOP/s", "frac": round(ach / pk["bf16_tflops"], 4), "traffic": None}
    kernel = _lib.KERNEL_NAMES[_lib.load().spira_b200_conv_kernel_choice(df, 27, args.cin, args.cout, n)]
    if df == 0 and _C.grouped_twin(m[2]) is not None and args.cin % 8 == 0:
        # Bytes that cross from L2 into the SMs per launch: gathered rows + one weight chunk per visited (tile, 64-wide
        # reduction chunk) + the map.  This, not HBM, is what the output-stationary kernels move most of.
        stats = _C.grouped_twin(m[2]).stats.cpu().tolist()
        tile_rows = 256 if kernel == "conv_os_n256_kernel" else 128
        visited = stats[1] if tile_rows == 256 else stats[0]              # non-empty (tile, offset) pairs of the grouped map
        xbar = nnz * args.cin * 2 + visited * (args.cin / 64.0) * args.cout * 128 + m[2].numel() * 4
        roof["l2_to_sm"] = {"bytes_per_launch": int(xbar), "achieved_gbs": round(xbar / (min_ms * 1e-3) / 1e9, 1),
                            "note": "gathered rows + weight chunks + map, over the fastest launch"}
    workload_label = f"single submanifold 3^3 layer {args.cin}->{args.cout}, {n} voxels ({args.scene}), dataflow {'WS' if df else 'OS'}"
    roof["traffic"] = captured_traffic(kernel, workload_label)
    roof.update(kernel=kernel, peak_source=f"of {pk_kind}", algorithmic_bytes=int(byts), algorithmic_flops=int(flops))
    return {"metric": "SpC layer TFLOP/s (FLOPs = 2*nnz*c_in*c_out)", "value": round(flops / (mean_ms * 1e-3) / 1e12, 3), "unit": "TFLOP/s",
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(mean_ms, 5), "min_ms": round(min_ms, 5), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16 (fp32 accumulate)", "data": "synthetic",
            "config": {"workload": workload_label,
                       "nnz": nnz, "nnz_per_voxel": round(nnz / n, 2), "l2": "256 MiB buffer rewritten between timed steps"},
            "kernel_map_build_ms": round(map_ms, 5), "roofline": roof, "gpu_launches": args.steps * (2 if df else 1)}


def run_kmap(args, device, pk, pk_kind):
    """Kernel-map workload: kernel maps only, 4 LiDAR-like scenes: 3^3, 5^3, stride-2 down-sampling + transposed reuse."""
    from spira_b200 import scenes as sc
    from spira_b200.nn.functional import _C
    scenes_k = []
    for seed in (1, 2, 3, 4):
        keys, _ = _C.cuda_flatten_sort(torch.from_numpy(sc.lidar_scene(seed)).to(device), False)
        scenes_k.append((keys, _C.cuda_downsample(keys, 2, 2, 2)))
    l2buf = torch.zeros(256 * 1024 * 1024 // 4, dtype=torch.float32, device=device)
    out = {}
    byts_all = 0

    def search_only(keys, tgt, ks, layout):
        return _C.cuda_binary_search(keys, tgt, ks, (1, 1, 1), layout)

    for name, ks, strided, df in (("3x3x3_os", (3, 3, 3), False, 0), ("3x3x3_ws", (3, 3, 3), False, 1), ("5x5x5_os", (5, 5, 5), False, 0),
                                  ("down_3x3x3_os", (3, 3, 3), True, 0), ("down_3x3x3_ws", (3, 3, 3), True, 1)):
        def fn():
            for keys, down in scenes_k:
                search_only(keys, down if strided else keys, ks, df)
        mean_ms, min_ms = _time_calls(fn, args.steps, args.warmup, l2buf)
        K = ks[0] * ks[1] * ks[2]
        byts = sum((k.numel() + (d.numel() if strided else k.numel())) * 4 + K * ((((d.numel() if strided else k.numel()) + 127) // 128) * 128) * 4
                   for k, d in scenes_k)
        out[name] = {"ms_per_scene": round(mean_ms / 4, 5), "min_ms_per_scene": round(min_ms / 4, 5), "algorithmic_bytes_per_scene": byts // 4,
                     "gbs": round(byts / (mean_ms * 1e-3) / 1e9, 1)}
    # the whole config per scene: 3^3 + 5^3 submanifold, 3^3 stride-2 map, inverse for the transposed layer
    def all_maps():
        for keys, down in scenes_k:
            maps = _C.cuda_binary_search_streamed([keys, down], [(3, 3, 3), (3, 3, 3)], [(1, 1, 1), (1, 1, 1)], [0, 0])
            _C.cuda_binary_search(keys, keys, (5, 5, 5), (1, 1, 1), 0)
            _C.cuda_convert_transposed_os(maps[1][2], keys.numel())
    mean_ms, min_ms = _time_calls(all_maps, args.steps, args.warmup, l2buf)
    # roofline of the search kernel alone on the 5^3 map of scene 0 (the largest single launch)
    from spira_b200 import _lib
    keys = scenes_k[0][0]
    n = keys.numel()
    Tal = (n + 127) // 128 * 128
    dense = torch.empty((Tal, 125), dtype=torch.int32, device=device)
    import ctypes as C
    d = (_lib.KmapDesc * 1)()
    d[0].sources = d[0].targets = keys.data_ptr()
    d[0].num_sources = d[0].num_targets = n
    d[0].kernel_size[:] = (5, 5, 5)
    d[0].source_stride[:] = (1, 1, 1)
    d[0].layout = 0
    d[0].map = dense.data_ptr()
    d[0].tile_counts = None
    stream = C.c_void_p(torch.cuda.current_stream(device).cuda_stream)
    k_ms, k_min = _time_calls(lambda: _lib.call("spira_b200_kmap_search", d, 1, 4, stream), max(args.steps, 10), args.warmup, l2buf)
    byts5 = 2 * n * 4 + 125 * Tal * 4
    ach = byts5 / (k_ms * 1e-3) / 1e9
    return {"metric": "kernel-map build (3^3 + 5^3 + stride-2 + transposed inverse)", "value": round(4 / (mean_ms * 1e-3), 2), "unit": "scenes/s",
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(mean_ms, 5), "ms_per_scene": round(mean_ms / 4, 5),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u32", "data": "synthetic",
            "config": {"workload": "kernel maps only, 4 LiDAR-like scenes ~125k voxels each", "voxels": [k.numel() for k, _ in scenes_k],
                       "l2": "256 MiB buffer rewritten between timed steps"},
            "maps": out,
            "roofline": {"bound": "hbm", "achieved": round(ach, 1), "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": round(ach / pk["hbm_gbs"], 4),
                         "traffic": captured_traffic("kmap_search_kernel<u32>", "kernel maps only, 4 LiDAR-like scenes ~125k voxels each"),
                         "kernel": "kmap_search_kernel<u32>, 5^3 map of scene 0", "peak_source": f"of {pk_kind}",
                         "algorithmic_bytes": byts5, "kernel_ms": round(k_ms, 5), "kernel_min_ms": round(k_min, 5)},
            "gpu_launches": args.steps * 4 * 4}


def _padded(t):
    """Same values with slack behind them: the reference's search reads ``sources[num_sources]``
    (csrc/spira/cuda/kernels/query_sorted.cuh:42,48)."""
    big = torch.zeros(t.shape[0] + 64, dtype=t.dtype, device=t.device)
    big[:t.shape[0]] = t
    return big[:t.shape[0]]


def run_layer_reference(args, device, pk, pk_kind):
    """The single-layer workload on the reference's own kernels: every dataflow's forward call on the map the reference
    builds for it (scripts/layerwise_experiment.py times the same calls through its module)."""
    from spira_b200 import scenes as sc
    ref = reference_tools().load_native()
    if args.scene == "c0":
        c, double = sc.planes_and_spheres(0), True
    else:
        c, double = sc.lidar_scene(1), False
    n = len(c)
    keys, _ = ref.cuda_flatten_sort(torch.from_numpy(c).to(device), double)
    keys = _padded(keys)
    feats = torch.from_numpy(sc.features(n, args.cin, 0)).to(device)
    rng = np.random.default_rng(0)
    if args.ksize == 1:
        # the reference's 1x1x1 layer is torch.mm (spira/nn/conv.py:312-316) followed by its BatchNorm module as a pass of its own
        w1 = torch.from_numpy((rng.normal(size=(1, args.cin, args.cout)) / np.sqrt(args.cin)).astype(np.float16)).to(device)
        gamma = torch.from_numpy(rng.uniform(0.5, 1.5, args.cout).astype(np.float16)).to(device)
        beta = torch.from_numpy(rng.normal(size=args.cout).astype(np.float16)).to(device)
        mean, var = torch.zeros(args.cout, dtype=torch.float16, device=device), torch.ones(args.cout, dtype=torch.float16, device=device)
        l2buf = torch.zeros(256 * 1024 * 1024 // 4, dtype=torch.float32, device=device)
        inputs = [feats] + [feats.clone() for _ in range(5)]      # six sets visited in turn, as in this engine's leg
        keep = [None] * len(inputs)

        def one_pass():
            for i, f in enumerate(inputs):
                keep[i] = torch.nn.functional.batch_norm(torch.mm(f, w1[0]), mean, var, gamma, beta, False, 0.0, 1e-5)

        pass_ms, pass_min_ms = _time_calls(one_pass, args.steps, args.warmup, l2buf)
        mean_ms, min_ms = pass_ms / len(inputs), pass_min_ms / len(inputs)
        byts = n * args.cin * 2 + args.cin * args.cout * 2 + n * args.cout * 2
        v = round(byts / (mean_ms * 1e-3) / 1e9, 1)
        return {"metric": "1x1x1 layer GB/s (bytes = n*(c_in + c_out)*2 + weights)", "value": v, "unit": "GB/s", "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": round(mean_ms, 5), "min_ms": round(min_ms, 5), "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "f16", "data": "synthetic",
                "config": {"workload": f"single 1x1x1 layer {args.cin}->{args.cout}, {n} voxels ({args.scene}), torch.mm + BatchNorm pass as in the reference",
                           "l2": "256 MiB buffer rewritten between timed steps"},
                "cpu_baseline": {"value": v, "unit": "GB/s", "cores": 0, "kind": "reference",
                                 "sample": "the reference's own path on the GPU (library GEMM + BatchNorm kernel): it has no CPU path"},
                "e2e": {"value": v, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    w = torch.from_numpy((rng.normal(size=(27, args.cin, args.cout)) / np.sqrt(27 * args.cin)).astype(np.float16)).to(device)
    l2buf = torch.zeros(256 * 1024 * 1024 // 4, dtype=torch.float32, device=device)
    gt, st_ = min(args.cin, 16), min(args.cout, 16)
    per_df, nnz = {}, None
    for df in range(9):
        try:
            m = ref.cuda_binary_search(keys, keys, (3, 3, 3), (1, 1, 1), df)
            if df == 0:
                nnz = int((m[2] >= 0).sum().item())
                fn = lambda: ref.cuda_sparse_convolution_forward_os(n, n, m[2], feats, w)
            elif df == 1:
                fn = lambda: ref.cuda_sparse_convolution_forward_ws_merged(n, n, feats, w, m[5], m[6], m[3], m[7], m[8], False)
            elif df == 2:
                fn = lambda: ref.cuda_sparse_convolution_forward_ws(n, n, gt, st_, 4, -1, feats, w, m[3], m[4], m[5])
            elif df % 2 == 1:
                fn = lambda: ref.cuda_sparse_convolution_forward_hs_merged(n, n, feats, w, m[5], m[6], m[3], None if df == 3 else m[2],
                                                                           m[7], m[8], False)
            else:
                fn = lambda: ref.cuda_sparse_convolution_forward_hs(n, n, gt, st_, 4, -1, feats, w, m[3], m[4], m[5],
                                                                    None if df == 4 else m[2])
            mean_ms, min_ms = _time_calls(fn, args.steps, args.warmup, l2buf)
            map_ms, _ = _time_calls(lambda: ref.cuda_binary_search(keys, keys, (3, 3, 3), (1, 1, 1), df), args.steps, args.warmup, l2buf)
            per_df[df] = {"ms": round(mean_ms, 5), "min_ms": round(min_ms, 5), "kernel_map_build_ms": round(map_ms, 5)}
        except RuntimeError as e:
            ref.cuda_reset_error()
            per_df[df] = {"error": str(e).splitlines()[0][:120]}
    ok = {d: v for d, v in per_df.items() if "ms" in v}
    best = min(ok, key=lambda d: ok[d]["ms"])
    flops = 2.0 * nnz * args.cin * args.cout
    mean_ms = ok[best]["ms"]
    return {"metric": "SpC layer TFLOP/s (FLOPs = 2*nnz*c_in*c_out)", "value": round(flops / (mean_ms * 1e-3) / 1e12, 3), "unit": "TFLOP/s",
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": mean_ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": f"single submanifold 3^3 layer {args.cin}->{args.cout}, {n} voxels ({args.scene}), the reference's best dataflow",
                       "nnz": nnz, "best_dataflow": best, "l2": "256 MiB buffer rewritten between timed steps"},
            "kernel_map_build_ms": ok[best]["kernel_map_build_ms"], "per_dataflow": {str(k): v for k, v in per_df.items()},
            "cpu_baseline": {"value": round(flops / (mean_ms * 1e-3) / 1e12, 3), "unit": "TFLOP/s", "cores": 0, "kind": "reference",
                             "sample": "the reference's own CUDA kernels on the GPU: it has no CPU path"},
            "e2e": {"value": round(flops / (mean_ms * 1e-3) / 1e12, 3), "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}


def run_kmap_reference(args, device, pk, pk_kind):
    """The kernel-map workload on the reference's own builder, with the protocol of scripts/mapping_experiment.py:84-105
    (the map-building call between two events) on the same four scenes and map kinds as this engine's leg."""
    from spira_b200 import scenes as sc
    ref = reference_tools().load_native()
    scenes_k = []
    for seed in (1, 2, 3, 4):
        keys, _ = ref.cuda_flatten_sort(torch.from_numpy(sc.lidar_scene(seed)).to(device), False)
        keys = _padded(keys)
        scenes_k.append((keys, ref.cuda_downsample(keys, 2, 2, 2)))
    l2buf = torch.zeros(256 * 1024 * 1024 // 4, dtype=torch.float32, device=device)
    out = {}
    for name, ks, strided, df in (("3x3x3_os", (3, 3, 3), False, 0), ("3x3x3_ws", (3, 3, 3), False, 1), ("5x5x5_os", (5, 5, 5), False, 0),
                                  ("down_3x3x3_os", (3, 3, 3), True, 0), ("down_3x3x3_ws", (3, 3, 3), True, 1)):
        def fn():
            for keys, down in scenes_k:
                ref.cuda_binary_search(keys, down if strided else keys, ks, (1, 1, 1), df)
        mean_ms, min_ms = _time_calls(fn, args.steps, args.warmup, l2buf)
        K = ks[0] * ks[1] * ks[2]
        byts = sum((k.numel() + (d.numel() if strided else k.numel())) * 4 + K * ((((d.numel() if strided else k.numel()) + 127) // 128) * 128) * 4
                   for k, d in scenes_k)
        out[name] = {"ms_per_scene": round(mean_ms / 4, 5), "min_ms_per_scene": round(min_ms / 4, 5), "algorithmic_bytes_per_scene": byts // 4,
                     "gbs": round(byts / (mean_ms * 1e-3) / 1e9, 1)}

    def all_maps():
        for keys, down in scenes_k:
            maps = ref.cuda_binary_search_streamed([keys, down], [(3, 3, 3), (3, 3, 3)], [(1, 1, 1), (1, 1, 1)], [0, 0])
            ref.cuda_binary_search(keys, keys, (5, 5, 5), (1, 1, 1), 0)
            ref.cuda_convert_transposed_os(maps[1][2], keys.numel())
    mean_ms, min_ms = _time_calls(all_maps, args.steps, args.warmup, l2buf)
    v = round(4 / (mean_ms * 1e-3), 2)
    return {"metric": "kernel-map build (3^3 + 5^3 + stride-2 + transposed inverse)", "value": v, "unit": "scenes/s",
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(mean_ms, 5), "ms_per_scene": round(mean_ms / 4, 5),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u32", "data": "synthetic",
            "config": {"workload": "kernel maps only, 4 LiDAR-like scenes ~125k voxels each", "voxels": [k.numel() for k, _ in scenes_k],
                       "l2": "256 MiB buffer rewritten between timed steps"},
            "maps": out,
            "cpu_baseline": {"value": v, "unit": "scenes/s", "cores": 0, "kind": "reference",
                             "sample": "the reference's own CUDA map builder on the GPU: it has no CPU path"},
            "e2e": {"value": v, "unit": "scenes/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}


def run_reference_port(args, wl, n_gpus):
    """Reference arm when the reference's native module is unavailable: the CPU oracle port."""
    from spira_b200 import scenes as sc
    sys.path.insert(0, str(ROOT / "oracle"))
    c = wl["scene"](wl["seeds"][0])
    layers = [dict(cin=32, cout=32, K=27, transposed=False, in_stride=(1, 1, 1), out_stride=(1, 1, 1), ksize=(3, 3, 3), flops=1.0)]
    times = []
    for _ in range(max(1, min(args.steps, 3))):
        est, spent, _, _ = cpu_scene_pass(c, layers, budget_s=20.0)
        times.append(spent)
    v = 1.0 / statistics.mean(times)
    print(json.dumps({"impl": "reference", "metric": "scene throughput", "value": round(v, 5), "unit": "scenes/s", "n_gpus": n_gpus,
                      "steps": len(times), "warmup": 0, "ms_per_step": round(1e3 / v, 2), "higher_is_better": True, "scaling": "weak",
                      "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": {"workload": wl["label"]},
                      "cpu_baseline": {"value": round(v, 5), "unit": "scenes/s", "cores": torch.get_num_threads(), "kind": "port",
                                       "sample": "oracle port: sort + level-0 3^3 map + one 32->32 layer of scene 0"},
                      "e2e": {"value": round(v, 5), "unit": "scenes/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


if __name__ == "__main__":
    main()
