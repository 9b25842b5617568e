#!/usr/bin/env python
"""Benchmark of the sparse-convolution hot path on synthetic LiDAR-like scenes.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload minkunet|indoor|second]

One step = one whole scene through the reference's timed region (scripts/end_to_end_experiment.py:191-207):
``SparseTensor.order()`` + network-wide kernel-map build (``KernelMapCache.add_all_kernel_maps``) + the network's
forward pass.  Default workload: MinkUNet18-style network, fp16, random init, one ~125k-voxel scene per step
(the headline workload).  With N > 1 (launched by torch.distributed.run) every rank owns one GPU and its own
scenes; nothing is exchanged on the data path, so scaling is weak and ``value`` = scenes of all ranks / slowest rank.

``--impl reference`` drives the reference's own native module (built from its unmodified sources into
``oracle/_ref/_C.so``) through the same Python glue, model definition and timing loop.  The reference has no CPU
implementation of this path; if its module is unavailable the arm times the CPU oracle port instead.

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
# the reference's native module behind this repo's Python glue
# ------------------------------------------------------------------------------------------------
class ReferenceModule:
    """Adapter: the reference's pybind module plus the three helpers this repo's glue calls that are plain torch
    operations in the reference's own Python (feature permutation ``features[index]``, ``map.T.contiguous()``)."""
    LAYOUT_OS, LAYOUT_WS = 0, 1
    CACHE_DERIVED = False   # the reference rebuilds the inverted map of a transposed layer on every forward

    def __init__(self, mod):
        self._mod = mod

    def __getattr__(self, name):
        return getattr(self._mod, name)

    def cuda_flatten_sort(self, coords, double=False):
        keys, perm = self._mod.cuda_flatten_sort(coords, double)
        if (keys.numel() * keys.element_size()) % 512 == 0:
            # the reference's search reads sources[num_sources] (kernels/query_sorted.cuh:42,48); keep that read
            # inside an allocation when the tensor ends exactly on an allocator block boundary
            big = torch.empty(keys.numel() + 64, dtype=keys.dtype, device=keys.device)
            big[:keys.numel()] = keys
            keys = big[:keys.numel()]
        return keys, perm

    @staticmethod
    def permute_rows(rows, perm):
        return rows[perm.to(torch.int64)]

    @staticmethod
    def transpose_map(m):
        return m.T.contiguous()

    @staticmethod
    def _aligned(n):
        return (n + 127) // 128 * 128

    @staticmethod
    def check_status(device=None):
        return None


def load_reference_module():
    so = ROOT / "oracle" / "_ref" / "_C.so"
    if not so.exists():
        return None
    import importlib.util
    spec = importlib.util.spec_from_file_location("_C", str(so))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return ReferenceModule(mod)


def install_native(module) -> None:
    """Points every glue module of the package at ``module`` instead of the built-in binding."""
    import spira_b200.nn.functional as F
    from spira_b200.nn import conv
    from spira_b200.nn.functional import indexing, convolution, memory
    for m in (F, conv, indexing, convolution, memory):
        m._C = module


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
                "reasons": sorted(reasons), "samples": len(sm)}


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
    total_ms = sharding.max_over_ranks(sum(per_step), torch.device("cuda"))
    return total_ms, wall + (per_step,)


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


# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of the 42 convolution launches of one default step, from the
# ncu launch list of that step (profiles/minkunet_step_launch_list.md); valid for the default workload only
NCU_CONV_DRAM_BYTES_PER_STEP = {"minkunet": 693_949_696}


def roofline_from_layers(layers, pk, pk_kind, workload=None):
    if not layers:
        return None
    t_ms = sum(l["ms"] for l in layers)
    step_traffic = NCU_CONV_DRAM_BYTES_PER_STEP.get(workload)
    traffic = None if step_traffic is None else int(step_traffic / len(layers))      # per launch, like `achieved`
    flops = sum(l["flops"] for l in layers)
    byts = sum(l["bytes"] for l in layers)
    ideal_tensor_ms = flops / (pk["bf16_tflops_sustained"] * 1e12) * 1e3
    ideal_hbm_ms = byts / (pk["hbm_gbs"] * 1e9) * 1e3
    if ideal_hbm_ms >= ideal_tensor_ms:
        ach = byts / (t_ms * 1e-3) / 1e9
        return {"bound": "hbm", "achieved": round(ach, 1), "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": round(ach / pk["hbm_gbs"], 4),
                "traffic": traffic, "kernel": "conv_os_n256_kernel / conv_tc_kernel / conv_os_stem_kernel (all sparse-convolution layers of one scene)",
                "peak_source": f"of {pk_kind}", "launches": len(layers), "kernel_ms_per_step": round(t_ms, 4),
                "algorithmic_bytes_per_step": int(byts), "tflops": round(flops / (t_ms * 1e-3) / 1e12, 2)}
    ach = flops / (t_ms * 1e-3) / 1e12
    return {"bound": "tensor", "achieved": round(ach, 2), "peak": pk["bf16_tflops_sustained"], "unit": "TFLOP/s",
            "frac": round(ach / pk["bf16_tflops_sustained"], 4), "traffic": traffic,
            "kernel": "conv_os_n256_kernel / conv_tc_kernel / conv_os_stem_kernel (all sparse-convolution layers of one scene)", "peak_source": f"of {pk_kind}",
            "launches": len(layers), "kernel_ms_per_step": round(t_ms, 4), "algorithmic_flops_per_step": int(flops),
            "gbs": round(byts / (t_ms * 1e-3) / 1e9, 1)}


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
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="minkunet", choices=["minkunet", "indoor", "second", "layer", "kmap"])
    ap.add_argument("--no-group", action="store_true", help="output-stationary maps keep their target order (no grouping by neighbour pattern)")
    ap.add_argument("--no-defer", action="store_true", help="add_all_kernel_maps completes all maps before it returns")
    ap.add_argument("--n256-min-targets", type=int, default=-1, help="layers with fewer targets use 128-target tiles (-1 = library default)")
    ap.add_argument("--no-n256", action="store_true", help="output-stationary layers always use the targets-as-M kernel")
    ap.add_argument("--gather", default="default", choices=["default", "tma", "cpasync"], help="row-gather engine of the tensor-core kernels")
    ap.add_argument("--cin", type=int, default=64)
    ap.add_argument("--cout", type=int, default=64)
    ap.add_argument("--scene", default="c0", choices=["c0", "lidar"], help="layer workload: 50k-voxel plane/sphere scene or a LiDAR scene")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--dataflow", default="auto", choices=["auto", "0", "1"], help="auto = per-group selector (tune); 0/1 = uniform")
    ap.add_argument("--no-compile", action="store_true", help="run the eager module path instead of the recorded tape (ours arm)")
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
        from spira_b200 import build, _lib
        build.build()
        _lib.load()
        line = {"layer": run_layer, "kmap": run_kmap}[args.workload](args, device, pk, pk_kind)
        line["n_gpus"] = n_gpus
        if rank == 0:
            print(json.dumps(line))
        if dist_ctx:
            torch.distributed.destroy_process_group()
        return
    wl = make_workload(args.workload)
    from spira_b200 import scenes as sc

    ref_mod = None
    if args.impl == "reference":
        ref_mod = load_reference_module()
        if ref_mod is None:
            if rank == 0:
                run_reference_port(args, wl, n_gpus)
            if dist_ctx:
                torch.distributed.destroy_process_group()
            return
        install_native(ref_mod)
    else:
        from spira_b200 import build, _lib
        build.build()
        _lib.load()

    # scenes of this rank: resident on the device AND in pinned host memory (for the end-to-end number)
    seeds = [s + 100 * rank for s in wl["seeds"]]
    host, dev = [], []
    for s in seeds:
        c = wl["scene"](s)
        f = sc.features(len(c), wl["channels"], s, wl["feat_kind"])
        hc, hf = torch.from_numpy(c).pin_memory(), torch.from_numpy(f).pin_memory()
        host.append((hc, hf))
        dev.append((hc.to(device), hf.to(device)))
    n_vox = [len(h[0]) for h in host]

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
                            tune_tag=f"{args.workload}_r{rank}", force_retune=True, return_dataflows=True, verify=False)
        engine.apply_groups(chosen)
        chosen_note = {str(k): v for k, v in chosen.items()}
    else:
        # the reference tunes per layer group with dozens of whole-model runs; here: the best UNIFORM dataflow of 0/1/2
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
        # then, like the reference's own tuner (spira/utils/helpers.py:388-618), per layer group: every group tries the
        # other dataflows on whole-model runs and keeps what is faster
        try:
            tuned = tune_reference_groups(engine, dev, best[0])
            if tuned is not None:
                chosen_note = {"per_group": {str(k): v for k, v in tuned.items()}, "start": best[0]}
        except RuntimeError:
            ref_mod.cuda_reset_error()
            engine.set_uniform_dataflow(best[0])

    if args.impl == "ours" and not args.no_compile:
        engine.compile(*dev[0])
    l2buf = torch.zeros(256 * 1024 * 1024 // 4, dtype=torch.float32, device=device)
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
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = _lib.launch_count
    total_ms, wall = timed_loop(step_resident, args.steps, args.warmup, l2buf, dist_ctx)
    launches = _lib.launch_count - launches0
    e2e_ms, _ = timed_loop(step_e2e, args.steps, args.warmup, l2buf, dist_ctx, drain_e2e)
    clocks = sampler.stop() if rank == 0 else None

    ms_per_step = total_ms / args.steps
    value = n_gpus * args.steps / (total_ms / 1e3)
    e2e_value = n_gpus * args.steps / (e2e_ms / 1e3)
    h2d = int(np.mean([h[0].numel() * 4 + h[1].numel() * 2 for h in host]))
    d2h = int(d2h_bytes[0])

    line = {
        "metric": "MinkUNet scene throughput (scene latency = ms_per_step)" if args.workload == "minkunet" else f"{args.workload} scene throughput",
        "value": round(value, 3), "unit": "scenes/s", "n_gpus": n_gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16 (fp32 accumulate); u32 packed keys", "data": "synthetic",
        "config": {"workload": wl["label"], "voxels_per_scene": n_vox, "scenes_per_rank": len(dev),
                   "timed_region": "order() + add_all_kernel_maps() + model forward, per scene",
                   "l2": "256 MiB buffer rewritten between timed steps",
                   "setup": "tune / compile, then every scene once untimed (allocator priming), then the W warm-up steps",
                   "dataflows": chosen_note, "sharding": "independent scenes per GPU, no collective",
                   "fused_epilogue": bool(args.impl == "ours" and not args.no_fuse),
                   "recorded_tape": bool(args.impl == "ours" and not args.no_compile)},
        "e2e": {"value": round(e2e_value, 3), "unit": "scenes/s", "ms_per_step": round(e2e_ms / args.steps, 4),
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches if args.impl == "ours" else 0,
        "host_enqueue_ms_per_step": round(wall[1] * 1e3 / args.steps, 4),
        "step_ms_min_median_max": [round(min(wall[2]), 4), round(statistics.median(wall[2]), 4), round(max(wall[2]), 4)],
        "step_ms_first": [round(v, 4) for v in wall[2][:8]],
        "clocks": clocks,
    }
    if args.impl == "reference":
        line["impl"] = "reference"
        line["cpu_baseline"] = {"value": line["value"], "unit": "scenes/s", "cores": 0, "kind": "reference",
                                "sample": "the reference's own CUDA kernels (its unmodified sources built for sm_100) on the GPU: it has no CPU path"}
    else:
        # roofline of the dominant kernel class + secondary metrics, measured live with CUDA events
        per_call, layers = profile_kernels(engine, dev[0])
        line["roofline"] = roofline_from_layers(layers, pk, pk_kind, args.workload if args.dataflow == "auto" else None)
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
    if rank == 0:
        print(json.dumps(line))
    if dist_ctx:
        torch.distributed.destroy_process_group()


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
    kernel = "conv_tc_kernel<WS>" if df else ("conv_os_n256_kernel" if 64 < args.cout <= 96 else "conv_tc_kernel<OS>")
    if df == 0 and m[2]._sb.get("grouped") is not None and args.cin % 8 == 0:
        # Bytes that cross from L2 into the SMs per launch: gathered rows + one weight chunk per visited (tile, 64-wide
        # reduction chunk) + the map.  This, not HBM, is what the output-stationary kernels move most of.
        stats = m[2]._sb["grouped"].stats.cpu().tolist()
        tile_rows = 256 if kernel == "conv_os_n256_kernel" else 128
        visited = stats[1] if tile_rows == 256 else stats[0]              # non-empty (tile, offset) pairs of the grouped map
        xbar = nnz * args.cin * 2 + visited * (args.cin / 64.0) * args.cout * 128 + m[2].numel() * 4
        roof["l2_to_sm"] = {"bytes_per_launch": int(xbar), "achieved_gbs": round(xbar / (min_ms * 1e-3) / 1e9, 1),
                            "note": "gathered rows + weight chunks + map, over the fastest launch"}
    # DRAM bytes per launch from an ncu capture of exactly this case (dram__bytes_read.sum + dram__bytes_write.sum)
    if args.scene == "lidar" and (args.cin, args.cout, df) == (96, 96, 0):
        roof["traffic"] = 39_471_000
    roof.update(kernel=kernel, peak_source=f"of {pk_kind}", algorithmic_bytes=int(byts), algorithmic_flops=int(flops))
    return {"metric": "SpC layer TFLOP/s (FLOPs = 2*nnz*c_in*c_out)", "value": round(flops / (mean_ms * 1e-3) / 1e12, 3), "unit": "TFLOP/s",
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(mean_ms, 5), "min_ms": round(min_ms, 5), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16 (fp32 accumulate)", "data": "synthetic",
            "config": {"workload": f"single submanifold 3^3 layer {args.cin}->{args.cout}, {n} voxels ({args.scene}), dataflow {'WS' if df else 'OS'}",
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
                         "traffic": None, "kernel": "kmap_search_kernel<u32>, 5^3 map of scene 0", "peak_source": f"of {pk_kind}",
                         "algorithmic_bytes": byts5, "kernel_ms": round(k_ms, 5), "kernel_min_ms": round(k_min, 5)},
            "gpu_launches": args.steps * 4 * 4}


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
