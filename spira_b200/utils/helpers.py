"""``as_tuple``, ``set_kernel_map_cache`` and ``tune`` with the reference's signatures
(spira/utils/helpers.py:20-47, 388-618).

``tune`` keeps the reference's entry point, grouping rule (layers grouped by
``(effective_stride, kernel_size, stride)``), return value and ``.pt`` result file, but chooses the
dataflow of each group from MEASURED layer shape and map density instead of timing nine
dataflows: the engine has two dataflows (output-stationary = reference dataflow 0, weight-stationary
= reference dataflow 1) and a cost model over the hit counts the map search already produced.
With ``verify=True`` the model-level timing of the reference (``helpers.py:122-143``) cross-checks
the choice.
"""
__all__ = ['as_tuple', 'make_divisible', 'tune', 'set_kernel_map_cache', 'DataflowConfig', 'choose_dataflow']

import functools
import itertools
import os.path
from collections import defaultdict
from typing import Dict, Iterable, List, Optional, Tuple, Union

import torch
from torch.nn import Module

from spira_b200.utils.typing import ScalarOrTuple


def set_kernel_map_cache(module: Module, cache):
    if hasattr(module, "set_kernel_map_cache"):
        module.set_kernel_map_cache(cache)
    for submodule in module.children():
        set_kernel_map_cache(submodule, cache=cache)
    return module


def as_tuple(value: ScalarOrTuple, *, size: int = 3, name: Optional[str] = None):
    name = name or "Value"
    if not isinstance(value, Iterable):
        return tuple(value for _ in range(size))
    value = tuple(value)
    if len(value) != size:
        raise ValueError(f"{name} must be a scalar or a iterable of size {size} but found {len(value)} elements")
    return value


def make_divisible(value: int, divisor: int) -> int:
    return (value + divisor - 1) // divisor * divisor


class DataflowConfig:
    """Per-group choice, same fields as the reference's record (helpers.py:81-93)."""

    def __init__(self, map_dataflow: int = 0, force_os: bool = False):
        self.map_dataflow = map_dataflow
        self.force_os = force_os

    def __repr__(self):
        return f"DataflowConfig(map_dataflow={self.map_dataflow}, force_os={self.force_os})"

    def to_dict(self):
        return {"map_dataflow": self.map_dataflow, "force_os": self.force_os}


# Calibration of the selector's cost model, measured on B200 with the kernels of this package (per-layer CUDA-event
# timings of a MinkUNet18-style network on ~125k-voxel scenes):
_CHUNK_US = (0.45, 0.0012)     # one pipeline stage of 128 rows x 64 channels (targets-as-M kernel): a + b * c_out us
_CHUNK256_US = 0.72            # one stage of 256 rows x 64 channels (targets-as-N kernel, 64 < c_out <= 96, K <= 32)
_GROUPED_REDUNDANCY = (1.2, 1.3)   # rows visited per real pair once the map rows are grouped (128- / 256-row tiles)
_IMBALANCE = (1.3, 1.3)        # heaviest CTA over the mean (128- / 256-row tiles)
_TILE_OVERHEAD_CHUNKS = (3.0, 6.0)   # per-tile prologue and epilogue, in units of one stage (128- / 256-row tiles)
_HEAVIEST_TILE = 0.75          # share of all offsets present in the fullest tile of a grouped map
_ATOMIC_BYTES_PER_US = 7.0e6   # fp32 vector reductions into the weight-stationary scratch (eight lanes per output row)
_STREAM_BYTES_PER_US = 1.0e7   # in-kernel conversion pass over the scratch (read fp32, write fp16, write zeros)
_WS_FIXED_US = 9.0             # launch, pipeline fill, grid barrier of the single cooperative launch
_OS_FIXED_US = 14.0
_INVERT_US = (150.0, 3.0e6)    # output-stationary map of a transposed layer: inverse, its rows in the grouping sort, its own
                               # grouped copy (measured end to end: the step gets slower unless the layer saves more than that)
_SM_COUNT = 148


_GROUP_COST_US = (12.0, 4.0e-4)    # grouping the rows of one map: fixed + per row (its share of the sort, the re-ordered copy)


def grouping_cost_us(num_targets: int) -> float:
    """Time the network-wide build spends on grouping one output-stationary map of ``num_targets`` rows."""
    return _GROUP_COST_US[0] + _GROUP_COST_US[1] * num_targets


def estimate_layer_us(c_in: int, c_out: int, kernel_volume: int, num_targets: int, nnz: int,
                      nonempty_tile_offsets: int = None, submanifold: bool = True, transposed: bool = False,
                      grouped: bool = True):
    """(output-stationary, weight-stationary) time estimates in microseconds.

    OS runs one persistent CTA per SM over tiles of 128 (or, for 64 < c_out <= 96, 256) map rows and streams one stage per
    (tile, 64 reduction elements) with a neighbour.  Maps with K <= 32 have their rows grouped by neighbour pattern,
    which leaves ~1.2-1.3 visited rows per real pair; other maps visit every non-empty (tile, offset) pair
    (``nonempty_tile_offsets``, from the search's hit counters).  WS streams one stage per 128 compacted pairs and 64
    input channels over all SMs but pays an fp32 read-modify-write of the output per pair plus a zero-fill and a
    conversion pass.  A transposed OS layer also pays for inverting (and grouping) the map of its twin.
    ``grouped=False`` gives the OS estimate for a map that keeps its target order."""
    import math
    chunk = _CHUNK_US[0] + _CHUNK_US[1] * c_out
    per_in = c_in / 64.0
    wide = not (64 < c_out <= 96 and kernel_volume <= 32)     # 128-row tiles (targets as M) unless the 256-target kernel applies
    rows_per_tile = 128 if wide else 256
    tiles = max(1, math.ceil(num_targets / rows_per_tile))
    ctas = min(_SM_COUNT, tiles)
    stage_us = chunk if wide else _CHUNK256_US
    grouped = grouped and kernel_volume <= 32
    if grouped:
        stages = _GROUPED_REDUNDANCY[0 if wide else 1] * nnz / rows_per_tile * per_in
    else:
        tiles128 = max(1, math.ceil(num_targets / 128))
        if nonempty_tile_offsets is None:
            nonempty_tile_offsets = tiles128 * kernel_volume
        stages = nonempty_tile_offsets * per_in * (128.0 / rows_per_tile)       # counted per 128-row tile
    which = 0 if wide else 1
    per_cta = _IMBALANCE[which] * stages / ctas + _TILE_OVERHEAD_CHUNKS[which] * math.ceil(tiles / ctas)
    if grouped:                 # no CTA finishes before the fullest tile of the grouped map
        per_cta = max(per_cta, _HEAVIEST_TILE * kernel_volume * per_in + _TILE_OVERHEAD_CHUNKS[which])
    os_us = _OS_FIXED_US + stage_us * per_cta
    if transposed:
        os_us += _INVERT_US[0] + num_targets * kernel_volume * 8 / _INVERT_US[1]
    rows = (kernel_volume + 1) // 2 if submanifold and kernel_volume % 2 == 1 else kernel_volume
    ws_stages = (nnz / 128.0 + rows / 2.0) * math.ceil(per_in)
    ws_us = (math.ceil(ws_stages / _SM_COUNT) * chunk + nnz * c_out * 4 / _ATOMIC_BYTES_PER_US
             + num_targets * c_out * 10 / _STREAM_BYTES_PER_US + _WS_FIXED_US)
    return os_us, ws_us


def choose_dataflow(c_in: int, c_out: int, kernel_volume: int, num_targets: int, nnz: int, nonempty_tile_offsets: int,
                    transposed_or_strided: bool = False) -> int:
    """Selector: 0 (output-stationary) or 1 (weight-stationary) from layer shape and measured map density.

    Channel counts the tensor-core kernels cannot tile run output-stationary on the SIMT kernel.  Otherwise the
    dataflow with the smaller :func:`estimate_layer_us` wins; in practice OS wins on the large, surface-dense levels
    (no atomics, one pass over the output) and WS on the small deep levels (16-40 tiles cannot fill 148 SMs
    output-stationary) and on transposed layers (about two neighbours per fine voxel)."""
    if c_in % 8 != 0 or c_out % 16 != 0 or c_out > 256 or num_targets == 0:
        return 0
    os_us, ws_us = estimate_layer_us(c_in, c_out, kernel_volume, num_targets, nnz, nonempty_tile_offsets,
                                     submanifold=not transposed_or_strided)
    return 1 if ws_us < os_us else 0


def _map_statistics(cache, conv, inputs_stride):
    """(num_targets, nnz, non-empty (tile, offset) count) of the layer's map from the search's hit counters."""
    from spira_b200.utils.helpers import as_tuple as _t
    s = _t(inputs_stride, size=3)
    if conv.transposed:
        key = (tuple(a // b for a, b in zip(s, conv.stride)), s, conv.kernel_size)
    else:
        key = (s, tuple(a * b for a, b in zip(s, conv.stride)), conv.kernel_size)
    entry = cache._kernel_maps_cache.get(key)
    if entry is None:
        return None
    sb = getattr(entry[3], "_sb", None)
    if sb is None:
        return None
    from spira_b200.nn.functional import _C
    counts = _C.map_counts(entry[3])
    if counts is None:
        return None
    nnz = int(counts.sum().item())
    nonempty = int((counts > 0).sum().item())
    return int(entry[2]), nnz, nonempty


def _time_model(model, samples, cache, skip: int = 1) -> float:
    times = []
    for i, x in enumerate(samples):
        if cache is not None:
            cache.reset()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        with torch.no_grad():
            model(x)
        b.record()
        b.synchronize()
        if i >= skip:
            times.append(a.elapsed_time(b))
    return sum(times) / max(len(times), 1)


def tune(model: Module, data_loader: Iterable, kernel_map_cache=None, map_dataflow_options: List[int] = None,
         test_force_os: bool = True, n_samples: int = 10, n_samples_for_gs: int = 1, save_dir: str = ".tune_configs",
         tune_tag: str = "default", force_retune: bool = False, allow_gs_tuning: bool = True, verbose: bool = False,
         return_dataflows: bool = False, verify: bool = False) -> Union[Module, Tuple[Module, Dict]]:
    """Chooses a dataflow per layer group and stores it in every layer's ``_tunable_config``.

    Result file ``<save_dir>/<tune_tag>.pt`` holds ``{name_to_group, best_configs, layer_configs}`` like the
    reference's (helpers.py:340-365) and is reloaded unless ``force_retune``.
    """
    from spira_b200.nn import SparseConv

    allowed = set(map_dataflow_options) if map_dataflow_options is not None else {0, 1}
    samples = list(itertools.islice(data_loader, max(1, min(n_samples, 4))))
    save_path = os.path.join(save_dir, f"{tune_tag}.pt")
    convs = {name: m for name, m in model.named_modules() if isinstance(m, SparseConv)}

    def apply(name_to_group, best):
        for name, m in convs.items():
            g = name_to_group.get(name)
            if g is not None and g in best:
                m._tunable_config['map_dataflow'] = best[g].map_dataflow
                m._tunable_config['force_os'] = best[g].force_os

    def apply_grouping(flags):
        # the cache groups the rows of every output-stationary map unless told otherwise: map key = (source stride,
        # target stride, kernel size) of the group's non-transposed layer
        if kernel_map_cache is not None and hasattr(kernel_map_cache, "set_group_policy"):
            policy = {}
            for (eff, ksize, stride), flag in flags.items():
                policy[(tuple(eff), tuple(a * b for a, b in zip(eff, stride)), tuple(ksize))] = bool(flag)
            kernel_map_cache.set_group_policy(policy)

    if os.path.exists(save_path) and not force_retune:
        try:
            blob = torch.load(save_path, weights_only=False)
            best = {g: DataflowConfig(**c) for g, c in blob["best_configs"].items()}
            apply(blob["name_to_group"], best)
            apply_grouping(blob.get("group_rows", {}))
            out = {g: c.map_dataflow for g, c in best.items()}
            return (model, out) if return_dataflows else model
        except Exception as e:  # unreadable cache -> tune again
            if verbose:
                print(f"could not load {save_path} ({e}); tuning again")

    # ---- one forward pass with hooks: group the layers and read the density of their maps
    name_to_group, group_to_name, stats = {}, defaultdict(list), defaultdict(list)

    def hook(module, inputs, outputs, name):
        x = inputs[0]
        stride = x._stride
        eff = tuple(stride[k] // module.stride[k] for k in range(3)) if module.transposed else stride
        g = (eff, module.kernel_size, module.stride)
        name_to_group[name] = g
        group_to_name[g].append(name)
        if not module.is_trivial and kernel_map_cache is not None:
            st = _map_statistics(kernel_map_cache, module, stride)
            if st is not None:
                T, nnz, nonempty = st
                if module.transposed:       # the map was built for the twin layer: its targets are this layer's sources
                    T, nonempty = outputs._features.shape[0], None
                stats[g].append((module.in_channels, module.out_channels, module.transposed, T, nnz, nonempty))

    handles = [m.register_forward_hook(functools.partial(hook, name=n)) for n, m in convs.items()]
    for m in convs.values():
        m._tunable_config['map_dataflow'] = 1  # weight-stationary maps carry every statistic the model needs
        m._tunable_config['force_os'] = False
    if kernel_map_cache is not None:
        kernel_map_cache.reset()
    with torch.no_grad():
        model(samples[0])
    for h in handles:
        h.remove()

    best: Dict[Tuple, DataflowConfig] = {}
    group_rows: Dict[Tuple, bool] = {}       # output-stationary groups: group the rows of their map by neighbour pattern?
    for g, names in group_to_name.items():
        # the layers of a group share their kernel maps, hence their dataflow: minimise the summed estimates
        os_total = ws_total = 0.0
        kv = g[1][0] * g[1][1] * g[1][2]
        for (cin, cout, transposed, T, nnz, nonempty) in stats.get(g, []):
            if choose_dataflow(cin, cout, kv, T, nnz, nonempty) == 0 and (cin % 8 or cout % 16 or cout > 256):
                ws_total = float("inf")      # a layer the tensor-core kernels cannot tile pins the group to OS
                continue
            o, w = estimate_layer_us(cin, cout, kv, T, nnz, nonempty, submanifold=not (transposed or any(v != 1 for v in g[2])),
                                     transposed=transposed)
            os_total += o
            ws_total += w
        df = 1 if ws_total < os_total else 0
        if df not in allowed:
            df = 0 if 0 in allowed else min(allowed)
        best[g] = DataflowConfig(map_dataflow=df, force_os=False)
        # Is grouping the rows of this map worth its sort?  Compare what the layers of the group save with the cost.
        layers_of_g = [st for st in stats.get(g, []) if not (st[0] % 8 or st[1] % 16 or st[1] > 256)]
        if df == 0 and kv <= 32 and layers_of_g:
            saved = 0.0
            for (cin, cout, transposed, T, nnz, nonempty) in layers_of_g:
                sub = not (transposed or any(v != 1 for v in g[2]))
                saved += (estimate_layer_us(cin, cout, kv, T, nnz, nonempty, submanifold=sub, grouped=False)[0]
                          - estimate_layer_us(cin, cout, kv, T, nnz, nonempty, submanifold=sub, grouped=True)[0])
            rows = max(st[3] for st in layers_of_g)
            group_rows[g] = saved > grouping_cost_us(rows)
        if verbose:
            print(f"group {g}: {len(names)} layer(s), estimated OS {os_total:.0f} us / WS {ws_total:.0f} us -> map_dataflow={df}"
                  + (f", rows grouped: {group_rows[g]}" if g in group_rows else ""))
    apply(name_to_group, best)

    if verify and len(best) > 0:
        base = _time_model(model, samples, kernel_map_cache)
        for g in list(best):
            if len(stats.get(g, [])) == 0:
                continue
            flipped = DataflowConfig(map_dataflow=1 - best[g].map_dataflow, force_os=False)
            if flipped.map_dataflow not in allowed:
                continue
            trial = dict(best)
            trial[g] = flipped
            apply(name_to_group, trial)
            t = _time_model(model, samples, kernel_map_cache)
            if t < 0.95 * base:
                best, base = trial, t
                if verbose:
                    print(f"group {g}: timing overrides the model -> map_dataflow={flipped.map_dataflow} ({t:.3f} ms)")
            apply(name_to_group, best)

    apply_grouping(group_rows)
    os.makedirs(save_dir, exist_ok=True)
    torch.save({"name_to_group": name_to_group,
                "best_configs": {g: c.to_dict() for g, c in best.items()},
                "group_rows": dict(group_rows),
                "layer_configs": {n: dict(m._tunable_config) for n, m in convs.items()}}, save_path)
    if kernel_map_cache is not None:
        kernel_map_cache.reset()
    out = {g: c.map_dataflow for g, c in best.items()}
    return (model, out) if return_dataflows else model
