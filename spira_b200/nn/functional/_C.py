"""Drop-in for the reference's pybind module ``spira.nn.functional._C``.

Same 18 function names, argument order and return structures as the reference registers
(``csrc/spira/torch/cuda_arg_sort_coordinates.cu:202-208``,
``csrc/spira/torch/cuda_sparse_convolution_mapping.cu:1832-1838``,
``csrc/spira/torch/cuda_sparse_convolution_forward.cu:500-507``,
``csrc/spira/torch/cuda_memory_buffer.cu:15-16``), implemented by calls into the C-ABI library
``libspira_b200.so``.  torch is used for device memory and the current stream only.

Kernel maps are returned as the reference's 9-tuple
``(num_sources, num_targets, map, opt, opt, opt, opt, mapsize, qmapsize)``; the tensors in it
additionally carry the engine's own structures in a ``_sb`` attribute so that the forward calls do
not have to rebuild them.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence, Tuple

import torch

from spira_b200 import _lib
from spira_b200._lib import KmapDesc, GroupDesc, WsDesc, Epilogue, LAYOUT_OS, LAYOUT_WS, PACK_OS, PACK_WS, MAX_MAPS, MAX_LEVELS


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream(device) -> C.c_void_p:
    idx = torch.device(device).index
    return C.c_void_p(torch._C._cuda_getCurrentRawStream(torch.cuda.current_device() if idx is None else idx))


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise NotImplementedError("spira_b200 runs on CUDA tensors only")


def _key_bytes(keys: torch.Tensor) -> int:
    if keys.dtype == torch.int32:
        return 4
    if keys.dtype == torch.int64:
        return 8
    raise RuntimeError(f"[spira_b200] packed keys must be int32 or int64, got {keys.dtype}")


def _aligned(n: int) -> int:
    return (n + 127) // 128 * 128


_status = {}


def status_word(device) -> torch.Tensor:
    """Per-device int32 the tensor-core kernels raise when one of their bounded waits expires."""
    idx = torch.device(device).index
    if idx is None:
        idx = torch.cuda.current_device()
    if idx not in _status:
        _status[idx] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
    return _status[idx]


def check_status(device=None) -> None:
    """Synchronises and raises if any kernel launched so far reported an expired wait."""
    for idx, t in list(_status.items()):
        if device is not None and torch.device(device).index not in (None, idx):
            continue
        if int(t.item()) != 0:
            t.zero_()
            _zero_scratch.pop(idx, None)     # a kernel that gave up may have left sums behind: start from a fresh zero scratch
            _split_scratch.pop(idx, None)    # ... or tile counters that are not back at zero
            with torch.cuda.device(idx):     # and bring the host's count of grid-barrier arrivals back in step with the device's
                _lib.call("spira_b200_ws_barrier_resync")
            raise RuntimeError("[spira_b200] a tensor-core kernel gave up on an internal wait (status word set)")


# ------------------------------------------------------------------------------------------------
# coordinates
# ------------------------------------------------------------------------------------------------
def cuda_flatten_sort(coordinates: torch.Tensor, is_double: bool = False):
    """``[N,3] int32`` -> ``(sorted packed keys [N] int32|int64, permutation [N] int32)``.
    Reference: ``CUDAFlattenSort`` (csrc/spira/torch/cuda_arg_sort_coordinates.cu:11-39)."""
    _require_cuda(coordinates)
    if coordinates.dim() != 2 or coordinates.shape[1] != 3 or coordinates.dtype != torch.int32:
        raise RuntimeError("[spira_b200] Tensor coordinates is expected to be int32 of shape [N, 3]")
    coordinates = coordinates.contiguous()
    n = coordinates.shape[0]
    kb = 8 if is_double else 4
    keys = torch.empty(n, dtype=torch.int64 if is_double else torch.int32, device=coordinates.device)
    perm = torch.empty(n, dtype=torch.int32, device=coordinates.device)
    need = C.c_size_t()
    _lib.call("spira_b200_flatten_sort_workspace", n, kb, C.byref(need))
    ws = torch.empty(need.value, dtype=torch.uint8, device=coordinates.device)
    _lib.call("spira_b200_flatten_sort", _ptr(coordinates), n, kb, _ptr(keys), _ptr(perm), _ptr(ws), need.value,
              _ptr(status_word(coordinates.device)), _stream(coordinates.device))
    return keys, perm


def cuda_unflatten(coordinates: torch.Tensor) -> torch.Tensor:
    """Packed keys ``[N]`` -> ``[N,3] int32`` (csrc/spira/torch/cuda_arg_sort_coordinates.cu:41-66)."""
    _require_cuda(coordinates)
    if coordinates.dim() != 1:
        raise RuntimeError("[spira_b200] Tensor coordinates is expected to have 1 dimension(s)")
    coordinates = coordinates.contiguous()
    n = coordinates.shape[0]
    out = torch.empty((n, 3), dtype=torch.int32, device=coordinates.device)
    _lib.call("spira_b200_unpack", _ptr(coordinates), n, _key_bytes(coordinates), _ptr(out), _stream(coordinates.device))
    return out


def permute_rows(rows: torch.Tensor, perm: torch.Tensor) -> torch.Tensor:
    """``rows[perm]`` for a 2-D tensor and an int32 permutation (the feature shuffle of ``SparseTensor.order``)."""
    _require_cuda(rows, perm)
    rows = rows.contiguous()
    row_bytes = rows.shape[1] * rows.element_size() if rows.dim() == 2 else 0
    if rows.dim() != 2 or perm.dtype != torch.int32 or row_bytes % 2 != 0 or row_bytes == 0:
        return rows[perm.long()]
    out = torch.empty_like(rows)
    _lib.call("spira_b200_permute_rows", _ptr(rows), _ptr(perm.contiguous()), rows.shape[0], row_bytes, _ptr(out),
              _stream(rows.device))
    return out


def cuda_streamed_output_generate(coordinates: torch.Tensor, target_strides: Sequence[Tuple[int, int, int]]) -> List[torch.Tensor]:
    """Down-sampled key sets of all levels from the level-0 keys; one host read of the level sizes.
    Reference: ``CUDAStreamedOutputGenerate`` (csrc/spira/torch/cuda_arg_sort_coordinates.cu:107-200)."""
    _require_cuda(coordinates)
    if coordinates.dim() != 1:
        raise RuntimeError("[spira_b200] Tensor coordinates is expected to have 1 dimension(s)")
    coordinates = coordinates.contiguous()
    strides = [tuple(int(v) for v in s) for s in target_strides]
    outputs: List[torch.Tensor] = []
    n, kb, dev = coordinates.shape[0], _key_bytes(coordinates), coordinates.device
    for first in range(0, len(strides), MAX_LEVELS):
        group = strides[first:first + MAX_LEVELS]
        L = len(group)
        bufs = torch.empty((L, n), dtype=coordinates.dtype, device=dev)
        host_strides = (C.c_int32 * (3 * L))(*[v for s in group for v in s])
        host_out = (C.c_void_p * L)(*[bufs[l].data_ptr() for l in range(L)])
        host_counts = None
        if first == 0 and SORT_FREE_DOWNSAMPLE and _strides_double(group):
            # sorted input (the usual case: the keys come from flatten_sort) needs no sort; the kernel reports an
            # unsorted input in the word behind the counts, which arrives with the same host read
            counts = torch.zeros(L + 1, dtype=torch.int32, device=dev)
            need = C.c_size_t()
            _lib.call("spira_b200_downsample_sorted_workspace", n, kb, C.byref(need))
            ws = torch.empty(need.value, dtype=torch.uint8, device=dev)
            _lib.call("spira_b200_downsample_sorted", _ptr(coordinates), n, kb, L, host_strides, host_out, _ptr(counts),
                      _ptr(ws), need.value, _ptr(counts[L:]), _stream(dev))
            host_counts = counts.cpu().tolist()
            if host_counts[L] != 0:
                host_counts = None
        if host_counts is None:
            counts = torch.empty(L, dtype=torch.int32, device=dev)
            need = C.c_size_t()
            _lib.call("spira_b200_downsample_workspace", n, kb, L, C.byref(need))
            ws = torch.empty(need.value, dtype=torch.uint8, device=dev)
            _lib.call("spira_b200_downsample", _ptr(coordinates), n, kb, L, host_strides, host_out, _ptr(counts), _ptr(ws),
                      need.value, _stream(dev))
            host_counts = counts.cpu().tolist()
        outputs += [bufs[l, :host_counts[l]] for l in range(L)]
    return outputs


SORT_FREE_DOWNSAMPLE = True


def _strides_double(strides) -> bool:
    prev = (1, 1, 1)
    for s in strides:
        if any(v != p and v != 2 * p for v, p in zip(s, prev)):
            return False
        prev = s
    return True


class PendingLevels:
    """Down-sampling whose kernels are enqueued and whose level sizes are on their way to the host.  Every pending
    build owns its landing slot (pinned buffer + event) until its sizes have been read, so that several builds --
    other caches, models or scenes -- can be in flight at once."""
    __slots__ = ("coordinates", "strides", "bufs", "counts", "host", "done", "levels", "slot", "device_index")

    def __del__(self):          # a build that was dropped without being completed gives its slot back
        _release_slot(self)


_side_stream = {}       # device index -> side stream of the size read-backs
_free_slots = {}        # device index -> [(pinned int32 buffer, its address, "sizes arrived" event, event handle), ...]


def _take_slot(idx: int, dev, side):
    free = _free_slots.setdefault(idx, [])
    if free:
        return free.pop()
    host = torch.zeros(MAX_LEVELS + 1, dtype=torch.int32).pin_memory()
    done = torch.cuda.Event()
    done.record(side)                       # creates the underlying event, whose handle the library records later
    return (host, host.data_ptr(), done, done.cuda_event)


def _release_slot(p) -> None:
    slot = getattr(p, "slot", None)
    if slot is not None:
        p.slot = None
        try:
            slot[2].synchronize()           # the copy into the buffer (if one is in flight) has landed
            _free_slots.setdefault(p.device_index, []).append(slot)
        except Exception:                   # interpreter shutdown: nothing to recycle
            pass


_ds_ws_bytes = {}       # (n, key bytes) -> workspace bytes of the sort-free down-sampling
_ds_strides = {}        # strides tuple -> ctypes int32 array


def streamed_output_generate_begin(coordinates: torch.Tensor, target_strides) -> Optional[PendingLevels]:
    """First half of :func:`cuda_streamed_output_generate` for sorted keys and doubling strides: launches the kernels and
    starts the copy of the level sizes on a side stream, so that the caller can enqueue work that does not depend on
    the sizes (the level-0 kernel map) before it waits in :func:`streamed_output_generate_end`.  Returns None when this
    path does not apply (then call the blocking function)."""
    strides = tuple(tuple(int(v) for v in s) for s in target_strides)
    L = len(strides)
    if not (SORT_FREE_DOWNSAMPLE and coordinates.is_cuda and coordinates.dim() == 1 and 1 <= L <= MAX_LEVELS
            and coordinates.shape[0] > 0):
        return None
    host_strides = _ds_strides.get(strides)
    if host_strides is None:
        if not _strides_double(strides):
            return None
        if len(_ds_strides) > 256:
            _ds_strides.clear()
        host_strides = _ds_strides[strides] = (C.c_int32 * (3 * L))(*[v for s in strides for v in s])
    coordinates = coordinates.contiguous()
    n, kb, dev = coordinates.shape[0], _key_bytes(coordinates), coordinates.device
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    side = _side_stream.get(idx)
    if side is None:
        side = _side_stream[idx] = torch.cuda.Stream(device=dev)
    need = _ds_ws_bytes.get((n, kb))
    if need is None:
        size = C.c_size_t()
        _lib.call("spira_b200_downsample_sorted_workspace", n, kb, C.byref(size))
        if len(_ds_ws_bytes) > 4096:
            _ds_ws_bytes.clear()
        need = _ds_ws_bytes[(n, kb)] = size.value
    p = PendingLevels()
    p.device_index, p.slot = idx, _take_slot(idx, dev, side)
    host, host_ptr, done, done_handle = p.slot
    p.coordinates, p.strides, p.levels = coordinates, strides, L
    p.bufs = torch.empty((L, n), dtype=coordinates.dtype, device=dev)
    p.counts = torch.empty(L + 1, dtype=torch.int32, device=dev)      # [L] = "the input was not sorted"
    ws = torch.empty(need, dtype=torch.uint8, device=dev)
    base, counts_ptr = p.bufs.data_ptr(), p.counts.data_ptr()
    host_out = (C.c_void_p * L)(*[base + l * n * kb for l in range(L)])
    main = _raw_stream(idx)
    _lib.call("spira_b200_downsample_sorted", coordinates.data_ptr(), n, kb, L, host_strides, host_out, counts_ptr, ws.data_ptr(),
              need, counts_ptr + 4 * L, main)
    _lib.call("spira_b200_read_back", counts_ptr, host_ptr, 4 * (L + 1), main, side.cuda_stream, done_handle)
    p.host, p.done = host, done
    return p


def streamed_output_generate_end(p: PendingLevels) -> List[torch.Tensor]:
    """Waits for the level sizes only (not for work enqueued since) and returns the level key sets."""
    p.done.synchronize()
    L = p.levels
    host_counts = p.host[:L + 1].tolist()
    _release_slot(p)
    if host_counts[L] != 0:      # the keys were not sorted: take the sorting path
        global SORT_FREE_DOWNSAMPLE
        SORT_FREE_DOWNSAMPLE, keep = False, SORT_FREE_DOWNSAMPLE
        try:
            return cuda_streamed_output_generate(p.coordinates, p.strides)
        finally:
            SORT_FREE_DOWNSAMPLE = keep
    return [p.bufs[l, :host_counts[l]] for l in range(L)]


def cuda_downsample(coordinates: torch.Tensor, stride_x: int, stride_y: int, stride_z: int) -> torch.Tensor:
    """``unique(sort(keys & mask))`` (csrc/spira/torch/cuda_arg_sort_coordinates.cu:68-105)."""
    return cuda_streamed_output_generate(coordinates, [(stride_x, stride_y, stride_z)])[0]


# ------------------------------------------------------------------------------------------------
# kernel maps
# ------------------------------------------------------------------------------------------------
class WsLists:
    """Compacted pair lists of a weight-stationary map (engine-native form of the reference's
    ``nbmaps / nbsizes / naddrs / qnaddrs`` slots).

    The kernels only need four device addresses (``in_ptr, out_ptr, naddrs_ptr, qnaddrs_ptr``).  The tensor views
    ``nbmaps [2, cap]``, ``in_idx``, ``out_idx``, ``nbsizes``, ``naddrs``, ``qnaddrs`` are either set directly or, for
    lists carved out of one arena by the network-wide builder, made on first access (``_lazy``: name -> (offset, shape)
    in int32 units of ``_arena``)."""

    def __getattr__(self, name):
        lazy = self.__dict__.get("_lazy")
        if lazy is not None and name in lazy:
            off, shape = lazy[name]
            n = 1
            for v in shape:
                n *= v
            t = self._arena[off:off + n].view(shape)
            setattr(self, name, t)
            return t
        raise AttributeError(name)

    def set_pointers(self):
        self.in_ptr, self.out_ptr = self.in_idx.data_ptr(), self.out_idx.data_ptr()
        self.naddrs_ptr, self.qnaddrs_ptr = self.naddrs.data_ptr(), self.qnaddrs.data_ptr()
        return self


def _dataflow_layout(dataflow: int) -> int:
    return LAYOUT_OS if dataflow == 0 else LAYOUT_WS


def _axis_range(k: int):
    lo = -(k // 2) if k % 2 == 1 else -(k // 2) + 1
    return range(lo, lo + k)


def l1_permutation(kernel_size, dataflow: int):
    """Row order of the hybrid dataflows 3-8 (``generate_indexes_L1``,
    csrc/spira/torch/cuda_sparse_convolution_mapping.cu:159-209): ``position[k]`` of every offset in natural order
    ``k = (ix*ky + iy)*kz + iz``.  Offsets whose L1 norm is below ``(dataflow - 1) // 2`` come first (the rows the
    output-stationary part takes), the others follow, both in natural order.  Returns ``(position, dense_offsets)``;
    like the reference, ``dense_offsets`` is read from ``position[0]`` (mapping.cu:682: the first natural offset is a
    corner, which is never among the leading rows of an odd kernel)."""
    threshold = (int(dataflow) - 1) // 2
    l1 = [abs(x) + abs(y) + abs(z) for x in _axis_range(kernel_size[0]) for y in _axis_range(kernel_size[1])
          for z in _axis_range(kernel_size[2])]
    front = sum(1 for v in l1 if v < threshold)
    position, f, b = [], 0, front
    for v in l1:
        if v < threshold:
            position.append(f)
            f += 1
        else:
            position.append(b)
            b += 1
    return position, position[0]


_l1_device = {}


def _l1_device_tensor(kernel_size, dataflow, device):
    key = (tuple(kernel_size), int(dataflow), str(device))
    t = _l1_device.get(key)
    if t is None:
        position, dense = l1_permutation(kernel_size, dataflow)
        t = _l1_device[key] = (torch.tensor(position, dtype=torch.int32, device=device), dense)
    return t


LAZY_SIZES = True   # cuda_binary_search_streamed(..., exact_sizes=False) keeps the list sizes on the device
WS_FUSED = True     # weight-stationary layers run as ONE cooperative launch over a persistent, always-zero scratch
DEFER_MAPS = True   # KernelMapCache.add_all_kernel_maps returns after the level-0 map; the rest is completed on first use
GROUP_OS = True     # output-stationary maps also get their rows grouped by neighbour pattern (spira_b200_kmap_group)
GROUP_MIN_TARGETS = 1024


class GroupedMap:
    """An output-stationary map with its rows sorted by presence mask: ``map [T_al, K]``, ``row_of [T_al]`` (the
    target of each grouped row), ``tile_masks [T_al / 128]`` and ``stats [2]`` (non-empty (tile, offset) pairs for
    128- and 256-row tiles, on the device).  The kernels take the three addresses; the tensors are views of one
    allocation shared by all maps of a call and are made on first access."""

    def __getattr__(self, name):
        lazy = self.__dict__.get("_lazy")
        if lazy is not None and name in lazy:
            off, shape = lazy[name]
            n = 1
            for v in shape:
                n *= v
            t = self._arena[off:off + n].view(shape)
            setattr(self, name, t)
            return t
        raise AttributeError(name)


_group_ws_bytes = {}


def group_os_maps(maps) -> list:
    """Groups the rows of engine-built ``[T_al, K]`` maps, ``maps = [(map, num_targets), ...]``, with one sort per
    <= 16 maps.  Returns one :class:`GroupedMap` (or None where grouping is off or does not apply) per input."""
    out = [None] * len(maps)
    todo = [i for i, (mp, T) in enumerate(maps) if GROUP_OS and mp.shape[1] <= 32 and T >= GROUP_MIN_TARGETS]
    for first in range(0, len(todo), MAX_MAPS):
        part = todo[first:first + MAX_MAPS]
        dev = maps[part[0]][0].device
        idx = dev.index if dev.index is not None else torch.cuda.current_device()
        total_rows, ints, offs = 0, 0, []
        for i in part:
            mp, T = maps[i]
            Tal, K = mp.shape
            o_map = ints
            ints += Tal * K
            o_row = ints
            ints += Tal
            o_mask = ints
            ints += (Tal // 128 + 63) & ~63
            o_stats = ints
            ints += 64
            offs.append((o_map, o_row, o_mask, o_stats))
            total_rows += int(T)
        need = _group_ws_bytes.get(total_rows)
        if need is None:
            size = C.c_size_t()
            _lib.call("spira_b200_kmap_group_workspace", total_rows, C.byref(size))
            if len(_group_ws_bytes) > 4096:
                _group_ws_bytes.clear()
            need = _group_ws_bytes[total_rows] = size.value
        arena = torch.empty(ints, dtype=torch.int32, device=dev)
        work = torch.empty(need, dtype=torch.uint8, device=dev)
        base = arena.data_ptr()
        descs = (GroupDesc * len(part))()
        for d, i, (o_map, o_row, o_mask, o_stats) in zip(descs, part, offs):
            mp, T = maps[i]
            Tal, K = mp.shape
            g = GroupedMap()
            g._arena = arena
            g._lazy = dict(map=(o_map, (Tal, K)), row_of=(o_row, (Tal,)), tile_masks=(o_mask, (Tal // 128,)), stats=(o_stats, (2,)))
            g.map_ptr, g.row_of_ptr, g.tile_masks_ptr = base + 4 * o_map, base + 4 * o_row, base + 4 * o_mask
            d.map_os, d.num_targets, d.K = mp.data_ptr(), int(T), K
            d.grouped_map, d.row_of, d.tile_masks, d.stats = g.map_ptr, g.row_of_ptr, g.tile_masks_ptr, base + 4 * o_stats
            out[i] = g
        _lib.call("spira_b200_kmap_group", descs, len(part), work.data_ptr(), need, _raw_stream(idx))
    return out


def group_os_map(map_os: torch.Tensor, num_targets: int) -> Optional[GroupedMap]:
    """Single-map form of :func:`group_os_maps`."""
    return group_os_maps([(map_os, int(num_targets))])[0]


def grouped_twin(map_os: torch.Tensor) -> Optional[GroupedMap]:
    """The grouped twin of an engine-built output-stationary map, or None.  Maps from the network-wide builder carry it
    already; a map from the single-map call (``cuda_binary_search``) gets it here, on the first convolution that runs
    over it -- the map build itself returns what the reference's returns and costs what a map build costs."""
    sb = getattr(map_os, "_sb", None)
    if sb is None:
        return None
    g = sb.get("grouped")
    if g is None and sb.get("group_lazy") is not None:
        num_targets, sb["group_lazy"] = sb["group_lazy"], None
        g = sb["grouped"] = group_os_map(map_os, num_targets)
    return g


def _build_maps(voxel_pairs, kernel_sizes, source_strides, dataflows, exact_sizes=True, group=True):
    """Shared implementation of the serial and the network-wide builders.

    ``voxel_pairs[i] = (sources, targets)``.  One search launch per group of <= 16 maps, one
    size scan per weight-stationary map, ONE host read of all list sizes, then the compactions.
    """
    n = len(voxel_pairs)
    dev = voxel_pairs[0][0].device
    kb = _key_bytes(voxel_pairs[0][0])
    stream = _stream(dev)
    info = []
    for i in range(n):
        src, tgt = voxel_pairs[i]
        _require_cuda(src, tgt)
        if _key_bytes(src) != kb or _key_bytes(tgt) != kb:
            raise RuntimeError("[spira_b200] all coordinate tensors of one call must share a key width")
        ks = tuple(int(v) for v in kernel_sizes[i])
        st = tuple(int(v) for v in source_strides[i])
        df = int(dataflows[i])
        if df < 0 or df > 8:
            raise RuntimeError(f"[spira_b200] unknown map dataflow {df}")
        S, T = src.shape[0], tgt.shape[0]
        K = ks[0] * ks[1] * ks[2]
        Tal = _aligned(T)
        layout = _dataflow_layout(df)
        shape = (Tal, K) if layout == LAYOUT_OS else (K, Tal)
        dense = torch.empty(shape, dtype=torch.int32, device=dev)
        counts = torch.empty((K, Tal // 128), dtype=torch.int32, device=dev)
        perm, n_dense = (None, 0)
        if df >= 3:
            # hybrid dataflows: the rows of the [K, T_al] map come in L1-norm order; the compacted half behind the leading
            # rows is mirrored, which presumes a submanifold map (the reference's tuner tries them on stride-1 layers only,
            # spira/utils/helpers.py:187-197)
            if S != T:
                raise RuntimeError(f"[spira_b200] map dataflow {df} (hybrid) needs a submanifold map: {S} sources, {T} targets")
            if ks[2] not in (3, 5):      # (csrc/spira/cuda/functions/query_sorted_index.cu:698-700)
                raise RuntimeError("[spira_b200] Currently Kernel Size in Z axis can only be 3, 5 for the hybrid dataflows")
            perm, n_dense = _l1_device_tensor(ks, df, dev)
            if (K - n_dense) % 2 != 0:
                raise RuntimeError(f"[spira_b200] map dataflow {df}: kernel size {ks} leaves an odd number of rows to mirror")
        info.append(dict(src=src, tgt=tgt, S=S, T=T, K=K, Tal=Tal, ks=ks, st=st, df=df, layout=layout, dense=dense,
                         counts=counts, perm=perm, n_dense=n_dense))
    for first in range(0, n, MAX_MAPS):
        batch = info[first:first + MAX_MAPS]
        descs = (KmapDesc * len(batch))()
        for d, m in zip(descs, batch):
            d.sources, d.targets = m["src"].data_ptr(), m["tgt"].data_ptr()
            d.num_sources, d.num_targets = m["S"], m["T"]
            d.kernel_size[:] = m["ks"]
            d.source_stride[:] = m["st"]
            d.layout = m["layout"]
            d.map, d.tile_counts = m["dense"].data_ptr(), m["counts"].data_ptr()
            d.row_perm = None if m["perm"] is None else m["perm"].data_ptr()
        _lib.call("spira_b200_kmap_search", descs, len(batch), kb, stream)

    hybrid_maps = [m for m in info if m["df"] >= 3]
    if hybrid_maps:
        _build_hybrid(hybrid_maps, dev, stream)

    # weight-stationary post-processing
    ws_maps = [m for m in info if m["layout"] == LAYOUT_WS and m["df"] < 3]
    for m in ws_maps:
        # submanifold map with an odd kernel volume: only the first (K+1)/2 rows are listed, the rest is applied by
        # symmetry (csrc/spira/torch/cuda_sparse_convolution_mapping.cu:269)
        m["half"] = (m["S"] == m["T"]) and (m["K"] % 2 == 1)
        m["rows"] = (m["K"] + 1) // 2 if m["half"] else m["K"]
    if ws_maps and not exact_sizes and all(m["Tal"] > 0 and m["T"] > 0 for m in ws_maps):
        # Nothing is read back: the lists get their worst-case capacity (rows * T pairs, allocated but never touched
        # beyond nnz), the kernels take the sizes from naddrs / qnaddrs on the device, and all maps share three launches.
        for first in range(0, len(ws_maps), MAX_MAPS):
            batch = ws_maps[first:first + MAX_MAPS]
            descs = (WsDesc * len(batch))()
            for d, m in zip(descs, batch):
                K, rows, nt = m["K"], m["rows"], m["Tal"] // 128
                small = torch.empty(K + 2 * (rows + 1) + 2, dtype=torch.int32, device=dev)
                m["nbsizes"], m["naddrs"] = small[:K], small[K:K + rows + 1]
                m["qnaddrs"], sizes = small[K + rows + 1:K + 2 * rows + 2], small[K + 2 * rows + 2:]
                m["tile_base"] = torch.empty((K, nt), dtype=torch.int32, device=dev)
                nbmaps = torch.empty((2, rows * m["T"]), dtype=torch.int32, device=dev)
                base = small.data_ptr()
                d.map_ws, d.tile_counts, d.aligned_targets = m["dense"].data_ptr(), m["counts"].data_ptr(), m["Tal"]
                d.K, d.rows = K, rows
                d.nbsizes, d.naddrs, d.qnaddrs, d.sizes = base, base + 4 * K, base + 4 * (K + rows + 1), base + 4 * (K + 2 * rows + 2)
                d.tile_base = m["tile_base"].data_ptr()
                d.in_idx, d.out_idx = nbmaps.data_ptr(), nbmaps.data_ptr() + 4 * rows * m["T"]
                w = WsLists()
                w.nbmaps, w.in_idx, w.out_idx = nbmaps, nbmaps[0], nbmaps[1]
                w.nbsizes, w.naddrs, w.qnaddrs = m["nbsizes"][:rows], m["naddrs"], m["qnaddrs"]
                w.rows, w.mirror, w.mapsize, w.qmapsize = rows, bool(m["half"]), None, None
                m["ws"] = w.set_pointers()
            _lib.call("spira_b200_kmap_ws_lists", descs, len(batch), stream)
    elif ws_maps:
        # sizes for every map, ONE host read of all list sizes (the reference reads them per map), then the pairs with
        # their exact shape [2, nnz]
        sizes = torch.empty((len(ws_maps), 2), dtype=torch.int32, device=dev)
        for j, m in enumerate(ws_maps):
            K, nt, rows = m["K"], m["Tal"] // 128, m["rows"]
            m["nbsizes"] = torch.empty(K, dtype=torch.int32, device=dev)
            m["naddrs"] = torch.empty(K + 1, dtype=torch.int32, device=dev)
            m["qnaddrs"] = torch.empty(K + 1, dtype=torch.int32, device=dev)
            m["tile_base"] = torch.empty((K, max(nt, 1)), dtype=torch.int32, device=dev)
            # tile_base / nbsizes are produced for all K rows (the mask format needs them); the
            # prefix sums below cover the `rows` rows the pair lists hold
            if nt > 0:
                if rows == K or m["df"] % 2 == 0:
                    _lib.call("spira_b200_kmap_ws_sizes", _ptr(m["counts"]), K, nt, _ptr(m["nbsizes"]), _ptr(m["naddrs"]),
                              _ptr(m["qnaddrs"]), _ptr(m["tile_base"]), _ptr(sizes[j]), stream)
                if rows != K:
                    _lib.call("spira_b200_kmap_ws_sizes", _ptr(m["counts"]), rows, nt, _ptr(m["nbsizes"]),
                              _ptr(m["naddrs"]), _ptr(m["qnaddrs"]), _ptr(m["tile_base"]), _ptr(sizes[j]), stream)
            else:
                m["nbsizes"].zero_(); m["naddrs"].zero_(); m["qnaddrs"].zero_(); sizes[j].zero_()
        host_sizes = sizes.cpu().tolist() if exact_sizes else None
        for j, m in enumerate(ws_maps):
            rows = m["rows"]
            if exact_sizes:
                mapsize, qmapsize = host_sizes[j]
                cap = mapsize
            else:
                mapsize = qmapsize = None
                cap = rows * m["T"]
            nbmaps = torch.empty((2, cap), dtype=torch.int32, device=dev)
            if cap > 0 and m["Tal"] > 0:
                _lib.call("spira_b200_kmap_ws_pairs", _ptr(m["dense"]), rows, m["Tal"], _ptr(m["naddrs"]),
                          _ptr(m["tile_base"]), _ptr(nbmaps[0]), _ptr(nbmaps[1]), stream)
            w = WsLists()
            w.nbmaps, w.in_idx, w.out_idx = nbmaps, nbmaps[0], nbmaps[1]
            w.nbsizes, w.naddrs, w.qnaddrs = m["nbsizes"][:rows], m["naddrs"][:rows + 1], m["qnaddrs"][:rows + 1]
            w.rows, w.mirror = rows, bool(m["half"])
            w.mapsize = None if mapsize is None else int(mapsize)
            w.qmapsize = None if qmapsize is None else int(qmapsize)
            m["ws"] = w.set_pointers()

    if group is True:       # False: the caller groups these maps together with others of its own; "lazy": on first use
        os_maps = [m for m in info if m["layout"] == LAYOUT_OS]
        for m, g in zip(os_maps, group_os_maps([(m["dense"], m["T"]) for m in os_maps])):
            m["grouped"] = g

    results = []
    for m in info:
        df, dense = m["df"], m["dense"]
        dense._sb = dict(counts=m["counts"], ws=m.get("ws"), kernel_size=m["ks"], layout=m["layout"], grouped=m.get("grouped"),
                         group_lazy=m["T"] if (group == "lazy" and m["layout"] == LAYOUT_OS) else None)
        if df >= 3:
            results.append(m["result"])
        elif df == 0:
            results.append((m["S"], m["T"], dense, None, None, None, None, None, None))
        elif df == 1:
            w = m["ws"]      # reachable from the dense map only: nothing in the lists points back (no reference cycle)
            results.append((m["S"], m["T"], dense, w.nbmaps, w.nbsizes, w.naddrs, w.qnaddrs, w.mapsize, w.qmapsize))
        else:
            w = m["ws"]
            K = m["K"]
            sm = torch.empty((K, m["S"]), dtype=torch.int32, device=dev)
            tm = torch.empty((K, m["T"]), dtype=torch.int32, device=dev)
            if m["half"]:
                # submanifold map with an odd kernel volume: the first (K+1)/2 rows are ranked, the others mirror them
                # (csrc/spira/cuda/functions/query_sorted_index.cu:516-640)
                _lib.call("spira_b200_kmap_masks_half", _ptr(dense), _ptr(m["tile_base"]), m["rows"], K, m["S"], m["T"], m["Tal"],
                          _ptr(sm), _ptr(tm), stream)
            else:
                _lib.call("spira_b200_kmap_masks", _ptr(dense), K, m["S"], m["T"], m["Tal"], _ptr(m["tile_base"]), _ptr(sm),
                          _ptr(tm), stream)
            results.append((m["S"], m["T"], dense, sm, tm, w.nbsizes, None, None, None))
    return results


def _build_maps_arena(voxel_pairs, kernel_sizes, source_strides, dataflows, group=True):
    """The network-wide builder's hot path (dataflows 0 and 1, nothing read back): every buffer of every map of the
    call lives in ONE int32 allocation; the kernels get addresses, tensor views are made only where a caller needs
    one (the dense map of every tuple; the list slots of a weight-stationary tuple on first access)."""
    n = len(voxel_pairs)
    dev = voxel_pairs[0][0].device
    kb = _key_bytes(voxel_pairs[0][0])
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    stream = _raw_stream(idx)
    metas, total = [], 0

    def take(ints):                       # offsets stay multiples of 64 ints (256 bytes)
        nonlocal total
        off = total
        total += (ints + 63) & ~63
        return off

    for i in range(n):
        src, tgt = voxel_pairs[i]
        ks, st, df = kernel_sizes[i], source_strides[i], dataflows[i]
        S, T = src.shape[0], tgt.shape[0]
        K = ks[0] * ks[1] * ks[2]
        Tal = (T + 127) & ~127
        nt = Tal >> 7
        m = [src, tgt, S, T, K, Tal, nt, ks, st, df, take(Tal * K), take(K * nt)]
        if df == 1:
            half = S == T and K % 2 == 1
            rows = (K + 1) // 2 if half else K
            # nbsizes [K], naddrs [rows + 1], qnaddrs [rows + 1], sizes [2]; tile_base [K][nt]; nbmaps [2][rows * T]
            m += [half, rows, take(K + 2 * (rows + 1) + 2), take(K * nt), take(2 * rows * T)]
        metas.append(m)
    arena = torch.empty(total, dtype=torch.int32, device=dev)
    base = arena.data_ptr()

    for first in range(0, n, MAX_MAPS):
        batch = metas[first:first + MAX_MAPS]
        descs = (KmapDesc * len(batch))()
        for d, m in zip(descs, batch):
            d.sources, d.targets, d.num_sources, d.num_targets = m[0].data_ptr(), m[1].data_ptr(), m[2], m[3]
            d.kernel_size[:] = m[7]
            d.source_stride[:] = m[8]
            d.layout = LAYOUT_OS if m[9] == 0 else LAYOUT_WS
            d.map, d.tile_counts = base + 4 * m[10], base + 4 * m[11]
        _lib.call("spira_b200_kmap_search", descs, len(batch), kb, stream)

    ws = [m for m in metas if m[9] == 1]
    for first in range(0, len(ws), MAX_MAPS):
        batch = ws[first:first + MAX_MAPS]
        descs = (WsDesc * len(batch))()
        for d, m in zip(descs, batch):
            K, T, rows, small = m[4], m[3], m[13], base + 4 * m[14]
            d.map_ws, d.tile_counts, d.aligned_targets, d.K, d.rows = base + 4 * m[10], base + 4 * m[11], m[5], K, rows
            d.nbsizes, d.naddrs, d.qnaddrs, d.sizes = small, small + 4 * K, small + 4 * (K + rows + 1), small + 4 * (K + 2 * rows + 2)
            d.tile_base = base + 4 * m[15]
            d.in_idx, d.out_idx = base + 4 * m[16], base + 4 * (m[16] + rows * T)
        _lib.call("spira_b200_kmap_ws_lists", descs, len(batch), stream)

    results, os_maps = [], []
    for m in metas:
        src, tgt, S, T, K, Tal, nt, ks, st, df, dense_off, counts_off = m[:12]
        if df == 0:
            dense = arena[dense_off:dense_off + Tal * K].view(Tal, K)
            dense._sb = dict(ws=None, kernel_size=ks, layout=LAYOUT_OS, grouped=None, _arena=arena, _counts=(counts_off, (K, nt)))
            os_maps.append((dense, T))
            results.append((S, T, dense, None, None, None, None, None, None))
        else:
            half, rows, small, tb_off, nb_off = m[12:]
            dense = arena[dense_off:dense_off + Tal * K].view(K, Tal)
            w = WsLists()
            w._arena = arena
            w._lazy = dict(nbmaps=(nb_off, (2, rows * T)), in_idx=(nb_off, (rows * T,)), out_idx=(nb_off + rows * T, (rows * T,)),
                           nbsizes=(small, (rows,)), naddrs=(small + K, (rows + 1,)), qnaddrs=(small + K + rows + 1, (rows + 1,)))
            w.in_ptr, w.out_ptr = base + 4 * nb_off, base + 4 * (nb_off + rows * T)
            w.naddrs_ptr, w.qnaddrs_ptr = base + 4 * (small + K), base + 4 * (small + K + rows + 1)
            w.rows, w.mirror, w.mapsize, w.qmapsize = rows, bool(half), None, None
            dense._sb = dict(ws=w, kernel_size=ks, layout=LAYOUT_WS, grouped=None, _arena=arena, _counts=(counts_off, (K, nt)))
            results.append(_WsTuple((S, T, dense, w)))
    if group and os_maps:
        for (dense, _), g in zip(os_maps, group_os_maps(os_maps)):
            dense._sb["grouped"] = g
    return results


def _build_hybrid(maps, dev, stream) -> None:
    """Post-processing of the hybrid dataflows 3-8 (``BinarySearch_Streamed_Hybrid_{WS,GS}``,
    csrc/spira/cuda/functions/query_sorted_index.cu:647-908, and the driver,
    csrc/spira/torch/cuda_sparse_convolution_mapping.cu:667-892).  The searched map has its rows in L1-norm order:
    ``dense`` leading rows for the output-stationary part, then ``K - dense`` rows of which the first half is compacted
    into pair lists (odd dataflows) or ranked into masks (even dataflows, both halves written by mirroring).  Dataflows
    above 4 return the leading rows as ``[T_al, dense]``; 3 and 4 (only the centre offset is dense) keep the whole map."""
    sizes = torch.empty((len(maps), 2), dtype=torch.int32, device=dev)
    for j, m in enumerate(maps):
        K, nt, nd = m["K"], m["Tal"] // 128, m["n_dense"]
        half = (K - nd) // 2
        m["half_rows"] = half
        m["nbsizes"] = torch.empty(max(half, 1), dtype=torch.int32, device=dev)[:half]
        m["naddrs"] = torch.zeros(half + 1, dtype=torch.int32, device=dev)
        m["qnaddrs"] = torch.zeros(half + 1, dtype=torch.int32, device=dev)
        m["tile_base"] = torch.empty((max(half, 1), max(nt, 1)), dtype=torch.int32, device=dev)
        if nt > 0 and half > 0:
            _lib.call("spira_b200_kmap_ws_sizes", m["counts"].data_ptr() + 4 * nd * nt, half, nt, _ptr(m["nbsizes"]),
                      _ptr(m["naddrs"]), _ptr(m["qnaddrs"]), _ptr(m["tile_base"]), _ptr(sizes[j]), stream)
        else:
            sizes[j].zero_()
    host_sizes = sizes.cpu().tolist()
    for j, m in enumerate(maps):
        K, nd, half, S, T, Tal, df, dense = m["K"], m["n_dense"], m["half_rows"], m["S"], m["T"], m["Tal"], m["df"], m["dense"]
        mapsize, qmapsize = host_sizes[j]
        rows_ptr = dense.data_ptr() + 4 * nd * Tal
        w = WsLists()
        nbmaps = torch.empty((2, mapsize), dtype=torch.int32, device=dev)
        if mapsize > 0:
            _lib.call("spira_b200_kmap_ws_pairs", rows_ptr, half, Tal, _ptr(m["naddrs"]), _ptr(m["tile_base"]), _ptr(nbmaps[0]),
                      _ptr(nbmaps[1]), stream)
        w.nbmaps, w.in_idx, w.out_idx = nbmaps, nbmaps[0], nbmaps[1]
        w.nbsizes, w.naddrs, w.qnaddrs = m["nbsizes"], m["naddrs"], m["qnaddrs"]
        w.rows, w.mirror, w.mapsize, w.qmapsize = half, True, int(mapsize), int(qmapsize)
        w.set_pointers()
        if df > 4:
            lead = torch.empty((Tal, nd), dtype=torch.int32, device=dev)
            if nd > 0 and Tal > 0:
                _lib.call("spira_b200_transpose_map", _ptr(dense), nd, Tal, _ptr(lead), stream)
            lead._sb = dict(layout=LAYOUT_OS, ws=None, grouped=None, counts=None, kernel_size=m["ks"])
            out_map = lead
        else:
            out_map = dense
        if df % 2 == 1:
            m["result"] = (S, T, out_map, w.nbmaps, w.nbsizes, w.naddrs, w.qnaddrs, w.mapsize, w.qmapsize)
        else:
            sm = torch.empty((K - nd, S), dtype=torch.int32, device=dev)
            tm = torch.empty((K - nd, T), dtype=torch.int32, device=dev)
            _lib.call("spira_b200_kmap_masks_half", rows_ptr, _ptr(m["tile_base"]), half, K - nd, S, T, Tal, _ptr(sm), _ptr(tm), stream)
            m["result"] = (S, T, out_map, sm, tm, w.nbsizes, None, None, None)


class _WsTuple(tuple):
    """The 9-slot result of a weight-stationary map whose list slots (3: nbmaps, 4: nbsizes, 5: naddrs, 6: qnaddrs) are
    views made when somebody reads them; slots 7 and 8 (the list sizes on the host) are None: nothing was read back."""

    def __new__(cls, head):
        return super().__new__(cls, (head[0], head[1], head[2], None, None, None, None, None, None))

    def __init__(self, head):
        self._lists = head[3]

    def __getitem__(self, i):
        if isinstance(i, int) and 3 <= (i if i >= 0 else i + 9) <= 6:
            w = self._lists
            return (w.nbmaps, w.nbsizes, w.naddrs, w.qnaddrs)[(i if i >= 0 else i + 9) - 3]
        if isinstance(i, slice):
            return tuple(self[j] for j in range(*i.indices(9)))
        return super().__getitem__(i)

    def __iter__(self):
        return (self[j] for j in range(9))


def map_counts(map_tensor: torch.Tensor) -> Optional[torch.Tensor]:
    """Hit counters ``[K, T_al / 128]`` of an engine-built map (``None`` for foreign maps)."""
    sb = getattr(map_tensor, "_sb", None)
    if sb is None:
        return None
    c = sb.get("counts")
    if c is None and sb.get("_counts") is not None:
        off, shape = sb["_counts"]
        c = sb["counts"] = sb["_arena"][off:off + shape[0] * shape[1]].view(shape)
    return c


def cuda_binary_search(sources, targets, kernel_size, source_stride, dataflow: int = 0):
    """One kernel map.  Reference: ``BinarySearch`` (csrc/spira/torch/cuda_sparse_convolution_mapping.cu:211-892)."""
    return _build_maps([(sources.contiguous(), targets.contiguous())], [kernel_size], [source_stride], [dataflow], group="lazy")[0]


def cuda_binary_search_streamed(voxels, kernel_sizes, source_strides, dataflow, exact_sizes=True):
    """All kernel maps of a network in one go; map ``i`` uses ``voxels[i // 2]`` as sources and
    ``voxels[(i + 1) // 2]`` as targets (csrc/spira/torch/cuda_sparse_convolution_mapping.cu:894-1645, :945-946)."""
    if not (len(kernel_sizes) == len(source_strides) == len(dataflow)):
        raise RuntimeError("[spira_b200] kernel_sizes, source_strides and dataflow must have the same length")
    voxels = [v.contiguous() for v in voxels]
    pairs = [(voxels[i // 2], voxels[(i + 1) // 2]) for i in range(len(kernel_sizes))]
    return _build_maps(pairs, kernel_sizes, source_strides, dataflow, exact_sizes, group="lazy")


def cuda_binary_search_pairs(voxel_pairs, kernel_sizes, source_strides, dataflow, exact_sizes=True, group=True):
    """Like :func:`cuda_binary_search_streamed` with the (sources, targets) pair of every map given explicitly.
    ``group=False`` leaves the output-stationary maps without their grouped twin (:func:`group_os_maps` adds it)."""
    if not (len(voxel_pairs) == len(kernel_sizes) == len(source_strides) == len(dataflow)):
        raise RuntimeError("[spira_b200] voxel_pairs, kernel_sizes, source_strides and dataflow must have the same length")
    pairs = [(a.contiguous(), b.contiguous()) for a, b in voxel_pairs]
    if not exact_sizes and _arena_path_applies(pairs, kernel_sizes, source_strides, dataflow):
        return _build_maps_arena(pairs, [tuple(int(v) for v in k) for k in kernel_sizes],
                                 [tuple(int(v) for v in t) for t in source_strides], [int(d) for d in dataflow], group)
    return _build_maps(pairs, kernel_sizes, source_strides, dataflow, exact_sizes, group)


def _arena_path_applies(pairs, kernel_sizes, source_strides, dataflow) -> bool:
    if not LAZY_SIZES or not pairs:
        return False
    dtype = pairs[0][0].dtype
    for (a, b), d in zip(pairs, dataflow):
        if d not in (0, 1) or not a.is_cuda or not b.is_cuda or a.dtype != dtype or b.dtype != dtype or a.dim() != 1 \
                or b.dim() != 1 or a.shape[0] == 0 or b.shape[0] == 0:
            return False
    return True


def cuda_binary_search_no_small_z(sources, targets, kernel_size, source_stride):
    """Ablation entry of the reference (full search for every offset, natural column order,
    csrc/spira/cuda/kernels/query_sorted.cuh:165-201): same result as the natural-order map, ``[T_al, K]``."""
    S, T, dense_ws, *_ = _build_maps([(sources.contiguous(), targets.contiguous())], [kernel_size], [source_stride], [1])[0]
    out = torch.empty((dense_ws.shape[1], dense_ws.shape[0]), dtype=torch.int32, device=dense_ws.device)
    _lib.call("spira_b200_transpose_map", _ptr(dense_ws), dense_ws.shape[0], dense_ws.shape[1], _ptr(out), _stream(out.device))
    return (S, T, out, None, None, None, None, None, None)


def transpose_map(m: torch.Tensor) -> torch.Tensor:
    """``m.T.contiguous()`` for an int32 map."""
    m = m.contiguous()
    out = torch.empty((m.shape[1], m.shape[0]), dtype=torch.int32, device=m.device)
    _lib.call("spira_b200_transpose_map", _ptr(m), m.shape[0], m.shape[1], _ptr(out), _stream(m.device))
    return out


def cuda_convert_transposed_os(out_in_map: torch.Tensor, num_sources: int) -> torch.Tensor:
    """Inverse of a ``[T_al, K]`` map: ``[S_al, K]`` (csrc/spira/torch/cuda_sparse_convolution_mapping.cu:1809-1830)."""
    _require_cuda(out_in_map)
    out_in_map = out_in_map.contiguous()
    Tal, K = out_in_map.shape
    Sal = _aligned(int(num_sources))
    out = torch.empty((Sal, K), dtype=torch.int32, device=out_in_map.device)
    _lib.call("spira_b200_convert_transposed_os", _ptr(out_in_map), Tal, K, _ptr(out), Sal, _stream(out.device))
    return out


# ------------------------------------------------------------------------------------------------
# feature compute
# ------------------------------------------------------------------------------------------------
def packed_weights(weights: torch.Tensor, mode: int) -> Optional[torch.Tensor]:
    """Tensor-core operand image of ``weights [K, c_in, c_out]``.

    The image is kept ON the weight tensor object (so it lives exactly as long as the tensor and can never be
    matched to a different tensor that happens to reuse the same address) and is rebuilt when the tensor's
    version counter or storage changes."""
    K, cin, cout = weights.shape
    if weights.dtype != torch.float16 or not _lib.load().spira_b200_tensor_core_eligible(K, cin, cout):
        return None
    stamp = (weights.data_ptr(), weights._version)
    store = getattr(weights, "_sb_packed", None)
    if store is None:
        store = {}
        weights._sb_packed = store
    hit = store.get(mode)
    if hit is not None and hit[0] == stamp:
        return hit[1]
    need = C.c_size_t()
    _lib.call("spira_b200_packed_weight_bytes", K, cin, cout, mode, C.byref(need))
    packed = torch.empty(need.value, dtype=torch.uint8, device=weights.device)
    _lib.call("spira_b200_pack_weights", _ptr(weights), K, cin, cout, mode, _ptr(packed), _stream(weights.device))
    store[mode] = (stamp, packed)
    return packed


def _epilogue(bias=None, scale=None, shift=None, residual=None, relu=False):
    if bias is None and scale is None and residual is None and not relu:
        return None, ()
    e = Epilogue()
    keep = []
    for name, t, dt in (("bias", bias, torch.float16), ("scale", scale, torch.float32), ("shift", shift, torch.float32),
                        ("residual", residual, torch.float16)):
        if t is not None:
            t = t.to(dt).contiguous()
            keep.append(t)
            setattr(e, name, t.data_ptr())
    e.relu = 1 if relu else 0
    return e, keep


def _check_feats(sources, weights):
    _require_cuda(sources, weights)
    if sources.dim() != 2:
        raise RuntimeError("[spira_b200] Tensor sources is expected to have 2 dimension(s)")
    if weights.dim() != 3:
        raise RuntimeError("[spira_b200] Tensor weights is expected to have 3 dimension(s)")
    if sources.shape[1] != weights.shape[1]:
        raise RuntimeError(f"[spira_b200] The dimension 1 of Tensor sources is expected to be {weights.shape[1]} but found {sources.shape[1]}")
    if sources.dtype != torch.float16 or weights.dtype != torch.float16:
        raise RuntimeError("[spira_b200] features and weights must be float16 (fp16 in/out, fp32 accumulate)")


def _check_second_source(sources, sources_b, weights):
    """Two-source form: the rows of ``sources`` and ``sources_b`` side by side are the input rows (a channel
    concatenation that is never materialised)."""
    _require_cuda(sources_b)
    if sources_b.dim() != 2 or sources_b.shape[0] != sources.shape[0] or sources_b.dtype != torch.float16:
        raise RuntimeError("[spira_b200] the second source must be float16 with the rows of the first")
    if sources.shape[1] + sources_b.shape[1] != weights.shape[1]:
        raise RuntimeError(f"[spira_b200] the sources hold {sources.shape[1]} + {sources_b.shape[1]} channels, the weights expect {weights.shape[1]}")
    if sources.shape[1] % 8 != 0 or sources_b.shape[1] % 8 != 0:
        raise RuntimeError("[spira_b200] both sources of a two-source convolution need a multiple of 8 channels")


def conv_desc_call(desc: "_lib.ConvDesc", device) -> None:
    """``spira_b200_conv`` on the current stream of ``device``."""
    _lib.call("spira_b200_conv", C.byref(desc), _ptr(status_word(device)), _stream(device))


def conv_identity(sources, weights, *, sources_b=None, bias=None, scale=None, shift=None, residual=None, relu=False) -> torch.Tensor:
    """1x1x1 layer ``[sources | sources_b] @ weights[0]`` with the fused epilogue, on the tensor-core output-stationary
    kernel through the identity map (no map tensor).  ``weights`` is ``[1, c_in, c_out]``."""
    if sources_b is None:
        _check_feats(sources, weights)
    else:
        _require_cuda(sources, weights)
        _check_second_source(sources, sources_b, weights)
        sources_b = sources_b.contiguous()
    sources, weights = sources.contiguous(), weights.contiguous()
    K, cin, cout = weights.shape
    if K != 1:
        raise RuntimeError("[spira_b200] conv_identity is for 1x1x1 layers")
    packed = packed_weights(weights, PACK_OS)
    if packed is None:
        raise RuntimeError(f"[spira_b200] a 1x1x1 layer {cin} -> {cout} is outside the tensor-core kernels")
    n = sources.shape[0]
    out = torch.empty((n, cout), dtype=torch.float16, device=sources.device)
    ep, keep = _epilogue(bias, scale, shift, residual, relu)
    d = _lib.ConvDesc(dataflow=0, K=1, c_in=cin, c_out=cout, c_in_a=sources.shape[1], num_sources=n, num_targets=n,
                      feats=_ptr(sources), feats_b=_ptr(sources_b), packed=_ptr(packed), out=_ptr(out))
    if ep is not None:
        d.epilogue = C.pointer(ep)
    conv_desc_call(d, sources.device)
    return out


def conv_os(num_sources, num_targets, out_in_map, sources, weights, *, bias=None, scale=None, shift=None, residual=None,
            relu=False, force_simt=False, grouped=True, splits=None, sources_b=None) -> torch.Tensor:
    """Output-stationary forward with the optional fused epilogue.  An engine-built map that carries a grouped twin
    (rows sorted by neighbour pattern) runs over the twin unless ``grouped=False``; the result is the same.
    ``splits`` (2, 4 or 8; default: ``os_splits`` decides) shares the reduction of every tile among that many CTAs; the
    fp32 partial sums are added in a fixed order, so the result is deterministic but rounds differently from one CTA's.
    ``sources_b``: second source tensor, see :func:`conv_ws`."""
    if sources_b is None:
        _check_feats(sources, weights)
    else:
        _require_cuda(sources, weights)
        _check_second_source(sources, sources_b, weights)
        sources_b = sources_b.contiguous()
    sources, weights, out_in_map = sources.contiguous(), weights.contiguous(), out_in_map.contiguous()
    K, cin, cout = weights.shape
    if out_in_map.dim() != 2 or out_in_map.shape[1] != K or out_in_map.shape[0] < num_targets:
        raise RuntimeError(f"[spira_b200] out_in_map must be [T_al, {K}] with T_al >= {num_targets}, got {tuple(out_in_map.shape)}")
    out = torch.empty((num_targets, cout), dtype=torch.float16, device=sources.device)
    if out_in_map.shape[0] != _aligned(num_targets):
        # the kernels read whole 128-row tiles of the map: bring a short map to T_al rows
        padded = torch.full((_aligned(num_targets), K), -1, dtype=torch.int32, device=out_in_map.device)
        padded[:num_targets] = out_in_map[:num_targets]
        out_in_map = padded
    packed = None if force_simt else packed_weights(weights, _lib.load().spira_b200_get_option(b"os_pack_mode"))
    ep, keep = _epilogue(bias, scale, shift, residual, relu)
    g = grouped_twin(out_in_map) if (grouped and GROUP_OS and (packed is not None or _stem_shape(cin, cout, K))) else None
    if splits is None:
        splits = os_splits(num_targets, K, cin, cout) if packed is not None else 1
    if sources_b is not None:
        if packed is None:
            raise RuntimeError(f"[spira_b200] two sources need a layer the tensor-core kernels take (K={K}, {cin} -> {cout})")
        d = _lib.ConvDesc(dataflow=0, K=K, c_in=cin, c_out=cout, c_in_a=sources.shape[1], splits=int(splits),
                          num_sources=int(num_sources), num_targets=int(num_targets), feats=_ptr(sources), feats_b=_ptr(sources_b),
                          packed=_ptr(packed), out=_ptr(out))
        if g is not None:
            d.map_os, d.row_of, d.tile_masks = g.map_ptr, g.row_of_ptr, g.tile_masks_ptr
        else:
            d.map_os = _ptr(out_in_map)
        if splits > 1:
            scratch = split_scratch(sources.device, 1024 + _aligned(num_targets) * splits * cout * 4)
            d.split_scratch, d.split_scratch_bytes = _ptr(scratch), scratch.numel()
        if ep is not None:
            d.epilogue = C.pointer(ep)
        conv_desc_call(d, sources.device)
        return out
    if splits > 1:
        scratch = split_scratch(sources.device, 1024 + _aligned(num_targets) * splits * cout * 4)
        _lib.call("spira_b200_conv_os_split", _ptr(sources), _ptr(packed), C.byref(ep) if ep is not None else None,
                  g.map_ptr if g is not None else _ptr(out_in_map), g.row_of_ptr if g is not None else None,
                  g.tile_masks_ptr if g is not None else None, int(num_sources), int(num_targets), K, cin, cout, int(splits),
                  _ptr(scratch), scratch.numel(), _ptr(out), _ptr(status_word(sources.device)), _stream(sources.device))
        return out
    if g is not None:
        _lib.call("spira_b200_conv_os_grouped", _ptr(sources), _ptr(weights), _ptr(packed), C.byref(ep) if ep is not None else None, g.map_ptr,
                  g.row_of_ptr, g.tile_masks_ptr, int(num_sources), int(num_targets), K, cin, cout, _ptr(out),
                  _ptr(status_word(sources.device)), _stream(sources.device))
        return out
    _lib.call("spira_b200_conv_os", _ptr(sources), _ptr(weights), _ptr(packed), C.byref(ep) if ep is not None else None,
              _ptr(out_in_map), int(num_sources), int(num_targets), K, cin, cout, _ptr(out), _ptr(status_word(sources.device)),
              _stream(sources.device))
    return out


def conv_ws(num_sources, num_targets, sources, weights, lists: WsLists, *, swap=False, bias=None, scale=None, shift=None,
            residual=None, relu=False, force_simt=False, fused=None, sources_b=None) -> torch.Tensor:
    """Weight-stationary forward over compacted pair lists with the optional fused epilogue.  ``fused`` (default:
    ``WS_FUSED`` where it applies) selects the single cooperative launch over the persistent zero scratch; the sums are
    the same (the order of the fp32 reductions varies from run to run on either path).
    ``sources_b``: a second source tensor with the rows of ``sources``; the layer then convolves the channel
    concatenation ``[sources | sources_b]`` without building it (the reference concatenates first:
    ``spira/operators.py:11-13``).  Tensor-core eligible layers only, fused call only."""
    if sources_b is None:
        _check_feats(sources, weights)
    else:
        _require_cuda(sources, weights)
        _check_second_source(sources, sources_b, weights)
        sources_b = sources_b.contiguous()
    sources, weights = sources.contiguous(), weights.contiguous()
    K, cin, cout = weights.shape
    out = torch.empty((num_targets, cout), dtype=torch.float16, device=sources.device)
    packed = None if force_simt else packed_weights(weights, PACK_WS)
    mirror = bool(lists.mirror)
    if mirror and swap:
        raise RuntimeError("[spira_b200] a mirrored (submanifold) list cannot be used transposed")
    ep, keep = _epilogue(bias, scale, shift, residual, relu)
    n_tiles = -1 if lists.qmapsize is None else lists.qmapsize // 128
    can_fuse = packed is not None and num_targets > 0 and get_option("gather_tma") == 0
    if fused is None:
        fused = WS_FUSED
    if sources_b is not None:
        if not can_fuse:
            raise RuntimeError(f"[spira_b200] two sources need a layer the tensor-core kernels take (K={K}, {cin} -> {cout})")
        accum = zero_scratch(sources.device, num_targets * cout)
        d = _lib.ConvDesc(dataflow=1, K=K, c_in=cin, c_out=cout, c_in_a=sources.shape[1], rows=lists.rows, mirror=1 if mirror else 0,
                          swap=1 if swap else 0, num_sources=int(num_sources), num_targets=int(num_targets), num_tiles128=n_tiles,
                          feats=_ptr(sources), feats_b=_ptr(sources_b), packed=_ptr(packed), in_idx=lists.in_ptr, out_idx=lists.out_ptr,
                          naddrs=lists.naddrs_ptr, qnaddrs=lists.qnaddrs_ptr, zeroed_accum=_ptr(accum), out=_ptr(out))
        if ep is not None:
            d.epilogue = C.pointer(ep)
        conv_desc_call(d, sources.device)
        return out
    if fused and can_fuse:
        accum = zero_scratch(sources.device, num_targets * cout)
        _lib.call("spira_b200_conv_ws_fused", _ptr(sources), _ptr(packed), C.byref(ep) if ep is not None else None,
                  lists.in_ptr, lists.out_ptr, lists.naddrs_ptr, lists.qnaddrs_ptr, lists.rows, n_tiles,
                  1 if mirror else 0, 1 if swap else 0, int(num_sources), int(num_targets), K, cin, cout, _ptr(accum), _ptr(out),
                  _ptr(status_word(sources.device)), _stream(sources.device))
        return out
    accum = torch.empty((num_targets, cout), dtype=torch.float32, device=sources.device)
    _lib.call("spira_b200_conv_ws", _ptr(sources), _ptr(weights), _ptr(packed), C.byref(ep) if ep is not None else None,
              lists.in_ptr, lists.out_ptr, lists.naddrs_ptr, lists.qnaddrs_ptr, lists.rows, n_tiles,
              1 if mirror else 0, 1 if swap else 0, int(num_sources), int(num_targets), K, cin, cout,
              _ptr(accum), _ptr(out), _ptr(status_word(sources.device)), _stream(sources.device))
    return out


# ---- prepared per-layer calls: the hot path of a network forward ----------------------------------------------------
_raw_stream = torch._C._cuda_getCurrentRawStream     # (device index) -> cudaStream_t as int, no Python object churn


def _no_call():
    return None


def _stem_shape(cin: int, cout: int, K: int) -> bool:
    """Narrow-input layers (network stems) that the one-thread-per-row kernel covers, also on grouped maps."""
    return cin <= 8 and cout in (16, 32, 64) and K * cin * cout * 4 + 128 * (2 if cout <= 32 else 1) * K * 4 <= 96 * 1024


class ConvCall:
    """Everything about one layer that does not change between forwards: the packed weight images, the epilogue
    struct, the resolved C functions.  ``SparseConv`` keeps one and the two ``run_*`` functions below add only the
    per-call pointers, so that a forward costs a few microseconds of Python per layer."""
    __slots__ = ("stamp", "weights", "K", "cin", "cout", "w_ptr", "packed", "ep", "ep_ref", "keep", "dev_index", "status",
                 "status_ptr", "fn_os", "fn_ws", "fn_os_grouped", "fn_ws_fused", "fn_os_split", "eligible", "stem")

    def __init__(self, weights: torch.Tensor, bias, fused):
        lib = _lib.load()
        if weights.dtype != torch.float16 or not weights.is_cuda or not weights.is_contiguous():
            raise RuntimeError("[spira_b200] layer weights must be contiguous float16 CUDA tensors")
        self.weights = weights
        self.K, self.cin, self.cout = weights.shape
        self.w_ptr = weights.data_ptr()
        self.eligible = bool(lib.spira_b200_tensor_core_eligible(self.K, self.cin, self.cout))
        self.stem = not self.eligible and _stem_shape(self.cin, self.cout, self.K)
        self.packed = {}
        scale = shift = None
        relu = False
        if fused is not None:
            scale, shift, relu = fused["scale"], fused["shift"], fused["relu"]
        self.ep, self.keep = _epilogue(bias, scale, shift, None, relu)
        if self.ep is None:
            self.ep = Epilogue()
        self.ep_ref = C.byref(self.ep)
        self.dev_index = weights.device.index
        self.status = status_word(weights.device)
        self.status_ptr = self.status.data_ptr()
        self.fn_os, self.fn_ws, self.fn_os_grouped = lib.spira_b200_conv_os, lib.spira_b200_conv_ws, lib.spira_b200_conv_os_grouped
        self.fn_ws_fused = lib.spira_b200_conv_ws_fused
        self.fn_os_split = lib.spira_b200_conv_os_split
        self.stamp = (weights.data_ptr(), weights._version, None if bias is None else (bias.data_ptr(), bias._version),
                      None if fused is None else (id(fused["scale"]), id(fused["shift"]), fused["relu"]))

    # a prepared call holds raw pointers: copies and pickles of a layer start without one and rebuild it lazily
    def __deepcopy__(self, memo):
        return None

    def __reduce__(self):
        return (_no_call, ())

    def packed_ptr(self, mode: int):
        if not self.eligible:
            return None
        p = self.packed.get(mode)
        if p is None:
            p = packed_weights(self.weights, mode)
            self.packed[mode] = p
        return p.data_ptr()


def conv_call_stamp(weights, bias, fused):
    return (weights.data_ptr(), weights._version, None if bias is None else (bias.data_ptr(), bias._version),
            None if fused is None else (id(fused["scale"]), id(fused["shift"]), fused["relu"]))


_pack_mode = [-1]       # SPIRA_B200_PACK_* image the output-stationary entry point expects (-1: ask the library)


def run_conv_os(call: ConvCall, num_sources: int, num_targets: int, out_in_map: torch.Tensor, feats: torch.Tensor,
                residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Output-stationary forward of a prepared layer.  ``out_in_map`` is an engine-built ``[T_al, K]`` map."""
    if not feats.is_contiguous():
        feats = feats.contiguous()
    out = torch.empty((num_targets, call.cout), dtype=torch.float16, device=feats.device)
    call.ep.residual = residual.data_ptr() if residual is not None else None
    sb = getattr(out_in_map, "_sb", None)
    g = None
    if sb is not None and (call.eligible or call.stem) and GROUP_OS:
        g = sb.get("grouped")
        if g is None and sb.get("group_lazy") is not None:
            g = grouped_twin(out_in_map)
    mode = _pack_mode[0]
    if mode < 0:
        mode = _pack_mode[0] = _lib.load().spira_b200_get_option(b"os_pack_mode")
    splits = os_splits(num_targets, call.K, call.cin, call.cout) if (call.eligible and mode == PACK_OS) else 1
    if splits > 1:
        scratch = split_scratch(feats.device, 1024 + _aligned(num_targets) * splits * call.cout * 4)
        name, fn = "spira_b200_conv_os_split", call.fn_os_split
        args = (feats.data_ptr(), call.packed_ptr(mode), call.ep_ref, g.map_ptr if g is not None else out_in_map.data_ptr(),
                g.row_of_ptr if g is not None else None, g.tile_masks_ptr if g is not None else None, num_sources, num_targets,
                call.K, call.cin, call.cout, splits, scratch.data_ptr(), scratch.numel(), out.data_ptr(), call.status_ptr,
                _raw_stream(call.dev_index))
    elif g is not None:
        name, fn = "spira_b200_conv_os_grouped", call.fn_os_grouped
        args = (feats.data_ptr(), call.w_ptr, call.packed_ptr(mode), call.ep_ref, g.map_ptr, g.row_of_ptr, g.tile_masks_ptr,
                num_sources, num_targets, call.K, call.cin, call.cout, out.data_ptr(), call.status_ptr,
                _raw_stream(call.dev_index))
    else:
        name, fn = "spira_b200_conv_os", call.fn_os
        args = (feats.data_ptr(), call.w_ptr, call.packed_ptr(mode), call.ep_ref, out_in_map.data_ptr(), num_sources,
                num_targets, call.K, call.cin, call.cout, out.data_ptr(), call.status_ptr, _raw_stream(call.dev_index))
    if _lib.profile_hook is not None:
        _lib.profile_hook(name, args, lambda: _lib.check(fn(*args)))
    else:
        rc = fn(*args)
        if rc != 0:
            _lib.check(rc)
    _lib.launch_count += 1
    return out


POINTWISE_HEAD = True   # 1x1x1 layers with at most 32 output channels run the engine's own kernel


def pointwise(feats: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    """``feats @ weight (+ bias)`` for a 1x1x1 layer with few output channels (``weight`` ``[c_in, c_out]``), or ``None``
    when the layer is outside what ``spira_b200_pointwise`` takes (the caller then uses the library GEMM, like the
    reference: spira/nn/conv.py:312-316)."""
    c_in, c_out = weight.shape
    if not POINTWISE_HEAD or c_out > 32 or c_in % 8 != 0 or c_in < 8 or c_in > 512 or not feats.is_cuda \
            or feats.dtype != torch.float16 or weight.dtype != torch.float16 or (bias is not None and bias.dtype != torch.float16):
        return None
    if not feats.is_contiguous():
        feats = feats.contiguous()
    if not weight.is_contiguous():
        weight = weight.contiguous()
    n = feats.shape[0]
    out = torch.empty((n, c_out), dtype=torch.float16, device=feats.device)
    idx = feats.device.index if feats.device.index is not None else torch.cuda.current_device()
    args = (feats.data_ptr(), weight.data_ptr(), bias.data_ptr() if bias is not None else None, n, c_in, c_out,
            out.data_ptr(), _raw_stream(idx))
    fn = _lib.load().spira_b200_pointwise
    if _lib.profile_hook is not None:
        _lib.profile_hook("spira_b200_pointwise", args, lambda: _lib.check(fn(*args)))
    else:
        rc = fn(*args)
        if rc != 0:
            _lib.check(rc)
    _lib.launch_count += 1
    return out


_zero_scratch = {}      # device index -> fp32 tensor that holds zeros whenever no weight-stationary call is in flight
_split_scratch = {}     # device index -> byte tensor of the split output-stationary calls (head: tile counters, zero when idle)
# Opt-in: output-stationary layers of at most ~4700 targets share every tile's reduction among 4 or 8 CTAs.  Measured on
# a 1961-voxel level (3x3x3, 256 -> 256): 57 us unsplit, 23 us with 8 CTAs per tile, 19.5 us for the fused weight-stationary
# call that the selector picks there anyway -- so the split only pays where a run is pinned to dataflow 0.
OS_SPLIT = False
_split_plans = {}


def os_split_plan(num_targets: int, K: int, cin: int, cout: int):
    """``(largest split count the library takes for this layer, scratch bytes it needs at that count)``; ``(1, 0)``
    when the layer cannot be split (too many tiles for the SMs, too narrow, not tensor-core eligible)."""
    key = (_aligned(num_targets), K, cin, cout)
    plan = _split_plans.get(key)
    if plan is None:
        n, b = C.c_int(0), C.c_size_t(0)
        _lib.call("spira_b200_conv_os_split_plan", int(num_targets), K, cin, cout, C.byref(n), C.byref(b))
        plan = _split_plans[key] = (int(n.value), int(b.value))
    return plan


def os_splits(num_targets: int, K: int, cin: int, cout: int) -> int:
    """Split count the output-stationary call uses for this layer (1: one CTA per tile)."""
    if not OS_SPLIT or num_targets <= 0:
        return 1
    limit = os_split_plan(num_targets, K, cin, cout)[0]
    return limit if limit >= 4 else 1      # (two CTAs per tile measured within 10 % of one)


def split_scratch(device, nbytes: int) -> torch.Tensor:
    """Persistent scratch of the split output-stationary call.  Its first 1024 bytes are tile counters that every call
    leaves at zero; it grows (a new zero-filled tensor) when a layer needs more; calls on one device are stream-ordered."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _split_scratch.get(idx)
    if t is None or t.numel() < nbytes:
        t = _split_scratch[idx] = torch.zeros(max(nbytes + nbytes // 2, 1 << 22), dtype=torch.uint8, device=device)
    return t



def zero_scratch(device, floats: int) -> torch.Tensor:
    """Persistent scratch of the fused weight-stationary call: zero on entry, zero again on completion.  It grows
    (a new zero-filled tensor) when a layer needs more; calls on one device are stream-ordered."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _zero_scratch.get(idx)
    if t is None or t.numel() < floats:
        t = _zero_scratch[idx] = torch.zeros(max(floats + floats // 2, 1 << 20), dtype=torch.float32, device=device)
    return t


def run_conv_ws(call: ConvCall, num_sources: int, num_targets: int, lists: WsLists, feats: torch.Tensor, swap: bool,
                residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Weight-stationary forward of a prepared layer over the engine's pair lists."""
    if not feats.is_contiguous():
        feats = feats.contiguous()
    if lists.mirror and swap:
        raise RuntimeError("[spira_b200] a mirrored (submanifold) list cannot be used transposed")
    out = torch.empty((num_targets, call.cout), dtype=torch.float16, device=feats.device)
    call.ep.residual = residual.data_ptr() if residual is not None else None
    n_tiles = -1 if lists.qmapsize is None else lists.qmapsize // 128
    mode = _pack_mode[0]
    if mode < 0:
        mode = _pack_mode[0] = _lib.load().spira_b200_get_option(b"os_pack_mode")
    if WS_FUSED and call.eligible and num_targets > 0 and mode == PACK_OS:      # (PACK_OS: the cp.async producers are in use)
        accum = zero_scratch(feats.device, num_targets * call.cout)
        name, fn, launches = "spira_b200_conv_ws_fused", call.fn_ws_fused, 1
        args = (feats.data_ptr(), call.packed_ptr(PACK_WS), call.ep_ref, lists.in_ptr, lists.out_ptr,
                lists.naddrs_ptr, lists.qnaddrs_ptr, lists.rows, n_tiles, 1 if lists.mirror else 0,
                1 if swap else 0, num_sources, num_targets, call.K, call.cin, call.cout, accum.data_ptr(), out.data_ptr(),
                call.status_ptr, _raw_stream(call.dev_index))
    else:
        accum = torch.empty((num_targets, call.cout), dtype=torch.float32, device=feats.device)
        name, fn, launches = "spira_b200_conv_ws", call.fn_ws, 2
        args = (feats.data_ptr(), call.w_ptr, call.packed_ptr(PACK_WS), call.ep_ref, lists.in_ptr,
                lists.out_ptr, lists.naddrs_ptr, lists.qnaddrs_ptr, lists.rows, n_tiles,
                1 if lists.mirror else 0, 1 if swap else 0, num_sources, num_targets, call.K, call.cin, call.cout,
                accum.data_ptr(), out.data_ptr(), call.status_ptr, _raw_stream(call.dev_index))
    if _lib.profile_hook is not None:
        _lib.profile_hook(name, args, lambda: _lib.check(fn(*args)))
    else:
        rc = fn(*args)
        if rc != 0:
            _lib.check(rc)
    _lib.launch_count += launches
    return out


def cuda_sparse_convolution_forward_os(num_sources, num_targets, out_in_map, sources, weights):
    """Reference: ``cuda_sparse_convolution_forward_os`` (csrc/spira/torch/cuda_sparse_convolution_forward.cu:11-80)."""
    return conv_os(num_sources, num_targets, out_in_map, sources, weights)


def _lists_from_reference_slots(naddrs, qnaddrs, nbmaps, mapsize, qmapsize, num_sources, num_targets, K, mirror=None) -> WsLists:
    w = WsLists()
    nbmaps = nbmaps.contiguous()
    w.nbmaps, w.in_idx, w.out_idx = nbmaps, nbmaps[0], nbmaps[1]
    w.naddrs, w.qnaddrs = naddrs.contiguous(), qnaddrs.contiguous()
    w.rows = naddrs.shape[0] - 1
    w.nbsizes = None
    if mirror is None:
        mirror = (w.rows == (K + 1) // 2) and K % 2 == 1 and num_sources == num_targets and w.rows != K
    w.mirror = bool(mirror)
    w.mapsize, w.qmapsize = int(mapsize), int(qmapsize)
    return w.set_pointers()


def cuda_sparse_convolution_forward_ws_merged(num_sources, num_targets, sources, weights, naddrs, qnaddrs, nbmaps, mapsize,
                                              qmapsize, transpose=False):
    """Reference: ``cuda_sparse_convolution_forward_ws_merged`` (csrc/spira/torch/cuda_sparse_convolution_forward.cu:183-246)."""
    K = weights.shape[0]
    lists = _lists_from_reference_slots(naddrs, qnaddrs, nbmaps, mapsize, qmapsize, num_sources, num_targets, K)
    return conv_ws(num_sources, num_targets, sources, weights, lists, swap=bool(transpose))


def lists_from_masks(source_masks: torch.Tensor, target_masks: torch.Tensor, kernel_map_sizes: torch.Tensor) -> WsLists:
    """Pair lists of ALL mask rows from the mask format alone: ``source_masks [Km, S]``, ``target_masks [Km, T]`` and
    the list sizes of all rows or of the first half of a mirrored map, whoever built them.  Nothing is read back: the
    lists get the capacity ``Km * min(S, T)`` and the kernels read their sizes on the device.  The result is kept on
    the mask tensor, so later forwards on the same map reuse it."""
    cached = getattr(source_masks, "_sb_lists", None)
    if cached is not None and cached[0] is target_masks and cached[1] == (source_masks._version, target_masks._version):
        return cached[2]
    _require_cuda(source_masks, target_masks, kernel_map_sizes)
    if source_masks.dim() != 2 or target_masks.dim() != 2 or source_masks.shape[0] != target_masks.shape[0]:
        raise RuntimeError("[spira_b200] source_masks and target_masks must be [K, S] and [K, T]")
    if source_masks.dtype != torch.int32 or target_masks.dtype != torch.int32 or kernel_map_sizes.dtype != torch.int32:
        raise RuntimeError("[spira_b200] masks and kernel_map_sizes must be int32")
    sm, tm, sizes = source_masks.contiguous(), target_masks.contiguous(), kernel_map_sizes.contiguous()
    Km, S = sm.shape
    T = tm.shape[1]
    n = sizes.shape[0]
    if n != Km and n != (Km + 1) // 2:
        raise RuntimeError(f"[spira_b200] kernel_map_sizes has {n} entries for {Km} mask rows (expected all rows or their first half)")
    dev = sm.device
    small = torch.empty(2 * (Km + 1), dtype=torch.int32, device=dev)
    nbmaps = torch.empty((2, max(Km * min(S, T), 1)), dtype=torch.int32, device=dev)
    w = WsLists()
    w.nbmaps, w.in_idx, w.out_idx = nbmaps, nbmaps[0], nbmaps[1]
    w.naddrs, w.qnaddrs, w.nbsizes = small[:Km + 1], small[Km + 1:], None
    w.rows, w.mirror, w.mapsize, w.qmapsize = Km, False, None, None
    w.set_pointers()
    _lib.call("spira_b200_kmap_lists_from_masks", _ptr(sm), _ptr(tm), _ptr(sizes), n, Km, S, T, w.naddrs_ptr, w.qnaddrs_ptr,
              w.in_ptr, w.out_ptr, _stream(dev))
    w._keep = (sm, tm, sizes)
    try:
        source_masks._sb_lists = (target_masks, (source_masks._version, target_masks._version), w)
    except Exception:
        pass
    return w


def cuda_sparse_convolution_forward_ws(num_sources, num_targets, gather_tile_size, scatter_tile_size, parallel, threshold,
                                       sources, weights, source_masks, target_masks, kernel_map_sizes):
    """Mask-format weight-stationary call (csrc/spira/torch/cuda_sparse_convolution_forward.cu:82-181,
    csrc/spira/cuda/functions/sparse_convolution.cu:1002-1124).  The pair lists are derived from the masks themselves
    (:func:`lists_from_masks`), so masks from any builder work; the masks of a transposed layer arrive exchanged
    (spira/nn/conv.py:353-360) and yield the exchanged lists.  The tile sizes, GEMM parallelism and padding threshold
    tune the reference's gather / cuBLAS / scatter pipeline and have no counterpart in the fused kernel; they are
    accepted and ignored."""
    if source_masks.shape[1] != num_sources or target_masks.shape[1] != num_targets:
        raise RuntimeError(f"[spira_b200] masks of shape {tuple(source_masks.shape)} / {tuple(target_masks.shape)} do not match "
                           f"{num_sources} sources and {num_targets} targets")
    if weights.shape[0] != source_masks.shape[0]:
        raise RuntimeError(f"[spira_b200] The dimension 0 of Tensor weights is expected to be {source_masks.shape[0]} but found {weights.shape[0]}")
    lists = lists_from_masks(source_masks, target_masks, kernel_map_sizes)
    return conv_ws(num_sources, num_targets, sources, weights, lists)


def _identity_map(n: int, device) -> torch.Tensor:
    """``[T_al, 1]`` output-stationary map of the centre offset of a submanifold layer: every voxel is its own neighbour."""
    m = torch.full((_aligned(n), 1), -1, dtype=torch.int32, device=device)
    m[:n, 0] = torch.arange(n, dtype=torch.int32, device=device)
    return m


def _hybrid_dense_part(num_sources, num_targets, sources, weights, out_in_map):
    """Output-stationary part of a hybrid call: the leading ``K_os`` weights over ``out_in_map [T_al, K_os]``, or -- no
    map given -- the centre offset alone, a plain matrix product in the reference
    (csrc/spira/cuda/functions/sparse_convolution.cu:1368-1380)."""
    if out_in_map is None:
        if num_sources != num_targets:
            raise RuntimeError("[spira_b200] a hybrid call without out_in_map is the centre offset of a submanifold layer")
        out_in_map = _identity_map(num_targets, sources.device)
    k_os = out_in_map.shape[1]
    return k_os, conv_os(num_sources, num_targets, out_in_map, sources, weights[:k_os].contiguous())


def cuda_sparse_convolution_forward_hs_merged(num_sources, num_targets, sources, weights, naddrs, qnaddrs, nbmaps, out_in_map,
                                              mapsize, qmapsize, transpose=False):
    """Hybrid call of the reference (csrc/spira/torch/cuda_sparse_convolution_forward.cu:338-420,
    csrc/spira/cuda/functions/sparse_convolution.cu:1299-1350): the leading ``K_os`` weights (L1-norm order,
    scripts/models/convert_weights.py:30-55) run output-stationary over ``out_in_map``, the remaining ``2 * rows`` weights
    weight-stationary over the half-compacted, mirrored pair lists, and the two parts are summed -- here in fp32 on top
    of the rounded output-stationary part."""
    _check_feats(sources, weights)
    rows = naddrs.shape[0] - 1
    k_os, dense_part = _hybrid_dense_part(num_sources, num_targets, sources, weights, out_in_map)
    if weights.shape[0] != k_os + 2 * rows:
        raise RuntimeError(f"[spira_b200] The dimension 0 of Tensor weights is expected to be {k_os + 2 * rows} but found {weights.shape[0]}")
    if rows == 0:
        return dense_part
    lists = _lists_from_reference_slots(naddrs, qnaddrs, nbmaps, mapsize, qmapsize, num_sources, num_targets, 2 * rows, mirror=True)
    return conv_ws(num_sources, num_targets, sources, weights[k_os:].contiguous(), lists, swap=bool(transpose), residual=dense_part)


def cuda_sparse_convolution_forward_hs(num_sources, num_targets, gather_tile_size, scatter_tile_size, parallel, threshold,
                                       sources, weights, source_masks, target_masks, kernel_map_sizes, out_in_map):
    """Hybrid mask-format call (csrc/spira/torch/cuda_sparse_convolution_forward.cu:248-336): like
    :func:`cuda_sparse_convolution_forward_hs_merged` with the weight-stationary part given as masks over
    ``K - K_os`` rows (both halves present, sizes for the first half)."""
    _check_feats(sources, weights)
    k_os, dense_part = _hybrid_dense_part(num_sources, num_targets, sources, weights, out_in_map)
    k_ws = target_masks.shape[0]
    if weights.shape[0] != k_os + k_ws or source_masks.shape[0] != k_ws:
        raise RuntimeError(f"[spira_b200] The dimension 0 of Tensor weights is expected to be {k_os + k_ws} but found {weights.shape[0]}")
    if k_ws == 0:
        return dense_part
    lists = lists_from_masks(source_masks, target_masks, kernel_map_sizes)
    return conv_ws(num_sources, num_targets, sources, weights[k_os:].contiguous(), lists, residual=dense_part)


def _time_ws(weights, source_masks, target_masks, kernel_map_sizes) -> float:
    S, T = source_masks.shape[1], target_masks.shape[1]
    lists = lists_from_masks(source_masks, target_masks, kernel_map_sizes)
    w = weights[weights.shape[0] - source_masks.shape[0]:].contiguous()     # (a hybrid layer: the weight-stationary rows)
    feats = torch.zeros((S, w.shape[1]), dtype=w.dtype, device=w.device)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    conv_ws(S, T, feats, w, lists)
    b.record()
    b.synchronize()
    return a.elapsed_time(b)


def cuda_time_gemm(parallel, threshold, is_hybrid, weights, source_masks, target_masks, kernel_map_sizes) -> float:
    """Timing probe used by the reference tuner (csrc/spira/torch/cuda_sparse_convolution_forward.cu:422-498).  The fused
    kernel has no separate GEMM stage: the time of the whole weight-stationary layer is returned."""
    return _time_ws(weights, source_masks, target_masks, kernel_map_sizes)


def cuda_time_gather(tile_size, threshold, is_hybrid, weights, source_masks, target_masks, kernel_map_sizes) -> float:
    """See :func:`cuda_time_gemm`."""
    return _time_ws(weights, source_masks, target_masks, kernel_map_sizes)


def cuda_time_scatter(tile_size, threshold, is_hybrid, weights, source_masks, target_masks, kernel_map_sizes) -> float:
    """See :func:`cuda_time_gemm`."""
    return _time_ws(weights, source_masks, target_masks, kernel_map_sizes)


_option_epoch = [0]      # bumped by set_option: prepared calls re-read the options they depend on


def set_option(name: str, value: int) -> None:
    """Process-wide kernel options, e.g. ``set_option("gather_tma", 1)`` (see include/spira_b200.h).  Set options
    through this function: the prepared per-layer calls cache the weight image mode that follows from them."""
    _lib.call("spira_b200_set_option", name.encode(), int(value))
    _option_epoch[0] += 1
    _pack_mode[0] = -1


def get_option(name: str) -> int:
    return int(_lib.load().spira_b200_get_option(name.encode()))


def cuda_free_buffers() -> None:
    """The reference releases its private stack allocator here (csrc/spira/torch/cuda_memory_buffer.cu:7-16).  This
    engine holds no pool of its own: scratch comes from torch's caching allocator, so there is nothing to release."""
    return None


def cuda_reset_error() -> None:
    """Clears a sticky CUDA error (csrc/spira/torch/cuda_memory_buffer.cu:11-16)."""
    _lib.call("spira_b200_reset_error")
