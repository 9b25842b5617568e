"""``KernelMapCache`` and ``SparseConv`` -- same public surface as the reference module
(spira/nn/conv.py:17-151 and :153-419): constructor arguments, ``kernel`` parameter of shape
``[K, c_in, c_out]``, ``_tunable_config`` keys, cache keys ``(source_stride, target_stride, kernel_size)`` and the
rule that a transposed layer reuses the map of its non-transposed twin.

Underneath there are two dataflows.  ``map_dataflow == 0`` (or ``force_os``) runs the output-stationary
implicit GEMM; every other value runs the weight-stationary gather-GEMM-scatter over compacted pair lists
(odd values through the reference's ``ws_merged`` slots, even values through its mask slots).
"""
__all__ = ['SparseConv', 'KernelMapCache', 'Conv3d']

import contextlib
import operator
from typing import Any, Dict, List, Optional, Tuple, Union

import numpy as np
import torch
from torch.nn import Module

from spira_b200.nn import functional as F
from spira_b200.nn.functional import _C
from spira_b200.tensors import SparseTensor
from spira_b200 import compile as _compile
from spira_b200.utils.helpers import as_tuple
from spira_b200.utils.typing import ScalarOrTuple


class KernelMapCache(object):
    """Coordinates per stride and kernel maps per ``(source_stride, target_stride, kernel_size)``.

    ``add_all_kernel_maps`` enqueues the down-sampling and the level-0 map and returns; everything that needs the level
    sizes on the host is completed on the first request that needs it (``finish()``).  The level-0 layers of a
    network are then enqueued first and keep the GPU busy while the remaining maps are being prepared."""

    def __init__(self):
        self._maps = dict()
        self._coords = dict()
        self._derived_maps = dict()   # maps derived from cached ones (transposed / inverted), built once
        self._pending = None          # arguments of a network-wide build that has not been completed yet
        # keys of the maps a transposed output-stationary layer asked the inverse of; kept across reset(): the next
        # network-wide build makes those inverses right away, grouped by the same sort as all other maps
        self._inverse_keys = set()
        # map key -> False: the rows of this output-stationary map keep their target order (set by spira.tune where the
        # layers that use the map save less than the grouping costs); maps not named here are grouped
        self._group_policy = dict()

    def set_group_policy(self, policy: Dict[tuple, bool]):
        self._group_policy = dict(policy)
        return self

    def _groups(self, key) -> bool:
        return self._group_policy.get(key, True)

    # the three dictionaries under their historical names: reading them completes a pending build first
    @property
    def _kernel_maps_cache(self):
        self.finish()
        return self._maps

    @property
    def _coordinates_cache(self):
        self.finish()
        return self._coords

    @property
    def _derived(self):
        self.finish()
        return self._derived_maps

    def reset(self):
        self._pending = None
        self._coords.clear()
        self._maps.clear()
        self._derived_maps.clear()

    def finish(self):
        """Completes a pending ``add_all_kernel_maps`` (no-op otherwise)."""
        if self._pending is not None:
            pending, self._pending = self._pending, None
            self._complete(*pending)
        return self

    def get_target_coordinates(self, source_coordinates: torch.Tensor, source_stride: ScalarOrTuple[int],
                               target_stride: ScalarOrTuple[int], transposed: bool = False):
        if type(source_stride) is not tuple:
            source_stride = as_tuple(source_stride, size=3, name="source_stride")
        if source_stride not in self._coords:
            self.finish()
            if source_stride not in self._coords:
                self._coords[source_stride] = source_coordinates
        if target_stride not in self._coords:
            self.finish()
        if target_stride in self._coords:
            return self._coords[target_stride]
        if transposed:
            raise RuntimeError("Layer must transpose=True must have its corresponding "
                               "non-transposed layer before its execution")
        target_coordinates = F.downsample(source_coordinates, target_stride)
        self._coords[target_stride] = target_coordinates
        return target_coordinates

    def get_kernel_map(self, source_coordinates: torch.Tensor, source_stride: ScalarOrTuple[int],
                       target_coordinates: torch.Tensor, target_stride: ScalarOrTuple[int],
                       kernel_size: ScalarOrTuple[int], map_dataflow: int, force_os: bool = False,
                       transposed: bool = False):
        if type(source_stride) is not tuple:
            source_stride = as_tuple(source_stride, size=3, name="source_stride")
        if type(target_stride) is not tuple:
            target_stride = as_tuple(target_stride, size=3, name="target_stride")
        if type(kernel_size) is not tuple:
            kernel_size = as_tuple(kernel_size, size=3, name="kernel_size")
        key = (target_stride, source_stride, kernel_size) if transposed else (source_stride, target_stride, kernel_size)

        if key not in self._maps:
            self.finish()
        if key not in self._maps:
            if transposed:
                raise RuntimeError("Layer must transpose=True must have its corresponding "
                                   "non-transposed layer before its execution")
            kernel_map = F.build_kmap(source_coordinates, target_coordinates, kernel_size, source_stride, map_dataflow)
            self._maps[key] = [False, *kernel_map]
        entry = self._maps[key]  # [flipped_flag, *tuple9]

        if force_os and not entry[0]:
            # a [K, T_al] map used output-stationary: transpose it once (reference: conv.py:80-83)
            sb = getattr(entry[3], "_sb", None)
            if sb is None or sb.get("layout") == _C.LAYOUT_WS:
                flipped = _C.transpose_map(entry[3])
                if sb is not None:
                    flipped._sb = dict(sb, layout=_C.LAYOUT_OS, group_lazy=None, grouped=_C.group_os_map(flipped, entry[2]))
                entry[3] = flipped
            entry[0] = True

        if (map_dataflow == 0 or force_os) and transposed:
            # output-stationary map of the transposed layer = inverse of the cached one.  The reference
            # rebuilds it on every forward (conv.py:85-89); it depends only on the cached map, so it is kept.
            dkey = (key, "inverted")
            if self._pending is not None and dkey not in self._derived_maps:
                self.finish()
            if dkey not in self._derived_maps or not getattr(_C, "CACHE_DERIVED", True):
                inv = F.convert_transposed_os(entry[3], entry[1])
                sb = getattr(entry[3], "_sb", None)
                if sb is not None:
                    inv._sb = dict(sb, ws=None, counts=None, _counts=None, group_lazy=None,
                                   grouped=_C.group_os_map(inv, entry[1]) if self._groups(key) else None)
                    self._inverse_keys.add(key)
                self._derived_maps[dkey] = inv
            new_entry = list(entry[1:])
            new_entry[2] = self._derived_maps[dkey]
            return new_entry
        return entry[1:]

    def add_all_kernel_maps(self, source_coordinates: torch.Tensor, kernel_sizes: List[ScalarOrTuple[int]],
                            source_strides: List[ScalarOrTuple[int]], target_strides: List[ScalarOrTuple[int]],
                            init_stride: Union[int, Tuple[int, ...]], dataflow: List[int]):
        """Network-wide precompute: all down-sampled coordinate sets, then all kernel maps in one batched
        search (reference: conv.py:116-151)."""
        self.finish()
        t_strides = [as_tuple(s, size=3, name="target_stride") for s in target_strides]
        k_sizes = [as_tuple(k, size=3, name="kernel_size") for k in kernel_sizes]
        s_strides = [as_tuple(s, size=3, name="kernel_stride") for s in source_strides]
        dataflow = list(dataflow)
        if not (len(k_sizes) == len(s_strides) - 1 == len(dataflow)):
            raise ValueError("All argument lists must have the same length in add_all_kernel_maps")
        source_coordinates = source_coordinates.contiguous()
        s0 = as_tuple(init_stride, size=3)
        self._coords[s0] = source_coordinates
        levels = _C.streamed_output_generate_begin(source_coordinates, t_strides) if len(t_strides) and len(k_sizes) \
            and hasattr(_C, "streamed_output_generate_begin") else None
        # The layers of this package read the pair lists through the engine's own structures, so the list sizes stay on
        # the device: the level sizes are the only host read of a scene.  Map 0 has the level-0 keys on both sides and
        # does not need them: it is built now, and the rest waits until somebody asks for it (finish()).
        first = None
        if levels is not None and getattr(_C, "DEFER_MAPS", True):
            first = _C.cuda_binary_search_pairs([(source_coordinates, source_coordinates)], k_sizes[:1], s_strides[:1],
                                                dataflow[:1], exact_sizes=False, group=self._groups((s0, s_strides[1], k_sizes[0])))
            self._maps[(s0, s_strides[1], k_sizes[0])] = self._entry(first[0])
        self._pending = (source_coordinates, k_sizes, s_strides, t_strides, s0, dataflow, levels, first)
        if levels is None or not getattr(_C, "DEFER_MAPS", True):
            self.finish()
        return self

    @staticmethod
    def _entry(kmap):
        """Cache entry ``[flipped_flag, *tuple9]``.  The network-wide build keeps the weight-stationary lists on the device
        (``map._sb["ws"]``, no list size is read back, slots 7 and 8 are None), so the reference-shaped list slots 3-6 of
        such an entry stay None as well instead of being materialised as tensor views for every map of every scene; the
        single-map path (``F.build_kmap``) fills all slots."""
        if type(kmap).__name__ == "_WsTuple":
            return [False, kmap[0], kmap[1], kmap[2], None, None, None, None, None, None]
        return [False, *kmap]

    def _complete(self, source_coordinates, k_sizes, s_strides, t_strides, s0, dataflow, levels, first):
        if levels is not None:
            output = _C.streamed_output_generate_end(levels)
        else:
            output = F.streamed_output_generate(source_coordinates, t_strides) if len(t_strides) else []
        voxels: List[torch.Tensor] = [source_coordinates] + output
        for i, t_stride in enumerate(t_strides):
            self._coords[t_stride] = voxels[i + 1]

        deferred = first is not None
        if deferred:
            # the remaining maps are grouped below, together with the inverses the transposed layers will ask for
            pairs = [(voxels[i // 2], voxels[(i + 1) // 2]) for i in range(1, len(k_sizes))]
            kmaps = first + (_C.cuda_binary_search_pairs(pairs, k_sizes[1:], s_strides[1:-1], dataflow[1:], exact_sizes=False,
                                                         group=False) if pairs else [])
        elif hasattr(_C, "cuda_binary_search_pairs"):
            # everything at once: one search launch, one grouping sort (inverses included)
            pairs = [(voxels[i // 2], voxels[(i + 1) // 2]) for i in range(len(k_sizes))]
            kmaps = _C.cuda_binary_search_pairs(pairs, k_sizes, s_strides[:-1], dataflow, exact_sizes=False, group=False)
            deferred = True
        else:
            kmaps = F.build_kmap_streamed(voxels, k_sizes, s_strides[:-1], dataflow, exact_sizes=False)

        keys = []
        s_stride = s0
        for i in range(len(k_sizes)):
            t_stride = s_strides[i + 1]
            key = (s_stride, t_stride, k_sizes[i])
            if not (first is not None and i == 0):
                self._maps[key] = self._entry(kmaps[i])
            keys.append(key)
            s_stride = t_stride

        if deferred:
            todo = []       # (tensor that carries the grouped twin, number of rows)
            for i, key in enumerate(keys):
                entry = self._maps[key]
                sb = getattr(entry[3], "_sb", None)
                if sb is None or sb.get("layout") != _C.LAYOUT_OS or not self._groups(key):
                    continue
                if i > 0 or first is None:
                    todo.append((entry[3], entry[2]))
                if key in self._inverse_keys and (key, "inverted") not in self._derived_maps:
                    inv = F.convert_transposed_os(entry[3], entry[1])
                    inv._sb = dict(sb, ws=None, counts=None, _counts=None, group_lazy=None, grouped=None)
                    self._derived_maps[(key, "inverted")] = inv
                    todo.append((inv, entry[1]))
            for (mp, _), g in zip(todo, _C.group_os_maps(todo)):
                mp._sb["grouped"] = g


class SparseConv(Module):

    __AVAILABLE_THRESHOLD__ = [-1, *list(np.linspace(0, 2, num=50)), None]
    __NUM_TUNING_ROUNDS__ = 5

    def __init__(self, in_channels: int, out_channels: int, kernel_size: ScalarOrTuple[int],
                 stride: ScalarOrTuple[int] = 1, bias: bool = False, transposed: bool = False, dilation: int = 1):
        super().__init__()
        if dilation != 1 and tuple(as_tuple(dilation, size=3)) != (1, 1, 1):
            raise ValueError("dilation other than 1 is not supported (the reference layer has no dilation argument)")
        self.in_channels = in_channels
        self.out_channels = out_channels
        self.kernel_size = as_tuple(kernel_size, size=3, name="kernel_size")
        self.stride = as_tuple(stride, size=3, name="stride")
        self.transposed = transposed

        kernel_volume = int(np.prod(self.kernel_size).item())
        self.kernel = torch.nn.Parameter(torch.empty(kernel_volume, in_channels, out_channels))
        if bias:
            self.bias = torch.nn.Parameter(torch.empty(out_channels))
        else:
            self.register_parameter('bias', None)
        self.reset_parameters()

        self._kernel_map_cache: Optional[KernelMapCache] = None
        self._tunable_config = {
            'threshold': -1,
            'gather_tile_size': min(in_channels, 16),
            'scatter_tile_size': min(out_channels, 16),
            'map_dataflow': 2,
            'force_os': False,
        }
        self._tuning_data = None
        # optional fused epilogue (set by spira_b200.fuse): per-channel fp32 scale / shift and a ReLU flag that the
        # kernels apply to the fp32 accumulator before the single rounding to fp16
        self._fused = None
        self._folded = None        # 1x1x1 layer with a BatchNorm folded into it by spira_b200.fuse: (weight, bias)
        self._call = None          # prepared native call (spira_b200.nn.functional._C.ConvCall)
        self._trivial = all(x == 1 for x in self.stride) and all(x == 1 for x in self.kernel_size)

    def set_fused_epilogue(self, scale: Optional[torch.Tensor], shift: Optional[torch.Tensor], relu: bool):
        """``y = relu?((conv(x) + bias) * scale + shift [+ residual])`` inside the convolution kernel."""
        if self.is_trivial:
            raise ValueError("the 1x1x1 stride-1 layer is a plain matrix product and has no fused epilogue")
        self._fused = dict(scale=None if scale is None else scale.detach().float().contiguous(),
                           shift=None if shift is None else shift.detach().float().contiguous(), relu=bool(relu))

    @property
    def tunable_config(self) -> Dict[str, Any]:
        return self._tunable_config

    def reset_parameters(self):
        std = (self.out_channels if self.transposed else self.in_channels)
        std = 1. / np.sqrt(std * len(self.kernel))
        self.kernel.data.uniform_(-std, std)
        if self.bias is not None:
            self.bias.data.uniform_(-std, std)

    def set_kernel_map_cache(self, cache: KernelMapCache):
        self._kernel_map_cache = cache

    @property
    def is_trivial(self):
        return self._trivial

    @contextlib.contextmanager
    def tune_gs(self, free_buffers: bool = True):
        """Kept for interface compatibility (reference: conv.py:217-307).  The gather / GEMM / scatter tile
        sizes and the padding threshold it searched belong to the reference's three-kernel pipeline; the fused
        weight-stationary kernel has none of them, so the context only records the calls."""
        try:
            self._tuning_data = list()
            yield
        finally:
            self._tuning_data = None

    def forward(self, inputs: SparseTensor, residual: Optional[torch.Tensor] = None):
        output = self._forward(inputs, residual)
        rec = _compile._recorder
        if rec is not None:
            rec.conv(self, inputs, residual, output)
        return output

    def _forward(self, inputs: SparseTensor, residual: Optional[torch.Tensor] = None):
        source_features = inputs._features
        if self.is_trivial:
            pointwise = getattr(_C, "pointwise", None)       # (absent when a reference-built binding is installed)
            if pointwise is not None and self.out_channels <= 32 and not torch.is_grad_enabled():
                # a head with few output channels runs the engine's own kernel (bias included)
                w, b = self._folded if self._folded is not None else (self.kernel.view(self.in_channels, self.out_channels), self.bias)
                y = pointwise(source_features, w, b)
                if y is not None:
                    return SparseTensor(features=y, coordinates=inputs._coordinates, stride=inputs._stride)
            if self._folded is not None:
                return SparseTensor(features=torch.addmm(self._folded[1], source_features, self._folded[0]),
                                    coordinates=inputs._coordinates, stride=inputs._stride)
            kernel = self.kernel.view(self.in_channels, self.out_channels)
            target_features = torch.mm(source_features, kernel)
            target_coordinates = inputs._coordinates
            target_stride = inputs._stride
        else:
            if self._kernel_map_cache is None:
                raise ValueError("Kernel map cache must be specified")
            op = operator.floordiv if self.transposed else operator.mul
            target_stride = tuple(op(a, b) for a, b in zip(inputs._stride, self.stride))
            cache = self._kernel_map_cache
            target_coordinates = cache.get_target_coordinates(inputs._coordinates, inputs._stride, target_stride, self.transposed)

            map_dataflow = self._tunable_config['map_dataflow']
            force_os = self._tunable_config['force_os']
            m = cache.get_kernel_map(inputs._coordinates, inputs._stride, target_coordinates, target_stride,
                                     self.kernel_size, map_dataflow, force_os, self.transposed)
            # m = (num_sources, num_targets, map, slot3, slot4, slot5, slot6, mapsize, qmapsize) of the
            # NON-transposed twin; a transposed layer exchanges the roles of sources and targets
            n_src, n_tgt = (m[1], m[0]) if self.transposed else (m[0], m[1])

            sb = getattr(m[2], "_sb", None) if hasattr(_C, "run_conv_os") else None
            if sb is not None and (map_dataflow == 0 or force_os or sb.get("ws") is not None):
                # engine-native call: bias / BatchNorm affine / residual / ReLU are applied in the kernel epilogue
                call = self._call
                if call is None or call.stamp != _C.conv_call_stamp(self.kernel, self.bias, self._fused):
                    call = self._call = _C.ConvCall(self.kernel, self.bias, self._fused)
                if map_dataflow == 0 or force_os:
                    target_features = _C.run_conv_os(call, n_src, n_tgt, m[2], source_features, residual)
                else:
                    if self._tuning_data is not None and map_dataflow % 2 == 0:
                        self._tuning_data.append(((m[4], m[3]) if self.transposed else (m[3], m[4])) + (m[5],))
                    target_features = _C.run_conv_ws(call, n_src, n_tgt, sb["ws"], source_features, self.transposed, residual)
                return SparseTensor(features=target_features, coordinates=target_coordinates, stride=target_stride)
            # reference-shaped calls: maps from another builder, and the hybrid dataflows 3-8 (an output-stationary and a
            # weight-stationary call per layer; a fused epilogue is applied as separate passes afterwards)
            epilogue_after = self._fused is not None or residual is not None
            if epilogue_after and not (sb is not None and map_dataflow >= 3):
                raise RuntimeError("[spira_b200] the fused epilogue needs kernel maps built by this engine")
            if map_dataflow == 0 or force_os:
                target_features = F.sparse_convolution_forward_os(n_src, n_tgt, m[2], source_features, self.kernel)
            elif map_dataflow % 2 == 1:
                if map_dataflow == 1:
                    target_features = F.sparse_convolution_forward_ws_merged(
                        n_src, n_tgt, source_features, self.kernel, m[5], m[6], m[3], m[7], m[8], self.transposed)
                else:
                    target_features = F.sparse_convolution_forward_hs_merged(
                        n_src, n_tgt, source_features, self.kernel, m[5], m[6], m[3],
                        None if map_dataflow == 3 else m[2], m[7], m[8], self.transposed)
            else:
                masks = (m[4], m[3]) if self.transposed else (m[3], m[4])
                if self._tuning_data is not None:
                    self._tuning_data.append((masks[0], masks[1], m[5]))
                if map_dataflow == 2:
                    target_features = F.sparse_convolution_forward_ws(
                        n_src, n_tgt, source_features, self.kernel, masks[0], masks[1], m[5],
                        self._tunable_config['gather_tile_size'], self._tunable_config['scatter_tile_size'],
                        None, self._tunable_config['threshold'])
                else:
                    target_features = F.sparse_convolution_forward_hs(
                        n_src, n_tgt, source_features, self.kernel, masks[0], masks[1], m[5],
                        None if map_dataflow == 4 else m[2],
                        self._tunable_config['gather_tile_size'], self._tunable_config['scatter_tile_size'],
                        None, self._tunable_config['threshold'])

            if epilogue_after:
                y = target_features.float()
                if self.bias is not None:
                    y = y + self.bias.float()
                if self._fused is not None and self._fused["scale"] is not None:
                    y = y * self._fused["scale"] + self._fused["shift"]
                if residual is not None:
                    y = y + residual.float()
                if self._fused is not None and self._fused["relu"]:
                    y = torch.relu(y)
                return SparseTensor(features=y.to(target_features.dtype), coordinates=target_coordinates, stride=target_stride)

        if self.bias is not None:
            target_features += self.bias
        return SparseTensor(features=target_features, coordinates=target_coordinates, stride=target_stride)


# TorchSparse's name for the same layer (the reference's comparison scripts use it, scripts/correctness.py:79-80)
Conv3d = SparseConv
