"""Record-and-replay execution of a network's forward pass.

A sparse network is a static sequence of a few operator kinds -- sparse convolution, a feature-wise torch function
(BatchNorm, ReLU, ...), channel concatenation, addition.  Going through ``torch.nn.Module.__call__``,
``SparseTensor`` wrappers and cache lookups for each of them costs more host time per scene than the GPU needs for
the kernels, so ``compile_model`` runs the model ONCE eagerly while a recorder notes every operator with the slots
of its inputs and output, and the returned ``CompiledModel`` replays that tape with a few microseconds of Python
per operator.  Shapes are free to change from scene to scene: kernel maps and coordinates are looked up in the
``KernelMapCache`` at replay time, only the operator sequence, strides and per-layer dataflow are frozen (compile
again after changing them).

The reference has no counterpart: its forward is plain eager PyTorch (``spira/nn/conv.py:310-419``).
"""
from __future__ import annotations

from typing import Any, List, Optional

import torch

from spira_b200.nn.functional import _C
from spira_b200.tensors import SparseTensor

__all__ = ["compile_model", "CompiledModel"]

_recorder = None      # the active Recorder, consulted by SparseConv.forward / fapply / cat / SparseTensor.__add__


class Recorder:
    def __init__(self):
        self.ops: List[tuple] = []
        self.slot_of = {}          # id(feature tensor) -> slot
        self.stride_of = {}        # slot -> stride
        self.keep = []             # keeps recorded tensors alive so that ids stay unique
        self.n_slots = 0

    def slot(self, feats: torch.Tensor, stride=None, create=False) -> int:
        s = self.slot_of.get(id(feats))
        if s is None:
            if not create:
                raise RuntimeError("[spira_b200] compile_model met a tensor that no recorded operator produced")
            s = self.n_slots
            self.n_slots += 1
            self.slot_of[id(feats)] = s
            self.keep.append(feats)
        if stride is not None:
            self.stride_of[s] = stride
        return s

    # -- operators ---------------------------------------------------------------------------------------------
    def conv(self, module, inputs: SparseTensor, residual, output: SparseTensor):
        i = self.slot(inputs._features)
        r = None if residual is None else self.slot(residual)
        o = self.slot(output._features, output._stride, create=True)
        self.ops.append(("conv", module, i, r, o, inputs._stride, output._stride))

    def apply(self, fn, args, kwargs, inputs: SparseTensor, output: SparseTensor):
        i = self.slot(inputs._features)
        o = self.slot(output._features, output._stride, create=True)
        self.ops.append(("apply", fn, args, kwargs, i, o))

    def cat(self, inputs, output: SparseTensor):
        ins = [self.slot(x._features) for x in inputs]
        o = self.slot(output._features, output._stride, create=True)
        self.ops.append(("cat", ins, o))

    def add(self, a: SparseTensor, b: SparseTensor, output: SparseTensor):
        o = self.slot(output._features, output._stride, create=True)
        self.ops.append(("add", self.slot(a._features), self.slot(b._features), o))


def _flatten_outputs(out, rec: Recorder):
    if isinstance(out, SparseTensor):
        return ("one", rec.slot(out._features), out._stride)
    if isinstance(out, (list, tuple)):
        return ("seq", type(out), [_flatten_outputs(x, rec) for x in out])
    raise RuntimeError("[spira_b200] compile_model supports models returning SparseTensors or lists of them")


class CompiledModel:
    """Replays the tape recorded by :func:`compile_model`; call it like the model: ``compiled(sparse_tensor)``."""

    def __init__(self, ops, n_slots, outputs, cache):
        self.cache = cache
        self.n_slots = n_slots
        self.outputs = outputs
        self.ops = []
        for op in ops:
            if op[0] == "conv":
                _, module, i, r, o, in_stride, out_stride = op
                cfg = module._tunable_config
                os_flow = cfg["map_dataflow"] == 0 or cfg["force_os"]
                # cache key of the layer's map (the non-transposed twin's for a transposed layer); the replay reads the
                # cache's dictionaries directly where the generic lookup would only confirm what the tape already knows
                key = (out_stride, in_stride, module.kernel_size) if module.transposed else (in_stride, out_stride, module.kernel_size)
                fast = not cfg["force_os"] and not module._trivial
                self.ops.append((0, module, i, r, o, in_stride, out_stride, os_flow, cfg["map_dataflow"], cfg["force_os"], key, fast))
            elif op[0] == "apply":
                self.ops.append((1,) + op[1:])
            elif op[0] == "cat":
                self.ops.append((2,) + op[1:])
            else:
                self.ops.append((3,) + op[1:])

    def _build(self, spec, slots):
        if spec[0] == "one":
            return SparseTensor(coordinates=self.cache._coordinates_cache.get(spec[2]), features=slots[spec[1]], stride=spec[2])
        return spec[1](self._build(x, slots) for x in spec[2])

    @torch.no_grad()
    def __call__(self, inputs: SparseTensor):
        cache = self.cache
        slots: List[Optional[torch.Tensor]] = [None] * self.n_slots
        slots[0] = inputs._features
        if inputs._stride not in cache._coords:           # (not the property: that would complete a pending map build)
            cache.finish()
            if inputs._stride not in cache._coords:
                cache._coords[inputs._stride] = inputs._coordinates
        for op in self.ops:
            kind = op[0]
            if kind == 0:
                _, module, i, r, o, in_stride, out_stride, os_flow, dataflow, force_os, key, fast = op
                x = slots[i]
                if module._trivial:
                    folded = module._folded
                    if module.out_channels <= 32:
                        y = _C.pointwise(x, *(folded if folded is not None else
                                              (module.kernel.view(module.in_channels, module.out_channels), module.bias)))
                        if y is not None:
                            slots[o] = y
                            continue
                    if folded is not None:
                        slots[o] = torch.addmm(folded[1], x, folded[0])
                    else:
                        y = torch.mm(x, module.kernel.view(module.in_channels, module.out_channels))
                        slots[o] = y if module.bias is None else y + module.bias
                    continue
                if dataflow >= 3 and not os_flow:
                    # hybrid dataflows run through the module's reference-shaped calls
                    xin = SparseTensor(coordinates=cache._coordinates_cache.get(in_stride), features=x, stride=in_stride)
                    slots[o] = module._forward(xin, None if r is None else slots[r])._features
                    continue
                m = None
                if fast:
                    e = cache._maps.get(key)
                    if e is not None and not e[0]:
                        if not (os_flow and module.transposed):
                            m = (e[1], e[2], e[3])
                        else:
                            inv = cache._derived_maps.get((key, "inverted"))
                            if inv is not None:
                                m = (e[1], e[2], inv)
                if m is None:
                    m = cache.get_kernel_map(None, in_stride, None, out_stride, module.kernel_size, dataflow, force_os, module.transposed)
                n_src, n_tgt = (m[1], m[0]) if module.transposed else (m[0], m[1])
                call = module._call
                if call is None or call.stamp != _C.conv_call_stamp(module.kernel, module.bias, module._fused):
                    call = module._call = _C.ConvCall(module.kernel, module.bias, module._fused)
                res = None if r is None else slots[r]
                if os_flow:
                    slots[o] = _C.run_conv_os(call, n_src, n_tgt, m[2], x, res)
                else:
                    slots[o] = _C.run_conv_ws(call, n_src, n_tgt, m[2]._sb["ws"], x, module.transposed, res)
            elif kind == 1:
                slots[op[5]] = op[1](slots[op[4]], *op[2], **op[3])
            elif kind == 2:
                slots[op[2]] = torch.cat([slots[j] for j in op[1]], dim=1)
            else:
                slots[op[3]] = slots[op[1]] + slots[op[2]]
        return self._build(self.outputs, slots)


def compile_model(model: torch.nn.Module, example: SparseTensor, cache) -> CompiledModel:
    """Runs ``model(example)`` once eagerly (kernel maps for ``example`` must be available through ``cache``, e.g.
    after ``cache.add_all_kernel_maps``) and returns the replayable :class:`CompiledModel`."""
    global _recorder
    if _recorder is not None:
        raise RuntimeError("[spira_b200] compile_model is not re-entrant")
    rec = Recorder()
    rec.slot(example._features, example._stride, create=True)
    _recorder = rec
    try:
        with torch.no_grad():
            out = model(example)
    finally:
        _recorder = None
    return CompiledModel(rec.ops, rec.n_slots, _flatten_outputs(out, rec), cache)
