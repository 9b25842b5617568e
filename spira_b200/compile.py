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

import ctypes as C

from spira_b200 import _lib
from spira_b200.nn.functional import _C
from spira_b200.tensors import SparseTensor

__all__ = ["compile_model", "CompiledModel"]

NATIVE_TAPE = True     # replay through spira_b200_run_tape (one library call per scene) where every operator allows it

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

    def __init__(self, ops, n_slots, outputs, cache, input_stride=(1, 1, 1)):
        self.cache = cache
        self.input_stride = input_stride
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

        # ``native``: the pass as tables for spira_b200_run_tape, or None with the reason in ``native_error``;
        # ``use_native`` switches between it and the operator-by-operator replay below (same results up to the rounding
        # of the 1x1x1 layers).  The native call costs a fraction of the host time; on the GPU its 1x1x1 layers run on the
        # engine's own kernel, which is slower than the library GEMM of the Python replay -- which one wins depends on
        # whether the host or the GPU is the bottleneck of the surrounding loop.
        self.native = None
        self.native_error = None
        if NATIVE_TAPE:
            try:
                self.native = _NativeTape(self)
            except _NotNative as e:
                self.native_error = str(e)
        self.use_native = self.native is not None

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
        if self.native is not None and self.use_native:
            # The layers on the level-0 map (built before the level sizes are known) are enqueued first, operator by
            # operator: the GPU works on them while the host waits for the sizes inside cache.finish().  The rest of the
            # pass is one call into the library.
            self._replay(self.ops[:self.native.prefix], slots)
            return self._build(self.outputs, self.native.run(slots))
        self._replay(self.ops, slots)
        return self._build(self.outputs, slots)

    def _replay(self, ops, slots):
        cache = self.cache
        for op in ops:
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


class _NotNative(Exception):
    """The recorded pass holds an operator the library's tape executor does not take; the Python replay runs it."""


def _output_slots(spec, acc):
    if spec[0] == "one":
        acc.append(spec[1])
    else:
        for x in spec[2]:
            _output_slots(x, acc)
    return acc


class _NativeTape:
    """The recorded pass as tables for ``spira_b200_run_tape``.

    Built once per compiled model: channel concatenations whose only readers are convolutions disappear (the readers take
    two sources), 1x1x1 layers become pointwise or identity-map operators, and every feature tensor that lives only
    inside the pass gets an arena buffer number from its lifetime (tensors of the same level and width take turns in one
    buffer).  Per scene only the map table, the row counts and the addresses of input and outputs are filled in."""

    def __init__(self, compiled: "CompiledModel"):
        cache = compiled.cache
        ops = compiled.ops
        n_slots = compiled.n_slots
        out_slots = set(_output_slots(compiled.outputs, []))
        # leading layers that share the map of the first one: they run before the other maps exist (see __call__)
        prefix = 0
        if ops and ops[0][0] == 0 and not ops[0][1]._trivial and ops[0][11]:
            while prefix < len(ops) and ops[prefix][0] == 0 and not ops[prefix][1]._trivial and ops[prefix][11] \
                    and ops[prefix][10] == ops[0][10] and not ops[prefix][1].transposed:
                prefix += 1
        self.prefix = prefix
        self.prefix_slots = {op[4]: op[1].out_channels for op in ops[:prefix]}      # produced by the prefix: external to the tape
        # ---- concatenations: (a | b) read only by convolutions -> two-source convolutions
        other_reads = set()     # slots read as a residual or by a concatenation
        for op in ops:
            if op[0] == 0:
                if op[3] is not None:
                    other_reads.add(op[3])
            elif op[0] == 2:
                other_reads.update(op[1])
            else:
                raise _NotNative("the pass holds a feature-wise torch operator or an addition outside a fused epilogue")
        parts = {}      # slot of a concatenation -> (slot a, slot b)
        for op in ops:
            if op[0] != 2:
                continue
            ins, o = op[1], op[2]
            if len(ins) != 2 or o in out_slots or o in other_reads:
                raise _NotNative("a concatenation that is not two tensors read only as convolution input")
            parts[o] = (ins[0], ins[1])
        # ---- operators
        self.modules = []
        self.stamps = []
        table = []          # (TapeOp fields dict, module)
        map_keys = []       # cache key per map index
        slot_channels = {0: None}
        slot_channels.update(self.prefix_slots)
        slot_stride = dict(compiled_strides(compiled))
        for op in ops[prefix:]:
            if op[0] == 2:
                continue
            _, module, i, r, o, in_stride, out_stride, os_flow, dataflow, force_os, key, fast = op
            in_a, in_b = parts.get(i, (i, -1))
            if in_a in parts or in_b in parts:
                raise _NotNative("nested concatenations")
            K = 1
            for v in module.kernel_size:
                K *= v
            cin, cout = module.in_channels, module.out_channels
            f = dict(in_a=in_a, in_b=in_b, residual=-1 if r is None else r, out=o, K=K, c_in=cin, c_out=cout, c_in_a=0,
                     map=-1, dataflow=0, transposed=0, grouped=0)
            if module._trivial:
                folded = module._folded
                w2d, bias = folded if folded is not None else (module.kernel.view(cin, cout), module.bias)
                if cout <= 32 and _C.POINTWISE_HEAD and cin % 8 == 0 and 8 <= cin <= 512 and in_b == -1 and r is None:
                    f.update(kind=_lib.TAPE_POINTWISE, weights=w2d.contiguous(), bias=bias)
                else:
                    call = _C.ConvCall(w2d.contiguous().view(1, cin, cout), bias, None)
                    if not call.eligible:
                        raise _NotNative(f"a 1x1x1 layer {cin} -> {cout} outside the tensor-core kernels")
                    f.update(kind=_lib.TAPE_IDENTITY, call=call, mode=_C.PACK_OS)
            else:
                if dataflow >= 3 and not os_flow:
                    raise _NotNative("hybrid dataflows run through the reference-shaped calls")
                call = module._call
                if call is None or call.stamp != _C.conv_call_stamp(module.kernel, module.bias, module._fused):
                    call = module._call = _C.ConvCall(module.kernel, module.bias, module._fused)
                if not call.eligible and (not os_flow or in_b >= 0):
                    raise _NotNative(f"a layer (K={K}, {cin} -> {cout}) outside the tensor-core kernels that is not a plain "
                                     f"output-stationary one")
                if not fast:
                    raise _NotNative("a layer pinned to the output-stationary dataflow on a map built for another")
                if key not in map_keys:
                    map_keys.append(key)
                f.update(kind=_lib.TAPE_CONV, call=call, mode=_C.PACK_OS if os_flow else _C.PACK_WS, map=map_keys.index(key),
                         dataflow=0 if os_flow else 1, transposed=1 if module.transposed else 0,
                         grouped=1 if (call.eligible or call.stem) else 0)
            table.append((f, module))
            slot_channels[o] = cout
            if in_a == 0 and in_b == -1 and slot_channels[0] is None:
                slot_channels[0] = cin
        if _lib.load().spira_b200_get_option(b"os_pack_mode") != _C.PACK_OS:
            raise _NotNative("the TMA gather engine is selected")
        # channel split of the two-source operators
        for f, module in table:
            if f["in_b"] >= 0:
                ca, cb = slot_channels.get(f["in_a"]), slot_channels.get(f["in_b"])
                if ca is None or cb is None or ca + cb != f["c_in"] or ca % 8 or cb % 8:
                    raise _NotNative("a concatenation whose parts the two-source kernels do not take")
                f["c_in_a"] = ca
        self.map_keys = map_keys
        self.n_slots = n_slots
        self.out_slots = sorted(out_slots)
        self.slot_stride = slot_stride
        # ---- lifetimes -> arena buffer numbers (an operator's output never shares storage with its own inputs)
        last_use = {}
        for n, (f, _) in enumerate(table):
            for sl in (f["in_a"], f["in_b"], f["residual"]):
                if sl >= 0:
                    last_use[sl] = n
        # A freed buffer goes to the next tensor of the same level (most recently freed first: its lines are still in
        # L2), else to one of a coarser level (fewer rows: it fits without growing the buffer); the executor sizes
        # every buffer for the largest tensor that passes through it.
        buffer_of = {}
        home = {}           # buffer number -> stride of the level it was created for (its finest, hence largest, tenant)
        free = []           # buffer numbers, most recently freed last
        n_buffers = 0

        def no_coarser(a, b):
            return all(x <= y for x, y in zip(a, b))

        for n, (f, _) in enumerate(table):
            o = f["out"]
            if o not in out_slots:
                st = slot_stride[o]
                pick = None
                for j in range(len(free) - 1, -1, -1):
                    if home[free[j]] == st:
                        pick = j
                        break
                if pick is None:
                    for j in range(len(free) - 1, -1, -1):
                        if no_coarser(home[free[j]], st):
                            pick = j
                            break
                if pick is not None:
                    buffer_of[o] = free.pop(pick)
                else:
                    buffer_of[o] = n_buffers
                    home[n_buffers] = st
                    n_buffers += 1
            for sl in {f["in_a"], f["in_b"], f["residual"]}:
                if sl >= 0 and last_use.get(sl) == n and sl in buffer_of:
                    free.append(buffer_of[sl])
        # ---- the C tables
        self.keep = []
        self.ops = (_lib.TapeOp * len(table))()
        for t, (f, module) in zip(self.ops, table):
            t.kind, t.dataflow, t.transposed, t.map = f["kind"], f["dataflow"], f["transposed"], f["map"]
            t.in_a, t.in_b, t.residual, t.out = f["in_a"], f["in_b"], f["residual"], f["out"]
            t.K, t.c_in, t.c_in_a, t.c_out = f["K"], f["c_in"], f["c_in_a"], f["c_out"]
            t.grouped = f["grouped"]
            if f["kind"] == _lib.TAPE_POINTWISE:
                t.weights = f["weights"].data_ptr()
                if f["bias"] is not None:
                    t.epilogue.bias = f["bias"].data_ptr()
                self.keep.append((f["weights"], f["bias"]))
            else:
                call = f["call"]
                t.packed = call.packed_ptr(f["mode"])          # (None outside the tensor-core kernels: plain weights then)
                if not call.eligible:
                    t.weights = call.w_ptr
                ep = call.ep
                t.epilogue.bias, t.epilogue.scale, t.epilogue.shift, t.epilogue.relu = ep.bias, ep.scale, ep.shift, ep.relu
                self.keep.append(call)
            self.modules.append(module)
            self.stamps.append((module.kernel.data_ptr(), module.kernel._version))
        self.n_ops = len(table)
        self.slots = (_lib.TapeSlot * n_slots)()
        for sl in range(n_slots):
            self.slots[sl].channels = slot_channels.get(sl) or 0
            self.slots[sl].buffer = buffer_of.get(sl, -1)
        self.arena_slots = [sl for sl in range(n_slots) if sl in buffer_of]
        self.used_slots = sorted(set(self.arena_slots) | out_slots | {0} | set(self.prefix_slots))
        self.maps = (_lib.TapeMap * max(len(map_keys), 1))()
        self.ws_outputs = [(f["out"], f["c_out"]) for f, _ in table if f["kind"] == _lib.TAPE_CONV and f["dataflow"] == 1]
        self.needs = {}     # map index -> (needs the output-stationary form, needs its inverse, needs the lists)
        for f, _ in table:
            if f["kind"] == _lib.TAPE_CONV:
                n = self.needs.setdefault(f["map"], [False, False, False])
                if f["dataflow"] == 1:
                    n[2] = True
                elif f["transposed"]:
                    n[1] = True
                else:
                    n[0] = True
        self.cache = cache
        self.arena = None
        self.needed = C.c_size_t(0)
        self.fn = _lib.load().spira_b200_run_tape

    def run(self, given):
        """``given``: the slot list of the pass with the network input in slot 0 and the outputs of the prefix layers in
        theirs; returns the list with the model's outputs filled in."""
        feats = given[0]
        cache = self.cache
        cache.finish()
        for module, stamp in zip(self.modules, self.stamps):
            k = module.kernel
            if k.data_ptr() != stamp[0] or k._version != stamp[1]:
                raise RuntimeError("[spira_b200] a layer's weights changed after compile_model; compile again")
        if not feats.is_contiguous():
            feats = feats.contiguous()
        device = feats.device
        # ---- maps of this scene
        maps = self.maps
        for n, key in enumerate(self.map_keys):
            e = cache._maps.get(key)
            if e is None or e[0]:
                raise RuntimeError(f"[spira_b200] the kernel map {key} of the compiled pass is not in the cache")
            m = maps[n]
            m.num_sources, m.num_targets = e[1], e[2]
            need_os, need_inv, need_ws = self.needs[n]
            sb = e[3]._sb
            if need_os:
                if sb.get("layout") != _C.LAYOUT_OS:
                    raise RuntimeError(f"[spira_b200] the kernel map {key} was not built output-stationary")
                m.map_os = e[3].data_ptr()
                g = sb.get("grouped") if _C.GROUP_OS else None
                if g is None and sb.get("group_lazy") is not None and _C.GROUP_OS:
                    g = _C.grouped_twin(e[3])
                if g is not None:
                    m.grouped_map, m.row_of, m.tile_masks = g.map_ptr, g.row_of_ptr, g.tile_masks_ptr
                else:
                    m.grouped_map, m.row_of, m.tile_masks = None, None, None
            if need_inv:
                inv = cache._derived_maps.get((key, "inverted"))
                if inv is None:
                    inv = cache.get_kernel_map(None, key[1], None, key[0], key[2], 0, False, True)[2]
                g = inv._sb.get("grouped") if (getattr(inv, "_sb", None) and _C.GROUP_OS) else None
                m.map_os_t = inv.data_ptr()
                if g is not None:
                    m.grouped_map_t, m.row_of_t, m.tile_masks_t = g.map_ptr, g.row_of_ptr, g.tile_masks_ptr
                else:
                    m.grouped_map_t, m.row_of_t, m.tile_masks_t = None, None, None
                self.keep_scene = inv
            if need_ws:
                lists = sb["ws"]
                m.in_idx, m.out_idx, m.naddrs, m.qnaddrs = lists.in_ptr, lists.out_ptr, lists.naddrs_ptr, lists.qnaddrs_ptr
                m.rows, m.mirror = lists.rows, 1 if lists.mirror else 0
                m.num_tiles128 = -1 if lists.qmapsize is None else lists.qmapsize // 128
        # ---- slots: rows per level, addresses of input and outputs
        slots = self.slots
        coords = cache._coords
        stride_of = self.slot_stride
        rows_of = {}
        for sl in self.used_slots:
            st = stride_of[sl]
            r = rows_of.get(st)
            if r is None:
                r = rows_of[st] = coords[st].shape[0]
            slots[sl].rows = r
            slots[sl].ptr = None
        slots[0].ptr = feats.data_ptr()
        if slots[0].channels == 0:
            slots[0].channels = feats.shape[1]
        result = [None] * self.n_slots
        result[0] = feats
        for sl in self.prefix_slots:
            t = given[sl]
            if not t.is_contiguous():
                t = given[sl] = t.contiguous()
            result[sl] = t
            slots[sl].ptr = t.data_ptr()
        for sl in self.out_slots:
            if sl == 0 or sl in self.prefix_slots:
                continue
            t = result[sl] = torch.empty((slots[sl].rows, slots[sl].channels), dtype=torch.float16, device=device)
            slots[sl].ptr = t.data_ptr()
        zero_floats = 0
        for sl, cout in self.ws_outputs:
            zero_floats = max(zero_floats, slots[sl].rows * cout)
        accum = _C.zero_scratch(device, zero_floats) if zero_floats else None
        status = _C.status_word(device)
        stream = _C._raw_stream(device.index if device.index is not None else torch.cuda.current_device())
        for attempt in range(2):
            arena = self.arena
            rc = self.fn(self.ops, self.n_ops, maps, len(self.map_keys), slots, self.n_slots,
                         arena.data_ptr() if arena is not None else None, arena.numel() if arena is not None else 0,
                         C.byref(self.needed), accum.data_ptr() if accum is not None else None,
                         accum.numel() if accum is not None else 0, status.data_ptr(), stream)
            if rc == 0:
                break
            if attempt == 0 and self.needed.value > (arena.numel() if arena is not None else 0):
                # the scene needs a larger arena (nothing was launched): grow it and run again
                self.arena = torch.empty(int(self.needed.value * 1.25) + 4096, dtype=torch.uint8, device=device)
                for sl in self.arena_slots:
                    slots[sl].ptr = None
                continue
            _lib.check(rc)
        _lib.launch_count += self.n_ops
        return result


def compiled_strides(compiled: "CompiledModel"):
    """(slot, stride) of every feature tensor of the recorded pass."""
    out = {0: compiled.input_stride}
    for op in compiled.ops:
        if op[0] == 0:
            out[op[4]] = op[6]
        elif op[0] == 2:
            out[op[2]] = out[op[1][0]]
    return out.items()


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
    return CompiledModel(rec.ops, rec.n_slots, _flatten_outputs(out, rec), cache, example._stride)
