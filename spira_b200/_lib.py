"""ctypes binding of ``libspira_b200.so`` -- the only route from Python to the CUDA kernels.

There is no fallback: if the library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "libspira_b200.so"

c_void_p, c_int, c_int32, c_int64, c_size_t = C.c_void_p, C.c_int, C.c_int32, C.c_int64, C.c_size_t


class KmapDesc(C.Structure):
    """Mirror of ``spira_b200_kmap_desc`` (include/spira_b200.h)."""
    _fields_ = [
        ("sources", c_void_p), ("targets", c_void_p),
        ("num_sources", c_int64), ("num_targets", c_int64),
        ("kernel_size", c_int32 * 3), ("source_stride", c_int32 * 3),
        ("layout", c_int32), ("reserved", c_int32),
        ("map", c_void_p), ("tile_counts", c_void_p), ("row_perm", c_void_p),
    ]


class GroupDesc(C.Structure):
    """Mirror of ``spira_b200_group_desc`` (include/spira_b200.h)."""
    _fields_ = [("map_os", c_void_p), ("num_targets", c_int64), ("K", c_int32), ("grouped_map", c_void_p),
                ("row_of", c_void_p), ("tile_masks", c_void_p), ("stats", c_void_p)]


class WsDesc(C.Structure):
    """Mirror of ``spira_b200_ws_desc`` (include/spira_b200.h)."""
    _fields_ = [("map_ws", c_void_p), ("tile_counts", c_void_p), ("aligned_targets", c_int64), ("K", c_int32), ("rows", c_int32),
                ("nbsizes", c_void_p), ("naddrs", c_void_p), ("qnaddrs", c_void_p), ("tile_base", c_void_p), ("sizes", c_void_p),
                ("in_idx", c_void_p), ("out_idx", c_void_p)]


class Epilogue(C.Structure):
    """Mirror of ``spira_b200_epilogue`` (include/spira_b200.h)."""
    _fields_ = [("bias", c_void_p), ("scale", c_void_p), ("shift", c_void_p), ("residual", c_void_p),
                ("relu", c_int32), ("reserved", c_int32)]


class ConvDesc(C.Structure):
    """Mirror of ``spira_b200_conv_desc`` (include/spira_b200.h)."""
    _fields_ = [("dataflow", c_int32), ("K", c_int32), ("c_in", c_int32), ("c_out", c_int32), ("c_in_a", c_int32),
                ("rows", c_int32), ("mirror", c_int32), ("swap", c_int32), ("splits", c_int32), ("reserved", c_int32),
                ("num_sources", c_int64), ("num_targets", c_int64), ("num_tiles128", c_int64),
                ("feats", c_void_p), ("feats_b", c_void_p), ("packed", c_void_p), ("weights", c_void_p), ("epilogue", C.POINTER(Epilogue)),
                ("map_os", c_void_p), ("row_of", c_void_p), ("tile_masks", c_void_p),
                ("in_idx", c_void_p), ("out_idx", c_void_p), ("naddrs", c_void_p), ("qnaddrs", c_void_p),
                ("zeroed_accum", c_void_p), ("split_scratch", c_void_p), ("split_scratch_bytes", c_size_t), ("out", c_void_p)]


class TapeMap(C.Structure):
    """Mirror of ``spira_b200_tape_map`` (include/spira_b200.h)."""
    _fields_ = [("num_sources", c_int64), ("num_targets", c_int64),
                ("map_os", c_void_p), ("grouped_map", c_void_p), ("row_of", c_void_p), ("tile_masks", c_void_p),
                ("map_os_t", c_void_p), ("grouped_map_t", c_void_p), ("row_of_t", c_void_p), ("tile_masks_t", c_void_p),
                ("in_idx", c_void_p), ("out_idx", c_void_p), ("naddrs", c_void_p), ("qnaddrs", c_void_p),
                ("rows", c_int32), ("mirror", c_int32), ("num_tiles128", c_int64)]


class TapeOp(C.Structure):
    """Mirror of ``spira_b200_tape_op`` (include/spira_b200.h)."""
    _fields_ = [("kind", c_int32), ("dataflow", c_int32), ("transposed", c_int32), ("map", c_int32),
                ("in_a", c_int32), ("in_b", c_int32), ("residual", c_int32), ("out", c_int32),
                ("K", c_int32), ("c_in", c_int32), ("c_in_a", c_int32), ("c_out", c_int32),
                ("grouped", c_int32), ("reserved", c_int32), ("packed", c_void_p), ("weights", c_void_p), ("epilogue", Epilogue)]


class TapeSlot(C.Structure):
    """Mirror of ``spira_b200_tape_slot`` (include/spira_b200.h)."""
    _fields_ = [("rows", c_int64), ("channels", c_int32), ("buffer", c_int32), ("ptr", c_void_p)]


TAPE_CONV, TAPE_IDENTITY, TAPE_POINTWISE = 0, 1, 2
LAYOUT_OS, LAYOUT_WS = 0, 1
KERNEL_NAMES = {0: "conv_os_simt_kernel", 1: "conv_os_stem_kernel", 2: "conv_tc_kernel<OS>", 3: "conv_os_n256_kernel",
                4: "conv_tc_kernel<WS>", 5: "conv_ws_simt_kernel"}
PACK_OS, PACK_WS = 0, 1
MAX_MAPS, MAX_LEVELS = 16, 8

# name -> argument types (every function returns int except the two noted below)
SIGNATURES = {
    "spira_b200_version": [],
    "spira_b200_reset_error": [],
    "spira_b200_read_back": [c_void_p, c_void_p, c_size_t, c_void_p, c_void_p, c_void_p],
    "spira_b200_set_option": [C.c_char_p, c_int],
    "spira_b200_get_option": [C.c_char_p],
    "spira_b200_ws_barrier_resync": [],
    "spira_b200_pack": [c_void_p, c_int64, c_int, c_void_p, c_void_p],
    "spira_b200_unpack": [c_void_p, c_int64, c_int, c_void_p, c_void_p],
    "spira_b200_flatten_sort_workspace": [c_int64, c_int, C.POINTER(c_size_t)],
    "spira_b200_flatten_sort": [c_void_p, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p, c_void_p],
    "spira_b200_permute_rows": [c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_void_p],
    "spira_b200_pointwise": [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p],
    "spira_b200_downsample_workspace": [c_int64, c_int, c_int, C.POINTER(c_size_t)],
    "spira_b200_downsample": [c_void_p, c_int64, c_int, c_int, C.POINTER(c_int32), C.POINTER(c_void_p), c_void_p,
                              c_void_p, c_size_t, c_void_p],
    "spira_b200_downsample_sorted_workspace": [c_int64, c_int, C.POINTER(c_size_t)],
    "spira_b200_downsample_sorted": [c_void_p, c_int64, c_int, c_int, C.POINTER(c_int32), C.POINTER(c_void_p), c_void_p,
                                     c_void_p, c_size_t, c_void_p, c_void_p],
    "spira_b200_kmap_search": [C.POINTER(KmapDesc), c_int, c_int, c_void_p],
    "spira_b200_kmap_ws_sizes": [c_void_p, c_int, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    "spira_b200_kmap_ws_pairs": [c_void_p, c_int, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    "spira_b200_kmap_ws_lists": [C.POINTER(WsDesc), c_int, c_void_p],
    "spira_b200_kmap_masks": [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_void_p],
    "spira_b200_kmap_masks_half": [c_void_p, c_void_p, c_int, c_int, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p],
    "spira_b200_kmap_lists_from_masks": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64, c_int64, c_void_p, c_void_p, c_void_p,
                                         c_void_p, c_void_p],
    "spira_b200_convert_transposed_os": [c_void_p, c_int64, c_int, c_void_p, c_int64, c_void_p],
    "spira_b200_transpose_map": [c_void_p, c_int64, c_int64, c_void_p, c_void_p],
    "spira_b200_tensor_core_eligible": [c_int, c_int, c_int],
    "spira_b200_conv_kernel_choice": [c_int, c_int, c_int, c_int, c_int64],
    "spira_b200_packed_weight_bytes": [c_int, c_int, c_int, c_int, C.POINTER(c_size_t)],
    "spira_b200_pack_weights": [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "spira_b200_conv_os": [c_void_p, c_void_p, c_void_p, C.POINTER(Epilogue), c_void_p, c_int64, c_int64, c_int, c_int,
                           c_int, c_void_p, c_void_p, c_void_p],
    "spira_b200_kmap_group_workspace": [c_int64, C.POINTER(c_size_t)],
    "spira_b200_kmap_group": [C.POINTER(GroupDesc), c_int, c_void_p, c_size_t, c_void_p],
    "spira_b200_conv_os_grouped": [c_void_p, c_void_p, c_void_p, C.POINTER(Epilogue), c_void_p, c_void_p, c_void_p, c_int64,
                                   c_int64, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p],
    "spira_b200_conv_os_split_plan": [c_int64, c_int, c_int, c_int, C.POINTER(c_int), C.POINTER(c_size_t)],
    "spira_b200_conv_os_split": [c_void_p, c_void_p, C.POINTER(Epilogue), c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int,
                                 c_int, c_int, c_int, c_void_p, c_size_t, c_void_p, c_void_p, c_void_p],
    "spira_b200_conv": [C.POINTER(ConvDesc), c_void_p, c_void_p],
    "spira_b200_run_tape": [C.POINTER(TapeOp), c_int, C.POINTER(TapeMap), c_int, C.POINTER(TapeSlot), c_int, c_void_p, c_size_t,
                            C.POINTER(c_size_t), c_void_p, c_size_t, c_void_p, c_void_p],
    "spira_b200_conv_ws": [c_void_p, c_void_p, c_void_p, C.POINTER(Epilogue), c_void_p, c_void_p, c_void_p, c_void_p,
                           c_int, c_int64, c_int, c_int, c_int64, c_int64, c_int, c_int, c_int, c_void_p, c_void_p,
                           c_void_p, c_void_p],
    "spira_b200_conv_ws_fused": [c_void_p, c_void_p, C.POINTER(Epilogue), c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64,
                                 c_int, c_int, c_int64, c_int64, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
    "spira_b200_conv_ws_static": [c_void_p, c_void_p, c_void_p, C.POINTER(Epilogue), c_void_p, c_void_p, c_void_p, c_void_p,
                                  c_int, c_int64, c_int, c_int, c_int64, c_int64, c_int, c_int, c_int, c_void_p, c_void_p,
                                  c_void_p],
}
STATIC_SCRATCH_FLOATS = 4 * 1024 * 1024
EXPORTS = sorted(list(SIGNATURES) + ["spira_b200_last_error"])

_lib = None


def load() -> C.CDLL:
    """Loads the library once; raises if it has not been built (``python -m spira_b200.build``)."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m spira_b200.build` "
                               "(the CUDA library is the only implementation; there is no fallback)")
        lib = C.CDLL(str(LIB_PATH))
        for name, args in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = c_int
        lib.spira_b200_last_error.argtypes = []
        lib.spira_b200_last_error.restype = C.c_char_p
        _lib = lib
    return _lib


def check(code: int) -> None:
    """Turns a non-zero return code into ``RuntimeError('[spira_b200] ...')`` like the reference's
    ``SpiraException`` -> ``RuntimeError`` (csrc/spira/common/exception.h:9-28)."""
    if code != 0:
        msg = load().spira_b200_last_error().decode(errors="replace")
        raise RuntimeError(f"[spira_b200] {msg} (code {code})")


# kernels of this library launched per successful call (library kernels such as the radix sort are not counted)
KERNELS_PER_CALL = {
    "spira_b200_pack": 1, "spira_b200_unpack": 1, "spira_b200_flatten_sort": 1, "spira_b200_permute_rows": 1,
    "spira_b200_downsample": 1, "spira_b200_pointwise": 1, "spira_b200_downsample_sorted": 1, "spira_b200_kmap_search": 1, "spira_b200_kmap_ws_sizes": 2, "spira_b200_kmap_ws_pairs": 1, "spira_b200_kmap_ws_lists": 3,
    "spira_b200_kmap_masks": 1, "spira_b200_kmap_masks_half": 1, "spira_b200_kmap_lists_from_masks": 3, "spira_b200_convert_transposed_os": 1, "spira_b200_transpose_map": 1,
    "spira_b200_pack_weights": 1, "spira_b200_conv_os": 1, "spira_b200_conv_os_grouped": 1, "spira_b200_conv_os_split": 1,
    "spira_b200_kmap_group": 2,
    "spira_b200_conv_ws": 2, "spira_b200_conv_ws_fused": 1, "spira_b200_conv_ws_static": 2,
}
launch_count = 0          # kernels launched through `call` since import (or since it was last reset by the caller)
profile_hook = None       # optional callable(name, args, run) -> None used by the benchmark to time single calls


def call(name: str, *args) -> None:
    global launch_count
    fn = getattr(load(), name)
    if profile_hook is not None:
        profile_hook(name, args, lambda: check(fn(*args)))
    else:
        check(fn(*args))
    launch_count += KERNELS_PER_CALL.get(name, 0)
