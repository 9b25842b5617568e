"""CPU: the C-ABI library builds, loads and exports every symbol the header declares (no compute calls)."""
import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def declared_symbols():
    text = (ROOT / "include" / "spira_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(spira_b200_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_surface():
    names = declared_symbols()
    for must in ("spira_b200_flatten_sort", "spira_b200_downsample", "spira_b200_kmap_search", "spira_b200_conv_os",
                 "spira_b200_conv_ws", "spira_b200_convert_transposed_os", "spira_b200_last_error"):
        assert must in names


def test_library_exports_every_declared_symbol(lib):
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} is declared in include/spira_b200.h but not exported"


def test_python_binding_covers_the_header(lib):
    from spira_b200 import _lib
    assert sorted(_lib.EXPORTS) == declared_symbols()


def test_struct_layouts_match_the_header():
    from spira_b200 import _lib
    assert ctypes.sizeof(_lib.KmapDesc) == 8 * 4 + 4 * 8 + 8 * 3      # 2 ptr, 2 i64, 8 i32, 3 ptr
    assert ctypes.sizeof(_lib.Epilogue) == 4 * 8 + 8
    assert ctypes.sizeof(_lib.ConvDesc) == 10 * 4 + 3 * 8 + 16 * 8         # the library static_asserts the same sizes
    assert ctypes.sizeof(_lib.TapeMap) == 2 * 8 + 12 * 8 + 2 * 4 + 8
    assert ctypes.sizeof(_lib.TapeOp) == 14 * 4 + 2 * 8 + ctypes.sizeof(_lib.Epilogue)
    assert ctypes.sizeof(_lib.TapeSlot) == 8 + 4 + 4 + 8


def test_argument_errors_without_a_gpu(lib):
    """Validation happens on the host before any CUDA call."""
    from spira_b200 import _lib
    import pytest
    n = ctypes.c_size_t()
    assert lib.spira_b200_flatten_sort_workspace(10, 5, ctypes.byref(n)) != 0
    assert b"key_bytes" in lib.spira_b200_last_error()
    assert lib.spira_b200_downsample_workspace(10, 4, 99, ctypes.byref(n)) != 0
    assert lib.spira_b200_tensor_core_eligible(27, 64, 64) == 1
    assert lib.spira_b200_tensor_core_eligible(27, 4, 32) == 0
    assert lib.spira_b200_tensor_core_eligible(27, 64, 19) == 0
    assert lib.spira_b200_packed_weight_bytes(27, 64, 64, 0, ctypes.byref(n)) == 0 and n.value == 27 * 64 * 128
    assert lib.spira_b200_packed_weight_bytes(27, 32, 64, 0, ctypes.byref(n)) == 0 and n.value == 14 * 64 * 128
    assert lib.spira_b200_packed_weight_bytes(27, 32, 64, 1, ctypes.byref(n)) == 0 and n.value == 27 * 64 * 128
    with pytest.raises(RuntimeError, match="spira_b200"):
        _lib.call("spira_b200_kmap_search", None, 99, 4, None)


def test_new_struct_layouts_match_the_header():
    from spira_b200 import _lib
    assert ctypes.sizeof(_lib.GroupDesc) == 8 + 8 + 8 + 4 * 8           # ptr, i64, i32 (+pad), 4 ptr
    assert ctypes.sizeof(_lib.WsDesc) == 2 * 8 + 8 + 2 * 4 + 7 * 8      # 2 ptr, i64, 2 i32, 7 ptr


def test_more_argument_errors_without_a_gpu(lib):
    from spira_b200 import _lib
    n = ctypes.c_size_t()
    assert lib.spira_b200_kmap_group_workspace(-1, ctypes.byref(n)) != 0
    assert lib.spira_b200_kmap_group(None, 99, None, 0, None) != 0 and b"n_maps" in lib.spira_b200_last_error()
    assert lib.spira_b200_kmap_ws_lists(None, 17, None) != 0 and b"n_maps" in lib.spira_b200_last_error()
    assert lib.spira_b200_kmap_group(None, 0, None, 0, None) == 0       # nothing to do
    assert lib.spira_b200_downsample_sorted_workspace(10, 3, ctypes.byref(n)) != 0
    assert lib.spira_b200_set_option(b"wait_limit_us", 1) != 0 and b"wait_limit_us" in lib.spira_b200_last_error()
    assert lib.spira_b200_set_option(b"no_such_option", 1) != 0 and lib.spira_b200_get_option(b"no_such_option") == -1
    assert lib.spira_b200_get_option(b"wait_limit_us") == 1500000 and lib.spira_b200_get_option(b"os_n256") == 1
    assert lib.spira_b200_read_back(None, None, 4, None, None, None) != 0
    assert lib.spira_b200_get_option(b"pdl") == 1 and lib.spira_b200_get_option(b"ws_cooperative_launch") == 0
    assert lib.spira_b200_set_option(b"pdl", 0) == 0 and lib.spira_b200_get_option(b"pdl") == 0
    assert lib.spira_b200_set_option(b"pdl", 1) == 0
    assert lib.spira_b200_get_option(b"identity_tma") == 1
    assert lib.spira_b200_set_option(b"identity_tma", 0) == 0 and lib.spira_b200_get_option(b"identity_tma") == 0
    assert lib.spira_b200_set_option(b"identity_tma", 1) == 0


def test_tape_and_descriptor_argument_checks_without_a_gpu(lib):
    """spira_b200_run_tape places its slots and validates the tables before anything is launched; the descriptor call
    rejects what it cannot run.  None of these reaches the device."""
    from spira_b200 import _lib
    need = ctypes.c_size_t(123)
    assert lib.spira_b200_run_tape(None, 0, None, 0, None, 0, None, 0, ctypes.byref(need), None, 0, None, None) == 0
    assert need.value == 0
    slots = (_lib.TapeSlot * 3)()
    for i, (rows, ch, buf) in enumerate(((1000, 64, -1), (1000, 96, 0), (500, 96, 0))):
        slots[i].rows, slots[i].channels, slots[i].buffer = rows, ch, buf
    slots[0].ptr = 4096
    # the arena is too small: nothing runs, the size it needs comes back (the two slots share buffer 0: the larger wins)
    rc = lib.spira_b200_run_tape(None, 0, None, 0, slots, 3, None, 0, ctypes.byref(need), None, 0, None, None)
    assert rc != 0
    assert need.value == 1000 * 96 * 2 and b"arena" in lib.spira_b200_last_error()
    # with an arena the slots get their addresses (same buffer, same address)
    rc = lib.spira_b200_run_tape(None, 0, None, 0, slots, 3, ctypes.c_void_p(1 << 20), 1 << 20, ctypes.byref(need), None, 0, None, None)
    assert rc == 0 and slots[1].ptr == slots[2].ptr == 1 << 20 and slots[0].ptr == 4096
    rc = lib.spira_b200_run_tape(None, 0, None, 0, slots, 3, ctypes.c_void_p((1 << 20) + 16), 1 << 20, ctypes.byref(need), None, 0, None, None)
    assert rc == 0      # (addresses already assigned: nothing left to place)
    slots[1].ptr = None
    rc = lib.spira_b200_run_tape(None, 0, None, 0, slots, 3, ctypes.c_void_p((1 << 20) + 16), 1 << 20, ctypes.byref(need), None, 0, None, None)
    assert rc != 0 and b"256-byte" in lib.spira_b200_last_error()
    # operators naming slots that do not exist, or whose channel counts do not match
    ops = (_lib.TapeOp * 1)()
    ops[0].kind, ops[0].in_a, ops[0].in_b, ops[0].residual, ops[0].out = _lib.TAPE_CONV, 0, -1, -1, 7
    rc = lib.spira_b200_run_tape(ops, 1, None, 0, slots, 3, ctypes.c_void_p(1 << 20), 1 << 20, ctypes.byref(need), None, 0, None, None)
    assert rc != 0 and b"slot" in lib.spira_b200_last_error()
    ops[0].out, ops[0].c_in, ops[0].c_out, ops[0].K = 1, 64, 32, 27
    rc = lib.spira_b200_run_tape(ops, 1, None, 0, slots, 3, ctypes.c_void_p(1 << 20), 1 << 20, ctypes.byref(need), None, 0, None, None)
    assert rc != 0 and b"channels" in lib.spira_b200_last_error()
    ops[0].c_out, ops[0].map = 96, 3
    rc = lib.spira_b200_run_tape(ops, 1, None, 0, slots, 3, ctypes.c_void_p(1 << 20), 1 << 20, ctypes.byref(need), None, 0, None, None)
    assert rc != 0 and b"map" in lib.spira_b200_last_error()
    # descriptor call
    d = _lib.ConvDesc(dataflow=5)
    assert lib.spira_b200_conv(ctypes.byref(d), None, None) != 0 and b"dataflow" in lib.spira_b200_last_error()
    d = _lib.ConvDesc(dataflow=0, K=27, c_in=64, c_out=64, c_in_a=32, packed=4096, feats=4096)
    assert lib.spira_b200_conv(ctypes.byref(d), None, None) != 0 and b"second tensor" in lib.spira_b200_last_error()
    assert lib.spira_b200_conv(None, None, None) != 0
    n, b = ctypes.c_int(0), ctypes.c_size_t(0)
    assert lib.spira_b200_conv_os_split_plan(1000, 27, 64, 64, None, None) != 0
