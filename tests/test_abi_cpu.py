"""The C-ABI library builds for sm_100a, loads without a GPU, and exports every entry
point include/soklyn_b200.h declares (no compute calls here)."""
import ctypes as C
import os
import re

from soklyn_b200 import _native

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "soklyn_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sk_[a-z0-9_]+)\s*\(", text)))


def test_header_and_bindings_agree():
    assert declared_symbols() == _native.exported_symbols()


def test_library_exports_every_declared_symbol():
    lib = _native.lib()
    for name in declared_symbols():
        assert hasattr(lib, name), name


def test_host_only_entry_points():
    lib = _native.lib()
    assert lib.sk_status_string(0) == b"ok"
    assert lib.sk_status_string(2) == b"Dimension mismatch"
    assert lib.sk_last_error(None) == b""
    assert lib.sk_launch_count(None) == 0
    # scramble_seed known answers, computed by hand from src/util/core.rs:90-94
    def scramble(step, lid):
        m = 0xFFFFFFFF
        h = (step * 1103515245 + lid) & m
        h = ((h ^ (h >> 16)) * 1103515245) & m
        return h ^ (h >> 15)
    for step, lid in [(0, 0), (1, 0), (1, 23), (7, 46), (100, 27), (0xFFFFFFFF, 0xFFFFFFFF)]:
        assert lib.sk_scramble_seed(step, lid) == scramble(step, lid)


def test_null_arguments_are_rejected_without_a_device():
    lib = _native.lib()
    assert lib.sk_ctx_create(0, 16, None, 0, 0, None) == 9          # NULL out pointer
    assert lib.sk_dense_forward(None, None, None, 0, 0, 0, 0, 0) == 9
    assert lib.sk_sync(None) == 9
    assert lib.sk_step_begin(None, 0) == 9 and lib.sk_step_end(None) == 9 and lib.sk_step_abort(None) == 9
    assert lib.sk_step_stats(None, None) == 9


def test_descriptor_layout_matches_header():
    # 5 u32 (+pad) + 28 pointers + 7 scalars: catches a field added on one side only
    assert C.sizeof(_native.SkDense) == 24 + 28 * 8 + 32
    assert C.sizeof(_native.SkOptim) == 20
