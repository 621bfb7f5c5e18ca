"""CPU suite, part 2: the C-ABI library builds, loads, exports every symbol
the header declares, and refuses to compute without a GPU (no CPU fallback)."""

import ctypes as C
import os
import re

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    src = open(os.path.join(ROOT, "include", "tiny_gemma_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(tg_[a-z0-9_]+)\s*\(", src)))


def test_library_exports_every_declared_symbol(capi):
    lib = capi.load()
    syms = header_symbols()
    assert len(syms) >= 30
    for s in syms:
        assert hasattr(lib, s), "missing export: " + s
    # and the Python binding knows every one of them
    assert sorted(capi.SIGNATURES) == syms


def test_config_table_matches_reference(capi):
    c = capi.config("270m")
    assert (c.hidden_size, c.intermediate_size, c.n_layers, c.n_vocab, c.n_pos, c.n_pos_local, c.head_dim, c.n_head,
            c.n_kv, c.window_pattern) == (640, 2048, 18, 262144, 32768, 512, 256, 4, 1, 6)
    c = capi.config("1B")
    assert (c.hidden_size, c.intermediate_size, c.n_layers) == (1152, 6912, 26)
    assert (c.rope_theta, c.rope_theta_local) == (1000000.0, 10000.0)
    try:
        capi.config("7B")
        assert False
    except capi.TgError as e:
        assert e.code == capi.TG_EINVAL
    n = C.c_size_t(0)
    cfg = capi.config("1B")
    assert capi.load().tg_model_file_bytes(C.byref(cfg), C.byref(n)) == 0 and n.value == 1305168896


def test_no_cpu_fallback(capi):
    if capi.device_count() > 0:
        return  # on a GPU box the parity tests cover the compute path
    for fn in (lambda: capi.Model("270m"), lambda: capi.qmatvec(np.zeros(640, np.float32), np.zeros((640, 1024), np.int8),
                                                                np.ones(1024, np.float32))):
        try:
            fn()
            assert False, "computed without a GPU"
        except capi.TgError as e:
            assert e.code == capi.TG_ENODEVICE


def test_shape_errors_come_before_device_use(capi):
    # unsupported K / N: the reference throws std::runtime_error (static_switch.hpp:27-29,55-57)
    try:
        capi.qmatvec(np.zeros(100, np.float32), np.zeros((100, 1024), np.int8), np.ones(1024, np.float32))
        assert False
    except capi.TgError as e:
        assert e.code == capi.TG_ESHAPE and "ROW" in str(e)
    try:
        capi.qmatvec(np.zeros(640, np.float32), np.zeros((640, 512), np.int8), np.ones(512, np.float32))
        assert False
    except capi.TgError as e:
        assert e.code == capi.TG_ESHAPE and "COL" in str(e)
