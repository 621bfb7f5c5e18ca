"""ctypes binding of ``libtinygemma_b200.so`` (the C ABI in
``include/tiny_gemma_b200.h``). Thin: every method is one C call plus NumPy
buffer handling. There is no fallback — if the library is missing or no GPU is
present the calls raise."""

from __future__ import annotations

import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libtinygemma_b200.so")

TG_OK, TG_EINVAL, TG_ENODEVICE, TG_ECUDA, TG_EIO, TG_ESHAPE, TG_ESTATE, TG_ENOMEM = range(8)


class TgError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__("tg error %d: %s" % (code, msg))
        self.code = code


class tg_config(C.Structure):
    _fields_ = [
        ("hidden_size", C.c_int), ("intermediate_size", C.c_int), ("n_layers", C.c_int), ("n_vocab", C.c_int),
        ("n_pos", C.c_int), ("n_pos_local", C.c_int), ("head_dim", C.c_int), ("n_head", C.c_int), ("n_kv", C.c_int),
        ("rope_theta", C.c_float), ("rope_theta_local", C.c_float), ("window_pattern", C.c_int),
    ]


# every symbol the header declares, with its argument types
_P = C.c_void_p
SIGNATURES = {
    "tg_last_error": (C.c_char_p, []),
    "tg_version": (C.c_char_p, []),
    "tg_device_count": (C.c_int, [C.POINTER(C.c_int)]),
    "tg_config_by_name": (C.c_int, [C.c_char_p, C.POINTER(tg_config)]),
    "tg_model_create": (C.c_int, [C.POINTER(tg_config), C.c_int, C.POINTER(_P)]),
    "tg_model_free": (C.c_int, [_P]),
    "tg_model_load_file": (C.c_int, [_P, C.c_char_p]),
    "tg_model_load_memory": (C.c_int, [_P, _P, C.c_size_t]),
    "tg_model_file_bytes": (C.c_int, [C.POINTER(tg_config), C.POINTER(C.c_size_t)]),
    "tg_model_set_rope": (C.c_int, [_P, C.c_int, _P, _P, C.c_int]),
    "tg_model_set_gelu_table": (C.c_int, [_P, C.c_float, C.c_float, _P, C.c_int]),
    "tg_model_build_tables": (C.c_int, [_P, C.c_int]),
    "tg_state_create": (C.c_int, [_P, C.c_int, C.c_int, C.POINTER(_P)]),
    "tg_state_free": (C.c_int, [_P]),
    "tg_state_reset": (C.c_int, [_P]),
    "tg_state_position": (C.c_int, [_P, C.c_int, C.POINTER(C.c_int)]),
    "tg_prefill": (C.c_int, [_P, _P, C.c_int, _P]),
    "tg_decode": (C.c_int, [_P, _P, _P]),
    "tg_append": (C.c_int, [_P, _P, C.c_int, _P]),
    "tg_sample_argmax": (C.c_int, [_P, _P]),
    "tg_sample_minp": (C.c_int, [_P, C.c_float, C.c_float, _P, _P]),
    "tg_logits_read": (C.c_int, [_P, _P]),
    "tg_generate": (C.c_int, [_P, _P, C.c_int, C.c_float, C.c_float, _P, _P]),
    "tg_kv_read": (C.c_int, [_P, C.c_int, C.c_int, C.c_int, C.c_int, _P, _P]),
    "tg_hidden_read": (C.c_int, [_P, _P]),
    "tg_qmatvec": (C.c_int, [_P, _P, _P, _P, C.c_int, C.c_int]),
    "tg_qgemm": (C.c_int, [_P, _P, _P, _P, C.c_int, C.c_int, C.c_int]),
    "tg_argmax_logits": (C.c_int, [_P, C.c_int, C.POINTER(C.c_int)]),
    "tg_minp_logits": (C.c_int, [_P, C.c_int, C.c_float, C.c_float, C.c_float, C.POINTER(C.c_int)]),
    "tg_inverse_cdf": (C.c_int, [_P, C.c_int, C.c_float, C.c_float, C.POINTER(C.c_int), C.POINTER(C.c_float)]),
    "tg_rmsnorm": (C.c_int, [_P, _P, C.c_int, C.c_int]),
    "tg_dev_qmatvec": (C.c_int, [_P, _P, _P, _P, C.c_int, C.c_int, _P]),
    "tg_dev_qmatvec_static": (C.c_int, [_P, _P, _P, _P, C.c_int, C.c_int, _P]),
    "tg_dev_qgemm": (C.c_int, [_P, _P, _P, _P, C.c_int, C.c_int, C.c_int, _P]),
    "tg_decode_hidden": (C.c_int, [_P, _P]),
    "tg_dev_hidden_copy": (C.c_int, [_P, _P]),
    "tg_dev_lm_head_top1": (C.c_int, [_P, _P, C.c_int, C.c_int, C.c_int, _P, _P, _P]),
    "tg_dev_set_tokens": (C.c_int, [_P, _P]),
    "tg_state_check": (C.c_int, [_P]),
    "tg_dev_resolve_top1": (C.c_int, [_P, C.c_int, C.c_int, C.c_int, C.c_int, _P, _P]),
    "tg_launch_count": (C.c_int, [C.c_int, C.POINTER(C.c_longlong)]),
    "tg_state_stream": (C.c_int, [_P, C.POINTER(_P)]),
    "tg_generate_async": (C.c_int, [_P, C.c_int, C.c_float, C.c_float]),
    "tg_state_set_randf": (C.c_int, [_P, _P, C.c_int]),
    "tg_state_tokens": (C.c_int, [_P, C.c_int, _P]),
    "tg_state_phase_clocks": (C.c_int, [_P, _P, C.c_int, C.POINTER(C.c_int)]),
}

_lib = None


def load() -> C.CDLL:
    """dlopen the library (once) and set signatures; raises if it is not built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FileNotFoundError(
                LIB_PATH + " is not built; run `python tiny-gemma_b200/build.py` (there is no CPU fallback)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def _ck(rc: int):
    if rc != TG_OK:
        raise TgError(rc, load().tg_last_error().decode())


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def device_count() -> int:
    n = C.c_int(0)
    _ck(load().tg_device_count(C.byref(n)))
    return n.value


def config(name: str) -> tg_config:
    c = tg_config()
    _ck(load().tg_config_by_name(name.encode(), C.byref(c)))
    return c


def launch_count(reset: bool = False) -> int:
    n = C.c_longlong(0)
    _ck(load().tg_launch_count(int(reset), C.byref(n)))
    return n.value


# ------------------------------------------------------------------ isolated ops
def qmatvec(x, w, scales) -> np.ndarray:
    K, N = w.shape
    x, scales = _f32(x), _f32(scales)
    w = np.ascontiguousarray(w, np.int8)
    y = np.empty(N, np.float32)
    _ck(load().tg_qmatvec(_ptr(y), _ptr(x), _ptr(w), _ptr(scales), K, N))
    return y


def qgemm(a, w, scales) -> np.ndarray:
    K, N = w.shape
    a, scales = _f32(a), _f32(scales)
    w = np.ascontiguousarray(w, np.int8)
    M = a.shape[0]
    c = np.empty((M, N), np.float32)
    _ck(load().tg_qgemm(_ptr(c), _ptr(a), _ptr(w), _ptr(scales), M, K, N))
    return c


def argmax_logits(logits) -> int:
    logits = _f32(logits)
    t = C.c_int(0)
    _ck(load().tg_argmax_logits(_ptr(logits), logits.size, C.byref(t)))
    return t.value


def minp_logits(logits, minp: float, temp: float, randf: float):
    """returns (token, probabilities); the input array is left untouched"""
    p = np.array(logits, np.float32, copy=True)
    t = C.c_int(0)
    _ck(load().tg_minp_logits(_ptr(p), p.size, minp, temp, randf, C.byref(t)))
    return t.value, p


def inverse_cdf(p, randf: float, cum0: float = 0.0):
    """First index whose sequential fp32 running sum reaches randf (-1 if none), and the sum there."""
    p = _f32(p)
    i = C.c_int(0)
    c = C.c_float(0.0)
    _ck(load().tg_inverse_cdf(_ptr(p), p.size, cum0, randf, C.byref(i), C.byref(c)))
    return i.value, c.value


def rmsnorm(x, w) -> np.ndarray:
    w = _f32(w)
    x = np.array(x, np.float32, copy=True).reshape(-1, w.shape[0])
    _ck(load().tg_rmsnorm(_ptr(x), _ptr(w), x.shape[0], x.shape[1]))
    return x


# ------------------------------------------------------------------ model / state
class Model:
    """gemma::Transformer + read_weights (reference transformer.hpp:22-47, 99-165)"""

    def __init__(self, size: str, device: int = 0):
        self.lib = load()
        self.size = size
        self.cfg = config(size)
        self.h = C.c_void_p()
        _ck(self.lib.tg_model_create(C.byref(self.cfg), device, C.byref(self.h)))

    def load_file(self, path: str):
        _ck(self.lib.tg_model_load_file(self.h, path.encode()))
        return self

    def load_bytes(self, blob: np.ndarray):
        blob = np.ascontiguousarray(blob, np.uint8)
        _ck(self.lib.tg_model_load_memory(self.h, _ptr(blob), blob.size))
        return self

    def file_bytes(self) -> int:
        n = C.c_size_t(0)
        _ck(self.lib.tg_model_file_bytes(C.byref(self.cfg), C.byref(n)))
        return n.value

    def set_tables(self, cos_g, sin_g, cos_l, sin_l, gelu, gmin=-4.0, gmax=4.0):
        cos_g, sin_g, cos_l, sin_l, gelu = map(_f32, (cos_g, sin_g, cos_l, sin_l, gelu))
        _ck(self.lib.tg_model_set_rope(self.h, 0, _ptr(cos_g), _ptr(sin_g), cos_g.shape[0]))
        _ck(self.lib.tg_model_set_rope(self.h, 1, _ptr(cos_l), _ptr(sin_l), cos_l.shape[0]))
        _ck(self.lib.tg_model_set_gelu_table(self.h, gmin, gmax, _ptr(gelu), gelu.size))
        return self

    def build_tables(self, gelu_size: int = 1024):
        _ck(self.lib.tg_model_build_tables(self.h, gelu_size))
        return self

    def lm_head_top1_dev(self, hidden_ptr: int, M: int, col0: int, ncols: int, max_ptr: int, idx_ptr: int, stream: int = 0):
        _ck(self.lib.tg_dev_lm_head_top1(self.h, C.c_void_p(hidden_ptr), M, col0, ncols, C.c_void_p(max_ptr),
                                         C.c_void_p(idx_ptr), C.c_void_p(stream)))

    def resolve_top1_dev(self, cand_ptr: int, world: int, M: int, row0: int, nrows: int, toks_ptr: int, stream: int = 0):
        _ck(self.lib.tg_dev_resolve_top1(C.c_void_p(cand_ptr), world, M, row0, nrows, C.c_void_p(toks_ptr), C.c_void_p(stream)))

    def state(self, batch: int = 1, max_pos_global: int = 0) -> "State":
        return State(self, batch, max_pos_global)

    def close(self):
        if self.h:
            self.lib.tg_model_free(self.h)
            self.h = C.c_void_p()


class State:
    """decode::DecodeState plus the forward / sampler calls"""

    def __init__(self, model: Model, batch: int, max_pos_global: int):
        self.m = model
        self.lib = model.lib
        self.B = batch
        self.V = model.cfg.n_vocab
        self.h = C.c_void_p()
        _ck(self.lib.tg_state_create(model.h, batch, max_pos_global, C.byref(self.h)))

    def reset(self):
        _ck(self.lib.tg_state_reset(self.h))

    def position(self, b: int = 0) -> int:
        p = C.c_int(0)
        _ck(self.lib.tg_state_position(self.h, b, C.byref(p)))
        return p.value

    def prefill(self, ids, want_logits: bool = True):
        ids = np.ascontiguousarray(ids, np.int32).reshape(self.B, -1)
        logits = np.empty((self.B, self.V), np.float32) if want_logits else None
        _ck(self.lib.tg_prefill(self.h, _ptr(ids), ids.shape[1], _ptr(logits)))
        return logits

    def decode(self, ids=None, want_logits: bool = True):
        if ids is not None:
            ids = np.ascontiguousarray(ids, np.int32).reshape(self.B)
        logits = np.empty((self.B, self.V), np.float32) if want_logits else None
        _ck(self.lib.tg_decode(self.h, _ptr(ids), _ptr(logits)))
        return logits

    def append(self, ids, want_logits: bool = True):
        """continue a non-empty context with the given tokens (one sequence per state)"""
        ids = np.ascontiguousarray(ids, np.int32).reshape(-1)
        logits = np.empty((1, self.V), np.float32) if want_logits else None
        _ck(self.lib.tg_append(self.h, _ptr(ids), ids.size, _ptr(logits)))
        return logits

    def sample_argmax(self) -> np.ndarray:
        t = np.empty(self.B, np.int32)
        _ck(self.lib.tg_sample_argmax(self.h, _ptr(t)))
        return t

    def sample_minp(self, minp: float, temp: float, randf) -> np.ndarray:
        randf = _f32(randf).reshape(self.B)
        t = np.empty(self.B, np.int32)
        _ck(self.lib.tg_sample_minp(self.h, minp, temp, _ptr(randf), _ptr(t)))
        return t

    def logits(self) -> np.ndarray:
        out = np.empty((self.B, self.V), np.float32)
        _ck(self.lib.tg_logits_read(self.h, _ptr(out)))
        return out

    def generate(self, first_ids, n_steps: int, minp: float = 2.0, temp: float = 1.0, randf=None) -> np.ndarray:
        first_ids = np.ascontiguousarray(first_ids, np.int32).reshape(self.B)
        rf = None if randf is None else _f32(randf).reshape(-1)
        out = np.empty((n_steps, self.B), np.int32)
        _ck(self.lib.tg_generate(self.h, _ptr(first_ids), n_steps, minp, temp, _ptr(rf), _ptr(out)))
        return out

    def set_randf(self, randf):
        rf = _f32(randf).reshape(-1, self.B)
        _ck(self.lib.tg_state_set_randf(self.h, _ptr(rf), rf.shape[0]))

    def generate_async(self, n_steps: int, minp: float = 2.0, temp: float = 1.0):
        _ck(self.lib.tg_generate_async(self.h, n_steps, minp, temp))

    def tokens(self, n_steps: int) -> np.ndarray:
        out = np.empty((n_steps, self.B), np.int32)
        _ck(self.lib.tg_state_tokens(self.h, n_steps, _ptr(out)))
        return out

    def phase_clocks(self) -> np.ndarray:
        out = np.zeros(4096, np.int64)
        n = C.c_int(0)
        _ck(self.lib.tg_state_phase_clocks(self.h, _ptr(out), out.size, C.byref(n)))
        return out[:n.value]

    def decode_hidden(self, ids=None):
        if ids is not None:
            ids = np.ascontiguousarray(ids, np.int32).reshape(self.B)
        _ck(self.lib.tg_decode_hidden(self.h, _ptr(ids)))

    def check(self):
        """synchronises the state's stream and raises if a kernel left an error word"""
        _ck(self.lib.tg_state_check(self.h))

    def hidden_copy_dev(self, dst_ptr: int):
        _ck(self.lib.tg_dev_hidden_copy(self.h, C.c_void_p(dst_ptr)))

    def set_tokens_dev(self, toks_ptr: int):
        _ck(self.lib.tg_dev_set_tokens(self.h, C.c_void_p(toks_ptr)))

    def stream(self) -> int:
        p = C.c_void_p()
        _ck(self.lib.tg_state_stream(self.h, C.byref(p)))
        return p.value or 0

    def kv_read(self, layer: int, slot0: int, nslots: int, b: int = 0):
        k = np.empty((nslots, 256), np.float32)
        v = np.empty((nslots, 256), np.float32)
        _ck(self.lib.tg_kv_read(self.h, b, layer, slot0, nslots, _ptr(k), _ptr(v)))
        return k, v

    def hidden(self) -> np.ndarray:
        out = np.empty((self.B, self.m.cfg.hidden_size), np.float32)
        _ck(self.lib.tg_hidden_read(self.h, _ptr(out)))
        return out

    def close(self):
        if self.h:
            self.lib.tg_state_free(self.h)
            self.h = C.c_void_p()
