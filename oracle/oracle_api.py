"""ctypes wrapper over the oracle libraries (TEST INFRASTRUCTURE, not the product).

``Oracle("port")`` loads ``oracle/libtgoracle.so`` (the scalar restatement);
``Oracle("reference")`` loads ``oracle/_ref/libtgref.so`` (the unmodified
reference headers behind a shim). Both export the same functions under the
prefixes ``orc_`` / ``ref_``.
"""

from __future__ import annotations

import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
VOCAB = 262144

_f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_i8p = np.ctypeslib.ndpointer(dtype=np.int8, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")


def lib_path(kind: str) -> str:
    return os.path.join(HERE, "libtgoracle.so") if kind == "port" else os.path.join(HERE, "_ref", "libtgref.so")


def available(kind: str) -> bool:
    return os.path.exists(lib_path(kind))


class Oracle:
    def __init__(self, kind: str = "port"):
        assert kind in ("port", "reference")
        self.kind = kind
        self.prefix = "orc_" if kind == "port" else "ref_"
        self.lib = C.CDLL(lib_path(kind))
        self._sig()

    def _fn(self, name):
        return getattr(self.lib, self.prefix + name)

    def _sig(self):
        f = self._fn
        f("last_error").restype = C.c_char_p
        f("model_create").restype = C.c_void_p
        f("model_create").argtypes = [C.c_char_p]
        f("model_free").argtypes = [C.c_void_p]
        f("model_load").argtypes = [C.c_void_p, C.c_char_p]
        f("state_create").restype = C.c_void_p
        f("state_create").argtypes = [C.c_void_p, C.c_int]
        f("state_free").argtypes = [C.c_void_p]
        f("prefill").argtypes = [C.c_void_p, _i32p, C.c_int, C.c_void_p]
        f("decode").argtypes = [C.c_void_p, C.c_int, C.c_void_p]
        f("decode_loop").argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_float, C.c_float, C.c_void_p, _i32p]
        f("kv_info").argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int)]
        f("kv_read").argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, _f32p, _f32p]
        f("hidden_read").argtypes = [C.c_void_p, _f32p]
        f("argmax_logits").argtypes = [_f32p, C.c_int]
        f("minp_logits").argtypes = [_f32p, C.c_int, C.c_float, C.c_float, C.c_float]
        for n in ("linear_decode", "lm_head_decode"):
            f(n).argtypes = [_f32p, _f32p, _i8p, _f32p, C.c_int, C.c_int]
        f("linear_prefill").argtypes = [_f32p, _f32p, _i8p, _f32p, C.c_int, C.c_int, C.c_int]
        f("time_linear").argtypes = [_f32p, _i8p, _f32p, C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_double)]
        f("rmsnorm").argtypes = [_f32p, _f32p, C.c_int, C.c_int]
        f("rope_tables").argtypes = [C.c_char_p, C.c_int, _f32p, _f32p]
        f("gelu_table").argtypes = [C.c_float, C.c_float, C.c_int, _f32p]
        f("state_tables").argtypes = [C.c_void_p] + [C.c_void_p] * 5
        f("module_mlp").argtypes = [_f32p, C.c_int, C.c_int, C.c_int, _i8p, _f32p, _i8p, _f32p, _i8p, _f32p, _f32p,
                                    _f32p, C.c_int]
        f("module_attention").argtypes = [_f32p, C.c_int, C.c_int, C.c_int, _i8p, _f32p, _i8p, _f32p, _i8p, _f32p,
                                          _i8p, _f32p, _f32p, _f32p, _f32p, _f32p, C.c_int, C.c_void_p, C.c_void_p]
        f("module_lm_head").argtypes = [_f32p, _f32p, C.c_int, C.c_int, _i8p, _f32p, _f32p]
        if self.kind == "port":
            f("state_set_tables").argtypes = [C.c_void_p] + [C.c_void_p] * 5
            f("mt19937_uniforms").argtypes = [C.c_uint, C.c_int, _f32p]

    def _check(self, rc):
        if rc != 0:
            raise RuntimeError("%s oracle: %s" % (self.kind, self._fn("last_error")().decode()))

    # ------------------------------------------------------------ isolated ops
    def linear_decode(self, x, w, s):
        K, N = w.shape
        y = np.zeros(N, np.float32)
        self._check(self._fn("linear_decode")(y, np.ascontiguousarray(x, np.float32), w, s, K, N))
        return y

    def lm_head_decode(self, x, w, s):
        K, N = w.shape
        y = np.zeros(N, np.float32)
        self._check(self._fn("lm_head_decode")(y, np.ascontiguousarray(x, np.float32), w, s, K, N))
        return y

    def linear_prefill(self, a, w, s):
        K, N = w.shape
        M = a.shape[0]
        c = np.zeros((M, N), np.float32)
        self._check(self._fn("linear_prefill")(c, np.ascontiguousarray(a, np.float32), w, s, M, K, N))
        return c

    def time_linear(self, x, w, s, M, reps):
        K, N = w.shape
        secs = C.c_double(0)
        self._check(self._fn("time_linear")(np.ascontiguousarray(x, np.float32), w, s, M, K, N, reps, C.byref(secs)))
        return secs.value

    def rmsnorm(self, x, w):
        x = np.array(x, np.float32, copy=True).reshape(-1, w.shape[0])
        self._check(self._fn("rmsnorm")(x, np.ascontiguousarray(w, np.float32), x.shape[0], x.shape[1]))
        return x

    def rope_tables(self, size, is_local, n_pos=32768, hd=256):
        c = np.zeros((n_pos, hd), np.float32)
        s = np.zeros((n_pos, hd), np.float32)
        self._check(self._fn("rope_tables")(size.encode(), int(is_local), c, s))
        return c, s

    def gelu_table(self, mn, mx, size):
        t = np.zeros(size, np.float32)
        self._check(self._fn("gelu_table")(mn, mx, size, t))
        return t

    def argmax_logits(self, logits):
        return int(self._fn("argmax_logits")(np.ascontiguousarray(logits, np.float32), logits.size))

    def minp_logits(self, logits, minp, temp, randf):
        """returns (token, probabilities) — the input is not modified"""
        p = np.array(logits, np.float32, copy=True)
        tok = int(self._fn("minp_logits")(p, p.size, minp, temp, randf))
        return tok, p

    def mt19937_uniforms(self, seed, n):
        assert self.kind == "port"
        out = np.zeros(n, np.float32)
        self._fn("mt19937_uniforms")(seed, n, out)
        return out

    def module_mlp(self, x, uw, us, gw, gs, dw, ds, pre, post, gelu_size):
        x = np.array(x, np.float32, copy=True)
        S, D = x.shape
        I = uw.shape[1]
        self._check(self._fn("module_mlp")(x, S, D, I, uw, us, gw, gs, dw, ds, pre, post, gelu_size))
        return x

    def module_attention(self, x, is_sw, qw, qs, kw, ks, vw, vs, ow, os_, rmsq, rmsk, pre, post, k_cache=None,
                         v_cache=None):
        x = np.array(x, np.float32, copy=True)
        S, D = x.shape
        n_cached = 0 if k_cache is None else k_cache.shape[0]
        kc = None if k_cache is None else np.ascontiguousarray(k_cache, np.float32).ctypes.data_as(C.c_void_p)
        vc = None if v_cache is None else np.ascontiguousarray(v_cache, np.float32).ctypes.data_as(C.c_void_p)
        self._check(self._fn("module_attention")(x, S, D, int(is_sw), qw, qs, kw, ks, vw, vs, ow, os_, rmsq, rmsk, pre,
                                                 post, n_cached, kc, vc))
        return x

    def module_lm_head(self, x, w, s, rmsw):
        x = np.ascontiguousarray(x, np.float32)
        S, D = x.shape
        logits = np.zeros(VOCAB, np.float32)
        self._check(self._fn("module_lm_head")(logits, x, S, D, w, s, rmsw))
        return logits

    # ------------------------------------------------------------------ model
    def model(self, size: str, path: str) -> "OracleModel":
        return OracleModel(self, size, path)


class OracleModel:
    def __init__(self, o: Oracle, size: str, path: str):
        self.o = o
        self.size = size
        self.h = o._fn("model_create")(size.encode())
        if not self.h:
            raise RuntimeError("model_create failed")
        o._check(o._fn("model_load")(self.h, path.encode()))

    def state(self, gelu_size=1024) -> "OracleState":
        return OracleState(self, gelu_size)

    def close(self):
        if self.h:
            self.o._fn("model_free")(self.h)
            self.h = None


class OracleState:
    def __init__(self, m: OracleModel, gelu_size: int):
        self.m = m
        self.o = m.o
        self.gelu_size = gelu_size
        self.h = self.o._fn("state_create")(m.h, gelu_size)
        if not self.h:
            raise RuntimeError("state_create failed")

    def prefill(self, ids):
        ids = np.ascontiguousarray(ids, np.int32)
        logits = np.zeros(VOCAB, np.float32)
        self.o._check(self.o._fn("prefill")(self.h, ids, ids.size, logits.ctypes.data_as(C.c_void_p)))
        return logits

    def decode(self, tok):
        logits = np.zeros(VOCAB, np.float32)
        self.o._check(self.o._fn("decode")(self.h, int(tok), logits.ctypes.data_as(C.c_void_p)))
        return logits

    def decode_loop(self, first_tok, n_steps, minp=2.0, temp=1.0, randf=None):
        out = np.zeros(n_steps, np.int32)
        rp = None
        if randf is not None:
            randf = np.ascontiguousarray(randf, np.float32)
            assert randf.size >= n_steps
            rp = randf.ctypes.data_as(C.c_void_p)
        self.o._check(self.o._fn("decode_loop")(self.h, int(first_tok), n_steps, minp, temp, rp, out))
        return out

    def kv_info(self, layer):
        a, b, c = C.c_int(), C.c_int(), C.c_int()
        self.o._fn("kv_info")(self.h, layer, C.byref(a), C.byref(b), C.byref(c))
        return a.value, b.value, c.value

    def kv_read(self, layer, slot0, nslots, hd=256):
        k = np.zeros((nslots, hd), np.float32)
        v = np.zeros((nslots, hd), np.float32)
        self.o._fn("kv_read")(self.h, layer, slot0, nslots, k, v)
        return k, v

    def hidden(self, D):
        h = np.zeros(D, np.float32)
        self.o._fn("hidden_read")(self.h, h)
        return h

    def tables(self, n_pos=32768, hd=256):
        t = [np.zeros((n_pos, hd), np.float32) for _ in range(4)] + [np.zeros(self.gelu_size, np.float32)]
        self.o._fn("state_tables")(self.h, *[a.ctypes.data_as(C.c_void_p) for a in t])
        return t

    def set_tables(self, cos_g, sin_g, cos_l, sin_l, gelu):
        assert self.o.kind == "port"
        arrs = [np.ascontiguousarray(a, np.float32) for a in (cos_g, sin_g, cos_l, sin_l, gelu)]
        self.o._fn("state_set_tables")(self.h, *[a.ctypes.data_as(C.c_void_p) for a in arrs])

    def close(self):
        if self.h:
            self.o._fn("state_free")(self.h)
            self.h = None
