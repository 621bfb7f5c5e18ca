"""Seeded inputs for the golden fixtures. Pure NumPy and deterministic, so the
big tensors (int8 weights) are rebuilt from their seed wherever the tests run
and only the expected OUTPUTS are committed (tests/golden/*.npz, written by
make_golden.py in a container that has the reference checkout)."""

from __future__ import annotations

import numpy as np

HEAD_DIM, N_HEAD, VOCAB = 256, 4, 262144


def quantize(w: np.ndarray):
    # reference py/weight_handlers.py:10-20
    s = (np.max(np.abs(w), axis=0, keepdims=True) / 127.0).astype(np.float32)
    return np.rint(w / s).astype(np.int8), np.ascontiguousarray(s.ravel())


def _lin(rng, K, N):
    w = (rng.standard_normal((K, N), dtype=np.float32) * np.float32(1.0 / np.sqrt(K))).astype(np.float32)
    return quantize(w)


def _vec(rng, n, std=1.0):
    return (rng.standard_normal(n, dtype=np.float32) * np.float32(std)).astype(np.float32)


def mlp_case(S: int, D: int = 640, I: int = 2048, seed: int = 11):
    """inputs of modules::mlp (reference tests/test_bench_modules.py:386-473 shapes)"""
    rng = np.random.default_rng(seed + S)
    uw, us = _lin(rng, D, I)
    gw, gs = _lin(rng, D, I)
    dw, ds = _lin(rng, I, D)
    return dict(x=_vec(rng, S * D).reshape(S, D), uw=uw, us=us, gw=gw, gs=gs, dw=dw, ds=ds,
                pre=_vec(rng, D), post=_vec(rng, D))


def attention_case(S: int, n_cached: int = 0, D: int = 640, seed: int = 23):
    """inputs of modules::attention: S > 1 prefill on an empty cache, or S == 1
    decode against n_cached pre-filled slots (keys already normed + roped at
    positions 0..n_cached-1, as reference tests/test_bench_modules.py:268-300)"""
    rng = np.random.default_rng(seed + 7 * S + n_cached)
    qd = N_HEAD * HEAD_DIM
    qw, qs = _lin(rng, D, qd)
    kw, ks = _lin(rng, D, HEAD_DIM)
    vw, vs = _lin(rng, D, HEAD_DIM)
    ow, os_ = _lin(rng, qd, D)
    c = dict(x=_vec(rng, S * D).reshape(S, D), qw=qw, qs=qs, kw=kw, ks=ks, vw=vw, vs=vs, ow=ow, os=os_,
             rmsq=_vec(rng, HEAD_DIM), rmsk=_vec(rng, HEAD_DIM), pre=_vec(rng, D), post=_vec(rng, D))
    if n_cached:
        c["k_raw"] = _vec(rng, n_cached * HEAD_DIM).reshape(n_cached, HEAD_DIM)
        c["v_cache"] = _vec(rng, n_cached * HEAD_DIM).reshape(n_cached, HEAD_DIM)
    return c


def lm_head_case(S: int, D: int = 640, seed: int = 37):
    rng = np.random.default_rng(seed + S)
    w = rng.integers(-127, 128, size=(D, VOCAB), dtype=np.int8)
    s = np.exp(rng.uniform(np.log(1e-4), np.log(1e-2), size=VOCAB)).astype(np.float32)
    return dict(x=_vec(rng, S * D).reshape(S, D), w=w, s=s, rmsw=_vec(rng, D, 0.1))


# the isolated-op sweep of the benchmark configuration: K x N shapes, int8
# weights uniform in [-127,127], scales log-uniform in [1e-4,1e-2], x ~ N(0,1)
SWEEP_SHAPES = [(640, 1024), (640, 2048), (2048, 640), (1152, 1024), (1152, 6912), (6912, 1152)]
LM_HEAD_SHAPE = (1152, 262144)


def linear_case(K: int, N: int, M: int, seed: int = 101):
    rng = np.random.default_rng(seed + K * 7 + N * 3 + M)
    w = rng.integers(-127, 128, size=(K, N), dtype=np.int8)
    s = np.exp(rng.uniform(np.log(1e-4), np.log(1e-2), size=N)).astype(np.float32)
    x = rng.standard_normal((M, K), dtype=np.float32)
    return x, w, s


def logits_case(kind: str, seed: int = 53):
    """synthetic logits rows for the sampler tests"""
    rng = np.random.default_rng(seed)
    x = (rng.standard_normal(VOCAB, dtype=np.float32) * np.float32(0.7)).astype(np.float32)
    if kind == "flat":
        x[200000] = 6.0
    elif kind == "peaked":
        x = (x * np.float32(4.0)).astype(np.float32)
        x[[17, 9000, 131071, 250000]] += np.float32(14.0)
    elif kind == "ties":
        x[[5, 77, 100000]] = np.float32(9.5)
    elif kind == "nan":
        x[3] = np.nan
        x[262143] = np.float32(8.0)
    return x


def subsample(v: np.ndarray, stride: int = 64) -> np.ndarray:
    return np.ascontiguousarray(v.reshape(-1)[::stride])
