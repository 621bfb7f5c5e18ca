"""Host-side model of the GPU's exact parallel inverse CDF (cdf_cross_block in
tiny-gemma_b200/csrc/kernels_sampler.cuh), checked against the sequential fp32 chain of
ops::minp_logits (reference ops.hpp:849-857).

Inside a binade [2^e, 2^(e+1)) the running sum is an integer S times u = 2^(e-23); adding p rounds
S + p/u to the nearest integer, ties to even. Element i is therefore the map S -> S + a0[i] (S even)
or S + a1[i] (S odd), such maps compose associatively, and the one addition that leaves the binade
is done in fp32. This file restates that arithmetic with NumPy scalars, composes blocks of maps the
way the kernel's scan does, and compares index and running sum with a plain sequential loop.
"""
import numpy as np

f32 = np.float32
SAT, BIG = 1 << 27, 1 << 25
TINY = f32(7.888609e-31)


def element(p, inv_u):
    x = f32(p) * f32(inv_u)
    if not (x < f32(33554432.0)):
        return (BIG, BIG)
    fl = np.floor(x)
    fr = f32(x - fl)
    q = int(fl)
    if fr == f32(0.5):
        return (q + (q & 1), q + 1 - (q & 1))
    a = q + (1 if fr > f32(0.5) else 0)
    return (a, a)


def compose(f, g):
    return (min(SAT, f[0] + (g[1] if f[0] & 1 else g[0])), min(SAT, f[1] + (g[0] if f[1] & 1 else g[1])))


def apply(f, S):
    return min(SAT, S + (f[1] if S & 1 else f[0]))


def scan_cross(p, randf, cum0=0.0, block=96):
    p = p.astype(f32)
    n, cum, pos, randf = len(p), f32(cum0), 0, f32(randf)
    while pos < n:
        bits = np.array(cum, dtype=f32).view(np.uint32)
        e = int((bits >> 23) & 0xFF) - 127
        if not (cum >= TINY) or e > 120:  # zero / tiny / inf / NaN: plain fp32 steps
            r = -1
            while pos < n and r < 0:
                cum = f32(cum + p[pos])
                if cum >= randf:
                    r = pos
                pos += 1
                if cum >= TINY and cum < f32(1e36):
                    break
            if r >= 0:
                return r, cum
            continue
        u, inv_u = f32(2.0) ** (e - 23), f32(2.0) ** (23 - e)
        S0 = int(cum * inv_u)
        y = randf * inv_u
        T = int(np.ceil(y)) if y < f32(33554432.0) else BIG
        Tmin = min(T, 1 << 24)
        els = [element(p[i], inv_u) for i in range(pos, min(n, pos + block))]
        whole = (0, 0)
        for f in els:
            whole = compose(whole, f)
        S, hit = S0, None
        for k, f in enumerate(els):
            nx = apply(f, S)
            if nx >= Tmin:
                hit = (k, S, nx)
                break
            S = nx
        if hit is None:
            assert apply(whole, S0) == S  # the composed map is the chain
            cum, pos = f32(S) * u, pos + block
            continue
        k, Sb, Sa = hit
        j = pos + k
        if Sa < (1 << 24):
            return j, f32(Sa) * u
        cum, pos = f32(f32(Sb) * u + p[j]), j + 1
        if cum >= randf:
            return j, cum
    return -1, cum


def seq_cross(p, randf, cum0=0.0):
    c = f32(cum0)
    for i, x in enumerate(p.astype(f32)):
        c = f32(c + x)
        if c >= f32(randf):
            return i, c
    return -1, c


def test_scan_model_equals_sequential_chain():
    rng = np.random.default_rng(3)
    for trial in range(120):
        n = int(rng.integers(1, 1500))
        kind = trial % 4
        if kind == 0:
            p = rng.random(n).astype(f32)
            p /= p.sum()
        elif kind == 1:  # dyadic: exact ties are common
            p = (rng.integers(0, 64, size=n) * 2.0 ** -26).astype(f32)
        elif kind == 2:  # wide range, zeros, a few large jumps
            p = (10.0 ** rng.uniform(-12, -4, size=n)).astype(f32)
            p[rng.integers(0, n, size=n // 7 + 1)] = 0
            p[rng.integers(0, n, size=2)] = 0.07
        else:
            p = (rng.integers(0, 8, size=n) * 2.0 ** -25).astype(f32)
        for r in (0.0, float(rng.random() * p.sum()), float(p.sum() * 0.999), 5.0):
            for c0 in (0.0, 0.25, 0.5000001):
                got, want = scan_cross(p, r, c0), seq_cross(p, r, c0)
                assert got[0] == want[0] and f32(got[1]) == f32(want[1]), (trial, r, c0, got, want)
