"""Writes tests/golden/*.npz from the reference itself. Needs the reference
checkout (default /root/reference) and oracle/_ref/libtgref.so; run it in the
build container, commit the outputs:

    python tests/golden/make_golden.py

Two families:
  * numpy_modules.npz — expected outputs of modules::mlp / attention / lm_head
    computed with the reference's own NumPy model (py/gemma.py), the way its
    unit tests do (tests/test_bench_modules.py): fp32 NumPy on dequantised
    weights. Tolerance of those tests: rel-L2 1e-3.
  * ref_e2e_270m.npz — the compiled reference (AVX2, Makefile flags) run end to
    end on seeded random 270m weights: greedy token ids for 256 steps and
    strided logits of selected steps, for GeLU tables of 1024 entries (what
    generate() uses) and 2^20 entries (isolates kernels from LUT bin flips).
  * ref_ops.npz — compiled-reference outputs of the isolated matvec / GEMM
    sweep (strided), RMSNorm, samplers.
"""

from __future__ import annotations

import importlib
import math
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REFERENCE = os.environ.get("TINY_GEMMA_REFERENCE", "/root/reference")
sys.path.insert(0, ROOT)
sys.path.insert(0, REFERENCE)
sys.path.insert(0, HERE)

import cases  # noqa: E402
from oracle.oracle_api import Oracle  # noqa: E402

synth = importlib.import_module("tiny-gemma_b200.synth")

# Prompt seed 10 gives a greedy run whose smallest top-1/top-2 logit gap over all
# 257 positions is 0.046 — far above the ~1e-2 logit noise that GeLU-table bin
# flips cause between any two implementations — so token-for-token equality is
# a meaningful test. Seed 123 has a 0.002 near-tie and is kept as the
# teacher-forced case.
E2E_PROMPT_SEED, E2E_PROMPT_LEN, E2E_STEPS = 10, 178, 256
NEAR_TIE_PROMPT_SEED = 123
E2E_LOGIT_STEPS = [0, 1, 2, 63, 255]
CACHE = os.environ.get("TG_CACHE_DIR", "/tmp")


def numpy_modules():
    import py.gemma as G
    from py.weight_handlers import dequantize
    from einops import rearrange

    out = {}
    cos, sin = G.precompute_freqs_cis(256, 32768, 1_000_000.0)

    for S in (1, 57):
        c = cases.mlp_case(S)
        x = c["x"][None]
        h = G.rmsnorm(x, c["pre"])
        act = G.gelu(G.linear(h, dequantize(c["gw"], c["gs"]))) * G.linear(h, dequantize(c["uw"], c["us"]))
        y = x + G.rmsnorm(G.linear(act, dequantize(c["dw"], c["ds"])), c["post"])
        out["mlp_S%d" % S] = y[0].astype(np.float32)

    def attn(c, S, n_cached):
        x = c["x"][None]
        a0 = G.rmsnorm(x, c["pre"])
        q = G.linear(a0, dequantize(c["qw"], c["qs"]))
        k = G.linear(a0, dequantize(c["kw"], c["ks"]))
        v = G.linear(a0, dequantize(c["vw"], c["vs"]))
        q = rearrange(q, "b l (h d) -> b h l d", h=4)
        k = rearrange(k, "b l d -> b 1 l d")
        v = rearrange(v, "b l d -> b 1 l d")
        q = G.rmsnorm(q, c["rmsq"])
        k = G.rmsnorm(k, c["rmsk"])
        q, k = G.apply_rotary_emb(q, k, cos, sin, offset=n_cached)
        if n_cached:
            kc = G.rmsnorm(c["k_raw"][None, None], c["rmsk"])
            kc, _ = G.apply_rotary_emb(kc, kc, cos, sin, offset=0)
            k = np.concatenate([kc, k], axis=-2)
            v = np.concatenate([c["v_cache"][None, None], v], axis=-2)
        o = G.attention(q, k, v, 1.0 / math.sqrt(256), max_len=32768)
        o = rearrange(o, "b h l d -> b l (h d)")
        y = x + G.rmsnorm(G.linear(o, dequantize(c["ow"], c["os"])), c["post"])
        return y[0].astype(np.float32), (kc[0, 0].astype(np.float32) if n_cached else None)

    for S in (57, 217):
        c = cases.attention_case(S)
        out["attn_prefill_S%d" % S], _ = attn(c, S, 0)
    for n in (57, 389):
        c = cases.attention_case(1, n)
        y, kc = attn(c, 1, n)
        out["attn_decode_N%d" % n] = y
        out["attn_decode_N%d_kcache" % n] = kc  # normed + roped keys handed to the C++ side

    for S in (1, 57):
        c = cases.lm_head_case(S)
        h = G.rmsnorm(c["x"][None, -1:], c["rmsw"])
        logits = G.linear(h, dequantize(c["w"], c["s"][None]))
        out["lm_head_S%d" % S] = cases.subsample(logits.astype(np.float32))
        out["lm_head_S%d_argmax" % S] = np.int32(np.argmax(logits))
    np.savez_compressed(os.path.join(HERE, "numpy_modules.npz"), **out)
    print("numpy_modules.npz:", sorted(out))


def ref_ops(R: Oracle):
    out = {}
    for K, N in cases.SWEEP_SHAPES + [cases.LM_HEAD_SHAPE]:
        for M in (1, 16):
            if N == 262144 and M > 1:
                continue
            x, w, s = cases.linear_case(K, N, M)
            if M == 1:
                y = R.lm_head_decode(x[0], w, s) if N == 262144 else R.linear_decode(x[0], w, s)
            else:
                y = R.linear_prefill(x, w, s)
            out["linear_%d_%d_M%d" % (K, N, M)] = cases.subsample(y, 16)
    rng = np.random.default_rng(5)
    for dim in (256, 640, 1152):
        x = (rng.standard_normal((8, dim), dtype=np.float32) * 3).astype(np.float32)
        w = (rng.standard_normal(dim, dtype=np.float32) * 0.1).astype(np.float32)
        out["rmsnorm_%d" % dim] = R.rmsnorm(x, w)
        out["rmsnorm_%d_x" % dim] = x
        out["rmsnorm_%d_w" % dim] = w
    for kind in ("flat", "peaked", "ties", "nan"):
        lg = cases.logits_case(kind)
        out["argmax_" + kind] = np.int32(R.argmax_logits(lg))
    for kind, minp, temp in (("flat", 0.1, 0.7), ("peaked", 0.1, 0.7), ("peaked", 0.05, 1.0)):
        lg = cases.logits_case(kind)
        toks = []
        for r in (0.01, 0.25, 0.5, 0.75, 0.99):
            t, p = R.minp_logits(lg, minp, temp, r)
            toks.append(t)
        key = "minp_%s_%g_%g" % (kind, minp, temp)
        out[key + "_tokens"] = np.array(toks, np.int32)
        out[key + "_probs"] = cases.subsample(p, 64)
        out[key + "_sum"] = np.float64(p.astype(np.float64).sum())
    out["gelu_1024"] = R.gelu_table(-4.0, 4.0, 1024)
    c, s = R.rope_tables("270m", 1)
    out["rope_local_cos_rows"] = c[[0, 1, 177, 511, 4095, 32767]]
    out["rope_local_sin_rows"] = s[[0, 1, 177, 511, 4095, 32767]]
    c, s = R.rope_tables("270m", 0)
    out["rope_global_cos_rows"] = c[[0, 1, 177, 511, 4095, 32767]]
    out["rope_global_sin_rows"] = s[[0, 1, 177, 511, 4095, 32767]]
    np.savez_compressed(os.path.join(HERE, "ref_ops.npz"), **out)
    print("ref_ops.npz:", len(out), "arrays")


def ref_e2e(R: Oracle):
    path = synth.write_random_model(os.path.join(CACHE, "tg_270m_s0.bin"), "270m", seed=0)
    m = R.model("270m", path)
    ids = synth.random_prompt(E2E_PROMPT_LEN, E2E_PROMPT_SEED)
    out = {"prompt": ids}
    for gsz in (1024, 1 << 20):
        st = m.state(gsz)
        logits = st.prefill(ids)
        out["g%d_prefill_logits" % gsz] = cases.subsample(logits)
        toks = [int(np.argmax(logits))]  # argmax_logits == first max
        assert toks[0] == R.argmax_logits(logits)
        top2 = np.partition(logits, -2)[-2:]
        gaps = [float(top2.max() - top2.min())]
        for step in range(E2E_STEPS):
            logits = st.decode(toks[-1])
            if step in E2E_LOGIT_STEPS:
                out["g%d_step%d_logits" % (gsz, step)] = cases.subsample(logits)
            top2 = np.partition(logits, -2)[-2:]
            gaps.append(float(top2.max() - top2.min()))
            toks.append(R.argmax_logits(logits))
        out["g%d_tokens" % gsz] = np.array(toks, np.int32)  # [0] from prefill, then 256 decode steps
        out["g%d_top2_gap" % gsz] = np.array(gaps, np.float32)
        out["g%d_hidden_last" % gsz] = st.hidden(640)
        k, v = st.kv_read(0, 0, 8)
        out["g%d_l0_k_first8" % gsz] = k
        out["g%d_l0_v_first8" % gsz] = v
        k, v = st.kv_read(5, 170, 16)
        out["g%d_l5_k_170_186" % gsz] = k
        out["g%d_l5_v_170_186" % gsz] = v
        st.close()
        print("gelu", gsz, "distinct tokens", len(set(toks)), "min gap", min(gaps))
    # near-tie prompt, reference configuration (1024-entry table): tokens + gaps only
    ids3 = synth.random_prompt(E2E_PROMPT_LEN, NEAR_TIE_PROMPT_SEED)
    st = m.state(1024)
    logits = st.prefill(ids3)
    toks, gaps = [], []
    for step in range(E2E_STEPS + 1):
        top2 = np.partition(logits, -2)[-2:]
        gaps.append(float(top2.max() - top2.min()))
        toks.append(R.argmax_logits(logits))
        if step < E2E_STEPS:
            logits = st.decode(toks[-1])
    out["tie_prompt"] = ids3
    out["tie_tokens"] = np.array(toks, np.int32)
    out["tie_top2_gap"] = np.array(gaps, np.float32)
    st.close()
    # short sliding-window case: prompt longer than the 512-slot ring
    ids2 = synth.random_prompt(600, 321)
    st = m.state(1 << 20)
    logits = st.prefill(ids2)
    out["sw_prompt"] = ids2
    out["sw_prefill_logits"] = cases.subsample(logits)
    toks = [int(R.argmax_logits(logits))]
    for step in range(8):
        logits = st.decode(toks[-1])
        toks.append(R.argmax_logits(logits))
    out["sw_tokens"] = np.array(toks, np.int32)
    out["sw_last_logits"] = cases.subsample(logits)
    out["sw_kv_info_l0"] = np.array(st.kv_info(0), np.int32)
    k, v = st.kv_read(0, 0, 10)
    out["sw_l0_k_first10"] = k
    st.close()
    np.savez_compressed(os.path.join(HERE, "ref_e2e_270m.npz"), **out)
    print("ref_e2e_270m.npz:", len(out), "arrays")


if __name__ == "__main__":
    R = Oracle("reference")
    numpy_modules()
    ref_ops(R)
    ref_e2e(R)
