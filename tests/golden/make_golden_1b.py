"""Writes tests/golden/ref_e2e_1b_*.npz from the compiled reference (oracle/_ref/libtgref.so) on the
Gemma-3-1B shape with seeded random weights. Run in the build container, commit the outputs:

    python tests/golden/make_golden_1b.py sampled     # ~4 min  -> ref_e2e_1b_sampled.npz
    python tests/golden/make_golden_1b.py long        # ~25 min -> ref_e2e_1b_long.npz
    python tests/golden/make_golden_1b.py batch       # ~5 min  -> ref_e2e_1b_batch.npz

  sampled  (plus 256 steps of the same run with a 2^20-entry table) the benchmarked configuration: 178-token prompt, 1024-entry GeLU table, 1024 decode steps
           with min-p 0.1 / temperature 0.7 and std::mt19937(1234) uniforms (reference
           transformer.hpp:204-234, ops.hpp:762-859): every sampled token, and strided logits of
           every 64th step for the teacher-forced comparison.
  long     16384-token prompt (sliding-window ring filled from the prompt tail, full cache on the
           global layers), 64 greedy steps: prefill logits, token ids, top-2 gaps, logits of the
           first and last step, cache bookkeeping of one local and one global layer.
  batch    16 independent 178-token prompts x 64 greedy steps: token ids, top-2 gaps, last logits.
"""

from __future__ import annotations

import importlib
import os
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, HERE)

import cases  # noqa: E402
from oracle.oracle_api import Oracle  # noqa: E402

synth = importlib.import_module("tiny-gemma_b200.synth")
CACHE = os.environ.get("TG_CACHE_DIR", "/tmp")

# the benchmark's seeds (bench.py)
WEIGHT_SEED, PROMPT_SEED, PROMPT_LEN, SAMPLER_SEED = 0, 77, 178, 1234
MINP, TEMP = 0.1, 0.7
SAMPLED_STEPS, SAMPLED_LOGIT_EVERY = 1024, 64
SMOOTH_STEPS = 256
LONG_PROMPT_SEED, LONG_PROMPT_LEN, LONG_STEPS = 4242, 16384, 64
BATCH_PROMPT_SEED0, BATCH_N, BATCH_STEPS = 9000, 16, 64


def top2_gap(logits):
    t = np.partition(logits, -2)[-2:]
    return float(t.max() - t.min())


def model(R):
    path = synth.write_random_model(os.path.join(CACHE, "tg_1B_s%d.bin" % WEIGHT_SEED), "1B", seed=WEIGHT_SEED)
    return R.model("1B", path)


def sampled(R):
    m = model(R)
    st = m.state(1024)
    ids = synth.random_prompt(PROMPT_LEN, PROMPT_SEED)
    rf = synth.mt19937_uniforms(1 + SAMPLED_STEPS, SAMPLER_SEED)
    out = {"prompt": ids, "uniforms": rf}
    logits = st.prefill(ids)
    out["prefill_logits"] = cases.subsample(logits)
    tok, _ = R.minp_logits(logits.copy(), MINP, TEMP, float(rf[0]))
    toks = [int(tok)]
    t0 = time.time()
    for step in range(SAMPLED_STEPS):
        logits = st.decode(toks[-1])
        if step % SAMPLED_LOGIT_EVERY == 0 or step == SAMPLED_STEPS - 1:
            out["step%d_logits" % step] = cases.subsample(logits)
        tok, _ = R.minp_logits(logits.copy(), MINP, TEMP, float(rf[1 + step]))
        toks.append(int(tok))
        if step % 128 == 0:
            print("sampled step", step, "%.1fs" % (time.time() - t0), flush=True)
    out["tokens"] = np.array(toks, np.int32)  # [0] sampled from the prefill logits, then one per decode step
    st.close()
    # the same run with a 2^20-entry table (no GeLU-bin flips between implementations): the sampler path end to end
    st = m.state(1 << 20)
    logits = st.prefill(ids)
    tok, _ = R.minp_logits(logits.copy(), MINP, TEMP, float(rf[0]))
    toks = [int(tok)]
    for step in range(SMOOTH_STEPS):
        logits = st.decode(toks[-1])
        if step in (0, SMOOTH_STEPS - 1):
            out["smooth_step%d_logits" % step] = cases.subsample(logits)
        tok, _ = R.minp_logits(logits.copy(), MINP, TEMP, float(rf[1 + step]))
        toks.append(int(tok))
    out["smooth_tokens"] = np.array(toks, np.int32)
    st.close()
    np.savez_compressed(os.path.join(HERE, "ref_e2e_1b_sampled.npz"), **out)
    print("ref_e2e_1b_sampled.npz:", len(out), "arrays, distinct tokens", len(set(toks)))


def long_context(R):
    m = model(R)
    out = {}
    ids = synth.random_prompt(LONG_PROMPT_LEN, LONG_PROMPT_SEED)
    for gsz in (1 << 20,):  # the smooth table isolates the kernels from GeLU-bin flips over 16384 positions
        st = m.state(gsz)
        t0 = time.time()
        logits = st.prefill(ids)
        print("long prefill %.0fs" % (time.time() - t0), flush=True)
        out["g%d_prefill_logits" % gsz] = cases.subsample(logits)
        toks, gaps = [int(R.argmax_logits(logits))], [top2_gap(logits)]
        for step in range(LONG_STEPS):
            logits = st.decode(toks[-1])
            if step in (0, LONG_STEPS - 1):
                out["g%d_step%d_logits" % (gsz, step)] = cases.subsample(logits)
            gaps.append(top2_gap(logits))
            toks.append(int(R.argmax_logits(logits)))
        out["g%d_tokens" % gsz] = np.array(toks, np.int32)
        out["g%d_top2_gap" % gsz] = np.array(gaps, np.float32)
        out["g%d_kv_info_l0" % gsz] = np.array(st.kv_info(0), np.int32)  # a sliding-window layer
        out["g%d_kv_info_l5" % gsz] = np.array(st.kv_info(5), np.int32)  # a global layer
        k, v = st.kv_read(0, 0, 4)
        out["g%d_l0_k_first4" % gsz] = k
        k, v = st.kv_read(5, LONG_PROMPT_LEN - 2, 4)
        out["g%d_l5_k_tail4" % gsz] = k
        out["g%d_l5_v_tail4" % gsz] = v
        st.close()
        print("long: min gap", min(gaps), "distinct tokens", len(set(toks)), flush=True)
    out["prompt_seed_len"] = np.array([LONG_PROMPT_SEED, LONG_PROMPT_LEN], np.int32)
    np.savez_compressed(os.path.join(HERE, "ref_e2e_1b_long.npz"), **out)
    print("ref_e2e_1b_long.npz:", len(out), "arrays")


def batch(R):
    m = model(R)
    out = {}
    toks_all, gaps_all, last = [], [], []
    for b in range(BATCH_N):
        st = m.state(1 << 20)
        ids = synth.random_prompt(PROMPT_LEN, BATCH_PROMPT_SEED0 + b)
        logits = st.prefill(ids)
        toks, gaps = [int(R.argmax_logits(logits))], [top2_gap(logits)]
        for step in range(BATCH_STEPS):
            logits = st.decode(toks[-1])
            gaps.append(top2_gap(logits))
            toks.append(int(R.argmax_logits(logits)))
        toks_all.append(toks)
        gaps_all.append(gaps)
        last.append(cases.subsample(logits))
        st.close()
        print("batch sequence", b, "min gap", min(gaps), flush=True)
    out["tokens"] = np.array(toks_all, np.int32)
    out["top2_gap"] = np.array(gaps_all, np.float32)
    out["last_logits"] = np.array(last, np.float32)
    out["prompt_seed0_n_len"] = np.array([BATCH_PROMPT_SEED0, BATCH_N, PROMPT_LEN], np.int32)
    np.savez_compressed(os.path.join(HERE, "ref_e2e_1b_batch.npz"), **out)
    print("ref_e2e_1b_batch.npz:", len(out), "arrays")


if __name__ == "__main__":
    R = Oracle("reference")
    part = sys.argv[1] if len(sys.argv) > 1 else "all"
    if part in ("sampled", "all"):
        sampled(R)
    if part in ("batch", "all"):
        batch(R)
    if part in ("long", "all"):
        long_context(R)
