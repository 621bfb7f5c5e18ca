"""Gemma-3-1B shape against goldens produced by the compiled reference (tests/golden/make_golden_1b.py):
the benchmarked configuration (min-p sampling, 1024-entry GeLU table), the 16384-token long-context
configuration and the batched configuration. All through the C ABI (ctypes)."""

import os

import numpy as np
import pytest

import cases
from conftest import ROOT, rel_l2

pytestmark = pytest.mark.gpu

MINP, TEMP = 0.1, 0.7


def _golden(name):
    p = os.path.join(ROOT, "tests", "golden", name + ".npz")
    if not os.path.exists(p):
        pytest.skip(name + ".npz not generated")
    return np.load(p)


def _tables(model, size, weights, gelu_size):
    """the compiled reference's own RoPE / GeLU tables when its library travelled with the repository
    (isolates the kernels from libm differences in the table builders), else the library's own"""
    from oracle import build_oracle
    from oracle.oracle_api import Oracle, available

    build_oracle.build_ref()
    if not available("reference"):
        model.build_tables(gelu_size)
        return False
    R = Oracle("reference")
    rm = R.model(size, weights)
    rs = rm.state(gelu_size)
    model.set_tables(*rs.tables())
    rs.close()
    rm.close()
    return True


def _ref_probs(logits, minp, temp):
    """ops::minp_logits steps 1-5 (reference ops.hpp:762-845) in float64: the reference's "probabilities"
    (tokens under the cut keep their mass, only the denominator is masked)"""
    z = logits.astype(np.float64) / temp
    p = np.exp(z - z.max())
    denom = p[p >= minp * p.max()].sum()
    return p / denom


def test_e2e_1b_minp_1024_vs_reference_golden(capi, weights_1b):
    """Configuration 3: 178-token prompt, 1024-entry GeLU table, 1024 steps of min-p 0.1 / temperature 0.7
    with the std::mt19937(1234) uniforms, compared with the compiled reference's run (reference
    transformer.hpp:204-234, ops.hpp:762-859).

    The reference's GeLU is a 1024-step lookup table, so two implementations of the same arithmetic differ
    by a few 1e-3 in the logits wherever an activation lands on the other side of a bin edge; on the flat
    distribution of random-init weights that moves the min-p draw to a neighbouring token often enough that
    a free-running comparison says little after the first divergence. The test therefore
      * runs free until the first divergence and requires the first mismatch to be explained: the
        reference's token must own the uniform within the logit noise, judged on our own logits;
      * then feeds the REFERENCE's tokens for all 1024 steps (teacher forced) and requires the logits of
        every stored step within rel-L2 3e-2 and every disagreeing draw explained the same way. The share
        of equal tokens is printed, not asserted: the reference's CDF runs over all 262144 tokens (those
        under the cut keep their mass), so logit noise of relative 1e-2 moves the crossing point by several
        token widths and equal draws are the exception. test_e2e_1b_minp_smooth_table_vs_reference_golden
        holds the token-level bar on the same run with a table that has no bin edges to flip."""
    g = _golden("ref_e2e_1b_sampled")
    m = capi.Model("1B").load_file(weights_1b)
    _tables(m, "1B", weights_1b, 1024)
    prompt, rf, ref_toks = g["prompt"], g["uniforms"], g["tokens"]
    n_steps = len(ref_toks) - 1

    def explained(logits, randf, ref_tok, slack=0.06):
        # the reference's token owns [cum[t-1], cum[t]) of its own CDF; on our logits the interval moves by the
        # logit noise (relative 3e-2 on a flat distribution shifts the CDF by a few percent of its value)
        p = _ref_probs(logits, MINP, TEMP)
        cum = np.cumsum(p)
        lo = cum[ref_tok - 1] if ref_tok > 0 else 0.0
        hi = cum[ref_tok]
        return lo * (1 - slack) - 1e-4 <= randf <= hi * (1 + slack) + 1e-4

    # free-running device loop
    st = m.state(1, 178 + n_steps + 8)
    lg = st.prefill(prompt)[0]
    assert rel_l2(cases.subsample(lg), g["prefill_logits"]) <= 3e-2
    first = st.sample_minp(MINP, TEMP, rf[0:1])
    toks = np.concatenate([first, st.generate(first, n_steps, MINP, TEMP, rf[1:1 + n_steps]).ravel()])
    diff = np.nonzero(toks != ref_toks)[0]
    match_len = int(diff[0]) if diff.size else len(ref_toks)
    print("free-running match length: %d of %d tokens" % (match_len, len(ref_toks)))
    st.close()

    # teacher forced on the reference's tokens
    st = m.state(1, 178 + n_steps + 8)
    lg = st.prefill(prompt)[0]
    agree, unexplained, worst = 0, 0, 0.0
    tok0 = int(st.sample_minp(MINP, TEMP, rf[0:1])[0])
    agree += tok0 == ref_toks[0]
    if tok0 != ref_toks[0] and not explained(lg, float(rf[0]), int(ref_toks[0])):
        unexplained += 1
    for step in range(n_steps):
        lg = st.decode([int(ref_toks[step])])[0]
        key = "step%d_logits" % step
        if key in g.files:
            worst = max(worst, rel_l2(cases.subsample(lg), g[key]))
        t = int(st.sample_minp(MINP, TEMP, rf[1 + step:2 + step])[0])
        if t == ref_toks[step + 1]:
            agree += 1
        elif not explained(lg, float(rf[1 + step]), int(ref_toks[step + 1])):
            unexplained += 1
    print("teacher forced: %d of %d tokens equal, %d unexplained, worst logits rel-L2 %.3g" % (agree, n_steps + 1, unexplained, worst))
    assert worst <= 3e-2
    assert unexplained == 0
    st.close()
    m.close()


def test_e2e_1b_minp_smooth_table_vs_reference_golden(capi, weights_1b):
    """The benchmarked run (same prompt, sampler and uniforms) with a 2^20-entry GeLU table, 256 steps: without
    bin edges the logits agree to 1e-4 and the min-p draw must pick the reference's token in at least 90 % of
    the teacher-forced steps, every other one explained by a CDF crossing within the logit noise."""
    g = _golden("ref_e2e_1b_sampled")
    if "smooth_tokens" not in g.files:
        pytest.skip("golden predates the smooth-table run")
    m = capi.Model("1B").load_file(weights_1b)
    exact = _tables(m, "1B", weights_1b, 1 << 20)
    tol = 2e-4 if exact else 1e-3
    prompt, rf, ref_toks = g["prompt"], g["uniforms"], g["smooth_tokens"]
    n_steps = len(ref_toks) - 1

    st = m.state(1, 178 + n_steps + 8)
    st.prefill(prompt, want_logits=False)
    first = st.sample_minp(MINP, TEMP, rf[0:1])
    toks = np.concatenate([first, st.generate(first, n_steps, MINP, TEMP, rf[1:1 + n_steps]).ravel()])
    diff = np.nonzero(toks != ref_toks)[0]
    match_len = int(diff[0]) if diff.size else len(ref_toks)
    print("smooth table, free-running match length: %d of %d tokens" % (match_len, len(ref_toks)))
    st.close()

    st = m.state(1, 178 + n_steps + 8)
    st.prefill(prompt, want_logits=False)
    agree = int(st.sample_minp(MINP, TEMP, rf[0:1])[0] == ref_toks[0])
    bad = []
    for step in range(n_steps):
        lg = st.decode([int(ref_toks[step])])[0]
        key = "smooth_step%d_logits" % step
        if key in g.files:
            assert rel_l2(cases.subsample(lg), g[key]) <= tol
        t = int(st.sample_minp(MINP, TEMP, rf[1 + step:2 + step])[0])
        if t == ref_toks[step + 1]:
            agree += 1
        else:
            cum = np.cumsum(_ref_probs(lg, MINP, TEMP))
            r, rt = float(rf[1 + step]), int(ref_toks[step + 1])
            lo, hi = (cum[rt - 1] if rt else 0.0), cum[rt]
            if not (lo * (1 - 2e-3) - 1e-5 <= r <= hi * (1 + 2e-3) + 1e-5):
                bad.append(step)
    print("smooth table, teacher forced: %d of %d tokens equal, unexplained steps %s" % (agree, n_steps + 1, bad))
    assert not bad
    assert agree >= 0.90 * (n_steps + 1)  # measured: 239 of 257
    st.close()
    m.close()


def test_e2e_1b_long_context_vs_reference_golden(capi, synth, weights_1b):
    """Configuration 4: 16384-token prompt (the sliding-window ring is filled from the prompt tail, reference
    decode.hpp:84-103; a sliding-window query sees 513 keys in the prefill, ops.hpp:437-443) and 64 greedy
    steps, 2^20-entry GeLU table, against the compiled reference's run."""
    g = _golden("ref_e2e_1b_long")
    seed, S = (int(v) for v in g["prompt_seed_len"])
    m = capi.Model("1B").load_file(weights_1b)
    exact = _tables(m, "1B", weights_1b, 1 << 20)
    tol = 2e-4 if exact else 1e-3
    ids = synth.random_prompt(S, seed)
    st = m.state(1, S + 80)
    lg = st.prefill(ids)[0]
    assert rel_l2(cases.subsample(lg), g["g1048576_prefill_logits"]) <= tol
    ref_toks, gaps = g["g1048576_tokens"], g["g1048576_top2_gap"]
    steps = len(ref_toks) - 1
    tok = int(st.sample_argmax()[0])
    if gaps[0] > 1e-3:
        assert tok == ref_toks[0]
    for step in range(steps):
        lg = st.decode([int(ref_toks[step])])[0]  # teacher forced: a near-tie must not derail the later steps
        key = "g1048576_step%d_logits" % step
        if key in g.files:
            assert rel_l2(cases.subsample(lg), g[key]) <= tol
        tok = int(st.sample_argmax()[0])
        if gaps[step + 1] > 1e-3:
            assert tok == ref_toks[step + 1], "step %d" % step
    assert st.position() == S + steps
    # cache rows: first slots of a sliding-window layer (prompt tail), last rows of a global layer
    k, v = st.kv_read(0, 0, 4)
    assert rel_l2(k, g["g1048576_l0_k_first4"]) <= tol
    k, v = st.kv_read(5, S - 2, 4)
    assert rel_l2(k, g["g1048576_l5_k_tail4"]) <= tol
    assert rel_l2(v, g["g1048576_l5_v_tail4"]) <= tol
    st.close()
    m.close()


def test_e2e_1b_batched_vs_reference_golden(capi, synth, weights_1b):
    """Configuration 5 (subset): the reference's 16 seeded 178-token prompts x 64 greedy steps are the first 16
    rows of a 32-sequence state (the batched tensor-core step: M = batch); the other rows are unrelated prompts.
    Tokens must equal the reference's wherever its own top-2 gap is above the noise, logits within tolerance."""
    g = _golden("ref_e2e_1b_batch")
    seed0, n_ref, plen = (int(v) for v in g["prompt_seed0_n_len"])
    m = capi.Model("1B").load_file(weights_1b)
    exact = _tables(m, "1B", weights_1b, 1 << 20)
    tol = 2e-4 if exact else 1e-3
    B = 32
    prompts = np.stack([synth.random_prompt(plen, seed0 + b) for b in range(B)])
    ref_toks, gaps = g["tokens"], g["top2_gap"]
    steps = ref_toks.shape[1] - 1
    st = m.state(B, plen + steps + 8)
    st.prefill(prompts, want_logits=False)
    tok = st.sample_argmax()
    feed = tok.copy()
    for b in range(n_ref):
        if gaps[b, 0] > 1e-3:
            assert tok[b] == ref_toks[b, 0]
        feed[b] = ref_toks[b, 0]
    for step in range(steps):
        lg = st.decode(feed, want_logits=(step == steps - 1))
        tok = st.sample_argmax()
        feed = tok.copy()
        for b in range(n_ref):
            if gaps[b, step + 1] > 1e-3:
                assert tok[b] == ref_toks[b, step + 1], "sequence %d step %d" % (b, step)
            feed[b] = ref_toks[b, step + 1]  # teacher forced on the reference rows
    for b in range(n_ref):
        assert rel_l2(cases.subsample(lg[b]), g["last_logits"][b]) <= tol
    st.close()
    m.close()


def test_append_equals_decode_steps_1b(capi, synth, weights_1b):
    """tg_append (continuation of a non-empty context) against the same tokens fed through tg_decode."""
    m = capi.Model("1B").load_file(weights_1b)
    m.build_tables(1 << 20)
    ids = synth.random_prompt(64, 5)
    more = synth.random_prompt(24, 6)
    a = m.state(1, 256)
    a.prefill(ids, want_logits=False)
    la = a.append(more)[0]
    b = m.state(1, 256)
    b.prefill(ids, want_logits=False)
    for t in more:
        lb = b.decode([int(t)])[0]
    assert a.position() == b.position() == 88
    assert rel_l2(la, lb) <= 1e-6
    # a second turn on top of it
    la = a.append(ids[:8])[0]
    for t in ids[:8]:
        lb = b.decode([int(t)])[0]
    assert rel_l2(la, lb) <= 1e-6
    a.close()
    b.close()
    m.close()


def test_chained_launches_equal_one_launch_1b(capi, synth, weights_1b):
    """The persistent decode kernel leaves its hand-off arena and its grid-barrier counter ready for the
    next launch instead of having the host reset them. 26 layers rotate over three arena copies, so launches
    of 1, 2 and 3 tokens end on every phase of the rotation; greedy and min-p launches (1 and 3 grid barriers
    per token) are mixed. The tokens must equal those of single launches over the same steps."""
    m = capi.Model("1B").load_file(weights_1b)
    m.build_tables(1 << 20)
    ids = synth.random_prompt(40, 17)
    rf = np.random.default_rng(3).random(24, dtype=np.float32)

    def start():
        st = m.state(1, 128)
        st.prefill(ids, want_logits=False)
        return st, st.sample_argmax()

    st, first = start()
    want_g = st.generate(first, 12).ravel()
    want_s = st.generate(want_g[-1:], 12, MINP, TEMP, rf[:12]).ravel()
    st.close()
    st, first = start()
    got, tok = [], first
    for n in (1, 2, 3, 1, 1, 2, 2):
        out = st.generate(tok, n).ravel()
        got += [int(t) for t in out]
        tok = out[-1:]
    assert got == [int(t) for t in want_g]
    got, used = [], 0
    for n in (1, 1, 3, 2, 1, 1, 3):
        out = st.generate(tok, n, MINP, TEMP, rf[used:used + n]).ravel()
        got += [int(t) for t in out]
        tok = out[-1:]
        used += n
    assert got == [int(t) for t in want_s]
    st.close()
    m.close()
