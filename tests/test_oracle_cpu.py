"""CPU suite, part 1: the oracle restatement (oracle/tg_oracle.cpp) pinned
against (a) fixtures computed by the reference's own NumPy model, (b) outputs
of the compiled reference committed as golden vectors, and (c) — where
oracle/_ref/libtgref.so is present — the compiled reference run live."""

import numpy as np
import pytest

import cases
from conftest import rel_l2, rel_max


# ---------------------------------------------------------------- (a) NumPy-model fixtures
# tolerances are the reference's own (tests/csrc/test_bench_modules.cpp:79,187,266,338,405,485):
# rel-L2 1e-3 on every module.
@pytest.mark.parametrize("S", [1, 57])
def test_port_mlp_vs_numpy_model(port, golden, S):
    c = cases.mlp_case(S)
    y = port.module_mlp(c["x"], c["uw"], c["us"], c["gw"], c["gs"], c["dw"], c["ds"], c["pre"], c["post"], 8192)
    assert rel_l2(y, golden["numpy_modules"]["mlp_S%d" % S]) < 1e-3


@pytest.mark.parametrize("S", [57, 217])
def test_port_attention_prefill_vs_numpy_model(port, golden, S):
    c = cases.attention_case(S)
    y = port.module_attention(c["x"], 0, c["qw"], c["qs"], c["kw"], c["ks"], c["vw"], c["vs"], c["ow"], c["os"],
                              c["rmsq"], c["rmsk"], c["pre"], c["post"])
    assert rel_l2(y, golden["numpy_modules"]["attn_prefill_S%d" % S]) < 1e-3


@pytest.mark.parametrize("N", [57, 389])
def test_port_attention_decode_vs_numpy_model(port, golden, N):
    c = cases.attention_case(1, N)
    kc = golden["numpy_modules"]["attn_decode_N%d_kcache" % N]
    y = port.module_attention(c["x"], 0, c["qw"], c["qs"], c["kw"], c["ks"], c["vw"], c["vs"], c["ow"], c["os"],
                              c["rmsq"], c["rmsk"], c["pre"], c["post"], kc, c["v_cache"])
    assert rel_l2(y, golden["numpy_modules"]["attn_decode_N%d" % N]) < 1e-3


@pytest.mark.parametrize("S", [1, 57])
def test_port_lm_head_vs_numpy_model(port, golden, S):
    c = cases.lm_head_case(S)
    logits = port.module_lm_head(c["x"], c["w"], c["s"], c["rmsw"])
    assert rel_l2(cases.subsample(logits), golden["numpy_modules"]["lm_head_S%d" % S]) < 1e-3
    assert int(np.argmax(logits)) == int(golden["numpy_modules"]["lm_head_S%d_argmax" % S])


# ---------------------------------------------------------------- (b) compiled-reference goldens
@pytest.mark.parametrize("K,N", cases.SWEEP_SHAPES)
@pytest.mark.parametrize("M", [1, 16])
def test_port_linear_bit_exact_vs_reference_golden(port, golden, K, N, M):
    x, w, s = cases.linear_case(K, N, M)
    y = port.linear_decode(x[0], w, s) if M == 1 else port.linear_prefill(x, w, s)
    want = golden["ref_ops"]["linear_%d_%d_M%d" % (K, N, M)]
    assert np.array_equal(cases.subsample(y, 16), want)  # integer->fp32 products and the k order are exact


def test_port_lm_head_matvec_bit_exact_vs_reference_golden(port, golden):
    K, N = cases.LM_HEAD_SHAPE
    x, w, s = cases.linear_case(K, N, 1)
    y = port.lm_head_decode(x[0], w, s)
    assert np.array_equal(cases.subsample(y, 16), golden["ref_ops"]["linear_%d_%d_M1" % (K, N)])


@pytest.mark.parametrize("dim", [256, 640, 1152])
def test_port_rmsnorm_vs_reference_golden(port, golden, dim):
    g = golden["ref_ops"]
    y = port.rmsnorm(g["rmsnorm_%d_x" % dim], g["rmsnorm_%d_w" % dim])
    # the compiled reference uses the RSQRTSS estimate + one Newton step; 1/sqrtf differs by <= ~2 ulp
    assert rel_max(y, g["rmsnorm_%d" % dim]) < 5e-7


def test_port_samplers_vs_reference_golden(port, golden):
    g = golden["ref_ops"]
    for kind in ("flat", "peaked", "ties", "nan"):
        assert port.argmax_logits(cases.logits_case(kind)) == int(g["argmax_" + kind])
    for kind, minp, temp in (("flat", 0.1, 0.7), ("peaked", 0.1, 0.7), ("peaked", 0.05, 1.0)):
        lg = cases.logits_case(kind)
        key = "minp_%s_%g_%g" % (kind, minp, temp)
        toks = [port.minp_logits(lg, minp, temp, r)[0] for r in (0.01, 0.25, 0.5, 0.75, 0.99)]
        assert toks == list(g[key + "_tokens"])
        p = port.minp_logits(lg, minp, temp, 0.5)[1]
        assert rel_max(cases.subsample(p, 64), g[key + "_probs"]) < 1e-6
        # the reference's quirk: sub-threshold tokens keep their mass, so the row sums to > 1
        assert abs(p.astype(np.float64).sum() - float(g[key + "_sum"])) < 1e-4 * float(g[key + "_sum"])


def test_argmax_edge_cases(port):
    x = np.full(262144, -np.inf, np.float32)
    assert port.argmax_logits(x) == -1  # nothing above -inf (ops.hpp:748-757)
    x[1000] = 1.0
    x[999] = 1.0
    assert port.argmax_logits(x) == 999  # lowest index wins ties
    x[5] = np.nan
    assert port.argmax_logits(x) == 999  # NaN never wins


def test_port_tables_vs_reference_golden(port, golden):
    g = golden["ref_ops"]
    assert np.array_equal(port.gelu_table(-4.0, 4.0, 1024), g["gelu_1024"])
    rows = [0, 1, 177, 511, 4095, 32767]
    for loc, name in ((1, "local"), (0, "global")):
        c, s = port.rope_tables("270m", loc)
        # float pow/cos/sin through scalar libm here vs glibc's vector libm in the
        # reference build: frequencies differ by a few ulp, which the position
        # multiplies (<= 2e-3 at position 32767)
        for i, r in enumerate(rows):
            tol = 1e-6 + 1.5e-7 * r
            assert np.abs(c[r] - g["rope_%s_cos_rows" % name][i]).max() <= tol
            assert np.abs(s[r] - g["rope_%s_sin_rows" % name][i]).max() <= tol


def test_port_e2e_270m_vs_reference_golden(port, golden, weights_270m):
    """short end-to-end run of the port against the committed reference run
    (same seeded weights): 2^20-entry GeLU table so that table bin flips do not
    mask arithmetic differences."""
    g = golden["ref_e2e_270m"]
    m = port.model("270m", weights_270m)
    st = m.state(1 << 20)
    ids = g["prompt"][:40]
    # the golden prompt is 178 tokens; run the port on it fully only for prefill
    logits = st.prefill(g["prompt"])
    # RoPE tables of the port differ slightly from the reference build's (see
    # above), hence 2e-4 rather than the ~1e-5 seen with identical tables
    assert rel_l2(cases.subsample(logits), g["g1048576_prefill_logits"]) < 2e-4
    toks = g["g1048576_tokens"]
    assert int(np.argmax(logits)) == int(toks[0])
    for step in range(3):
        logits = st.decode(int(toks[step]))
        assert int(np.argmax(logits)) == int(toks[step + 1])
        assert rel_l2(cases.subsample(logits), g["g1048576_step%d_logits" % step]) < 2e-4
    k, v = st.kv_read(0, 0, 8)
    assert rel_max(k, g["g1048576_l0_k_first8"]) < 1e-5
    assert rel_max(v, g["g1048576_l0_v_first8"]) < 1e-5
    st.close()
    m.close()
    del ids


# ---------------------------------------------------------------- (c) live compiled reference
def test_port_vs_live_reference_ops(port, ref):
    for K, N in [(640, 1024), (1152, 6912), (6912, 1152)]:
        x, w, s = cases.linear_case(K, N, 5, seed=7)
        assert np.array_equal(port.linear_decode(x[0], w, s), ref.linear_decode(x[0], w, s))
        assert np.array_equal(port.linear_prefill(x, w, s), ref.linear_prefill(x, w, s))
    c = cases.mlp_case(7)
    a = port.module_mlp(c["x"], c["uw"], c["us"], c["gw"], c["gs"], c["dw"], c["ds"], c["pre"], c["post"], 8192)
    b = ref.module_mlp(c["x"], c["uw"], c["us"], c["gw"], c["gs"], c["dw"], c["ds"], c["pre"], c["post"], 8192)
    assert rel_l2(a, b) < 5e-6
    for sw in (0, 1):
        c = cases.attention_case(40)
        args = (c["qw"], c["qs"], c["kw"], c["ks"], c["vw"], c["vs"], c["ow"], c["os"], c["rmsq"], c["rmsk"], c["pre"],
                c["post"])
        assert rel_l2(port.module_attention(c["x"], sw, *args), ref.module_attention(c["x"], sw, *args)) < 5e-6


def test_mt19937_uniforms_match_libstdcxx(port, synth):
    for seed in (0, 1, 1234567):
        assert np.array_equal(synth.mt19937_uniforms(64, seed), port.mt19937_uniforms(seed, 64))


def test_weight_file_layout(synth, weights_270m):
    import os

    assert os.path.getsize(weights_270m) == synth.file_size("270m") == 437586944
    assert synth.file_size("1B") == 1305168896
    lay = dict((n, (dt, sh, off)) for n, dt, sh, off in synth.layout("270m"))
    assert lay["wte.q"][2] == 0 and lay["final_norm"][2] == 262144 * 640 + 4 * 640
    # every tensor starts on a 256-byte boundary (what the kernels' 128-bit loads rely on)
    assert all(off % 256 == 0 for _, _, _, off in synth.layout("270m"))
    assert all(off % 256 == 0 for _, _, _, off in synth.layout("1B"))
    # quantiser: one scale per column, max|q| == 127 in every column
    q, s = synth.quantize_weight(np.random.default_rng(0).standard_normal((64, 32)).astype(np.float32))
    assert s.shape == (1, 32) and np.all(np.abs(q).max(axis=0) == 127)
