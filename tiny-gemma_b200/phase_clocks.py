"""Per-phase timing of the persistent decode kernel.

    python tiny-gemma_b200/phase_clocks.py [270m|1B] [minp|greedy]

Arms the kernel's recorder (tg_state_phase_clocks), runs 16 tokens twice and
prints, for the last token of the second run, the time CTA 0 spent in each
section of each layer (SM clock stamps / 1965 MHz), the lm_head and the sampler.
"""
import importlib
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import numpy as np
capi = importlib.import_module("tiny-gemma_b200.capi"); synth = importlib.import_module("tiny-gemma_b200.synth")
size = sys.argv[1] if len(sys.argv)>1 else "1B"
sampler = sys.argv[2] if len(sys.argv)>2 else "minp"
path = synth.write_random_model(os.path.join(os.environ.get("TG_CACHE_DIR", "/tmp"), "tg_%s_s0.bin" % size), size, 0)
m = capi.Model(size).load_file(path); m.build_tables(1024)
st = m.state(1, 1024)
st.prefill(synth.random_prompt(178, 77), want_logits=False)
tok = st.sample_argmax()
st.phase_clocks()
rf = synth.mt19937_uniforms(64, 1)
for rep in range(2):
    if sampler=="minp": toks = st.generate(tok, 16, 0.1, 0.7, rf[:16])
    else: toks = st.generate(tok, 16)
    tok = toks[-1]
    c = st.phase_clocks()
L = m.cfg.n_layers
print("stamps", len(c))
d = np.diff(c)/1965.0  # us at 1965 MHz
# layout: 1 (step start) + 16 stamps per layer (see names); then lm_head prologue, lm_head, sampler
names = ["A.pro","A.wait","A.comp","A.post","B.work","C.pro","C.comp","C.post","D.pro","D.wait","D.up","D.gate","D.issue","E.wait","E.comp","E.bar"]
NS=len(names)
per = d[:NS*L].reshape(L,NS)
for i,nm in enumerate(names):
    print("%-7s mean %7.2f us  min %7.2f max %7.2f  total %8.1f"%(nm, per[:,i].mean(), per[:,i].min(), per[:,i].max(), per[:,i].sum()))
print("layers total %.1f us"%per.sum())
rest = d[NS*L:]
print("tail (lm.pro, lm_head, sampler):", np.round(rest,1))
print("step total %.1f us"%((c[-1]-c[0])/1965.0))

