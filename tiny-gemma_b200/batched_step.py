"""Time the batched decode step in isolation (no prefill, caches filled by the steps themselves).

    python tiny-gemma_b200/batched_step.py [270m|1B] [batch] [steps]

Runs `steps` greedy decode steps of `batch` sequences from an empty cache and prints the mean
step time. It launches nothing but the step's own kernels, so a kernel launch list taken over
this command is the per-kernel breakdown of the batched step (set TG_USE_GRAPH=0 to see the
kernels individually rather than as one graph launch).
"""
import importlib
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import numpy as np

capi = importlib.import_module("tiny-gemma_b200.capi")
synth = importlib.import_module("tiny-gemma_b200.synth")
size = sys.argv[1] if len(sys.argv) > 1 else "1B"
batch = int(sys.argv[2]) if len(sys.argv) > 2 else 256
steps = int(sys.argv[3]) if len(sys.argv) > 3 else 16
path = synth.write_random_model(os.path.join(os.environ.get("TG_CACHE_DIR", "/tmp"), "tg_%s_s0.bin" % size), size, 0)
m = capi.Model(size).load_file(path)
m.build_tables(1024)
st = m.state(batch, steps + 16)
tok = np.random.default_rng(0).integers(0, 262144, size=batch).astype(np.int32)
for _ in range(3):  # eager step, graph capture, first replay
    st.decode(tok, want_logits=False)
    tok = st.sample_argmax()
t0 = time.perf_counter()
for _ in range(steps):
    st.decode(tok, want_logits=False)
    tok = st.sample_argmax()
dt = (time.perf_counter() - t0) / steps
print("batch %d: %.3f ms per step, %.0f tok/s (launches per step: %d)" % (
    batch, dt * 1e3, batch / dt, capi.launch_count() // (steps + 3)))
