#!/usr/bin/env python
"""Benchmark of the int8 weight-only Gemma-3 decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (N=1): Gemma-3-1B architecture, seeded random-init int8 weights in the
gemma_i8.bin layout, batch 1, a 178-token random prompt prefilled once, then
decode steps with the min-p sampler (minp 0.1, temperature 0.7, std::mt19937
seed 1234). One "step" = one token: forward_decode + sampler. The prompt and
weights stand in for the reference README's ultrachat prompts / real
checkpoint, which are not available offline.

Numbers on the JSON line
  value     device-resident decode tok/s: token fed back on the GPU, CUDA-event
            timed on the launching stream, no host round trip per token.
  e2e       decode tok/s through the C ABI with host buffers: per step the token
            id and the uniform go host->device and the sampled id comes back
            (one tg_generate call of one step per token; the two-call variant,
            tg_decode then tg_sample_minp, is reported beside it).
  roofline  whole decode step against the measured HBM copy bandwidth:
            algorithmic bytes per token (weights + scales + norms once, plus
            the KV rows the step reads) / device time per token.
  cpu_baseline  the reference's own single-threaded AVX2 code (oracle/_ref) on
            this box's host, bounded sample.
With N>1 (torchrun): one process per GPU, each decoding its own independent
sequence from a full weight replica — no data-path collective; value is the sum
over ranks / max time over ranks.
"""

from __future__ import annotations

import argparse
import importlib
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODEL = "1B"
PROMPT_LEN = 178
MINP, TEMP, SAMPLER_SEED = 0.1, 0.7, 1234
WEIGHT_SEED, PROMPT_SEED = 0, 77
CACHE = os.environ.get("TG_CACHE_DIR", "/tmp")
PUBLISHED_DECODE_TOK_S = 16.45  # reference README.md:69, Ryzen 5 5500, 1 thread, real weights
# dram__bytes_read.sum + dram__bytes_write.sum per decoded token from one ncu capture of the decode kernel
# (profiles/mega_decode_kernel_1B_dram_traffic.md, profiles/mega_decode_kernel_270m_ncu_full.md)
DRAM_TRAFFIC_PER_STEP = {"1B": 1005668181, "270m": 273534288}
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0


def algorithmic_bytes_per_token(cfg, positions) -> float:
    """int8 weights + fp32 scales + norm weights read once per token, plus the
    fp32 K and V rows attention reads at each position (2 * 256 * 4 B per slot)."""
    D, I, L, V = cfg.hidden_size, cfg.intermediate_size, cfg.n_layers, cfg.n_vocab
    qd, kd = cfg.n_head * cfg.head_dim, cfg.n_kv * cfg.head_dim
    per_layer = (D * qd + 4 * qd) + 2 * (D * kd + 4 * kd) + (qd * D + 4 * D) + 2 * 4 * cfg.head_dim + 2 * 4 * D \
        + 2 * (D * I + 4 * I) + (I * D + 4 * D) + 2 * 4 * D
    weights = L * per_layer + (D * V + 4 * V) + 4 * D + (D + 4 * D)  # + final norm + one embedding row and its scales
    n_local = sum(1 for l in range(L) if (l % cfg.window_pattern) != cfg.window_pattern - 1)
    n_global = L - n_local
    kv = 0.0
    for p in positions:
        kv += 2048.0 * (n_local * min(p + 1, cfg.n_pos_local) + n_global * (p + 1))
    return weights + kv / max(len(positions), 1)


def measured_tensor_peak():
    """burst dense bf16 TFLOP/s of MEASURED_PEAKS.json (a kernel timed alone), else the 1590 fallback"""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["bf16_tflops"])
    except Exception:
        return 1590.0


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """nvidia-smi clock / throttle sampling while the timed region runs"""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.p = None

    def start(self):
        try:
            self.p = subprocess.Popen(["nvidia-smi", "-i", str(self.idx), "--query-gpu=" + self.Q,
                                       "--format=csv,noheader,nounits", "-lms", "100"], stdout=self.f,
                                      stderr=subprocess.DEVNULL)
        except Exception:
            self.p = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.p is None:
            return out
        self.p.terminate()  # the exact process started above
        try:
            self.p.wait(timeout=5)
        except Exception:
            pass
        self.f.flush()
        rows = [r.split(",") for r in open(self.f.name).read().strip().splitlines() if r.strip()]
        os.unlink(self.f.name)
        sm, reasons = [], set()
        for r in rows:
            try:
                sm.append(float(r[1]))
                out["sm_max_mhz"] = float(r[2])
            except Exception:
                continue
            names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
            for name, v in zip(names, r[5:9]):
                if v.strip().lower().startswith("active"):
                    reasons.add(name)
        if sm:
            out["sm_mhz"] = float(np.median(sm))
        out["reasons"] = sorted(reasons)
        out["samples"] = len(sm)
        return out


def dist_env():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))


# =============================================================================== reference arm
def run_reference(args):
    """times the reference's own CPU implementation of the same workload"""
    rank, _, world = dist_env()
    if rank != 0:
        return 0
    from oracle import build_oracle
    from oracle.oracle_api import Oracle, available

    synth = importlib.import_module("tiny-gemma_b200.synth")
    build_oracle.build_ref()
    kind = "reference" if available("reference") else "port"
    if kind == "port":
        build_oracle.build_port()
    O = Oracle(kind)
    path = synth.write_random_model(os.path.join(CACHE, "tg_%s_s%d.bin" % (MODEL, WEIGHT_SEED)), MODEL, WEIGHT_SEED)
    m = O.model(MODEL, path)
    st = m.state(1024)
    ids = synth.random_prompt(PROMPT_LEN, PROMPT_SEED)
    W = max(args.warmup, 1)
    K = min(args.steps, 48)  # bounded sample: ~0.2 s per token on one core
    rf = synth.mt19937_uniforms(1 + W + K, SAMPLER_SEED)
    t0 = time.perf_counter()
    logits = st.prefill(ids)
    t_prefill = time.perf_counter() - t0
    tok, _ = O.minp_logits(logits, MINP, TEMP, float(rf[0]))
    toks = st.decode_loop(tok, W, MINP, TEMP, rf[1:1 + W])
    t0 = time.perf_counter()
    toks = st.decode_loop(int(toks[-1]), K, MINP, TEMP, rf[1 + W:1 + W + K])
    dt = time.perf_counter() - t0
    v = K / dt
    cpu = ""
    try:
        cpu = [l.split(":", 1)[1].strip() for l in open("/proc/cpuinfo") if l.startswith("model name")][0]
    except Exception:
        pass
    line = {
        "impl": "reference", "metric": "decode_tok_s", "value": v, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": K, "warmup": W, "ms_per_step": 1e3 * dt / K, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": v / PUBLISHED_DECODE_TOK_S, "dtype": "int8w/f32", "data": "synthetic",
        "config": {"workload": "gemma3-%s int8 weight-only, batch 1, 178-token random prompt, min-p 0.1 temp 0.7 decode" % MODEL,
                   "model_size": MODEL, "prompt_len": PROMPT_LEN, "batch": 1},
        "cpu_baseline": {"value": v, "unit": "tok/s", "cores": 1, "kind": kind,
                         "sample": "%d decode steps after a %d-token prefill, single thread (the reference is "
                                   "single-threaded), host CPU: %s" % (K, PROMPT_LEN, cpu)},
        "e2e": {"value": v, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "prefill_tok_s": PROMPT_LEN / t_prefill,
    }
    print(json.dumps(line), flush=True)
    return 0


# =============================================================================== our arm
def cpu_baseline_sample(synth, path, ids, rf):
    """reference's CPU path on a bounded sample (rank 0, N=1 only)"""
    from oracle import build_oracle
    from oracle.oracle_api import Oracle, available

    build_oracle.build_ref()
    kind = "reference" if available("reference") else "port"
    if kind == "port":
        build_oracle.build_port()
    O = Oracle(kind)
    m = O.model(MODEL, path)
    st = m.state(1024)
    t0 = time.perf_counter()
    logits = st.prefill(ids)
    t_prefill = time.perf_counter() - t0
    tok, _ = O.minp_logits(logits, MINP, TEMP, float(rf[0]))
    n = 32
    t0 = time.perf_counter()
    st.decode_loop(tok, n, MINP, TEMP, rf[1:1 + n])
    dt = time.perf_counter() - t0
    st.close()
    m.close()
    cpu = ""
    try:
        cpu = [l.split(":", 1)[1].strip() for l in open("/proc/cpuinfo") if l.startswith("model name")][0]
    except Exception:
        pass
    return {"value": n / dt, "unit": "tok/s", "cores": 1, "kind": kind, "prefill_tok_s": PROMPT_LEN / t_prefill,
            "sample": "%d decode steps after the %d-token prefill, 1 thread (the reference is single-threaded); "
                      "host CPU: %s, %d cores online" % (n, PROMPT_LEN, cpu, os.cpu_count() or 0)}


def matvec_sweep(capi, torch, hbm_peak):
    """isolated int8 matvec at the Gemma-3 shapes, device-resident, rotating
    over enough weight copies that the working set exceeds L2"""
    import ctypes as C

    cases = [(640, 1024), (640, 2048), (2048, 640), (1152, 1024), (1152, 6912), (6912, 1152), (1152, 262144)]
    lib = capi.load()
    out = []
    g = torch.Generator(device="cuda").manual_seed(5)
    for K, N in cases:
        nbytes = K * N
        copies = max(2, min(512, int(np.ceil(300e6 / nbytes))))
        w = torch.randint(-127, 128, (copies, K, N), dtype=torch.int8, device="cuda", generator=g)
        s = torch.rand(N, device="cuda", generator=g) * 1e-2 + 1e-4
        x = torch.randn(K, device="cuda", generator=g)
        y = torch.empty(N, device="cuda")
        stream = torch.cuda.current_stream()
        sp = C.c_void_p(stream.cuda_stream)

        def run(i):
            rc = lib.tg_dev_qmatvec(C.c_void_p(y.data_ptr()), C.c_void_p(x.data_ptr()),
                                    C.c_void_p(w[i % copies].data_ptr()), C.c_void_p(s.data_ptr()), K, N, sp)
            if rc:
                raise RuntimeError(lib.tg_last_error().decode())

        for i in range(5):
            run(i)
        reps = max(20, copies)
        # The launches are captured into a CUDA graph and the graph is timed: at 5-20 us per kernel a Python
        # loop of ctypes calls enqueues more slowly than the GPU executes, and the events would time the host.
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            cs = torch.cuda.current_stream()
            spc = C.c_void_p(cs.cuda_stream)
            for i in range(reps):
                rc = lib.tg_dev_qmatvec(C.c_void_p(y.data_ptr()), C.c_void_p(x.data_ptr()),
                                        C.c_void_p(w[i % copies].data_ptr()), C.c_void_p(s.data_ptr()), K, N, spc)
                if rc:
                    raise RuntimeError(lib.tg_last_error().decode())
        graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(3):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        us = 1e3 * e0.elapsed_time(e1) / (3 * reps)
        alg = K * N + 4 * N + 4 * K + 4 * N
        out.append({"K": K, "N": N, "us": us, "GBs": alg / us / 1e3, "frac": alg / us / 1e3 / hbm_peak})
        del w
    return out


def gemm_sweep(capi, torch, tf_peak):
    """isolated int8-weight GEMM (prefill / batched-step operator) at Gemma-3-1B shapes, device-resident.
    TFLOP/s counts the algorithmic 2*M*K*N; the tensor cores execute three bf16 products per fp32
    activation (split into three bf16 terms), so the tensor-pipe work is three times that."""
    import ctypes as C

    lib = capi.load()
    out = []
    g = torch.Generator(device="cuda").manual_seed(6)
    for K, N in [(1152, 6912), (6912, 1152), (1152, 1024)]:
        # enough weight copies that the rotating working set exceeds L2
        copies = int(np.ceil(300e6 / (K * N)))
        w = torch.randint(-127, 128, (copies, K, N), dtype=torch.int8, device="cuda", generator=g)
        s = torch.rand(N, device="cuda", generator=g) * 1e-2 + 1e-4
        for M in (16, 178, 1024, 4096):
            a = torch.randn(M, K, device="cuda", generator=g)
            c = torch.empty(M, N, device="cuda")

            def run(i, sp):
                rc = lib.tg_dev_qgemm(C.c_void_p(c.data_ptr()), C.c_void_p(a.data_ptr()),
                                      C.c_void_p(w[i % copies].data_ptr()), C.c_void_p(s.data_ptr()), M, K, N, sp)
                if rc:
                    raise RuntimeError(lib.tg_last_error().decode())

            for i in range(3):
                run(i, C.c_void_p(torch.cuda.current_stream().cuda_stream))
            # Outside a capture every call synchronises (it reads the error word), which at small M costs more
            # than the kernels; the launches are captured into a graph and the graph is timed.
            reps = max(10, min(copies, 40))
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                spc = C.c_void_p(torch.cuda.current_stream().cuda_stream)
                for i in range(reps):
                    run(i, spc)
            graph.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(3):
                graph.replay()
            e1.record()
            torch.cuda.synchronize()
            us = 1e3 * e0.elapsed_time(e1) / (3 * reps)
            # one uncaptured call afterwards reports an error word a replay may have set
            run(0, C.c_void_p(torch.cuda.current_stream().cuda_stream))
            tf = 2.0 * M * K * N / us / 1e6
            out.append({"M": M, "K": K, "N": N, "us": us, "TFLOPs": tf, "tensor_TFLOPs": 3 * tf,
                        "tensor_frac": 3 * tf / tf_peak if tf_peak else None})
    return out


def run_ours(args):
    rank, local_rank, world = dist_env()
    import torch

    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device: this benchmark has no CPU path"}), flush=True)
        return 1
    torch.cuda.set_device(local_rank)
    use_dist = world > 1
    if use_dist:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    build = importlib.import_module("tiny-gemma_b200.build")
    if rank == 0 or not use_dist:
        build.build()
    if use_dist:
        dist.barrier()
    capi = importlib.import_module("tiny-gemma_b200.capi")
    synth = importlib.import_module("tiny-gemma_b200.synth")

    path = os.path.join(CACHE, "tg_%s_s%d.bin" % (MODEL, WEIGHT_SEED))
    if local_rank == 0:
        synth.write_random_model(path, MODEL, WEIGHT_SEED)
    if use_dist:
        dist.barrier()
    W, K = max(args.warmup, 3), args.steps
    model = capi.Model(MODEL, device=local_rank).load_file(path)
    model.build_tables(1024)
    cfg = model.cfg
    st = model.state(1, PROMPT_LEN + 3 * (W + K) + 80)
    stream = torch.cuda.ExternalStream(st.stream())
    ids = synth.random_prompt(PROMPT_LEN, PROMPT_SEED + rank)  # every rank its own sequence
    rf = synth.mt19937_uniforms(3 * (1 + W + K) + 16, SAMPLER_SEED + rank)

    def ev():
        return torch.cuda.Event(enable_timing=True)

    # ---- prefill (timed once on the device; includes the lm_head of the last position)
    st.prefill(synth.random_prompt(PROMPT_LEN, 999), want_logits=False)  # warm-up of the prefill kernels
    st.reset()
    e0, e1 = ev(), ev()
    torch.cuda.synchronize()
    e0.record(stream)
    st.prefill(ids, want_logits=False)
    e1.record(stream)
    torch.cuda.synchronize()
    prefill_ms = e0.elapsed_time(e1)
    first = st.sample_minp(MINP, TEMP, rf[0:1])

    # ---- device-resident decode loop (value): (decode, sample) pairs, token fed back on the GPU.
    # The state's first decode step runs eagerly, the second captures the CUDA graph, the rest replay it.
    st.set_randf(rf[1:1 + W + K])
    pos0 = st.position()
    st.generate_async(W, MINP, TEMP)
    torch.cuda.synchronize()
    if use_dist:
        dist.barrier()
    clocks = ClockSampler(local_rank)
    clocks.start()
    capi.launch_count(reset=True)
    torch.cuda.synchronize()
    e0, e1 = ev(), ev()
    e0.record(stream)
    st.generate_async(K, MINP, TEMP)
    e1.record(stream)
    torch.cuda.synchronize()
    launches = capi.launch_count()
    clk = clocks.stop()
    dev_ms = e0.elapsed_time(e1)
    toks = st.tokens(K)
    positions = list(range(pos0 + W, pos0 + W + K))

    # ---- e2e through the C ABI with host buffers (token + uniform in, token out, every step)
    tok = toks[-1].copy()
    rf2 = rf[2 + W + K:]
    # The calls go straight to the C ABI with buffers and pointers prepared once: the Python wrapper's
    # per-call numpy conversions cost 50-60 us, which a C++ caller of the library does not pay.
    import ctypes as C

    lib = capi.load()
    ids_buf = np.array(tok, np.int32).reshape(1)
    out_buf = np.zeros(1, np.int32)
    rf2 = np.ascontiguousarray(rf2, np.float32)
    p_ids, p_out, rf_base = ids_buf.ctypes.data, out_buf.ctypes.data, rf2.ctypes.data

    def check(rc):
        if rc:
            raise RuntimeError(lib.tg_last_error().decode())

    # (a) one call per token: tg_generate with n_steps = 1 (ids + uniform in, one launch of the persistent
    #     kernel with its sampler, token out, one synchronisation)
    def step_one_call(i):
        check(lib.tg_generate(st.h, p_ids, 1, MINP, TEMP, rf_base + 4 * i, p_out))
        ids_buf[0] = out_buf[0]

    # (b) the reference's call granularity: forward_decode, then minp_logits (two calls, two launches)
    def step_two_calls(i):
        check(lib.tg_decode(st.h, p_ids, None))
        check(lib.tg_sample_minp(st.h, MINP, TEMP, rf_base + 4 * i, p_out))
        ids_buf[0] = out_buf[0]

    n_e2e = min(K, (len(rf2) - 6) // 2)
    e2e_times = []
    for step, first in ((step_one_call, 0), (step_two_calls, 3 + n_e2e)):
        # each variant decodes the positions the device-resident loop was timed on: same prompt again
        st.reset()
        st.prefill(ids, want_logits=False)
        ids_buf[0] = st.sample_minp(MINP, TEMP, rf[0:1])[0]
        for i in range(3):
            step(first + i)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for i in range(n_e2e):
            step(first + 3 + i)
        torch.cuda.synchronize()
        e2e_times.append(time.perf_counter() - t0)
    e2e_s, e2e2_s = e2e_times

    # ---- reduce over ranks
    t = torch.tensor([dev_ms, e2e_s * 1e3 * K / max(n_e2e, 1), prefill_ms, e2e2_s * 1e3 * K / max(n_e2e, 1)],
                     dtype=torch.float64, device="cuda")
    if use_dist:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms_max, e2e_ms_max, prefill_ms_max, e2e2_ms_max = [float(v) for v in t.tolist()]
    value = world * K / (dev_ms_max / 1e3)
    e2e_value = world * K / (e2e_ms_max / 1e3)

    hbm_peak, peak_kind = measured_peaks()
    alg = algorithmic_bytes_per_token(cfg, positions)
    achieved = alg / (dev_ms_max / 1e3 / K) / 1e9
    line = {
        "metric": "decode_tok_s", "value": value, "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": dev_ms_max / K, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": value / PUBLISHED_DECODE_TOK_S, "dtype": "int8w/f32", "data": "synthetic",
        "config": {"workload": "gemma3-%s int8 weight-only, batch 1 per GPU, 178-token random prompt, min-p 0.1 "
                               "temp 0.7 decode" % MODEL, "model_size": MODEL, "prompt_len": PROMPT_LEN, "batch_per_gpu": 1,
                   "parallelism": "replica-dp%d (independent sequences, no collective)" % world,
                   "l2": "inputs larger than L2: every step streams 1.0 GB of weights through a 126 MB L2",
                   "timing": "CUDA events on the launching stream, max over ranks"},
        "e2e": {"value": e2e_value, "unit": "tok/s", "h2d_bytes_per_step": 8, "d2h_bytes_per_step": 8,
                "steps": n_e2e, "call": "tg_generate(n_steps=1) per token: host ids + uniform in, host token out",
                "two_calls_tok_s": world * K / (e2e2_ms_max / 1e3),
                "two_calls": "tg_decode then tg_sample_minp per token (the reference's forward_decode / minp_logits granularity)"},
        "gpu_launches": int(launches),
        "clocks": clk,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                     "frac": achieved / hbm_peak, "traffic": DRAM_TRAFFIC_PER_STEP.get(MODEL), "peak_kind": peak_kind,
                     "what": "one decode step of the persistent decode kernel (forward + sampler)",
                     "algorithmic_bytes_per_token": alg, "frac_of_nominal_8TBs": achieved / NOMINAL_HBM_GBS},
        "prefill_tok_s": world * PROMPT_LEN / (prefill_ms_max / 1e3),
        "prefill_ms": prefill_ms_max,
    }
    if rank == 0 and world == 1 and not args.no_extras:
        try:
            line["matvec_sweep"] = matvec_sweep(capi, torch, hbm_peak)
            line["gemm_sweep"] = gemm_sweep(capi, torch, measured_tensor_peak())
        except Exception as e:  # the sweep is an extra; the headline line must still print
            line["matvec_sweep_error"] = str(e)
        st.close()
        model.close()
        try:
            line["cpu_baseline"] = cpu_baseline_sample(synth, path, ids, rf)
        except Exception as e:
            line["cpu_baseline"] = {"value": None, "unit": "tok/s", "cores": 1, "kind": "unavailable", "sample": str(e)}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if use_dist:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def run_batched(args):
    """Batched greedy throughput: `--batch` independent sequences in total, split evenly over the
    ranks (strong scaling), each a 178-token random prompt followed by greedy decode steps. Every
    weight matrix is read once per step for all of a rank's sequences (tensor-core GEMMs, M = batch);
    attention runs per sequence against its own cache. No data-path collective."""
    rank, local_rank, world = dist_env()
    import torch

    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device: this benchmark has no CPU path"}), flush=True)
        return 1
    torch.cuda.set_device(local_rank)
    use_dist = world > 1
    if use_dist:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    build = importlib.import_module("tiny-gemma_b200.build")
    if rank == 0 or not use_dist:
        build.build()
    if use_dist:
        dist.barrier()
    capi = importlib.import_module("tiny-gemma_b200.capi")
    synth = importlib.import_module("tiny-gemma_b200.synth")
    path = os.path.join(CACHE, "tg_%s_s%d.bin" % (MODEL, WEIGHT_SEED))
    if local_rank == 0:
        synth.write_random_model(path, MODEL, WEIGHT_SEED)
    if use_dist:
        dist.barrier()
    W, K = max(args.warmup, 3), args.steps
    B = args.batch // world
    model = capi.Model(MODEL, device=local_rank).load_file(path)
    model.build_tables(1024)
    st = model.state(B, PROMPT_LEN + W + K + 72)
    stream = torch.cuda.ExternalStream(st.stream())
    prompts = np.stack([synth.random_prompt(PROMPT_LEN, PROMPT_SEED + rank * B + b) for b in range(B)])

    def ev():
        return torch.cuda.Event(enable_timing=True)

    e0, e1 = ev(), ev()
    torch.cuda.synchronize()
    e0.record(stream)
    st.prefill(prompts, want_logits=False)
    e1.record(stream)
    torch.cuda.synchronize()
    prefill_ms = e0.elapsed_time(e1)
    st.sample_argmax()
    st.generate_async(W, 1.0, 1.0)
    torch.cuda.synchronize()
    if use_dist:
        dist.barrier()
    clocks = ClockSampler(local_rank)
    clocks.start()
    capi.launch_count(reset=True)
    torch.cuda.synchronize()
    e0, e1 = ev(), ev()
    e0.record(stream)
    st.generate_async(K, 1.0, 1.0)
    e1.record(stream)
    torch.cuda.synchronize()
    launches = capi.launch_count()
    clk = clocks.stop()
    dev_ms = e0.elapsed_time(e1)
    toks = st.tokens(K)

    # e2e: tokens in from the host and out to the host every step
    tok = toks[-1].copy()
    n_e2e = min(K, 32)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(n_e2e):
        st.decode(tok, want_logits=False)
        tok = st.sample_argmax()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0

    t = torch.tensor([dev_ms, e2e_s * 1e3 * K / n_e2e, prefill_ms], dtype=torch.float64, device="cuda")
    if use_dist:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms_max, e2e_ms_max, prefill_ms_max = [float(v) for v in t.tolist()]
    value = world * B * K / (dev_ms_max / 1e3)
    hbm_peak, peak_kind = measured_peaks()
    cfg = model.cfg
    # weights once per step + every sequence's cache reads
    pos_mid = PROMPT_LEN + W + K // 2
    alg = algorithmic_bytes_per_token(cfg, [pos_mid])
    weight_bytes = algorithmic_bytes_per_token(cfg, [0])
    step_bytes = weight_bytes + B * (alg - weight_bytes)
    achieved = step_bytes / (dev_ms_max / 1e3 / K) / 1e9
    line = {
        "metric": "decode_tok_s", "value": value, "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": dev_ms_max / K, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "int8w/f32 (bf16x3 tensor-core GEMM)", "data": "synthetic",
        "config": {"workload": "gemma3-%s int8 weight-only, %d independent sequences in total, 178-token random "
                               "prompts, greedy decode" % (MODEL, B * world), "model_size": MODEL,
                   "prompt_len": PROMPT_LEN, "batch_per_gpu": B,
                   "parallelism": "sequence-sharded dp%d (no collective)" % world,
                   "l2": "inputs larger than L2: every step streams 1.0 GB of weights and the sequences' caches",
                   "timing": "CUDA events on the launching stream, max over ranks"},
        "e2e": {"value": world * B * K / (e2e_ms_max / 1e3), "unit": "tok/s", "h2d_bytes_per_step": 4 * B,
                "d2h_bytes_per_step": 4 * B, "steps": n_e2e},
        "gpu_launches": int(launches), "clocks": clk,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                     "frac": achieved / hbm_peak, "traffic": None, "peak_kind": peak_kind,
                     "what": "one batched decode step: weights once + %d sequences' KV reads" % B},
        "prefill_tok_s": world * B * PROMPT_LEN / (prefill_ms_max / 1e3), "prefill_ms": prefill_ms_max,
    }
    if rank == 0:
        print(json.dumps(line), flush=True)
    if use_dist:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=512)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=1, help="total independent sequences (greedy); >1 selects the batched step")
    ap.add_argument("--no-extras", action="store_true", help="skip the matvec sweep and the CPU baseline sample")
    ap.add_argument("--model", default=MODEL, choices=["270m", "1B"],
                    help="architecture; 1B is the benchmark configuration, 270m is the small case used for profiling")
    ap.add_argument("--prompt-len", type=int, default=PROMPT_LEN,
                    help="prompt tokens; 178 is the benchmark configuration, 16384 the long-context one "
                         "(use --no-extras: the CPU baseline sample would prefill the same prompt)")
    args = ap.parse_args()
    globals()["MODEL"] = args.model
    globals()["PROMPT_LEN"] = args.prompt_len
    if args.impl == "reference":
        return run_reference(args)
    if args.batch > 1:
        return run_batched(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
