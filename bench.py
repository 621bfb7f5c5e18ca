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
            this box's host, bounded sample; its tokens are compared with the
            device loop's ("parity").
  batched_256   sub-record: 256 independent greedy sequences split evenly over
            the ranks (strong scaling), every weight matrix read once per step
            for all of a rank's sequences (tensor-core GEMMs).
  sharded_lm_head  sub-record (N > 1): the same 256 sequences with the lm_head
            split by vocabulary columns over the ranks (two NCCL all-gathers per
            step), tokens checked against the unsharded step.
The device loop and both e2e legs are timed as repeats of --steps (state reset
and prompt prefilled again in between) until at least a second has been timed;
value / ms_per_step are the median repeat, the list is kept.
With N>1 (torchrun): one process per GPU, each decoding its own independent
sequence from a full weight replica — no data-path collective; value is the sum
over ranks / max time over ranks.

Other modes (one JSON line each, 1 GPU):
    python bench.py --phase-clocks [--greedy]   where a decoded token's time goes (in-kernel recorder)
    python bench.py --batched-step --batch B    the batched step alone, from an empty cache
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
DRAM_TRAFFIC_PER_STEP = {"1B": 1003642432, "270m": (1080847104 + 9990400) // 4}
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


def headline_config(world: int) -> dict:
    """the workload both arms run (the reference arm prints the same dict)"""
    return {"workload": "gemma3-%s int8 weight-only, batch 1 per GPU, %d-token random prompt, min-p 0.1 temp 0.7 decode"
                        % (MODEL, PROMPT_LEN), "model_size": MODEL, "prompt_len": PROMPT_LEN, "batch_per_gpu": 1,
            "parallelism": "replica-dp%d (independent sequences, no collective)" % world,
            "l2": "inputs larger than L2: every step streams 1.0 GB of weights through a 126 MB L2",
            "timing": "CUDA events on the launching stream, max over ranks"}


def host_cpu_name() -> str:
    try:
        return [l.split(":", 1)[1].strip() for l in open("/proc/cpuinfo") if l.startswith("model name")][0]
    except Exception:
        return ""


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
    cpu = host_cpu_name()
    line = {
        "impl": "reference", "metric": "decode_tok_s", "value": v, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": K, "warmup": W, "ms_per_step": 1e3 * dt / K, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": v / PUBLISHED_DECODE_TOK_S, "dtype": "int8w/f32", "data": "synthetic",
        "config": headline_config(world),
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
    toks = st.decode_loop(tok, n, MINP, TEMP, rf[1:1 + n])
    dt = time.perf_counter() - t0
    st.close()
    m.close()
    rec = {"value": n / dt, "unit": "tok/s", "cores": 1, "kind": kind, "prefill_tok_s": PROMPT_LEN / t_prefill,
           "sample": "%d decode steps after the %d-token prefill, 1 thread (the reference is single-threaded); "
                     "host CPU: %s, %d cores online" % (n, PROMPT_LEN, host_cpu_name(), os.cpu_count() or 0)}
    return rec, np.concatenate([[int(tok)], toks]).astype(np.int64)


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


def setup(args):
    """device, process group, library, weights: what every mode of the repo's arm needs"""
    rank, local_rank, world = dist_env()
    import torch

    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device: this benchmark has no CPU path"}), flush=True)
        return None
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    build = importlib.import_module("tiny-gemma_b200.build")
    if rank == 0 or dist is None:
        build.build()
    if dist is not None:
        dist.barrier()
    capi = importlib.import_module("tiny-gemma_b200.capi")
    synth = importlib.import_module("tiny-gemma_b200.synth")
    path = os.path.join(CACHE, "tg_%s_s%d.bin" % (MODEL, WEIGHT_SEED))
    if local_rank == 0:
        synth.write_random_model(path, MODEL, WEIGHT_SEED)
    if dist is not None:
        dist.barrier()
    t0 = time.perf_counter()
    model = capi.Model(MODEL, device=local_rank).load_file(path)
    load_s = time.perf_counter() - t0
    model.build_tables(1024)
    return {"load_s": load_s, "load_bytes": os.path.getsize(path), "rank": rank, "local_rank": local_rank, "world": world, "torch": torch, "dist": dist, "capi": capi,
            "synth": synth, "path": path, "model": model}


def max_over_ranks(env, values):
    torch, dist = env["torch"], env["dist"]
    t = torch.tensor(list(values), dtype=torch.float64, device="cuda")
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t.tolist()]


def repeats_for(first_ms: float, floor: int = 3, cap: int = 20) -> int:
    """repeats so that at least one second is timed in total"""
    return int(min(cap, max(floor, np.ceil(1000.0 / max(first_ms, 1e-3)))))


def batched_record(env, total: int, K: int, W: int, sharded: bool = False):
    """`total` independent greedy sequences split evenly over the ranks (strong scaling), each a 178-token
    random prompt followed by K timed decode steps. Every weight matrix is read once per step for all of a
    rank's sequences (tensor-core GEMMs, M = sequences per rank); attention runs per sequence against its own
    cache. sharded: the lm_head is split by vocabulary columns over the ranks (two all-gathers per step);
    otherwise there is no data-path collective."""
    torch, dist, capi, synth, model = env["torch"], env["dist"], env["capi"], env["synth"], env["model"]
    rank, world = env["rank"], env["world"]
    B = total // world
    cfg = model.cfg
    st = model.state(B, PROMPT_LEN + W + K + 72)
    stream = torch.cuda.ExternalStream(st.stream())
    prompts = np.stack([synth.random_prompt(PROMPT_LEN, PROMPT_SEED + rank * B + b) for b in range(B)])

    def ev():
        return torch.cuda.Event(enable_timing=True)

    # (an untimed prefill first: the first one allocates the state's prefill scratch, which the events would time)
    st.prefill(prompts, want_logits=False)
    st.reset()
    e0, e1 = ev(), ev()
    torch.cuda.synchronize()
    e0.record(stream)
    st.prefill(prompts, want_logits=False)
    e1.record(stream)
    torch.cuda.synchronize()
    prefill_ms = e0.elapsed_time(e1)
    first = st.sample_argmax()
    rec = {}
    if sharded:
        sh = importlib.import_module("tiny-gemma_b200.sharded")
        # the unsharded step on the same sequences: the tokens the sharded step must reproduce
        want = st.generate(first, 8)
        st.reset()
        st.prefill(prompts, want_logits=False)
        dec = sh.ShardedGreedyDecoder(torch, dist, model, st, rank, world)
        dec.step(first)
        got = [dec.tokens_host()]
        for _ in range(7):
            dec.step(None)
            got.append(dec.tokens_host())
        st.check()
        bad = int((np.stack(got) != want).sum())
        for _ in range(max(W - 8, 0)):
            dec.step(None)
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        capi.launch_count(reset=True)
        e0, e1 = ev(), ev()
        e0.record(stream)
        for _ in range(K):
            dec.step(None)
        e1.record(stream)
        torch.cuda.synchronize()
        st.check()
        launches = capi.launch_count()
        rec["tokens_equal_unsharded_8_steps"] = bad == 0
        rec["token_mismatches"] = bad
    else:
        st.generate_async(W, 1.0, 1.0)
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        capi.launch_count(reset=True)
        torch.cuda.synchronize()
        e0, e1 = ev(), ev()
        e0.record(stream)
        st.generate_async(K, 1.0, 1.0)
        e1.record(stream)
        torch.cuda.synchronize()
        launches = capi.launch_count()
    dev_ms = e0.elapsed_time(e1)
    e2e_ms = None
    n_e2e = min(K, 32)
    if not sharded:
        # e2e: tokens in from the host and out to the host every step
        tok = st.tokens(K)[-1].copy()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(n_e2e):
            st.decode(tok, want_logits=False)
            tok = st.sample_argmax()
        torch.cuda.synchronize()
        e2e_ms = (time.perf_counter() - t0) * 1e3 * K / n_e2e
    st.close()
    dev_ms_max, e2e_ms_max, prefill_ms_max = max_over_ranks(env, [dev_ms, e2e_ms or 0.0, prefill_ms])
    hbm_peak, peak_kind = measured_peaks()
    # per rank and step: the weights once (only its column slice of the lm_head when sharded) + every sequence's cache reads
    pos_mid = PROMPT_LEN + W + K // 2
    weight_bytes = algorithmic_bytes_per_token(cfg, [])
    kv_bytes = algorithmic_bytes_per_token(cfg, [pos_mid]) - weight_bytes
    lm_bytes = cfg.hidden_size * cfg.n_vocab + 4 * cfg.n_vocab
    step_bytes = weight_bytes - (lm_bytes * (1.0 - 1.0 / world) if sharded else 0.0) + B * kv_bytes
    achieved = step_bytes / (dev_ms_max / 1e3 / K) / 1e9
    rec.update({
        "sequences": B * world, "sequences_per_gpu": B, "steps": K, "warmup": W, "scaling": "strong",
        "ms_per_step": dev_ms_max / K, "tok_s": world * B * K / (dev_ms_max / 1e3),
        "gpu_launches": int(launches), "prefill_ms": prefill_ms_max,
        "prefill_tok_s": world * B * PROMPT_LEN / (prefill_ms_max / 1e3),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                     "traffic": None, "peak_kind": peak_kind, "per": "GPU",
                     "what": "one batched decode step on one rank: weights once%s + %d sequences' KV reads"
                             % (" (1/%d of the lm_head)" % world if sharded else "", B)},
    })
    if e2e_ms is not None:
        rec["e2e"] = {"value": world * B * K / (e2e_ms_max / 1e3), "unit": "tok/s", "h2d_bytes_per_step": 4 * B,
                      "d2h_bytes_per_step": 4 * B, "steps": n_e2e}
    return rec


def run_ours(args):
    env = setup(args)
    if env is None:
        return 1
    torch, dist, capi, synth, model = env["torch"], env["dist"], env["capi"], env["synth"], env["model"]
    rank, local_rank, world, path = env["rank"], env["local_rank"], env["world"], env["path"]
    W, K = max(args.warmup, 3), args.steps
    cfg = model.cfg
    st = model.state(1, PROMPT_LEN + W + K + 80)
    stream = torch.cuda.ExternalStream(st.stream())
    ids = synth.random_prompt(PROMPT_LEN, PROMPT_SEED + rank)  # every rank its own sequence
    rf = synth.mt19937_uniforms(2 * (1 + W + K) + 16, SAMPLER_SEED + rank)

    def ev():
        return torch.cuda.Event(enable_timing=True)

    st.prefill(synth.random_prompt(PROMPT_LEN, 999), want_logits=False)  # warm-up of the prefill kernels
    clocks = ClockSampler(local_rank)
    clocks.start()

    # ---- device-resident decode loop (value): repeats of [reset, prefill, first token, W warm-up steps, K timed
    # steps]; (decode, sample) pairs with the token fed back on the GPU. The prefill (with the lm_head of the last
    # position) is timed once per repeat on the device.
    def one_repeat(count_launches=False):
        st.reset()
        e0, e1 = ev(), ev()
        torch.cuda.synchronize()
        e0.record(stream)
        st.prefill(ids, want_logits=False)
        e1.record(stream)
        torch.cuda.synchronize()
        pre_ms = e0.elapsed_time(e1)
        first = st.sample_minp(MINP, TEMP, rf[0:1])
        st.set_randf(rf[1:1 + W + K])
        pos0 = st.position()
        st.generate_async(W, MINP, TEMP)
        torch.cuda.synchronize()
        warm = st.tokens(W)
        if dist is not None:
            dist.barrier()
        if count_launches:
            capi.launch_count(reset=True)
        torch.cuda.synchronize()
        e0, e1 = ev(), ev()
        e0.record(stream)
        st.generate_async(K, MINP, TEMP)
        e1.record(stream)
        torch.cuda.synchronize()
        n_launch = capi.launch_count() if count_launches else None
        seq = np.concatenate([first.ravel(), warm.ravel(), st.tokens(K).ravel()]).astype(np.int64)
        return e0.elapsed_time(e1), pre_ms, pos0, n_launch, seq

    ms0, pre0, pos0, launches, dev_seq = one_repeat(count_launches=True)
    R = args.repeats if args.repeats > 0 else int(max_over_ranks(env, [repeats_for(ms0)])[0])
    rep_ms, rep_pre = [ms0], [pre0]
    for _ in range(R - 1):
        ms, pre, _, _, _ = one_repeat()
        rep_ms.append(ms)
        rep_pre.append(pre)
    positions = list(range(pos0 + W, pos0 + W + K))

    # ---- e2e through the C ABI with host buffers (token + uniform in, token out, every step)
    # The calls go straight to the C ABI with buffers and pointers prepared once: the Python wrapper's
    # per-call numpy conversions cost 50-60 us, which a C++ caller of the library does not pay.
    import ctypes as C

    lib = capi.load()
    ids_buf = np.zeros(1, np.int32)
    out_buf = np.zeros(1, np.int32)
    rf2 = np.ascontiguousarray(rf[1:], np.float32)
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

    n_e2e = K
    e2e_reps = []
    for step in (step_one_call, step_two_calls):
        times = []
        Re = None
        while Re is None or len(times) < Re:
            # every repeat decodes the positions the device-resident loop was timed on: same prompt again
            st.reset()
            st.prefill(ids, want_logits=False)
            ids_buf[0] = st.sample_minp(MINP, TEMP, rf[0:1])[0]
            for i in range(W):
                step(i)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for i in range(n_e2e):
                step(W + i)
            torch.cuda.synchronize()
            times.append((time.perf_counter() - t0) * 1e3)
            if Re is None:
                Re = args.repeats if args.repeats > 0 else int(max_over_ranks(env, [repeats_for(times[0])])[0])
        e2e_reps.append(times)
    clk = clocks.stop()
    st.close()

    # ---- reduce over ranks: the median repeat of every rank, then the max over ranks
    dev_ms_max, e2e_ms_max, prefill_ms_max, e2e2_ms_max = max_over_ranks(
        env, [np.median(rep_ms), np.median(e2e_reps[0]), np.median(rep_pre), np.median(e2e_reps[1])])
    value = world * K / (dev_ms_max / 1e3)
    e2e_value = world * K / (e2e_ms_max / 1e3)

    hbm_peak, peak_kind = measured_peaks()
    alg = algorithmic_bytes_per_token(cfg, positions)
    achieved = alg / (dev_ms_max / 1e3 / K) / 1e9
    line = {
        "metric": "decode_tok_s", "value": value, "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": dev_ms_max / K, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": value / PUBLISHED_DECODE_TOK_S, "dtype": "int8w/f32", "data": "synthetic",
        "config": headline_config(world),
        "repeats": {"n": R, "ms_per_step": [m / K for m in rep_ms], "prefill_ms": rep_pre, "reported": "median",
                    "timed_s": sum(rep_ms) / 1e3},
        "e2e": {"value": e2e_value, "unit": "tok/s", "h2d_bytes_per_step": 8, "d2h_bytes_per_step": 8,
                "steps": n_e2e, "call": "tg_generate(n_steps=1) per token: host ids + uniform in, host token out",
                "repeats_ms_per_step": [m / n_e2e for m in e2e_reps[0]],
                "two_calls_tok_s": world * K / (e2e2_ms_max / 1e3),
                "two_calls_repeats_ms_per_step": [m / n_e2e for m in e2e_reps[1]],
                "two_calls": "tg_decode then tg_sample_minp per token (the reference's forward_decode / minp_logits granularity)"},
        "gpu_launches": int(launches),
        "clocks": clk,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                     "frac": achieved / hbm_peak, "traffic": DRAM_TRAFFIC_PER_STEP.get(MODEL), "peak_kind": peak_kind,
                     "what": "one decode step of the persistent decode kernel (forward + sampler)",
                     "algorithmic_bytes_per_token": alg, "frac_of_nominal_8TBs": achieved / NOMINAL_HBM_GBS},
        "prefill_tok_s": world * PROMPT_LEN / (prefill_ms_max / 1e3),
        "prefill_ms": prefill_ms_max,
        "weight_load": {"seconds": env["load_s"], "GBs": env["load_bytes"] / env["load_s"] / 1e9, "bytes": env["load_bytes"],
                        "what": "tg_model_load_file on rank 0: file (page cache) -> pinned double buffer -> HBM, then the "
                                "decode kernel's re-tiling"},
    }
    if not args.no_extras:
        try:
            line["batched_256"] = batched_record(env, 256, max(64, min(K, 128)), 8)
            if world > 1:
                line["sharded_lm_head"] = batched_record(env, 256, max(64, min(K, 128)), 8, sharded=True)
        except Exception as e:  # a sub-record is an extra; the headline line must still print
            line["batched_error"] = repr(e)
    if rank == 0 and world == 1 and not args.no_extras:
        try:
            line["matvec_sweep"] = matvec_sweep(capi, torch, hbm_peak)
            line["gemm_sweep"] = gemm_sweep(capi, torch, measured_tensor_peak())
        except Exception as e:  # the sweep is an extra; the headline line must still print
            line["matvec_sweep_error"] = str(e)
        model.close()
        try:
            line["cpu_baseline"], ref_seq = cpu_baseline_sample(synth, path, ids, rf)
            n = int(min(len(ref_seq), len(dev_seq)))
            diff = np.nonzero(ref_seq[:n] != dev_seq[:n])[0]
            line["parity"] = {"compared": n, "match_len": int(diff[0]) if diff.size else n,
                              "what": "tokens of the device-resident loop against the reference's CPU run: same weights, "
                                      "prompt and std::mt19937 uniforms; the reference's token 0 is drawn from its own "
                                      "prefill logits. With the 1024-entry GeLU table on random-init weights a draw flips "
                                      "on logit noise of 1e-3 (tests/test_e2e_1b_gpu.py holds the teacher-forced bar)"}
        except Exception as e:
            line["cpu_baseline"] = {"value": None, "unit": "tok/s", "cores": 1, "kind": "unavailable", "sample": str(e)}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def run_batched(args):
    """stand-alone form of the batched sub-record: --batch sequences in total over the ranks"""
    env = setup(args)
    if env is None:
        return 1
    world, dist = env["world"], env["dist"]
    W, K = max(args.warmup, 3), args.steps
    clocks = ClockSampler(env["local_rank"])
    clocks.start()
    rec = batched_record(env, args.batch, K, W, sharded=args.sharded and world > 1)
    clk = clocks.stop()
    line = {
        "metric": "decode_tok_s", "value": rec["tok_s"], "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": rec["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "int8w/f32 (bf16x3 tensor-core GEMM)", "data": "synthetic",
        "config": {"workload": "gemma3-%s int8 weight-only, %d independent sequences in total, %d-token random "
                               "prompts, greedy decode" % (MODEL, rec["sequences"], PROMPT_LEN), "model_size": MODEL,
                   "prompt_len": PROMPT_LEN, "batch_per_gpu": rec["sequences_per_gpu"],
                   "parallelism": "sequence-sharded dp%d (%s)" % (world, "vocab-sharded lm_head, two all-gathers per step"
                                                                   if args.sharded and world > 1 else "no collective"),
                   "l2": "inputs larger than L2: every step streams 1.0 GB of weights and the sequences' caches",
                   "timing": "CUDA events on the launching stream, max over ranks"},
        "gpu_launches": rec["gpu_launches"], "clocks": clk, "roofline": rec["roofline"],
        "prefill_tok_s": rec["prefill_tok_s"], "prefill_ms": rec["prefill_ms"],
    }
    if "e2e" in rec:
        line["e2e"] = rec["e2e"]
    for k in ("tokens_equal_unsharded_8_steps", "token_mismatches"):
        if k in rec:
            line[k] = rec[k]
    if env["rank"] == 0:
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def run_batched_step(args):
    """The batched decode step alone: --batch sequences from an empty cache (the steps fill it), greedy, host
    tokens in and out every step. It launches nothing but the step's own kernels, so a kernel launch list taken
    over this command is the per-kernel breakdown of the step (TG_USE_GRAPH=0 shows the kernels one by one
    instead of one graph launch)."""
    env = setup(args)
    if env is None:
        return 1
    capi, model = env["capi"], env["model"]
    B, K = args.batch, args.steps
    st = model.state(B, K + 16)
    tok = np.random.default_rng(0).integers(0, model.cfg.n_vocab, size=B).astype(np.int32)
    for _ in range(3):  # eager step, graph capture, first replay
        st.decode(tok, want_logits=False)
        tok = st.sample_argmax()
    capi.launch_count(reset=True)
    t0 = time.perf_counter()
    for _ in range(K):
        st.decode(tok, want_logits=False)
        tok = st.sample_argmax()
    dt = (time.perf_counter() - t0) / K
    print(json.dumps({"mode": "batched-step", "model_size": MODEL, "batch": B, "steps": K, "ms_per_step": dt * 1e3,
                      "tok_s": B / dt, "launches_per_step": capi.launch_count() // K,
                      "timing": "host clock around decode + argmax calls with host tokens, synchronised every step"}), flush=True)
    st.close()
    return 0


# sections of a layer as the kernel's recorder stamps them (CTA 0); the count per layer tells the kernel
PHASES = {
    16: ["A.pro", "A.wait", "A.comp", "A.post", "B.work", "C.pro", "C.comp", "C.post", "D.pro", "D.wait", "D.up", "D.gate",
         "D.issue", "E.wait", "E.comp", "E.bar"],
    17: ["A.pro", "A.bulk", "A.sum", "A.issue", "A.wipe", "B.work", "C.pro", "C.bulk", "C.sum", "C.issue", "D.pro", "D.wait",
         "D.comp", "E.pro", "E.bulk", "E.sum", "E.issue"],
}


def run_phase_clocks(args):
    """Where a decoded token's time goes: arms the persistent kernel's recorder (tg_state_phase_clocks), decodes
    16 tokens twice after the benchmark's prompt and reports, for the last token, the time CTA 0 spent in every
    section of a layer (mean / min / max over the layers), in the lm_head and in the sampler. SM clock stamps are
    converted with the SM clock sampled while the tokens ran."""
    env = setup(args)
    if env is None:
        return 1
    synth, model = env["synth"], env["model"]
    st = model.state(1, 1024)
    prompt = synth.random_prompt(PROMPT_LEN, PROMPT_SEED)
    rf = synth.mt19937_uniforms(64, 1)
    st.phase_clocks()  # arms the recorder
    clocks = ClockSampler(env["local_rank"])
    clocks.start()
    t_end = time.perf_counter() + 1.5  # (the clock sampler needs about a second of load)
    while True:
        st.reset()
        st.prefill(prompt, want_logits=False)
        tok = st.sample_argmax()
        for _ in range(2):
            toks = st.generate(tok, 16, MINP, TEMP, rf[:16]) if not args.greedy else st.generate(tok, 16)
            tok = toks[-1]
        if time.perf_counter() > t_end:
            break
    c = st.phase_clocks()
    clk = clocks.stop()
    mhz = clk["sm_mhz"] or clk["sm_max_mhz"] or 1965.0
    L = model.cfg.n_layers
    d = np.diff(c) / mhz  # us
    ns = (len(d) - 3) // L
    names = PHASES.get(ns, ["s%d" % i for i in range(ns)])
    per = d[:ns * L].reshape(L, ns)
    out = {"mode": "phase-clocks", "model_size": MODEL, "sampler": "greedy" if args.greedy else "minp", "sm_mhz": mhz,
           "clocks": clk, "stamps": int(len(c)),
           "sections_us": {nm: {"mean": float(per[:, i].mean()), "min": float(per[:, i].min()), "max": float(per[:, i].max())}
                           for i, nm in enumerate(names)},
           "layer_mean_us": float(per.sum(axis=1).mean()), "layers_total_us": float(per.sum()),
           "tail_us": {"lm_head.pro": float(d[ns * L]), "lm_head": float(d[ns * L + 1]), "sampler": float(d[ns * L + 2])},
           "step_total_us": float((c[-1] - c[0]) / mhz)}
    print(json.dumps(out), flush=True)
    st.close()
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
    ap.add_argument("--repeats", type=int, default=0,
                    help="repeats of the timed loops; 0: as many as it takes to time one second (use 1 under a profiler)")
    ap.add_argument("--sharded", action="store_true", help="with --batch under torchrun: vocab-sharded lm_head")
    ap.add_argument("--phase-clocks", action="store_true", help="per-section timing of one decoded token (in-kernel recorder)")
    ap.add_argument("--greedy", action="store_true", help="with --phase-clocks: argmax instead of the min-p sampler")
    ap.add_argument("--batched-step", action="store_true", help="time the batched step alone (--batch sequences, empty cache)")
    args = ap.parse_args()
    globals()["MODEL"] = args.model
    globals()["PROMPT_LEN"] = args.prompt_len
    if args.impl == "reference":
        return run_reference(args)
    if args.phase_clocks:
        return run_phase_clocks(args)
    if args.batched_step:
        return run_batched_step(args)
    if args.batch > 1:
        return run_batched(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
