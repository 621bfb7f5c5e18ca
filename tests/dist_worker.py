"""Worker for the multi-process tests; launched with torch.distributed.run.

    ... tests/dist_worker.py cpu     gloo, world_size 2: the sharding / candidate-resolution
                                     logic of tiny-gemma_b200/sharded.py against an unsharded argmax
    ... tests/dist_worker.py gpu     nccl, one GPU per rank: sharded greedy decoding of 270m
                                     against the same sequences decoded with the whole lm_head
"""

import importlib
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sharded = importlib.import_module("tiny-gemma_b200.sharded")


def first_max(x):
    return int(np.argmax(x))  # numpy returns the first maximum = reference tie rule


def run_cpu(rank, world):
    V, D, b = 128 * world * 4, 64, 3
    rng = np.random.default_rng(0)  # same data on every rank
    w = rng.integers(-127, 128, size=(D, V), dtype=np.int8)
    s = np.exp(rng.uniform(np.log(1e-4), np.log(1e-2), size=V)).astype(np.float32)
    # exact ties across shards: duplicate one column of shard 0 into the other shards
    s[7] = 1.0  # a scale far above the others, so that column 7 (and its copies) can be made the maximum
    for r in range(1, world):
        w[:, r * (V // world) + 5] = w[:, 7]
        s[r * (V // world) + 5] = s[7]
    hidden = rng.standard_normal((world * b, D)).astype(np.float32)
    hidden[1] = 0.0  # all logits equal (0): lowest index overall must win
    boost = np.zeros(D, np.float32)
    boost[:] = w[:, 7].astype(np.float32)  # makes column 7 (and its duplicates) the maximum
    hidden[2] = boost

    def score(hidden_all, col0, ncols):
        h = hidden_all.numpy()
        lg = (h @ w[:, col0:col0 + ncols].astype(np.float32)) * s[col0:col0 + ncols]
        idx = np.array([first_max(r) for r in lg], np.int32)
        mx = lg[np.arange(lg.shape[0]), idx].astype(np.float32)
        return torch.from_numpy(mx), torch.from_numpy(idx + col0)

    mine = torch.from_numpy(hidden[rank * b:(rank + 1) * b].copy())
    toks = sharded.sharded_greedy_step(torch, dist, mine, score, rank, world, V)
    full = (hidden @ w.astype(np.float32)) * s
    want = [first_max(full[i]) for i in range(rank * b, (rank + 1) * b)]
    assert toks.tolist() == want, (rank, toks.tolist(), want)
    if rank == 0:
        assert want[1] == 0 and want[2] == 7  # the tie cases resolved to the lowest index
    # shard arithmetic and the no-candidate case
    assert sharded.shard_columns(262144, 3, 8) == (98304, 32768)
    g = torch.tensor([[[float("-inf"), -1.0]], [[1.5, 40.0]]], dtype=torch.float64)
    assert sharded.resolve_candidates(torch, g).tolist() == [40]
    g = torch.tensor([[[float("-inf"), -1.0]], [[float("-inf"), -1.0]]], dtype=torch.float64)
    assert sharded.resolve_candidates(torch, g).tolist() == [-1]


def run_gpu(rank, world):
    capi = importlib.import_module("tiny-gemma_b200.capi")
    synth = importlib.import_module("tiny-gemma_b200.synth")
    torch.cuda.set_device(rank)
    path = os.path.join(os.environ.get("TG_CACHE_DIR", "/tmp"), "tg_270m_s0.bin")
    if rank == 0:
        synth.write_random_model(path, "270m", 0)
    dist.barrier()
    m = capi.Model("270m", device=rank).load_file(path).build_tables(1024)
    b, steps = 2, 12
    prompts = np.stack([synth.random_prompt(48, 100 + rank * b + i) for i in range(b)])
    # reference run on this rank: whole lm_head, greedy
    ref = m.state(b, 128)
    ref.prefill(prompts, want_logits=False)
    first = ref.sample_argmax()
    want = ref.generate(first, steps)  # [steps, b]
    ref.close()
    st = m.state(b, 128)
    st.prefill(prompts, want_logits=False)
    dec = sharded.ShardedGreedyDecoder(torch, dist, m, st, rank, world)
    got = []
    dec.step(first)
    got.append(dec.tokens_host())
    for _ in range(steps - 1):
        dec.step(None)
        got.append(dec.tokens_host())
    got = np.stack(got)
    assert np.array_equal(got, want), (rank, got.T, want.T)
    st.close()
    m.close()


def main():
    mode = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    if mode == "cpu":
        dist.init_process_group("gloo")
        run_cpu(rank, world)
    else:
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
        run_gpu(rank, world)
    dist.barrier()
    dist.destroy_process_group()
    print("rank %d ok" % rank)


if __name__ == "__main__":
    main()
