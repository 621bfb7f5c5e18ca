"""Vocab-sharded lm_head over several GPUs, one process per GPU.

The [D, V] lm_head is split by columns: rank r owns vocabulary columns
[r * V/world, (r+1) * V/world). Sequences are data-parallel: every rank runs the
layers for its own sequences. Per decode step

  1. all-gather of the final-normed hidden states  [b, D] -> [world * b, D]
  2. every rank scores ALL sequences against its column slice and keeps, per
     sequence, the maximum logit and its global index (lowest index on ties)
  3. all-gather of those candidates  [M, 2] -> [world, M, 2]
  4. every rank resolves its own sequences: largest maximum, and among equal
     maxima the lowest global index — the tie rule of the reference's
     argmax_logits (ops.hpp:744-760).

Both exchanges are a few KB to ~1 MB: latency-bound NCCL all-gathers over NVLink.
The collectives go through torch.distributed (NCCL on GPUs, gloo in the CPU
tests of this logic); the forward, the scoring (one tensor-core GEMM over the
slice with a row-maximum epilogue) and the resolution of the candidates are the
library's kernels. resolve_candidates / sharded_greedy_step below are the same
logic in torch operations: the form the gloo tests run, and the checker of the
device kernel.
"""

from __future__ import annotations

import numpy as np


def shard_columns(n_vocab: int, rank: int, world: int, align: int = 128) -> tuple[int, int]:
    """(first column, number of columns) of rank's slice; every slice a multiple of `align`"""
    if n_vocab % (world * align):
        raise ValueError("n_vocab must be a multiple of world * %d" % align)
    n = n_vocab // world
    return rank * n, n


def pack_candidates(torch, maxs, idxs):
    """[M] float32 maxima + [M] int32 indices -> [M, 2] float64 (both exactly representable)"""
    return torch.stack([maxs.to(torch.float64), idxs.to(torch.float64)], dim=1).contiguous()


def resolve_candidates(torch, gathered):
    """gathered: [world, M, 2] float64 -> [M] int64 token ids.

    Largest maximum wins; among equal maxima the lowest index; a slice with no
    candidate (index -1, nothing above -inf) never wins; -1 if no slice has one.
    """
    vals, idxs = gathered[..., 0], gathered[..., 1]
    valid = idxs >= 0
    vals = torch.where(valid, vals, torch.full_like(vals, -float("inf")))
    best = vals.max(dim=0).values  # [M]
    is_best = (vals == best.unsqueeze(0)) & valid
    big = torch.full_like(idxs, float(2**52))
    pick = torch.where(is_best, idxs, big).min(dim=0).values
    return torch.where(pick >= big[0], torch.full_like(pick, -1.0), pick).to(torch.int64)


def sharded_greedy_step(torch, dist, hidden_local, score_slice, rank: int, world: int, n_vocab: int):
    """One exchange: hidden_local [b, D] (this rank's sequences) -> token ids [b] (int64).

    score_slice(hidden_all [M, D], col0, ncols) -> (max [M] float32, idx [M] int32, global indices)
    """
    b = hidden_local.shape[0]
    hidden_all = torch.empty((world * b, hidden_local.shape[1]), dtype=hidden_local.dtype, device=hidden_local.device)
    dist.all_gather_into_tensor(hidden_all, hidden_local.contiguous())
    col0, ncols = shard_columns(n_vocab, rank, world)
    maxs, idxs = score_slice(hidden_all, col0, ncols)
    cand = pack_candidates(torch, maxs, idxs)
    gathered = torch.empty((world * cand.shape[0], 2), dtype=cand.dtype, device=cand.device)
    dist.all_gather_into_tensor(gathered, cand)  # concatenated along dim 0, rank-major
    toks = resolve_candidates(torch, gathered.view(world, cand.shape[0], 2))
    return toks[rank * b:(rank + 1) * b]


class ShardedGreedyDecoder:
    """Greedy decoding of this rank's sequences with the lm_head sharded over `world` GPUs.

    A step only enqueues: the layers, both all-gathers (NCCL, ordered after the state's stream, which is
    made torch's current stream), the slice scoring and the candidate resolution run back to back on the
    device; nothing waits on the host until the caller reads the tokens or calls state.check()."""

    def __init__(self, torch, dist, model, state, rank: int, world: int):
        self.torch, self.dist = torch, dist
        self.model, self.state = model, state
        self.rank, self.world = rank, world
        self.V = model.cfg.n_vocab
        self.D = model.cfg.hidden_size
        b, M = state.B, world * state.B
        dev = torch.device("cuda", torch.cuda.current_device())
        self.stream = torch.cuda.ExternalStream(state.stream())
        self.hidden = torch.empty((b, self.D), dtype=torch.float32, device=dev)
        self.hidden_all = torch.empty((M, self.D), dtype=torch.float32, device=dev)
        self.cand = torch.empty((2, M), dtype=torch.int32, device=dev)  # row 0: maxima (fp32 bits), row 1: global indices
        self.cand_all = torch.empty((world * 2, M), dtype=torch.int32, device=dev)
        self.toks = torch.empty(b, dtype=torch.int32, device=dev)
        self.col0, self.ncols = shard_columns(self.V, rank, world)

    def step(self, ids=None):
        """feed `ids` (host, [b]) or the tokens of the previous step; returns the new tokens [b] (device int32,
        valid in stream order on the state's stream)"""
        torch, st = self.torch, self.stream.cuda_stream
        M = self.hidden_all.shape[0]
        with torch.cuda.stream(self.stream):
            self.state.decode_hidden(ids)
            self.state.hidden_copy_dev(self.hidden.data_ptr())
            self.dist.all_gather_into_tensor(self.hidden_all, self.hidden)
            self.model.lm_head_top1_dev(self.hidden_all.data_ptr(), M, self.col0, self.ncols, self.cand[0].data_ptr(),
                                        self.cand[1].data_ptr(), st)
            self.dist.all_gather_into_tensor(self.cand_all, self.cand)
            self.model.resolve_top1_dev(self.cand_all.data_ptr(), self.world, M, self.rank * self.state.B, self.state.B,
                                        self.toks.data_ptr(), st)
            self.state.set_tokens_dev(self.toks.data_ptr())
        return self.toks

    def tokens_host(self):
        """the tokens of the last step as a numpy array (waits for the state's stream)"""
        with self.torch.cuda.stream(self.stream):
            return self.toks.cpu().numpy().copy()
