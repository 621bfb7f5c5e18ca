"""Multi-process tests of the vocab-sharded lm_head (tiny-gemma_b200/sharded.py)."""

import os
import socket
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _launch(mode, nproc, timeout):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(nproc), "--master-addr",
           "127.0.0.1", "--master-port", str(_free_port()), os.path.join(ROOT, "tests", "dist_worker.py"), mode]
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, cwd=ROOT)


def test_sharded_lm_head_logic_gloo_world2():
    r = _launch("cpu", 2, 300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "rank 0 ok" in r.stdout and "rank 1 ok" in r.stdout


@pytest.mark.gpu
def test_sharded_lm_head_nccl_matches_unsharded(capi):
    import torch

    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs 2 GPUs")
    r = _launch("gpu", 2, 900)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]


@pytest.mark.gpu
@pytest.mark.parametrize("batch", [3, 160])
def test_lm_head_top1_eight_slices_one_gpu(capi, synth, weights_270m, batch):
    """The entry points of the sharded step on one device: 8 column slices scored with tg_dev_lm_head_top1
    (one tensor-core GEMM with the row-maximum epilogue each), resolved with tg_dev_resolve_top1, against the
    whole-vocabulary logits of tg_decode: the maximum must be the logits' maximum (the GEMM and the decode
    step sum in different orders: 1e-5 relative) and the index the lowest index holding it (ops::argmax_logits,
    reference ops.hpp:744-760) wherever the top-2 gap is above that noise. batch 160 takes the 256-column tile
    shape, whose last tile reaches past a slice of 128-column granularity."""
    import importlib

    import numpy as np
    import torch

    sharded = importlib.import_module("tiny-gemma_b200.sharded")
    m = capi.Model("270m").load_file(weights_270m).build_tables(1 << 20)
    V, D, world = m.cfg.n_vocab, m.cfg.hidden_size, 8
    st = m.state(batch, 64)
    prompts = np.stack([synth.random_prompt(12, 300 + b) for b in range(batch)])
    st.prefill(prompts, want_logits=False)
    first = st.sample_argmax()
    logits = st.decode(first)  # [batch, V]
    st.close()
    st = m.state(batch, 64)  # the same step again, stopped before the lm_head
    st.prefill(prompts, want_logits=False)
    st.decode_hidden(first)
    hidden = torch.empty((batch, D), dtype=torch.float32, device="cuda")
    stream = st.stream()
    st.hidden_copy_dev(hidden.data_ptr())
    cand_all = torch.empty((world * 2, batch), dtype=torch.int32, device="cuda")
    for r in range(world):
        col0, ncols = sharded.shard_columns(V, r, world)
        m.lm_head_top1_dev(hidden.data_ptr(), batch, col0, ncols, cand_all[2 * r].data_ptr(), cand_all[2 * r + 1].data_ptr(), stream)
    toks = torch.empty(batch, dtype=torch.int32, device="cuda")
    m.resolve_top1_dev(cand_all.data_ptr(), world, batch, 0, batch, toks.data_ptr(), stream)
    st.check()
    torch.cuda.synchronize()
    got = toks.cpu().numpy()
    c = cand_all.cpu().numpy().reshape(world, 2, batch)
    maxs, idxs = c[:, 0, :].view(np.float32), c[:, 1, :]
    # every slice's candidate against the logits of that slice
    for r in range(world):
        col0, ncols = sharded.shard_columns(V, r, world)
        sl = logits[:, col0:col0 + ncols]
        assert np.all((idxs[r] >= col0) & (idxs[r] < col0 + ncols))
        np.testing.assert_allclose(maxs[r], sl.max(axis=1), rtol=2e-5, atol=1e-6)
        np.testing.assert_allclose(logits[np.arange(batch), idxs[r]], sl.max(axis=1), rtol=2e-5, atol=1e-6)
    # the torch form of the resolution on the same candidates
    g = torch.stack([torch.from_numpy(maxs.astype(np.float64)), torch.from_numpy(idxs.astype(np.float64))], dim=2)
    assert np.array_equal(sharded.resolve_candidates(torch, g).numpy(), got)
    top2 = np.partition(logits, -2, axis=1)[:, -2:]
    clear = (top2[:, 1] - top2[:, 0]) > 1e-4 * np.abs(top2[:, 1])
    assert clear.sum() >= batch // 2
    assert np.array_equal(got[clear], logits.argmax(axis=1)[clear])
    # a second call on the same scratch, slices in another order, must give the same candidates
    cand2 = torch.empty_like(cand_all)
    for r in reversed(range(world)):
        col0, ncols = sharded.shard_columns(V, r, world)
        m.lm_head_top1_dev(hidden.data_ptr(), batch, col0, ncols, cand2[2 * r].data_ptr(), cand2[2 * r + 1].data_ptr(), stream)
    torch.cuda.synchronize()
    assert torch.equal(cand2, cand_all)
    st.close()
    m.close()


@pytest.mark.gpu
def test_two_devices_in_one_process(capi, synth, weights_270m):
    """Models on two GPUs of one process (the C ABI takes the device per model): the kernels' per-device
    attributes (dynamic shared memory opt-in) must be set on each device, so prefill, the persistent decode
    kernel, the batch-2 per-phase path and the batched tensor-core step all have to work on device 1 after
    device 0 has used them, and give the same tokens."""
    import numpy as np
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    out = []
    for dev in (0, 1):
        m = capi.Model("270m", device=dev).load_file(weights_270m).build_tables(1 << 20)
        ids = synth.random_prompt(40, 21)
        st = m.state(1, 128)
        st.prefill(ids, want_logits=False)
        t1 = st.generate(st.sample_argmax(), 8).ravel()
        st.close()
        st = m.state(2, 128)
        st.prefill(np.stack([ids, ids[::-1]]), want_logits=False)
        t2 = st.generate(st.sample_argmax(), 4).ravel()
        st.close()
        st = m.state(8, 128)
        st.prefill(np.stack([synth.random_prompt(40, 30 + b) for b in range(8)]), want_logits=False)
        t8 = st.generate(st.sample_argmax(), 4).ravel()
        st.close()
        m.close()
        out.append((t1, t2, t8))
    for a, b in zip(out[0], out[1]):
        assert np.array_equal(a, b)
