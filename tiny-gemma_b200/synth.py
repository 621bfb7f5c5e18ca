"""Seeded random-init Gemma-3 weights in the ``gemma_i8.bin`` layout, plus prompts.

There is no checkpoint to download where this runs, so benchmarks and parity
tests use random weights of the real architecture. The file produced here is
byte-for-byte what the reference converter would write for the same float
tensors:

* layout and order  — reference ``py/gemma.py:27-77``
  (``write_from_transformer_weights_quantized``), read back by
  ``csrc/include/transformer.hpp:99-165`` (``read_weights``);
* quantiser         — reference ``py/weight_handlers.py:10-20``: one fp32 scale
  per column of the stored 2-D array, ``scale = max|W| / 127`` over axis 0,
  ``q = rint(W / scale)`` as int8.

No header, no padding, native little-endian.
"""

from __future__ import annotations

import os
from dataclasses import dataclass

import numpy as np


@dataclass(frozen=True)
class Config:
    """Field order follows reference ``csrc/include/config.hpp:7-20``."""

    hidden_size: int
    intermediate_size: int
    n_layers: int
    n_vocab: int
    n_pos: int
    n_pos_local: int
    head_dim: int
    n_head: int
    n_kv: int
    rope_theta: float
    rope_theta_local: float
    window_pattern: int

    @property
    def q_dim(self) -> int:
        return self.n_head * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.n_kv * self.head_dim

    def is_local(self, layer: int) -> bool:
        # reference transformer.hpp:43
        return (layer % self.window_pattern) != (self.window_pattern - 1)


# reference config.hpp:46-48
CONFIGS = {
    "270m": Config(640, 2048, 18, 262144, 32768, 512, 256, 4, 1, 1_000_000.0, 10_000.0, 6),
    "1B": Config(1152, 6912, 26, 262144, 32768, 512, 256, 4, 1, 1_000_000.0, 10_000.0, 6),
}


def quantize_weight(w: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """Per-column int8 quantiser (reference ``py/weight_handlers.py:10-20``)."""
    assert w.ndim == 2
    scales = (np.max(np.abs(w), axis=0, keepdims=True) / 127.0).astype(np.float32)
    q = np.rint(w / scales).astype(np.int8)
    return q, scales


def layout(size: str) -> list[tuple[str, str, tuple[int, ...], int]]:
    """[(name, dtype, shape, byte offset)] of every tensor in file order."""
    c = CONFIGS[size]
    out = []
    off = 0

    def add(name, dtype, shape):
        nonlocal off
        out.append((name, dtype, shape, off))
        off += int(np.prod(shape)) * (1 if dtype == "i1" else 4)

    def addq(name, rows, cols):
        add(name + ".q", "i1", (rows, cols))
        add(name + ".s", "f4", (cols,))

    addq("wte", c.n_vocab, c.hidden_size)
    add("final_norm", "f4", (c.hidden_size,))
    for l in range(c.n_layers):
        p = f"l{l}."
        addq(p + "q", c.hidden_size, c.q_dim)
        addq(p + "k", c.hidden_size, c.kv_dim)
        addq(p + "v", c.hidden_size, c.kv_dim)
        addq(p + "o", c.q_dim, c.hidden_size)
        add(p + "q_norm", "f4", (c.head_dim,))
        add(p + "k_norm", "f4", (c.head_dim,))
        add(p + "attn_pre", "f4", (c.hidden_size,))
        add(p + "attn_post", "f4", (c.hidden_size,))
        addq(p + "up", c.hidden_size, c.intermediate_size)
        addq(p + "gate", c.hidden_size, c.intermediate_size)
        addq(p + "down", c.intermediate_size, c.hidden_size)
        add(p + "mlp_pre", "f4", (c.hidden_size,))
        add(p + "mlp_post", "f4", (c.hidden_size,))
    addq("lm_head", c.hidden_size, c.n_vocab)
    out.append(("<end>", "i1", (0,), off))
    return out


def file_size(size: str) -> int:
    return layout(size)[-1][3]


def random_tensors(size: str, seed: int = 0, std: float = 0.02):
    """The seeded N(0, std) fp32 tensors of a model in file order, as (name, array): wte [V, D], final_norm,
    then per layer q, k, v, o, q_norm, k_norm, attn_pre, attn_post, up, gate, down, mlp_pre, mlp_post
    (names prefixed l<layer>.). The lm_head is tied: wte.T."""
    c = CONFIGS[size]
    rng = np.random.default_rng(seed)

    def normal(*shape):
        return (rng.standard_normal(shape, dtype=np.float32) * np.float32(std)).astype(np.float32)

    yield "wte", normal(c.n_vocab, c.hidden_size)
    yield "final_norm", normal(c.hidden_size)
    for l in range(c.n_layers):
        p = "l%d." % l
        yield p + "q", normal(c.hidden_size, c.q_dim)
        yield p + "k", normal(c.hidden_size, c.kv_dim)
        yield p + "v", normal(c.hidden_size, c.kv_dim)
        yield p + "o", normal(c.q_dim, c.hidden_size)
        yield p + "q_norm", normal(c.head_dim)
        yield p + "k_norm", normal(c.head_dim)
        yield p + "attn_pre", normal(c.hidden_size)
        yield p + "attn_post", normal(c.hidden_size)
        yield p + "up", normal(c.hidden_size, c.intermediate_size)
        yield p + "gate", normal(c.hidden_size, c.intermediate_size)
        yield p + "down", normal(c.intermediate_size, c.hidden_size)
        yield p + "mlp_pre", normal(c.hidden_size)
        yield p + "mlp_post", normal(c.hidden_size)


def write_random_model(path: str, size: str, seed: int = 0, std: float = 0.02) -> str:
    """Write the tensors of random_tensors (norm weights included, lm_head tied to
    wte before quantisation) to ``path`` in the gemma_i8.bin layout (reference
    ``py/gemma.py:27-77``); returns ``path``. Skips the work if a file of the
    right size is already there (callers encode size/seed in the name)."""
    want = file_size(size)
    if os.path.exists(path) and os.path.getsize(path) == want:
        return path
    tmp = path + ".tmp%d" % os.getpid()
    with open(tmp, "wb") as f:
        wte = None
        for name, w in random_tensors(size, seed, std):
            if w.ndim == 2:
                q, s = quantize_weight(w)
                f.write(np.ascontiguousarray(q).data)
                f.write(np.ascontiguousarray(s).data)
                if name == "wte":
                    wte = w
            else:
                f.write(w.data)
        # tied embeddings: lm_head = wte.T as floats, quantised per vocab column
        s_v = (np.max(np.abs(wte), axis=1) / 127.0).astype(np.float32)  # [V]
        q = np.rint(wte / s_v[:, None]).astype(np.int8)  # [V, D]
        f.write(np.ascontiguousarray(q.T).data)
        f.write(s_v.data)
    assert os.path.getsize(tmp) == want, (os.path.getsize(tmp), want)
    os.replace(tmp, path)
    return path


def random_prompt(n: int, seed: int, vocab: int = 262144) -> np.ndarray:
    """``n`` token ids uniform in [0, vocab) — stands in for the reference's
    ultrachat prompts (mean length 178, reference ``README.md:50``)."""
    return np.random.default_rng(seed).integers(0, vocab, size=n, dtype=np.int32)


def mt19937_uniforms(n: int, seed: int) -> np.ndarray:
    """``n`` draws of ``std::uniform_real_distribution<float>(0,1)`` over
    ``std::mt19937(seed)`` (reference ``transformer.hpp:170-172``): libstdc++'s
    ``generate_canonical<float,24>`` takes one 32-bit word per draw, scales it
    by 2^-32 in float and maps a result of 1.0 to the float just below 1."""
    rs = np.random.RandomState()
    key = np.zeros(624, dtype=np.uint32)
    # std::mt19937 seeding: x[0]=seed, x[i] = 1812433253*(x[i-1]^(x[i-1]>>30)) + i
    x = np.uint64(seed & 0xFFFFFFFF)
    key[0] = x
    for i in range(1, 624):
        x = (np.uint64(1812433253) * (x ^ (x >> np.uint64(30))) + np.uint64(i)) & np.uint64(0xFFFFFFFF)
        key[i] = x
    rs.set_state(("MT19937", key, 624))
    words = rs.randint(0, 2**32, size=n, dtype=np.uint64).astype(np.uint32)
    out = words.astype(np.float32) * np.float32(2.0**-32)
    out[out >= np.float32(1.0)] = np.nextafter(np.float32(1.0), np.float32(0.0))
    return out.astype(np.float32)
