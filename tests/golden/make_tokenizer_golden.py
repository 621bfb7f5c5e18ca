"""Synthetic tokenizer vocabulary in the reference's file format (py/convert.py:108-113) and, from it, the golden
encodings of the reference's own csrc/include/tokenizer.hpp:

    python tests/golden/make_tokenizer_golden.py     # -> tests/golden/tokenizer_golden.json

The driver tiny-gemma_b200/host/tokenizer_check.cpp is compiled against the reference's header (a copy of the
driver in a scratch directory, so that its #include "tokenizer.hpp" resolves to the reference's include
directory) and run on TEXTS; its output is stored. The reference's decode throws on byte-fallback tokens, so
decoded text is stored only for the texts in DECODABLE."""

from __future__ import annotations

import json
import os
import shutil
import struct
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
DRIVER = os.path.join(ROOT, "tiny-gemma_b200", "host", "tokenizer_check.cpp")
REFERENCE = os.environ.get("TINY_GEMMA_REFERENCE", os.path.join(os.sep, "root", "reference"))
VOCAB_SIZE = 5000

TEXTS = [
    "hello world",
    " the theatre in an anthem",
    "aaaaaaa ab abc",
    "é 日本語 🙂🙂🚀 ✓",
    "",
    "  leading and\ttab",  # tab has no entry: byte fallback
    "xyz\x01\x7f",
    b"bad \xc3 tail \xe6\x97\xa5\x80\x80\x80\x80z".decode("latin-1"),  # written as raw bytes below
    "The quick brown fox jumps over the lazy dog and then the other one",
]
RAW = {7}  # indices of TEXTS whose latin-1 code points are the raw bytes (malformed UTF-8)
DECODABLE = [0, 1, 2, 3, 4, 8]


def text_bytes(i: int) -> bytes:
    return TEXTS[i].encode("latin-1") if i in RAW else TEXTS[i].encode("utf-8")


def write_vocab(path: str, n: int = VOCAB_SIZE, seed: int = 0) -> list[bytes]:
    """n entries: <unk> <eos> <bos>, the 256 byte tokens "<0xNN>" at ids 3..258 (where the reference's byte
    fallback expects them), printable ASCII and some multi-byte code points, a few hand-made merges, one
    duplicated text, then random lower-case strings (more duplicates); the chat-template ids hold their texts.
    Scores fall with the id, with a band of equal scores so that ties between different merges occur."""
    rng = np.random.default_rng(seed)
    toks = [b"<unk>", b"<eos>", b"<bos>"] + [b"<0x%02X>" % b for b in range(256)]
    toks += [chr(c).encode() for c in range(32, 127)] + [c.encode() for c in "äöüéèñçßøåμπλ中文日本語한국어✓€→🙂🚀"]
    toks += [w.encode() for w in ["the", " the", "he", "th", " t", "in", " a", "er", "an", " an", "re", "on", " on", "at", "en", "nd",
                                  " th", "ing", " in", "llo", "hel", "hello", " hello", " wor", "ld", " world", "wor", "orl", "lo",
                                  "ll", "  ", "\n\n", "ab", "abc", "bc", "aa", "aaa", "aaaa", "é ", "日本", "本語", "日本語", "🙂🙂"]]
    toks.append(b"ab")
    while len(toks) < n:
        toks.append(bytes(rng.choice(list(b"abcdefghijklmnopqrstuvwxyz "), size=int(rng.integers(2, 6))).tolist()))
    toks[105], toks[106], toks[107], toks[2364], toks[4368] = b"<start_of_turn>", b"<end_of_turn>", b"\n", b"user", b"model"
    scores = (-np.arange(n) * 0.25).astype(np.float32)
    scores[rng.integers(300, n, size=200)] = -7.0
    with open(path, "wb") as f:
        f.write(struct.pack("I", max(len(t) for t in toks)))
        for t, s in zip(toks, scores):
            f.write(struct.pack("fI", float(s), len(t)))
            f.write(t)
    return toks


def build_driver(out: str, include_dir: str | None) -> str:
    """include_dir None: this repository's header (beside the driver); else a copy of the driver compiled with -I include_dir"""
    if include_dir is None:
        subprocess.check_call(["g++", "-std=c++20", "-O2", "-Wall", "-Werror", "-o", out, DRIVER])
    else:
        d = tempfile.mkdtemp()
        try:
            shutil.copy(DRIVER, d)
            subprocess.check_call(["g++", "-std=c++20", "-O2", "-I", include_dir, "-o", out, os.path.join(d, "tokenizer_check.cpp")])
        finally:
            shutil.rmtree(d)
    return out


def run_driver(exe: str, vocab: str, chat: int, texts: list[bytes], decode: bool, n: int = VOCAB_SIZE) -> list[str]:
    with tempfile.NamedTemporaryFile("wb", suffix=".txt", delete=False) as f:
        f.write(b"\n".join(texts) + b"\n")
    try:
        r = subprocess.run([exe, vocab, str(n), str(chat), f.name] + (["--decode"] if decode else []), capture_output=True)
    finally:
        os.unlink(f.name)
    if r.returncode:
        raise RuntimeError(r.stderr.decode(errors="replace"))
    return r.stdout.decode("latin-1").split("\n")


def main():
    inc = os.path.join(REFERENCE, "csrc", "include")
    if not os.path.exists(os.path.join(inc, "tokenizer.hpp")):
        sys.exit("reference checkout not found")
    tmp = tempfile.mkdtemp()
    try:
        vocab = os.path.join(tmp, "tok.bin")
        write_vocab(vocab)
        exe = build_driver(os.path.join(tmp, "ref_check"), inc)
        out = {"vocab_size": VOCAB_SIZE, "seed": 0}
        for chat in (0, 1):
            out["ids_chat%d" % chat] = run_driver(exe, vocab, chat, [text_bytes(i) for i in range(len(TEXTS))], False)
            out["decode_chat%d" % chat] = run_driver(exe, vocab, chat, [text_bytes(i) for i in DECODABLE], True)
        with open(os.path.join(HERE, "tokenizer_golden.json"), "w") as f:
            json.dump(out, f, indent=1)
        print("tokenizer_golden.json:", sum(len(v) for v in out.values() if isinstance(v, list)), "lines")
    finally:
        shutil.rmtree(tmp)


if __name__ == "__main__":
    main()
