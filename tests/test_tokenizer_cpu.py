"""CPU suite: sentencepiece::Tokenizer of the host layer (tiny-gemma_b200/host/tokenizer.hpp) against the
reference's tokenizer (csrc/include/tokenizer.hpp:77-239) on a synthetic vocabulary file in the format of
py/convert.py:108-113: committed golden output of the reference, and, where the reference checkout is present,
the reference's header compiled live on random texts. The gemma CLI's argument handling needs no GPU either."""

import json
import os
import subprocess

import numpy as np
import pytest

import make_tokenizer_golden as tk

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HOST = os.path.join(ROOT, "tiny-gemma_b200", "host")
LIBDIR = os.path.join(ROOT, "tiny-gemma_b200")


@pytest.fixture(scope="module")
def vocab(tmp_path_factory):
    p = str(tmp_path_factory.mktemp("tok") / "tok.bin")
    tk.write_vocab(p)
    return p


@pytest.fixture(scope="module")
def ours(tmp_path_factory):
    return tk.build_driver(str(tmp_path_factory.mktemp("tokexe") / "check"), None)


def test_tokenizer_matches_reference_golden(ours, vocab):
    """ids for every text (malformed UTF-8, byte fallback, duplicate vocabulary texts, equal merge scores,
    chat template on and off) and decoded text / pieces for the texts the reference can decode. (Which of two
    entries with the same text is found follows std::sort's order of equal keys: the golden file holds for
    the standard library of this image.)"""
    g = json.load(open(os.path.join(ROOT, "tests", "golden", "tokenizer_golden.json")))
    for chat in (0, 1):
        got = tk.run_driver(ours, vocab, chat, [tk.text_bytes(i) for i in range(len(tk.TEXTS))], False)
        assert got == g["ids_chat%d" % chat]
        got = tk.run_driver(ours, vocab, chat, [tk.text_bytes(i) for i in tk.DECODABLE], True)
        assert got == g["decode_chat%d" % chat]


def test_tokenizer_round_trip_and_byte_tokens(ours, vocab):
    """decode(encode(text)) gives "<bos>" + text when every code point is in the vocabulary; a byte-fallback
    token decodes to its byte (the reference throws there)."""
    texts = ["hello world and the other", "é 日本語 ✓", "tab\there", "\x01"]
    out = tk.run_driver(ours, vocab, 0, [t.encode() for t in texts], True)
    lines = [l for l in out if l.startswith("text: ")]
    assert [l[len("text: "):].encode("latin-1").decode("utf-8") for l in lines] == ["<bos>" + t for t in texts]
    ids = [l for l in out if l.startswith("ids:")]
    assert ids[2].split()[1:] == ["2"] + ids[2].split()[2:] and str(9 + 3) in ids[2].split()  # the tab is token 9 + 3
    assert ids[3].split()[1:] == ["2", "4"]


def test_tokenizer_matches_live_reference_on_random_texts(ours, vocab, tmp_path):
    inc = os.path.join(tk.REFERENCE, "csrc", "include")
    if not os.path.exists(os.path.join(inc, "tokenizer.hpp")):
        pytest.skip("reference checkout not present")
    ref = tk.build_driver(str(tmp_path / "ref_check"), inc)
    rng = np.random.default_rng(5)
    alphabet = list("abcdefghijklmnopqrstuvwxyz      theinanerlo") + ["é", "日", "本", "語", "🙂", "✓", "Q", "7"]
    texts = ["".join(rng.choice(alphabet, size=int(rng.integers(1, 120)))).encode() for _ in range(200)]
    texts += [bytes(rng.integers(1, 256, size=int(rng.integers(1, 40))).tolist()).replace(b"\n", b" ") for _ in range(50)]  # arbitrary bytes
    for chat in (0, 1):
        assert tk.run_driver(ours, vocab, chat, texts, False) == tk.run_driver(ref, vocab, chat, texts, False)
        assert tk.run_driver(ours, vocab, chat, texts[:200], True) == tk.run_driver(ref, vocab, chat, texts[:200], True)


def test_tokenizer_missing_file_error(ours, tmp_path):
    r = subprocess.run([ours, str(tmp_path / "none.bin"), "10", "0", "/dev/null"], capture_output=True, text=True)
    assert r.returncode == 1 and "Cannot open model file: " in r.stderr  # tokenizer.hpp:85


def test_gemma_cli_argument_errors(tmp_path, capi):
    """the option grammar of the reference's argparse.hpp:30-52 (every option is "--name value"): the three usage
    errors return 1 with the message and the option list, a value that does not parse is a "Parse error"."""
    capi.load()
    exe = str(tmp_path / "gemma")
    subprocess.check_call(["g++", "-std=c++20", "-O2", "-Wall", "-Werror", "-o", exe, os.path.join(HOST, "gemma.cpp"), "-L", LIBDIR,
                           "-ltinygemma_b200", "-Wl,-rpath," + LIBDIR])
    for args, msg in ((["stray"], "Error: unexpected token: stray"), (["--nope", "1"], "Error: unknown option: --nope"),
                      (["--n_dec"], "Error: missing value for --n_dec"), (["--n_dec", "many"], "Parse error: expected integer for many"),
                      (["--temp", "warm"], "Parse error: expected float for warm")):
        r = subprocess.run([exe] + args, capture_output=True, text=True)
        assert r.returncode == 1 and msg in r.stderr, (args, r.stderr)
    r = subprocess.run([exe, "--model_size", "7B"], capture_output=True, text=True)
    assert r.returncode == 1  # CONFIG_MAP.at throws std::out_of_range (gemma.cpp:38)
