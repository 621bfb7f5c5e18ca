"""The C++20 host layer (tiny-gemma_b200/host/tiny_gemma.hpp): the reference's
own names and signatures on top of the C ABI, driven the way the reference's
gemma.cpp / test_generation.cpp drive theirs."""

import os
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HOST = os.path.join(ROOT, "tiny-gemma_b200", "host")
LIBDIR = os.path.join(ROOT, "tiny-gemma_b200")


def _build(tmp_path, capi):
    capi.load()  # makes sure the shared library is built
    exe = str(tmp_path / "gemma_tokens")
    subprocess.check_call(["g++", "-std=c++20", "-O2", "-Wall", "-Werror", "-o", exe, os.path.join(HOST, "gemma_tokens.cpp"),
                           "-L", LIBDIR, "-ltinygemma_b200", "-Wl,-rpath," + LIBDIR])
    return exe


def test_host_layer_compiles_and_fails_loudly_without_gpu(tmp_path, capi):
    exe = _build(tmp_path, capi)
    if capi.device_count() > 0:
        return
    r = subprocess.run([exe, "/nonexistent.bin", "270m", "/dev/null", "1"], capture_output=True, text=True)
    assert r.returncode == 1 and "no CUDA device" in r.stderr  # no CPU fallback behind the C++ API either


@pytest.mark.gpu
def test_cpp_driver_matches_reference_tokens(tmp_path, capi, golden, weights_270m):
    exe = _build(tmp_path, capi)
    g = golden["ref_e2e_270m"]
    ids = tmp_path / "ids.txt"
    ids.write_text(" ".join(str(int(t)) for t in g["prompt"]))
    want = [int(t) for t in g["g1024_tokens"][:41]]
    for extra in ([], ["2.0", "1.0", "0", "--device-loop"]):
        r = subprocess.run([exe, weights_270m, "270m", str(ids), "40"] + extra, capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr
        got = [int(t) for t in r.stdout.split()]
        # the driver builds its own RoPE/GeLU tables (reference constructors' formulas); greedy ids
        # equal the compiled reference's on this prompt (top-2 gaps >= 0.046)
        assert got == want, (got, want)
    # sampled: per-token loop and device-resident loop draw the same std::mt19937 uniforms
    a = subprocess.run([exe, weights_270m, "270m", str(ids), "24", "0.1", "0.7", "1234"], capture_output=True, text=True)
    b = subprocess.run([exe, weights_270m, "270m", str(ids), "24", "0.1", "0.7", "1234", "--device-loop"], capture_output=True,
                       text=True)
    assert a.returncode == 0 and b.returncode == 0, (a.stderr, b.stderr)
    ta, tb = [int(t) for t in a.stdout.split()], [int(t) for t in b.stdout.split()]
    assert len(ta) == len(tb) == 25 and ta[0] == tb[0]
    # the two samplers may differ by one index at a CDF step (different denominator order); once they
    # differ the sequences part, so compare up to the first difference
    first = next((i for i in range(25) if ta[i] != tb[i]), 25)
    assert first >= 8 and (first == 25 or abs(ta[first] - tb[first]) <= 1), (ta, tb)


@pytest.mark.gpu
def test_cpp_driver_error_behaviour(tmp_path, capi, weights_270m):
    exe = _build(tmp_path, capi)
    ids = tmp_path / "ids.txt"
    ids.write_text("1 2 3")
    r = subprocess.run([exe, str(tmp_path / "missing.bin"), "270m", str(ids), "1"], capture_output=True, text=True)
    assert r.returncode == 1 and "Could not open file." in r.stderr  # transformer.hpp:163
    r = subprocess.run([exe, weights_270m, "7B", str(ids), "1"], capture_output=True, text=True)
    assert r.returncode == 1  # CONFIG_MAP.at throws std::out_of_range (gemma.cpp:38)


@pytest.mark.gpu
def test_gemma_cli_generates_text(tmp_path, capi, synth, weights_270m):
    """The text CLI (host/gemma.cpp: the reference's gemma.cpp flags and output, transformer.hpp:167-258) on a
    synthetic 262144-entry tokenizer file: prompt length, streamed text and the statistics line; the generated
    text equals the pieces of the tokens the C ABI generates for the same ids; a seeded sampled run repeats."""
    import re

    import make_tokenizer_golden as tk

    capi.load()
    exe = str(tmp_path / "gemma")
    subprocess.check_call(["g++", "-std=c++20", "-O2", "-Wall", "-Werror", "-o", exe, os.path.join(HOST, "gemma.cpp"), "-L", LIBDIR,
                           "-ltinygemma_b200", "-Wl,-rpath," + LIBDIR])
    check = tk.build_driver(str(tmp_path / "check"), None)
    tok_path = str(tmp_path / "tok.bin")
    vocab = tk.write_vocab(tok_path, n=262144)
    prompt = "hello world and the other one"
    ids = [int(t) for t in tk.run_driver(check, tok_path, 1, [prompt.encode()], False, n=262144)[0].split()[1:]]
    base = [exe, "--weights_path", weights_270m, "--model_size", "270m", "--prompt", prompt, "--chat_format", "1",
            "--terminate_on_eos", "0", "--tokenizer_path", tok_path]
    r = subprocess.run(base + ["--n_dec", "12", "--temp", "1.0"], capture_output=True, timeout=600)
    out = r.stdout.decode("latin-1")
    assert r.returncode == 0, r.stderr
    assert "Weights loaded!\n" in out and ("Prompt length: %d\n" % len(ids)) in out
    m = re.search(r"\n\nGenerating 12 tokens took [0-9.]+ seconds\. Prefill Tok/s: [0-9.]+  Decode Tok/s [0-9.]+ ms/token: [0-9.]+\n$", out)
    assert m, out[-300:]
    # the same ids through the C ABI
    model = capi.Model("270m").load_file(weights_270m).build_tables(1024)
    st = model.state(1, 256)
    st.prefill(np.array(ids, np.int32), want_logits=False)
    first = st.sample_argmax()
    toks = [int(first[0])] + [int(t) for t in st.generate(first, 12).ravel()]
    st.close()
    model.close()

    def piece(t, prev):
        p = vocab[t]
        if prev == 1 and p[:1] == b" ":
            p = p[1:]
        mm = re.fullmatch(rb"<0x([0-9A-Fa-f]{2})>", p)
        return bytes([int(mm.group(1), 16)]) if mm else p

    want, prev = b"", ids[-1]
    for t in toks:
        want += piece(t, prev)
        prev = t
    body = out[out.index("Prompt length"):m.start()].encode("latin-1")
    assert body.endswith(want), (body[-200:], want)
    # sampled, seeded: repeatable
    a = subprocess.run(base + ["--n_dec", "20", "--minp", "0.1", "--temp", "0.7", "--seed", "7"], capture_output=True, timeout=600)
    b = subprocess.run(base + ["--n_dec", "20", "--minp", "0.1", "--temp", "0.7", "--seed", "7"], capture_output=True, timeout=600)
    assert a.returncode == 0 and b.returncode == 0
    strip = lambda s: s[:s.rindex(b"\n\nGenerating")]
    assert strip(a.stdout) == strip(b.stdout)
