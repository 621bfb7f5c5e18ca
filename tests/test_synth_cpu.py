"""CPU suite: the synthetic weight file is byte-compatible with the reference's own writer."""

import importlib.util
import os
import sys

import numpy as np
import pytest

REFERENCE = os.environ.get("TINY_GEMMA_REFERENCE", os.path.join(os.sep, "root", "reference"))


def _reference_py():
    """the reference's numpy package (py/), loaded under a private name where its checkout is present"""
    init = os.path.join(REFERENCE, "py", "__init__.py")
    if not os.path.exists(init):
        pytest.skip("reference checkout not present")
    try:
        spec = importlib.util.spec_from_file_location("tgref_py", init, submodule_search_locations=[os.path.dirname(init)])
        pkg = importlib.util.module_from_spec(spec)
        sys.modules["tgref_py"] = pkg
        spec.loader.exec_module(pkg)
        gemma = importlib.import_module("tgref_py.gemma")
        wh = importlib.import_module("tgref_py.weight_handlers")
    except Exception as e:  # a dependency of the reference's package missing here
        pytest.skip("reference py package not importable: %r" % (e,))
    return gemma, wh


def test_random_model_bytes_equal_reference_writer(synth, tmp_path):
    """synth.write_random_model against write_from_transformer_weights_quantized (reference py/gemma.py:27-77,
    quantiser py/weight_handlers.py:10-20) on the same fp32 tensors, 270m shape: every byte of the file."""
    gemma, wh = _reference_py()
    t = dict(synth.random_tensors("270m", seed=3))
    c = synth.CONFIGS["270m"]
    layers = []
    for l in range(c.n_layers):
        p = "l%d." % l
        attn = wh.AttentionWeights(q_proj=t[p + "q"], k_proj=t[p + "k"], v_proj=t[p + "v"], o_proj=t[p + "o"],
                                   q_rms_weight=t[p + "q_norm"], k_rms_weight=t[p + "k_norm"],
                                   rms_weight_pre=t[p + "attn_pre"], rms_weight_post=t[p + "attn_post"],
                                   heads=c.n_head, is_sliding=c.is_local(l))
        mlp = wh.MLPWeights(gate_proj=t[p + "gate"], up_proj=t[p + "up"], down_proj=t[p + "down"],
                            rms_weight_post=t[p + "mlp_post"], rms_weight_pre=t[p + "mlp_pre"])
        layers.append(wh.LayerWeights(attn=attn, mlp=mlp))
    w = wh.TransformerWeights(wte=t["wte"], layers=layers, rms_weight=t["final_norm"], lm_head=np.ascontiguousarray(t["wte"].T))
    ref_path = str(tmp_path / "ref.bin")
    gemma.write_from_transformer_weights_quantized(w, ref_path)
    ours = synth.write_random_model(str(tmp_path / "ours.bin"), "270m", seed=3)
    assert os.path.getsize(ours) == os.path.getsize(ref_path) == synth.file_size("270m")
    with open(ours, "rb") as a, open(ref_path, "rb") as b:
        off = 0
        while True:
            x, y = a.read(1 << 24), b.read(1 << 24)
            assert x == y, "files differ in the 16 MiB block at offset %d" % off
            if not x:
                break
            off += len(x)
