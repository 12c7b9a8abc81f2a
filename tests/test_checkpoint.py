"""Checkpoint import: the reference's ModelSerializer format (persistence/ModelSerializer.java:44-98) read back
into named decoder weights.  The expected bytes are built here with `struct`, independently of the module."""
import struct

import numpy as np
import pytest

from deepj_b200.checkpoint import named_parameters, parameter_layout, read_parameters, weight_getter, write_parameters
from deepj_b200.decoder import DecoderConfig


def java_bytes(params):
    """DataOutputStream: writeInt(count); per tensor writeInt(rows), writeInt(cols), writeDouble((double) v)…"""
    out = [struct.pack(">i", len(params))]
    for p in params:
        out.append(struct.pack(">ii", p.shape[0], p.shape[1]))
        out.append(b"".join(struct.pack(">d", float(v)) for v in p.reshape(-1)))
    return b"".join(out)


def random_params(cfg, seed=0):
    rng = np.random.default_rng(seed)
    return [rng.standard_normal(shape).astype(np.float32) for _, _, shape in parameter_layout(cfg)]


def test_layout_follows_parameters_order():
    cfg = DecoderConfig("llama", 11, 16, 8, 2, 2, 24)
    names = [(n, l) for n, l, _ in parameter_layout(cfg)]
    assert names[0] == ("emb", -1)
    assert names[1:13] == [("g1", 0), ("g2", 0), ("Wq", 0), ("Wk", 0), ("Wv", 0), ("Wo", 0), ("Wg", 0), ("bg", 0),
                           ("Wu", 0), ("bu", 0), ("Wd", 0), ("bd", 0)]          # ln1, ln2, attn, mlp — W before b
    assert names[-3:] == [("gF", -1), ("Wlm", -1), ("blm", -1)]
    assert len(names) == 1 + 2 * 12 + 3
    ds = DecoderConfig("deepseek", 11, 16, 8, 2, 1, 24, q_rank=4, kv_rank=2)
    lay = parameter_layout(ds)
    assert [n for n, _, _ in lay[3:9]] == ["Wdq", "Wuq", "Wdkv", "Wuk", "Wuv", "Wo"]
    assert [s for _, _, s in lay[3:9]] == [(8, 4), (4, 8), (8, 2), (2, 8), (2, 8), (8, 8)]


def test_gpt_layout_follows_parameters_order():
    """GPTModel.embeddingParameters (token, position), GPTTransformerBlock.subLayers (ln1, ln2, attn, mlp) with
    LayerNorm1D's (gamma, beta) and FNN's (W, b) pairs, final norm, LM head."""
    cfg = DecoderConfig("gpt", 11, 16, 8, 2, 2, 24)
    lay = parameter_layout(cfg)
    names = [(n, l) for n, l, _ in lay]
    assert names[:2] == [("emb", -1), ("pos", -1)] and lay[1][2] == (16, 8)
    assert names[2:14] == [("g1", 0), ("b1", 0), ("g2", 0), ("b2", 0), ("Wq", 0), ("Wk", 0), ("Wv", 0), ("Wo", 0),
                           ("W1", 0), ("c1", 0), ("W2", 0), ("c2", 0)]
    assert names[-4:] == [("gF", -1), ("bF", -1), ("Wlm", -1), ("blm", -1)]
    assert len(names) == 2 + 2 * 12 + 4
    get = weight_getter(cfg, random_params(cfg, 3))
    assert get("c1", 1).shape == (24,) and get("W1", 1).shape == (8, 24) and get("pos", -1).shape == (16, 8)


def test_reads_the_java_stream_bit_for_bit(tmp_path):
    cfg = DecoderConfig("llama", 11, 16, 8, 2, 2, 24)
    params = random_params(cfg)
    path = tmp_path / "model.bin"
    path.write_bytes(java_bytes(params))
    back = read_parameters(path)
    assert len(back) == len(params)
    for a, b in zip(params, back):
        assert a.shape == b.shape and np.array_equal(a.view(np.uint32), b.view(np.uint32))
    # and the writer produces the same bytes
    out = tmp_path / "copy.bin"
    write_parameters(out, params)
    assert out.read_bytes() == path.read_bytes()
    get = weight_getter(cfg, path)
    assert get("Wq", 1).shape == (8, 8) and get("g1", 0).shape == (8,) and get("blm", -1).shape == (11,)
    assert np.array_equal(get("Wd", 1), params[1 + 12 + 10])


def test_rejects_what_the_reference_rejects(tmp_path):
    cfg = DecoderConfig("llama", 11, 16, 8, 2, 1, 24)
    params = random_params(cfg)
    with pytest.raises(IOError, match="Parameter count mismatch"):
        named_parameters(cfg, params[:-1])
    bad = list(params)
    bad[3] = np.zeros((8, 7), dtype=np.float32)
    with pytest.raises(IOError, match="Shape mismatch at parameter 3"):
        named_parameters(cfg, bad)
    blob = java_bytes(params)
    p = tmp_path / "cut.bin"
    p.write_bytes(blob[:-5])
    with pytest.raises(IOError):
        read_parameters(p)
    p.write_bytes(blob + b"\0")
    with pytest.raises(IOError, match="trailing"):
        read_parameters(p)
    p.write_bytes(b"")
    with pytest.raises(IOError):
        read_parameters(p)
