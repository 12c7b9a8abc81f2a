"""GPT family on the reference-style layer stack (deepj_b200.layers) over the oracle's op interpreter, against an
independent numpy restatement — LayerNorm, GELU MLP, learned positions, un-rotated causal attention."""
import numpy as np

import gpt_ref
import oracle
from deepj_b200.layers import LayerNorm1D, TextGenerator, build_gpt_model
from deepj_b200.tensor import GraphBackend, Tensor

SHAPE = dict(vocab=97, max_seq=16, d=32, heads=4, layers=2, d_ff=80)


def on_oracle():
    b = GraphBackend(oracle.OracleRuntime())
    Tensor.setBackend(b)
    return b


def test_layer_norm_rows_are_standardised():
    b = on_oracle()
    x = np.random.default_rng(0).standard_normal((5, 32)).astype(np.float32) * 3 + 1
    y = LayerNorm1D(32).forward(Tensor(5, 32, x)).numpy()
    assert np.allclose(y.mean(axis=1), 0.0, atol=1e-5)
    assert np.allclose(y.var(axis=1), 1.0, atol=1e-4)
    g = np.linspace(0.5, 1.5, 32).astype(np.float32)
    s = np.linspace(-1, 1, 32).astype(np.float32)
    z = LayerNorm1D(32, g, s).forward(Tensor(5, 32, x)).numpy()
    assert np.allclose(z, y * g + s, atol=1e-5)
    b.releaseResources()


def test_gpt_forward_matches_numpy_restatement_and_is_causal():
    b = on_oracle()
    w, get = gpt_ref.make_weights(seed=5, **SHAPE)
    model = build_gpt_model(get=get, **SHAPE)
    ids = [3, 96, 0, 41, 41, 7, 12, 88, 5]
    got = model.forward(ids).numpy()
    want = gpt_ref.forward(w, ids, SHAPE["d"], SHAPE["heads"], SHAPE["layers"])
    assert got.shape == (len(ids), SHAPE["vocab"])
    assert float(np.abs(got - want).max()) <= 1e-4 * float(np.abs(want).max())
    # a later token does not change earlier rows (DecoderOnlyModelTest's no-leak property)
    ids2 = list(ids)
    ids2[-1] = 50
    got2 = model.forward(ids2).numpy()
    assert float(np.abs(got2[:-1] - got[:-1]).max()) <= 1e-6
    assert float(np.abs(got2[-1] - got[-1]).max()) > 1e-3
    # greedy generation appends the argmax of the last row
    out = TextGenerator.generate(model.forward, SHAPE["max_seq"], ids, 3, 1.0, 1)
    assert out[:len(ids)] == ids and out[len(ids)] == int(np.argmax(got[-1]))
    b.releaseResources()
