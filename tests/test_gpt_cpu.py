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


GPT_NAMES = [("emb", -1), ("pos", -1), ("gF", -1), ("bF", -1), ("Wlm", -1), ("blm", -1)]
GPT_LAYER_NAMES = ["g1", "b1", "g2", "b2", "Wq", "Wk", "Wv", "Wo", "W1", "c1", "W2", "c2"]


def native_gpt(seed=11, init_mode=0, **shape):
    return oracle.OracleModel("gpt", shape["vocab"], shape["max_seq"], shape["d"], shape["heads"], shape["layers"], shape["d_ff"],
                              seed=seed, init_mode=init_mode, std=0.1)


def test_native_gpt_equals_the_layer_stack_bit_for_bit_and_the_numpy_restatement():
    """The C++ GPT forward pass, the Python layer stack over the oracle's op interpreter (two independent restatements of
    GPTModel.forward) and the numpy one: the first two agree bit for bit, the third to rounding."""
    om = native_gpt(**SHAPE)
    rng = np.random.default_rng(2)
    for l in range(SHAPE["layers"]):          # the constructors leave biases at zero and gains constant: make them count
        for n in ("g1", "b1", "g2", "b2", "c1", "c2"):
            a = om.weight(n, l)
            om.set_weight(n, l, a + 0.05 * rng.standard_normal(a.size).astype(np.float32))
    om.set_weight("bF", -1, 0.05 * rng.standard_normal(SHAPE["d"]).astype(np.float32))
    om.set_weight("blm", -1, 0.05 * rng.standard_normal(SHAPE["vocab"]).astype(np.float32))
    shapes = {"emb": (SHAPE["vocab"], SHAPE["d"]), "pos": (SHAPE["max_seq"], SHAPE["d"]), "Wlm": (SHAPE["d"], SHAPE["vocab"]),
              "Wq": (SHAPE["d"],) * 2, "Wk": (SHAPE["d"],) * 2, "Wv": (SHAPE["d"],) * 2, "Wo": (SHAPE["d"],) * 2,
              "W1": (SHAPE["d"], SHAPE["d_ff"]), "W2": (SHAPE["d_ff"], SHAPE["d"])}

    def get(name, layer):
        a = om.weight(name, layer)
        return a.reshape(shapes[name]) if name in shapes else a

    ids = [3, 96, 0, 41, 41, 7, 12, 88, 5, 60]
    native = om.forward(ids)
    b = on_oracle()
    stack = build_gpt_model(get=get, **SHAPE).forward(ids).numpy()
    b.releaseResources()
    assert np.array_equal(native.view(np.uint32), stack.view(np.uint32))
    w = {(n, l): get(n, l) for n, l in GPT_NAMES}
    w.update({(n, l): get(n, l) for l in range(SHAPE["layers"]) for n in GPT_LAYER_NAMES})
    want = gpt_ref.forward(w, ids, SHAPE["d"], SHAPE["heads"], SHAPE["layers"])
    assert float(np.abs(native - want).max()) <= 1e-4 * float(np.abs(want).max())
    # the KV-cached step reproduces the last row of the full forward bit for bit
    om.reset_cache()
    for t, tok in enumerate(ids):
        row = om.decode_step(tok)
        assert np.array_equal(row.view(np.uint32), native[t].view(np.uint32)), t


def test_native_gpt_draw_order_and_init_scale():
    """GPTModel's constructor (models/gpt/GPTModel.java:31-46,78-83): token table from Random(seed), the blocks from one
    fresh Random(seed) (Wq, Wk, Wv, Wo, then the MLP's two matrices), the LM head from Random(seed + 1), the position
    table from Random(seed + 2), and every parameter — gains included — times initScale 0.2."""
    seed = 11
    om = native_gpt(seed=seed, **SHAPE)
    d, F, V, S = SHAPE["d"], SHAPE["d_ff"], SHAPE["vocab"], SHAPE["max_seq"]

    def draws(r, n):
        return (np.asarray([np.float32(r.next_gaussian() * 0.1) for _ in range(n)], dtype=np.float32) * np.float32(0.2))

    assert np.array_equal(om.weight("emb"), draws(oracle.JRandom(seed), V * d))
    r = oracle.JRandom(seed)
    for l in range(SHAPE["layers"]):
        for name, n in (("Wq", d * d), ("Wk", d * d), ("Wv", d * d), ("Wo", d * d), ("W1", d * F), ("W2", F * d)):
            assert np.array_equal(om.weight(name, l), draws(r, n)), (name, l)
        assert np.all(om.weight("g1", l) == np.float32(0.2)) and np.all(om.weight("b1", l) == 0.0) and np.all(om.weight("c1", l) == 0.0)
    assert np.array_equal(om.weight("Wlm"), draws(oracle.JRandom(seed + 1), d * V))
    assert np.array_equal(om.weight("pos"), draws(oracle.JRandom(seed + 2), S * d))
    assert np.all(om.weight("gF") == np.float32(0.2))
