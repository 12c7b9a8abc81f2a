"""An independent numpy restatement of the reference's GPT forward pass (models/gpt/GPTModel.java:52-54,
blocks/GPTTransformerBlock.java:66-74, norm/LayerNorm1D.java:33-71, MultiHeadSelfAttention.java:60-86,
tensor/cpu/CpuBackend.java gelu) for the tests: fp32 numpy, row-major, no framework objects."""
import numpy as np


def make_weights(vocab, max_seq, d, heads, layers, d_ff, seed):
    rng = np.random.default_rng(seed)
    w = {("emb", -1): rng.standard_normal((vocab, d)) * 0.1, ("pos", -1): rng.standard_normal((max_seq, d)) * 0.1,
         ("gF", -1): 1 + 0.1 * rng.standard_normal(d), ("bF", -1): 0.1 * rng.standard_normal(d),
         ("Wlm", -1): rng.standard_normal((d, vocab)) * 0.1, ("blm", -1): 0.1 * rng.standard_normal(vocab)}
    for l in range(layers):
        for n in ("g1", "g2"):
            w[(n, l)] = 1 + 0.1 * rng.standard_normal(d)
        for n in ("b1", "b2", "c2"):
            w[(n, l)] = 0.1 * rng.standard_normal(d)
        for n in ("Wq", "Wk", "Wv", "Wo"):
            w[(n, l)] = rng.standard_normal((d, d)) * 0.1
        w[("W1", l)] = rng.standard_normal((d, d_ff)) * 0.1
        w[("c1", l)] = 0.1 * rng.standard_normal(d_ff)
        w[("W2", l)] = rng.standard_normal((d_ff, d)) * 0.1
    w = {k: v.astype(np.float32) for k, v in w.items()}
    return w, (lambda name, layer: w[(name, layer)])


def layer_norm(x, g, b):
    mean = x.mean(axis=1, keepdims=True, dtype=np.float32)
    var = ((x - mean) ** 2).mean(axis=1, keepdims=True, dtype=np.float32)
    return ((x - mean) / np.sqrt(var + np.float32(1e-5))) * g + b


def gelu(x):
    x = x.astype(np.float64)
    return (0.5 * x * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (x + 0.044715 * x ** 3)))).astype(np.float32)


def forward(w, ids, d, heads, layers):
    L = len(ids)
    hd = d // heads
    x = w[("emb", -1)][ids] + w[("pos", -1)][:L]
    mask = np.triu(np.ones((L, L), dtype=bool), 1)
    for l in range(layers):
        h = layer_norm(x, w[("g1", l)], w[("b1", l)])
        q, k, v = h @ w[("Wq", l)], h @ w[("Wk", l)], h @ w[("Wv", l)]
        out = np.zeros_like(x)
        for a in range(heads):
            sl = slice(a * hd, (a + 1) * hd)
            s = (q[:, sl] @ k[:, sl].T) * np.float32(1.0 / np.sqrt(hd))
            s = np.where(mask, np.float32(-1e9), s)
            p = np.exp(s - s.max(axis=1, keepdims=True))
            p = p / p.sum(axis=1, keepdims=True)
            out[:, sl] = p @ v[:, sl]
        x = x + out @ w[("Wo", l)]
        h = layer_norm(x, w[("g2", l)], w[("b2", l)])
        x = x + (gelu(h @ w[("W1", l)] + w[("c1", l)]) @ w[("W2", l)] + w[("c2", l)])
    return layer_norm(x, w[("gF", -1)], w[("bF", -1)]) @ w[("Wlm", -1)] + w[("blm", -1)]
