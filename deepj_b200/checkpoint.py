"""DeepJ checkpoints → the Q8 decoder.

`ModelSerializer` (persistence/ModelSerializer.java:44-98) writes a model as a big-endian
stream: `int count`, then per parameter `int rows, int cols` and `rows·cols` doubles (each
the widened fp32 value, row-major).  The parameters come in `model.parameters()` order
(models/DecoderOnlyModel.java:78-85): token embedding; per block `ln1.gamma, ln2.gamma`,
the attention matrices, `gate.W, gate.b, up.W, up.b, down.W, down.b`
(blocks/LlamaTransformerBlock.java:45-47, SwiGLULayer.java:91-97, Linear.java:54-56); the
final norm's gamma; `lmHead.W, lmHead.b`.  Attention matrices: `Wq, Wk, Wv, Wo`
(MultiHeadSelfAttention.java:256-258) or, for DeepSeek blocks, `Wdq, Wuq, Wdkv, Wuk, Wuv, Wo`
(MultiHeadLatentAttention.java:174-176).  A GPT model (`kind="gpt"`) adds the position table after the token
embedding, has `gamma, beta` per LayerNorm, and `W1, c1, W2, c2` for its MLP (models/gpt/GPTModel.java:63-67,
blocks/GPTTransformerBlock.java:61-63, norm/LayerNorm1D.java:80-82, layers/FNN.java:110-114).

`read_parameters` parses the file, `named_parameters` checks the shapes against a
`DecoderConfig` and names them the way `Q8Decoder.load_weights` asks for them, and
`weight_getter` is the callable to hand over:

    dec = Q8Decoder(cfg); dec.load_weights(weight_getter(cfg, "model.bin"))

`write_parameters` produces the same format (tests, and exporting weights back).
"""
from __future__ import annotations

import os
from typing import Callable, Dict, List, Tuple, Union

import numpy as np

from .decoder import DecoderConfig

PathLike = Union[str, "os.PathLike[str]"]


def read_parameters(path: PathLike) -> List[np.ndarray]:
    """All parameters of a checkpoint as fp32 [rows × cols] arrays, in file order."""
    with open(path, "rb") as f:
        blob = f.read()
    if len(blob) < 4:
        raise IOError("checkpoint is shorter than its parameter count")
    count = int(np.frombuffer(blob, dtype=">i4", count=1)[0])
    if count < 0:
        raise IOError(f"negative parameter count {count}")
    pos, out = 4, []
    for i in range(count):
        if pos + 8 > len(blob):
            raise IOError(f"checkpoint ends inside the header of parameter {i}")
        rows, cols = (int(v) for v in np.frombuffer(blob, dtype=">i4", count=2, offset=pos))
        pos += 8
        if rows < 0 or cols < 0:
            raise IOError(f"negative shape at parameter {i}")
        n = rows * cols
        if pos + 8 * n > len(blob):
            raise IOError(f"checkpoint ends inside the data of parameter {i}")
        out.append(np.frombuffer(blob, dtype=">f8", count=n, offset=pos).astype(np.float32).reshape(rows, cols))
        pos += 8 * n
    if pos != len(blob):
        raise IOError(f"{len(blob) - pos} trailing bytes after parameter {count - 1}")
    return out


def write_parameters(path: PathLike, params: List[np.ndarray]) -> None:
    """The inverse of `read_parameters` (ModelSerializer.save)."""
    with open(path, "wb") as f:
        f.write(np.asarray([len(params)], dtype=">i4").tobytes())
        for p in params:
            a = np.asarray(p, dtype=np.float32)
            if a.ndim != 2:
                raise ValueError("parameters are [rows × cols] tensors")
            f.write(np.asarray(a.shape, dtype=">i4").tobytes())
            f.write(a.astype(">f8").tobytes())


def parameter_layout(cfg: DecoderConfig) -> List[Tuple[str, int, Tuple[int, int]]]:
    """(name, layer, shape) of every parameter in `parameters()` order; layer −1 = not in a block."""
    d, F, V = cfg.d_model, cfg.d_ff, cfg.vocab_size
    out: List[Tuple[str, int, Tuple[int, int]]] = [("emb", -1, (V, d))]
    if cfg.kind == "gpt":
        # GPTModel.embeddingParameters (models/gpt/GPTModel.java:63-67), GPTTransformerBlock.subLayers
        # (ln1, ln2, attn, mlp), LayerNorm1D.parameters (gamma, beta), FNN.parameters (W, b per Linear)
        out.append(("pos", -1, (cfg.max_seq_len, d)))
        for l in range(cfg.n_layers):
            out += [("g1", l, (1, d)), ("b1", l, (1, d)), ("g2", l, (1, d)), ("b2", l, (1, d))]
            out += [(n, l, (d, d)) for n in ("Wq", "Wk", "Wv", "Wo")]
            out += [("W1", l, (d, F)), ("c1", l, (1, F)), ("W2", l, (F, d)), ("c2", l, (1, d))]
        return out + [("gF", -1, (1, d)), ("bF", -1, (1, d)), ("Wlm", -1, (d, V)), ("blm", -1, (1, V))]
    if cfg.kind == "llama":
        attn = [("Wq", (d, d)), ("Wk", (d, d)), ("Wv", (d, d)), ("Wo", (d, d))]
    else:
        attn = [("Wdq", (d, cfg.q_rank)), ("Wuq", (cfg.q_rank, d)), ("Wdkv", (d, cfg.kv_rank)), ("Wuk", (cfg.kv_rank, d)),
                ("Wuv", (cfg.kv_rank, d)), ("Wo", (d, d))]
    for l in range(cfg.n_layers):
        out += [("g1", l, (1, d)), ("g2", l, (1, d))]
        out += [(n, l, s) for n, s in attn]
        out += [("Wg", l, (d, F)), ("bg", l, (1, F)), ("Wu", l, (d, F)), ("bu", l, (1, F)), ("Wd", l, (F, d)), ("bd", l, (1, d))]
    out += [("gF", -1, (1, d)), ("Wlm", -1, (d, V)), ("blm", -1, (1, V))]
    return out


def named_parameters(cfg: DecoderConfig, params: List[np.ndarray]) -> Dict[Tuple[str, int], np.ndarray]:
    """Check count and shapes the way ModelSerializer.load does and key the tensors by (name, layer)."""
    layout = parameter_layout(cfg)
    if len(params) != len(layout):
        raise IOError("Parameter count mismatch")                       # ModelSerializer.java: readAndValidateParameterCount
    named = {}
    for i, ((name, layer, shape), p) in enumerate(zip(layout, params)):
        if tuple(p.shape) != shape:
            raise IOError(f"Shape mismatch at parameter {i}")           # readAndValidateShape
        named[(name, layer)] = p
    return named


def weight_getter(cfg: DecoderConfig, source: Union[PathLike, List[np.ndarray]]) -> Callable[[str, int], np.ndarray]:
    """`get(name, layer)` for `Q8Decoder.load_weights`, from a checkpoint file or its parameter list."""
    params = read_parameters(source) if isinstance(source, (str, os.PathLike)) else list(source)
    named = named_parameters(cfg, params)

    def get(name: str, layer: int) -> np.ndarray:
        a = named[(name, layer if (name, layer) in named else -1)]
        return a.reshape(-1) if a.shape[0] == 1 and name[0] in "gbc" else a
    return get
