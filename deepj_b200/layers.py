"""The reference's inference layers, written against the `Tensor` façade only.

These classes restate the forward passes of DeepJ's layer stack op for op, so that the
same code runs on any `TensorBackend` — in particular on `CudaBackend`, where it
demonstrates the drop-in path: the unmodified layer structure, including the
reference's materialise-and-copy head reshapes (which force a flush per head), over
libdeepj_cuda_jni.  It is correct but flush-bound; the fast path is
`deepj_b200.decoder.Q8Decoder`.  Weights are passed in as arrays (the reference draws
them from java.util.Random in its constructors).
"""
from __future__ import annotations

import math
from typing import Callable, List, Optional, Sequence

import numpy as np

from .decoder import rope_tables
from .tensor import Tensor


class Linear:
    """layers/Linear.java:31-36 — y = x·W + b, W [dIn × dOut], b [1 × dOut]."""

    def __init__(self, W: np.ndarray, b: Optional[np.ndarray] = None):
        self.dIn, self.dOut = W.shape
        self.W = Tensor(self.dIn, self.dOut, W)
        self.b = Tensor(1, self.dOut, b if b is not None else np.zeros(self.dOut, dtype=np.float32))

    def forward(self, x: Tensor) -> Tensor:
        if x.cols != self.dIn:
            raise ValueError(f"Expected input cols={self.dIn} got {x.cols}")
        return x.matmul(self.W).addRowVector(self.b)


class RMSNorm1D:
    """layers/transformer/norm/RMSNorm1D.java:46-57, eps 1e-6, gain only."""

    EPS = 1e-6

    def __init__(self, dim: int, gamma: Optional[np.ndarray] = None):
        if dim <= 0:
            raise ValueError("dim must be > 0")
        self.dim = dim
        self.gamma = Tensor(1, dim, gamma if gamma is not None else np.ones(dim, dtype=np.float32))

    def forward(self, x: Tensor) -> Tensor:
        if x.cols != self.dim:
            raise ValueError(f"Expected cols={self.dim} got {x.cols}")
        mean_sq = x.multiply(x).meanAlongRows()
        rms = mean_sq.addScalar(self.EPS).sqrt()
        return x.divideBroadcastCols(rms).multiplyBroadcastRows(self.gamma)


class LayerNorm1D:
    """layers/transformer/norm/LayerNorm1D.java:33-71 — per-row mean and (population) variance,
    (x − mean) / sqrt(var + 1e-5) · γ + β."""

    EPS = 1e-5

    def __init__(self, dim: int, gamma: Optional[np.ndarray] = None, beta: Optional[np.ndarray] = None):
        if dim <= 0:
            raise ValueError("dim must be > 0")
        self.dim = dim
        self.gamma = Tensor(1, dim, gamma if gamma is not None else np.ones(dim, dtype=np.float32))
        self.beta = Tensor(1, dim, beta if beta is not None else np.zeros(dim, dtype=np.float32))

    def forward(self, x: Tensor) -> Tensor:
        if x.cols != self.dim:
            raise ValueError(f"Expected cols={self.dim} got {x.cols}")
        mean = x.meanAlongRows()
        std = x.varianceAlongRows().addScalar(self.EPS).sqrt()
        xhat = x.subtractBroadcastCols(mean).divideBroadcastCols(std)
        return xhat.multiplyBroadcastRows(self.gamma).addBroadcastRows(self.beta)


class FNN:
    """layers/FNN.java:62-80 with one hidden layer and GELU, the GPT block's MLP
    (blocks/GPTTransformerBlock.java:54): Linear → GELU → Linear."""

    def __init__(self, hidden: Linear, out: Linear):
        self.hidden, self.out = hidden, out

    def forward(self, x: Tensor) -> Tensor:
        return self.out.forward(self.hidden.forward(x).geluActivation())


class RotaryEmbedding:
    """transformer/embeddings/RotaryEmbedding.java:52-122 — interleaved pairs, applied
    on the host after a materialise, as the reference does."""

    def __init__(self, headDim: int, maxSeqLen: int):
        self.cos, self.sin = rope_tables(headDim, maxSeqLen)
        self.halfDim = headDim // 2
        self.maxSeqLen = maxSeqLen

    def apply(self, t: Tensor, seqLen: int, nHeads: int) -> Tensor:
        if seqLen > self.maxSeqLen:
            raise ValueError(f"seqLen {seqLen} exceeds maxSeqLen {self.maxSeqLen}")
        src = t.numpy().reshape(nHeads, seqLen, -1)
        c, s = self.cos[:seqLen][None], self.sin[:seqLen][None]
        x0, x1 = src[:, :, 0::2], src[:, :, 1::2]
        out = np.empty_like(src)
        out[:, :, 0::2] = x0 * c - x1 * s
        out[:, :, 1::2] = x0 * s + x1 * c
        return Tensor(t.rows, t.cols, out)


class HeadOps:
    """layers/transformer/attention/HeadOps.java:33-140."""

    @staticmethod
    def splitHeads(t: Tensor, seqLen, nHeads, headDim, dModel) -> Tensor:
        src = t.numpy().reshape(seqLen, nHeads, headDim)
        return Tensor(nHeads * seqLen, headDim, src.transpose(1, 0, 2).copy())

    @staticmethod
    def mergeHeads(t: Tensor, seqLen, nHeads, headDim, dModel) -> Tensor:
        src = t.numpy().reshape(nHeads, seqLen, headDim)
        return Tensor(seqLen, dModel, src.transpose(1, 0, 2).copy())

    @staticmethod
    def extractBlock(t: Tensor, rowStart, numRows, numCols) -> Tensor:
        return Tensor(numRows, numCols, t.numpy()[rowStart:rowStart + numRows].copy())

    @staticmethod
    def insertBlock(target: Tensor, block: Tensor, rowStart, numRows, numCols) -> None:
        target.data[rowStart:rowStart + numRows] = block.numpy()

    @staticmethod
    def scaledDotProductScores(qh, kh, nHeads, seqLen, headDim, scale) -> Tensor:
        out = Tensor(nHeads * seqLen, seqLen)
        for h in range(nHeads):
            q = HeadOps.extractBlock(qh, h * seqLen, seqLen, headDim)
            k = HeadOps.extractBlock(kh, h * seqLen, seqLen, headDim)
            s = q.matmul(k.transpose())
            s.multiplyScalarInPlace(scale)
            HeadOps.insertBlock(out, s, h * seqLen, seqLen, seqLen)
        return out

    @staticmethod
    def applyCausalMask(scores, nHeads, seqLen) -> Tensor:
        mask = Tensor.causalMask(seqLen)
        out = Tensor(nHeads * seqLen, seqLen)
        for h in range(nHeads):
            block = HeadOps.extractBlock(scores, h * seqLen, seqLen, seqLen)
            HeadOps.insertBlock(out, block.add(mask), h * seqLen, seqLen, seqLen)
        return out

    @staticmethod
    def applyAttentionToValues(attnProb, vh, nHeads, seqLen, headDim) -> Tensor:
        out = Tensor(nHeads * seqLen, headDim)
        for h in range(nHeads):
            a = HeadOps.extractBlock(attnProb, h * seqLen, seqLen, seqLen)
            v = HeadOps.extractBlock(vh, h * seqLen, seqLen, headDim)
            HeadOps.insertBlock(out, a.matmul(v), h * seqLen, seqLen, headDim)
        return out


class MultiHeadSelfAttention:
    """layers/transformer/attention/MultiHeadSelfAttention.java:60-86; bias-free projections."""

    def __init__(self, dModel, nHeads, causalMask, Wq, Wk, Wv, Wo):
        if dModel % nHeads != 0:
            raise ValueError("dModel must be divisible by nHeads")
        self.dModel, self.nHeads, self.headDim, self.causalMask = dModel, nHeads, dModel // nHeads, causalMask
        self.scale = float(np.float32(1.0 / math.sqrt(self.headDim)))
        self.Wq, self.Wk, self.Wv, self.Wo = (Tensor(w.shape[0], w.shape[1], w) for w in (Wq, Wk, Wv, Wo))

    def transformQueryKey(self, heads: Tensor, seqLen: int) -> Tensor:
        return heads

    def project(self, x: Tensor):
        return x.matmul(self.Wq), x.matmul(self.Wk), x.matmul(self.Wv)

    def forward(self, x: Tensor) -> Tensor:
        if x.cols != self.dModel:
            raise ValueError(f"Expected cols={self.dModel} got {x.cols}")
        n, H, hd, d = x.rows, self.nHeads, self.headDim, self.dModel
        Q, K, V = self.project(x)
        qh = self.transformQueryKey(HeadOps.splitHeads(Q, n, H, hd, d), n)
        kh = self.transformQueryKey(HeadOps.splitHeads(K, n, H, hd, d), n)
        vh = HeadOps.splitHeads(V, n, H, hd, d)
        scores = HeadOps.scaledDotProductScores(qh, kh, H, n, hd, self.scale)
        if self.causalMask:
            scores = HeadOps.applyCausalMask(scores, H, n)
        prob = scores.softmaxRows()
        merged = HeadOps.mergeHeads(HeadOps.applyAttentionToValues(prob, vh, H, n, hd), n, H, hd, d)
        return merged.matmul(self.Wo)


class RoPEMultiHeadSelfAttention(MultiHeadSelfAttention):
    """layers/transformer/attention/RoPEMultiHeadSelfAttention.java:56-58."""

    def __init__(self, dModel, nHeads, causalMask, rope: RotaryEmbedding, Wq, Wk, Wv, Wo):
        super().__init__(dModel, nHeads, causalMask, Wq, Wk, Wv, Wo)
        self.rope = rope

    def transformQueryKey(self, heads, seqLen):
        return self.rope.apply(heads, seqLen, self.nHeads)


class MultiHeadLatentAttention(RoPEMultiHeadSelfAttention):
    """layers/transformer/attention/MultiHeadLatentAttention.java:93-124: low-rank Q and a
    shared KV latent, RoPE on the whole head of the expanded K, then the MHSA tail."""

    def __init__(self, dModel, nHeads, rope, Wdq, Wuq, Wdkv, Wuk, Wuv, Wo):
        z = np.zeros((dModel, dModel), dtype=np.float32)
        super().__init__(dModel, nHeads, True, rope, z, z, z, Wo)
        self.Wdq, self.Wuq, self.Wdkv, self.Wuk, self.Wuv = (Tensor(w.shape[0], w.shape[1], w) for w in (Wdq, Wuq, Wdkv, Wuk, Wuv))

    def project(self, x):
        cQ = x.matmul(self.Wdq)
        cKV = x.matmul(self.Wdkv)
        return cQ.matmul(self.Wuq), cKV.matmul(self.Wuk), cKV.matmul(self.Wuv)


class SwiGLULayer:
    """layers/transformer/SwiGLULayer.java:63-70 with SiLU = x·σ(x) (activations/SiLU.java:20-24)."""

    def __init__(self, gate: Linear, up: Linear, down: Linear):
        self.gateProj, self.upProj, self.downProj = gate, up, down

    def forward(self, x: Tensor) -> Tensor:
        gate = self.gateProj.forward(x)
        up = self.upProj.forward(x)
        silu = gate.multiply(gate.sigmoidActivation())
        return self.downProj.forward(silu.multiply(up))


class TransformerBlock:
    """Pre-norm residual block (LlamaTransformerBlock.java:50-53, DeepSeekTransformerBlock.java:54-57)."""

    def __init__(self, ln1: RMSNorm1D, ln2: RMSNorm1D, attn, mlp: SwiGLULayer):
        self.ln1, self.ln2, self.attn, self.mlp = ln1, ln2, attn, mlp

    def forward(self, x: Tensor) -> Tensor:
        x2 = x.add(self.attn.forward(self.ln1.forward(x)))
        return x2.add(self.mlp.forward(self.ln2.forward(x2)))


class DecoderOnlyModel:
    """models/DecoderOnlyModel.java:58-64: embed → blocks → final norm → LM head."""

    def __init__(self, emb: np.ndarray, blocks: List[TransformerBlock], normF: RMSNorm1D, lmHead: Linear, maxSeqLen: int):
        self.vocabSize, self.dModel = emb.shape
        self.tokEmb = Tensor(emb.shape[0], emb.shape[1], emb)
        self.blocks, self.normF, self.lmHead, self.maxSeqLen = blocks, normF, lmHead, maxSeqLen

    def forward(self, inputIds: Sequence[int]) -> Tensor:
        for i in inputIds:
            if i < 0 or i >= self.vocabSize:
                raise ValueError(f"Token id out of range: {i}")       # Embedding.java:30-32
        x = Tensor.sliceRows(self.tokEmb, inputIds, self.dModel)
        for b in self.blocks:
            x = b.forward(x)
        return self.lmHead.forward(self.normF.forward(x))


class GPTModel(DecoderOnlyModel):
    """models/gpt/GPTModel.java:26-54: learned positional embedding added to the token embedding,
    LayerNorm blocks with a GELU MLP, plain (un-rotated) causal attention, final LayerNorm."""

    def __init__(self, emb, pos: np.ndarray, blocks, normF: LayerNorm1D, lmHead: Linear, maxSeqLen: int):
        super().__init__(emb, blocks, normF, lmHead, maxSeqLen)
        self.posEmb = Tensor(pos.shape[0], pos.shape[1], pos)

    def forward(self, inputIds: Sequence[int]) -> Tensor:
        for i in inputIds:
            if i < 0 or i >= self.vocabSize:
                raise ValueError(f"Token id out of range: {i}")       # Embedding.java:30-32
        if len(inputIds) > self.maxSeqLen:
            raise ValueError(f"seqLen {len(inputIds)} exceeds maxSeq {self.maxSeqLen}")      # PositionalEmbedding.java:27
        x = Tensor.sliceRows(self.tokEmb, inputIds, self.dModel).add(
            Tensor.sliceRows(self.posEmb, list(range(len(inputIds))), self.dModel))
        for b in self.blocks:
            x = b.forward(x)
        return self.lmHead.forward(self.normF.forward(x))


def build_gpt_model(vocab: int, max_seq: int, d: int, heads: int, layers: int, d_ff: int,
                    get: Callable[[str, int], np.ndarray]) -> GPTModel:
    """A GPT model from a weight getter: "emb" [V×d], "pos" [maxSeq×d]; per layer "g1","b1","g2","b2" (LayerNorm
    gain / shift), "Wq","Wk","Wv","Wo" [d×d], "W1" [d×dFF], "c1", "W2" [dFF×d], "c2"; "gF","bF","Wlm" [d×V], "blm"."""
    def arr(name, layer, shape=None):
        a = np.asarray(get(name, layer), dtype=np.float32)
        return a.reshape(shape) if shape else a.reshape(-1)

    blocks = []
    for l in range(layers):
        attn = MultiHeadSelfAttention(d, heads, True, arr("Wq", l, (d, d)), arr("Wk", l, (d, d)), arr("Wv", l, (d, d)), arr("Wo", l, (d, d)))
        mlp = FNN(Linear(arr("W1", l, (d, d_ff)), arr("c1", l)), Linear(arr("W2", l, (d_ff, d)), arr("c2", l)))
        blocks.append(TransformerBlock(LayerNorm1D(d, arr("g1", l), arr("b1", l)), LayerNorm1D(d, arr("g2", l), arr("b2", l)), attn, mlp))
    return GPTModel(arr("emb", -1, (vocab, d)), arr("pos", -1, (max_seq, d)), blocks, LayerNorm1D(d, arr("gF", -1), arr("bF", -1)),
                    Linear(arr("Wlm", -1, (d, vocab)), arr("blm", -1)), max_seq)


def build_model(cfg, get: Callable[[str, int], np.ndarray]) -> DecoderOnlyModel:
    """Assemble a Llama / DeepSeek model from a `DecoderConfig` and a weight getter with the
    names `Q8Decoder.load_weights` uses."""
    shapes = {n: (k, w) for n, k, w in cfg.matmul_shapes()}
    d = cfg.d_model

    def mat(name, layer):
        return np.asarray(get(name, layer), dtype=np.float32).reshape(shapes[name])

    blocks = []
    for l in range(cfg.n_layers):
        rope = RotaryEmbedding(cfg.head_dim, cfg.max_seq_len)
        if cfg.kind == "llama":
            attn = RoPEMultiHeadSelfAttention(d, cfg.n_heads, True, rope, mat("Wq", l), mat("Wk", l), mat("Wv", l), mat("Wo", l))
        else:
            attn = MultiHeadLatentAttention(d, cfg.n_heads, rope, mat("Wdq", l), mat("Wuq", l), mat("Wdkv", l),
                                            mat("Wuk", l), mat("Wuv", l), mat("Wo", l))
        mlp = SwiGLULayer(Linear(mat("Wg", l), get("bg", l)), Linear(mat("Wu", l), get("bu", l)), Linear(mat("Wd", l), get("bd", l)))
        blocks.append(TransformerBlock(RMSNorm1D(d, get("g1", l)), RMSNorm1D(d, get("g2", l)), attn, mlp))
    emb = np.asarray(get("emb", -1), dtype=np.float32).reshape(cfg.vocab_size, d)
    head = Linear(np.asarray(get("Wlm", -1), dtype=np.float32).reshape(d, cfg.vocab_size), get("blm", -1))
    return DecoderOnlyModel(emb, blocks, RMSNorm1D(d, get("gF", -1)), head, cfg.max_seq_len)


class TextGenerator:
    """models/TextGenerator.java:66-181 for token ids.  topK = 1 is the greedy pick; the
    stable descending sort keeps the lowest index among equal logits."""

    @staticmethod
    def argsortDescending(a: np.ndarray) -> np.ndarray:
        # Float.compare order: -0.0 < +0.0, NaN above everything; stable
        bits = np.where(np.isnan(a), np.int32(0x7fc00000), a.view(np.int32)).astype(np.int64)
        key = np.where(bits < 0, bits ^ 0x7fffffff, bits)
        return np.argsort(-key, kind="stable")

    @staticmethod
    def nextToken(forward: Callable[[Sequence[int]], Tensor], maxSeqLen: int, ids: List[int], temperature: float, topK: int,
                  nextFloat: Callable[[], float]) -> int:
        context = ids if len(ids) <= maxSeqLen else ids[-maxSeqLen:]
        logits = forward(context).numpy()[-1].copy()
        order = TextGenerator.argsortDescending(logits)
        k = len(logits) if topK == 0 else min(topK, len(logits))
        top = order[:k]
        scaled = (logits[top] / np.float32(temperature)).astype(np.float32)
        mx = scaled.max()
        probs = np.array([np.float32(math.exp(float(np.float32(v - mx)))) for v in scaled], dtype=np.float32)
        total = np.float32(0.0)
        for p in probs:
            total = np.float32(total + p)
        probs = (probs / total).astype(np.float32)
        r = np.float32(nextFloat())
        cum = np.float32(0.0)
        for i, p in enumerate(probs):
            cum = np.float32(cum + p)
            if r <= cum:
                return int(top[i])
        return int(top[-1])

    @staticmethod
    def generate(forward, maxSeqLen: int, promptIds: Sequence[int], maxNewTokens: int, temperature: float, topK: int,
                 nextFloat: Callable[[], float] = lambda: 0.0) -> List[int]:
        if maxNewTokens < 0:
            raise ValueError("maxNewTokens must be >= 0")
        if temperature <= 0.0:
            raise ValueError("temperature must be > 0")
        if topK < 0:
            raise ValueError("topK must be >= 0")
        ids = list(promptIds)
        for _ in range(maxNewTokens):
            ids.append(TextGenerator.nextToken(forward, maxSeqLen, ids, temperature, topK, nextFloat))
        return ids
