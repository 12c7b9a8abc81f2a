"""Q8 decoder runner: DeepJ's LlamaModel / DeepSeekModel / GPTModel forward for ONE new token per
sequence, recorded as a ComputeGraph command stream of fused decode ops and replayed
through `deepj_cuda_flush_ops` (one flush per token; the library turns the repeated
stream into a CUDA graph).

What the stream computes, per token, is the last row of the reference's
`DecoderOnlyModel.forward` (models/DecoderOnlyModel.java:58-64): embedding row →
per block `x2 = x + attn(rmsnorm(x)); x = x2 + swiglu(rmsnorm(x2))`
(layers/transformer/blocks/LlamaTransformerBlock.java:50-53,
DeepSeekTransformerBlock.java:54-57) → final RMSNorm → LM head, then the greedy pick
of models/TextGenerator.java (topK = 1).  K and V of earlier positions come from a
cache in HBM instead of being recomputed.

`kind="gpt"` records the GPT family instead (models/gpt/GPTModel.java:52-54,
blocks/GPTTransformerBlock.java:66-74): token + learned position embedding, per block
`x2 = x + attn(layernorm(x)); x = x2 + W2·gelu(W1·layernorm(x2) + c1) + c2` with plain
(un-rotated) causal attention, a final LayerNorm and the LM head.  LayerNorm and GELU are
fused into the Q8 projections (op 75); the attention op runs with an identity rotation table.
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass
from typing import Tuple, Callable, Dict, List, Optional

import numpy as np

from . import _lib
from .compute_graph import (OP_ADD, OP_DECODE_STEP, OP_Q8_LINEAR_LN, OP_ADD_SCALAR_INPLACE, OP_ARGMAX_ROWS, OP_ATTN_DECODE, OP_ATTN_PREFILL, OP_COPY, OP_EMBED_GATHER, OP_SAMPLE_TOPK,
                            OP_Q8_LINEAR, OP_Q8_SWIGLU, OP_TP_ALLGATHER, OP_TP_ALLREDUCE, float_bits)

RMS_EPS = 1e-6      # layers/transformer/norm/RMSNorm1D.java:30
LN_EPS = 1e-5       # layers/transformer/norm/LayerNorm1D.java (EPS)


@dataclass(frozen=True)
class DecoderConfig:
    """Field-for-field the reference's LlamaConfig / DeepSeekConfig records
    (models/llama/LlamaConfig.java:10-22, models/deepseek/DeepSeekConfig.java)."""
    kind: str            # "llama" | "deepseek" | "gpt"
    vocab_size: int
    max_seq_len: int
    d_model: int
    n_heads: int
    n_layers: int
    d_ff: int
    q_rank: int = 0
    kv_rank: int = 0

    def __post_init__(self):
        # models/TransformerConfig.java:19-31
        if self.kind not in ("llama", "deepseek", "gpt"):
            raise ValueError("kind must be 'llama', 'deepseek' or 'gpt'")
        for name in ("vocab_size", "max_seq_len", "d_model", "n_heads", "n_layers", "d_ff"):
            if getattr(self, name) <= 0:
                raise ValueError(f"{name} must be > 0")
        if self.d_model % self.n_heads != 0:
            raise ValueError("dModel must be divisible by nHeads")
        if (self.d_model // self.n_heads) % 2 != 0:
            raise ValueError("headDim must be a positive even number")
        if self.kind == "deepseek" and (self.q_rank <= 0 or self.kv_rank <= 0):
            raise ValueError("qRank and kvRank must be > 0")

    @property
    def head_dim(self) -> int:
        return self.d_model // self.n_heads

    def matmul_shapes(self) -> List[tuple]:
        """(name, K, N) of the matmul weights of one block, in the reference's
        construction order (MultiHeadSelfAttention.java:47-50,
        MultiHeadLatentAttention.java:82-87, SwiGLULayer.java:56-58)."""
        d, f = self.d_model, self.d_ff
        if self.kind in ("llama", "gpt"):
            attn = [("Wq", d, d), ("Wk", d, d), ("Wv", d, d), ("Wo", d, d)]
        else:
            attn = [("Wdq", d, self.q_rank), ("Wuq", self.q_rank, d), ("Wdkv", d, self.kv_rank),
                    ("Wuk", self.kv_rank, d), ("Wuv", self.kv_rank, d), ("Wo", d, d)]
        if self.kind == "gpt":
            return attn + [("W1", d, f), ("W2", f, d)]          # layers/FNN.java: one hidden layer
        return attn + [("Wg", d, f), ("Wu", d, f), ("Wd", f, d)]

    def q8_weight_bytes(self) -> int:
        """Q8 bytes of every matmul weight streamed for one token (codes + scales)."""
        def q8(k, n):
            return k * n + ((k + 31) // 32) * n * 4
        per_layer = sum(q8(k, n) for _, k, n in self.matmul_shapes())
        return per_layer * self.n_layers + q8(self.d_model, self.vocab_size)

    def kv_bytes_per_position(self, kv_dtype: str = "f32") -> int:
        """K and V rows of one cached position, all layers (fp32, or fp16 with kv_dtype "f16")."""
        return 2 * self.n_layers * self.d_model * (2 if kv_dtype == "f16" else 4)


def rope_tables(head_dim: int, max_seq: int):
    """cos/sin tables with the reference's exact expression order
    (transformer/embeddings/RotaryEmbedding.java:52-71): float exponent, double pow,
    float theta, double cos/sin rounded to float."""
    if head_dim <= 0 or head_dim % 2 != 0:
        raise ValueError(f"headDim must be a positive even number, got {head_dim}")
    if max_seq <= 0:
        raise ValueError("maxSeqLen must be > 0")
    half = head_dim // 2
    f32 = np.float32
    inv = [math.pow(float(f32(10000.0)), float(f32(f32(2.0) * f32(i)) / f32(head_dim))) for i in range(half)]
    cos = np.empty((max_seq, half), dtype=np.float32)
    sin = np.empty((max_seq, half), dtype=np.float32)
    for pos in range(max_seq):
        for i in range(half):
            theta = float(f32(pos / inv[i]))
            cos[pos, i] = math.cos(theta)
            sin[pos, i] = math.sin(theta)
    return cos, sin


def shard_plan(cfg: DecoderConfig, rank: int, world: int) -> List[tuple]:
    """(device object, K_local, [(reference name, first row, first column, columns)]) of one block for
    one tensor-parallel rank.  Megatron-style split: Wq/Wk/Wv (or MLA's up-projections), gate and up
    by output columns (whole heads per rank); Wo and down by reduction rows — every split lands on a
    32-element Q8 block boundary.  MLA's low-rank down-projections are replicated."""
    c, r = cfg, rank
    d, dl, Fl = c.d_model, c.d_model // world, c.d_ff // world
    if c.kind == "gpt":
        if world != 1:
            raise ValueError("the GPT stream runs on one GPU")
        return [("Wqkv", d, [("Wq", 0, 0, d), ("Wk", 0, 0, d), ("Wv", 0, 0, d)]), ("Wo", d, [("Wo", 0, 0, d)]),
                ("W1", d, [("W1", 0, 0, c.d_ff)]), ("W2", c.d_ff, [("W2", 0, 0, d)])]
    if c.kind == "llama":
        plan = [("Wqkv", d, [("Wq", 0, r * dl, dl), ("Wk", 0, r * dl, dl), ("Wv", 0, r * dl, dl)])]
    else:
        plan = [("Wdqkv", d, [("Wdq", 0, 0, c.q_rank), ("Wdkv", 0, 0, c.kv_rank)]),
                ("Wuq", c.q_rank, [("Wuq", 0, r * dl, dl)]),
                ("Wukv", c.kv_rank, [("Wuk", 0, r * dl, dl), ("Wuv", 0, r * dl, dl)])]
    return plan + [("Wo", dl, [("Wo", r * dl, 0, d)]), ("Wg", d, [("Wg", 0, r * Fl, Fl)]),
                   ("Wu", d, [("Wu", 0, r * Fl, Fl)]), ("Wd", Fl, [("Wd", r * Fl, 0, d)])]


class Q8Decoder:
    """Owns the device-side weights, KV cache and the per-token command stream.

    Buffer ids are taken from `id_base` upwards so they never collide with the ids a
    `ComputeGraph` hands out (those start at 0).
    """

    def __init__(self, cfg: DecoderConfig, batch: int = 1, device: int = 0, id_base: int = 1 << 24,
                 tp_rank: int = 0, tp_world: int = 1, tp_slot_floats: int = 0, share_weights: Optional["Q8Decoder"] = None,
                 fused_step: Optional[bool] = None, kv_dtype: str = "f32"):
        """`tp_slot_floats`: the slot size the exchange buffer was (or will be) connected with (`tp.connect`); it
        bounds the rows a tensor-parallel prompt chunk may have (rows × dModel floats per exchange).
        `share_weights`: another decoder of the same configuration and sharding whose device weights this one reads
        (its own activations and KV cache, a different `id_base`); the other decoder must outlive this one.
        `fused_step`: run a token step as ONE persistent kernel (op 76) instead of one kernel per operator; the model must
        qualify (a Llama-shaped model, one sequence, every reduction length a multiple of 32, head dim 32 / 64 / 128).
        Under tensor parallelism the plan is made at the first step, after `tp.connect`.
        `kv_dtype`: "f32" (the reference's precision) or "f16" — keys rounded after the rotation, values rounded, fp32
        arithmetic; half the bytes a step's attention reads."""
        self.cfg = cfg
        self.B = int(batch)
        if kv_dtype not in ("f32", "f16"):
            raise ValueError("kv_dtype must be 'f32' or 'f16'")
        if kv_dtype == "f16" and (fused_step or cfg.head_dim % 16 != 0):
            raise ValueError("an fp16 KV cache needs a head dim that is a multiple of 16 and the per-operator step")
        self.kv_dtype = kv_dtype
        self.tp_slot_floats = int(tp_slot_floats)
        if tp_world < 1 or not (0 <= tp_rank < tp_world):
            raise ValueError("bad tensor-parallel rank / world size")
        if tp_world > 1 and cfg.kind == "gpt":
            raise ValueError("the GPT stream runs on one GPU")
        if tp_world > 1 and (cfg.n_heads % tp_world or cfg.d_ff % tp_world or cfg.vocab_size % tp_world or
                             (cfg.d_ff // tp_world) % 32 or (cfg.d_model // tp_world) % 32):
            raise ValueError("heads, dFF and vocab must divide by the tensor-parallel size, on 32-element block boundaries")
        self.tp_rank, self.tp_world = int(tp_rank), int(tp_world)
        self.h_local = cfg.n_heads // tp_world
        self.d_local = cfg.d_model // tp_world
        self.f_local = cfg.d_ff // tp_world
        self.v_local = cfg.vocab_size // tp_world
        self._ref_shapes = {n: (k, w) for n, k, w in cfg.matmul_shapes()}
        self._ref_shapes["Wlm"] = (cfg.d_model, cfg.vocab_size)
        self.lib = _lib.load()
        _lib.check(self.lib.deepj_cuda_init(device))
        self._next_id = id_base
        self._owned: List[int] = []
        self.ids: Dict[str, int] = {}
        self.loaded = False
        self._stream_host: Optional[np.ndarray] = None
        self._stream_dev: Optional[np.ndarray] = None
        self._op_labels: List[str] = []
        self._pin_ptr = None
        self._prefill_ids: Dict[str, int] = {}
        self._prefill_cap = 0
        self._prefill_streams: Dict[int, np.ndarray] = {}
        self.position = 0
        self._plan_id: Optional[int] = None
        if fused_step and not self.fused_step_eligible(cfg, self.B, tp_world):
            raise ValueError("this configuration does not qualify for the single-kernel token step")
        self.fused_step = bool(fused_step)          # opt-in: measured slower than the per-operator stream on one GPU so far
        self._alloc_state()
        if share_weights is not None:
            o = share_weights
            if o.cfg != cfg or (o.tp_rank, o.tp_world) != (self.tp_rank, self.tp_world) or not o.loaded:
                raise ValueError("share_weights needs a loaded decoder of the same configuration and sharding")
            for name, buf_id in o.ids.items():
                if name not in self.ids:          # everything that is not per-decoder state: the weights
                    self.ids[name] = buf_id
            self.loaded = True

    @staticmethod
    def fused_step_eligible(cfg: DecoderConfig, batch: int, tp_world: int = 1) -> bool:
        """Whether op 76 covers this model: see `deepj_cuda_decode_plan` in include/deepj_cuda.h."""
        if cfg.kind != "llama" or batch != 1 or cfg.head_dim not in (32, 64, 128):
            return False
        ks = (cfg.d_model, cfg.d_model // tp_world, cfg.d_ff // tp_world)
        return all(k % 32 == 0 for k in ks) and max(ks) <= 16384

    # ── id / buffer helpers ──
    def _new_id(self) -> int:
        i = self._next_id
        self._next_id += 1
        self._owned.append(i)
        return i

    def _f32(self, name: str, n: int, data: Optional[np.ndarray] = None) -> int:
        i = self._new_id()
        ids = (ctypes.c_int32 * 1)(i)
        sizes = (ctypes.c_int32 * 1)(n)
        _lib.check(self.lib.deepj_cuda_alloc_buffers(ids, sizes, 1))
        if data is not None:
            self._upload(i, data)
        if name:
            self.ids[name] = i
        return i

    def _upload(self, buf_id: int, data: np.ndarray) -> None:
        data = np.ascontiguousarray(data, dtype=np.float32)
        _lib.check(self.lib.deepj_cuda_upload_buffer(buf_id, data.ctypes.data, data.size))

    def _download(self, buf_id: int, n: int) -> np.ndarray:
        out = np.empty(n, dtype=np.float32)
        _lib.check(self.lib.deepj_cuda_download_buffer(buf_id, out.ctypes.data, n))
        return out

    def _release(self, ids: List[int]) -> None:
        arr = (ctypes.c_int32 * len(ids))(*ids)
        _lib.check(self.lib.deepj_cuda_release_buffers(arr, len(ids)))
        for i in ids:
            if i in self._owned:
                self._owned.remove(i)

    def _alloc_state(self) -> None:
        c, B = self.cfg, self.B
        d = c.d_model
        if c.kind == "gpt":
            # no rotary embedding: cos 1 / sin 0 make the attention op's rotation the identity
            half = c.head_dim // 2
            cos, sin = np.ones((c.max_seq_len, half), dtype=np.float32), np.zeros((c.max_seq_len, half), dtype=np.float32)
            self._f32("xp", B * d)       # the positional-embedding rows of the current tokens
        else:
            cos, sin = rope_tables(c.head_dim, c.max_seq_len)
        self._f32("cos", cos.size, cos)
        self._f32("sin", sin.size, sin)
        self._f32("tok", B)              # current token ids (floats holding ints)
        self._f32("pos", B)              # write position of every sequence
        self._f32("x", B * d)
        self._f32("x2", B * d)
        self._f32("qkv", B * 3 * self.d_local)
        self._f32("att", B * self.d_local)
        self._f32("h", B * self.f_local)
        self._f32("logits", B * c.vocab_size)
        if self.tp_world > 1:
            self._f32("part", B * d)
            self._f32("logits_local", B * self.v_local)
        self._f32("next", B)
        self._f32("r", B)                # one Random.nextFloat() per sequence for the device sampler
        if c.kind == "deepseek":
            self._f32("lat", B * (c.q_rank + c.kv_rank))
        kv = self._new_id()
        alloc = self.lib.deepj_cuda_kv_alloc_f16 if self.kv_dtype == "f16" else self.lib.deepj_cuda_kv_alloc
        _lib.check(alloc(kv, c.n_layers, B, self.h_local, c.max_seq_len, c.head_dim))
        self.ids["kv"] = kv

    # ── weights ──
    def _layer_plan(self) -> List[tuple]:
        """(device object name, K, [reference weight names concatenated along N]) of the
        unsharded model."""
        c = self.cfg
        d = c.d_model
        if c.kind == "gpt":
            return [("Wqkv", d, ["Wq", "Wk", "Wv"]), ("Wo", d, ["Wo"]), ("W1", d, ["W1"]), ("W2", c.d_ff, ["W2"])]
        if c.kind == "llama":
            plan = [("Wqkv", d, ["Wq", "Wk", "Wv"]), ("Wo", d, ["Wo"])]
        else:
            plan = [("Wdqkv", d, ["Wdq", "Wdkv"]), ("Wuq", c.q_rank, ["Wuq"]), ("Wukv", c.kv_rank, ["Wuk", "Wuv"]),
                    ("Wo", d, ["Wo"])]
        return plan + [("Wg", d, ["Wg"]), ("Wu", d, ["Wu"]), ("Wd", c.d_ff, ["Wd"])]

    def _shard_plan(self) -> List[tuple]:
        return shard_plan(self.cfg, self.tp_rank, self.tp_world)

    def _q8_from_parts(self, name: str, K: int, parts: List[tuple], fill: Callable[[str, int], None]) -> None:
        """Allocate a Q8 object [K × ΣN] and quantize each window into its column range.
        `fill(ref_name, tmp_id)` must fill the float buffer tmp_id with the whole reference matrix."""
        shapes = self._ref_shapes
        q = self._new_id()
        _lib.check(self.lib.deepj_cuda_q8_alloc(q, K, sum(p[3] for p in parts)))
        col = 0
        for ref, k0, n0, n in parts:
            rows, cols = shapes[ref]
            tmp = self._f32("", rows * cols)
            fill(ref, tmp)
            _lib.check(self.lib.deepj_cuda_q8_quantize_into(q, col, tmp, k0, n0, cols, n))
            self._release([tmp])
            col += n
        self.ids[name] = q

    def _load(self, fill_layer: Callable[[int], Callable[[str, int], None]], vec: Callable[[str, int, int], np.ndarray]) -> None:
        c, r = self.cfg, self.tp_rank
        Fl, Vl = self.f_local, self.v_local
        for l in range(c.n_layers):
            self._f32(f"g1.{l}", c.d_model, vec("g1", l, c.d_model))
            self._f32(f"g2.{l}", c.d_model, vec("g2", l, c.d_model))
            for obj, K, parts in self._shard_plan():
                self._q8_from_parts(f"{obj}.{l}", K, parts, fill_layer(l))
            if c.kind == "gpt":
                for name, n in (("b1", c.d_model), ("b2", c.d_model), ("c1", c.d_ff), ("c2", c.d_model)):
                    self._f32(f"{name}.{l}", n, vec(name, l, n))
                continue
            self._f32(f"bg.{l}", Fl, vec("bg", l, c.d_ff)[r * Fl:(r + 1) * Fl])
            self._f32(f"bu.{l}", Fl, vec("bu", l, c.d_ff)[r * Fl:(r + 1) * Fl])
            self._f32(f"bd.{l}", c.d_model, vec("bd", l, c.d_model))
        self._f32("gF", c.d_model, vec("gF", -1, c.d_model))
        if c.kind == "gpt":
            self._f32("bF", c.d_model, vec("bF", -1, c.d_model))
        self._q8_from_parts("Wlm", c.d_model, [("Wlm", 0, r * Vl, Vl)], fill_layer(-1))
        self._f32("blm", Vl, vec("blm", -1, c.vocab_size)[r * Vl:(r + 1) * Vl])
        self.loaded = True

    def load_weights(self, get: Callable[[str, int], np.ndarray]) -> None:
        """Upload fp32 weights and quantize them on the device.

        `get(name, layer)` returns the reference tensor as a numpy array: matmul
        weights as [dIn × dOut] (layers/Linear.java:26), vectors 1-D.  Names: "emb",
        per layer "g1","g2", the block's matmul names (`DecoderConfig.matmul_shapes`),
        "bg","bu","bd"; then "gF","Wlm","blm" (layer = -1 for model-level tensors).
        Under tensor parallelism every rank is given the full tensors and keeps its shard.
        """
        c = self.cfg
        self._f32("emb", c.vocab_size * c.d_model, get("emb", -1))
        if c.kind == "gpt":
            self._f32("posemb", c.max_seq_len * c.d_model, get("pos", -1))
        self._load(lambda l: (lambda ref, tmp: self._upload(tmp, get(ref, l))),
                   lambda name, l, n: np.asarray(get(name, l), dtype=np.float32).reshape(-1))

    def load_synthetic(self, seed: int, std: float) -> None:
        """Random-init weights of this architecture generated on the device with the
        library's counter-based generator; one ordinal per matrix in the reference's
        construction order (embedding, then every block's matrices, then the LM
        head).  Norm gains are ones and biases zeros, as the reference initialises them."""
        c = self.cfg
        per_layer = c.matmul_shapes()
        shapes = self._ref_shapes

        def fill_layer(l):
            def fill(ref, tmp):
                ordinal = 1 + c.n_layers * len(per_layer) if ref == "Wlm" else \
                    1 + l * len(per_layer) + [n for n, _, _ in per_layer].index(ref)
                _lib.check(self.lib.deepj_cuda_synth_fill(tmp, seed, ordinal, std, 0, shapes[ref][0] * shapes[ref][1]))
            return fill

        emb = self._f32("emb", c.vocab_size * c.d_model)
        _lib.check(self.lib.deepj_cuda_synth_fill(emb, seed, 0, std, 0, c.vocab_size * c.d_model))
        if c.kind == "gpt":
            pos = self._f32("posemb", c.max_seq_len * c.d_model)
            _lib.check(self.lib.deepj_cuda_synth_fill(pos, seed, 2 + c.n_layers * len(per_layer), std, 0, c.max_seq_len * c.d_model))
        self._load(fill_layer, lambda name, l, n: (np.ones(n, dtype=np.float32) if name.startswith("g") else np.zeros(n, dtype=np.float32)))

    def q8_arrays(self, name: str):
        """Canonical (codes[N][K] int8, scales[N][ceil(K/32)] fp32) of a device Q8 object."""
        c = self.cfg
        base = name.split(".")[0]
        plan = {o: (k, sum(p[3] for p in parts)) for o, k, parts in self._shard_plan()}
        K, N = plan.get(base, (c.d_model, self.v_local))
        codes = np.empty((N, K), dtype=np.int8)
        scales = np.empty((N, (K + 31) // 32), dtype=np.float32)
        _lib.check(self.lib.deepj_cuda_q8_download(self.ids[name], codes.ctypes.data, scales.ctypes.data))
        return codes, scales

    # ── the per-token stream ──
    def _build(self, feed_back: bool, sampler: Optional[Tuple[int, float]] = None) -> np.ndarray:
        c, B, I = self.cfg, self.B, self.ids
        d, V = c.d_model, c.vocab_size
        dl, Fl, Vl, Hl = self.d_local, self.f_local, self.v_local, self.h_local
        tp = self.tp_world > 1
        eps = float_bits(RMS_EPS)
        s: List[int] = []
        labels: List[str] = []

        bounds: List[Tuple[int, int]] = []

        def op(label, *ints):
            bounds.append((len(s), len(s) + len(ints)))
            s.extend(int(v) for v in ints)
            labels.append(label)

        def linear(label, x, x_off, ldx, gamma, w, bias, res, res_off, ldr, out, out_off, ldo):
            op(label, OP_Q8_LINEAR, x, x_off, ldx, gamma, eps, w, bias, res, res_off, ldr, out, out_off, ldo, B)

        op("embed", OP_EMBED_GATHER, I["emb"], I["tok"], I["x"], B, d, V)
        if c.kind == "gpt":
            self._gpt_blocks(op, I["x"], I["x2"], I["xp"], I["qkv"], I["att"], I["h"], I["pos"], B, 1)
            op("lm_head", OP_Q8_LINEAR_LN, I["x"], 0, d, I["gF"], I["bF"], float_bits(LN_EPS), I["Wlm"], I["blm"], -1, 0, 0,
               I["logits"], 0, V, B, 0)
        for l in range(c.n_layers if c.kind != "gpt" else 0):
            if c.kind == "llama":
                linear("qkv", I["x"], 0, d, I[f"g1.{l}"], I[f"Wqkv.{l}"], -1, -1, 0, 0, I["qkv"], 0, 3 * dl)
            else:
                r = c.q_rank + c.kv_rank
                linear("mla_down", I["x"], 0, d, I[f"g1.{l}"], I[f"Wdqkv.{l}"], -1, -1, 0, 0, I["lat"], 0, r)
                linear("mla_up_q", I["lat"], 0, r, -1, I[f"Wuq.{l}"], -1, -1, 0, 0, I["qkv"], 0, 3 * dl)
                linear("mla_up_kv", I["lat"], c.q_rank, r, -1, I[f"Wukv.{l}"], -1, -1, 0, 0, I["qkv"], dl, 3 * dl)
            op("attn", OP_ATTN_DECODE, I["qkv"], 0, dl, 2 * dl, 3 * dl, I["kv"], l, I["pos"], I["cos"], I["sin"],
               I["att"], 0, dl, B, Hl, c.head_dim)
            if tp:
                # row-parallel: every rank holds a partial sum; the exchange adds them (+ residual, + bias)
                linear("wo", I["att"], 0, dl, -1, I[f"Wo.{l}"], -1, -1, 0, 0, I["part"], 0, d)
                op("allreduce", OP_TP_ALLREDUCE, I["part"], -1, I["x"], I["x2"], B, d)
            else:
                linear("wo", I["att"], 0, dl, -1, I[f"Wo.{l}"], -1, I["x"], 0, d, I["x2"], 0, d)
            op("swiglu", OP_Q8_SWIGLU, I["x2"], 0, d, I[f"g2.{l}"], eps, I[f"Wg.{l}"], I[f"bg.{l}"], I[f"Wu.{l}"],
               I[f"bu.{l}"], I["h"], 0, Fl, B)
            if tp:
                linear("down", I["h"], 0, Fl, -1, I[f"Wd.{l}"], -1, -1, 0, 0, I["part"], 0, d)
                op("allreduce", OP_TP_ALLREDUCE, I["part"], I[f"bd.{l}"], I["x2"], I["x"], B, d)
            else:
                linear("down", I["h"], 0, Fl, -1, I[f"Wd.{l}"], I[f"bd.{l}"], I["x2"], 0, d, I["x"], 0, d)
        if tp:
            linear("lm_head", I["x"], 0, d, I["gF"], I["Wlm"], I["blm"], -1, 0, 0, I["logits_local"], 0, Vl)
            op("allgather", OP_TP_ALLGATHER, I["logits_local"], I["logits"], B, Vl)
        elif c.kind != "gpt":
            linear("lm_head", I["x"], 0, d, I["gF"], I["Wlm"], I["blm"], -1, 0, 0, I["logits"], 0, V)
        if sampler is None:
            op("argmax", OP_ARGMAX_ROWS, I["logits"], I["next"], B, V)
        else:
            op("sample", OP_SAMPLE_TOPK, I["logits"], I["r"], I["next"], B, V, sampler[0], float_bits(sampler[1]))
        op("advance", OP_ADD_SCALAR_INPLACE, I["pos"], float_bits(1.0), B)
        if feed_back:
            op("feed_back", OP_COPY, I["next"], 0, I["tok"], 0, B)
        self._op_labels = labels
        self._op_bounds = bounds
        return np.asarray(s, dtype=np.int32)

    def _gpt_blocks(self, op, x, x2, xp, qkv, att, h, pos_ids, B: int, T: int) -> None:
        """The GPT part of a stream between the token gather and the final norm, for M = B·T rows: add the learned
        position rows (embeddings/PositionalEmbedding.java:26-33; `pos_ids` holds one position per row), then per
        block LayerNorm→QKV, attention, Wo + residual, LayerNorm→W1 + c1→GELU, W2 + c2 + residual."""
        c, I = self.cfg, self.ids
        d, F, M = c.d_model, c.d_ff, B * T
        eps = float_bits(LN_EPS)
        op("pos_embed", OP_EMBED_GATHER, I["posemb"], pos_ids, xp, M, d, c.max_seq_len)
        op("pos_add", OP_ADD, x, xp, x, M * d)
        for l in range(c.n_layers):
            op("qkv", OP_Q8_LINEAR_LN, x, 0, d, I[f"g1.{l}"], I[f"b1.{l}"], eps, I[f"Wqkv.{l}"], -1, -1, 0, 0, qkv, 0, 3 * d, M, 0)
            if T == 1:
                op("attn", OP_ATTN_DECODE, qkv, 0, d, 2 * d, 3 * d, I["kv"], l, I["pos"], I["cos"], I["sin"], att, 0, d, B, c.n_heads, c.head_dim)
            else:
                op("attn", OP_ATTN_PREFILL, qkv, 0, d, 2 * d, 3 * d, I["kv"], l, I["pos"], I["cos"], I["sin"], att, 0, d, B, c.n_heads,
                   c.head_dim, T)
            op("wo", OP_Q8_LINEAR, att, 0, d, -1, 0, I[f"Wo.{l}"], -1, x, 0, d, x2, 0, d, M)
            op("ffn_up", OP_Q8_LINEAR_LN, x2, 0, d, I[f"g2.{l}"], I[f"b2.{l}"], eps, I[f"W1.{l}"], I[f"c1.{l}"], -1, 0, 0, h, 0, F, M, 1)
            op("ffn_down", OP_Q8_LINEAR, h, 0, F, -1, 0, I[f"W2.{l}"], I[f"c2.{l}"], x2, 0, d, x, 0, d, M)

    def _streams(self):
        if not self.loaded:
            raise RuntimeError("weights are not loaded")
        if self._stream_host is None:
            if self.fused_step:
                plan = self._decode_plan()
                self._stream_dev = np.asarray([OP_DECODE_STEP, plan, 1], dtype=np.int32)
                self._stream_host = np.asarray([OP_DECODE_STEP, plan, 0], dtype=np.int32)
            else:
                self._stream_dev = self._build(feed_back=True)
                self._stream_host = self._build(feed_back=False)
        return self._stream_host, self._stream_dev

    def _decode_plan(self) -> int:
        """The plan object behind op 76: every buffer and weight of a token step, resolved once by the library."""
        if self._plan_id is None:
            c, I = self.cfg, self.ids
            logits = I["logits_local"] if self.tp_world > 1 else I["logits"]
            desc = [1, c.n_layers, self.h_local, c.head_dim, float_bits(RMS_EPS),
                    I["tok"], I["pos"], I["emb"], I["cos"], I["sin"], I["kv"], I["x"], I["x2"], I["qkv"], I["att"], I["h"],
                    logits, I["next"], I["gF"], I["Wlm"], I["blm"]]
            for l in range(c.n_layers):
                desc += [I[f"g1.{l}"], I[f"Wqkv.{l}"], I[f"Wo.{l}"], I[f"g2.{l}"], I[f"Wg.{l}"], I[f"bg.{l}"], I[f"Wu.{l}"], I[f"bu.{l}"],
                         I[f"Wd.{l}"], I[f"bd.{l}"]]
            arr = np.asarray(desc, dtype=np.int32)
            plan = self._new_id()
            _lib.check(self.lib.deepj_cuda_decode_plan(plan, arr.ctypes.data, arr.size))
            self._plan_id = plan
        return self._plan_id

    # ── stepping ──
    def reset(self) -> None:
        """Start every sequence at position 0 (cache contents are overwritten as it refills)."""
        self._upload(self.ids["pos"], np.zeros(self.B, dtype=np.float32))
        self.position = 0

    def set_position(self, position: int) -> None:
        """Rewind (or advance) every sequence to `position`; cache rows at and beyond it are
        overwritten by the following steps."""
        if position < 0 or position > self.cfg.max_seq_len:
            raise ValueError(f"position {position} outside 0..{self.cfg.max_seq_len}")
        self._upload(self.ids["pos"], np.full(self.B, float(position), dtype=np.float32))
        self.position = int(position)

    def _pinned(self) -> Tuple[np.ndarray, np.ndarray]:
        """Page-locked staging for the ids going up and the picks coming down each step ([B] floats each)."""
        if self._pin_ptr is None:
            ptr = ctypes.c_void_p()
            _lib.check(self.lib.deepj_cuda_pinned_alloc(ctypes.byref(ptr), 8 * self.B))
            self._pin_ptr = ptr
            buf = (ctypes.c_float * (2 * self.B)).from_address(ptr.value)
            arr = np.frombuffer(buf, dtype=np.float32)
            self._pin_tok, self._pin_next = arr[:self.B], arr[self.B:]
        return self._pin_tok, self._pin_next

    def set_tokens(self, tokens) -> None:
        t = np.asarray(tokens, dtype=np.int64).reshape(-1)
        if t.size != self.B:
            raise ValueError(f"expected {self.B} token ids, got {t.size}")
        # Embedding.forward range check (transformer/embeddings/Embedding.java:30-32)
        if t.min() < 0 or t.max() >= self.cfg.vocab_size:
            bad = t[(t < 0) | (t >= self.cfg.vocab_size)][0]
            raise ValueError(f"Token id out of range: {int(bad)}")
        tok, _ = self._pinned()
        tok[:] = t
        _lib.check(self.lib.deepj_cuda_upload_buffer(self.ids["tok"], tok.ctypes.data, self.B))

    def step(self, tokens) -> np.ndarray:
        """One token per sequence through host buffers: upload the ids, flush the
        stream (synchronous), download the greedy picks."""
        if self.position >= self.cfg.max_seq_len:
            raise ValueError(f"seqLen {self.position + 1} exceeds maxSeqLen {self.cfg.max_seq_len}")
        host, _ = self._streams()
        self.set_tokens(tokens)
        # enqueue the stream behind the upload and let the download's synchronisation be the only one of the step
        _lib.check(self.lib.deepj_cuda_flush_ops_async(host.ctypes.data, host.size))
        self.position += 1
        _, nxt = self._pinned()
        _lib.check(self.lib.deepj_cuda_download_buffer(self.ids["next"], nxt.ctypes.data, self.B))
        return nxt.astype(np.int64)

    def step_device(self, n_steps: int = 1, sync: bool = True) -> None:
        """n greedy steps with the picked token fed back on the device (no host copies)."""
        if self.position + n_steps > self.cfg.max_seq_len:
            raise ValueError(f"seqLen {self.position + n_steps} exceeds maxSeqLen {self.cfg.max_seq_len}")
        _, dev = self._streams()
        for _ in range(n_steps):
            _lib.check(self.lib.deepj_cuda_flush_ops_async(dev.ctypes.data, dev.size))
        self.position += n_steps
        if sync:
            _lib.check(self.lib.deepj_cuda_synchronize())

    def logits(self) -> np.ndarray:
        if self.fused_step and self.tp_world > 1:
            # the single-kernel step leaves this rank's vocabulary columns; gather the ranks' shards (every rank calls this)
            I = self.ids
            g = np.asarray([OP_TP_ALLGATHER, I["logits_local"], I["logits"], self.B, self.v_local], dtype=np.int32)
            _lib.check(self.lib.deepj_cuda_flush_ops(g.ctypes.data, g.size))
        return self._download(self.ids["logits"], self.B * self.cfg.vocab_size).reshape(self.B, self.cfg.vocab_size)

    def next_tokens(self) -> np.ndarray:
        return self._download(self.ids["next"], self.B).astype(np.int64)

    PREFILL_CHUNK = 2048     # prompt tokens per sequence and pass of the many-row path (enough 128 × 256 tiles for the GEMM to pair them)

    def _build_prefill(self, T: int) -> np.ndarray:
        """The stream of one prompt chunk: T tokens of every sequence at once, B·T activation rows through the
        many-row Q8 kernels and the chunk attention op; the last token's hidden state lands in the decode
        buffers and the positions advance by T.  The row-major layout is row = b·T + t.  Under tensor parallelism
        the Wo and down projections leave partial sums that the exchange op adds over the ranks, M rows at a time."""
        c, B, I, P = self.cfg, self.B, self.ids, self._prefill_ids
        d, dl, Fl, Hl = c.d_model, self.d_local, self.f_local, self.h_local
        M = B * T
        eps = float_bits(RMS_EPS)
        s: List[int] = []

        def linear(x, x_off, ldx, gamma, w, bias, res, ldr, out, ldo):
            s.extend(int(v) for v in (OP_Q8_LINEAR, x, x_off, ldx, gamma, eps, w, bias, res, 0, ldr, out, 0, ldo, M))

        s.extend((OP_EMBED_GATHER, I["emb"], P["tok"], P["x"], M, d, c.vocab_size))
        if c.kind == "gpt":
            self._gpt_blocks(lambda _label, *ints: s.extend(int(v) for v in ints), P["x"], P["x2"], P["xp"], P["qkv"], P["att"], P["h"],
                             P["ppos"], B, T)
        for l in range(c.n_layers if c.kind != "gpt" else 0):
            if c.kind == "llama":
                linear(P["x"], 0, d, I[f"g1.{l}"], I[f"Wqkv.{l}"], -1, -1, 0, P["qkv"], 3 * dl)
            else:
                r = c.q_rank + c.kv_rank
                linear(P["x"], 0, d, I[f"g1.{l}"], I[f"Wdqkv.{l}"], -1, -1, 0, P["lat"], r)
                linear(P["lat"], 0, r, -1, I[f"Wuq.{l}"], -1, -1, 0, P["qkv"], 3 * dl)
                s.extend(int(v) for v in (OP_Q8_LINEAR, P["lat"], c.q_rank, r, -1, eps, I[f"Wukv.{l}"], -1, -1, 0, 0, P["qkv"], dl, 3 * dl, M))
            s.extend(int(v) for v in (OP_ATTN_PREFILL, P["qkv"], 0, dl, 2 * dl, 3 * dl, I["kv"], l, I["pos"], I["cos"], I["sin"],
                                      P["att"], 0, dl, B, Hl, c.head_dim, T))
            if self.tp_world > 1:       # row-parallel projections leave partial sums; the exchange adds them (+ residual, + bias)
                linear(P["att"], 0, dl, -1, I[f"Wo.{l}"], -1, -1, 0, P["part"], d)
                s.extend((OP_TP_ALLREDUCE, P["part"], -1, P["x"], P["x2"], M, d))
            else:
                linear(P["att"], 0, dl, -1, I[f"Wo.{l}"], -1, P["x"], d, P["x2"], d)
            s.extend(int(v) for v in (OP_Q8_SWIGLU, P["x2"], 0, d, I[f"g2.{l}"], eps, I[f"Wg.{l}"], I[f"bg.{l}"], I[f"Wu.{l}"],
                                      I[f"bu.{l}"], P["h"], 0, Fl, M))
            if self.tp_world > 1:
                linear(P["h"], 0, Fl, -1, I[f"Wd.{l}"], -1, -1, 0, P["part"], d)
                s.extend((OP_TP_ALLREDUCE, P["part"], I[f"bd.{l}"], P["x2"], P["x"], M, d))
            else:
                linear(P["h"], 0, Fl, -1, I[f"Wd.{l}"], I[f"bd.{l}"], P["x2"], d, P["x"], d)
        for b in range(B):
            s.extend((OP_COPY, P["x"], (b * T + T - 1) * d, I["x"], b * d, d))
        s.extend((OP_ADD_SCALAR_INPLACE, I["pos"], float_bits(float(T)), B))
        return np.asarray(s, dtype=np.int32)

    def _head_stream(self) -> np.ndarray:
        """Final norm + LM head + greedy pick on the hidden state in the decode buffer."""
        c, B, I = self.cfg, self.B, self.ids
        if c.kind == "gpt":
            s = [OP_Q8_LINEAR_LN, I["x"], 0, c.d_model, I["gF"], I["bF"], float_bits(LN_EPS), I["Wlm"], I["blm"], -1, 0, 0, I["logits"], 0,
                 c.vocab_size, B, 0]
        elif self.tp_world > 1:
            s = [OP_Q8_LINEAR, I["x"], 0, c.d_model, I["gF"], float_bits(RMS_EPS), I["Wlm"], I["blm"], -1, 0, 0, I["logits_local"], 0, self.v_local, B,
                 OP_TP_ALLGATHER, I["logits_local"], I["logits"], B, self.v_local]
        else:
            s = [OP_Q8_LINEAR, I["x"], 0, c.d_model, I["gF"], float_bits(RMS_EPS), I["Wlm"], I["blm"], -1, 0, 0, I["logits"], 0, c.vocab_size, B]
        s += [OP_ARGMAX_ROWS, I["logits"], I["next"], B, c.vocab_size]
        return np.asarray(s, dtype=np.int32)

    def prefill(self, prompts, chunked: Optional[bool] = None) -> np.ndarray:
        """Feed the prompt (every sequence the same length); returns the greedy pick after its last token.
        Prompts of 32 tokens or more go through the many-row path in chunks of PREFILL_CHUNK tokens per
        sequence (tensor-core GEMMs, chunk attention); shorter ones one decode step per position.  Under tensor
        parallelism a chunk's rows × dModel must fit the exchange slot (`tp_slot_floats`), which bounds the chunk."""
        p = np.asarray(prompts, dtype=np.int64).reshape(self.B, -1)
        T_all = p.shape[1]
        tp_rows = self.tp_slot_floats // self.cfg.d_model // self.B if self.tp_world > 1 else 0      # tokens per sequence and chunk
        if chunked is None:
            chunked = T_all >= 32 and (self.tp_world == 1 or tp_rows >= 16)
        if not chunked or T_all == 0:
            nxt = None
            for t in range(T_all):
                nxt = self.step(p[:, t])
            return nxt
        if self.tp_world > 1 and tp_rows < 1:
            raise ValueError("the exchange slot (tp_slot_floats) is smaller than one token per sequence")
        if np.any(p < 0) or np.any(p >= self.cfg.vocab_size):
            raise ValueError(f"Token id out of range: {int(p[(p < 0) | (p >= self.cfg.vocab_size)][0])}")
        if self.position + T_all > self.cfg.max_seq_len:
            raise ValueError(f"seqLen {self.position + T_all} exceeds maxSeqLen {self.cfg.max_seq_len}")
        C = min(self.PREFILL_CHUNK, T_all, max(1, 65535 // self.B))
        if self.tp_world > 1:
            C = min(C, tp_rows)
        self._ensure_prefill_buffers(C)
        done = 0
        while done < T_all:
            T = min(C, T_all - done)
            if T not in self._prefill_streams:
                self._prefill_streams[T] = self._build_prefill(T)
            st = self._prefill_streams[T]
            self._upload(self._prefill_ids["tok"], p[:, done:done + T].astype(np.float32).reshape(-1))
            if self.cfg.kind == "gpt":       # row b·T + t sits at position (start of the chunk) + t
                rows = np.tile(np.arange(self.position, self.position + T, dtype=np.float32), self.B)
                self._upload(self._prefill_ids["ppos"], rows)
            _lib.check(self.lib.deepj_cuda_flush_ops(st.ctypes.data, st.size))
            done += T
            self.position += T
        hs = self._head_stream()
        _lib.check(self.lib.deepj_cuda_flush_ops(hs.ctypes.data, hs.size))
        return self.next_tokens()

    def _ensure_prefill_buffers(self, C: int) -> None:
        if self._prefill_cap >= C:
            return
        if self._prefill_ids:
            self._release(list(self._prefill_ids.values()))
        c, M = self.cfg, self.B * C
        sizes = {"tok": M, "x": M * c.d_model, "x2": M * c.d_model, "qkv": M * 3 * self.d_local, "att": M * self.d_local,
                 "h": M * self.f_local}
        if c.kind == "deepseek":
            sizes["lat"] = M * (c.q_rank + c.kv_rank)
        if c.kind == "gpt":
            sizes["xp"], sizes["ppos"] = M * c.d_model, M
        if self.tp_world > 1:
            sizes["part"] = M * c.d_model
        self._prefill_ids = {}
        for name, n in sizes.items():
            self._prefill_ids[name] = self._f32("", n)
        self._prefill_cap = C
        self._prefill_streams = {}

    def generate(self, prompt, max_new_tokens: int, temperature: float = 1.0, top_k: int = 40, seed: int = 0) -> np.ndarray:
        """TextGenerator.generate for batch 1 (models/TextGenerator.java:66-151) with the draw on the device:
        temperature / top-k sampling, one `java.util.Random(seed).nextFloat()` per new token, the logits never
        leave the GPU.  topK = 0 means the whole vocabulary, as in the reference (TextGenerator.java:111-115)."""
        from .jrandom import JavaRandom
        if max_new_tokens < 0:
            raise ValueError("maxNewTokens must be >= 0")
        if not temperature > 0.0:
            raise ValueError("temperature must be > 0")
        if top_k < 0:
            raise ValueError("topK must be >= 0")
        if self.B != 1:
            raise ValueError("generate drives one sequence")
        rnd = JavaRandom(seed)
        c, I = self.cfg, self.ids
        pick = np.asarray([OP_SAMPLE_TOPK, I["logits"], I["r"], I["next"], 1, c.vocab_size, top_k, float_bits(float(temperature))], dtype=np.int32)
        step = self._build(feed_back=False, sampler=(top_k, float(temperature)))
        self.reset()
        self.prefill(np.asarray(prompt).reshape(1, -1))              # leaves the last prompt position's logits on the device
        out = []
        for i in range(max_new_tokens):
            self._upload(I["r"], np.asarray([rnd.next_float()], dtype=np.float32))
            if i == 0:
                _lib.check(self.lib.deepj_cuda_flush_ops(pick.ctypes.data, pick.size))
            else:
                if self.position + 1 > c.max_seq_len:
                    raise ValueError(f"seqLen {self.position + 1} exceeds maxSeqLen {c.max_seq_len}")
                self._upload(I["tok"], np.asarray([out[-1]], dtype=np.float32))
                _lib.check(self.lib.deepj_cuda_flush_ops(step.ctypes.data, step.size))
                self.position += 1
            out.append(int(self.next_tokens()[0]))
        return np.asarray(out, dtype=np.int64)

    def generate_greedy(self, prompt, max_new_tokens: int, keep_logits: bool = False):
        """TextGenerator.generate with topK = 1 (models/TextGenerator.java:66-100)
        for batch 1: returns the new token ids (and the logits row behind each)."""
        if max_new_tokens < 0:
            raise ValueError("maxNewTokens must be >= 0")
        if self.B != 1:
            raise ValueError("generate_greedy drives one sequence")
        self.reset()
        nxt = self.prefill(np.asarray(prompt).reshape(1, -1))
        out, rows = [], []
        for i in range(max_new_tokens):
            if keep_logits:
                rows.append(self.logits()[0].copy())
            tok = int(nxt[0])
            out.append(tok)
            if i + 1 < max_new_tokens:
                nxt = self.step([tok])
        return (np.asarray(out, dtype=np.int64), np.stack(rows) if rows else None) if keep_logits else np.asarray(out, dtype=np.int64)

    def profile_step(self):
        """Device time of every op of one token step, run op by op as the per-operator stream (also when the
        decoder itself steps with the single-kernel op): [(label, ms)]."""
        if not self.loaded:
            raise RuntimeError("weights are not loaded")
        host = self._build(feed_back=False)
        n = len(self._op_labels) + 1
        ms = np.zeros(n, dtype=np.float32)
        cnt = ctypes.c_int32(0)
        _lib.check(self.lib.deepj_cuda_profile_ops(host.ctypes.data, host.size, ms.ctypes.data, n, ctypes.byref(cnt)))
        self.position += 1
        return list(zip(self._op_labels, ms[: cnt.value].tolist()))

    def time_ops(self, labels, iters: int = 20, warmup: int = 3) -> Tuple[float, int]:
        """Device time of the ops whose label is in `labels`, run back to back as their own stream
        (graph-replayed like the full step, at the current position): (ms per pass, ops per pass)."""
        full = self._build(feed_back=False)
        keep = [full[a:b] for lbl, (a, b) in zip(self._op_labels, self._op_bounds) if lbl in labels]
        if not keep:
            return 0.0, 0
        sub = np.ascontiguousarray(np.concatenate(keep))
        for _ in range(max(warmup, 3)):
            _lib.check(self.lib.deepj_cuda_flush_ops(sub.ctypes.data, sub.size))
        _lib.check(self.lib.deepj_cuda_timer_begin())
        for _ in range(iters):
            _lib.check(self.lib.deepj_cuda_flush_ops_async(sub.ctypes.data, sub.size))
        ms = ctypes.c_float(0)
        _lib.check(self.lib.deepj_cuda_timer_end(ctypes.byref(ms)))
        return ms.value / iters, len(keep)

    def stats(self) -> Dict[str, int]:
        v = (ctypes.c_int64 * 6)()
        _lib.check(self.lib.deepj_cuda_stats(v, 6))
        return {"eager_launches": v[0], "graph_replays": v[1], "graphs_captured": v[2],
                "kernels_per_replay": v[3], "workspace_bytes": v[4], "device_error": v[5]}

    def close(self) -> None:
        if self._pin_ptr is not None:
            self.lib.deepj_cuda_pinned_free(self._pin_ptr)
            self._pin_ptr = None
        if self._owned:
            self._release(list(self._owned))
