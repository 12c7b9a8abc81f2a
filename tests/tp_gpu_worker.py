"""One rank of the tensor-parallel GPU parity check (launched by torchrun, one process per GPU):
a small Llama decoded with the weights sharded over the ranks must reproduce the oracle's
logits and greedy tokens, and every rank must end up with the same tokens."""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, HERE)

import oracle
from deepj_b200 import tp
from deepj_b200.decoder import DecoderConfig, Q8Decoder
from test_decoder_gpu import weight_getter


def main():
    rank, world = tp.init_process_group()
    local = int(os.environ.get("LOCAL_RANK", rank))
    kind = sys.argv[1] if len(sys.argv) > 1 else "llama"
    batch = int(sys.argv[2]) if len(sys.argv) > 2 else 2          # 1: the decode steps run as the single whole-token kernel
    if kind == "llama":
        cfg = DecoderConfig("llama", 512, 64, 512, 8, 2, 1024)
    else:
        cfg = DecoderConfig("deepseek", 512, 64, 512, 8, 2, 1024, q_rank=256, kv_rank=128)
    om = oracle.OracleModel(cfg.kind, cfg.vocab_size, cfg.max_seq_len, cfg.d_model, cfg.n_heads, cfg.n_layers, cfg.d_ff,
                            cfg.q_rank, cfg.kv_rank, seed=21)
    B, T = batch, 40
    # slots large enough for a 24-token chunk per sequence: the 40-token prompt goes through the many-row path in
    # two chunks (24 + 16 tokens, 48 and 32 rows per exchange), the steps after it through the decode path
    slot = max(B * 24 * cfg.d_model, B * cfg.vocab_size // world)
    dec = Q8Decoder(cfg, batch=B, device=local, tp_rank=rank, tp_world=world, tp_slot_floats=slot, fused_step=(B == 1))
    tp.connect(rank, world, slot, large_message_floats=8192)      # both exchange grids and both slot regions get used
    dec.load_weights(weight_getter(om, cfg))
    om.apply_q8()
    tp.barrier()              # the exchange kernel's wait for a peer is bounded: start stepping together
    rng = np.random.default_rng(5)
    prompts = rng.integers(0, cfg.vocab_size, size=(B, T))
    dec.reset()
    nxt = dec.prefill(prompts)
    got_tokens = [nxt.copy()]
    got_logits = [dec.logits().copy()]
    for _ in range(7):
        nxt = dec.step(nxt)
        got_tokens.append(nxt.copy())
        got_logits.append(dec.logits().copy())
    got_tokens = np.stack(got_tokens, axis=1)
    for b in range(B):
        toks, logits = om.generate_greedy(list(prompts[b]), 8, use_cache=True)
        mine = np.stack([g[b] for g in got_logits])
        rng_ = float(logits.max() - logits.min())
        err = float(np.abs(mine - logits).max())
        assert err <= 2e-3 * rng_, (rank, b, err, rng_)
        assert np.array_equal(toks, got_tokens[b]), (rank, b, toks, got_tokens[b])
    st = dec.stats()
    assert st["device_error"] == 0, st
    blobs = tp.all_gather_bytes(got_tokens.astype(np.int64).tobytes())
    assert all(b == blobs[0] for b in blobs)
    dec.close()
    tp.disconnect()
    if rank == 0:
        print(f"TP_GPU_OK world={world} kind={kind} batch={B} fused_step={dec.fused_step}", flush=True)


if __name__ == "__main__":
    main()
