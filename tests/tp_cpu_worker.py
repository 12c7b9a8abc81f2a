"""World-size-2 (gloo, CPU) check of the tensor-parallel host logic: handle exchange order,
max-over-ranks, and that the shard plan's partial products add up to the unsharded layer."""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, HERE)

import torch
import torch.distributed as dist

import oracle
from deepj_b200 import tp
from deepj_b200.decoder import DecoderConfig, shard_plan


def main():
    rank, world = tp.init_process_group()
    blobs = tp.all_gather_bytes(bytes([rank]) * 64)
    assert [b[0] for b in blobs] == list(range(world)) and all(len(b) == 64 for b in blobs)
    assert tp.max_over_ranks(float(rank)) == float(world - 1)

    cfg = DecoderConfig("llama", 256, 16, 128, 4, 1, 384)
    om = oracle.OracleModel("llama", 256, 16, 128, 4, 1, 384, seed=4)
    shapes = {n: (k, w) for n, k, w in cfg.matmul_shapes()}
    W = {n: oracle.q8_dequantize(*oracle.q8_quantize(om.weight(n, 0).reshape(shapes[n]))) for n in shapes}
    plan = dict((o, (k, parts)) for o, k, parts in shard_plan(cfg, rank, world))

    def shard(obj):
        k, parts = plan[obj]
        return np.concatenate([W[ref][k0:k0 + k, n0:n0 + n] for ref, k0, n0, n in parts], axis=1)

    # quantizing a shard equals the shard of the quantized matrix (blocks never straddle a split)
    for obj, (k, parts) in plan.items():
        for ref, k0, n0, n in parts:
            full = om.weight(ref, 0).reshape(shapes[ref])
            c_full, s_full = oracle.q8_quantize(full)
            c_sh, s_sh = oracle.q8_quantize(np.ascontiguousarray(full[k0:k0 + k, n0:n0 + n]))
            assert np.array_equal(c_sh, c_full[n0:n0 + n, k0:k0 + k]) and np.array_equal(s_sh, s_full[n0:n0 + n, k0 // 32:(k0 + k) // 32])

    rng = np.random.default_rng(0)
    x = rng.standard_normal((2, cfg.d_model)).astype(np.float32)
    dl, Fl = cfg.d_model // world, cfg.d_ff // world
    # column-parallel QKV then row-parallel Wo: sum of partials == full product
    qkv_local = x @ shard("Wqkv")
    v_local = qkv_local[:, 2 * dl:]
    part = torch.from_numpy((v_local @ shard("Wo")).astype(np.float64))
    dist.all_reduce(part)
    full = (x @ W["Wv"]) @ W["Wo"]
    assert np.abs(part.numpy() - full).max() < 1e-4
    # column-parallel gate/up then row-parallel down
    g, u = x @ shard("Wg"), x @ shard("Wu")
    part = torch.from_numpy(((g * u) @ shard("Wd")).astype(np.float64))
    dist.all_reduce(part)
    full = ((x @ W["Wg"]) * (x @ W["Wu"])) @ W["Wd"]
    assert np.abs(part.numpy() - full).max() < 1e-4
    # a rank that never joins is detected on the host: a short timeout ends the collective with an error
    tp.barrier()
    if rank == 0:
        print("TP_CPU_OK", flush=True)


if __name__ == "__main__":
    main()
