"""Tensor-parallel host logic on CPU ranks (gloo, world size 2)."""
import os
import subprocess
import sys

import pytest

from deepj_b200.decoder import DecoderConfig, shard_plan

HERE = os.path.dirname(os.path.abspath(__file__))


def test_shard_plan_covers_every_weight_exactly_once():
    for kind, kw in (("llama", {}), ("deepseek", dict(q_rank=1024, kv_rank=512))):
        cfg = DecoderConfig(kind, 32000, 64, 2048 if kind == "deepseek" else 4096, 16 if kind == "deepseek" else 32, 2,
                            5632 if kind == "deepseek" else 11008, **kw)
        shapes = {n: (k, w) for n, k, w in cfg.matmul_shapes()}
        for world in (1, 2, 4, 8):
            cover = {n: 0 for n in shapes}
            for rank in range(world):
                for obj, K, parts in shard_plan(cfg, rank, world):
                    for ref, k0, n0, n in parts:
                        assert k0 % 32 == 0 and K % 32 == 0 and k0 + K <= shapes[ref][0] and n0 + n <= shapes[ref][1]
                        cover[ref] += K * n
            for n, (k, w) in shapes.items():
                replicated = kind == "deepseek" and n in ("Wdq", "Wdkv")
                assert cover[n] == k * w * (world if replicated else 1), (n, world)


def test_two_cpu_ranks_agree_with_the_unsharded_layer():
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29611", os.path.join(HERE, "tp_cpu_worker.py")]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=240, env=env)
    assert res.returncode == 0 and "TP_CPU_OK" in res.stdout, res.stdout[-2000:] + res.stderr[-4000:]
