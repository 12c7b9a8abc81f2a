#!/usr/bin/env python
"""Q8 decode throughput of the Llama-7B-shaped configuration on B200.

One "step" = one greedy decode step (one new token per sequence) of the Q8 decoder
through `deepj_cuda_flush_ops`, with the KV cache already holding the prompt.

  value      tokens/s with the token fed back on the device (inputs resident in HBM),
             timed with CUDA events on the library's stream.
  e2e        tokens/s through the host-buffer call: every step uploads the token ids
             from host memory, flushes synchronously and downloads the picked ids.
  roofline   the Q8 GEMV kernel: algorithmic bytes of every GEMV launch of one step ÷
             their summed device time (op-by-op CUDA-event profile of the same step).
  cpu_baseline / --impl reference: the CPU oracle's KV-cached decode of the same
             configuration on the host cores, on a bounded sample (see `sample`).

Synthetic data: random-init weights of the named architecture (device-side
counter-based generator, N(0,0.02)-like), uniform random prompt ids.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # BASELINE configs[4]: Llama-7B shape, 2048-token prompts, 128 generated tokens
    "llama7b_q8_decode_b1": dict(kind="llama", vocab=32000, d=4096, heads=32, layers=32, d_ff=11008, max_seq=2176,
                                 prompt=2048, batch=1, seed=9, std=0.02),
    "llama7b_q8_decode_b16": dict(kind="llama", vocab=32000, d=4096, heads=32, layers=32, d_ff=11008, max_seq=2176,
                                  prompt=2048, batch=16, seed=9, std=0.02),
    # BASELINE configs[2]: Llama-1B shape
    "llama1b_q8_decode_b1": dict(kind="llama", vocab=32000, d=2048, heads=32, layers=22, d_ff=5632, max_seq=768,
                                 prompt=512, batch=1, seed=3, std=0.02),
    # BASELINE configs[3]: DeepSeek shape (qRank = dModel/2 assumed)
    "deepseek_q8_decode_b1": dict(kind="deepseek", vocab=32000, d=2048, heads=16, layers=16, d_ff=5632, max_seq=1280,
                                  prompt=1024, batch=1, seed=5, std=0.02, q_rank=1024, kv_rank=512),
    # the GPT family at GPT-2 XL's shape (not a BASELINE config: the fused LayerNorm / GELU projections at speed)
    "gpt2xl_q8_decode_b1": dict(kind="gpt", vocab=50257, d=1600, heads=25, layers=48, d_ff=6400, max_seq=1024,
                                prompt=512, batch=1, seed=11, std=0.02),
    # BASELINE configs[0]: tiny Llama (latency-bound; no roofline claim)
    "tiny_llama_q8_decode_b1": dict(kind="llama", vocab=256, d=256, heads=8, layers=4, d_ff=688, max_seq=256,
                                    prompt=32, batch=1, seed=42, std=0.1),
}


def measured_peak_gbs():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples during the timed region."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.tmp = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "20", "-i", str(self.idx)], stdout=self.tmp, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def wait_ready(self, timeout_s: float = 3.0):
        """nvidia-smi takes a moment to come up (longer on a box with many GPUs): hold the timed region back until
        its first sample is in the file."""
        if self.proc is None:
            return
        t0 = time.perf_counter()
        while time.perf_counter() - t0 < timeout_s:
            try:
                if os.path.getsize(self.tmp.name) > 0:
                    return
            except OSError:
                return
            time.sleep(0.02)

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.tmp.flush()
        self.tmp.seek(0)
        sm, smax, reasons = [], [], set()
        for line in self.tmp.read().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); smax.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.tmp.name)
        if sm:
            out.update(sm_mhz=float(np.median(sm)), sm_max_mhz=float(max(smax)), reasons=sorted(reasons), samples=len(sm))
        return out


def cpu_decode_sample(w, threads: int):
    """CPU oracle, KV-cached decode of workload `w`: time one block + the LM head at a
    short context and extrapolate to the full depth.  Returns (tok/s, description)."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle
    oracle.lib().oracle_set_threads(threads)
    used = oracle.lib().oracle_get_threads()
    built = 1
    om = oracle.OracleModel(w["kind"], w["vocab"], 8, w["d"], w["heads"], w["layers"], w["d_ff"],
                            w.get("q_rank", 0), w.get("kv_rank", 0), seed=w["seed"], init_mode=1, std=w["std"],
                            layers_built=built)
    rng = np.random.default_rng(w["seed"] + 1000)
    toks = rng.integers(0, w["vocab"], size=8)
    om.reset_cache()
    om.decode_step(int(toks[0]))                     # warm the pages
    t0 = time.perf_counter()
    n = 3
    for i in range(n):
        om.decode_step(int(toks[1 + i]))
    t_layer_head = (time.perf_counter() - t0) / n
    x = rng.standard_normal((1, w["d"])).astype(np.float32)
    Wlm = om.weight("Wlm").reshape(w["d"], w["vocab"])
    oracle.matmul(x, Wlm)
    t0 = time.perf_counter()
    for i in range(n):
        oracle.matmul(x, Wlm)
    t_head = (time.perf_counter() - t0) / n
    t_layer = max(t_layer_head - t_head, 1e-9)
    t_token = t_layer * w["layers"] + t_head
    sample = (f"C++ restatement of CpuBackend, KV-cached decode, fp32 weights: {n} steps of {built} of {w['layers']} blocks "
              f"+ LM head at context <= 4, extrapolated x{w['layers']} blocks (block {t_layer * 1e3:.1f} ms, head {t_head * 1e3:.1f} ms); "
              f"batch 1; the reference itself re-forwards the whole context per token and is slower still")
    return 1.0 / t_token, used, sample


def cpu_full_reforward_sample(w, threads: int, n_new: int = 8):
    """The reference's own generation loop on the CPU oracle: every new token re-forwards the whole
    context (models/TextGenerator.java:91-100), fp32 weights.  Only for shapes a CPU finishes in seconds."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle
    oracle.lib().oracle_set_threads(threads)
    om = oracle.OracleModel(w["kind"], w["vocab"], w["max_seq"], w["d"], w["heads"], w["layers"], w["d_ff"],
                            w.get("q_rank", 0), w.get("kv_rank", 0), seed=w["seed"], init_mode=1, std=w["std"])
    prompt = list(np.random.default_rng(w["seed"] + 1000).integers(0, w["vocab"], size=w["prompt"]))
    t0 = time.perf_counter()
    om.generate_greedy(prompt, n_new, use_cache=False)
    return n_new / (time.perf_counter() - t0)


def run_reference(args, w, name):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = max(1, (os.cpu_count() or 2) - 1)      # DeepJExecutor default: cores - 1
    t0 = time.perf_counter()
    vals = []
    used, sample = threads, ""
    for _ in range(max(1, min(args.steps, 2))):
        v, used, sample = cpu_decode_sample(w, threads)
        vals.append(v)
    v = float(np.median(vals)) * w["batch"] / w["batch"]
    line = {
        "impl": "reference", "metric": "q8_decode_tokens_per_s", "value": v, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 / v, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": name, "parallelism": "cpu"},
        "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": used, "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "wall_s": time.perf_counter() - t0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="llama7b_q8_decode_b1", choices=sorted(WORKLOADS))
    ap.add_argument("--prompt-len", type=int, default=0, help="override the prompt length (debugging)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    w = dict(WORKLOADS[args.workload])
    if args.prompt_len > 0:
        w["prompt"] = args.prompt_len
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args, w, args.workload)
        return

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world:
        if args.gpus == 1 and world == 1:
            pass
        else:
            raise SystemExit(f"--gpus {args.gpus} needs torchrun with {args.gpus} ranks (WORLD_SIZE={world})")
    from deepj_b200.decoder import DecoderConfig, Q8Decoder
    from deepj_b200 import tp
    if world > 1:
        tp.init_process_group()

    cfg = DecoderConfig(w["kind"], w["vocab"], w["max_seq"], w["d"], w["heads"], w["layers"], w["d_ff"],
                        w.get("q_rank", 0), w.get("kv_rank", 0))
    B = w["batch"]
    room = w["max_seq"] - w["prompt"] - 1          # decode steps that fit behind the prompt
    if room < 8:
        raise SystemExit("the context window of this workload leaves no room to decode")
    # exchange slots sized for a prompt chunk (rows x d partial sums per exchange), capped at 64 MB per slot.  The chunked
    # tensor-parallel prompt pass has been run on 2 GPUs only; larger worlds take one decode step per prompt position
    # (measured on 4 and 8 GPUs) unless DEEPJ_BENCH_TP_CHUNKED=1 asks for chunks there too.
    slot = max(B * cfg.d_model, B * cfg.vocab_size // world)
    if world == 2 or os.environ.get("DEEPJ_BENCH_TP_CHUNKED") == "1":
        slot = max(slot, min(B * min(w["prompt"], Q8Decoder.PREFILL_CHUNK) * cfg.d_model, 16 << 20))
    dec = Q8Decoder(cfg, batch=B, device=local_rank, tp_rank=rank, tp_world=world, tp_slot_floats=slot if world > 1 else 0)
    if world > 1:
        # weights are split by rows/columns over the ranks; [rows x d] partial sums and the logits
        # shards cross NVLink through the library's own peer-memory exchange kernel
        tp.connect(rank, world, slot)
    t_load = time.perf_counter()
    dec.load_synthetic(w["seed"], w["std"])
    if world > 1:
        tp.barrier()          # the exchange kernel's wait for a peer is bounded: start stepping together
    rng = np.random.default_rng(w["seed"] + 1000)
    prompts = rng.integers(0, w["vocab"], size=(B, w["prompt"]))
    dec.reset()
    t_load = time.perf_counter() - t_load
    t_prefill = time.perf_counter()
    nxt = dec.prefill(prompts)          # many-row path (tcgen05 GEMMs, chunk attention; partial sums exchanged per chunk under tensor parallelism)
    t_prefill = time.perf_counter() - t_prefill

    lib = dec.lib
    from deepj_b200 import _lib
    import ctypes

    def run_device(n):
        """n steps with device feedback; when the window fills up, rewind to the end of the prompt."""
        done = 0
        while done < n:
            if dec.position >= w["max_seq"] - 1:
                dec.set_position(w["prompt"])
            k = min(n - done, w["max_seq"] - 1 - dec.position)
            dec.step_device(k, sync=False)
            done += k

    # ── device-resident loop (value) ──
    dec.set_tokens(nxt)
    run_device(args.warmup)
    if dec.position + min(args.steps, room) > w["max_seq"] - 1:
        dec.set_position(w["prompt"])
    ctx0 = dec.position
    sampler = ClockSampler(local_rank)
    sampler.start()
    sampler.wait_ready()
    _lib.check(lib.deepj_cuda_synchronize())
    if world > 1:
        tp.barrier()
    st0 = dec.stats()
    _lib.check(lib.deepj_cuda_timer_begin())
    run_device(args.steps)
    ms = ctypes.c_float(0)
    _lib.check(lib.deepj_cuda_timer_end(ctypes.byref(ms)))
    _lib.check(lib.deepj_cuda_synchronize())
    if world > 1:
        tp.barrier()
    clocks = sampler.stop()
    st1 = dec.stats()
    elapsed_ms = tp.max_over_ranks(ms.value) if world > 1 else ms.value      # device time, max over ranks
    ms_per_step = elapsed_ms / args.steps
    value = B * 1e3 / ms_per_step
    launches = (st1["graph_replays"] - st0["graph_replays"]) * st1["kernels_per_replay"] + (st1["eager_launches"] - st0["eager_launches"])

    # ── host-buffer loop (e2e): same context range, token ids through host memory every step ──
    tok = dec.next_tokens()
    dec.set_position(ctx0)
    for _ in range(3):
        tok = dec.step(tok)
    dec.set_position(ctx0)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        if dec.position >= w["max_seq"] - 1:
            dec.set_position(w["prompt"])
        tok = dec.step(tok)
    e2e_s = time.perf_counter() - t0
    if world > 1:
        e2e_s = tp.max_over_ranks(e2e_s)
    e2e = B * args.steps / e2e_s
    dec.set_position(min(ctx0 + min(args.steps, room) // 2, w["max_seq"] - 3))

    # ── the GEMV kernel against the HBM roofline ──
    peak, peak_kind = measured_peak_gbs()
    prof = dec.profile_step()
    prof = dec.profile_step()
    shapes = {n: (k, n_) for n, k, n_ in cfg.matmul_shapes()}

    def q8b(k, n):
        return k * n + ((k + 31) // 32) * n * 4
    d = cfg.d_model
    dl, Fl, Vl = d // world, cfg.d_ff // world, cfg.vocab_size // world      # this rank's shard
    op_bytes = {"qkv": q8b(d, 3 * dl) + 4 * B * (d + 3 * dl), "wo": q8b(dl, d) + 4 * B * (dl + 2 * d),
                "swiglu": 2 * q8b(d, Fl) + 4 * B * (d + Fl), "down": q8b(Fl, d) + 4 * B * (Fl + 2 * d),
                "lm_head": q8b(d, Vl) + 4 * B * (d + Vl)}
    if cfg.kind == "gpt":
        F = cfg.d_ff
        op_bytes = {"qkv": q8b(d, 3 * d) + 4 * B * (d + 3 * d), "wo": q8b(d, d) + 4 * B * (d + 2 * d), "ffn_up": q8b(d, F) + 4 * B * (d + F),
                    "ffn_down": q8b(F, d) + 4 * B * (F + 2 * d), "lm_head": q8b(d, Vl) + 4 * B * (d + Vl)}
    if cfg.kind == "deepseek":
        r = cfg.q_rank + cfg.kv_rank
        op_bytes.update({"mla_down": q8b(d, r) + 4 * B * (d + r), "mla_up_q": q8b(cfg.q_rank, dl) + 4 * B * (cfg.q_rank + dl),
                         "mla_up_kv": q8b(cfg.kv_rank, 2 * dl) + 4 * B * (cfg.kv_rank + 2 * dl)})
    gemv_ms = sum(t for lbl, t in prof if lbl in op_bytes)
    gemv_bytes = sum(op_bytes[lbl] for lbl, _ in prof if lbl in op_bytes)
    n_gemv = sum(1 for lbl, _ in prof if lbl in op_bytes)
    attn_ms = sum(t for lbl, t in prof if lbl == "attn")
    exch_ms = sum(t for lbl, t in prof if lbl in ("allreduce", "allgather"))
    total_prof_ms = sum(t for _, t in prof)
    # the same kernels back to back as their own graph-replayed stream: this is the launch duration the
    # roofline line uses (the op-by-op profile adds an event and a drained pipeline to every launch)
    gemv_stream_ms, n_gemv_stream = dec.time_ops(set(op_bytes), iters=10)
    attn_stream_ms, n_attn = dec.time_ops({"attn"}, iters=10)
    if world > 1:
        gemv_stream_ms = tp.max_over_ranks(gemv_stream_ms)
        attn_stream_ms = tp.max_over_ranks(attn_stream_ms)
    achieved = gemv_bytes / (gemv_stream_ms * 1e-3) / 1e9
    ctx = min(ctx0 + min(args.steps, room) // 2, w["max_seq"] - 3)
    step_bytes = cfg.q8_weight_bytes() + B * ctx * cfg.kv_bytes_per_position()      # whole job, all ranks
    step_achieved = step_bytes / world / (ms_per_step * 1e-3) / 1e9                  # per GPU
    attn_bytes = B * ctx * cfg.kv_bytes_per_position() // world                      # this rank's heads

    line = {
        "metric": "q8_decode_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "q8 weights, f32 activations/accumulate", "data": "synthetic",
        "config": {"workload": args.workload, "batch": B, "prompt_len": w["prompt"], "context_at_timing": ctx,
                   "parallelism": f"tp{world}", "kv_cache": "f32", "l2": "weights+KV per step exceed L2 (inputs larger than L2)"},
        "e2e": {"value": e2e, "unit": "tokens/s", "h2d_bytes_per_step": 4 * B, "d2h_bytes_per_step": 4 * B},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     # DRAM bytes per launch (read + write), scaled by K·N from the ncu capture of the K=4096, N=12288
                     # launch (56.869 MB measured against 56.69 MB algorithmic): the full-size step is too large to capture
                     "traffic": (gemv_bytes / max(n_gemv, 1)) * (56.869 / 56.69), "traffic_unit": "bytes per launch (average)",
                     "traffic_source": "profiles/q8_gemv_i8_k4096_n12288_ncu.md, scaled by algorithmic bytes",
                     "peak_kind": peak_kind, "kernel": "k_q8_gemv", "launches_per_step": n_gemv,
                     "bytes_per_step": gemv_bytes, "us_per_launch": 1e3 * gemv_stream_ms / max(n_gemv_stream, 1),
                     "ms_per_step_back_to_back": gemv_stream_ms, "ms_per_step_op_by_op": gemv_ms},
        "roofline_attention": {"bound": "hbm", "kernel": "k_attn_decode", "launches_per_step": n_attn,
                               "bytes_per_step": attn_bytes, "ms_per_step_back_to_back": attn_stream_ms,
                               "achieved": attn_bytes / max(attn_stream_ms * 1e-3, 1e-12) / 1e9, "peak": peak, "unit": "GB/s",
                               "frac": attn_bytes / max(attn_stream_ms * 1e-3, 1e-12) / 1e9 / peak},
        "roofline_step": {"bytes_per_token": step_bytes, "achieved_per_gpu": step_achieved, "frac": step_achieved / peak,
                          "roofline_tokens_per_s": B * world * peak * 1e9 / step_bytes},
        "profile_ms": {"gemv": gemv_ms, "attention": attn_ms, "exchange": exch_ms, "all_ops": total_prof_ms},
        "setup_s": t_load,
        "prefill": {"tokens": int(B * w["prompt"]), "seconds": t_prefill, "tokens_per_s": B * w["prompt"] / max(t_prefill, 1e-9),
                    "path": "chunked, many-row kernels" if w["prompt"] >= 32 and (world == 1 or slot >= 16 * B * cfg.d_model) else "one decode step per position"},
    }
    if not args.no_cpu_baseline and rank == 0:
        v, used, sample = cpu_decode_sample(w, max(1, (os.cpu_count() or 2) - 1))
        line["cpu_baseline"] = {"value": v, "unit": "tokens/s", "cores": used, "kind": "port", "sample": sample}
        if w["d"] <= 256:      # the tiny configuration: also the reference-faithful loop, full re-forward per token
            line["cpu_baseline"]["full_reforward_tokens_per_s"] = cpu_full_reforward_sample(w, used)
    if rank == 0:
        print(json.dumps(line), flush=True)
    dec.close()
    if world > 1:
        tp.disconnect()


if __name__ == "__main__":
    main()
