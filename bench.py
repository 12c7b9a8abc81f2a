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


# DRAM bytes (read + write) over algorithmic bytes of one k_decode_step launch, from the ncu capture of a reduced-depth
# model of the same width (profiles/); None until a capture exists.  Traffic grows with the weights and K/V rows streamed.
DECODE_STEP_DRAM_RATIO = (742.42 + 60.54) / 737.0
DECODE_STEP_DRAM_SOURCE = "profiles/decode_step_2blocks_7bwidth_ncu.md (742.4 MB read + 60.5 MB written for 737 MB algorithmic on a 2-block model), scaled by algorithmic bytes"


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
    short context and extrapolate to the full depth.  Returns (tok/s, threads used, description, steps run)."""
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
              f"+ LM head at context <= 4, EXTRAPOLATED x{w['layers']} blocks (block {t_layer * 1e3:.1f} ms, head {t_head * 1e3:.1f} ms); "
              f"batch 1; CPU attention over the timed GPU context ({w['prompt']}+ cached positions) is NOT included, which flatters the CPU; "
              f"the reference itself re-forwards the whole context per token and is slower still")
    return 1.0 / t_token, used, sample, n


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


def timing_context(w, steps, warmup):
    """The cached context length the timed steps are centred on — what `measure_decode` arrives at: warm-up steps
    behind the prompt (rewinding to the end of the prompt when the window is full), then `steps` steps."""
    room = w["max_seq"] - w["prompt"] - 1
    pos, done = w["prompt"], 0
    while done < warmup:
        if pos >= w["max_seq"] - 1:
            pos = w["prompt"]
        k = min(warmup - done, w["max_seq"] - 1 - pos)
        pos += k
        done += k
    if pos + min(steps, room) > w["max_seq"] - 1:
        pos = w["prompt"]
    return min(pos + min(steps, room) // 2, w["max_seq"] - 3)


def workload_config(name, w, world, kv_dtype, ctx=None):
    """The `config` object of the JSON line; the reference arm prints the same keys and values."""
    return {"workload": name, "batch": w["batch"], "prompt_len": w["prompt"], "context_at_timing": ctx,
            "parallelism": f"tp{world}", "kv_cache": kv_dtype, "l2": "weights+KV per step exceed L2 (inputs larger than L2)"}


def run_reference(args, w, name):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = max(1, (os.cpu_count() or 2) - 1)      # DeepJExecutor default: cores - 1
    t0 = time.perf_counter()
    vals = []
    used, sample, ran = threads, "", 0
    for _ in range(max(1, min(args.steps, 2))):
        v, used, sample, n = cpu_decode_sample(w, threads)
        vals.append(v)
        ran += n
    v = float(np.median(vals))
    line = {
        "impl": "reference", "metric": "q8_decode_tokens_per_s", "value": v, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 / v, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        # the same keys and values as the GPU arm prints for this command line (the work is the same; it runs on the host cores)
        "config": workload_config(name, w, args.gpus, args.kv, timing_context(w, args.steps, args.warmup)),
        # value and ms_per_step are extrapolated from a bounded sample, not measured over `steps` full tokens
        "extrapolated": True, "steps_run": ran, "steps_run_what": "decode steps of 1 block + LM head at context <= 4",
        "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": used, "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "wall_s": time.perf_counter() - t0,
    }
    print(json.dumps(line), flush=True)


def measure_decode(dec, w, args, world, local_rank, tp, repeats):
    """The timed regions of one decoder whose cache already holds the prompt: `repeats` device-resident regions of
    exactly `steps` steps each (median reported, all kept), then the host-buffer loop over the same context range."""
    import ctypes
    from deepj_b200 import _lib
    lib = dec.lib
    B = dec.B
    room = w["max_seq"] - w["prompt"] - 1

    def run_device(n):
        """n steps with device feedback; when the window fills up, rewind to the end of the prompt."""
        done = 0
        while done < n:
            if dec.position >= w["max_seq"] - 1:
                dec.set_position(w["prompt"])
            k = min(n - done, w["max_seq"] - 1 - dec.position)
            dec.step_device(k, sync=False)
            done += k

    run_device(args.warmup)
    if dec.position + min(args.steps, room) > w["max_seq"] - 1:
        dec.set_position(w["prompt"])
    ctx0 = dec.position
    sampler = ClockSampler(local_rank)
    sampler.start()
    sampler.wait_ready()
    regions = []
    launches = 0
    for rep in range(repeats):
        dec.set_position(ctx0)
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
        st1 = dec.stats()
        regions.append(tp.max_over_ranks(ms.value) if world > 1 else ms.value)      # device time, max over ranks
        launches = (st1["graph_replays"] - st0["graph_replays"]) * st1["kernels_per_replay"] + (st1["eager_launches"] - st0["eager_launches"])
    clocks = sampler.stop()
    per_step = sorted(r / args.steps for r in regions)
    ms_per_step = float(np.median(per_step))

    # host-buffer loop (e2e): same context range, token ids through host memory every step
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
    ctx = min(ctx0 + min(args.steps, room) // 2, w["max_seq"] - 3)
    dec.set_position(ctx)
    return {"ms_per_step": ms_per_step, "ms_per_step_regions": per_step, "value": B * 1e3 / ms_per_step,
            "e2e": B * args.steps / e2e_s, "launches": int(launches), "clocks": clocks, "ctx": ctx, "dev_error": dec.stats()["device_error"]}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="llama7b_q8_decode_b1", choices=sorted(WORKLOADS))
    ap.add_argument("--prompt-len", type=int, default=0, help="override the prompt length (debugging)")
    ap.add_argument("--repeats", type=int, default=5, help="timed regions of `steps` steps each; the median is reported")
    ap.add_argument("--kv", default="f32", choices=["f32", "f16"], help="dtype of the K/V cache of the headline run (fp32 = the reference's precision)")
    ap.add_argument("--no-kv16", action="store_true", help="skip the fp16-K/V sub-record")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="skip the reduced-depth check against the CPU oracle")
    ap.add_argument("--no-batch16", action="store_true", help="skip the 16-sequence sub-record of the 7B workload")
    ap.add_argument("--fused-step", action="store_true", help="the single whole-token kernel (op 76) instead of one kernel per operator")
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
    batch16 = args.workload == "llama7b_q8_decode_b1" and not args.no_batch16 and args.prompt_len == 0
    # exchange slots hold a prompt chunk's partial sums (rows x dModel per exchange), capped at 2048 rows
    slot = max((16 if batch16 else B) * cfg.d_model, (16 if batch16 else B) * cfg.vocab_size // world,
               min(B * min(w["prompt"], Q8Decoder.PREFILL_CHUNK), 2048) * cfg.d_model)
    dec = Q8Decoder(cfg, batch=B, device=local_rank, tp_rank=rank, tp_world=world, tp_slot_floats=slot if world > 1 else 0,
                    fused_step=args.fused_step, kv_dtype=args.kv)
    kv16 = not args.no_kv16 and args.kv == "f32" and not args.fused_step and args.prompt_len == 0
    if world > 1:
        # weights are split by rows/columns over the ranks; [rows x d] partial sums and the logits
        # shards cross NVLink through the library's own peer-memory exchange
        tp.connect(rank, world, slot)

    # ── correctness first: the same architecture at full width, two blocks deep, against the CPU oracle ──
    parity = None
    if not args.no_parity:
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        from parity_util import reduced_depth_parity_variants
        variants = [dict(kv_dtype=args.kv, fused_step=args.fused_step)] + ([dict(kv_dtype="f16")] if kv16 else [])
        checks = reduced_depth_parity_variants(w, variants, layers=2, prompt_len=48, n_new=8, rank=rank, world=world, device=local_rank,
                                               tp_slot_floats=slot if world > 1 else 0, check_codes=False)
        parity = checks[0]
        parity16 = checks[1] if kv16 else None
        if kv16 and not (parity16["tokens_equal"] and parity16["max_err_over_range"] <= parity16["tolerance"]):
            kv16 = False          # the option does not pass its gate on this configuration: it is reported as failed, not timed
        if not (parity["tokens_equal"] and parity["max_err_over_range"] <= parity["tolerance"]):
            if rank == 0:
                print(json.dumps({"metric": "q8_decode_tokens_per_s", "error": "parity check failed", "parity": parity}), flush=True)
            raise SystemExit(3)

    t_load = time.perf_counter()
    dec.load_synthetic(w["seed"], w["std"])
    if world > 1:
        tp.barrier()          # the exchange's wait for a peer is bounded: start stepping together
    rng = np.random.default_rng(w["seed"] + 1000)
    prompts = rng.integers(0, w["vocab"], size=(B, w["prompt"]))
    dec.reset()
    t_load = time.perf_counter() - t_load
    t_prefill = time.perf_counter()
    nxt = dec.prefill(prompts)          # many-row path (tcgen05 GEMMs, chunk attention; partial sums exchanged per chunk under tensor parallelism)
    t_prefill = time.perf_counter() - t_prefill
    prefill_chunked = w["prompt"] >= 32 and (world == 1 or slot // cfg.d_model // B >= 16)

    dec.set_tokens(nxt)
    m = measure_decode(dec, w, args, world, local_rank, tp, max(1, args.repeats))
    ms_per_step, value, ctx = m["ms_per_step"], m["value"], m["ctx"]

    # ── the dominant kernels against the HBM roofline ──
    peak, peak_kind = measured_peak_gbs()
    prof = dec.profile_step()
    prof = dec.profile_step()

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
    kv_pos_bytes = cfg.kv_bytes_per_position(args.kv)
    step_bytes = cfg.q8_weight_bytes() + B * ctx * kv_pos_bytes                      # whole job, all ranks
    step_achieved = step_bytes / world / (ms_per_step * 1e-3) / 1e9                  # per GPU
    attn_bytes = B * ctx * kv_pos_bytes // world                                     # this rank's heads

    line = {
        "metric": "q8_decode_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "q8 weights, f32 activations/accumulate", "data": "synthetic",
        "config": workload_config(args.workload, w, world, args.kv, ctx),
        "timed_regions": {"count": len(m["ms_per_step_regions"]), "steps_each": args.steps, "ms_per_step_median": ms_per_step,
                          "ms_per_step_min": m["ms_per_step_regions"][0], "ms_per_step_max": m["ms_per_step_regions"][-1]},
        "e2e": {"value": m["e2e"], "unit": "tokens/s", "h2d_bytes_per_step": 4 * B, "d2h_bytes_per_step": 4 * B},
        "gpu_launches": m["launches"],
        "clocks": m["clocks"],
        "parity": parity,
        "roofline_gemv" if dec.fused_step else "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     # DRAM bytes per launch (read + write), scaled by K·N from the ncu capture of the K=4096, N=12288
                     # launch (56.869 MB measured against 56.69 MB algorithmic): the full-size step is too large to capture
                     "traffic": (gemv_bytes / max(n_gemv, 1)) * (56.826 / 56.689), "traffic_unit": "bytes per launch (average)",
                     "traffic_source": "profiles/q8_gemv_tma_k4096_n12288_ncu.md (56.709 MB read + 0.117 MB written per launch, mean of two, for 56.689 MB algorithmic), scaled by algorithmic bytes",
                     "peak_kind": peak_kind, "kernel": "k_q8_gemv_tma", "launches_per_step": n_gemv,
                     "bytes_per_step": gemv_bytes, "us_per_launch": 1e3 * gemv_stream_ms / max(n_gemv_stream, 1),
                     "ms_per_step_back_to_back": gemv_stream_ms, "ms_per_step_op_by_op": gemv_ms},
        "roofline_attention": {"bound": "hbm", "kernel": "k_attn_decode", "launches_per_step": n_attn,
                               "bytes_per_step": attn_bytes, "ms_per_step_back_to_back": attn_stream_ms,
                               "achieved": attn_bytes / max(attn_stream_ms * 1e-3, 1e-12) / 1e9, "peak": peak, "unit": "GB/s",
                               "frac": attn_bytes / max(attn_stream_ms * 1e-3, 1e-12) / 1e9 / peak},
        "roofline_step": {"bytes_per_token": step_bytes, "achieved_per_gpu": step_achieved, "frac": step_achieved / peak,
                          "roofline_tokens_per_s": B * world * peak * 1e9 / step_bytes},
        "profile_ms": {"gemv": gemv_ms, "attention": attn_ms, "exchange": exch_ms, "all_ops": total_prof_ms},
        "device_error": m["dev_error"],
        "setup_s": t_load,
        "prefill": {"tokens": int(B * w["prompt"]), "seconds": t_prefill, "tokens_per_s": B * w["prompt"] / max(t_prefill, 1e-9),
                    "path": "chunked, many-row kernels" if prefill_chunked else "one decode step per position"},
    }

    if dec.fused_step:
        # the step is ONE launch of the whole-token kernel: its algorithmic bytes are this GPU's share of the Q8 weights and of
        # the K/V rows of the timed context, its launch duration the device time per step (CUDA events over the timed regions)
        line["roofline"] = {"bound": "hbm", "kernel": "k_decode_step", "launches_per_step": 1, "achieved": step_achieved, "peak": peak,
                            "unit": "GB/s", "frac": step_achieved / peak, "peak_kind": peak_kind, "bytes_per_launch": step_bytes / world,
                            "us_per_launch": 1e3 * ms_per_step,
                            "traffic": (step_bytes / world) * DECODE_STEP_DRAM_RATIO if DECODE_STEP_DRAM_RATIO else None,
                            "traffic_unit": "bytes per launch", "traffic_source": DECODE_STEP_DRAM_SOURCE}
        line["step_kernel"] = "k_decode_step: one cooperative launch per token (op 76)"
    else:
        line["step_kernel"] = "one kernel per operator, CUDA-graph replay"

    # ── the same step with the K/V cache in fp16 (an option behind the same parity gate; the headline stays at the reference's fp32) ──
    if not args.no_parity and not args.no_kv16 and args.kv == "f32" and not args.fused_step and args.prompt_len == 0:
        line["kv_f16"] = {"parity": parity16}
    if kv16 and not args.no_parity:
        d16 = Q8Decoder(cfg, batch=B, device=local_rank, id_base=6 << 24, tp_rank=rank, tp_world=world,
                        tp_slot_floats=slot if world > 1 else 0, share_weights=dec, kv_dtype="f16")
        if world > 1:
            tp.barrier()
        d16.reset()
        nx = d16.prefill(prompts)
        d16.set_tokens(nx)
        mk = measure_decode(d16, w, args, world, local_rank, tp, max(1, min(args.repeats, 3)))
        bk = cfg.q8_weight_bytes() + B * mk["ctx"] * cfg.kv_bytes_per_position("f16")
        ak = bk / world / (mk["ms_per_step"] * 1e-3) / 1e9
        line["kv_f16"].update({"value": mk["value"], "unit": "tokens/s", "ms_per_step": mk["ms_per_step"], "ms_per_step_regions": mk["ms_per_step_regions"],
                               "e2e": {"value": mk["e2e"], "unit": "tokens/s", "h2d_bytes_per_step": 4 * B, "d2h_bytes_per_step": 4 * B},
                               "roofline_step": {"bytes_per_token": bk, "achieved_per_gpu": ak, "frac": ak / peak,
                                                 "roofline_tokens_per_s": B * world * peak * 1e9 / bk},
                               "device_error": mk["dev_error"]})
        d16.close()

    # ── the same model at 16 concurrent sequences (BASELINE configs[4] asks for 1 and 16), sharing the weights ──
    fail16 = False
    if batch16:
        w16 = dict(WORKLOADS["llama7b_q8_decode_b16"])
        dec16 = Q8Decoder(cfg, batch=16, device=local_rank, id_base=5 << 24, tp_rank=rank, tp_world=world,
                          tp_slot_floats=slot if world > 1 else 0, share_weights=dec)
        if world > 1:
            tp.barrier()
        p16 = np.random.default_rng(w16["seed"] + 1016).integers(0, w16["vocab"], size=(16, w16["prompt"]))
        dec16.reset()
        t16 = time.perf_counter()
        nxt16 = dec16.prefill(p16)
        t16 = time.perf_counter() - t16
        par16 = None
        if not args.no_parity:
            # full-depth check of the several-row kernels: sequence 0 of the batch against the same prompt decoded alone
            # (single-row kernels, themselves held to the oracle above), logits of the prompt's last token and of four
            # teacher-forced steps
            dec.reset()
            n1 = dec.prefill(p16[:1])
            rows1, rows16, toks1, toks16 = [dec.logits()[0].copy()], [dec16.logits()[0].copy()], [int(n1[0])], [int(nxt16[0])]
            for _ in range(4):
                fed = np.asarray(nxt16[:1]).copy()           # both decoders get the batch's own pick for sequence 0
                nxt16 = dec16.step(nxt16)
                n1 = dec.step(fed)
                rows1.append(dec.logits()[0].copy()); rows16.append(dec16.logits()[0].copy())
                toks1.append(int(n1[0])); toks16.append(int(nxt16[0]))
            r1, r16 = np.stack(rows1), np.stack(rows16)
            err16 = float(np.abs(r1 - r16).max()) / float(r1.max() - r1.min())
            par16 = {"max_err_over_range": err16, "tokens_equal": toks1 == toks16, "tolerance": 2e-3,
                     "checked": f"all {cfg.n_layers} blocks, 16 sequences at context {w16['prompt']}: sequence 0's logits after the prompt and after "
                                "four steps vs the same prompt decoded alone (single-row kernels)"}
        dec16.set_tokens(nxt16)
        m16 = measure_decode(dec16, w16, args, world, local_rank, tp, max(1, min(args.repeats, 3)))
        prof16 = dec16.profile_step()
        prof16 = dec16.profile_step()
        by_label = {}
        for lbl, t in prof16:
            by_label[lbl] = by_label.get(lbl, 0.0) + t
        bytes16 = cfg.q8_weight_bytes() + 16 * m16["ctx"] * kv_pos_bytes
        ach16 = bytes16 / world / (m16["ms_per_step"] * 1e-3) / 1e9
        line["batch16"] = {
            "workload": "llama7b_q8_decode_b16", "value": m16["value"], "unit": "tokens/s", "ms_per_step": m16["ms_per_step"],
            "ms_per_step_regions": m16["ms_per_step_regions"], "context_at_timing": m16["ctx"],
            "e2e": {"value": m16["e2e"], "unit": "tokens/s", "h2d_bytes_per_step": 64, "d2h_bytes_per_step": 64},
            "roofline_step": {"bytes_per_step": bytes16, "achieved_per_gpu": ach16, "frac": ach16 / peak,
                              "roofline_tokens_per_s": 16 * world * peak * 1e9 / bytes16},
            "gpu_launches": m16["launches"], "device_error": m16["dev_error"],
            "prefill": {"tokens": 16 * w16["prompt"], "seconds": t16},
            "profile_ms_op_by_op": by_label,
        }
        if par16 is not None:
            line["batch16"]["parity_vs_single_sequence"] = par16
            if not (par16["tokens_equal"] and par16["max_err_over_range"] <= par16["tolerance"]):
                line["batch16"]["error"] = "parity check failed: the timings of this sub-record do not count"
                fail16 = True
        dec16.close()
        if kv16 and not args.no_parity:
            # … and with the fp16 K/V cache (16 sequences read 16 caches per step: the K/V rows are most of the bytes)
            dec16h = Q8Decoder(cfg, batch=16, device=local_rank, id_base=7 << 24, tp_rank=rank, tp_world=world,
                               tp_slot_floats=slot if world > 1 else 0, share_weights=dec, kv_dtype="f16")
            if world > 1:
                tp.barrier()
            dec16h.reset()
            nxt16 = dec16h.prefill(p16)
            dec16h.set_tokens(nxt16)
            m16h = measure_decode(dec16h, w16, args, world, local_rank, tp, max(1, min(args.repeats, 3)))
            b16h = cfg.q8_weight_bytes() + 16 * m16h["ctx"] * cfg.kv_bytes_per_position("f16")
            a16h = b16h / world / (m16h["ms_per_step"] * 1e-3) / 1e9
            line["batch16"]["kv_f16"] = {"value": m16h["value"], "unit": "tokens/s", "ms_per_step": m16h["ms_per_step"],
                                         "e2e": {"value": m16h["e2e"], "unit": "tokens/s", "h2d_bytes_per_step": 64, "d2h_bytes_per_step": 64},
                                         "roofline_step": {"bytes_per_step": b16h, "achieved_per_gpu": a16h, "frac": a16h / peak,
                                                           "roofline_tokens_per_s": 16 * world * peak * 1e9 / b16h},
                                         "device_error": m16h["dev_error"]}
            dec16h.close()

    if not args.no_cpu_baseline and rank == 0:
        v, used, sample, _ = cpu_decode_sample(w, max(1, (os.cpu_count() or 2) - 1))
        line["cpu_baseline"] = {"value": v, "unit": "tokens/s", "cores": used, "kind": "port", "sample": sample, "extrapolated": True}
        if w["d"] <= 256:      # the tiny configuration: also the reference-faithful loop, full re-forward per token
            line["cpu_baseline"]["full_reforward_tokens_per_s"] = cpu_full_reforward_sample(w, used)
    if rank == 0:
        print(json.dumps(line), flush=True)
    dec.close()
    if world > 1:
        tp.disconnect()
    if fail16:
        raise SystemExit(3)


if __name__ == "__main__":
    main()
