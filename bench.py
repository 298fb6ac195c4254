"""Decode benchmark: batch-1 greedy decode tok/s of the Qwen3-1.7B architecture on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step: one token through embed -> 28 layers -> lm_head ->
greedy pick.  The sequence is a 64-token uniform-random prompt followed by greedy
continuation; the first W steps (default 63, the prompt walk) are untimed warm-up
and the next K steps (default 2048) are timed, so the defaults time exactly the
2048 new tokens the metric names.  Weights are seeded bf16 N(0, 0.02) (norm gains
1 + N(0, 0.02)); nothing is read from disk.

One JSON line is printed by rank 0.  `value` is measured with the whole state
resident on the device (CUDA-graph replays between two CUDA events); `e2e` drives
the same captured step the way the reference's generation loop drives a model --
token id in from pinned host memory, picked token back to the host, every step.
The dense Qwen3 path does not shard ("replicas only"): with --gpus N each rank
decodes its own sequence and `value` is the sum over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

PROMPT_TOKENS = 64
METRIC = "batch-1 decode tok/s (2048 new tokens)"


def peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return json.loads(path.read_text())["hbm_gbs"], "measured"
    return 6650.0, "fallback"


def make_weights(cfg, seed=0):
    from tilefoundry_b200.authored import qwen3_1_7b as q
    from tilefoundry_b200.authored.weights import random_weights

    return q.tie_head(random_weights(q.build(cfg), seed=seed, std=0.02))


def prompt_ids(cfg, seed=0):
    return torch.randint(0, cfg.vocab_size, (PROMPT_TOKENS,), generator=torch.Generator().manual_seed(seed + 1))


class ClockSampler:
    """nvidia-smi samples of SM clock and throttle reasons while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(index), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            pass

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        out, _ = self.proc.communicate(timeout=10)
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) != 6:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[2:]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def time_kernel_gate_up(sess, reps=10):
    """Average device time of the dominant kernel (gate/up projection + SwiGLU): one launch per layer's
    weights (28 x 50 MB, far larger than L2, so every launch streams from HBM), recorded as a CUDA
    graph so host launch cost does not limit it, launched the way the step launches it (programmatic
    dependent launch), timed with CUDA events on the launching stream."""
    from tilefoundry_b200 import lib

    cfg = sess.cfg

    def launches():
        for layer in sess.layers:
            lib.gemv(layer["w_gate"], sess.hidden, sess.act, w2=layer["w_up"], gamma=layer["gamma_post"],
                     prologue=lib.NORM_CAST_THEN_GAIN, epilogue=lib.EPI_SWIGLU, eps=cfg.rms_norm_eps, pdl=True)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        launches()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        launches()
    torch.cuda.synchronize()
    for _ in range(3):
        graph.replay()
    stream = torch.cuda.current_stream()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record(stream)
    for _ in range(reps):
        graph.replay()
    end.record(stream)
    torch.cuda.synchronize()
    return start.elapsed_time(end) / (reps * len(sess.layers))      # ms per launch


def cpu_baseline(cfg, weights, prompt, steps, warm):
    """The CPU oracle (a port of the reference evaluator's arithmetic) on the host cores."""
    from oracle import evaluator, generation, qwen3_1_7b as oq
    from tilefoundry_b200.authored import qwen3_1_7b as q
    from tilefoundry_b200.runtime import DictResource

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    ref = evaluator.load(q.build(cfg), DictResource(weights), oq.make(cfg))
    run = generation.decode_ids(ref, prompt[:warm], steps)
    return {"value": steps / run["seconds"], "unit": "tok/s", "cores": threads, "kind": "port",
            "sample": f"{warm} prompt steps (untimed) then {steps} greedy decode steps of the same "
                      f"model and seed, torch CPU bf16, {threads} threads"}, run


def run_reference(args):
    """Reference arm: the reference's own CPU implementation of the path.  The reference package
    does not import here (isl/ortools missing), so this is the oracle port of its evaluator."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from tilefoundry_b200.authored import qwen3_1_7b as q

    cfg = q.QWEN3_1_7B
    steps = max(1, min(args.steps, 32))
    warm = max(1, min(args.warmup + 1, PROMPT_TOKENS))
    base, _ = cpu_baseline(cfg, make_weights(cfg), prompt_ids(cfg), steps, warm)
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": "tok/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": warm, "ms_per_step": 1e3 / base["value"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "Qwen3-1.7B architecture, batch 1, greedy decode on host cores",
                   "note": f"bounded sample: {steps} of the requested {args.steps} steps"},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_ours(args):
    import torch.distributed as dist

    from tilefoundry_b200.authored import qwen3_1_7b as q
    from tilefoundry_b200.engine.qwen3 import Qwen3Session
    from tilefoundry_b200.runtime import DictResource

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")

    cfg = q.QWEN3_1_7B
    K, W = args.steps, max(args.warmup, 3)
    weights = make_weights(cfg, seed=0)                       # same model on every rank
    prompt = prompt_ids(cfg, seed=rank)                       # its own sequence per rank
    max_ctx = max(W + K + 8, PROMPT_TOKENS + 8)
    sess = Qwen3Session(cfg, DictResource({k: v.to(dev) for k, v in weights.items()}), max_ctx=max_ctx, device=dev)
    sess.reset(prompt)
    sess.capture()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing ----------------------------------------------------------
    sess.reset(prompt)
    sess.run(W)
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    stream = torch.cuda.current_stream()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(stream)
    sess.run(K)
    end.record(stream)
    barrier()
    clocks = sampler.stop() if sampler else None
    ms = start.elapsed_time(end)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t)
    tokens_out = sess.tokens[W + 1: W + 1 + K].tolist()

    # ---- end to end: token in from pinned host memory, picked token back, every step ---------
    sess.reset(prompt)
    sess.run(W)
    pin_in = torch.empty(1, dtype=torch.int64).pin_memory()
    pin_out = torch.empty(1, dtype=torch.int64).pin_memory()
    pin_in[0] = int(sess.tokens[W])
    barrier()
    t0 = time.perf_counter()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for i in range(K):
        pos = W + i
        sess.tokens[pos: pos + 1].copy_(pin_in, non_blocking=True)         # H2D: this step's input
        sess.graph.replay()
        pin_out.copy_(sess.tokens[pos + 1: pos + 2], non_blocking=True)    # D2H: this step's result
        stream.synchronize()
        pin_in[0] = pin_out[0]
    e1.record(stream)
    barrier()
    e2e_ms = max(e0.elapsed_time(e1), (time.perf_counter() - t0) * 1e3)
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- roofline ---------------------------------------------------------------------------------
    peak, peak_kind = peaks()
    w_bytes = sess.weight_bytes()
    kv_pos = sess.kv_bytes_per_position()
    # a step at position p reads the p cached positions and its weights, writes one position
    step_bytes = [w_bytes + kv_pos * (W + i + 1) for i in range(K)]
    step_gbs = sum(step_bytes) / (ms * 1e-3) / 1e9
    k_ms = time_kernel_gate_up(sess)
    k_bytes = 2 * cfg.intermediate_size * cfg.hidden_size * 2
    k_gbs = k_bytes / (k_ms * 1e-3) / 1e9
    roofline = {
        "kernel": "gemv_kernel<SwiGLU> (post-attention norm + gate/up projection)", "bound": "hbm",
        "achieved": k_gbs, "peak": peak, "peak_kind": peak_kind + " (MEASURED_PEAKS.json hbm_gbs)" if peak_kind == "measured" else "fallback",
        "unit": "GB/s", "frac": k_gbs / peak, "traffic": None,
        "algorithmic_bytes_per_launch": k_bytes, "us_per_launch": k_ms * 1e3,
        "whole_step": {"achieved": step_gbs, "frac": step_gbs / peak,
                       "bytes_per_token_mean": sum(step_bytes) / K, "frac_of_8TBs_nominal": step_gbs / 8000.0},
    }

    base = None
    if world == 1 and not args.no_cpu:
        base, _ = cpu_baseline(cfg, weights, prompt, 32, PROMPT_TOKENS)

    line = {
        "metric": METRIC, "value": world * K / (ms * 1e-3), "unit": "tok/s", "n_gpus": world, "steps": K,
        "warmup": W, "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "Qwen3-1.7B architecture (28 layers, hidden 2048, 16q/8kv x128, SwiGLU 6144, "
                               "vocab 151936, tied head), batch 1, 64-token random prompt, greedy decode, "
                               "paged bf16 KV cache (page 64)",
                   "timed_positions": [W, W + K], "parallelism": "replicas only" if world > 1 else "1 gpu",
                   "l2": "inputs larger than L2: 3.44 GB of weights are streamed every step",
                   "first_tokens": tokens_out[:8]},
        "e2e": {"value": world * K / (e2e_ms * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": 8,
                "d2h_bytes_per_step": 8},
        "gpu_launches": sess.launches_per_step * K,
        "clocks": clocks, "roofline": roofline, "cpu_baseline": base,
    }
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2048)
    ap.add_argument("--warmup", type=int, default=PROMPT_TOKENS - 1)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
