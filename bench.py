"""Decode benchmark: batch-1 greedy decode tok/s of the Qwen3-1.7B architecture on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step: one token through embed -> 28 layers -> lm_head ->
greedy pick.  The sequence is a 64-token uniform-random prompt followed by greedy
continuation; the prompt walk (63 steps) and W further decode steps (default 3) are
untimed warm-up and the next K steps (default 2048) are timed, so the defaults time
the 2048 new tokens the metric names.  Weights are seeded bf16 N(0, 0.02) (norm gains
1 + N(0, 0.02)); nothing is read from disk.

One JSON line is printed by rank 0.  `value` is measured with the whole state
resident on the device (CUDA-graph replays between two CUDA events); `e2e` drives
the same captured step the way the reference's generation loop drives a model --
token id in from pinned host memory, picked token back to the host, every step.
The dense Qwen3 path does not shard ("replicas only"): with --gpus N each rank
decodes its own sequence and `value` is the sum over ranks.

Side modes, each printing one JSON line that is not the metric: --config (the other
three architectures), --batch B (B sequences per step), --batch32-projection,
--moe-batch T (the Qwen3.5 expert block for T tokens at once), --profile-layers /
--dominant-only (the small cases profiler captures run).
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


class Workload:
    """One benchmark configuration: how to build the authored Module, the session, the oracle."""

    def __init__(self, key):
        self.key = key
        self.dtype = "bf16"                      # the arithmetic type of the path: bf16 storage, f32 accumulation
        if key == "qwen3_1_7b":
            from tilefoundry_b200.authored import qwen3_1_7b as a
            from tilefoundry_b200.engine.qwen3 import Qwen3Session as S
            self.authored, self.cfg, self.session_cls, self.overrides = a, a.QWEN3_1_7B, S, None
            self.describe = ("Qwen3-1.7B architecture (28 layers, hidden 2048, 16q/8kv x128, SwiGLU 6144, vocab "
                             "151936, tied head), batch 1, 64-token random prompt, greedy decode, paged bf16 KV "
                             "cache (page 64)")
            self.oracle_name, self.cpu_layers = "qwen3_1_7b", None
        elif key == "minicpm3_4b":
            from tilefoundry_b200.authored import minicpm3_4b as a
            from tilefoundry_b200.engine.minicpm3 import MiniCPM3Session as S
            self.authored, self.cfg, self.session_cls, self.overrides = a, a.MINICPM3_4B, S, None
            self.describe = ("MiniCPM3-4B architecture (62 layers, hidden 2560, 40 heads, MLA q_lora 768 / kv_lora "
                             "256, nope 64 + rope 32, v 64, SwiGLU 6400, vocab 73448), batch 1, 64-token random "
                             "prompt, greedy decode, paged bf16 cache of latents (kv_lora 256 + rope 32 per position), kv_b absorbed")
            self.oracle_name, self.cpu_layers = "minicpm3_4b", 8
        elif key == "granite_4_0_h_small":
            from tilefoundry_b200.authored import granite_4_0_h_small as a
            from tilefoundry_b200.engine.granite import GraniteSession as S
            self.authored, self.cfg, self.session_cls, self.overrides = a, a.GRANITE_4_0_H_SMALL, S, a.weight_overrides
            self.describe = ("granite-4.0-h-small architecture (36 Mamba-2 + 4 attention layers, hidden 4096, MoE 72 "
                             "experts top-10 + shared expert, vocab 100352), batch 1, 64-token random prompt, greedy "
                             "decode, f32 recurrent state in place, paged bf16 KV for the attention layers")
            self.oracle_name, self.cpu_layers = "granite_4_0_h_small", 3
        elif key == "qwen3_5_35b_a3b":
            from tilefoundry_b200.authored import qwen3_5_35b_a3b as a
            from tilefoundry_b200.engine.qwen3_5 import Qwen35Session as S
            self.authored, self.cfg, self.session_cls, self.overrides = a, a.QWEN3_5_35B_A3B, S, a.weight_overrides
            self.describe = ("Qwen3.5-35B-A3B architecture (30 Gated DeltaNet + 10 gated-attention layers, hidden 2048, "
                             "MoE 256 experts top-8 + gated shared expert, vocab 248320), f32 activations and state, "
                             "bf16 contracted weights, batch 1, 64-token random prompt, greedy decode, paged f32 KV "
                             "for the attention layers")
            self.oracle_name, self.cpu_layers = "qwen3_5_35b_a3b", 4
            self.dtype = "f32 activations/state, bf16 weights and products"
        else:
            raise SystemExit(f"unknown --config {key!r}")

    def module(self, cfg=None):
        return self.authored.build(self.cfg if cfg is None else cfg)

    def host_weights(self, cfg=None, seed=0):
        from tilefoundry_b200.authored.weights import random_weights

        w = random_weights(self.module(cfg), seed=seed, std=0.02, overrides=self.overrides)
        return self.authored.tie_head(w) if hasattr(self.authored, "tie_head") else w

    def device_weights(self, dev, seed=0):
        from tilefoundry_b200.authored.weights import random_weights_on

        tied = hasattr(self.authored, "tie_head")
        w = random_weights_on(self.module(), dev, seed=seed, std=0.02, overrides=self.overrides,
                              skip=("w_head",) if tied else ())
        if tied:
            w["w_head"] = w["w_embed"].t()          # a view: the session recognises the tie and shares the table
        return w

    def oracle(self, cfg, weights):
        import importlib

        from oracle import evaluator
        from tilefoundry_b200.runtime import DictResource

        impl = importlib.import_module(f"oracle.{self.oracle_name}").make(cfg)
        return evaluator.load(self.module(cfg), DictResource(weights), impl)

    def truncated(self):
        """The same architecture with fewer layers, for a CPU baseline that fits host memory and time."""
        import dataclasses

        if self.cpu_layers is None:
            return self.cfg, 1.0
        kw = {"num_hidden_layers": self.cpu_layers}
        if self.key == "qwen3_5_35b_a3b":
            kw = {"n_layers": self.cpu_layers}               # one 3 : 1 cycle of the layer pattern
        if self.key == "granite_4_0_h_small":
            kw["attention_layers"] = (self.cpu_layers - 1,)
        small = dataclasses.replace(self.cfg, **kw)
        return small, self.cfg.num_hidden_layers / self.cpu_layers


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


def _graph_time(launches, n_launches, reps=10):
    """ms per launch of *launches()* recorded as one CUDA graph (host launch cost excluded), CUDA events on
    the launching stream."""
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
    return start.elapsed_time(end) / (reps * n_launches)


#: dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel from one ncu capture
#: (profiles/qwen3_step_kernel_qwen3_1_7b.md: the one-launch step at context 1087: 3.569 GB read + 20.1 MB written);
#: None where no capture was taken for that configuration.
NCU_TRAFFIC = {"qwen3_1_7b": 3569151000 + 20059392}


def dominant_kernel(work, sess):
    """(name, ms per launch, algorithmic bytes per launch) of the projection that moves the most bytes per
    layer, launched over every layer's weights in turn (far more than L2), the way the step launches it."""
    from tilefoundry_b200 import lib

    cfg = sess.cfg
    if getattr(sess, "fused", False):
        # the whole step is ONE kernel: time it alone, the position word parked at the mean context of the run
        saved = sess.snapshot()
        sess.pos.fill_(PROMPT_TOKENS - 1 + NEW_TOKENS // 2)

        def launches():
            sess.step()
            sess.pos.fill_(PROMPT_TOKENS - 1 + NEW_TOKENS // 2)       # (a memset node: the kernel advanced it)
        ms = _graph_time(launches, 1)
        sess.restore(saved)
        sess.check_status()
        nbytes = sess.weight_bytes() + sess.kv_bytes_per_position() * (PROMPT_TOKENS + NEW_TOKENS // 2)
        return ("qwen3_step_kernel (the whole decode step as one cooperative launch, at the run's mean context)", ms, nbytes)
    if work.key in ("qwen3_1_7b", "minicpm3_4b"):
        def launches():
            for layer in sess.layers:
                lib.gemv(layer["w_gate"], sess.hidden, sess.act, w2=layer["w_up"], gamma=layer["gamma_post"],
                         prologue=lib.NORM_CAST_THEN_GAIN, epilogue=lib.EPI_SWIGLU, eps=cfg.rms_norm_eps, pdl=True)
        nbytes = 2 * cfg.intermediate_size * cfg.hidden_size * 2
        return ("gemv_persist_kernel<SwiGLU> (post-attention norm + gate/up projection)",
                _graph_time(launches, len(sess.layers)), nbytes)
    if work.key == "qwen3_5_35b_a3b":
        import ctypes as C
        gdn = [l for l in sess.layers if l["kind"] == "linear_attention"]
        n = cfg.conv_dim + cfg.val_dim + 2 * cfg.gdn_n_v_heads
        calls = [lib.GemvF32Args(w=lib.ptr(l["w_in"]), x=lib.ptr(sess.hidden), gamma=lib.ptr(l["gamma_in"]),
                                 y=lib.ptr(sess.proj), n=n, k=cfg.hidden, prologue=lib.NORM_F32GAIN, epilogue=lib.EPI_STORE,
                                 eps=cfg.rms_eps, pdl=1) for l in gdn]

        def launches():
            for a in calls:
                lib.check(lib.load().tfb_gemv_f32(C.byref(a), lib.stream()), "tfb_gemv_f32")
        return ("gemv_f32_kernel<store> (input norm + Gated DeltaNet in-projection)", _graph_time(launches, len(gdn)),
                n * cfg.hidden * 2)
    mamba = [l for l in sess.layers if l["kind"] == "linear_attention"]

    def launches():
        for layer in mamba:
            lib.gemv(layer["w_in"], sess.hidden, sess.proj, gamma=layer["gamma_in"], prologue=lib.NORM_F32GAIN,
                     eps=cfg.rms_norm_eps, pdl=True)
    return ("gemv_kernel<store> (input norm + Mamba-2 in_projection)", _graph_time(launches, len(mamba)),
            cfg.proj * cfg.hidden_size * 2)


def cpu_baseline(work, steps, warm, seed=0, start_at=None):
    """The CPU oracle (a port of the reference evaluator's arithmetic) on all host cores.  Models too
    large for a host run use a truncated layer stack and the time is scaled per layer (labelled).
    *start_at*: walk the whole 64-token prompt and decode greedily, untimed, up to that position, then time
    *steps* steps there (the reference arm: the positions the GPU arm times); default: *warm* prompt tokens then
    *steps* timed steps straight after them (the short sample the GPU arm carries along)."""
    from oracle import generation

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    cfg, scale = work.truncated()
    ref = work.oracle(cfg, work.host_weights(cfg, seed))
    if start_at is None:
        run = generation.decode_ids(ref, prompt_ids(cfg, 0)[:warm], steps)
        per_token = run["seconds"] / steps
        sample = f"{warm} prompt steps (untimed) then {steps} greedy decode steps"
    else:
        ahead = start_at - PROMPT_TOKENS                       # untimed greedy steps between the prompt and the window
        lead = generation.decode_ids(ref, prompt_ids(cfg, 0), ahead)
        history = torch.cat([prompt_ids(cfg, 0), torch.tensor(lead["tokens"], dtype=torch.int64)])
        run = generation.decode_ids(ref, history, steps, caches=lead["caches"], logits=lead["last_logits"])
        per_token = run["seconds"] / steps
        sample = (f"{PROMPT_TOKENS} prompt steps and {ahead} greedy steps (untimed), then {steps} greedy decode steps "
                  f"timed at positions {start_at}..{start_at + steps - 1}")
    sample += f", same architecture and seed, torch CPU bf16, {threads} threads"
    if scale != 1.0:
        # head and embedding are not per-layer: the whole truncated step is scaled, which over-counts the head slightly
        sample += (f"; truncated to {cfg.num_hidden_layers} of {work.cfg.num_hidden_layers} layers and scaled "
                   f"x{scale:.2f} per layer (extrapolated)")
        per_token *= scale
    return {"value": 1.0 / per_token, "unit": "tok/s", "cores": threads, "kind": "port", "sample": sample}


def run_reference(args):
    """Reference arm: the reference's own CPU implementation of the path.  The reference package does not
    import here (isl / ortools missing), so this is the oracle port of its evaluator, on all host cores, over
    the same prompt and the same timed positions as the GPU arm.  Rank 0 alone runs it."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    work = Workload(args.config)
    K, W = args.steps, max(args.warmup, 3)
    first, mid = windows(K, W)
    at = mid if mid is not None else first
    base = cpu_baseline(work, K, None, start_at=at)
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": "tok/s", "n_gpus": args.gpus,
        "steps": K, "warmup": W, "ms_per_step": 1e3 / base["value"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": work.dtype, "data": "synthetic",
        "config": {"workload": work.describe, "positions": describe_positions(K, W), "name": work.key,
                   "timed_positions": [at, at + K]},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_moe_batch(args):
    print(json.dumps(moe_batch_summary(args.moe_batch)))


def moe_batch_summary(T, dev=None, compare=True):
    """The Qwen3.5-35B-A3B expert block for a batch of tokens (`tfb_moe_batch`): 256 experts of 512, top-8, the shared
    expert, hidden 2048; random tokens routed by a random router, so ~222 experts are touched by 64 tokens.  Timed over
    several layers' expert sets (1.6 GB each, far more than L2) in one CUDA graph; bytes = the touched experts' three
    matrices once, plus the shared expert's.  For scale, the same tokens one at a time through the one-token kernels
    (gathered gate/up GEMV + down), which read an expert once per token that selected it."""
    import ctypes as C

    from tilefoundry_b200 import lib

    lib.load()
    dev = dev or torch.device("cuda:0")
    E, K, H, I = 256, 8, 2048, 512
    g = torch.Generator(device=dev).manual_seed(0)
    bf = torch.bfloat16
    rnd = lambda *shape, std=0.02: (torch.randn(*shape, device=dev, generator=g) * std).to(bf)
    n_layers = 3
    layers = [dict(w_gate=rnd(E, I, H), w_up=rnd(E, I, H), w_down=rnd(E, H, I), sg=rnd(I, H), su=rnd(I, H), sd=rnd(H, I),
                   router=rnd(E, H, std=0.05)) for _ in range(n_layers)]
    x = torch.randn(T, H, device=dev, generator=g)
    status = torch.zeros(1, device=dev, dtype=torch.int32)
    out = torch.empty(T, H, device=dev)
    scratch = dict(x_bf16=torch.empty(T, H, device=dev, dtype=bf), inner=torch.empty(T, K + 1, I, device=dev, dtype=bf),
                   y=torch.empty(T, K + 1, H, device=dev, dtype=bf), counts=torch.empty(2 * (E + 1) + 1, device=dev, dtype=torch.int32),
                   lists=torch.empty(E + 1, T, device=dev, dtype=torch.int32))
    calls, touched = [], []
    for L in layers:
        probs = torch.softmax((x.to(bf) @ L["router"].t()).float(), dim=-1)
        top, idx = torch.topk(probs, K, dim=-1)
        L["idx"], L["w"] = idx.contiguous(), (top / top.sum(-1, keepdim=True)).contiguous()
        L["gate"] = torch.zeros(T, device=dev)
        touched.append(int(torch.unique(idx).numel()))
        calls.append(lib.MoeBatchArgs(x=lib.ptr(x), indices=lib.ptr(L["idx"]), weights=lib.ptr(L["w"]), shared_gate=lib.ptr(L["gate"]),
                                      residual=None, w_gate=lib.ptr(L["w_gate"]), w_up=lib.ptr(L["w_up"]), w_down=lib.ptr(L["w_down"]),
                                      w_shared_gate=lib.ptr(L["sg"]), w_shared_up=lib.ptr(L["su"]), w_shared_down=lib.ptr(L["sd"]),
                                      out=lib.ptr(out), status=lib.ptr(status), tokens=T, hidden=H, inter=I, experts=E, top_k=K,
                                      pdl=0, **{k: lib.ptr(v) for k, v in scratch.items()}))

    def grouped():
        for a in calls:
            lib.check(lib.load().tfb_moe_batch(C.byref(a), lib.stream()), "tfb_moe_batch")
    ms = _graph_time(grouped, n_layers)
    if int(status):
        raise RuntimeError(f"tfb_moe_batch: a bounded wait gave up (status {int(status):#x})")
    expert_bytes = 3 * I * H * 2
    bytes_grouped = (sum(touched) / n_layers + 1) * expert_bytes

    # the whole block: post-norm of the residual stream, routing on the device, experts -- ten launches whatever T is
    gamma = torch.ones(H, device=dev)
    normed = torch.empty(T, H, device=dev)
    r_idx = torch.empty(T, K, device=dev, dtype=torch.int64)
    r_w, r_gate = torch.empty(T, K, device=dev), torch.empty(T, device=dev)
    r_logits = torch.empty(T, E + 1, device=dev)
    whole = []
    for L in layers:
        L["scale"] = rnd(1, H)
        route = lib.MoeRouteArgs(x=lib.ptr(normed), w_router=lib.ptr(L["router"]), w_shared_scale=lib.ptr(L["scale"]),
                                 logits=lib.ptr(r_logits), indices=lib.ptr(r_idx), weights=lib.ptr(r_w), shared_gate=lib.ptr(r_gate),
                                 tokens=T, hidden=H, experts=E, top_k=K, mode=1, pdl=0)
        block = lib.MoeBatchArgs(x=lib.ptr(normed), indices=lib.ptr(r_idx), weights=lib.ptr(r_w), shared_gate=lib.ptr(r_gate),
                                 residual=lib.ptr(x), w_gate=lib.ptr(L["w_gate"]), w_up=lib.ptr(L["w_up"]), w_down=lib.ptr(L["w_down"]),
                                 w_shared_gate=lib.ptr(L["sg"]), w_shared_up=lib.ptr(L["su"]), w_shared_down=lib.ptr(L["sd"]),
                                 out=lib.ptr(out), status=lib.ptr(status), tokens=T, hidden=H, inter=I, experts=E, top_k=K,
                                 pdl=0, **{k: lib.ptr(v) for k, v in scratch.items()})
        whole.append((route, block))

    def block_forward():
        for route, block in whole:
            lib.check(lib.load().tfb_rmsnorm_f32(lib.ptr(x), lib.ptr(gamma), lib.ptr(normed), T, H, 1e-6, 0, lib.stream()), "tfb_rmsnorm_f32")
            lib.check(lib.load().tfb_moe_batch_route(C.byref(route), lib.stream()), "tfb_moe_batch_route")
            lib.check(lib.load().tfb_moe_batch(C.byref(block), lib.stream()), "tfb_moe_batch")
    ms_whole = _graph_time(block_forward, n_layers)
    peak, kind = peaks()

    # the same work token by token through the one-token kernels (gathered gate/up + SwiGLU, then down + combine)
    inner1 = torch.empty((K + 1) * I, device=dev)
    out1 = torch.empty(H, device=dev)
    one = []
    for L in layers:
        for t in range(T):
            one.append((lib.GemvF32Args(w=lib.ptr(L["w_gate"]), w2=lib.ptr(L["w_up"]), w_extra=lib.ptr(L["sg"]), w2_extra=lib.ptr(L["su"]),
                                        x=lib.ptr(x[t]), y=lib.ptr(inner1), n=K * I + I, k=H, eps=1e-6, pdl=1, epilogue=lib.EPI_SWIGLU,
                                        expert_idx=lib.ptr(L["idx"][t]), rows_per_expert=I, routed_slots=K),
                        lib.MoeDownF32Args(w_down=lib.ptr(L["w_down"]), w_shared=lib.ptr(L["sd"]), inner=lib.ptr(inner1),
                                           indices=lib.ptr(L["idx"][t]), weights=lib.ptr(L["w"][t]),
                                           shared_gate_logit=lib.ptr(L["gate"][t:t + 1]), out=lib.ptr(out1), hidden=H, inter=I,
                                           shared_inter=I, top_k=K, pdl=1)))

    def token_by_token():
        for ga, da in one:
            lib.check(lib.load().tfb_gemv_f32(C.byref(ga), lib.stream()), "tfb_gemv_f32")
            lib.check(lib.load().tfb_moe_down_f32(C.byref(da), lib.stream()), "tfb_moe_down_f32")
    try:
        per_token_ms = _graph_time(token_by_token, n_layers, reps=3) if compare else None
    except Exception as exc:                                    # the comparison is a courtesy, not the measurement
        per_token_ms = f"{type(exc).__name__}: {exc}"
    line = {"mode": "moe_batch", "kernel": "moe_grouped_kernel (tcgen05.mma, K folded into N: 16 rows x 128 elements x 8 tokens per MMA)",
            "config": {"workload": "Qwen3.5-35B-A3B expert block: 256 experts of 512 + shared expert, top-8, hidden 2048", "tokens": T},
            "experts_touched_mean": sum(touched) / n_layers, "us_per_block": ms * 1e3,
            "algorithmic_bytes": bytes_grouped, "GBs": bytes_grouped / (ms * 1e-3) / 1e9,
            "frac_of_hbm_peak": bytes_grouped / (ms * 1e-3) / 1e9 / peak, "peak_GBs": peak, "peak_kind": kind,
            "us_per_block_with_norm_and_routing": ms_whole * 1e3,
            "one_token_kernels_us_for_the_same_tokens": per_token_ms * 1e3 if isinstance(per_token_ms, float) else per_token_ms}
    return line


def run_batch32_projection(args):
    """The batch-32 form of the projections of the Qwen3-1.7B architecture: y[32, n] = x[32, k] . w[n, k]^T on the
    tensor cores, timed over distinct weight matrices (far more than L2) in one CUDA graph, as HBM GB/s of weight
    bytes and as TFLOP/s.  Qwen3-1.7B shapes: head, fused gate|up, down, q|k|v, o."""
    import ctypes as C

    from tilefoundry_b200 import lib

    lib.load()
    dev = torch.device("cuda:0")
    cfg = Workload("qwen3_1_7b").cfg
    H, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    QKV = (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * cfg.head_dim
    M, out = 32, []
    peak, kind = peaks()
    for name, n, k in (("lm_head", V, H), ("gate|up", 2 * I, H), ("down", H, I), ("q|k|v", QKV, H), ("o", H, H)):
        L = max(2, min(24, int(2e9 // (n * k * 2))))
        W = [torch.randn(n, k, device=dev).to(torch.bfloat16) for _ in range(L)]
        x = torch.randn(M, k, device=dev).to(torch.bfloat16)
        y = torch.empty(M, n, device=dev, dtype=torch.bfloat16)
        splits = lib.load().tfb_gemm_small_m_splits(n, k)
        status = torch.zeros(1, device=dev, dtype=torch.int32)
        calls = [lib.GemmSmallMArgs(w=lib.ptr(w), x=lib.ptr(x), y=lib.ptr(y),
                                    status=lib.ptr(status), m=M, n=n, k=k, pdl=1) for w in W]

        def launches():
            for a in calls:
                lib.check(lib.load().tfb_gemm_small_m(C.byref(a), lib.stream()), "tfb_gemm_small_m")
        ms = _graph_time(launches, L)
        if int(status):
            raise RuntimeError(f"tfb_gemm_small_m: a bounded wait gave up (role {int(status)})")
        gbs = n * k * 2 / (ms * 1e-3) / 1e9
        out.append({"projection": name, "n": n, "k": k, "k_splits": splits, "us_per_launch": ms * 1e3, "weight_GBs": gbs,
                    "frac_of_hbm_peak": gbs / peak, "TFLOPs": 2 * M * n * k / (ms * 1e-3) / 1e12})
        del W
    print(json.dumps({"mode": "batch32_projection", "kernel": "gemm_tc_kernel (tcgen05.mma, TMEM accumulator, TMA ring)",
                      "batch": M, "dtype": "bf16", "peak_GBs": peak, "peak_kind": kind, "shapes": out}))


def run_batch_decode(args):
    """Several sequences at once: `--batch B` independent sequences of the Qwen3-1.7B
    architecture, each a 64-token random prompt walked token by token and then `--steps` greedy tokens; every
    projection on the tensor cores, the KV cache of every sequence read once per step.  One JSON line: total
    tokens/s over all sequences and the fraction of the measured HBM peak the step's algorithmic bytes reach."""
    from tilefoundry_b200.engine.qwen3_batch import Qwen3BatchSession
    from tilefoundry_b200.runtime import DictResource

    work = Workload("qwen3_1_7b")
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    B, steps = args.batch, args.steps
    n_prompt = args.prompt_tokens or PROMPT_TOKENS
    max_ctx = n_prompt + max(steps, 8) + 8
    sess = Qwen3BatchSession(work.cfg, DictResource(work.device_weights(dev)), batch=B, max_ctx=max_ctx, device=dev)
    prompts = torch.randint(0, work.cfg.vocab_size, (B, n_prompt), generator=torch.Generator().manual_seed(1))
    if args.skip_prompt_walk:
        # the profiler-sized case: positions set straight to the end of the prompt (cache rows below stay zero, the
        # bytes moved are the same), a few eager steps and no graph, so a capture meets few launches before its own
        from tilefoundry_b200.engine.session import Generated
        sess.reset(prompts)
        sess.pos.fill_(n_prompt - 1)
        for _ in range(3):
            sess.step()
        sess.pos.fill_(n_prompt - 1)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sampler = ClockSampler(0)
        torch.cuda.synchronize()
        start.record()
        for _ in range(steps):
            sess.step()
        end.record()
        torch.cuda.synchronize()
        sess.check_status()
        clocks = sampler.stop()
        gen = Generated([], start.elapsed_time(end) / 1e3, 0.0, 1)
    else:
        sess.generate(prompts, 8)                               # capture + warm-up
        sampler = ClockSampler(0)
        gen = sess.generate(prompts, steps)
        clocks = sampler.stop()
    W, kv = sess.weight_bytes(), sess.kv_bytes_per_position()
    # bytes(t) = weights + batch * kv_per_position * (context read + the entry written)
    total_bytes = sum(W + B * kv * (n_prompt + t + 1) for t in range(steps))
    peak, kind = peaks()
    achieved = total_bytes / gen.seconds / 1e9
    print(json.dumps({
        "mode": "batch_decode", "metric": "decode tok/s, all sequences", "value": B * steps / gen.seconds,
        "unit": "tok/s", "batch": B, "steps": steps, "ms_per_step": gen.seconds * 1e3 / steps,
        "prompt_ms_per_step": gen.prompt_seconds * 1e3 / max(gen.prompt_steps - 1, 1),
        "dtype": "bf16", "data": "synthetic", "gpu_launches": sess.launches_per_step * steps,
        "launch": "eager, prompt walk skipped" if args.skip_prompt_walk else "one captured graph per step",
        "config": {"workload": work.describe.replace("batch 1", f"batch {B}").replace("64-token", f"{n_prompt}-token"),
                   "l2": "inputs larger than L2"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_kind": kind, "weights_bytes_per_step": W, "kv_bytes_per_step_at_end":
                     B * kv * (n_prompt + steps)},
        "clocks": clocks}))


def batch32_summary(work, dev, packed_from, steps):
    """The batch-32 clause of the headline configuration inside the default run: 32 sequences per step on the
    tensor-core projections, sharing the weights the one-sequence session already holds."""
    from tilefoundry_b200.engine.packed import PackedQwen3
    from tilefoundry_b200.engine.qwen3_batch import Qwen3BatchSession

    B, n_prompt = 32, PROMPT_TOKENS
    weights = PackedQwen3({"w_embed": packed_from.w_embed, "gamma_final": packed_from.gamma_final,
                           "w_head": None if packed_from.w_head is packed_from.w_embed else packed_from.w_head},
                          packed_from.layers)
    sess = Qwen3BatchSession(work.cfg, weights, batch=B, max_ctx=n_prompt + steps + 8, device=dev)
    prompts = torch.randint(0, work.cfg.vocab_size, (B, n_prompt), generator=torch.Generator().manual_seed(1))
    sess.generate(prompts, 8)
    gen = sess.generate(prompts, steps)
    W, kv = sess.weight_bytes(), sess.kv_bytes_per_position()
    total_bytes = sum(W + B * kv * (n_prompt + t + 1) for t in range(steps))
    peak, _ = peaks()
    achieved = total_bytes / gen.seconds / 1e9
    return {"batch": B, "value": B * steps / gen.seconds, "unit": "tok/s over all sequences", "steps": steps,
            "ms_per_step": gen.seconds * 1e3 / steps, "gpu_launches": sess.launches_per_step * steps,
            "roofline_frac": achieved / peak, "achieved_GBs": achieved}


NEW_TOKENS = 2048                      # the run the metric names: 2048 greedy tokens after the 64-token prompt


def windows(K, W):
    """Positions of the timed steps inside that run.  A step at position p reads p cached positions and writes
    one; position 63 consumes the last prompt token and yields the first new one.  The prompt (positions 0..62)
    is always walked untimed, then W untimed decode steps, then K timed steps ("after_prompt").  When K is
    shorter than the whole run a second window of K steps is timed around the run's mean position (1087): time
    per token grows linearly with the context, so that window estimates the mean over all 2048 tokens, and it
    is the one `value` reports."""
    first = PROMPT_TOKENS - 1 + W
    if K + W >= NEW_TOKENS:
        return first, None
    mid = PROMPT_TOKENS - 1 + NEW_TOKENS // 2 - K // 2
    return first, max(mid, first + K)


def describe_positions(K, W):
    first, mid = windows(K, W)
    at = mid if mid is not None else first
    return (f"{PROMPT_TOKENS}-token prompt walked untimed, {W} untimed decode steps, then {K} timed steps at positions "
            f"{at}..{at + K - 1} of the 2048-token greedy run" + (" (centred on its mean context)" if mid is not None else ""))


def measure(work, sess, prompt, K, W, dev, rank, world, units, sample_clocks):
    """Device-resident and end-to-end timing of K decode steps of *sess*, in the window(s) `windows` gives."""
    import torch.distributed as dist

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t)
        return ms

    stream = torch.cuda.current_stream()

    def timed(K):
        barrier()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(stream)
        sess.run(K)
        end.record(stream)
        barrier()
        return max_over_ranks(start.elapsed_time(end))

    first, mid = windows(K, W)
    sess.reset(prompt)
    sess.run(first)                                  # prompt walk + W warm-up decode steps
    sampler = ClockSampler(dev.index) if sample_clocks else None
    snap = sess.snapshot() if mid is None else None
    ms_first = timed(K)
    at, ms = first, ms_first
    if mid is not None:
        sess.run(mid - (first + K))                  # the same greedy run, continued untimed up to the second window
        torch.cuda.synchronize()
        snap = sess.snapshot()
        at, ms = mid, timed(K)
    clocks = sampler.stop() if sampler else None
    tokens_out = sess.tokens[at + 1: at + 1 + min(K, 8)].tolist()

    # ---- end to end over the same positions: token in from pinned host memory, picked token back, every step ----
    sess.restore(snap)
    pin_in = torch.empty(1, dtype=torch.int64).pin_memory()
    pin_in[0] = int(sess.tokens[at])
    barrier()
    t0 = time.perf_counter()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    sess.generate_host(at, K, pin_in)                   # every step: H2D its input token, the step, D2H its pick, wait
    e1.record(stream)
    barrier()
    e2e_ms = max_over_ranks(max(e0.elapsed_time(e1), (time.perf_counter() - t0) * 1e3))

    peak, peak_kind = peaks()
    w_bytes, kv_pos = sess.weight_bytes(), sess.kv_bytes_per_position()
    state = sess.state_bytes() if hasattr(sess, "state_bytes") else 0
    # a step at position p reads its weights, the p cached positions and the recurrent state, writes one
    # position and the state back
    step_bytes = [w_bytes + state + kv_pos * (at + i + 1) for i in range(K)]
    step_gbs = sum(step_bytes) / (ms * 1e-3) / 1e9
    out = {
        "value": units * K / (ms * 1e-3), "ms_per_step": ms / K, "timed_positions": [at, at + K],
        "e2e": {"value": units * K / (e2e_ms * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": 8, "d2h_bytes_per_step": 8},
        "gpu_launches": sess.launches_per_step * K, "clocks": clocks, "first_tokens": tokens_out,
        "whole_step": {"achieved": step_gbs, "frac": step_gbs / peak, "bytes_per_token_mean": sum(step_bytes) / K,
                       "weights_bytes": w_bytes, "state_bytes": state, "kv_bytes_per_position": kv_pos,
                       "frac_of_8TBs_nominal": step_gbs / 8000.0},
    }
    if mid is not None:
        first_bytes = sum(w_bytes + state + kv_pos * (first + i + 1) for i in range(K))
        out["after_prompt"] = {"value": units * K / (ms_first * 1e-3), "ms_per_step": ms_first / K,
                               "timed_positions": [first, first + K],
                               "whole_step_frac": first_bytes / (ms_first * 1e-3) / 1e9 / peak}
    return out


def roofline_of(work, sess, whole_step):
    peak, peak_kind = peaks()
    k_name, k_ms, k_bytes = dominant_kernel(work, sess)
    k_gbs = k_bytes / (k_ms * 1e-3) / 1e9
    return {"kernel": k_name, "bound": "hbm", "achieved": k_gbs, "peak": peak,
            "peak_kind": "measured (MEASURED_PEAKS.json hbm_gbs)" if peak_kind == "measured" else "fallback",
            "unit": "GB/s", "frac": k_gbs / peak, "traffic": NCU_TRAFFIC.get(work.key),
            "algorithmic_bytes_per_launch": k_bytes, "us_per_launch": k_ms * 1e3, "whole_step": whole_step}


def side_config(key, dev, K, W, with_cpu):
    """One of the other single-GPU configurations, measured the same way, as a bounded side entry of the line."""
    from tilefoundry_b200.runtime import DictResource

    work = Workload(key)
    first, mid = windows(K, W)
    max_ctx = (mid if mid is not None else first) + K + 8
    sess = work.session_cls(work.cfg, DictResource(work.device_weights(dev, seed=0)), max_ctx=max_ctx, device=dev)
    sess.reset(prompt_ids(work.cfg, 0))
    sess.capture()
    m = measure(work, sess, prompt_ids(work.cfg, 0), K, W, dev, 0, 1, 1, False)
    whole = m.pop("whole_step")
    out = {"workload": work.describe, "dtype": work.dtype, "unit": "tok/s", **m, "roofline": roofline_of(work, sess, whole)}
    if hasattr(sess, "prefill"):
        # prompt processing, outside the metric: the 64-token prompt walked one decode step per token against the
        # same prompt in chunks of 32 tokens (tensor-core projections)
        try:
            prompt = prompt_ids(work.cfg, 0)
            walk = sess.generate(prompt, 4)
            sess.generate(prompt, 4, prefill=True)                                  # warm-up: buffers, tensor maps
            chunked = sess.generate(prompt, 4, prefill=True)
            out["prompt"] = {"tokens": PROMPT_TOKENS, "walk_ms": walk.prompt_seconds * 1e3,
                             "chunked_prefill_ms": chunked.prompt_seconds * 1e3,
                             "same_continuation": walk.tokens == chunked.tokens}
        except Exception as exc:                      # a side measurement: it must not cost the entry
            out["prompt"] = {"error": f"{type(exc).__name__}: {exc}"}
    del sess
    torch.cuda.empty_cache()
    if with_cpu:
        out["cpu_baseline"] = cpu_baseline(work, 8, 8)
    return out


def sharded_config(key, dev, K, W, rank, world):
    """One sequence of a MoE configuration split over all ranks (routed experts by expert, shared expert and head
    by slice; exchange kernels over NVLink peer memory): strong scaling, every rank the same tokens."""
    import torch.distributed as dist

    from tilefoundry_b200.runtime import DictResource

    work = Workload(key)
    first, mid = windows(K, W)
    max_ctx = (mid if mid is not None else first) + K + 8
    sess = work.session_cls(work.cfg, DictResource(work.device_weights(dev, seed=0)), max_ctx=max_ctx, device=dev,
                            group=dist.group.WORLD)
    prompt = prompt_ids(work.cfg, 0)
    sess.reset(prompt)
    sess.capture()
    m = measure(work, sess, prompt, K, W, dev, rank, world, 1, False)
    status = int(sess.peer_status) if getattr(sess, "collectives", "") == "peer" else 0
    whole = m.pop("whole_step")
    exchanges = len(sess.layers) + 1
    out = {"workload": work.describe, "scaling": "strong", "gpus": world, "unit": "tok/s", **m,
           "collectives": getattr(sess, "collectives", "nccl"), "exchanges_per_token": exchanges,
           "bounded_wait_status": status, "per_gpu": whole,
           "frac_of_n_gpu_roofline": whole["frac"],      # per-GPU bytes / time against ONE GPU's peak = total / (N x peak)
           "parallelism": f"ep{world} routed experts + tp{world} shared expert + vocabulary-parallel head, mixers replicated"}
    sess.graph = None
    del sess
    torch.cuda.empty_cache()
    return out


def run_ours(args):
    import datetime
    import threading

    import torch.distributed as dist

    from tilefoundry_b200.runtime import DictResource

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    # The exchange kernels use plain peer stores only: keep NCCL and symmetric memory from binding any buffer to an
    # NVLink multicast object (a rank that ends while bound to one disturbs its peers).
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    if world > 1:
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=600))

    work = Workload(args.config)
    cfg = work.cfg
    K, W = args.steps, max(args.warmup, 3)
    # `--config <MoE model> --gpus N` shards one sequence over the GPUs; the dense ones do not shard: each rank
    # decodes its own sequence ("replicas only").
    sharded = world > 1 and work.key in ("granite_4_0_h_small", "qwen3_5_35b_a3b")
    prompt = prompt_ids(cfg, seed=0 if sharded else rank)
    first, mid = windows(K, W)
    max_ctx = (mid if mid is not None else first) + K + 8
    extra = {"group": dist.group.WORLD} if sharded else {}
    if work.key == "qwen3_1_7b" and args.kernel >= 0:
        extra["kernel"] = args.kernel
    sess = work.session_cls(cfg, DictResource(work.device_weights(dev, seed=0)), max_ctx=max_ctx, device=dev, **extra)
    units = 1 if sharded else world                           # sequences decoded per step over all ranks
    sess.reset(prompt)
    if args.dominant_only:
        name, ms_launch, nbytes = dominant_kernel(work, sess)
        print(json.dumps({"kernel": name, "us_per_launch": ms_launch * 1e3, "algorithmic_bytes_per_launch": nbytes,
                          "achieved_gbs": nbytes / (ms_launch * 1e-3) / 1e9}))
        return
    sess.capture()
    m = measure(work, sess, prompt, K, W, dev, rank, world, units, rank == 0)
    whole = m.pop("whole_step")
    line = None
    if rank == 0:
        roofline = roofline_of(work, sess, whole)
        # prompt processing, outside the metric: the 64-token prompt walked one decode step per token against the same
        # prompt in chunks of 32 tokens on the tensor-core projections (Qwen3 only)
        prompt_info = batch32 = None
        if world == 1 and hasattr(sess, "prefill") and not args.no_sides:
            walk = sess.generate(prompt, 4)
            sess.generate(prompt, 4, prefill=True)                                  # warm-up: buffers, tensor maps
            chunked = sess.generate(prompt, 4, prefill=True)
            prompt_info = {"tokens": PROMPT_TOKENS, "walk_ms": walk.prompt_seconds * 1e3,
                           "chunked_prefill_ms": chunked.prompt_seconds * 1e3,
                           "same_continuation": walk.tokens == chunked.tokens}
        if world == 1 and work.key == "qwen3_1_7b" and not args.no_sides:
            try:
                batch32 = batch32_summary(work, dev, sess, min(K, 2048))
            except Exception as exc:                      # a side measurement: it must not cost the headline line
                batch32 = {"error": f"{type(exc).__name__}: {exc}"}
        base = None
        if world == 1 and not args.no_cpu:
            base = cpu_baseline(work, 32 if work.cpu_layers is None else 8, PROMPT_TOKENS if work.cpu_layers is None else 8)
        line = {
            "metric": METRIC, "value": m["value"], "unit": "tok/s", "n_gpus": world, "steps": K,
            "warmup": W, "ms_per_step": m["ms_per_step"], "higher_is_better": True,
            "scaling": "strong" if sharded else "weak", "vs_baseline": None,
            "dtype": work.dtype, "data": "synthetic",
            # (the reference arm prints the very same `config`)
            "config": {"workload": work.describe, "positions": describe_positions(K, W), "name": work.key,
                       "timed_positions": m["timed_positions"]},
            "parallelism": (f"ep{world} routed experts + tp{world} shared expert + vocabulary-parallel head, mixers "
                            f"replicated, one exchange per MoE block ({getattr(sess, 'collectives', 'nccl')} collectives)"
                            if sharded else "replicas only" if world > 1 else "1 gpu"),
            "l2": f"inputs larger than L2: {whole['weights_bytes'] / 1e9:.2f} GB of weights are streamed every step",
            "first_tokens": m["first_tokens"],
            "e2e": m["e2e"], "gpu_launches": m["gpu_launches"], "clocks": m["clocks"], "roofline": roofline,
            "cpu_baseline": base, "after_prompt": m.get("after_prompt"), "prompt": prompt_info, "batch32": batch32,
        }
    sess.graph = None
    del sess
    torch.cuda.empty_cache()

    # ---- the other configurations, bounded, so that their numbers come from the same run ----------------------------
    def guarded(fn, *a):
        try:
            return fn(*a)
        except Exception as exc:                          # side measurements must not cost the headline line
            return {"error": f"{type(exc).__name__}: {exc}"}

    if world == 1 and work.key == "qwen3_1_7b" and not args.no_sides:
        Ks = min(K, 256)
        line["configs"] = {key: guarded(side_config, key, dev, Ks, W, not args.no_cpu)
                           for key in ("minicpm3_4b", "granite_4_0_h_small", "qwen3_5_35b_a3b")}
        torch.cuda.empty_cache()
        line["moe_batch64"] = guarded(moe_batch_summary, 64, dev, False)     # the Qwen3.5 expert block for 64 tokens at once
    if world > 1 and work.key == "qwen3_1_7b" and not args.no_sides:
        # The sharded MoE steps wait on one another across ranks inside kernels (bounded) and in barriers (not): a
        # watchdog prints the headline line and ends the process if this part does not finish in time.
        def give_up():
            if rank == 0:
                line["sharded"] = {"error": "the sharded measurements did not finish within 420 s"}
                print(json.dumps(line), flush=True)
            os._exit(0)
        dog = threading.Timer(420.0, give_up)
        dog.daemon = True
        dog.start()
        Ks = min(K, 256)
        res = {key: guarded(sharded_config, key, dev, Ks, W, rank, world)
               for key in ("granite_4_0_h_small", "qwen3_5_35b_a3b")}
        dog.cancel()
        if rank == 0:
            line["sharded"] = res
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        # every rank stays until all of them are done, then they leave together (no captured graph is alive any more)
        from tilefoundry_b200.engine.peer import leave_together
        leave_together()


def run_profile_case(args):
    """A few eager decode steps of a configuration cut to --profile-layers layers, the position parked at the mean
    context of the benchmark: small enough (a few GB) for a profiler to replay single launches of any kernel of the
    step.  Prints what it ran; not a benchmark line."""
    import dataclasses

    import torch

    from tilefoundry_b200.runtime import DictResource

    work = Workload(args.config)
    n = args.profile_layers
    kw = {"n_layers": n} if work.key == "qwen3_5_35b_a3b" else {"num_hidden_layers": n}
    if work.key == "granite_4_0_h_small":
        kw["attention_layers"] = (n - 1,)
    work.cfg = dataclasses.replace(work.cfg, **kw)
    dev = torch.device("cuda:0")
    extra = {"kernel": args.kernel} if work.key == "qwen3_1_7b" and args.kernel >= 0 else {}
    sess = work.session_cls(work.cfg, DictResource(work.device_weights(dev, seed=0)), max_ctx=PROMPT_TOKENS + NEW_TOKENS,
                            device=dev, **extra)
    sess.reset(prompt_ids(work.cfg, 0))
    steps = min(max(args.steps, 1), 16)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for i in range(steps + 1):
        sess.pos.fill_(PROMPT_TOKENS - 1 + NEW_TOKENS // 2)
        if i == 1:
            t0.record()
        sess.step()
    t1.record()
    torch.cuda.synchronize()
    print(json.dumps({"profile_case": True, "config": work.key, "layers": n, "eager_steps": steps,
                      "context": PROMPT_TOKENS - 1 + NEW_TOKENS // 2, "launches_per_step": sess.launches_per_step,
                      "ms_per_eager_step": t0.elapsed_time(t1) / steps}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2048)
    ap.add_argument("--warmup", type=int, default=3,
                    help="untimed decode steps after the (always untimed) 64-token prompt walk")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="qwen3_1_7b",
                    choices=["qwen3_1_7b", "minicpm3_4b", "granite_4_0_h_small", "qwen3_5_35b_a3b"],
                    help="which configuration to run (default: the one the metric is quoted on)")
    ap.add_argument("--kernel", type=int, default=-1,
                    help="Qwen3 only: TFB_KERNEL_* of the step (0 = one launch per kernel, 6 = the whole step as one "
                         "cooperative launch; default: the session's own choice, which is 6 for this architecture)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-sides", action="store_true",
                    help="only the headline configuration: no prompt / batch-32 / other-configuration / sharded side entries")
    ap.add_argument("--batch32-projection", action="store_true",
                    help="time the batch-32 tensor-core projection (tcgen05) on this configuration's projection shapes, "
                         "print one JSON line and exit")
    ap.add_argument("--moe-batch", type=int, default=0,
                    help="time the Qwen3.5 expert block for this many tokens at once (tfb_moe_batch, e.g. 64), print one JSON "
                         "line and exit")
    ap.add_argument("--batch", type=int, default=1,
                    help="decode this many independent Qwen3-1.7B sequences per step (2..32) on the tensor-core "
                         "projections, print one JSON line and exit")
    ap.add_argument("--prompt-tokens", type=int, default=0,
                    help="with --batch: prompt length per sequence (default 64); a long prompt puts the timed steps at a "
                         "long context, e.g. for a profiler capture of the batched attention kernel")
    ap.add_argument("--skip-prompt-walk", action="store_true",
                    help="with --batch: start at the end of the prompt without walking it and launch eagerly (for profiler "
                         "captures; the number includes host launch time)")
    ap.add_argument("--profile-layers", type=int, default=0,
                    help="the small case a profiler capture runs: the configuration cut to this many layers (same widths, one "
                         "attention layer among them where the model mixes layer kinds), --steps eager decode steps at "
                         "the run's mean context, one JSON line that is NOT the metric")
    ap.add_argument("--dominant-only", action="store_true",
                    help="build the session, time only the dominant kernel over every layer's weights, print it and exit "
                         "(the small case a profiler capture of that kernel runs)")
    args = ap.parse_args()
    if args.profile_layers > 0:
        run_profile_case(args)
    elif args.impl == "reference":
        run_reference(args)
    elif args.moe_batch > 0:
        run_moe_batch(args)
    elif args.batch32_projection:
        run_batch32_projection(args)
    elif args.batch > 1:
        run_batch_decode(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
