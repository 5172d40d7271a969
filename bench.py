#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, on the Llama-3.1-8B shape with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L] [--impl reference]
                    [--shape llama-3.1-8b | llama-2-13b | llama-3.2-1b]

One JSON line: `value` is decoded tokens per second at batch 8 (K captured decode steps back to back on the
device, timed with CUDA events); `e2e` is the same through the public entry point (`LocalModel.generate`, host
token ids in and out every step); `prefill` is one 2,048-token prompt; `roofline` compares the bytes a decode
step must read (weights once, the live requests' keys and values) with the measured copy bandwidth; `points`
holds batch 1 and 64. A step reads 16 GB of weights, far more than the 126 MB L2, so no flush is needed between
steps. For more than one GPU it prints one line saying so and exits with 2: this engine runs on one GPU.

`--shape llama-2-13b` measures the same line on the Llama-2-13B shape (40 key/value heads, context 4,096,
2,048-token prompts, an explicit page pool for batch 64). `--shape llama-3.2-1b` runs the mixed workload of that
shape instead: 64 requests with prompts of 16 to 2,048 random ids and 128 tokens each under continuous batching
through `LocalModel.generate`; `value` is then generated tokens per second from submission to the last token,
and `points.decode_b64` / `roofline` describe the steady decode step of all 64 at head size 64.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LLAMA_31_8B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 32, "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 128, "intermediate_size": 14336, "vocab_size": 128256, "max_position_embeddings": 131072,
    "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "tie_word_embeddings": False,
}
LLAMA_2_13B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 40, "hidden_size": 5120, "num_attention_heads": 40, "num_key_value_heads": 40,
    "head_dim": 128, "intermediate_size": 13824, "vocab_size": 32000, "max_position_embeddings": 4096,
    "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "rope_scaling": None, "tie_word_embeddings": False,
}
LLAMA_32_1B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 16, "hidden_size": 2048, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 64, "intermediate_size": 8192, "vocab_size": 128256, "max_position_embeddings": 131072,
    "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "tie_word_embeddings": True,
}
# name -> (config.json, label, context, prompt tokens of the decode points, seed of the random weights, rope in words)
SHAPES = {
    "llama-3.1-8b": (LLAMA_31_8B, "Llama-3.1-8B shape", 8192, 1024, 5,
                     "theta 5e5, llama3 factor 8 low 1 high 4 original 8192"),
    "llama-2-13b": (LLAMA_2_13B, "Llama-2-13B shape", 4096, 2048, 7, "theta 1e4, no scaling"),
    "llama-3.2-1b": (LLAMA_32_1B, "Llama-3.2-1B shape", 8192, 1024, 6,
                     "theta 5e5, llama3 factor 32 low 1 high 4 original 8192"),
}
PREFILL_TOKENS = 2048
SETTLE_S = 0.3  # idle time between the prompts' prefill and a decode measurement's warm-up steps


def peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    try:
        with open(path) as f:
            m = json.load(f)
        if "hbm_gbs" in m:
            out["hbm_gbs"] = float(m["hbm_gbs"])
        if "bf16_tflops" in m:
            out["bf16_tflops"] = float(m["bf16_tflops"])
        if "bf16_tflops_sustained" in m:
            out["bf16_tflops_sustained"] = float(m["bf16_tflops_sustained"])
        out["source"] = "measured"
    except (OSError, ValueError):
        pass
    return out


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed regions run."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.perf_counter(), line.strip()))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, windows) -> dict:
        mhz, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for t, line in self.samples:
            if not any(a - 0.15 <= t <= b + 0.15 for a, b in windows):
                continue
            parts = [p.strip() for p in line.split(",")]
            try:
                mhz.append(int(parts[0]))
                mx = max(mx, int(parts[1]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": int(statistics.median(mhz)) if mhz else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(mhz)}


def contraction_table(args, token_counts) -> int:
    """The four contractions of one layer (q/k/v with store, output projection into the 32-bit stream, gate/up
    with SwiGLU, down into the stream) at the shape's widths: this library's kernels beside cuBLAS through
    torch.matmul (the plain product only; its epilogues would be further launches). Six sets of weights take
    turns, so weights always come from memory; CUDA events around six launches, best of five."""
    import math

    import torch

    from cuca_b200.kernels import ops

    cfg = SHAPES[args.shape][0]
    E, ff = cfg["hidden_size"], cfg["intermediate_size"]
    qkv = (cfg["num_attention_heads"] + 2 * cfg["num_key_value_heads"]) * cfg["head_dim"]
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(1)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    shapes = [("qkv", qkv, E, ops.EPI_STORE, torch.bfloat16), ("o", E, cfg["num_attention_heads"] * cfg["head_dim"],
                                                                  ops.EPI_RESIDUAL, torch.float32),
              ("gate_up", ff, E, ops.EPI_SWIGLU, torch.bfloat16), ("down", E, ff, ops.EPI_RESIDUAL, torch.float32)]
    sets = 6

    def best_us(fn):
        fn()
        torch.cuda.synchronize()
        out = []
        for _ in range(5):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            out.append(a.elapsed_time(b) * 1e3 / sets)
        return min(out)

    for M in token_counts:
        line = {"tokens": M, "shape": SHAPES[args.shape][1], "unit": "us per launch, cold weights"}
        for name, N, K, epi, odt in shapes:
            a = torch.randn(M, K, device=dev, generator=g).bfloat16()
            rows = (2 if epi == ops.EPI_SWIGLU else 1) * N
            ws = [(torch.randn(rows, K, device=dev, generator=g) / math.sqrt(K)).bfloat16() for _ in range(sets)]
            out = torch.zeros(M, N, device=dev, dtype=odt)
            ref = torch.empty(M, rows, device=dev, dtype=torch.bfloat16)
            if epi != ops.EPI_SWIGLU and ops.gemm_partial_supported(a, ws[0]) and \
                    (name != "qkv" or M <= ops.ROPE_PARTIAL_MAX_ROWS):
                # as the engine runs it over few tokens: K slices left unadded for the kernel that reads them next
                ours = best_us(lambda: [ops.gemm_partial(a, w, err) for w in ws])
                line.setdefault("unadded_slices", []).append(name)
            else:
                ours = best_us(lambda: [ops.gemm_tc(a, w, out, epi, None, err) for w in ws])
            cublas = best_us(lambda: [torch.matmul(a, w.T, out=ref) for w in ws])
            line[name] = {"ours": round(ours, 1), "cublas": round(cublas, 1), "ratio": round(ours / cublas, 2)}
        assert int(err.item()) == 0
        print(json.dumps(line))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the model has (reported)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-points", action="store_true", help="skip batch 1 and 64")
    ap.add_argument("--shape", default="llama-3.1-8b", choices=sorted(SHAPES))
    ap.add_argument("--prompt-tokens", type=int, default=None, help="prompt length of the decode points (the shape's default else)")
    ap.add_argument("--prefill-tokens", type=int, default=None,
                    help="length of the timed prefill prompt (2,048 else; longer prompts run in portions of 2,048)")
    ap.add_argument("--context", type=int, default=None, help="context length (the shape's default else)")
    ap.add_argument("--contractions", default=None, metavar="M,M,...",
                    help="instead of the bench: time the four contractions of a layer at these token counts, this "
                         "library's kernels beside cuBLAS (torch.matmul), cold weights; one JSON line per count")
    ap.add_argument("--decode-only", action="store_true",
                    help="with --shape llama-3.2-1b: the plain decode line at --batch instead of the mixed workload")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "nassor/cuca is a Rust crate (rust-toolchain 1.100.0): no cargo/rustc in this image and "
                          "no network for crates.io, so it cannot be built or installed; its CUDA backend was "
                          "never run by its authors either"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not measured (use --gpus 1)")
        return 2
    args.warmup = max(3, args.warmup)
    if args.steps + args.warmup + 2 > 1000:
        print("bench.py: --steps + --warmup must stay below 1000")
        return 2

    import numpy as np
    import torch

    if args.contractions:
        return contraction_table(args, [int(m) for m in args.contractions.split(",")])

    from cuca_b200 import BatchingConfig, LocalModel, LocalModelConfig, RandomWeights
    from cuca_b200.engine.scheduler import DECODE, Request
    from cuca_b200.kernels import library

    base_cfg, label, CONTEXT, PROMPT, SEED, rope_words = SHAPES[args.shape]
    mixed = args.shape == "llama-3.2-1b" and not args.decode_only
    PREFILL_TOKENS = args.prefill_tokens or globals()["PREFILL_TOKENS"]
    STEP_TOKENS = 2048  # rows of one step: longer prompts are prefilled in portions of this many
    PROMPT = args.prompt_tokens or PROMPT
    CONTEXT = args.context or max(CONTEXT, PROMPT + args.steps + args.warmup + 256, PREFILL_TOKENS + 16)
    cfg = dict(base_cfg)
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    layers = cfg["num_hidden_layers"]
    pk = peaks()
    max_batch = args.batch if args.no_points and not mixed else max(64, args.batch)
    point_steps = min(args.steps, 64)  # steps of the batch-1 and batch-64 points

    def pages_for(batch, steps):
        """Positions the pool must hold for `batch` requests that decode `steps` timed steps after their prompt
        (requests that finish their prompt early decode while the others are still being prefilled)."""
        per_request = PROMPT + steps + args.warmup + 2 * (-(-batch * PROMPT // STEP_TOKENS)) + 48
        return batch * (-(-per_request // 16) * 16)

    kv_tokens = max(CONTEXT + 16, pages_for(args.batch, args.steps), 0 if args.no_points else pages_for(64, point_steps),
                    64 * (2048 + 128 + 16) if mixed else 0, PREFILL_TOKENS + 64) + STEP_TOKENS + 64
    t0 = time.perf_counter()
    model = LocalModel.load(LocalModelConfig(
        model_config=cfg, random_weights=RandomWeights(seed=SEED, std=0.02), dtype="bfloat16", context_length=CONTEXT,
        kv_block_size=16, batching=BatchingConfig(max_sequences=max_batch, kv_tokens=kv_tokens,
                                                  max_step_tokens=max(STEP_TOKENS, max_batch),
                                                  prefill_chunk=STEP_TOKENS)))
    load_s = time.perf_counter() - t0
    core, sched, backend = model.core, model.scheduler, model.backend
    vocab = cfg["vocab_size"]
    rng = np.random.default_rng(SEED)
    clocks = ClockSampler()
    clocks.start()
    windows = []

    def prompts(n, length):
        return [rng.integers(0, vocab, size=length).tolist() for _ in range(n)]

    # ------------------------------------------------------------ prefill: one 2,048-token prompt, one step
    def prefill_once():
        p = prompts(1, PREFILL_TOKENS)[0]
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        model.generate(p, max_tokens=1, temperature=0.0)
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b)

    for _ in range(3):
        prefill_once()
    w0 = time.perf_counter()
    torch.cuda.nvtx.range_push("prefill_timed")
    prefill_ms = statistics.median(prefill_once() for _ in range(5))
    torch.cuda.nvtx.range_pop()
    windows.append((w0, time.perf_counter()))
    E, ff, nh, nkv, d = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_attention_heads"], \
        cfg["num_key_value_heads"], cfg["head_dim"]
    gemm_params = layers * (E * (nh + 2 * nkv) * d + nh * d * E + 3 * E * ff)
    T = PREFILL_TOKENS
    prefill_flops = 2.0 * T * gemm_params + layers * 4.0 * nh * d * (T * (T + 1) / 2) + 2.0 * E * vocab
    prefill = {"value": round(T / (prefill_ms / 1e3), 1), "tokens": T, "ms": round(prefill_ms, 3),
               "frac": round(prefill_flops / (prefill_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
               "tflops": round(prefill_flops / (prefill_ms / 1e3) / 1e12, 1)}
    if "bf16_tflops_sustained" in pk:  # the prompts are timed back to back, under the power cap
        prefill["frac_of_sustained"] = round(prefill_flops / (prefill_ms / 1e3) / (pk["bf16_tflops_sustained"] * 1e12), 4)

    # ------------------------------------------------------------ decode, device only: K captured steps
    def decode_device(batch, steps, warmup):
        # requests that finish their prompt early decode while the others are still being prefilled: give every
        # request room for that, and never spin if the scheduler stops making progress
        turns_needed = -(-batch * PROMPT // sched.cfg.max_step_tokens) + 2
        seqs = [sched.submit(Request(p, max_tokens=steps + warmup + 2 * turns_needed + 8, temperature=0.0))
                for p in prompts(batch, PROMPT)]
        for _ in range(4 * turns_needed + 16):
            if all(s.phase == DECODE for s in seqs):
                break
            if sched.turn() == 0:
                break
        if not all(s.phase == DECODE for s in seqs):
            raise RuntimeError("bench: the prompts did not all reach the decode phase: "
                               + ", ".join(sorted({s.phase for s in seqs})))
        tokens = [s.pending for s in seqs]
        # The prompts' prefill leaves the SM clock where the power cap held it, and it comes back in stages over
        # the next 70 ms: the first ten decode steps after it take 4.2 ms, the next ten 3.7, then 3.57. A short
        # idle pause lets the clock recover before the warm-up steps, so that K = 20 timed steps show the steady
        # decode rate that K = 128 shows without it (named in `config.settle`).
        torch.cuda.synchronize()
        time.sleep(SETTLE_S)
        hist = backend.burst(seqs, tokens, warmup)
        tokens = hist[-1].tolist()
        ctx0 = seqs[0].blocks.length
        launches0 = library.launches
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        w = time.perf_counter()
        torch.cuda.nvtx.range_push("decode_timed_b%d" % batch)
        a.record()
        hist = backend.burst(seqs, tokens, steps, check=False)
        b.record()
        torch.cuda.synchronize()
        torch.cuda.nvtx.range_pop()
        windows.append((w, time.perf_counter()))
        ms = a.elapsed_time(b)
        out_tokens = hist.cpu()
        assert out_tokens.shape == (steps, batch) and int(out_tokens.min()) >= 0
        core.rt.check_device_errors()
        g = backend.graphs.get(batch, seqs[0].blocks.length, False)
        for s in list(seqs):
            sched.cancel(s)
        sched.finished.clear()
        mean_ctx = ctx0 + (steps - 1) / 2.0 + 1
        return ms / steps, mean_ctx, g

    def roofline_of(batch, ms, ctx):
        step_bytes = model.core.model.weight_bytes() + batch * ctx * core.cache.bytes_per_token()
        achieved = step_bytes / (ms / 1e3) / 1e9
        return {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": int(step_bytes), "peaks": pk["source"]}

    points, fracs = {}, {}
    if mixed:
        # ---------------------------------------------------- 64 requests of mixed length, continuous batching
        n_req, new_tokens = 64, 128
        lengths = rng.integers(16, 2049, size=n_req).tolist()
        ps = [rng.integers(0, vocab, size=n).tolist() for n in lengths]
        model.generate(ps[:4], max_tokens=4, temperature=0.0)  # warm-up: kernels configured, first graphs captured
        done_at = []
        steps0 = core.stepper.steps
        staging = core.stepper._staging
        h2d0, d2h0 = staging.bytes_sent + backend.h2d_bytes, backend.d2h_bytes
        torch.cuda.synchronize()
        w = time.perf_counter()
        outs = model.generate(ps, max_tokens=new_tokens, temperature=0.0,
                              on_token=lambda seq, tok: done_at.append(time.perf_counter()))
        torch.cuda.synchronize()
        wall = time.perf_counter() - w
        windows.append((w, time.perf_counter()))
        generated = sum(len(o.tokens) for o in outs)
        assert generated == n_req * new_tokens and all(o.report.finish_reason == "length" for o in outs)
        mixed_steps = core.stepper.steps - steps0
        value = generated / wall
        ms_step, mean_ctx, g8 = decode_device(64, point_steps, args.warmup)
        roofline = roofline_of(64, ms_step, mean_ctx)
        points["decode_b64"] = round(64 / (ms_step / 1e3), 1)
        fracs["decode_b64"] = roofline["frac"]
        e2e = {"value": round(value, 1), "unit": "tokens/s", "seconds": round(wall, 4), "steps": mixed_steps,
               "prompt_tokens": int(sum(lengths)), "generated_tokens": generated,
               "h2d_bytes_per_step": round((staging.bytes_sent + backend.h2d_bytes - h2d0) / max(1, mixed_steps)),
               "d2h_bytes_per_step": round((backend.d2h_bytes - d2h0) / max(1, mixed_steps))}
        metric = ("generated tokens/s, %s, bf16, 64 requests with prompts of 16..2048 ids and 128 tokens each, "
                  "continuous batching, submission to last token" % label)
        batch_of_value, steps_of_value = 64, mixed_steps
        ms_per_step = wall / max(1, mixed_steps) * 1e3
    else:
        ms_step, mean_ctx, g8 = decode_device(args.batch, args.steps, args.warmup)
        value = args.batch / (ms_step / 1e3)
        roofline = roofline_of(args.batch, ms_step, mean_ctx)

        # -------------------------------------------------------- decode, end to end through generate()
        # Requests whose prompt is done decode while later prompts are still prefilled; the clock runs on the LAST
        # request's tokens, which are all produced by steps that decode the whole batch, and every request gets
        # enough tokens to still be running then.
        # The first decode steps after the prompts run 3 to 18 % slower on the device itself (4.23 ms, then 3.68,
        # then 3.57 per step at batch 8): the SM clock comes back in stages from where the power cap held it
        # during the prefill, over some 70 ms. The device-timed figure above never sees that (capturing its
        # graph leaves the GPU idle first), so the end-to-end window starts after at least 24 decode steps.
        e2e_warmup = max(args.warmup, 24)
        stamps = []
        turns = -(-args.batch * PROMPT // sched.cfg.max_step_tokens) + 2
        last_id = sched._next_id + args.batch - 1

        def on_token(seq, tok):
            if seq.id == last_id:
                stamps.append(time.perf_counter())

        ps = prompts(args.batch, PROMPT)
        w = time.perf_counter()
        model.generate(ps, max_tokens=e2e_warmup + args.steps + 1 + turns, temperature=0.0, on_token=on_token)
        windows.append((w, time.perf_counter()))
        e2e_s = stamps[e2e_warmup + args.steps] - stamps[e2e_warmup]
        bucket = g8.bucket
        e2e = {"value": round(args.batch * args.steps / e2e_s, 1), "unit": "tokens/s",
               "h2d_bytes_per_step": 3 * bucket * 4, "d2h_bytes_per_step": (bucket + 1) * 4,
               "ms_per_step": round(e2e_s / args.steps * 1e3, 4), "warmup": e2e_warmup}
        if not args.no_points:
            for b in (1, 64):
                ms_b, ctx_b, _ = decode_device(b, point_steps, args.warmup)
                points[f"decode_b{b}"] = round(b / (ms_b / 1e3), 1)
                fracs[f"decode_b{b}"] = roofline_of(b, ms_b, ctx_b)["frac"]
        metric = "decode tokens/s, %s, bf16, batch %d, %d-token prompts" % (label, args.batch, PROMPT)
        batch_of_value, steps_of_value = args.batch, args.steps
        ms_per_step = ms_step
    launches_per_step = getattr(g8, "launches", 0)
    step_bytes = roofline["bytes_per_step"]
    clocks.stop()

    line = {
        "metric": metric,
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps_of_value, "warmup": args.warmup,
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded random token ids, random weights N(0, 0.02) seed %d" % SEED,
        "config": {
            "model": label, "layers": layers, "layers_of_model": full_layers,
            "hidden_size": E, "heads": nh, "kv_heads": nkv, "head_dim": d, "intermediate_size": ff,
            "vocab_size": vocab, "rms_norm_eps": cfg["rms_norm_eps"], "rope": rope_words,
            "global_batch": batch_of_value, "seq_len": CONTEXT, "prompt_tokens": "16..2048" if mixed else PROMPT,
            "kv_block_size": 16, "decode_context": round(mean_ctx, 1), "prefill_tokens": PREFILL_TOKENS,
            "l2": "no flush: a step reads %.1f GB, far above the 126 MB L2" % (step_bytes / 1e9),
            "parallelism": "1 GPU",
            "settle": "%.1f s idle between the prompts and a decode measurement's warm-up steps" % SETTLE_S,
        },
        "e2e": e2e, "gpu_launches": int(launches_per_step * (point_steps if mixed else args.steps)),
        "launches_per_step": launches_per_step,
        "clocks": clocks.summary(windows), "prefill": prefill, "roofline": roofline, "points": points,
        "points_frac": fracs, "load_seconds": round(load_s, 1), "impl": "ours",
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
