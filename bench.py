#!/usr/bin/env python3
"""Decode and prefill throughput of rllm_b200 on one B200, Llama-3.2-1B shape.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  A "step" is one decode step of a batch of 8 sequences
at the benchmark context (each sequence ends the run holding ``context_len``
tokens).  ``value`` is decoded tokens per second timed on the device with CUDA
events around exactly K steps that stay on the device (graph replay, argmax,
next-token feed-back); ``e2e`` is the same metric through the Python entry
point (``LLM.step``): host token ids in, pinned-memory copy of the step's
inputs to the device, sampled tokens read back to the host, every step.
Weights are random (N(0, 0.02), seed 0), token ids uniform random: synthetic
data, as in the reference's own workloads.  No flush of L2 is needed between
steps: every step reads all weights (2.5 GB) and the live KV cache, far more
than the 126 MB of L2.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LLAMA_1B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 16,
    "hidden_size": 2048, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64,
    "intermediate_size": 8192, "vocab_size": 128256, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    "max_position_embeddings": 131072, "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
    "hidden_act": "silu", "torch_dtype": "bfloat16", "bos_token_id": 128000, "eos_token_id": 128001,
}
CONTEXT_LEN = 4096
BLOCK_SIZE = 16
PREFILL_TOKENS = 2048


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while it runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.time(), line.strip()))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()

    def summary(self, windows):
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for t, line in self.samples:
            if not any(a <= t <= b for a, b in windows):
                continue
            parts = [p.strip() for p in line.split(",")]
            try:
                sm.append(int(parts[0]))
                mx = max(mx, int(parts[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, parts[2:]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


def layer_param_count(c, layers):
    h, i, d = c["hidden_size"], c["intermediate_size"], c["head_dim"]
    nq, nkv = c["num_attention_heads"], c["num_key_value_heads"]
    per_layer = h * (nq + 2 * nkv) * d + nq * d * h + 3 * h * i
    return per_layer * layers


def prefill_flops(c, layers, T):
    linear = 2 * T * layer_param_count(c, layers) + 2 * c["hidden_size"] * c["vocab_size"]
    attn = layers * 4 * c["head_dim"] * c["num_attention_heads"] * T * (T + 1) // 2
    return linear + attn


def decode_bytes(c, layers, batch, ctx_mid):
    weights = 2 * (layer_param_count(c, layers) + c["hidden_size"] * c["vocab_size"])
    kv = batch * ctx_mid * layers * 2 * c["num_key_value_heads"] * c["head_dim"] * 2
    return weights + kv


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the model has (stated in config)")
    ap.add_argument("--context", type=int, default=CONTEXT_LEN)
    ap.add_argument("--no-points", action="store_true", help="skip decode at batch 1 and 64")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "rLLM is a Rust workspace (cargo, Candle and ~300 crates); no Rust toolchain and no "
                          "network here, and its paged CUDA path does not compile (paged_attention.cu:409)"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not measured")
        return 2
    K, W = args.steps, max(3, args.warmup)

    import numpy as np
    import torch

    from rllm_b200 import LLM, SamplingParams
    from rllm_b200.engine.runner import StepEntry
    from rllm_b200.kernels import ops

    cfg = dict(LLAMA_1B)
    layers = args.layers or cfg["num_hidden_layers"]
    cfg["num_hidden_layers"] = layers
    model_dir = tempfile.mkdtemp(prefix="rllm_bench_")
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(cfg, f)
    max_batch = args.batch if args.no_points else max(args.batch, 64)
    pages = max_batch * (-(-args.context // BLOCK_SIZE) + 2) + -(-PREFILL_TOKENS // BLOCK_SIZE) + 64
    t0 = time.time()
    llm = LLM(model_dir, dtype="bf16", max_model_len=args.context, max_num_seqs=max_batch,
              max_num_batched_tokens=8192, long_prefill_token_threshold=8192, block_size=BLOCK_SIZE,
              num_gpu_blocks=pages, enable_prefix_caching=False, random_weights=True, seed=0,
              draw_on_device=True)
    load_s = time.time() - t0
    eng, runner = llm.engine, llm.engine.runner
    rng = np.random.default_rng(0)
    pk = peaks()
    clocks = ClockSampler()
    clocks.start()
    windows = []

    def decode_point(batch, steps, warm, with_e2e):
        """(device tok/s, ms per step, e2e dict or None) at this batch."""
        total_new = 2 * (steps + warm) + 2
        prompt_len = args.context - total_new
        prompts = [[int(t) for t in rng.integers(0, cfg["vocab_size"], size=prompt_len)] for _ in range(batch)]
        sp = SamplingParams(temperature=0.0, max_tokens=total_new, ignore_eos=True)
        ids = [llm.add_request(p, sp) for p in prompts]
        while any(eng.scheduler.requests[i].num_computed < prompt_len for i in ids):
            llm.step()                                         # prefill
        e2e = None
        if with_e2e:
            for _ in range(warm):
                llm.step()
            torch.cuda.synchronize()
            h2d0 = sum(g.h2d_bytes for g in runner.graphs.values())
            a = time.time()
            t_a = time.perf_counter()
            n_tok = 0
            for _ in range(steps):
                n_tok += len(llm.step())
            torch.cuda.synchronize()
            dt = time.perf_counter() - t_a
            windows.append((a, time.time()))
            # host -> device: the step's positions, lengths and block tables from pinned memory, on the steps
            # where a block table changed (the token ids of a decode step are the step before's samples and
            # stay on the device); device -> host: the sampled tokens, every step, and the error words
            h2d = sum(g.h2d_bytes for g in runner.graphs.values()) - h2d0
            e2e = {"value": n_tok / dt, "unit": "tok/s", "h2d_bytes_per_step": int(h2d / steps),
                   "d2h_bytes_per_step": int(batch * 4 + 1), "ms_per_step": 1e3 * dt / steps}
        # the device-timed run goes on from where the requests are
        entries = []
        for i in ids:
            r = eng.scheduler.requests[i]
            assert eng.cache.ensure(i, r.num_computed, r.num_computed + steps + warm)
            entries.append(StepEntry(i, [r.all_token_ids[r.num_computed]], r.num_computed, [0]))
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a = time.time()
        runner.greedy_decode_run(entries, warm + steps, timing=(warm, ev0, ev1))
        torch.cuda.synchronize()
        windows.append((a, time.time()))
        ms = ev0.elapsed_time(ev1)
        runner.check_errors()
        for i in ids:
            llm.abort_request(i)
        return batch * steps / (ms / 1e3), ms / steps, e2e

    # launches of this engine's own kernels in one decode step (counted on an eager step)
    value, ms_step, e2e = decode_point(args.batch, K, W, True)
    points = {}
    if not args.no_points:
        for b in (1, 64):
            pv, _, _ = decode_point(b, min(K, 64), W, False)
            points[f"decode_b{b}"] = round(pv, 1)

    # prefill of one 2,048-token prompt, device-timed
    eng.cache.admit("prefill")
    assert eng.cache.ensure("prefill", 0, PREFILL_TOKENS)
    ptoks = [int(t) for t in rng.integers(0, cfg["vocab_size"], size=PREFILL_TOKENS)]
    entry = [StepEntry("prefill", ptoks, 0, [PREFILL_TOKENS - 1])]
    for _ in range(3):
        runner.step(entry)
    n0 = ops.LAUNCHES[0]
    torch.cuda.synchronize()
    reps = 5
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(reps + 1)]
    a = time.time()
    for i in range(reps):
        evs[i].record()
        runner.step(entry)
    evs[reps].record()
    torch.cuda.synchronize()
    windows.append((a, time.time()))
    prefill_launches = (ops.LAUNCHES[0] - n0) // reps
    p_ms = min(evs[i].elapsed_time(evs[i + 1]) for i in range(reps))
    eng.cache.free("prefill")
    pf = prefill_flops(cfg, layers, PREFILL_TOKENS)
    prefill = {"value": round(PREFILL_TOKENS / (p_ms / 1e3), 1), "tokens": PREFILL_TOKENS, "ms": round(p_ms, 3),
               "frac": round(pf / (p_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}

    # own kernel launches of one decode step, counted on an eager step of the same shape
    eng.cache.admit("count")
    assert eng.cache.ensure("count", 0, 8)
    was = runner.capture_graphs
    runner.capture_graphs = False
    n0 = ops.LAUNCHES[0]
    runner.step([StepEntry("count", [1], 0, [0])])
    per_step = ops.LAUNCHES[0] - n0 + 2                        # + argmax and the feed-back kernel
    runner.capture_graphs = was
    eng.cache.free("count")
    torch.cuda.synchronize()
    clocks.stop()

    ctx_mid = args.context - K // 2
    nbytes = decode_bytes(cfg, layers, args.batch, ctx_mid)
    achieved = nbytes / (ms_step / 1e3) / 1e9
    out = {
        "metric": "decode tok/s at batch 8 (Llama-3.2-1B shape, bf16)", "value": round(value, 1),
        "unit": "tok/s", "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": round(ms_step, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic (random weights N(0,0.02) seed 0, uniform random token ids)", "impl": "ours",
        "config": {"model": "Llama-3.2-1B shape", "layers": layers, "layers_of_model": LLAMA_1B["num_hidden_layers"],
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                   "global_batch": args.batch, "seq_len": args.context, "block_size": BLOCK_SIZE,
                   "prefill_tokens": PREFILL_TOKENS, "parallelism": "single GPU", "cuda_graphs": True,
                   "l2": "inputs larger than L2 (2.5 GB of weights per step)", "peaks": pk["source"],
                   "load_s": round(load_s, 1)},
        "e2e": {k: (round(v, 3) if isinstance(v, float) else v) for k, v in e2e.items()},
        "gpu_launches": int(per_step * K),
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "clocks": clocks.summary(windows),
        "launches_per_decode_step": int(per_step), "launches_per_prefill": int(prefill_launches),
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
