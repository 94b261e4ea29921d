#!/usr/bin/env python3
"""Decode and prefill throughput of rllm_b200 on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--no-workloads]

Prints ONE JSON line.

Headline (Llama-3.2-1B shape, bfloat16, random weights): a batch of 8 sequences, each holding a 2,048-token
prompt, decodes greedily; a "step" is one decode step.  After W warm-up steps exactly K steps are timed
(K = 256 by default: the sequences then go from 2,048 to 2,304 tokens).  ``value`` is decoded tokens per
second timed on the device with CUDA events around K steps that stay on the device (graph replay, argmax,
next-token feed-back), the median of three such runs; SETTLE_STEPS further untimed steps come before the W warm-up steps of every
device-timed point (``config.settle_steps``: the first steps behind the prompts run slower than the rest).  ``e2e`` is the same metric through the Python entry point (``LLM.step``): host token
ids in, pinned-memory copy of the step's inputs to the device, sampled tokens read back to the host, every
step, timed by the host's clock between two device synchronisations.  ``points`` holds the same two figures
at batch 1 and 64, and device-timed decoding at the full context of 4,096 tokens.  ``prefill`` is one
2,048-token prompt as one step, device-timed as a burst after ``prefill_idle_s`` seconds of rest (its ``frac`` is
against the burst peak of the library's product).  ``roofline`` is the decode step against the measured copy bandwidth: the
bytes it has to read (every weight once, the keys and values of the live requests) over its time.

``workloads`` holds two serving runs through ``LLM.add_request`` / ``LLM.step`` with continuous batching:
the Llama-3.2-3B shape (32 requests, prompts of 128 to 4,096 tokens, at most 4,096 tokens a step, 128 tokens
each at temperature 0.8) and the Llama-3.1-8B shape (16 requests that share a 1,024-token prefix, 512-token
portions beside decoded tokens, 256 greedy tokens, prefix caching on), after the reference's synthetic
workload generator (crates/rllm-bench/src/workload.rs:74-90).  Each gives wall time, generated and prompt
tokens per second, preemptions, prefix-hit tokens, steps launched ahead, and the fraction of the roofline:
the sum over the steps that ran of max(flops / peak flops, bytes / peak bandwidth), over the wall time.

``library_standin`` is not the reference (which cannot be built here): it is the same model shape written
with PyTorch's library operators only, timed the same way, so that the figures above have something
beside the roofline to stand against.

Weights are random (N(0, 0.02), seed 0), token ids uniform random: synthetic data, as in the reference's own
workloads.  No flush of L2 is needed between steps: every step reads all weights (2.5 GB and more) and the
live KV cache, far more than the 126 MB of L2.
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


def llama(layers, hidden, heads, kv_heads, head_dim, inter, factor, tied):
    return {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": layers,
        "hidden_size": hidden, "num_attention_heads": heads, "num_key_value_heads": kv_heads, "head_dim": head_dim,
        "intermediate_size": inter, "vocab_size": 128256, "rope_theta": 500000.0,
        "rope_scaling": {"rope_type": "llama3", "factor": factor, "low_freq_factor": 1.0,
                         "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
        "max_position_embeddings": 131072, "rms_norm_eps": 1e-5, "tie_word_embeddings": tied,
        "hidden_act": "silu", "torch_dtype": "bfloat16", "bos_token_id": 128000, "eos_token_id": 128001,
    }


LLAMA_1B = llama(16, 2048, 32, 8, 64, 8192, 32.0, True)
LLAMA_3B = llama(28, 3072, 24, 8, 128, 8192, 32.0, True)
LLAMA_8B = llama(32, 4096, 32, 8, 128, 14336, 8.0, False)
CONTEXT_LEN = 4096
PROMPT_LEN = 2048
DECODE_TOKENS = 256
BLOCK_SIZE = 16
PREFILL_TOKENS = 2048
PREFILL_IDLE_S = 1.5       # the GPU rests this long before the prefill point's burst (see there)
SETTLE_STEPS = 48          # untimed decode steps of a device-timed point before its warm-up steps (see device_point)


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


# -- what a step has to read and to compute ---------------------------------------------------------------
def layer_param_count(c, layers):
    h, i, d = c["hidden_size"], c["intermediate_size"], c["head_dim"]
    nq, nkv = c["num_attention_heads"], c["num_key_value_heads"]
    per_layer = h * (nq + 2 * nkv) * d + nq * d * h + 3 * h * i
    return per_layer * layers


def kv_bytes_per_token(c, layers):
    return layers * 2 * c["num_key_value_heads"] * c["head_dim"] * 2


def prefill_flops(c, layers, T):
    linear = 2 * T * layer_param_count(c, layers) + 2 * c["hidden_size"] * c["vocab_size"]
    attn = layers * 4 * c["head_dim"] * c["num_attention_heads"] * T * (T + 1) // 2
    return linear + attn


def decode_bytes(c, layers, batch, ctx_mid):
    weights = 2 * (layer_param_count(c, layers) + c["hidden_size"] * c["vocab_size"])
    return weights + batch * ctx_mid * kv_bytes_per_token(c, layers)


def step_floor_seconds(c, layers, scheduled, pk):
    """The least time a step of these (start, tokens, wants logits) entries can take: the larger of its
    flops over the tensor peak and the bytes it must read over the copy bandwidth."""
    tokens = sum(n for _, n, _ in scheduled)
    rows = sum(1 for _, _, w in scheduled if w)
    flops = 2 * tokens * layer_param_count(c, layers) + 2 * rows * c["hidden_size"] * c["vocab_size"]
    nbytes = 2 * (layer_param_count(c, layers) + c["hidden_size"] * c["vocab_size"])
    for start, n, _ in scheduled:
        # token i of the portion sees start + i + 1 keys; the keys are read once per portion
        flops += layers * 4 * c["head_dim"] * c["num_attention_heads"] * (n * start + n * (n + 1) // 2)
        nbytes += (start + n) * kv_bytes_per_token(c, layers)
    return max(flops / (pk["bf16_tflops"] * 1e12), nbytes / (pk["hbm_gbs"] * 1e9))


def write_config(cfg):
    d = tempfile.mkdtemp(prefix="rllm_bench_")
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    return d


# -- a serving workload through the entry point -------------------------------------------------------------
def run_workload(cfg, prompts, params, pk, windows, warm_prompts, **llm_kw):
    """All requests are added at once and stepped until none is left.  A workload of the same shape with
    other tokens (``warm_prompts``) runs once untimed first (graphs are captured, libraries warmed, and
    nothing of the timed prompts is in the prefix cache), then the workload itself three times, each timed
    by the host's clock with the prefix cache emptied in between; the pass with the median wall time is
    reported."""
    import torch

    from rllm_b200 import LLM
    layers = cfg["num_hidden_layers"]
    t0 = time.time()
    llm = LLM(write_config(cfg), dtype="bf16", random_weights=True, seed=0, draw_on_device=True,
              block_size=BLOCK_SIZE, **llm_kw)
    load_s = time.time() - t0
    eng = llm.engine
    results = []
    for timed in (False, True, True, True):
        before = dict(eng.stats())
        floor = 0.0
        n_out = n_prompt_steps = 0
        prompt_tokens = prompt_time = 0.0
        torch.cuda.synchronize()
        a_wall = time.time()
        a = time.perf_counter()
        for p, sp in zip(prompts if timed else warm_prompts, params):
            llm.add_request(p, sp)
        while llm.has_work():
            t_step = time.perf_counter()
            outs = llm.step()
            sched = eng.last_schedule
            n_out += len(outs)
            if sched is not None and sched.scheduled:
                floor += step_floor_seconds(cfg, layers, [(s.start, s.num_tokens, s.want_logits)
                                                          for s in sched.scheduled], pk)
                if sched.num_prefill_tokens:
                    # a step with prompt tokens is never launched ahead: its host time is its own
                    torch.cuda.synchronize()
                    prompt_time += time.perf_counter() - t_step
                    prompt_tokens += sched.num_prefill_tokens
                    n_prompt_steps += 1
        torch.cuda.synchronize()
        wall = time.perf_counter() - a
        eng.runner.check_errors()
        if timed:
            windows.append((a_wall, time.time()))
            st = eng.stats()
            results.append({
                "wall_s": round(wall, 4), "requests": len(prompts), "generated_tokens": n_out,
                "prompt_tokens": sum(len(p) for p in prompts),
                "output_tok_s": round(n_out / wall, 1),
                "total_tok_s": round((n_out + prompt_tokens) / wall, 1),
                "prefill_tok_s": round(prompt_tokens / prompt_time, 1) if prompt_time else None,
                "prompt_tokens_computed": int(prompt_tokens), "steps": st["num_steps"] - before["num_steps"],
                "steps_with_prompt_tokens": n_prompt_steps,
                "preemptions": st["num_preemptions"] - before["num_preemptions"],
                "prefix_hit_tokens": st["prefix_hit_tokens"] - before["prefix_hit_tokens"],
                "steps_launched_ahead": st["num_steps_ahead"] - before["num_steps_ahead"],
                "roofline_frac": round(floor / wall, 4), "cache_pages": eng.num_pages[0],
                "layers": layers, "load_s": round(load_s, 1),
            })
            # the prompts of this pass must not be found in the prefix cache by the next one
            if eng.cache.prefix_caching:
                eng.cache.reset_prefix_cache()
    results.sort(key=lambda r: r["wall_s"])
    result = dict(results[len(results) // 2], timed_passes=len(results),
                  wall_s_all=" ".join(str(r["wall_s"]) for r in results))
    del llm, eng
    import gc
    gc.collect()
    torch.cuda.empty_cache()
    return result


# -- a stand-in for the missing reference arm: the same model through library operators only --------------
def library_standin(cfg, batches, prompt_len, steps, warm, windows):
    """The reference cannot be built here (no Rust toolchain), so nothing of this engine can be compared with
    it.  This is NOT the reference: it is the same Llama shape written with PyTorch's library operators
    alone (torch.mm -> cuBLAS, scaled_dot_product_attention, rms_norm, silu), random weights, a contiguous
    key/value cache of exactly the context (no paging, no scheduler), greedy decoding captured in one CUDA
    graph a batch size, timed with CUDA events like ``value``.  It says what stock library kernels reach on
    this GPU for the same arithmetic; none of this engine's code runs in it."""
    import torch
    import torch.nn.functional as F
    dev = torch.device("cuda:0")
    L, H, I = cfg["num_hidden_layers"], cfg["hidden_size"], cfg["intermediate_size"]
    nq, nkv, d, V = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["vocab_size"]
    eps = cfg["rms_norm_eps"]
    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *shape: (torch.randn(*shape, generator=g, device=dev) * 0.02).bfloat16()
    emb = rnd(V, H)
    layers = [dict(qkv=rnd((nq + 2 * nkv) * d, H), o=rnd(H, nq * d), gu=rnd(2 * I, H), down=rnd(H, I),
                   n1=torch.ones(H, device=dev, dtype=torch.bfloat16), n2=torch.ones(H, device=dev, dtype=torch.bfloat16))
              for _ in range(L)]
    nf = torch.ones(H, device=dev, dtype=torch.bfloat16)
    inv = 1.0 / (cfg["rope_theta"] ** (torch.arange(0, d, 2, device=dev, dtype=torch.float32) / d))

    def rope(x, pos):                                  # x [B, T, heads, d], pos [B, T]
        ang = pos[..., None].float() * inv
        cos, sin = ang.cos()[:, :, None, :], ang.sin()[:, :, None, :]
        a, b = x[..., : d // 2].float(), x[..., d // 2:].float()
        return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1).to(x.dtype)

    def forward(ids, pos, kc, vc, causal):
        """ids, pos [B, T]; kc, vc: per layer [B, nkv, C, d]; the T tokens sit at positions pos."""
        B, T = ids.shape
        x = emb[ids]
        for w, k_l, v_l in zip(layers, kc, vc):
            h = F.rms_norm(x, (H,), w["n1"], eps)
            qkv = (h.view(B * T, H) @ w["qkv"].t()).view(B, T, nq + 2 * nkv, d)
            q, k, v = rope(qkv[:, :, :nq], pos), rope(qkv[:, :, nq:nq + nkv], pos), qkv[:, :, nq + nkv:]
            idx = pos[:, None, :, None].expand(B, nkv, T, d)
            k_l.scatter_(2, idx, k.transpose(1, 2))
            v_l.scatter_(2, idx, v.transpose(1, 2))
            if causal:
                att = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                                     is_causal=True, enable_gqa=True)
            else:
                att = F.scaled_dot_product_attention(q.transpose(1, 2), k_l, v_l, enable_gqa=True)
            x = x + (att.transpose(1, 2).reshape(B * T, nq * d) @ w["o"].t()).view(B, T, H)
            h = F.rms_norm(x, (H,), w["n2"], eps)
            gu = h.view(B * T, H) @ w["gu"].t()
            x = x + ((F.silu(gu[:, :I]) * gu[:, I:]) @ w["down"].t()).view(B, T, H)
        last = F.rms_norm(x[:, -1], (H,), nf, eps)
        return (last @ emb.t()).float().argmax(dim=-1)

    out = {"what": "PyTorch library operators only (cuBLAS, SDPA), contiguous cache, CUDA graph; not the reference"}
    with torch.no_grad():
        for B in batches:
            C = prompt_len + warm + steps                 # the cache holds exactly what the run needs
            kc = [torch.randn(B, nkv, C, d, device=dev).bfloat16() for _ in range(L)]
            vc = [torch.randn(B, nkv, C, d, device=dev).bfloat16() for _ in range(L)]
            ids = torch.randint(0, V, (B, 1), device=dev)
            pos = torch.full((B, 1), prompt_len, device=dev, dtype=torch.long)

            def step():
                nxt = forward(ids, pos, kc, vc, causal=False)
                ids.copy_(nxt[:, None])
            # every step attends over the whole cache (a few more keys than the engine's sequences hold on
            # average: C against prompt_len + warm + steps / 2)
            side = torch.cuda.Stream()
            with torch.cuda.stream(side):
                for _ in range(3):
                    step()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step()
            for _ in range(warm):
                graph.replay()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a = time.time()
            e0.record()
            for _ in range(steps):
                graph.replay()
            e1.record()
            torch.cuda.synchronize()
            windows.append((a, time.time()))
            out[f"decode_b{B}"] = round(B * steps / (e0.elapsed_time(e1) / 1e3), 1)
            del kc, vc, graph
            torch.cuda.empty_cache()
        T = PREFILL_TOKENS
        kc = [torch.zeros(1, nkv, T, d, device=dev, dtype=torch.bfloat16) for _ in range(L)]
        vc = [torch.zeros(1, nkv, T, d, device=dev, dtype=torch.bfloat16) for _ in range(L)]
        ids = torch.randint(0, V, (1, T), device=dev)
        pos = torch.arange(T, device=dev)[None]
        for _ in range(3):
            forward(ids, pos, kc, vc, causal=True)
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(6)]
        torch.cuda.synchronize()
        a = time.time()
        for i in range(5):
            evs[i].record()
            forward(ids, pos, kc, vc, causal=True)
        evs[5].record()
        torch.cuda.synchronize()
        windows.append((a, time.time()))
        ms = min(evs[i].elapsed_time(evs[i + 1]) for i in range(5))
        out["prefill_tok_s"] = round(T / (ms / 1e3), 1)
        out["prefill_ms"] = round(ms, 3)
    del emb, layers, kc, vc
    torch.cuda.empty_cache()
    return out


def workload_3b(pk, windows):
    """BASELINE.json configs[3]: 32 requests, prompts uniform in [128, 4096], at most 4,096 tokens a step with
    chunked prefill, 128 tokens each at temperature 0.8, context 8,192."""
    import numpy as np

    from rllm_b200 import SamplingParams
    rng = np.random.default_rng(3)
    lengths = rng.integers(128, 4097, size=32)
    prompts = [[int(t) for t in rng.integers(0, 128256, size=int(n))] for n in lengths]
    warm = [[int(t) for t in rng.integers(0, 128256, size=int(n))] for n in lengths]
    params = [SamplingParams(temperature=0.8, seed=1000 + i, max_tokens=128, ignore_eos=True) for i in range(32)]
    return run_workload(LLAMA_3B, prompts, params, pk, windows, warm, max_model_len=8192, max_num_seqs=32,
                        max_num_batched_tokens=4096, long_prefill_token_threshold=4096,
                        enable_prefix_caching=False)


def workload_8b(pk, windows):
    """BASELINE.json configs[4]: 16 requests that share a 1,024-token prefix, followed by suffixes of 256 to
    2,048 tokens of their own; 512-token portions beside decoded tokens; 256 greedy tokens each; context 8,192;
    prefix caching on."""
    import numpy as np

    from rllm_b200 import SamplingParams
    rng = np.random.default_rng(4)
    lengths = rng.integers(256, 2049, size=16)
    shared, shared_warm = ([int(t) for t in rng.integers(0, 128256, size=1024)] for _ in range(2))
    prompts = [shared + [int(t) for t in rng.integers(0, 128256, size=int(n))] for n in lengths]
    warm = [shared_warm + [int(t) for t in rng.integers(0, 128256, size=int(n))] for n in lengths]
    params = [SamplingParams(temperature=0.0, max_tokens=256, ignore_eos=True) for _ in range(16)]
    return run_workload(LLAMA_8B, prompts, params, pk, windows, warm, max_model_len=8192, max_num_seqs=16,
                        max_num_batched_tokens=4096, long_prefill_token_threshold=512,
                        enable_prefix_caching=True)


def main():
    global SETTLE_STEPS
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=DECODE_TOKENS)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the model has (stated in config)")
    ap.add_argument("--prompt-len", type=int, default=PROMPT_LEN)
    ap.add_argument("--no-points", action="store_true", help="skip the other batch sizes and contexts")
    ap.add_argument("--no-workloads", action="store_true", help="skip the 3B and 8B serving workloads")
    ap.add_argument("--no-standin", action="store_true", help="skip the library-operator stand-in")
    ap.add_argument("--settle-steps", type=int, default=SETTLE_STEPS,
                    help="untimed decode steps of a device-timed point before its warm-up steps (0 for a short capture under a profiler)")
    args = ap.parse_args()
    SETTLE_STEPS = max(0, args.settle_steps)

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "rLLM is a Rust workspace (cargo, Candle and ~300 crates); no Rust toolchain and no "
                          "network here, and its paged CUDA path does not compile (paged_attention.cu:409)"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not measured")
        return 2
    K, W = args.steps, max(3, args.warmup)
    if args.prompt_len + K + W + SETTLE_STEPS + 4 > CONTEXT_LEN:
        print(f"bench.py: a prompt of {args.prompt_len} tokens and {K} + {W} steps do not fit the context of {CONTEXT_LEN}")
        return 2

    import numpy as np
    import torch

    from rllm_b200 import LLM, SamplingParams
    from rllm_b200.engine.runner import StepEntry
    from rllm_b200.kernels import ops

    cfg = dict(LLAMA_1B)
    layers = args.layers or cfg["num_hidden_layers"]
    cfg["num_hidden_layers"] = layers
    model_dir = write_config(cfg)
    max_batch = args.batch if args.no_points else max(args.batch, 64)
    pages = max_batch * (-(-CONTEXT_LEN // BLOCK_SIZE) + 2) + -(-PREFILL_TOKENS // BLOCK_SIZE) + 64
    t0 = time.time()
    llm = LLM(model_dir, dtype="bf16", max_model_len=CONTEXT_LEN, max_num_seqs=max_batch,
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

    def e2e_point(batch, prompt_len, steps, warm):
        """Through ``LLM.step``: tokens a second, ms a step, bytes to and from the device a step."""
        prompts = [[int(t) for t in rng.integers(0, cfg["vocab_size"], size=prompt_len)] for _ in range(batch)]
        # no request may end inside the timed steps (those whose prompts are computed first decode a few
        # tokens while the others' prompts are still being computed)
        sp = SamplingParams(temperature=0.0, max_tokens=CONTEXT_LEN - prompt_len, ignore_eos=True)
        ids = [llm.add_request(p, sp) for p in prompts]
        while any(eng.scheduler.requests[i].num_computed < prompt_len for i in ids):
            llm.step()                                         # the prompts
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
        assert n_tok == batch * steps, (n_tok, batch, steps)
        # host -> device: the step's positions, lengths and block tables from pinned memory, on the steps
        # where a block table changed (the token ids of a decode step are the step before's samples and
        # stay on the device); device -> host: the sampled tokens, every step, and the error words
        h2d = sum(g.h2d_bytes for g in runner.graphs.values()) - h2d0
        for i in ids:
            llm.abort_request(i)
        return {"value": n_tok / dt, "unit": "tok/s", "h2d_bytes_per_step": int(h2d / steps),
                "d2h_bytes_per_step": int(batch * 4 + 1), "ms_per_step": 1e3 * dt / steps}

    def device_point(batch, prompt_len, steps, warm):
        """(tokens a second, ms a step) timed on the device around ``steps`` steps that stay there, every
        sequence holding ``prompt_len`` tokens when they begin.  The step function is driven directly.
        SETTLE_STEPS more untimed steps come before the ``warm`` ones: right behind the prompts (tens of
        milliseconds at the power cap) the first decode steps run 3 to 6 % slower than the rest."""
        warm += SETTLE_STEPS
        ids = [f"dev{i}" for i in range(batch)]
        for i in ids:
            eng.cache.admit(i)
            assert eng.cache.ensure(i, 0, prompt_len + steps + warm + 1)
        per_step = max(1, 8192 // prompt_len)
        for a in range(0, batch, per_step):                    # the prompts, some at a time
            runner.step([StepEntry(i, [int(t) for t in rng.integers(0, cfg["vocab_size"], size=prompt_len)], 0, [])
                         for i in ids[a:a + per_step]])
        entries = [StepEntry(i, [int(rng.integers(0, cfg["vocab_size"]))], prompt_len, [0]) for i in ids]
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a = time.time()
        runner.greedy_decode_run(entries, warm + steps, timing=(warm, ev0, ev1))
        torch.cuda.synchronize()
        windows.append((a, time.time()))
        ms = ev0.elapsed_time(ev1)
        runner.check_errors()
        for i in ids:
            eng.cache.free(i)
        return batch * steps / (ms / 1e3), ms / steps

    def frac(batch, ms, ctx_mid):
        return decode_bytes(cfg, layers, batch, ctx_mid) / (ms / 1e3) / 1e9 / pk["hbm_gbs"]

    P = args.prompt_len
    ctx_mid = P + SETTLE_STEPS + W + K // 2
    e2e = e2e_point(args.batch, P, K, W)
    # three such runs, each with requests and pages of its own (where the pages lie moves the step by a few
    # per cent); the median is reported
    runs = sorted((device_point(args.batch, P, K, W) for _ in range(3)), key=lambda r: r[1])
    value, ms_step = runs[1]
    points = {}
    if not args.no_points:
        for b in (1, 64):
            pv, pms = device_point(b, P, K, W)
            pe = e2e_point(b, P, K, W)
            points[f"decode_b{b}"] = round(pv, 1)
            points[f"decode_b{b}_e2e"] = round(pe["value"], 1)
            points[f"decode_b{b}_hbm_frac"] = round(frac(b, pms, ctx_mid), 4)
        # the whole context of the configuration: sequences that end the run with 4,096 tokens
        k4 = min(K, 64)
        for b in (1, 8, 64):
            pv, pms = device_point(b, CONTEXT_LEN - (k4 + W + SETTLE_STEPS) - 4, k4, W)      # ends with 4,092 tokens
            points[f"decode_b{b}_ctx4096"] = round(pv, 1)
            points[f"decode_b{b}_ctx4096_hbm_frac"] = round(frac(b, pms, CONTEXT_LEN - 4 - k4 // 2), 4)

    # prefill of one 2,048-token prompt, device-timed
    eng.cache.admit("prefill")
    assert eng.cache.ensure("prefill", 0, PREFILL_TOKENS)
    ptoks = [int(t) for t in rng.integers(0, cfg["vocab_size"], size=PREFILL_TOKENS)]
    entry = [StepEntry("prefill", ptoks, 0, [PREFILL_TOKENS - 1])]
    for _ in range(3):
        runner.step(entry)
    n0 = ops.LAUNCHES[0]
    torch.cuda.synchronize()
    # A burst, like the peak it is divided by: the GPU rests PREFILL_IDLE_S first (right behind other work the
    # same prefill takes 4.5 to 4.9 ms instead of 4.4 under the power cap, and its time then says more about
    # what ran before it than about the prefill), then two more untimed repetitions.
    time.sleep(PREFILL_IDLE_S)
    for _ in range(2):
        runner.step(entry)
    torch.cuda.synchronize()
    n0 = ops.LAUNCHES[0]
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

    workloads = {}
    standin = None
    del llm, eng, runner
    import gc
    gc.collect()
    torch.cuda.empty_cache()
    if not args.no_standin:
        try:
            standin = library_standin(cfg, (args.batch,) if args.no_points else (1, args.batch, 64), P, min(K, 64), W,
                                      windows)
        except Exception as e:                             # a stand-in must never take the measurement down with it
            standin = {"unavailable": f"{type(e).__name__}: {e}"[:200]}
        gc.collect()
        torch.cuda.empty_cache()
    if not args.no_workloads and args.layers is None:
        workloads["llama3b_continuous_batching"] = workload_3b(pk, windows)
        workloads["llama8b_shared_prefix"] = workload_8b(pk, windows)
    clocks.stop()

    nbytes = decode_bytes(cfg, layers, args.batch, ctx_mid)
    achieved = nbytes / (ms_step / 1e3) / 1e9
    out = {
        "metric": f"decode tok/s at batch {args.batch}, 2,048-token prompts + 256 tokens (Llama-3.2-1B shape, bf16)",
        "value": round(value, 1),
        "unit": "tok/s", "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": round(ms_step, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic (random weights N(0,0.02) seed 0, uniform random token ids)", "impl": "ours",
        "config": {"model": "Llama-3.2-1B shape", "layers": layers, "layers_of_model": LLAMA_1B["num_hidden_layers"],
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                   "global_batch": args.batch, "seq_len": P + SETTLE_STEPS + W + K, "prompt_len": P, "context_cap": CONTEXT_LEN,
                   "block_size": BLOCK_SIZE, "prefill_tokens": PREFILL_TOKENS, "parallelism": "single GPU",
                   "cuda_graphs": True, "l2": "inputs larger than L2 (2.5 GB of weights per step)",
                   "peaks": pk["source"], "settle_steps": SETTLE_STEPS},
        "load_s": round(load_s, 1), "value_runs_ms": " ".join(f"{r[1]:.4f}" for r in runs),
        "e2e": {k: (round(v, 3) if isinstance(v, float) else v) for k, v in e2e.items()},
        "gpu_launches": int(per_step * K),
        "prefill": prefill, "prefill_idle_s": PREFILL_IDLE_S,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "workloads": workloads,
        "library_standin": standin,
        "clocks": clocks.summary(windows),
        "launches_per_decode_step": int(per_step), "launches_per_prefill": int(prefill_launches),
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
