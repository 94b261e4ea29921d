"""Timing of single kernels at the sizes of a model, for profiling.

    python -m rllm_b200.kernels.microbench attention_decode --batch 8 --context 4096
    python -m rllm_b200.kernels.microbench attention_prefill --tokens 2048 [--impl tcgen05]
    python -m rllm_b200.kernels.microbench gemm_small_m --rows 8 [--variant residual|rstd]
    python -m rllm_b200.kernels.microbench gemm_tcgen05 --rows 2048

Sizes default to the Llama-3.2-1B shape (32 heads, 8 kv heads, head 64, hidden
2048, intermediate 8192).  Times are CUDA-event times over ``--iters`` launches
after warm-up; inputs rotate over several buffers larger than L2 together, so
that weights and caches come from HBM as in a model step.  One line per case:
microseconds, and GB/s (memory-bound kernels) or TFLOP/s (products, attention
over prompts).
"""
from __future__ import annotations

import argparse
import math
import sys

import torch

from . import ops

DEV = "cuda:0"


def time_us(fn, iters: int, warmup: int = 3) -> float:
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / iters


def time_graph_us(fn, iters: int) -> float:
    """Back-to-back launches inside one CUDA graph: no host gaps between kernels."""
    for i in range(3):
        fn(i)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        with torch.cuda.graph(g):
            for i in range(iters):
                fn(i)
    torch.cuda.synchronize()
    g.replay()                      # the first replay also uploads the graph
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / iters


def attention_decode(args) -> None:
    nq, nkv, d, page = args.heads, args.kv_heads, args.head_dim, args.page
    B, ctx = args.batch, args.context
    pages = B * (ctx // page) + 8
    nc = max(2, min(8, int(300e6 // (pages * nkv * page * d * 4)) + 1))
    caches = [(torch.randn(pages, nkv, page, d, device=DEV).bfloat16(),
               torch.randn(pages, nkv, page, d, device=DEV).bfloat16()) for _ in range(nc)]
    table = torch.randperm(pages - 8, device=DEV).int().view(B, ctx // page).contiguous()
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    q = torch.randn(B, nq * d, device=DEV).bfloat16()
    out = torch.empty_like(q)
    seq_lens = torch.full((B,), ctx, dtype=torch.int32, device=DEV)
    ws = torch.empty(ops.attention_decode_workspace(B, nq, d, ctx), device=DEV)
    scale = 1 / math.sqrt(d)

    def run(i):
        k, v = caches[i % nc]
        ops.attention_decode_bf16(q, nq * d, out, k, v, table, seq_lens, B, ctx, nq, nkv, d, 0, scale, err, ws)
    us = time_graph_us(run, args.iters)
    nbytes = B * ctx * nkv * d * 2 * 2
    print(f"attention_decode batch {B} context {ctx}: {us:.1f} us, {nbytes / us / 1e3:.0f} GB/s of K and V")


def attention_prefill(args) -> None:
    nq, nkv, d, page = args.heads, args.kv_heads, args.head_dim, args.page
    T = args.tokens
    pages = T // page + 8
    k = torch.randn(pages, nkv, page, d, device=DEV).bfloat16()
    v = torch.randn(pages, nkv, page, d, device=DEV).bfloat16()
    table = torch.randperm(pages - 8, device=DEV).int().view(1, T // page).contiguous()
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    q = torch.randn(T, nq * d, device=DEV).bfloat16()
    out = torch.empty_like(q)
    seq_lens = torch.tensor([T], dtype=torch.int32, device=DEV)
    q_start = torch.tensor([0, T], dtype=torch.int32, device=DEV)
    scale = 1 / math.sqrt(d)

    fn = ops.attention_prefill_tcgen05 if args.impl == "tcgen05" else ops.attention_prefill_bf16

    def run(i):
        fn(q, nq * d, out, k, v, table, q_start, seq_lens, 0, 1, T, nq, nkv, d, 0, scale, err)
    us = time_us(run, args.iters)
    flops = 4 * d * nq * T * (T + 1) // 2
    print(f"attention_prefill ({args.impl}) tokens {T}: {us:.1f} us, {flops / us / 1e6:.0f} TFLOP/s (causal)")
    if int(err.item()):
        print(f"error word {int(err.item())}", file=sys.stderr)


def _shapes(args):
    H, I = args.hidden, args.intermediate
    qkv = (args.heads + 2 * args.kv_heads) * args.head_dim
    return [("qkv", qkv, H), ("o_proj", H, args.heads * args.head_dim), ("gate_up", 2 * I, H), ("down", H, I)]


def gemm_small_m(args) -> None:
    """--variant plain: the four projections.  residual: o and down adding into a float32 stream and
    preparing the next norm.  rstd: qkv and gate_up applying the norm's row factors."""
    M = args.rows
    for name, N, K in _shapes(args):
        silu = name == "gate_up"
        if args.only and name != args.only:
            continue
        if args.variant == "residual" and name not in ("o_proj", "down"):
            continue
        if args.variant == "rstd" and name not in ("qkv", "gate_up"):
            continue
        nw = max(2, int(300e6 // (N * K * 2)) + 1)
        ws = [(torch.randn(N, K, device=DEV) * 0.02).bfloat16() for _ in range(nw)]
        x = torch.randn(M, K, device=DEV).bfloat16()
        out = torch.empty(M, N // 2 if silu else N, device=DEV, dtype=torch.bfloat16)
        h = torch.randn(M, N, device=DEV)
        wn = torch.ones(N, device=DEV)
        parts = torch.ones(128, M, device=DEV)

        def run(i):
            if args.variant == "residual":
                ops.gemm_small_m_residual(x, ws[i % nw], h, wn)
            elif args.variant == "rstd":
                ops.gemm_small_m_rstd(x, parts, 1e-5, ws[i % nw], out, "silu_mul" if silu else "store")
            else:
                ops.gemm_small_m(x, ws[i % nw], out, "silu_mul" if silu else "store")
        us = time_graph_us(run, args.iters)
        print(f"gemm_small_m ({args.variant}) rows {M} {name}{' +silu' if silu else ''} [{N} x {K}]: {us:.1f} us, "
              f"{N * K * 2 / us / 1e3:.0f} GB/s of weight")


def gemm_tcgen05(args) -> None:
    M = args.rows
    for name, N, K in _shapes(args):
        if args.only and name != args.only:
            continue
        w = (torch.randn(N, K, device=DEV) * 0.02).bfloat16()
        x = torch.randn(M, K, device=DEV).bfloat16()
        silu = name == "gate_up"
        out = torch.empty(M, N // 2 if silu else N, device=DEV, dtype=torch.bfloat16)

        def run(i):
            ops.gemm_tcgen05(x, w, out, "silu_mul" if silu else "store")
        us = time_us(run, args.iters)
        print(f"gemm_tcgen05 rows {M} {name}{' +silu' if silu else ''} [{N} x {K}]: {us:.1f} us, "
              f"{2 * M * N * K / us / 1e6:.0f} TFLOP/s")
    ops.check_gemm_errors(torch.device(DEV))


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="python -m rllm_b200.kernels.microbench", description=__doc__.split("\n\n")[0])
    p.add_argument("kernel", choices=["attention_decode", "attention_prefill", "gemm_small_m", "gemm_tcgen05"])
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--context", type=int, default=4096)
    p.add_argument("--tokens", type=int, default=2048)
    p.add_argument("--rows", type=int, default=8)
    p.add_argument("--iters", type=int, default=20)
    p.add_argument("--heads", type=int, default=32)
    p.add_argument("--kv-heads", type=int, default=8)
    p.add_argument("--head-dim", type=int, default=64)
    p.add_argument("--hidden", type=int, default=2048)
    p.add_argument("--intermediate", type=int, default=8192)
    p.add_argument("--page", type=int, default=16)
    p.add_argument("--variant", choices=["plain", "residual", "rstd"], default="plain",
                   help="gemm_small_m: which epilogue / operand form")
    p.add_argument("--only", choices=["qkv", "o_proj", "gate_up", "down"], default=None,
                   help="gemm_small_m, gemm_tcgen05: this projection alone")
    p.add_argument("--impl", choices=["mma", "tcgen05"], default="mma",
                   help="attention_prefill: the mma.sync kernel or the tcgen05 kernel")
    args = p.parse_args(argv)
    if not torch.cuda.is_available():
        print("microbench needs a CUDA device", file=sys.stderr)
        return 1
    {"attention_decode": attention_decode, "attention_prefill": attention_prefill,
     "gemm_small_m": gemm_small_m, "gemm_tcgen05": gemm_tcgen05}[args.kernel](args)
    return 0


if __name__ == "__main__":
    sys.exit(main())
