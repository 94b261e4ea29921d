"""The ``rllm`` command line.

    rllm generate <model_dir> --prompt-ids 1,2,3 [--max-tokens 64] [--temperature 1.0] ...
    rllm init-random <model_dir> --config config.json [--seed 0] [--dtype bfloat16]

``generate`` is the reference's offline example made real
(examples/offline_generate.rs:5-21: ``--model/-m``, ``--prompt/-p``,
``--max-tokens`` 64, ``--temperature`` 1.0 with 0 = greedy; the example only
prints its arguments).  Prompts are token ids here.  Engine options carry the
names and defaults of ``rllm serve`` (crates/rllm-server/src/cli.rs:27-49:
``--dtype auto``, ``--max-model-len``, ``--max-num-seqs 256``,
``--max-num-batched-tokens 4096``, ``--gpu-memory-utilization 0.9``,
``--enable-prefix-caching``).  ``init-random`` is the random-weights mode: it
writes config.json and model.safetensors drawn from a seed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from typing import List


def _gpu_util(s: str) -> float:
    v = float(s)
    if not 0.01 <= v <= 1.0:
        raise argparse.ArgumentTypeError(f"gpu_memory_utilization must be in range 0.01..=1.0, got {v}")
    return v


def _bool(s: str) -> bool:
    if s.lower() in ("1", "true", "yes", "on"):
        return True
    if s.lower() in ("0", "false", "no", "off"):
        return False
    raise argparse.ArgumentTypeError(f"not a boolean: {s!r}")


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="rllm", description="rllm_b200: LLM inference engine for one B200")
    sub = p.add_subparsers(dest="command", required=True)

    g = sub.add_parser("generate", help="generate from token-id prompts")
    g.add_argument("model", nargs="?", help="model folder (config.json + safetensors)")
    g.add_argument("--model", "-m", dest="model_opt", help="same as the positional argument")
    g.add_argument("--prompt-ids", "-p", action="append", default=[],
                   help="a prompt as comma-separated token ids; may be repeated")
    g.add_argument("--prompt-file", help="JSON file: a list of prompts, each a list of token ids")
    g.add_argument("--random-prompts", metavar="N:LEN", help="N random prompts of LEN tokens")
    g.add_argument("--max-tokens", type=int, default=64)
    g.add_argument("--temperature", type=float, default=1.0, help="0 = greedy")
    g.add_argument("-n", "--n", type=int, default=1, help="samples per prompt (the prompt is computed once)")
    g.add_argument("--top-k", type=int, default=-1)
    g.add_argument("--top-p", type=float, default=1.0)
    g.add_argument("--min-p", type=float, default=0.0)
    g.add_argument("--repetition-penalty", type=float, default=1.0)
    g.add_argument("--presence-penalty", type=float, default=0.0)
    g.add_argument("--frequency-penalty", type=float, default=0.0)
    g.add_argument("--seed", type=int, default=None, help="sampling seed of the first prompt; prompt i uses seed+i")
    g.add_argument("--ignore-eos", action="store_true")
    g.add_argument("--stop-token-ids", default="", metavar="ID,ID", help="token ids that end a request (beside the model's EOS)")
    g.add_argument("--bad-words-token-ids", default="", metavar="ID,ID;ID",
                   help="token sequences, separated by ';': a sequence's last token cannot follow its first ones")
    g.add_argument("--skip-reading-prefix-cache", action="store_true",
                   help="compute the whole prompt even where shared pages hold a part of it")
    g.add_argument("--min-tokens", type=int, default=0, help="the model's EOS cannot be drawn before this many tokens have been generated")
    g.add_argument("--logprobs", type=int, default=None, metavar="N",
                   help="report every generated token's log-probability and the N likeliest tokens of its place (with --json)")
    g.add_argument("--dtype", default="auto", help="auto | bf16 | fp32")
    g.add_argument("--max-model-len", type=int, default=None)
    g.add_argument("--max-num-seqs", type=int, default=256)
    g.add_argument("--max-num-batched-tokens", type=int, default=4096)
    g.add_argument("--long-prefill-token-threshold", type=int, default=2048)
    g.add_argument("--gpu-memory-utilization", type=_gpu_util, default=0.9)
    g.add_argument("--enable-prefix-caching", type=_bool, nargs="?", const=True, default=True)
    g.add_argument("--scheduling-policy", choices=["fcfs", "priority"], default="fcfs")
    g.add_argument("--priorities", default="", metavar="P,P", help="a priority for each prompt (priority policy: larger first)")
    g.add_argument("--step-row-multiple", type=int, default=128,
                   help="a step that ends up to a quarter of this many rows over a multiple of it gives them back (0: off)")
    g.add_argument("--block-size", type=int, default=16)
    g.add_argument("--num-gpu-blocks", type=int, default=None)
    g.add_argument("--random-weights", action="store_true",
                   help="draw weights from --weights-seed; the folder needs config.json only")
    g.add_argument("--weights-seed", type=int, default=0)
    g.add_argument("--json", action="store_true", help="one JSON object per request on stdout")
    g.add_argument("--log-level", default=None,
                   help="error | warn | info | debug (one line of statistics per step) | trace; "
                        "default: the environment variable RLLM_LOG, else info")

    sub.add_parser("replay", add_help=False,
                   help="feed token ids through the model step by step and write logits (options of bin/trace_run)")
    sub.add_parser("bench", add_help=False,
                   help="time one kernel alone: attention_decode | attention_prefill | gemm_small_m | gemm_tcgen05 "
                        "(options of python -m rllm_b200.kernels.microbench)")
    r = sub.add_parser("init-random", help="write a model folder with random weights")
    r.add_argument("model", help="folder to write")
    r.add_argument("--config", required=True, help="config.json to build the model from")
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--dtype", default=None, help="storage dtype (default: the config's torch_dtype)")
    return p


def _prompts(args) -> List[List[int]]:
    prompts: List[List[int]] = []
    for s in args.prompt_ids:
        prompts.append([int(x) for x in s.replace(" ", "").split(",") if x])
    if args.prompt_file:
        with open(args.prompt_file) as f:
            prompts += [[int(t) for t in p] for p in json.load(f)]
    return prompts


def cmd_generate(args) -> int:
    from . import LLM, SamplingParams
    from .config import read_config_json
    from . import log
    log.set_level(args.log_level or os.environ.get("RLLM_LOG") or "info")
    model_dir = args.model or args.model_opt
    if not model_dir:
        print("rllm generate: a model folder is required", file=sys.stderr)
        return 2
    prompts = _prompts(args)
    if args.random_prompts:
        import numpy as np
        n, length = (int(x) for x in args.random_prompts.split(":"))
        vocab = int(read_config_json(model_dir).get("vocab_size", 32000))
        rng = np.random.default_rng(0)
        prompts += [[int(t) for t in rng.integers(0, vocab, size=length)] for _ in range(n)]
    if not prompts:
        print("rllm generate: no prompt (use --prompt-ids, --prompt-file or --random-prompts)", file=sys.stderr)
        return 2
    llm = LLM(model_dir, dtype=args.dtype, max_model_len=args.max_model_len, max_num_seqs=args.max_num_seqs,
              max_num_batched_tokens=args.max_num_batched_tokens,
              gpu_memory_utilization=args.gpu_memory_utilization,
              enable_prefix_caching=args.enable_prefix_caching, block_size=args.block_size,
              num_gpu_blocks=args.num_gpu_blocks,
              long_prefill_token_threshold=args.long_prefill_token_threshold,
              step_row_multiple=args.step_row_multiple, scheduling_policy=args.scheduling_policy,
              random_weights=args.random_weights, seed=args.weights_seed)
    params = [SamplingParams(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p,
                             min_p=args.min_p, repetition_penalty=args.repetition_penalty,
                             presence_penalty=args.presence_penalty,
                             frequency_penalty=args.frequency_penalty, max_tokens=args.max_tokens,
                             ignore_eos=args.ignore_eos, logprobs=args.logprobs, n=args.n,
                             stop_token_ids=[int(x) for x in args.stop_token_ids.replace(" ", "").split(",") if x],
                             min_tokens=args.min_tokens,
                             bad_words_token_ids=[[int(x) for x in w.split(",") if x]
                                                  for w in args.bad_words_token_ids.replace(" ", "").split(";") if w],
                             skip_reading_prefix_cache=args.skip_reading_prefix_cache,
                             seed=None if args.seed is None else args.seed + i)
              for i in range(len(prompts))]
    t0 = time.time()
    prios = [int(x) for x in args.priorities.replace(" ", "").split(",") if x] or None
    outs = llm.generate(prompts, params, priorities=prios)
    dt = time.time() - t0
    n_out = sum(o.usage.completion_tokens for o in outs)
    def sample(c):
        return {"index": c.index, "token_ids": c.token_ids, "finish_reason": c.finish_reason,
                "logprobs": None if c.logprobs is None else
                [{"token_id": e.token_id, "logprob": e.logprob, "top_logprobs": e.top_logprobs} for e in c.logprobs]}

    for o in outs:
        if args.json:
            first = sample(o.outputs[0])
            print(json.dumps({"request_id": o.request_id, "prompt_token_ids": o.prompt_token_ids,
                              "token_ids": first["token_ids"], "finish_reason": first["finish_reason"],
                              "logprobs": first["logprobs"], "outputs": [sample(c) for c in o.outputs],
                              "usage": vars(o.usage)}))
        else:
            for c in o.outputs:
                name = f"request {o.request_id}" + (f" sample {c.index}" if len(o.outputs) > 1 else "")
                print(f"{name}: {c.token_ids}  [{c.finish_reason}; "
                      f"{o.usage.prompt_tokens} prompt + {len(c.token_ids)} generated]")
    log.logger.info(f"{n_out} tokens in {dt:.3f} s ({n_out / max(dt, 1e-9):.1f} tok/s), "
                    f"{llm.engine.num_steps} steps; {json.dumps(llm.engine.stats())}")
    return 0


def cmd_init_random(args) -> int:
    from .engine.loading import write_random_model
    with open(args.config) as f:
        cfg = json.load(f)
    write_random_model(args.model, cfg, args.seed, args.dtype)
    print(f"wrote {args.model}/config.json and model.safetensors (seed {args.seed})")
    return 0


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] == "replay":
        # trace replay (the program behind bin/trace_run) takes its own options: --model --dtype --out --max-tokens
        from .engine.replay import main as replay_main
        return replay_main(argv[1:])
    if argv and argv[0] == "bench":
        from .kernels.microbench import main as bench_main
        return bench_main(argv[1:])
    args = build_parser().parse_args(argv)
    if args.command == "generate":
        return cmd_generate(args)
    if args.command == "init-random":
        return cmd_init_random(args)
    return 2


if __name__ == "__main__":
    sys.exit(main())
