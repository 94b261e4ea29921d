"""Generation through the Python entry point against the plain implementation:
greedy tokens, seeded temperature sampling, and that a request's output does
not depend on batching, portion sizes, preemption or prefix sharing."""
import numpy as np
import pytest
import torch

import plain_llama as pl
from conftest import TINY

pytestmark = pytest.mark.gpu


def prompts_for(name, lengths, seed):
    cfg, _, _ = TINY[name]
    rng = np.random.default_rng(seed)
    return [[int(t) for t in rng.integers(8, cfg["vocab_size"], size=n)] for n in lengths]


def make_llm(model_dirs, name, dtype="fp32", **kw):
    from rllm_b200 import LLM
    _, _, page = TINY[name]
    kw.setdefault("num_gpu_blocks", 256)
    kw.setdefault("max_num_seqs", 8)
    return LLM(model_dirs[name], dtype=dtype, block_size=page, **kw)


@pytest.mark.parametrize("name,lengths,seed,steps", [("A", [5, 12, 17], 1, 8), ("B", [1, 31, 70, 150], 3, 10)])
def test_greedy_generation_equals_plain_greedy(model_dirs, name, lengths, seed, steps):
    from rllm_b200 import SamplingParams
    prompts = prompts_for(name, lengths, seed)
    llm = make_llm(model_dirs, name, max_num_batched_tokens=64, long_prefill_token_threshold=16)
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=steps, ignore_eos=True))
    plain = pl.read_model_dir(model_dirs[name])
    for p, o in zip(prompts, outs):
        assert o.outputs[0].token_ids == plain.greedy(p, steps)
        assert o.outputs[0].finish_reason == "length" and o.finished
        assert (o.usage.prompt_tokens, o.usage.completion_tokens, o.usage.total_tokens) == \
            (len(p), steps, len(p) + steps)
    assert llm.engine.cache.usage()["num_requests"] == 0


def test_greedy_generation_in_bfloat16(model_dirs):
    """bfloat16 follows the oracle (run on bfloat16-rounded weights) wherever
    the oracle's own choice is clear: top-two margin above the bf16 tolerance."""
    from rllm_b200 import SamplingParams
    prompts = prompts_for("B", [31, 70], 3)
    llm = make_llm(model_dirs, "B", dtype="bf16")
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))
    plain = pl.read_model_dir(model_dirs["B"], round_to=torch.bfloat16)
    for p, o in zip(prompts, outs):
        toks = list(p)
        for t in o.outputs[0].token_ids:
            row = plain.logits(toks)[-1]
            top = torch.topk(row, 2).values
            if float(top[0] - top[1]) > 4e-2 * float(row.abs().max()):
                assert t == int(torch.argmax(row))
            toks.append(t)


@pytest.mark.parametrize("name", ["B", "B0"])
def test_temperature_sampling_matches_plain_and_ignores_batching(model_dirs, name):
    """Four requests with prompts of 1, 31, 70 and 150 tokens, portions of 16 tokens beside decoded tokens of
    the others, 10 tokens each at temperature 0.7 with a Philox stream per request."""
    from rllm_b200 import SamplingParams
    prompts = prompts_for(name, [1, 31, 70, 150], 3)
    params = [SamplingParams(temperature=0.7, max_tokens=10, seed=100 + i, ignore_eos=True) for i in range(4)]
    together = make_llm(model_dirs, name, max_num_batched_tokens=40, long_prefill_token_threshold=16)
    outs = together.generate(prompts, params)
    # the plain model, given the engine's own tokens so far, draws the same next token
    plain = pl.read_model_dir(model_dirs[name])
    for i, (p, o) in enumerate(zip(prompts, outs)):
        toks = list(p)
        for j, t in enumerate(o.outputs[0].token_ids):
            x = pl.process_logits(plain.logits(toks)[-1].numpy(), temperature=0.7)
            assert t == pl.sample_row(x, 0.7, -1, pl.uniform_for(100 + i, j)), (i, j)
            toks.append(t)
    # one by one gives the same tokens (crates/rllm-bench/tests/correctness.rs:73-117)
    alone = make_llm(model_dirs, name)
    for p, sp, o in zip(prompts, params, outs):
        assert alone.generate([p], sp)[0].outputs[0].token_ids == o.outputs[0].token_ids


def test_stop_conditions(model_dirs):
    from rllm_b200 import SamplingParams
    llm = make_llm(model_dirs, "A")
    p = prompts_for("A", [9], 5)[0]
    free_run = llm.generate([p], SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))[0].outputs[0].token_ids
    stop_at = free_run[4]
    first = free_run.index(stop_at)
    out = llm.generate([p], SamplingParams(temperature=0.0, max_tokens=12, stop_token_ids=[stop_at], ignore_eos=True))[0]
    assert out.outputs[0].token_ids == free_run[:first + 1] and out.outputs[0].finish_reason == "stop"
    # an EOS of config.json stops unless ignore_eos; min_tokens keeps it away
    eos_cfg = dict(TINY["A"][0], eos_token_id=stop_at)
    import json, os, shutil, tempfile
    d = tempfile.mkdtemp()
    shutil.copy(os.path.join(model_dirs["A"], "model.safetensors"), d)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(eos_cfg, f)
    from rllm_b200 import LLM
    llm2 = LLM(d, dtype="fp32", num_gpu_blocks=64, max_num_seqs=4)
    out = llm2.generate([p], SamplingParams(temperature=0.0, max_tokens=12))[0]
    assert out.outputs[0].token_ids == free_run[:first + 1] and out.outputs[0].finish_reason == "stop"
    out = llm2.generate([p], SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))[0]
    assert out.outputs[0].token_ids == free_run
    out = llm2.generate([p], SamplingParams(temperature=0.0, max_tokens=first + 3, min_tokens=first + 2))[0]
    assert stop_at not in out.outputs[0].token_ids[:first + 2]
    shutil.rmtree(d)


@pytest.mark.parametrize("dtype,temperature", [("fp32", 0.0), ("fp32", 0.8)])
def test_steps_launched_ahead_keep_every_request_right(model_dirs, dtype, temperature):
    """Decode steps go to the GPU before the tokens of the step before them are read.  Requests that
    end at different steps (length, a stop token), one that is aborted and one that arrives in the
    middle each leave a step in flight that holds a row to drop or forces a fresh schedule: every
    request's tokens are those of the plain implementation, and all pages come back."""
    from rllm_b200 import SamplingParams
    name = "A"
    prompts = prompts_for(name, [9, 14, 6, 11, 7], 21)
    plain = pl.read_model_dir(model_dirs[name])
    llm = make_llm(model_dirs, name, dtype=dtype, enable_prefix_caching=False)
    free = llm.engine.cache.num_free_pages()

    def sp(i, n, **kw):
        return SamplingParams(temperature=temperature, max_tokens=n, seed=40 + i, ignore_eos=True, **kw)

    def want(i, n):
        if temperature == 0.0:
            return plain.greedy(prompts[i], n)
        toks = list(prompts[i])
        for j in range(n):
            x = pl.process_logits(plain.logits(toks)[-1].numpy(), temperature=temperature)
            toks.append(pl.sample_row(x, temperature, -1, pl.uniform_for(40 + i, j)))
        return toks[len(prompts[i]):]
    full1 = want(1, 40)
    stop_tok = full1[17]
    n_stop = full1.index(stop_tok) + 1
    ids = [llm.add_request(prompts[0], sp(0, 40)), llm.add_request(prompts[1], sp(1, 40, stop_token_ids=[stop_tok])),
           llm.add_request(prompts[2], sp(2, 23)), llm.add_request(prompts[3], sp(3, 40))]
    got = {i: [] for i in ids}
    reasons = {}
    steps = 0
    late = None
    while llm.has_work():
        for out in llm.step():
            got.setdefault(out.request_id, []).extend(out.outputs[0].token_ids)
            if out.finished:
                reasons[out.request_id] = out.outputs[0].finish_reason
        steps += 1
        if steps == 12:
            assert llm.abort_request(ids[3])
        if steps == 27:
            late = llm.add_request(prompts[4], sp(4, 15))
    assert got[ids[0]] == want(0, 40) and reasons[ids[0]] == "length"
    assert got[ids[1]] == full1[:n_stop] and reasons[ids[1]] == "stop"
    assert got[ids[2]] == want(2, 23) and reasons[ids[2]] == "length"
    assert got[ids[3]] == want(3, 40)[:len(got[ids[3]])] and 0 < len(got[ids[3]]) < 40
    assert got[late] == want(4, 15)
    assert llm.engine.stats()["num_steps_ahead"] > 10
    llm.engine.cache.check()
    assert llm.engine.cache.num_free_pages() == free and llm.engine.cache.usage()["num_requests"] == 0


@pytest.mark.parametrize("name,dtype", [("A", "fp32"), ("C", "bf16")])
def test_batches_padded_to_captured_sizes(model_dirs, name, dtype):
    """More than 8 requests decode in graphs of padded batch sizes (12, 16, ...): requests that end one
    after the other walk the batch down through the sizes; every request's tokens are what it gets alone,
    and (float32) what the plain implementation generates."""
    from rllm_b200 import SamplingParams
    from rllm_b200.engine.decode_graph import batch_bucket
    assert [batch_bucket(n) for n in (1, 8, 9, 12, 13, 33, 64, 65, 129)] == [1, 8, 12, 12, 16, 40, 64, 80, 160]
    lengths = [5, 9, 3, 14, 7, 11, 4, 6, 13, 8, 10, 12, 15]
    prompts = prompts_for(name, lengths, 31)
    budgets = [6 + 3 * i for i in range(len(prompts))]            # 6 .. 42 tokens: one request ends every third step
    params = [SamplingParams(temperature=0.0, max_tokens=n, ignore_eos=True) for n in budgets]
    llm = make_llm(model_dirs, name, dtype=dtype, max_num_seqs=16, enable_prefix_caching=False)
    free = llm.engine.cache.num_free_pages()
    outs = llm.generate(prompts, params)
    sizes = sorted(k[0] for k in llm.engine.runner.graphs)
    assert 16 in sizes and 12 in sizes and not any(8 < n and n % 4 for n in sizes), sizes
    if dtype == "fp32":
        plain = pl.read_model_dir(model_dirs[name])
        for p, n, o in zip(prompts, budgets, outs):
            assert o.outputs[0].token_ids == plain.greedy(p, n)
    else:
        alone = make_llm(model_dirs, name, dtype=dtype, max_num_seqs=16, enable_prefix_caching=False)
        for p, sp, o in list(zip(prompts, params, outs))[::4]:
            assert alone.generate([p], sp)[0].outputs[0].token_ids == o.outputs[0].token_ids
    llm.engine.cache.check()
    assert llm.engine.cache.num_free_pages() == free


def test_preemption_does_not_change_outputs(model_dirs):
    from rllm_b200 import SamplingParams
    name = "B"
    prompts = prompts_for(name, [40, 33, 25, 47], 8)
    params = [SamplingParams(temperature=0.9, top_p=0.95, max_tokens=40, seed=7 + i, ignore_eos=True) for i in range(4)]
    roomy = make_llm(model_dirs, name)
    want = [o.outputs[0].token_ids for o in roomy.generate(prompts, params)]
    tight = make_llm(model_dirs, name, num_gpu_blocks=24, enable_prefix_caching=False)   # 192 tokens of cache
    got = [o.outputs[0].token_ids for o in tight.generate(prompts, params)]
    assert tight.engine.scheduler.num_preemptions > 0
    assert got == want
    assert tight.engine.cache.num_free_pages() == 24


def test_prefix_sharing_does_not_change_outputs(model_dirs):
    from rllm_b200 import SamplingParams
    name = "A"
    common = prompts_for(name, [50], 2)[0]
    prompts = [common + tail for tail in prompts_for(name, [3, 9, 1], 4)] + [list(common[:48])]
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    off = make_llm(model_dirs, name, enable_prefix_caching=False)
    want = [o.outputs[0].token_ids for o in off.generate(prompts, sp)]
    on = make_llm(model_dirs, name, enable_prefix_caching=True, max_num_seqs=1)     # one after the other
    got = [o.outputs[0].token_ids for o in on.generate(prompts, sp)]
    assert on.engine.scheduler.prefix_hit_tokens == 48 + 48 + 32    # the last prompt is cached whole: one page is redone
    assert got == want
    on.engine.cache.check()


def sample_seed(seed, index):
    """The seed of sample ``index`` of a request: the request's seed moved on by the index."""
    return (seed + index * 0x9E3779B97F4A7C15) & 0x7FFFFFFFFFFFFFFF


@pytest.mark.parametrize("name,prefix,pages", [("B", False, 256), ("B", True, 256), ("B0", False, 20), ("A", True, 256)])
def test_several_samples_of_one_prompt(model_dirs, name, prefix, pages):
    """n = 3 samples of prompts of 1, 33, 70 and 16 k + 1 tokens beside a request with one sample: the
    prompt is computed once up to its last token, the samples take its pages over and go on by
    themselves; every sample is what the plain model draws with the sample's own random stream.  With
    20 pages the samples do not all fit: some wait like new requests, some are preempted and computed
    again."""
    from rllm_b200 import SamplingParams
    _, _, page = TINY[name]
    lengths = [1, 33, 70, 4 * page + 1, 21]
    prompts = prompts_for(name, lengths, 12)
    params = [SamplingParams(temperature=0.9, max_tokens=9, seed=300 + i, ignore_eos=True, n=3) for i in range(4)]
    params.append(SamplingParams(temperature=0.9, max_tokens=9, seed=304, ignore_eos=True))
    llm = make_llm(model_dirs, name, num_gpu_blocks=pages, max_num_seqs=16, max_num_batched_tokens=48,
                   long_prefill_token_threshold=16, enable_prefix_caching=prefix)
    outs = llm.generate(prompts, params)
    plain = pl.read_model_dir(model_dirs[name])
    for i, (p, sp, o) in enumerate(zip(prompts, params, outs)):
        assert [c.index for c in o.outputs] == list(range(sp.n)) and all(c.finish_reason == "length" for c in o.outputs)
        assert o.usage.completion_tokens == 9 * sp.n and o.usage.prompt_tokens == len(p)
        for c in o.outputs:
            toks = list(p)
            for j, t in enumerate(c.token_ids):
                x = pl.process_logits(plain.logits(toks)[-1].numpy(), temperature=0.9)
                assert t == pl.sample_row(x, 0.9, -1, pl.uniform_for(sample_seed(300 + i, c.index), j)), (i, c.index, j)
                toks.append(t)
        if sp.n > 1:
            assert len({tuple(c.token_ids) for c in o.outputs}) > 1         # streams of their own
    stats = llm.engine.stats()
    if pages == 256:
        # prompts of 33, 70 and 4 pages + 1: two samples each took over all but the last token
        assert stats["num_copied_tokens"] == 2 * (32 + 69 + 4 * page)
    else:
        assert stats["num_preemptions"] > 0 and 0 < stats["num_copied_tokens"] < 2 * (32 + 69 + 4 * page)
    llm.engine.cache.check()
    assert llm.engine.cache.num_free_pages() == pages and not llm.engine._families


def test_samples_of_one_prompt_can_be_aborted_and_greedy_refuses_them(model_dirs):
    from rllm_b200 import SamplingParams
    from rllm_b200.sampling.params import InvalidSamplingParams
    llm = make_llm(model_dirs, "A")
    with pytest.raises(InvalidSamplingParams):
        llm.add_request([9, 10, 11], SamplingParams(temperature=0.0, n=2))
    p = prompts_for("A", [40], 3)[0]
    rid = llm.add_request(p, SamplingParams(temperature=1.0, max_tokens=30, n=4, seed=5, ignore_eos=True))
    seen = set()
    for _ in range(6):
        for o in llm.step():
            assert o.request_id == rid and not o.finished
            seen.update(c.index for c in o.outputs)
    assert seen == {0, 1, 2, 3}
    assert llm.abort_request(rid) and not llm.has_work() and not llm.abort_request(rid)
    llm.engine.cache.check()
    assert llm.engine.cache.num_free_pages() == 256
    # the engine goes on as before
    out = llm.generate([p], SamplingParams(temperature=1.0, max_tokens=5, n=2, seed=5, ignore_eos=True))[0]
    assert [len(c.token_ids) for c in out.outputs] == [5, 5]


def test_requests_beyond_the_limits_are_refused(model_dirs):
    from rllm_b200 import SamplingParams
    from rllm_b200.engine.scheduler import RequestRefused
    llm = make_llm(model_dirs, "A", num_gpu_blocks=4)
    with pytest.raises(RequestRefused):
        llm.add_request(list(range(100)), SamplingParams(max_tokens=40))     # beyond max_position_embeddings 128
    with pytest.raises(RequestRefused):
        llm.add_request(list(range(60)), SamplingParams(max_tokens=16))      # beyond 4 pages of 16
    with pytest.raises(ValueError, match="vocabulary"):
        llm.add_request([1, 2, 256])


def test_priorities_decide_who_runs_first_and_change_no_token(model_dirs):
    from rllm_b200 import SamplingParams
    plain = pl.read_model_dir(model_dirs["A"])
    prompts = prompts_for("A", [9, 4, 13], 5)
    llm = make_llm(model_dirs, "A", max_num_seqs=1, scheduling_policy="priority")
    sp = SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True)
    ids = [llm.add_request(p, sp, priority=pr) for p, pr in zip(prompts, [0, 7, 3])]
    finished, got = [], {i: [] for i in ids}
    while llm.has_work():
        for out in llm.step():
            got[out.request_id] += out.outputs[0].token_ids
            if out.finished:
                finished.append(out.request_id)
    assert finished == [ids[1], ids[2], ids[0]]
    assert [got[i] for i in ids] == [plain.greedy(p, 3) for p in prompts]
    outs = llm.generate(prompts, sp, priorities=[1, 2, 3])
    assert [o.outputs[0].token_ids for o in outs] == [plain.greedy(p, 3) for p in prompts]


def test_bad_words_keep_their_last_token_out_behind_their_first_ones(model_dirs):
    """Greedy generation with a one-token word (never drawn) and a two-token word (its second token is not
    drawn behind its first, but elsewhere it is), against the plain implementation with the same rule."""
    from rllm_b200 import SamplingParams
    plain = pl.read_model_dir(model_dirs["A"])
    prompt = [5, 6, 7, 8]
    free = plain.greedy(prompt, 10)
    one = [free[1]]                               # the token that greedy decoding would draw second
    two = [free[3], free[4]]                      # and the pair that it would draw fourth and fifth
    words = [one, two]

    def plain_with_rule(n):
        toks, out = list(prompt), []
        for _ in range(n):
            row = plain.logits(toks)[-1].clone()
            for w in words:
                k = len(w) - 1
                if k == 0 or toks[-k:] == w[:k]:
                    row[w[-1]] = float("-inf")
            t = int(torch.argmax(row))
            out.append(t)
            toks.append(t)
        return out

    want = plain_with_rule(10)
    assert one[0] not in want and want != free
    llm = make_llm(model_dirs, "A")
    got = llm.generate([prompt], SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True,
                                                bad_words_token_ids=words))[0].outputs[0].token_ids
    assert got == want
    for a, b in zip([prompt[-1]] + got, got):
        assert not (a == two[0] and b == two[1])


def test_command_line(model_dirs, capsys):
    from rllm_b200.cli import main
    import json
    code = main(["generate", model_dirs["A"], "--prompt-ids", "5,6,7", "-p", "9,10", "--max-tokens", "4",
                 "--temperature", "0", "--dtype", "fp32", "--num-gpu-blocks", "32", "--max-num-seqs", "4",
                 "--ignore-eos", "--json"])
    assert code == 0
    lines = [json.loads(l) for l in capsys.readouterr().out.strip().split("\n")]
    plain = pl.read_model_dir(model_dirs["A"])
    assert [l["token_ids"] for l in lines] == [plain.greedy([5, 6, 7], 4), plain.greedy([9, 10], 4)]
    assert lines[0]["finish_reason"] == "length" and lines[0]["usage"]["total_tokens"] == 7
    # a stop token ends the request at its first appearance
    want = plain.greedy([5, 6, 7], 8)
    stop = want[2]
    first = want.index(stop)
    code = main(["generate", model_dirs["A"], "--prompt-ids", "5,6,7", "--max-tokens", "8", "--temperature", "0",
                 "--dtype", "fp32", "--num-gpu-blocks", "32", "--max-num-seqs", "4", "--ignore-eos",
                 "--stop-token-ids", f"{stop}", "--json"])
    assert code == 0
    line = json.loads(capsys.readouterr().out.strip())
    assert line["token_ids"] == want[:first + 1] and line["finish_reason"] == "stop"
    # two samples of a prompt, each from a stream of its own
    code = main(["generate", model_dirs["A"], "--prompt-ids", "5,6,7,8,9", "--max-tokens", "6", "--temperature", "1.0",
                 "-n", "2", "--seed", "11", "--dtype", "fp32", "--num-gpu-blocks", "32", "--max-num-seqs", "4",
                 "--ignore-eos", "--json"])
    assert code == 0
    line = json.loads(capsys.readouterr().out.strip())
    assert [o["index"] for o in line["outputs"]] == [0, 1] and all(len(o["token_ids"]) == 6 for o in line["outputs"])
    assert line["token_ids"] == line["outputs"][0]["token_ids"] and line["usage"]["completion_tokens"] == 12
    for o in line["outputs"]:
        toks = [5, 6, 7, 8, 9]
        for j, t in enumerate(o["token_ids"]):
            x = pl.process_logits(plain.logits(toks)[-1].numpy(), temperature=1.0)
            assert t == pl.sample_row(x, 1.0, -1, pl.uniform_for(sample_seed(11, o["index"]), j))
            toks.append(t)


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_random_serving_keeps_every_request_right(model_dirs, seed):
    """Requests of random lengths, some with a common beginning, arrive while others run; there are few
    pages (requests get preempted), few sequences at a time, a small token budget, prefix sharing, an
    abort, request names that come back after their request has ended, and requests that want two or three
    samples at a temperature.  Every request that ends has the tokens that the plain implementation
    generates (or draws, with the sample's own random stream) for its prompt alone."""
    from rllm_b200 import SamplingParams
    name = "A"
    cfg, _, page = TINY[name]
    rng = np.random.default_rng(100 + seed)
    V = cfg["vocab_size"]
    plain = pl.read_model_dir(model_dirs[name])
    llm = make_llm(model_dirs, name, num_gpu_blocks=10, max_num_seqs=4, max_num_batched_tokens=40,
                   long_prefill_token_threshold=24, enable_prefix_caching=True)
    bases = [[int(t) for t in rng.integers(8, V, size=48)] for _ in range(2)]
    todo = []
    for i in range(22):
        n = int(rng.integers(1, 70))
        if rng.random() < 0.4:
            b = bases[int(rng.integers(0, 2))]
            k = int(rng.integers(16, 49))
            prompt = b[:k] + [int(t) for t in rng.integers(8, V, size=max(1, n - k))]
        else:
            prompt = [int(t) for t in rng.integers(8, V, size=n)]
        steps = int(rng.integers(1, 20))
        prompt = prompt[: 100 - steps]
        todo.append((f"q{i % 9}", prompt, steps))         # names come back
    live, done, aborted = {}, [], 0
    guard = 0
    while todo or live:
        guard += 1
        assert guard < 5000
        # admit: a name only when its earlier request has ended; every fourth request wants several samples
        while todo and todo[0][0] not in live and len(live) < 7 and rng.random() < 0.7:
            rid, prompt, steps = todo.pop(0)
            n = int(rng.integers(2, 4)) if len(todo) % 4 == 0 else 1
            sp = SamplingParams(temperature=0.8 if n > 1 else 0.0, max_tokens=steps, ignore_eos=True, n=n, seed=1000 + len(todo))
            llm.add_request(prompt, sp, request_id=rid)
            live[rid] = (prompt, steps, {i: [] for i in range(n)}, sp)
        if live and aborted == 0 and guard == 25:
            rid = sorted(live)[0]
            assert llm.abort_request(rid)
            del live[rid]
            aborted = 1
        for out in llm.step():
            prompt, steps, toks, sp = live[out.request_id]
            for c in out.outputs:
                toks[c.index] += c.token_ids
            if out.finished:
                done.append((prompt, steps, toks, sp))
                del live[out.request_id]
    assert len(done) >= 20 and any(sp.n > 1 for _, _, _, sp in done)
    for prompt, steps, toks, sp in done:
        if sp.n == 1:
            assert toks[0] == plain.greedy(prompt, steps), (len(prompt), steps)
            continue
        for i, got in toks.items():
            assert len(got) == steps
            seq = list(prompt)
            for j, t in enumerate(got):
                x = pl.process_logits(plain.logits(seq)[-1].numpy(), temperature=0.8)
                assert t == pl.sample_row(x, 0.8, -1, pl.uniform_for(sample_seed(sp.seed, i), j)), (len(prompt), i, j)
                seq.append(t)
    llm.engine.cache.check()
    assert llm.engine.cache.usage()["num_requests"] == 0 and not llm.engine._families
    print("preemptions", llm.engine.scheduler.num_preemptions, "prefix hits", llm.engine.scheduler.prefix_hit_tokens)


@pytest.mark.parametrize("hidden,heads,kv_heads,head_dim,inter", [(2048, 32, 8, 64, 8192), (3072, 24, 8, 128, 8192)])
def test_layers_of_real_size_in_bfloat16_follow_float32(tmp_path, hidden, heads, kv_heads, head_dim, inter):
    """Two layers with the sizes of a Llama-3.2-1B (or 3B: heads of 128) layer and its vocabulary, random weights: the logits of
    the bfloat16 path (tensor-core products and attention on tcgen05 for the 1,024-token prompt, the
    weight-streaming products and split-KV attention for the decode steps that follow, as CUDA graphs)
    agree with those of the float32 path, whose kernels the tiny configurations check against the plain
    implementation.  Sizes of this kind reach code that the tiny configurations do not (full tiles, the
    one-wave form of the decode products, several CTAs a sequence in decode attention)."""
    import json
    from rllm_b200 import LLM
    from rllm_b200.engine.runner import StepEntry
    cfg = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 2, "hidden_size": hidden,
           "num_attention_heads": heads, "num_key_value_heads": kv_heads, "head_dim": head_dim, "intermediate_size": inter,
           "vocab_size": 128256, "rope_theta": 500000.0,
           "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                            "original_max_position_embeddings": 8192},
           "max_position_embeddings": 131072, "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
           "hidden_act": "silu", "torch_dtype": "bfloat16", "bos_token_id": 128000, "eos_token_id": 128001}
    d = str(tmp_path / "real_size")
    import os
    os.makedirs(d)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    rng = np.random.default_rng(3)
    prompts = {"long": [int(t) for t in rng.integers(0, 128256, size=1024)],
               "mid": [int(t) for t in rng.integers(0, 128256, size=700)],
               "short": [int(t) for t in rng.integers(0, 128256, size=5)]}
    feed = {k: [int(t) for t in rng.integers(0, 128256, size=6)] for k in prompts}
    rows = {}
    for dt in ("fp32", "bf16"):
        llm = LLM(d, dtype=dt, max_model_len=2048, max_num_seqs=16, max_num_batched_tokens=2048, num_gpu_blocks=200,
                  enable_prefix_caching=False, random_weights=True, draw_on_device=True, seed=1)
        eng, runner = llm.engine, llm.engine.runner
        got = []
        for k, p in prompts.items():
            eng.cache.admit(k)
            assert eng.cache.ensure(k, 0, len(p) + 12)
        # the prompts as one step, then decode steps of all three
        logits = runner.step([StepEntry(k, p, 0, [len(p) - 1]) for k, p in prompts.items()])
        got.append(logits.float().cpu())
        for i in range(6):
            logits = runner.step([StepEntry(k, [feed[k][i]], len(prompts[k]) + i, [0]) for k in prompts])
            got.append(logits.float().cpu())
        # nine more requests: decode steps of twelve rows go through the decode products in their form for
        # two batch tiles
        more = {f"m{i}": [int(t) for t in np.random.default_rng(50 + i).integers(0, 128256, size=4 + i)] for i in range(9)}
        for k, p in more.items():
            eng.cache.admit(k)
            assert eng.cache.ensure(k, 0, len(p) + 4)
        got.append(runner.step([StepEntry(k, p, 0, [len(p) - 1]) for k, p in more.items()]).float().cpu())
        for i in range(3):
            entries = [StepEntry(k, [feed[k][i]], len(prompts[k]) + 6 + i, [0]) for k in prompts]
            entries += [StepEntry(k, [7 + i], len(p) + i, [0]) for k, p in more.items()]
            got.append(runner.step(entries).float().cpu())
        runner.check_errors()
        rows[dt] = torch.cat(got)
        del llm, eng, runner
        torch.cuda.empty_cache()
    a, b = rows["fp32"].double(), rows["bf16"].double()
    err = (a - b).abs().amax(dim=1) / a.abs().amax(dim=1)
    same = (a.argmax(dim=1) == b.argmax(dim=1)).float().mean()
    print(f"layers of real size (hidden {hidden}): bfloat16 against float32 worst {float(err.max()):.3e}, "
          f"mean {float(err.mean()):.3e}, same argmax {float(same):.3f}")
    assert float(err.max()) <= 2.5e-2, err
    # and the two paths agree on the likeliest token except at near-ties (a vocabulary of 128,256 has some)
    assert float(same) >= 0.9, same
    top = torch.topk(a, 2, dim=1).values
    clear = (top[:, 0] - top[:, 1]) > 2 * 2.5e-2 * a.abs().amax(dim=1)
    assert bool((a.argmax(dim=1) == b.argmax(dim=1))[clear].all())


def test_logprobs_come_from_the_raw_logits(model_dirs):
    """A request that asks for log-probabilities gets, for every generated token, its log-probability and
    the N likeliest tokens of its place, from the raw logits: also when penalties and a temperature change
    what is sampled, and beside requests that did not ask."""
    from rllm_b200 import SamplingParams
    name = "A"
    prompts = prompts_for(name, [9, 30, 4], 12)
    params = [SamplingParams(temperature=0.0, max_tokens=7, ignore_eos=True, logprobs=3),
              SamplingParams(temperature=0.0, max_tokens=9, ignore_eos=True),
              SamplingParams(temperature=0.8, seed=4, repetition_penalty=1.3, max_tokens=6, ignore_eos=True, logprobs=0)]
    llm = make_llm(model_dirs, name)
    outs = llm.generate(prompts, params)
    plain = pl.read_model_dir(model_dirs[name])
    assert outs[1].outputs[0].logprobs is None
    for p, sp, o in zip(prompts, params, outs):
        if sp.logprobs is None:
            continue
        got = o.outputs[0]
        assert len(got.logprobs) == len(got.token_ids) == sp.max_tokens
        toks = list(p)
        for t, entry in zip(got.token_ids, got.logprobs):
            row = plain.logits(toks)[-1].numpy()
            assert entry.token_id == t
            assert abs(entry.logprob - pl.logprob_of(row, t)) <= 1e-3
            top = pl.top_logprobs(row, sp.logprobs)
            assert [i for i, _ in entry.top_logprobs] == [i for i, _ in top]
            np.testing.assert_allclose([v for _, v in entry.top_logprobs], [v for _, v in top], atol=1e-3)
            toks.append(t)
    # greedy: the chosen token is the likeliest one
    assert all(e.top_logprobs[0][0] == e.token_id for e in outs[0].outputs[0].logprobs)
