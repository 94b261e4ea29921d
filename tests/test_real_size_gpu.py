"""Layers of real size: two layers with the widths of Llama-3.2-1B (hidden 2048, 32 / 8 heads of 64,
intermediate 8192) and its whole vocabulary (128,256, tied head), random weights.

The float32 path is compared with the plain implementation (float64, whole sequences) in every way of
cutting, as the tiny configurations are; sizes of this kind reach code that the tiny ones do not (full
tiles of every product, many CTAs a row in the vocabulary product and in sampling, several CTAs a sequence
in decode attention).  The bfloat16 path is then compared with the float32 path on schedules that only real
widths reach: decode steps of 32 and 64 rows (the library's products with the norm and SiLU kernels between
them), and generation with a shared prefix and so few pages that requests are preempted.

The weights are drawn on the device; the plain implementation gets the same tensors (the generator gives the
same bits wherever it runs, see test_kernels_gpu.py).
"""
import json
import os

import numpy as np
import pytest
import torch

import plain_llama as pl
import replay_util as ru

pytestmark = pytest.mark.gpu

V = 128256
CFG = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 2, "hidden_size": 2048,
       "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64, "intermediate_size": 8192,
       "vocab_size": V, "rope_theta": 500000.0,
       "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                        "original_max_position_embeddings": 8192},
       "max_position_embeddings": 131072, "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
       "hidden_act": "silu", "torch_dtype": "bfloat16", "bos_token_id": 128000, "eos_token_id": 128001}
SEED = 0


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    d = str(tmp_path_factory.mktemp("llama_1b_two_layers"))
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(CFG, f)
    return d


@pytest.fixture(scope="module")
def plain(folder):
    """The plain implementation on the tensors that ``random_weights=True, seed=SEED`` draws."""
    from rllm_b200.config import load_model_description
    from rllm_b200.models import DecoderModel
    from rllm_b200.weights import draw_tensor
    _, spec = load_model_description(folder)
    tensors = {}
    for ts in DecoderModel(spec).tensor_specs():
        if not ts.optional:
            tensors[ts.name] = draw_tensor(ts, SEED, "cuda:0").cpu().to(pl.DTYPE)
    torch.cuda.empty_cache()
    return pl.PlainLlama(CFG, tensors)


@pytest.fixture(scope="module")
def model_f32(folder):
    from rllm_b200.engine.loading import load_model
    _, model = load_model(folder, dtype="fp32", random_weights=True, seed=SEED, draw_on_device=True)
    return model


REQS = {f"r{i}": [int(t) for t in np.random.default_rng(40 + i).integers(0, V, size=n)]
        for i, n in enumerate([70, 33, 100, 49])}


def wanted(rid, pos):
    """A ninth of the rows and each request's last two: the vocabulary product of the oracle is what costs."""
    return pos % 9 == 4 or pos >= len(REQS[rid]) - 2


@pytest.fixture(scope="module")
def plain_rows(plain):
    out = {}
    for rid, toks in REQS.items():
        rows = [p for p in range(len(toks)) if wanted(rid, p)]
        out[rid] = dict(zip(rows, plain.logits_at(toks, rows).numpy()))
    return out


@pytest.mark.parametrize("mode", ["whole", "tail_decode", "portions", "mixed"])
def test_float32_path_at_real_widths_matches_plain(model_f32, plain_rows, mode):
    tb = {"whole": lambda: ru.trace_whole(REQS, want=wanted),
          "tail_decode": lambda: ru.trace_tail_decode(REQS, 32, want=wanted),
          "portions": lambda: ru.trace_portions(REQS, seed=5, want=wanted),
          "mixed": lambda: ru.trace_mixed(REQS, seed=11, live=3, tail=32, want=wanted)}[mode]()
    if mode == "mixed":
        assert tb.peak < sum(ru.round64(len(t)) for t in REQS.values())      # pages are used again
    got = ru.run_trace_on_model(model_f32, tb, page_size=16)
    assert set(got) == {(rid, p) for rid, rows in plain_rows.items() for p in rows}
    worst = 0.0
    for (rid, pos), row in got.items():
        want = plain_rows[rid][pos]
        err = float(np.abs(row - want).max() / np.abs(want).max())
        assert err <= 1e-4, (mode, rid, pos, err)
        assert int(row.argmax()) == int(want.argmax()), (mode, rid, pos)
        worst = max(worst, err)
    print(f"real widths, float32, {mode}: worst relative error {worst:.3e}")


def test_float32_greedy_tokens_at_real_widths_equal_plain_greedy(model_f32, plain):
    from rllm_b200 import SamplingParams
    from rllm_b200.config.engine_args import EngineArgs
    from rllm_b200.engine.engine_core import EngineCore
    eng = EngineCore(model_f32, EngineArgs(dtype="fp32", max_model_len=256, max_num_seqs=4, num_gpu_blocks=32,
                                           max_num_batched_tokens=16, long_prefill_token_threshold=16,
                                           enable_prefix_caching=False))
    prompts = [REQS["r1"][:12], REQS["r3"][:25]]
    ids = [eng.add_request(p, SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True)) for p in prompts]
    out = {i: [] for i in ids}
    while eng.has_work():
        for o in eng.step():
            out[o.request_id] += o.outputs[0].token_ids
    eng.runner.check_errors()
    for rid, p in zip(ids, prompts):
        toks = list(p)
        for _ in range(5):
            toks.append(int(torch.argmax(plain.logits_at(toks, [len(toks) - 1])[0])))
        assert out[rid] == toks[len(p):]
    assert eng.cache.usage()["num_requests"] == 0


def _llm(folder, dtype, **kw):
    from rllm_b200 import LLM
    kw.setdefault("max_model_len", 2048)
    kw.setdefault("enable_prefix_caching", False)
    return LLM(folder, dtype=dtype, random_weights=True, draw_on_device=True, seed=SEED, **kw)


def test_decode_steps_of_32_and_64_rows_in_bfloat16_follow_float32(folder):
    """64 requests of 3 to 200 tokens, all prompts in one step (1,6xx rows: the tcgen05 products and prompt
    attention), then decode steps of 64, 64, 32 and 32 rows: too many rows for the weight-streaming products,
    too few tiles for the tcgen05 kernel, so the library's product runs with this engine's norm, SiLU and
    attention kernels around it.  Every row of the bfloat16 path is compared with the float32 path."""
    from rllm_b200.engine.runner import StepEntry
    rng = np.random.default_rng(9)
    prompts = {f"q{i}": [int(t) for t in rng.integers(0, V, size=int(n))]
               for i, n in enumerate(rng.integers(3, 200, size=64))}
    feed = rng.integers(0, V, size=(4, 64))
    rows = {}
    for dt in ("fp32", "bf16"):
        llm = _llm(folder, dt, max_num_seqs=64, max_num_batched_tokens=16384, num_gpu_blocks=64 * 14)
        eng, runner = llm.engine, llm.engine.runner
        for k, p in prompts.items():
            eng.cache.admit(k)
            assert eng.cache.ensure(k, 0, len(p) + 4)
        got = [runner.step([StepEntry(k, p, 0, [len(p) - 1]) for k, p in prompts.items()]).float().cpu()]
        keys = list(prompts)
        for i in range(4):
            live = keys if i < 2 else keys[::2]
            entries = [StepEntry(k, [int(feed[i][keys.index(k)])], len(prompts[k]) + i, [0]) for k in live]
            for _ in range(3 if i in (1, 3) else 1):        # the same step again: eager twice, then as a graph
                logits = runner.step(entries)
            got.append(logits.float().cpu())
        runner.check_errors()
        rows[dt] = torch.cat(got)
        del llm, eng, runner
        torch.cuda.empty_cache()
    a, b = rows["fp32"].double(), rows["bf16"].double()
    assert a.shape == (64 + 64 + 64 + 32 + 32, V)
    err = (a - b).abs().amax(dim=1) / a.abs().amax(dim=1)
    same = float((a.argmax(dim=1) == b.argmax(dim=1)).float().mean())
    print(f"real widths, bfloat16 against float32, 32 and 64 rows: worst {float(err.max()):.3e}, "
          f"mean {float(err.mean()):.3e}, same argmax {same:.3f}")
    assert float(err.max()) <= 2.5e-2, err
    # where float32's choice is clear (top-two margin above the error just measured) bfloat16 makes the same
    top = torch.topk(a, 2, dim=1).values
    clear = (top[:, 0] - top[:, 1]) > 2 * 2.5e-2 * a.abs().amax(dim=1)
    assert bool((a.argmax(dim=1) == b.argmax(dim=1))[clear].all())


@pytest.mark.parametrize("n_long,portion", [(6100, 2048), (33_000, 4096)])
def test_a_long_prompt_in_portions_and_decoding_behind_it_in_bfloat16_follow_float32(folder, n_long, portion):
    """One request of 6,100 (33,000) tokens in portions of 2,048 (4,096): prompt attention over up to 48 (258)
    key tiles a row, the later portions with thousands of keys of context before them; a second, short
    request beside it; then decode steps of both (decode attention with 48 (258) chunks a kv head for the
    long one).  Rows of the bfloat16 path against the float32 path."""
    from rllm_b200.engine.runner import StepEntry
    rng = np.random.default_rng(21)
    long_p = [int(t) for t in rng.integers(0, V, size=n_long)]
    short_p = [int(t) for t in rng.integers(0, V, size=37)]
    feed = rng.integers(0, V, size=(6, 2))
    rows = {}
    for dt in ("fp32", "bf16"):
        llm = _llm(folder, dt, max_num_seqs=4, max_num_batched_tokens=portion + 64, num_gpu_blocks=(n_long + 8) // 16 + 8,
                   max_model_len=n_long + 64)
        eng, runner = llm.engine, llm.engine.runner
        for k, n in (("long", n_long + 8), ("short", 37 + 8)):
            eng.cache.admit(k)
            assert eng.cache.ensure(k, 0, n)
        got = []
        for a in range(0, n_long, portion):
            part = long_p[a:a + portion]
            entries = [StepEntry("long", part, a, [0, len(part) // 2, len(part) - 1])]
            if a == portion:
                entries.append(StepEntry("short", short_p, 0, [len(short_p) - 1]))
            got.append(runner.step(entries).float().cpu())
        for i in range(6):
            entries = [StepEntry("long", [int(feed[i][0])], n_long + i, [0]), StepEntry("short", [int(feed[i][1])], 37 + i, [0])]
            got.append(runner.step(entries).float().cpu())
        runner.check_errors()
        rows[dt] = torch.cat(got)
        del llm, eng, runner
        torch.cuda.empty_cache()
    a, b = rows["fp32"].double(), rows["bf16"].double()
    assert a.shape == (3 * -(-n_long // portion) + 1 + 12, V)
    err = (a - b).abs().amax(dim=1) / a.abs().amax(dim=1)
    same = float((a.argmax(dim=1) == b.argmax(dim=1)).float().mean())
    print(f"real widths, {n_long} tokens: bfloat16 against float32 worst {float(err.max()):.3e}, mean {float(err.mean()):.3e}, "
          f"same argmax {same:.3f}")
    assert float(err.max()) <= 2.5e-2, err
    top = torch.topk(a, 2, dim=1).values
    clear = (top[:, 0] - top[:, 1]) > 2 * 2.5e-2 * a.abs().amax(dim=1)
    assert bool((a.argmax(dim=1) == b.argmax(dim=1))[clear].all())


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_generation_at_real_widths_with_a_shared_prefix_and_preemption(folder, dtype):
    """Twelve requests that share a 96-token prefix, with prefix caching on, 48-token portions and a page
    pool that holds about half of what they need: some are preempted and compute again.  In float32 every
    request's tokens equal those of the same request run alone in a roomy engine (a row's arithmetic does
    not depend on the batch there).  In bfloat16 the batch decides which product kernel a step uses, so
    tokens may part from the lone runs at a near-tie; there the same schedule must give the same tokens
    twice."""
    from rllm_b200 import SamplingParams
    rng = np.random.default_rng(77)
    shared = [int(t) for t in rng.integers(0, V, size=96)]
    prompts = [shared + [int(t) for t in rng.integers(0, V, size=int(n))] for n in rng.integers(5, 90, size=12)]
    params = [SamplingParams(temperature=0.0, max_tokens=24, ignore_eos=True) for _ in prompts]
    roomy = _llm(folder, dtype, max_num_seqs=1, num_gpu_blocks=64)
    alone = [roomy.generate([p], [sp])[0].outputs[0].token_ids for p, sp in zip(prompts, params)]
    del roomy
    torch.cuda.empty_cache()
    # pages the twelve need when the six pages of the prefix are held once; half of that is the pool
    need = sum(-(-(len(p) + 24) // 16) for p in prompts) - 11 * (96 // 16)
    tight = _llm(folder, dtype, max_num_seqs=12, num_gpu_blocks=need // 2, max_num_batched_tokens=128,
                 long_prefill_token_threshold=48, enable_prefix_caching=True)
    outs = tight.generate(prompts, params)
    st = tight.engine.stats()
    agree = [next((i for i, (x, y) in enumerate(zip(o.outputs[0].token_ids, a)) if x != y), 24)
             for o, a in zip(outs, alone)]
    print(f"real widths, {dtype}, shared prefix, {need // 2} of {need} pages: {st['num_preemptions']} preemptions, "
          f"{st['prefix_hit_tokens']} prefix-hit tokens, {st['num_steps_ahead']} steps launched ahead; "
          f"tokens equal to the lone runs up to {agree}")
    assert st["num_preemptions"] > 0 and st["prefix_hit_tokens"] >= 96
    assert all(len(o.outputs[0].token_ids) == 24 for o in outs)
    if dtype == "fp32":
        assert agree == [24] * 12
    else:
        # where the tokens part from the lone runs is a matter of near-ties; what must hold is that the
        # same schedule gives the same tokens again (no page or prefix hit is read before it is written)
        again = _llm(folder, dtype, max_num_seqs=12, num_gpu_blocks=need // 2, max_num_batched_tokens=128,
                     long_prefill_token_threshold=48, enable_prefix_caching=True)
        outs2 = again.generate(prompts, params)
        assert [o.outputs[0].token_ids for o in outs2] == [o.outputs[0].token_ids for o in outs]
    tight.engine.cache.check()
    assert tight.engine.cache.usage()["num_requests"] == 0


def test_cache_sized_from_free_memory(folder):
    """No ``num_gpu_blocks``: the pool is sized from the device's free memory, capped at what the limits can
    use (crates/rllm-cache/src/spec.rs:45-60, crates/rllm-server/src/server.rs:367-370).  The engine
    generates with it and gives every page back."""
    from rllm_b200 import SamplingParams
    free0, total = torch.cuda.mem_get_info()
    llm = _llm(folder, "bf16", max_model_len=4096, max_num_seqs=32, gpu_memory_utilization=0.5)
    pages = llm.engine.num_pages
    assert pages == [32 * 256]                 # half of a B200 is far more than 32 x 4096 tokens: the cap applies
    held = llm.engine.storage.num_bytes()
    assert held == (pages[0] + 1) * 2 * 2 * 8 * 16 * 64 * 2          # pages + the spare, K and V, two layers
    assert held < 0.5 * total
    rng = np.random.default_rng(5)
    prompts = [[int(t) for t in rng.integers(0, V, size=int(n))] for n in (40, 300, 7)]
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
    assert all(len(o.outputs[0].token_ids) == 8 for o in outs)
    llm.engine.cache.check()
    u = llm.engine.cache.usage()
    assert u["num_requests"] == 0 and u["groups"][0]["free"] == pages[0]
    # a small share of the memory: fewer pages than the cap, and within the budget
    del llm
    torch.cuda.empty_cache()
    free, total = torch.cuda.mem_get_info()
    used_frac = (total - free) / total
    tiny_share = min(0.99, used_frac + (6 << 30) / total)          # about 6 GiB beyond what is in use now
    small = _llm(folder, "bf16", max_model_len=65536, max_num_seqs=256, gpu_memory_utilization=tiny_share)
    n = small.engine.num_pages[0]
    assert 4 <= n < 256 * 4096
    assert small.engine.storage.num_bytes() <= 6 << 30
    outs = small.generate(prompts[:1], SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
    assert len(outs[0].outputs[0].token_ids) == 4


def test_steps_launched_ahead_in_bfloat16_with_temperature(folder):
    """Decode steps that are put on the GPU before the tokens of the step before are read, with seeded
    temperature sampling in bfloat16: the same tokens as with CUDA graphs (and with them launching ahead)
    switched off."""
    from rllm_b200 import SamplingParams
    rng = np.random.default_rng(123)
    prompts = [[int(t) for t in rng.integers(0, V, size=int(n))] for n in (30, 9, 64, 17, 5)]
    params = [SamplingParams(temperature=0.7, seed=100 + i, max_tokens=20 + i, ignore_eos=True)
              for i in range(len(prompts))]
    ahead = _llm(folder, "bf16", max_num_seqs=8, num_gpu_blocks=64)
    a = [o.outputs[0].token_ids for o in ahead.generate(prompts, params)]
    assert ahead.engine.num_steps_ahead > 10
    del ahead
    torch.cuda.empty_cache()
    plainly = _llm(folder, "bf16", max_num_seqs=8, num_gpu_blocks=64, enable_cuda_graphs=False)
    b = [o.outputs[0].token_ids for o in plainly.generate(prompts, params)]
    assert plainly.engine.num_steps_ahead == 0
    assert a == b
