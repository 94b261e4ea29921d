"""Trace replay against the plain implementation: the same requests whole, with
the last 32 tokens decoded one by one, in portions of changing size, and mixed
with other requests so that pages are used again; in float32 and in bfloat16;
for both tiny configurations.  Every logits row of every mode is compared with
the plain implementation's row for the same (request, position)."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import plain_llama
import replay_util as ru
from conftest import TINY

pytestmark = pytest.mark.gpu

# max |engine - plain| over a request's logits, relative to max |plain|
TOL = {"float32": 1e-4, "bfloat16": 2e-2}

LENGTHS = {"A": [5, 12, 17, 70, 100, 33, 64, 49], "B": [1, 31, 70, 150, 300, 97, 2, 210],
           "C": [3, 130, 257, 400, 129, 64, 500, 33], "D": [2, 40, 67, 150, 9, 101],
           "B0": [1, 31, 70, 150, 97, 2, 210, 256]}


def make_requests(name: str):
    cfg, _, _ = TINY[name]
    rng = np.random.default_rng({"A": 1, "B": 3, "C": 8, "D": 4, "B0": 3}[name])
    return {f"r{i}": [int(t) for t in rng.integers(0, cfg["vocab_size"], size=n)]
            for i, n in enumerate(LENGTHS[name])}


_plain_cache = {}


def plain_logits(model_dirs, name: str, dtype: str):
    key = (name, dtype)
    if key not in _plain_cache:
        model = plain_llama.read_model_dir(model_dirs[name],
                                           round_to=torch.bfloat16 if dtype == "bfloat16" else None)
        _plain_cache[key] = {rid: model.logits(toks).numpy() for rid, toks in make_requests(name).items()}
    return _plain_cache[key]


def compare(got, want_by_req, reqs, dtype, what):
    worst = 0.0
    for rid, toks in reqs.items():
        want = want_by_req[rid]
        have = np.stack([got[(rid, p)] for p in range(len(toks))])
        assert np.isfinite(have).all(), f"{what}: request {rid} has non-finite logits"
        err = np.abs(have - want).max(axis=1) / np.abs(want).max()
        bad = np.nonzero(err > TOL[dtype])[0]
        assert bad.size == 0, (f"{what}: request {rid} (length {len(toks)}): first wrong position "
                               f"{int(bad[0])}, error {err[bad[0]]:.3e} > {TOL[dtype]:.0e}; "
                               f"wrong positions {bad[:20].tolist()}")
        worst = max(worst, float(err.max()))
    return worst


MODES = {
    "whole": lambda reqs: ru.trace_whole(reqs),
    "tail_decode": lambda reqs: ru.trace_tail_decode(reqs, 32),
    "portions": lambda reqs: ru.trace_portions(reqs, seed=5),
    "mixed": lambda reqs: ru.trace_mixed(reqs, seed=11, live=4, tail=32),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "B0"])
@pytest.mark.parametrize("mode", list(MODES))
def test_replay_matches_plain(model_dirs, name, dtype, mode):
    cfg, _, page = TINY[name]
    reqs = make_requests(name)
    tb = MODES[mode](reqs)
    if mode == "mixed":
        # so few pages that later requests get pages that earlier ones gave back
        total = sum(ru.round64(len(t)) for t in reqs.values())
        assert tb.peak < total
    got = ru.run_trace(model_dirs[name], dtype, tb, cfg["vocab_size"], page_size=page)
    worst = compare(got, plain_logits(model_dirs, name, dtype), reqs, dtype, f"{name}/{dtype}/{mode}")
    print(f"{name} {dtype} {mode}: worst relative error {worst:.3e}")


def test_modes_agree_in_float32(model_dirs):
    """The cuts agree with each other far more closely than with the oracle's
    float64: a row's arithmetic does not depend on the cut."""
    cfg, _, page = TINY["B"]
    reqs = make_requests("B")
    a = ru.run_trace(model_dirs["B"], "float32", ru.trace_whole(reqs), cfg["vocab_size"], page_size=page)
    b = ru.run_trace(model_dirs["B"], "float32", ru.trace_mixed(reqs, seed=2), cfg["vocab_size"], page_size=page)
    for key in a:
        scale = np.abs(a[key]).max()
        assert np.abs(a[key] - b[key]).max() <= 2e-6 * scale, key


def test_trace_run_program(model_dirs):
    """The program itself, as a child process: bin/trace_run."""
    cfg, _, page = TINY["A"]
    reqs = {k: v for k, v in list(make_requests("A").items())[:3]}
    tb = ru.trace_mixed(reqs, seed=4, live=2, tail=4)
    got = ru.run_trace(model_dirs["A"], "float32", tb, cfg["vocab_size"], page_size=page, subprocess_mode=True)
    compare(got, plain_logits(model_dirs, "A", "float32"), reqs, "float32", "program")


def test_too_few_pages_is_an_error(model_dirs):
    cfg, _, page = TINY["A"]
    reqs = {"r0": list(range(100))}
    tb = ru.trace_whole(reqs)
    with pytest.raises(AssertionError):
        ru.run_trace(model_dirs["A"], "float32", tb, cfg["vocab_size"], page_size=page, max_tokens=64)


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("mode", ["whole", "mixed"])
def test_replay_through_the_tcgen05_gemm(model_dirs, name, mode, monkeypatch):
    """Tiny models are too small for the tcgen05 GEMM to be chosen by itself (it
    wants enough tiles to fill the GPU); RLLM_GEMM=tcgen05 sends every product of
    more than 8 rows through it, tails in all three dimensions included."""
    monkeypatch.setenv("RLLM_GEMM", "tcgen05")
    cfg, _, page = TINY[name]
    reqs = make_requests(name)
    got = ru.run_trace(model_dirs[name], "bfloat16", MODES[mode](reqs), cfg["vocab_size"], page_size=page)
    compare(got, plain_logits(model_dirs, name, "bfloat16"), reqs, "bfloat16", f"{name}/tcgen05/{mode}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", list(MODES))
def test_replay_with_head_size_64(model_dirs, dtype, mode):
    """tiny-C has the head size of the tcgen05 attention kernel: in bfloat16 its prompt portions
    run there, over several 128-key tiles, in every way of cutting."""
    cfg, _, page = TINY["C"]
    reqs = make_requests("C")
    got = ru.run_trace(model_dirs["C"], dtype, MODES[mode](reqs), cfg["vocab_size"], page_size=page)
    compare(got, plain_logits(model_dirs, "C", dtype), reqs, dtype, f"C/{dtype}/{mode}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", list(MODES))
def test_replay_with_head_size_48(model_dirs, dtype, mode):
    """tiny-D: heads of 48 (no tensor-core attention kernel takes them: the general kernel runs in both
    dtypes), one kv head a head, pages of 4 keys, one layer, tied embeddings."""
    cfg, _, page = TINY["D"]
    reqs = make_requests("D")
    got = ru.run_trace(model_dirs["D"], dtype, MODES[mode](reqs), cfg["vocab_size"], page_size=page)
    compare(got, plain_logits(model_dirs, "D", dtype), reqs, dtype, f"D/{dtype}/{mode}")


def test_attention_kernels_agree_through_replay(model_dirs, monkeypatch):
    """RLLM_ATTENTION=mma keeps prompt portions on the mma.sync kernel: the same trace through
    both kernels gives logits that differ by bfloat16 rounding only."""
    cfg, _, page = TINY["C"]
    reqs = make_requests("C")
    a = ru.run_trace(model_dirs["C"], "bfloat16", MODES["portions"](reqs), cfg["vocab_size"], page_size=page)
    monkeypatch.setenv("RLLM_ATTENTION", "mma")
    b = ru.run_trace(model_dirs["C"], "bfloat16", MODES["portions"](reqs), cfg["vocab_size"], page_size=page)
    compare(b, plain_logits(model_dirs, "C", "bfloat16"), reqs, "bfloat16", "C/mma/portions")
    worst = max(float(np.abs(a[k] - b[k]).max() / np.abs(b[k]).max()) for k in a)
    assert 0 < worst <= TOL["bfloat16"], worst       # not the same kernel, and close


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_decoding_with_and_without_norm_kernels(model_dirs, name, monkeypatch):
    """Steps of up to 8 tokens run a layer without norm kernels (the products carry the RMSNorm);
    RLLM_FUSED_NORM=0 runs the same steps with them.  Both match the plain implementation, and
    they differ from each other (so both ways were taken) by rounding only."""
    cfg, _, page = TINY[name]
    reqs = make_requests(name)
    tb = ru.trace_mixed(reqs, seed=6, live=3, tail=32)
    a = ru.run_trace(model_dirs[name], "bfloat16", tb, cfg["vocab_size"], page_size=page)
    monkeypatch.setenv("RLLM_FUSED_NORM", "0")
    b = ru.run_trace(model_dirs[name], "bfloat16", ru.trace_mixed(reqs, seed=6, live=3, tail=32), cfg["vocab_size"],
                     page_size=page)
    want = plain_logits(model_dirs, name, "bfloat16")
    compare(a, want, reqs, "bfloat16", f"{name}/fused norm")
    compare(b, want, reqs, "bfloat16", f"{name}/norm kernels")
    worst = max(float(np.abs(a[k] - b[k]).max() / np.abs(b[k]).max()) for k in a)
    assert 0 < worst <= TOL["bfloat16"], worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_long_decoding(model_dirs, name, dtype):
    """A short prompt, then one token a step for as long as the model allows: over many pages, past
    split and chunk edges of the decode kernels and (tiny-B) far past the rotary scaling's original
    context.  Two more requests decode beside it, starting at other steps."""
    cfg, _, page = TINY[name]
    n = cfg["max_position_embeddings"] - 1
    rng = np.random.default_rng(17)
    reqs = {"long": [int(t) for t in rng.integers(0, cfg["vocab_size"], size=n)],
            "mid": [int(t) for t in rng.integers(0, cfg["vocab_size"], size=n // 3)],
            "late": [int(t) for t in rng.integers(0, cfg["vocab_size"], size=n // 5)]}
    tb = ru.TraceBuilder()
    fed = {k: 0 for k in reqs}
    tb.step([("long", reqs["long"][:3])])
    fed["long"] = 3
    step = 0
    while any(fed[k] < len(v) for k, v in reqs.items()):
        entries, end = [], []
        for k, v in reqs.items():
            if k == "mid" and step < 10 or k == "late" and step < n // 2:
                continue
            if fed[k] < len(v):
                entries.append((k, v[fed[k]:fed[k] + 1]))
                fed[k] += 1
                if fed[k] == len(v):
                    end.append(k)
        tb.step(entries, end=end)
        step += 1
    got = ru.run_trace(model_dirs[name], dtype, tb, cfg["vocab_size"], page_size=page)
    model = plain_llama.read_model_dir(model_dirs[name], round_to=torch.bfloat16 if dtype == "bfloat16" else None)
    want = {k: model.logits(v).numpy() for k, v in reqs.items()}
    compare(got, want, reqs, dtype, f"{name}/{dtype}/long decoding")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_first_tokens_of_a_sequence(model_dirs, name, dtype):
    """Sequences of 1 to 5 tokens, whole and token by token: position 0 sees only itself, and the
    first page is only partly filled."""
    cfg, _, page = TINY[name]
    rng = np.random.default_rng(23)
    reqs = {f"s{n}": [int(t) for t in rng.integers(0, cfg["vocab_size"], size=n)] for n in range(1, 6)}
    model = plain_llama.read_model_dir(model_dirs[name], round_to=torch.bfloat16 if dtype == "bfloat16" else None)
    want = {k: model.logits(v).numpy() for k, v in reqs.items()}
    whole = ru.run_trace(model_dirs[name], dtype, ru.trace_whole(reqs), cfg["vocab_size"], page_size=page)
    compare(whole, want, reqs, dtype, f"{name}/{dtype}/first tokens whole")
    single = ru.run_trace(model_dirs[name], dtype, ru.trace_tail_decode(reqs, tail=8), cfg["vocab_size"], page_size=page)
    compare(single, want, reqs, dtype, f"{name}/{dtype}/first tokens one by one")
    # all five first tokens in one step, as a batch of single-token prompts
    tb = ru.TraceBuilder()
    tb.step([(k, v[:1]) for k, v in reqs.items()], end=list(reqs))
    batch = ru.run_trace(model_dirs[name], dtype, tb, cfg["vocab_size"], page_size=page)
    for k in reqs:
        err = np.abs(batch[(k, 0)] - want[k][0]).max() / np.abs(want[k]).max()
        assert err <= TOL[dtype], (k, err)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_request_id_used_again_after_its_end(model_dirs, dtype):
    """Request "a" decodes and ends; "b" takes the pages it gave back and stays alive; a new request, again
    called "a", of the same length but with other tokens, decodes alone in its steps.  Its decode steps
    have the shape of the first a's (one request, the same number of pages), on other pages: nothing of
    the first a's block table may be taken for the second's."""
    cfg, _, page = TINY["A"]
    rng = np.random.default_rng(21)
    V = cfg["vocab_size"]
    first = [int(t) for t in rng.integers(0, V, size=40)]
    other = [int(t) for t in rng.integers(0, V, size=50)]
    second = [int(t) for t in rng.integers(0, V, size=40)]
    tb = ru.TraceBuilder()
    tb.step([("a", first[:34])])
    for i in range(34, 40):
        tb.step([("a", first[i:i + 1])], end=["a"] if i == 39 else [])
    tb.step([("b", other)])                      # gets the pages that a gave back
    n_first = len(tb.steps)
    tb.step([("a", second[:34])])
    for i in range(34, 40):
        tb.step([("a", second[i:i + 1])])
    tb.step([("b", [7])], end=["a", "b"])
    # the second life of "a" under a name of its own
    for i in range(n_first, len(tb.rows) - 1):
        tb.rows[i] = [("a2", pos) for _, pos in tb.rows[i]]
    got = ru.run_trace(model_dirs["A"], dtype, tb, V, page_size=page, max_tokens=192)
    model = plain_llama.read_model_dir(model_dirs["A"], round_to=torch.bfloat16 if dtype == "bfloat16" else None)
    want = {"a": model.logits(first).numpy(), "a2": model.logits(second).numpy(), "b": model.logits(other + [7]).numpy()}
    tol = 1e-4 if dtype == "float32" else 3e-2
    for (rid, pos), row in got.items():
        ref = want[rid][pos]
        err = float(np.abs(row - ref).max() / np.abs(ref).max())
        assert err <= tol, (rid, pos, err)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,common_len", [("A", 37), ("A", 48), ("B", 21), ("C", 150)])
def test_fork_parent_and_child_diverge(model_dirs, name, common_len, dtype):
    """A request is fed ``common_len`` tokens (in two portions), then forked: the child shares its full pages
    and gets a copy of the partly filled last one (none at a page's edge: 48 = 3 pages of 16).  Parent and
    child go on with different tokens, portions of one beside decoded tokens of the other, a second child is
    forked from the first a few tokens later, and every row of all three matches the plain implementation on
    its own whole sequence: nobody saw a key that another wrote after the fork
    (crates/rllm-cache/src/manager.rs:220-245, block_pool.rs:292-302)."""
    cfg, _, page = TINY[name]
    V = cfg["vocab_size"]
    rng = np.random.default_rng(31)
    draw = lambda n: [int(t) for t in rng.integers(0, V, size=n)]
    common, tail_p, tail_c, tail_d = draw(common_len), draw(24), draw(24), draw(9)
    tb = ru.TraceBuilder()
    tb.step([("p", common[:common_len - 5])])
    tb.step([("p", common[common_len - 5:])])
    tb.step([("p", tail_p[:1]), ("c", tail_c[:7])], fork=[("p", "c")])
    tb.step([("p", tail_p[1:2]), ("c", tail_c[7:8])])
    tb.step([("p", tail_p[2:13]), ("c", tail_c[8:9]), ("d", tail_d[:2])], fork=[("c", "d")])
    for i in range(9, 20):
        entries = [("p", tail_p[4 + i:5 + i]), ("c", tail_c[i:i + 1])]
        if i - 7 < len(tail_d):
            entries.append(("d", tail_d[i - 7:i - 6]))
        tb.step(entries)
    tb.step([("c", tail_c[20:])], end=["p", "c", "d"])
    seqs = {"p": common + tail_p, "c": common + tail_c, "d": common + tail_c[:8] + tail_d}
    got = ru.run_trace(model_dirs[name], dtype, tb, V, page_size=page)
    model = plain_llama.read_model_dir(model_dirs[name], round_to=torch.bfloat16 if dtype == "bfloat16" else None)
    want = {k: model.logits(v).numpy() for k, v in seqs.items()}
    assert {k for k, _ in got} == {"p", "c", "d"}
    assert max(pos for k, pos in got if k == "d") == len(seqs["d"]) - 1
    for (rid, pos), row in got.items():
        ref = want[rid][pos]
        err = float(np.abs(row - ref).max() / np.abs(want[rid]).max())
        assert err <= TOL[dtype], (rid, pos, err)
