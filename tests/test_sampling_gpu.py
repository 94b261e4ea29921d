"""The sampling kernels against the plain sampler (tests/plain_llama.py), on
vocabularies that are no power of two."""
import numpy as np
import pytest
import torch

import plain_llama as pl

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


@pytest.fixture(scope="module")
def sampler():
    from rllm_b200.sampling import Sampler
    return Sampler(DEV)


def rows_for(params_list, seeds, gen_index, contexts=None, eos=()):
    from rllm_b200.sampling import SamplingRow
    return [SamplingRow(p, s, g, (contexts[i] if contexts else ()), eos)
            for i, (p, s, g) in enumerate(zip(params_list, seeds, gen_index))]


def banned(p, context):
    """Tokens that the bad words rule out behind ``context``: a word's last token, if the tokens before it are
    the context's last ones (the plain restatement; the reference masks it whatever the context,
    crates/rllm-sampling/src/sampler.rs:95-98)."""
    out = []
    for w in p.bad_words_token_ids:
        k = len(w) - 1
        if k == 0 or list(context[-k:]) == list(w[:k]) and len(context) >= k:
            out.append(int(w[-1]))
    return out


def plain_pick(logits_row, p, seed, gen_index, context=(), eos=()):
    suppress = list(eos) if (p.min_tokens > 0 and gen_index < p.min_tokens) else []
    suppress += banned(p, context)
    x = pl.process_logits(logits_row, context=context, logit_bias=p.logit_bias,
                          repetition_penalty=p.repetition_penalty, frequency_penalty=p.frequency_penalty,
                          presence_penalty=p.presence_penalty, allowed_token_ids=p.allowed_token_ids,
                          suppress=suppress, temperature=p.temperature, top_k=p.top_k, top_p=p.top_p,
                          min_p=p.min_p)
    return pl.sample_row(x, p.temperature, p.top_k, pl.uniform_for(seed, gen_index))


@pytest.mark.parametrize("V", [1, 255, 4096, 4097, 128256, 128259, 300001])
def test_argmax_kernel_at_any_width(V):
    """Rows are cut into ranges for several CTAs: the largest value wins wherever it lies, ties go to
    the lowest index also across the ranges' edges, and a row of -inf gives token 0."""
    from rllm_b200.kernels import ops
    torch.manual_seed(V)
    R = 7
    logits = torch.randn(R, V, device=DEV)
    if V > 4:
        logits[1, V - 1] = 40.0                       # the last element
        logits[2, 0] = logits[2, V - 1] = 41.0        # a tie between the first and the last range
        logits[3, V // 2] = logits[3, V // 2 + 1] = 42.0
        logits[4] = -float("inf")
        logits[5, min(V - 1, 4096)] = logits[5, min(V - 1, 4095)] = 43.0   # a tie across an edge between ranges
    out = torch.full((R,), -1, dtype=torch.int32, device=DEV)
    ops.argmax(logits, out)
    want = logits.argmax(dim=1).tolist()
    if V > 4:
        want[2], want[3], want[4], want[5] = 0, V // 2, 0, min(V - 1, 4095)
    assert out.tolist() == want
    ops.argmax(logits[:, : V - V // 3], out)           # a view: rows are not contiguous
    assert out.tolist()[0] == int(logits[0, : V - V // 3].argmax())


@pytest.mark.parametrize("V", [7, 256, 4097, 128256, 300001])
def test_sampling_by_several_ctas_a_row_draws_the_same_tokens(V):
    """The chain of kernels that cuts a row into ranges draws the tokens of the one-CTA kernel: every
    mix of temperature, top-k, top-p and min-p, seeds and steps, greedy rows, rows of -inf, ties."""
    from rllm_b200.kernels import ops
    torch.manual_seed(V)
    R = 16
    logits = torch.randn(R, V, device=DEV) * 4
    logits[3] = -float("inf")
    logits[4, : V // 2] = -float("inf")
    logits[13] = torch.round(logits[13])              # many equal values: ties at every threshold
    temperature = torch.tensor([0.7, 1.3, 0.0, 0.9, 0.5, 2.0, 0.8, 1.0, 0.3, 1.0, 0.8, 5.0, 1.0, 1.0, 0.6, 1.5],
                               device=DEV)
    top_k = torch.tensor([-1, 0, -1, 5, -1, 1, 3, V + 5, 50, -1, 2, -1, 40, 7, V - 1, 1000], dtype=torch.int32,
                         device=DEV)
    top_p = torch.tensor([1, 1, 1, 0.9, 1, 1, 1, 0.5, 0.95, 0.3, 1, 0.999, 0.8, 0.9, 0.7, 0.6], dtype=torch.float32,
                         device=DEV)
    min_p = torch.tensor([0, 0, 0, 0, 0.1, 0, 0.3, 0, 0, 0.01, 0, 0, 0.05, 0, 0, 0.2], dtype=torch.float32,
                         device=DEV)
    for select in (True, False):
        if not select:
            top_k = torch.where((top_k > 1) & (top_k < V), torch.full_like(top_k, -1), top_k)
            top_p = torch.ones_like(top_p)
        for step in range(5):
            seeds = torch.arange(R, dtype=torch.int64, device=DEV) * 7919 + step
            gen = torch.full((R,), step * 3, dtype=torch.int64, device=DEV)
            a = torch.full((R,), -1, dtype=torch.int32, device=DEV)
            b = torch.full((R,), -2, dtype=torch.int32, device=DEV)
            ops.sample_one_cta(logits, temperature, top_k, top_p, min_p, seeds, gen, a)
            ops.sample(logits, temperature, top_k, top_p, min_p, seeds, gen, b, with_select=select)
            assert a.tolist() == b.tolist(), (select, step)
    assert len(set(a.tolist())) > 3


def test_greedy_is_argmax_with_lowest_index_on_ties(sampler):
    from rllm_b200.sampling import SamplingParams
    torch.manual_seed(0)
    logits = torch.randn(5, 128256 + 3, device=DEV)
    logits[2, 77] = logits[2, 90000] = 50.0
    logits[3, 128258] = 60.0
    p = SamplingParams(temperature=0.0)
    got = sampler.sample(logits.clone(), rows_for([p] * 5, range(5), [0] * 5)).tolist()
    assert got == logits.argmax(dim=1).tolist() and got[2] == 77 and got[3] == 128258
    # top_k == 1 is greedy too (crates/rllm-sampling/src/sampler.rs:117)
    p1 = SamplingParams(temperature=0.9, top_k=1)
    assert sampler.sample(logits.clone(), rows_for([p1] * 5, range(5), [0] * 5)).tolist() == got


@pytest.mark.parametrize("V", [389, 5003, 128256])
def test_draws_match_the_plain_sampler(sampler, V):
    from rllm_b200.sampling import SamplingParams
    rng = np.random.default_rng(V)
    variants = [SamplingParams(temperature=0.7), SamplingParams(temperature=1.3, top_k=40),
                SamplingParams(temperature=1.0, top_p=0.8), SamplingParams(temperature=0.9, min_p=0.05),
                SamplingParams(temperature=1.1, top_k=200, top_p=0.9, min_p=0.01),
                SamplingParams(temperature=2.0, top_k=3)]
    R = 48
    logits = (rng.standard_normal((R, V)) * 3).astype(np.float32)
    params = [variants[i % len(variants)] for i in range(R)]
    seeds = [int(s) for s in rng.integers(0, 2 ** 62, size=R)]
    gen = [int(g) for g in rng.integers(0, 5000, size=R)]
    got = sampler.sample(torch.from_numpy(logits).to(DEV), rows_for(params, seeds, gen)).tolist()
    want = [plain_pick(logits[r], params[r], seeds[r], gen[r]) for r in range(R)]
    assert got == want


def test_a_row_does_not_depend_on_its_batch(sampler):
    from rllm_b200.sampling import SamplingParams
    rng = np.random.default_rng(7)
    V = 2000
    logits = (rng.standard_normal((9, V)) * 2).astype(np.float32)
    p = SamplingParams(temperature=0.8, top_p=0.95)
    seeds, gen = list(range(100, 109)), list(range(9))
    full = sampler.sample(torch.from_numpy(logits).to(DEV), rows_for([p] * 9, seeds, gen)).tolist()
    for r in (0, 4, 8):
        alone = sampler.sample(torch.from_numpy(logits[r:r + 1]).to(DEV), rows_for([p], [seeds[r]], [gen[r]]))
        assert alone.tolist() == [full[r]]
    # mixed with greedy rows
    mixed = [p, SamplingParams(temperature=0.0)] * 4 + [p]
    got = sampler.sample(torch.from_numpy(logits).to(DEV), rows_for(mixed, seeds, gen)).tolist()
    assert got[0::2] == full[0::2] and got[1::2] == logits[1::2].argmax(axis=1).tolist()


def test_draw_frequencies(sampler):
    from rllm_b200.sampling import SamplingParams
    probs = np.array([0.5, 0.25, 0.125, 0.125, 0.0], dtype=np.float64)
    with np.errstate(divide="ignore"):
        row = np.log(probs).astype(np.float32)
    R = 4000
    logits = torch.from_numpy(np.tile(row, (R, 1))).to(DEV)
    p = SamplingParams(temperature=1.0)
    got = sampler.sample(logits, rows_for([p] * R, [5] * R, list(range(R)))).cpu().numpy()
    freq = np.bincount(got, minlength=5) / R
    assert freq[4] == 0 and np.allclose(freq[:4], probs[:4], atol=0.03)
    again = sampler.sample(logits, rows_for([p] * R, [5] * R, list(range(R)))).cpu().numpy()
    assert (again == got).all()                      # same seed and index: same token


def test_processors_match_the_plain_ones(sampler):
    from rllm_b200.sampling import SamplingParams
    rng = np.random.default_rng(3)
    V, R = 777, 12
    logits = (rng.standard_normal((R, V)) * 2).astype(np.float32)
    contexts = [[int(t) for t in rng.integers(0, 50, size=rng.integers(1, 60))] for _ in range(R)]
    eos = (5, 9)
    ps = []
    for r in range(R):
        ps.append(SamplingParams(
            temperature=[0.0, 0.8][r % 2], repetition_penalty=[1.0, 1.3, 0.7][r % 3],
            frequency_penalty=[0.0, 0.4][(r // 2) % 2], presence_penalty=[0.0, 1.5][(r // 3) % 2],
            logit_bias={3: 5.0, 700: -2.0} if r % 4 == 0 else {},
            allowed_token_ids=list(range(0, V, 3)) if r % 5 == 0 else None,
            # a one-token word, a word whose first tokens are the context's last ones, and one that does not fit
            bad_words_token_ids=[[int(np.argmax(logits[r]))], contexts[r][-2:] + [int(np.argsort(logits[r])[-2])],
                                 [contexts[r][-1] + 1, int(np.argsort(logits[r])[-3])]] if r % 3 == 1 else (),
            min_tokens=4 if r % 2 else 0))
    seeds, gen = list(range(R)), [r % 6 for r in range(R)]
    dev = torch.from_numpy(logits).to(DEV)
    got = sampler.sample(dev, rows_for(ps, seeds, gen, contexts, eos)).tolist()
    want = [plain_pick(logits[r], ps[r], seeds[r], gen[r], contexts[r], eos) for r in range(R)]
    assert got == want
    # and the edited logits themselves
    dev = torch.from_numpy(logits).to(DEV)
    sampler.apply_processors(dev, rows_for(ps, seeds, gen, contexts, eos))
    for r in range(R):
        suppress = list(eos) if (ps[r].min_tokens > 0 and gen[r] < ps[r].min_tokens) else []
        suppress += banned(ps[r], contexts[r])
        if ps[r].bad_words_token_ids:
            top3 = [int(t) for t in np.argsort(logits[r])[-3:]]
            assert top3[2] in suppress and top3[0] not in banned(ps[r], contexts[r])
            assert (top3[1] in suppress) == (len(contexts[r]) >= 2)
        x = pl.process_logits(logits[r], context=contexts[r], logit_bias=ps[r].logit_bias,
                              repetition_penalty=ps[r].repetition_penalty,
                              frequency_penalty=ps[r].frequency_penalty,
                              presence_penalty=ps[r].presence_penalty,
                              allowed_token_ids=ps[r].allowed_token_ids, suppress=suppress, temperature=0.0)
        np.testing.assert_allclose(dev[r].cpu().numpy(), x, rtol=1e-6, atol=1e-6)


def test_params_are_validated():
    from rllm_b200.sampling import InvalidSamplingParams, SamplingParams
    SamplingParams().validate()
    SamplingParams(n=3).validate()
    assert SamplingParams().max_tokens == 16 and SamplingParams().temperature == 1.0
    for bad in (dict(temperature=-1.0), dict(top_p=1.5), dict(n=0), dict(n=2, temperature=0.0), dict(n=2, top_k=1),
                dict(repetition_penalty=0.0),
                dict(presence_penalty=3.0), dict(logprobs=-1), dict(logprobs=33), dict(bad_words_token_ids=[[1], []])):
        with pytest.raises(InvalidSamplingParams):
            SamplingParams(**bad).validate()


@pytest.mark.parametrize("V", [311, 4097, 128256])
def test_logprobs_kernel_matches_the_plain_formulas(V):
    """The log-probability of a chosen token and the N likeliest tokens of a row, from raw logits; equal
    logits come lower index first; -inf logits are left out; N beyond what is left gives id -1."""
    from rllm_b200.kernels import ops
    g = torch.Generator().manual_seed(V)
    R, N = 5, 6
    logits = torch.randn(R, V, generator=g) * 3
    logits[1, 7] = logits[1, 3] = logits[1].max() + 1.0            # a tie at the top
    logits[2, :] = float("-inf")
    logits[2, [5, 9, 11]] = torch.tensor([0.5, 0.5, -2.0])          # three tokens left: N runs out
    logits[3, 100:] = float("-inf")
    tokens = torch.tensor([0, 7, 9, 50, V - 1], dtype=torch.int32)
    lp, ids, vals = ops.logprobs(logits.cuda(), tokens.cuda(), N)
    lp0, ids0, _ = ops.logprobs(logits.cuda(), tokens.cuda(), 0)
    assert ids0.shape == (R, 0) and torch.equal(lp0, lp)
    for r in range(R):
        row = logits[r].numpy()
        want = pl.logprob_of(row, int(tokens[r]))
        assert abs(float(lp[r]) - want) <= 1e-4 * max(1.0, abs(want)), (r, float(lp[r]), want)
        top = pl.top_logprobs(row, N)
        got_ids = ids[r].tolist()
        assert got_ids[: len(top)] == [i for i, _ in top] and all(i == -1 for i in got_ids[len(top):])
        np.testing.assert_allclose(vals[r, : len(top)].cpu().numpy(), [v for _, v in top], rtol=1e-4, atol=1e-4)
