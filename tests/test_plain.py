"""The plain implementation itself: each part against a hand-computed case or
an independent formulation."""
import math

import numpy as np
import pytest
import torch

import plain_llama as pl
from conftest import TINY_B


def test_rms_norm_by_hand():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    w = torch.tensor([2.0, 0.5], dtype=torch.float64)
    got = pl.rms_norm(x, w, 0.5)
    inv = 1.0 / math.sqrt((9 + 16) / 2 + 0.5)
    assert torch.allclose(got, torch.tensor([[3 * inv * 2, 4 * inv * 0.5]], dtype=torch.float64))


def test_rope_position_zero_is_identity_and_rotation_keeps_length():
    inv = pl.rope_inv_freq(8, 10000.0, None)
    x = torch.randn(3, 2, 8, dtype=torch.float64)
    assert torch.allclose(pl.apply_rope(x, torch.tensor([0, 0, 0]), inv), x)
    y = pl.apply_rope(x, torch.tensor([5, 17, 100]), inv)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1))
    # the rotate-half pairing: dims (i, i + d/2) rotate by position * f_i
    i, p = 1, 17
    a = p * float(inv[i])
    assert math.isclose(float(y[1, 0, i]), float(x[1, 0, i]) * math.cos(a) - float(x[1, 0, i + 4]) * math.sin(a))
    assert math.isclose(float(y[1, 0, i + 4]), float(x[1, 0, i + 4]) * math.cos(a) + float(x[1, 0, i]) * math.sin(a))


def test_rope_dot_product_depends_on_distance_only():
    inv = pl.rope_inv_freq(16, 500000.0, TINY_B["rope_scaling"])
    q, k = torch.randn(1, 1, 16, dtype=torch.float64), torch.randn(1, 1, 16, dtype=torch.float64)
    def dot(pq, pk):
        return float((pl.apply_rope(q, torch.tensor([pq]), inv) * pl.apply_rope(k, torch.tensor([pk]), inv)).sum())
    assert math.isclose(dot(10, 3), dot(107, 100), rel_tol=1e-9, abs_tol=1e-9)


def test_llama3_scaling_hits_all_three_branches():
    sc = TINY_B["rope_scaling"]
    plain = pl.rope_inv_freq(32, 500000.0, None)
    scaled = pl.rope_inv_freq(32, 500000.0, sc)
    kinds = set()
    for f, g in zip(plain.tolist(), scaled.tolist()):
        wl = 2 * math.pi / f
        if wl < sc["original_max_position_embeddings"] / sc["high_freq_factor"]:
            assert g == f; kinds.add("kept")
        elif wl > sc["original_max_position_embeddings"] / sc["low_freq_factor"]:
            assert math.isclose(g, f / sc["factor"]); kinds.add("divided")
        else:
            assert f / sc["factor"] < g < f; kinds.add("blended")
    assert kinds == {"kept", "divided", "blended"}


def test_llama3_scaling_is_continuous_and_monotone_in_the_frequency():
    """What a misreading of the rule would break.  The ratio f'/f as a function of f: 1 for short
    wavelengths, 1/factor for long ones, and between the two bounds a blend that meets both ends without a
    jump, rises with f, and is halfway at the middle of the band in orig / wavelength.  A blend in the
    wrong direction, swapped bounds or a blend in the wavelength instead of its inverse jumps at a bound
    or misses the middle.  Checked for the oracle and for the engine's table."""
    from rllm_b200.parts.rotary import rotary_frequencies
    sc = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
          "original_max_position_embeddings": 8192}
    orig, low, high, factor = 8192.0, 1.0, 4.0, 8.0
    f_keep, f_divide = 2 * math.pi * high / orig, 2 * math.pi * low / orig     # wavelength orig/high, orig/low

    def ratio_plain(f):
        return float(pl.rope_inv_freq(4, 1.0 / (f * f), sc)[1]) / f          # the second of the two frequencies is f

    def ratio_engine(f):
        return rotary_frequencies(4, 1.0 / (f * f), sc)[1] / f
    for ratio in (ratio_plain, ratio_engine):
        assert math.isclose(ratio(f_keep * 1.5), 1.0, rel_tol=1e-12) and math.isclose(ratio(f_divide / 1.5), 1 / factor, rel_tol=1e-12)
        for eps in (1e-6, 1e-9):
            assert math.isclose(ratio(f_keep * (1 - eps)), 1.0, rel_tol=0, abs_tol=10 * eps)
            assert math.isclose(ratio(f_keep * (1 + eps)), 1.0, rel_tol=0, abs_tol=10 * eps)
            assert math.isclose(ratio(f_divide * (1 - eps)), 1 / factor, rel_tol=0, abs_tol=10 * eps)
            assert math.isclose(ratio(f_divide * (1 + eps)), 1 / factor, rel_tol=0, abs_tol=10 * eps)
        grid = [f_divide * (f_keep / f_divide) ** (i / 200) for i in range(1, 200)]
        vals = [ratio(f) for f in grid]
        assert all(a < b for a, b in zip(vals, vals[1:])) and 1 / factor < vals[0] and vals[-1] < 1.0
        # orig / wavelength = orig f / (2 pi) runs from low to high; at its middle the blend is half and half
        f_mid = 2 * math.pi * (low + high) / 2 / orig
        assert math.isclose(ratio(f_mid), 0.5 * (1 + 1 / factor), rel_tol=1e-9)


def test_attention_matches_a_per_query_loop_and_respects_window_and_groups():
    torch.manual_seed(0)
    T, nq, nkv, d = 9, 4, 2, 8
    q, k, v = (torch.randn(T, n, d, dtype=torch.float64) for n in (nq, nkv, nkv))
    pos = torch.arange(T)
    for window in (None, 3):
        got = pl.attention(q, k, v, pos, window=window).reshape(T, nq, d)
        for t in range(T):
            lo = 0 if window is None else max(0, t - window + 1)
            for h in range(nq):
                kv = h // (nq // nkv)
                s = torch.stack([q[t, h] @ k[j, kv] for j in range(lo, t + 1)]) / math.sqrt(d)
                p = torch.softmax(s, 0)
                want = sum(p[j - lo] * v[j, kv] for j in range(lo, t + 1))
                assert torch.allclose(got[t, h], want)


def test_gated_mlp_by_hand():
    x = torch.tensor([[1.0, -2.0]], dtype=torch.float64)
    wg = torch.tensor([[1.0, 0.0], [0.0, 1.0], [1.0, 1.0]], dtype=torch.float64)
    wu = torch.tensor([[2.0, 0.0], [0.0, 3.0], [1.0, -1.0]], dtype=torch.float64)
    wd = torch.tensor([[1.0, 1.0, 1.0]], dtype=torch.float64)
    g = [1.0, -2.0, -1.0]
    u = [2.0, -6.0, 3.0]
    want = sum(gi / (1 + math.exp(-gi)) * ui for gi, ui in zip(g, u))
    assert math.isclose(float(pl.gated_mlp(x, wg, wu, wd)), want)


def test_model_is_causal_and_tied(model_dirs):
    m = pl.read_model_dir(model_dirs["A"])
    assert "lm_head.weight" not in m.t and m.head_weight() is m.t["model.embed_tokens.weight"]
    toks = [5, 9, 200, 31, 77, 8]
    full = m.logits(toks)
    assert torch.allclose(m.logits(toks[:4]), full[:4], atol=1e-12)
    other = m.logits(toks[:4] + [1, 2])
    assert torch.allclose(other[:4], full[:4], atol=1e-12) and not torch.allclose(other[5], full[5])
    assert m.greedy(toks, 3) == m.greedy(toks, 5)[:3]


def test_philox_known_answers():
    # Random123's published known-answer tests for philox4x32-10
    assert pl.philox4x32_10([0, 0, 0, 0], [0, 0]) == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    assert pl.philox4x32_10([0xFFFFFFFF] * 4, [0xFFFFFFFF] * 2) == [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]
    assert pl.philox4x32_10([0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344], [0xA4093822, 0x299F31D0]) == \
        [0xD16CFE09, 0x94FDCCEB, 0x5001E420, 0x24126EA1]
    us = [pl.uniform_for(3, i) for i in range(2000)]
    assert all(0.0 <= u < 1.0 for u in us) and 0.45 < sum(us) / len(us) < 0.55


def test_logits_processors():
    x = np.array([1.0, 3.0, -2.0, 0.5, 2.0], dtype=np.float32)
    got = pl.process_logits(x, context=[1, 1, 2], repetition_penalty=2.0, frequency_penalty=0.5,
                            presence_penalty=0.25, logit_bias={3: 1.0}, temperature=1.0)
    assert np.allclose(got, [1.0, 3.0 / 4 - 1.0 - 0.25, -4.0 - 0.5 - 0.25, 1.5, 2.0])
    got = pl.process_logits(x, temperature=0.5, top_k=2)
    assert np.isneginf(got[[0, 2, 3]]).all() and np.allclose(got[[1, 4]], [6.0, 4.0])
    probs = np.exp(x) / np.exp(x).sum()                     # sorted: 3.0, 2.0, 1.0, 0.5, -2.0
    p_two = float(np.sort(probs)[::-1][:2].sum())
    got = pl.process_logits(x, top_p=p_two - 1e-3)
    assert np.isfinite(got).sum() == 2
    got = pl.process_logits(x, top_p=p_two + 1e-3)
    assert np.isfinite(got).sum() == 3
    got = pl.process_logits(x, min_p=0.2)                   # keep p >= 0.2 * p_max: x >= 3 + ln 0.2 = 1.39
    assert np.isfinite(got).tolist() == [False, True, False, False, True]
    got = pl.process_logits(x, allowed_token_ids=[0, 2], suppress=[2])
    assert np.isfinite(got).tolist() == [True, False, False, False, False]
    assert pl.sample_row(pl.process_logits(x, temperature=0.0), 0.0, -1, 0.3) == 1
    assert pl.sample_row(np.array([1.0, 5.0, 5.0], dtype=np.float32), 0.0, -1, 0.0) == 1   # lowest index wins


def test_draws_follow_the_distribution():
    x = np.log(np.array([0.5, 0.25, 0.125, 0.125], dtype=np.float64)).astype(np.float32)
    counts = np.zeros(4)
    for i in range(4000):
        counts[pl.sample_row(x, 1.0, -1, pl.uniform_for(11, i))] += 1
    assert np.allclose(counts / 4000, [0.5, 0.25, 0.125, 0.125], atol=0.03)
    masked = np.array([-np.inf, 0.0, 0.0], dtype=np.float32)
    assert pl.sample_row(masked, 1.0, -1, 0.0) == 1         # a masked token is never drawn


def test_logprobs_by_hand():
    """log softmax of [0, ln 2, ln 5] is [-ln 8, ln 2 - ln 8, ln 5 - ln 8]; the largest first, equal logits
    lower index first, -inf left out (crates/rllm-sampling/src/logprobs.rs:5-28, 34-70)."""
    import math
    import numpy as np
    import plain_llama as pl
    x = np.array([0.0, math.log(2.0), math.log(5.0)], dtype=np.float32)
    assert abs(pl.logprob_of(x, 0) + math.log(8.0)) < 1e-6
    assert abs(pl.logprob_of(x, 2) - (math.log(5.0) - math.log(8.0))) < 1e-6
    assert pl.logprob_of(x, 3) == -math.inf
    top = pl.top_logprobs(x, 2)
    assert [i for i, _ in top] == [2, 1] and abs(top[1][1] - (math.log(2.0) - math.log(8.0))) < 1e-6
    y = np.array([1.0, -np.inf, 1.0, 0.0], dtype=np.float32)
    assert [i for i, _ in pl.top_logprobs(y, 5)] == [0, 2, 3]
    assert pl.top_logprobs(np.array([-np.inf, -np.inf]), 1) == [] and pl.top_logprobs(x, 0) == []
