"""A toy mixer with state of its own, a toy feed-forward and a toy architecture
are defined HERE, registered, written as a model folder, loaded, and stepped
through trace replay - without a change to the framework's files.  The toy
model mixes kinds layer by layer: its first layer keeps a running state per
request, its second is the framework's attention."""
import json
import math
import os

import numpy as np
import pytest
import torch

import plain_llama as pl
from conftest import ATT_NAMES, MLP_NAMES
import replay_util as ru

pytestmark = pytest.mark.gpu

H, V, STATE = 40, 131, 24
DECAY = 0.9


def register_toy():
    from rllm_b200.config import register_architecture
    from rllm_b200.parts import (FeedForward, LayerSpec, Mixer, ModelSpec, PartSpec, Run, StateNeed,
                                 TensorSpec, register_part)

    @register_part("mixer", "toy_decay_state")
    class DecayState(Mixer):
        """s_t = decay * s_{t-1} + W_in x_t ;  y_t = W_out s_t, state float32 [STATE] per request.
        A step in which every sequence brings one token is computed for all rows at once from the device's
        slot indices, without a look at the host's lists: such steps may be captured in a CUDA graph, so
        the class says ``graph_safe``."""
        graph_safe = True

        def __init__(self, spec, prefix=""):
            super().__init__(spec, prefix)
            self.hidden, self.size, self.decay = spec["hidden_size"], spec["state_size"], spec["decay"]

        def tensor_specs(self):
            return [TensorSpec(self.prefix + "in.weight", (self.size, self.hidden), init=("normal", 0.2)),
                    TensorSpec(self.prefix + "out.weight", (self.hidden, self.size), init=("normal", 0.2))]

        def load(self, tensors):
            self.w_in, self.w_out = tensors[self.prefix + "in.weight"], tensors[self.prefix + "out.weight"]

        def cache_need(self):
            return StateNeed((self.size,))

        def forward(self, x, ctx, cache):
            u = x.float() @ self.w_in.float().t()                      # [T, STATE]
            if ctx.num_decode == ctx.num_seqs:                         # one token a sequence: all rows at once
                slots = ctx.state_slots.long()
                state = cache.state.index_select(0, slots) * self.decay + u
                cache.state.index_copy_(0, slots, state)
                return (state @ self.w_out.float().t()).to(x.dtype)
            out = torch.empty_like(u)
            off = 0
            for s, n in enumerate(ctx.q_lens_host):                    # a sequence's tokens in order
                state = cache.state[ctx.state_slots_host[s]]
                for t in range(off, off + n):
                    state.mul_(self.decay).add_(u[t])
                    out[t] = state
                off += n
            return (out @ self.w_out.float().t()).to(x.dtype)

    @register_part("feed_forward", "toy_scale")
    class Scale(FeedForward):
        graph_safe = True

        def __init__(self, spec, prefix=""):
            super().__init__(spec, prefix)
            self.hidden = spec["hidden_size"]

        def tensor_specs(self):
            return [TensorSpec(self.prefix + "scale", (self.hidden,), role="vector", init=("one_plus_normal", 0.3))]

        def load(self, tensors):
            self.scale = tensors[self.prefix + "scale"]

        def forward(self, x):
            return (x.float() * self.scale.float()).to(x.dtype)

    def parse(raw):
        return dict(raw)

    def build(cfg):
        norms = lambda: (PartSpec.of("rmsnorm", size=H, eps=cfg["eps"], name="n0.weight"),
                         PartSpec.of("rmsnorm", size=H, eps=cfg["eps"], name="n1.weight"))
        pos = PartSpec.of("rotary", head_dim=16, rotary_dim=16, theta=100.0, scaling=None)
        layers = (
            LayerSpec("pre_norm", PartSpec.of("toy_decay_state", hidden_size=H, state_size=STATE, decay=DECAY,
                                              tensor_prefix="state."),
                      PartSpec.of("toy_scale", hidden_size=H, tensor_prefix="ff."), norms(), "toy.0."),
            LayerSpec("pre_norm", PartSpec.of("attention", **ATT_NAMES, hidden_size=H, num_heads=2, num_kv_heads=1, head_dim=16,
                                              window=None, scale=None, position=pos),
                      PartSpec.of("gated_mlp", **MLP_NAMES, hidden_size=H, intermediate_size=56), norms(), "toy.1."),
        )
        return ModelSpec(hidden_size=H, vocab_size=V,
                         embedding=PartSpec.of("token_embedding", vocab_size=V, hidden_size=H, name="toy.embed"),
                         layers=layers, order=(Run(0, 0), Run(1, 1)),
                         final_norm=PartSpec.of("rmsnorm", size=H, eps=cfg["eps"], name="toy.norm"),
                         head=PartSpec.of("lm_head", vocab_size=V, hidden_size=H, name="toy.head", tied_to="toy.embed"),
                         max_positions=512)

    register_architecture("ToyStateForCausalLM", parse, build)


def plain_toy(w, tokens, eps):
    x = pl.embedding(w["toy.embed"], tokens)
    t = len(tokens)
    # layer 0: decaying state, scale feed-forward
    xn = pl.rms_norm(x, w["toy.0.n0.weight"], eps)
    u = xn @ w["toy.0.state.in.weight"].t()
    s, outs = torch.zeros(STATE, dtype=torch.float64), []
    for i in range(t):
        s = DECAY * s + u[i]
        outs.append(s)
    x = x + torch.stack(outs) @ w["toy.0.state.out.weight"].t()
    x = x + pl.rms_norm(x, w["toy.0.n1.weight"], eps) * w["toy.0.ff.scale"]
    # layer 1: attention, gated mlp
    xn = pl.rms_norm(x, w["toy.1.n0.weight"], eps)
    inv = pl.rope_inv_freq(16, 100.0, None)
    pos = torch.arange(t)
    q = pl.apply_rope((xn @ w["toy.1.self_attn.q_proj.weight"].t()).reshape(t, 2, 16), pos, inv)
    k = pl.apply_rope((xn @ w["toy.1.self_attn.k_proj.weight"].t()).reshape(t, 1, 16), pos, inv)
    v = (xn @ w["toy.1.self_attn.v_proj.weight"].t()).reshape(t, 1, 16)
    x = x + pl.attention(q, k, v, pos) @ w["toy.1.self_attn.o_proj.weight"].t()
    xn = pl.rms_norm(x, w["toy.1.n1.weight"], eps)
    x = x + pl.gated_mlp(xn, w["toy.1.mlp.gate_proj.weight"], w["toy.1.mlp.up_proj.weight"], w["toy.1.mlp.down_proj.weight"])
    return pl.rms_norm(x, w["toy.norm"], eps) @ w["toy.embed"].t()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_is_registered_built_and_stepped(tmp_path, dtype):
    from safetensors import safe_open
    from rllm_b200.engine.loading import write_random_model
    register_toy()
    cfg = {"architectures": ["ToyStateForCausalLM"], "eps": 1e-4, "torch_dtype": "float32"}
    d = str(tmp_path / "toy")
    write_random_model(d, cfg, seed=3)
    w = {}
    with safe_open(os.path.join(d, "model.safetensors"), framework="pt") as f:
        for n in f.keys():
            t = f.get_tensor(n)
            w[n] = (t.to(torch.bfloat16) if dtype == "bfloat16" and t.dim() == 2 else t).double()
    assert "toy.0.state.in.weight" in w and "toy.head" not in w
    rng = np.random.default_rng(5)
    reqs = {f"r{i}": [int(t) for t in rng.integers(0, V, size=n)] for i, n in enumerate([40, 3, 77, 21, 64, 9])}
    want = {r: plain_toy(w, toks, 1e-4).numpy() for r, toks in reqs.items()}
    tol = 1e-4 if dtype == "float32" else 3e-2
    for tb in (ru.trace_whole(reqs), ru.trace_portions(reqs, seed=1), ru.trace_mixed(reqs, seed=2, live=3, tail=5)):
        got = ru.run_trace(d, dtype, tb, V, page_size=16)
        for r, toks in reqs.items():
            have = np.stack([got[(r, p)] for p in range(len(toks))])
            err = np.abs(have - want[r]).max(axis=1) / np.abs(want[r]).max()
            assert err.max() <= tol, (r, int(err.argmax()), float(err.max()))


def _toy_folder(tmp_path, name="toy"):
    from safetensors import safe_open
    from rllm_b200.engine.loading import write_random_model
    register_toy()
    cfg = {"architectures": ["ToyStateForCausalLM"], "eps": 1e-4, "torch_dtype": "float32"}
    d = str(tmp_path / name)
    write_random_model(d, cfg, seed=3)
    with safe_open(os.path.join(d, "model.safetensors"), framework="pt") as f:
        w = {n: f.get_tensor(n).double() for n in f.keys()}
    return d, w


def test_a_forked_request_takes_a_copy_of_the_state(tmp_path):
    """Fork with a mixer that keeps state of fixed size: the child's slot starts as a copy of the parent's
    (not zeroed, not shared), both go on with different tokens and match the plain formulas."""
    d, w = _toy_folder(tmp_path)
    rng = np.random.default_rng(8)
    common, tail_p, tail_c = ([int(t) for t in rng.integers(0, V, size=n)] for n in (21, 12, 12))
    tb = ru.TraceBuilder()
    tb.step([("p", common)])
    tb.step([("p", tail_p[:1]), ("c", tail_c[:5])], fork=[("p", "c")])
    for i in range(1, 8):
        tb.step([("p", tail_p[i:i + 1]), ("c", tail_c[4 + i:5 + i])])
    tb.step([("p", tail_p[8:])], end=["p", "c"])
    got = ru.run_trace(d, "float32", tb, V, page_size=16)
    want = {"p": plain_toy(w, common + tail_p, 1e-4).numpy(), "c": plain_toy(w, common + tail_c, 1e-4).numpy()}
    assert max(pos for r, pos in got if r == "c") == len(common) + len(tail_c) - 1
    for (r, pos), row in got.items():
        err = np.abs(row - want[r][pos]).max() / np.abs(want[r]).max()
        assert err <= 1e-4, (r, pos, float(err))


def test_a_stateful_mixer_decodes_in_captured_graphs_and_padded_batches(tmp_path):
    """Eleven requests generate through the entry point with the toy model: decode steps of 9 to 11 rows are
    padded to captured sizes (12), whose spare rows use the storage's spare state slot; the next step is
    prepared and launched ahead like the Llama's.  Tokens are those of the plain formulas, and a request's
    state is untouched by the padding rows beside it."""
    from rllm_b200 import LLM, SamplingParams
    d, w = _toy_folder(tmp_path, "toy_gen")
    rng = np.random.default_rng(4)
    prompts = [[int(t) for t in rng.integers(0, V, size=int(n))] for n in rng.integers(2, 30, size=11)]
    budgets = [8 + 2 * i for i in range(11)]
    params = [SamplingParams(temperature=0.0, max_tokens=n, ignore_eos=True) for n in budgets]
    llm = LLM(d, dtype="fp32", num_gpu_blocks=64, max_num_seqs=12, enable_prefix_caching=False)
    assert llm.engine.runner.capture_graphs
    outs = llm.generate(prompts, params)
    captured = [k for k, g in llm.engine.runner.graphs.items() if g.graph is not None]
    assert any(k[0] == 12 for k in captured), captured
    assert llm.engine.stats()["num_steps_ahead"] > 5
    for p, n, o in zip(prompts, budgets, outs):
        toks = list(p)
        for _ in range(n):
            toks.append(int(torch.argmax(plain_toy(w, toks, 1e-4)[-1])))
        assert o.outputs[0].token_ids == toks[len(p):]
    llm.engine.cache.check()
    assert llm.engine.cache.usage()["num_requests"] == 0


def test_several_samples_of_one_prompt_branch_with_the_state(tmp_path):
    """n = 3 samples with the toy model: the samples branch off before the prompt's last token, each with a
    copy of the first sample's state slot as it was there, so every sample's tokens are those that the plain
    formulas draw with the sample's random stream."""
    from rllm_b200 import LLM, SamplingParams
    d, w = _toy_folder(tmp_path, "toy_samples")
    rng = np.random.default_rng(6)
    prompts = [[int(t) for t in rng.integers(0, V, size=n)] for n in (19, 2, 33)]
    llm = LLM(d, dtype="fp32", num_gpu_blocks=64, max_num_seqs=12, max_num_batched_tokens=24,
              long_prefill_token_threshold=8, enable_prefix_caching=False)
    outs = llm.generate(prompts, [SamplingParams(temperature=0.8, max_tokens=7, seed=50 + i, ignore_eos=True, n=3)
                                  for i in range(3)])
    assert llm.engine.stats()["num_copied_tokens"] == 2 * (18 + 1 + 32)
    for i, (p, o) in enumerate(zip(prompts, outs)):
        assert len(o.outputs) == 3
        for c in o.outputs:
            seed = (50 + i + c.index * 0x9E3779B97F4A7C15) & 0x7FFFFFFFFFFFFFFF
            toks = list(p)
            for j, t in enumerate(c.token_ids):
                x = pl.process_logits(plain_toy(w, toks, 1e-4)[-1].numpy(), temperature=0.8)
                assert t == pl.sample_row(x, 0.8, -1, pl.uniform_for(seed, j)), (i, c.index, j)
                toks.append(t)
    llm.engine.cache.check()
    assert llm.engine.cache.usage()["num_requests"] == 0


# ---------------------------------------------------------------------------
# A feed-forward with routing and another position encoding, defined here too
# ---------------------------------------------------------------------------
E, FF = 3, 48
AMP = 0.5


def register_routed():
    from rllm_b200.config import register_architecture
    from rllm_b200.parts import FeedForward, LayerSpec, ModelSpec, PartSpec, Run, TensorSpec, register_part
    from rllm_b200.parts.base import PositionEncoding

    @register_part("feed_forward", "toy_top1_experts")
    class Top1Experts(FeedForward):
        """Router logits in float32, the expert with the largest logit (lowest index on ties) alone computes
        the token: y = softmax(logits)[e] * W2[e] relu(W1[e] x).  A row depends on nothing but itself."""

        def __init__(self, spec, prefix=""):
            super().__init__(spec, prefix)
            self.hidden, self.inner, self.experts = spec["hidden_size"], spec["inner_size"], spec["num_experts"]

        def tensor_specs(self):
            specs = [TensorSpec(self.prefix + "router.weight", (self.experts, self.hidden), init=("normal", 0.5))]
            for e in range(self.experts):
                specs += [TensorSpec(self.prefix + f"experts.{e}.w1", (self.inner, self.hidden), init=("normal", 0.2)),
                          TensorSpec(self.prefix + f"experts.{e}.w2", (self.hidden, self.inner), init=("normal", 0.2))]
            return specs

        def load(self, tensors):
            self.router = tensors[self.prefix + "router.weight"]
            self.w1 = [tensors[self.prefix + f"experts.{e}.w1"] for e in range(self.experts)]
            self.w2 = [tensors[self.prefix + f"experts.{e}.w2"] for e in range(self.experts)]

        def forward(self, x):
            xf = x.float()
            logits = xf @ self.router.float().t()
            choice = logits.argmax(dim=1)
            gate = torch.softmax(logits, dim=1).gather(1, choice[:, None])
            out = torch.zeros_like(xf)
            for e in range(self.experts):                       # tokens sorted by expert, one product per expert
                rows = (choice == e).nonzero().flatten()
                if rows.numel():
                    hid = torch.relu(xf[rows] @ self.w1[e].float().t())
                    out[rows] = hid @ self.w2[e].float().t()
            return (out * gate).to(x.dtype)

    @register_part("position_encoding", "toy_additive_waves")
    class AdditiveWaves(PositionEncoding):
        """q += amp * sin(p f_i), k += amp * cos(p f_i) on every head dim i: not a rotation, so the mixer
        calls ``apply`` and fuses nothing."""

        def __init__(self, spec, prefix=""):
            super().__init__(spec, prefix)
            self.dim, self.amp = spec["head_dim"], spec["amp"]
            self.freq = torch.tensor([1.0 / (3.0 + i) for i in range(self.dim)], dtype=torch.float64)

        def tensor_specs(self):
            return []

        def load(self, tensors):
            pass

        def apply(self, q, k, positions):
            ang = positions.double()[:, None, None] * self.freq.to(q.device)[None, None, :]
            q.add_((self.amp * torch.sin(ang)).to(q.dtype))
            if k is not None:
                k.add_((self.amp * torch.cos(ang)).to(k.dtype))

    def build(cfg):
        norms = lambda: (PartSpec.of("rmsnorm", size=H, eps=cfg["eps"], name="n0.weight"),
                         PartSpec.of("rmsnorm", size=H, eps=cfg["eps"], name="n1.weight"))
        waves = PartSpec.of("toy_additive_waves", head_dim=16, amp=AMP)
        rot = PartSpec.of("rotary", head_dim=16, rotary_dim=16, theta=100.0, scaling=None)
        layers = (
            LayerSpec("pre_norm", PartSpec.of("attention", **ATT_NAMES, hidden_size=H, num_heads=2, num_kv_heads=2, head_dim=16,
                                              window=24, scale=None, position=waves),
                      PartSpec.of("gated_mlp", **MLP_NAMES, hidden_size=H, intermediate_size=56), norms(), "toy.0."),
            LayerSpec("pre_norm", PartSpec.of("attention", **ATT_NAMES, hidden_size=H, num_heads=2, num_kv_heads=1, head_dim=16,
                                              window=None, scale=None, position=rot),
                      PartSpec.of("toy_top1_experts", hidden_size=H, inner_size=FF, num_experts=E, tensor_prefix="moe."),
                      norms(), "toy.1."),
        )
        return ModelSpec(hidden_size=H, vocab_size=V,
                         embedding=PartSpec.of("token_embedding", vocab_size=V, hidden_size=H, name="toy.embed"),
                         layers=layers, order=(Run(0, 0), Run(1, 1)),
                         final_norm=PartSpec.of("rmsnorm", size=H, eps=cfg["eps"], name="toy.norm"),
                         head=PartSpec.of("lm_head", vocab_size=V, hidden_size=H, name="toy.head", tied_to=None),
                         max_positions=512)

    register_architecture("ToyRoutedForCausalLM", lambda raw: dict(raw), build)


def plain_routed(w, tokens, eps):
    """Logits and, per token, the margin between the router's two largest logits."""
    x = pl.embedding(w["toy.embed"], tokens)
    t = len(tokens)
    pos = torch.arange(t)
    # layer 0: attention over a window of 24 keys with the additive waves, gated mlp
    xn = pl.rms_norm(x, w["toy.0.n0.weight"], eps)
    ang = pos.double()[:, None, None] * torch.tensor([1.0 / (3.0 + i) for i in range(16)], dtype=torch.float64)
    q = (xn @ w["toy.0.self_attn.q_proj.weight"].t()).reshape(t, 2, 16) + AMP * torch.sin(ang)
    k = (xn @ w["toy.0.self_attn.k_proj.weight"].t()).reshape(t, 2, 16) + AMP * torch.cos(ang)
    v = (xn @ w["toy.0.self_attn.v_proj.weight"].t()).reshape(t, 2, 16)
    x = x + pl.attention(q, k, v, pos, window=24) @ w["toy.0.self_attn.o_proj.weight"].t()
    xn = pl.rms_norm(x, w["toy.0.n1.weight"], eps)
    x = x + pl.gated_mlp(xn, w["toy.0.mlp.gate_proj.weight"], w["toy.0.mlp.up_proj.weight"], w["toy.0.mlp.down_proj.weight"])
    # layer 1: attention with rotation, routed experts
    xn = pl.rms_norm(x, w["toy.1.n0.weight"], eps)
    inv = pl.rope_inv_freq(16, 100.0, None)
    q = pl.apply_rope((xn @ w["toy.1.self_attn.q_proj.weight"].t()).reshape(t, 2, 16), pos, inv)
    k = pl.apply_rope((xn @ w["toy.1.self_attn.k_proj.weight"].t()).reshape(t, 1, 16), pos, inv)
    v = (xn @ w["toy.1.self_attn.v_proj.weight"].t()).reshape(t, 1, 16)
    x = x + pl.attention(q, k, v, pos) @ w["toy.1.self_attn.o_proj.weight"].t()
    xn = pl.rms_norm(x, w["toy.1.n1.weight"], eps)
    logits = xn @ w["toy.1.moe.router.weight"].t()
    top = torch.topk(logits, 2, dim=1).values
    choice = logits.argmax(dim=1)
    gate = torch.softmax(logits, dim=1).gather(1, choice[:, None])
    y = torch.zeros_like(xn)
    for i in range(t):
        e = int(choice[i])
        y[i] = torch.relu(xn[i] @ w[f"toy.1.moe.experts.{e}.w1"].t()) @ w[f"toy.1.moe.experts.{e}.w2"].t()
    x = x + y * gate
    return pl.rms_norm(x, w["toy.norm"], eps) @ w["toy.head"].t(), (top[:, 0] - top[:, 1])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_routed_feed_forward_and_another_position_encoding(tmp_path, dtype):
    """A feed-forward that routes every token to one of three experts and a position encoding that is no
    rotation, both defined in this file, in a model whose first layer keeps a window of 24 keys (its pages
    are given back as the window passes them): whole, in portions and mixed, against plain formulas.
    The routed layer is the last one, so a token whose two best router logits are too close to call in
    bfloat16 changes its own logits only; such tokens are left out of the comparison."""
    from safetensors import safe_open
    from rllm_b200.engine.loading import write_random_model
    register_routed()
    cfg = {"architectures": ["ToyRoutedForCausalLM"], "eps": 1e-5, "torch_dtype": "float32"}
    d = str(tmp_path / "routed")
    write_random_model(d, cfg, seed=11)
    w = {}
    with safe_open(os.path.join(d, "model.safetensors"), framework="pt") as f:
        for n in f.keys():
            t = f.get_tensor(n)
            w[n] = (t.to(torch.bfloat16) if dtype == "bfloat16" and t.dim() == 2 else t).double()
    assert "toy.1.moe.experts.2.w2" in w and "toy.head" in w
    rng = np.random.default_rng(9)
    reqs = {f"r{i}": [int(t) for t in rng.integers(0, V, size=n)] for i, n in enumerate([90, 5, 130, 33, 64, 17])}
    want, clear = {}, {}
    for r, toks in reqs.items():
        logits, margin = plain_routed(w, toks, 1e-5)
        want[r] = logits.numpy()
        clear[r] = (margin > (1e-6 if dtype == "float32" else 0.15)).numpy()
    assert sum(int(c.sum()) for c in clear.values()) > 0.7 * sum(len(t) for t in reqs.values())
    tol = 1e-4 if dtype == "float32" else 3e-2
    for tb in (ru.trace_whole(reqs), ru.trace_portions(reqs, seed=3), ru.trace_mixed(reqs, seed=4, live=3, tail=6)):
        got = ru.run_trace(d, dtype, tb, V, page_size=8)
        for r, toks in reqs.items():
            have = np.stack([got[(r, p)] for p in range(len(toks))])
            err = np.abs(have - want[r]).max(axis=1) / np.abs(want[r]).max()
            assert err[clear[r]].max() <= tol, (r, int(np.argmax(err * clear[r])), float(err[clear[r]].max()))


# ---------------------------------------------------------------------------
# The engine's own parts in another arrangement: a layer that sees a window of 20 keys, a layer that sees all
# ---------------------------------------------------------------------------
def register_windowed():
    from rllm_b200.config import register_architecture
    from rllm_b200.parts import LayerSpec, ModelSpec, PartSpec, Run

    def build(cfg):
        norms = lambda: (PartSpec.of("rmsnorm", size=H, eps=cfg["eps"], name="n0.weight"),
                         PartSpec.of("rmsnorm", size=H, eps=cfg["eps"], name="n1.weight"))
        rot = PartSpec.of("rotary", head_dim=16, rotary_dim=16, theta=1000.0, scaling=None)
        att = lambda window, nkv: PartSpec.of("attention", **ATT_NAMES, hidden_size=H, num_heads=2, num_kv_heads=nkv, head_dim=16,
                                              window=window, scale=None, position=rot)
        mlp = lambda: PartSpec.of("gated_mlp", **MLP_NAMES, hidden_size=H, intermediate_size=56)
        layers = (LayerSpec("pre_norm", att(20, 2), mlp(), norms(), "toy.0."),
                  LayerSpec("pre_norm", att(None, 1), mlp(), norms(), "toy.1."))
        return ModelSpec(hidden_size=H, vocab_size=V,
                         embedding=PartSpec.of("token_embedding", vocab_size=V, hidden_size=H, name="toy.embed"),
                         layers=layers, order=(Run(0, 0), Run(1, 1)),
                         final_norm=PartSpec.of("rmsnorm", size=H, eps=cfg["eps"], name="toy.norm"),
                         head=PartSpec.of("lm_head", vocab_size=V, hidden_size=H, name="toy.head", tied_to=None),
                         max_positions=512)

    register_architecture("ToyWindowedForCausalLM", lambda raw: dict(raw), build)


def plain_windowed(w, tokens, eps):
    x = pl.embedding(w["toy.embed"], tokens)
    t = len(tokens)
    pos = torch.arange(t)
    inv = pl.rope_inv_freq(16, 1000.0, None)
    for layer, (window, nkv) in enumerate([(20, 2), (None, 1)]):
        p = f"toy.{layer}."
        xn = pl.rms_norm(x, w[p + "n0.weight"], eps)
        q = pl.apply_rope((xn @ w[p + "self_attn.q_proj.weight"].t()).reshape(t, 2, 16), pos, inv)
        k = pl.apply_rope((xn @ w[p + "self_attn.k_proj.weight"].t()).reshape(t, nkv, 16), pos, inv)
        v = (xn @ w[p + "self_attn.v_proj.weight"].t()).reshape(t, nkv, 16)
        x = x + pl.attention(q, k, v, pos, window=window) @ w[p + "self_attn.o_proj.weight"].t()
        xn = pl.rms_norm(x, w[p + "n1.weight"], eps)
        x = x + pl.gated_mlp(xn, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    return pl.rms_norm(x, w["toy.norm"], eps) @ w["toy.head"].t()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_windowed_layer_beside_a_full_one(tmp_path, dtype):
    """Two groups of pages with different needs: the windowed layer's pages are given back as the window
    passes them and are used again, the other layer keeps all.  Every part is the engine's own, so decode
    steps run as CUDA graphs, over a long decode, in portions and mixed with other requests."""
    from safetensors import safe_open
    from rllm_b200.engine.loading import write_random_model
    register_windowed()
    cfg = {"architectures": ["ToyWindowedForCausalLM"], "eps": 1e-5, "torch_dtype": "float32"}
    d = str(tmp_path / "windowed")
    write_random_model(d, cfg, seed=5)
    w = {}
    with safe_open(os.path.join(d, "model.safetensors"), framework="pt") as f:
        for n in f.keys():
            t = f.get_tensor(n)
            w[n] = (t.to(torch.bfloat16) if dtype == "bfloat16" and t.dim() == 2 else t).double()
    rng = np.random.default_rng(13)
    reqs = {f"r{i}": [int(t) for t in rng.integers(0, V, size=n)] for i, n in enumerate([120, 7, 64, 33, 150, 21])}
    want = {r: plain_windowed(w, toks, 1e-5).numpy() for r, toks in reqs.items()}
    tol = 1e-4 if dtype == "float32" else 3e-2
    traces = (ru.trace_whole(reqs), ru.trace_tail_decode(reqs, 60), ru.trace_portions(reqs, seed=6),
              ru.trace_mixed(reqs, seed=8, live=3, tail=40))
    for tb in traces:
        got = ru.run_trace(d, dtype, tb, V, page_size=4)
        for r, toks in reqs.items():
            have = np.stack([got[(r, p)] for p in range(len(toks))])
            err = np.abs(have - want[r]).max(axis=1) / np.abs(want[r]).max()
            assert err.max() <= tol, (r, int(np.argmax(err)), float(err.max()))


def test_generation_with_a_windowed_layer(tmp_path):
    """The same arrangement through the scheduler and the entry point: pages of the windowed layer go back
    to the pool while requests decode, several requests at a time, and the tokens are the plain ones."""
    from safetensors import safe_open
    from rllm_b200 import LLM, SamplingParams
    from rllm_b200.engine.loading import write_random_model
    register_windowed()
    cfg = {"architectures": ["ToyWindowedForCausalLM"], "eps": 1e-5, "torch_dtype": "float32"}
    d = str(tmp_path / "windowed_gen")
    write_random_model(d, cfg, seed=6)
    with safe_open(os.path.join(d, "model.safetensors"), framework="pt") as f:
        w = {n: f.get_tensor(n).double() for n in f.keys()}
    rng = np.random.default_rng(2)
    prompts = [[int(t) for t in rng.integers(0, V, size=n)] for n in (30, 3, 45)]
    steps = 40
    llm = LLM(d, dtype="fp32", block_size=4, num_gpu_blocks=80, max_num_seqs=3, max_num_batched_tokens=32,
              long_prefill_token_threshold=16)
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=steps, ignore_eos=True))
    for p, o in zip(prompts, outs):
        toks = list(p)
        for _ in range(steps):
            toks.append(int(torch.argmax(plain_windowed(w, toks, 1e-5)[-1])))
        assert o.outputs[0].token_ids == toks[len(p):]
    llm.engine.cache.check()
    assert llm.engine.cache.usage()["num_requests"] == 0


def test_prefix_sharing_with_a_windowed_layer(tmp_path):
    """Requests with a common prefix of 50 tokens on a model whose first layer sees 20 keys: later requests take
    the prefix's pages over (all of the layer that sees every key; of the windowed layer those that reach into
    their first query's window, found again although the window gave them back long ago) and generate the
    plain tokens."""
    from safetensors import safe_open
    from rllm_b200 import LLM, SamplingParams
    from rllm_b200.engine.loading import write_random_model
    register_windowed()
    cfg = {"architectures": ["ToyWindowedForCausalLM"], "eps": 1e-5, "torch_dtype": "float32"}
    d = str(tmp_path / "windowed_prefix")
    write_random_model(d, cfg, seed=6)
    with safe_open(os.path.join(d, "model.safetensors"), framework="pt") as f:
        w = {n: f.get_tensor(n).double() for n in f.keys()}
    rng = np.random.default_rng(9)
    common = [int(t) for t in rng.integers(0, V, size=50)]
    prompts = [common + [int(t) for t in rng.integers(0, V, size=n)] for n in (3, 11, 1)] + [common[:48], common[:21]]
    steps = 12
    llm = LLM(d, dtype="fp32", block_size=4, num_gpu_blocks=80, max_num_seqs=2, max_num_batched_tokens=32,
              long_prefill_token_threshold=16, enable_prefix_caching=True)
    assert llm.engine.cache.prefix_caching
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=steps, ignore_eos=True))
    for p, o in zip(prompts, outs):
        toks = list(p)
        for _ in range(steps):
            toks.append(int(torch.argmax(plain_windowed(w, toks, 1e-5)[-1])))
        assert o.outputs[0].token_ids == toks[len(p):]
    # 48 tokens of the prefix lie in full pages: the second and third prompt take them, the fourth (48 tokens, cached
    # whole) computes its last page again; the fifth needs the windowed layer's first pages, which may have been
    # used again by then (that layer has 20 pages in all)
    hits = llm.engine.stats()["prefix_hit_tokens"]
    assert 48 + 48 + 44 <= hits <= 48 + 48 + 44 + 20, hits
    llm.engine.cache.check()
    assert llm.engine.cache.usage()["num_requests"] == 0
