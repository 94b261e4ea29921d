"""Each part a layer is put together from, alone, against the plain functions,
at sizes that differ from the tiny models'; and the generality of the layer
list: a layer that runs twice, a layer that reads another layer's cache, and
mixers of different kinds (with and without a window) in one model."""
import math

import numpy as np
import pytest
import torch

import plain_llama as pl
from conftest import ATT_NAMES, MLP_NAMES

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
DTYPES = [torch.float32, torch.bfloat16]


def tol(dt):
    return 1e-5 if dt is torch.float32 else 2e-2


def rel_err(got, want):
    want = want.double().cpu()
    return float((got.double().cpu() - want).abs().max() / want.abs().max().clamp_min(1e-30))


def load_part(part, dt, seed=0):
    """Random weights for a part through the framework's own loader."""
    from rllm_b200.weights import RandomSource, load_tensors
    specs = part.tensor_specs()
    tensors = load_tensors(specs, RandomSource(specs, seed), dt, DEV)
    part.load(tensors)
    return {k: v.double().cpu() for k, v in tensors.items()}


def context_for(needs, page, pages, entries, dt, cache=None):
    from rllm_b200.cache import CacheManager
    from rllm_b200.engine.runner import BatchBuilder, StepEntry
    cache = cache or CacheManager(needs, page, pages, 8)
    es = []
    for rid, toks, start in entries:
        if rid not in cache.requests:
            cache.admit(rid)
        assert cache.ensure(rid, start, start + len(toks))
        es.append(StepEntry(rid, toks, start, []))
    ctx, _, _ = BatchBuilder(cache, DEV, dt).build_context(es)
    return ctx, cache


@pytest.mark.parametrize("dt", DTYPES)
def test_norm_part(dt):
    from rllm_b200.parts import PartSpec, build_part
    norm = build_part("norm", PartSpec.of("rmsnorm", size=200, eps=3e-4, name="n.weight"), prefix="x.")
    w = load_part(norm, dt)["x.n.weight"]
    assert norm.weight.dtype is torch.float32            # stored in 32-bit by the random source: stays so
    x = torch.randn(6, 200, device=DEV)
    delta = torch.randn(6, 200, device=DEV).to(dt)
    assert rel_err(norm.forward(x.clone(), dt), pl.rms_norm(x.double().cpu(), w, 3e-4)) <= tol(dt)
    h = x.clone()
    got = norm.add_forward(h, delta)
    assert torch.equal(h, x + delta.float())
    assert rel_err(got, pl.rms_norm(h.double().cpu(), w, 3e-4)) <= tol(dt)
    rows = torch.tensor([4, 1], dtype=torch.int32, device=DEV)
    assert torch.equal(norm.gather_forward(x.clone(), delta, rows, dt), got[rows.long()])


def test_rotary_part_builds_the_scaled_table():
    from rllm_b200.parts import PartSpec, build_part
    sc = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
          "original_max_position_embeddings": 64}
    rot = build_part("position_encoding", PartSpec.of("rotary", head_dim=48, rotary_dim=32, theta=77777.0, scaling=sc))
    table, rd = rot.fused_rotary(DEV)
    assert rd == 32 and table.dtype is torch.float64
    assert torch.allclose(table.cpu(), pl.rope_inv_freq(32, 77777.0, sc), rtol=1e-15)
    with pytest.raises(ValueError):
        build_part("position_encoding", PartSpec.of("rotary", head_dim=48, rotary_dim=50, theta=1e4, scaling=None))


@pytest.mark.parametrize("dt", DTYPES)
def test_feed_forward_part(dt):
    from rllm_b200.parts import PartSpec, build_part
    mlp = build_part("feed_forward", PartSpec.of("gated_mlp", **MLP_NAMES, hidden_size=72, intermediate_size=200), prefix="m.")
    w = load_part(mlp, dt)
    x = (torch.randn(9, 72, device=DEV) * 2).to(dt)
    want = pl.gated_mlp(x.double().cpu(), w["m.gate_proj.weight"], w["m.up_proj.weight"], w["m.down_proj.weight"])
    assert rel_err(mlp.forward(x), want) <= tol(dt)


@pytest.mark.parametrize("dt", DTYPES)
def test_embedding_and_head_parts(dt):
    from rllm_b200.parts import PartSpec
    from rllm_b200.parts.embedding import OutputHead, TokenEmbedding
    emb = TokenEmbedding(PartSpec.of("token_embedding", vocab_size=301, hidden_size=40, name="e.weight"))
    table = load_part(emb, dt)["e.weight"]
    ids = torch.tensor([0, 300, 17], dtype=torch.int32, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    assert torch.equal(emb.forward(ids, err).double().cpu(), table[[0, 300, 17]])
    tied = OutputHead(PartSpec.of("lm_head", vocab_size=301, hidden_size=40, name="h.weight", tied_to="e.weight"))
    assert tied.tensor_specs()[0].optional
    tied.load({"e.weight": emb.weight})
    x = torch.randn(5, 40, device=DEV).to(dt)
    logits = tied.forward(x)
    assert logits.dtype is torch.float32 and rel_err(logits, x.double().cpu() @ table.t()) <= tol(dt)
    own = OutputHead(PartSpec.of("lm_head", vocab_size=301, hidden_size=40, name="h.weight", tied_to=None))
    assert not own.tensor_specs()[0].optional


def plain_attention_part(w, prefix, x, positions, nq, nkv, d, inv, window, rd=None):
    t = x.shape[0]
    q = pl.linear(x, w[prefix + "q_proj.weight"]).reshape(t, nq, d)
    k = pl.linear(x, w[prefix + "k_proj.weight"]).reshape(t, nkv, d)
    v = pl.linear(x, w[prefix + "v_proj.weight"]).reshape(t, nkv, d)
    rd = rd or d
    q = torch.cat([pl.apply_rope(q[..., :rd], positions, inv), q[..., rd:]], -1)
    k = torch.cat([pl.apply_rope(k[..., :rd], positions, inv), k[..., rd:]], -1)
    return pl.linear(pl.attention(q, k, v, positions, window=window), w[prefix + "o_proj.weight"])


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,rd,window,page", [(6, 3, 48, 48, None, 4), (4, 1, 64, 32, 9, 8), (5, 5, 16, 16, None, 16)])
def test_attention_part_in_portions(dt, nq, nkv, d, rd, window, page):
    """The mixer alone, fed a sequence in portions beside another sequence."""
    from rllm_b200.cache import CacheStorage
    from rllm_b200.models.decoder import CacheLayout
    from rllm_b200.parts import PartSpec, build_part
    hidden = 56
    pos = PartSpec.of("rotary", head_dim=d, rotary_dim=rd, theta=5000.0, scaling=None)
    att = build_part("mixer", PartSpec.of("attention", **ATT_NAMES, hidden_size=hidden, num_heads=nq, num_kv_heads=nkv,
                                          head_dim=d, window=window, scale=None, position=pos), prefix="a.")
    w = load_part(att, dt)
    need = att.cache_need()
    assert (need.num_kv_heads, need.head_dim, need.window) == (nkv, d, window)
    layout = CacheLayout([need], [[0]], [0], [0])
    storage = CacheStorage(layout, page, [32], 8, dt, DEV)
    torch.manual_seed(1)
    xs = {"a": torch.randn(41, hidden).to(dt), "b": torch.randn(13, hidden).to(dt)}
    inv = pl.rope_inv_freq(rd, 5000.0, None)
    want = {r: plain_attention_part(w, "a.", x.double(), torch.arange(len(x)), nq, nkv, d, inv, window, rd)
            for r, x in xs.items()}
    cuts = {"a": [17, 1, 2, 20, 1], "b": [1, 1, 11]}
    cache, fed, got = None, {"a": 0, "b": 0}, {"a": [], "b": []}
    for step in range(5):
        entries = []
        for r in ("a", "b"):
            if step < len(cuts[r]):
                n = cuts[r][step]
                entries.append((r, list(range(n)), fed[r]))
        ctx, cache = context_for([need], page, 32, entries, dt, cache)
        order = sorted(range(len(entries)), key=lambda i: (len(entries[i][1]) != 1, i))
        x = torch.cat([xs[entries[i][0]][entries[i][2]:entries[i][2] + len(entries[i][1])] for i in order]).to(DEV)
        y = att.forward(x, ctx, storage.view(0))
        off = 0
        for i in order:
            r, toks, _ = entries[i]
            got[r].append(y[off:off + len(toks)].cpu())
            off += len(toks)
            fed[r] += len(toks)
        assert int(ctx.err.item()) == 0
    for r in xs:
        assert rel_err(torch.cat(got[r]), want[r]) <= tol(dt), r


def toy_spec(kind):
    """Four-run models over two or three layers, built from registered parts only."""
    from rllm_b200.parts import LayerSpec, ModelSpec, PartSpec, Run
    H, V = 48, 97
    def layer(i, window=None, shares_kv=False, nkv=2):
        pos = PartSpec.of("rotary", head_dim=16, rotary_dim=16, theta=1000.0, scaling=None)
        return LayerSpec(
            block="pre_norm",
            mixer=PartSpec.of("attention", **ATT_NAMES, hidden_size=H, num_heads=4, num_kv_heads=nkv, head_dim=16,
                              window=window, scale=None, position=pos, shares_kv=shares_kv),
            ffn=PartSpec.of("gated_mlp", **MLP_NAMES, hidden_size=H, intermediate_size=80 + 8 * i),
            norms=(PartSpec.of("rmsnorm", size=H, eps=1e-5, name="input_layernorm.weight"),
                   PartSpec.of("rmsnorm", size=H, eps=1e-5, name="post_attention_layernorm.weight")),
            prefix=f"model.layers.{i}.")
    if kind == "twice":          # layer 1 runs twice, each run with a cache of its own
        layers, order = (layer(0), layer(1)), (Run(0, 0), Run(1, 1), Run(1, 2), Run(0, 3))
    elif kind == "shared":       # layer 2 has no k/v projections: it reads the cache that run 0 wrote
        layers, order = (layer(0), layer(1), layer(2, shares_kv=True)), (Run(0, 0), Run(1, 1), Run(2, 0))
    else:                        # a windowed layer between layers that keep all keys
        layers, order = (layer(0), layer(1, window=6, nkv=1), layer(2)), (Run(0, 0), Run(1, 1), Run(2, 2))
    return ModelSpec(hidden_size=H, vocab_size=V,
                     embedding=PartSpec.of("token_embedding", vocab_size=V, hidden_size=H, name="model.embed_tokens.weight"),
                     layers=layers, order=order,
                     final_norm=PartSpec.of("rmsnorm", size=H, eps=1e-5, name="model.norm.weight"),
                     head=PartSpec.of("lm_head", vocab_size=V, hidden_size=H, name="lm_head.weight", tied_to=None),
                     max_positions=256)


def plain_toy_logits(spec, w, tokens):
    """The toy models computed with the plain functions, following the order list."""
    x = pl.embedding(w["model.embed_tokens.weight"], tokens)
    positions = torch.arange(len(tokens))
    inv = pl.rope_inv_freq(16, 1000.0, None)
    kv_of_run = {}
    for i, run in enumerate(spec.order):
        ls = spec.layers[run.layer]
        p, m = ls.prefix, ls.mixer.get()
        nq, nkv, d = m["num_heads"], m["num_kv_heads"], m["head_dim"]
        xn = pl.rms_norm(x, w[p + "input_layernorm.weight"], 1e-5)
        t = len(tokens)
        q = pl.apply_rope(pl.linear(xn, w[p + "self_attn.q_proj.weight"]).reshape(t, nq, d), positions, inv)
        if run.cache == i:
            k = pl.apply_rope(pl.linear(xn, w[p + "self_attn.k_proj.weight"]).reshape(t, nkv, d), positions, inv)
            v = pl.linear(xn, w[p + "self_attn.v_proj.weight"]).reshape(t, nkv, d)
            kv_of_run[i] = (k, v)
        k, v = kv_of_run[run.cache]
        a = pl.linear(pl.attention(q, k, v, positions, window=m["window"]), w[p + "self_attn.o_proj.weight"])
        x = x + a
        xn = pl.rms_norm(x, w[p + "post_attention_layernorm.weight"], 1e-5)
        x = x + pl.gated_mlp(xn, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    return pl.linear(pl.rms_norm(x, w["model.norm.weight"], 1e-5), w["lm_head.weight"])


@pytest.mark.parametrize("kind", ["twice", "shared", "mixed_windows"])
def test_layer_list_is_data(kind):
    from rllm_b200.cache import CacheManager, CacheStorage
    from rllm_b200.engine.runner import ModelRunner, StepEntry
    from rllm_b200.models import DecoderModel
    from rllm_b200.weights import RandomSource
    spec = toy_spec(kind)
    model = DecoderModel(spec)
    specs = model.tensor_specs()
    names = {s.name for s in specs}
    if kind == "shared":
        assert "model.layers.2.self_attn.k_proj.weight" not in names
        assert model.layout.owners == [[0, 1]] and model.layout.run_owner == [0, 1, 0]
    if kind == "twice":
        assert len([n for n in names if n.startswith("model.layers.1.")]) == 9       # one set of weights
        assert model.layout.owners == [[0, 1, 2, 3]]                                   # four caches
    if kind == "mixed_windows":
        assert len(model.layout.groups) == 2 and model.layout.run_group == [0, 1, 0]
    src = RandomSource(specs, 4)
    model.load(src, torch.float32, DEV)
    w = {n: src.read(n).double() for n in src.names()}
    n_paged = len(model.layout.groups)
    cache = CacheManager(model.layout.groups, 4, [24] * n_paged, 4)
    storage = CacheStorage(model.layout, 4, [24] * n_paged, 4, torch.float32, DEV)
    runner = ModelRunner(model, cache, storage)
    rng = np.random.default_rng(0)
    seqs = {"a": [int(t) for t in rng.integers(0, 97, size=37)], "b": [int(t) for t in rng.integers(0, 97, size=21)]}
    want = {r: plain_toy_logits(spec, w, toks) for r, toks in seqs.items()}
    cuts = {"a": [5, 2, 9, 1, 1, 19], "b": [1, 17, 1, 1, 1]}
    fed = {"a": 0, "b": 0}
    for r in seqs:
        cache.admit(r)
    for step in range(6):
        entries = []
        for r in seqs:
            if step < len(cuts[r]):
                n = cuts[r][step]
                assert cache.ensure(r, fed[r], fed[r] + n)
                entries.append(StepEntry(r, seqs[r][fed[r]:fed[r] + n], fed[r], list(range(n))))
        logits = runner.step(entries)
        runner.check_errors()
        off = 0
        for e in entries:
            n = len(e.tokens)
            assert rel_err(logits[off:off + n], want[e.req][e.start:e.start + n]) <= 1e-4, (kind, step, e.req)
            off += n
            fed[e.req] += n
        cache.check()
    if kind == "mixed_windows":      # the windowed group has given back what its window passed
        # the last portion began at position 18: with a window of 6 it sees keys from 13 on (page 3)
        assert cache.table("a", 1)[:3] == [-1] * 3 and all(p >= 0 for p in cache.table("a", 1)[3:])
        assert all(p >= 0 for p in cache.table("a", 0))
