"""Weights by name: the writer, the reader and the one error that lists what
does not fit (the reference's loader tests: crates/rllm-model/src/loader.rs:381-444)."""
import json
import os

import pytest
import torch

from conftest import TINY_A, TINY_B
from rllm_b200.config import load_model_description
from rllm_b200.engine.loading import write_random_model
from rllm_b200.models import DecoderModel
from rllm_b200.weights import (FolderSource, RandomSource, SafetensorsFile, WeightsError, WeightsMismatch,
                               check_tensors, draw_tensor, find_weight_files, load_tensors,
                               write_safetensors)


def specs_of(model_dir):
    _, spec = load_model_description(model_dir)
    return DecoderModel(spec).tensor_specs()


def test_written_folder_is_read_by_the_safetensors_library(model_dirs):
    from safetensors import safe_open
    src = FolderSource(model_dirs["B"])
    with safe_open(os.path.join(model_dirs["B"], "model.safetensors"), framework="pt") as f:
        assert sorted(f.keys()) == sorted(src.names())
        for name in f.keys():
            assert torch.equal(f.get_tensor(name), src.read(name))
    assert "lm_head.weight" in src.names()


def test_tied_model_has_no_head_tensor(model_dirs):
    assert "lm_head.weight" not in FolderSource(model_dirs["A"]).names()
    check_tensors(specs_of(model_dirs["A"]), FolderSource(model_dirs["A"]))


def test_same_seed_same_weights_and_names_are_independent(tmp_path):
    write_random_model(str(tmp_path / "a"), TINY_A, 5, "float32")
    write_random_model(str(tmp_path / "b"), TINY_A, 5, "float32")
    write_random_model(str(tmp_path / "c"), TINY_A, 6, "float32")
    a, b, c = (FolderSource(str(tmp_path / x)) for x in "abc")
    name = "model.layers.1.mlp.down_proj.weight"
    assert torch.equal(a.read(name), b.read(name)) and not torch.equal(a.read(name), c.read(name))
    assert abs(float(a.read(name).std()) - 0.02) < 2e-3
    norm = a.read("model.layers.0.input_layernorm.weight")
    assert abs(float(norm.mean()) - 1.0) < 0.1 and 0.03 < float(norm.std()) < 0.2
    # a tensor's values depend on seed and name only, not on the rest of the model
    cfg = dict(TINY_A, num_hidden_layers=1)
    write_random_model(str(tmp_path / "d"), cfg, 5, "float32")
    assert torch.equal(FolderSource(str(tmp_path / "d")).read("model.layers.0.mlp.up_proj.weight"),
                       a.read("model.layers.0.mlp.up_proj.weight"))


def test_bfloat16_storage_round_trip(tmp_path):
    write_random_model(str(tmp_path / "m"), dict(TINY_B, torch_dtype="bfloat16"), 1)
    src = FolderSource(str(tmp_path / "m"))
    dt, shape = src.info("model.embed_tokens.weight")
    assert dt is torch.bfloat16 and shape == (389, 96)
    t = src.read("model.embed_tokens.weight")
    spec = [s for s in specs_of(str(tmp_path / "m")) if s.name == "model.embed_tokens.weight"][0]
    assert torch.equal(t, draw_tensor(spec, 1).to(torch.bfloat16))


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path, model_dirs):
    src = FolderSource(model_dirs["B"])
    tensors = {n: src.read(n) for n in src.names()}
    del tensors["model.layers.1.self_attn.k_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.9.extra.weight"] = torch.zeros(3)
    tensors["model.layers.0.mlp.gate_proj.weight"] = torch.zeros(264, 95)
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(16)   # ignored, as in checkpoints
    d = tmp_path / "broken"
    d.mkdir()
    write_safetensors(str(d / "model.safetensors"), tensors)
    (d / "config.json").write_text(json.dumps(TINY_B))
    _, spec = load_model_description(str(d))
    model = DecoderModel(spec)
    ignored = [n for part in model.parts() for n in part.ignored_tensors()]
    assert "model.layers.0.self_attn.rotary_emb.inv_freq" in ignored      # declared by the rotary part's spec
    with pytest.raises(WeightsMismatch) as e:
        check_tensors(model.tensor_specs(), FolderSource(str(d)), ignored)
    err = e.value
    assert err.missing == ["model.layers.1.self_attn.k_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.9.extra.weight"]
    assert err.wrong_shape == [("model.layers.0.mlp.gate_proj.weight", (264, 95), (264, 96))]
    text = str(err)
    for word in ("missing (2)", "unexpected (1)", "wrong shape (1)", "k_proj", "extra", "[264, 95]"):
        assert word in text


def test_untied_model_needs_its_head(tmp_path, model_dirs):
    src = FolderSource(model_dirs["B"])
    tensors = {n: src.read(n) for n in src.names() if n != "lm_head.weight"}
    d = tmp_path / "nohead"
    d.mkdir()
    write_safetensors(str(d / "model.safetensors"), tensors)
    (d / "config.json").write_text(json.dumps(TINY_B))
    with pytest.raises(WeightsMismatch, match="lm_head.weight"):
        check_tensors(specs_of(str(d)), FolderSource(str(d)))


def test_held_dtypes(model_dirs):
    specs = specs_of(model_dirs["A"])
    got = load_tensors(specs, FolderSource(model_dirs["A"]), torch.bfloat16, torch.device("cpu"))
    assert got["model.embed_tokens.weight"].dtype is torch.bfloat16
    assert got["model.norm.weight"].dtype is torch.float32       # stored in 32-bit: stays so
    got = load_tensors(specs, FolderSource(model_dirs["A"]), torch.float32, torch.device("cpu"))
    assert all(t.dtype is torch.float32 for t in got.values())


def test_integer_tables_become_int32():
    from rllm_b200.parts.spec import TensorSpec
    specs = [TensorSpec("table", (7, 3), role="int", init=("randint", 100))]
    got = load_tensors(specs, RandomSource(specs, 0), torch.bfloat16, torch.device("cpu"))
    assert got["table"].dtype is torch.int32 and int(got["table"].max()) < 100


def test_shard_discovery(tmp_path):
    with pytest.raises(WeightsError, match="does not exist"):
        find_weight_files(str(tmp_path / "nope"))
    with pytest.raises(WeightsError, match="no safetensors"):
        find_weight_files(str(tmp_path))
    for n in ("model-00001-of-00002.safetensors", "model-00002-of-00002.safetensors"):
        write_safetensors(str(tmp_path / n), {n[:11]: torch.zeros(2)})
    assert [os.path.basename(p) for p in find_weight_files(str(tmp_path))] == [
        "model-00001-of-00002.safetensors", "model-00002-of-00002.safetensors"]
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"a": "model-00002-of-00002.safetensors", "b": "model-00002-of-00002.safetensors"}}))
    assert [os.path.basename(p) for p in find_weight_files(str(tmp_path))] == ["model-00002-of-00002.safetensors"]
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"a": "../evil.safetensors"}}))
    with pytest.raises(WeightsError, match="leaves the model folder"):
        find_weight_files(str(tmp_path))
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"a": "gone.safetensors"}}))
    with pytest.raises(WeightsError, match="does not exist"):
        find_weight_files(str(tmp_path))


def test_corrupt_file(tmp_path):
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"\xff" * 20)
    with pytest.raises(WeightsError, match="header"):
        SafetensorsFile(str(p))


def test_an_architecture_with_other_tensor_names_loads_without_a_change_to_the_framework(tmp_path):
    """Same parts, a checkpoint that calls its tensors otherwise: the names are the spec's, so a new
    architecture registered from here writes, checks and loads its folder."""
    from rllm_b200.config.registry import register_architecture
    from rllm_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, Run

    def parse(cfg):
        return dict(cfg)

    def build(cfg):
        H, V = cfg["width"], cfg["vocab"]
        pos = PartSpec.of("rotary", head_dim=16, rotary_dim=16, theta=100.0, scaling=None,
                          ignored_tensors=("freq_table",))
        layer = lambda i: LayerSpec(
            "pre_norm",
            PartSpec.of("attention", hidden_size=H, num_heads=2, num_kv_heads=1, head_dim=16, window=None,
                        scale=None, position=pos, tensor_prefix="att/",
                        tensor_names={"q": "wq", "k": "wk", "v": "wv", "o": "wo"}),
            PartSpec.of("gated_mlp", hidden_size=H, intermediate_size=40, tensor_prefix="ff/",
                        tensor_names={"gate": "w1", "up": "w3", "down": "w2"}),
            (PartSpec.of("rmsnorm", size=H, eps=1e-5, name="ln1"), PartSpec.of("rmsnorm", size=H, eps=1e-5, name="ln2")),
            f"blk{i}/")
        return ModelSpec(hidden_size=H, vocab_size=V,
                         embedding=PartSpec.of("token_embedding", vocab_size=V, hidden_size=H, name="tok"),
                         layers=(layer(0), layer(1)), order=(Run(0, 0), Run(1, 1)),
                         final_norm=PartSpec.of("rmsnorm", size=H, eps=1e-5, name="ln_f"),
                         head=PartSpec.of("lm_head", vocab_size=V, hidden_size=H, name="out", tied_to="tok"),
                         max_positions=64)

    register_architecture("ToyRenamedForTest", parse, build)
    cfg = {"architectures": ["ToyRenamedForTest"], "width": 32, "vocab": 50, "torch_dtype": "float32"}
    d = str(tmp_path / "renamed")
    write_random_model(d, cfg, 3, "float32")
    src = FolderSource(d)
    assert sorted(src.names()) == sorted(
        ["tok", "ln_f"] + [f"blk{i}/{n}" for i in (0, 1)
                           for n in ("att/wq", "att/wk", "att/wv", "att/wo", "ff/w1", "ff/w2", "ff/w3", "ln1", "ln2")])
    # a stored frequency table under the name the spec declared is passed over; any other extra is not
    tensors = {n: src.read(n) for n in src.names()}
    tensors["blk1/att/freq_table"] = torch.zeros(8)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    _, spec = load_model_description(d)
    model = DecoderModel(spec)
    model.load(FolderSource(d), torch.float32, torch.device("cpu"))
    assert model.blocks[1].mixer.w_qkv.shape == (64, 32) and model.blocks[0].ffn.w_gate_up.shape == (80, 32)
    tensors["blk1/att/other"] = torch.zeros(8)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    with pytest.raises(WeightsMismatch, match="blk1/att/other"):
        DecoderModel(spec).load(FolderSource(d), torch.float32, torch.device("cpu"))


def test_counter_generator_known_answers_and_shape_of_the_distribution():
    """Philox4x32-10: the published known-answer vector for an all-zero counter and key.  The normals: right
    moments, and element i is a function of (key, i) alone, whatever the tensor's length."""
    import numpy as np
    from rllm_b200.weights import counter_rng as cr
    w = cr.philox4x32_10(np.array([0], dtype=np.uint64), 0)
    assert [hex(int(x)) for x in w[0]] == ["0x6627e8d5", "0xe169c58d", "0xbc57ac4c", "0x9b00dbd8"]
    z = cr.standard_normal(400_003, 0x0123456789ABCDEF)
    assert abs(z.mean()) < 5e-3 and abs(z.std() - 1) < 5e-3 and abs((z ** 4).mean() - 3) < 0.05
    assert abs(np.corrcoef(z[:-1], z[1:])[0, 1]) < 5e-3
    assert np.array_equal(cr.standard_normal(1001, 7), cr.standard_normal(5000, 7)[:1001])
    assert not np.array_equal(cr.standard_normal(64, 7), cr.standard_normal(64, 8))
    # the pieces that replace the library's logarithm, cosine and sine are accurate to a few ulp
    words = np.random.default_rng(0).integers(0, 2 ** 32, size=20000, dtype=np.uint64).astype(np.uint32)
    c, s = cr._cos_sin(words)
    angle = 2 * np.pi * words.astype(np.float64) / 2 ** 32
    assert np.abs(c - np.cos(angle)).max() < 2e-15 and np.abs(s - np.sin(angle)).max() < 2e-15
    u = (words.astype(np.float64) + 0.5) / 2 ** 32
    assert np.abs(cr._ln(u) / np.log(u) - 1).max() < 2e-15
    r = cr.randint(1000, 3, 17)
    assert r.min() >= 0 and r.max() == 16 and r.dtype == np.int32


def test_draw_tensor_rules():
    from rllm_b200.parts.spec import TensorSpec
    a = draw_tensor(TensorSpec("x.weight", (33, 7), init=("normal", 0.02)), 4)
    b = draw_tensor(TensorSpec("x.weight", (33, 7), role="vector", init=("one_plus_normal", 0.1)), 4)
    assert a.dtype is torch.float32 and a.shape == (33, 7) and abs(float(a.std()) - 0.02) < 4e-3
    # the same stream under both rules: 1 + 0.1 z against 0.02 z
    assert torch.allclose((b - 1.0) / 0.1, a / 0.02, atol=1e-5)
    other = draw_tensor(TensorSpec("y.weight", (33, 7), init=("normal", 0.02)), 4)
    assert not torch.equal(a, other) and not torch.equal(a, draw_tensor(TensorSpec("x.weight", (33, 7)), 5))
