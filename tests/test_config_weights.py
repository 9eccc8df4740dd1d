"""Configuration, registry, safetensors and weight-loading errors (no GPU)."""
import json

import pytest
import torch

import locus_b200.models  # noqa: F401
from locus_b200.config import ConfigError, Qwen2MoeConfig, archs, find_arch, load_config
from locus_b200.models.model import Model
from locus_b200.weights.loader import RandomSource, WeightError, load_weights, random_tensor
from locus_b200.weights.safetensors_io import ModelFiles, SafetensorsError, write_safetensors
from tiny_configs import config, make_model_dir


def test_config_reads_every_size_from_the_keys():
    for name in "ABC":
        raw = config(name)
        cfg = Qwen2MoeConfig.from_dict(raw)
        for key in ("vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
                    "head_dim", "rope_theta", "rms_norm_eps", "num_experts", "num_experts_per_tok", "norm_topk_prob",
                    "moe_intermediate_size", "shared_expert_intermediate_size", "tie_word_embeddings", "qkv_bias"):
            assert getattr(cfg, key) == raw[key], key
        assert Qwen2MoeConfig.from_dict(cfg.to_dict()) == cfg


def test_layer_kinds_and_windows():
    b = Qwen2MoeConfig.from_dict(config("B"))
    assert [b.is_moe_layer(l) for l in range(3)] == [False, True, False]  # decoder_sparse_step 2
    c = Qwen2MoeConfig.from_dict(config("C"))
    assert [c.is_moe_layer(l) for l in range(4)] == [True, False, True, True]  # mlp_only_layers [1]
    assert [c.layer_window(l) for l in range(4)] == [0, 0, 24, 24]
    a = Qwen2MoeConfig.from_dict(config("A"))
    assert all(a.layer_window(l) == 0 for l in range(2))


def test_head_dim_defaults_to_hidden_over_heads():
    raw = config("A")
    del raw["head_dim"]
    assert Qwen2MoeConfig.from_dict(raw).head_dim == 16


@pytest.mark.parametrize("change,fragment", [
    ({"num_attention_heads": 5, "head_dim": None}, "invalid head configuration"),
    ({"num_key_value_heads": 3}, "invalid kv head configuration"),
    ({"num_experts_per_tok": 9}, "invalid num_experts_per_tok"),
    ({"num_experts_per_tok": 0}, "invalid num_experts_per_tok"),
    ({"hidden_size": None}, "missing key: hidden_size"),
    ({"vocab_size": None}, "missing key: vocab_size"),
    ({"moe_intermediate_size": 0}, "moe_intermediate_size"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_scaling": {"type": "yarn", "factor": 4}}, "rope_scaling"),
    ({"use_sliding_window": True, "sliding_window": 0}, "sliding_window"),
    ({"num_hidden_layers": "two"}, "must be an integer"),
    ({"decoder_sparse_step": 0}, "decoder_sparse_step"),
])
def test_config_errors(change, fragment):
    raw = config("A")
    raw.update(change)
    with pytest.raises(ConfigError, match=fragment):
        Qwen2MoeConfig.from_dict(raw)


def test_registry(tmp_path):
    assert [a.name for a in archs()] == ["Qwen2MoeForCausalLM"] or "Qwen2MoeForCausalLM" in [a.name for a in archs()]
    assert find_arch("Qwen2MoeForCausalLM").description
    with pytest.raises(ConfigError, match=r"unsupported architecture: 'LlamaForCausalLM' \(supported: .*Qwen2MoeForCausalLM"):
        find_arch("LlamaForCausalLM")
    with pytest.raises(ConfigError, match="no config.json"):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text(json.dumps({"hidden_size": 8}))
    with pytest.raises(ConfigError, match="missing key: architectures"):
        load_config(str(tmp_path))


def test_plan_is_data_layer_by_layer():
    entry = find_arch("Qwen2MoeForCausalLM")
    plan = entry.build_plan(entry.parse_config(config("C")))
    assert [l.feed_forward.kind for l in plan.layers] == ["sparse_moe", "dense_mlp", "sparse_moe", "sparse_moe"]
    assert [l.mixer.args["window"] for l in plan.layers] == [0, 0, 24, 24]
    assert [c.layer for c in plan.order] == [0, 1, 2, 3]
    model = Model(plan, torch.float32, "cpu")
    needs = model.cache_needs()
    assert needs[0][0].window == 0 and needs[3][0].window == 24 and needs[0][0].n_kv_heads == 1


def test_safetensors_round_trip_against_the_library(tmp_path):
    from safetensors import safe_open

    tensors = {"a.weight": torch.randn(3, 5).to(torch.bfloat16), "b": torch.arange(7, dtype=torch.int64),
               "c": torch.randn(4), "d.e": torch.randn(2, 3, 4).to(torch.float16)}
    path = str(tmp_path / "model.safetensors")
    write_safetensors(path, [(k, tuple(v.shape), v.dtype) for k, v in tensors.items()], lambda n: tensors[n])
    with safe_open(path, framework="pt") as f:  # the library reads what we wrote
        assert set(f.keys()) == set(tensors)
        for k in tensors:
            assert torch.equal(f.get_tensor(k), tensors[k])
    mf = ModelFiles(str(tmp_path))  # and we read it back
    for k, v in tensors.items():
        assert mf.info(k) == (v.dtype, tuple(v.shape))
        assert torch.equal(mf.tensor(k), v)
    mf.close()


def test_sharded_folder_and_bad_files(tmp_path):
    t1, t2 = {"x": torch.randn(2, 2)}, {"y": torch.randn(3)}
    write_safetensors(str(tmp_path / "s1.safetensors"), [("x", (2, 2), torch.float32)], lambda n: t1[n])
    write_safetensors(str(tmp_path / "s2.safetensors"), [("y", (3,), torch.float32)], lambda n: t2[n])
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"x": "s1.safetensors", "y": "s2.safetensors"}}))
    mf = ModelFiles(str(tmp_path))
    assert sorted(mf.names()) == ["x", "y"] and torch.equal(mf.tensor("y"), t2["y"])
    mf.close()
    bad = tmp_path / "bad"
    bad.mkdir()
    with pytest.raises(SafetensorsError, match="no model.safetensors"):
        ModelFiles(str(bad))
    (bad / "model.safetensors").write_bytes(b"\xff" * 7)
    with pytest.raises(SafetensorsError, match="too short"):
        ModelFiles(str(bad))
    (bad / "model.safetensors").write_bytes((10 ** 9).to_bytes(8, "little") + b"{}")
    with pytest.raises(SafetensorsError, match="exceeds the file"):
        ModelFiles(str(bad))


def _cpu_model(name):
    entry = find_arch("Qwen2MoeForCausalLM")
    return Model(entry.build_plan(entry.parse_config(config(name))), torch.bfloat16, "cpu")


def test_random_model_folder_loads_and_is_reproducible(tmp_path):
    d1 = make_model_dir(tmp_path / "1", "B", torch.bfloat16)
    d2 = make_model_dir(tmp_path / "2", "B", torch.bfloat16)
    m1, m2 = ModelFiles(d1), ModelFiles(d2)
    assert sorted(m1.names()) == sorted(m2.names())
    for n in m1.names():
        assert torch.equal(m1.tensor(n), m2.tensor(n))
    names = set(m1.names())
    assert "lm_head.weight" not in names  # tied head
    assert "model.layers.1.mlp.experts.11.down_proj.weight" in names and "model.layers.0.mlp.gate_proj.weight" in names
    assert "model.layers.1.mlp.shared_expert_gate.weight" in names and "model.layers.2.self_attn.k_proj.bias" in names
    w = m1.tensor("model.layers.1.mlp.experts.3.up_proj.weight").float()
    assert abs(float(w.std()) - 0.02) < 0.004 and abs(float(w.mean())) < 0.004
    nw = m1.tensor("model.norm.weight").float()
    assert abs(float(nw.mean()) - 1.0) < 0.01 and float(nw.std()) < 0.03
    # another seed gives other weights; the value of a tensor does not depend on the others
    assert not torch.equal(random_tensor(1, "x", (4, 4), "linear", torch.float32),
                           random_tensor(2, "x", (4, 4), "linear", torch.float32))
    model = _cpu_model("B")
    load_weights(model, m1)
    m1.close(), m2.close()
    att = model.blocks[0].mixer
    assert att.params["wqkv"].shape == (6 * 32 + 2 * 2 * 32, 192) and att.params["wqkv"].dtype == torch.bfloat16
    moe = model.blocks[1].ff
    assert moe.params["gate_exps"].shape == (12, 48, 192) and moe.params["down_exps"].shape == (12, 192, 48)


def test_element_types_follow_storage(tmp_path):
    d = make_model_dir(tmp_path, "A", torch.float32)
    files = ModelFiles(d)
    m16 = _cpu_model("A")  # a bfloat16 model keeps tensors stored in 32 bits as they are
    load_weights(m16, files)
    assert all(p.dtype == torch.float32 for part in m16.all_parts() for p in part.params.values())
    entry = find_arch("Qwen2MoeForCausalLM")
    m32 = Model(entry.build_plan(entry.parse_config(config("A"))), torch.float32, "cpu")
    d16 = make_model_dir(tmp_path, "A", torch.bfloat16)
    f16 = ModelFiles(d16)
    load_weights(m32, f16)  # a float32 model widens everything
    assert all(p.dtype == torch.float32 for part in m32.all_parts() for p in part.params.values())
    m = _cpu_model("A")
    load_weights(m, f16)
    assert all(p.dtype == torch.bfloat16 for part in m.all_parts() for p in part.params.values())
    files.close(), f16.close()


def test_one_error_lists_missing_unexpected_and_wrong(tmp_path):
    model = _cpu_model("A")
    src = RandomSource(model, 0, torch.bfloat16)

    class Broken:
        def names(self):
            n = [x for x in src.names() if x not in ("model.norm.weight", "model.layers.0.mlp.experts.2.up_proj.weight")]
            return n + ["model.layers.0.self_attn.rotary.extra", "lm_head.bias"]

        def info(self, name):
            dt, shape = src.info(name)
            if name == "model.layers.1.self_attn.q_proj.weight":
                return dt, (shape[0], shape[1] + 1)
            return dt, shape

        def tensor(self, name):
            return src.tensor(name)

    with pytest.raises(WeightError) as ei:
        load_weights(model, Broken())
    e = ei.value
    assert e.missing == ["model.layers.0.mlp.experts.2.up_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["lm_head.bias", "model.layers.0.self_attn.rotary.extra"]
    assert len(e.wrong_shape) == 1 and "q_proj.weight" in e.wrong_shape[0] and "(64, 65)" in e.wrong_shape[0]
    msg = str(e)
    assert "2 missing, 2 unexpected, 1 with a wrong shape" in msg and "model.norm.weight" in msg
    assert not model.loaded


def test_tied_head_tolerates_a_stored_head(tmp_path):
    model = _cpu_model("B")
    src = RandomSource(model, 1, torch.bfloat16)

    class WithHead:
        def names(self):
            return src.names() + ["lm_head.weight"]

        info, tensor = src.info, src.tensor

    load_weights(model, WithHead())
    assert model.loaded


def test_tied_head_and_embedding_are_one_tensor_and_the_plan_says_what_to_ignore(tmp_path):
    model = _cpu_model("B")
    src = RandomSource(model, 1, torch.bfloat16)
    assert src.names().count("model.embed_tokens.weight") == 1

    class WithLeftovers:
        def names(self):
            return src.names() + ["lm_head.weight", "model.layers.0.self_attn.rotary_emb.inv_freq"]

        info, tensor = src.info, src.tensor

    load_weights(model, WithLeftovers())
    assert model.head.params["weight"].data_ptr() == model.embedding.params["table"].data_ptr()
    assert model.param_bytes() == sum(t.numel() * 2 for _, s in {s.name: (0, s) for _, s in model.tensor_sources()}.items()
                                      for t in [torch.empty(s[1].shape, device="meta")])
    # an untied model has a head of its own, and a stored tensor that its plan does not name is an error
    a = _cpu_model("A")
    srca = RandomSource(a, 0, torch.bfloat16)

    class Extra:
        def names(self):
            return srca.names() + ["model.layers.0.self_attn.rotary_emb.inv_freq", "model.extra"]

        info, tensor = srca.info, srca.tensor

    with pytest.raises(WeightError) as ei:
        load_weights(a, Extra())
    assert ei.value.unexpected == ["model.extra"]
    load_weights(a, srca)
    assert a.head.params["weight"].data_ptr() != a.embedding.params["table"].data_ptr()


def test_random_draws_are_a_function_of_seed_name_and_index():
    from locus_b200.weights import random_init as R

    key = R.tensor_key(7, "some.tensor")
    whole = R.normal_slice(key, 0, 5000)
    parts = torch.cat([R.normal_slice(key, 0, 1), R.normal_slice(key, 1, 1233), R.normal_slice(key, 1234, 3766)])
    assert torch.equal(whole, parts)                      # any cut, any order
    assert not torch.equal(whole, R.normal_slice(R.tensor_key(7, "other.tensor"), 0, 5000))
    u = R.uniform_slice(key, 0, 200000)
    assert 0.0 < float(u.min()) and float(u.max()) < 1.0 and abs(float(u.mean()) - 0.5) < 0.005
    z = R.normal_slice(key, 0, 200000)
    assert abs(float(z.mean())) < 0.01 and abs(float(z.std()) - 1.0) < 0.01
    assert abs(float((z.abs() < 1.0).double().mean()) - 0.6827) < 0.01 and float(z.abs().max()) > 3.5
    # the logarithm made of exact operations agrees with the library's to the last bits
    x = torch.cat([u[:1000], torch.tensor([2.0 ** -53, 1e-300, 0.02425, 0.999999, 7.5], dtype=torch.float64)])
    assert float(((R._log(x) - torch.log(x)).abs() / torch.log(x).abs()).max()) < 1e-14
    assert float(R._log(torch.ones(1, dtype=torch.float64))) == 0.0
    # a tensor larger than one slice is the slices side by side
    old, R.SLICE = R.SLICE, 1000
    try:
        t = R.random_tensor(3, "w", (7, 500), "linear", torch.float32)
    finally:
        R.SLICE = old
    assert torch.equal(t, R.random_tensor(3, "w", (7, 500), "linear", torch.float32))
    assert torch.equal(R.random_tensor(3, "w", (7, 500), "linear", torch.bfloat16), t.to(torch.bfloat16))
    n = R.random_tensor(3, "n", (4000,), "norm", torch.float32)
    assert abs(float(n.mean()) - 1.0) < 0.002 and abs(float(n.std()) - 0.01) < 0.002
    with pytest.raises(ValueError, match="init kind"):
        R.random_tensor(3, "w", (2,), "uniform", torch.float32)
