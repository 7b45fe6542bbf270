"""CPU tests: configuration, registry, safetensors container, weight errors, random weights."""
import json
import os
import struct

import pytest
import torch

from tiny import CONFIG_A, CONFIG_B, CONFIG_C


def test_config_reads_every_key():
    from llm_b200.config import parse_config
    arch, cfg = parse_config(CONFIG_B)
    assert arch.name == "LlamaForCausalLM"
    assert (cfg.hidden_size, cfg.intermediate_size, cfg.num_hidden_layers) == (96, 256, 3)
    assert (cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim) == (3, 1, 32)
    assert cfg.vocab_size == 384 and cfg.rms_norm_eps == 1e-6 and cfg.rope_theta == 500000.0
    assert cfg.max_position_embeddings == 256 and cfg.sliding_window is None
    _, c = parse_config(CONFIG_C)
    assert c.sliding_window == 37 and c.tie_word_embeddings and c.head_dim == 48


def test_config_defaults_and_errors():
    from llm_b200.config import ConfigError, parse_config
    d = dict(CONFIG_A)
    del d["num_key_value_heads"], d["head_dim"], d["rope_theta"]
    _, cfg = parse_config(d)
    assert cfg.num_key_value_heads == 4 and cfg.head_dim == 16 and cfg.rope_theta == 10000.0
    for key in ("hidden_size", "intermediate_size", "num_hidden_layers", "vocab_size", "rms_norm_eps",
                "max_position_embeddings"):
        bad = dict(CONFIG_A)
        del bad[key]
        with pytest.raises(ConfigError, match=key):
            parse_config(bad)
    with pytest.raises(ConfigError, match="multiple"):
        parse_config(dict(CONFIG_A, num_key_value_heads=3))
    with pytest.raises(ConfigError, match="unknown architecture"):
        parse_config(dict(CONFIG_A, architectures=["NoSuchModel"]))
    with pytest.raises(ConfigError, match="rope_scaling"):
        parse_config(dict(CONFIG_A, rope_scaling={"type": "linear", "factor": 2}))
    with pytest.raises(ConfigError, match="hidden_act"):
        parse_config(dict(CONFIG_A, hidden_act="gelu"))
    with pytest.raises(ConfigError, match="even"):
        parse_config(dict(CONFIG_A, head_dim=15))


def test_spec_is_data_with_sizes_from_config():
    from llm_b200.config import parse_config
    arch, cfg = parse_config(CONFIG_B)
    spec = arch.build_spec(cfg)
    assert spec.order == (0, 1, 2) and len(spec.layers) == 3
    mixer = spec.layers[1].parts["mixer"]
    assert mixer.kind == "attention" and mixer.params["num_kv_heads"] == 1 and mixer.params["head_dim"] == 32
    assert mixer.params["position"].params["theta"] == 500000.0
    assert spec.layers[2].parts["norm2"].params["eps"] == 1e-6
    assert spec.layers[0].parts["ffn"].params["intermediate_size"] == 256


def test_safetensors_round_trip_and_errors(tmp_path):
    from llm_b200.weights import SafetensorsError, SafetensorsFile, write_safetensors
    t = {"a": torch.arange(6, dtype=torch.float32).reshape(2, 3),
         "b": torch.randn(5, 7).to(torch.bfloat16), "c": torch.tensor([1, 2, 3], dtype=torch.int32)}
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, t, {"k": "v"})
    f = SafetensorsFile(p)
    assert set(f.names()) == set(t) and f.metadata == {"k": "v"}
    for k in t:
        assert f.tensor(k).dtype == t[k].dtype and torch.equal(f.tensor(k), t[k])

    def write_raw(header: bytes, data: bytes = b"", name="bad.safetensors"):
        q = str(tmp_path / name)
        with open(q, "wb") as fh:
            fh.write(struct.pack("<Q", len(header)) + header + data)
        return q

    with open(tmp_path / "short", "wb") as fh:
        fh.write(b"abc")
    with pytest.raises(SafetensorsError, match="shorter"):
        SafetensorsFile(str(tmp_path / "short"))
    with open(tmp_path / "big", "wb") as fh:
        fh.write(struct.pack("<Q", 1000) + b"{}")
    with pytest.raises(SafetensorsError, match="exceeds"):
        SafetensorsFile(str(tmp_path / "big"))
    with pytest.raises(SafetensorsError, match="JSON"):
        SafetensorsFile(write_raw(b"{not json"))
    with pytest.raises(SafetensorsError, match="data_offsets"):
        SafetensorsFile(write_raw(json.dumps({"t": {"dtype": "F32", "shape": [1]}}).encode()))
    with pytest.raises(SafetensorsError, match="reversed"):
        SafetensorsFile(write_raw(json.dumps({"t": {"dtype": "F32", "shape": [1], "data_offsets": [4, 0]}}).encode(), b"0000"))
    with pytest.raises(SafetensorsError, match="past the data"):
        SafetensorsFile(write_raw(json.dumps({"t": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}).encode(), b"0000"))
    with pytest.raises(SafetensorsError, match="unsupported dtype"):
        SafetensorsFile(write_raw(json.dumps({"t": {"dtype": "F8_E4M3", "shape": [4], "data_offsets": [0, 4]}}).encode(), b"0000"))
    with pytest.raises(SafetensorsError, match="needs 8"):
        SafetensorsFile(write_raw(json.dumps({"t": {"dtype": "F32", "shape": [2], "data_offsets": [0, 4]}}).encode(), b"0000"))


def test_random_model_is_seeded_and_complete(tmp_path):
    from llm_b200.weights import SafetensorsFile, write_random_model
    from llm_b200.weights.loader import expected_tensors
    a = write_random_model(str(tmp_path / "a"), CONFIG_A, 5, "bfloat16")
    b = write_random_model(str(tmp_path / "b"), CONFIG_A, 5, "bfloat16")
    c = write_random_model(str(tmp_path / "c"), CONFIG_A, 6, "float32")
    fa, fb, fc = (SafetensorsFile(os.path.join(d, "model.safetensors")) for d in (a, b, c))
    exp = expected_tensors(CONFIG_A)
    assert set(fa.names()) == set(exp) and len(exp) == 2 * 9 + 3
    for n in fa.names():
        assert torch.equal(fa.tensor(n), fb.tensor(n))
        assert tuple(fa.tensor(n).shape) == exp[n].shape
    assert fa.tensor("model.layers.0.mlp.down_proj.weight").dtype == torch.bfloat16
    assert fa.tensor("model.norm.weight").dtype == torch.float32
    assert fc.tensor("lm_head.weight").dtype == torch.float32
    assert not torch.equal(fa.tensor("lm_head.weight").float(), fc.tensor("lm_head.weight"))
    w = fc.tensor("model.layers.1.self_attn.q_proj.weight")
    assert abs(float(w.std()) - 0.02) < 0.002 and abs(float(w.mean())) < 0.002
    g = fc.tensor("model.layers.1.input_layernorm.weight")
    assert abs(float(g.mean()) - 1.0) < 0.01
    with open(os.path.join(a, "config.json")) as fh:
        assert json.load(fh)["hidden_size"] == 64
    # tied head: no lm_head tensor is expected
    assert "lm_head.weight" not in expected_tensors(CONFIG_C)


def test_weight_errors_are_listed_together(tmp_path):
    from llm_b200.weights import SafetensorsFile, WeightError, load_tensors, write_random_model, write_safetensors
    from llm_b200.weights.loader import expected_tensors
    d = write_random_model(str(tmp_path / "m"), CONFIG_A, 1, "float32")
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    t = {n: f.tensor(n).clone() for n in f.names()}
    del t["model.layers.1.mlp.up_proj.weight"], t["model.norm.weight"]
    t["model.layers.0.extra.weight"] = torch.zeros(3)
    t["lm_head.weight"] = torch.zeros(255, 64)
    write_safetensors(os.path.join(d, "model.safetensors"), t)
    with pytest.raises(WeightError) as ei:
        load_tensors(d, expected_tensors(CONFIG_A), torch.float32, torch.device("cpu"))
    e = ei.value
    assert e.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["model.layers.0.extra.weight"]
    assert len(e.wrong) == 1 and "lm_head.weight" in e.wrong[0] and "[255, 64]" in e.wrong[0]
    msg = str(e)
    assert "missing" in msg and "unexpected" in msg and "wrong shape" in msg


def test_loaded_dtypes(tmp_path):
    from llm_b200.weights import load_tensors, write_random_model
    from llm_b200.weights.loader import expected_tensors
    d = write_random_model(str(tmp_path / "m"), CONFIG_A, 1, "bfloat16")
    t = load_tensors(d, expected_tensors(CONFIG_A), torch.bfloat16, torch.device("cpu"))
    assert t["lm_head.weight"].dtype == torch.bfloat16 and t["model.norm.weight"].dtype == torch.float32
    t32 = load_tensors(d, expected_tensors(CONFIG_A), torch.float32, torch.device("cpu"))
    assert t32["lm_head.weight"].dtype == torch.float32
    assert torch.equal(t32["lm_head.weight"], t["lm_head.weight"].float())


def test_buffers_that_checkpoints_carry_are_not_an_error(tmp_path):
    """Rotary inverse-frequency buffers and an lm_head.weight beside tied embeddings load; any other
    extra tensor is still refused."""
    from llm_b200.weights import SafetensorsFile, WeightError, load_tensors, write_random_model, write_safetensors
    from llm_b200.weights.loader import expected_tensors
    from tiny import CONFIG_C
    d = write_random_model(str(tmp_path / "m"), CONFIG_C, 1, "float32")            # tied embeddings
    path = os.path.join(d, "model.safetensors")
    f = SafetensorsFile(path)
    t = {n: f.tensor(n).clone() for n in f.names()}
    f.close()
    t["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(24)
    t["lm_head.weight"] = t["model.embed_tokens.weight"].clone()
    write_safetensors(path, t)
    got = load_tensors(d, expected_tensors(CONFIG_C), torch.float32, torch.device("cpu"))
    assert set(got) == set(expected_tensors(CONFIG_C))
    t["lm_head.bias"] = torch.zeros(301)
    write_safetensors(path, t)
    with pytest.raises(WeightError) as ei:
        load_tensors(d, expected_tensors(CONFIG_C), torch.float32, torch.device("cpu"))
    assert ei.value.unexpected == ["lm_head.bias"]


def test_bias_flags_add_bias_tensors():
    from llm_b200.config import parse_config
    from llm_b200.weights.loader import expected_tensors
    from tiny import CONFIG_F, CONFIG_G
    _, cfg = parse_config(CONFIG_F)
    assert cfg.attention_bias and cfg.mlp_bias and cfg.head_dim == 80
    names = expected_tensors(CONFIG_F)
    for n, shape in (("self_attn.q_proj.bias", (320,)), ("self_attn.k_proj.bias", (160,)), ("self_attn.v_proj.bias", (160,)),
                     ("self_attn.o_proj.bias", (160,)), ("mlp.gate_proj.bias", (208,)), ("mlp.up_proj.bias", (208,)),
                     ("mlp.down_proj.bias", (160,))):
        assert names[f"model.layers.1.{n}"].shape == shape
    g = expected_tensors(CONFIG_G)
    assert "model.layers.0.self_attn.o_proj.bias" in g and "model.layers.0.mlp.up_proj.bias" not in g
    assert not any(n.endswith(".bias") for n in expected_tensors(CONFIG_A))


def test_sharded_checkpoint_with_an_index(tmp_path):
    """A folder whose tensors are spread over several files named by model.safetensors.index.json
    loads like a single file, and its errors name what is missing or misplaced."""
    from llm_b200.weights import SafetensorsError, SafetensorsFile, WeightError, load_tensors, write_random_model, write_safetensors
    from llm_b200.weights.loader import expected_tensors
    d = write_random_model(str(tmp_path / "m"), CONFIG_A, 4, "bfloat16")
    single = os.path.join(d, "model.safetensors")
    f = SafetensorsFile(single)
    t = {n: f.tensor(n).clone() for n in f.names()}
    f.close()
    want = load_tensors(d, expected_tensors(CONFIG_A), torch.float32, torch.device("cpu"))
    os.remove(single)
    names = sorted(t)
    parts = {"model-00001-of-00002.safetensors": names[:9], "model-00002-of-00002.safetensors": names[9:]}
    for fname, ns in parts.items():
        write_safetensors(os.path.join(d, fname), {n: t[n] for n in ns})
    index = {"metadata": {"total_size": 0}, "weight_map": {n: fname for fname, ns in parts.items() for n in ns}}
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as fh:
        json.dump(index, fh)
    got = load_tensors(d, expected_tensors(CONFIG_A), torch.float32, torch.device("cpu"))
    assert set(got) == set(want) and all(torch.equal(got[n], want[n]) for n in want)
    # the index names a tensor that its file does not hold
    index["weight_map"][names[0]] = "model-00002-of-00002.safetensors"
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as fh:
        json.dump(index, fh)
    with pytest.raises(SafetensorsError, match="does not hold it"):
        load_tensors(d, expected_tensors(CONFIG_A), torch.float32, torch.device("cpu"))
    # a tensor that no file holds is reported as missing
    del index["weight_map"][names[0]]
    write_safetensors(os.path.join(d, "model-00001-of-00002.safetensors"), {n: t[n] for n in names[1:9]})
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as fh:
        json.dump(index, fh)
    with pytest.raises(WeightError) as ei:
        load_tensors(d, expected_tensors(CONFIG_A), torch.float32, torch.device("cpu"))
    assert ei.value.missing == [names[0]]
