"""Configuration, registry, safetensors and weight errors (no GPU)."""

import json

import pytest
import torch

from configs import CONFIGS, TINY_A, TINY_B
from scratch_llm_b200.config import (LlamaConfig, config_from_dict, load_config,
                                     register_architecture)
from scratch_llm_b200.config.spec import ModelSpec, PartSpec, Run
from scratch_llm_b200.engine import build_model
from scratch_llm_b200.weights import (ParamSpec, SafetensorsError, SafetensorsFile, WeightError,
                                      load_tensors, random_tensors, write_random_model,
                                      write_safetensors)


def test_config_reads_its_keys():
    cfg = config_from_dict(TINY_B)
    assert isinstance(cfg, LlamaConfig)
    assert (cfg.kv_heads, cfg.head_size, cfg.rms_norm_eps, cfg.rope_theta) == (1, 32, 1e-6, 500000.0)
    assert cfg.tie_word_embeddings and cfg.max_position_embeddings == 256
    spec = cfg.model_spec()
    assert len(spec.layers) == 3 and [r.layer for r in spec.order] == [0, 1, 2]
    assert spec.layers[1].parts["mixer"].args["n_kv_heads"] == 1
    assert spec.layers[1].parts["mixer_norm"].args["eps"] == 1e-6
    assert config_from_dict(cfg.to_dict()) == cfg


def test_config_defaults_and_derived_head_size():
    cfg = config_from_dict(dict(architectures=["LlamaForCausalLM"], hidden_size=96,
                                num_hidden_layers=1, num_attention_heads=6,
                                intermediate_size=100, vocab_size=50))
    assert cfg.kv_heads == 6 and cfg.head_size == 16 and cfg.rope_theta == 10000.0
    assert cfg.rms_norm_eps == 1e-5 and not cfg.tie_word_embeddings


@pytest.mark.parametrize("change, message", [
    (dict(num_attention_heads=5, head_dim=None), "not divisible"),
    (dict(num_key_value_heads=3), "group"),
    (dict(head_dim=15), "even"),
    (dict(vocab_size=0), "positive"),
    (dict(rms_norm_eps=0.0), "rms_norm_eps"),
    (dict(attention_bias=True), "unsupported"),
    (dict(rope_scaling={"type": "llama3"}), "rope_scaling"),
    (dict(sliding_window=128), "sliding_window"),
])
def test_config_rejects(change, message):
    raw = {**TINY_A, **change}
    raw = {k: v for k, v in raw.items() if v is not None}
    with pytest.raises(ValueError, match=message):
        config_from_dict(raw)


def test_config_missing_keys_and_unknown_architecture(tmp_path):
    raw = dict(TINY_A)
    del raw["intermediate_size"], raw["vocab_size"]
    with pytest.raises(ValueError, match="intermediate_size, vocab_size"):
        config_from_dict(raw)
    with pytest.raises(ValueError, match="unknown architecture 'Nope'.*LlamaForCausalLM"):
        config_from_dict({**TINY_A, "architectures": ["Nope"]})
    with pytest.raises(FileNotFoundError):
        load_config(tmp_path)
    with pytest.raises(ValueError, match="already registered"):
        register_architecture("LlamaForCausalLM", LlamaConfig)


def test_run_order_is_checked():
    cfg = config_from_dict(TINY_A)
    spec = cfg.model_spec()
    fields = {f: getattr(spec, f) for f in spec.__dataclass_fields__}
    ModelSpec(**{**fields, "order": (Run(0, 0), Run(1, 1), Run(1, 1, write=False))})
    with pytest.raises(ValueError, match="written by two runs"):
        ModelSpec(**{**fields, "order": (Run(0, 0), Run(1, 0))})
    with pytest.raises(ValueError, match="before any run wrote"):
        ModelSpec(**{**fields, "order": (Run(0, 1, write=False),)})
    with pytest.raises(ValueError, match="names layer 7"):
        ModelSpec(**{**fields, "order": (Run(7, 0),)})


def test_unknown_part_names_the_registered_ones():
    cfg = config_from_dict(TINY_A)
    spec = cfg.model_spec()
    import dataclasses
    from scratch_llm_b200.engine.model import DecoderModel
    first = spec.layers[0]
    bad = dataclasses.replace(first, parts={**first.parts, "mixer": PartSpec("no_such_mixer")})
    with pytest.raises(ValueError, match="unknown mixer 'no_such_mixer'.*gqa_attention"):
        DecoderModel(dataclasses.replace(spec, layers=(bad, spec.layers[1])))
    # a layer must give exactly the roles its block arrangement has
    short = dataclasses.replace(first, parts={k: v for k, v in first.parts.items()
                                              if k != "feed_forward_norm"})
    with pytest.raises(ValueError, match="has the roles.*feed_forward_norm"):
        DecoderModel(dataclasses.replace(spec, layers=(short, spec.layers[1])))


def test_safetensors_roundtrip(tmp_path):
    t = {"a": torch.arange(6, dtype=torch.float32).reshape(2, 3),
         "b": torch.randn(5).to(torch.bfloat16), "c": torch.tensor([1, 2, 3], dtype=torch.int64)}
    path = write_safetensors(tmp_path / "x.safetensors", t, {"k": "v"})
    f = SafetensorsFile(path)
    assert dict(f.metadata) == {"k": "v"} and set(f) == {"a", "b", "c"}
    for k in t:
        assert f.entries[k].shape == tuple(t[k].shape)
        assert torch.equal(f.tensor(k), t[k])
    # the library's reader agrees with the file we write
    from safetensors.torch import load_file
    other = load_file(str(path))
    assert all(torch.equal(other[k], t[k]) for k in t)


def test_safetensors_truncated(tmp_path):
    path = write_safetensors(tmp_path / "x.safetensors", {"a": torch.zeros(100)})
    raw = path.read_bytes()
    path.write_bytes(raw[:-40])
    with pytest.raises(SafetensorsError, match="truncated"):
        SafetensorsFile(path)
    path.write_bytes(raw[:5])
    with pytest.raises(SafetensorsError, match="too short"):
        SafetensorsFile(path)


def test_random_model_folder_and_loading(tmp_path):
    cfg = config_from_dict(TINY_B)
    d = write_random_model(cfg, tmp_path / "m", seed=3)
    assert json.loads((d / "config.json").read_text())["architectures"] == ["LlamaForCausalLM"]
    model = build_model(load_config(d))
    specs = model.param_specs()
    assert "lm_head.weight" not in specs  # tied
    assert len(specs) == 9 * 3 + 2
    tensors = load_tensors(d, specs)
    assert tensors["model.layers.2.mlp.down_proj.weight"].shape == (256, 688)
    assert tensors["model.embed_tokens.weight"].dtype == torch.float32  # stored in 32-bit, stays so
    assert torch.all(tensors["model.norm.weight"] == 1)
    w = tensors["model.layers.0.self_attn.q_proj.weight"]
    assert abs(float(w.std()) - 0.02) < 1e-3
    # same seed, same values, whatever the order; another seed, other values
    again = random_tensors(dict(reversed(list(specs.items()))), 3, torch.float32)
    assert torch.equal(again["model.layers.0.self_attn.q_proj.weight"], w)
    assert not torch.equal(random_tensors(specs, 4, torch.float32)
                           ["model.layers.0.self_attn.q_proj.weight"], w)
    # bfloat16 storage stays bfloat16
    d2 = write_random_model(cfg, tmp_path / "m2", seed=3, dtype="bfloat16")
    assert load_tensors(d2, specs)["model.embed_tokens.weight"].dtype == torch.bfloat16


def test_weight_error_lists_everything(tmp_path):
    cfg = config_from_dict(TINY_A)
    d = write_random_model(cfg, tmp_path / "m", seed=0)
    specs = build_model(cfg).param_specs()
    f = SafetensorsFile(d / "model.safetensors")
    t = {k: f.tensor(k).clone() for k in f}
    del t["model.layers.1.mlp.up_proj.weight"], t["model.norm.weight"]
    t["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(16, 64)
    t["extra.bias"] = torch.zeros(3)
    t["lm_head.weight"] = t["lm_head.weight"].to(torch.int32)
    write_safetensors(d / "model.safetensors", t)
    with pytest.raises(WeightError) as info:
        load_tensors(d, specs)
    e = info.value
    assert e.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["extra.bias"]
    assert e.wrong_shape == [("model.layers.0.self_attn.k_proj.weight", (16, 64), (32, 64))]
    assert e.wrong_dtype == [("lm_head.weight", "int32")]
    msg = str(e)
    for part in ("missing (2)", "unexpected (1)", "wrong shape (1)", "is [16, 64], expected [32, 64]"):
        assert part in msg


def test_reference_names_and_tied_head(tmp_path):
    cfg = config_from_dict(TINY_B)
    d = write_random_model(cfg, tmp_path / "m", seed=1)
    specs = build_model(cfg).param_specs()
    f = SafetensorsFile(d / "model.safetensors")
    back = {v: k for k, v in cfg.reference_aliases().items()}
    renamed = {back[k]: f.tensor(k).clone() for k in f}
    renamed["lm_head.weight"] = renamed["token_emb.weight"].clone()  # a state_dict lists both
    write_safetensors(d / "model.safetensors", renamed)
    optional = {"lm_head.weight": "model.embed_tokens.weight"}
    got = load_tensors(d, specs, cfg.reference_aliases(), optional)
    assert set(got) == set(specs)
    renamed["lm_head.weight"][0, 0] += 1
    write_safetensors(d / "model.safetensors", renamed)
    with pytest.raises(WeightError, match="ties it"):
        load_tensors(d, specs, cfg.reference_aliases(), optional)


def test_integer_tables_become_int32(tmp_path):
    write_safetensors(tmp_path / "model.safetensors",
                      {"t": torch.tensor([1, 2], dtype=torch.int64), "h": torch.ones(2, dtype=torch.float16)})
    got = load_tensors(tmp_path, {"t": ParamSpec((2,), "int"), "h": ParamSpec((2,), "gain")})
    assert got["t"].dtype == torch.int32 and got["h"].dtype == torch.bfloat16


def test_sharded_model_folder(tmp_path):
    """A model stored as two shards with ``model.safetensors.index.json``: the loader opens every
    shard the index names and finds each tensor by name; a tensor that is missing from its shard
    is reported by name in the one error."""
    from scratch_llm_b200.weights import write_safetensors
    cfg = config_from_dict(TINY_A)
    whole = write_random_model(cfg, tmp_path / "whole", 7)
    specs = build_model(cfg).param_specs()
    want = load_tensors(whole, specs)
    names = sorted(want)
    first, second = names[:len(names) // 2], names[len(names) // 2:]

    def write(folder, parts):
        folder.mkdir()
        (folder / "config.json").write_text((whole / "config.json").read_text())
        weight_map = {}
        for k, part in enumerate(parts, 1):
            shard = f"model-{k:05d}-of-{len(parts):05d}.safetensors"
            write_safetensors(folder / shard, {n: want[n] for n in part})
            weight_map.update({n: shard for n in part})
        (folder / "model.safetensors.index.json").write_text(json.dumps(
            {"metadata": {}, "weight_map": weight_map}))

    write(tmp_path / "sharded", [first, second])
    got = load_tensors(tmp_path / "sharded", specs)
    assert got.keys() == want.keys()
    for n in names:
        assert torch.equal(got[n], want[n])

    gone = second[0]
    write(tmp_path / "short", [first, second[1:]])
    with pytest.raises(WeightError) as err:
        load_tensors(tmp_path / "short", specs)
    assert err.value.missing == [gone] and not err.value.unexpected
