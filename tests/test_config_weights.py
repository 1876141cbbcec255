"""Configuration, registry and weight-loading errors (no GPU)."""
import copy
import json
import os
import shutil

import numpy as np
import pytest
import torch

import tiny
from xyntetik_runner_b200 import architectures  # noqa: F401
from xyntetik_runner_b200.architectures.llama import build_llama
from xyntetik_runner_b200.config import registry
from xyntetik_runner_b200.config.llama import ConfigError, LlamaConfig
from xyntetik_runner_b200.weights.loader import FolderSource, WeightsError, load_tensors
from xyntetik_runner_b200.weights.safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors


def test_reads_every_key():
    c = LlamaConfig.from_dict(tiny.TINY_B)
    assert (c.hidden_size, c.num_hidden_layers, c.num_attention_heads, c.num_key_value_heads) == (96, 3, 3, 1)
    assert (c.head_dim, c.intermediate_size, c.vocab_size) == (32, 200, 387)
    assert c.rms_norm_eps == 1e-6 and c.rope_theta == 500000.0 and not c.tie_word_embeddings
    assert c.rope_scaling.factor == 8.0 and c.rope_scaling.original_max_position_embeddings == 64
    assert c.eos_token_ids == (5, 7) and c.q_dim == 96 and c.kv_dim == 32
    a = LlamaConfig.from_dict(tiny.TINY_A)
    assert a.tie_word_embeddings and a.rope_scaling is None and a.eos_token_ids == (2,) and a.bos_token_id == 1
    assert LlamaConfig.from_dict(a.to_dict()) == a


def test_defaults_follow_the_reference():
    d = {k: v for k, v in tiny.TINY_A.items() if k not in ("num_key_value_heads", "head_dim", "rope_theta")}
    c = LlamaConfig.from_dict(d)
    assert c.num_key_value_heads == c.num_attention_heads and c.head_dim == 16 and c.rope_theta == 10000.0


@pytest.mark.parametrize("key,value", [
    ("hidden_size", 0), ("num_hidden_layers", 0), ("num_hidden_layers", 100001), ("num_attention_heads", 0),
    ("num_key_value_heads", 3), ("num_key_value_heads", 8), ("head_dim", 15), ("intermediate_size", -4),
    ("vocab_size", 0), ("rms_norm_eps", 0.0), ("rope_theta", -1.0), ("hidden_size", (1 << 20) + 1),
    ("hidden_act", "gelu"), ("mlp_bias", True), ("torch_dtype", "int8"), ("hidden_size", "64"),
    ("rope_scaling", {"rope_type": "yarn", "factor": 2.0}), ("rope_scaling", {"rope_type": "llama3", "factor": 8.0}),
    ("eos_token_id", 999), ("sliding_window", 0), ("layer_types", ["full_attention"]),
])
def test_refuses_bad_values(key, value):
    d = copy.deepcopy(tiny.TINY_A)
    d[key] = value
    with pytest.raises(ConfigError):
        LlamaConfig.from_dict(d)


def test_refuses_missing_keys():
    for key in ("hidden_size", "num_hidden_layers", "num_attention_heads", "intermediate_size", "vocab_size",
                "rms_norm_eps", "max_position_embeddings"):
        d = copy.deepcopy(tiny.TINY_A)
        del d[key]
        with pytest.raises(ConfigError, match=key):
            LlamaConfig.from_dict(d)


def test_registry_refuses_unknown_architectures(tmp_path):
    assert "LlamaForCausalLM" in registry.known_architectures()
    with pytest.raises(registry.UnknownArchitecture, match="Gemma2ForCausalLM.*LlamaForCausalLM"):
        registry.resolve("Gemma2ForCausalLM")
    d = copy.deepcopy(tiny.TINY_A)
    d["architectures"] = ["MixtralForCausalLM"]
    (tmp_path / "config.json").write_text(json.dumps(d))
    with pytest.raises(ConfigError, match="MixtralForCausalLM"):
        registry.load_config(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError):
        registry.load_config(str(tmp_path))
    with pytest.raises(ConfigError):
        registry.load_config(str(tmp_path / "nowhere"))


def test_layer_windows():
    c = LlamaConfig.from_dict(tiny.TINY_C)
    assert [c.layer_window(i) for i in range(3)] == [24, None, 24]
    plan = build_llama(c)
    assert [b.mixer.window for b in plan.blocks] == [24, None, 24]


def _specs(name):
    return build_llama(LlamaConfig.from_dict(tiny.CONFIGS[name])).tensor_specs()


def test_tensor_names_and_shapes():
    s = _specs("B")
    assert s["model.embed_tokens.weight"].shape == (387, 96)
    assert s["lm_head.weight"].shape == (387, 96)
    assert s["model.layers.2.self_attn.k_proj.weight"].shape == (32, 96)
    assert s["model.layers.0.mlp.down_proj.weight"].shape == (96, 200)
    assert s["model.norm.weight"].shape == (96,)
    assert "lm_head.weight" not in _specs("A")           # tied
    assert _specs("C")["model.layers.1.self_attn.o_proj.bias"].shape == (80,)
    assert len(s) == 2 + 1 + 3 * 9


def test_random_folder_round_trip_and_reproducible(tmp_path):
    a = tiny.make_folder(str(tmp_path / "a"), "A")
    b = tiny.make_folder(str(tmp_path / "b"), "A")
    fa, fb = SafetensorsFile(os.path.join(a, "model.safetensors")), SafetensorsFile(os.path.join(b, "model.safetensors"))
    assert fa.names() == fb.names()
    for n in fa.names():
        assert torch.equal(fa.get(n), fb.get(n))
    got = load_tensors(_specs("A"), FolderSource(a), torch.device("cpu"))
    w = got["model.layers.1.mlp.up_proj.weight"]
    assert w.dtype == torch.float32 and abs(float(w.std()) - 0.1) < 0.01
    assert abs(float(got["model.norm.weight"].mean()) - 1.0) < 0.1
    assert json.load(open(os.path.join(a, "config.json")))["intermediate_size"] == 176
    # bfloat16 folders keep bfloat16
    c = tiny.make_folder(str(tmp_path / "c"), "A", "bfloat16")
    got = load_tensors(_specs("A"), FolderSource(c), torch.device("cpu"))
    assert got["model.layers.0.self_attn.q_proj.weight"].dtype == torch.bfloat16


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = tiny.make_folder(str(tmp_path / "m"), "B")
    f = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    tensors = {n: f.get(n).clone() for n in f.names()}
    del tensors["model.layers.1.mlp.gate_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(16)
    tensors["model.layers.2.self_attn.v_proj.weight"] = torch.zeros(32, 95)
    tensors["lm_head.weight"] = torch.zeros(387, 96, dtype=torch.int32)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors.items())
    with pytest.raises(WeightsError) as ei:
        load_tensors(_specs("B"), FolderSource(folder), torch.device("cpu"))
    e = ei.value
    assert e.missing == ["model.layers.1.mlp.gate_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert e.wrong_shape == [("model.layers.2.self_attn.v_proj.weight", (32, 95), (32, 96))]
    assert e.bad_dtype and e.bad_dtype[0][0] == "lm_head.weight"
    msg = str(e)
    for needle in ("gate_proj", "model.norm.weight", "inv_freq", "[32, 95]", "[32, 96]", "lm_head.weight"):
        assert needle in msg


def test_tied_model_refuses_a_head_tensor(tmp_path):
    folder = tiny.make_folder(str(tmp_path / "m"), "A")
    f = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    tensors = {n: f.get(n).clone() for n in f.names()}
    tensors["lm_head.weight"] = torch.zeros(256, 64)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors.items())
    with pytest.raises(WeightsError, match="unexpected.*lm_head.weight"):
        load_tensors(_specs("A"), FolderSource(folder), torch.device("cpu"))


def test_broken_container(tmp_path):
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(str(p))
    p.write_bytes((10 ** 9).to_bytes(8, "little") + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        SafetensorsFile(str(p))
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [4, 4], "data_offsets": [0, 64]}}).encode()
    p.write_bytes(len(hdr).to_bytes(8, "little") + hdr + b"\0" * 32)       # data cut short
    with pytest.raises(SafetensorsError, match="outside the file"):
        SafetensorsFile(str(p))
    with pytest.raises(SafetensorsError):
        FolderSource(str(tmp_path / "none"))


def test_float16_is_widened_and_tables_are_int32(tmp_path):
    from xyntetik_runner_b200.weights.loader import TensorSpec
    write_safetensors(str(tmp_path / "model.safetensors"),
                      [("h", torch.tensor([[1.5, -2.25]], dtype=torch.float16)), ("t", torch.tensor([3, 4], dtype=torch.int64))])
    got = load_tensors({"h": TensorSpec((1, 2)), "t": TensorSpec((2,), "table")}, FolderSource(str(tmp_path)), torch.device("cpu"))
    assert got["h"].dtype == torch.float32 and got["h"].tolist() == [[1.5, -2.25]]
    assert got["t"].dtype == torch.int32 and got["t"].tolist() == [3, 4]


def test_rope_table_matches_the_plain_formula():
    from plain_llama import rope_inv_freq
    from xyntetik_runner_b200.parts.position import Rope
    for name in "ABC":
        c = LlamaConfig.from_dict(tiny.CONFIGS[name])
        mine = Rope(c.head_dim, c.rope_theta, scaling=c.rope_scaling).inv_freq_host
        ref = rope_inv_freq(c.rope_theta, c.head_dim, tiny.CONFIGS[name].get("rope_scaling"))
        assert mine.dtype == np.float32 and np.array_equal(mine, ref)
    b = LlamaConfig.from_dict(tiny.TINY_B)
    plain = Rope(b.head_dim, b.rope_theta).inv_freq_host
    scaled = Rope(b.head_dim, b.rope_theta, scaling=b.rope_scaling).inv_freq_host
    ratio = plain / scaled
    assert ratio[0] == 1.0 and abs(ratio[-1] - 8.0) < 1e-5 and (np.diff(ratio) >= -1e-6).all()
    assert ((ratio > 1.001) & (ratio < 7.999)).any()          # the interpolated band is exercised
    # linear scaling: every frequency divided by the factor
    lin = LlamaConfig.from_dict(dict(tiny.TINY_A, rope_scaling={"type": "linear", "factor": 2.5}))
    assert lin.rope_scaling.rope_type == "linear" and LlamaConfig.from_dict(lin.to_dict()) == lin
    mine = Rope(lin.head_dim, lin.rope_theta, scaling=lin.rope_scaling).inv_freq_host
    assert np.array_equal(mine, rope_inv_freq(lin.rope_theta, lin.head_dim, {"type": "linear", "factor": 2.5}))
    assert np.allclose(Rope(lin.head_dim, lin.rope_theta).inv_freq_host / mine, 2.5, rtol=1e-6)
    with pytest.raises(ConfigError, match="factor"):
        LlamaConfig.from_dict(dict(tiny.TINY_A, rope_scaling={"type": "linear", "factor": 0.0}))


def test_llama3_divisors_against_constants():
    """The per-frequency divisors of rope_scaling type llama3, pinned by numbers: how many frequencies stay as they
    are, how many are divided by the whole factor, and the divisors of the band between (worked out in float64 from
    the turns a frequency makes over the original context, turns = orig * f / 2 pi: more than `high` turns keeps f,
    fewer than `low` divides by `factor`, between them f' = (1 - s) f / factor + s f with
    s = (turns - low) / (high - low)), for the parameters of Llama-3.1, Llama-3.2 and tiny configuration B."""
    from xyntetik_runner_b200.parts.position import llama3_divisors
    cases = {
        # (theta, head size, factor, low, high, original context): (kept, fully divided, {index: divisor})
        (5e5, 128, 8.0, 1.0, 4.0, 8192): (29, 29, {29: 1.207483871283662, 30: 1.5534146285049257, 31: 2.0263132059050557,
                                                     32: 2.694529687894733, 33: 3.6842525277457185, 34: 5.257326588708465}),
        (5e5, 64, 32.0, 1.0, 4.0, 8192): (15, 14, {15: 1.6513292457638984, 16: 3.292262102940884, 17: 9.666728978753287}),
        (5e5, 32, 8.0, 1.0, 4.0, 64): (2, 13, {2: 2.4422593898300864}),
    }
    for (theta, hd, factor, low, high, orig), (kept, full, band) in cases.items():
        j = np.arange(hd // 2, dtype=np.float32)
        inv = np.power(np.float32(theta), (np.float32(-2.0) * j / np.float32(hd)).astype(np.float32)).astype(np.float32)
        div = llama3_divisors(inv, factor, low, high, orig)
        assert div.dtype == np.float32 and int((div == 1.0).sum()) == kept and int((div == np.float32(factor)).sum()) == full
        assert len(band) == hd // 2 - kept - full
        for idx, want in band.items():
            assert abs(float(div[idx]) - want) <= 3e-6 * want, (hd, idx, float(div[idx]), want)      # inv is float32: 1e-7 relative, amplified near s = 0
        assert (np.diff(div) >= 0).all()


def _write_shards(folder, tensors, split_at, weight_map=None, extra_in_second=None):
    """Write `tensors` as two shards and an index; the first `split_at` names go to the first shard."""
    from xyntetik_runner_b200.weights.safetensors_io import write_safetensors
    names = list(tensors)
    shards = {"model-00001-of-00002.safetensors": names[:split_at], "model-00002-of-00002.safetensors": names[split_at:]}
    wm = {}
    for fn, ns in shards.items():
        items = [(n, tensors[n]) for n in ns]
        if fn.startswith("model-00002") and extra_in_second:
            items += list(extra_in_second.items())
        write_safetensors(os.path.join(folder, fn), items)
        wm.update({n: fn for n in ns})
    with open(os.path.join(folder, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {}, "weight_map": wm if weight_map is None else weight_map(wm)}, f)


def test_sharded_folder_loads_and_its_errors_come_as_one(tmp_path):
    """Two shards and model.safetensors.index.json (the layout of a real multi-gigabyte checkpoint): the same tensors
    as the single file; a name stored twice, one that the index does not list, and one that the index lists but no
    shard holds are all named in ONE error."""
    src = tiny.make_folder(str(tmp_path / "one"), "B")
    single = SafetensorsFile(os.path.join(src, "model.safetensors"))
    tensors = {n: single.get(n).clone() for n in single.names()}
    specs = _specs("B")
    good = tmp_path / "two"
    good.mkdir()
    shutil.copy(os.path.join(src, "config.json"), good / "config.json")
    _write_shards(str(good), tensors, split_at=11)
    got = load_tensors(specs, FolderSource(str(good)), torch.device("cpu"))
    want = load_tensors(specs, FolderSource(src), torch.device("cpu"))
    assert set(got) == set(want) and all(torch.equal(got[n], want[n]) for n in want)
    assert len(FolderSource(str(good)).files) == 2
    # broken: a tensor of the first shard stored again in the second, one extra tensor that the index does not list,
    # and the index lists one name more than the shards hold
    names = list(tensors)
    bad = tmp_path / "bad"
    bad.mkdir()
    _write_shards(str(bad), tensors, split_at=11, extra_in_second={names[0]: tensors[names[0]], "model.stray": torch.zeros(3)},
                  weight_map=lambda wm: dict(wm, **{"model.ghost.weight": "model-00001-of-00002.safetensors"}))
    with pytest.raises(WeightsError) as ei:
        FolderSource(str(bad))
    msg = str(ei.value)
    assert "stored twice" in msg and names[0] in msg and "model.stray" in msg and "not in the index" in msg
    assert "model.ghost.weight" in msg and "in no shard" in msg
    # the index names a shard that is not there: a clear error as well
    os.remove(bad / "model-00002-of-00002.safetensors")
    with pytest.raises(Exception, match="model-00002-of-00002.safetensors"):
        FolderSource(str(bad))
    # a name in the index only, nothing else wrong: reported as missing with the other mismatches by load_tensors
    part = tmp_path / "part"
    part.mkdir()
    fewer = {n: t for n, t in tensors.items() if n != "model.norm.weight"}
    _write_shards(str(part), fewer, split_at=5, weight_map=lambda wm: dict(wm, **{"model.norm.weight": "model-00001-of-00002.safetensors"}))
    with pytest.raises(WeightsError) as ei:
        load_tensors(specs, FolderSource(str(part)), torch.device("cpu"))
    assert ei.value.missing == ["model.norm.weight"]


def test_random_values_do_not_depend_on_how_they_are_drawn():
    """The counter-based generator: a tensor's values are a function of (seed, name, element) alone -- whole or in
    pieces, whatever else was drawn before -- normal, and the same numbers forever (pinned below: a change of the
    recipe would change every seeded model)."""
    from xyntetik_runner_b200.weights import random_fill as rf
    from xyntetik_runner_b200.weights.loader import RandomSource, TensorSpec
    key = rf.tensor_key(7, "model.layers.3.mlp.up_proj.weight")
    whole = rf.normal_values(key, 0, 5000, 0.0, 0.02)
    assert np.array_equal(np.concatenate([rf.normal_values(key, 0, 1234, 0.0, 0.02), rf.normal_values(key, 1234, 3766, 0.0, 0.02)]), whole)
    assert np.array_equal(rf.unit_normal_at(key, np.array([4999, 0, 17]))[[1, 2, 0]] * np.float32(0.02), whole[[0, 17, 4999]])
    assert not np.array_equal(rf.normal_values(rf.tensor_key(7, "other"), 0, 100, 0.0, 0.02), whole[:100])
    z = rf.normal_values(key, 0, 1 << 18, 0.0, 1.0)
    assert abs(float(z.mean())) < 0.01 and abs(float(z.std()) - 1) < 0.01 and abs(float((z ** 4).mean()) - 3) < 0.1
    assert abs(float(np.corrcoef(z[:-1], z[1:])[0, 1])) < 0.01
    assert rf.unit_normal_at(rf.tensor_key(2, "model.embed_tokens.weight"), np.arange(3)).view(np.uint32).tolist() == PINNED_DRAWS
    # bfloat16 rounding to nearest even, as torch rounds
    x = rf.normal_values(key, 0, 4096, 0.0, 1.0)
    assert np.array_equal(rf.to_bfloat16_bits(x), torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16))
    # through the source: the order of fetches and the other tensors' sizes change nothing
    specs = {"a": TensorSpec((5, 7)), "b": TensorSpec((3,), "vector", "ones_jitter"), "c": TensorSpec((2, 2), init="zeros")}
    s1 = RandomSource(specs, 11, torch.float32, std=0.1, norm_jitter=0.1)
    s2 = RandomSource(dict(specs, a2=TensorSpec((900, 9))), 11, torch.float32, std=0.1, norm_jitter=0.1)
    dev = torch.device("cpu")
    s2.fetch("a2", dev)
    for n in ("b", "a", "c"):
        assert torch.equal(s1.fetch(n, dev), s2.fetch(n, dev))
    assert float(s1.fetch("c", dev).abs().sum()) == 0 and abs(float(s1.fetch("b", dev).mean()) - 1) < 0.2


PINNED_DRAWS = [3197608319, 3192270923, 1071824072]      # float32 bit patterns of z(seed 2, "model.embed_tokens.weight", 0..2)
