"""Configurations drawn at random: every size and option of config.json at values that no hand-made tiny
configuration has, replayed in two cuttings, in 32 bit and in bfloat16, against the plain implementation.

The draws are seeded, so a failure names its configuration and can be run again.
"""
import copy

import numpy as np
import pytest

import tiny
import traces
from plain_llama import PlainLlama

pytestmark = pytest.mark.gpu

N_CONFIGS = 24


def draw_config(seed):
    """A LlamaForCausalLM config.json: sizes that are no power of two, any number of heads and groups, even head
    sizes whether or not they are multiples of 16, windows on some layers, every kind of position scaling."""
    rng = np.random.RandomState(1000 + seed)
    kv = int(rng.randint(1, 5))
    groups = int(rng.choice([1, 2, 3, 4, 5, 7, 8]))
    head_dim = int(rng.choice([8, 16, 24, 32, 40, 48, 64, 72, 80, 96, 112, 128, 136]))
    layers = int(rng.randint(1, 5))
    cfg = {
        "architectures": ["LlamaForCausalLM"],
        "hidden_size": 2 * int(rng.randint(20, 120)),
        "num_hidden_layers": layers,
        "num_attention_heads": kv * groups,
        "num_key_value_heads": kv,
        "head_dim": head_dim,
        "intermediate_size": 2 * int(rng.randint(15, 200)),
        "vocab_size": int(rng.randint(90, 900)),
        "rms_norm_eps": float(rng.choice([1e-6, 3e-6, 1e-5, 2e-5, 1e-4])),
        "rope_theta": float(rng.choice([1e4, 2.5e4, 1e5, 5e5, 1e6])),
        "rope_scaling": None,
        "max_position_embeddings": 1024,
        "tie_word_embeddings": bool(rng.randint(2)),
        "attention_bias": bool(rng.randint(2)),
        "hidden_act": "silu",
        "torch_dtype": "float32",
    }
    kind = int(rng.randint(3))
    if kind == 1:
        cfg["rope_scaling"] = {"rope_type": "linear", "factor": float(rng.choice([1.5, 2.0, 4.0]))}
    elif kind == 2:
        cfg["rope_scaling"] = {"rope_type": "llama3", "factor": float(rng.choice([2.0, 8.0, 32.0])),
                               "low_freq_factor": 1.0, "high_freq_factor": float(rng.choice([2.0, 4.0])),
                               "original_max_position_embeddings": int(rng.choice([32, 64, 256]))}
    if rng.randint(2):
        cfg["sliding_window"] = int(rng.randint(5, 70))
        types = [str(rng.choice(["sliding_attention", "full_attention"])) for _ in range(layers)]
        if "sliding_attention" not in types:
            types[int(rng.randint(layers))] = "sliding_attention"
        cfg["layer_types"] = types
    page = int(rng.choice([4, 8, 16, 32, 64]))
    lengths = [int(n) for n in rng.randint(1, 170, size=5)]
    return cfg, page, lengths


@pytest.fixture(scope="module")
def drawn(tmp_path_factory):
    out = {}
    for seed in range(N_CONFIGS):
        cfg, page, lengths = draw_config(seed)
        name = f"R{seed}"
        tiny.CONFIGS[name] = cfg
        tiny.SEEDS[name] = 50 + seed
        try:
            folders = {dt: tiny.make_folder(str(tmp_path_factory.mktemp(f"drawn{seed}_{dt}")), name, dt)
                       for dt in ("float32", "bfloat16")}
        finally:
            del tiny.CONFIGS[name], tiny.SEEDS[name]
        reqs = {f"r{i}": traces.random_tokens(7 * seed + i, n, cfg["vocab_size"]) for i, n in enumerate(lengths)}
        out[seed] = (copy.deepcopy(cfg), page, reqs, folders)
    return out


CUTS = {"tail": lambda reqs: traces.tail_decoded(reqs, 12), "mixed": lambda reqs: traces.mixed(reqs, seed=11)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(N_CONFIGS))
def test_a_drawn_configuration_matches_plain(drawn, seed, dtype):
    from xyntetik_runner_b200.engine.engine import Engine, EngineParams
    from xyntetik_runner_b200.engine.replay import replay
    cfg, page, reqs, folders = drawn[seed]
    what = {k: cfg[k] for k in ("hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
                                "head_dim", "intermediate_size", "vocab_size")}
    what.update(page=page, window=cfg.get("sliding_window"), scaling=(cfg["rope_scaling"] or {}).get("rope_type"))
    plain = PlainLlama(folders[dtype])
    ref = {rid: plain.logits(t) for rid, t in reqs.items()}
    for cut, make in CUTS.items():
        steps = make(reqs)
        eng = Engine(folders[dtype], EngineParams(dtype=dtype, max_tokens=traces.pool_tokens(steps, max(64, page)),
                                                  page_size=page, max_requests=4))
        res = replay(eng, steps)
        eng.cache.audit()
        assert not eng.cache.live_requests()
        got = traces.collect(steps, res, cfg["vocab_size"])
        for rid in reqs:
            traces.assert_close(got[rid], ref[rid], dtype, f"drawn configuration {seed} {what} / {cut} / {dtype} / {rid}")
