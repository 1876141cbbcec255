"""Layer sizes of the models the benchmarks name (a few layers of each, so that the test takes seconds) with random bfloat16 weights:
the serving path against the engine's own true 32-bit path on the same weights, whole and cut.  The tiny
configurations anchor the arithmetic on the plain implementation; this anchors the kernels at the sizes
they are tuned for (head size 128, four heads per kv head, widths 4096/14336, a 128,256-entry vocabulary)."""
import numpy as np
import pytest
import torch

import traces

pytestmark = pytest.mark.gpu

SHAPE = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 4096, "num_hidden_layers": 4, "num_attention_heads": 32,
    "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 14336, "vocab_size": 128256, "rms_norm_eps": 1e-5,
    "rope_theta": 500000.0, "rope_scaling": None, "max_position_embeddings": 8192, "tie_word_embeddings": False,
    "hidden_act": "silu", "torch_dtype": "bfloat16",
}


# Llama-3.2-1B layer sizes: head size 64, tied head, llama3 rope scaling x32
SHAPE_1B = dict(SHAPE, hidden_size=2048, num_hidden_layers=3, num_attention_heads=32, num_key_value_heads=8, head_dim=64,
                intermediate_size=8192, tie_word_embeddings=True,
                rope_scaling={"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                              "original_max_position_embeddings": 8192})
# Llama-2-13B layer sizes: as many kv heads as heads, a 32,000-entry vocabulary, theta 10000
SHAPE_13B = dict(SHAPE, hidden_size=5120, num_hidden_layers=2, num_attention_heads=40, num_key_value_heads=40, head_dim=128,
                 intermediate_size=13824, vocab_size=32000, rope_theta=10000.0, max_position_embeddings=4096)


@pytest.mark.parametrize("shape", [SHAPE, SHAPE_1B, SHAPE_13B], ids=["llama-3-8b", "llama-3.2-1b", "llama-2-13b"])
def test_serving_path_matches_the_32_bit_path_at_8b_layer_sizes(shape):
    from xyntetik_runner_b200.config.llama import LlamaConfig
    from xyntetik_runner_b200.engine.engine import EngineParams, random_engine
    from xyntetik_runner_b200.engine.replay import replay
    from xyntetik_runner_b200.parts import linear
    cfg = LlamaConfig.from_dict(shape)
    V = cfg.vocab_size
    reqs = {"a": traces.random_tokens(1, 150, V), "b": traces.random_tokens(2, 70, V), "c": traces.random_tokens(3, 600, V)}     # 600: several token tiles of the CTA-pair product

    def only_last(steps, keep=3):
        """ask for logits at the last `keep` tokens of every entry only (a row of logits is half a megabyte)"""
        for st in steps:
            for e in st["entries"]:
                e["want"] = list(range(max(0, len(e["tokens"]) - keep), len(e["tokens"])))
        return steps

    results = {}
    for dtype in ("float32", "bfloat16"):
        for cut_name, cut in (("whole", traces.whole), ("mixed", lambda r: traces.mixed(r, seed=4, max_live=3))):
            steps = only_last(cut(reqs))
            # weights: the same seeded draw for both engines
            eng = random_engine(cfg, 2, EngineParams(dtype=dtype, max_tokens=traces.pool_tokens(steps), page_size=64, max_requests=3),
                                std=0.02, norm_jitter=0.0)
            before = dict(linear.counters)
            res = replay(eng, steps)
            eng.cache.audit()
            used_tc = linear.counters["tcgen05"] - before["tcgen05"]
            assert (used_tc > 0) == (dtype == "bfloat16")          # the tensor-core kernel ran iff serving path
            out = {}
            for st in steps:
                if st["step"] not in res:
                    continue
                arr, at = res[st["step"]], 0
                for e in st["entries"]:
                    p0 = sum(len(x["tokens"]) for s2 in steps[:steps.index(st)] for x in s2["entries"] if x["id"] == e["id"])
                    for w in e["want"]:
                        out[e["id"], p0 + w] = arr[at]
                        at += 1
            results[dtype, cut_name] = out
            del eng
            torch.cuda.empty_cache()
    ref = results["float32", "whole"]
    # 32 bit: cutting changes nothing but rounding
    for key, row in results["float32", "mixed"].items():
        if key in ref:
            scale = np.abs(ref[key]).max()
            assert np.abs(row - ref[key]).max() <= 1e-4 * scale, key
    # bfloat16 against 32 bit, whole and mixed
    common = 0
    for cut_name in ("whole", "mixed"):
        for key, row in results["bfloat16", cut_name].items():
            if key not in ref:
                continue
            common += 1
            scale = np.abs(ref[key]).max()
            d = np.abs(row - ref[key])
            assert d.max() <= traces.TOL["bfloat16"]["max_rel"] * scale and d.mean() <= traces.TOL["bfloat16"]["mean_rel"] * scale, (cut_name, key)
    assert common >= 12
