"""Random loads through the runner: many requests of random lengths, token budgets of 256 or 2,048, pools so tight that
requests are preempted, greedy and sampled (top-k, top-p, a repeat penalty whose window is completed on the device),
with the next step launched ahead and one step at a time.

In 32-bit a position's logits do not depend on the batch it shared a step with, so the two ways of stepping give the
same tokens for every request, whatever the order in which they were admitted, preempted and ended.  In bfloat16
(where they agree to rounding only, and 64 requests of 8 kv heads take the decode attention in even shares) the
invariants are checked: every request ends with its length, no page is lost, the flags that pieces of the attention
are handed over with are lowered again, no kernel reported a wait that ran out."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

CONFIG = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 256, "num_hidden_layers": 2, "num_attention_heads": 16,
    "num_key_value_heads": 8, "head_dim": 64, "intermediate_size": 512, "vocab_size": 600, "rms_norm_eps": 1e-5,
    "rope_theta": 10000.0, "rope_scaling": None, "max_position_embeddings": 2048, "tie_word_embeddings": True,
    "hidden_act": "silu", "torch_dtype": "bfloat16",
}


def one_round(seed, dtype, ahead):
    from xyntetik_runner_b200 import kernels
    from xyntetik_runner_b200.config.llama import LlamaConfig
    from xyntetik_runner_b200.engine.runner import Runner
    cfg = LlamaConfig.from_dict(CONFIG)
    rng = np.random.RandomState(seed)
    n_req = int(rng.choice([3, 12, 40, 64]))
    tight, sampled, budget = bool(rng.rand() < 0.4), bool(rng.rand() < 0.5), int(rng.choice([256, 2048]))
    prompts = [[int(t) for t in rng.randint(0, cfg.vocab_size, size=int(rng.randint(1, 500)))] for _ in range(n_req)]
    lens = [int(rng.randint(1, 40)) for _ in range(n_req)]
    kw = dict(config=cfg, random_seed=3, ctx=1024, batch=budget, parallel=min(n_req, 48), page_size=64, dtype=dtype)
    if tight:
        kw["max_tokens"] = 64 * max(14, sum(len(p) for p in prompts) // 64 // 2)
    r = Runner(**kw)
    r.scheduler.params.look_ahead = ahead
    ids = []
    for i, (p, n) in enumerate(zip(prompts, lens)):
        if sampled:
            ids.append(r.submit(p, n=n, temp=0.9, top_k=40 if i % 2 else 0, top_p=0.9, repeat_penalty=1.2 if i % 3 else 1.0,
                                seed=100 + i, ignore_eos=True, stop_ids=[5, 9]))
        else:
            ids.append(r.submit(p, n=n, temp=0.0, ignore_eos=True))
    steps = 0
    while r.scheduler.has_work():
        r.scheduler.step()
        steps += 1
        if steps % 16 == 0:
            r.engine.cache.audit()
        assert steps < 5000
    torch.cuda.synchronize()
    r.engine.check_status()
    r.engine.cache.audit()
    assert not r.engine.cache.live_requests()
    assert int(kernels.workspace(torch.device("cuda:0")).flags.abs().sum()) == 0
    done = [r.scheduler.finished[i] for i in ids]
    assert [len(q.generated) for q in done] == lens and all(q.finish_reason == "length" for q in done)
    stats = dict(r.scheduler.stats)
    del r
    torch.cuda.empty_cache()
    return [q.generated for q in done], stats, n_req


def test_random_loads_in_32_bit_give_the_same_tokens_ahead_and_stepwise():
    ahead_steps = preemptions = 0
    sizes = set()
    for seed in range(1, 15):
        got, stats, n_req = one_round(seed, "float32", True)
        want, _, _ = one_round(seed, "float32", False)
        assert got == want, f"round {seed}: {sum(a != b for a, b in zip(got, want))} of {n_req} requests differ"
        ahead_steps += stats.get("steps_launched_ahead", 0)
        preemptions += stats.get("preemptions", 0)
        sizes.add(n_req)
    assert ahead_steps > 100 and preemptions >= 1 and len(sizes) >= 3          # what the rounds are for


def test_random_loads_in_bfloat16_keep_the_invariants():
    from xyntetik_runner_b200 import kernels
    even0 = kernels.attention_even_launches()
    for seed in range(1, 11):
        for ahead in (True, False):
            one_round(seed, "bfloat16", ahead)
    assert kernels.attention_even_launches() > even0                           # rounds of 40 and 64 requests took even shares
