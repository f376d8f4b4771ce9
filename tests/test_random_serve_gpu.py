"""Random configurations, random engine settings and random requests through ``LLM.serve``
(fixed seeds): greedy generation in 32-bit must give the plain implementation's greedy
continuation whatever the page size, the token budget, the portion size, the number of live
requests, the admission rule, the lookahead and the size of the page pool are; several of the
seeds have so few pages that requests are preempted and run again.  Nothing may stay held."""

import random

import pytest
import torch

from plain import llama_plain as P

pytestmark = pytest.mark.gpu

# (seeds 1, 10, 34, 45 and 47 preempt between 4 and 10 times; the others never)
SEEDS = (0, 1, 2, 3, 10, 34, 45, 47, 58, 59)


def draw(seed):
    """(config dict, [(prompt length, new tokens)], LLM settings) from one seed."""
    rng = random.Random(seed)
    hd = rng.choice((16, 32, 48, 64, 80, 128))
    kv = rng.choice((1, 2, 3, 4))
    heads = kv * rng.choice((1, 2, 4))
    width = 512 if rng.random() < 0.25 else 8 * rng.randint(4, 48)
    cfg = dict(architectures=["LlamaForCausalLM"], hidden_size=width,
               num_hidden_layers=rng.randint(1, 2), num_attention_heads=heads,
               num_key_value_heads=kv, head_dim=hd,
               intermediate_size=512 if width == 512 else 8 * rng.randint(5, 60),
               vocab_size=rng.randint(50, 600), rope_theta=10000.0, rms_norm_eps=1e-5,
               tie_word_embeddings=rng.random() < 0.5, max_position_embeddings=512,
               rope_interleaved=rng.random() < 0.5, torch_dtype="float32")
    page = rng.choice((8, 16, 64))
    reqs = []
    for _ in range(rng.randint(3, 14)):
        plen = rng.choice((1, 2, rng.randint(3, 30), rng.randint(30, 200)))
        new = rng.choice((1, 2, rng.randint(3, 20), rng.randint(20, 60)))
        reqs.append((plen, new))
    need = max(-(-(p + n) // page) * page for p, n in reqs)     # the longest request fits
    settings = dict(page_size=page, max_requests=rng.randint(1, 8),
                    max_batch_tokens=rng.choice((8, 16, 33, 64, 200, 2048)),
                    chunk_size=rng.choice((None, None, 2, 7, 32)),
                    admission=rng.choice(("optimistic", "optimistic", "reserve_full")),
                    lookahead=rng.random() < 0.7,
                    max_tokens=need * rng.choice((1, 1, 2, 3, 8)))
    return cfg, reqs, settings


@pytest.mark.parametrize("seed", SEEDS)
def test_random_serving(seed, tmp_path):
    from scratch_llm_b200.config import config_from_dict
    from scratch_llm_b200.engine import LLM, Request
    from scratch_llm_b200.sampling import SamplingParams
    from scratch_llm_b200.weights import write_random_model
    raw, reqs, settings = draw(seed)
    d = write_random_model(config_from_dict(raw), tmp_path / "m", seed=seed, std=0.02,
                           dtype="float32")
    cfg, w = P.read_model_dir(d)
    g = torch.Generator().manual_seed(seed)
    prompts = [torch.randint(0, raw["vocab_size"], (p,), generator=g).tolist() for p, _ in reqs]
    llm = LLM(d, dtype="float32", **settings)
    llm.runner.capture_padded_after = 2
    result = llm.serve([Request(i, p, SamplingParams(temperature=0.0, max_tokens=n))
                        for i, (p, (_, n)) in enumerate(zip(prompts, reqs))])
    for done, prompt, (_, n) in zip(result.completed, prompts, reqs):
        want = P.greedy(cfg, w, prompt, n)
        got = list(done.token_ids)
        if got != want:
            # two logits closer than 32-bit rounding may swap; anything else is a fault
            k = next(i for i, (a, b) in enumerate(zip(got, want)) if a != b)
            top = P.forward(cfg, w, prompt + want[:k])[-1].topk(2).values
            assert float(top[0] - top[1]) < 1e-5, (seed, raw, settings, done.request.request_id, k)
    if seed in (1, 10, 34, 45, 47):
        assert sum(c.n_preempted for c in result.completed) >= 4
    cache = llm.runner.cache
    assert not cache.requests
    assert all(grp.pool.n_free == grp.pool.n_pages for grp in cache.groups)
