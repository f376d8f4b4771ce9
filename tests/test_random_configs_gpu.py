"""Configurations drawn at random (fixed seeds): every size and option of the architecture
changes from draw to draw, within what config.json allows, and the engine must give the plain
implementation's logits for whole prompts and for a mixed trace, in 32-bit and in bfloat16,
with free cache pages holding NaN.  The four named configurations of the other tests were
chosen by hand; these were not.  Weights are N(0, 0.02) as there, and so are the tolerances
(an absolute tolerance belongs to a scale of the logits)."""

import random

import pytest
import torch

import trace_util as T
from plain import llama_plain as P

pytestmark = pytest.mark.gpu

# head sizes whose attention kernels the build step prepares (another size would be compiled
# on first use, which is covered elsewhere and takes a minute each)
HEAD_SIZES = (16, 32, 48, 64, 80, 128)
TOL = {"float32": dict(rtol=2e-5, atol=5e-6), "bfloat16": dict(rtol=3e-2, atol=3e-2)}


def draw(seed):
    """(config dict, page size, prompt lengths) from one seed."""
    rng = random.Random(seed)
    hd = rng.choice(HEAD_SIZES)
    kv = rng.choice((1, 2, 3, 4))
    heads = kv * rng.choice((1, 2, 3, 4, 8))
    # the width need not be heads x head size, nor a power of two; multiples of 8 keep rows of
    # bfloat16 weights on 16 bytes, which the loader's products ask for
    width = 8 * rng.randint(4, 96) if rng.random() < 0.7 else heads * hd
    ff = 8 * rng.randint(5, 200)
    cfg = dict(architectures=["LlamaForCausalLM"], hidden_size=width,
               num_hidden_layers=rng.randint(1, 4), num_attention_heads=heads,
               num_key_value_heads=kv, head_dim=hd, intermediate_size=ff,
               vocab_size=rng.randint(50, 1500),
               rope_theta=rng.choice((100.0, 10000.0, 500000.0, 1234.5)),
               rms_norm_eps=rng.choice((1e-6, 1e-5, 1e-3, 3e-4)),
               tie_word_embeddings=rng.random() < 0.5, max_position_embeddings=512,
               rope_interleaved=rng.random() < 0.5, torch_dtype="float32")
    page = rng.choice((8, 16, 32, 64))
    lengths = [rng.choice((1, 2, rng.randint(3, 40), rng.randint(40, 300))) for _ in range(6)]
    lengths[rng.randrange(6)] = rng.randint(200, 420)
    return cfg, page, lengths


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(16))
def test_random_configuration(seed, dtype, tmp_path):
    from scratch_llm_b200.config import config_from_dict
    from scratch_llm_b200.engine import ModelRunner, load_model
    from scratch_llm_b200.kernels import ops
    from scratch_llm_b200.weights import write_random_model
    raw, page, lengths = draw(seed)
    config = config_from_dict(raw)
    d = write_random_model(config, tmp_path / "m", seed=seed, std=0.02, dtype="float32")
    cfg, w = P.read_model_dir(d)
    if dtype == "bfloat16":
        w = {k: v.to(torch.bfloat16).float() for k, v in w.items()}
    reqs = T.make_requests(cfg["vocab_size"], lengths, seed=seed)
    want = {rid: P.forward(cfg, w, toks) for rid, toks in reqs.items()}
    model = load_model(d, dtype, verbose=False)
    for way in (T.whole, T.mixed):
        steps = way(reqs)
        peak = T.peak_tokens(steps, round_to=max(64, page))
        runner = ModelRunner(model, page, -(-peak // page), 4, poison_free_pages=True)
        runner.capture_padded_after = 2
        with torch.no_grad():
            got = T.run_in_process(runner, steps)
        ops.check_kernel_errors()
        assert len(got) == sum(lengths)
        for (rid, pos), row in sorted(got.items()):
            torch.testing.assert_close(
                row, want[rid][pos], **TOL[dtype],
                msg=lambda m: f"seed {seed} {raw} page {page} {way.__name__} request {rid} "
                              f"position {pos}: {m}")
        assert not runner.cache.requests and all(
            g.pool.n_free == g.pool.n_pages for g in runner.cache.groups)
