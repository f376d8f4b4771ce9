#!/usr/bin/env python3
"""Headline benchmark: decode tokens per second at Llama-3-8B layer sizes with random weights
on one B200, plus the prefill of 2,048 tokens, the decode roofline and the end-to-end number
through the Python entry point.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--batch B] [--context T]

Prints ONE JSON line.  A "step" is one decode step of the whole batch.  ``value`` is timed on
the device with CUDA events around K steps of the step function plus the sampling kernel;
``e2e`` is the same through ``LLM.submit``/``LLM.step`` with host token ids in (pinned memory,
one copy per step) and the chosen tokens read back to the host every step.
"""

from __future__ import annotations

import argparse
import json
import statistics
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

from baseline.common import (SIZE_LABELS, SIZES_BY_NAME, ClockSampler, kv_bytes_per_token,
                             model_config, peaks, prefill_flops, spread, weight_bytes)

# the headline configuration: Llama-3-8B layer sizes
SIZES = SIZES_BY_NAME["llama-3-8b"]
#: up to this many layers the random model is written as a model folder and opened through
#: ``load_model`` like any user's; above, each tensor is drawn on the device when the model
#: asks for it (a folder of 16 GB takes minutes to draw on the CPU and to write)
FOLDER_MAX_LAYERS = 4


def build_engine(n_layers: int, capacity_tokens: int, max_requests: int, page_size: int,
                 sizes: dict | None = None):
    """The engine with random weights N(0, 0.02): (config, model, LLM, how the weights came)."""
    import tempfile

    import torch

    from scratch_llm_b200.config import config_from_dict
    from scratch_llm_b200.engine import LLM, build_model, load_model
    from scratch_llm_b200.kernels import ops
    from scratch_llm_b200.parts import BuildContext
    from scratch_llm_b200.weights import write_random_model
    from scratch_llm_b200.weights.random_init import random_tensors

    cfg = config_from_dict({**(sizes or SIZES), "num_hidden_layers": n_layers,
                            "architectures": ["LlamaForCausalLM"]})
    if n_layers <= FOLDER_MAX_LAYERS:
        # the way a user's model comes in: a folder with config.json and model.safetensors
        with tempfile.TemporaryDirectory() as tmp:
            write_random_model(cfg, tmp, seed=0)
            model = load_model(tmp, "bfloat16", verbose=False)
        how = "model folder (config.json + model.safetensors) through load_model"
    else:
        model = build_model(cfg)
        ops.prepare(model.head_dims(), verbose=False)
        specs = model.param_specs()
        device = torch.device("cuda", 0)

        class Lazy(dict):
            """Draws each tensor on the device when the model asks for it, so that the random
            weights never exist twice."""

            def __missing__(self, name):
                return random_tensors({name: specs[name]}, 0, torch.bfloat16, device=device)[name]

        model.load(Lazy(), BuildContext(dtype=torch.bfloat16, device=device))
        model.config = cfg
        how = "drawn on the device tensor by tensor (no folder of this size is written)"
    llm = LLM(model, max_tokens=capacity_tokens, page_size=page_size, max_requests=max_requests,
              max_batch_tokens=4096, chunk_size=2048)
    return cfg, model, llm, how


def time_serve(llm, cfg, n_requests: int, seed: int = 3):
    """The baseline's continuous-batching workload: `n_requests` requests with prompt lengths
    16-2048 and output lengths 16-512 (seeded, uniform), all queued at once, through LLM.serve
    (host token ids in and out).  Returns (generated tok/s, prompt tokens, generated tokens,
    seconds, steps)."""
    import random

    from scratch_llm_b200 import Request, SamplingParams

    rng = random.Random(seed)
    reqs = []
    for i in range(n_requests):
        n_in, n_out = rng.randint(16, 2048), rng.randint(16, 512)
        reqs.append(Request(f"s{i}", [rng.randrange(cfg.vocab_size) for _ in range(n_in)],
                            SamplingParams(temperature=0.0, max_tokens=n_out)))
    llm.serve(reqs[:4])          # warm-up: compiles nothing, but pages in the kernels
    res = llm.serve(reqs)
    n_out = sum(len(c.token_ids) for c in res.completed)
    n_in = sum(len(r.prompt_ids) for r in reqs)
    return n_out / res.wall_s, n_in, n_out, res.wall_s, res.stats.steps


def random_prompts(n: int, length: int, vocab: int, seed: int):
    import torch
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (length,), generator=g).tolist() for _ in range(n)]


def time_decode_device(llm, cfg, batch: int, context: int, steps: int, warmup: int, tag: str):
    """Device time of `steps` decode steps at `batch` x `context`: (ms/step over the whole
    timed region, launches, per-step times).  One CUDA event after every step."""
    import torch

    from scratch_llm_b200.engine import RowInput
    from scratch_llm_b200.kernels import ops

    runner = llm.runner
    ids = [f"{tag}{i}" for i in range(batch)]
    prompts = random_prompts(batch, context, cfg.vocab_size, seed=batch)
    for rid, p in zip(ids, prompts):
        assert runner.admit(rid)
    for start in range(0, batch, 2):   # prefill two prompts per step
        runner.step([RowInput(rid, p) for rid, p in zip(ids[start:start + 2],
                                                        prompts[start:start + 2])])
    nxt = random_prompts(warmup + steps, batch, cfg.vocab_size, seed=99)
    out = torch.empty(batch, dtype=torch.int32, device=runner.device)
    scratch = torch.zeros(ops.argmax_scratch_bytes(batch), dtype=torch.uint8, device=runner.device)

    def one(k):
        logits = runner.step([RowInput(rid, [nxt[k][i]], [0]) for i, rid in enumerate(ids)])
        ops.argmax(logits, out, scratch, batch)   # greedy choice, as LLM.step does

    for k in range(warmup):
        one(k)
    torch.cuda.synchronize()
    before = ops.launch_count + runner.replayed_kernels
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    marks[0].record()
    for k in range(steps):
        one(warmup + k)
        marks[k + 1].record()
    torch.cuda.synchronize()
    launches = ops.launch_count + runner.replayed_kernels - before
    for rid in ids:
        runner.release(rid)
    ops.check_kernel_errors()
    per_step = [marks[k].elapsed_time(marks[k + 1]) for k in range(steps)]
    return marks[0].elapsed_time(marks[-1]) / steps, launches, per_step


def time_decode_e2e(llm, cfg, batch: int, context: int, steps: int, warmup: int):
    """Wall time of `steps` scheduler steps through LLM.submit/LLM.step: (ms/step, h2d, d2h)."""
    import torch

    from scratch_llm_b200 import Request, SamplingParams

    prompts = random_prompts(batch, context, cfg.vocab_size, seed=1000 + batch)
    # room for the steps in which later prompts are still read while earlier requests decode
    params = SamplingParams(temperature=0.0,
                            max_tokens=warmup + steps + 8 + batch + batch * context // 1024)
    for i, p in enumerate(prompts):
        llm.submit(Request(f"e{i}", p, params))
    produced = set()
    while len(produced) < batch:            # prompts are read; every request has a first token
        produced.update(llm.step())
    for _ in range(warmup):
        llm.step()
    stager = llm.runner._stager
    torch.cuda.synchronize()
    h0, d0 = stager.bytes_uploaded, llm.sampler.bytes_read
    t0 = time.perf_counter()
    n_tokens = 0
    for _ in range(steps):
        n_tokens += len(llm.step())
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    h2d = (stager.bytes_uploaded - h0) / steps
    d2h = (llm.sampler.bytes_read - d0) / steps
    llm.abort_all()
    assert n_tokens == batch * steps
    return wall * 1e3 / steps, h2d, d2h


def time_prefill(llm, cfg, tokens: int, reps: int = 9):
    """Times of `reps` prompt steps of `tokens` tokens (after three untimed ones), each from an
    empty cache."""
    import torch

    from scratch_llm_b200.engine import RowInput

    runner = llm.runner
    prompt = random_prompts(1, tokens, cfg.vocab_size, seed=7)[0]
    times = []
    for r in range(reps + 3):
        assert runner.admit("prefill")
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        runner.step([RowInput("prefill", prompt, [tokens - 1])])
        e1.record()
        torch.cuda.synchronize()
        if r >= 3:
            times.append(e0.elapsed_time(e1))
        runner.release("prefill")
    return times


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=SIZES["num_hidden_layers"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=1024)
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--page-size", type=int, default=64)
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 and 64 points")
    ap.add_argument("--sizes", default="llama-3-8b", choices=sorted(SIZES_BY_NAME),
                    help="layer sizes (the default is the configuration the metric is quoted on)")
    ap.add_argument("--serve", type=int, default=0, metavar="N",
                    help="also run the continuous-batching workload with N requests")
    args = ap.parse_args()
    sizes = SIZES_BY_NAME[args.sizes]
    if args.layers == SIZES["num_hidden_layers"] and args.sizes != "llama-3-8b":
        args.layers = sizes["num_hidden_layers"]
    if args.gpus != 1:
        print(f"bench.py measures one GPU: this engine has no multi-GPU path (--gpus {args.gpus})")
        return 2
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        from baseline import reference_arm
        return reference_arm.main(args, sizes)

    import torch

    torch.cuda.set_device(0)
    pk = peaks()
    big = max(64, args.batch)
    capacity = big * (args.context + args.warmup + args.steps + 64) + 4096
    if args.serve:
        capacity = max(capacity, min(args.serve, 64) * 2600)
    cfg, model, llm, how = build_engine(args.layers, capacity, big + 1, args.page_size, sizes)

    with torch.no_grad():
        with ClockSampler(0) as clk_prefill:
            prefill_times = time_prefill(llm, cfg, args.prefill_tokens)
        with ClockSampler(0) as clk:
            ms, launches, per_step = time_decode_device(llm, cfg, args.batch, args.context,
                                                        args.steps, args.warmup, "d")
        with ClockSampler(0) as clk_e2e:
            e2e_ms, h2d, d2h = time_decode_e2e(llm, cfg, args.batch, args.context, args.steps,
                                               args.warmup)
        points = {}
        with ClockSampler(0) as clk_points:
            if not args.no_points:
                for b in (1, 64):
                    pms, _, _ = time_decode_device(llm, cfg, b, args.context,
                                                   max(8, args.steps // 2), args.warmup,
                                                   f"p{b}_")
                    points[f"decode_b{b}"] = round(b / pms * 1e3, 1)
        serve = None
        if args.serve:
            tok_s, n_in, n_out, seconds, steps = time_serve(llm, cfg, args.serve)
            serve = {"requests": args.serve, "generated_tok_s": round(tok_s, 1),
                     "prompt_tokens": n_in, "generated_tokens": n_out,
                     "seconds": round(seconds, 3), "steps": steps}

    prefill_ms = statistics.median(prefill_times)
    value = args.batch / ms * 1e3
    ctx_mid = args.context + args.warmup + args.steps / 2
    step_bytes = weight_bytes(sizes, args.layers) + \
        args.batch * ctx_mid * kv_bytes_per_token(sizes, args.layers)
    achieved = step_bytes / (ms * 1e-3) / 1e9
    flops = prefill_flops(sizes, args.layers, args.prefill_tokens)
    out = {
        "metric": f"decode tok/s at batch {args.batch} ({SIZE_LABELS[args.sizes]} sizes, "
                  "random weights)",
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms, 4), "spread": spread(per_step),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "impl": "ours",
        "config": model_config(args.sizes, sizes, args.layers, args.batch, args.context,
                               args.prefill_tokens, pk["source"]),
        "engine": {"page_size": args.page_size, "weights_from": how},
        "e2e": {"value": round(args.batch / e2e_ms * 1e3, 1), "unit": "tok/s",
                "ms_per_step": round(e2e_ms, 4), "h2d_bytes_per_step": int(h2d),
                "d2h_bytes_per_step": int(d2h)},
        "gpu_launches": launches,
        "prefill": {"value": round(args.prefill_tokens / prefill_ms * 1e3, 1),
                    "tokens": args.prefill_tokens, "ms": round(prefill_ms, 3),
                    "frac": round(flops / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                    "spread": spread(prefill_times)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "clocks": clk.summary,
        "clocks_regions": {"prefill": clk_prefill.summary, "e2e": clk_e2e.summary,
                           "points": clk_points.summary},
    }
    if serve is not None:
        out["serve"] = serve
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
