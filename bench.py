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
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# the headline configuration: Llama-3-8B layer sizes
SIZES = dict(hidden_size=4096, num_hidden_layers=32, num_attention_heads=32,
             num_key_value_heads=8, head_dim=128, intermediate_size=14336, vocab_size=128256,
             rope_theta=500000.0, rms_norm_eps=1e-5, tie_word_embeddings=False,
             max_position_embeddings=8192, torch_dtype="bfloat16")
# the other two configurations at full size that the baseline names; chosen with --sizes
SIZES_BY_NAME = {
    "llama-3-8b": SIZES,
    "llama-3.2-1b": dict(hidden_size=2048, num_hidden_layers=16, num_attention_heads=32,
                         num_key_value_heads=8, head_dim=64, intermediate_size=8192,
                         vocab_size=128256, rope_theta=500000.0, rms_norm_eps=1e-5,
                         tie_word_embeddings=True, max_position_embeddings=8192,
                         torch_dtype="bfloat16"),
    "llama-2-13b": dict(hidden_size=5120, num_hidden_layers=40, num_attention_heads=40,
                        num_key_value_heads=40, head_dim=128, intermediate_size=13824,
                        vocab_size=32000, rope_theta=10000.0, rms_norm_eps=1e-5,
                        tie_word_embeddings=False, max_position_embeddings=4096,
                        torch_dtype="bfloat16"),
}
SIZE_LABELS = {"llama-3-8b": "Llama-3-8B", "llama-3.2-1b": "Llama-3.2-1B",
               "llama-2-13b": "Llama-2-13B"}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            raw = json.loads(path.read_text())
            return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]),
                    "bf16_tflops_sustained": float(raw.get("bf16_tflops_sustained",
                                                           raw["bf16_tflops"])),
                    "source": "measured"}
        except (KeyError, ValueError, json.JSONDecodeError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int) -> None:
        self.index, self.proc = index, None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        self.summary = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out = ""
        clocks, reasons, mx = [], set(), None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) != 6:
                continue
            try:
                clocks.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for name, val in zip(names, parts[2:]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if clocks:
            self.summary = {"sm_mhz": statistics.median(clocks), "sm_max_mhz": mx,
                            "reasons": sorted(reasons), "samples": len(clocks)}


def reference_arm() -> int:
    # The one offline install this arm may use,
    #   python -m pip install --no-index --no-build-isolation --find-links /opt/wheelhouse
    #       --target baseline/_ref <reference>
    # fails: the reference's build backend (hatchling) is not in the wheelhouse.
    ref = ROOT / "baseline" / "_ref" / "scratch_llm"
    why = ("offline install failed: the reference's build backend 'hatchling' is not in the "
           "wheelhouse (ModuleNotFoundError), so baseline/_ref is empty")
    if ref.is_dir():
        why = ("baseline/_ref holds the reference, but it has no engine for Llama-3-8B sizes "
               "on one call: not wired")
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def build_engine(n_layers: int, capacity_tokens: int, max_requests: int, page_size: int,
                 sizes: dict | None = None):
    import torch

    from scratch_llm_b200.config import config_from_dict
    from scratch_llm_b200.engine import LLM, build_model
    from scratch_llm_b200.kernels import ops
    from scratch_llm_b200.parts import BuildContext
    from scratch_llm_b200.weights.random_init import random_tensors

    cfg = config_from_dict({**(sizes or SIZES), "num_hidden_layers": n_layers,
                            "architectures": ["LlamaForCausalLM"]})
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
    llm = LLM(model, max_tokens=capacity_tokens, page_size=page_size, max_requests=max_requests,
              max_batch_tokens=4096, chunk_size=2048)
    return cfg, model, llm


def weight_bytes(cfg) -> int:
    """Bytes of weights a decode step reads (a tied output matrix is still read; the embedding
    table is not: a step gathers a few rows of it)."""
    d, f, v = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    hq, hk = cfg.num_attention_heads * cfg.head_size, cfg.kv_heads * cfg.head_size
    per_layer = (hq + 2 * hk) * d + d * hq + 3 * f * d
    return 2 * (cfg.num_hidden_layers * per_layer + v * d) + 4 * (2 * cfg.num_hidden_layers + 1) * d


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


def prefill_flops(cfg, t: int) -> float:
    d, f, v = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    hq, hk = cfg.num_attention_heads * cfg.head_size, cfg.kv_heads * cfg.head_size
    linear = 2.0 * t * cfg.num_hidden_layers * ((hq + 2 * hk) * d + d * hq + 3 * f * d)
    attn = cfg.num_hidden_layers * 4.0 * hq * (t * (t + 1) / 2)   # causal half of QK^T and PV
    return linear + attn + 2.0 * v * d   # the output matrix on the one wanted row


def random_prompts(n: int, length: int, vocab: int, seed: int):
    import torch
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (length,), generator=g).tolist() for _ in range(n)]


def time_decode_device(llm, cfg, batch: int, context: int, steps: int, warmup: int, tag: str):
    """Device time of `steps` decode steps at `batch` x `context`; returns (ms/step, launches)."""
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
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for k in range(warmup, warmup + steps):
        one(k)
    e1.record()
    torch.cuda.synchronize()
    launches = ops.launch_count + runner.replayed_kernels - before
    for rid in ids:
        runner.release(rid)
    return e0.elapsed_time(e1) / steps, launches


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


def time_prefill(llm, cfg, tokens: int, reps: int = 3):
    import torch

    from scratch_llm_b200.engine import RowInput

    runner = llm.runner
    prompt = random_prompts(1, tokens, cfg.vocab_size, seed=7)[0]
    times = []
    for r in range(reps + 2):
        assert runner.admit("prefill")
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        runner.step([RowInput("prefill", prompt, [tokens - 1])])
        e1.record()
        torch.cuda.synchronize()
        if r >= 2:
            times.append(e0.elapsed_time(e1))
        runner.release("prefill")
    return statistics.median(times)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
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
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print(f"bench.py measures one GPU: this engine has no multi-GPU path (--gpus {args.gpus})")
        return 2
    args.warmup = max(args.warmup, 3)

    import torch

    torch.cuda.set_device(0)
    pk = peaks()
    big = max(64, args.batch)
    capacity = big * (args.context + args.warmup + args.steps + 64) + 4096
    if args.serve:
        capacity = max(capacity, min(args.serve, 64) * 2600)
    cfg, model, llm = build_engine(args.layers, capacity, big + 1, args.page_size, sizes)

    with torch.no_grad():
        prefill_ms = time_prefill(llm, cfg, args.prefill_tokens)
        with ClockSampler(0) as clk:
            ms, launches = time_decode_device(llm, cfg, args.batch, args.context, args.steps,
                                              args.warmup, "d")
        e2e_ms, h2d, d2h = time_decode_e2e(llm, cfg, args.batch, args.context, args.steps,
                                           args.warmup)
        points = {}
        if not args.no_points:
            for b in (1, 64):
                pms, _ = time_decode_device(llm, cfg, b, args.context, max(8, args.steps // 2),
                                            args.warmup, f"p{b}_")
                points[f"decode_b{b}"] = round(b / pms * 1e3, 1)
        serve = None
        if args.serve:
            tok_s, n_in, n_out, seconds, steps = time_serve(llm, cfg, args.serve)
            serve = {"requests": args.serve, "generated_tok_s": round(tok_s, 1),
                     "prompt_tokens": n_in, "generated_tokens": n_out,
                     "seconds": round(seconds, 3), "steps": steps}

    value = args.batch / ms * 1e3
    ctx_mid = args.context + args.warmup + args.steps / 2
    kv_bytes = args.batch * ctx_mid * 2 * cfg.kv_heads * cfg.head_size * 2 * cfg.num_hidden_layers
    step_bytes = weight_bytes(cfg) + kv_bytes
    achieved = step_bytes / (ms * 1e-3) / 1e9
    flops = prefill_flops(cfg, args.prefill_tokens)
    out = {
        "metric": f"decode tok/s at batch {args.batch} ({SIZE_LABELS[args.sizes]} sizes, "
                  "random weights)",
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "ours",
        "config": {"model": f"{args.sizes}-sizes", "layers": cfg.num_hidden_layers,
                   "layers_of_config": sizes["num_hidden_layers"], "hidden": cfg.hidden_size,
                   "heads": cfg.num_attention_heads, "kv_heads": cfg.kv_heads,
                   "head_dim": cfg.head_size, "intermediate": cfg.intermediate_size,
                   "vocab": cfg.vocab_size, "global_batch": args.batch, "seq_len": args.context,
                   "prefill_tokens": args.prefill_tokens, "page_size": args.page_size,
                   "parallelism": "single-gpu", "weights": "random N(0,0.02)",
                   "l2": "inputs larger than L2 (weights read once per step)",
                   "peaks": pk["source"]},
        "e2e": {"value": round(args.batch / e2e_ms * 1e3, 1), "unit": "tok/s",
                "ms_per_step": round(e2e_ms, 4), "h2d_bytes_per_step": int(h2d),
                "d2h_bytes_per_step": int(d2h)},
        "gpu_launches": launches,
        "prefill": {"value": round(args.prefill_tokens / prefill_ms * 1e3, 1),
                    "tokens": args.prefill_tokens, "ms": round(prefill_ms, 3),
                    "frac": round(flops / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "clocks": clk.summary,
    }
    if serve is not None:
        out["serve"] = serve
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
