"""``bench.py --impl reference``: the unmodified reference, through its own public classes, at
the configuration of the bench line.

What runs is the reference's fastest stock decode path: ``TransformerLM`` in bfloat16,
``PagedKVCache(use_kernel=True)`` filled through ``PrefillView``, one decode step captured and
replayed by ``CudaGraphDecoder`` (src/scratch_llm/serving/cudagraph.py:31-96; the recipe is the
reference's own bench/cudagraph_decode.py:34-57, 91-103).  Where its Triton kernel cannot be
imported or compiled, the eager decode over the same paged cache (the loop of
bench/cudagraph_decode.py:60-69 with ``use_kernel=False``) runs instead, and the line says so.
Prefill is the reference's stock forward over a ``PrefillView`` (logits at every position, as
its model computes them).  Nothing of ``scratch_llm_b200`` is imported here.
"""

from __future__ import annotations

import json
import random
import sys
import time
from pathlib import Path

from .common import (SIZE_LABELS, ClockSampler, kv_bytes_per_token, model_config, peaks,
                     prefill_flops, spread, weight_bytes)

REF = Path(__file__).resolve().parent / "_ref"
PREFILL_GROUP = 8      # prompts per PrefillView forward (its eager attention holds all scores)


def unavailable(why: str) -> int:
    print(json.dumps({"impl": "reference", "unavailable": " ".join(why.split())[:400]}))
    return 0


def _prompts(n: int, length: int, vocab: int, seed: int) -> list[list[int]]:
    rng = random.Random(seed)
    return [[rng.randrange(vocab) for _ in range(length)] for _ in range(n)]


class _Arm:
    def __init__(self, sizes: dict, n_layers: int) -> None:
        import torch
        from scratch_llm.model import ModelConfig, TransformerLM

        self.torch = torch
        self.device = torch.device("cuda", 0)
        d, h = sizes["hidden_size"], sizes["num_attention_heads"]
        if sizes["head_dim"] * h != d:
            raise ValueError("the reference derives head_dim = d_model / n_heads")
        self.cfg = ModelConfig(vocab_size=sizes["vocab_size"], d_model=d, n_layers=n_layers,
                               n_heads=h, n_kv_heads=sizes["num_key_value_heads"],
                               d_ff=sizes["intermediate_size"],
                               context_length=sizes["max_position_embeddings"],
                               rope_theta=sizes["rope_theta"],
                               tie_embeddings=sizes["tie_word_embeddings"])
        torch.manual_seed(0)
        with torch.device(self.device):
            model = TransformerLM(self.cfg)      # its own construction and init, on the device
        model = model.to(torch.bfloat16).eval()
        with torch.no_grad():
            for p in model.parameters():
                if p.dim() == 2:
                    p.normal_(0.0, 0.02)         # the bench line's weights: N(0, 0.02)
        self.model = model
        self.path = "CudaGraphDecoder over PagedKVCache(use_kernel=True)"
        self.why_eager = None
        try:
            from scratch_llm.kernels.attention.dispatch import paged_decode_attention  # noqa: F401
        except Exception as exc:   # Triton missing or broken: the reference's eager decode
            self.why_eager = f"{type(exc).__name__}: {exc}"
            self.path = "eager decode over PagedKVCache (gather view)"

    # ------------------------------------------------------------------------------ cache

    def filled_cache(self, batch: int, context: int, room: int, seed: int):
        """A paged cache with ``batch`` prompts of ``context`` tokens read, and the first
        greedy token of each."""
        torch = self.torch
        from scratch_llm.model import PagedKVCache, PrefillView

        block = PagedKVCache.BLOCK
        per_row = -(-(context + room) // block)
        cache = PagedKVCache(n_layers=self.cfg.n_layers, n_slots=batch,
                             n_kv_heads=self.cfg.kv_heads, max_ctx=self.cfg.context_length,
                             head_dim=self.cfg.head_dim, n_blocks=batch * per_row + 1,
                             device=self.device, dtype=torch.bfloat16)
        cache.use_kernel = self.why_eager is None
        prompts = _prompts(batch, context, self.cfg.vocab_size, seed)
        first = torch.empty(batch, dtype=torch.long, device=self.device)
        with torch.no_grad():
            for lo in range(0, batch, PREFILL_GROUP):
                slots = list(range(lo, min(batch, lo + PREFILL_GROUP)))
                x = torch.tensor([prompts[s] for s in slots], dtype=torch.long,
                                 device=self.device)
                logits = self.model(x, PrefillView(cache, slots, [context] * len(slots)))
                cache.mirror_admit(slots, [context] * len(slots))
                first[lo:lo + len(slots)] = logits[:, context - 1].argmax(dim=-1)
                del logits
        return cache, first

    def stepper(self, cache):
        """step(last_tokens (B,) long on the device) -> next greedy tokens (B,)."""
        torch = self.torch
        if cache.use_kernel:
            from scratch_llm.serving.cudagraph import CudaGraphDecoder
            dec = CudaGraphDecoder(self.model, cache)
            try:
                dec.capture()
                return dec.step
            except Exception as exc:
                if "CUDA error" in str(exc) or "illegal" in str(exc):
                    raise
                self.why_eager = f"{type(exc).__name__}: {exc}"
                self.path = "eager decode over PagedKVCache (gather view)"
                cache.use_kernel = False

        @torch.no_grad()
        def eager(last):
            cache.pre_decode_reserve()
            logits = self.model(last.unsqueeze(1), cache)
            nxt = logits[:, -1].argmax(dim=-1)
            cache.mirror_advance()
            return nxt
        return eager

    # ----------------------------------------------------------------------------- timing

    def time_decode(self, batch: int, context: int, steps: int, warmup: int, seed: int):
        """Device time of ``steps`` greedy decode steps: (ms/step, per-step times)."""
        torch = self.torch
        cache, last = self.filled_cache(batch, context, warmup + steps + 8, seed)
        step = self.stepper(cache)
        for _ in range(warmup):
            last = step(last)
        torch.cuda.synchronize()
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        marks[0].record()
        for k in range(steps):
            last = step(last)
            marks[k + 1].record()
        torch.cuda.synchronize()
        per_step = [marks[k].elapsed_time(marks[k + 1]) for k in range(steps)]
        return marks[0].elapsed_time(marks[-1]) / steps, per_step

    def time_decode_e2e(self, batch: int, context: int, steps: int, warmup: int, seed: int):
        """Wall time with host token ids in (pinned memory, one copy per step) and the chosen
        tokens read back to the host every step: (ms/step, bytes up, bytes down)."""
        torch = self.torch
        cache, first = self.filled_cache(batch, context, warmup + steps + 8, seed)
        step = self.stepper(cache)
        staging = torch.empty(batch, dtype=torch.long).pin_memory()
        host = first.tolist()

        def one(tokens: list[int]) -> list[int]:
            staging.copy_(torch.tensor(tokens, dtype=torch.long))
            return step(staging.to(self.device, non_blocking=True)).tolist()

        for _ in range(warmup):
            host = one(host)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            host = one(host)
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        return wall * 1e3 / steps, batch * 8, batch * 8

    def time_prefill(self, tokens: int, reps: int = 9):
        torch = self.torch
        from scratch_llm.model import PagedKVCache, PrefillView

        prompt = torch.tensor(_prompts(1, tokens, self.cfg.vocab_size, 7), dtype=torch.long,
                              device=self.device)
        times = []
        for r in range(reps + 3):
            cache = PagedKVCache(n_layers=self.cfg.n_layers, n_slots=1,
                                 n_kv_heads=self.cfg.kv_heads, max_ctx=self.cfg.context_length,
                                 head_dim=self.cfg.head_dim,
                                 n_blocks=-(-tokens // PagedKVCache.BLOCK) + 1,
                                 device=self.device, dtype=torch.bfloat16)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            with torch.no_grad():
                logits = self.model(prompt, PrefillView(cache, [0], [tokens]))
                logits[0, tokens - 1].argmax()
            e1.record()
            torch.cuda.synchronize()
            if r >= 3:
                times.append(e0.elapsed_time(e1))
            del logits, cache
        return times


def main(args, sizes: dict) -> int:
    if not (REF / "scratch_llm" / "model.py").is_file():
        return unavailable("baseline/_ref does not hold the reference package: run "
                           "baseline/install_reference.py with a checkout of it (the offline "
                           "pip install needs its build backend hatchling, which the "
                           "wheelhouse does not have)")
    sys.path.insert(0, str(REF))
    try:
        import torch
        if not torch.cuda.is_available():
            return unavailable("no CUDA device")
        torch.cuda.set_device(0)
        arm = _Arm(sizes, args.layers)
        pk = peaks()
        with ClockSampler(0) as clk_prefill:
            prefill_times = arm.time_prefill(args.prefill_tokens)
        with ClockSampler(0) as clk:
            ms, per_step = arm.time_decode(args.batch, args.context, args.steps, args.warmup,
                                           seed=args.batch)
        with ClockSampler(0) as clk_e2e:
            e2e_ms, h2d, d2h = arm.time_decode_e2e(args.batch, args.context, args.steps,
                                                   args.warmup, seed=1000 + args.batch)
        points = {}
        with ClockSampler(0) as clk_points:
            if not args.no_points:
                for b in (1, 64):
                    pms, _ = arm.time_decode(b, args.context, max(8, args.steps // 2),
                                             args.warmup, seed=b)
                    points[f"decode_b{b}"] = round(b / pms * 1e3, 1)
    except Exception as exc:   # the reference's own code failed here: say how, run nothing again
        return unavailable(f"the reference failed on this box: {type(exc).__name__}: {exc}")

    import statistics
    prefill_ms = statistics.median(prefill_times)
    ctx_mid = args.context + args.warmup + args.steps / 2
    step_bytes = weight_bytes(sizes, args.layers) + \
        args.batch * ctx_mid * kv_bytes_per_token(sizes, args.layers)
    achieved = step_bytes / (ms * 1e-3) / 1e9
    flops = prefill_flops(sizes, args.layers, args.prefill_tokens)
    out = {
        "metric": f"decode tok/s at batch {args.batch} ({SIZE_LABELS[args.sizes]} sizes, "
                  "random weights)",
        "value": round(args.batch / ms * 1e3, 1), "unit": "tok/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 4),
        "spread": spread(per_step), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "reference",
        "config": model_config(args.sizes, sizes, args.layers, args.batch, args.context,
                               args.prefill_tokens, pk["source"]),
        "engine": {"path": arm.path, "page_size": 16,
                   **({"eager_because": arm.why_eager[:200]} if arm.why_eager else {})},
        "e2e": {"value": round(args.batch / e2e_ms * 1e3, 1), "unit": "tok/s",
                "ms_per_step": round(e2e_ms, 4), "h2d_bytes_per_step": int(h2d),
                "d2h_bytes_per_step": int(d2h)},
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
    print(json.dumps(out))
    return 0
