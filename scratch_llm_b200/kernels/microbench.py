"""Times single kernels of the engine with CUDA events, beside the library product where one
exists, at sizes given on the command line.

    python -m scratch_llm_b200.kernels.microbench linear --tokens 16 64 128 256 [--n 28672]
        [--k 4096] [--swiglu]
    python -m scratch_llm_b200.kernels.microbench attn_prefill --tokens 2048 4096 [--page 64]
    python -m scratch_llm_b200.kernels.microbench attn_decode --batch 8 64 [--context 1024]
    python -m scratch_llm_b200.kernels.microbench sample --rows 1 8 64 [--vocab 128256]

Method: ``--inner`` launches (16 by default) are recorded into a CUDA graph, so that no
launch waits for the host; after warm-up each replay is timed by an event pair on the
launching stream, and the median over the replays of (replay time / launches) is reported.
Products rotate through enough copies of the weight to
exceed the L2 cache several times over (``--rotate-mb``, 512 MB by default), so that every
launch streams its weight from memory as a decode step does.  Fractions are of the measured
copy bandwidth and of the measured bf16 product rate of this pool's GPUs when the file that
holds them lies at the repository's root, else of the fallback figures.

The reference's harness reports the median with p10/p90 after warm-up in the same manner
(src/scratch_llm/bench/harness.py:52-91).
"""

from __future__ import annotations

import argparse
import json
import math
import statistics
from pathlib import Path

import torch

from . import ops

ROOT = Path(__file__).resolve().parent.parent.parent


def _peaks() -> tuple[float, float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            raw = json.loads(path.read_text())
            return float(raw["hbm_gbs"]), float(raw["bf16_tflops"]), "measured"
        except (KeyError, ValueError, json.JSONDecodeError):
            pass
    return 6650.0, 1590.0, "fallback"


INNER = 16   # launches per timed graph replay (set by --inner)


def time_us(launch, reps: int, warmup: int = 3) -> dict:
    """``launch(i)`` is recorded for i = 0 .. INNER-1 into one graph; returns the median / p10 /
    p90 over ``reps`` replays of the time per launch, in microseconds."""
    for i in range(2):
        launch(i)               # whatever a first call sets up must not be recorded
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        graph.capture_begin()
        for i in range(INNER):
            launch(i)
        graph.capture_end()
    torch.cuda.current_stream().wait_stream(stream)
    for _ in range(warmup):
        graph.replay()
    torch.cuda.synchronize()
    marks = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
             for _ in range(reps)]
    for a, b in marks:
        a.record()
        graph.replay()
        b.record()
    torch.cuda.synchronize()
    t = sorted(a.elapsed_time(b) * 1e3 / INNER for a, b in marks)
    return {"median_us": round(statistics.median(t), 2), "p10_us": round(t[len(t) // 10], 2),
            "p90_us": round(t[(9 * len(t)) // 10], 2)}


def bench_linear(args) -> list[dict]:
    from ..parts.linear import Linear
    hbm, tf, src = _peaks()
    n, k = args.n, args.k
    copies = max(2, -(-args.rotate_mb * (1 << 20) // (n * k * 2)))
    g = torch.Generator(device="cuda").manual_seed(0)
    weights = [(torch.randn(n, k, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
               for _ in range(copies)]
    layers = [Linear(w) for w in weights]
    out = []
    for m in args.tokens:
        x = (torch.randn(m, k, device="cuda", generator=g)).to(torch.bfloat16)
        half = n // 2
        if args.swiglu:
            ours = time_us(lambda i: layers[i % copies].swiglu(x), args.reps)
            buf = torch.empty(m, half, dtype=torch.bfloat16, device="cuda")
            lib = time_us(lambda i: ops.swiglu(torch.mm(x, weights[i % copies].t()), buf),
                          args.reps)
        else:
            ours = time_us(lambda i: layers[i % copies](x), args.reps)
            lib = time_us(lambda i: torch.mm(x, weights[i % copies].t()), args.reps)
        byts = n * k * 2 + m * k * 2 + m * (half if args.swiglu else n) * 2
        flops = 2.0 * m * n * k
        row = {"kernel": "linear+swiglu" if args.swiglu else "linear", "tokens": m, "n": n, "k": k,
               "engine": ours, "library": lib,
               "engine_gbs": round(byts / ours["median_us"] / 1e3, 1),
               "engine_hbm_frac": round(byts / ours["median_us"] / 1e3 / hbm, 3),
               "engine_tflops": round(flops / ours["median_us"] / 1e6, 1),
               "engine_tensor_frac": round(flops / ours["median_us"] / 1e6 / tf, 3),
               "library_gbs": round(byts / lib["median_us"] / 1e3, 1), "peaks": src}
        out.append(row)
    return out


def _paged(batch: int, context: int, g_heads: int, hd: int, page: int, gen):
    per = -(-context // page)
    pages = torch.randn(batch * per, 2, g_heads, page, hd, device="cuda", generator=gen
                        ).to(torch.bfloat16)
    table = torch.randperm(batch * per, device="cuda", generator=gen).to(torch.int32).view(batch, per)
    return pages, table.contiguous()


def bench_attn_prefill(args) -> list[dict]:
    hbm, tf, src = _peaks()
    H, G, hd, page = args.heads, args.kv_heads, args.head_dim, args.page
    ops.prepare([hd], verbose=False)
    gen = torch.Generator(device="cuda").manual_seed(0)
    out = []
    for t in args.tokens:
        pages, table = _paged(1, t, G, hd, page, gen)
        q = torch.randn(t, H * hd, device="cuda", generator=gen).to(torch.bfloat16)
        o = torch.empty_like(q)
        row_start = torch.tensor([0, t], dtype=torch.int32, device="cuda")
        pos0 = torch.zeros(1, dtype=torch.int32, device="cuda")
        scale = 1.0 / math.sqrt(hd)
        flops = 4.0 * H * hd * (t * (t + 1) / 2)
        row = {"kernel": "attn_prefill", "tokens": t, "heads": H, "kv_heads": G, "head_dim": hd,
               "page": page, "peaks": src}
        if ops.attention_tc_supports(H, G, hd, page, None):
            for name, two in (("tcgen05", None), ("tcgen05_two_tiles", True),
                              ("tcgen05_one_tile", False)):
                if two and hd > 128:
                    continue
                ops.attention_tc_set_two_tiles(hd, two)
                r = time_us(lambda i: ops.attention_tc(q, pages, table, page, row_start, pos0, o,
                                                       None, 1, t, H, G, hd, scale), args.reps)
                assert ops.attention_tc_error(hd) == 0
                row[name] = r
                row[name + "_tflops"] = round(flops / r["median_us"] / 1e6, 1)
                row[name + "_tensor_frac"] = round(flops / r["median_us"] / 1e6 / tf, 3)
            ops.attention_tc_set_two_tiles(hd, None)
        r = time_us(lambda i: ops.attention_mma(q, pages, table, page, row_start, pos0, o, None, 1,
                                                t, H, G, hd, scale, None, split=False), args.reps)
        row["mma_sync"] = r
        row["mma_sync_tflops"] = round(flops / r["median_us"] / 1e6, 1)
        out.append(row)
    return out


def bench_attn_decode(args) -> list[dict]:
    from ..parts.attention import decode_splits
    hbm, tf, src = _peaks()
    H, G, hd, page, ctx = args.heads, args.kv_heads, args.head_dim, args.page, args.context
    ops.prepare([hd], verbose=False)
    gen = torch.Generator(device="cuda").manual_seed(0)
    out = []
    for b in args.batch:
        # several copies of the keys and values, taken in turn, so that they come from memory
        byts = b * ctx * 2 * G * hd * 2
        copies = max(2, -(-512 * (1 << 20) // byts))
        caches = [_paged(b, ctx, G, hd, page, gen) for _ in range(copies)]
        q = torch.randn(b, H * hd, device="cuda", generator=gen).to(torch.bfloat16)
        o = torch.empty_like(q)
        row_start = torch.arange(b + 1, dtype=torch.int32, device="cuda")
        pos0 = torch.full((b,), ctx - 1, dtype=torch.int32, device="cuda")
        n_splits = decode_splits(b * G * (-(-(H // G) // 16)), ctx,
                                 ops.attention_decode_slots(hd))
        scratch = torch.empty(max(1, ops.attention_mma_scratch_floats(b, H, hd, n_splits)),
                              dtype=torch.float32, device="cuda")

        def launch(i):
            pages, table = caches[i % copies]
            ops.attention_mma(q, pages, table, page, row_start, pos0, o, None, b, 1, H, G, hd,
                              1.0 / math.sqrt(hd), None, split=True, n_splits=n_splits,
                              scratch=scratch)
        r = time_us(launch, args.reps)
        byts = b * ctx * 2 * G * hd * 2
        out.append({"kernel": "attn_decode", "batch": b, "context": ctx, "splits": n_splits,
                    "page": page, "engine": r, "kv_mb": round(byts / 1e6, 1),
                    "engine_gbs": round(byts / r["median_us"] / 1e3, 1),
                    "engine_hbm_frac": round(byts / r["median_us"] / 1e3 / hbm, 3), "peaks": src})
    return out


def bench_sample(args) -> list[dict]:
    """The choice of the next token over a vocabulary of ``--vocab`` entries: greedy (the argmax
    kernel), a draw at a temperature, a draw from a nucleus, and the latter with the drawn
    token's log-probability."""
    gen = torch.Generator(device="cuda").manual_seed(0)
    out = []
    for n in args.rows:
        logits = torch.randn(n, args.vocab, device="cuda", generator=gen) * 3
        tok = torch.empty(n, dtype=torch.int32, device="cuda")
        temp = torch.full((n,), 0.8, device="cuda")
        top = torch.full((n,), 0.9, device="cuda")
        seed = torch.arange(n, dtype=torch.int64, device="cuda")
        ctr = torch.zeros(n, dtype=torch.int64, device="cuda")
        lp = torch.empty(n, device="cuda")
        scratch = torch.zeros(ops.argmax_scratch_bytes(n), dtype=torch.uint8, device="cuda")
        out.append({
            "kernel": "sample", "rows": n, "vocab": args.vocab,
            "argmax": time_us(lambda i: ops.argmax(logits, tok, scratch, n), args.reps),
            "temperature": time_us(lambda i: ops.sample(logits, tok, temp, None, seed, ctr),
                                   args.reps),
            "nucleus": time_us(lambda i: ops.sample(logits, tok, temp, top, seed, ctr), args.reps),
            "nucleus_logprob": time_us(lambda i: ops.sample(logits, tok, temp, top, seed, ctr, lp),
                                       args.reps)})
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    sub = ap.add_subparsers(dest="what", required=True)
    p = sub.add_parser("linear")
    p.add_argument("--tokens", type=int, nargs="+", default=[1, 8, 16, 64, 128, 256])
    p.add_argument("--n", type=int, default=28672)
    p.add_argument("--k", type=int, default=4096)
    p.add_argument("--swiglu", action="store_true")
    p.add_argument("--rotate-mb", type=int, default=512)
    p = sub.add_parser("attn_prefill")
    p.add_argument("--tokens", type=int, nargs="+", default=[2048, 4096])
    p = sub.add_parser("attn_decode")
    p.add_argument("--batch", type=int, nargs="+", default=[8, 64])
    p.add_argument("--context", type=int, default=1024)
    p = sub.add_parser("sample")
    p.add_argument("--rows", type=int, nargs="+", default=[1, 8, 64])
    p.add_argument("--vocab", type=int, default=128256)
    for name in ("attn_prefill", "attn_decode"):
        q = sub.choices[name]
        q.add_argument("--heads", type=int, default=32)
        q.add_argument("--kv-heads", type=int, default=8)
        q.add_argument("--head-dim", type=int, default=128)
        q.add_argument("--page", type=int, default=64)
    for q in sub.choices.values():
        q.add_argument("--reps", type=int, default=30)
        q.add_argument("--inner", type=int, default=16)
    args = ap.parse_args(argv)
    global INNER
    INNER = max(1, args.inner)
    if not torch.cuda.is_available():
        raise SystemExit("microbench needs a CUDA device")
    ops.prepare([], verbose=False)
    with torch.no_grad():
        rows = {"linear": bench_linear, "attn_prefill": bench_attn_prefill,
                "attn_decode": bench_attn_decode, "sample": bench_sample}[args.what](args)
    for r in rows:
        print(json.dumps(r))
    ops.check_kernel_errors()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
