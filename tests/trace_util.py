"""Builds replay traces (the ways of cutting requests into steps) and runs them, either in
process through ``ModelRunner.step`` or through the ``bin/trace_run`` program."""

import json
import random
import subprocess
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent


def whole(requests):
    """Each request alone and whole in one step, logits wanted everywhere."""
    return [{"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}],
             "end": [rid]} for i, (rid, toks) in enumerate(requests.items())]


def tail_one_by_one(requests, tail=32):
    """Most of a request in one step, the last ``tail`` tokens one by one."""
    steps = []
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        cuts = [(0, head)] + [(i, i + 1) for i in range(head, len(toks))]
        for k, (a, b) in enumerate(cuts):
            steps.append({"step": len(steps), "entries": [
                {"id": rid, "tokens": toks[a:b], "want": list(range(b - a))}],
                "end": [rid] if k == len(cuts) - 1 else []})
    return steps


def changing_portions(requests, sizes=(7, 2, 16, 3, 33, 2, 5, 64, 2, 17)):
    """Portions of changing size, down to two tokens."""
    steps = []
    for rid, toks in requests.items():
        a, k = 0, 0
        while a < len(toks):
            b = min(len(toks), a + sizes[k % len(sizes)])
            if len(toks) - b == 1:  # never leave a single token over by accident
                b = len(toks)
            steps.append({"step": len(steps), "entries": [
                {"id": rid, "tokens": toks[a:b], "want": list(range(b - a))}],
                "end": [rid] if b == len(toks) else []})
            a, k = b, k + 1
    return steps


def mixed(requests, seed=0, max_live=4, prefill_part=0.6, sizes=(2, 3, 5, 8, 13, 21, 40)):
    """Up to ``max_live`` requests live at a time; each first gets the larger part of its tokens
    in portions of random size (a 'prompt') and then the rest one token per step (as decoding
    would feed them), so that steps hold portions of some requests beside single tokens of
    others; a request is sometimes left out of a step; finished requests end and later ones
    take over their pages."""
    rng = random.Random(seed)
    waiting = list(requests.items())
    live = {}  # rid -> [tokens, fed, prompt_len]
    steps = []
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, toks = waiting.pop(0)
            live[rid] = [toks, 0, max(1, int(len(toks) * prefill_part))]
        entries, end = [], []
        for rid, st in list(live.items()):
            toks, fed, prompt = st
            if len(live) > 1 and rng.random() < 0.15:
                continue  # left out of this step
            if fed < prompt:
                n = min(prompt - fed, rng.choice(list(sizes)))
                if prompt - fed - n == 1:
                    n += 1
            else:
                n = 1
            entries.append({"id": rid, "tokens": toks[fed:fed + n], "want": list(range(n))})
            st[1] = fed + n
            if st[1] == len(toks):
                end.append(rid)
                del live[rid]
        if entries:
            steps.append({"step": len(steps), "entries": entries, "end": end})
    return steps


def large_mixed(requests, max_live=4, tail=3, sizes=(300, 150, 260, 130, 340)):
    """Up to ``max_live`` requests live; each gets all but its last ``tail`` tokens in portions
    whose sizes cycle through ``sizes`` (hundreds of tokens), then the rest one by one: steps of
    several hundred tokens with two or three long portions beside single tokens of others."""
    waiting = list(requests.items())
    live, steps, k = {}, [], 0
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, toks = waiting.pop(0)
            live[rid] = [toks, 0, max(1, len(toks) - tail)]
        entries, end = [], []
        for rid, st in list(live.items()):
            toks, fed, prompt = st
            if fed < prompt:
                n = min(prompt - fed, sizes[k % len(sizes)])
                k += 1
                if prompt - fed - n == 1:
                    n += 1
            else:
                n = 1
            entries.append({"id": rid, "tokens": toks[fed:fed + n], "want": list(range(n))})
            st[1] = fed + n
            if st[1] == len(toks):
                end.append(rid)
                del live[rid]
        steps.append({"step": len(steps), "entries": entries, "end": end})
    return steps


def peak_tokens(steps, round_to=64):
    """The most tokens live requests hold at any time, each rounded up to ``round_to``."""
    held, peak = {}, 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-n // round_to) * round_to for n in held.values()))
        for rid in s["end"]:
            held.pop(rid, None)
    return peak


def run_in_process(runner, steps, after_step=None):
    """{(request, position): logits row} of a trace through ModelRunner.step.  ``after_step``
    is called after every step, before the step's finished requests are released."""
    from scratch_llm_b200.engine import RowInput

    out, fed = {}, {}
    for s in steps:
        rows = []
        for e in s["entries"]:
            if e["id"] not in runner.cache.requests:
                assert runner.admit(e["id"])
                fed[e["id"]] = 0
            rows.append(RowInput(e["id"], e["tokens"], e["want"]))
        logits = runner.step(rows)
        k = 0
        for e in s["entries"]:
            for w in e["want"]:
                out[(e["id"], fed[e["id"]] + w)] = logits[k].float().cpu()
                k += 1
            fed[e["id"]] += len(e["tokens"])
        if after_step is not None:
            after_step()
        for rid in s["end"]:
            runner.release(rid)
        runner.cache.check()
    return out


def run_program(model_dir, dtype, steps, out_dir, max_tokens, vocab, extra=()):
    """The same through bin/trace_run as a child process."""
    text = "".join(json.dumps(s) + "\n" for s in steps)
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model",
                           str(model_dir), "--dtype", dtype, "--out", str(out_dir),
                           "--max-tokens", str(max_tokens), *extra],
                          input=text, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-3000:]
    done = [l for l in proc.stdout.splitlines() if l.startswith("done ")]
    assert done == [f"done {s['step']}" for s in steps]
    out, fed = {}, {}
    for s in steps:
        n_want = sum(len(e["want"]) for e in s["entries"])
        path = Path(out_dir) / f"{s['step']}.f32"
        if n_want == 0:
            assert not path.exists()
        else:
            data = torch.from_numpy(np.fromfile(path, dtype="<f4").reshape(n_want, vocab).copy())
        k = 0
        for e in s["entries"]:
            fed.setdefault(e["id"], 0)
            for w in e["want"]:
                out[(e["id"], fed[e["id"]] + w)] = data[k]
                k += 1
            fed[e["id"]] += len(e["tokens"])
    return out


def chunks_of(requests, chunk, tail=3):
    """Each request alone: its tokens but the last ``tail`` in chunks of ``chunk`` (the last one
    ragged), then the rest one by one, as a scheduler with that chunk size would feed them."""
    steps = []
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        cuts = [(a, min(head, a + chunk)) for a in range(0, head, chunk)]
        cuts += [(i, i + 1) for i in range(head, len(toks))]
        for k, (a, b) in enumerate(cuts):
            steps.append({"step": len(steps), "entries": [
                {"id": rid, "tokens": toks[a:b], "want": list(range(b - a))}],
                "end": [rid] if k == len(cuts) - 1 else []})
    return steps


def make_requests(vocab, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    return {f"r{i}": torch.randint(0, vocab, (n,), generator=g).tolist()
            for i, n in enumerate(lengths)}
