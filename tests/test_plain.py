"""The plain implementation against the reference's own model (golden files), and against
itself where the formulas imply an identity."""

import math
from pathlib import Path

import numpy as np
import pytest
import torch

from configs import CONFIGS
from plain import llama_plain as P

GOLDEN = Path(__file__).parent / "golden"


@pytest.mark.parametrize("name", ["A", "B"])
def test_plain_matches_reference_model(name, model_dirs):
    gold = np.load(GOLDEN / f"reference_{name}.npz")
    cfg, w = P.read_model_dir(model_dirs[name])
    sums = np.array([float(w[k].double().sum()) for k in sorted(w)])
    np.testing.assert_allclose(sums, gold["weight_sums"], rtol=0, atol=1e-9,
                               err_msg="seeded weights differ from the ones the golden file "
                                       "was made with")
    logits = P.forward(cfg, w, gold["tokens"].tolist())
    torch.testing.assert_close(logits, torch.from_numpy(gold["logits"]), rtol=1e-5, atol=2e-6)


def test_float64_agrees_with_float32(model_dirs):
    cfg, w = P.read_model_dir(model_dirs["C"])
    ids = list(range(3, 60))
    a = P.forward(cfg, w, ids)
    b = P.forward(cfg, w, ids, dtype=torch.float64)
    torch.testing.assert_close(a.double(), b, rtol=1e-4, atol=2e-6)


def test_causal_no_leak(model_dirs):
    # logits up to a cut do not change when later tokens do (tests/test_model.py:60-75 of the
    # reference)
    cfg, w = P.read_model_dir(model_dirs["A"])
    ids = list(range(10, 40))
    other = ids[:20] + [(t * 7 + 3) % 256 for t in ids[20:]]
    a, b = P.forward(cfg, w, ids), P.forward(cfg, w, other)
    assert torch.equal(a[:20], b[:20])
    assert not torch.equal(a[20:], b[20:])


def test_rope_score_depends_on_offset_only():
    cos, sin = P.rope_tables(32, 64, 10000.0)
    g = torch.Generator().manual_seed(0)
    q, k = torch.randn(1, 1, 32, generator=g), torch.randn(1, 1, 32, generator=g)
    for inter in (True, False):
        def score(pq, pk):
            a = P.apply_rope(q, torch.tensor([pq]), cos, sin, inter)
            b = P.apply_rope(k, torch.tensor([pk]), cos, sin, inter)
            return float((a * b).sum())
        assert score(5, 2) == pytest.approx(score(40, 37), abs=1e-4)
        assert score(5, 2) != pytest.approx(score(5, 3), abs=1e-4)


def test_rmsnorm_and_swiglu_formulas():
    x = torch.tensor([[3.0, 4.0]])
    out = P.rmsnorm(x, torch.tensor([2.0, 0.5]), 0.0)
    torch.testing.assert_close(out, torch.tensor([[3 / math.sqrt(12.5) * 2, 4 / math.sqrt(12.5) * 0.5]]))
    wg, wu, wd = torch.tensor([[1.0, 0.0]]), torch.tensor([[0.0, 1.0]]), torch.tensor([[1.0], [2.0]])
    y = P.swiglu(x, wg, wu, wd)
    s = 3.0 / (1 + math.exp(-3.0)) * 4.0
    torch.testing.assert_close(y, torch.tensor([[s, 2 * s]]))


def test_attention_window_and_groups():
    g = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(4, 6, 8, generator=g), torch.randn(2, 6, 8, generator=g),
               torch.randn(2, 6, 8, generator=g))
    pos = torch.arange(6)
    full = P.attention(q, k, v, pos, pos, 0.3)
    # the first query sees only key 0: its output is v[0] of its kv head
    torch.testing.assert_close(full[:, 0], v.repeat_interleave(2, 0)[:, 0])
    win = P.attention(q, k, v, pos, pos, 0.3, window=1)  # each query sees itself only
    torch.testing.assert_close(win, v.repeat_interleave(2, 0))
    assert torch.equal(P.attention(q, k, v, pos, pos, 0.3, window=100), full)


def test_top_p_keeps_crossing_token():
    p = torch.tensor([0.5, 0.3, 0.15, 0.05])
    out = P.top_p_filter(p, 0.7)
    torch.testing.assert_close(out, torch.tensor([0.5 / 0.8, 0.3 / 0.8, 0.0, 0.0]))
    assert torch.equal(P.top_p_filter(p, 1.0), p)


def test_greedy_is_deterministic_and_run_order_is_data(model_dirs):
    cfg, w = P.read_model_dir(model_dirs["A"])
    assert P.greedy(cfg, w, [1, 2, 3], 4) == P.greedy(cfg, w, [1, 2, 3], 4)
    ids = [5, 9, 200, 31, 7]
    default = P.forward(cfg, w, ids)
    explicit = P.forward(cfg, w, ids, order=[(0, 0, True), (1, 1, True)])
    assert torch.equal(default, explicit)
    shared = P.forward(cfg, w, ids, order=[(0, 0, True), (1, 0, False)])
    assert not torch.equal(default, shared)
