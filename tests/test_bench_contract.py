"""The measuring program's contract, as far as it can be checked without a GPU: more than one
GPU is refused with one line and exit code 2, the ``config`` of the line is flat and short, and
the byte and flop counts behind the roofline fractions are the architecture's."""

import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from baseline import common  # noqa: E402


def test_more_than_one_gpu_is_refused_with_one_line():
    for n in ("2", "8"):
        proc = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--gpus", n, "--steps", "2",
                               "--warmup", "1"], capture_output=True, text=True, timeout=120)
        assert proc.returncode == 2
        lines = [line for line in proc.stdout.splitlines() if line.strip()]
        assert len(lines) == 1 and "one GPU" in lines[0]


def test_config_is_flat_and_names_every_size():
    sizes = common.SIZES_BY_NAME["llama-3-8b"]
    cfg = common.model_config("llama-3-8b", sizes, 32, 8, 1024, 2048, "measured")
    assert len(cfg) <= 20
    assert all(isinstance(v, (int, float, str, bool)) for v in cfg.values())
    assert cfg["layers"] == cfg["layers_of_config"] == 32
    for key, size in (("hidden", 4096), ("heads", 32), ("kv_heads", 8), ("head_dim", 128),
                      ("intermediate", 14336), ("vocab", 128256), ("global_batch", 8),
                      ("seq_len", 1024), ("prefill_tokens", 2048)):
        assert cfg[key] == size
    json.dumps(cfg)


def test_bytes_and_flops_of_the_named_configuration():
    sizes = common.SIZES_BY_NAME["llama-3-8b"]
    # 8.03 billion parameters, of which the embedding table (0.53 billion) is not streamed
    w = common.weight_bytes(sizes, 32)
    per_layer = (4096 * 6144 + 4096 * 4096 + 3 * 14336 * 4096)
    assert w == 2 * (32 * per_layer + 128256 * 4096) + 4 * 65 * 4096
    assert abs(w / 1e9 - 15.01) < 0.01
    assert common.kv_bytes_per_token(sizes, 32) == 128 * 1024
    # a 2,048-token prompt: 28.59 TFLOP of products and 1.10 of causal attention
    f = common.prefill_flops(sizes, 32, 2048)
    assert abs(f / 1e12 - 29.69) < 0.02
    # fewer layers: the layers' share shrinks, the output matrix stays
    assert common.weight_bytes(sizes, 2) == 2 * (2 * per_layer + 128256 * 4096) + 4 * 5 * 4096
    tied = common.SIZES_BY_NAME["llama-3.2-1b"]
    assert abs(common.weight_bytes(tied, 16) / 1e9 - 2.47) < 0.01   # the tied output matrix is read


def test_spread_and_peaks():
    s = common.spread([3.0, 1.0, 2.0, 10.0, 2.5])
    assert s["median_ms"] == 2.5 and s["n"] == 5 and s["p10_ms"] <= s["median_ms"] <= s["p90_ms"]
    assert common.spread([]) == {}
    p = common.peaks()
    assert p["source"] in ("measured", "fallback") and p["hbm_gbs"] > 1000 and p["bf16_tflops"] > 100
