"""Measuring helpers shared by both arms of ``bench.py``: the roofline denominators, the clock
sampler and the spread of per-step times.

The reference reports the median with the 10th and 90th percentile of CUDA-event times after
warm-up (src/scratch_llm/bench/harness.py:52-91); :func:`spread` is the same summary.
"""

from __future__ import annotations

import json
import statistics
import subprocess
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
                  "source": "fallback"}

# the configurations at full size that the baseline names; bench.py --sizes chooses one
SIZES_BY_NAME = {
    "llama-3-8b": dict(hidden_size=4096, num_hidden_layers=32, num_attention_heads=32,
                       num_key_value_heads=8, head_dim=128, intermediate_size=14336,
                       vocab_size=128256, rope_theta=500000.0, rms_norm_eps=1e-5,
                       tie_word_embeddings=False, max_position_embeddings=8192,
                       torch_dtype="bfloat16"),
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


def peaks() -> dict:
    """Measured copy bandwidth and bf16 product rate of this pool's GPUs if the file that holds
    them is there, else the stated fallback."""
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


def spread(times_ms: list[float]) -> dict:
    """Median, 10th and 90th percentile of per-step times in milliseconds."""
    if not times_ms:
        return {}
    s = sorted(times_ms)

    def pick(q: float) -> float:
        return s[min(len(s) - 1, max(0, round(q * (len(s) - 1))))]

    return {"median_ms": round(statistics.median(s), 4), "p10_ms": round(pick(0.1), 4),
            "p90_ms": round(pick(0.9), 4), "n": len(s)}


def model_config(name: str, sizes: dict, n_layers: int, batch: int, context: int,
                 prefill_tokens: int, peaks_source: str) -> dict:
    """The ``config`` of the bench line: every size, flat, the same for both arms."""
    return {"model": f"{name}-sizes", "layers": n_layers,
            "layers_of_config": sizes["num_hidden_layers"], "hidden": sizes["hidden_size"],
            "heads": sizes["num_attention_heads"], "kv_heads": sizes["num_key_value_heads"],
            "head_dim": sizes["head_dim"], "intermediate": sizes["intermediate_size"],
            "vocab": sizes["vocab_size"], "rope_theta": sizes["rope_theta"],
            "rms_norm_eps": sizes["rms_norm_eps"], "max_position": sizes["max_position_embeddings"],
            "tied": sizes["tie_word_embeddings"], "global_batch": batch, "seq_len": context,
            "prefill_tokens": prefill_tokens, "parallelism": "single-gpu",
            "weights": "random N(0,0.02)",
            "l2": "inputs larger than L2 (weights read once per step)", "peaks": peaks_source}


def weight_bytes(sizes: dict, n_layers: int) -> int:
    """Bytes of bf16 weights a decode step reads (a tied output matrix is still read; the
    embedding table is not: a step gathers a few rows of it) plus the 32-bit norm gains."""
    d, f, v = sizes["hidden_size"], sizes["intermediate_size"], sizes["vocab_size"]
    hq = sizes["num_attention_heads"] * sizes["head_dim"]
    hk = sizes["num_key_value_heads"] * sizes["head_dim"]
    per_layer = (hq + 2 * hk) * d + d * hq + 3 * f * d
    return 2 * (n_layers * per_layer + v * d) + 4 * (2 * n_layers + 1) * d


def kv_bytes_per_token(sizes: dict, n_layers: int) -> int:
    return 2 * sizes["num_key_value_heads"] * sizes["head_dim"] * 2 * n_layers


def prefill_flops(sizes: dict, n_layers: int, t: int) -> float:
    d, f, v = sizes["hidden_size"], sizes["intermediate_size"], sizes["vocab_size"]
    hq = sizes["num_attention_heads"] * sizes["head_dim"]
    hk = sizes["num_key_value_heads"] * sizes["head_dim"]
    linear = 2.0 * t * n_layers * ((hq + 2 * hk) * d + d * hq + 3 * f * d)
    attn = n_layers * 4.0 * hq * (t * (t + 1) / 2)   # causal half of QK^T and PV
    return linear + attn + 2.0 * v * d   # the output matrix on the one wanted row


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs (a
    query only: no setting of the GPU is touched)."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0) -> None:
        self.index, self.proc = index, None
        self.summary: dict = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}

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
