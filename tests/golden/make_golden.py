"""Writes tests/golden/reference_{A,B}.npz: logits of the reference's own TransformerLM
(andreidhoang/scratch_llm, src/scratch_llm/model.py) on the CPU in 32-bit, for the tiny
configurations A and B with the engine's seeded random weights loaded under the reference's
tensor names.  tests/test_plain.py compares the plain implementation with these files.

Run from the repository root, with the reference checked out beside it:

    python tests/golden/make_golden.py /path/to/scratch_llm/src

The reference's RMSNorm eps is a constructor default that the model never sets
(model.py:153, 410-412, 456); for configuration B it is set on the built modules.
"""

import sys
import tempfile
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

from configs import CONFIGS, SEED  # noqa: E402
from scratch_llm_b200.config import config_from_dict  # noqa: E402
from scratch_llm_b200.weights import write_random_model  # noqa: E402
from plain.llama_plain import read_model_dir  # noqa: E402

LENGTHS = {"A": 33, "B": 40}


def main(reference_src: str) -> None:
    sys.path.insert(0, reference_src)
    from scratch_llm.model import ModelConfig, RMSNorm, TransformerLM

    for name in ("A", "B"):
        raw = CONFIGS[name]
        cfg = config_from_dict(raw)
        with tempfile.TemporaryDirectory() as tmp:
            write_random_model(cfg, tmp, SEED[name])
            _, w = read_model_dir(tmp)
        ref_cfg = ModelConfig(vocab_size=raw["vocab_size"], d_model=raw["hidden_size"],
                              n_layers=raw["num_hidden_layers"],
                              n_heads=raw["num_attention_heads"],
                              n_kv_heads=raw["num_key_value_heads"],
                              d_ff=raw["intermediate_size"],
                              context_length=raw["max_position_embeddings"],
                              rope_theta=raw["rope_theta"],
                              tie_embeddings=raw["tie_word_embeddings"])
        assert ref_cfg.head_dim == raw["head_dim"]
        model = TransformerLM(ref_cfg).eval()
        alias = cfg.reference_aliases()
        sd = {ref: w[ours] for ref, ours in alias.items() if ours in w}
        if raw["tie_word_embeddings"]:
            sd["lm_head.weight"] = sd["token_emb.weight"]
        model.load_state_dict(sd, strict=True)
        for mod in model.modules():
            if isinstance(mod, RMSNorm):
                mod.eps = raw["rms_norm_eps"]
        gen = torch.Generator().manual_seed(1234 + SEED[name])
        ids = torch.randint(0, raw["vocab_size"], (1, LENGTHS[name]), generator=gen)
        with torch.no_grad():
            logits = model(ids)[0]
        checksum = np.array([float(w[k].double().sum()) for k in sorted(w)])
        out = Path(__file__).parent / f"reference_{name}.npz"
        np.savez_compressed(out, tokens=ids[0].numpy().astype(np.int32),
                            logits=logits.numpy().astype(np.float32), weight_sums=checksum)
        print(out, logits.shape, float(logits.abs().max()))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/scratch_llm/src")
    main(sys.argv[1])
