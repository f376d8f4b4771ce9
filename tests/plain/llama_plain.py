"""A plain, slow implementation of the Llama-style dense GQA decoder: whole sequences, no
cache, one function per part, PyTorch on the CPU only.

It is written from the formulas of the reference (andreidhoang/scratch_llm), each function
citing the file and lines it restates, and shares no code with ``scratch_llm_b200``: it has
its own safetensors reader and takes ``config.json`` as a plain dict.  ``tests/golden/`` holds
outputs of the reference's own ``TransformerLM`` on a tiny random model, against which
``tests/test_plain.py`` checks this file once.
"""

from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch


# ---------------------------------------------------------------------------- model folder

def read_model_dir(model_dir, dtype=torch.float32):
    """(config dict, {name: tensor}) of a folder with config.json and model.safetensors."""
    model_dir = Path(model_dir)
    config = json.loads((model_dir / "config.json").read_text())
    raw = (model_dir / "model.safetensors").read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    header.pop("__metadata__", None)
    tensors = {}
    for name, info in header.items():
        b, e = info["data_offsets"]
        buf = raw[8 + n + b:8 + n + e]
        if info["dtype"] == "F32":
            t = torch.from_numpy(np.frombuffer(buf, dtype="<f4").copy())
        elif info["dtype"] == "BF16":
            bits = np.frombuffer(buf, dtype="<u2").astype(np.uint32) << 16
            t = torch.from_numpy(bits.view(np.float32).copy())
        else:
            raise ValueError(f"{name}: dtype {info['dtype']}")
        tensors[name] = t.reshape(info["shape"]).to(dtype)
    return config, tensors


# ---------------------------------------------------------------------------------- parts

def embed(token_ids, table):
    """Row gather, no scaling and no position added: src/scratch_llm/model.py:145-146, 499."""
    return table[token_ids]


def rmsnorm(x, weight, eps):
    """x * rsqrt(mean(x^2) + eps) * weight, eps inside the root, the weight after the
    normalisation: src/scratch_llm/model.py:158-162."""
    rms = torch.rsqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)
    return x * rms * weight


def rope_tables(head_dim, n_positions, theta, dtype=torch.float32):
    """cos and sin of position * theta^(-2j/head_dim), j = 0..head_dim/2-1, built in 32-bit:
    src/scratch_llm/model.py:195-202."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2).float() / head_dim))
    freqs = torch.outer(torch.arange(n_positions).float(), inv_freq)
    return freqs.cos().to(dtype), freqs.sin().to(dtype)


def apply_rope(x, positions, cos, sin, interleaved=True):
    """Rotate pairs of x (..., seq, head_dim) by their position's angles.  interleaved: the
    pairs are (x[2j], x[2j+1]), src/scratch_llm/model.py:204-220.  Otherwise the pairs are
    (x[j], x[j + head_dim/2]), the layout of checkpoints saved for the split-half rotation."""
    c, s = cos[positions], sin[positions]
    if interleaved:
        even, odd = x[..., 0::2], x[..., 1::2]
        return torch.stack((even * c - odd * s, even * s + odd * c), dim=-1).flatten(-2)
    half = x.shape[-1] // 2
    a, b = x[..., :half], x[..., half:]
    return torch.cat((a * c - b * s, a * s + b * c), dim=-1)


def attention(q, k, v, q_positions, k_positions, scale, window=None):
    """softmax(q k^T * scale + mask) v with max-subtracted softmax; a query at position p sees
    key j iff j <= p (and j > p - window if a window is given).  q (H, S, hd); k, v (G, T, hd);
    query head h uses kv head h // (H / G): src/scratch_llm/model.py:172-182, 330-345."""
    n_heads, n_kv = q.shape[0], k.shape[0]
    k = k.repeat_interleave(n_heads // n_kv, dim=0)
    v = v.repeat_interleave(n_heads // n_kv, dim=0)
    scores = (q @ k.transpose(-2, -1)) * scale
    allowed = k_positions[None, :] <= q_positions[:, None]
    if window is not None:
        allowed &= k_positions[None, :] > q_positions[:, None] - window
    scores = scores.masked_fill(~allowed, float("-inf"))
    scores = scores - scores.amax(dim=-1, keepdim=True)
    e = scores.exp()
    return (e / e.sum(dim=-1, keepdim=True)) @ v


def swiglu(x, w_gate, w_up, w_down):
    """W_down( silu(W_gate x) * (W_up x) ), silu(z) = z * sigmoid(z); w1 = gate, w3 = up,
    w2 = down: src/scratch_llm/model.py:223-237."""
    g = x @ w_gate.T
    return ((g * torch.sigmoid(g)) * (x @ w_up.T)) @ w_down.T


def attention_layer(h, positions, w, prefix, cfg, cos, sin, shared_kv=None):
    """Projections, rotary positions on q and k, attention, output projection:
    src/scratch_llm/model.py:265-366.  Returns (output, (k, v)); with ``shared_kv`` the layer
    attends to another run's keys and values instead of its own."""
    n_heads = cfg["num_attention_heads"]
    n_kv = cfg.get("num_key_value_heads") or n_heads
    hd = cfg.get("head_dim") or cfg["hidden_size"] // n_heads
    s = h.shape[0]
    q = (h @ w[f"{prefix}.q_proj.weight"].T).view(s, n_heads, hd).transpose(0, 1)
    q = apply_rope(q, positions, cos, sin, cfg.get("rope_interleaved", True))
    if shared_kv is None:
        k = (h @ w[f"{prefix}.k_proj.weight"].T).view(s, n_kv, hd).transpose(0, 1)
        v = (h @ w[f"{prefix}.v_proj.weight"].T).view(s, n_kv, hd).transpose(0, 1)
        k = apply_rope(k, positions, cos, sin, cfg.get("rope_interleaved", True))
    else:
        k, v = shared_kv
    out = attention(q, k, v, positions, positions, 1.0 / math.sqrt(hd), cfg.get("sliding_window"))
    out = out.transpose(0, 1).reshape(s, n_heads * hd)
    return out @ w[f"{prefix}.o_proj.weight"].T, (k, v)


def block(x, positions, w, layer, cfg, cos, sin, shared_kv=None):
    """x + Attn(Norm(x)), then x + FFN(Norm(x)): src/scratch_llm/model.py:423-436."""
    p = f"model.layers.{layer}"
    eps = cfg.get("rms_norm_eps", 1e-5)
    a, kv = attention_layer(rmsnorm(x, w[f"{p}.input_layernorm.weight"], eps), positions, w,
                            f"{p}.self_attn", cfg, cos, sin, shared_kv)
    x = x + a
    h = rmsnorm(x, w[f"{p}.post_attention_layernorm.weight"], eps)
    x = x + swiglu(h, w[f"{p}.mlp.gate_proj.weight"], w[f"{p}.mlp.up_proj.weight"],
                   w[f"{p}.mlp.down_proj.weight"])
    return x, kv


def forward(cfg, w, token_ids, order=None, dtype=torch.float32):
    """Logits (S, V) at every position of one whole sequence starting at position 0:
    src/scratch_llm/model.py:471-505.  ``order`` is a list of (layer, cache entry, write);
    the default runs every layer once in index order."""
    ids = torch.as_tensor(token_ids, dtype=torch.long)
    n_heads = cfg["num_attention_heads"]
    hd = cfg.get("head_dim") or cfg["hidden_size"] // n_heads
    w = {k: v.to(dtype) for k, v in w.items()}
    cos, sin = rope_tables(hd, len(ids), cfg.get("rope_theta", 10000.0), dtype)
    positions = torch.arange(len(ids))
    x = embed(ids, w["model.embed_tokens.weight"])
    if order is None:
        order = [(i, i, True) for i in range(cfg["num_hidden_layers"])]
    kept = {}
    for layer, entry, write in order:
        x, kv = block(x, positions, w, layer, cfg, cos, sin, None if write else kept[entry])
        if write:
            kept[entry] = kv
    x = rmsnorm(x, w["model.norm.weight"], cfg.get("rms_norm_eps", 1e-5))
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings") else w["lm_head.weight"]
    return x @ head.T


# ------------------------------------------------------------------------------- sampling

def greedy(cfg, w, prompt, n_new, dtype=torch.float32):
    """Greedy continuation by full recompute, the reference's oracle path
    (src/scratch_llm/sampling.py:172-182 with temperature 0: argmax, first maximum on ties)."""
    ids = list(prompt)
    out = []
    for _ in range(n_new):
        nxt = int(forward(cfg, w, ids, dtype=dtype)[-1].argmax())
        ids.append(nxt)
        out.append(nxt)
    return out


def top_p_filter(probs, top_p):
    """Keep the smallest set of most probable tokens whose mass reaches top_p (the token that
    crosses it is kept), renormalise: src/scratch_llm/sampling.py:60-77."""
    if top_p >= 1.0:
        return probs
    sorted_probs, idx = torch.sort(probs, descending=True)
    remove = torch.cumsum(sorted_probs, dim=-1) > top_p
    remove[1:] = remove[:-1].clone()
    remove[0] = False
    sorted_probs = sorted_probs.masked_fill(remove, 0.0)
    sorted_probs = sorted_probs / sorted_probs.sum()
    return torch.zeros_like(probs).scatter_(-1, idx, sorted_probs)


def sampling_distribution(logits, temperature, top_p=1.0):
    """The distribution that the next token is drawn from: softmax(logits / T), then the
    nucleus filter: src/scratch_llm/sampling.py:80-86."""
    z = logits / temperature
    z = z - z.max()
    p = z.exp() / z.exp().sum()
    return top_p_filter(p, top_p)
