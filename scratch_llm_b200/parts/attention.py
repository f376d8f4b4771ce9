"""Grouped-query attention over the paged cache.

q, k, v projections without bias (fused into one matrix at load), position encoding on q and
k, the new keys and values stored into the request's pages, causal attention in which query
head h reads kv head ``h // (n_heads / n_kv_heads)``, and the output projection:
src/scratch_llm/model.py:265-366 of the reference.  ``scale`` multiplies the scores
(``1/sqrt(head_dim)`` for this architecture, src/scratch_llm/model.py:177); ``window`` None
attends to every earlier key, a number to the last ``window`` of them.
"""

from __future__ import annotations

from typing import Mapping

import torch

from ..kernels import ops
from ..weights.loader import ParamSpec
from .base import BuildContext, CacheView, KVSpec, Mixer, PositionEncoding
from .linear import Linear
from .registry import register_mixer


#: rows with several new tokens go to the tcgen05 attention kernel when the longest of them
#: fills at least one of its 128-query tiles (packed queries = new tokens x group size)
TC_MIN_PACKED_QUERIES = 128


def decode_splits(base_ctas: int, context: int, slots: int) -> int:
    """How many CTAs share the keys of one (row, kv head) in the split decode kernel: the count
    that minimises waves x (key tiles per CTA + fixed cost), a function of the batch's shape
    and of the context bucket alone, so that it is the same for every step that replays one
    captured graph.  ``slots``: CTAs of the split kernel resident on the GPU at once
    (:func:`scratch_llm_b200.kernels.ops.attention_decode_slots` reads it from the device)."""
    tiles = max(1, -(-context // 64))
    best, best_cost = 1, None
    for n in range(1, min(64, tiles) + 1):
        # waves x (key tiles per CTA + a CTA's fixed cost) + what the merge reads per split
        cost = -(-base_ctas * n // slots) * (-(-tiles // n) + 2) + (0.1 * n if n > 1 else 0)
        if best_cost is None or cost < best_cost:
            best, best_cost = n, cost
    return best


@register_mixer("gqa_attention")
class GQAttention(Mixer):
    pad_safe = True   # padding tokens are not stored, rows without tokens leave the kernels at once
    accepts_sink = True   # forward() takes sink=: the output projection may feed the stream itself

    def accepts_normed(self, n_tokens: int) -> bool:
        return self.qkv is not None and self.qkv.takes_normed(n_tokens)

    def __init__(self, hidden_size: int, n_heads: int, n_kv_heads: int, head_dim: int,
                 scale: float, window: int | None = None,
                 names: Mapping[str, str] | None = None) -> None:
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} query heads do not group evenly over {n_kv_heads} "
                             "kv heads")
        if head_dim % 16 or not 16 <= head_dim <= 512:
            raise ValueError(f"head size {head_dim}: the attention kernels take multiples of "
                             "16 from 16 to 512")
        self.hidden_size, self.n_heads, self.n_kv_heads = hidden_size, n_heads, n_kv_heads
        self.head_dim, self.scale, self.window = head_dim, float(scale), window
        self.names = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight",
                      "o": "o_proj.weight", **(names or {})}
        self.qkv: Linear | None = None
        self.o: Linear | None = None

    def kv_spec(self) -> KVSpec:
        return KVSpec(self.n_kv_heads, self.head_dim, self.window)

    def param_specs(self) -> dict[str, ParamSpec]:
        hq, hk = self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim
        return {self.names["q"]: ParamSpec((hq, self.hidden_size)),
                self.names["k"]: ParamSpec((hk, self.hidden_size)),
                self.names["v"]: ParamSpec((hk, self.hidden_size)),
                self.names["o"]: ParamSpec((self.hidden_size, hq))}

    def load(self, tensors: Mapping[str, torch.Tensor], ctx: BuildContext) -> None:
        put = lambda t: t.to(device=ctx.device, dtype=ctx.dtype)  # noqa: E731
        self.qkv = Linear(torch.cat([put(tensors[self.names[n]]) for n in "qkv"], 0).contiguous())
        self.o = Linear(put(tensors[self.names["o"]]).contiguous())

    def forward(self, x, batch, cache: CacheView, write: bool, position: PositionEncoding,
                sink=None):
        """``x``: the normed activations (or a :class:`~.stream.Normed`, see accepts_normed);
        ``sink``: where the output projection may put its result (a
        :class:`~.stream.StreamSink`), else the result is returned."""
        out = self._attend(x, batch, cache, write, position)
        return self.o(out) if sink is None else sink.finish(self.o, out)

    def _attend(self, x, batch, cache: CacheView, write: bool,
                position: PositionEncoding) -> torch.Tensor:
        H, G, hd = self.n_heads, self.n_kv_heads, self.head_dim
        qkv = self.qkv(x)
        if position.rotary_tables:
            cos, sin, interleaved = position.cos, position.sin, position.interleaved
        else:
            n = qkv.shape[0]
            position.apply(qkv[:, :H * hd].view(n, H, hd), qkv[:, H * hd:(H + G) * hd].view(n, G, hd),
                           batch.positions)
            cos = sin = None
            interleaved = True
        # (padding tokens get no attention output: zeros, so that what follows stays finite)
        out = (torch.zeros if batch.padded else torch.empty)(
            (qkv.shape[0], H * hd), dtype=qkv.dtype, device=qkv.device)
        if (cos is not None and qkv.dtype == torch.bfloat16 and batch.n_multi == 0
                and batch.n_single > 0 and H // G <= 16
                and ops.attention_decode_fused_supported(hd)):
            # a step of single tokens: the decode kernel rotates q and the new keys itself and
            # stores the new keys and values (one launch fewer, q and k make no round trip)
            self._decode_fused(qkv, out, batch, cache, (cos, sin, interleaved, write))
            return out
        ops.rope_kv_write(qkv, batch.positions, batch.token_row, cos, sin, cache.pages,
                          cache.block_table, cache.page_size, H, G, hd, interleaved, write)
        q = qkv[:, :H * hd]
        if qkv.dtype == torch.bfloat16 and hd <= ops.MMA_MAX_HEAD_DIM:
            self._attend_tensor_cores(q, out, batch, cache)
        else:
            ops.attention_simt(q, cache.pages, cache.block_table, cache.page_size,
                               batch.row_start, batch.row_pos0, out, batch.n_rows,
                               batch.max_new, H, G, hd, self.scale, self.window)
        return out

    def _n_splits(self, batch) -> int:
        H, G = self.n_heads, self.n_kv_heads
        return decode_splits(batch.n_single * G * (-(-(H // G) // 16)),
                             batch.context_bucket if self.window is None
                             else min(batch.context_bucket, self.window + 64),
                             ops.attention_decode_slots(self.head_dim))

    def _decode_fused(self, qkv, out, batch, cache: CacheView, rope) -> None:
        H, G, hd = self.n_heads, self.n_kv_heads, self.head_dim
        n_splits = self._n_splits(batch)
        scratch = None
        if n_splits > 1:
            scratch = torch.empty(ops.attention_mma_scratch_floats(qkv.shape[0], H, hd, n_splits),
                                  dtype=torch.float32, device=qkv.device)
        cos, sin, interleaved, write = rope
        # every row is single and the list names them in order: the kernel needs no list
        # (one load less on the way to a CTA's first keys)
        rows = None if batch.n_single == batch.n_rows else batch.single_rows
        # Where the launch fits the device at once, what counts is the chain of kernels: the CTA
        # that finishes last for a row and kv head merges the splits itself and no merge kernel
        # follows.  A launch of several rounds of CTAs is bound by its work, to which the count
        # and its fence in every CTA would add (5.57 against 5.38 ms a step at batch 64).
        ctas = batch.n_single * G * (-(-(H // G) // 16)) * n_splits
        inside = ctas <= ops.attention_decode_slots(hd)
        ops.attention_mma_decode(qkv, cache.pages, cache.block_table, cache.page_size,
                                 batch.row_start, batch.row_pos0, out, rows,
                                 batch.n_single, H, G, hd, self.scale, self.window, cos, sin,
                                 interleaved, write, n_splits, scratch, merge_inside=inside)

    def _attend_tensor_cores(self, q, out, batch, cache: CacheView) -> None:
        """Rows with several new tokens go to the wide kernel, rows with one to the split
        kernel, whose number of splits along the keys comes from :func:`decode_splits`."""
        H, G, hd = self.n_heads, self.n_kv_heads, self.head_dim
        common = (q, cache.pages, cache.block_table, cache.page_size, batch.row_start,
                  batch.row_pos0, out)
        if batch.n_multi:
            if ops.attention_tc_supports(H, G, hd, cache.page_size, self.window) \
                    and batch.max_new_multi * (H // G) >= TC_MIN_PACKED_QUERIES:
                # tcgen05 kernel: scores, probabilities and output in tensor memory
                ops.attention_tc(*common, batch.multi_rows, batch.n_multi, batch.max_new_multi,
                                 H, G, hd, self.scale)
            else:
                ops.attention_mma(*common, batch.multi_rows, batch.n_multi,
                                  batch.max_new_multi, H, G, hd, self.scale, self.window,
                                  split=False)
        if batch.n_single:
            n_splits = self._n_splits(batch)
            scratch = None
            if n_splits > 1:
                scratch = torch.empty(ops.attention_mma_scratch_floats(q.shape[0], H, hd, n_splits),
                                      dtype=torch.float32, device=q.device)
            ops.attention_mma(*common, batch.single_rows, batch.n_single, 1, H, G, hd,
                              self.scale, self.window, split=True, n_splits=n_splits,
                              scratch=scratch)
