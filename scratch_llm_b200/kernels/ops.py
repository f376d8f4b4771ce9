"""Python bindings of the engine's CUDA kernels: one function per launcher of ``csrc/``.

Each function checks devices, dtypes and layouts, passes raw pointers and the current CUDA
stream through ctypes, and raises :class:`KernelError` on a non-zero return code.  There is no
other implementation behind these functions: if a library cannot be compiled or loaded, the
call fails.

The reference reaches its compiled kernels through one pybind module (csrc/pybind.cpp:89-127)
and a lazy dispatch table (src/scratch_llm/kernels/attention/dispatch.py:68-90).
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_int64, c_void_p
from typing import Sequence

import torch

from . import build

_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}


class KernelError(RuntimeError):
    pass


# library name -> (sources, defines)
CORE_LIBRARIES: dict[str, tuple[tuple[str, ...], tuple[str, ...]]] = {
    "sllm_elementwise": (("elementwise.cu",), ()),
    "sllm_rope_cache": (("rope_cache.cu",), ()),
    "sllm_gemm_simt": (("gemm_simt.cu",), ()),
    "sllm_sampling": (("sampling.cu",), ()),
    "sllm_gemv_mma": (("gemv_mma.cu",), ()),
    "sllm_gemm_tcgen05": (("gemm_tcgen05.cu",), ()),
    "sllm_gemv_tma": (("gemv_tma.cu",), ()),
}


def attention_library(head_dim: int) -> tuple[str, tuple[str, ...], tuple[str, ...]]:
    return (f"sllm_attention_simt_hd{head_dim}", ("attention_simt.cu",),
            (f"SLLM_HEAD_DIM={head_dim}",))


def attention_mma_library(head_dim: int) -> tuple[str, tuple[str, ...], tuple[str, ...]]:
    return (f"sllm_attention_mma_hd{head_dim}", ("attention_mma.cu",),
            (f"SLLM_HEAD_DIM={head_dim}",))


def attention_tc_library(head_dim: int) -> tuple[str, tuple[str, ...], tuple[str, ...]]:
    return (f"sllm_attention_tc_hd{head_dim}", ("attention_tc.cu",),
            (f"SLLM_HEAD_DIM={head_dim}",))


def attention_tc_supports(n_heads: int, n_kv_heads: int, head_dim: int, page_size: int,
                          window: int | None) -> bool:
    """Whether the tcgen05 attention kernel takes this shape (else attention_mma serves it)."""
    if head_dim % 64 or not 64 <= head_dim <= 256 or window:
        return False
    gs = n_heads // n_kv_heads
    return n_heads % n_kv_heads == 0 and 128 % gs == 0 and page_size > 0 and 128 % page_size == 0


#: the tensor-core attention kernels take head sizes up to this; larger ones use the CUDA cores
MMA_MAX_HEAD_DIM = 256

_loaded: dict[str, ctypes.CDLL] = {}


def _load(name: str, sources: Sequence[str], defines: Sequence[str]) -> ctypes.CDLL:
    lib = _loaded.get(name)
    if lib is None:
        path = build.compile_library(name, sources, defines)
        try:
            lib = ctypes.CDLL(str(path))
        except OSError as exc:
            raise KernelError(f"cannot load {path}: {exc}") from None
        _loaded[name] = lib
    return lib


def _core(name: str) -> ctypes.CDLL:
    return _load(name, *CORE_LIBRARIES[name])


def prepare(head_dims: Sequence[int] = (), verbose: bool = True) -> None:
    """Compile (in parallel) and load everything a model with these head sizes needs."""
    jobs = [(n, s, d) for n, (s, d) in CORE_LIBRARIES.items()]
    jobs += [attention_library(hd) for hd in sorted(set(head_dims))]
    jobs += [attention_mma_library(hd) for hd in sorted(set(head_dims)) if hd <= MMA_MAX_HEAD_DIM]
    jobs += [attention_tc_library(hd) for hd in sorted(set(head_dims))
             if hd % 64 == 0 and hd <= 256]
    build.compile_many(jobs, verbose=verbose)
    for n, s, d in jobs:
        _load(n, s, d)


#: kernels of this package launched so far in this process (one per successful op call)
launch_count = 0
#: the same per op name ("gemv_tma", "attention_tc", ...): which kernels a workload reached.
#: Calls recorded into a CUDA graph count once, at the capture; replays are counted by the runner.
launch_counts: dict[str, int] = {}


def _check(code: int, what: str) -> None:
    global launch_count
    launch_count += 1
    launch_counts[what] = launch_counts.get(what, 0) + 1
    if code != 0:
        raise KernelError(f"{what} failed with CUDA error {code} "
                          f"({'invalid value: a size this kernel does not take' if code == 1 else 'see cudaError_t'})")


# the current stream's handle without building a torch.cuda.Stream object (3 us a call, which
# is a third of a launch's host cost in steps that run outside a captured graph)
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_current_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> c_void_p:
    if _raw_stream is not None and _current_device is not None:
        return c_void_p(_raw_stream(_current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: torch.Tensor | None) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def _need(t: torch.Tensor, dtype: torch.dtype | None, name: str, contiguous: bool = True) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor: the engine has no CPU path")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


def _code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"unsupported dtype {dtype}: kernels take float32 and bfloat16") from None


# ------------------------------------------------------------------------------ elementwise

def embed(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor,
          pending: torch.Tensor | None = None, scale: float = 1.0) -> torch.Tensor:
    """out[n] = table[ids[n]] widened to 32-bit, times ``scale`` (an architecture's embedding
    multiplier).  ids int32 [N]; table [V, d]; out f32 [N, d].
    An id ``-1 - j`` stands for ``pending[j]`` (int32, on the device): a token that an earlier
    kernel of the stream chose and the host has not read yet."""
    _need(ids, torch.int32, "ids")
    if pending is not None:
        _need(pending, torch.int32, "pending")
    _need(table, None, "table")
    _need(out, torch.float32, "out")
    n, d = ids.numel(), table.shape[1]
    if out.shape != (n, d):
        raise KernelError(f"out must be [{n}, {d}], got {list(out.shape)}")
    _check(_core("sllm_elementwise").sllm_embed(
        _ptr(ids), _ptr(pending) if pending is not None else c_void_p(0), _ptr(table), _ptr(out),
        c_int(n), c_int(d), c_int(_code(table.dtype)), c_float(scale), _stream()), "embed")
    return out


def embed_prepare(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor,
                  pending: torch.Tensor | None, scale: float, gain: torch.Tensor,
                  x_out: torch.Tensor, shares: torch.Tensor) -> None:
    """:func:`embed` for up to 8 tokens of a bfloat16 table, with the norm after it prepared for
    the product that follows: ``x_out`` [N, d] = bfloat16(out * gain), ``shares`` [d / 8, 8] the
    tokens' sums of squares in groups of 8 features (see scratch_llm_b200.parts.stream)."""
    _need(ids, torch.int32, "ids")
    if pending is not None:
        _need(pending, torch.int32, "pending")
    _need(table, torch.bfloat16, "table")
    _need(out, torch.float32, "out")
    _need(gain, torch.float32, "gain")
    _need(x_out, torch.bfloat16, "x_out", contiguous=False)
    _need(shares, torch.float32, "shares")
    n, d = ids.numel(), table.shape[1]
    if n > 8 or d % 8 or out.shape != (n, d) or x_out.shape != (n, d) or gain.numel() != d \
            or shares.shape != (d // 8, 8) or x_out.stride(1) != 1:
        raise KernelError("embed_prepare shapes")
    _check(_core("sllm_elementwise").sllm_embed_prepare(
        _ptr(ids), _ptr(pending) if pending is not None else c_void_p(0), _ptr(table), _ptr(out),
        c_int(n), c_int(d), c_float(scale), _ptr(gain), _ptr(x_out), c_int64(x_out.stride(0)),
        _ptr(shares), _stream()), "embed_prepare")


def logit_cap(logits: torch.Tensor, scale: float = 1.0, cap: float = 0.0) -> torch.Tensor:
    """In place on 32-bit logits: ``cap * tanh(logits * scale / cap)``, or ``logits * scale``
    when ``cap`` is 0."""
    _need(logits, torch.float32, "logits")
    if not logits.is_contiguous():
        raise KernelError("logits must be contiguous")
    if cap < 0:
        raise KernelError(f"cap must not be negative, got {cap}")
    _check(_core("sllm_elementwise").sllm_logit_cap(
        _ptr(logits), c_int64(logits.numel()), c_float(scale), c_float(cap), _stream()),
        "logit_cap")
    return logits


def add_rmsnorm(resid: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor,
                eps: float, out: torch.Tensor, index: torch.Tensor | None = None) -> torch.Tensor:
    """resid += delta (if given), out = rmsnorm(resid) * weight.  With ``index`` only the rows
    ``index`` are normed into out[0..len(index)) and resid is left as it was."""
    _need(resid, torch.float32, "resid")
    _need(weight, torch.float32, "weight")
    _need(out, None, "out")
    d = resid.shape[-1]
    if delta is not None:
        _need(delta, out.dtype, "delta")
        if delta.shape != resid.shape:
            raise KernelError("delta and resid differ in shape")
    if weight.numel() != d or out.shape[-1] != d:
        raise KernelError("norm width mismatch")
    if index is not None:
        _need(index, torch.int32, "index")
        n_out = index.numel()
    else:
        n_out = resid.shape[0]
    if out.shape[0] != n_out:
        raise KernelError("out has the wrong number of rows")
    _check(_core("sllm_elementwise").sllm_add_rmsnorm(
        _ptr(resid), _ptr(delta), _ptr(index), _ptr(weight), c_float(eps), _ptr(out),
        c_int(n_out), c_int(d), c_int(_code(out.dtype)), _stream()), "add_rmsnorm")
    return out


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[n, f] = silu(gate_up[n, f]) * gate_up[n, F + f]."""
    _need(gate_up, None, "gate_up")
    _need(out, gate_up.dtype, "out")
    n, two_f = gate_up.shape
    if two_f % 2 or out.shape != (n, two_f // 2):
        raise KernelError("swiglu shapes")
    _check(_core("sllm_elementwise").sllm_swiglu(
        _ptr(gate_up), _ptr(out), c_int(n), c_int(two_f // 2), c_int(_code(out.dtype)),
        _stream()), "swiglu")
    return out


# ------------------------------------------------------------------------------------ gemm

def gemm_simt(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = x[M, K] @ w[N, K]^T with 32-bit fused multiply-adds on the CUDA cores."""
    _need(x, None, "x", contiguous=False)
    _need(w, x.dtype, "w", contiguous=False)
    _need(out, None, "out", contiguous=False)
    (m, k), (n, k2) = x.shape, w.shape
    if k != k2 or out.shape != (m, n) or x.stride(1) != 1 or w.stride(1) != 1 \
            or out.stride(1) != 1:
        raise KernelError(f"gemm shapes/strides: x {list(x.shape)}, w {list(w.shape)}, "
                          f"out {list(out.shape)}")
    _check(_core("sllm_gemm_simt").sllm_gemm_simt(
        _ptr(x), _ptr(w), _ptr(out), c_int(m), c_int(n), c_int(k), c_int64(x.stride(0)),
        c_int64(w.stride(0)), c_int64(out.stride(0)), c_int(_code(x.dtype)),
        c_int(_code(out.dtype)), _stream()), "gemm_simt")
    return out


#: the streaming small-batch product takes up to this many tokens
GEMV_MAX_TOKENS = 64


def gemv_mma(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, swiglu: bool = False
             ) -> torch.Tensor:
    """out[M, N] = x[M, K] @ w[N, K]^T for M <= 64 tokens (bfloat16 operands, tensor cores,
    32-bit accumulation), streaming w once.  ``swiglu``: w = [gate rows; up rows] and
    out[M, N/2] = silu(x gate^T) * (x up^T).  ``out`` is bfloat16 or float32."""
    _need(x, torch.bfloat16, "x", contiguous=False)
    _need(w, torch.bfloat16, "w", contiguous=False)
    _need(out, None, "out", contiguous=False)
    (m, k), (n, k2) = x.shape, w.shape
    n_out = n // 2 if swiglu else n
    if k != k2 or out.shape != (m, n_out) or x.stride(1) != 1 or w.stride(1) != 1 \
            or out.stride(1) != 1:
        raise KernelError(f"gemv shapes/strides: x {list(x.shape)}, w {list(w.shape)}, "
                          f"out {list(out.shape)}")
    if m > GEMV_MAX_TOKENS or k % 8 or x.stride(0) % 8 or w.stride(0) % 8:
        raise KernelError(f"gemv_mma takes up to {GEMV_MAX_TOKENS} tokens and rows that are "
                          f"multiples of 8 elements; got M={m}, K={k}")
    _check(_core("sllm_gemv_mma").sllm_gemv_mma(
        _ptr(x), _ptr(w), _ptr(out), c_int(m), c_int(n), c_int(k), c_int64(x.stride(0)),
        c_int64(w.stride(0)), c_int64(out.stride(0)), c_int(int(swiglu)),
        c_int(_code(out.dtype)), _stream()), "gemv_mma")
    return out


#: workspaces of the persistent small-batch product, per device: the words through which the
#: ranges of K exchange partial sums (zero between launches).  A
#: workspace that has been handed to a launch is never freed (a captured CUDA graph may hold its
#: address), so a larger one is made beside it when a wider matrix comes.
_gemv_workspaces: dict[int, list[torch.Tensor]] = {}
_sm_counts: dict[int, int] = {}


def _sm_count(device: torch.device | int | None = None) -> int:
    index = device.index if isinstance(device, torch.device) else device
    if index is None:
        index = torch.cuda.current_device()
    if index not in _sm_counts:
        _sm_counts[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return _sm_counts[index]


def sm_count(device: torch.device | int | None = None) -> int:
    """SMs of ``device`` (the current one by default)."""
    return _sm_count(device)


def gemv_tma_supports(m: int, n: int, k: int, swiglu: bool = False) -> bool:
    """Whether :func:`gemv_tma` takes a product of these sizes (on the current device)."""
    return bool(_core("sllm_gemv_tma").sllm_gemv_tma_supports(
        c_int(m), c_int(n), c_int(k), c_int(int(swiglu)), c_int(_sm_count())))


def gemv_tma_reserve(n: int, k: int, swiglu: bool, device: torch.device) -> torch.Tensor:
    """A zeroed workspace on ``device`` that is large enough for a weight [n, k].  Called when a
    model is built, so that no step allocates it."""
    lib = _core("sllm_gemv_tma")
    lib.sllm_gemv_tma_workspace_bytes.restype = ctypes.c_int64
    need = int(lib.sllm_gemv_tma_workspace_bytes(c_int(n), c_int(k), c_int(int(swiglu)),
                                                 c_int(_sm_count(device))))
    index = device.index if device.index is not None else torch.cuda.current_device()
    held = _gemv_workspaces.setdefault(index, [])
    if not held or held[-1].numel() < need:
        held.append(torch.zeros(need, dtype=torch.uint8, device=device))
    return held[-1]


def gemv_tma(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None, swiglu: bool = False,
             scale: tuple[torch.Tensor, int, float] | None = None,
             sink: tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor] | None = None
             ) -> torch.Tensor | None:
    """out[M, N] = x[M, K] @ w[N, K]^T for M <= 8 tokens by the persistent kernel that streams w
    through shared memory with bulk copies (one CTA per SM, four ranges of K whose partial sums
    the last CTA of a row tile adds in a fixed order).  ``swiglu`` as in :func:`gemv_mma`.
    Launches share one workspace per device and must be ordered by their stream.

    ``scale = (shares, dim, eps)``: x is a stream times a norm's gain whose RMS norm is not
    finished; every output of token t is multiplied by ``rsqrt(shares[:, t].sum() / dim + eps)``
    (``shares`` float32 [parts, 8]).  ``sink = (resid, gain, x_out, shares_out)`` (not with
    ``swiglu``): the output is added into the 32-bit stream ``resid`` [M, N] instead of being
    stored (``out`` may be None), ``x_out`` [M, N] bfloat16 gets ``resid * gain`` and
    ``shares_out`` float32 [ceil(N / 8), 8] the tokens' sums of squares over each 8 features."""
    _need(x, torch.bfloat16, "x", contiguous=False)
    _need(w, torch.bfloat16, "w", contiguous=False)
    (m, k), (n, k2) = x.shape, w.shape
    n_out = n // 2 if swiglu else n
    if out is not None:
        _need(out, None, "out", contiguous=False)
        if out.shape != (m, n_out) or out.stride(1) != 1:
            raise KernelError(f"gemv out must be [{m}, {n_out}] with contiguous rows")
    elif sink is None:
        raise KernelError("gemv_tma needs an output or a sink")
    if k != k2 or x.stride(1) != 1 or w.stride(1) != 1:
        raise KernelError(f"gemv shapes/strides: x {list(x.shape)}, w {list(w.shape)}")
    if not gemv_tma_supports(m, n, k, swiglu) or x.stride(0) % 8 or w.stride(0) % 8:
        raise KernelError(f"gemv_tma takes 1 to 8 tokens, K a multiple of 256 and at least 1024, "
                          f"and rows that are multiples of 8 elements; got M={m}, N={n}, K={k}")
    ss_in, ss_parts, ss_dim, ss_eps = None, 0, 1, 0.0
    if scale is not None:
        ss_in, ss_dim, ss_eps = scale
        _need(ss_in, torch.float32, "scale shares")
        if ss_in.dim() != 2 or ss_in.shape[1] != 8 or ss_dim < 1:
            raise KernelError("scale shares must be float32 [parts, 8]")
        ss_parts = ss_in.shape[0]
    resid = gain = x_out = ss_out = None
    if sink is not None:
        if swiglu:
            raise KernelError("a sink cannot follow the fused activation")
        resid, gain, x_out, ss_out = sink
        _need(resid, torch.float32, "resid", contiguous=False)
        _need(gain, torch.float32, "gain")
        _need(x_out, torch.bfloat16, "x_out", contiguous=False)
        _need(ss_out, torch.float32, "shares_out")
        if resid.shape != (m, n) or x_out.shape != (m, n) or gain.numel() != n \
                or resid.stride(1) != 1 or x_out.stride(1) != 1 \
                or ss_out.numel() < -(-n // 8) * 8:
            raise KernelError("sink shapes: resid and x_out [M, N], gain [N], shares [ceil(N/8), 8]")
    workspace = gemv_tma_reserve(n, k, swiglu, x.device)
    _check(_core("sllm_gemv_tma").sllm_gemv_tma(
        _ptr(x), _ptr(w), _ptr(out), _ptr(workspace), c_int(m), c_int(n), c_int(k),
        c_int64(x.stride(0)), c_int64(w.stride(0)), c_int64(out.stride(0) if out is not None else 0),
        c_int(int(swiglu)), c_int(_code(out.dtype) if out is not None else 1),
        c_int(_sm_count(x.device)), _ptr(ss_in), c_int(ss_parts), c_int(ss_dim), c_float(ss_eps),
        _ptr(resid), c_int64(resid.stride(0) if resid is not None else 0), _ptr(gain), _ptr(x_out),
        c_int64(x_out.stride(0) if x_out is not None else 0), _ptr(ss_out), _stream()), "gemv_tma")
    if sink is not None:    # (counted beside "gemv_tma": which steps handed a norm over)
        launch_counts["gemv_tma_sink"] = launch_counts.get("gemv_tma_sink", 0) + 1
    return out


def gemv_tma_error() -> int:
    """The first error a gemv_tma kernel recorded since the last call (0 = none)."""
    return int(_core("sllm_gemv_tma").sllm_gemv_tma_error())


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, swiglu: bool = False
            ) -> torch.Tensor:
    """out[M, N] = x[M, K] @ w[N, K]^T in bfloat16 on tcgen05 tensor cores (TMA-fed, accumulator
    in tensor memory).  ``swiglu``: w = [gate rows; up rows], out[M, N/2] = silu(gate) * up."""
    _need(x, torch.bfloat16, "x", contiguous=False)
    _need(w, torch.bfloat16, "w", contiguous=False)
    _need(out, torch.bfloat16, "out", contiguous=False)
    (m, k), (n, k2) = x.shape, w.shape
    n_out = n // 2 if swiglu else n
    if k != k2 or out.shape != (m, n_out) or x.stride(1) != 1 or w.stride(1) != 1 \
            or out.stride(1) != 1:
        raise KernelError(f"gemm shapes/strides: x {list(x.shape)}, w {list(w.shape)}, "
                          f"out {list(out.shape)}")
    if k % 8 or x.stride(0) % 8 or w.stride(0) % 8:
        raise KernelError("gemm_tc needs rows that are multiples of 8 elements (16 bytes)")
    _check(_core("sllm_gemm_tcgen05").sllm_gemm_tc(
        _ptr(x), _ptr(w), _ptr(out), c_int(m), c_int(n), c_int(k), c_int64(x.stride(0)),
        c_int64(w.stride(0)), c_int64(out.stride(0)), c_int(int(swiglu)), _stream()), "gemm_tc")
    return out


def gemm_tc_set_pairs(on: bool) -> None:
    """Choose the tcgen05 GEMM kernel: pairs of SMs with 256 x 256 tiles (the default) or single
    SMs with 128 x 256 tiles."""
    _core("sllm_gemm_tcgen05").sllm_gemm_tc_set_pairs(c_int(int(on)))


def gemm_tc_set_tile(features: int | None) -> None:
    """Features per tile of the pair kernel's fused gate/up product: None lets the launcher
    choose (the width whose tiles fill the SM pairs' rounds best), else a multiple of 16 from 16
    to 128."""
    _core("sllm_gemm_tcgen05").sllm_gemm_tc_set_tile(c_int(int(features or 0)))


def gemm_tc_swiglu_tile(m: int, half: int, pairs: int) -> int:
    """The tile width the pair kernel uses for gate/up + SwiGLU of ``m`` tokens and ``half``
    features on ``pairs`` SM pairs."""
    return int(_core("sllm_gemm_tcgen05").sllm_gemm_tc_swiglu_tile(c_int(m), c_int(half),
                                                                   c_int(pairs)))


def gemm_tc_error() -> int:
    """The first error a bounded wait inside gemm_tc recorded since the last call (0 = none).
    Synchronises the device."""
    return int(_core("sllm_gemm_tcgen05").sllm_gemm_tc_error())


# --------------------------------------------------------------------------- rope and cache

def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, token_row: torch.Tensor,
                  cos: torch.Tensor | None, sin: torch.Tensor | None, pages: torch.Tensor,
                  block_table: torch.Tensor, page_size: int, n_heads: int, n_kv_heads: int,
                  head_dim: int, interleaved: bool, write: bool) -> None:
    """Rotate q (in place) and k by their positions' angles; store k and v into the pages.
    ``cos``/``sin`` None stores k as it is (the position encoding was applied before)."""
    _need(qkv, None, "qkv")
    _need(positions, torch.int32, "positions")
    _need(token_row, torch.int32, "token_row")
    _need(pages, qkv.dtype, "pages")
    _need(block_table, torch.int32, "block_table", contiguous=False)
    n = qkv.shape[0]
    if qkv.shape[1] != (n_heads + 2 * n_kv_heads) * head_dim:
        raise KernelError("qkv width does not match the head counts")
    if pages.shape[1:] != (2, n_kv_heads, page_size, head_dim):
        raise KernelError(f"pages must be [n_pages, 2, {n_kv_heads}, {page_size}, {head_dim}], "
                          f"got {list(pages.shape)}")
    rotate = cos is not None
    if rotate:
        _need(cos, torch.float32, "cos")
        _need(sin, torch.float32, "sin")
        if cos.shape[1] != head_dim // 2 or sin.shape != cos.shape:
            raise KernelError("rotary table width")
    if block_table.stride(1) != 1:
        raise KernelError("block_table rows must be contiguous")
    _check(_core("sllm_rope_cache").sllm_rope_kv_write(
        _ptr(qkv), _ptr(positions), _ptr(token_row), _ptr(cos), _ptr(sin), _ptr(pages),
        _ptr(block_table), c_int(block_table.stride(0)), c_int(page_size), c_int(n),
        c_int(n_heads), c_int(n_kv_heads), c_int(head_dim), c_int(int(rotate)),
        c_int(int(interleaved)), c_int(int(write)), c_int(_code(qkv.dtype)), _stream()),
        "rope_kv_write")


# -------------------------------------------------------------------------------- attention

def attention_simt(q: torch.Tensor, pages: torch.Tensor, block_table: torch.Tensor,
                   page_size: int, row_start: torch.Tensor, row_pos0: torch.Tensor,
                   out: torch.Tensor, n_rows: int, max_new: int, n_heads: int, n_kv_heads: int,
                   head_dim: int, scale: float, window: int | None) -> torch.Tensor:
    """Causal attention of the packed batch over the paged cache (CUDA cores, 32-bit math).
    ``q`` may be a column slice of a wider buffer (the fused qkv)."""
    _need(q, None, "q", contiguous=False)
    _need(pages, q.dtype, "pages")
    _need(out, q.dtype, "out", contiguous=False)
    _need(block_table, torch.int32, "block_table", contiguous=False)
    _need(row_start, torch.int32, "row_start")
    _need(row_pos0, torch.int32, "row_pos0")
    if q.stride(1) != 1 or out.stride(1) != 1 or q.shape[1] != n_heads * head_dim \
            or out.shape != q.shape:
        raise KernelError("attention q/out layout")
    if pages.shape[1:] != (2, n_kv_heads, page_size, head_dim):
        raise KernelError(f"pages must be [n_pages, 2, {n_kv_heads}, {page_size}, {head_dim}], "
                          f"got {list(pages.shape)}")
    if head_dim % 16 or not 16 <= head_dim <= 512:
        raise KernelError(f"head size {head_dim}: the attention kernels take multiples of 16 "
                          "from 16 to 512")
    lib = _load(*attention_library(head_dim))
    _check(lib.sllm_attn_simt(
        _ptr(q), c_int64(q.stride(0)), _ptr(pages), _ptr(block_table),
        c_int(block_table.stride(0)), c_int(page_size), _ptr(row_start), _ptr(row_pos0),
        _ptr(out), c_int64(out.stride(0)), c_int(n_rows), c_int(max_new), c_int(n_heads),
        c_int(n_kv_heads), c_float(scale), c_int(window or 0), c_int(_code(q.dtype)),
        _stream()), "attention_simt")
    return out


def attention_mma(q: torch.Tensor, pages: torch.Tensor, block_table: torch.Tensor,
                  page_size: int, row_start: torch.Tensor, row_pos0: torch.Tensor,
                  out: torch.Tensor, row_list: torch.Tensor | None, n_list: int, max_new: int,
                  n_heads: int, n_kv_heads: int, head_dim: int, scale: float,
                  window: int | None, split: bool, n_splits: int = 1,
                  scratch: torch.Tensor | None = None) -> torch.Tensor:
    """Causal attention of the listed rows over the paged cache on the tensor cores
    (bfloat16).  ``split`` False: the wide kernel for rows with many new tokens; True: the
    split kernel for decode rows, ``n_splits`` CTAs along the keys, partial results in
    ``scratch`` (32-bit, :func:`attention_mma_scratch_floats` entries) when ``n_splits`` > 1."""
    _need(q, torch.bfloat16, "q", contiguous=False)
    _need(pages, torch.bfloat16, "pages")
    _need(out, torch.bfloat16, "out", contiguous=False)
    _need(block_table, torch.int32, "block_table", contiguous=False)
    _need(row_start, torch.int32, "row_start")
    _need(row_pos0, torch.int32, "row_pos0")
    if row_list is not None:
        _need(row_list, torch.int32, "row_list")
    if q.stride(1) != 1 or out.stride(1) != 1 or q.shape[1] != n_heads * head_dim \
            or out.shape != q.shape:
        raise KernelError("attention q/out layout")
    if pages.shape[1:] != (2, n_kv_heads, page_size, head_dim):
        raise KernelError(f"pages must be [n_pages, 2, {n_kv_heads}, {page_size}, {head_dim}], "
                          f"got {list(pages.shape)}")
    if head_dim % 16 or not 16 <= head_dim <= MMA_MAX_HEAD_DIM:
        raise KernelError(f"head size {head_dim}: the tensor-core attention kernels take "
                          f"multiples of 16 up to {MMA_MAX_HEAD_DIM}")
    n_tokens = q.shape[0]
    if split and n_splits > 1:
        need = attention_mma_scratch_floats(n_tokens, n_heads, head_dim, n_splits)
        if scratch is None:
            raise KernelError("the split kernel needs scratch memory for its partial results")
        _need(scratch, torch.float32, "scratch")
        if scratch.numel() < need:
            raise KernelError(f"scratch holds {scratch.numel()} floats, {need} are needed")
    lib = _load(*attention_mma_library(head_dim))
    _check(lib.sllm_attn_mma(
        _ptr(q), c_int64(q.stride(0)), _ptr(pages), _ptr(block_table),
        c_int(block_table.stride(0)), c_int(page_size), _ptr(row_start), _ptr(row_pos0),
        _ptr(row_list), c_int(n_list), c_int(max_new), _ptr(out), c_int64(out.stride(0)),
        c_int(n_heads), c_int(n_kv_heads), c_float(scale), c_int(window or 0),
        c_int(int(split)), c_int(n_splits), _ptr(scratch), c_int64(n_tokens), _stream()),
        "attention_mma")
    return out


_decode_slots: dict[tuple[int, int], int] = {}


def attention_decode_slots(head_dim: int) -> int:
    """CTAs of the split decode attention kernel that the current device holds at once (SMs x
    resident CTAs per SM, asked of the occupancy calculator once per device and head size)."""
    key = (torch.cuda.current_device(), head_dim)
    if key not in _decode_slots:
        n = int(_load(*attention_mma_library(head_dim)).sllm_attn_mma_decode_slots())
        if n <= 0:
            raise KernelError("the occupancy of the decode attention kernel could not be read")
        _decode_slots[key] = n
    return _decode_slots[key]


def attention_decode_fused_supported(head_dim: int) -> bool:
    """Whether this head size has the decode attention kernel that rotates q and the new key and
    stores the new key and value itself (head sizes that are multiples of 64)."""
    if head_dim % 16 or not 16 <= head_dim <= MMA_MAX_HEAD_DIM:
        return False
    return bool(_load(*attention_mma_library(head_dim)).sllm_attn_mma_decode_fused_supported())


#: counters of the decode attention's in-kernel merge, per device (zero between launches; a
#: buffer that has been handed to a launch is never freed: a captured graph may hold its address)
_merge_counters: dict[int, list[torch.Tensor]] = {}


def _merge_counter(device: torch.device, n: int) -> torch.Tensor:
    index = device.index if device.index is not None else torch.cuda.current_device()
    held = _merge_counters.setdefault(index, [])
    if not held or held[-1].numel() < n:
        held.append(torch.zeros(max(n, 4096), dtype=torch.int32, device=device))
    return held[-1]


def attention_mma_decode(qkv: torch.Tensor, pages: torch.Tensor, block_table: torch.Tensor,
                         page_size: int, row_start: torch.Tensor, row_pos0: torch.Tensor,
                         out: torch.Tensor, row_list: torch.Tensor | None, n_list: int,
                         n_heads: int, n_kv_heads: int, head_dim: int, scale: float,
                         window: int | None, cos: torch.Tensor, sin: torch.Tensor,
                         interleaved: bool, write: bool, n_splits: int = 1,
                         scratch: torch.Tensor | None = None,
                         merge_inside: bool = True) -> torch.Tensor:
    """Decode attention (rows of one new token) over the paged cache on the tensor cores, for
    head sizes that are multiples of 64, straight from the step's fused projection ``qkv``
    [tokens, (H + 2 G) * hd] as the product left it: the kernel rotates q and the new key itself
    (``cos``/``sin`` tables, adjacent pairs if ``interleaved``) and, if ``write``, stores the new
    key and value into ``pages``: no separate rotate-and-store kernel runs.  ``scratch`` as in
    :func:`attention_mma` for several splits; with ``merge_inside`` the CTA that finishes last for
    a row and kv head merges the splits itself (same arithmetic, no merge kernel, nobody waits),
    else a merge kernel follows.  Launches share the merge's counters per device and must be
    ordered by their stream."""
    _need(qkv, torch.bfloat16, "qkv", contiguous=False)
    _need(pages, torch.bfloat16, "pages")
    _need(out, torch.bfloat16, "out", contiguous=False)
    _need(block_table, torch.int32, "block_table", contiguous=False)
    _need(row_start, torch.int32, "row_start")
    _need(row_pos0, torch.int32, "row_pos0")
    _need(cos, torch.float32, "cos")
    _need(sin, torch.float32, "sin")
    if row_list is not None:
        _need(row_list, torch.int32, "row_list")
    if qkv.stride(1) != 1 or out.stride(1) != 1 \
            or qkv.shape[1] != (n_heads + 2 * n_kv_heads) * head_dim \
            or out.shape != (qkv.shape[0], n_heads * head_dim):
        raise KernelError("attention qkv/out layout")
    if pages.shape[1:] != (2, n_kv_heads, page_size, head_dim):
        raise KernelError(f"pages must be [n_pages, 2, {n_kv_heads}, {page_size}, {head_dim}], "
                          f"got {list(pages.shape)}")
    if not attention_decode_fused_supported(head_dim) or n_heads % n_kv_heads \
            or n_heads // n_kv_heads > 16:
        raise KernelError(f"attention_mma_decode takes head sizes that are multiples of 64 and "
                          f"groups of up to 16 query heads; got {head_dim}, {n_heads}/{n_kv_heads}")
    if cos.shape[1] != head_dim // 2 or sin.shape != cos.shape:
        raise KernelError("rotary table width")
    n_tokens = qkv.shape[0]
    if n_splits > 1:
        need = attention_mma_scratch_floats(n_tokens, n_heads, head_dim, n_splits)
        if scratch is None:
            raise KernelError("several splits need scratch memory for their partial results")
        _need(scratch, torch.float32, "scratch")
        if scratch.numel() < need:
            raise KernelError(f"attention scratch holds {scratch.numel()} floats, {need} needed")
    if block_table.stride(1) != 1:
        raise KernelError("block_table rows must be contiguous")
    counters = _merge_counter(qkv.device, n_list * n_kv_heads) \
        if merge_inside and n_splits > 1 else None
    _check(_load(*attention_mma_library(head_dim)).sllm_attn_mma_decode(
        _ptr(qkv), c_int64(qkv.stride(0)), _ptr(pages), _ptr(block_table),
        c_int(block_table.stride(0)), c_int(page_size), _ptr(row_start), _ptr(row_pos0),
        _ptr(row_list), c_int(n_list), _ptr(out), c_int64(out.stride(0)), c_int(n_heads),
        c_int(n_kv_heads), c_float(scale), c_int(window or 0), c_int(n_splits), _ptr(scratch),
        c_int64(n_tokens), _ptr(cos), _ptr(sin), c_int(int(interleaved)), c_int(int(write)),
        _ptr(counters), _stream()), "attention_mma_decode")
    return out


def attention_tc(q: torch.Tensor, pages: torch.Tensor, block_table: torch.Tensor, page_size: int,
                 row_start: torch.Tensor, row_pos0: torch.Tensor, out: torch.Tensor,
                 row_list: torch.Tensor | None, n_list: int, max_new: int, n_heads: int,
                 n_kv_heads: int, head_dim: int, scale: float) -> torch.Tensor:
    """Causal attention of the listed rows (prompt portions) over the paged cache on tcgen05
    tensor cores with S, P and O in tensor memory.  What the cache holds in places beyond a
    row's context never reaches a result (NaN included)."""
    _need(q, torch.bfloat16, "q", contiguous=False)
    _need(pages, torch.bfloat16, "pages")
    _need(out, torch.bfloat16, "out", contiguous=False)
    _need(block_table, torch.int32, "block_table", contiguous=False)
    _need(row_start, torch.int32, "row_start")
    _need(row_pos0, torch.int32, "row_pos0")
    if row_list is not None:
        _need(row_list, torch.int32, "row_list")
    if not attention_tc_supports(n_heads, n_kv_heads, head_dim, page_size, None):
        raise KernelError("attention_tc does not take this shape")
    if q.stride(1) != 1 or out.stride(1) != 1 or q.shape[1] != n_heads * head_dim \
            or out.shape != q.shape:
        raise KernelError("attention q/out layout")
    if pages.shape[1:] != (2, n_kv_heads, page_size, head_dim):
        raise KernelError(f"pages must be [n_pages, 2, {n_kv_heads}, {page_size}, {head_dim}], "
                          f"got {list(pages.shape)}")
    lib = _load(*attention_tc_library(head_dim))
    _check(lib.sllm_attn_tc(
        _ptr(q), c_int64(q.stride(0)), c_int64(q.shape[0]), _ptr(pages), c_int64(pages.shape[0]),
        _ptr(block_table), c_int(block_table.stride(0)), c_int(page_size), _ptr(row_start),
        _ptr(row_pos0), _ptr(row_list), c_int(n_list), c_int(max_new), _ptr(out),
        c_int64(out.stride(0)), c_int(n_heads), c_int(n_kv_heads), c_float(scale), _stream()),
        "attention_tc")
    return out


def attention_tc_set_two_tiles(head_dim: int, mode: int | bool | None) -> None:
    """Choose the tcgen05 attention kernel for head sizes up to 128.  None (the default):
    two query tiles per CTA, which share every key/value tile, when the launch has at least as
    many such CTAs as the device has SMs, else one; True: always two; False: always one."""
    code = 1 if mode is None else (2 if mode else 0)
    _load(*attention_tc_library(head_dim)).sllm_attn_tc_set_two_tiles(c_int(code))


def attention_tc_error(head_dim: int) -> int:
    return int(_load(*attention_tc_library(head_dim)).sllm_attn_tc_error())


def check_kernel_errors() -> None:
    """Raise if a kernel of a loaded library gave up a bounded wait since the last check (the
    kernels that use mbarriers or flags record a code instead of hanging).  Synchronises the
    device: call it where the host waits anyway (the end of a request batch, of a trace)."""
    found = []
    for name, lib in list(_loaded.items()):
        for symbol in ("sllm_gemm_tc_error", "sllm_gemv_tma_error", "sllm_attn_tc_error"):
            if hasattr(lib, symbol):
                code = int(getattr(lib, symbol)())
                if code:
                    found.append(f"{name}: code {code}")
    if found:
        raise KernelError("a kernel gave up waiting (its results are not valid): " +
                          "; ".join(found))


def attention_mma_scratch_floats(n_tokens: int, n_heads: int, head_dim: int, n_splits: int) -> int:
    return n_tokens * n_heads * n_splits * (head_dim + 1) if n_splits > 1 else 0


# --------------------------------------------------------------------------------- sampling

def argmax_scratch_bytes(n_rows: int) -> int:
    lib = _core("sllm_sampling")
    lib.sllm_argmax_scratch_bytes.restype = c_int64
    return int(lib.sllm_argmax_scratch_bytes(c_int(n_rows)))


def argmax(logits: torch.Tensor, out: torch.Tensor, scratch: torch.Tensor, rows_capacity: int
           ) -> torch.Tensor:
    """out[r] = first maximum of logits[r] (32-bit, [n, V]), many blocks per row.  ``scratch``:
    uint8 of ``argmax_scratch_bytes(rows_capacity)``, zero-filled once; its layout depends on
    ``rows_capacity``, which must be the same on every call with this scratch."""
    _need(logits, torch.float32, "logits", contiguous=False)
    _need(out, torch.int32, "out")
    _need(scratch, torch.uint8, "scratch")
    n, v = logits.shape
    if logits.stride(1) != 1 or out.numel() != n or n != rows_capacity \
            or scratch.numel() < argmax_scratch_bytes(rows_capacity):
        raise KernelError("argmax shapes")
    _check(_core("sllm_sampling").sllm_argmax(
        _ptr(logits), c_int64(logits.stride(0)), c_int(n), c_int(v), _ptr(scratch), _ptr(out),
        _stream()), "argmax")
    return out


def sample(logits: torch.Tensor, out: torch.Tensor, temperature: torch.Tensor | None = None,
           top_p: torch.Tensor | None = None, seed: torch.Tensor | None = None,
           counter: torch.Tensor | None = None, logprob_out: torch.Tensor | None = None,
           probs_out: torch.Tensor | None = None) -> torch.Tensor:
    """Choose one token per row of ``logits`` [n, V] (32-bit).  Rows whose temperature is 0
    (or all rows when ``temperature`` is None) take the argmax.  seed/counter: int64 [n]."""
    _need(logits, torch.float32, "logits", contiguous=False)
    _need(out, torch.int32, "out")
    n, v = logits.shape
    if logits.stride(1) != 1 or out.numel() != n:
        raise KernelError("sample shapes")
    for t, dt, name in ((temperature, torch.float32, "temperature"), (top_p, torch.float32, "top_p"),
                        (seed, torch.int64, "seed"), (counter, torch.int64, "counter"),
                        (logprob_out, torch.float32, "logprob_out")):
        if t is not None:
            _need(t, dt, name)
            if t.numel() != n:
                raise KernelError(f"{name} must have one entry per row")
    if probs_out is not None:
        _need(probs_out, torch.float32, "probs_out")
        if probs_out.shape != (n, v):
            raise KernelError("probs_out shape")
    _check(_core("sllm_sampling").sllm_sample(
        _ptr(logits), c_int64(logits.stride(0)), c_int(n), c_int(v), _ptr(temperature),
        _ptr(top_p), _ptr(seed), _ptr(counter), _ptr(out), _ptr(logprob_out), _ptr(probs_out),
        _stream()), "sample")
    return out


def log_softmax(logits: torch.Tensor, rows_out: torch.Tensor | None = None,
                taken: torch.Tensor | None = None, taken_out: torch.Tensor | None = None) -> None:
    """log_softmax of each row of ``logits`` [n, V] (32-bit).  ``rows_out`` [n, V] gets the whole
    rows; ``taken`` (int32 [n]) and ``taken_out`` (float32 [n]) the log-probability of one given
    token per row."""
    _need(logits, torch.float32, "logits", contiguous=False)
    n, v = logits.shape
    if logits.stride(1) != 1:
        raise KernelError("log_softmax: rows must be contiguous")
    if rows_out is not None:
        _need(rows_out, torch.float32, "rows_out")
        if rows_out.shape != (n, v):
            raise KernelError("rows_out shape")
    if (taken is None) != (taken_out is None):
        raise KernelError("taken and taken_out come together")
    if taken is not None:
        _need(taken, torch.int32, "taken")
        _need(taken_out, torch.float32, "taken_out")
        if taken.numel() != n or taken_out.numel() != n:
            raise KernelError("taken / taken_out must have one entry per row")
    _check(_core("sllm_sampling").sllm_log_softmax(
        _ptr(logits), c_int64(logits.stride(0)), c_int(n), c_int(v), _ptr(rows_out), _ptr(taken),
        _ptr(taken_out), _stream()), "log_softmax")
