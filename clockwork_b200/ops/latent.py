"""Python faces of the kernels for attention over a cached latent (``csrc/latent_attention.cu``)."""

from __future__ import annotations

import torch

from . import _need, _ptr, _stream, dtype_code
from .library import check, library


def set_tensor_cores(on: bool) -> None:
    """bfloat16 attention over the latent runs on the tensor cores when its sizes allow (the default); ``False`` keeps
    it on the CUDA-core kernel that float32 runs use (for comparisons)."""
    library().cw_latent_attention_set_mma(1 if on else 0)


def latent_prepare(down: torch.Tensor, q: torch.Tensor, qa: torch.Tensor, view, norm_weight: torch.Tensor,
                   inv_freq: torch.Tensor, positions: torch.Tensor, heads: int, dim: int, rot: int, rank: int, eps: float,
                   status: torch.Tensor) -> None:
    """Writes each token's cache row [normed latent | rotated shared key part] at its slot and the rotated
    parts of the queries into ``qa`` [N, heads*(rank+rot)] at [.., rank:] of every head."""
    _need(down, torch.float32, "down", 2)
    _need(q, None, "q", 2)
    _need(qa, q.dtype, "qa", 2)
    cache = view.k_cache
    _need(cache, q.dtype, "cache", 4)
    n = q.shape[0]
    if down.shape[1] != rank + rot or q.shape[1] != heads * (dim + rot) or qa.shape[1] != heads * (rank + rot):
        raise ValueError("widths do not match the head count and sizes")
    if cache.shape[2] * cache.shape[3] != rank + rot:
        raise ValueError("cache rows do not hold rank + rot numbers")
    write = bool(view.write)
    check(library().cw_latent_prepare(_ptr(down), _ptr(q), _ptr(qa), _ptr(cache), _ptr(norm_weight), _ptr(inv_freq), _ptr(positions),
                                      _ptr(view.slots), n, heads, dim, rot, rank, cache.shape[0] * cache.shape[1], float(eps),
                                      1 if write else 0, dtype_code(q.dtype), _ptr(status), _stream()), "latent_prepare")


def latent_attention(qa: torch.Tensor, view, ctx, sink: torch.Tensor | None, heads: int, rank: int, rot: int,
                     scale: float) -> torch.Tensor:
    """[N, heads*rank]: per head the softmax-weighted sum of the cached latents (the sink in the denominator)."""
    _need(qa, None, "qa", 2)
    cache = view.k_cache
    n = qa.shape[0]
    out = torch.empty((n, heads * rank), dtype=qa.dtype, device=qa.device)
    check(library().cw_latent_attention(_ptr(qa), _ptr(out), _ptr(cache), _ptr(view.block_tables), _ptr(ctx.tok_seq),
                                        _ptr(ctx.positions), _ptr(sink), n, heads, rank, rot, cache.shape[1],
                                        view.block_tables.shape[1], cache.shape[0], float(scale), dtype_code(qa.dtype),
                                        _ptr(ctx.status), _stream()), "latent_attention")
    return out
