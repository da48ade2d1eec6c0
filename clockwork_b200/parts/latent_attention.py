"""Attention that caches a latent instead of keys and values, with a softmax sink and an output gate.

Parameters: ``hidden_size, heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, rope_base, eps``.
Tensors: ``dq`` [q_rank, H], ``dq.norm`` [q_rank], ``uq`` [heads*(dim+rot_dim), q_rank], ``dkv``
[kv_rank+rot_dim, H], ``dkv.norm`` [kv_rank], ``uk`` [heads*dim, kv_rank], ``uv`` [heads*vdim, kv_rank],
``sink`` [heads], ``g`` [heads*vdim, H], ``o`` [H, heads*vdim].

Queries: ``c_q = rmsnorm(dq x) * dq.norm``, ``q = uq c_q``, per head ``[dim plain | rot_dim rotated]``.
Keys and values: the first kv_rank rows of ``dkv x``, RMS-normed with ``dkv.norm``, are the latent c;
the last rot_dim are one rotated key part shared by all heads (rotate-half pairing, angle
``p * base^(-2i/rot_dim)``).  Per head the plain key is ``uk c`` and the value ``uv c``; the score is
``(q_plain . k_plain + q_rot . k_rot) * scale``, causal, and the softmax denominator also holds
``exp(sink_h)``.  The heads' outputs are multiplied by ``sigmoid(g x)`` and go through ``o``.

Only ``[c | k_rot]`` is cached (one row of kv_rank + rot_dim numbers per token, one plane of pages).
The per-head products are moved to the query side: the query row of a head is ``[uk_h^T q_plain | q_rot]``
and the kernel returns ``sum_j p_j c_j`` per head, which ``uv_h`` then maps to the head's value
(``csrc/latent_attention.cu``).
"""

from __future__ import annotations

import torch

from .. import ops
from ..ops import grouped as grouped_ops
from ..ops import latent as latent_ops
from ..weights.decl import TensorDecl
from .base import Mixer, PagedKVNeed, PagedView, ResidualStream, StepContext
from .linear import Linear
from .registry import register_mixer


class LatentAttention(Mixer):
    graph_safe = True
    graph_safe_portions = True

    def __init__(self, spec, prefix, dtype, device) -> None:
        super().__init__(spec, prefix, dtype, device)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.heads, self.dim, self.rot, self.vdim = int(p["heads"]), int(p["dim"]), int(p["rot_dim"]), int(p["vdim"])
        self.kv_rank, self.q_rank = int(p["kv_rank"]), int(p["q_rank"])
        self.scale, self.eps, self.base = float(p["scale"]), float(p["eps"]), float(p["rope_base"])
        if self.rot % 2:
            raise ValueError(f"rot_dim {self.rot} must be even")
        # float32 angles' frequencies, computed on the host in float64 and rounded once
        half = self.rot // 2
        self.inv_freq = torch.tensor([self.base ** (-2.0 * i / self.rot) for i in range(half)] or [0.0],
                                     dtype=torch.float32).to(device)

    def cache_need(self) -> PagedKVNeed:
        return PagedKVNeed(1, self.kv_rank + self.rot, None, planes=1)

    def tensor_decls(self):
        h, heads = self.hidden_size, self.heads
        yield TensorDecl(self.name("dq"), (self.q_rank, h), "matrix", "linear")
        yield TensorDecl(self.name("dq.norm"), (self.q_rank,), "vector", "norm")
        yield TensorDecl(self.name("uq"), (heads * (self.dim + self.rot), self.q_rank), "matrix", "linear")
        yield TensorDecl(self.name("dkv"), (self.kv_rank + self.rot, h), "matrix", "linear")
        yield TensorDecl(self.name("dkv.norm"), (self.kv_rank,), "vector", "norm")
        yield TensorDecl(self.name("uk"), (heads * self.dim, self.kv_rank), "matrix", "linear")
        yield TensorDecl(self.name("uv"), (heads * self.vdim, self.kv_rank), "matrix", "linear")
        yield TensorDecl(self.name("sink"), (heads,), "vector", "bias")
        yield TensorDecl(self.name("g"), (heads * self.vdim, h), "matrix", "linear")
        yield TensorDecl(self.name("o"), (h, heads * self.vdim), "matrix", "linear")

    def load_weights(self, fetch) -> None:
        self.dq, self.uq, self.dkv = Linear(fetch(self.name("dq"))), Linear(fetch(self.name("uq"))), Linear(fetch(self.name("dkv")))
        self.dq_norm, self.dkv_norm = fetch(self.name("dq.norm")), fetch(self.name("dkv.norm"))
        # per head [kv_rank, dim]: the key product's transpose, applied to the query instead of the latent
        self.uk_t = fetch(self.name("uk")).view(self.heads, self.dim, self.kv_rank).transpose(1, 2).contiguous()
        self.uv = fetch(self.name("uv")).view(self.heads, self.vdim, self.kv_rank).contiguous()
        self.sink = fetch(self.name("sink"))
        self.gate, self.o = Linear(fetch(self.name("g"))), Linear(fetch(self.name("o")))

    def forward(self, ctx: StepContext, x, view: PagedView, stream: ResidualStream):
        n, heads, rank, rot = x.shape[0], self.heads, self.kv_rank, self.rot
        c_q = ops.add_rmsnorm(self.dq.to_float32(x), None, self.dq_norm, self.eps, self.dtype, ctx.status)
        q = self.uq(c_q)                      # [N, heads*(dim+rot)]
        down = self.dkv.to_float32(x)         # [N, kv_rank+rot], float32: the latent is normed from it
        qa = torch.empty((n, heads * (rank + rot)), dtype=self.dtype, device=x.device)
        latent_ops.latent_prepare(down, q, qa, view, self.dkv_norm, self.inv_freq, ctx.positions, heads, self.dim, rot, rank,
                                  self.eps, ctx.status)
        grouped_ops.per_head_product(q, self.dim + rot, self.uk_t, qa, rank + rot)
        mixed = latent_ops.latent_attention(qa, view, ctx, self.sink, heads, rank, rot, self.scale)  # [N, heads*rank]
        out = torch.empty((n, heads * self.vdim), dtype=self.dtype, device=x.device)
        grouped_ops.per_head_product(mixed, rank, self.uv, out, self.vdim, gate=self.gate(x))
        return self.o.add_or_defer(out, stream)


register_mixer("latent_attention", LatentAttention, replace=True)
