"""Feed-forwards besides SwiGLU: a dense two-matrix layer with GELU, and a mixture of experts.

``gelu_mlp``: ``down(gelu_tanh(up(x)))``, no biases.  Parameters: ``hidden_size, intermediate_size``;
tensors ``up`` [I, H], ``down`` [H, I].

``moe``: ``experts`` SwiGLU experts without biases (``e<i>.gate``, ``e<i>.up`` [F, H], ``e<i>.down``
[H, F]), a router ``router`` [E, H] with bias ``router.b``.  Router logits are a product with float32
accumulation and stay float32; each token takes
the ``top`` experts with the largest logits, weighted by the softmax over the chosen logits only; the
output is the weighted sum of the chosen experts' outputs, added into the float32 residual in the order
of the choices.  Tokens are grouped by expert on the device (no host round trip), so the part is safe
to capture in a CUDA graph.  Parameters: ``hidden_size, expert_size, experts, top``.
"""

from __future__ import annotations

import torch

from ..ops import grouped as grouped_ops
from ..ops import recurrence as rec_ops
from ..weights.decl import TensorDecl
from .base import FeedForward, ResidualStream, StepContext
from .linear import Linear
from .registry import register_ffn


class GeluMLP(FeedForward):
    graph_safe = True
    graph_safe_portions = True

    def __init__(self, spec, prefix, dtype, device) -> None:
        super().__init__(spec, prefix, dtype, device)
        self.hidden_size = int(spec["hidden_size"])
        self.intermediate_size = int(spec["intermediate_size"])
        self.up: Linear | None = None
        self.down: Linear | None = None

    def tensor_decls(self):
        h, i = self.hidden_size, self.intermediate_size
        yield TensorDecl(self.name("up"), (i, h), "matrix", "linear")
        yield TensorDecl(self.name("down"), (h, i), "matrix", "linear")

    def load_weights(self, fetch) -> None:
        self.up = Linear(fetch(self.name("up")))
        self.down = Linear(fetch(self.name("down")))

    def forward(self, ctx: StepContext, x, stream: ResidualStream):
        act = rec_ops.activation_(self.up(x), rec_ops.ACT_GELU_TANH)
        return self.down.add_or_defer(act, stream)


class MixtureOfExperts(FeedForward):
    graph_safe = True
    graph_safe_portions = True

    def __init__(self, spec, prefix, dtype, device) -> None:
        super().__init__(spec, prefix, dtype, device)
        self.hidden_size = int(spec["hidden_size"])
        self.expert_size = int(spec["expert_size"])
        self.experts = int(spec["experts"])
        self.top = int(spec["top"])
        if not 0 < self.top <= self.experts:
            raise ValueError(f"top {self.top} must lie in 1..experts ({self.experts})")
        self.w_gate = self.w_up = self.w_down = self.router = self.router_bias = None

    def tensor_decls(self):
        h, f = self.hidden_size, self.expert_size
        for e in range(self.experts):
            yield TensorDecl(self.name(f"e{e}.gate"), (f, h), "matrix", "linear")
            yield TensorDecl(self.name(f"e{e}.up"), (f, h), "matrix", "linear")
            yield TensorDecl(self.name(f"e{e}.down"), (h, f), "matrix", "linear")
        yield TensorDecl(self.name("router"), (self.experts, h), "matrix", "linear")
        yield TensorDecl(self.name("router.b"), (self.experts,), "vector", "bias")

    def load_weights(self, fetch) -> None:
        stack = lambda what: torch.stack([fetch(self.name(f"e{e}.{what}")) for e in range(self.experts)]).contiguous()  # noqa: E731
        self.w_gate, self.w_up, self.w_down = stack("gate"), stack("up"), stack("down")
        self.router = Linear(fetch(self.name("router")))
        self.router_bias = fetch(self.name("router.b"))

    def forward(self, ctx: StepContext, x, stream: ResidualStream):
        sel, weights = grouped_ops.moe_choose(self.router.to_float32(x), self.router_bias, ctx.tok_seq, self.top)
        offsets, order = grouped_ops.moe_group(sel, self.experts)
        act = grouped_ops.expert_gate_up(x, self.w_gate, self.w_up, offsets, order, self.top)
        y = grouped_ops.expert_down(act, self.w_down, offsets, order)
        grouped_ops.moe_combine(stream.residual_after_flush(), y, sel, weights)
        return None


register_ffn("gelu_mlp", GeluMLP, replace=True)
register_ffn("moe", MixtureOfExperts, replace=True)
