"""Parallel residual block: a single norm feeds the mixer and the feed-forward alike:
``n = norm(h); h += mixer(n) + ffn(n)``.

Tensor prefixes: ``<layer>.norm1``, ``<layer>.mix``, ``<layer>.mlp`` (the names of the Rapitar
checkpoints).  A layer without a feed-forward names the kind ``none``.  The sublayers' output
products add into the float32 residual in their epilogues, the mixer first, so the sum is
``(h + mixer) + ffn`` in float32 whatever the run precision.
"""

from __future__ import annotations

from ..config.model_spec import LayerSpec
from .base import Block, ResidualStream, StepContext
from .registry import build_part, register_block


class ParallelResidualBlock(Block):
    def __init__(self, layer: LayerSpec, dtype, device) -> None:
        self.layer = layer
        self.prefix = layer.prefix
        self.dtype, self.device = dtype, device
        self.norm = build_part("norm", layer.mixer_norm, f"{layer.prefix}.norm1", dtype, device)
        self.mixer = build_part("mixer", layer.mixer, f"{layer.prefix}.mix", dtype, device)
        self.ffn = None if layer.ffn.kind == "none" else build_part("ffn", layer.ffn, f"{layer.prefix}.mlp", dtype, device)

    def parts(self):
        return (self.norm, self.mixer) + (() if self.ffn is None else (self.ffn,))

    @property
    def graph_safe(self) -> bool:
        return all(part.graph_safe for part in self.parts())

    def tensor_decls(self):
        for part in self.parts():
            yield from part.tensor_decls()

    def load_weights(self, fetch) -> None:
        for part in self.parts():
            part.load_weights(fetch)

    def first_norm(self):
        return self.norm

    def forward(self, ctx: StepContext, stream: ResidualStream, view, following_norm=None) -> None:
        x = self.norm.forward(stream, ctx.status)  # a plain tensor: two sublayers read it
        stream.next_norm = None if self.ffn is not None else following_norm
        stream.push(self.mixer.forward(ctx, x, view, stream))
        if self.ffn is not None:
            stream.next_norm = following_norm  # what the feed-forward's last product may begin or leave in parts
            stream.push(self.ffn.forward(ctx, x, stream))
        stream.next_norm = None


register_block("parallel_residual", ParallelResidualBlock, replace=True)
