"""Gamesun: a decoder whose layers are listed one by one in ``config.json``, each with two mixers side by side
(attention over a sliding window beside linear attention with a state of fixed size) and a gated feed-forward.

``config.json`` keys: ``architecture`` ("Gamesun"), ``vocab``, ``width``, ``norm.eps``, ``embedding.scale`` and
``layers``, a list of ``{"type", "mixer": {"left", "right"}, "mlp"}``.  ``type`` names the pair of mixers:

* ``parallel``: left = windowed attention with biases, the heads' scores mixed by ``talk``, a number per head added
  (``pb``) and sigmoid weights; right = linear attention with a decay per key channel (``tau``, low-rank decay products);
* ``parallel_2``: left = windowed softmax attention with a number per head multiplied into the score (``temp``);
  right = linear attention with a constant decay per head (``decay``).

``left`` holds ``heads, kv_heads, dim, vdim, scale, mask.size`` (the window), ``right`` holds ``heads, dim, vdim`` and
``tau`` or ``decay``; ``mlp`` is ``null`` or ``{"kind": "dense", "ff"}`` (silu(gate) * up, then down).  The embedding
rows are multiplied by ``embedding.scale`` and a sinusoidal position vector (base 10000) is added; the output head is
the embedding table itself.  Every layer is a pre-norm residual block with plain RMS-norm weights.  Tensor names:
``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.left.*``, ``l<i>.mix.right.*``, ``l<i>.mix.left.out``,
``l<i>.mix.right.out``, ``l<i>.mlp.gate|up|down``, ``final.norm``.  Nothing here fixes a size.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from ..config.model_spec import LayerSpec, ModelSpec, PartSpec, sequential_schedule
from ..config.registry import register_architecture
from .rapitar import _need

LAYER_TYPES = ("parallel", "parallel_2")
POSITION_BASE = 10000.0  # of the sinusoidal position vector; the design fixes it
PAIR_FACTOR = 0.5        # a layer's mixer is half the sum of its two normed mixers


@dataclass(frozen=True)
class GamesunConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    layers: tuple  # of (mixer PartSpec, feed-forward PartSpec)
    raw: dict


def _layers_2k(repeats: int) -> list:
    """Layer sizes of a model of 2,048 width: 16 query heads of 128 on 4 key/value heads; windows of 1,024 and 4,096;
    linear attention of 16 heads of 128; a feed-forward of 3.5 widths."""
    dense = {"kind": "dense", "ff": 7168}
    soft = {"type": "parallel_2", "mlp": dense, "mixer": {
        "left": {"heads": 16, "kv_heads": 4, "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "mask": {"size": 4096}},
        "right": {"heads": 16, "dim": 128, "vdim": 128, "decay": [1.0 - 2.0 ** (-5 - 3 * h / 15) for h in range(16)]}}}
    gated = {"type": "parallel", "mlp": dense, "mixer": {
        "left": {"heads": 16, "kv_heads": 4, "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "mask": {"size": 1024}},
        "right": {"heads": 16, "dim": 64, "vdim": 128, "tau": 16.0, "decay_rank": 16}}}
    return [soft, gated] * repeats


class GamesunArchitecture:
    name = "Gamesun"
    layer_count_key = None  # the layers are a list: a shape with fewer layers is another list
    named_shapes = {
        "gamesun-2k": {"architecture": "Gamesun", "vocab": 32768, "width": 2048, "norm": {"eps": 1e-6},
                       "embedding": {"scale": 45.25}, "layers": _layers_2k(4)},
        "gamesun-tiny": {"architecture": "Gamesun", "vocab": 256, "width": 64, "norm": {"eps": 1e-6}, "embedding": {"scale": 8.0},
                         "layers": [
            {"type": "parallel_2", "mlp": {"kind": "dense", "ff": 96}, "mixer": {
                "left": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.25, "mask": {"size": 24}},
                "right": {"heads": 2, "dim": 16, "vdim": 16, "decay": [0.9, 0.99]}}},
            {"type": "parallel", "mlp": None, "mixer": {
                "left": {"heads": 2, "kv_heads": 1, "dim": 24, "vdim": 16, "scale": 0.2, "mask": {"size": 9}},
                "right": {"heads": 2, "dim": 8, "vdim": 16, "tau": 8.0, "decay_rank": 4}}}]},
    }

    @staticmethod
    def _mixer(kind: str, m: dict[str, Any], width: int, eps: float, where: str) -> PartSpec:
        if kind not in LAYER_TYPES:
            raise ValueError(f"config.json: {where}: unknown layer type {kind!r}; known: {list(LAYER_TYPES)}")
        left, right = m.get("left") or {}, m.get("right") or {}
        lw, rw = where + ".left", where + ".right"
        gated = kind == "parallel"
        attention = dict(hidden_size=width, heads=_need(left, "heads", lw), kv_heads=_need(left, "kv_heads", lw),
                         dim=_need(left, "dim", lw), vdim=_need(left, "vdim", lw), scale=_need(left, "scale", lw, float),
                         window=_need(left.get("mask") or {}, "size", lw + ".mask"), bias=gated, talk=gated, head_bias=gated,
                         head_scale=not gated, weights="sigmoid" if gated else "softmax")
        linear = dict(hidden_size=width, heads=_need(right, "heads", rw), dim=_need(right, "dim", rw), vdim=_need(right, "vdim", rw),
                      eps=eps)
        if gated:
            linear.update(tau=_need(right, "tau", rw, float), decay_rank=right.get("decay_rank"))
            right_spec = PartSpec("gated_linear", linear)
        else:
            decay = right.get("decay")
            if not isinstance(decay, list) or len(decay) != linear["heads"] or any(isinstance(d, bool) or not isinstance(d, (int, float)) for d in decay):
                raise ValueError(f"config.json: {rw}.decay must list one number per head ({linear['heads']}), got {decay!r}")
            linear.update(decay=[float(d) for d in decay])
            right_spec = PartSpec("decay_linear", linear)
        return PartSpec("side_by_side", dict(hidden_size=width, eps=eps, factor=PAIR_FACTOR,
                                             left=PartSpec("window_attention", attention), right=right_spec))

    @staticmethod
    def _ffn(f, width: int, where: str) -> PartSpec:
        if f is None:
            return PartSpec("none", {})
        if f.get("kind") != "dense":
            raise ValueError(f"config.json: {where}: unknown feed-forward kind {f.get('kind')!r}")
        return PartSpec("swiglu", dict(hidden_size=width, intermediate_size=_need(f, "ff", where), names=("gate", "up", "down")))

    def parse_config(self, raw: dict[str, Any]) -> GamesunConfig:
        width = _need(raw, "width", "the model")
        eps = _need(raw.get("norm") or {}, "eps", "norm", float)
        scale = _need(raw.get("embedding") or {}, "scale", "embedding", float)
        listed = raw.get("layers")
        if not isinstance(listed, list) or not listed:
            raise ValueError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(listed):
            where = f"layers[{i}]"
            layers.append((self._mixer(entry.get("type"), entry.get("mixer") or {}, width, eps, where + ".mixer"),
                           self._ffn(entry.get("mlp"), width, where + ".mlp")))
        return GamesunConfig(_need(raw, "vocab", "the model"), width, eps, scale, tuple(layers), dict(raw))

    def model_spec(self, config: GamesunConfig) -> ModelSpec:
        norm = PartSpec("rmsnorm", {"size": config.width, "eps": config.eps, "weight_suffix": ""})
        layers = [LayerSpec(block="prenorm_residual_short", mixer=mixer, ffn=ffn, mixer_norm=norm, ffn_norm=norm, prefix=f"l{i}")
                  for i, (mixer, ffn) in enumerate(config.layers)]
        return ModelSpec(architecture=self.name, vocab_size=config.vocab, hidden_size=config.width, layers=layers,
                         schedule=sequential_schedule(len(layers)), final_norm=norm, embedding_name="embed",
                         final_norm_prefix="final.norm", head_name="head", tie_word_embeddings=True,
                         embedding_scale=config.embedding_scale,
                         absolute_positions=PartSpec("sinusoidal_absolute", {"size": config.width, "base": POSITION_BASE}),
                         raw=config.raw)


register_architecture(GamesunArchitecture(), replace=True)
