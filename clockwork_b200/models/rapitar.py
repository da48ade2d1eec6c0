"""Rapitar: a decoder whose layers are listed one by one in ``config.json``.

``config.json`` keys: ``architecture`` ("Rapitar"), ``vocab``, ``width``, ``norm.eps`` and ``layers``, a
list of ``{"type", "mixer", "mlp"}``: ``type`` names the layer's mixer (``mamba2``, ``wkv`` or
``latent_attention``), ``mixer`` holds that mixer's sizes and constants, ``mlp`` is ``null`` (no
feed-forward), ``{"kind": "dense", "ff"}`` or ``{"kind": "moe", "expert": {"ff"}, "router": {"experts",
"top"}}``.  Every layer is a parallel residual block (a single norm, whose stored weight is the distance from one,
feeds mixer and feed-forward).  Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.mix.*``, ``l<i>.mlp.*``,
``final.norm``, ``head``.  Nothing here fixes a size: another model of the design has other sizes,
another order of layers and other constants.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from ..config.model_spec import LayerSpec, ModelSpec, PartSpec, sequential_schedule
from ..config.registry import register_architecture

MIXER_TYPES = ("mamba2", "wkv", "latent_attention")


def _need(raw: dict[str, Any], key: str, where: str, kind=int):
    if not isinstance(raw, dict) or key not in raw or raw[key] is None:
        raise ValueError(f"config.json: {where} lacks {key!r}")
    value = raw[key]
    if kind is int:
        if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
            raise ValueError(f"config.json: {where}.{key} must be a positive integer, got {value!r}")
        return value
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ValueError(f"config.json: {where}.{key} must be a number, got {value!r}")
    return float(value)


@dataclass(frozen=True)
class RapitarConfig:
    vocab: int
    width: int
    eps: float
    layers: tuple  # of (mixer PartSpec, feed-forward PartSpec)
    raw: dict


def _layers_2k(repeats: int) -> list:
    """Layer sizes of published models of about 2,048 width: a time-mixing layer of 32 heads of 64, latent attention
    of 16 heads over a latent of 512 + 64, a state-space layer of 64 heads of 64 with 128 states; dense feed-forwards
    of 3.5 widths and 64 experts of 1,408 of which 6 are chosen."""
    dense = {"kind": "dense", "ff": 7168}
    moe = {"kind": "moe", "expert": {"ff": 1408}, "router": {"experts": 64, "top": 6}}
    wkv = {"type": "wkv", "mixer": {"heads": 32, "dim": 64, "decay_rank": 64}, "mlp": dense}
    latent = {"type": "latent_attention", "mlp": moe,
              "mixer": {"heads": 16, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": 512, "q_rank": 1536,
                        "rot": {"base": 10000.0, "dims": 64}, "scale": 192 ** -0.5}}
    mamba = {"heads": 64, "vdim": 64, "state": 128, "groups": 1, "conv": 4, "norm_groups": 1}
    return [wkv, latent, {"type": "mamba2", "mixer": mamba, "mlp": moe}, {"type": "mamba2", "mixer": mamba, "mlp": dense}] * repeats


class RapitarArchitecture:
    name = "Rapitar"
    layer_count_key = None  # the layers are a list: a shape with fewer layers is another list
    # config.json contents of the sizes that the benchmarks and the command line know by name
    named_shapes = {
        "rapitar-2k": {"architecture": "Rapitar", "vocab": 32768, "width": 2048, "norm": {"eps": 1e-6}, "layers": _layers_2k(2)},
        "rapitar-tiny": {"architecture": "Rapitar", "vocab": 256, "width": 64, "norm": {"eps": 1e-6}, "layers": [
            {"type": "wkv", "mixer": {"heads": 2, "dim": 16, "decay_rank": 8}, "mlp": {"kind": "dense", "ff": 96}},
            {"type": "latent_attention", "mlp": {"kind": "moe", "expert": {"ff": 32}, "router": {"experts": 4, "top": 2}},
             "mixer": {"heads": 2, "dim": 16, "rot_dim": 8, "vdim": 16, "kv_rank": 24, "q_rank": 16,
                       "rot": {"base": 10000.0, "dims": 8}, "scale": 0.2}},
            {"type": "mamba2", "mixer": {"heads": 2, "vdim": 16, "state": 8, "groups": 1, "conv": 4, "norm_groups": 1}, "mlp": None}]},
    }

    @staticmethod
    def _mixer(kind: str, m: dict[str, Any], width: int, eps: float, where: str) -> PartSpec:
        if kind == "mamba2":
            return PartSpec("mamba2", dict(hidden_size=width, heads=_need(m, "heads", where), vdim=_need(m, "vdim", where),
                                           state=_need(m, "state", where), groups=_need(m, "groups", where),
                                           conv=_need(m, "conv", where), norm_groups=_need(m, "norm_groups", where), eps=eps))
        if kind == "wkv":
            return PartSpec("wkv", dict(hidden_size=width, heads=_need(m, "heads", where), dim=_need(m, "dim", where),
                                        decay_rank=m.get("decay_rank"), eps=eps))
        if kind == "latent_attention":
            rot = m.get("rot") or {}
            rot_dim = _need(m, "rot_dim", where)
            if int(rot.get("dims", rot_dim)) != rot_dim:
                raise ValueError(f"config.json: {where}: rot.dims {rot.get('dims')} differs from rot_dim {rot_dim}")
            return PartSpec("latent_attention", dict(
                hidden_size=width, heads=_need(m, "heads", where), dim=_need(m, "dim", where), rot_dim=rot_dim,
                vdim=_need(m, "vdim", where), kv_rank=_need(m, "kv_rank", where), q_rank=_need(m, "q_rank", where),
                scale=_need(m, "scale", where, float), rope_base=_need(rot, "base", where + ".rot", float), eps=eps))
        raise ValueError(f"config.json: {where}: unknown layer type {kind!r}; known: {list(MIXER_TYPES)}")

    @staticmethod
    def _ffn(f, width: int, where: str) -> PartSpec:
        if f is None:
            return PartSpec("none", {})
        kind = f.get("kind")
        if kind == "dense":
            return PartSpec("gelu_mlp", dict(hidden_size=width, intermediate_size=_need(f, "ff", where)))
        if kind == "moe":
            router = f.get("router") or {}
            return PartSpec("moe", dict(hidden_size=width, expert_size=_need(f.get("expert") or {}, "ff", where + ".expert"),
                                        experts=_need(router, "experts", where + ".router"),
                                        top=_need(router, "top", where + ".router")))
        raise ValueError(f"config.json: {where}: unknown feed-forward kind {kind!r}")

    def parse_config(self, raw: dict[str, Any]) -> RapitarConfig:
        width = _need(raw, "width", "the model")
        eps = _need(raw.get("norm") or {}, "eps", "norm", float)
        listed = raw.get("layers")
        if not isinstance(listed, list) or not listed:
            raise ValueError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(listed):
            where = f"layers[{i}]"
            kind = entry.get("type")
            layers.append((self._mixer(kind, entry.get("mixer") or {}, width, eps, where + ".mixer"),
                           self._ffn(entry.get("mlp"), width, where + ".mlp")))
        return RapitarConfig(_need(raw, "vocab", "the model"), width, eps, tuple(layers), dict(raw))

    def model_spec(self, config: RapitarConfig) -> ModelSpec:
        norm = PartSpec("rmsnorm", {"size": config.width, "eps": config.eps, "offset": 1.0, "weight_suffix": ""})
        layers = [LayerSpec(block="parallel_residual", mixer=mixer, ffn=ffn, mixer_norm=norm, ffn_norm=norm, prefix=f"l{i}")
                  for i, (mixer, ffn) in enumerate(config.layers)]
        return ModelSpec(architecture=self.name, vocab_size=config.vocab, hidden_size=config.width, layers=layers,
                         schedule=sequential_schedule(len(layers)), final_norm=norm, embedding_name="embed",
                         final_norm_prefix="final.norm", head_name="head", tie_word_embeddings=False, raw=config.raw)


register_architecture(RapitarArchitecture(), replace=True)
