"""Small Rapitar configurations of the tests and random weights for them, drawn here (tensor names and
shapes are written out from the configuration by this file's own rules, not asked of the package).

The three differ in every size, in the order and mix of layers, and in the values that a model may
happen to make equal or 1: groups and norm parts above 1, one head, one expert chosen, all experts
chosen, a layer without feed-forward, a rotated part as wide as the plain part, a latent wider than 128,
an inner size of the decay products that is no multiple of 8, two attention layers of different sizes
(two groups of pages), and a model without any attention layer (no pages at all)."""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch


def _latent(heads, dim, rot, vdim, rank, q_rank, base, scale):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": rank,
                                                   "q_rank": q_rank, "rot": {"base": base, "dims": rot}, "scale": scale}}


def _mamba(heads, vdim, state, groups, conv, norm_groups):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
                                         "norm_groups": norm_groups}}


def _wkv(heads, dim):
    return {"type": "wkv", "mixer": {"heads": heads, "dim": dim}}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def _model(vocab, width, eps, layers):
    return {"architecture": "Rapitar", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "layers": [dict(layer, mlp=mlp) for layer, mlp in layers]}


CONFIG_A = _model(96, 64, 1e-5, [
    (_latent(3, 24, 8, 20, 40, 24, 1000.0, 0.21), _dense(100)),
    (_mamba(4, 12, 20, 2, 3, 2), _moe(5, 2, 36)),
    (_wkv(3, 20), None),
    (_mamba(2, 40, 9, 1, 2, 4), _moe(3, 3, 24)),
])
CONFIG_B = _model(80, 48, 1e-6, [  # no attention layer: requests hold state slots and no pages
    (_wkv(1, 16), _moe(4, 1, 40)),
    (_mamba(2, 24, 8, 2, 5, 1), _dense(72)),
])
CONFIG_C = _model(120, 72, 1e-5, [  # two attention layers of different sizes: two groups of pages
    (_latent(1, 16, 16, 16, 16, 8, 10000.0, 0.18), _moe(6, 2, 20)),
    (_wkv(2, 36), _dense(64)),
    (_latent(5, 8, 4, 12, 136, 32, 500.0, 0.3), None),
])
CONFIGS = {"A": (CONFIG_A, 4, 5), "B": (CONFIG_B, 8, 8), "C": (CONFIG_C, 16, 3)}  # name -> (config, page size, decay rank)


def tensor_shapes(config: dict, decay_rank: int) -> dict[str, tuple]:
    w = config["width"]
    out = {"embed": (config["vocab"], w), "final.norm": (w,), "head": (config["vocab"], w)}
    for i, layer in enumerate(config["layers"]):
        m, p = layer["mixer"], f"l{i}.mix"
        out[f"l{i}.norm1"] = (w,)
        if layer["type"] == "latent_attention":
            h = m["heads"]
            out.update({f"{p}.dq": (m["q_rank"], w), f"{p}.dq.norm": (m["q_rank"],), f"{p}.uq": (h * (m["dim"] + m["rot_dim"]), m["q_rank"]),
                        f"{p}.dkv": (m["kv_rank"] + m["rot_dim"], w), f"{p}.dkv.norm": (m["kv_rank"],),
                        f"{p}.uk": (h * m["dim"], m["kv_rank"]), f"{p}.uv": (h * m["vdim"], m["kv_rank"]), f"{p}.sink": (h,),
                        f"{p}.g": (h * m["vdim"], w), f"{p}.o": (w, h * m["vdim"])})
        elif layer["type"] == "mamba2":
            inner, gn = m["heads"] * m["vdim"], m["groups"] * m["state"]
            out.update({f"{p}.in": (2 * inner + 2 * gn + m["heads"], w), f"{p}.conv": (inner + 2 * gn, m["conv"]),
                        f"{p}.conv.b": (inner + 2 * gn,), f"{p}.dt_bias": (m["heads"],), f"{p}.A_log": (m["heads"],),
                        f"{p}.D": (m["heads"],), f"{p}.norm": (inner,), f"{p}.o": (w, inner)})
        else:
            a = m["heads"] * m["dim"]
            out.update({f"{p}.mu.{s}": (w,) for s in "rkvgw"})
            out.update({f"{p}.{s}": (a, w) for s in "rkvg"})
            out.update({f"{p}.w1": (decay_rank, w), f"{p}.w2": (a, decay_rank), f"{p}.w0": (a,), f"{p}.u": (m["heads"], m["dim"]),
                        f"{p}.norm": (a,), f"{p}.o": (w, a)})
        f, p = layer["mlp"], f"l{i}.mlp"
        if f is None:
            continue
        if f["kind"] == "dense":
            out.update({f"{p}.up": (f["ff"], w), f"{p}.down": (w, f["ff"])})
        else:
            for e in range(f["router"]["experts"]):
                out.update({f"{p}.e{e}.gate": (f["expert"]["ff"], w), f"{p}.e{e}.up": (f["expert"]["ff"], w),
                            f"{p}.e{e}.down": (w, f["expert"]["ff"])})
            out.update({f"{p}.router": (f["router"]["experts"], w), f"{p}.router.b": (f["router"]["experts"],)})
    return out


def draw_weights(config: dict, decay_rank: int, seed: int) -> dict[str, torch.Tensor]:
    """bfloat16 tensors.  Matrices N(0, 1/in) so that activations keep their size; attention peaked (query and
    key sides scaled up) and sinks of the size of the scores, so that a missed key or a dropped sink moves the
    logits; slow decays (a state remembers a few dozen tokens), so that a lost state does."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config, decay_rank).items():
        leaf = name.split(".", 2)[-1] if name.startswith("l") else name
        n = lambda scale=1.0: torch.randn(shape, generator=gen) * scale  # noqa: E731
        if leaf in ("norm1", "final.norm"):
            t = n(0.2)
        elif leaf in ("embed",):
            t = n()
        elif leaf.endswith("norm"):
            t = 1.0 + n(0.2)
        elif leaf in ("sink",):
            t = 1.0 + n(1.5)
        elif leaf in ("uq", "dkv"):
            t = n(3.0 / math.sqrt(shape[-1]))
        elif leaf in ("A_log",):
            t = math.log(0.3) + n(0.5)
        elif leaf in ("dt_bias",):
            t = -2.5 + n(0.5)
        elif leaf in ("D",):
            t = 1.0 + n(0.3)
        elif leaf in ("w0",):
            t = -3.5 + n(0.7)
        elif leaf in ("u",):
            t = n(0.5)
        elif leaf.startswith("mu."):
            t = torch.rand(shape, generator=gen)
        elif leaf in ("conv",):
            t = n(0.5)
        elif leaf in ("conv.b", "router.b"):
            t = n(0.3)
        elif leaf in ("router",):
            t = n(4.0 / math.sqrt(shape[-1]))
        else:
            t = n(1.0 / math.sqrt(shape[-1]))
        out[name] = t.to(torch.bfloat16)
    return out


def write_model(folder, name: str, seed: int = 0) -> Path:
    from clockwork_b200.weights import save_safetensors

    config, _, decay_rank = CONFIGS[name]
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config))
    save_safetensors(folder / "model.safetensors", draw_weights(config, decay_rank, seed))
    return folder


def tokens_for(config: dict, length: int, salt: int = 0) -> list[int]:
    state = (7919 * salt + 104729 * length + 12345) & 0x7FFFFFFF
    out = []
    for _ in range(length):
        state = (1103515245 * state + 12345) & 0x7FFFFFFF
        out.append((state >> 8) % config["vocab"])
    return out
