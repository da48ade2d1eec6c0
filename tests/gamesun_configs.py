"""Small Gamesun configurations of the tests and random weights for them, drawn here (tensor names and shapes are
written out from the configuration by this file's own rules, not asked of the package).

The four differ in every size, in the order of layers, and in the values that a model may happen to make equal
or 1: one key/value head for all query heads, as many key/value heads as query heads, three query heads per
key/value head; values narrower and wider than keys; linear-attention heads whose keys and values differ in size,
a single head; windows of 1 (a token sees itself only), smaller than a page, no multiple of a page, and longer than
the prompts; a layer without feed-forward; a decay of exactly 1; widths that are no power of two; an inner size of
the decay products that is no multiple of 8."""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch


def _soft(heads, kv_heads, dim, vdim, window, scale, r_heads, r_dim, r_vdim, decay):
    return {"type": "parallel_2", "mixer": {
        "left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": window}},
        "right": {"heads": r_heads, "dim": r_dim, "vdim": r_vdim, "decay": decay}}}


def _gated(heads, kv_heads, dim, vdim, window, scale, r_heads, r_dim, r_vdim, tau):
    return {"type": "parallel", "mixer": {
        "left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": window}},
        "right": {"heads": r_heads, "dim": r_dim, "vdim": r_vdim, "tau": tau}}}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _model(vocab, width, eps, scale, layers):
    return {"architecture": "Gamesun", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": scale},
            "layers": [dict(layer, mlp=mlp) for layer, mlp in layers]}


CONFIG_A = _model(96, 64, 1e-5, 8.0, [
    (_gated(4, 2, 24, 12, 21, 0.3, 3, 20, 12, 8.0), _dense(100)),
    (_soft(3, 1, 16, 40, 7, 0.25, 2, 24, 8, [0.97, 1.0]), None),
    (_soft(6, 2, 8, 8, 50, 0.4, 1, 16, 48, [0.9]), _dense(72)),
    (_gated(2, 2, 32, 16, 1, 0.2, 4, 8, 8, 3.0), _dense(40)),
])
CONFIG_B = _model(80, 48, 1e-6, 3.5, [
    (_soft(2, 2, 12, 20, 200, 0.3, 3, 8, 16, [0.5, 0.95, 0.995]), _dense(64)),
    (_gated(3, 3, 16, 8, 33, 0.25, 2, 12, 24, 20.0), None),
])
CONFIG_C = _model(120, 72, 1e-5, 1.0, [
    (_gated(6, 1, 8, 24, 16, 0.35, 1, 40, 16, 1.0), _dense(56)),
    (_gated(1, 1, 40, 8, 3, 0.15, 5, 8, 8, 12.0), _dense(88)),
    (_soft(4, 4, 16, 16, 19, 0.25, 2, 16, 16, [0.99, 0.8]), _dense(30)),
])
CONFIG_D = _model(1000, 320, 1e-6, 12.0, [  # sizes that the tensor-core attention takes, in each of its arrangements
    (_soft(8, 2, 32, 64, 100, 32 ** -0.5, 3, 24, 40, [0.75, 0.875, 0.9375]), _dense(500)),   # four query heads per key/value head
    (_gated(12, 3, 48, 80, 60, 48 ** -0.5, 2, 32, 64, 4.0), _dense(260)),                    # twelve heads mixed: twelve warps a block
    (_gated(20, 4, 16, 24, 64, 0.25, 5, 16, 16, 16.0), None),                                # twenty heads mixed: the CUDA-core kernel
    (_soft(4, 4, 80, 200, 30, 80 ** -0.5, 4, 64, 32, [0.5, 0.9, 0.99, 0.999]), _dense(384)),  # one query head per key/value head, wide values
])
CONFIGS = {"A": (CONFIG_A, 4, 5), "B": (CONFIG_B, 8, 8), "C": (CONFIG_C, 16, 3), "D": (CONFIG_D, 16, 6)}  # name -> (config, page size, decay rank)


def tensor_shapes(config: dict, decay_rank: int) -> dict[str, tuple]:
    w = config["width"]
    out = {"embed": (config["vocab"], w), "final.norm": (w,)}
    for i, layer in enumerate(config["layers"]):
        left, right, p = layer["mixer"]["left"], layer["mixer"]["right"], f"l{i}.mix"
        gated = layer["type"] == "parallel"
        out[f"l{i}.norm1"] = (w,)
        h, g, dk, dv = left["heads"], left["kv_heads"], left["dim"], left["vdim"]
        out.update({f"{p}.left.q": (h * dk, w), f"{p}.left.k": (g * dk, w), f"{p}.left.v": (g * dv, w), f"{p}.left.o": (w, h * dv),
                    f"{p}.left.out": (w,), f"{p}.right.out": (w,)})
        if gated:
            out.update({f"{p}.left.q.b": (h * dk,), f"{p}.left.k.b": (g * dk,), f"{p}.left.v.b": (g * dv,), f"{p}.left.o.b": (w,),
                        f"{p}.left.talk": (h, h), f"{p}.left.pb": (h,)})
        else:
            out[f"{p}.left.temp"] = (h,)
        rh, rk, rv = right["heads"], right["dim"], right["vdim"]
        out.update({f"{p}.right.q": (rh * rk, w), f"{p}.right.k": (rh * rk, w), f"{p}.right.v": (rh * rv, w),
                    f"{p}.right.g": (rh * rv, w), f"{p}.right.o": (w, rh * rv)})
        if gated:
            out.update({f"{p}.right.a1": (decay_rank, w), f"{p}.right.a2": (rh * rk, decay_rank), f"{p}.right.a2.b": (rh * rk,),
                        f"{p}.right.norm": (rv,)})
        else:
            out[f"{p}.right.norm"] = (rh * rv,)
        if layer["mlp"] is not None:
            ff = layer["mlp"]["ff"]
            out.update({f"l{i}.norm2": (w,), f"l{i}.mlp.gate": (ff, w), f"l{i}.mlp.up": (ff, w), f"l{i}.mlp.down": (w, ff)})
    return out


def draw_weights(config: dict, decay_rank: int, seed: int) -> dict[str, torch.Tensor]:
    """bfloat16 tensors.  Matrices N(0, 1/in) so that activations keep their size; attention peaked (query and key
    sides scaled up) so that a key that is missed or seen wrongly moves the logits; decays close to one (the decay
    product's bias large), so that a state remembers dozens of tokens and a lost or stale state shows."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config, decay_rank).items():
        leaf = name.split(".", 1)[-1] if name.startswith("l") else name
        n = lambda scale=1.0: torch.randn(shape, generator=gen) * scale  # noqa: E731
        if leaf == "embed":
            t = n(0.5)
        elif leaf in ("norm1", "norm2", "final.norm", "mix.left.out", "mix.right.out", "mix.right.norm"):
            t = 1.0 + n(0.2)
        elif leaf in ("mix.left.q", "mix.left.k"):
            t = n(2.5 / math.sqrt(shape[-1]))
        elif leaf == "mix.left.talk":
            t = torch.eye(shape[0]) + n(0.3)
        elif leaf == "mix.left.pb":
            t = -1.0 + n(1.0)
        elif leaf == "mix.left.temp":
            t = 1.0 + n(0.4)
        elif leaf == "mix.right.a2.b":
            t = 3.0 + n(1.0)
        elif leaf.endswith(".b"):
            t = n(0.3)
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
    state = (6007 * salt + 15485863 * length + 777) & 0x7FFFFFFF
    out = []
    for _ in range(length):
        state = (1103515245 * state + 12345) & 0x7FFFFFFF
        out.append((state >> 8) % config["vocab"])
    return out
