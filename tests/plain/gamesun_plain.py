"""A plain, slow forward pass of the Gamesun design: whole sequences, no cache, one function per
mechanism, float32 or float64 torch on the CPU.  It is the yardstick of the tests and shares no
code with ``clockwork_b200``.

The design in this file's notation (x: residual row, h: its norm, W: a stored [out, in] matrix,
n(x) = x / sqrt(mean(x^2) + eps), t: position in the sequence from 0):

* input:   x_t = E[token] s_e + pe(t),  pe(t)[2i] = sin(t b^(-2i/width)),  pe(t)[2i+1] = cos(same),  b = 10000
* layer:   x <- x + mixer(n(x) g1);  x <- x + ff(n(x) g2)  (a layer may have no ff)
* mixer:   two mixers read the same h:  0.5 (n(left(h)) g_left + n(right(h)) g_right), norms over the width
* left:    attention over the last `window` positions (t - j < window), H query heads on G key/value heads,
           keys of size dk, values of size dv, no rotation;  s_h = (q_h . k) scale
           - `parallel`   : biases on q, k, v, o;  s_h <- sum_g T[h, g] s_g;  weight = sigmoid(s_h + pb_h), not normalised
           - `parallel_2` : no biases;  s_h <- s_h temp_h;  weights = softmax over the visible keys
* right of `parallel` (linear attention, a decay per key channel):
           q = W_q h dk^(-1/2);  a = sigmoid(W_a2 W_a1 h + b)^(1/tau);  S <- diag(a) S + k v^T;  o = S^T q;
           out = W_o (concat_heads(n(o_head) g) silu(W_g h))      (g of size dv, shared by the heads)
* right of `parallel_2` (linear attention, a constant decay per head):
           q, k, v = silu(W_q h), silu(W_k h), silu(W_v h);  S <- d_head S + k v^T;  o = S^T q;
           out = W_o (n(concat_heads(o)) g sigmoid(W_g h))
* ff:      W_down (silu(W_gate h) (W_up h))
* output:  logits = E (n(x) g_final)
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def exact(x):
    return x


def to_bfloat16_and_back(x):
    return x.to(torch.bfloat16).to(x.dtype)


def unit_rms(x, eps):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def scaled_norm(x, g, eps):
    return unit_rms(x, eps) * g


def position_vectors(count, width, dtype, base=10000.0):
    t = torch.arange(count, dtype=dtype)[:, None]
    i = torch.arange(0, width, 2, dtype=dtype)[None, :]
    angle = t * base ** (-i / width)
    out = torch.zeros(count, width, dtype=dtype)
    out[:, 0::2] = torch.sin(angle)
    out[:, 1::2] = torch.cos(angle)
    return out


def embed(tokens, w, scale, dtype):
    table = w["embed"]
    return table[tokens] * scale + position_vectors(len(tokens), table.shape[1], dtype)


def window_mask(count, window):
    t = torch.arange(count)
    d = t[:, None] - t[None, :]
    return (d >= 0) & (d < window)


def window_scores(h, w, p, m, biased, rnd=exact):
    """[H, T, T] scaled scores of every query head against its key/value head, and the values [G, T, dv].
    (``rnd``: a bfloat16 run stores queries, keys and values in bfloat16.)"""
    heads, groups, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    t = h.shape[0]
    q, k, v = h @ w[f"{p}.q"].T, h @ w[f"{p}.k"].T, h @ w[f"{p}.v"].T
    if biased:
        q, k, v = q + w[f"{p}.q.b"], k + w[f"{p}.k.b"], v + w[f"{p}.v.b"]
    q, k, v = rnd(q), rnd(k), rnd(v)
    q = q.reshape(t, heads, dk).transpose(0, 1)
    k = k.reshape(t, groups, dk).transpose(0, 1)
    v = v.reshape(t, groups, dv).transpose(0, 1)
    per = heads // groups
    k_of_head = k.repeat_interleave(per, dim=0)
    scores = torch.einsum("htd,hsd->hts", q, k_of_head) * m["scale"]
    return scores, v.repeat_interleave(per, dim=0)


def sigmoid_window_attention(h, w, p, m, rnd=exact):
    """The left mixer of a `parallel` layer."""
    scores, v = window_scores(h, w, p, m, biased=True, rnd=rnd)
    scores = torch.einsum("hg,gts->hts", w[f"{p}.talk"], scores)
    weights = torch.sigmoid(scores + w[f"{p}.pb"][:, None, None])
    weights = weights * window_mask(h.shape[0], m["mask"]["size"])
    o = torch.einsum("hts,hsd->thd", weights, v).reshape(h.shape[0], -1)
    return rnd(o) @ w[f"{p}.o"].T + w[f"{p}.o.b"]


def softmax_window_attention(h, w, p, m, rnd=exact):
    """The left mixer of a `parallel_2` layer."""
    scores, v = window_scores(h, w, p, m, biased=False, rnd=rnd)
    scores = scores * w[f"{p}.temp"][:, None, None]
    scores = scores.masked_fill(~window_mask(h.shape[0], m["mask"]["size"]), float("-inf"))
    o = torch.einsum("hts,hsd->thd", torch.softmax(scores, dim=-1), v).reshape(h.shape[0], -1)
    return rnd(o) @ w[f"{p}.o"].T


def decayed_outer_product_scan(q, k, v, decay):
    """q, k [T, H, dk], v [T, H, dv], decay [T, H, dk] (or broadcastable): S <- diag(decay) S + k v^T, o = S^T q."""
    t, heads, dk = q.shape
    state = torch.zeros(heads, dk, v.shape[-1], dtype=q.dtype)
    out = []
    for i in range(t):
        state = decay[i][..., None] * state + k[i][..., None] * v[i][:, None, :]
        out.append(torch.einsum("hkv,hk->hv", state, q[i]))
    return torch.stack(out)


def channel_decay_mixer(h, w, p, m, eps, rnd=exact):
    """The right mixer of a `parallel` layer."""
    heads, dk, dv = m["heads"], m["dim"], m["vdim"]
    t = h.shape[0]
    q = (h @ w[f"{p}.q"].T) * dk ** -0.5
    k, v = h @ w[f"{p}.k"].T, h @ w[f"{p}.v"].T
    z = rnd(h @ w[f"{p}.a1"].T) @ w[f"{p}.a2"].T + w[f"{p}.a2.b"]
    decay = torch.exp(F.logsigmoid(z) / m["tau"])
    o = decayed_outer_product_scan(q.reshape(t, heads, dk), k.reshape(t, heads, dk), v.reshape(t, heads, dv),
                                   decay.reshape(t, heads, dk))
    o = scaled_norm(o, w[f"{p}.norm"], eps).reshape(t, heads * dv)
    return rnd(o * F.silu(h @ w[f"{p}.g"].T)) @ w[f"{p}.o"].T


def head_decay_mixer(h, w, p, m, eps, rnd=exact):
    """The right mixer of a `parallel_2` layer."""
    heads, dk, dv = m["heads"], m["dim"], m["vdim"]
    t = h.shape[0]
    q, k, v = F.silu(h @ w[f"{p}.q"].T), F.silu(h @ w[f"{p}.k"].T), F.silu(h @ w[f"{p}.v"].T)
    decay = torch.tensor(m["decay"], dtype=h.dtype)[None, :, None].expand(t, heads, 1)
    o = decayed_outer_product_scan(q.reshape(t, heads, dk), k.reshape(t, heads, dk), v.reshape(t, heads, dv), decay)
    o = scaled_norm(o.reshape(t, heads * dv), w[f"{p}.norm"], eps)
    return rnd(o * torch.sigmoid(h @ w[f"{p}.g"].T)) @ w[f"{p}.o"].T


def side_by_side(h, w, p, kind, m, eps, rnd=exact):
    if kind == "parallel":
        left = sigmoid_window_attention(h, w, f"{p}.left", m["left"], rnd)
        right = channel_decay_mixer(h, w, f"{p}.right", m["right"], eps, rnd)
    elif kind == "parallel_2":
        left = softmax_window_attention(h, w, f"{p}.left", m["left"], rnd)
        right = head_decay_mixer(h, w, f"{p}.right", m["right"], eps, rnd)
    else:
        raise ValueError(kind)
    return 0.5 * (scaled_norm(left, w[f"{p}.left.out"], eps) + scaled_norm(right, w[f"{p}.right.out"], eps))


def gated_ff(h, w, p, rnd=exact):
    return rnd(F.silu(h @ w[f"{p}.gate"].T) * (h @ w[f"{p}.up"].T)) @ w[f"{p}.down"].T


def forward(config, weights, tokens, dtype=torch.float64, rnd=exact, keep_layers=False):
    """Logits [T, vocab] of one whole sequence (and, with ``keep_layers``, the residual after every layer)."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = config["norm"]["eps"]
    x = embed(torch.as_tensor(tokens, dtype=torch.long), w, config["embedding"]["scale"], dtype)
    kept = []
    for i, layer in enumerate(config["layers"]):
        h = rnd(scaled_norm(x, w[f"l{i}.norm1"], eps))
        x = x + side_by_side(h, w, f"l{i}.mix", layer["type"], layer["mixer"], eps, rnd)
        if layer.get("mlp") is not None:
            h = rnd(scaled_norm(x, w[f"l{i}.norm2"], eps))
            x = x + gated_ff(h, w, f"l{i}.mlp", rnd)
        kept.append(x)
    logits = rnd(scaled_norm(x, w["final.norm"], eps)) @ w["embed"].T
    return (logits, torch.stack(kept)) if keep_layers else logits


def greedy_generate(config, weights, prompt, count, dtype=torch.float64):
    tokens = list(prompt)
    for _ in range(count):
        tokens.append(int(forward(config, weights, tokens, dtype=dtype)[-1].argmax()))
    return tokens[len(prompt):]


def first_position_margin(config, weights, token, dtype=torch.float64):
    """At position 0 a head of the linear attention with a norm per head puts out sign(q.k) n(v): the smallest
    |cos(q, k)| over those heads says how far the first token is from a sign that rounding could flip."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = config["norm"]["eps"]
    x = embed(torch.as_tensor([token], dtype=torch.long), w, config["embedding"]["scale"], dtype)
    margin = 1.0
    for i, layer in enumerate(config["layers"]):
        h = scaled_norm(x, w[f"l{i}.norm1"], eps)
        if layer["type"] == "parallel":
            m = layer["mixer"]["right"]
            q = (h @ w[f"l{i}.mix.right.q"].T).reshape(m["heads"], m["dim"])
            k = (h @ w[f"l{i}.mix.right.k"].T).reshape(m["heads"], m["dim"])
            margin = min(margin, float(((q * k).sum(-1) / (q.norm(dim=-1) * k.norm(dim=-1))).abs().min()))
        x = x + side_by_side(h, w, f"l{i}.mix", layer["type"], layer["mixer"], eps)
        if layer.get("mlp") is not None:
            x = x + gated_ff(scaled_norm(x, w[f"l{i}.norm2"], eps), w, f"l{i}.mlp")
    return margin


def steady_first_token(config, weights, candidates=range(48)):
    """The candidate whose answer at position 0 is farthest from such a flip."""
    return max(candidates, key=lambda token: first_position_margin(config, weights, token))
