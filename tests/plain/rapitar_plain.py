"""A plain, slow forward pass of the Rapitar design: whole sequences, no cache, one function per
mechanism, float32 or float64 torch on the CPU.  It is the yardstick of the tests and shares no
code with ``clockwork_b200``.

The design in this file's notation (x: residual row, h: its norm, W: a stored [out, in] matrix):

* layer (parallel):  h = n(x) (1 + g),  n(x) = x / sqrt(mean(x^2) + eps);  x <- x + mixer(h) + ff(h)
* mamba2:  [z | u | B | C | dt] = W_in h;  (u, B, C) <- silu(causal_conv(u, B, C));
           dt <- softplus(dt + dt_bias);  S <- exp(-exp(A_log) dt) S + dt B u^T;  y = S^T C + D u;
           out = W_o (n_groups(y silu(z)) g)
* wkv:     m_s = h + (h_prev - h) mu_s;  r, k, v = W_r m_r, W_k m_k, W_v m_v;  gate = silu(W_g m_g);
           w = exp(-exp(W_w2 tanh(W_w1 m_w) + w0));  o = (S + diag(u) k v^T)^T r;  S <- diag(w) S + k v^T;
           out = W_o (n_head(o) g gate)
* latent attention:  c_q = n(W_dq h) g_q;  q = W_uq c_q (per head [plain | rotated]);
           [c_raw | k_r] = W_dkv h;  c = n(c_raw) g_kv;  k = [W_uk c | rot(k_r)];  v = W_uv c;
           p = exp(s_j) / (exp(sink) + sum_j exp(s_j)),  s = q.k scale, causal;
           out = W_o (concat(p v) sigmoid(W_g h))
* feed-forward:  dense W_down gelu_tanh(W_up h);  experts: top-k of W_router h + b, softmax over the
           chosen logits, sum of weight * W_down (silu(W_gate h) (W_up h))
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


def offset_norm(x, g, eps):
    """The layer norm: the checkpoint holds the weight's distance from one."""
    return unit_rms(x, eps) * (1.0 + g)


def plain_norm(x, g, eps):
    return unit_rms(x, eps) * g


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z**3)))


def dense_ff(h, w, p, rnd=exact):
    return rnd(gelu_tanh(h @ w[f"{p}.up"].T)) @ w[f"{p}.down"].T


def routed_ff(h, w, p, cfg, rnd=exact):
    experts, top = cfg["router"]["experts"], cfg["router"]["top"]
    logits = h @ w[f"{p}.router"].T + w[f"{p}.router.b"]
    chosen = torch.topk(logits, top, dim=-1)
    weights = torch.softmax(chosen.values, dim=-1)
    out = torch.zeros(h.shape[0], w[f"{p}.e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(chosen.indices[t, j])
            assert 0 <= e < experts
            a = rnd(F.silu(w[f"{p}.e{e}.gate"] @ h[t]) * (w[f"{p}.e{e}.up"] @ h[t]))
            out[t] += weights[t, j] * (w[f"{p}.e{e}.down"] @ a)
    return out


def causal_conv_silu(x, weight, bias):
    """x [T, C]; weight [C, taps]: the newest input meets the last tap, inputs before position 0 count as zero."""
    t, c = x.shape
    taps = weight.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, c, dtype=x.dtype), x])
    out = bias.expand(t, c).clone()
    for j in range(taps):
        out = out + padded[j : j + t] * weight[:, j]
    return F.silu(out)


def mamba2_mixer(h, w, p, cfg, eps, rnd=exact):
    heads, vdim, n, groups = cfg["heads"], cfg["vdim"], cfg["state"], cfg["groups"]
    inner = heads * vdim
    t = h.shape[0]
    proj = h @ w[f"{p}.in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner : 2 * inner + 2 * groups * n], proj[:, 2 * inner + 2 * groups * n :]
    xbc = rnd(causal_conv_silu(xbc, w[f"{p}.conv"], w[f"{p}.conv.b"]))
    u = xbc[:, :inner].reshape(t, heads, vdim)
    b = xbc[:, inner : inner + groups * n].reshape(t, groups, n)
    c = xbc[:, inner + groups * n :].reshape(t, groups, n)
    dt = F.softplus(dt + w[f"{p}.dt_bias"], threshold=1e9)
    decay = torch.exp(-torch.exp(w[f"{p}.A_log"]) * dt)  # [T, heads]
    y = torch.zeros(t, heads, vdim, dtype=h.dtype)
    per_group = heads // groups
    for hd in range(heads):
        g = hd // per_group
        s = torch.zeros(n, vdim, dtype=h.dtype)
        for i in range(t):
            s = decay[i, hd] * s + dt[i, hd] * torch.outer(b[i, g], u[i, hd])
            y[i, hd] = s.T @ c[i, g] + w[f"{p}.D"][hd] * u[i, hd]
    y = y.reshape(t, inner) * F.silu(z)
    parts = cfg["norm_groups"]
    y = unit_rms(y.reshape(t, parts, inner // parts), eps).reshape(t, inner) * w[f"{p}.norm"]
    return rnd(y) @ w[f"{p}.o"].T


def wkv_mixer(h, w, p, cfg, eps, rnd=exact):
    heads, dim = cfg["heads"], cfg["dim"]
    t = h.shape[0]
    prev = torch.cat([torch.zeros(1, h.shape[1], dtype=h.dtype), h[:-1]])

    def mix(s):
        return rnd(h + (prev - h) * w[f"{p}.mu.{s}"])

    r = (mix("r") @ w[f"{p}.r"].T).reshape(t, heads, dim)
    k = (mix("k") @ w[f"{p}.k"].T).reshape(t, heads, dim)
    v = (mix("v") @ w[f"{p}.v"].T).reshape(t, heads, dim)
    gate = F.silu(mix("g") @ w[f"{p}.g"].T)
    decay = torch.exp(-torch.exp(rnd(torch.tanh(mix("w") @ w[f"{p}.w1"].T)) @ w[f"{p}.w2"].T + w[f"{p}.w0"])).reshape(t, heads, dim)
    bonus = w[f"{p}.u"]
    o = torch.zeros(t, heads, dim, dtype=h.dtype)
    for hd in range(heads):
        s = torch.zeros(dim, dim, dtype=h.dtype)  # [key channel, value channel]
        for i in range(t):
            kv = torch.outer(k[i, hd], v[i, hd])
            o[i, hd] = (s + bonus[hd][:, None] * kv).T @ r[i, hd]
            s = decay[i, hd][:, None] * s + kv
    o = unit_rms(o, eps).reshape(t, heads * dim) * w[f"{p}.norm"] * gate
    return rnd(o) @ w[f"{p}.o"].T


def rotate_pairs(x, positions, base):
    """x [T, ..., dims]: dimension i is paired with i + dims/2."""
    dims = x.shape[-1]
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=torch.float32)
    angle = positions.to(torch.float32)[:, None] * freq[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    cos, sin = angle.cos().to(x.dtype).reshape(shape), angle.sin().to(x.dtype).reshape(shape)
    a, b = x[..., :half], x[..., half:]
    return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)


def latent_attention_mixer(h, w, p, cfg, eps, positions=None, rnd=exact):
    heads, dim, rot, vdim, rank = cfg["heads"], cfg["dim"], cfg["rot_dim"], cfg["vdim"], cfg["kv_rank"]
    t = h.shape[0]
    positions = torch.arange(t) if positions is None else positions
    base = cfg["rot"]["base"]
    assert cfg["rot"]["dims"] == rot
    cq = rnd(plain_norm(h @ w[f"{p}.dq"].T, w[f"{p}.dq.norm"], eps))
    q = rnd(cq @ w[f"{p}.uq"].T).reshape(t, heads, dim + rot)
    q_plain, q_rot = q[..., :dim], rotate_pairs(q[..., dim:], positions, base)
    down = h @ w[f"{p}.dkv"].T
    c = rnd(plain_norm(down[:, :rank], w[f"{p}.dkv.norm"], eps))
    k_rot = rnd(rotate_pairs(down[:, rank:], positions, base))  # shared by all heads
    k_plain = (c @ w[f"{p}.uk"].T).reshape(t, heads, dim)
    v = (c @ w[f"{p}.uv"].T).reshape(t, heads, vdim)
    scores = (torch.einsum("qhd,khd->hqk", q_plain, k_plain) + torch.einsum("qhd,kd->hqk", q_rot, k_rot)) * cfg["scale"]
    hidden = positions[None, :] > positions[:, None]
    scores = scores.masked_fill(hidden, float("-inf"))
    sink = w[f"{p}.sink"].to(h.dtype)
    top = torch.maximum(scores.max(-1).values, sink[:, None])
    e = torch.exp(scores - top[..., None])
    probs = e / (e.sum(-1, keepdim=True) + torch.exp(sink[:, None] - top)[..., None])
    out = torch.einsum("hqk,khd->qhd", probs, v).reshape(t, heads * vdim)
    out = out * torch.sigmoid(h @ w[f"{p}.g"].T)
    return rnd(out) @ w[f"{p}.o"].T


MIXERS = {"mamba2": mamba2_mixer, "wkv": wkv_mixer, "latent_attention": latent_attention_mixer}


def feed_forward(h, w, p, cfg, rnd=exact):
    if cfg is None:
        return 0.0
    if cfg["kind"] == "dense":
        return dense_ff(h, w, p, rnd)
    if cfg["kind"] == "moe":
        return routed_ff(h, w, p, cfg, rnd)
    raise ValueError(cfg["kind"])


def greedy_generate(config, w, prompt, count, dtype=torch.float64):
    tokens = list(prompt)
    for _ in range(count):
        tokens.append(int(forward(config, w, tokens, dtype=dtype)[-1].argmax()))
    return tokens[len(prompt):]


def forward(config, w, tokens, rnd=exact, dtype=torch.float32, keep_layers=False):
    """Logits [T, vocab] of one whole sequence (and, on request, the residual after every layer)."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    eps = config["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens)]
    after = []
    for i, layer in enumerate(config["layers"]):
        h = rnd(offset_norm(x, w[f"l{i}.norm1"], eps))
        mixed = MIXERS[layer["type"]](h, w, f"l{i}.mix", layer["mixer"], eps, rnd=rnd)
        x = x + (mixed + feed_forward(h, w, f"l{i}.mlp", layer["mlp"], rnd))
        after.append(x)
    logits = rnd(offset_norm(x, w["final.norm"], eps)) @ w["head"].T
    return (logits, torch.stack(after)) if keep_layers else logits
