"""Python faces of the kernels for layers that carry a state of fixed size from token to token
(``csrc/recurrence.cu``): token shift, short causal convolution, the rows kept for the next step,
the recurrence itself in its two forms, the gated norm in parts, and in-place activations.

A request's state is one float32 row of the cache manager's slot tensor (``StateView``); a part
lays several pieces out in that row and names each by its offset."""

from __future__ import annotations

import torch

from . import _need, _ptr, _stream, dtype_code
from .library import check, library

FORM_CHANNEL_DECAY, FORM_STEP_SIZE = 0, 1
ACT_GELU_TANH, ACT_TANH = 0, 1


def _state_args(view) -> tuple:
    state = view.state
    _need(state, torch.float32, "state", 2)
    _need(view.slots, torch.int64, "state slots", 1)
    return state.data_ptr(), state.stride(0), view.slots.data_ptr()


def shift_mix(x: torch.Tensor, mu: torch.Tensor, view, offset: int, ctx) -> torch.Tensor:
    """[mixes, N, W]: ``x + (x_prev - x) * mu[s]``; the row before a portion's first comes from the state."""
    _need(x, None, "x", 2)
    _need(mu, torch.float32, "mu", 2)
    n, w = x.shape
    if mu.shape[1] != w:
        raise ValueError("mu must be [mixes, width]")
    out = torch.empty((mu.shape[0], n, w), dtype=x.dtype, device=x.device)
    state, stride, slots = _state_args(view)
    check(library().cw_shift_mix(_ptr(x), _ptr(mu), state, stride, offset, slots, _ptr(ctx.tok_seq), _ptr(ctx.q_start),
                                 _ptr(out), n, w, mu.shape[0], dtype_code(x.dtype), _stream()), "shift_mix")
    return out


def causal_conv(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, view, offset: int, ctx) -> torch.Tensor:
    """silu(conv(x) + bias) per channel; ``x`` float32 [N, C] (may be a column slice), ``weight`` [C, taps]."""
    if x.dtype != torch.float32 or x.dim() != 2 or x.stride(1) != 1:
        raise ValueError("x must be float32 [N, C] with unit column stride")
    _need(weight, torch.float32, "weight", 2)
    n, c = x.shape
    if weight.shape[0] != c:
        raise ValueError("conv weight must be [channels, taps]")
    out = torch.empty((n, c), dtype=torch.float32, device=x.device)
    state, stride, slots = _state_args(view)
    check(library().cw_causal_conv(_ptr(x), x.stride(0) if n > 1 else max(x.stride(0), c), _ptr(weight), _ptr(bias), state, stride,
                                   offset, slots, _ptr(ctx.tok_seq), _ptr(ctx.q_start), _ptr(out), n, c, weight.shape[1],
                                   _stream()), "causal_conv")
    return out


def carry_rows(x: torch.Tensor, rows: int, view, offset: int, ctx) -> None:
    """Keeps the last ``rows`` rows of every request's portion of ``x`` [N, C] in its state (older kept rows shift)."""
    if x.dim() != 2 or x.stride(1) != 1:
        raise ValueError("x must be [N, C] with unit column stride")
    n, c = x.shape
    state, stride, slots = _state_args(view)
    check(library().cw_carry_rows(_ptr(x), x.stride(0) if n > 1 else max(x.stride(0), c), state, stride, offset, slots,
                                  _ptr(ctx.tok_seq), _ptr(ctx.q_start), ctx.num_seqs, c, rows, dtype_code(x.dtype), _stream()),
          "carry_rows")


def recurrence_scan(form: int, q, k, v, pre, p0, p1, p2, view, offset: int, ctx, heads: int, dk: int, dv: int,
                    heads_per_group: int = 1) -> torch.Tensor:
    """float32 [N, heads*dv].  ``q``, ``k`` [N, groups*dk], ``v`` [N, heads*dv], ``pre`` [N, heads*dk] (form 0) or
    [N, heads] (form 1): float32, unit column stride, any row stride.  The state piece at ``offset`` holds
    heads*dk*dv numbers.  Form 0 turns ``pre`` into the decays in place (it is a product's output that nothing
    else reads)."""
    for name, t in (("q", q), ("k", k), ("v", v), ("pre", pre)):
        if t.dtype != torch.float32 or t.dim() != 2 or t.stride(1) != 1:
            raise ValueError(f"{name} must be float32 [N, *] with unit column stride")
    n = v.shape[0]
    out = torch.empty((n, heads * dv), dtype=torch.float32, device=v.device)
    state, stride, slots = _state_args(view)

    def ld(t):
        return t.stride(0) if n > 1 else max(t.stride(0), t.shape[1])

    # decays and step sizes once per token, ahead of the scan
    if form == FORM_CHANNEL_DECAY:
        check(library().cw_recurrence_coefficients(form, _ptr(pre), ld(pre), _ptr(p0), None, None, n, heads * dk, _stream()),
              "recurrence_coefficients")
    else:
        coef = torch.empty((n, 2 * heads), dtype=torch.float32, device=v.device)
        check(library().cw_recurrence_coefficients(form, _ptr(pre), ld(pre), _ptr(p0), _ptr(p1), _ptr(coef), n, heads, _stream()),
              "recurrence_coefficients")
        pre = coef
    check(library().cw_recurrence_scan(form, _ptr(q), ld(q), _ptr(k), ld(k), _ptr(v), ld(v), _ptr(pre), ld(pre), _ptr(p0), _ptr(p1),
                                       _ptr(p2), state, stride, offset, slots, _ptr(ctx.tok_seq), _ptr(ctx.q_start), ctx.num_seqs,
                                       heads, dk, dv, heads_per_group, _ptr(out), heads * dv, _stream()), "recurrence_scan")
    return out


def gated_group_norm(y: torch.Tensor, z: torch.Tensor, weight: torch.Tensor, parts: int, eps: float, gate_first: bool,
                     out_dtype: torch.dtype) -> torch.Tensor:
    """``gate_first``: norm_parts(y * silu(z)) * weight; else norm_parts(y) * weight * silu(z).  y, z float32."""
    _need(y, torch.float32, "y", 2)
    if z.dtype != torch.float32 or z.dim() != 2 or z.stride(1) != 1:
        raise ValueError("z must be float32 [N, C] with unit column stride")
    _need(weight, torch.float32, "weight", 1)
    n, c = y.shape
    out = torch.empty((n, c), dtype=out_dtype, device=y.device)
    check(library().cw_gated_group_norm(_ptr(y), _ptr(z), z.stride(0) if n > 1 else max(z.stride(0), c), _ptr(weight), _ptr(out), n, c,
                                        parts, float(eps), 1 if gate_first else 0, dtype_code(out_dtype), _stream()),
          "gated_group_norm")
    return out


def activation_(x: torch.Tensor, kind: int) -> torch.Tensor:
    """In place: gelu in its tanh form, or tanh."""
    _need(x, None, "x")
    check(library().cw_activation(_ptr(x), x.numel(), kind, dtype_code(x.dtype), _stream()), "activation")
    return x
