"""A mixture-of-experts feed-forward as launches: the router, the pick, and the choice of kernels for the two grouped
products."""
from __future__ import annotations

from typing import Optional

import torch

from . import lib as K
from . import linear as L


def feed_forward(ctx, y: torch.Tensor, wr: torch.Tensor, br: Optional[torch.Tensor], wup: torch.Tensor,
                 wdown: torch.Tensor, top: int, act: str, dtype: torch.dtype, *, score: str = "softmax",
                 gated: bool = False, weight_on: str = "output", n_experts: Optional[int] = None):
    """32-bit planes ``[top, T, width]`` whose sum in order is the feed-forward's output: router logits ``y wr^T + br``
    with 32-bit accumulation, the ``top`` largest per row weighted by the softmax over those alone (``score``
    "sigmoid": by each one's own sigmoid), plane k of a row = its k-th weight times ``W_down[e] act(W_up[e] y)``.
    ``wr`` may hold rows beyond the ``n_experts`` experts' (another per-row logit that rides in the same product):
    the return value is then ``(planes, logits)``"""
    logits = L.linear(ctx, y, wr, torch.float32)
    idx, wts = K.moe_topk(logits, br, top, score, n_experts)
    planes = experts(ctx, y, idx, wts, wup, wdown, top, act, dtype, gated=gated, weight_on=weight_on)
    return planes if n_experts is None else (planes, logits)


def gate_mul(gu: torch.Tensor, wts: Optional[torch.Tensor], plan, act: str, h: torch.Tensor, act_params=None) -> None:
    """the gated experts' ``act(g) * u`` over the plan's sorted rows ``gu`` = [gate | up]; ``act`` "glu_clamp" with
    ``act_params`` = (limit, alpha, group): ``g' sigmoid(alpha g') (u' + 1)``, gate clamped from above, up from both
    sides; the expert's gate and up columns alternate in groups of ``group`` (the inner size: all gates, then all ups)"""
    if act == "glu_clamp":
        if wts is not None:
            raise ValueError("a weight on the input of experts with the clamped unit")
        limit, alpha, group = act_params
        K.glu_clamp(gu, h, group, limit, alpha)
    else:
        K.moe_gate_mul(gu, wts, plan, act, h)


def experts(ctx, y: torch.Tensor, idx: torch.Tensor, wts: torch.Tensor, wup: torch.Tensor, wdown: torch.Tensor,
            top: int, act: str, dtype: torch.dtype, *, gated: bool = False, weight_on: str = "output",
            act_params=None) -> torch.Tensor:
    """32-bit planes ``[top, T, width]``: plane k holds ``wts[t, k] * W_down[e] act(W_up[e] y[t])`` for ``e = idx[t,
    k]``. ``wup`` ``[E, F, width]``, ``wdown`` ``[E, width, F]``. ``gated``: ``wup`` is ``[E, 2 F, width]``, every
    expert's gate rows followed by its up rows, and the expert is ``W_down (act(W_gate y) * (W_up y))``.
    ``weight_on`` "input": the weight multiplies the expert's input instead of its output (for a gated expert:
    ``act(w g) * (w u)``, the two products being linear in their input). Picks whose index is not one of the E experts
    (below 0, or from E on) take no part in the products: their rows of the planes are left unwritten"""
    T, width = y.shape
    E, F, _ = wup.shape
    if weight_on not in ("output", "input") or (weight_on == "input" and not gated):
        raise ValueError("a weight on the experts' input is built for gated experts")
    if ctx.fast:
        from . import fast
        planes = fast.moe_experts(ctx, y, idx, wts, wup, wdown, top, act, gated, weight_on, act_params)
        if planes is not None:
            return planes
    plan = K.moe_plan(idx, E, K.moe_gemm_tile())
    h = torch.empty((T * top, F), dtype=dtype, device=y.device)
    K.moe_gemm_up(y, wup, plan, top, "none" if gated else act, h)
    if gated:
        gu, h = h, torch.empty((T * top, F // 2), dtype=dtype, device=y.device)
        gate_mul(gu, wts if weight_on == "input" else None, plan, act, h, act_params)
    planes = torch.empty((top, T, width), dtype=torch.float32, device=y.device)
    if weight_on == "input":
        from . import fast
        wts = fast._ones_like(wts)
    K.moe_gemm_down(h, wdown, plan, wts, top, planes)
    return planes
