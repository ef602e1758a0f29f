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


def experts(ctx, y: torch.Tensor, idx: torch.Tensor, wts: torch.Tensor, wup: torch.Tensor, wdown: torch.Tensor,
            top: int, act: str, dtype: torch.dtype, *, gated: bool = False, weight_on: str = "output") -> torch.Tensor:
    """32-bit planes ``[top, T, width]``: plane k holds ``wts[t, k] * W_down[e] act(W_up[e] y[t])`` for ``e = idx[t,
    k]``. ``wup`` ``[E, F, width]``, ``wdown`` ``[E, width, F]``. ``gated``: ``wup`` is ``[E, 2 F, width]``, every
    expert's gate rows followed by its up rows, and the expert is ``W_down (act(W_gate y) * (W_up y))``.
    ``weight_on`` "input": the weight multiplies the expert's input instead of its output (for a gated expert:
    ``act(w g) * (w u)``, the two products being linear in their input)"""
    T, width = y.shape
    E, F, _ = wup.shape
    if weight_on not in ("output", "input") or (weight_on == "input" and not gated):
        raise ValueError("a weight on the experts' input is built for gated experts")
    if ctx.fast:
        from . import fast
        planes = fast.moe_experts(ctx, y, idx, wts, wup, wdown, top, act, gated, weight_on)
        if planes is not None:
            return planes
    plan = K.moe_plan(idx, E, K.moe_gemm_tile())
    h = torch.empty((T * top, F), dtype=dtype, device=y.device)
    K.moe_gemm_up(y, wup, plan, top, "none" if gated else act, h)
    if gated:
        gu, h = h, torch.empty((T * top, F // 2), dtype=dtype, device=y.device)
        K.moe_gate_mul(gu, wts if weight_on == "input" else None, plan, act, h)
    planes = torch.empty((top, T, width), dtype=torch.float32, device=y.device)
    if weight_on == "input":
        from . import fast
        wts = fast._ones_like(wts)
    K.moe_gemm_down(h, wdown, plan, wts, top, planes)
    return planes
