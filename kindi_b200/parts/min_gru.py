"""minGRU: a gated recurrence, element by element, whose gates read only the current token.

``z = sigmoid(W_z y + b_z)``, ``u = W_x y + b_x`` (both of size ``inner``); the candidate is ``u + 1/2`` where
``u >= 0`` and ``sigmoid(u)`` where ``u < 0`` (continuous at zero, positive everywhere);
``S_t = (1 - z) S_(t-1) + z * candidate``; the output is ``W_o (S_t * silu(W_g y))``.

The three projections are one product; gates, candidate and recurrence are 32-bit. The state (``[inner]`` per
sequence, zero when it starts) lives in the cache's state storage. ``inner``, whether z and x have biases (``bias``)
and the tensors' suffixes (``names``) are parameters of the part.
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from ..config.registry import register_part
from ..config.spec import PartSpec
from ..kernels import lib as K
from ..kernels import linear as L
from .base import Branch, Mixer, StateNeed, StepContext, WeightView
from .gated_delta import pad_rows

_DEFAULT_NAMES = {"z": "z", "x": "x", "gate": "g", "o": "o", "bias": "%s.b"}


class MinGRU(Mixer):
    @classmethod
    def _names(cls, spec: PartSpec):
        n = dict(_DEFAULT_NAMES)
        n.update(spec.get("names") or {})
        return n

    @classmethod
    def tensor_shapes(cls, spec: PartSpec, width: int) -> Dict[str, Tuple[int, ...]]:
        W = int(spec["inner"])
        n = cls._names(spec)
        out = {n["z"]: (W, width), n["x"]: (W, width), n["gate"]: (W, width), n["o"]: (width, W)}
        if spec.get("bias", True):
            out.update({n["bias"] % n["z"]: (W,), n["bias"] % n["x"]: (W,)})
        return out

    @classmethod
    def tensor_init(cls, spec: PartSpec, width: int) -> Dict[str, str]:
        return {}

    @classmethod
    def cache_need(cls, spec: PartSpec, width: int):
        return StateNeed((int(spec["inner"]),))

    def __init__(self, spec, width, weights: WeightView, *, dtype, device):
        super().__init__(spec, width, weights, dtype=dtype, device=device)
        self.W = int(spec["inner"])
        n = self._names(spec)
        ws = [weights(n["z"]), weights(n["x"]), weights(n["gate"])]
        if len({w.dtype for w in ws}) != 1:
            raise ValueError("the projections of %s are stored in different dtypes" % weights.prefix)
        self.w_in = pad_rows(torch.cat(ws, dim=0))              # [z | x | gate]
        self.bz = self.bx = None
        if spec.get("bias", True):
            self.bz = weights(n["bias"] % n["z"]).to(torch.float32).contiguous()
            self.bx = weights(n["bias"] % n["x"]).to(torch.float32).contiguous()
        self.w_o = weights(n["o"])

    def forward(self, ctx: StepContext, y: torch.Tensor) -> Branch:
        W = self.W
        a = L.rows_or_planes(ctx, y, self.w_in, self.dtype)
        state = ctx.cache.state_view(ctx.entry.cache, self.state_base)
        h = (torch.zeros if ctx.graph else torch.empty)((ctx.T, W), dtype=self.dtype, device=y.device)
        K.min_gru(a, 0, W, 2 * W, W, self.bz, self.bx, ctx.B, ctx.q_start, ctx.slot, state, h,
                  max_rows=ctx.max_q)
        return Branch(L.planes(ctx, h, self.w_o))

    def bytes_read(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.w_o))


register_part("mixer", "min_gru", MinGRU)
