"""The gated delta rule: a recurrent mixer whose cache is a fixed-size state per head.

``q = W_q y``, ``k = W_k y`` (G heads of ``head_dim``), ``v = W_v y`` (H heads of ``v_head_dim``; head h uses query/key
head ``h // (H / G)``), no biases. Each passes a short causal convolution over time per channel (``conv`` taps, the
last tap meets the current token, zeros before the sequence's start) and silu. q and k become unit vectors per head,
``x / sqrt(sum x^2 + unit_eps)``, q also times ``head_dim^(-1/2)``. Per head, with ``beta = sigmoid(W_b y)`` and the
decay ``g = exp(-exp(A_log) * softplus(W_a y + dt_bias))``:

    S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q

so the read-out sees the current token's write. Each head's o is divided by its root mean square over ``v_head_dim``
(``eps``), multiplied by the gains ``norm`` (shared by the heads) and by ``silu(W_g y)``; then ``W_o``.

All six projections are one product. The convolution, the unit norms, beta, the decay, the recurrence and the norm
are 32-bit. The cache entry holds two states per sequence, zero when it starts: S (``[H, v_head_dim, head_dim]``) and
the last ``conv - 1`` projected rows of q, k and v. Sizes, ``conv``, ``eps``, ``unit_eps`` and the tensors' suffixes
(``names``) are parameters of the part.
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from ..config.registry import register_part
from ..config.spec import PartSpec
from ..kernels import lib as K
from ..kernels import linear as L
from .base import Branch, Mixer, StateNeed, StepContext, WeightView

_DEFAULT_NAMES = {"q": "q", "k": "k", "v": "v", "conv": "%s.conv", "beta": "b", "decay": "a", "A_log": "A_log",
                  "dt_bias": "dt_bias", "norm": "norm", "gate": "g", "o": "o"}


def pad_rows(w: torch.Tensor, multiple: int = 8) -> torch.Tensor:
    """zero rows below a joined weight so that its row count is a multiple the tensor-core products take"""
    pad = -w.shape[0] % multiple
    if not pad:
        return w.contiguous()
    return torch.cat([w, torch.zeros((pad,) + tuple(w.shape[1:]), dtype=w.dtype, device=w.device)], dim=0).contiguous()


class GatedDeltaRule(Mixer):
    @classmethod
    def _names(cls, spec: PartSpec):
        n = dict(_DEFAULT_NAMES)
        n.update(spec.get("names") or {})
        return n

    @classmethod
    def _sizes(cls, spec: PartSpec):
        H, G = int(spec["n_heads"]), int(spec.get("n_kv_heads") or spec["n_heads"])
        return H, G, int(spec["head_dim"]), int(spec["v_head_dim"]), int(spec.get("conv") or 0)

    @classmethod
    def tensor_shapes(cls, spec: PartSpec, width: int) -> Dict[str, Tuple[int, ...]]:
        H, G, d, dv, taps = cls._sizes(spec)
        n = cls._names(spec)
        out = {n["q"]: (G * d, width), n["k"]: (G * d, width), n["v"]: (H * dv, width), n["beta"]: (H, width),
               n["decay"]: (H, width), n["A_log"]: (H,), n["dt_bias"]: (H,), n["norm"]: (dv,),
               n["gate"]: (H * dv, width), n["o"]: (width, H * dv)}
        if taps >= 1:
            out.update({n["conv"] % n["q"]: (G * d, taps), n["conv"] % n["k"]: (G * d, taps),
                        n["conv"] % n["v"]: (H * dv, taps)})
        return out

    @classmethod
    def tensor_init(cls, spec: PartSpec, width: int) -> Dict[str, str]:
        return {cls._names(spec)["norm"]: "gain"}

    @classmethod
    def cache_need(cls, spec: PartSpec, width: int):
        H, G, d, dv, taps = cls._sizes(spec)
        needs = [StateNeed((H, dv, d))]
        if taps > 1:
            needs.append(StateNeed((taps - 1, 2 * G * d + H * dv)))
        return tuple(needs)

    def __init__(self, spec, width, weights: WeightView, *, dtype, device):
        super().__init__(spec, width, weights, dtype=dtype, device=device)
        self.H, self.G, self.d, self.dv, self.taps = self._sizes(spec)
        if self.H % self.G:
            raise ValueError("n_heads %d is not a multiple of n_kv_heads %d" % (self.H, self.G))
        if self.d > 256:
            raise ValueError("the delta rule supports key sizes up to 256, found %d" % self.d)
        if not (0 <= self.taps <= 8):
            raise ValueError("a short convolution has up to 8 taps (0: none), found %d" % self.taps)
        self.eps = float(spec["eps"])
        self.unit_eps = float(spec.get("unit_eps", 1e-6))
        n = self._names(spec)
        ws = [weights(n[k]) for k in ("q", "k", "v", "beta", "decay", "gate")]
        if len({w.dtype for w in ws}) != 1:
            raise ValueError("the projections of %s are stored in different dtypes" % weights.prefix)
        self.w_in = pad_rows(torch.cat(ws, dim=0))              # [q | k | v | beta | decay | gate]
        self.C = 2 * self.G * self.d + self.H * self.dv
        if self.taps >= 1:
            conv = torch.cat([weights(n["conv"] % n[k]) for k in ("q", "k", "v")], dim=0)
        else:
            conv = torch.ones((self.C, 1), device=device)
        self.w_conv = conv.to(torch.float32).contiguous()
        self.a_log = weights(n["A_log"]).to(torch.float32).contiguous()
        self.dt_bias = weights(n["dt_bias"]).to(torch.float32).contiguous()
        self.g_norm = weights(n["norm"]).to(torch.float32).contiguous()
        self.w_o = weights(n["o"])
        self._no_tails = torch.zeros((1, 1), dtype=torch.float32, device=device)

    def forward(self, ctx: StepContext, y: torch.Tensor) -> Branch:
        H, G, d, dv, C = self.H, self.G, self.d, self.dv, self.C
        a = L.rows_or_planes(ctx, y, self.w_in, self.dtype)
        entry = ctx.entry.cache
        state = ctx.cache.state_view(entry, self.state_base).view(-1, H * dv * d)
        tails = ctx.cache.state_view(entry, self.state_base + 1).view(-1, (self.taps - 1) * C) if self.taps > 1 \
            else self._no_tails
        new = torch.zeros if ctx.graph else torch.empty       # (padding rows of a recorded step are written by nobody)
        c = new((ctx.T, C), dtype=torch.float32, device=y.device)
        K.short_conv(a, 0, C, None, self.w_conv, True, tails, ctx.pos, ctx.seq, ctx.slot, ctx.q_start, c)
        o = new((ctx.T, H * dv), dtype=torch.float32, device=y.device)
        # prompts of the serving path: the chunked form (32-bit sums that differ from the token-by-token kernel's by
        # rounding); single tokens, short steps and the true 32-bit path: token by token
        K.delta_rule(c, a, C, C + H, self.a_log, self.dt_bias, ctx.B, H, G, d, dv, self.unit_eps, ctx.q_start,
                     ctx.slot, state, o, max_rows=ctx.max_q if ctx.fast and not ctx.decode else 0)
        yn = torch.empty((ctx.T, H * dv), dtype=self.dtype, device=y.device)
        K.head_norm_gate(o, H, dv, self.g_norm, self.eps, a, C + 2 * H, "silu", yn)
        return Branch(L.planes(ctx, yn, self.w_o))

    def bytes_read(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.w_o))


register_part("mixer", "gated_delta", GatedDeltaRule)
