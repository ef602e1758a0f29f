"""Mixture-of-experts feed-forward: a router picks ``top_k`` of ``n_experts`` small feed-forwards for every row.

Router: ``z = W_r y + b_r`` with 32-bit accumulation (``y`` in the run dtype); the ``top_k`` experts with the largest
``z`` are chosen and weighted by the softmax over the chosen values only. Expert: ``W_down act(W_up y)``, no biases,
no gate; ``act`` is a parameter (``relu2``: the square of relu; ``silu``; ``gelu_tanh``; ``none``). The branch is the
weighted sum of the chosen experts' outputs: it is returned as ``top_k`` 32-bit planes (plane k holds each row's k-th
expert, already weighted), which the next norm adds in order, so every row's sum has the same order in every batch.

All rows of a step go through the experts as grouped products over (row, pick) pairs sorted by expert; the sort
happens on the device, so the part can be recorded. Sizes, the activation, whether the router has a bias and the
tensors' suffixes (``router``, ``router_bias``, ``up`` and ``down`` with ``%d`` for the expert) are parameters.

Further options, all parameters:

* ``gated``: an expert is ``W_down (act(W_gate y) * (W_up y))`` (suffix ``gate``, with ``%d``).
* ``score`` = ``sigmoid``: the weights are the chosen experts' own ``sigmoid(z)``, not normalised over the chosen
  ones (the order of the logits is the order of their sigmoids, so the pick is the same).
* ``weight_on`` = ``input`` (gated experts): the weight multiplies the expert's input, ``expert(w y)``, which is
  ``W_down (act(w g) * (w u))`` with ``g = W_gate y``, ``u = W_up y``.
* ``score`` = ``softmax_all``: the scores are the softmax over ALL router outputs. The choice goes by score +
  ``correction`` (a tensor suffix, one number per output, or None), the weights by the scores alone, divided by the
  chosen ones' sum. ``groups`` (``{"count", "keep"}``): the outputs form ``count`` equal groups of neighbours, a
  group's value is its largest choice score, and only outputs of the ``keep`` best groups can be chosen.
* ``identity`` (n): the router has ``n_experts + n`` outputs (groups are formed over all of them); the last n are
  experts without tensors whose output is their input, times the weight.
* ``activation`` = ``glu_clamp`` (gated experts; ``limit``, ``alpha`` default 1.702): an expert is
  ``W_down (g' sigmoid(alpha g') (u' + 1))`` with ``g' = min(W_gate y, limit)``, ``u' = clamp(W_up y, -limit, limit)``.
  A shared expert may have the same activation with a limit of its own (``shared.limit``).
* ``shared`` (``{"intermediate", "activation", "names": {gate, up, down}, "row_gate": suffix or None}``): a gated
  feed-forward that every row passes through, added as one more plane; with ``row_gate`` (a ``[1, width]`` tensor)
  it is multiplied by ``sigmoid(W_sg y)``, one number per row, whose logit rides in the router's product.
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from ..config.registry import register_part
from ..config.spec import PartSpec
from ..kernels import lib as K
from ..kernels import linear as L
from ..kernels import moe as M
from .base import Branch, FeedForward, StepContext, WeightView

_DEFAULT_NAMES = {"router": "router.weight", "router_bias": "router.bias", "up": "experts.%d.up_proj.weight",
                  "down": "experts.%d.down_proj.weight", "gate": "experts.%d.gate_proj.weight"}
_SHARED_NAMES = {"gate": "shared.gate_proj.weight", "up": "shared.up_proj.weight", "down": "shared.down_proj.weight"}


class MixtureOfExperts(FeedForward):
    @classmethod
    def _names(cls, spec: PartSpec):
        n = dict(_DEFAULT_NAMES)
        n.update(spec.get("names") or {})
        return n

    @classmethod
    def _sizes(cls, spec: PartSpec):
        return int(spec["n_experts"]), int(spec["top_k"]), int(spec["intermediate"])

    @classmethod
    def tensor_shapes(cls, spec: PartSpec, width: int) -> Dict[str, Tuple[int, ...]]:
        E, top, f = cls._sizes(spec)
        n = cls._names(spec)
        n_out = E + int(spec.get("identity") or 0)
        out = {n["router"]: (n_out, width)}
        if spec.get("router_bias", True):
            out[n["router_bias"]] = (E,)
        if spec.get("correction"):
            out[spec["correction"]] = (n_out,)
        for e in range(E):
            out[n["up"] % e] = (f, width)
            out[n["down"] % e] = (width, f)
            if spec.get("gated"):
                out[n["gate"] % e] = (f, width)
        sh = spec.get("shared")
        if sh:
            sn = cls._shared_names(sh)
            fs = int(sh["intermediate"])
            out.update({sn["gate"]: (fs, width), sn["up"]: (fs, width), sn["down"]: (width, fs)})
            if sh.get("row_gate"):
                out[sh["row_gate"]] = (1, width)
        return out

    @classmethod
    def _shared_names(cls, sh):
        n = dict(_SHARED_NAMES)
        n.update(sh.get("names") or {})
        return n

    @classmethod
    def tensor_init(cls, spec: PartSpec, width: int) -> Dict[str, str]:
        return {cls._names(spec)["router_bias"]: "zero"} if spec.get("router_bias", True) else {}

    def __init__(self, spec, width, weights: WeightView, *, dtype, device):
        super().__init__(spec, width, weights, dtype=dtype, device=device)
        self.E, self.top, self.f = self._sizes(spec)
        if not (1 <= self.top <= self.E + int(spec.get("identity") or 0)):
            raise ValueError("top_k %d must lie between 1 and the %d experts" % (self.top, self.E + int(spec.get("identity") or 0)))
        self.act = str(spec.get("activation", "relu2"))
        if self.act not in K.ACT and not (self.act == "glu_clamp" and spec.get("gated")):
            raise ValueError("unknown activation %r; known: %s, and glu_clamp for gated experts"
                             % (self.act, ", ".join(sorted(K.ACT))))
        # (the clamped unit's gate and up rows alternate in groups that the products' epilogues can finish, like a dense
        # gated feed-forward's)
        self.act_params = (float(spec["limit"]), float(spec.get("alpha", 1.702)),
                           L.GATE_UP_GROUP if self.f % L.GATE_UP_GROUP == 0 else self.f) if self.act == "glu_clamp" else None
        self.n_identity = int(spec.get("identity") or 0)
        self.n_out = self.E + self.n_identity
        n = self._names(spec)
        self.wr = weights(n["router"])
        self.br = weights(n["router_bias"]).to(torch.float32).contiguous() if spec.get("router_bias", True) else None
        ups = [weights(n["up"] % e) for e in range(self.E)]
        downs = [weights(n["down"] % e) for e in range(self.E)]
        if len({w.dtype for w in ups + downs}) != 1:
            raise ValueError("the expert weights of %s are stored in different dtypes" % weights.prefix)
        self.gated = bool(spec.get("gated"))
        self.score = str(spec.get("score") or "softmax")
        self.weight_on = str(spec.get("weight_on") or "output")
        if self.score not in K.MOE_SCORE and self.score != "softmax_all":
            raise ValueError("unknown router score %r; known: %s, softmax_all"
                             % (self.score, ", ".join(sorted(K.MOE_SCORE))))
        self.correction = None
        self.groups = (1, 1)
        if self.score == "softmax_all":
            if self.br is not None:
                raise ValueError("a router that scores over all its outputs takes a correction, not a bias")
            if spec.get("correction"):
                self.correction = weights(spec["correction"]).to(torch.float32).contiguous()
            g = spec.get("groups") or {}
            self.groups = (int(g.get("count", 1)), int(g.get("keep", g.get("count", 1))))
            if self.groups[0] < 1 or self.n_out % self.groups[0] or not (1 <= self.groups[1] <= self.groups[0]):
                raise ValueError("%d router outputs do not form %d equal groups of which %d are kept"
                                 % (self.n_out, self.groups[0], self.groups[1]))
            if self.top > self.groups[1] * (self.n_out // self.groups[0]):
                raise ValueError("top_k %d exceeds the %d outputs of the kept groups"
                                 % (self.top, self.groups[1] * (self.n_out // self.groups[0])))
            if self.weight_on != "output":
                raise ValueError("a router that scores over all its outputs weighs the experts' outputs")
            pad = -self.n_out % 8           # (the products take row counts that are multiples of eight)
            if pad:
                self.wr = torch.cat([self.wr, torch.zeros((pad, width), dtype=self.wr.dtype, device=self.wr.device)])
                self.wr = self.wr.contiguous()
        elif self.n_identity or spec.get("correction") or spec.get("groups"):
            raise ValueError("identity experts, a correction and groups belong to the score softmax_all")
        if self.weight_on not in ("output", "input") or (self.weight_on == "input" and not self.gated):
            raise ValueError("weight_on is 'output', or 'input' for gated experts; found %r" % self.weight_on)
        if self.gated:
            gates = [weights(n["gate"] % e) for e in range(self.E)]
            if {w.dtype for w in gates} != {ups[0].dtype}:
                raise ValueError("the expert weights of %s are stored in different dtypes" % weights.prefix)
            if self.act == "glu_clamp":
                ups = [L.join_gate_up(g, u)[0] for g, u in zip(gates, ups)]   # gate and up rows in groups of 16 (or all)
            else:
                ups = [torch.cat([g, u], dim=0) for g, u in zip(gates, ups)]  # every expert: its gate rows, then up
        self.wup = torch.stack(ups).contiguous()            # [E, f (gated: 2 f), width]
        self.wdown = torch.stack(downs).contiguous()        # [E, width, f]
        self.shared = None
        sh = spec.get("shared")
        if sh:
            sn = self._shared_names(sh)
            act = str(sh.get("activation") or "silu")
            wgu, group = L.join_gate_up(weights(sn["gate"]), weights(sn["up"]))
            self.shared = (wgu, group, int(sh["intermediate"]), act, weights(sn["down"]))
            self.shared_params = (float(sh["limit"]), float(sh.get("alpha", 1.702))) if act == "glu_clamp" else None
            self.row_gate = bool(sh.get("row_gate"))
            if self.row_gate and self.score == "softmax_all":
                raise NotImplementedError("a row gate beside a router that scores over all its outputs")
            if self.row_gate:
                # the gate's logit is one more row of the router's product (zero rows fill up to a multiple of eight)
                rows = [self.wr, weights(sh["row_gate"]).to(self.wr.dtype)]
                pad = -(self.E + 1) % 8
                if pad:
                    rows.append(torch.zeros((pad, width), dtype=self.wr.dtype, device=self.wr.device))
                self.wr = torch.cat(rows, dim=0).contiguous()

    def _forward_all(self, ctx: StepContext, y: torch.Tensor) -> torch.Tensor:
        """the planes of a router that scores over all its outputs: pick inside the kept groups, the experts'
        grouped products, and the rows of picks that name an identity expert"""
        logits = L.linear(ctx, y, self.wr, torch.float32)
        idx, wts = K.moe_route(logits, self.correction, self.n_out, self.top, self.groups[0], self.groups[1])
        planes = M.experts(ctx, y, idx, wts, self.wup, self.wdown, self.top, self.act, self.dtype, gated=self.gated,
                           act_params=self.act_params)
        K.moe_identity(y, idx, wts, planes, self.E)
        return planes

    def forward(self, ctx: StepContext, y: torch.Tensor) -> Branch:
        if self.score == "softmax_all":
            planes = self._forward_all(ctx, y)
            if self.shared is None:
                return Branch(planes)
            wgu, group, fs, act, wd = self.shared
            if act == "glu_clamp":
                h = L.gate_up_glu_clamp(ctx, y, wgu, group, fs, self.dtype, *self.shared_params)
            else:
                h = L.gate_up_swiglu(ctx, y, wgu, group, fs, self.dtype, act)
            return Branch(torch.cat([planes, L.planes(ctx, h, wd)], dim=0))
        out = M.feed_forward(ctx, y, self.wr, self.br, self.wup, self.wdown, self.top, self.act, self.dtype,
                             score=self.score, gated=self.gated, weight_on=self.weight_on,
                             n_experts=self.E if self.shared is not None and self.row_gate else None)
        if self.shared is None:
            return Branch(out)
        planes, logits = out if self.row_gate else (out, None)
        wgu, group, fs, act, wd = self.shared
        h = L.gate_up_swiglu(ctx, y, wgu, group, fs, self.dtype, act)
        if logits is not None:
            K.row_gate(h, logits[:, self.E])            # W_down (s h) = s W_down h: the gate scales the row once
        return Branch(torch.cat([planes, L.planes(ctx, h, wd)], dim=0))

    def bytes_read(self) -> int:
        """the router and, of the experts, the share a single row reads (a large step reads up to all of them)"""
        per_expert = (self.wup.numel() + self.wdown.numel()) // self.E * self.wup.element_size()
        shared = 0 if self.shared is None else (self.shared[0].numel() + self.shared[4].numel()) * self.wup.element_size()
        return self.wr.numel() * self.wr.element_size() + self.top * per_expert + shared


register_part("feed_forward", "moe", MixtureOfExperts)
