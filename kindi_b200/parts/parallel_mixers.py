"""Several mixers side by side on the same input: the result is the mean of their outputs, each first RMS-normed over
the model width with gains of its own (stored as they multiply, not around zero).

``branches`` lists the mixers: ``{"mixer": PartSpec, "prefix": sub-prefix of its tensors, "gain": suffix of its
gains}``; ``eps`` is the norms'. Every mixer keeps what it needs in the layer's ONE cache entry: the entry asks for
the tuple of all their needs (at most one of them may ask for keys and values), and each mixer is told where its
states begin among the entry's (``state_base``).
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from ..config.registry import part_class, register_part
from ..config.spec import PartSpec
from ..kernels import lib as K
from .base import Branch, KVNeed, Mixer, StateNeed, StepContext, WeightView


def _as_list(need):
    return [n for n in (need if isinstance(need, (tuple, list)) else [need]) if n is not None]


class ParallelMixers(Mixer):
    @classmethod
    def _branches(cls, spec: PartSpec):
        return [(b["mixer"], b.get("prefix", ""), b["gain"]) for b in spec["branches"]]

    @classmethod
    def tensor_shapes(cls, spec: PartSpec, width: int) -> Dict[str, Tuple[int, ...]]:
        out = {}
        for ps, prefix, gain in cls._branches(spec):
            for suffix, shape in part_class("mixer", ps.kind).tensor_shapes(ps, width).items():
                out[prefix + suffix] = shape
            out[gain] = (width,)
        return out

    @classmethod
    def tensor_init(cls, spec: PartSpec, width: int) -> Dict[str, str]:
        out = {}
        for ps, prefix, gain in cls._branches(spec):
            for suffix, kind in part_class("mixer", ps.kind).tensor_init(ps, width).items():
                out[prefix + suffix] = kind
            out[gain] = "gain"
        return out

    @classmethod
    def cache_need(cls, spec: PartSpec, width: int):
        needs = []
        for ps, _, _ in cls._branches(spec):
            needs += _as_list(part_class("mixer", ps.kind).cache_need(ps, width))
        if sum(isinstance(n, KVNeed) for n in needs) > 1:
            raise ValueError("mixers side by side share one cache entry: only one of them may keep keys and values")
        return tuple(needs) if needs else None

    def __init__(self, spec, width, weights: WeightView, *, dtype, device):
        super().__init__(spec, width, weights, dtype=dtype, device=device)
        self.eps = float(spec["eps"])
        self.mixers, self.gains = [], []
        n_states = 0
        branches = self._branches(spec)
        if not (1 <= len(branches) <= 4):
            raise ValueError("one to four mixers run side by side, found %d" % len(branches))
        for ps, prefix, gain in branches:
            cls = part_class("mixer", ps.kind)
            m = cls(ps, width, weights.sub(prefix), dtype=dtype, device=device)
            m.state_base = self.state_base + n_states
            n_states += sum(isinstance(n, StateNeed) for n in _as_list(cls.cache_need(ps, width)))
            self.mixers.append(m)
            self.gains.append(weights(gain).to(torch.float32).contiguous())
        self.graph_safe = all(m.graph_safe for m in self.mixers)

    def forward(self, ctx: StepContext, y: torch.Tensor) -> Branch:
        parts = []
        for m, gain in zip(self.mixers, self.gains):
            b = m.forward(ctx, y)
            if b.scale is not None:
                raise NotImplementedError("a scaled branch among mixers side by side")
            parts.append((b.parts, b.bias, gain))
        out = torch.empty((1, ctx.T, self.width), dtype=torch.float32, device=y.device)
        K.branch_norm_mean(parts, self.eps, out[0])
        return Branch(out)

    def bytes_read(self) -> int:
        return sum(m.bytes_read() for m in self.mixers)


register_part("mixer", "parallel", ParallelMixers)
