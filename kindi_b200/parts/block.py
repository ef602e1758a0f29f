"""The pre-norm residual block: ``x += mixer(norm1(x)); x += feed_forward(norm2(x))``.

The adds are deferred: each norm first adds the branch that the part before it produced, so a block receives the
previous block's pending branch and returns its own (the reference's arrangement, ``kindi/nanbeige.py:688-718``:
``nbq_add_rms_q8`` adds ``br`` into ``x`` before it normalises). Which mixer, feed-forward and norms a block has is
given by its spec; the names of the sub-prefixes of its tensors are parameters too. A block whose spec gives no
feed-forward (``None``) is ``x += mixer(norm1(x))`` alone and has no second norm. ``layer_scale`` (``{"mixer": name,
"feed_forward": name}``, names under the layer's prefix): each sub-layer's output is multiplied, column by column,
by that tensor before the add: ``x += ls1 * mixer(norm1(x))``.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..config.registry import part_class, register_part
from ..config.spec import PartSpec
from ..kernels import lib as K
from .base import Block, Branch, StepContext, WeightView

_DEFAULT_NAMES = {"norm1": "input_layernorm.", "mixer": "self_attn.", "norm2": "post_attention_layernorm.",
                  "feed_forward": "mlp."}
_CATEGORY = {"norm1": "norm", "mixer": "mixer", "norm2": "norm", "feed_forward": "feed_forward"}


class PreNormBlock(Block):
    @classmethod
    def _names(cls, spec: PartSpec):
        n = dict(_DEFAULT_NAMES)
        n.update(spec.get("names") or {})
        return n

    @classmethod
    def _roles(cls, spec: PartSpec):
        """(role, sub-prefix) of the parts the block has: without a feed-forward there is no second norm either"""
        has_ff = spec.get("feed_forward") is not None
        return [(role, sub) for role, sub in cls._names(spec).items()
                if has_ff or role not in ("norm2", "feed_forward")]

    @classmethod
    def _scales(cls, spec: PartSpec):
        """{role: tensor name} of the sub-layers whose output has a learned per-column scale"""
        has_ff = spec.get("feed_forward") is not None
        return {role: name for role, name in (spec.get("layer_scale") or {}).items()
                if role == "mixer" or (role == "feed_forward" and has_ff)}

    @classmethod
    def tensor_shapes(cls, spec: PartSpec, width: int) -> Dict[str, Tuple[int, ...]]:
        out = {}
        for role, sub in cls._roles(spec):
            ps: PartSpec = spec[role]
            for suffix, shape in part_class(_CATEGORY[role], ps.kind).tensor_shapes(ps, width).items():
                out[sub + suffix] = shape
        for name in cls._scales(spec).values():
            out[name] = (width,)
        return out

    @classmethod
    def tensor_init(cls, spec: PartSpec, width: int) -> Dict[str, str]:
        out = {}
        for role, sub in cls._roles(spec):
            ps: PartSpec = spec[role]
            for suffix, kind in part_class(_CATEGORY[role], ps.kind).tensor_init(ps, width).items():
                out[sub + suffix] = kind
        for name in cls._scales(spec).values():
            out[name] = "gain"
        return out

    @classmethod
    def cache_need(cls, spec: PartSpec, width: int):
        ps: PartSpec = spec["mixer"]
        return part_class("mixer", ps.kind).cache_need(ps, width)

    def __init__(self, spec, width, weights: WeightView, *, dtype, device):
        super().__init__(spec, width, weights, dtype=dtype, device=device)
        names = self._names(spec)

        def make(role):
            ps: PartSpec = spec[role]
            return part_class(_CATEGORY[role], ps.kind)(ps, width, weights.sub(names[role]), dtype=dtype,
                                                        device=device)
        self.norm1, self.mixer = make("norm1"), make("mixer")
        self.norm2 = self.feed_forward = None
        if spec.get("feed_forward") is not None:
            self.norm2, self.feed_forward = make("norm2"), make("feed_forward")
        scales = self._scales(spec)
        self.scale1 = weights(scales["mixer"]) if "mixer" in scales else None
        self.scale2 = weights(scales["feed_forward"]) if "feed_forward" in scales else None
        self.graph_safe = all(p.graph_safe for p in self._parts())

    def _parts(self):
        return [p for p in (self.norm1, self.mixer, self.norm2, self.feed_forward) if p is not None]

    def forward(self, ctx: StepContext, x, pending: Optional[Branch]) -> Optional[Branch]:
        y = self.norm1.add_norm(ctx, x, pending)
        pending = self.mixer.forward(ctx, y).with_bias_plane()
        pending.scale = self.scale1
        if self.feed_forward is None:
            return pending
        y = self.norm2.add_norm(ctx, x, pending)
        pending = self.feed_forward.forward(ctx, y)
        pending.scale = self.scale2
        return pending

    def bytes_read(self) -> int:
        return sum(p.bytes_read() for p in self._parts())


class ParallelBlock(PreNormBlock):
    """mixer and feed-forward side by side on the same residual: ``x += m * (mixer(norm1(x)) + feed_forward(norm2(x)))``,
    each with a norm of its own. ``residual_mult`` (m, default 1) is a parameter; without a feed-forward the block is
    ``x += m * mixer(norm1(x))``. The block returns ONE pending branch: the mixer's planes followed by the
    feed-forward's, with m as the branch's per-column scale, so the next norm adds ``m * (sum of the planes)``."""

    def __init__(self, spec, width, weights: WeightView, *, dtype, device):
        super().__init__(spec, width, weights, dtype=dtype, device=device)
        if self.scale1 is not None or self.scale2 is not None:
            raise ValueError("a parallel block has one residual multiplier, not a learned scale per sub-layer")
        m = float(spec.get("residual_mult", 1.0))
        self.mult = None if m == 1.0 else torch.full((width,), m, dtype=torch.float32, device=device)

    def forward(self, ctx: StepContext, x, pending: Optional[Branch]) -> Optional[Branch]:
        y1 = self.norm1.add_norm(ctx, x, pending)              # (adds the pending branch into x)
        y2 = self.norm2.add_norm(ctx, x, None) if self.feed_forward is not None else None
        a = self.mixer.forward(ctx, y1).with_bias_plane()
        if a.scale is not None:
            raise NotImplementedError("a scaled branch inside a parallel block")
        planes = a.parts
        if self.feed_forward is not None:
            b = self.feed_forward.forward(ctx, y2)
            if b.scale is not None:
                raise NotImplementedError("a scaled branch inside a parallel block")
            planes = torch.cat([a.parts, b.parts], dim=0)
        return Branch(planes, self.mult)


class PostNormBlock(PreNormBlock):
    """the norm sits on each sub-layer's OUTPUT and the sub-layers read the residual stream itself:
    ``x += ls1 * norm1(mixer(x))``, then ``x += ls2 * norm2(feed_forward(x))`` (``layer_scale`` as in the pre-norm
    block; without it the factor is one). The norms must be RMS norms (they are given as parts so that their eps and
    the gains' names are parameters; the block reads ``weight`` and ``eps`` of them). One kernel sums a branch's
    planes, normalises, scales, adds into the 32-bit stream and writes the stream in the run dtype for the next
    sub-layer to read; the block therefore returns no pending branch, and hands the run-dtype rows of ITS output to
    the next block of its kind through the step's scratch (a block of another kind, or the final norm, reads the
    32-bit stream)."""

    def __init__(self, spec, width, weights: WeightView, *, dtype, device):
        super().__init__(spec, width, weights, dtype=dtype, device=device)
        for n in (self.norm1, self.norm2):
            if n is not None and not (hasattr(n, "weight") and hasattr(n, "eps") and not hasattr(n, "bias")):
                raise ValueError("a post-norm block takes RMS norms")
        for sc, n in ((self.scale1, self.norm1), (self.scale2, self.norm2)):
            if sc is not None and sc.dtype != n.weight.dtype:
                raise ValueError("layer scale and norm gains of %s are stored in different dtypes" % weights.prefix)

    def _rows(self, ctx: StepContext, x):
        """the stream in the run dtype: what the block before left for this step, else a copy made now"""
        y = ctx.scratch.pop(("stream rows", x.data_ptr()), None)
        if y is not None:
            return y
        if self.dtype == torch.float32:
            return x
        y = torch.empty(x.shape, dtype=self.dtype, device=x.device)
        K.cast_rows(x, y)
        return y

    def _add(self, ctx: StepContext, x, branch: Branch, norm, scale):
        if branch.scale is not None:
            raise NotImplementedError("a branch with a scale of its own inside a post-norm block")
        y = x if self.dtype == torch.float32 else torch.empty(x.shape, dtype=self.dtype, device=x.device)
        K.postnorm_add(x, branch.parts, branch.bias, norm.weight, scale, norm.eps,
                       None if self.dtype == torch.float32 else y)
        return y

    def forward(self, ctx: StepContext, x, pending: Optional[Branch]) -> Optional[Branch]:
        if pending is not None:
            # a block of another kind ran before: its branch joins the stream as it is
            if pending.scale is not None:
                raise NotImplementedError("a scaled pending branch in front of a post-norm block")
            K.residual_add(x, pending.with_bias_plane().parts, None)
        y = self._rows(ctx, x)
        y = self._add(ctx, x, self.mixer.forward(ctx, y), self.norm1, self.scale1)
        if self.feed_forward is not None:
            y = self._add(ctx, x, self.feed_forward.forward(ctx, y), self.norm2, self.scale2)
        ctx.scratch[("stream rows", x.data_ptr())] = y
        return None


register_part("block", "prenorm", PreNormBlock)
register_part("block", "postnorm", PostNormBlock)
register_part("block", "parallel", ParallelBlock)
