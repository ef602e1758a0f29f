"""Causal attention without a softmax, with a learned distance bias, over the paged cache.

``q, k, v = W y (+ biases)`` with H query heads and G key/value heads (query head h reads key/value head
``h // (H / G)``); each then passes a short causal convolution over time per channel (``conv`` taps, no activation;
the last ``conv - 1`` projected rows of a sequence are part of its state). There is no rotation; positions enter in
two ways only: the query at position p is multiplied by ``1 + coef * ln((p + 1) // every + 1)`` (``q_temp``), and the
score of query i and key j gets the bias ``rel[bucket(i - j), h]`` with, for a table of B rows and ``far`` = the
distance at which the last row is reached,

    bucket(n) = n                                                            for n < B / 2
                min(B - 1, B / 2 + floor(ln(n / (B / 2)) / ln(far / (B / 2)) * (B - B / 2)))   otherwise.

Values are divided per head by their root mean square (``v_norm``: its eps) before they are cached. The weight of a
visible key (j <= i) is ``sigmoid(q . k * scale + bias + pb[h])``; weights are not normalised over keys; the heads'
weighted sums of values go through ``W_o`` (+ bias), which the branch carries as its ``bias``.

The three projections are one product. The convolution, the temperature, the value norm, scores, weights and sums are
32-bit. The bias table and the per-head constant are folded into one table over the distance when the part is built
(64-bit on the host): ``[H, ceil(far) + 1]``, whose last entry stands for every larger distance. The cache and the
kernels know one head size: keys and values are stored ``max(head_dim, v_head_dim)`` wide, rounded up to 64 or 128
(the head sizes of the tensor-core kernel for prompts) or, beyond 128, to a multiple of eight, zero beyond their own
size. ``conv``: the taps of the tensors ``<projection>.conv`` (one tap is a factor per channel; absent or 0: no
convolution). Sizes, ``scale``, ``conv``, ``bias``, ``q_temp``, ``v_norm``, ``rel`` (``{"name", "far"}`` and
optionally ``"rows"``; without it the table's own shape gives its rows), ``head_bias`` and the tensors' suffixes
(``names``) are parameters of the part.
"""
from __future__ import annotations

import math
from typing import Dict, Tuple

import torch

from ..config.registry import register_part
from ..config.spec import PartSpec
from ..kernels import attention as A
from ..kernels import lib as K
from ..kernels import linear as L
from .base import Branch, KVNeed, Mixer, StateNeed, StepContext, WeightView
from .gated_delta import pad_rows

_DEFAULT_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "conv": "%s.conv", "bias": "%s.b"}
DEFAULT_REL_ROWS = 16


def distance_bucket(n: int, rows: int, far: float) -> int:
    """the row of a distance-bias table of ``rows`` rows for the distance ``n >= 0``: one row per distance below
    ``rows // 2``, then rows spaced evenly in the logarithm up to ``far``, where the last row begins"""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def _pad_heads(w: torch.Tensor, n: int, have: int, want: int) -> torch.Tensor:
    if have == want:
        return w
    out = torch.zeros((n, want) + tuple(w.shape[1:]), dtype=w.dtype, device=w.device)
    out[:, :have] = w.view((n, have) + tuple(w.shape[1:]))
    return out.view((n * want,) + tuple(w.shape[1:]))


class SigmoidAttention(Mixer):
    @classmethod
    def _names(cls, spec: PartSpec):
        n = dict(_DEFAULT_NAMES)
        n.update(spec.get("names") or {})
        return n

    @classmethod
    def _sizes(cls, spec: PartSpec):
        H, G = int(spec["n_heads"]), int(spec.get("n_kv_heads") or spec["n_heads"])
        d = int(spec["head_dim"])
        return H, G, d, int(spec.get("v_head_dim") or d), int(spec.get("conv") or 0)

    @classmethod
    def _cache_dim(cls, spec: PartSpec) -> int:
        _, _, d, dv, _ = cls._sizes(spec)
        n = max(d, dv)
        # (the tensor-core kernel knows head sizes 64 and 128: smaller heads are stored that wide)
        return 64 if n <= 64 else 128 if n <= 128 else (n + 7) // 8 * 8

    @classmethod
    def tensor_shapes(cls, spec: PartSpec, width: int) -> Dict[str, Tuple[int, ...]]:
        H, G, d, dv, taps = cls._sizes(spec)
        n = cls._names(spec)
        rows = {"q": H * d, "k": G * d, "v": G * dv}
        out = {n[k]: (r, width) for k, r in rows.items()}
        out[n["o"]] = (width, H * dv)
        if spec.get("bias"):
            out.update({n["bias"] % n[k]: (r,) for k, r in rows.items()})
            out[n["bias"] % n["o"]] = (width,)
        if taps >= 1:
            out.update({n["conv"] % n[k]: (r, taps) for k, r in rows.items()})
        rel = spec.get("rel")
        if rel:
            # (the table's own shape gives its rows unless the spec fixes them; a random model gets DEFAULT_REL_ROWS)
            out[rel["name"]] = (int(rel["rows"]) if rel.get("rows") else -DEFAULT_REL_ROWS, H)
        if spec.get("head_bias"):
            out[spec["head_bias"]] = (H,)
        return out

    @classmethod
    def cache_need(cls, spec: PartSpec, width: int):
        H, G, d, dv, taps = cls._sizes(spec)
        needs = [KVNeed(G, cls._cache_dim(spec))]
        if taps > 1:
            needs.append(StateNeed((taps - 1, H * d + G * d + G * dv)))
        return tuple(needs)

    def __init__(self, spec, width, weights: WeightView, *, dtype, device):
        super().__init__(spec, width, weights, dtype=dtype, device=device)
        self.H, self.G, self.d, self.dv, self.taps = self._sizes(spec)
        self.hd = self._cache_dim(spec)
        H, G, d, dv = self.H, self.G, self.d, self.dv
        if H % G:
            raise ValueError("n_heads %d is not a multiple of n_kv_heads %d" % (H, G))
        if self.hd > 512:
            raise ValueError("head sizes up to 512 are supported, found %d" % self.hd)
        if not (0 <= self.taps <= 8):
            raise ValueError("a short convolution has up to 8 taps (0: none), found %d" % self.taps)
        self.scale = float(spec.get("scale") or 1.0 / math.sqrt(d))
        n = self._names(spec)
        ws = [weights(n[k]) for k in ("q", "k", "v")]
        if len({w.dtype for w in ws}) != 1:
            raise ValueError("q, k and v weights of %s are stored in different dtypes" % weights.prefix)
        self.C = H * d + G * d + G * dv
        self.w_in = pad_rows(torch.cat(ws, dim=0))
        self.b_in = self.b_o = None
        if spec.get("bias"):
            self.b_in = torch.cat([weights(n["bias"] % n[k]) for k in ("q", "k", "v")]).to(torch.float32).contiguous()
            self.b_o = weights(n["bias"] % n["o"]).to(torch.float32).contiguous()
        if self.taps >= 1:
            conv = torch.cat([weights(n["conv"] % n[k]) for k in ("q", "k", "v")], dim=0)
        else:
            conv = torch.ones((self.C, 1), device=device)
        self.w_conv = conv.to(torch.float32).contiguous()
        qt = spec.get("q_temp") or {}
        self.q_coef, self.q_every = float(qt.get("coef", 0.0)), int(qt.get("every", 1))
        if self.q_every < 1:
            raise ValueError("q_temp.every must be at least 1, found %d" % self.q_every)
        vn = spec.get("v_norm")
        self.v_norm, self.v_eps = vn is not None, float(vn or 0.0)
        # the heads' outputs come hd wide out of the attention kernel: zero columns of W_o meet what lies beyond v_dim
        wo = weights(n["o"])
        if dv != self.hd:
            wo = _pad_heads(wo.t().contiguous(), H, dv, self.hd).t().contiguous()
        self.w_o = wo
        self.bias_table = self._bias_table(spec, weights, device)
        self._no_tails = torch.zeros((1, 1), dtype=torch.float32, device=device)

    def _bias_table(self, spec: PartSpec, weights: WeightView, device):
        """float32 [H, n]: entry (h, dist) = rel[bucket(dist), h] + head_bias[h]; the last entry stands for every larger
        distance. None when the part has neither"""
        rel, hb = spec.get("rel"), spec.get("head_bias")
        if not rel and not hb:
            return None
        H = self.H
        const = weights(hb).to(torch.float64).cpu() if hb else torch.zeros(H, dtype=torch.float64)
        if not rel:
            return const.view(H, 1).to(torch.float32).to(device).contiguous()
        table = weights(rel["name"]).to(torch.float64).cpu()                       # [rows, H]
        rows, far = int(table.shape[0]), float(rel["far"])
        if rows < 2 or not (far > rows // 2):
            raise ValueError("a distance bias needs at least two rows and far > rows / 2; found rows %d, far %r"
                             % (rows, far))
        n = int(math.ceil(far)) + 1
        idx = torch.tensor([distance_bucket(k, rows, far) if k < far else rows - 1 for k in range(n)])
        return (table[idx].t() + const.view(H, 1)).to(torch.float32).to(device).contiguous()

    def forward(self, ctx: StepContext, y: torch.Tensor) -> Branch:
        H, G, d, dv, hd, C = self.H, self.G, self.d, self.dv, self.hd, self.C
        a = L.rows_or_planes(ctx, y, self.w_in, self.dtype)
        entry = ctx.entry.cache
        pool, table, n_pages = ctx.cache.kv_view(entry)
        tails = ctx.cache.state_view(entry, self.state_base).view(-1, (self.taps - 1) * C) if self.taps > 1 \
            else self._no_tails
        c = (torch.zeros if ctx.graph else torch.empty)((ctx.T, C), dtype=torch.float32, device=y.device)
        K.short_conv(a, 0, C, self.b_in, self.w_conv, False, tails, ctx.pos, ctx.seq, ctx.slot, ctx.q_start, c)
        q = torch.empty((ctx.T, H * hd), dtype=self.dtype, device=y.device)
        K.sigattn_prep(c, H, G, d, dv, hd, self.q_coef, self.q_every, self.v_norm, self.v_eps, ctx.pos, ctx.seq,
                       ctx.slot, q, pool, table, n_pages, ctx.status)
        att = torch.empty((ctx.T, H * hd), dtype=self.dtype, device=y.device)
        A.sigmoid_attention(ctx, q, att, H, G, hd, self.scale, self.bias_table, pool, table, n_pages)
        return Branch(L.planes(ctx, att, self.w_o), bias=self.b_o)

    def bytes_read(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.w_o))


register_part("mixer", "sigmoid_attention", SigmoidAttention)
