"""Causal softmax attention with grouped queries whose query and key heads pass a norm of their OWN (per head, not
over the whole projection), with a temperature on the queries, a gate per head, or two softmax maps per head that are
subtracted ("differential" attention).

``q, k, v = W y`` without biases, one product over the concatenated weights. Every query head and every key head is
divided by its root mean square over the head's ``head_dim`` elements (``head_norm``: ``{"eps", "when": "before" |
"after" the rotation, "q", "k"}``; ``q`` / ``k`` name gains of size ``head_dim`` that all heads share, None for a
unit norm). ``position`` is a rotation (``rotary`` with either pairing, partial rotation allowed) or ``none``.
``q_temp`` (``{"coef", "every"}``): queries at position p are multiplied by ``1 + coef ln(floor((p + 1) / every) + 1)``.
Scores are ``scale (q . k)``, causal, softmax over all earlier positions; softmax and the weighted sums are 32-bit.

* ``head_gate`` (a tensor suffix, ``[n_heads, width]``): head h's output is multiplied by ``sigmoid(W_g y)_h``, one
  number per head and row; the gate's rows ride in the joined product.
* ``differential`` (``{"diff", "eps", "lq1", "lk1", "lq2", "lk2"}``): the query projection holds, per head, two maps
  ``[map 1 | map 2]`` of ``head_dim`` each, and so does the key projection per key/value head; both maps attend over
  the same values. With ``lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff`` (one number for the layer) head h is
  ``o = a1 - lambda a2``, divided by its root mean square over the head's values (no gain) and multiplied by
  ``1 - diff``.

How it runs. An interleaved rotation (pairs ``(2i, 2i + 1)``) is turned into the rotate-half form the kernels know by
permuting the rows of W_q and W_k inside every head, evens first: a score is a sum over the head's elements and does
not see their order, and neither does the head's norm. Differential attention runs the library's attention kernels
on ``2 n_heads`` query heads and ``2 n_kv_heads`` key/value heads: query heads are laid out (group, map, head of the
group) so that the plain grouped-query rule ``kv = q // (heads per group)`` pairs every map with its own keys, and the
value rows of W_v are stored once per map; a small kernel then subtracts, normalises and scales. The cache and the
kernels know one head size, so the smaller of ``head_dim`` and ``v_head_dim`` is widened with zero rows as in the
``attention`` part.
"""
from __future__ import annotations

import math
from typing import Dict, Tuple

import torch

from ..config.registry import part_class, register_part
from ..config.spec import PartSpec
from ..kernels import attention as A
from ..kernels import lib as K
from ..kernels import linear as L
from .attention import _pad_heads
from .base import Branch, KVNeed, Mixer, StepContext, WeightView

_DEFAULT_NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight"}


class HeadNormAttention(Mixer):
    @classmethod
    def _sizes(cls, spec: PartSpec):
        return int(spec["n_heads"]), int(spec["n_kv_heads"]), int(spec["head_dim"]), \
            int(spec.get("v_head_dim") or spec["head_dim"])

    @classmethod
    def _maps(cls, spec: PartSpec) -> int:
        return 2 if spec.get("differential") else 1

    @classmethod
    def _cache_dim(cls, spec: PartSpec) -> int:
        """the one head size the cache and the kernels see (64 or 128 where that is near: the tensor-core kernels'
        sizes)"""
        _, _, hd, vd = cls._sizes(spec)
        m = max(hd, vd)
        if hd == vd and (hd % 8 == 0 or hd > 128):
            return hd
        return 64 if m <= 64 else 128 if m <= 128 else (m + 7) // 8 * 8

    @classmethod
    def _names(cls, spec: PartSpec):
        n = dict(_DEFAULT_NAMES)
        n.update(spec.get("names") or {})
        return n

    @classmethod
    def tensor_shapes(cls, spec: PartSpec, width: int) -> Dict[str, Tuple[int, ...]]:
        nh, nkv, hd, vd = cls._sizes(spec)
        maps = cls._maps(spec)
        n = cls._names(spec)
        out = {n["q"]: (nh * maps * hd, width), n["k"]: (nkv * maps * hd, width), n["v"]: (nkv * vd, width),
               n["o"]: (width, nh * vd)}
        hn = spec.get("head_norm")
        if hn:
            for key in ("q", "k"):
                if hn.get(key):
                    out[hn[key]] = (hd,)
        if spec.get("head_gate"):
            out[spec["head_gate"]] = (nh, width)
        d = spec.get("differential")
        if d:
            for key in ("lq1", "lk1", "lq2", "lk2"):
                out[d[key]] = (hd,)
        return out

    @classmethod
    def tensor_init(cls, spec: PartSpec, width: int) -> Dict[str, str]:
        hn = spec.get("head_norm") or {}
        return {hn[key]: "gain" for key in ("q", "k") if hn.get(key)}

    @classmethod
    def cache_need(cls, spec: PartSpec, width: int):
        _, nkv, _, _ = cls._sizes(spec)
        return KVNeed(nkv * cls._maps(spec), cls._cache_dim(spec), None, 0)

    def __init__(self, spec, width, weights: WeightView, *, dtype, device):
        super().__init__(spec, width, weights, dtype=dtype, device=device)
        self.nh, self.nkv, self.qk_dim, self.v_dim = self._sizes(spec)
        self.maps = self._maps(spec)
        self.hd = hd = self._cache_dim(spec)
        if self.nh % self.nkv:
            raise ValueError("n_heads %d is not a multiple of n_kv_heads %d" % (self.nh, self.nkv))
        if hd > 512:
            raise ValueError("head sizes up to 512 are supported, found %d" % hd)
        self.group = self.nh // self.nkv
        self.scale = float(spec.get("scale") or 1.0 / math.sqrt(self.qk_dim))
        n = self._names(spec)
        # ---- the rotation: frequencies from the position part; an interleaved pairing becomes a row permutation
        pspec: PartSpec = spec["position"]
        self.position = part_class("position", pspec.kind)(pspec, width, weights, dtype=dtype, device=device)
        self.rot = int(getattr(self.position, "rotary_dim", 0) or 0)
        if self.rot > self.qk_dim:
            raise ValueError("rotary_dim %d exceeds head_dim %d" % (self.rot, self.qk_dim))
        if self.rot and getattr(self.position, "mult", 1.0) != 1.0:
            raise NotImplementedError("a rotation with scaled cosines and sines in this mixer")
        self.inv_freq = self.position.inv_freq if self.rot else None
        self.inv_freq64 = self.position.inv_freq64 if self.rot else None
        perm = None
        if self.rot and getattr(self.position, "pairing", "half") == "interleaved":
            perm = torch.tensor(list(range(0, self.rot, 2)) + list(range(1, self.rot, 2))
                                + list(range(self.rot, self.qk_dim)), dtype=torch.long, device=device)

        def heads_of(w, n_heads):
            """[n_heads * maps * qk_dim, width] -> [n_heads, maps, qk_dim, width], rows permuted for the rotation"""
            w = w.view(n_heads, self.maps, self.qk_dim, width)
            return w if perm is None else w[:, :, perm.to(w.device)]

        wq = heads_of(weights(n["q"]), self.nh)                                 # [nh, maps, d, width]
        wk = heads_of(weights(n["k"]), self.nkv)                                # [nkv, maps, d, width]
        wv = weights(n["v"]).view(self.nkv, 1, self.v_dim, width)
        # query heads in the order (group, map, head of the group); key heads (group, map); values once per map
        wq = wq.view(self.nkv, self.group, self.maps, self.qk_dim, width).transpose(1, 2)
        wq = wq.reshape(self.nh * self.maps * self.qk_dim, width)
        wk = wk.reshape(self.nkv * self.maps * self.qk_dim, width)
        wv = wv.expand(self.nkv, self.maps, self.v_dim, width).reshape(self.nkv * self.maps * self.v_dim, width)
        self.nhq, self.nkvq = self.nh * self.maps, self.nkv * self.maps
        ws = [_pad_heads(wq, self.nhq, self.qk_dim, hd), _pad_heads(wk, self.nkvq, self.qk_dim, hd),
              _pad_heads(wv, self.nkvq, self.v_dim, hd)]
        self.n_main = sum(w.shape[0] for w in ws)
        self.has_gate = bool(spec.get("head_gate"))
        if self.has_gate:
            if self.maps != 1:
                raise NotImplementedError("a gate per head on differential attention")
            wg = weights(spec["head_gate"])
            pad = -self.nh % 8                      # (the products take column counts that are multiples of eight)
            ws.append(wg if not pad else torch.cat([wg, torch.zeros((pad, width), dtype=wg.dtype, device=wg.device)]))
        if len({w.dtype for w in ws}) != 1:
            raise ValueError("q, k and v weights of %s are stored in different dtypes" % weights.prefix)
        self.wqkv = torch.cat(ws, dim=0).contiguous()
        wo = weights(n["o"])
        if self.v_dim != hd:
            wo = _pad_heads(wo.t().contiguous(), self.nh, self.v_dim, hd).t().contiguous()
        self.wo = wo
        # ---- the heads' norm
        hn = spec.get("head_norm")
        self.norm_when, self.norm_eps, self.gq, self.gk = "none", 0.0, None, None
        if hn:
            self.norm_when = str(hn.get("when") or "before")
            if self.norm_when not in ("before", "after"):
                raise ValueError("head_norm.when is 'before' or 'after' the rotation, found %r" % self.norm_when)
            self.norm_eps = float(hn["eps"])
            if bool(hn.get("q")) != bool(hn.get("k")):
                raise ValueError("a head norm has gains for queries and keys, or for neither")
            if hn.get("q"):
                def gain(name):
                    g = weights(name).to(torch.float32)
                    if perm is not None:
                        g = g[perm.to(g.device)]
                    out = torch.zeros(hd, dtype=torch.float32, device=g.device)
                    out[:self.qk_dim] = g
                    return out.contiguous()
                self.gq, self.gk = gain(hn["q"]), gain(hn["k"])
        qt = spec.get("q_temp")
        self.t_coef, self.t_every = (float(qt["coef"]), int(qt["every"])) if qt else (0.0, 1)
        if qt and self.t_every < 1:
            raise ValueError("q_temp.every must be at least 1, found %d" % self.t_every)
        # ---- differential attention's constants
        d = spec.get("differential")
        self.diff = None
        if d:
            f64 = [weights(d[key]).to(torch.float64).cpu() for key in ("lq1", "lk1", "lq2", "lk2")]
            diff = float(d["diff"])
            lam = math.exp(float((f64[0] * f64[1]).sum())) - math.exp(float((f64[2] * f64[3]).sum())) + diff
            self.diff = (lam, float(d["eps"]), 1.0 - diff)

    def forward(self, ctx: StepContext, y: torch.Tensor) -> Branch:
        nhq, nkvq, hd = self.nhq, self.nkvq, self.hd
        n_q = nhq * hd
        qkv = L.rows_or_planes(ctx, y, self.wqkv, self.dtype)
        pool, table, n_pages = ctx.cache.kv_view(ctx.entry.cache)
        q = qkv if qkv.dim() == 2 else torch.empty((ctx.T, n_q), dtype=self.dtype, device=y.device)
        K.headnorm_rope_store(qkv[..., :self.n_main], q, self.gq, self.gk, self.norm_eps, self.qk_dim, self.norm_when,
                              self.inv_freq, self.inv_freq64, self.rot, self.t_coef, self.t_every, ctx.pos, ctx.seq,
                              ctx.slot, nhq, nkvq, nkvq, hd, pool, table, n_pages, ctx.status)
        att = torch.empty((ctx.T, n_q), dtype=self.dtype, device=y.device)
        A.attention(ctx, q[:, :n_q] if q.shape[1] != n_q else q, att, nhq, nkvq, hd, self.scale, 0, pool, table,
                    n_pages)
        if self.diff is not None:
            lam, eps, mult = self.diff
            out = torch.empty((ctx.T, self.nh * hd), dtype=self.dtype, device=y.device)
            K.diff_combine(att, out, self.nh, self.group, hd, self.v_dim, lam, eps, mult)
            att = out
        elif self.has_gate:
            K.head_gate_mul(att, qkv[..., self.n_main:], att, hd)
        return Branch(L.planes(ctx, att, self.wo))

    def bytes_read(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.wqkv, self.wo))


register_part("mixer", "headnorm_attention", HeadNormAttention)
